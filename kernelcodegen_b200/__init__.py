"""B200 (sm_100a) kernels for the two operators KernelCodeGen generates: fused matmul+ReLU
and FMHA, behind a C-ABI (`include/kcg_capi.h`)."""
from . import capi  # noqa: F401

__all__ = ["capi", "ops"]


def __getattr__(name):
    if name == "ops":
        import importlib

        return importlib.import_module(".ops", __name__)
    raise AttributeError(name)
