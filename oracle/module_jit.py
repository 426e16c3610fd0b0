"""Runs the module the product's Frontend builds on the host CPU.  TEST INFRASTRUCTURE ONLY.

`module_lower.cc` (linked against the product's operator API) builds a graph through
`PlaceHolder / Matmul / Relu / BatchedMatmul / Softmax / Transpose::build` and lowers the
resulting loop nests to scalar LLVM IR; this file JIT-compiles that IR with llvmlite (MCJIT,
host CPU, O2, no fast-math) and executes the module-level calls on numpy arrays.

This is the literal form of "the repo's own affine module lowered to CPU": the reference
declares that lowering (`Rewriter::loweringAffineDialect`, include/Optimizer/Rewriter.h:221)
but never wrote it (src/Optimizer/Rewriter.cc:1605-1612).  It is a second execution of the
operator definitions, derived from the IR rather than written by hand like `oracle.c`, and the
two are compared bit for bit in tests/test_oracle_module.py.  Only tests/ and bench.py's CPU
baseline legs may import it.
"""
from __future__ import annotations

import ctypes
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Sequence

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle_module.so"
_lib = None
_llvm_ready = False


def build(force: bool = False) -> Path:
    src = HERE / "module_lower.cc"
    runtime = HERE.parent / "kernelcodegen_b200" / "libkcg_runtime.so"
    stale = (not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime or
             (runtime.exists() and LIB_PATH.stat().st_mtime < runtime.stat().st_mtime))
    if force or stale:
        if not runtime.exists():
            from kernelcodegen_b200 import build as kbuild

            kbuild.build_host()
        subprocess.run(["make", "-C", str(HERE), "-B", "liboracle_module.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return LIB_PATH


def _load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(str(LIB_PATH))
        lib.oracle_module_lower.restype = ctypes.c_long
        lib.oracle_module_lower.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_int,
                                            ctypes.c_char_p, ctypes.c_size_t]
        _lib = lib
    return _lib


def lower(graph: str, dims: Sequence[int], dtype: str = "float32") -> str:
    """Program lines + ';;;IR' + LLVM IR of the Frontend's module for `graph` (see module_lower.cc)."""
    lib = _load()
    arr = (ctypes.c_int64 * len(dims))(*dims)
    cap = 1 << 20
    while True:
        buf = ctypes.create_string_buffer(cap)
        n = lib.oracle_module_lower(graph.encode(), dtype.encode(), arr, len(dims), buf, cap)
        if n < 0:
            raise RuntimeError(f"lowering {graph}{tuple(dims)} failed: {buf.value.decode()}")
        if n < cap:
            return buf.value.decode()
        cap = n + 1


def _llvm():
    global _llvm_ready
    import llvmlite.binding as llvm

    if not _llvm_ready:
        try:
            llvm.initialize()
        except Exception:
            pass            # newer llvmlite initialises itself
        llvm.initialize_native_target()
        llvm.initialize_native_asmprinter()
        for name in ("libm.so.6", "libc.so.6"):
            try:
                llvm.load_library_permanently(name)
            except Exception:
                pass
        _llvm_ready = True
    return llvm


class LoweredModule:
    """The Frontend's module for one graph, compiled for the host.

    graph / dims as in module_lower.cc: "matmul" | "matmul_relu" (m n k), "relu" | "softmax" |
    "transpose" (shape...), "batched_matmul_nn" | "batched_matmul_nt" (batch... m n k),
    "attention" (batch... sq skv hd).
    """

    def __init__(self, graph: str, dims: Sequence[int], dtype: str = "float32", opt: int = 2):
        llvm = _llvm()
        text = lower(graph, dims, dtype)
        prog, ir = text.split(";;;IR\n", 1)
        self.ir = ir
        self.np_dtype = np.float64 if dtype == "float64" else np.float32
        self.allocs = {}        # value id -> shape
        self.calls = []         # (callee, [arg ids], result id)
        for line in prog.splitlines():
            f = line.split()
            if not f:
                continue
            if f[0] == "alloc":
                rank = int(f[3])
                self.allocs[int(f[1])] = tuple(int(x) for x in f[4:4 + rank])
            elif f[0] == "call":
                n = int(f[2])
                self.calls.append((f[1], [int(x) for x in f[3:3 + n]], int(f[3 + n + 1])))
        # value ids that are results of calls are not placeholders; an alloc that is only ever the
        # LAST operand of a call whose result it becomes is an output buffer
        self.inputs = self._input_ids()
        mod = llvm.parse_assembly(ir)
        mod.verify()
        target = llvm.Target.from_default_triple()
        self.tm = target.create_target_machine(cpu=llvm.get_host_cpu_name(), features=llvm.get_host_cpu_features().flatten(),
                                               opt=opt)
        try:
            pto = llvm.create_pipeline_tuning_options(speed_level=opt, size_level=0)
            pb = llvm.create_pass_builder(self.tm, pto)
            pm = pb.getModulePassManager()
            pm.run(mod, pb)
        except AttributeError:      # older llvmlite: legacy pass manager
            pmb = llvm.create_pass_manager_builder()
            pmb.opt_level = opt
            pm = llvm.create_module_pass_manager()
            pmb.populate(pm)
            pm.run(mod)
        self.engine = llvm.create_mcjit_compiler(mod, self.tm)
        self.engine.finalize_object()
        self._mod = mod
        self._fns = {}

    def _input_ids(self) -> List[int]:
        produced = set()
        for callee, args, res in self.calls:
            # operators that take their output buffer as the last operand (Matmul, BatchedMatmul,
            # Transpose): that alloc is written, not read
            if callee.startswith(("Matmul_", "BatchMatmul_", "Transpose_")):
                produced.add(args[-1])
            produced.add(res)
        return [i for i in sorted(self.allocs) if i not in produced]

    def _fn(self, name: str, nargs: int, rows: bool):
        key = (name, rows)
        if key not in self._fns:
            addr = self.engine.get_function_address(name + (".rows" if rows else ""))
            if not addr:
                raise RuntimeError(f"function {name} not found in the compiled module")
            sig = [ctypes.c_void_p] * nargs + ([ctypes.c_int64, ctypes.c_int64] if rows else [])
            self._fns[key] = ctypes.CFUNCTYPE(ctypes.c_void_p, *sig)(addr)
        return self._fns[key]

    def run(self, *inputs: np.ndarray, threads: int = 1) -> np.ndarray:
        """Executes the module's calls in order on copies of `inputs` (the graph's PlaceHolders in
        creation order) and returns the last call's result.  `threads` > 1 spreads the outermost
        loop of every call over host threads (rows are independent in every nest: same bits)."""
        if len(inputs) != len(self.inputs):
            raise ValueError(f"the graph has {len(self.inputs)} placeholders, got {len(inputs)} arrays")
        bufs = {}
        for vid, arr in zip(self.inputs, inputs):
            a = np.array(arr, dtype=self.np_dtype, order="C", copy=True)
            if a.shape != self.allocs[vid]:
                raise ValueError(f"placeholder {vid} has shape {self.allocs[vid]}, got {a.shape}")
            bufs[vid] = a
        for vid, shape in self.allocs.items():
            if vid not in bufs:
                bufs[vid] = np.empty(shape, dtype=self.np_dtype)
        result = None
        for callee, args, res in self.calls:
            ptrs = [bufs[i].ctypes.data for i in args]
            if threads > 1:
                outer = self._outer_extent(callee, bufs, args)
                fn = self._fn(callee, len(args), rows=True)
                n = min(threads, outer)
                cuts = [outer * i // n for i in range(n + 1)]
                with ThreadPoolExecutor(max_workers=n) as ex:
                    rets = list(ex.map(lambda i: fn(*ptrs, cuts[i], cuts[i + 1]), range(n)))
                ret = rets[0]
            else:
                ret = self._fn(callee, len(args), rows=False)(*ptrs)
            # every operator here returns one of its operands (its output buffer, or its input when in place)
            hit = [i for i in args if bufs[i].ctypes.data == ret]
            if not hit:
                raise RuntimeError(f"{callee} returned a buffer the module does not know")
            bufs[res] = bufs[hit[-1]]
            result = bufs[res]
        return result

    def _outer_extent(self, callee: str, bufs, args) -> int:
        # the outermost loop of every nest runs over the first dimension of the result (Matmul,
        # BatchedMatmul: last operand; Relu, Softmax: the only operand) -- of the input for Transpose
        if callee.startswith("Transpose_"):
            return int(bufs[args[0]].shape[0])
        return int(bufs[args[-1]].shape[0])
