"""Child process of tests/test_bounds_build_gpu.py: runs with KCG_DEBUG_BOUNDS=1, so that
`capi.load()` picks the bounds-checking build of the library.  Prints one JSON line."""
import ctypes
import json
import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from kernelcodegen_b200 import capi, ops  # noqa: E402
from oracle import oracle  # noqa: E402


def rel(x, ref):
    return float(np.abs(np.asarray(x, np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def main():
    dev = torch.device("cuda:0")
    lib = capi.load()
    out = {"enabled": int(lib.kcg_debug_bounds_enabled()), "cases": []}
    g = torch.Generator().manual_seed(1)
    # ragged GEMMs through every kernel variant: CTA pairs with the shared-K tail, single CTAs, bf16, batched
    for m, n, k, kw in [(300, 520, 132, {}), (300, 520, 132, {"cta_group": 1}), (1000, 264, 96, {"cta_group": 2, "tile_n": 256}),
                        (130, 72, 64, {"precision": "tf32"})]:
        a = torch.rand((m, k), generator=g) * 2 - 1
        b = torch.rand((k, n), generator=g) * 2 - 1
        c = ops.matmul_relu(a.to(dev), b.to(dev), **kw)
        out["cases"].append({"what": f"gemm {m}x{n}x{k} {kw}", "err": rel(c.cpu().numpy(), oracle.matmul_relu(a.numpy(), b.numpy())),
                             "tol": 5e-3 if kw.get("precision") == "tf32" else 1e-4, "status": ops.last_device_status()})
    a = (torch.rand((300, 136), generator=g) * 2 - 1).bfloat16()
    b = (torch.rand((136, 200), generator=g) * 2 - 1).bfloat16()
    c = ops.matmul(a.to(dev), b.to(dev))
    out["cases"].append({"what": "gemm bf16 300x200x136", "err": rel(c.float().cpu().numpy(), oracle.matmul(a.float().numpy(), b.float().numpy())),
                         "tol": 2e-2, "status": ops.last_device_status()})
    a = torch.rand((5, 130, 40), generator=g) * 2 - 1
    b = torch.rand((5, 40, 72), generator=g) * 2 - 1
    c = ops.batched_matmul(a.to(dev), b.to(dev))
    out["cases"].append({"what": "batched 5x130x72x40", "err": rel(c.cpu().numpy(), oracle.batched_matmul(a.numpy(), b.numpy())),
                         "tol": 1e-4, "status": ops.last_device_status()})
    # ragged attention, causal with fewer keys than queries
    q = torch.randn((1, 2, 384, 64), generator=g).bfloat16()
    k_, v = (torch.randn((1, 2, 130, 64), generator=g).bfloat16() for _ in range(2))
    o = ops.fmha(q.to(dev), k_.to(dev), v.to(dev), scale=0.125, causal=True)
    want = oracle.fmha(q.float().numpy(), k_.float().numpy(), v.float().numpy(), scale=0.125, causal=True)
    out["cases"].append({"what": "fmha 384x130 causal", "err": rel(o.float().cpu().numpy(), want), "tol": 2e-2,
                         "status": ops.last_device_status()})

    # the reporting path: cap the extent the kernel checks against at half of C (the buffer itself is
    # large enough, nothing is really out of bounds): the stores beyond the cap are skipped and reported
    m, n, k = 512, 256, 64
    a = (torch.rand((m, k), generator=g) * 2 - 1).to(dev)
    b = (torch.rand((k, n), generator=g) * 2 - 1).to(dev)
    c = torch.full((m, n), -7.0, device=dev)
    cap = m * n * 4 // 2
    lib.kcg_debug_set_extent_limit(cap)
    ops.matmul(a, b, out=c)
    status = ops.last_device_status()
    detail = (ctypes.c_uint64 * 2)()
    lib.kcg_debug_bounds_detail(detail)
    lib.kcg_debug_set_extent_limit(0)
    want = oracle.matmul(a.cpu().numpy(), b.cpu().numpy())
    cn = c.cpu().numpy()
    out["capped"] = {"status": status, "offset": int(detail[0]), "extent": int(detail[1]), "cap": cap,
                     "below_cap_err": rel(cn[: m // 2], want[: m // 2]), "beyond_cap_untouched": bool((cn[m // 2:] == -7.0).all())}
    # and the context is still usable, with the cap lifted everything is written again
    ops.matmul(a, b, out=c)
    out["after"] = {"status": ops.last_device_status(), "err": rel(c.cpu().numpy(), want)}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
