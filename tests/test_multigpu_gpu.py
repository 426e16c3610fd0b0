"""Two-GPU test of the row-block GEMM whose epilogue stores every C tile into both ranks'
copies of C (fused all-gather over peer memory).  Skipped on a box with a single GPU."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from kernelcodegen_b200 import ops, peer, sharding
    from oracle import oracle

    m, n, k = 1024, 640, 384
    g = torch.Generator().manual_seed(3)
    a = (torch.rand((m, k), generator=g) * 2 - 1).bfloat16()
    b = (torch.rand((k, n), generator=g) * 2 - 1).bfloat16()
    lo, hi = sharding.row_block(m, rank, world)
    cm = peer.PeerMatrix(m, n, torch.bfloat16, dev)
    cm.tensor.fill_(-1.0)
    torch.cuda.synchronize()
    dist.barrier()
    token = torch.zeros(1, device=dev)
    ops.matmul_relu(a[lo:hi].to(dev), b.to(dev), out=cm.tensor[lo:hi], peers=cm.peer_row_ptrs(lo))
    dist.all_reduce(token)  # every rank's kernel, and so every store into this copy, has finished
    torch.cuda.synchronize()
    got = cm.tensor.float().cpu().numpy()
    want = oracle.matmul_relu(a.float().numpy(), b.float().numpy())
    err = float(np.abs(got - want).max() / np.abs(want).max())
    # the same with single CTAs (the kernel long launches use: two epilogue warp groups)
    cm.tensor.fill_(-1.0)
    torch.cuda.synchronize()
    dist.barrier()
    ops.matmul_relu(a[lo:hi].to(dev), b.to(dev), out=cm.tensor[lo:hi], peers=cm.peer_row_ptrs(lo), cta_group=1)
    dist.all_reduce(token)
    torch.cuda.synchronize()
    got = cm.tensor.float().cpu().numpy()
    err = max(err, float(np.abs(got - want).max() / np.abs(want).max()))
    # the same all-gather through the host-buffer entry: strips computed from chunked copies
    # must land in both ranks' copies of C and in this rank's host block
    cm.tensor.fill_(-1.0)
    torch.cuda.synchronize()
    dist.barrier()
    a_h, b_h = a[lo:hi].contiguous().pin_memory(), b.pin_memory()
    c_h = torch.empty((hi - lo, n), dtype=torch.bfloat16).pin_memory()
    a_d, b_d = torch.zeros_like(a_h, device=dev), torch.zeros_like(b_h, device=dev)
    ops.matmul_host(a_h, b_h, c_h, a_d, b_d, cm.tensor[lo:hi], relu=True, peers=cm.peer_row_ptrs(lo), chunks=2)
    dist.all_reduce(token)
    torch.cuda.synchronize()
    got = cm.tensor.float().cpu().numpy()
    err = max(err, float(np.abs(got - want).max() / np.abs(want).max()))
    err = max(err, float(np.abs(c_h.float().numpy() - want[lo:hi]).max() / np.abs(want).max()))
    status = ops.last_device_status()
    Path(out_dir, f"r{rank}.txt").write_text(f"{err} {status}")
    cm.close()
    dist.destroy_process_group()


def test_two_ranks_fill_both_copies_of_c(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from kernelcodegen_b200 import build

    build.build()
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        err, status = (tmp_path / f"r{r}.txt").read_text().split()
        assert float(err) <= 2e-2, f"rank {r}: full C (own and peer rows) off by {err}"
        assert int(status) == 0
