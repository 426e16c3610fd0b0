"""The row-block GEMM whose epilogue stores every C tile into all ranks' copies of C (fused
all-gather over peer memory) and publishes a completion flag: two-GPU tests (skipped on a box
with a single GPU) and single-GPU tests of the flag / bounded-wait protocol."""
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


def _worker(rank, world, port, out_dir, backend):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"      # NCCL is only the rendezvous and the barrier here
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
    want = oracle.matmul_relu(a.float().numpy(), b.float().numpy())
    lo, hi = sharding.row_block(m, rank, world)
    cm = peer.PeerMatrix(m, n, torch.bfloat16, dev, backend=backend)
    a_d, b_d = a[lo:hi].to(dev), b.to(dev)
    err = 0.0
    step = 0

    def check():
        # own rows and the peer's rows, as they arrived in THIS rank's copy
        got = cm.tensor.float().cpu().numpy()
        return float(np.abs(got - want).max() / np.abs(want).max())

    # CTA pairs / single CTAs (the kernel long launches use: two epilogue warp groups); with the
    # multicast address when the copies have one, and with plain unicast peer stores
    for cta_group in (0, 1):
        for multicast in (True, False):
            step += 1
            cm.tensor.fill_(-1.0)
            torch.cuda.synchronize()
            dist.barrier()
            ops.matmul_relu(a_d, b_d, out=cm.tensor[lo:hi], cta_group=cta_group,
                            **cm.store_args(lo, step, multicast=multicast))
            cm.wait(step)            # every rank's launch, and so every store into this copy, has finished
            ops.peer_wait_status()   # synchronises; raises if the bounded wait ran out
            err = max(err, check())
    # the same all-gather through the host-buffer entry: strips computed from chunked copies
    # must land in both ranks' copies of C and in this rank's host block
    cm.tensor.fill_(-1.0)
    torch.cuda.synchronize()
    dist.barrier()
    token = torch.zeros(1, device=dev)
    a_h, b_h = a[lo:hi].contiguous().pin_memory(), b.pin_memory()
    c_h = torch.empty((hi - lo, n), dtype=torch.bfloat16).pin_memory()
    a_s, b_s = torch.zeros_like(a_h, device=dev), torch.zeros_like(b_h, device=dev)
    ops.matmul_host(a_h, b_h, c_h, a_s, b_s, cm.tensor[lo:hi], relu=True, peers=cm.peer_row_ptrs(lo), chunks=2)
    dist.all_reduce(token)
    torch.cuda.synchronize()
    err = max(err, check())
    err = max(err, float(np.abs(c_h.float().numpy() - want[lo:hi]).max() / np.abs(want).max()))
    status = ops.last_device_status()
    Path(out_dir, f"r{rank}.txt").write_text(f"{err} {status} {cm.backend} {int(cm.mc_ptr != 0)}")
    cm.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("backend", ["ipc", "symmetric"])
def test_two_ranks_fill_both_copies_of_c(tmp_path, backend):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from kernelcodegen_b200 import build

    build.build()
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), backend), nprocs=2, join=True)
    for r in range(2):
        err, status, used, mc = (tmp_path / f"r{r}.txt").read_text().split()
        assert float(err) <= 2e-2, f"rank {r}: full C (own and peer rows) off by {err}"
        assert int(status) == 0
        assert used == backend


def test_completion_flag_follows_the_stores_single_gpu(cuda_device):
    """One rank: the launch publishes its flag, the bounded wait passes, C matches the oracle."""
    from kernelcodegen_b200 import ops, peer
    from oracle import oracle

    g = torch.Generator().manual_seed(5)
    a = (torch.rand((512, 256), generator=g) * 2 - 1).bfloat16()
    b = (torch.rand((256, 384), generator=g) * 2 - 1).bfloat16()
    cm = peer.PeerMatrix(512, 384, torch.bfloat16, cuda_device)
    try:
        for step, cta_group in ((1, 0), (2, 1), (7, 2)):
            cm.tensor.fill_(-1.0)
            ops.matmul_relu(a.to(cuda_device), b.to(cuda_device), out=cm.tensor, cta_group=cta_group,
                            **cm.store_args(0, step))
            cm.wait(step)
            ops.peer_wait_status()
            assert int(cm.flags[0].item()) == step
            want = oracle.matmul_relu(a.float().numpy(), b.float().numpy())
            err = np.abs(cm.tensor.float().cpu().numpy() - want).max() / np.abs(want).max()
            assert err <= 2e-2
    finally:
        cm.close()


def test_wait_for_an_absent_rank_times_out_and_context_survives(cuda_device):
    """A flag nothing sets: the wait gives up after its poll limit, the status call reports
    KCG_PEER_TIMEOUT, and the device is usable afterwards."""
    from kernelcodegen_b200 import capi, ops, peer

    cm = peer.PeerMatrix(128, 128, torch.float32, cuda_device)
    try:
        cm.wait(3, max_polls=2000)
        with pytest.raises(capi.KcgError) as ei:
            ops.peer_wait_status()
        assert ei.value.status == capi.KCG_PEER_TIMEOUT
        ops.peer_wait_status()           # cleared
        x = torch.ones(8, device=cuda_device)
        assert float((x + 1).sum().item()) == 16.0
    finally:
        cm.close()
