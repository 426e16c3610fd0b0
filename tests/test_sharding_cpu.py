"""Host-side multi-rank logic on CPU: partitioning, and a world_size-2 gloo run of the
row-block scheme with the check-in barrier (including a rank that never arrives)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernelcodegen_b200 import sharding

ROOT = Path(__file__).resolve().parents[1]


def test_row_blocks_cover_and_align():
    for m in (128, 4096, 32768, 1000, 130):
        for world in (1, 2, 4, 8):
            spans = [sharding.row_block(m, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b
            for lo, hi in spans:
                assert lo % 128 == 0 or lo == m
    assert sharding.row_block(32768, 3, 8) == (12288, 16384)


def test_weighted_row_blocks():
    # equal weights = the even split
    for m in (128, 4096, 32768, 1000, 130):
        for world in (1, 2, 4, 8):
            assert sharding.weighted_row_blocks(m, [1.0] * world) == [sharding.row_block(m, r, world) for r in range(world)]
    # a rank measured 10 % slower gets about 10 % fewer rows; the blocks still tile [0, m)
    spans = sharding.weighted_row_blocks(32768, [1.0, 1.0, 0.9, 1.0, 1.0, 1.0, 1.0, 1.0])
    assert spans[0][0] == 0 and spans[-1][1] == 32768
    for (a, b), (c, d) in zip(spans, spans[1:]):
        assert b == c
    sizes = [hi - lo for lo, hi in spans]
    assert all(s % 128 == 0 for s in sizes) and sum(sizes) == 32768
    assert sizes[2] == min(sizes) and abs(sizes[2] / sizes[0] - 0.9) < 0.04
    # finishing times are closer together than with the even split
    rates = [1.0, 1.0, 0.9, 1.0, 1.0, 1.0, 1.0, 1.0]
    assert max(s / r for s, r in zip(sizes, rates)) < max(4096 / r for r in rates)
    # every rank keeps at least one block; fewer blocks than ranks leaves empty ranks at the end
    assert all(hi > lo for lo, hi in sharding.weighted_row_blocks(1024, [100.0, 1.0, 1.0, 1.0]))
    assert sharding.weighted_row_blocks(256, [1.0, 1.0, 1.0]) == [(0, 128), (128, 256), (256, 256)]
    with pytest.raises(ValueError):
        sharding.weighted_row_blocks(1024, [1.0, 0.0])


def test_bh_shards():
    assert [sharding.bh_shard(256, r, 8) for r in range(8)] == [(32 * r, 32 * r + 32) for r in range(8)]
    assert [sharding.bh_shard(5, r, 2) for r in range(2)] == [(0, 3), (3, 5)]
    with pytest.raises(ValueError):
        sharding.bh_shard(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, absent_rank, result_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    try:
        # step 0: everyone checks in, then the row-block all-gather of C is emulated with gloo
        sharding.check_in(store, rank, world, step=0, timeout_s=20)
        m, n, k = 512, 64, 96
        g = torch.Generator().manual_seed(5)
        a = torch.rand(m, k, generator=g) * 2 - 1
        b = torch.rand(k, n, generator=g) * 2 - 1
        lo, hi = sharding.row_block(m, rank, world)
        c_local = torch.relu(a[lo:hi] @ b)
        parts = [torch.empty(sharding.row_block(m, r, world)[1] - sharding.row_block(m, r, world)[0], n) for r in range(world)]
        dist.all_gather(parts, c_local)
        c = torch.cat(parts)
        ok = torch.allclose(c, torch.relu(a @ b), atol=1e-5)
        # step 1: one rank stays away; the others must time out on the host
        outcome = "skipped"
        if rank != absent_rank:
            try:
                sharding.check_in(store, rank, world, step=1, timeout_s=1.0)
                outcome = "passed"
            except sharding.PeerTimeout:
                outcome = "timeout"
        Path(result_dir, f"r{rank}.txt").write_text(f"{int(ok)} {outcome}")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_rows_and_detect_a_missing_peer(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 1, str(tmp_path)), nprocs=world, join=True)
    r0 = (tmp_path / "r0.txt").read_text().split()
    r1 = (tmp_path / "r1.txt").read_text().split()
    assert r0[0] == "1" and r1[0] == "1"
    assert r0[1] == "timeout"       # rank 0 waited for rank 1, which never checked in for step 1
    assert r1[1] == "skipped"
