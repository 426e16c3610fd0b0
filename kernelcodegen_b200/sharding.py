"""How the two operators are split over the GPUs of one node.

GEMM: rows of C are independent, so rank r owns a contiguous block of rows of A and C
(B is replicated).  FMHA: (batch, head) pairs are independent, so rank r owns a contiguous range
of the flattened batch*head axis and no data moves between ranks.  The functions here are pure
host logic (tested on CPU with gloo ranks); `check_in` is the host-side rendezvous every rank
passes before a step that writes into peers' memory is launched, so that a missing rank is
noticed on the host instead of by a kernel waiting on it.
"""
from __future__ import annotations

import time
from typing import List, Sequence, Tuple


def row_block(m: int, rank: int, world: int, align: int = 128) -> Tuple[int, int]:
    """[lo, hi) rows of rank `rank`: blocks of `align` rows dealt out as evenly as possible."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    blocks = (m + align - 1) // align
    base, extra = divmod(blocks, world)
    lo_b = rank * base + min(rank, extra)
    hi_b = lo_b + base + (1 if rank < extra else 0)
    return min(lo_b * align, m), min(hi_b * align, m)


def weighted_row_blocks(m: int, weights: Sequence[float], align: int = 128) -> List[Tuple[int, int]]:
    """[lo, hi) rows of every rank when rank r should receive a share of the rows proportional to
    weights[r] (for instance its measured rate: the GPUs of one node differ by several per cent
    under their power caps, and a step ends when the slowest rank ends).  Blocks of `align` rows;
    every rank receives at least one block while there are enough; equal weights give the split
    of `row_block`."""
    world = len(weights)
    if world <= 0 or any((not w > 0) or w != w or w == float("inf") for w in weights):
        raise ValueError("weights must be positive and finite")
    blocks = (m + align - 1) // align
    total = float(sum(weights))
    ideal = [w / total * blocks for w in weights]
    counts = [int(x) for x in ideal]
    if blocks >= world:
        counts = [max(1, c) for c in counts]
    # hand the remaining blocks to the largest fractional parts (ties: lowest rank, like row_block);
    # take back from the smallest if the minimum of one block per rank overshot
    while sum(counts) < blocks:
        r = max(range(world), key=lambda i: (ideal[i] - counts[i], -i))
        counts[r] += 1
    while sum(counts) > blocks:
        r = max((i for i in range(world) if counts[i] > (1 if blocks >= world else 0)),
                key=lambda i: (counts[i] - ideal[i], i))
        counts[r] -= 1
    out, lo = [], 0
    for c in counts:
        hi = lo + c
        out.append((min(lo * align, m), min(hi * align, m)))
        lo = hi
    return out


def bh_shard(batch_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """[lo, hi) of the flattened batch*head axis owned by `rank`."""
    return row_block(batch_heads, rank, world, align=1)


class PeerTimeout(RuntimeError):
    """A rank did not check in within the time limit (maps to KCG_PEER_TIMEOUT)."""


def check_in(store, rank: int, world: int, step: int, timeout_s: float = 30.0, poll_s: float = 0.002) -> None:
    """Host-side barrier over a torch.distributed store (TCPStore/FileStore/HashStore).

    Every rank adds 1 to the counter of `step` and waits until it reaches `world`.  Raises
    PeerTimeout if some rank never arrives -- before any kernel that stores into that rank's
    memory has been launched.
    """
    key = f"kcg/checkin/{step}"
    store.add(key, 1)
    deadline = time.monotonic() + timeout_s
    while True:
        if int(store.add(key, 0)) >= world:
            return
        if time.monotonic() > deadline:
            raise PeerTimeout(f"rank {rank}: only {int(store.add(key, 0))} of {world} ranks checked in for step {step}")
        time.sleep(poll_s)
