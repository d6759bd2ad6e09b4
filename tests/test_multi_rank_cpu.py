"""CPU (gloo, world_size 2 and 3) check of the multi-rank decode plan: the
token-range partition, per-rank partials, the exchange and the log-sum-exp
merge reproduce the single-rank answer.  The arithmetic is the oracle's; what
is under test is the host logic the GPU path shares (bench.token_ranges, the
layout of the gathered partials, the merge order)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import bench
from oracle import oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_token_ranges_partition_on_block_borders():
    for L in (1, 15, 16, 17, 4097, 131072, 131073):
        for n in (1, 2, 3, 4, 8):
            r = bench.token_ranges(L, n)
            assert r[0][0] == 0 and r[-1][1] == L and len(r) == n
            for (a, b), (c, d) in zip(r[:-1], r[1:]):
                assert b == c and a <= b
            assert all(a % 16 == 0 for a, _ in r)


def _worker(rank, world, port, L, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(11)  # same data on every rank
    k = orc.randn_bf16(rng, (8, L, 64), 0.5)
    v = orc.randn_bf16(rng, (8, L, 64), 0.5)
    q = orc.randn_bf16(rng, (32, 64))
    lo, hi = bench.token_ranges(L, world)[rank]
    # this rank's pool holds only its own range, in its own (shuffled) blocks
    n = hi - lo
    nb = (n + 15) // 16 + 3
    table = np.random.default_rng(100 + rank).permutation(nb)[: (n + 15) // 16].astype(np.int32)
    pool = np.zeros((nb, 8, 2, 16, 64), np.uint16)
    if n:
        orc.paged_append(pool, table, k[:, lo:hi], v[:, lo:hi], 0)
    o, lse = orc.decode_paged(q, pool, table, 0, n)
    part = torch.from_numpy(np.concatenate([o.reshape(-1), lse]).astype(np.float32))
    gathered = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(gathered, part)
    g = torch.stack(gathered).numpy()
    O, merged_lse = orc.lse_merge(g[:, :2048].reshape(world, 32, 64), g[:, 2048:])
    want, want_lse = orc.attention(q[:, None, :], k, v, L)
    ok = bool(np.max(np.abs(O - want[:, 0])) < 1e-5 and np.max(np.abs(merged_lse - want_lse[:, 0])) < 1e-5)
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        q_out.put(all(flags))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,L", [(2, 513), (3, 40)])
def test_range_sharded_decode_over_gloo(world, L):
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, L, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q_out.get(timeout=5) is True


def _exchange_schedule_is_safe(world, layers, combiners, slots, rng, steps=20000):
    """Model of the in-kernel exchange under a random schedule.  Every rank has `combiners` actors;
    actor c handles layers c, c + combiners, ...: it pushes its words of layer l (tagged l) into slot
    l % slots of EVERY rank's buffer, then polls its own buffer until the words of all ranks in that
    slot carry l.  A word tagged with a later layer in a slot somebody still polls means the protocol
    overwrote data in use.  Returns False on such an overwrite, True when all actors finish."""
    buf = [[[-1] * world for _ in range(slots)] for _ in range(world)]   # buf[rank][slot][src] = tag
    state = {(r, c): ("push", c) for r in range(world) for c in range(combiners)}
    for _ in range(steps):
        live = [a for a, (_, l) in state.items() if l < layers]
        if not live:
            return True
        r, c = live[rng.integers(len(live))]
        phase, l = state[(r, c)]
        if phase == "push":
            for dst in range(world):
                buf[dst][l % slots][r] = l
            state[(r, c)] = ("poll", l)
        else:
            tags = buf[r][l % slots]
            if any(t > l for t in tags):
                return False            # a needed word was overwritten before it was read
            if all(t == l for t in tags):
                state[(r, c)] = ("push", l + combiners)
    return all(l >= layers for _, l in state.values())


def test_exchange_slot_count_is_enough_for_the_combining_ctas():
    """C combining CTAs per (sequence, head) on alternate layers need a slot count that is a
    multiple of C and at least 2 C (a peer can be C layers ahead of a slot still being polled): the
    library uses 8 slots with C in {1, 2, 4}.  The model finds no overwrite for those over many
    random schedules, and does find one with too few slots."""
    rng = np.random.default_rng(2024)
    for world in (1, 2, 3, 8):
        for _ in range(40):
            assert _exchange_schedule_is_safe(world, 16, 1, 2, rng)
            assert _exchange_schedule_is_safe(world, 16, 2, 4, rng)
            for combiners in (1, 2, 4):
                assert _exchange_schedule_is_safe(world, 16, combiners, 8, rng)
                assert _exchange_schedule_is_safe(world, 3, combiners, 8, rng)   # fewer layers than slots
    unsafe = sum(not _exchange_schedule_is_safe(2, 16, 2, 2, rng) for _ in range(200))
    assert unsafe > 0, "two slots with two combining CTAs should be caught by some schedule"
    unsafe = sum(not _exchange_schedule_is_safe(2, 16, 4, 4, rng) for _ in range(200))
    assert unsafe > 0, "four slots with four combining CTAs should be caught by some schedule"
