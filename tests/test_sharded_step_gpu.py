"""GPU parity of the one-launch sharded decode step (pa_decode_step_sharded): the in-kernel
{value, step} word exchange and merge, with SEVERAL ranks, against the fp32 oracle.

On one GPU the ranks are pools in this process and their steps run as ONE cooperative launch
(pa_decode_step_sharded_colocated): ranks wait on each other's words, and separate launches on one
GPU are not guaranteed to run at the same time.  The kernel code per rank is the one the multi-GPU
path runs (same step body, same exchange buffers, peers reached through plain pointers)."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import _lib, paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, check_close, f32_dev, to_dev, to_u16

pytestmark = pytest.mark.gpu


def _fill(pool, seq, layers, k, v):
    """k, v [layers][8, n, 64] final cache values -> positions 0..n-1 of `seq` (identity rotation)."""
    n = k[0].shape[1]
    if n == 0:
        return
    pool.reserve(seq, n)
    pool.batch_set([seq], [n])
    ones = torch.ones(n, 32, dtype=torch.float32, device=DEV)
    zeros = torch.zeros(n, 32, dtype=torch.float32, device=DEV)
    for layer in range(layers):
        pool.append(layer, None, to_dev(k[layer].transpose(1, 0, 2)), to_dev(v[layer].transpose(1, 0, 2)),
                    ones, zeros, None)
    torch.cuda.synchronize()


@pytest.mark.parametrize("world,cuts,chunk_blocks", [
    (2, [0, 304, 700], 8),          # two ranks, several chunks per (sequence, head)
    (3, [0, 256, 256, 700], 16),    # an empty middle range
    (4, [0, 64, 256, 512, 700], 0),  # planner's own split on a quarter of the SMs
])
def test_colocated_ranks_step_matches_whole_sequence(cuda, world, cuts, chunk_blocks):
    """3 layers, 6 consecutive steps (the 4 word slots wrap, two combining CTAs alternate over the
    layers), every layer's merged rows on every rank against the oracle over the WHOLE sequence;
    all ranks must hold the same bits."""
    rng = np.random.default_rng(400 + world)
    layers, steps, L = 3, 6, cuts[-1]
    cos, sin = orc.build_rope_tables(L + steps + 1)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    K = [orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)]
    V = [orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)]
    pools, seqs = [], []
    for r in range(world):
        lo, hi = cuts[r], cuts[r + 1]
        nb = (hi - lo + steps + 15) // 16 + 4
        pool = paged.KVPool(layers, nb, 8, 1)
        pool.set_free_order(rng.permutation(nb))
        if chunk_blocks:
            pool.set_decode_chunk_blocks(chunk_blocks)
        s = pool.create_seq()
        _fill(pool, s, layers, [k[:, lo:hi] for k in K], [v[:, lo:hi] for v in V])
        pools.append(pool)
        seqs.append(s)
    xs = [paged.Exchange(0, r, world, 1, 8) for r in range(world)]
    bufs = [x.buffer()[0] for x in xs]
    for x in xs:
        x.connect_ptrs(bufs)
    owner = world - 1
    for step in range(steps):
        pos = L + step
        q_new = orc.randn_bf16(rng, (layers, 1, 32, 64))
        k_new = orc.randn_bf16(rng, (layers, 1, 8, 64))
        v_new = orc.randn_bf16(rng, (layers, 1, 8, 64))
        qd, kd, vd = to_dev(q_new), to_dev(k_new), to_dev(v_new)
        q_rots = [torch.zeros_like(qd) for _ in range(world)]
        outs = [torch.full((layers, 1, 2048), 9.0, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
        pools[owner].reserve(seqs[owner], pools[owner].length(seqs[owner]) + 1)
        for r in range(world):
            pools[r].batch_set_sharded([seqs[r]], [1 if r == owner else 0], [1], [pos], [cuts[r]])
        before = [p.step_launches() for p in pools]
        paged.decode_step_sharded_colocated(
            pools, xs, 0, layers, [qd] * world, [kd if r == owner else None for r in range(world)],
            [vd if r == owner else None for r in range(world)], 2048, 512, cos_d, sin_d, q_rots, outs, 2048, 2048)
        torch.cuda.synchronize()
        for p in pools:
            p.check()
        assert [p.step_launches() for p in pools] == [b + 1 for b in before]
        for layer in range(layers):
            K[layer][:, pos] = orc.rope(k_new[layer], cos, sin, pos, 1)[:, 0]
            V[layer][:, pos] = v_new[layer, 0]
            q_rot = orc.rope(q_new[layer], cos, sin, pos, 1)
            O, _ = orc.attention(q_rot, K[layer], V[layer], pos + 1)
            for r in range(world):
                check_close(orc.bf16_to_f32(to_u16(outs[r][layer, 0])), O[:, 0].reshape(-1),
                            f"step {step} layer {layer} rank {r}")
                assert np.array_equal(to_u16(q_rots[r][layer, 0]), orc.rope(q_new[layer], cos, sin, pos, 1, True)[0])
        for r in range(1, world):
            assert torch.equal(outs[r], outs[0]), f"step {step}: rank {r} merged other bits than rank 0"
    # the owner's cache holds the appended rows bit for bit
    gk = torch.zeros(8, pools[owner].length(seqs[owner]), 64, dtype=torch.bfloat16, device=DEV)
    gv = torch.zeros_like(gk)
    for layer in range(layers):
        pools[owner].gather_kv(layer, seqs[owner], gk, gv, gk.shape[1])
        torch.cuda.synchronize()
        assert np.array_equal(to_u16(gk), K[layer][:, cuts[owner]:L + steps])
        assert np.array_equal(to_u16(gv), V[layer][:, cuts[owner]:L + steps])
    for x in xs:
        x.close()
    for p in pools:
        p.close()


def test_colocated_step_is_refused_when_it_cannot_be_coresident(cuda):
    """Too many chunks for a share of the SMs: PA_ERR_UNSUPPORTED, the exchanges' step numbers are
    handed back, and the next (fitting) step still works."""
    rng = np.random.default_rng(410)
    layers, L = 2, 4096
    cos, sin = orc.build_rope_tables(L + 4)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    K = [orc.randn_bf16(rng, (8, L + 1, 64), 0.5) for _ in range(layers)]
    V = [orc.randn_bf16(rng, (8, L + 1, 64), 0.5) for _ in range(layers)]
    cuts = [0, 2048, L]
    pools, seqs = [], []
    for r in range(2):
        nb = 2048 // 16 + 6
        pool = paged.KVPool(layers, nb, 8, 1)
        s = pool.create_seq()
        _fill(pool, s, layers, [k[:, cuts[r]:cuts[r + 1]] for k in K], [v[:, cuts[r]:cuts[r + 1]] for v in V])
        pools.append(pool)
        seqs.append(s)
    xs = [paged.Exchange(0, r, 2, 1, 8) for r in range(2)]
    bufs = [x.buffer()[0] for x in xs]
    for x in xs:
        x.connect_ptrs(bufs)
    q_new = orc.randn_bf16(rng, (layers, 1, 32, 64))
    k_new = orc.randn_bf16(rng, (layers, 1, 8, 64))
    v_new = orc.randn_bf16(rng, (layers, 1, 8, 64))
    qd, kd, vd = to_dev(q_new), to_dev(k_new), to_dev(v_new)
    q_rots = [torch.zeros_like(qd) for _ in range(2)]
    outs = [torch.zeros(layers, 1, 2048, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    pools[1].reserve(seqs[1], 2049)
    for r in range(2):
        pools[r].batch_set_sharded([seqs[r]], [r], [1], [L], [cuts[r]])
        pools[r].set_decode_chunk_blocks(2)  # 64 chunks x 8 heads: far more CTAs than half the SMs
    args = (pools, xs, 0, layers, [qd, qd], [None, kd], [None, vd], 2048, 512, cos_d, sin_d, q_rots, outs, 2048, 2048)
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.decode_step_sharded_colocated(*args)
    assert ei.value.code == 3
    for r in range(2):
        pools[r].set_decode_chunk_blocks(32)
    paged.decode_step_sharded_colocated(*args)
    torch.cuda.synchronize()
    for p in pools:
        p.check()
    for layer in range(layers):
        K[layer][:, L] = orc.rope(k_new[layer], cos, sin, L, 1)[:, 0]
        V[layer][:, L] = v_new[layer, 0]
        O, _ = orc.attention(orc.rope(q_new[layer], cos, sin, L, 1), K[layer], V[layer], L + 1)
        for r in range(2):
            check_close(orc.bf16_to_f32(to_u16(outs[r][layer, 0])), O[:, 0].reshape(-1), f"layer {layer} rank {r}")
    for x in xs:
        x.close()
    for p in pools:
        p.close()


def test_step_kernel_wait_on_a_silent_peer_times_out_and_the_pool_recovers(cuda):
    """The one-launch step with an exchange whose peer never publishes: the combining CTAs' bounded
    polls run out (about a second per layer turn), the kernel returns, pa_pool_check reports
    PA_ERR_TIMEOUT and clears the status word and the arrival counters; a clean step on the same
    pool afterwards equals the per-layer path.  Nothing faults: the wait simply is never satisfied."""
    rng = np.random.default_rng(420)
    layers, L = 2, 300
    cos, sin = orc.build_rope_tables(L + 4)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    K = [orc.randn_bf16(rng, (8, L, 64), 0.5) for _ in range(layers)]
    V = [orc.randn_bf16(rng, (8, L, 64), 0.5) for _ in range(layers)]
    pool = paged.KVPool(layers, 40, 8, 1)
    s = pool.create_seq()
    _fill(pool, s, layers, K, V)
    x = paged.Exchange(0, 0, 2, 1, 8)
    ptr, nbytes = x.buffer()
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    x.connect_ptrs([ptr, silent_peer])
    q = to_dev(orc.randn_bf16(rng, (layers, 1, 32, 64)))
    q_rot = torch.zeros_like(q)
    out = torch.zeros(layers, 1, 2048, dtype=torch.bfloat16, device=DEV)
    pool.batch_set_sharded([s], [0], [1], [L - 1], [0])
    paged.decode_step_sharded(pool, x, 0, layers, q, None, None, 2048, 512, cos_d, sin_d, q_rot, out, 2048, 2048)
    torch.cuda.synchronize()
    with pytest.raises(_lib.PagedAttentionError) as ei:
        pool.check()
    assert ei.value.code == 5
    pool.check()  # cleared
    x.close()
    # the pool still serves: one-launch step == per-layer kernels, and both match the oracle
    pool.batch_set_sharded([s], [0], [1], [L - 1], [0])
    got = torch.zeros(layers, 1, 2048, dtype=torch.bfloat16, device=DEV)
    pool.decode_step(0, layers, q, None, None, 2048, 512, cos_d, sin_d, q_rot, got, 2048, 2048)
    assert pool.step_launches() >= 2
    pool.set_step_kernel(False)
    want = torch.zeros_like(got)
    pool.decode_step(0, layers, q, None, None, 2048, 512, cos_d, sin_d, q_rot, want, 2048, 2048)
    torch.cuda.synchronize()
    pool.check()
    assert torch.equal(got, want)
    for layer in range(layers):
        qr = orc.rope(to_u16(q[layer]), cos, sin, L - 1, 1)
        O, _ = orc.attention(qr, K[layer], V[layer], L)
        check_close(orc.bf16_to_f32(to_u16(got[layer, 0])), O[:, 0].reshape(-1), f"layer {layer} after a timeout")
    pool.close()
