"""GPU tests of the cross-rank partial exchange used by sequence-range sharded
decode, on ONE GPU: the ranks are pools in this process and every kernel that
waits on a flag is launched only after the kernels that raise it, so nothing
waits on a later launch.  Also: a wait that nothing satisfies runs out after
about a second and comes back as PA_ERR_TIMEOUT with the context intact."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import _lib, paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, check_close, f32_dev, fill_cache, to_dev, to_u16

pytestmark = pytest.mark.gpu


def make_rank(rng, k, v, lo, hi, extra_tokens):
    n = hi - lo
    nb = (n + extra_tokens + 15) // 16 + 4
    pool = paged.KVPool(1, nb, 8, 1)
    pool.set_free_order(rng.permutation(nb))
    s = pool.create_seq()
    if n:
        fill_cache(pool, 0, s, k[:, lo:hi], v[:, lo:hi])
    return pool, s


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_decode_steps_match_whole_sequence(cuda, world):
    rng = np.random.default_rng(90 + world)
    L, steps = 700, 3
    k = orc.randn_bf16(rng, (8, L + steps, 64), 0.5)
    v = orc.randn_bf16(rng, (8, L + steps, 64), 0.5)
    cos, sin = orc.build_rope_tables(L + steps)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    cuts = [0, 256, 256, L] if world == 3 else [0, 304, L]  # world 3 has an empty middle range
    ranks = [make_rank(rng, k, v, cuts[r], cuts[r + 1], steps) for r in range(world)]
    xs = [paged.Exchange(0, r, world, 1, 8) for r in range(world)]
    bufs = [x.buffer()[0] for x in xs]
    for x in xs:
        x.connect_ptrs(bufs)
    owner = world - 1
    for step in range(steps):
        pos = L + step
        q_new = orc.randn_bf16(rng, (1, 32, 64))
        k_new = orc.randn_bf16(rng, (1, 8, 64))
        v_new = orc.randn_bf16(rng, (1, 8, 64))
        k[:, pos] = orc.rope(k_new, cos, sin, pos, 1)[:, 0]  # the cache row the owner will hold
        v[:, pos] = v_new[0]
        q_rots = []
        for r, (pool, s) in enumerate(ranks):
            if r == owner:
                pool.reserve(s, pool.length(s) + 1)
            pool.batch_set_sharded([s], [1 if r == owner else 0], [1], [pos], [cuts[r]])
            qd = to_dev(q_new)
            pool.append(0, qd, to_dev(k_new) if r == owner else None, to_dev(v_new) if r == owner else None,
                        cos_d, sin_d, qd)
            q_rots.append(qd)
        for r, (pool, s) in enumerate(ranks):  # every rank pushes its partial to all ranks ...
            xs[r].push(pool, 0, q_rots[r])
        outs = []
        for r, (pool, s) in enumerate(ranks):  # ... only then does any rank wait and merge
            o = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
            xs[r].merge(pool, o, 2048)
            outs.append(o)
        torch.cuda.synchronize()
        for pool, _ in ranks:
            pool.check()
        q_rot = orc.rope(q_new, cos, sin, pos, 1)
        O, _ = orc.attention(q_rot, k, v, pos + 1)
        for r in range(world):
            check_close(orc.bf16_to_f32(to_u16(outs[r]))[0], O[:, 0].reshape(-1), f"step {step} rank {r}")
            assert torch.equal(outs[r], outs[0])  # every rank merges the same bits
    for x in xs:
        x.close()
    for pool, _ in ranks:
        pool.close()


def test_wait_that_nothing_satisfies_times_out_cleanly(cuda):
    rng = np.random.default_rng(95)
    k = orc.randn_bf16(rng, (8, 100, 64), 0.5)
    v = orc.randn_bf16(rng, (8, 100, 64), 0.5)
    pool, s = make_rank(rng, k, v, 0, 100, 0)
    x = paged.Exchange(0, 0, 2, 1, 8)
    ptr, nbytes = x.buffer()
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)  # a rank that never publishes
    x.connect_ptrs([ptr, silent_peer])
    q = to_dev(orc.randn_bf16(rng, (1, 32, 64)))
    out = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
    pool.batch_set([s], [0])
    x.push(pool, 0, q)
    x.merge(pool, out, 2048)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    torch.cuda.synchronize()
    with pytest.raises(_lib.PagedAttentionError) as ei:
        pool.check()
    assert ei.value.code == 5
    # the status word is cleared and the device still works
    pool.check()
    want = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
    pool.decode(0, q, want, 2048)
    torch.cuda.synchronize()
    pool.check()
    O, _ = orc.attention(to_u16(q)[0][:, None, :], k, v, 100)
    check_close(orc.bf16_to_f32(to_u16(want))[0], O[:, 0].reshape(-1), "decode after a timed-out wait")
    x.close()
    pool.close()


def test_sharded_step_with_one_rank_equals_plain_step(cuda):
    """pa_decode_step_sharded (append fused in, partials pushed, the combining CTA
    waits for the flags and merges in the kernel) with a world of one rank: it
    pushes to its own buffer and must reproduce pa_decode_step bit for bit."""
    rng = np.random.default_rng(97)
    layers, lens = 2, [300, 17, 1]
    n = len(lens)
    cos, sin = orc.build_rope_tables(400)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    q = to_dev(orc.randn_bf16(rng, (layers, n, 32, 64)))
    k = to_dev(orc.randn_bf16(rng, (layers, n, 8, 64)))
    v = to_dev(orc.randn_bf16(rng, (layers, n, 8, 64)))
    outs = []
    for sharded in (False, True):
        prng = np.random.default_rng(98)
        pool = paged.KVPool(layers, 64, 8, n, 24)
        pool.set_free_order(prng.permutation(64))
        seqs = []
        for L in lens:
            s = pool.create_seq()
            pool.reserve(s, L)
            pool.batch_set([s], [L])
            for layer in range(layers):
                pool.append(layer, None, to_dev(orc.randn_bf16(prng, (L, 8, 64), 0.5)),
                            to_dev(orc.randn_bf16(prng, (L, 8, 64), 0.5)),
                            torch.ones(L, 32, device=DEV), torch.zeros(L, 32, device=DEV), None)
            seqs.append(s)
        for s, L in zip(seqs, lens):
            pool.reserve(s, L + 1)
        pool.batch_set(seqs)
        out = torch.zeros(layers, n, 2048, dtype=torch.bfloat16, device=DEV)
        q_rot = torch.zeros_like(q)
        if sharded:
            x = paged.Exchange(0, 0, 1, n, 8)
            paged.decode_step_sharded(pool, x, 0, layers, q, k, v, n * 2048, n * 512, cos_d, sin_d, q_rot, out,
                                      2048, n * 2048)
        else:
            pool.decode_step(0, layers, q, k, v, n * 2048, n * 512, cos_d, sin_d, q_rot, out, 2048, n * 2048)
        torch.cuda.synchronize()
        pool.check()
        outs.append((to_u16(out), to_u16(q_rot)))
        if sharded:
            x.close()
        pool.close()
    # the merge of a single partial renormalises through exp/log of the LSE: equal within bf16 rounding
    check_close(orc.bf16_to_f32(outs[1][0]), orc.bf16_to_f32(outs[0][0]), "sharded (1 rank) vs plain step")
    assert np.array_equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("world", [2, 4])
def test_head_sharded_step_gathers_full_rows(cuda, world):
    """KV heads sharded over `world` pools (ranks in this process, one GPU): each
    rank's decode kernels store its column slice into every rank's row buffer;
    after all ranks' steps every rank holds the full [layers, seqs, 2048] rows."""
    rng = np.random.default_rng(110 + world)
    layers, lens, steps = 2, [70, 300, 16], 2
    n = len(lens)
    kvh = 8 // world
    qh = 4 * kvh
    max_len = max(lens) + steps
    cos, sin = orc.build_rope_tables(max_len + 1)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    # full caches per layer and sequence (final, i.e. already rotated, values)
    K = [[orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for L in lens] for _ in range(layers)]
    V = [[orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for L in lens] for _ in range(layers)]
    pools, seqs = [], []
    for r in range(world):
        prng = np.random.default_rng(5)  # the same allocator decisions on every rank
        pool = paged.KVPool(layers, 80, kvh, n, 24)
        pool.set_free_order(prng.permutation(80))
        ids = []
        for i, L in enumerate(lens):
            s = pool.create_seq()
            pool.reserve(s, L)
            pool.batch_set([s], [L])
            for layer in range(layers):
                kk = K[layer][i][r * kvh:(r + 1) * kvh, :L].transpose(1, 0, 2)
                vv = V[layer][i][r * kvh:(r + 1) * kvh, :L].transpose(1, 0, 2)
                pool.append(layer, None, to_dev(kk), to_dev(vv), torch.ones(L, 32, device=DEV),
                            torch.zeros(L, 32, device=DEV), None)
            ids.append(s)
        pools.append(pool)
        seqs.append(ids)
    gs = [paged.HeadGather(0, r, world, n, layers, kvh) for r in range(world)]
    bufs = [g.buffer()[0] for g in gs]
    for g in gs:
        g.connect_ptrs(bufs)
    cur = list(lens)
    for step in range(steps):
        q = orc.randn_bf16(rng, (layers, n, 32, 64))
        k_new = orc.randn_bf16(rng, (layers, n, 8, 64))
        v_new = orc.randn_bf16(rng, (layers, n, 8, 64))
        keep = []
        for r in range(world):
            for s, L in zip(seqs[r], cur):
                pools[r].reserve(s, L + 1)
            pools[r].batch_set(seqs[r])
            qd = to_dev(q[:, :, r * qh:(r + 1) * qh])
            kd = to_dev(k_new[:, :, r * kvh:(r + 1) * kvh])
            vd = to_dev(v_new[:, :, r * kvh:(r + 1) * kvh])
            qr = torch.zeros_like(qd)
            keep.append((qd, kd, vd, qr))
            gs[r].step(pools[r], qd, kd, vd, n * qh * 64, n * kvh * 64, cos_d, sin_d, qr, wait=False)
        rows = []
        for r in range(world):  # all ranks have launched their stores: now each may wait
            ptr = gs[r].wait(pools[r])
            out = torch.empty(layers, n, 2048, dtype=torch.bfloat16, device=DEV)
            import ctypes
            cudart = ctypes.CDLL("libcudart.so.12")
            torch.cuda.synchronize()
            assert cudart.cudaMemcpy(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(ptr),
                                     ctypes.c_size_t(out.numel() * 2), 3) == 0
            rows.append(out)
        torch.cuda.synchronize()
        for pool in pools:
            pool.check()
        for layer in range(layers):
            for i in range(n):
                pos = cur[i]
                K[layer][i][:, pos] = orc.rope(k_new[layer, i][None], cos, sin, pos, 1)[:, 0]
                V[layer][i][:, pos] = v_new[layer, i]
                q_rot = orc.rope(q[layer, i][None], cos, sin, pos, 1)
                O, _ = orc.attention(q_rot, K[layer][i], V[layer][i], pos + 1)
                for r in range(world):
                    check_close(orc.bf16_to_f32(to_u16(rows[r][layer, i])), O[:, 0].reshape(-1),
                                f"step {step} layer {layer} seq {i} rank {r}")
        for r in range(1, world):
            assert torch.equal(rows[r], rows[0])
        cur = [c + 1 for c in cur]
    for g in gs:
        g.close()
    for pool in pools:
        pool.close()
