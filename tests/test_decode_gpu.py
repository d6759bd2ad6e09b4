"""GPU parity of K2 (paged split-KV GQA decode): against the fp32 oracle and the
reference's own kernel, tolerance max-abs 2e-2 / rel 1e-2 on bf16 outputs."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, check_close, f32_dev, fill_cache, to_dev, to_u16

pytestmark = pytest.mark.gpu


def oracle_decode(q, k, v, L):
    """q [32,64], k/v [8,>=L,64] -> fp32 [2048], lse [32]."""
    O, lse = orc.attention(q[:, None, :], k, v, L, causal=True)
    return O[:, 0].reshape(-1), lse[:, 0]


def gpu_decode(pool, seqs, q_rows, want_f32=False):
    n = len(seqs)
    qd = to_dev(q_rows)
    out = torch.zeros(n, pool.q_heads * 64, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(n, pool.q_heads, dtype=torch.float32, device=DEV)
    o32 = torch.zeros(n, pool.q_heads, 64, dtype=torch.float32, device=DEV) if want_f32 else None
    pool.batch_set(seqs)
    pool.decode(0, qd, out, None, o32, lse)
    torch.cuda.synchronize()
    pool.check()
    res = orc.bf16_to_f32(to_u16(out)), lse.cpu().numpy()
    return res + (o32.cpu().numpy(),) if want_f32 else res


def test_config1_ctx512_plus_one(cuda):
    """1 sequence, context 512 + 1 appended token, 33 blocks through a seeded
    random permutation table, RoPE theta 500000 on the new K and Q at position
    512, scale 1/8, against fp32 naive attention."""
    rng = np.random.default_rng(1)
    k = orc.randn_bf16(rng, (8, 513, 64), 0.5)
    v = orc.randn_bf16(rng, (8, 513, 64), 0.5)
    cos, sin = orc.build_rope_tables(513)
    q_new = orc.randn_bf16(rng, (1, 32, 64))
    k_new = orc.randn_bf16(rng, (1, 8, 64))
    v_new = orc.randn_bf16(rng, (1, 8, 64))
    pool = paged.KVPool(1, 40, 8, 1)
    pool.set_free_order(rng.permutation(40))
    s = pool.create_seq()
    fill_cache(pool, 0, s, k[:, :512], v[:, :512])
    pool.reserve(s, 513)
    assert pool.block_table(s).size == 33
    pool.batch_set([s])
    qd = to_dev(q_new)
    qo = torch.empty_like(qd)
    pool.append(0, qd, to_dev(k_new), to_dev(v_new), f32_dev(cos), f32_dev(sin), qo)
    out = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(1, 32, dtype=torch.float32, device=DEV)
    pool.decode(0, qo, out, 2048, None, lse, 0.125)
    torch.cuda.synchronize()
    pool.check()
    k[:, 512] = orc.rope(k_new, cos, sin, 512, 1)[:, 0]
    v[:, 512] = v_new[0]
    q_rot = orc.rope(q_new, cos, sin, 512, 1)[:, 0]
    want, want_lse = oracle_decode(q_rot, k, v, 513)
    check_close(orc.bf16_to_f32(to_u16(out))[0], want, "cfg1 out")
    assert np.max(np.abs(lse.cpu().numpy()[0] - want_lse)) < 1e-2
    pool.close()


@pytest.mark.parametrize("chunk_blocks", [0, 1, 3, 4, 7])
def test_every_length_residue(cuda, chunk_blocks):
    """Context 1..130 covers every length mod 16 and mod 64; chunk_blocks 1..7
    forces one-block chunks, chunks smaller than the warp count and ragged last
    chunks through the in-kernel combine."""
    rng = np.random.default_rng(2)
    lens = list(range(1, 131))
    n = len(lens)
    nb = sum((L + 15) // 16 for L in lens) + 7
    pool = paged.KVPool(1, nb, 8, n, 9)
    pool.set_free_order(rng.permutation(nb))
    pool.set_decode_chunk_blocks(chunk_blocks)
    ks, vs, seqs = [], [], []
    for L in lens:
        k = orc.randn_bf16(rng, (8, L, 64), 0.5)
        v = orc.randn_bf16(rng, (8, L, 64), 0.5)
        s = pool.create_seq()
        fill_cache(pool, 0, s, k, v)
        ks.append(k), vs.append(v), seqs.append(s)
    q = orc.randn_bf16(rng, (n, 32, 64))
    got, lse, o32 = gpu_decode(pool, seqs, q, want_f32=True)
    for i, L in enumerate(lens):
        want, want_lse = oracle_decode(q[i], ks[i], vs[i], L)
        check_close(got[i], want, f"len {L}")
        check_close(o32[i].reshape(-1), want, f"len {L} f32")
        assert np.max(np.abs(lse[i] - want_lse)) < 1e-2, L
    pool.close()


@pytest.mark.parametrize("kv_heads", [1, 2, 4])
def test_sharded_heads_write_their_columns(cuda, kv_heads):
    """A pool holding 8/n KV heads serves 32/n query heads and writes only its
    column slice of the [sequences, 2048] output."""
    rng = np.random.default_rng(3)
    lens = [70, 1, 333, 16]
    pool = paged.KVPool(1, 64, kv_heads, len(lens), 32)
    pool.set_free_order(rng.permutation(64))
    qh = 4 * kv_heads
    seqs, want = [], []
    q = orc.randn_bf16(rng, (len(lens), qh, 64))
    for i, L in enumerate(lens):
        k = orc.randn_bf16(rng, (kv_heads, L, 64), 0.5)
        v = orc.randn_bf16(rng, (kv_heads, L, 64), 0.5)
        s = pool.create_seq()
        fill_cache(pool, 0, s, k, v)
        seqs.append(s)
        O, _ = orc.attention(q[i][:, None, :], k, v, L)
        want.append(O[:, 0].reshape(-1))
    full = torch.full((len(lens), 2048), 7.0, dtype=torch.bfloat16, device=DEV)
    col0 = 2 * qh * 64 if kv_heads < 4 else 0  # some shard's column offset
    pool.batch_set(seqs)
    pool.decode(0, to_dev(q), full[:, col0:], 2048)
    torch.cuda.synchronize()
    pool.check()
    got = orc.bf16_to_f32(to_u16(full))
    for i in range(len(lens)):
        check_close(got[i, col0:col0 + qh * 64], want[i], f"row {i}")
    mask = np.ones(2048, bool)
    mask[col0:col0 + qh * 64] = False
    assert np.all(got[:, mask] == 7.0)
    pool.close()


def test_fragmented_pool_after_free_and_realloc(cuda):
    """Sequences freed and re-created between steps interleave their blocks;
    stale contents of recycled and never-used blocks must not leak in."""
    rng = np.random.default_rng(4)
    nb = 300
    pool = paged.KVPool(1, nb, 8, 8, 64)
    pool.set_free_order(rng.permutation(nb))
    live = {}
    for rnd in range(4):
        for s in list(live):
            if rng.random() < 0.5:
                pool.free_seq(s)
                del live[s]
        while len(live) < 6:
            L = int(rng.integers(1, 400))
            if (L + 15) // 16 > pool.free_blocks():
                break
            k = orc.randn_bf16(rng, (8, L, 64), 0.5)
            v = orc.randn_bf16(rng, (8, L, 64), 0.5)
            s = pool.create_seq()
            fill_cache(pool, 0, s, k, v)
            live[s] = (k, v, L)
        seqs = sorted(live)
        q = orc.randn_bf16(rng, (len(seqs), 32, 64))
        got, lse = gpu_decode(pool, seqs, q)
        for i, s in enumerate(seqs):
            k, v, L = live[s]
            want, want_lse = oracle_decode(q[i], k, v, L)
            check_close(got[i], want, f"round {rnd} seq {s} len {L}")
    pool.close()


def test_token_range_partials_merge_to_whole(cuda):
    """Split-KV across pools (as across GPUs): each pool holds one token range
    of the same sequence; normalised fp32 partials + LSE merge to the whole."""
    rng = np.random.default_rng(5)
    L = 1000
    k = orc.randn_bf16(rng, (8, L, 64), 0.5)
    v = orc.randn_bf16(rng, (8, L, 64), 0.5)
    q = orc.randn_bf16(rng, (1, 32, 64))
    cuts = [0, 256, 256, 640, L]  # one empty range
    parts_o = torch.zeros(4, 32, 64, dtype=torch.float32, device=DEV)
    parts_l = torch.zeros(4, 32, dtype=torch.float32, device=DEV)
    pools = []
    for i, (a, b) in enumerate(zip(cuts[:-1], cuts[1:])):
        pool = paged.KVPool(1, 64, 8, 1)
        pool.set_free_order(rng.permutation(64))
        s = pool.create_seq()
        if b > a:
            fill_cache(pool, 0, s, k[:, a:b], v[:, a:b])
        pool.batch_set([s], [0])
        pool.decode(0, to_dev(q), None, 0, parts_o[i], parts_l[i])
        pools.append(pool)
    torch.cuda.synchronize()
    assert torch.isneginf(parts_l[1]).all() and not parts_o[1].any()
    out = torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(32, dtype=torch.float32, device=DEV)
    paged.merge_partials(parts_o, parts_l, 4, 32, out, None, lse)
    torch.cuda.synchronize()
    want, want_lse = oracle_decode(q[0], k, v, L)
    check_close(orc.bf16_to_f32(to_u16(out)).reshape(-1), want, "merged")
    assert np.max(np.abs(lse.cpu().numpy() - want_lse)) < 1e-2
    Om, _ = orc.lse_merge(parts_o.cpu().numpy(), parts_l.cpu().numpy())
    check_close(orc.bf16_to_f32(to_u16(out)), Om, "merge kernel vs oracle merge")
    for p in pools:
        p.close()


@pytest.mark.skipif(not orc.ref_available(), reason="reference kernels were not built")
@pytest.mark.parametrize("L", [1, 63, 64, 513, 4097])
def test_decode_vs_reference_kernel(cuda, L):
    """The reference decodes with its prefill kernel at q_seq_len = 1 over the
    contiguous cache, then transposes the output."""
    rng = np.random.default_rng(6)
    ref = orc.ref()
    k = orc.randn_bf16(rng, (8, L, 64), 0.5)
    v = orc.randn_bf16(rng, (8, L, 64), 0.5)
    q = orc.randn_bf16(rng, (1, 32, 64))
    kc, vc = to_dev(k), to_dev(v)
    qd = to_dev(q[0][:, None, :])  # [32, 1, 64]
    o_flash = torch.zeros(32, 1, 64, dtype=torch.bfloat16, device=DEV)
    ref_lse = torch.zeros(32, 1, dtype=torch.float32, device=DEV)
    o_ref = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    ref.ref_flash_attention(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), o_flash.data_ptr(),
                            ref_lse.data_ptr(), 1, 32, 8, 1, L, L, 0.125, 1, None)
    ref.ref_flash_output_layout(o_flash.data_ptr(), o_ref.data_ptr(), 1)
    torch.cuda.synchronize()
    nb = (L + 15) // 16 + 5
    pool = paged.KVPool(1, nb, 8, 1)
    pool.set_free_order(rng.permutation(nb))
    s = pool.create_seq()
    fill_cache(pool, 0, s, k, v)
    got, lse = gpu_decode(pool, [s], q)
    want = orc.bf16_to_f32(to_u16(o_ref))[0]
    check_close(got[0], want, f"vs reference kernel, L={L}")
    assert np.max(np.abs(lse[0] - ref_lse.cpu().numpy()[:, 0])) < 1e-2
    oracle_o, _ = oracle_decode(q[0], k, v, L)
    check_close(want, oracle_o, "reference kernel vs oracle")
    pool.close()


@pytest.mark.parametrize("chunk_blocks", [0, 2, 5])
def test_fused_step_equals_append_then_decode(cuda, chunk_blocks):
    """pa_decode_step runs RoPE(Q), RoPE(K) + append and the decode in ONE kernel
    per layer; cache contents, rotated Q and outputs must equal the two-kernel
    path bit for bit (same arithmetic, same placement)."""
    from tests.gpu_helpers import read_logical_pool
    rng = np.random.default_rng(70 + chunk_blocks)
    lens = [47, 16, 130, 1, 255]  # new tokens land mid-block, at slot 0 of a fresh block, ...
    layers = 2
    cos, sin = orc.build_rope_tables(300)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    n = len(lens)
    q = to_dev(orc.randn_bf16(rng, (layers, n, 32, 64)))
    k = to_dev(orc.randn_bf16(rng, (layers, n, 8, 64)))
    v = to_dev(orc.randn_bf16(rng, (layers, n, 8, 64)))
    results = []
    for fused in (True, False):
        prng = np.random.default_rng(71)
        pool = paged.KVPool(layers, 64, 8, n, 20)
        pool.set_free_order(prng.permutation(64))
        pool.set_decode_chunk_blocks(chunk_blocks)
        pool.set_decode_cluster(-1)  # the step kernel has no cluster form: same chunking on both sides
        seqs = []
        for L in lens:
            s = pool.create_seq()
            for layer in range(layers):
                kk = orc.randn_bf16(prng, (8, L, 64), 0.5)
                vv = orc.randn_bf16(prng, (8, L, 64), 0.5)
                if layer == 0:
                    fill_cache(pool, 0, s, kk, vv)
                else:  # the same positions of the other layer
                    pool.batch_set([s], [L])
                    pool.append(layer, None, to_dev(kk.transpose(1, 0, 2)), to_dev(vv.transpose(1, 0, 2)),
                                torch.ones(L, 32, device=DEV), torch.zeros(L, 32, device=DEV), None)
            seqs.append(s)
        for s, L in zip(seqs, lens):
            pool.reserve(s, L + 1)
        pool.batch_set(seqs)
        out = torch.zeros(layers, n, 2048, dtype=torch.bfloat16, device=DEV)
        q_rot = torch.zeros_like(q)
        if fused:
            pool.decode_step(0, layers, q, k, v, n * 2048, n * 512, cos_d, sin_d, q_rot, out, 2048, n * 2048)
        else:
            for layer in range(layers):
                pool.append(layer, q[layer], k[layer], v[layer], cos_d, sin_d, q_rot[layer])
                pool.decode(layer, q_rot[layer], out[layer], 2048)
        torch.cuda.synchronize()
        pool.check()
        results.append((to_u16(out), to_u16(q_rot), [read_logical_pool(pool, l) for l in range(layers)]))
        pool.close()
    (of, qf, cf), (o2, q2, c2) = results
    assert np.array_equal(qf, q2)
    for l in range(layers):
        assert np.array_equal(cf[l], c2[l])
    assert np.array_equal(of, o2)


@pytest.mark.gpu
@pytest.mark.parametrize("chunk_blocks", [0, 5])
def test_step_kernel_equals_one_kernel_per_layer(cuda, chunk_blocks):
    """A decode step of several layers runs as ONE cooperative launch (streaming
    CTAs layer after layer, one combining CTA per (sequence, head)); outputs,
    rotated Q, LSE-free rows and cache contents must equal the one-kernel-per-layer
    path and the separate append + decode path bit for bit."""
    from tests.gpu_helpers import read_logical_pool
    rng = np.random.default_rng(170 + chunk_blocks)
    lens = [47, 130, 255]
    layers = 3
    cos, sin = orc.build_rope_tables(300)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    n = len(lens)
    q = to_dev(orc.randn_bf16(rng, (layers, n, 32, 64)))
    k = to_dev(orc.randn_bf16(rng, (layers, n, 8, 64)))
    v = to_dev(orc.randn_bf16(rng, (layers, n, 8, 64)))
    results = []
    for mode in ("step", "per_layer", "separate"):
        prng = np.random.default_rng(171)
        pool = paged.KVPool(layers, 64, 8, n, 20)
        pool.set_free_order(prng.permutation(64))
        pool.set_decode_chunk_blocks(chunk_blocks)
        pool.set_decode_cluster(-1)  # the step kernel has no cluster form: same chunking in all three modes
        pool.set_step_kernel(mode == "step")
        seqs = []
        for L in lens:
            s = pool.create_seq()
            for layer in range(layers):
                kk = orc.randn_bf16(prng, (8, L, 64), 0.5)
                vv = orc.randn_bf16(prng, (8, L, 64), 0.5)
                if layer == 0:
                    fill_cache(pool, 0, s, kk, vv)
                else:
                    pool.batch_set([s], [L])
                    pool.append(layer, None, to_dev(kk.transpose(1, 0, 2)), to_dev(vv.transpose(1, 0, 2)),
                                torch.ones(L, 32, device=DEV), torch.zeros(L, 32, device=DEV), None)
            seqs.append(s)
        outs = []
        for step in range(2):  # two steps in a row: counters and rings start clean each launch
            for s, L in zip(seqs, lens):
                pool.reserve(s, L + 1 + step)
            pool.batch_set(seqs)
            out = torch.zeros(layers, n, 2048, dtype=torch.bfloat16, device=DEV)
            q_rot = torch.zeros_like(q)
            if mode == "separate":
                for layer in range(layers):
                    pool.append(layer, q[layer], k[layer], v[layer], cos_d, sin_d, q_rot[layer])
                    pool.decode(layer, q_rot[layer], out[layer], 2048)
            else:
                pool.decode_step(0, layers, q, k, v, n * 2048, n * 512, cos_d, sin_d, q_rot, out, 2048, n * 2048)
            torch.cuda.synchronize()
            pool.check()
            outs.append((to_u16(out), to_u16(q_rot)))
        assert pool.step_launches() == (2 if mode == "step" else 0)
        results.append((outs, [read_logical_pool(pool, l) for l in range(layers)]))
        pool.close()
    (o_a, c_a), (o_b, c_b), (o_c, c_c) = results
    for step in range(2):
        for other in (o_b, o_c):
            assert np.array_equal(o_a[step][0], other[step][0])
            assert np.array_equal(o_a[step][1], other[step][1])
    for l in range(layers):
        assert np.array_equal(c_a[l], c_b[l]) and np.array_equal(c_a[l], c_c[l])


@pytest.mark.parametrize("mode,lens", [(0, [4097]), (16, [4097]), (8, [513, 2000]), (4, [70, 1000, 64]), (2, [33, 300, 17, 129]),
                                       (0, [300, 1200]), (16, [16])])
def test_cluster_form_of_the_one_layer_kernel(cuda, mode, lens):
    """The chunks of a (sequence, head) as one thread-block cluster that combines through distributed
    shared memory (mode 0: the planner's choice; 2..16: that cluster size, with CTAs beyond a short
    sequence's own chunk count idling).  Against the oracle, and against the workspace form of the
    same pool within one bf16 rounding of the row scale (the chunking differs, so not bit for bit)."""
    rng = np.random.default_rng(400 + mode + len(lens))
    n = len(lens)
    nb = sum((L + 15) // 16 for L in lens) + 5
    pool = paged.KVPool(1, nb, 8, n, max((L + 15) // 16 for L in lens) + 1)
    pool.set_free_order(rng.permutation(nb))
    ks, vs, seqs = [], [], []
    for L in lens:
        k = orc.randn_bf16(rng, (8, L, 64), 0.5)
        v = orc.randn_bf16(rng, (8, L, 64), 0.5)
        s = pool.create_seq()
        fill_cache(pool, 0, s, k, v)
        ks.append(k), vs.append(v), seqs.append(s)
    q = orc.randn_bf16(rng, (n, 32, 64))
    pool.set_decode_cluster(mode)
    got, lse, o32 = gpu_decode(pool, seqs, q, want_f32=True)
    got2, _, _ = gpu_decode(pool, seqs, q, want_f32=True)  # a second launch: nothing left behind by the first
    assert np.array_equal(got, got2)
    pool.set_decode_cluster(-1)
    ws, ws_lse, _ = gpu_decode(pool, seqs, q, want_f32=True)
    for i, L in enumerate(lens):
        want, want_lse = oracle_decode(q[i], ks[i], vs[i], L)
        check_close(got[i], want, f"len {L}")
        check_close(o32[i].reshape(-1), want, f"len {L} f32")
        assert np.max(np.abs(lse[i] - want_lse)) < 1e-2, L
        check_close(got[i], ws[i], f"len {L} vs the workspace form")
    pool.close()


def test_cluster_form_with_the_fused_append(cuda):
    """pa_decode_step of one layer (RoPE + append fused in) in the cluster form, against append + decode."""
    rng = np.random.default_rng(431)
    lens = [1000, 257]
    n = len(lens)
    cos, sin = orc.build_rope_tables(1100)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    q = to_dev(orc.randn_bf16(rng, (1, n, 32, 64)))
    k = to_dev(orc.randn_bf16(rng, (1, n, 8, 64)))
    v = to_dev(orc.randn_bf16(rng, (1, n, 8, 64)))
    outs = []
    for fused in (True, False):
        prng = np.random.default_rng(432)
        pool = paged.KVPool(1, 100, 8, n, 70)
        pool.set_free_order(prng.permutation(100))
        pool.set_decode_cluster(8)
        seqs = []
        for L in lens:
            s = pool.create_seq()
            fill_cache(pool, 0, s, orc.randn_bf16(prng, (8, L, 64), 0.5), orc.randn_bf16(prng, (8, L, 64), 0.5))
            seqs.append(s)
        for s, L in zip(seqs, lens):
            pool.reserve(s, L + 1)
        pool.batch_set(seqs)
        out = torch.zeros(1, n, 2048, dtype=torch.bfloat16, device=DEV)
        q_rot = torch.zeros_like(q)
        if fused:
            pool.decode_step(0, 1, q, k, v, n * 2048, n * 512, cos_d, sin_d, q_rot, out, 2048, n * 2048)
        else:
            pool.append(0, q[0], k[0], v[0], cos_d, sin_d, q_rot[0])
            pool.decode(0, q_rot[0], out[0], 2048)
        torch.cuda.synchronize()
        pool.check()
        outs.append((to_u16(out), to_u16(q_rot)))
        pool.close()
    assert np.array_equal(outs[0][1], outs[1][1])
    assert np.array_equal(outs[0][0], outs[1][0])  # same cluster size, same chunking: bit for bit
