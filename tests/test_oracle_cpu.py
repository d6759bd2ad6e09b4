"""CPU checks of the oracle itself: each restated function against an
independent float64 numpy statement of the same definition, plus the golden
vectors made by the reference's own kernels (tests/golden/)."""
import glob
import os

import numpy as np
import pytest

from oracle import oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_bf16_roundtrip_and_rounding():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(4096).astype(np.float32)
    b = orc.f32_to_bf16(x)
    for i in range(0, 4096, 97):
        assert int(b[i]) == int(orc.lib().orc_f32_to_bf16(float(x[i])))
    assert np.array_equal(orc.f32_to_bf16(orc.bf16_to_f32(b)), b)
    # ties to even: 1 + 2^-8 is exactly between two bf16 values
    assert orc.f32_to_bf16(np.array([1.0 + 2.0 ** -8], np.float32))[0] == 0x3F80
    assert orc.f32_to_bf16(np.array([1.0 + 3 * 2.0 ** -8], np.float32))[0] == 0x3F82


def test_rope_tables_match_definition():
    cos, sin = orc.build_rope_tables(300)
    pair = np.arange(32)
    inv = (1.0 / np.power(np.float32(500000.0), (2 * pair).astype(np.float32) / np.float32(64))).astype(np.float32)
    wl = (np.float32(2.0) * np.float32(np.pi) / inv).astype(np.float32)
    smooth = (np.float32(8192.0) / wl - 1.0) / 3.0
    scaled = np.where(wl < 2048, inv, np.where(wl <= 8192, (1 - smooth) * inv / 32 + smooth * inv, inv / 32))
    ang = np.arange(300)[:, None].astype(np.float64) * scaled[None, :].astype(np.float64)
    assert np.allclose(cos, np.cos(ang), atol=2e-4)
    assert np.allclose(sin, np.sin(ang), atol=2e-4)
    assert cos.dtype == np.float32 and cos.shape == (300, 32)
    # position 0 is the identity rotation
    assert np.all(cos[0] == 1.0) and np.all(sin[0] == 0.0)


@pytest.mark.parametrize("variant", [0, 1, 2])
def test_rope_half_split_pairs(variant):
    rng = np.random.default_rng(1)
    tokens, heads, off = 5, 3, 7
    x = orc.randn_bf16(rng, (tokens, heads, 64))
    cos, sin = orc.build_rope_tables(off + tokens)
    y = orc.rope(x, cos, sin, off, variant)
    assert y.shape == (heads, tokens, 64)
    xf = orc.bf16_to_f32(x).astype(np.float64)
    c = cos[off:off + tokens].astype(np.float64)[:, None, :]
    s = sin[off:off + tokens].astype(np.float64)[:, None, :]
    y0 = xf[..., :32] * c - xf[..., 32:] * s
    y1 = xf[..., :32] * s + xf[..., 32:] * c
    want = np.concatenate([y0, y1], -1).transpose(1, 0, 2)
    got = orc.bf16_to_f32(y).astype(np.float64)
    assert np.max(np.abs(got - want)) <= 2.0 ** -8 * np.max(np.abs(want)) + 1e-6
    # the three roundings of y0 differ by at most one bf16 step, y1 is identical
    y_tm = orc.rope(x, cos, sin, off, variant, out_token_major=True)
    assert np.array_equal(y_tm.transpose(1, 0, 2), y)


def test_transpose_append_layout():
    rng = np.random.default_rng(2)
    v = orc.randn_bf16(rng, (6, 8, 64))
    vt = orc.transpose_v(v)
    assert np.array_equal(vt, v.transpose(1, 0, 2))
    cache = np.zeros((8, 40, 64), np.uint16)
    orc.append_contig(cache, vt, 9)
    assert np.array_equal(cache[:, 9:15], vt)
    assert not cache[:, :9].any() and not cache[:, 15:].any()
    o = orc.randn_bf16(rng, (32, 6, 64))
    assert np.array_equal(orc.output_layout(o), o.transpose(1, 0, 2).reshape(6, 2048))


def test_paged_placement_equals_contiguous():
    rng = np.random.default_rng(3)
    nb, heads, L = 12, 8, 70
    table = rng.permutation(nb)[: (L + 15) // 16].astype(np.int32)
    pool = np.zeros((nb, heads, 2, 16, 64), np.uint16)
    kc = np.zeros((heads, L, 64), np.uint16)
    vc = np.zeros((heads, L, 64), np.uint16)
    pos = 0
    for tok in (33, 1, 1, 35):  # ragged appends crossing block borders
        k = orc.randn_bf16(rng, (heads, tok, 64))
        v = orc.randn_bf16(rng, (heads, tok, 64))
        orc.paged_append(pool, table, k, v, pos)
        orc.append_contig(kc, k, pos)
        orc.append_contig(vc, v, pos)
        pos += tok
    gk, gv = orc.paged_gather(pool, table, L)
    assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
    for p in (0, 15, 16, 69):
        assert np.array_equal(pool[table[p // 16], :, 0, p % 16], kc[:, p])


def _attention_f64(Q, K, V, kv_len, causal, scale=0.125):
    q = orc.bf16_to_f32(Q).astype(np.float64)
    k = orc.bf16_to_f32(K).astype(np.float64)[:, :kv_len]
    v = orc.bf16_to_f32(V).astype(np.float64)[:, :kv_len]
    hq, sq, _ = q.shape
    g = hq // k.shape[0]
    O = np.zeros((hq, sq, 64))
    L = np.zeros((hq, sq))
    for h in range(hq):
        s = q[h] @ k[h // g].T * scale
        if causal:
            i = np.arange(sq)[:, None]
            j = np.arange(kv_len)[None, :]
            s = np.where(j <= i + (kv_len - sq), s, -np.inf)
        m = s.max(-1, keepdims=True)
        p = np.exp(s - m)
        O[h] = p @ v[h // g] / p.sum(-1, keepdims=True)
        L[h] = (m + np.log(p.sum(-1, keepdims=True)))[:, 0]
    return O, L


@pytest.mark.parametrize("sq,kv,causal", [(1, 513, True), (17, 17, True), (40, 100, True), (9, 33, False)])
def test_attention_matches_float64(sq, kv, causal):
    rng = np.random.default_rng(4)
    Q = orc.randn_bf16(rng, (32, sq, 64))
    K = orc.randn_bf16(rng, (8, kv + 3, 64), 0.5)
    V = orc.randn_bf16(rng, (8, kv + 3, 64), 0.5)
    O, L = orc.attention(Q, K, V, kv, causal=causal)
    Ow, Lw = _attention_f64(Q, K, V, kv, causal)
    assert np.max(np.abs(O - Ow)) < 2e-5
    assert np.max(np.abs(L - Lw)) < 2e-5
    Or, _ = orc.attention(Q, K, V, kv, causal=causal, round_p_bf16=True)
    assert np.max(np.abs(Or - Ow)) < 5e-3  # bf16 probabilities: the reference's P*V rounding


def test_long_decode_is_chunked_consistently():
    rng = np.random.default_rng(5)
    kv = 9000  # more than one internal chunk
    Q = orc.randn_bf16(rng, (32, 1, 64))
    K = orc.randn_bf16(rng, (8, kv, 64), 0.5)
    V = orc.randn_bf16(rng, (8, kv, 64), 0.5)
    O, L = orc.attention(Q, K, V, kv)
    Ow, Lw = _attention_f64(Q, K, V, kv, True)
    assert np.max(np.abs(O - Ow)) < 2e-5 and np.max(np.abs(L - Lw)) < 2e-5


def test_decode_paged_and_lse_merge():
    rng = np.random.default_rng(6)
    nb, L = 40, 513
    table = rng.permutation(nb)[:33].astype(np.int32)
    pool = np.zeros((nb, 8, 2, 16, 64), np.uint16)
    k = orc.randn_bf16(rng, (8, L, 64), 0.5)
    v = orc.randn_bf16(rng, (8, L, 64), 0.5)
    orc.paged_append(pool, table, k, v, 0)
    q = orc.randn_bf16(rng, (32, 64))
    full, lse = orc.decode_paged(q, pool, table, 0, L)
    Ow, Lw = orc.attention(q[:, None, :], k, v, L)
    assert np.max(np.abs(full - Ow[:, 0])) < 1e-5 and np.max(np.abs(lse - Lw[:, 0])) < 1e-5
    # merge of disjoint ranges (one of them empty) reproduces the whole
    cuts = [0, 100, 100, 257, L]
    parts = [orc.decode_paged(q, pool, table, a, b) for a, b in zip(cuts[:-1], cuts[1:])]
    Om, lm = orc.lse_merge(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]))
    assert np.isneginf(parts[1][1]).all()
    assert np.max(np.abs(Om - full)) < 1e-5 and np.max(np.abs(lm - lse)) < 1e-5


def test_block_pool_model_is_lifo_and_all_or_nothing():
    m = orc.BlockPoolModel(6, [3, 1, 4, 0, 5, 2])
    a = m.create()
    assert m.reserve(a, 17) and m.tables[a] == [3, 1]
    b = m.create()
    assert m.reserve(b, 16 * 3) and m.tables[b] == [4, 0, 5]
    assert not m.reserve(a, 16 * 4) and m.tables[a] == [3, 1] and m.lens[a] == 17
    m.release(b)
    assert m.reserve(a, 33) and m.tables[a] == [3, 1, 4]  # first block of the freed table comes back first
    assert m.create() == b


@pytest.mark.skipif(not glob.glob(os.path.join(GOLDEN, "*.npz")), reason="no golden fixtures yet")
def test_golden_vectors_from_reference_kernels():
    """Fixtures hold inputs and the outputs of the reference's own CUDA kernels
    (made by tests/golden/make_golden.py on a B200)."""
    for path in sorted(glob.glob(os.path.join(GOLDEN, "*.npz"))):
        g = np.load(path)
        if "y0_variant" not in g.files:
            continue  # the element-wise fixture has its own test
        variant = int(g["y0_variant"])
        pos, tokens, max_seq = int(g["position"]), int(g["tokens"]), int(g["max_seq"])
        cos, sin = orc.build_rope_tables(max_seq)
        assert np.array_equal(cos, g["cos"]) and np.array_equal(sin, g["sin"]), path
        qf = orc.rope(g["q_in"], cos, sin, pos, variant)
        kf = orc.rope(g["k_in"], cos, sin, pos, variant)
        vf = orc.transpose_v(g["v_in"])
        assert np.array_equal(qf, g["q_flash"]), path
        assert np.array_equal(kf, g["k_flash"]), path
        assert np.array_equal(vf, g["v_flash"]), path
        kc = g["k_cache_before"].copy()
        vc = g["v_cache_before"].copy()
        orc.append_contig(kc, kf, pos)
        orc.append_contig(vc, vf, pos)
        assert np.array_equal(kc, g["k_cache_after"]) and np.array_equal(vc, g["v_cache_after"]), path
        O, L = orc.attention(qf, kc, vc, pos + tokens, causal=True)
        ref_o = orc.bf16_to_f32(g["o_flash"])
        err = np.abs(ref_o - O)
        assert np.all(err <= 2e-2 + 1e-2 * np.abs(O)), (path, err.max())
        assert np.max(np.abs(g["lse"] - L)) < 2e-2, path
        assert np.array_equal(orc.output_layout(g["o_flash"]), g["o_layout"]), path


def test_gemm_restatement_against_numpy():
    """orc_gemm_bf16 (the projection GEMMs' contract) against float64 numpy, rounded once."""
    rng = np.random.default_rng(77)
    a = orc.randn_bf16(rng, (3, 256))
    b = orc.randn_bf16(rng, (256, 96), 0.05)
    got = orc.gemm_bf16(a, b)
    ref = orc.bf16_to_f32(a).astype(np.float64) @ orc.bf16_to_f32(b).astype(np.float64)
    want = orc.f32_to_bf16(ref.astype(np.float32))
    # float64 -> float32 -> bf16 can differ from the oracle's path only by double rounding: none here
    assert np.array_equal(got, want)


@pytest.mark.skipif(not os.path.exists(os.path.join(GOLDEN, "elementwise_rmsnorm_silu.npz")), reason="fixture not made yet")
def test_golden_rmsnorm_and_silu_mul_from_reference_kernels():
    """RMSNorm: the oracle restates the reference kernel's summation order, so the bits are equal.
    SiLU(gate) * up: the device evaluates exp with __expf, the oracle with expf; equal to within one
    bf16 unit everywhere, bit-equal almost everywhere."""
    g = np.load(os.path.join(GOLDEN, "elementwise_rmsnorm_silu.npz"))
    assert np.array_equal(orc.rmsnorm(g["x"], g["norm_w"], 1e-5), g["rmsnorm_out"])
    got = orc.silu_mul(g["gate"], g["up"])
    a = orc.bf16_to_f32(got).astype(np.float64)
    b = orc.bf16_to_f32(g["silu_mul_out"]).astype(np.float64)
    assert np.all(np.abs(a - b) <= np.maximum(np.abs(a), np.abs(b)) * 2.0 ** -7 + 1e-30)
    assert float((got == g["silu_mul_out"]).mean()) > 0.99


def test_silu_mul_and_ffn_restatement_against_numpy():
    rng = np.random.default_rng(78)
    gate = orc.randn_bf16(rng, (2, 512), 2.0)
    up = orc.randn_bf16(rng, (2, 512), 1.0)
    gf, uf = orc.bf16_to_f32(gate).astype(np.float64), orc.bf16_to_f32(up).astype(np.float64)
    want = gf / (1.0 + np.exp(-gf)) * uf
    got = orc.bf16_to_f32(orc.silu_mul(gate, up)).astype(np.float64)
    assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -7 + 1e-30)
    # the block: RMSNorm -> gate/up GEMMs -> SiLU * up -> down GEMM -> residual, piece by piece
    x = orc.randn_bf16(rng, (2, 128), 1.0)
    nw = orc.randn_bf16(rng, (128,), 0.7)
    wg = orc.randn_bf16(rng, (128, 256), 0.1)
    wu = orc.randn_bf16(rng, (128, 256), 0.1)
    wd = orc.randn_bf16(rng, (256, 128), 0.1)
    xn = orc.rmsnorm(x, nw, 1e-5)
    h = orc.silu_mul(orc.gemm_bf16(xn, wg), orc.gemm_bf16(xn, wu))
    y = orc.gemm_bf16(h, wd)
    assert np.array_equal(orc.ffn(x, nw, wg, wu, wd, 1e-5, False), y)
    assert np.array_equal(orc.ffn(x, nw, wg, wu, wd, 1e-5, True), orc.f32_to_bf16(orc.bf16_to_f32(x) + orc.bf16_to_f32(y)))


def test_argmax_rule_of_the_reference_kernel():
    """A host model of the reference's argmax kernel (256 threads, strided scan with a strict ">",
    shuffle-down reductions that keep the lower lane on ties) against the closed-form rule."""
    rng = np.random.default_rng(79)

    def kernel_model(v):
        best_v = np.full(256, -np.inf, np.float32)
        best_i = np.full(256, -1, np.int64)
        for t in range(256):
            idx = np.arange(t, v.size, 256)
            j = int(np.argmax(v[idx]))  # first occurrence of the largest: the strict ">" scan
            best_v[t], best_i[t] = v[idx][j], idx[j]
        def warp_reduce(vals, idxs):
            vals, idxs = vals.copy(), idxs.copy()
            for off in (16, 8, 4, 2, 1):
                for lane in range(32 - off):  # lanes past the end read themselves: no change
                    if vals[lane + off] > vals[lane]:
                        vals[lane], idxs[lane] = vals[lane + off], idxs[lane + off]
            return vals[0], idxs[0]
        wv, wi = zip(*(warp_reduce(best_v[32 * w:32 * w + 32], best_i[32 * w:32 * w + 32]) for w in range(8)))
        pv = np.full(32, -np.inf, np.float32)
        pi = np.full(32, -1, np.int64)
        pv[:8], pi[:8] = wv, wi
        return warp_reduce(pv, pi)[1]

    for trial in range(20):
        n = 128256 if trial < 2 else 3000
        lg = orc.randn_bf16(rng, (1, n), 1.0)
        ties = rng.choice(n, size=rng.integers(1, 5), replace=False)
        lg[0, ties] = orc.f32_to_bf16(np.array([60.0], np.float32))[0]
        assert orc.argmax_reference_rule(lg)[0] == kernel_model(orc.bf16_to_f32(lg[0]))
