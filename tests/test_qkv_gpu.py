"""GPU parity of the decode-shape Q/K/V projection (pa_qkv_project) against the
CPU oracle (double accumulation, one rounding) and the reference's own GEMM
kernels (gemm_2048x2048.cu, gemm_2048x512.cu as Attention::forward calls them)."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import _lib, paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, to_dev, to_u16

pytestmark = pytest.mark.gpu


def bf16_close(got_u16, want_u16, what):
    """Equal up to one bf16 ulp (2^-8 relative) plus the rounding of sums that cancel."""
    g = orc.bf16_to_f32(got_u16).astype(np.float64)
    w = orc.bf16_to_f32(want_u16).astype(np.float64)
    tol = np.abs(w) * 2.0 ** -7 + 0.02
    bad = np.abs(g - w) > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} differ, worst {np.abs(g - w).max()}"
    exact = float((got_u16 == want_u16).mean())
    assert exact > 0.9, f"{what}: only {exact:.3f} of the values are bit-equal"


@pytest.mark.parametrize("rows,layers", [(1, 1), (1, 3), (2, 2), (3, 1), (8, 2)])
def test_qkv_project_vs_oracle(cuda, rows, layers):
    rng = np.random.default_rng(500 + rows * 10 + layers)
    x = orc.randn_bf16(rng, (layers, rows, 2048))
    wq = orc.randn_bf16(rng, (layers, 2048, 2048), 0.03)
    wk = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
    wv = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
    q = torch.full((layers, rows, 2048), 7.0, dtype=torch.bfloat16, device=DEV)
    k = torch.full((layers, rows, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    v = torch.full((layers, rows, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    xd, wqd, wkd, wvd = to_dev(x), to_dev(wq), to_dev(wk), to_dev(wv)
    paged.qkv_project(xd, wqd, wkd, wvd, q, k, v, rows, layers)
    torch.cuda.synchronize()
    for l in range(layers):
        bf16_close(to_u16(q[l]), orc.gemm_bf16(x[l], wq[l]), f"q layer {l}")
        bf16_close(to_u16(k[l]), orc.gemm_bf16(x[l], wk[l]), f"k layer {l}")
        bf16_close(to_u16(v[l]), orc.gemm_bf16(x[l], wv[l]), f"v layer {l}")


@pytest.mark.parametrize("hidden,rows", [(64, 1), (192, 3), (1088, 8), (1984, 2)])
def test_qkv_project_hidden_sizes_that_end_inside_a_step(cuda, hidden, rows):
    """The kernel walks the weight rows in steps of 128; a hidden size that is a multiple of 64 but not of
    128 (or shorter than a step) ends inside one: the tile rows past the end must count as zeros, whatever
    the memory behind the matrix holds (here: NaN patterns)."""
    rng = np.random.default_rng(520 + hidden + rows)
    x = orc.randn_bf16(rng, (1, rows, hidden))
    n_q, n_kv = 256, 64
    # each matrix sits in front of a guard filled with NaNs: rows past the end would read it
    def guarded(n):
        buf = np.full((hidden + 128, n), 0x7FC0, np.uint16)
        buf[:hidden] = orc.randn_bf16(rng, (hidden, n), 0.05)
        return buf
    wq, wk, wv = guarded(n_q), guarded(n_kv), guarded(n_kv)
    q = torch.full((1, rows, n_q), 7.0, dtype=torch.bfloat16, device=DEV)
    k = torch.full((1, rows, n_kv), 7.0, dtype=torch.bfloat16, device=DEV)
    v = torch.full((1, rows, n_kv), 7.0, dtype=torch.bfloat16, device=DEV)
    wqd, wkd, wvd = to_dev(wq), to_dev(wk), to_dev(wv)
    paged.qkv_project(to_dev(x), wqd[:hidden].unsqueeze(0), wkd[:hidden].unsqueeze(0), wvd[:hidden].unsqueeze(0), q, k, v,
                      rows, 1, hidden=hidden)
    torch.cuda.synchronize()
    bf16_close(to_u16(q[0]), orc.gemm_bf16(x[0], wq[:hidden]), "q")
    bf16_close(to_u16(k[0]), orc.gemm_bf16(x[0], wk[:hidden]), "k")
    bf16_close(to_u16(v[0]), orc.gemm_bf16(x[0], wv[:hidden]), "v")


@pytest.mark.parametrize("rows,layers", [(1, 2), (3, 1), (8, 2)])
def test_qkv_project_packed_equals_row_major(cuda, rows, layers):
    """The packed-weight kernel adds the same products in a different order: compare with the
    oracle like the row-major kernel, and require near-complete bit agreement between the two."""
    rng = np.random.default_rng(520 + rows + layers)
    x = orc.randn_bf16(rng, (layers, rows, 2048))
    wq = orc.randn_bf16(rng, (layers, 2048, 2048), 0.03)
    wk = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
    wv = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
    xd, wqd, wkd, wvd = to_dev(x), to_dev(wq), to_dev(wk), to_dev(wv)
    outs = []
    for packed in (False, True):
        q = torch.full((layers, rows, 2048), 7.0, dtype=torch.bfloat16, device=DEV)
        k = torch.full((layers, rows, 512), 7.0, dtype=torch.bfloat16, device=DEV)
        v = torch.full((layers, rows, 512), 7.0, dtype=torch.bfloat16, device=DEV)
        if packed:
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            pq, pk, pv = (paged.pack_projection_weights(w) for w in (wqd, wkd, wvd))
            paged.qkv_project_packed(xd, pq, pk, pv, q, k, v, rows, status, layers)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
        else:
            paged.qkv_project(xd, wqd, wkd, wvd, q, k, v, rows, layers)
            torch.cuda.synchronize()
        outs.append((to_u16(q), to_u16(k), to_u16(v)))
    for l in range(layers):
        bf16_close(outs[1][0][l], orc.gemm_bf16(x[l], wq[l]), f"packed q layer {l}")
        bf16_close(outs[1][1][l], orc.gemm_bf16(x[l], wk[l]), f"packed k layer {l}")
        bf16_close(outs[1][2][l], orc.gemm_bf16(x[l], wv[l]), f"packed v layer {l}")
    for a_, b_ in zip(outs[0], outs[1]):
        assert float((a_ == b_).mean()) > 0.9


@pytest.mark.skipif(not orc.ref_available(), reason="reference kernels were not built")
@pytest.mark.parametrize("rows", [1, 4])
def test_qkv_project_vs_reference_gemm(cuda, rows):
    rng = np.random.default_rng(540 + rows)
    x = to_dev(orc.randn_bf16(rng, (1, rows, 2048)))
    wq = to_dev(orc.randn_bf16(rng, (1, 2048, 2048), 0.03))
    wk = to_dev(orc.randn_bf16(rng, (1, 2048, 512), 0.03))
    wv = to_dev(orc.randn_bf16(rng, (1, 2048, 512), 0.03))
    q = torch.zeros(1, rows, 2048, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(1, rows, 512, dtype=torch.bfloat16, device=DEV)
    v = torch.zeros(1, rows, 512, dtype=torch.bfloat16, device=DEV)
    paged.qkv_project(x, wq, wk, wv, q, k, v, rows, 1)
    r = orc.ref()
    for w, got, n in ((wq, q, 2048), (wk, k, 512), (wv, v, 512)):
        want = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
        assert r.ref_gemm(x.data_ptr(), w.data_ptr(), want.data_ptr(), rows, n, 2048) == 0
        torch.cuda.synchronize()
        bf16_close(to_u16(got[0]), to_u16(want), f"N={n} rows={rows} against the reference GEMM")


def test_qkv_project_rejects_prefill_shapes(cuda):
    from llama_transformer_runtime_b200._lib import PagedAttentionError
    t = torch.zeros(1, 9, 2048, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(1, 2048, 2048, dtype=torch.bfloat16, device=DEV)
    wk = torch.zeros(1, 2048, 512, dtype=torch.bfloat16, device=DEV)
    o = torch.zeros(1, 9, 2048, dtype=torch.bfloat16, device=DEV)
    ok = torch.zeros(1, 9, 512, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(PagedAttentionError):
        paged.qkv_project(t, w, wk, wk, o, ok, ok, 9, 1)


def _project_append_case(rng, position, tokens):
    """Cache holds `position` tokens; `tokens` new rows are projected, rotated and appended by ONE
    tcgen05 GEMM launch.  Returns GPU results and the oracle chain (GEMM -> bf16 -> RoPE -> placement)."""
    from tests.gpu_helpers import f32_dev, fill_cache
    L = position + tokens
    cos, sin = orc.build_rope_tables(L)
    nb = (L + 15) // 16 + 4
    pool = paged.KVPool(1, nb, 8, 1)
    pool.set_free_order(rng.permutation(nb))
    s = pool.create_seq()
    k_old = orc.randn_bf16(rng, (8, position, 64), 0.5)
    v_old = orc.randn_bf16(rng, (8, position, 64), 0.5)
    if position:
        fill_cache(pool, 0, s, k_old, v_old)
    x = orc.randn_bf16(rng, (tokens, 2048))
    wq = orc.randn_bf16(rng, (2048, 2048), 0.03)
    wk = orc.randn_bf16(rng, (2048, 512), 0.03)
    wv = orc.randn_bf16(rng, (2048, 512), 0.03)
    pool.reserve(s, L)
    pool.batch_set([s], [tokens])
    q_out = torch.full((tokens, 2048), 3.0, dtype=torch.bfloat16, device=DEV)
    pq, pk, pv = (paged.pack_projection_weights(to_dev(w)) for w in (wq, wk, wv))
    pool.qkv_project_append(0, to_dev(x), pq, pk, pv, f32_dev(cos), f32_dev(sin), q_out)
    torch.cuda.synchronize()
    pool.check()
    gk = torch.zeros(8, L, 64, dtype=torch.bfloat16, device=DEV)
    gv = torch.zeros_like(gk)
    pool.gather_kv(0, s, gk, gv, L)
    torch.cuda.synchronize()
    got = (to_u16(q_out), to_u16(gk), to_u16(gv))
    pool.close()
    # oracle chain
    q_lin = orc.gemm_bf16(x, wq).reshape(tokens, 32, 64)
    k_lin = orc.gemm_bf16(x, wk).reshape(tokens, 8, 64)
    v_lin = orc.gemm_bf16(x, wv).reshape(tokens, 8, 64)
    q_want = orc.rope(q_lin, cos, sin, position, 1, out_token_major=True).reshape(tokens, 2048)
    k_want = np.concatenate([k_old, orc.rope(k_lin, cos, sin, position, 1)], 1)
    v_want = np.concatenate([v_old, orc.transpose_v(v_lin)], 1)
    return got, (q_want, k_want, v_want), (x, wq, wk, wv, cos, sin)


def rotated_close(got_u16, want_u16, what):
    """RoPE mixes two GEMM outputs, each within one bf16 ulp of the oracle's: allow two ulps of
    the larger partner (bounded by 2^-6 of 4 sigma here) and ask that most values are bit-equal."""
    g = orc.bf16_to_f32(got_u16).astype(np.float64)
    w = orc.bf16_to_f32(want_u16).astype(np.float64)
    tol = np.abs(w) * 2.0 ** -6 + 0.05
    bad = np.abs(g - w) > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} differ, worst {np.abs(g - w).max()}"
    assert float((got_u16 == want_u16).mean()) > 0.85, f"{what}: too few bit-equal values"


@pytest.mark.parametrize("position,tokens", [(0, 128), (0, 37), (45, 200), (16, 300)])
def test_qkv_project_append_vs_oracle_chain(cuda, position, tokens):
    rng = np.random.default_rng(600 + position + tokens)
    (q, k, v), (qw, kw, vw), _ = _project_append_case(rng, position, tokens)
    # tokens that were already in the cache are untouched, bit for bit
    assert np.array_equal(k[:, :position], kw[:, :position]) and np.array_equal(v[:, :position], vw[:, :position])
    rotated_close(q, qw, "rotated Q")
    rotated_close(k[:, position:], kw[:, position:], "rotated K in the cache")
    bf16_close(v[:, position:], vw[:, position:], "V in the cache")


@pytest.mark.skipif(not orc.ref_available(), reason="reference kernels were not built")
def test_qkv_project_append_vs_reference_chain(cuda):
    """Against the reference's own kernels: its GEMMs, then its RoPE kernels on their outputs."""
    rng = np.random.default_rng(650)
    tokens = 200
    (q, k, v), _, (x, wq, wk, wv, cos, sin) = _project_append_case(rng, 0, tokens)
    from tests.gpu_helpers import f32_dev
    r = orc.ref()
    xd = to_dev(x)
    lin = {}
    for name, w, n in (("q", wq, 2048), ("k", wk, 512), ("v", wv, 512)):
        o = torch.zeros(tokens, n, dtype=torch.bfloat16, device=DEV)
        assert r.ref_gemm(xd.data_ptr(), to_dev(w).data_ptr(), o.data_ptr(), tokens, n, 2048) == 0
        lin[name] = o
    qo = torch.zeros(32, tokens, 64, dtype=torch.bfloat16, device=DEV)
    ko = torch.zeros(8, tokens, 64, dtype=torch.bfloat16, device=DEV)
    vo = torch.zeros(8, tokens, 64, dtype=torch.bfloat16, device=DEV)
    cd, sd = f32_dev(cos), f32_dev(sin)
    r.ref_rope_qkv(lin["q"].data_ptr(), qo.data_ptr(), lin["k"].data_ptr(), ko.data_ptr(), lin["v"].data_ptr(),
                   vo.data_ptr(), cd.data_ptr(), sd.data_ptr(), tokens, 0)
    torch.cuda.synchronize()
    q_ref = to_u16(qo).transpose(1, 0, 2).reshape(tokens, 2048)  # [heads, tokens, 64] -> token-major
    rotated_close(q, q_ref, "rotated Q against the reference chain")
    rotated_close(k, to_u16(ko), "rotated K against the reference chain")
    bf16_close(v, to_u16(vo), "V against the reference chain")


def test_qkv_project_append_two_sequences(cuda):
    """A batch of two sequences with different lengths and cache positions: rows of x are in batch
    order, every row finds its own sequence, position and cache block."""
    from tests.gpu_helpers import f32_dev, fill_cache
    rng = np.random.default_rng(700)
    positions, news = [19, 0], [70, 133]
    cos, sin = orc.build_rope_tables(256)
    pool = paged.KVPool(1, 40, 8, 2)
    pool.set_free_order(rng.permutation(40))
    seqs, olds = [], []
    for pos in positions:
        s = pool.create_seq()
        k_old = orc.randn_bf16(rng, (8, pos, 64), 0.5)
        v_old = orc.randn_bf16(rng, (8, pos, 64), 0.5)
        if pos:
            fill_cache(pool, 0, s, k_old, v_old)
        seqs.append(s)
        olds.append((k_old, v_old))
    rows = sum(news)
    x = orc.randn_bf16(rng, (rows, 2048))
    wq = orc.randn_bf16(rng, (2048, 2048), 0.03)
    wk = orc.randn_bf16(rng, (2048, 512), 0.03)
    wv = orc.randn_bf16(rng, (2048, 512), 0.03)
    for s, pos, n in zip(seqs, positions, news):
        pool.reserve(s, pos + n)
    pool.batch_set(seqs, news)
    q_out = torch.zeros(rows, 2048, dtype=torch.bfloat16, device=DEV)
    pq, pk, pv = (paged.pack_projection_weights(to_dev(w)) for w in (wq, wk, wv))
    # the activations are read in place through a tensor map: a base that is not 16-byte aligned is refused
    x_odd = torch.zeros(rows * 2048 + 1, dtype=torch.bfloat16, device=DEV)[1:].view(rows, 2048)
    with pytest.raises(_lib.PagedAttentionError) as ei:
        pool.qkv_project_append(0, x_odd, pq, pk, pv, f32_dev(cos), f32_dev(sin), q_out)
    assert ei.value.code == 1 and "16-byte" in str(ei.value)
    pool.qkv_project_append(0, to_dev(x), pq, pk, pv, f32_dev(cos), f32_dev(sin), q_out)
    torch.cuda.synchronize()
    pool.check()
    q_lin = orc.gemm_bf16(x, wq).reshape(rows, 32, 64)
    k_lin = orc.gemm_bf16(x, wk).reshape(rows, 8, 64)
    v_lin = orc.gemm_bf16(x, wv).reshape(rows, 8, 64)
    got_q = to_u16(q_out)
    r0 = 0
    for s, pos, n, (k_old, v_old) in zip(seqs, positions, news, olds):
        L = pos + n
        gk = torch.zeros(8, L, 64, dtype=torch.bfloat16, device=DEV)
        gv = torch.zeros_like(gk)
        pool.gather_kv(0, s, gk, gv, L)
        torch.cuda.synchronize()
        k, v = to_u16(gk), to_u16(gv)
        assert np.array_equal(k[:, :pos], k_old) and np.array_equal(v[:, :pos], v_old)
        rotated_close(got_q[r0:r0 + n],
                      orc.rope(q_lin[r0:r0 + n], cos, sin, pos, 1, out_token_major=True).reshape(n, 2048),
                      f"rotated Q of sequence {s}")
        rotated_close(k[:, pos:], orc.rope(k_lin[r0:r0 + n], cos, sin, pos, 1), f"rotated K of sequence {s}")
        bf16_close(v[:, pos:], orc.transpose_v(v_lin[r0:r0 + n]), f"V of sequence {s}")
        r0 += n
    pool.close()


@pytest.mark.parametrize("rows,layers,with_residual", [(1, 2, True), (4, 1, True), (2, 1, False)])
def test_out_project_with_residual(cuda, rows, layers, with_residual):
    """Output projection of a decode step with the attention residual folded in, against the oracle
    (GEMM rounded to bf16, fp32 sum of two bf16 rounded once) and the reference GEMM kernel."""
    rng = np.random.default_rng(800 + rows + layers)
    a = orc.randn_bf16(rng, (layers, rows, 2048))
    wo = orc.randn_bf16(rng, (layers, 2048, 2048), 0.03)
    res = orc.randn_bf16(rng, (layers, rows, 2048))
    out = torch.full((layers, rows, 2048), 5.0, dtype=torch.bfloat16, device=DEV)
    ad, wd, rd = to_dev(a), to_dev(wo), to_dev(res)
    paged.out_project(ad, wd, rd if with_residual else None, out, rows, layers)
    torch.cuda.synchronize()
    got = to_u16(out)
    for l in range(layers):
        lin = orc.gemm_bf16(a[l], wo[l])
        want = orc.f32_to_bf16(orc.bf16_to_f32(res[l]) + orc.bf16_to_f32(lin)) if with_residual else lin
        bf16_close(got[l], want, f"out_project layer {l}")
    if orc.ref_available():
        r = orc.ref()
        lin = torch.zeros(rows, 2048, dtype=torch.bfloat16, device=DEV)
        assert r.ref_gemm(ad[0].data_ptr(), wd[0].data_ptr(), lin.data_ptr(), rows, 2048, 2048) == 0
        torch.cuda.synchronize()
        want = (rd[0].float() + lin.float()).to(torch.bfloat16) if with_residual else lin
        bf16_close(got[0], to_u16(want), "out_project against the reference GEMM + residual")


@pytest.mark.parametrize("rows,with_residual", [(300, True), (128, False), (2400, True)])
def test_out_project_rows_on_tensor_cores(cuda, rows, with_residual):
    """Output projection of a prompt chunk (the projection GEMM with a plain epilogue) against the
    oracle and the reference GEMM + residual.  2400 rows are more pair tiles than SM pairs: the persistent
    form of the kernel (two accumulator sets in tensor memory), with a last row pair of one CTA's rows."""
    rng = np.random.default_rng(900 + rows)
    a = orc.randn_bf16(rng, (rows, 2048))
    wo = orc.randn_bf16(rng, (2048, 2048), 0.03)
    res = orc.randn_bf16(rng, (rows, 2048))
    pool = paged.KVPool(1, 8, 8, 1)
    out = torch.full((rows, 2048), 5.0, dtype=torch.bfloat16, device=DEV)
    ad, wd, rd = to_dev(a), to_dev(wo), to_dev(res)
    pool.out_project_rows(ad, paged.pack_projection_weights(wd), rd if with_residual else None, out, rows)
    torch.cuda.synchronize()
    pool.check()
    got = to_u16(out)
    lin = orc.gemm_bf16(a, wo)
    want = orc.f32_to_bf16(orc.bf16_to_f32(res) + orc.bf16_to_f32(lin)) if with_residual else lin
    bf16_close(got, want, "out_project_rows")
    if orc.ref_available():
        r = orc.ref()
        lr = torch.zeros(rows, 2048, dtype=torch.bfloat16, device=DEV)
        assert r.ref_gemm(ad.data_ptr(), wd.data_ptr(), lr.data_ptr(), rows, 2048, 2048) == 0
        torch.cuda.synchronize()
        wr = (rd.float() + lr.float()).to(torch.bfloat16) if with_residual else lr
        bf16_close(got, to_u16(wr), "out_project_rows against the reference GEMM + residual")
    pool.close()
