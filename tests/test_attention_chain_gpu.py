"""GPU parity of the steps either side of the attention path chained by their data: RMSNorm (as the
projection kernel's prologue and as a kernel of its own), and pa_attention_step — per layer
RMSNorm -> Q/K/V projections -> RoPE + append + decode attention -> output projection + residual,
the next layer fed by the previous one.  Against the CPU oracle chain and against the reference's own
kernels driven as Attention::forward drives them (src/runtime/attention.cu:99-390)."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import _lib, paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, check_close, f32_dev, to_dev, to_u16

pytestmark = pytest.mark.gpu

EPS = 1e-5


def ulp_close(got_u16, want_u16, what, min_equal=0.9, ulps=1, slack=0.0):
    """bf16 values equal up to `ulps` units in the last place (a bf16 neighbour is at most 2^-7 of the
    value away), most of them bit-equal.  `slack` is an absolute allowance for sums of many terms that
    cancel (GEMM outputs accumulated in another order)."""
    g = orc.bf16_to_f32(got_u16).astype(np.float64)
    w = orc.bf16_to_f32(want_u16).astype(np.float64)
    tol = np.maximum(np.abs(w), np.abs(g)) * 2.0 ** -7 * ulps + slack + 1e-30
    bad = np.abs(g - w) > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} differ by more than {ulps} ulp, worst {np.abs(g - w).max()}"
    exact = float((got_u16 == want_u16).mean())
    assert exact >= min_equal, f"{what}: only {exact:.4f} of the values are bit-equal"


@pytest.mark.parametrize("rows", [1, 5, 300])
def test_rmsnorm_rows_vs_reference_kernel_and_oracle(cuda, rows):
    rng = np.random.default_rng(700 + rows)
    x = orc.randn_bf16(rng, (rows, 2048), 1.5)
    w = orc.randn_bf16(rng, (2048,), 0.7)
    xd, wd = to_dev(x), to_dev(w)
    y = torch.full((rows, 2048), 9.0, dtype=torch.bfloat16, device=DEV)
    paged.rmsnorm(xd, wd, y, rows)
    torch.cuda.synchronize()
    got = to_u16(y)
    ulp_close(got, orc.rmsnorm(x, w, EPS), "pa_rmsnorm vs oracle", min_equal=0.99)
    if orc.ref_available():
        want = torch.zeros_like(y)
        orc.ref().ref_rmsnorm(xd.data_ptr(), wd.data_ptr(), want.data_ptr(), rows, EPS)
        torch.cuda.synchronize()
        assert np.array_equal(got, to_u16(want)), "pa_rmsnorm differs from the reference kernel's bits"
    # in place
    paged.rmsnorm(xd, wd, xd, rows)
    torch.cuda.synchronize()
    assert np.array_equal(to_u16(xd), got)


@pytest.mark.parametrize("rows,layers", [(1, 2), (3, 1), (8, 1)])
def test_rmsnorm_qkv_project_vs_oracle_and_reference(cuda, rows, layers):
    rng = np.random.default_rng(720 + rows)
    x = orc.randn_bf16(rng, (layers, rows, 2048), 1.5)
    nw = orc.randn_bf16(rng, (layers, 2048), 0.7)
    wq = orc.randn_bf16(rng, (layers, 2048, 2048), 0.03)
    wk = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
    wv = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
    q = torch.full((layers, rows, 2048), 7.0, dtype=torch.bfloat16, device=DEV)
    k = torch.full((layers, rows, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    v = torch.full((layers, rows, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    xd, nwd, wqd, wkd, wvd = to_dev(x), to_dev(nw), to_dev(wq), to_dev(wk), to_dev(wv)
    paged.rmsnorm_qkv_project(xd, nwd, wqd, wkd, wvd, q, k, v, rows, layers)
    torch.cuda.synchronize()
    for l in range(layers):
        xn = orc.rmsnorm(x[l], nw[l], EPS)
        for got, wmat, name in ((q, wq, "q"), (k, wk, "k"), (v, wv, "v")):
            ulp_close(to_u16(got[l]), orc.gemm_bf16(xn, wmat[l]), f"{name} layer {l} vs oracle chain", slack=0.02)
    if orc.ref_available():
        r = orc.ref()
        xn = torch.zeros(rows, 2048, dtype=torch.bfloat16, device=DEV)
        r.ref_rmsnorm(xd[0].data_ptr(), nwd[0].data_ptr(), xn.data_ptr(), rows, EPS)
        for got, wmat, n in ((q, wqd, 2048), (k, wkd, 512), (v, wvd, 512)):
            want = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
            assert r.ref_gemm(xn.data_ptr(), wmat[0].data_ptr(), want.data_ptr(), rows, n, 2048) == 0
            torch.cuda.synchronize()
            ulp_close(to_u16(got[0]), to_u16(want), f"N={n} vs the reference's RMSNorm + GEMM", slack=0.02)


def _model(rng, layers):
    nw = orc.randn_bf16(rng, (layers, 2048), 0.7)
    wq = orc.randn_bf16(rng, (layers, 2048, 2048), 0.03)
    wk = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
    wv = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
    wo = orc.randn_bf16(rng, (layers, 2048, 2048), 0.03)
    return nw, wq, wk, wv, wo


def _oracle_layer(x, nw, wq, wk, wv, wo, K, V, pos, cos, sin, residual=True):
    """One attention block for ONE sequence on the CPU.  x [1, 2048] bf16 bits; K, V [8, >= pos + 1, 64]
    (row pos is written).  Returns the block output [1, 2048] bf16 bits and the attention row (fp32)."""
    xn = orc.rmsnorm(x, nw, EPS)
    q = orc.gemm_bf16(xn, wq).reshape(1, 32, 64)
    k = orc.gemm_bf16(xn, wk).reshape(1, 8, 64)
    v = orc.gemm_bf16(xn, wv).reshape(1, 8, 64)
    K[:, pos] = orc.rope(k, cos, sin, pos, 1)[:, 0]
    V[:, pos] = v[0]
    O, _ = orc.attention(orc.rope(q, cos, sin, pos, 1), K, V, pos + 1)
    attn = orc.f32_to_bf16(O[:, 0].reshape(1, 2048))
    lin = orc.gemm_bf16(attn, wo)
    out = orc.f32_to_bf16(orc.bf16_to_f32(x) + orc.bf16_to_f32(lin)) if residual else lin
    return out, O[:, 0].reshape(-1)


def _fill(pool, seq, layers, Ks, Vs, n):
    pool.reserve(seq, n)
    pool.batch_set([seq], [n])
    ones = torch.ones(n, 32, dtype=torch.float32, device=DEV)
    zeros = torch.zeros(n, 32, dtype=torch.float32, device=DEV)
    for l in range(layers):
        pool.append(l, None, to_dev(Ks[l][:, :n].transpose(1, 0, 2)), to_dev(Vs[l][:, :n].transpose(1, 0, 2)),
                    ones, zeros, None)
    torch.cuda.synchronize()


@pytest.mark.parametrize("lens", [(777,), (40, 1300, 16)])
def test_attention_step_layer_by_layer_vs_oracle_chain(cuda, lens):
    """3 layers, 2 steps.  Each layer is fed the GPU's own previous output, so every layer is compared
    with the oracle on identical inputs (no error build-up); then one 3-layer call must reproduce the
    layer-by-layer rows bit for bit, and the caches must hold the appended rows."""
    rng = np.random.default_rng(800 + len(lens))
    layers, steps, n = 3, 2, len(lens)
    nw, wq, wk, wv, wo = _model(rng, layers)
    cos, sin = orc.build_rope_tables(max(lens) + steps + 1)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    nb = sum((L + steps + 15) // 16 for L in lens) + 8
    Ks = [[orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)] for L in lens]
    Vs = [[orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)] for L in lens]
    results = []
    for mode in ("by_layer", "one_call"):
        pool = paged.KVPool(layers, nb, 8, n, max((L + steps + 15) // 16 for L in lens) + 1)
        pool.set_free_order(np.random.default_rng(3).permutation(nb))
        seqs = [pool.create_seq() for _ in lens]
        for i, L in enumerate(lens):
            _fill(pool, seqs[i], layers, Ks[i], Vs[i], L)
        tens = [to_dev(a) for a in (nw, wq, wk, wv, wo)]  # the descriptor holds raw addresses: keep them alive
        W = paged.attention_weights(*tens)
        xrng = np.random.default_rng(55)
        outs = []
        for step in range(steps):
            x0 = orc.randn_bf16(xrng, (n, 2048), 1.0)
            for i, L in enumerate(lens):
                pool.reserve(seqs[i], L + step + 1)
            pool.batch_set(seqs)
            if mode == "one_call":
                y = torch.zeros(n, 2048, dtype=torch.bfloat16, device=DEV)
                paged.attention_step(pool, W, 0, layers, to_dev(x0), y, cos_d, sin_d)
                torch.cuda.synchronize()
                pool.check()
                outs.append(to_u16(y))
                continue
            cur = to_dev(x0)
            per_layer = []
            for l in range(layers):
                y = torch.zeros(n, 2048, dtype=torch.bfloat16, device=DEV)
                paged.attention_step(pool, W, l, l + 1, cur, y, cos_d, sin_d)
                torch.cuda.synchronize()
                pool.check()
                xin = to_u16(cur)
                for i, L in enumerate(lens):
                    K, V = Ks[i][l].copy(), Vs[i][l].copy()
                    want, _ = _oracle_layer(xin[i:i + 1], nw[l], wq[l], wk[l], wv[l], wo[l], K, V, L + step, cos, sin)
                    # projections may differ by an ulp, which attention and the output projection pass
                    # on: compare on the scale of the row
                    g = orc.bf16_to_f32(to_u16(y[i])).astype(np.float64)
                    w_ = orc.bf16_to_f32(want[0]).astype(np.float64)
                    assert np.max(np.abs(g - w_)) <= 2.0 ** -6 * np.max(np.abs(w_)), (step, l, i, np.max(np.abs(g - w_)))
                    assert float((to_u16(y[i]) == want[0]).mean()) > 0.8
                per_layer.append(to_u16(y))
                cur = y
            outs.append(per_layer[-1])
            # this step's appended rows become part of the cache the next step sees (GPU's own values)
            for i, L in enumerate(lens):
                for l in range(layers):
                    gk = torch.zeros(8, L + step + 1, 64, dtype=torch.bfloat16, device=DEV)
                    gv = torch.zeros_like(gk)
                    pool.gather_kv(l, seqs[i], gk, gv, L + step + 1)
                    torch.cuda.synchronize()
                    Ks[i][l][:, L + step] = to_u16(gk)[:, L + step]
                    Vs[i][l][:, L + step] = to_u16(gv)[:, L + step]
        results.append(outs)
        pool.close()
    for a, b in zip(results[0], results[1]):
        assert np.array_equal(a, b), "a 3-layer call differs from three 1-layer calls"


@pytest.mark.skipif(not orc.ref_available(), reason="reference kernels were not built")
def test_attention_step_vs_reference_chain(cuda):
    """One layer, one sequence at position 600, without the residual (what Attention::forward returns)
    and with it (after TransformerBlock's residual_add): the reference's own kernels in its own order."""
    rng = np.random.default_rng(830)
    L = 600
    nw, wq, wk, wv, wo = _model(rng, 1)
    cos, sin = orc.build_rope_tables(L + 2)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    K = orc.randn_bf16(rng, (8, L + 1, 64), 0.5)
    V = orc.randn_bf16(rng, (8, L + 1, 64), 0.5)
    x = orc.randn_bf16(rng, (1, 2048), 1.0)
    tens = [to_dev(a) for a in (nw, wq, wk, wv, wo)]
    W = paged.attention_weights(*tens)
    xd = to_dev(x)
    got = {}
    for residual in (False, True):
        pool = paged.KVPool(1, 48, 8, 1)
        s = pool.create_seq()
        _fill(pool, s, 1, [K], [V], L)
        pool.reserve(s, L + 1)
        pool.batch_set([s])
        y = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
        paged.attention_step(pool, W, 0, 1, xd, y, cos_d, sin_d, add_residual=residual)
        torch.cuda.synchronize()
        pool.check()
        got[residual] = to_u16(y)
        pool.close()
    r = orc.ref()
    nwd, wqd, wkd, wvd, wod = tens
    max_seq = L + 8
    xn = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
    ql = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
    kl = torch.zeros(1, 512, dtype=torch.bfloat16, device=DEV)
    vl = torch.zeros(1, 512, dtype=torch.bfloat16, device=DEV)
    qf = torch.empty(32, 1, 64, dtype=torch.bfloat16, device=DEV)
    kf = torch.empty(8, 1, 64, dtype=torch.bfloat16, device=DEV)
    vf = torch.empty(8, 1, 64, dtype=torch.bfloat16, device=DEV)
    of = torch.empty(32, 1, 64, dtype=torch.bfloat16, device=DEV)
    arow = torch.empty(1, 2048, dtype=torch.bfloat16, device=DEV)
    lin = torch.empty(1, 2048, dtype=torch.bfloat16, device=DEV)
    res = torch.empty(1, 2048, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(8, max_seq, 64, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    kc[:, :L] = to_dev(K[:, :L])
    vc[:, :L] = to_dev(V[:, :L])
    torch.cuda.synchronize()
    r.ref_rmsnorm(xd.data_ptr(), nwd[0].data_ptr(), xn.data_ptr(), 1, EPS)
    for wmat, o, ncol in ((wqd, ql, 2048), (wkd, kl, 512), (wvd, vl, 512)):
        assert r.ref_gemm(xn.data_ptr(), wmat[0].data_ptr(), o.data_ptr(), 1, ncol, 2048) == 0
        torch.cuda.synchronize()
    r.ref_rope_qkv(ql.data_ptr(), qf.data_ptr(), kl.data_ptr(), kf.data_ptr(), vl.data_ptr(), vf.data_ptr(),
                   cos_d.data_ptr(), sin_d.data_ptr(), 1, L)
    assert r.ref_append_memcpy_loop(kc.data_ptr(), vc.data_ptr(), kf.data_ptr(), vf.data_ptr(), max_seq, L, 1) == 0
    r.ref_flash_attention(qf.data_ptr(), kc.data_ptr(), vc.data_ptr(), of.data_ptr(), None, 1, 32, 8, 1, L + 1,
                          max_seq, 0.125, 1, None)
    r.ref_flash_output_layout(of.data_ptr(), arow.data_ptr(), 1)
    assert r.ref_gemm(arow.data_ptr(), wod[0].data_ptr(), lin.data_ptr(), 1, 2048, 2048) == 0
    torch.cuda.synchronize()
    assert r.ref_residual_add(xd.data_ptr(), lin.data_ptr(), res.data_ptr(), 2048) == 0
    torch.cuda.synchronize()
    for residual, want in ((False, to_u16(lin)), (True, to_u16(res))):
        g = orc.bf16_to_f32(got[residual]).astype(np.float64)
        w_ = orc.bf16_to_f32(want).astype(np.float64)
        # the two attention kernels round their rows differently in the last bit, and the output
        # projection sums 2048 such terms: compare on the scale of the row, not bit by bit
        assert np.max(np.abs(g - w_)) <= 2.0 ** -6 * np.max(np.abs(w_)), (residual, np.max(np.abs(g - w_)))


def test_attention_step_with_a_one_rank_exchange_and_argument_errors(cuda):
    rng = np.random.default_rng(840)
    L = 200
    nw, wq, wk, wv, wo = _model(rng, 2)
    cos, sin = orc.build_rope_tables(L + 2)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    Ks = [orc.randn_bf16(rng, (8, L + 1, 64), 0.5) for _ in range(2)]
    Vs = [orc.randn_bf16(rng, (8, L + 1, 64), 0.5) for _ in range(2)]
    tens = [to_dev(a) for a in (nw, wq, wk, wv, wo)]
    W = paged.attention_weights(*tens)
    x = to_dev(orc.randn_bf16(rng, (1, 2048), 1.0))
    outs = []
    for sharded in (False, True):
        pool = paged.KVPool(2, 24, 8, 1)
        s = pool.create_seq()
        _fill(pool, s, 2, Ks, Vs, L)
        pool.reserve(s, L + 1)
        pool.batch_set([s])
        xchg = paged.Exchange(0, 0, 1, 1, 8) if sharded else None
        y = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
        paged.attention_step(pool, W, 0, 2, x, y, cos_d, sin_d, xchg=xchg)
        torch.cuda.synchronize()
        pool.check()
        outs.append(to_u16(y))
        if not sharded:
            with pytest.raises(_lib.PagedAttentionError) as ei:  # several layers in place
                paged.attention_step(pool, W, 0, 2, x, x, cos_d, sin_d)
            assert ei.value.code == 1
            with pytest.raises(_lib.PagedAttentionError) as ei:
                paged.attention_step(pool, W, 1, 3, x, y, cos_d, sin_d)
            assert ei.value.code == 1
        if xchg is not None:
            xchg.close()
        pool.close()
    g = orc.bf16_to_f32(outs[1]).astype(np.float64)
    w_ = orc.bf16_to_f32(outs[0]).astype(np.float64)
    assert np.max(np.abs(g - w_)) <= 2.0 ** -6 * np.max(np.abs(w_))
