"""GPU parity of the feed-forward block of a decode step (pa_ffn) and of whole transformer blocks
chained by their data (pa_block_step), against the CPU oracle chain and against the reference's own
kernels driven as FeedForward::forward drives them (src/runtime/ffn.cu:34-145: RMSNorm, two
2048x8192 GEMMs, SiLU(gate) * up, the 8192x2048 GEMM) plus the block's residual add
(src/runtime/transformer_block.cu:76-81)."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import _lib, paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, f32_dev, to_dev, to_u16
from tests.test_attention_chain_gpu import _fill, _model, _oracle_layer

pytestmark = pytest.mark.gpu

EPS = 1e-5
# floating point: the block output is a sum of 8192 products of bf16 values, rounded to bf16; the
# bar is 2^-6 of the row's largest magnitude (two bf16 roundings of slack)
ROW_TOL = 2.0 ** -6


def row_rel(got_u16, want_u16):
    g = orc.bf16_to_f32(got_u16).astype(np.float64)
    w = orc.bf16_to_f32(want_u16).astype(np.float64)
    return float(np.max(np.abs(g - w).max(axis=-1) / np.maximum(np.abs(w).max(axis=-1), 1e-30)))


def _ffn_model(rng, layers):
    fn = orc.randn_bf16(rng, (layers, 2048), 0.7)
    wg = orc.randn_bf16(rng, (layers, 2048, 8192), 0.03)
    wu = orc.randn_bf16(rng, (layers, 2048, 8192), 0.03)
    wd = orc.randn_bf16(rng, (layers, 8192, 2048), 0.02)
    return fn, wg, wu, wd


@pytest.mark.parametrize("rows,residual,norm", [(1, True, True), (2, True, True), (3, False, True), (4, True, False),
                                               (7, True, True), (8, True, True)])
def test_ffn_vs_oracle_and_reference(cuda, rows, residual, norm):
    rng = np.random.default_rng(900 + rows)
    layers = 2
    fn, wg, wu, wd = _ffn_model(rng, layers)
    x = orc.randn_bf16(rng, (rows, 2048), 1.2)
    tens = [to_dev(a) for a in (fn, wg, wu, wd)]
    W = paged.ffn_weights(tens[0] if norm else None, tens[1], tens[2], tens[3], EPS)
    xd = to_dev(x)
    h = torch.full((rows, 8192), 3.0, dtype=torch.bfloat16, device=DEV)
    out = torch.full((rows, 2048), 5.0, dtype=torch.bfloat16, device=DEV)
    layer = 1
    paged.ffn(W, layer, xd, h, out, rows, add_residual=residual)
    torch.cuda.synchronize()
    got, got_h = to_u16(out), to_u16(h)
    # ---- CPU oracle chain
    xn = orc.rmsnorm(x, fn[layer], EPS) if norm else x
    want_h = orc.silu_mul(orc.gemm_bf16(xn, wg[layer]), orc.gemm_bf16(xn, wu[layer]))
    assert row_rel(got_h, want_h) <= ROW_TOL, "activated rows vs oracle"
    want = orc.ffn(x, fn[layer] if norm else None, wg[layer], wu[layer], wd[layer], EPS, residual)
    assert row_rel(got, want) <= ROW_TOL, "block output vs oracle"
    # the kernel's own h through the oracle's down projection: isolates the second kernel
    y = orc.gemm_bf16(got_h, wd[layer])
    want2 = orc.f32_to_bf16(orc.bf16_to_f32(x) + orc.bf16_to_f32(y)) if residual else y
    assert row_rel(got, want2) <= 2.0 ** -7, "down projection on identical activated rows"
    # ---- the reference's kernels
    if orc.ref_available():
        r = orc.ref()
        xn_d = torch.zeros(rows, 2048, dtype=torch.bfloat16, device=DEV)
        if norm:
            r.ref_rmsnorm(xd.data_ptr(), tens[0][layer].data_ptr(), xn_d.data_ptr(), rows, EPS)
        else:
            xn_d.copy_(xd)
        g = torch.zeros(rows, 8192, dtype=torch.bfloat16, device=DEV)
        u = torch.zeros_like(g)
        hr = torch.zeros_like(g)
        yr = torch.zeros(rows, 2048, dtype=torch.bfloat16, device=DEV)
        assert r.ref_gemm(xn_d.data_ptr(), tens[1][layer].data_ptr(), g.data_ptr(), rows, 8192, 2048) == 0
        assert r.ref_gemm(xn_d.data_ptr(), tens[2][layer].data_ptr(), u.data_ptr(), rows, 8192, 2048) == 0
        r.ref_silu_mul(g.data_ptr(), u.data_ptr(), hr.data_ptr(), rows)
        assert r.ref_gemm(hr.data_ptr(), tens[3][layer].data_ptr(), yr.data_ptr(), rows, 2048, 8192) == 0
        if residual:
            assert r.ref_residual_add(xd.data_ptr(), yr.data_ptr(), yr.data_ptr(), rows * 2048) == 0
        torch.cuda.synchronize()
        assert row_rel(got_h, to_u16(hr)) <= ROW_TOL, "activated rows vs the reference's kernels"
        assert row_rel(got, to_u16(yr)) <= ROW_TOL, "block output vs the reference's kernels"
        # SiLU(gate) * up alone, on the reference's own gate and up rows: the oracle's restatement
        # (expf on the CPU, __expf on the device) within one bf16 unit of the reference kernel
        oh = orc.silu_mul(to_u16(g), to_u16(u))
        a = orc.bf16_to_f32(oh).astype(np.float64)
        b = orc.bf16_to_f32(to_u16(hr)).astype(np.float64)
        assert np.all(np.abs(a - b) <= np.maximum(np.abs(a), np.abs(b)) * 2.0 ** -7 + 1e-30)
        assert float((oh == to_u16(hr)).mean()) > 0.99
    # in place: out may alias x
    x2 = xd.clone()
    paged.ffn(W, layer, x2, h, x2, rows, add_residual=residual)
    torch.cuda.synchronize()
    assert np.array_equal(to_u16(x2), got)


@pytest.mark.parametrize("rows,residual", [(5, True), (300, True), (130, False), (700, True)])
def test_ffn_rows_on_the_tensor_cores_vs_oracle(cuda, rows, residual):
    """The prompt-chunk form: RMSNorm kernel, two tcgen05 GEMM launches on packed weights (gate and up as
    one, SiLU * up in its epilogue; down + residual).  Up to 256 rows the gate/up GEMM is one tile per CTA
    pair, above that the persistent form.  Against the oracle chain, and (for few rows) against the
    decode-shape kernels."""
    rng = np.random.default_rng(930 + rows)
    fn, wg, wu, wd = _ffn_model(rng, 1)
    x = orc.randn_bf16(rng, (rows, 2048), 1.2)
    tens = [to_dev(a) for a in (fn, wg, wu, wd)]
    packed = [paged.pack_projection_weights(t) for t in tens[1:]]
    WP = paged.ffn_weights(tens[0], packed[0], packed[1], packed[2], EPS)
    pool = paged.KVPool(1, 8, 8, 1)
    xd = to_dev(x)
    scratch = torch.zeros(rows * (2048 + 8192), dtype=torch.bfloat16, device=DEV)
    out = torch.full((rows, 2048), 5.0, dtype=torch.bfloat16, device=DEV)
    paged.ffn_rows(pool, WP, 0, xd, scratch, out, rows, add_residual=residual)
    torch.cuda.synchronize()
    pool.check()
    got = to_u16(out)
    want = orc.ffn(x, fn[0], wg[0], wu[0], wd[0], EPS, residual)
    assert row_rel(got, want) <= ROW_TOL
    if rows <= 8:
        W = paged.ffn_weights(*tens, EPS)
        h = torch.zeros(rows, 8192, dtype=torch.bfloat16, device=DEV)
        out2 = torch.zeros_like(out)
        paged.ffn(W, 0, xd, h, out2, rows, add_residual=residual)
        torch.cuda.synchronize()
        assert row_rel(got, to_u16(out2)) <= ROW_TOL
    pool.close()


def test_ffn_argument_errors(cuda):
    rng = np.random.default_rng(5)
    fn, wg, wu, wd = _ffn_model(rng, 1)
    tens = [to_dev(a) for a in (fn, wg, wu, wd)]
    W = paged.ffn_weights(*tens)
    x = torch.zeros(9, 2048, dtype=torch.bfloat16, device=DEV)
    h = torch.zeros(9, 8192, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.ffn(W, 0, x, h, x, 9)
    assert ei.value.code == 3  # PA_ERR_UNSUPPORTED: more than 8 rows
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.ffn(W, 0, None, h, x, 1)
    assert ei.value.code == 1


@pytest.mark.parametrize("lens", [(300,), (40, 520)])
def test_block_step_layer_by_layer_vs_oracle_chain(cuda, lens):
    """2 layers, 2 steps of whole blocks.  Each layer is fed the GPU's own previous rows, so every layer is
    compared with the oracle on identical inputs; one 2-layer call must reproduce those rows bit for bit."""
    rng = np.random.default_rng(950 + len(lens))
    layers, steps, n = 2, 2, len(lens)
    nw, wq, wk, wv, wo = _model(rng, layers)
    fn, wg, wu, wd = _ffn_model(rng, layers)
    cos, sin = orc.build_rope_tables(max(lens) + steps + 1)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    nb = sum((L + steps + 15) // 16 for L in lens) + 8
    Ks = [[orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)] for L in lens]
    Vs = [[orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)] for L in lens]
    xs = [orc.randn_bf16(rng, (n, 2048), 1.0) for _ in range(steps)]
    results = []
    for mode in ("by_layer", "one_call"):
        pool = paged.KVPool(layers, nb, 8, n, max((L + steps + 15) // 16 for L in lens) + 1)
        pool.set_free_order(np.random.default_rng(3).permutation(nb))
        seqs = [pool.create_seq() for _ in lens]
        for i, L in enumerate(lens):
            _fill(pool, seqs[i], layers, Ks[i], Vs[i], L)
        at = [to_dev(a) for a in (nw, wq, wk, wv, wo)]
        ft = [to_dev(a) for a in (fn, wg, wu, wd)]
        WA, WF = paged.attention_weights(*at), paged.ffn_weights(*ft)
        Kc = [[k.copy() for k in Ks[i]] for i in range(n)]
        Vc = [[v.copy() for v in Vs[i]] for i in range(n)]
        rows_out = []
        for step in range(steps):
            for i in range(n):
                pool.reserve(seqs[i], lens[i] + step + 1)
            pool.batch_set(seqs, [1] * n)
            cur = to_dev(xs[step])
            if mode == "one_call":
                y = torch.zeros(n, 2048, dtype=torch.bfloat16, device=DEV)
                paged.block_step(pool, WA, WF, 0, layers, cur, y, cos_d, sin_d)
                torch.cuda.synchronize()
                pool.check()
                rows_out.append(to_u16(y))
                continue
            for l in range(layers):
                y = torch.zeros(n, 2048, dtype=torch.bfloat16, device=DEV)
                paged.block_step(pool, WA, WF, l, l + 1, cur, y, cos_d, sin_d)
                torch.cuda.synchronize()
                pool.check()
                x_u = to_u16(cur)
                for i in range(n):
                    pos = lens[i] + step
                    a, _ = _oracle_layer(x_u[i:i + 1], nw[l], wq[l], wk[l], wv[l], wo[l], Kc[i][l], Vc[i][l], pos, cos, sin)
                    want = orc.ffn(a, fn[l], wg[l], wu[l], wd[l], EPS, True)
                    rel = row_rel(to_u16(y[i:i + 1]), want)
                    assert rel <= 2.0 ** -5, f"step {step} layer {l} sequence {i}: {rel}"
                cur = y
            rows_out.append(to_u16(cur))
        results.append(rows_out)
        pool.close()
    for a, b in zip(*results):
        assert np.array_equal(a, b), "one 2-layer call differs from two 1-layer calls"
