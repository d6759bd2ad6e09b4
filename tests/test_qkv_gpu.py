"""GPU parity of the decode-shape Q/K/V projection (pa_qkv_project) against the
CPU oracle (double accumulation, one rounding) and the reference's own GEMM
kernels (gemm_2048x2048.cu, gemm_2048x512.cu as Attention::forward calls them)."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import paged
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
