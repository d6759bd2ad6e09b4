"""GPU parity of the end of a decode step: the language-model head (pa_lm_head: final RMSNorm + the
2048 x 128256 weight stream) and greedy sampling (pa_argmax), against the CPU oracle and against the
reference's own kernels (rmsnorm_launch<2048>, launch_gemm_2048x128256, launch_argmax as
src/runtime/llama_runtime.cu:880-930 calls them)."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import _lib, paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, to_dev, to_u16
from tests.test_attention_chain_gpu import ulp_close

pytestmark = pytest.mark.gpu

VOCAB = 128256
EPS = 1e-5


@pytest.mark.parametrize("rows", [1, 3])
def test_lm_head_logits_and_token_vs_oracle_and_reference(cuda, rows):
    rng = np.random.default_rng(1100 + rows)
    x = orc.randn_bf16(rng, (rows, 2048), 1.3)
    nw = orc.randn_bf16(rng, (2048,), 0.7)
    w = orc.randn_bf16(rng, (2048, VOCAB), 0.03)
    xd, nd, wd = to_dev(x), to_dev(nw), to_dev(w)
    logits = torch.full((rows, VOCAB), 7.0, dtype=torch.bfloat16, device=DEV)
    tokens = torch.full((rows,), -5, dtype=torch.int32, device=DEV)
    paged.lm_head(xd, nd, wd, logits, rows, EPS)
    paged.argmax(logits, tokens, rows)
    torch.cuda.synchronize()
    got = to_u16(logits)
    want = orc.gemm_bf16(orc.rmsnorm(x, nw, EPS), w)
    # sums of 2048 products accumulated in another order: one bf16 unit, plus an absolute allowance for
    # sums that cancel
    ulp_close(got, want, "logits vs oracle", min_equal=0.9, slack=0.02)
    # the token is the reference rule's answer on the logits the GPU produced
    assert np.array_equal(tokens.cpu().numpy(), orc.argmax_reference_rule(got))
    if orc.ref_available():
        r = orc.ref()
        xn = torch.zeros(1, 2048, dtype=torch.bfloat16, device=DEV)
        ref_logits = torch.zeros(1, VOCAB, dtype=torch.bfloat16, device=DEV)
        ref_tok = torch.zeros(1, dtype=torch.int32, device=DEV)
        r.ref_rmsnorm(xd[0:1].data_ptr(), nd.data_ptr(), xn.data_ptr(), 1, EPS)
        assert r.ref_gemm(xn.data_ptr(), wd.data_ptr(), ref_logits.data_ptr(), 1, VOCAB, 2048) == 0
        torch.cuda.synchronize()
        ulp_close(got[0:1], to_u16(ref_logits), "logits vs the reference's RMSNorm + GEMM", min_equal=0.9, slack=0.02)
        # the reference's argmax kernel on this library's logits gives this library's token
        for i in range(rows):
            r.ref_argmax(logits[i].data_ptr(), ref_tok.data_ptr())
            torch.cuda.synchronize()
            assert int(ref_tok.item()) == int(tokens[i].item())


def test_argmax_breaks_ties_as_the_reference_kernel_does(cuda):
    """Equal largest values at chosen places: the winner is decided by the reference kernel's reduction
    tree (thread = index mod 256; warps, then lanes, in bit-reversed order; then the smallest index) —
    not simply the first index."""
    rng = np.random.default_rng(1200)
    rows = 6
    lg = orc.randn_bf16(rng, (rows, VOCAB), 1.0)
    big = orc.f32_to_bf16(np.array([50.0], np.float32))[0]
    places = [[300, 5], [5, 261, 517], [1000, 999], [VOCAB - 1, 255], [256 * 7 + 3, 3 + 256 * 400, 4], [77]]
    for i, idxs in enumerate(places):
        lg[i, idxs] = big
    d = to_dev(lg)
    tokens = torch.zeros(rows, dtype=torch.int32, device=DEV)
    paged.argmax(d, tokens, rows)
    torch.cuda.synchronize()
    got = tokens.cpu().numpy()
    assert np.array_equal(got, orc.argmax_reference_rule(lg))
    # [300, 5]: threads 44 (warp 1) and 5 (warp 0): warp 0 first.  [5, 261, 517]: all thread 5: smallest index.
    # [1000, 999]: threads 232 (warp 7, lane 8) and 231 (warp 7, lane 7): lane 8 (reversed 2) before lane 7 (28).
    assert list(got[:3]) == [5, 5, 1000]
    if orc.ref_available():
        r = orc.ref()
        ref_tok = torch.zeros(1, dtype=torch.int32, device=DEV)
        for i in range(rows):
            r.ref_argmax(d[i].data_ptr(), ref_tok.data_ptr())
            torch.cuda.synchronize()
            assert int(ref_tok.item()) == int(got[i]), i


def test_lm_head_argument_errors(cuda):
    x = torch.zeros(9, 2048, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(2048, 64, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(9, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.lm_head(x, None, w, out, 9)
    assert ei.value.code == 3
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.lm_head(None, None, w, out, 1)
    assert ei.value.code == 1
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.lm_head(x, None, torch.zeros(2048, 40, dtype=torch.bfloat16, device=DEV), out, 1)
    assert ei.value.code == 3  # vocab must be a multiple of 32
