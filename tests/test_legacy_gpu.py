"""GPU parity of the reference-compatible launchers (include/flashattention.h,
rope.hpp, layout.hpp -> lt_* entries): same layouts as the reference, checked
against the reference's own kernels and the oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import _lib
from oracle import oracle as orc
from tests.gpu_helpers import DEV, check_close, f32_dev, to_dev, to_u16

pytestmark = pytest.mark.gpu


def flash(Q, K, V, O, L, batch, q_len, kv_len, stride, causal=True, heads=32, kv_heads=8, d_head=64, dtype=1):
    p = _lib.FlashAttentionParams(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(),
                                  0 if L is None else L.data_ptr(), batch, heads, kv_heads, q_len, kv_len,
                                  stride, d_head, 0.125, int(causal), dtype, None)
    return _lib.lib().lt_launch_flash_attention(C.byref(p))


@pytest.mark.parametrize("tokens,position", [(1, 512), (37, 0), (300, 45)])
def test_rope_and_layout_bit_exact(cuda, tokens, position):
    rng = np.random.default_rng(200 + tokens)
    cos, sin = orc.build_rope_tables(position + tokens)
    q = orc.randn_bf16(rng, (tokens, 32, 64))
    k = orc.randn_bf16(rng, (tokens, 8, 64))
    v = orc.randn_bf16(rng, (tokens, 8, 64))
    qo = torch.zeros(32, tokens, 64, dtype=torch.bfloat16, device=DEV)
    ko = torch.zeros(8, tokens, 64, dtype=torch.bfloat16, device=DEV)
    vo = torch.zeros_like(ko)
    qd, kd, vd, cd, sd = to_dev(q), to_dev(k), to_dev(v), f32_dev(cos), f32_dev(sin)  # kept alive past the launch
    rc = _lib.lib().lt_launch_rope_qkv(qd.data_ptr(), qo.data_ptr(), kd.data_ptr(), ko.data_ptr(),
                                       vd.data_ptr(), vo.data_ptr(), cd.data_ptr(), sd.data_ptr(), tokens,
                                       position, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.array_equal(to_u16(qo), orc.rope(q, cos, sin, position, 1))
    assert np.array_equal(to_u16(ko), orc.rope(k, cos, sin, position, 1))
    assert np.array_equal(to_u16(vo), orc.transpose_v(v))
    if orc.ref_available():
        rq, rk, rv = torch.zeros_like(qo), torch.zeros_like(ko), torch.zeros_like(vo)
        orc.ref().ref_rope_qkv(qd.data_ptr(), rq.data_ptr(), kd.data_ptr(), rk.data_ptr(), vd.data_ptr(),
                               rv.data_ptr(), cd.data_ptr(), sd.data_ptr(), tokens, position)
        torch.cuda.synchronize()
        assert torch.equal(rq.view(torch.int16), qo.view(torch.int16))
        assert torch.equal(rk.view(torch.int16), ko.view(torch.int16))
        assert torch.equal(rv.view(torch.int16), vo.view(torch.int16))
    lay = torch.zeros(tokens, 2048, dtype=torch.bfloat16, device=DEV)
    assert _lib.lib().lt_launch_flash_output_layout(qo.data_ptr(), lay.data_ptr(), tokens, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(to_u16(lay), orc.output_layout(to_u16(qo)))


@pytest.mark.parametrize("batch,q_len,kv_len,stride,causal", [
    (1, 1, 513, 600, True), (1, 200, 200, 256, True), (1, 20, 65, 80, True),
    (2, 1, 300, 300, True), (2, 130, 190, 200, True), (1, 70, 150, 150, False),
])
def test_flash_attention_contiguous_cache(cuda, batch, q_len, kv_len, stride, causal):
    rng = np.random.default_rng(300 + q_len + kv_len)
    Q = orc.randn_bf16(rng, (batch * 32, q_len, 64))
    K = orc.randn_bf16(rng, (batch * 8, stride, 64), 0.5)
    V = orc.randn_bf16(rng, (batch * 8, stride, 64), 0.5)
    Qd, Kd, Vd = to_dev(Q), to_dev(K), to_dev(V)
    O = torch.zeros(batch * 32, q_len, 64, dtype=torch.bfloat16, device=DEV)
    L = torch.zeros(batch * 32, q_len, dtype=torch.float32, device=DEV)
    for rep in range(2):  # the second call reuses the private pool
        assert flash(Qd, Kd, Vd, O, L, batch, q_len, kv_len, stride, causal) == 0, _lib.lib().pa_last_error()
    torch.cuda.synchronize()
    got, got_l = orc.bf16_to_f32(to_u16(O)), L.cpu().numpy()
    for b in range(batch):
        want, want_l = orc.attention(Q[b * 32:(b + 1) * 32], K[b * 8:(b + 1) * 8], V[b * 8:(b + 1) * 8], kv_len,
                                     causal=causal)
        check_close(got[b * 32:(b + 1) * 32], want, f"batch {b}")
        assert np.max(np.abs(got_l[b * 32:(b + 1) * 32] - want_l)) < 1e-2
    if orc.ref_available():
        Or = torch.zeros_like(O)
        orc.ref().ref_flash_attention(Qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), Or.data_ptr(), None, batch, 32,
                                      8, q_len, kv_len, stride, 0.125, int(causal), None)
        torch.cuda.synchronize()
        check_close(got, orc.bf16_to_f32(to_u16(Or)), "vs reference kernel")


def test_unsupported_requests_are_refused(cuda):
    t = torch.zeros(32, 1, 64, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(8, 16, 64, dtype=torch.bfloat16, device=DEV)
    assert flash(t, k, k, t, None, 1, 1, 16, 16, d_head=128) == 3
    assert flash(t, k, k, t, None, 1, 1, 16, 16, dtype=0) == 3
    assert flash(t, k, k, t, None, 1, 1, 16, 16, heads=32, kv_heads=32) == 3
    assert flash(t, k, k, t, None, 1, 4, 2, 16) == 1  # causal with fewer keys than queries
