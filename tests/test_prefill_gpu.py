"""GPU parity of K3 (causal GQA prefill on tcgen05): against the fp32 oracle and
the reference's own kernel, tolerance max-abs 2e-2 / rel 1e-2 on bf16 outputs."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, check_close, f32_dev, fill_cache, to_dev, to_u16

pytestmark = pytest.mark.gpu


def run_prefill(rng, position, tokens, kv_heads=8, want_lse=True):
    """Cache holds `position` earlier tokens; `tokens` new ones are appended with
    RoPE and attend causally.  Returns (out [tokens, heads*64] fp32, lse, inputs)."""
    qh = 4 * kv_heads
    L = position + tokens
    cos, sin = orc.build_rope_tables(L)
    nb = (L + 15) // 16 + 6
    pool = paged.KVPool(1, nb, kv_heads, 1)
    pool.set_free_order(rng.permutation(nb))
    s = pool.create_seq()
    k_old = orc.randn_bf16(rng, (kv_heads, position, 64), 0.5)
    v_old = orc.randn_bf16(rng, (kv_heads, position, 64), 0.5)
    if position:
        fill_cache(pool, 0, s, k_old, v_old)
    q = orc.randn_bf16(rng, (tokens, qh, 64))
    k = orc.randn_bf16(rng, (tokens, kv_heads, 64))
    v = orc.randn_bf16(rng, (tokens, kv_heads, 64))
    pool.reserve(s, L)
    pool.batch_set([s], [tokens])
    qd = to_dev(q)
    pool.append(0, qd, to_dev(k), to_dev(v), f32_dev(cos), f32_dev(sin), qd)
    out = torch.full((tokens, qh * 64), 9.0, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(qh, tokens, dtype=torch.float32, device=DEV) if want_lse else None
    pool.prefill(0, qd, out, lse, 0.125)
    torch.cuda.synchronize()
    pool.check()
    q_rot = orc.rope(q, cos, sin, position, 1)                      # [qh, tokens, 64]
    kc = np.concatenate([k_old, orc.rope(k, cos, sin, position, 1)], 1)
    vc = np.concatenate([v_old, orc.transpose_v(v)], 1)
    pool.close()
    return (orc.bf16_to_f32(to_u16(out)), None if lse is None else lse.cpu().numpy(), q_rot, kc, vc)


@pytest.mark.parametrize("position,tokens", [
    (0, 1), (0, 37), (0, 128), (0, 129), (0, 200), (45, 20), (100, 300), (128, 128), (7, 512),
])
def test_prefill_vs_oracle(cuda, position, tokens):
    rng = np.random.default_rng(1000 + position * 7 + tokens)
    got, lse, q_rot, kc, vc = run_prefill(rng, position, tokens)
    O, L = orc.attention(q_rot, kc, vc, position + tokens, causal=True)
    want = orc.output_layout(O)
    check_close(got, want, f"prefill pos {position} tokens {tokens}")
    assert np.max(np.abs(lse - L)) < 1e-2


def test_prefill_config3_one_layer(cuda):
    """2048 tokens at position 0 (one layer of the 2048-token prefill configuration)."""
    rng = np.random.default_rng(3)
    got, lse, q_rot, kc, vc = run_prefill(rng, 0, 2048)
    O, L = orc.attention(q_rot, kc, vc, 2048, causal=True)
    check_close(got, orc.output_layout(O), "prefill 2048")
    assert np.max(np.abs(lse - L)) < 1e-2


@pytest.mark.parametrize("kv_heads", [1, 2])
def test_prefill_sharded_heads(cuda, kv_heads):
    rng = np.random.default_rng(40 + kv_heads)
    got, lse, q_rot, kc, vc = run_prefill(rng, 33, 150, kv_heads)
    O, _ = orc.attention(q_rot, kc, vc, 183, causal=True)
    check_close(got, orc.output_layout(O), f"prefill {kv_heads} kv heads")


@pytest.mark.skipif(not orc.ref_available(), reason="reference kernels were not built")
@pytest.mark.parametrize("position,tokens", [(0, 256), (45, 20), (0, 2048)])
def test_prefill_vs_reference_kernel(cuda, position, tokens):
    rng = np.random.default_rng(50 + tokens)
    got, lse, q_rot, kc, vc = run_prefill(rng, position, tokens)
    ref = orc.ref()
    L = position + tokens
    qd, kd, vd = to_dev(q_rot), to_dev(kc), to_dev(vc)
    of = torch.zeros(32, tokens, 64, dtype=torch.bfloat16, device=DEV)
    rl = torch.zeros(32, tokens, dtype=torch.float32, device=DEV)
    ol = torch.zeros(tokens, 2048, dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    ref.ref_flash_attention(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), of.data_ptr(), rl.data_ptr(),
                            1, 32, 8, tokens, L, L, 0.125, 1, None)
    ref.ref_flash_output_layout(of.data_ptr(), ol.data_ptr(), tokens)
    torch.cuda.synchronize()
    check_close(got, orc.bf16_to_f32(to_u16(ol)), "vs reference kernel")
    assert np.max(np.abs(lse - rl.cpu().numpy())) < 1e-2
