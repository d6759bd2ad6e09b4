"""GPU parity of K1 (fused RoPE + paged append): bit-exact against the oracle,
against the raw physical layout, and against the reference's own kernels."""
import ctypes as C

import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, f32_dev, read_logical_pool, to_dev, to_u16

pytestmark = pytest.mark.gpu

DEFAULT_VARIANT = 1  # must equal the library's default (pinned against the reference below)


def run_append(pool, seqs, new_tokens, q, k, v, cos_d, sin_d, want_q=True):
    pool.batch_set(seqs, new_tokens)
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    qo = torch.empty_like(qd) if want_q else None
    pool.append(0, qd, kd, vd, cos_d, sin_d, qo)
    torch.cuda.synchronize()
    pool.check()
    return None if qo is None else to_u16(qo)


def test_append_bit_exact_vs_oracle(cuda):
    variant = DEFAULT_VARIANT
    rng = np.random.default_rng(10 + variant)
    nb, max_pos = 24, 300
    cos, sin = orc.build_rope_tables(max_pos)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    pool = paged.KVPool(1, nb, 8, 1)
    pool.set_free_order(rng.permutation(nb))
    s = pool.create_seq()
    model = np.zeros((nb, 8, 2, 16, 64), np.uint16)
    pos = 0
    for tok in (37, 1, 1, 26, 1, 130):  # ragged, crossing block borders, single-token steps
        q = orc.randn_bf16(rng, (tok, 32, 64))
        k = orc.randn_bf16(rng, (tok, 8, 64))
        v = orc.randn_bf16(rng, (tok, 8, 64))
        pool.reserve(s, pos + tok)
        qo = run_append(pool, [s], [tok], q, k, v, cos_d, sin_d)
        table = pool.block_table(s)
        assert np.array_equal(qo, orc.rope(q, cos, sin, pos, variant, out_token_major=True))
        orc.paged_append(model, table, orc.rope(k, cos, sin, pos, variant), orc.transpose_v(v), pos)
        pos += tok
    # placement in the raw storage, decoded with the documented layout only
    assert np.array_equal(read_logical_pool(pool, 0), model)
    # and through the product's gather
    kd = torch.zeros(8, pos + 5, 64, dtype=torch.bfloat16, device=DEV)
    vd = torch.zeros_like(kd)
    pool.gather_kv(0, s, kd, vd, pos + 5)
    torch.cuda.synchronize()
    gk, gv = orc.paged_gather(model, pool.block_table(s), pos)
    assert np.array_equal(to_u16(kd)[:, :pos], gk) and np.array_equal(to_u16(vd)[:, :pos], gv)
    assert not to_u16(kd)[:, pos:].any()
    pool.close()


@pytest.mark.parametrize("kv_heads", [1, 2, 4, 8])
def test_append_multi_sequence_and_sharded_heads(cuda, kv_heads):
    rng = np.random.default_rng(20 + kv_heads)
    nb, n_seq = 64, 5
    cos, sin = orc.build_rope_tables(200)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    pool = paged.KVPool(2, nb, kv_heads, n_seq, 16)
    pool.set_free_order(rng.permutation(nb))
    seqs = [pool.create_seq() for _ in range(n_seq)]
    lens = [0] * n_seq
    model = np.zeros((nb, kv_heads, 2, 16, 64), np.uint16)
    for step in range(4):
        new = [int(x) for x in rng.integers(0 if step else 1, 40, n_seq)]
        if step == 3:
            new = [1] * n_seq
        for s, n in zip(seqs, new):
            pool.reserve(s, lens[s] + n)
        rows = sum(new)
        q = orc.randn_bf16(rng, (rows, 4 * kv_heads, 64))
        k = orc.randn_bf16(rng, (rows, kv_heads, 64))
        v = orc.randn_bf16(rng, (rows, kv_heads, 64))
        qo = run_append(pool, seqs, None if step == 3 else new, q, k, v, cos_d, sin_d)
        r = 0
        for s, n in zip(seqs, new):
            if n:
                assert np.array_equal(qo[r:r + n],
                                      orc.rope(q[r:r + n], cos, sin, lens[s], DEFAULT_VARIANT, True))
                orc.paged_append(model, pool.block_table(s),
                                 orc.rope(k[r:r + n], cos, sin, lens[s], DEFAULT_VARIANT),
                                 orc.transpose_v(v[r:r + n]), lens[s])
            lens[s] += n
            r += n
    assert np.array_equal(read_logical_pool(pool, 0), model)
    assert not read_logical_pool(pool, 1).any()  # the other layer is untouched
    pool.close()


@pytest.mark.skipif(not orc.ref_available(), reason="reference kernels were not built")
@pytest.mark.parametrize("position,tokens", [(0, 37), (512, 1), (45, 20), (0, 256)])
def test_append_equals_reference_cache(cuda, position, tokens):
    """The reference: launch_rope_qkv, then its 128-byte copy loop into the
    contiguous [8, max_seq, 64] cache.  Ours: one pa_append.  Same bits."""
    rng = np.random.default_rng(30 + position)
    ref = orc.ref()
    max_seq = position + tokens + 11
    cos, sin = orc.build_rope_tables(max_seq)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    q = orc.randn_bf16(rng, (tokens, 32, 64))
    k = orc.randn_bf16(rng, (tokens, 8, 64))
    v = orc.randn_bf16(rng, (tokens, 8, 64))
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    qf = torch.empty(32, tokens, 64, dtype=torch.bfloat16, device=DEV)
    kf = torch.empty(8, tokens, 64, dtype=torch.bfloat16, device=DEV)
    vf = torch.empty(8, tokens, 64, dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    ref.ref_rope_qkv(qd.data_ptr(), qf.data_ptr(), kd.data_ptr(), kf.data_ptr(), vd.data_ptr(),
                     vf.data_ptr(), cos_d.data_ptr(), sin_d.data_ptr(), tokens, position)
    kc = torch.zeros(8, max_seq, 64, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    torch.cuda.synchronize()
    assert ref.ref_append_memcpy_loop(kc.data_ptr(), vc.data_ptr(), kf.data_ptr(), vf.data_ptr(),
                                      max_seq, position, tokens) == 0
    torch.cuda.synchronize()

    # which rounding of y0 did the compiler give the reference kernel?
    matches = [var for var in (0, 1, 2)
               if np.array_equal(to_u16(kf), orc.rope(k, cos, sin, position, var))
               and np.array_equal(to_u16(qf), orc.rope(q, cos, sin, position, var))]
    assert DEFAULT_VARIANT in matches, f"reference rope matches oracle variants {matches}"

    nb = (max_seq + 15) // 16 + 3
    pool = paged.KVPool(1, nb, 8, 1)
    pool.set_free_order(rng.permutation(nb))
    s = pool.create_seq()
    pool.reserve(s, position + tokens)
    pool.batch_set([s], [tokens])
    qo = torch.empty_like(qd)
    pool.append(0, qd, kd, vd, cos_d, sin_d, qo)
    gk = torch.zeros(8, max_seq, 64, dtype=torch.bfloat16, device=DEV)
    gv = torch.zeros_like(gk)
    pool.gather_kv(0, s, gk, gv, max_seq)
    torch.cuda.synchronize()
    pool.check()
    # positions below `position` were never written on either side (zero)
    assert torch.equal(gk.view(torch.int16), kc.view(torch.int16))
    assert torch.equal(gv.view(torch.int16), vc.view(torch.int16))
    assert torch.equal(qo.view(torch.int16).permute(1, 0, 2), qf.view(torch.int16))
    pool.close()
