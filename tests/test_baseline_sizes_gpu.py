"""GPU parity at the sizes the benchmark configurations are quoted on: the 16-layer decode step at
context 4096 + 1 through pa_decode_step (every layer against the oracle, layer 0 against the
reference's own kernel chain), and a 64-sequence ragged batch over a pool fragmented by freeing and
re-creating sequences (more (sequence, head) pairs than SMs, so the 4-warp ragged-wave plan runs)."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, check_close, f32_dev, to_dev, to_u16

pytestmark = pytest.mark.gpu


def _append_identity(pool, layers, seq, k, v):
    """k, v [8, n, 64]: final cache values of a fresh sequence, the same in every layer of `layers`."""
    n = k.shape[1]
    pool.reserve(seq, n)
    pool.batch_set([seq], [n])
    ones = torch.ones(n, 32, dtype=torch.float32, device=DEV)
    zeros = torch.zeros(n, 32, dtype=torch.float32, device=DEV)
    kd, vd = to_dev(k.transpose(1, 0, 2)), to_dev(v.transpose(1, 0, 2))
    for layer in layers:
        pool.append(layer, None, kd, vd, ones, zeros, None)


def test_decode_step_16_layers_ctx4096_plus_one(cuda):
    """16 layers, batch 1, context 4096 + 1: per layer a fused append + decode, all layers in one
    pa_decode_step call (one cooperative launch).  Every layer against the fp32 oracle; layer 0
    also against the reference chain (its RoPE kernels, its 128-byte append copies into the
    contiguous cache, its attention kernel at q_seq_len 1, its output layout kernel)."""
    rng = np.random.default_rng(2)
    layers, L = 16, 4096
    cos, sin = orc.build_rope_tables(L + 1)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    nb = (L + 1 + 15) // 16
    pool = paged.KVPool(layers, nb + nb // 4, 8, 1, nb + 1)
    pool.set_free_order(rng.permutation(nb + nb // 4))
    s = pool.create_seq()
    K = [orc.randn_bf16(rng, (8, L + 1, 64), 0.5) for _ in range(layers)]
    V = [orc.randn_bf16(rng, (8, L + 1, 64), 0.5) for _ in range(layers)]
    for layer in range(layers):  # reserving an unchanged length is a no-op
        _append_identity(pool, [layer], s, K[layer][:, :L], V[layer][:, :L])
    q_new = orc.randn_bf16(rng, (layers, 1, 32, 64))
    k_new = orc.randn_bf16(rng, (layers, 1, 8, 64))
    v_new = orc.randn_bf16(rng, (layers, 1, 8, 64))
    pool.reserve(s, L + 1)
    assert pool.block_table(s).size == 257
    pool.batch_set([s])
    qd, kd, vd = to_dev(q_new), to_dev(k_new), to_dev(v_new)
    q_rot = torch.zeros_like(qd)
    out = torch.zeros(layers, 1, 2048, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(layers, 1, 32, dtype=torch.float32, device=DEV)
    before = pool.step_launches()
    pool.decode_step(0, layers, qd, kd, vd, 2048, 512, cos_d, sin_d, q_rot, out, 2048, 2048, lse)
    torch.cuda.synchronize()
    pool.check()
    assert pool.step_launches() == before + 1, "the 16-layer step did not run as one launch"
    got = orc.bf16_to_f32(to_u16(out))
    for layer in range(layers):
        K[layer][:, L] = orc.rope(k_new[layer], cos, sin, L, 1)[:, 0]
        V[layer][:, L] = v_new[layer, 0]
        O, want_lse = orc.attention(orc.rope(q_new[layer], cos, sin, L, 1), K[layer], V[layer], L + 1)
        check_close(got[layer, 0], O[:, 0].reshape(-1), f"layer {layer}")
        assert np.max(np.abs(lse[layer, 0].cpu().numpy() - want_lse[:, 0])) < 1e-2, layer
    # the appended rows are in the cache bit for bit
    gk = torch.zeros(8, L + 1, 64, dtype=torch.bfloat16, device=DEV)
    gv = torch.zeros_like(gk)
    pool.gather_kv(5, s, gk, gv, L + 1)
    torch.cuda.synchronize()
    assert np.array_equal(to_u16(gk), K[5]) and np.array_equal(to_u16(gv), V[5])
    if orc.ref_available():
        ref = orc.ref()
        max_seq = L + 8
        kc = torch.zeros(8, max_seq, 64, dtype=torch.bfloat16, device=DEV)
        vc = torch.zeros_like(kc)
        kc[:, :L] = to_dev(K[0][:, :L])
        vc[:, :L] = to_dev(V[0][:, :L])
        qf = torch.empty(32, 1, 64, dtype=torch.bfloat16, device=DEV)
        kf = torch.empty(8, 1, 64, dtype=torch.bfloat16, device=DEV)
        vf = torch.empty(8, 1, 64, dtype=torch.bfloat16, device=DEV)
        of = torch.empty(32, 1, 64, dtype=torch.bfloat16, device=DEV)
        orow = torch.empty(1, 2048, dtype=torch.bfloat16, device=DEV)
        torch.cuda.synchronize()
        ref.ref_rope_qkv(qd[0].data_ptr(), qf.data_ptr(), kd[0].data_ptr(), kf.data_ptr(), vd[0].data_ptr(),
                         vf.data_ptr(), cos_d.data_ptr(), sin_d.data_ptr(), 1, L)
        assert ref.ref_append_memcpy_loop(kc.data_ptr(), vc.data_ptr(), kf.data_ptr(), vf.data_ptr(), max_seq, L, 1) == 0
        ref.ref_flash_attention(qf.data_ptr(), kc.data_ptr(), vc.data_ptr(), of.data_ptr(), None, 1, 32, 8, 1, L + 1,
                                max_seq, 0.125, 1, None)
        ref.ref_flash_output_layout(of.data_ptr(), orow.data_ptr(), 1)
        torch.cuda.synchronize()
        check_close(got[0, 0], orc.bf16_to_f32(to_u16(orow))[0], "layer 0 vs the reference chain")
    pool.close()


def test_ragged_batch_of_64_over_a_fragmented_pool(cuda):
    """64 sequences with seeded-uniform lengths in [128, 4096] (the batched-decode configuration's
    [1024, 32768] scaled by 1/8), a shared pool, two rounds of freeing and re-creating a third of the
    sequences, then a 2-layer decode step with the append fused in: 512 (sequence, head) pairs, more
    than the SMs, so the CTAs are 4 warps wide and come in ragged waves.  Every sequence and layer
    against the oracle; the appended rows bit-exact."""
    rng = np.random.default_rng(2024)
    n, layers = 64, 2
    lens = rng.integers(128, 4097, n).astype(int)
    blocks = int(sum((l + 1 + 15) // 16 for l in lens))
    nb = blocks + blocks // 2 + 64
    pool = paged.KVPool(layers, nb, 8, n, (4096 + 1 + 15) // 16 + 1)
    pool.set_free_order(rng.permutation(nb))
    data = {}

    def create(L):
        s = pool.create_seq()
        k = orc.randn_bf16(rng, (8, L + 1, 64), 0.5)
        v = orc.randn_bf16(rng, (8, L + 1, 64), 0.5)
        _append_identity(pool, range(layers), s, k[:, :L], v[:, :L])
        data[s] = (k, v, L)

    for L in lens:
        create(int(L))
    for _ in range(2):
        victims = rng.choice(sorted(data), n // 3, replace=False)
        for s in victims:
            pool.free_seq(int(s))
            del data[int(s)]
        for L in rng.integers(128, 4097, len(victims)):
            create(int(L))
    torch.cuda.synchronize()
    ids = sorted(data)
    assert len(ids) == n
    # fragmentation really happened: some table is not a run of the free order
    tabs = [pool.block_table(s) for s in ids]
    cos, sin = orc.build_rope_tables(4096 + 2)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    q_new = orc.randn_bf16(rng, (layers, n, 32, 64))
    k_new = orc.randn_bf16(rng, (layers, n, 8, 64))
    v_new = orc.randn_bf16(rng, (layers, n, 8, 64))
    for s in ids:
        pool.reserve(s, data[s][2] + 1)
    pool.batch_set(ids)
    qd, kd, vd = to_dev(q_new), to_dev(k_new), to_dev(v_new)
    q_rot = torch.zeros_like(qd)
    out = torch.zeros(layers, n, 2048, dtype=torch.bfloat16, device=DEV)
    pool.decode_step(0, layers, qd, kd, vd, n * 2048, n * 512, cos_d, sin_d, q_rot, out, 2048, n * 2048)
    torch.cuda.synchronize()
    pool.check()
    got = orc.bf16_to_f32(to_u16(out))
    for i, s in enumerate(ids):
        k, v, L = data[s]
        for layer in range(layers):
            kk, vv = k.copy(), v.copy()
            kk[:, L] = orc.rope(k_new[layer, i][None], cos, sin, L, 1)[:, 0]
            vv[:, L] = v_new[layer, i]
            O, _ = orc.attention(orc.rope(q_new[layer, i][None], cos, sin, L, 1), kk, vv, L + 1)
            check_close(got[layer, i], O[:, 0].reshape(-1), f"sequence {s} (length {L}) layer {layer}")
            if i % 16 == 0:
                gk = torch.zeros(8, L + 1, 64, dtype=torch.bfloat16, device=DEV)
                gv = torch.zeros_like(gk)
                pool.gather_kv(layer, s, gk, gv, L + 1)
                torch.cuda.synchronize()
                assert np.array_equal(to_u16(gk), kk) and np.array_equal(to_u16(gv), vv)
    assert any(np.any(np.diff(t) != 1) for t in tabs)
    pool.close()
