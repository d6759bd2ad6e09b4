"""pa_decode_noalloc: decode for hosts that may not allocate device memory
(a plug-in inside a server that owns the GPU's memory, a loop that cannot take
an allocation's device-wide synchronisation, a fixed memory budget).  It runs
the decode kernel over caller-owned buffers with its split-KV scratch in a
fixed array inside the library, so it must give the same answer as pa_decode,
call after call, although every call reuses that array.

The file name sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import _lib, paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, check_close, fill_cache, to_dev, to_u16

pytestmark = pytest.mark.gpu


def _pool_with_sequences(rng, lens, kv_heads=8):
    nb = sum((L + 15) // 16 for L in lens) + 9
    stride = max((L + 15) // 16 for L in lens) + 2
    pool = paged.KVPool(1, nb, kv_heads, len(lens), stride)
    pool.set_free_order(rng.permutation(nb))
    seqs, caches = [], []
    for L in lens:
        k = orc.randn_bf16(rng, (kv_heads, L, 64), 0.5)
        v = orc.randn_bf16(rng, (kv_heads, L, 64), 0.5)
        s = pool.create_seq()
        fill_cache(pool, 0, s, k, v)
        seqs.append(s)
        caches.append((k, v))
    tables = np.zeros((len(lens), stride), np.int32)
    for i, s in enumerate(seqs):
        t = pool.block_table(s)
        tables[i, :t.size] = t
    return pool, seqs, torch.from_numpy(tables).to(DEV), stride, caches


def test_noalloc_matches_pool_decode_twice_in_a_row(cuda):
    rng = np.random.default_rng(77)
    # call 1: three ragged sequences, several split-KV chunks each; call 2: other
    # lengths and another pool, so stale partials/tickets of call 1 would show
    for call, lens in enumerate([(3000, 17, 640), (5, 2049)]):
        pool, seqs, tables_d, stride, caches = _pool_with_sequences(rng, lens)
        n = len(lens)
        q = to_dev(orc.randn_bf16(rng, (n, 32, 64)))
        want = torch.zeros(n, 2048, dtype=torch.bfloat16, device=DEV)
        want_lse = torch.zeros(n, 32, dtype=torch.float32, device=DEV)
        pool.batch_set(seqs)
        pool.decode(0, q, want, 2048, None, want_lse)
        got = torch.full((n, 2048), 3.0, dtype=torch.bfloat16, device=DEV)
        got_lse = torch.zeros(n, 32, dtype=torch.float32, device=DEV)
        ptr, _ = pool.layer_storage(0)
        paged.decode_noalloc(ptr, pool.num_blocks, 8, tables_d, stride, list(lens), q, got, 2048, got_lse)
        torch.cuda.synchronize()
        pool.check()
        paged.decode_noalloc_check()  # this entry's own status word (the pool's is another one)
        # same kernel, same arithmetic; only the split may differ (the pool may plan other chunks)
        check_close(orc.bf16_to_f32(to_u16(got)), orc.bf16_to_f32(to_u16(want)), f"call {call}")
        assert torch.max(torch.abs(got_lse - want_lse)).item() < 1e-2
        # and against the CPU oracle directly
        for i, L in enumerate(lens):
            O, want_l = orc.attention(to_u16(q[i])[:, None, :], caches[i][0], caches[i][1], L)
            check_close(orc.bf16_to_f32(to_u16(got[i])), O[:, 0].reshape(-1), f"call {call} sequence {i} vs oracle")
            assert np.max(np.abs(got_lse[i].cpu().numpy() - want_l[:, 0])) < 1e-2
        pool.close()


def test_noalloc_reports_a_block_id_outside_the_cache(cuda):
    """The caller owns the block tables here, so a bad id is this entry's most likely misuse.  The
    kernel's range check reads block 0 instead of the bad one (no access outside the cache), records
    it, and pa_decode_noalloc_check hands it back as PA_ERR_INVALID_ARG and clears the word."""
    rng = np.random.default_rng(79)
    lens = (40, 333)
    pool, seqs, tables_d, stride, _ = _pool_with_sequences(rng, lens)
    q = to_dev(orc.randn_bf16(rng, (2, 32, 64)))
    out = torch.zeros(2, 2048, dtype=torch.bfloat16, device=DEV)
    ptr, _ = pool.layer_storage(0)
    bad = tables_d.clone()
    bad[1, 3] = pool.num_blocks + 5
    paged.decode_noalloc(ptr, pool.num_blocks, 8, bad, stride, list(lens), q, out, 2048)
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.decode_noalloc_check()
    assert ei.value.code == 1
    paged.decode_noalloc_check()  # cleared
    # a good call afterwards is clean and right
    paged.decode_noalloc(ptr, pool.num_blocks, 8, tables_d, stride, list(lens), q, out, 2048)
    paged.decode_noalloc_check()
    want = torch.zeros(2, 2048, dtype=torch.bfloat16, device=DEV)
    pool.batch_set(seqs)
    pool.decode(0, q, want, 2048)
    torch.cuda.synchronize()
    check_close(orc.bf16_to_f32(to_u16(out)), orc.bf16_to_f32(to_u16(want)), "after a reported bad block id")
    # a stream under capture is refused (the entry copies its descriptor from host memory)
    import ctypes
    cudart = ctypes.CDLL("libcudart.so.12")
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    graph = ctypes.c_void_p()
    assert cudart.cudaStreamBeginCapture(ctypes.c_void_p(side.cuda_stream), 2) == 0  # relaxed mode
    try:
        with pytest.raises(_lib.PagedAttentionError) as ei:
            paged.decode_noalloc(ptr, pool.num_blocks, 8, tables_d, stride, list(lens), q, out, 2048,
                                 stream=side.cuda_stream)
        assert ei.value.code == 6
    finally:
        assert cudart.cudaStreamEndCapture(ctypes.c_void_p(side.cuda_stream), ctypes.byref(graph)) == 0
        if graph.value:
            cudart.cudaGraphDestroy(graph)
    pool.close()


def test_noalloc_rejects_more_than_its_fixed_scratch_holds(cuda):
    rng = np.random.default_rng(78)
    lens = [20] * 9
    pool, seqs, tables_d, stride, _ = _pool_with_sequences(rng, lens)
    q = to_dev(orc.randn_bf16(rng, (9, 32, 64)))
    out = torch.zeros(9, 2048, dtype=torch.bfloat16, device=DEV)
    ptr, _ = pool.layer_storage(0)
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.decode_noalloc(ptr, pool.num_blocks, 8, tables_d, stride, lens, q, out, 2048)
    assert ei.value.code == 3 and "PA_NOALLOC_MAX_SEQS" in str(ei.value)
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.decode_noalloc(ptr, pool.num_blocks, 8, tables_d, stride, [16 * stride + 1], q, out, 2048)
    assert ei.value.code == 1
    # and the first eight of them are served
    paged.decode_noalloc(ptr, pool.num_blocks, 8, tables_d, stride, lens[:8], q, out, 2048)
    want = torch.zeros(9, 2048, dtype=torch.bfloat16, device=DEV)
    pool.batch_set(seqs)
    pool.decode(0, q, want, 2048)
    torch.cuda.synchronize()
    check_close(orc.bf16_to_f32(to_u16(out[:8])), orc.bf16_to_f32(to_u16(want[:8])), "eight sequences")
    pool.close()
