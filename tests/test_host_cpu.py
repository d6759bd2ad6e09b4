"""CPU checks of the product's host side: the C-ABI library loads and exports
what the header declares, the C++ block allocator matches the model, argument
errors come back as status codes.  No kernel is launched."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from llama_transformer_runtime_b200 import _lib, paged
from oracle import oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    src = open(os.path.join(ROOT, "include", header)).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b((?:pa|lt)_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    names = _declared("paged_attention.h")
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), n
    for n in _declared("legacy_kernels.h"):
        assert hasattr(L, n), n
    assert sorted(_declared("legacy_kernels.h")) == sorted(_lib.LEGACY_SYMBOLS)
    assert sorted(set(_lib.SYMBOLS)) == [n for n in names if n in _lib.SYMBOLS]
    assert set(names) <= set(_lib.SYMBOLS), set(names) - set(_lib.SYMBOLS)


def test_rope_tables_equal_oracle_bits():
    cos, sin = paged.build_rope_tables(4200)
    oc, os_ = orc.build_rope_tables(4200)
    assert np.array_equal(cos, oc) and np.array_equal(sin, os_)


def host_pool(nb, max_seqs=8, mb=None):
    return paged.KVPool(1, nb, 8, max_seqs, mb, device=-1)


def test_allocator_matches_model_under_random_traffic():
    rng = np.random.default_rng(7)
    nb = 257
    order = rng.permutation(nb)
    pool = host_pool(nb, 16, 64)
    pool.set_free_order(order)
    model = orc.BlockPoolModel(nb, order)
    live = []
    for step in range(3000):
        op = rng.integers(0, 10)
        if op < 2 and len(live) < 16:
            s = pool.create_seq()
            assert s == model.create()
            live.append(s)
        elif op < 3 and live:
            s = live.pop(rng.integers(0, len(live)))
            pool.free_seq(s)
            model.release(s)
        elif live:
            s = live[rng.integers(0, len(live))]
            new_len = model.lens[s] + int(rng.integers(0, 40))
            if (new_len + 15) // 16 > 64:
                continue
            ok = model.reserve(s, new_len)
            if ok:
                pool.reserve(s, new_len)
            else:
                with pytest.raises(_lib.PagedAttentionError) as ei:
                    pool.reserve(s, new_len)
                assert ei.value.code == 2
            assert pool.length(s) == model.lens[s]
            assert pool.block_table(s).tolist() == model.tables[s]
        assert pool.free_blocks() == len(model.free)
    used = [b for s in live for b in pool.block_table(s).tolist()]
    assert len(used) == len(set(used)) and len(used) + pool.free_blocks() == nb


def test_reserve_semantics():
    pool = host_pool(4, 2, 4)
    s = pool.create_seq()
    pool.reserve(s, 0)
    assert pool.block_table(s).size == 0
    pool.reserve(s, 1)
    assert pool.block_table(s).tolist() == [0]
    pool.reserve(s, 16)
    pool.reserve(s, 5)  # never shrinks, no-op
    assert pool.length(s) == 16 and pool.block_table(s).tolist() == [0]
    pool.reserve(s, 17)
    assert pool.block_table(s).tolist() == [0, 1]  # entry i covers positions [16i, 16i+16)
    with pytest.raises(_lib.PagedAttentionError) as ei:
        pool.reserve(s, 16 * 4 + 1)  # table too small
    assert ei.value.code == 1
    t = pool.create_seq()
    with pytest.raises(_lib.PagedAttentionError) as ei:
        pool.reserve(t, 16 * 3)  # only 2 blocks left
    assert ei.value.code == 2 and pool.length(t) == 0 and pool.free_blocks() == 2
    with pytest.raises(_lib.PagedAttentionError):
        pool.create_seq()  # both ids in use
    with pytest.raises(_lib.PagedAttentionError):
        pool.set_free_order(np.arange(4))  # blocks in use
    pool.free_seq(s)
    pool.free_seq(t)
    with pytest.raises(_lib.PagedAttentionError):
        pool.free_seq(t)
    with pytest.raises(_lib.PagedAttentionError):
        pool.set_free_order([0, 1, 1, 2])
    pool.set_free_order([3, 2, 1, 0])
    s = pool.create_seq()
    pool.reserve(s, 40)
    assert pool.block_table(s).tolist() == [3, 2, 1]


def test_argument_errors_are_status_codes():
    L = _lib.lib()
    h = C.c_void_p()
    assert L.pa_pool_create(C.byref(h), -1, 1, 0, 8, 1, 1) == 1
    assert L.pa_pool_create(C.byref(h), -1, 1, 4, 3, 1, 1) == 3
    assert b"kv_heads" in L.pa_last_error()
    pool = host_pool(4)
    s = pool.create_seq()
    pool.reserve(s, 3)
    with pytest.raises(_lib.PagedAttentionError) as ei:
        pool.batch_set([s])  # host-only pool has no device side
    assert ei.value.code == 6
    with pytest.raises(_lib.PagedAttentionError):
        pool.decode(0, 1, out=1)
    assert L.pa_merge_partials(None, None, 1, 1, None, None, None, None) == 1


def test_physical_layout_formula():
    # 16-byte chunks of one tile are a permutation of its 2048 bytes
    offs = sorted(paged.physical_chunk_offset(0, 8, 0, 0, r, c) for r in range(16) for c in range(8))
    assert offs == list(range(0, 2048, 16))
    assert paged.physical_chunk_offset(5, 8, 3, 1, 0, 0) == ((5 * 8 + 3) * 2 + 1) * 2048
    assert paged.physical_chunk_offset(0, 8, 0, 0, 9, 2) == 9 * 128 + ((2 ^ 1) << 4)


def test_drop_in_headers_compile(tmp_path):
    """A translation unit written against the reference's headers (same names,
    namespace, struct fields) compiles against the shims in include/."""
    import subprocess
    src = tmp_path / "caller.cu"
    src.write_text("""
#include "flashattention.h"
#include "rope.hpp"
#include "layout.hpp"
int caller(__nv_bfloat16* q, __nv_bfloat16* k, __nv_bfloat16* v, float* c, float* s) {
  launch_rope_qkv(q, q, k, k, v, v, c, s, 1, 0);
  transformer::FlashAttentionParams p = {};
  p.Q = q; p.K = k; p.V = v; p.O = q; p.L = nullptr;
  p.batch_size = 1; p.num_heads = ROPE_HEADS; p.num_kv_heads = ROPE_KV_HEADS;
  p.q_seq_len = 1; p.kv_seq_len = 1; p.kv_stride = 1; p.d_head = ROPE_HEAD_DIM;
  p.scale = 0.125f; p.causal = true; p.dtype = transformer::DType::BF16; p.stream = 0;
  transformer::launch_flash_attention(p);
  launch_flash_output_layout(q, q, 1);
  return 0;
}
""")
    r = subprocess.run(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                        os.path.join(ROOT, "include"), "-c", str(src), "-o", str(tmp_path / "caller.o")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_drop_in_class_headers_compile(tmp_path):
    """A translation unit that builds the reference's per-layer objects and its Transformer from a
    llama::LlamaWeights (src/runtime/transformer.cu:6-40) compiles against include/attention.hpp, ffn.hpp,
    weights.hpp and transformer.hpp (raw device pointers where the reference passes its Tensor)."""
    import subprocess
    src = tmp_path / "model_caller.cu"
    src.write_text("""
#include "attention.hpp"
#include "ffn.hpp"
#include "transformer.hpp"
int caller(llama::LlamaWeights& weights, float* cos_table, float* sin_table, __nv_bfloat16* in, __nv_bfloat16* out) {
  static_assert(llama::NUM_LAYERS == 16 && llama::VOCAB_SIZE == 128256, "model constants");
  runtime::Attention attention(weights.layers[0].input_layernorm, weights.layers[0].q_proj, weights.layers[0].k_proj,
                               weights.layers[0].v_proj, weights.layers[0].o_proj, cos_table, sin_table, 128, 0);
  runtime::FeedForward ffn(weights.layers[0].post_attention_layernorm, weights.layers[0].gate_proj,
                           weights.layers[0].up_proj, weights.layers[0].down_proj);
  attention.forward(in, out, 0, 1);
  ffn.forward(in, out, 1);
  runtime::Transformer transformer(weights, cos_table, sin_table, 128);
  transformer.forward(in, out, 0, 1);
  return transformer.get_key_cache(3) != nullptr && transformer.get_value_cache(15) != nullptr;
}
""")
    r = subprocess.run(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                        os.path.join(ROOT, "include"), "-c", str(src), "-o", str(tmp_path / "model_caller.o")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_projection_entries_validate_before_touching_a_device():
    """Argument checks of the projection entries run on the host, before any CUDA call: they must
    answer with a status and a message, never crash, with no GPU present."""
    import ctypes as C
    from llama_transformer_runtime_b200 import _lib
    L = _lib.lib()
    buf = (C.c_char * 64)()
    ptr = C.addressof(buf)
    # NULL argument
    assert L.pa_qkv_project(None, ptr, ptr, ptr, ptr, ptr, ptr, 1, 1, 2048, 2048, 512, 0, 0, 0, 0, 0, None) == 1
    assert b"NULL" in L.pa_last_error()
    # more rows than a decode step may bring
    rc = L.pa_qkv_project(ptr, ptr, ptr, ptr, ptr, ptr, ptr, 9, 1, 2048, 2048, 512, 0, 0, 0, 0, 0, None)
    assert rc != 0 and b"at most 8 rows" in L.pa_last_error()
    # hidden not a multiple of 64
    rc = L.pa_qkv_project(ptr, ptr, ptr, ptr, ptr, ptr, ptr, 1, 1, 2000, 2048, 512, 0, 0, 0, 0, 0, None)
    assert rc != 0 and b"hidden" in L.pa_last_error()
    rc = L.pa_out_project(ptr, ptr, None, ptr, 1, 1, 2048, 2040, 0, 0, 0, None)
    assert rc != 0 and b"cols" in L.pa_last_error()
    rc = L.pa_pack_projection_weights(ptr, ptr, 2048, 2048, None)
    assert rc != 0 and b"aliased" in L.pa_last_error()
    rc = L.pa_qkv_project_packed(ptr, ptr, ptr, ptr, ptr, ptr, ptr, 1, 1, 2048, 2048, 500, 0, 0, 0, 0, 0, ptr, None)
    assert rc != 0 and b"multiples of 64" in L.pa_last_error()
