"""Thin Python view of the C-ABI, used by the tests and the bench.

Every method forwards to one ``pa_*`` entry of ``libpaged_attention.so``; no
arithmetic happens here.  Device buffers are passed as torch CUDA tensors (or
raw integer addresses); torch is only the owner of that memory.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import AttentionWeights, FfnWeights, ModelWeights, check, lib

HEAD_DIM = 64
GROUP = 4
BLOCK_TOKENS = 16
TILE_BYTES = 2048


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    return x.data_ptr()


def build_rope_tables(seq_len: int):
    """fp32 cos/sin tables [seq_len, 32] (host), as the reference's runtime builds them."""
    cos = np.empty((seq_len, 32), np.float32)
    sin = np.empty((seq_len, 32), np.float32)
    check(lib().pa_build_rope_tables(cos.ctypes.data, sin.ctypes.data, seq_len))
    return cos, sin


def physical_chunk_offset(block: int, kv_heads: int, head: int, kv: int, slot: int, chunk: int) -> int:
    """Byte offset, inside one layer's storage, of 16-byte chunk ``chunk`` of token
    slot ``slot`` of tile (block, head, K if kv == 0 else V)."""
    return (((block * kv_heads + head) * 2 + kv) * TILE_BYTES + slot * 128
            + ((chunk ^ (slot & 7)) << 4))


class KVPool:
    """Paged KV cache of one GPU: storage, block allocator, block tables."""

    def __init__(self, num_layers: int, num_blocks: int, kv_heads: int = 8, max_seqs: int = 1,
                 max_blocks_per_seq: int | None = None, device: int = 0):
        self._h = C.c_void_p()
        self.num_layers, self.num_blocks, self.kv_heads = num_layers, num_blocks, kv_heads
        self.q_heads = kv_heads * GROUP
        self.max_seqs = max_seqs
        self.max_blocks_per_seq = max_blocks_per_seq or num_blocks
        self.device = device
        check(lib().pa_pool_create(C.byref(self._h), device, num_layers, num_blocks, kv_heads,
                                   max_seqs, self.max_blocks_per_seq))

    def close(self) -> None:
        if self._h:
            lib().pa_pool_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- allocator / tables (host) ----
    def free_blocks(self) -> int:
        n = C.c_int()
        check(lib().pa_pool_free_blocks(self._h, C.byref(n)))
        return n.value

    def set_free_order(self, order) -> None:
        o = np.ascontiguousarray(order, np.int32)
        check(lib().pa_pool_set_free_order(self._h, o.ctypes.data, int(o.size)))

    def create_seq(self) -> int:
        s = C.c_int()
        check(lib().pa_seq_create(self._h, C.byref(s)))
        return s.value

    def free_seq(self, seq: int) -> None:
        check(lib().pa_seq_free(self._h, seq))

    def reserve(self, seq: int, new_len: int) -> None:
        check(lib().pa_seq_reserve(self._h, seq, new_len))

    def length(self, seq: int) -> int:
        n = C.c_int()
        check(lib().pa_seq_length(self._h, seq, C.byref(n)))
        return n.value

    def block_table(self, seq: int) -> np.ndarray:
        t = C.POINTER(C.c_int32)()
        n = C.c_int()
        check(lib().pa_seq_block_table(self._h, seq, C.byref(t), C.byref(n)))
        if n.value == 0:
            return np.zeros((0,), np.int32)
        return np.ctypeslib.as_array(t, shape=(n.value,)).copy()

    def layer_storage(self, layer: int):
        p = C.c_void_p()
        b = C.c_uint64()
        check(lib().pa_pool_layer_storage(self._h, layer, C.byref(p), C.byref(b)))
        return p.value, b.value

    # ---- device work ----
    def batch_set(self, seq_ids, new_tokens=None, stream: int = 0) -> None:
        s = np.ascontiguousarray(seq_ids, np.int32)
        nt = None if new_tokens is None else np.ascontiguousarray(new_tokens, np.int32)
        check(lib().pa_batch_set(self._h, s.ctypes.data, None if nt is None else nt.ctypes.data,
                                 int(s.size), stream))

    def batch_set_sharded(self, seq_ids, new_tokens=None, q_rows=None, q_pos=None,
                          kv_pos_offset=None, stream: int = 0) -> None:
        arrs = [None if a is None else np.ascontiguousarray(a, np.int32)
                for a in (seq_ids, new_tokens, q_rows, q_pos, kv_pos_offset)]
        check(lib().pa_batch_set_sharded(self._h, *[None if a is None else a.ctypes.data for a in arrs],
                                         int(arrs[0].size), stream))

    def append(self, layer: int, q_in, k_in, v_in, cos, sin, q_out, stream: int = 0) -> None:
        check(lib().pa_append(self._h, layer, _ptr(q_in), _ptr(k_in), _ptr(v_in), _ptr(cos),
                              _ptr(sin), _ptr(q_out), stream))

    def decode(self, layer: int, q, out=None, out_stride: int | None = None, out_f32=None,
               lse=None, scale: float = 0.125, stream: int = 0) -> None:
        if out_stride is None:
            out_stride = self.q_heads * HEAD_DIM
        check(lib().pa_decode(self._h, layer, _ptr(q), _ptr(out), out_stride, _ptr(out_f32),
                              _ptr(lse), scale, stream))

    def decode_step(self, layer_begin: int, layer_end: int, q_in, k_in, v_in, q_layer_stride: int,
                    kv_layer_stride: int, cos, sin, q_rot, out, out_stride: int,
                    out_layer_stride: int, lse=None, scale: float = 0.125, stream: int = 0) -> None:
        check(lib().pa_decode_step(self._h, layer_begin, layer_end, _ptr(q_in), _ptr(k_in),
                                   _ptr(v_in), q_layer_stride, kv_layer_stride, _ptr(cos), _ptr(sin),
                                   _ptr(q_rot), _ptr(out), out_stride, out_layer_stride, _ptr(lse),
                                   scale, stream))

    def qkv_project_append(self, layer: int, x, wq, wk, wv, cos, sin, q_out, hidden: int = 2048,
                           stream: int = 0) -> None:
        """Projections of the batch's new tokens on the tensor cores, RoPE and cache append fused in."""
        check(lib().pa_qkv_project_append(self._h, layer, _ptr(x), _ptr(wq), _ptr(wk), _ptr(wv), _ptr(cos),
                                          _ptr(sin), _ptr(q_out), hidden, stream))

    def out_project_rows(self, attn, wo_packed, residual, out, rows: int, hidden: int = 2048, stream: int = 0) -> None:
        """out = bf16(residual + bf16(attn W_o)) for a prompt chunk, on the tensor cores."""
        check(lib().pa_out_project_rows(self._h, _ptr(attn), _ptr(wo_packed), _ptr(residual), _ptr(out), rows,
                                        hidden, int(wo_packed.shape[-1]), stream))

    def prefill(self, layer: int, q, out, lse=None, scale: float = 0.125, stream: int = 0) -> None:
        check(lib().pa_prefill(self._h, layer, _ptr(q), _ptr(out), _ptr(lse), scale, stream))

    def gather_kv(self, layer: int, seq: int, k_out, v_out, out_stride_tokens: int,
                  stream: int = 0) -> None:
        check(lib().pa_gather_kv(self._h, layer, seq, _ptr(k_out), _ptr(v_out), out_stride_tokens,
                                 stream))

    def check(self, stream: int = 0) -> None:
        check(lib().pa_pool_check(self._h, stream))

    def set_decode_cluster(self, mode: int) -> None:
        """One-layer decode kernel: -1 never clusters, 0 planner, 2/4/8/16 that cluster size."""
        check(lib().pa_pool_set_decode_cluster(self._h, mode))

    def set_decode_chunk_blocks(self, n: int) -> None:
        check(lib().pa_pool_set_decode_chunk_blocks(self._h, n))

    def set_step_kernel(self, enable: bool) -> None:
        """decode_step as one cooperative launch per step (default) or one kernel per layer."""
        check(lib().pa_pool_set_step_kernel(self._h, 1 if enable else 0))

    def set_layer_overlap(self, allow: bool) -> None:
        """False: layers of a decode step run strictly one after the other (dependent layers)."""
        check(lib().pa_pool_set_layer_overlap(self._h, 1 if allow else 0))

    def set_step_combiners(self, n: int) -> None:
        check(lib().pa_pool_set_step_combiners(self._h, n))

    def step_launches(self) -> int:
        """Decode steps of this pool that ran as one launch."""
        n = C.c_longlong(0)
        check(lib().pa_pool_step_launches(self._h, C.byref(n)))
        return int(n.value)

    def set_decode_shape(self, warps: int, stages: int) -> None:
        check(lib().pa_pool_set_decode_shape(self._h, warps, stages))


class Exchange:
    """Receive buffer + peer mappings for sequence-range sharded decode (one per rank).

    ``handle()`` gives the 64-byte CUDA IPC handle of this rank's buffer; after every
    rank's handle has been gathered (in rank order) ``connect()`` maps the peers."""

    HANDLE_BYTES = 64

    def __init__(self, device: int, rank: int, world: int, n_seqs: int = 1, kv_heads: int = 8):
        self._h = C.c_void_p()
        self.rank, self.world = rank, world
        check(lib().pa_exchange_create(C.byref(self._h), device, rank, world, n_seqs, kv_heads))

    def handle(self) -> bytes:
        buf = C.create_string_buffer(self.HANDLE_BYTES)
        check(lib().pa_exchange_handle(self._h, buf))
        return buf.raw

    def connect(self, handles) -> None:
        blob = b"".join(handles)
        assert len(blob) == self.world * self.HANDLE_BYTES
        check(lib().pa_exchange_connect(self._h, C.create_string_buffer(blob, len(blob))))

    def buffer(self):
        p, b = C.c_void_p(), C.c_uint64()
        check(lib().pa_exchange_buffer(self._h, C.byref(p), C.byref(b)))
        return p.value, b.value

    def connect_ptrs(self, peer_buffers) -> None:
        """Same-process variant: every rank's receive buffer as a device address."""
        arr = (C.c_void_p * self.world)(*[C.c_void_p(_ptr(b)) for b in peer_buffers])
        check(lib().pa_exchange_connect_ptrs(self._h, arr))

    def push(self, pool: "KVPool", layer: int, q, scale: float = 0.125, stream: int = 0) -> None:
        check(lib().pa_decode_push(pool._h, self._h, layer, _ptr(q), scale, stream))

    def merge(self, pool: "KVPool", out, out_stride: int, stream: int = 0) -> None:
        check(lib().pa_exchange_merge(pool._h, self._h, _ptr(out), out_stride, stream))

    def close(self) -> None:
        if self._h:
            lib().pa_exchange_destroy(self._h)
            self._h = C.c_void_p()


class HeadGather:
    """Row buffers + peer mappings for KV-head sharded decode (one per rank): the
    decode kernels of a step store every rank's head outputs into every rank's
    [layers, n_seqs, 2048] rows; ``step`` returns the device address of this
    step's rows once all ranks' contributions have arrived."""

    HANDLE_BYTES = 64

    def __init__(self, device: int, rank: int, world: int, n_seqs: int, layers: int, kv_heads: int):
        self._h = C.c_void_p()
        self.rank, self.world = rank, world
        check(lib().pa_gather_create(C.byref(self._h), device, rank, world, n_seqs, layers, kv_heads))

    def handle(self) -> bytes:
        buf = C.create_string_buffer(self.HANDLE_BYTES)
        check(lib().pa_gather_handle(self._h, buf))
        return buf.raw

    def connect(self, handles) -> None:
        blob = b"".join(handles)
        check(lib().pa_gather_connect(self._h, C.create_string_buffer(blob, len(blob))))

    def buffer(self):
        p, b = C.c_void_p(), C.c_uint64()
        check(lib().pa_gather_buffer(self._h, C.byref(p), C.byref(b)))
        return p.value, b.value

    def connect_ptrs(self, peer_buffers) -> None:
        arr = (C.c_void_p * self.world)(*[C.c_void_p(_ptr(b)) for b in peer_buffers])
        check(lib().pa_gather_connect_ptrs(self._h, arr))

    def step(self, pool: "KVPool", q_in, k_in, v_in, q_layer_stride: int, kv_layer_stride: int, cos, sin,
             q_rot, scale: float = 0.125, wait: bool = True, stream: int = 0):
        rows = C.c_void_p()
        check(lib().pa_decode_step_gathered(pool._h, self._h, _ptr(q_in), _ptr(k_in), _ptr(v_in),
                                            q_layer_stride, kv_layer_stride, _ptr(cos), _ptr(sin), _ptr(q_rot),
                                            scale, int(wait), stream, C.byref(rows)))
        return rows.value

    def wait(self, pool: "KVPool", stream: int = 0):
        rows = C.c_void_p()
        check(lib().pa_gather_wait(pool._h, self._h, stream, C.byref(rows)))
        return rows.value

    def close(self) -> None:
        if self._h:
            lib().pa_gather_destroy(self._h)
            self._h = C.c_void_p()


def decode_step_sharded(pool: "KVPool", xchg: Exchange, layer_begin: int, layer_end: int, q_in, k_in,
                        v_in, q_layer_stride: int, kv_layer_stride: int, cos, sin, q_rot, out,
                        out_stride: int, out_layer_stride: int, scale: float = 0.125,
                        stream: int = 0) -> None:
    check(lib().pa_decode_step_sharded(pool._h, xchg._h, layer_begin, layer_end, _ptr(q_in), _ptr(k_in),
                                       _ptr(v_in), q_layer_stride, kv_layer_stride, _ptr(cos), _ptr(sin),
                                       _ptr(q_rot), _ptr(out), out_stride, out_layer_stride, scale, stream))


def decode_step_sharded_colocated(pools, xchgs, layer_begin: int, layer_end: int, q_in, k_in, v_in,
                                  q_layer_stride: int, kv_layer_stride: int, cos, sin, q_rot, out,
                                  out_stride: int, out_layer_stride: int, scale: float = 0.125,
                                  stream: int = 0) -> None:
    """The sharded step of several ranks whose pools share one GPU, as one cooperative launch.
    pools, xchgs, q_in, k_in, v_in, q_rot, out are per-rank lists (k_in/v_in entries may be None)."""
    n = len(pools)
    arr = lambda xs: (C.c_void_p * n)(*[C.c_void_p(_ptr(x)) for x in xs])
    check(lib().pa_decode_step_sharded_colocated(
        (C.c_void_p * n)(*[p._h for p in pools]), (C.c_void_p * n)(*[x._h for x in xchgs]), n, layer_begin,
        layer_end, arr(q_in), arr(k_in), arr(v_in), q_layer_stride, kv_layer_stride, _ptr(cos), _ptr(sin),
        arr(q_rot), arr(out), out_stride, out_layer_stride, scale, stream))


def decode_noalloc_check(stream: int = 0) -> None:
    """Read and clear the status word of pa_decode_noalloc's scratch (raises on a recorded error)."""
    check(lib().pa_decode_noalloc_check(stream))


def decode_noalloc(cache_layer, num_blocks: int, kv_heads: int, block_tables, table_stride: int,
                   kv_lens, q, out, out_stride: int, lse=None, scale: float = 0.125,
                   stream: int = 0) -> None:
    """pa_decode_noalloc: decode over caller-owned buffers, for hosts that may not
    allocate device memory; at most PA_NOALLOC_MAX_SEQS (8) sequences per call."""
    lens = np.ascontiguousarray(kv_lens, np.int32)
    check(lib().pa_decode_noalloc(_ptr(cache_layer), num_blocks, kv_heads, _ptr(block_tables),
                                  table_stride, lens.ctypes.data, int(lens.size), _ptr(q), _ptr(out),
                                  out_stride, _ptr(lse), scale, stream))


def merge_partials(o_parts, lse_parts, n_parts: int, rows: int, out=None, out_f32=None,
                   lse_out=None, stream: int = 0) -> None:
    check(lib().pa_merge_partials(_ptr(o_parts), _ptr(lse_parts), n_parts, rows, _ptr(out),
                                  _ptr(out_f32), _ptr(lse_out), stream))


def qkv_project(x, wq, wk, wv, q, k, v, rows: int, layers: int = 1, hidden: int = 2048, stream: int = 0) -> None:
    """q, k, v = x Wq, x Wk, x Wv for the rows of a decode step, all layers in one launch.
    x [layers, rows, hidden]; wq [layers, hidden, q_cols]; wk, wv [layers, hidden, kv_cols]
    (the reference's row-major weights); outputs [layers, rows, cols]; contiguous bf16 tensors."""
    q_cols, kv_cols = int(wq.shape[-1]), int(wk.shape[-1])
    check(lib().pa_qkv_project(_ptr(x), _ptr(wq), _ptr(wk), _ptr(wv), _ptr(q), _ptr(k), _ptr(v), rows, layers,
                               hidden, q_cols, kv_cols, rows * hidden, hidden * q_cols, hidden * kv_cols,
                               rows * q_cols, rows * kv_cols, stream))


def rmsnorm_qkv_project(x, norm_w, wq, wk, wv, q, k, v, rows: int, layers: int = 1, hidden: int = 2048,
                        eps: float = 1e-5, stream: int = 0) -> None:
    """qkv_project with the RMSNorm in front of it as the kernel's prologue; norm_w [layers, hidden]."""
    q_cols, kv_cols = int(wq.shape[-1]), int(wk.shape[-1])
    check(lib().pa_rmsnorm_qkv_project(_ptr(x), _ptr(norm_w), hidden, eps, _ptr(wq), _ptr(wk), _ptr(wv), _ptr(q),
                                       _ptr(k), _ptr(v), rows, layers, hidden, q_cols, kv_cols, rows * hidden,
                                       hidden * q_cols, hidden * kv_cols, rows * q_cols, rows * kv_cols, stream))


def rmsnorm(x, w, y, rows: int, hidden: int = 2048, eps: float = 1e-5, stream: int = 0) -> None:
    check(lib().pa_rmsnorm(_ptr(x), _ptr(w), _ptr(y), rows, hidden, eps, stream))


def attention_weights(input_norm, wq, wk, wv, wo, hidden: int = 2048, eps: float = 1e-5) -> AttentionWeights:
    """Descriptor of per-layer weights stacked along a leading layer dimension (contiguous bf16 tensors):
    input_norm [layers, hidden] or None, wq [layers, hidden, q_cols], wk/wv [layers, hidden, kv_cols],
    wo [layers, q_cols, hidden]."""
    w = AttentionWeights()
    w.input_norm = _ptr(input_norm)
    w.wq, w.wk, w.wv, w.wo = _ptr(wq), _ptr(wk), _ptr(wv), _ptr(wo)
    w.norm_layer_stride = hidden
    w.wq_layer_stride = int(wq.shape[-2]) * int(wq.shape[-1])
    w.wkv_layer_stride = int(wk.shape[-2]) * int(wk.shape[-1])
    w.wo_layer_stride = int(wo.shape[-2]) * int(wo.shape[-1])
    w.rms_eps = eps
    w.hidden = hidden
    return w


def attention_step(pool: "KVPool", weights: AttentionWeights, layer_begin: int, layer_end: int, x_in, x_out,
                   cos, sin, add_residual: bool = True, xchg: "Exchange | None" = None, scale: float = 0.125,
                   stream: int = 0) -> None:
    """One decode step through the attention blocks of [layer_begin, layer_end), layers chained by their data."""
    check(lib().pa_attention_step(pool._h, xchg._h if xchg is not None else None, layer_begin, layer_end,
                                  C.byref(weights), _ptr(x_in), _ptr(x_out), int(add_residual), _ptr(cos), _ptr(sin),
                                  scale, stream))


def ffn_weights(ffn_norm, gate, up, down, eps: float = 1e-5) -> "FfnWeights":
    """Descriptor of per-layer feed-forward weights stacked along a leading layer dimension (contiguous
    bf16): ffn_norm [layers, hidden] or None, gate/up [layers, hidden, inter], down [layers, inter, hidden]."""
    w = FfnWeights()
    w.ffn_norm = _ptr(ffn_norm)
    w.gate, w.up, w.down = _ptr(gate), _ptr(up), _ptr(down)
    hidden, inter = int(gate.shape[-2]), int(gate.shape[-1])
    w.norm_layer_stride = hidden
    w.gate_layer_stride = w.up_layer_stride = w.down_layer_stride = hidden * inter
    w.rms_eps = eps
    w.hidden, w.inter = hidden, inter
    return w


def ffn(weights: "FfnWeights", layer: int, x, h_scratch, out, rows: int, add_residual: bool = True,
        stream: int = 0) -> None:
    """out = (x +) FeedForward(x) of one layer for 1 to 8 rows; h_scratch [rows, inter] bf16."""
    check(lib().pa_ffn(C.byref(weights), layer, _ptr(x), _ptr(h_scratch), _ptr(out), rows, int(add_residual), stream))


def ffn_rows(pool: "KVPool", packed_weights: "FfnWeights", layer: int, x, scratch, out, rows: int,
             add_residual: bool = True, stream: int = 0) -> None:
    """The feed-forward block for a prompt chunk on the tensor cores; gate/up/down of the descriptor packed by
    pack_projection_weights; scratch holds rows * (hidden + inter) bf16."""
    check(lib().pa_ffn_rows(pool._h, C.byref(packed_weights), layer, _ptr(x), _ptr(scratch), _ptr(out), rows,
                            int(add_residual), stream))


def block_step(pool: "KVPool", attention: AttentionWeights, ffn_w: "FfnWeights", layer_begin: int, layer_end: int,
               x_in, x_out, cos, sin, xchg: "Exchange | None" = None, scale: float = 0.125, stream: int = 0) -> None:
    """One decode step through the transformer blocks of [layer_begin, layer_end): attention block and
    feed-forward block with their residuals, layers chained by their data."""
    check(lib().pa_block_step(pool._h, xchg._h if xchg is not None else None, layer_begin, layer_end,
                              C.byref(attention), C.byref(ffn_w), _ptr(x_in), _ptr(x_out), _ptr(cos), _ptr(sin), scale,
                              stream))


def lm_head(x, final_norm, w_lm, logits, rows: int, eps: float = 1e-5, stream: int = 0) -> None:
    """logits [rows, vocab] bf16 = RMSNorm(x, final_norm) W_lm; w_lm [hidden, vocab] row-major."""
    check(lib().pa_lm_head(_ptr(x), _ptr(final_norm), eps, _ptr(w_lm), _ptr(logits), rows, int(w_lm.shape[-2]),
                           int(w_lm.shape[-1]), stream))


def argmax(logits, tokens, rows: int, stream: int = 0) -> None:
    """tokens[r] (int32) = index of the largest logit of row r, ties as the reference's kernel breaks them."""
    check(lib().pa_argmax(_ptr(logits), _ptr(tokens), rows, int(logits.shape[-1]), stream))


def embedding(tokens, table, out, rows: int, stream: int = 0) -> None:
    """out[r, :] = table[tokens[r], :]; tokens int32 on the device, table [vocab, hidden] bf16."""
    check(lib().pa_embedding(_ptr(tokens), _ptr(table), _ptr(out), rows, int(table.shape[-1]), int(table.shape[-2]),
                             stream))


def model_weights(embed_tokens, attention: AttentionWeights, ffn_w: "FfnWeights", final_norm, w_lm,
                  eps: float = 1e-5) -> "ModelWeights":
    """Descriptor of a whole model for decode_token; keeps the two block descriptors alive."""
    m = ModelWeights()
    m.embed_tokens = _ptr(embed_tokens)
    m.attention = C.pointer(attention)
    m.ffn = C.pointer(ffn_w)
    m.final_norm = _ptr(final_norm)
    m.lm_head = _ptr(w_lm)
    m.vocab = int(w_lm.shape[-1])
    m.rms_eps = eps
    m._keep = (attention, ffn_w)
    return m


def decode_token(pool: "KVPool", model: "ModelWeights", tokens_in, tokens_out, logits, cos, sin, scale: float = 0.125,
                 chained: bool = False, stream: int = 0) -> None:
    """One decode step of the whole model for the active batch: token ids (device int32) -> embedding ->
    every layer's block -> final norm + language-model head -> greedy token ids (device int32)."""
    check(lib().pa_decode_token(pool._h, C.byref(model), _ptr(tokens_in), _ptr(tokens_out), _ptr(logits), _ptr(cos),
                                _ptr(sin), scale, int(chained), stream))


def pack_projection_weights(w, stream: int = 0):
    """Row-major [..., hidden, cols] bf16 weights -> the tile image qkv_project_append reads (a new tensor)."""
    import torch
    packed = torch.empty_like(w)
    hidden, cols = int(w.shape[-2]), int(w.shape[-1])
    flat_in = w.reshape(-1, hidden, cols)
    flat_out = packed.reshape(-1, hidden, cols)
    for i in range(flat_in.shape[0]):
        check(lib().pa_pack_projection_weights(_ptr(flat_in[i]), _ptr(flat_out[i]), hidden, cols, stream))
    return packed


def qkv_project_packed(x, wq_packed, wk_packed, wv_packed, q, k, v, rows: int, status, layers: int = 1,
                       hidden: int = 2048, stream: int = 0) -> None:
    """qkv_project on weights repacked by pack_projection_weights; `status` is a device int32 tensor
    that receives the timeout code if a bounded wait runs out."""
    q_cols, kv_cols = int(wq_packed.shape[-1]), int(wk_packed.shape[-1])
    check(lib().pa_qkv_project_packed(_ptr(x), _ptr(wq_packed), _ptr(wk_packed), _ptr(wv_packed), _ptr(q), _ptr(k),
                                      _ptr(v), rows, layers, hidden, q_cols, kv_cols, rows * hidden,
                                      hidden * q_cols, hidden * kv_cols, rows * q_cols, rows * kv_cols,
                                      _ptr(status), stream))


def out_project(attn, wo, residual, out, rows: int, layers: int = 1, hidden: int = 2048, stream: int = 0) -> None:
    """out = bf16(residual + bf16(attn W_o)) for the rows of a decode step, all layers in one launch.
    attn [layers, rows, hidden]; wo [layers, hidden, cols]; residual (or None) and out [layers, rows, cols]."""
    cols = int(wo.shape[-1])
    check(lib().pa_out_project(_ptr(attn), _ptr(wo), _ptr(residual), _ptr(out), rows, layers, hidden, cols,
                               rows * hidden, hidden * cols, rows * cols, stream))
