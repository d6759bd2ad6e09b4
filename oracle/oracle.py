"""TEST INFRASTRUCTURE — ctypes binding of the CPU oracle (oracle.c) and of the
reference's own CUDA kernels (``_ref/libref.so``, GPU only).

Only tests, ``__graft_entry__.smoke()`` and the CPU/reference legs of
``bench.py`` may import this module.  The product package never does.

bf16 tensors are numpy ``uint16`` arrays holding the bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

HEAD_DIM = 64
ROTARY_DIM = 32
BLOCK_TOKENS = 16


def build(ref_dir: str | None = None) -> None:
    """Compile liboracle.so and, when the reference checkout is reachable,
    ``_ref/libref.so`` from the reference's sources where they lie."""
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    cmd = ["make", "-C", _HERE, "ref"]
    if ref_dir:
        cmd.append(f"REF={ref_dir}")
    subprocess.run(cmd, check=True, capture_output=True)
    cmd[3] = "callers"
    subprocess.run(cmd, check=True, capture_output=True)


def _p(a, t=C.c_void_p):
    if a is None:
        return None
    return a.ctypes.data_as(t)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
        _LIB = C.CDLL(path)
        _LIB.orc_f32_to_bf16.restype = C.c_uint16
        _LIB.orc_f32_to_bf16.argtypes = [C.c_float]
        _LIB.orc_bf16_to_f32.restype = C.c_float
        _LIB.orc_bf16_to_f32.argtypes = [C.c_uint16]
        _LIB.orc_num_threads.restype = C.c_int
    return _LIB


# ---- bf16 helpers (numpy, vectorised; same rounding as orc_f32_to_bf16) ----
def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + (0x7FFF + ((u >> 16) & 1))) >> 16
    r = np.where(nan, 0x7FFF, r)
    return r.astype(np.uint16)


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def randn_bf16(rng: np.random.Generator, shape, scale: float = 1.0) -> np.ndarray:
    return f32_to_bf16((rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)))


# ---- oracle entry points ----------------------------------------------------
def build_rope_tables(seq_len: int):
    cos = np.empty((seq_len, ROTARY_DIM), np.float32)
    sin = np.empty((seq_len, ROTARY_DIM), np.float32)
    lib().orc_build_rope_tables(_p(cos), _p(sin), C.c_int(seq_len))
    return cos, sin


def rope(x: np.ndarray, cos, sin, position_offset: int, y0_variant: int = 1,
         out_token_major: bool = False) -> np.ndarray:
    """x [tokens, heads, 64] -> [heads, tokens, 64] (or token-major)."""
    tokens, heads, d = x.shape
    assert d == HEAD_DIM
    x = np.ascontiguousarray(x, np.uint16)
    out = np.empty((tokens, heads, d) if out_token_major else (heads, tokens, d), np.uint16)
    lib().orc_rope(_p(x), _p(out), _p(cos), _p(sin), C.c_int(tokens), C.c_int(heads),
                   C.c_int(position_offset), C.c_int(y0_variant), C.c_int(int(out_token_major)))
    return out


def transpose_v(v: np.ndarray) -> np.ndarray:
    tokens, heads, d = v.shape
    v = np.ascontiguousarray(v, np.uint16)
    out = np.empty((heads, tokens, d), np.uint16)
    lib().orc_transpose_v(_p(v), _p(out), C.c_int(tokens), C.c_int(heads))
    return out


def append_contig(cache: np.ndarray, flash: np.ndarray, position: int) -> None:
    heads, max_seq, d = cache.shape
    _, tokens, _ = flash.shape
    assert cache.flags.c_contiguous and cache.dtype == np.uint16
    flash = np.ascontiguousarray(flash, np.uint16)
    lib().orc_append_contig(_p(cache), _p(flash), C.c_int(heads), C.c_int(max_seq),
                            C.c_int(position), C.c_int(tokens))


def paged_append(pool: np.ndarray, table: np.ndarray, k_flash, v_flash, position: int) -> None:
    """pool: logical [num_blocks, kv_heads, 2, 16, 64] uint16, updated in place."""
    nb, heads, two, bt, d = pool.shape
    assert (two, bt, d) == (2, BLOCK_TOKENS, HEAD_DIM) and pool.flags.c_contiguous
    table = np.ascontiguousarray(table, np.int32)
    k_flash = np.ascontiguousarray(k_flash, np.uint16)
    v_flash = np.ascontiguousarray(v_flash, np.uint16)
    tokens = k_flash.shape[1]
    lib().orc_paged_append(_p(pool), C.c_int(heads), _p(table), _p(k_flash), _p(v_flash),
                           C.c_int(position), C.c_int(tokens))


def paged_gather(pool: np.ndarray, table: np.ndarray, length: int):
    nb, heads, _, _, d = pool.shape
    table = np.ascontiguousarray(table, np.int32)
    k = np.zeros((heads, length, d), np.uint16)
    v = np.zeros((heads, length, d), np.uint16)
    lib().orc_paged_gather(_p(pool), C.c_int(heads), _p(table), C.c_int(length), _p(k), _p(v),
                           C.c_int(length))
    return k, v


def attention(Q, K, V, kv_seq_len: int, scale: float = 0.125, causal: bool = True,
              round_p_bf16: bool = False, want_lse: bool = True):
    """Q [Hq, Sq, 64], K/V [Hkv, kv_stride, 64] -> O fp32 [Hq, Sq, 64], LSE [Hq, Sq]."""
    Q = np.ascontiguousarray(Q, np.uint16)
    K = np.ascontiguousarray(K, np.uint16)
    V = np.ascontiguousarray(V, np.uint16)
    hq, sq, _ = Q.shape
    hkv, stride, _ = K.shape
    O = np.empty((hq, sq, HEAD_DIM), np.float32)
    L = np.empty((hq, sq), np.float32) if want_lse else None
    lib().orc_attention(_p(Q), _p(K), _p(V), _p(O), _p(L), C.c_int(hq), C.c_int(hkv),
                        C.c_int(sq), C.c_int(kv_seq_len), C.c_int(stride), C.c_float(scale),
                        C.c_int(int(causal)), C.c_int(int(round_p_bf16)))
    return O, L


def decode_paged(q, pool, table, tok_begin: int, tok_end: int, scale: float = 0.125):
    """q [Hq, 64] -> out fp32 [Hq, 64], lse [Hq] over tokens [tok_begin, tok_end)."""
    q = np.ascontiguousarray(q, np.uint16)
    hq = q.shape[0]
    heads = pool.shape[1]
    table = np.ascontiguousarray(table, np.int32)
    out = np.empty((hq, HEAD_DIM), np.float32)
    lse = np.empty((hq,), np.float32)
    lib().orc_decode_paged(_p(q), _p(pool), C.c_int(hq), C.c_int(heads), _p(table),
                           C.c_int(tok_begin), C.c_int(tok_end), C.c_float(scale), _p(out), _p(lse))
    return out, lse


def lse_merge(O_parts: np.ndarray, lse_parts: np.ndarray):
    """O_parts [n, rows, 64] fp32, lse_parts [n, rows] -> (O [rows, 64], lse [rows])."""
    O_parts = np.ascontiguousarray(O_parts, np.float32)
    lse_parts = np.ascontiguousarray(lse_parts, np.float32)
    n, rows, _ = O_parts.shape
    O = np.empty((rows, HEAD_DIM), np.float32)
    lse = np.empty((rows,), np.float32)
    lib().orc_lse_merge(_p(O_parts), _p(lse_parts), C.c_int(n), C.c_int(rows), _p(O), _p(lse))
    return O, lse


def output_layout(x: np.ndarray) -> np.ndarray:
    """[heads, tokens, 64] -> [tokens, heads*64]."""
    heads, tokens, d = x.shape
    x = np.ascontiguousarray(x)
    out = np.empty((tokens, heads * d), x.dtype)
    if x.dtype == np.float32:
        lib().orc_output_layout_f32(_p(x), _p(out), C.c_int(heads), C.c_int(tokens))
    else:
        lib().orc_output_layout_bf16(_p(x), _p(out), C.c_int(heads), C.c_int(tokens))
    return out


def gemm_bf16(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """bf16 bit patterns: a [M, K] times b [K, N] -> [M, N] (double accumulation, one rounding)."""
    a = np.ascontiguousarray(a, dtype=np.uint16)
    b = np.ascontiguousarray(b, dtype=np.uint16)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    out = np.empty((M, N), np.uint16)
    lib().orc_gemm_bf16(_p(a), _p(b), _p(out), C.c_int(M), C.c_int(N), C.c_int(K))
    return out


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    """bf16 bit patterns: x [rows, hidden], w [hidden] -> y [rows, hidden] (the reference kernel's arithmetic)."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.uint16)
    rows, hidden = x.shape
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), _p(y), C.c_int(rows), C.c_int(hidden), C.c_float(eps))
    return y


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """bf16 bit patterns: bf16(SiLU(gate) * up), element-wise (src/kernels/silu/silu_8192.cu:55-100)."""
    gate = np.ascontiguousarray(gate, dtype=np.uint16)
    up = np.ascontiguousarray(up, dtype=np.uint16)
    assert gate.shape == up.shape
    out = np.empty_like(gate)
    lib().orc_silu_mul(_p(gate), _p(up), _p(out), C.c_longlong(gate.size))
    return out


def ffn(x: np.ndarray, norm_w, wg: np.ndarray, wu: np.ndarray, wd: np.ndarray, eps: float = 1e-5,
        add_residual: bool = True) -> np.ndarray:
    """The reference's feed-forward block on bf16 bit patterns (src/runtime/ffn.cu:34-145 and the residual
    add of src/runtime/transformer_block.cu:76-81): x [rows, hidden] -> [rows, hidden]."""
    xn = rmsnorm(x, norm_w, eps) if norm_w is not None else np.ascontiguousarray(x, dtype=np.uint16)
    h = silu_mul(gemm_bf16(xn, wg), gemm_bf16(xn, wu))
    y = gemm_bf16(h, wd)
    if not add_residual:
        return y
    return f32_to_bf16(bf16_to_f32(x) + bf16_to_f32(y))


def _bitrev5(x):
    x = np.asarray(x)
    return ((x & 1) << 4) | ((x & 2) << 2) | (x & 4) | ((x & 8) >> 2) | ((x & 16) >> 4)


def argmax_reference_rule(logits: np.ndarray) -> np.ndarray:
    """bf16 bit patterns [rows, vocab] -> int32 [rows]: index of the largest logit, ties broken as the
    structure of the reference's argmax kernel breaks them (src/kernels/sampling/argmax_128256.cu:43-96):
    256 threads scan t, t + 256, ... with a strict ">" (the smallest index of a thread wins), lanes and
    then warps are combined by shuffle-down with a strict ">" — a tree whose left operand wins a tie, and
    whose leaves from left to right are the lanes in bit-reversed order.  So among equal largest values
    the winner has the smallest (bit-reversed warp number, bit-reversed lane number, index), with
    thread = index mod 256."""
    v = bf16_to_f32(np.ascontiguousarray(logits, dtype=np.uint16))
    out = np.empty(v.shape[0], np.int32)
    for r in range(v.shape[0]):
        cand = np.flatnonzero(v[r] == v[r].max())
        t = cand % 256
        out[r] = cand[np.lexsort((cand, _bitrev5(t % 32), _bitrev5(t // 32)))[0]]
    return out


def num_threads() -> int:
    return int(lib().orc_num_threads())


# ---- block allocator model (pure Python; the reference has none) -----------
class BlockPoolModel:
    """Host model of the paged block allocator the product's C++ pool must match:
    a LIFO free list initialised so that block ids pop in ``free_order`` order;
    ``reserve`` grows a sequence's table to cover ``new_len`` tokens, never
    shrinks, and is all-or-nothing; ``free`` pushes a sequence's blocks back in
    reverse table order, so the most recently freed block is handed out first."""

    def __init__(self, num_blocks: int, free_order=None):
        order = list(range(num_blocks)) if free_order is None else [int(b) for b in free_order]
        assert sorted(order) == list(range(num_blocks))
        self.free = order[::-1]  # pop() from the end yields order[0] first
        self.tables: dict[int, list[int]] = {}
        self.lens: dict[int, int] = {}

    def create(self) -> int:
        s = 0
        while s in self.tables:  # lowest unused id
            s += 1
        self.tables[s] = []
        self.lens[s] = 0
        return s

    def reserve(self, s: int, new_len: int) -> bool:
        if new_len <= self.lens[s]:
            return True
        need = (new_len + BLOCK_TOKENS - 1) // BLOCK_TOKENS - len(self.tables[s])
        if need > len(self.free):
            return False
        for _ in range(max(need, 0)):
            self.tables[s].append(self.free.pop())
        self.lens[s] = max(self.lens[s], new_len)
        return True

    def release(self, s: int) -> None:
        for b in reversed(self.tables.pop(s)):
            self.free.append(b)
        self.lens.pop(s)


# ---- the reference's own CUDA kernels (GPU box only) ------------------------
def ref_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libref.so"))


def ref():
    """Load ``_ref/libref.so`` (the reference's flashattention.cu, rope.cu, layout.cu
    and its two projection GEMMs compiled unmodified for sm_100a).  Needs a GPU."""
    global _REF
    if _REF is None:
        r = C.CDLL(os.path.join(_HERE, "_ref", "libref.so"))
        vp, i, f = C.c_void_p, C.c_int, C.c_float
        r.ref_rope_qkv.argtypes = [vp] * 8 + [i, i]
        r.ref_rope_qkv.restype = None
        r.ref_flash_attention.argtypes = [vp] * 5 + [i] * 6 + [f, i, vp]
        r.ref_flash_attention.restype = None
        r.ref_flash_output_layout.argtypes = [vp, vp, i]
        r.ref_flash_output_layout.restype = None
        r.ref_append_memcpy_loop.argtypes = [vp] * 4 + [i] * 3
        r.ref_append_memcpy_loop.restype = i
        r.ref_append_strided.argtypes = [vp] * 4 + [i] * 3 + [vp]
        r.ref_append_strided.restype = i
        r.ref_gemm.argtypes = [vp, vp, vp, i, i, i]
        r.ref_gemm.restype = i
        r.ref_argmax.argtypes = [vp, vp]
        r.ref_argmax.restype = None
        r.ref_embedding.argtypes = [vp, vp, vp, i]
        r.ref_embedding.restype = None
        r.ref_silu_mul.argtypes = [vp, vp, vp, i]
        r.ref_silu_mul.restype = None
        r.ref_residual_add.argtypes = [vp, vp, vp, C.c_longlong]
        r.ref_residual_add.restype = i
        r.ref_rmsnorm.argtypes = [vp, vp, vp, i, f]
        r.ref_rmsnorm.restype = None
        _REF = r
    return _REF
