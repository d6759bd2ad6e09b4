"""Shared plumbing of the GPU tests: bf16 bit patterns <-> torch tensors and
cache set-up through the product's own append entry."""
import numpy as np
import torch

from llama_transformer_runtime_b200 import paged
from oracle import oracle as orc

DEV = "cuda:0"


def to_dev(u16: np.ndarray) -> torch.Tensor:
    """numpy uint16 bit patterns -> CUDA bf16 tensor of the same shape."""
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).view(torch.bfloat16).to(DEV)


def to_u16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def f32_dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(DEV)


def identity_tables(n: int):
    return (torch.ones(n, 32, dtype=torch.float32, device=DEV),
            torch.zeros(n, 32, dtype=torch.float32, device=DEV))


def fill_cache(pool: paged.KVPool, layer: int, seq: int, k: np.ndarray, v: np.ndarray) -> None:
    """Put K/V [kv_heads, L, 64] (final cache values) at positions 0..L-1 of a
    fresh sequence: an append with the identity rotation (cos 1, sin 0)."""
    heads, L, _ = k.shape
    pool.reserve(seq, L)
    pool.batch_set([seq], [L])
    cos, sin = identity_tables(L)
    kin = to_dev(k.transpose(1, 0, 2))
    vin = to_dev(v.transpose(1, 0, 2))
    pool.append(layer, None, kin, vin, cos, sin, None)
    torch.cuda.synchronize()


def read_logical_pool(pool: paged.KVPool, layer: int) -> np.ndarray:
    """Raw device storage of one layer -> logical [blocks, heads, 2, 16, 64]
    uint16, undoing the documented physical layout with numpy only."""
    ptr, nbytes = pool.layer_storage(layer)
    raw = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    # device-to-device copy of the raw bytes through a typed view of the address
    import ctypes
    cudart = ctypes.CDLL("libcudart.so.12")
    assert cudart.cudaMemcpy(ctypes.c_void_p(raw.data_ptr()), ctypes.c_void_p(ptr),
                             ctypes.c_size_t(nbytes), 3) == 0
    b = raw.cpu().numpy().reshape(pool.num_blocks, pool.kv_heads, 2, 16, 8, 16)
    out = np.empty_like(b)
    for r in range(16):
        for c in range(8):
            out[:, :, :, r, c] = b[:, :, :, r, c ^ (r & 7)]
    return out.reshape(pool.num_blocks, pool.kv_heads, 2, 16, 128).view(np.uint16).reshape(
        pool.num_blocks, pool.kv_heads, 2, 16, 64)


ROW_REL = 2.0 ** -7  # per-row bar: a few bf16 output roundings (2^-9 each) of the row's largest value


def check_close(got: np.ndarray, want: np.ndarray, what: str = "", row: int = 64) -> None:
    """Two bars, both must hold.  (1) The tolerance of the path: max-abs 2e-2 or relative 1e-2 per
    element.  (2) A bar that scales with the data: within each output row of one head (`row` = 64
    consecutive values) max|got - want| <= 2^-7 * max|want|.  At long contexts attention outputs
    shrink like 1/sqrt(L) and fall below the absolute term of (1), which an all-zero output would
    then pass; (2) cannot be passed that way.  row = 0 switches (2) off."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    err = np.abs(got - want)
    bad = err > 2e-2 + 1e-2 * np.abs(want)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, max err {err.max():.4g}"
    if row and want.size % row == 0 and want.size:
        e = err.reshape(-1, row).max(axis=1)
        m = np.abs(want).reshape(-1, row).max(axis=1)
        worst = int(np.argmax(e - ROW_REL * m))
        assert np.all(e <= ROW_REL * m + 1e-30), (
            f"{what}: row {worst}: max err {e[worst]:.4g} exceeds 2^-7 of the row's largest value {m[worst]:.4g} "
            f"({(e > ROW_REL * m).sum()} of {e.size} rows)")


def max_row_rel_err(got: np.ndarray, want: np.ndarray, row: int = 64) -> float:
    """max over rows of max|got - want| / max|want| (the quantity bar (2) of check_close bounds)."""
    err = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)).reshape(-1, row).max(axis=1)
    m = np.abs(np.asarray(want, np.float64)).reshape(-1, row).max(axis=1)
    return float(np.max(err / np.maximum(m, 1e-30)))
