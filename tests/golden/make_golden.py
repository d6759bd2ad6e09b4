"""Makes the golden fixtures of this folder by running the REFERENCE's own CUDA
kernels (oracle/_ref/libref.so: its flashattention.cu, rope.cu, layout.cu, rmsnorm.cu and
silu_8192.cu compiled unmodified for sm_100a) on seeded inputs.  Needs a B200.

    python tests/golden/make_golden.py <output folder>

Each .npz holds the inputs and what the reference produced for one call of its
path: launch_rope_qkv -> 128-byte append loop -> launch_flash_attention (causal,
kv_len = position + tokens) -> launch_flash_output_layout.  The CPU tests check
the oracle against these files bit for bit (RoPE, append, layout) and within
the path's tolerance (attention).
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from oracle import oracle as orc  # noqa: E402

DEV = "cuda:0"


def dev(u16):
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).view(torch.bfloat16).to(DEV)


def host(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def one_case(name, seed, position, tokens, max_seq, out_dir):
    rng = np.random.default_rng(seed)
    ref = orc.ref()
    cos, sin = orc.build_rope_tables(max_seq)
    cos_d = torch.from_numpy(cos).to(DEV)
    sin_d = torch.from_numpy(sin).to(DEV)
    q = orc.randn_bf16(rng, (tokens, 32, 64))
    k = orc.randn_bf16(rng, (tokens, 8, 64))
    v = orc.randn_bf16(rng, (tokens, 8, 64))
    # earlier cache contents: N(0,1)*0.5 at positions < position, zero elsewhere
    kc0 = np.zeros((8, max_seq, 64), np.uint16)
    vc0 = np.zeros((8, max_seq, 64), np.uint16)
    kc0[:, :position] = orc.randn_bf16(rng, (8, position, 64), 0.5)
    vc0[:, :position] = orc.randn_bf16(rng, (8, position, 64), 0.5)
    qd, kd, vd = dev(q), dev(k), dev(v)
    qf = torch.empty(32, tokens, 64, dtype=torch.bfloat16, device=DEV)
    kf = torch.empty(8, tokens, 64, dtype=torch.bfloat16, device=DEV)
    vf = torch.empty(8, tokens, 64, dtype=torch.bfloat16, device=DEV)
    kc, vc = dev(kc0), dev(vc0)
    of = torch.zeros(32, tokens, 64, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(32, tokens, dtype=torch.float32, device=DEV)
    ol = torch.zeros(tokens, 2048, dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    ref.ref_rope_qkv(qd.data_ptr(), qf.data_ptr(), kd.data_ptr(), kf.data_ptr(), vd.data_ptr(),
                     vf.data_ptr(), cos_d.data_ptr(), sin_d.data_ptr(), tokens, position)
    assert ref.ref_append_memcpy_loop(kc.data_ptr(), vc.data_ptr(), kf.data_ptr(), vf.data_ptr(),
                                      max_seq, position, tokens) == 0
    ref.ref_flash_attention(qf.data_ptr(), kc.data_ptr(), vc.data_ptr(), of.data_ptr(),
                            lse.data_ptr(), 1, 32, 8, tokens, position + tokens, max_seq, 0.125, 1,
                            None)
    ref.ref_flash_output_layout(of.data_ptr(), ol.data_ptr(), tokens)
    torch.cuda.synchronize()
    variants = [var for var in (0, 1, 2)
                if np.array_equal(host(kf), orc.rope(k, cos, sin, position, var))
                and np.array_equal(host(qf), orc.rope(q, cos, sin, position, var))]
    print(name, "reference rope equals oracle y0 variants", variants)
    np.savez_compressed(
        os.path.join(out_dir, name + ".npz"), position=position, tokens=tokens, max_seq=max_seq,
        y0_variant=(1 if 1 in variants else (variants[0] if variants else -1)), y0_variants=np.array(variants, np.int32),
        cos=cos, sin=sin, q_in=q, k_in=k, v_in=v, q_flash=host(qf), k_flash=host(kf),
        v_flash=host(vf), k_cache_before=kc0, v_cache_before=vc0, k_cache_after=host(kc),
        v_cache_after=host(vc), o_flash=host(of), lse=lse.cpu().numpy(), o_layout=host(ol))


def elementwise_cases(out_dir):
    """The kernels either side of the attention path that have no free parameters: RMSNorm over rows of
    2048 (rmsnorm_launch<2048>, 256 threads) and SiLU(gate) * up over rows of 8192 (launch_silu_mul)."""
    rng = np.random.default_rng(105)
    ref = orc.ref()
    x = orc.randn_bf16(rng, (3, 2048), 1.5)
    w = orc.randn_bf16(rng, (2048,), 0.7)
    y = torch.zeros(3, 2048, dtype=torch.bfloat16, device=DEV)
    xd, wd = dev(x), dev(w)
    ref.ref_rmsnorm(xd.data_ptr(), wd.data_ptr(), y.data_ptr(), 3, 1e-5)
    gate = orc.randn_bf16(rng, (2, 8192), 2.0)
    up = orc.randn_bf16(rng, (2, 8192), 1.0)
    gate[0, :8] = orc.f32_to_bf16(np.array([0.0, -0.0, 30.0, -30.0, 88.0, -88.0, 1e-3, -1e-3], np.float32))
    h = torch.zeros(2, 8192, dtype=torch.bfloat16, device=DEV)
    gd, ud = dev(gate), dev(up)
    ref.ref_silu_mul(gd.data_ptr(), ud.data_ptr(), h.data_ptr(), 2)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, "elementwise_rmsnorm_silu.npz"), x=x, norm_w=w, rmsnorm_out=host(y),
                        gate=gate, up=up, silu_mul_out=host(h))
    print("elementwise: rmsnorm equal to oracle", np.array_equal(host(y), orc.rmsnorm(x, w, 1e-5)),
          "; silu_mul bit-equal fraction", float((host(h) == orc.silu_mul(gate, up)).mean()))


if __name__ == "__main__":
    out_dir = sys.argv[1]
    os.makedirs(out_dir, exist_ok=True)
    one_case("prefill_37_at_0", 101, 0, 37, 48, out_dir)
    one_case("decode_1_at_100", 102, 100, 1, 112, out_dir)
    one_case("chunked_prefill_20_at_45", 103, 45, 20, 80, out_dir)
    one_case("prefill_66_at_0", 104, 0, 66, 66, out_dir)
    elementwise_cases(out_dir)
