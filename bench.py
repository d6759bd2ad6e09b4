"""Benchmark of the paged KV-cache decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode128k|decode4k]

Default workload (decode128k): long-context decode, batch 1, context 131072 x 16
layers (about 4.3 GB of bf16 paged KV, 16-token blocks, seeded random fragmented
block table), KV values N(0,1)*0.5.  One step = one new token: per layer a fused
RoPE + paged append, then paged GQA decode attention over the whole cache.
With N GPUs the sequence is split by token range over the ranks (strong
scaling); every layer ends with an exchange of the ranks' (O, LSE) partials and
a log-sum-exp merge.

metric  paged_decode_attn_hbm_gbs = algorithmic cache bytes streamed per second,
        sum over ranks: steps x layers x (2048 L + 8192 + 4 ceil(L/16)) / time.
        The line also carries us_per_token (time per step).
value   inputs resident in HBM.      e2e   host buffers: per step the new
        token's q/k/v for all layers go host->device from pinned memory and the
        attention outputs come back, inside the timed region.
The cache is 4.3 GB per step (268 MB per layer) — larger than L2, no flush needed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYERS = 16
Q_HEADS, KV_HEADS, D = 32, 8, 64
BLOCK = 16
WORKLOADS = {
    "decode128k": dict(ctx=131072, name="decode_ctx131072_x16layers_batch1"),
    "decode4k": dict(ctx=4096, name="decode_ctx4096_x16layers_batch1"),
}


def decode_bytes(L: int) -> int:
    """Algorithmic bytes of one layer's decode over a context of L tokens:
    K+V read once, Q read, O written, block table read."""
    return 2 * KV_HEADS * L * D * 2 + 2 * Q_HEADS * D * 2 + 4 * ((L + BLOCK - 1) // BLOCK)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ncu capture (profiles/): dram read+write bytes per layer of the workload, or
# None when not captured.
# per layer: the 2-layer decode_step_kernel capture read 537.09 MB and wrote 6.00 MB
NCU_TRAFFIC_BYTES = {"decode128k": 271544320, "decode4k": None}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self, lo: int = 0, hi: int | None = None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        rows = [r for r in self.rows[lo:hi] if len(r) >= 6] or [r for r in self.rows if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": float(rows[0][1]) if rows[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def token_ranges(L: int, n: int):
    """Split [0, L) into n contiguous ranges on 16-token block borders."""
    blocks = (L + BLOCK - 1) // BLOCK
    cuts = [min(L, (blocks * r // n) * BLOCK) for r in range(n)] + [L]
    return [(cuts[r], cuts[r + 1]) for r in range(n)]


# =============================================================================
# our arm
# =============================================================================
def run_ours(args):
    import torch
    import torch.distributed as dist

    from llama_transformer_runtime_b200 import paged

    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    wl = WORKLOADS[args.workload]
    ctx = wl["ctx"]
    total_steps = args.warmup + 2 * args.steps + 8
    lo, hi = token_ranges(ctx, world)[rank]
    local_len = hi - lo
    owner = world - 1  # the last range takes the appended tokens
    cap_tokens = local_len + (total_steps if rank == owner else 0)
    need_blocks = (cap_tokens + BLOCK - 1) // BLOCK
    num_blocks = need_blocks + need_blocks // 4 + 8  # fragmented: table scattered over a larger pool

    pool = paged.KVPool(LAYERS, num_blocks, KV_HEADS, 1, need_blocks + 1, device=local_rank)
    rng = np.random.default_rng(1234 + rank)
    pool.set_free_order(rng.permutation(num_blocks))
    seq = pool.create_seq()
    if args.chunk_blocks:
        pool.set_decode_chunk_blocks(args.chunk_blocks)
    if args.decode_shape:
        w, s = args.decode_shape.lower().split("x")
        pool.set_decode_shape(int(w), int(s))
    if args.combiners:
        pool.set_step_combiners(args.combiners)

    # ---- fill the cache: N(0,1)*0.5, generated on the device, appended with the identity rotation
    gen = torch.Generator(device=dev)
    gen.manual_seed(4321 + rank)
    chunk = 8192
    # tables are indexed by absolute position, so they cover the whole local range
    ones = torch.ones(local_len + 1, 32, dtype=torch.float32, device=dev)
    zeros = torch.zeros(local_len + 1, 32, dtype=torch.float32, device=dev)
    for c0 in range(0, local_len, chunk):
        n = min(chunk, local_len - c0)
        pool.reserve(seq, c0 + n)
        pool.batch_set([seq], [n])
        for layer in range(LAYERS):
            k = (torch.randn(n, KV_HEADS, D, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
            v = (torch.randn(n, KV_HEADS, D, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
            pool.append(layer, None, k, v, ones, zeros, None)
    torch.cuda.synchronize()
    del ones, zeros

    cos_h, sin_h = paged.build_rope_tables(ctx + total_steps + 1)
    cos = torch.from_numpy(cos_h).to(dev)
    sin = torch.from_numpy(sin_h).to(dev)

    # ---- per-step inputs (all layers), host pinned + device
    q_host = (torch.randn(LAYERS, 1, Q_HEADS, D, generator=torch.Generator().manual_seed(7))).to(torch.bfloat16).pin_memory()
    k_host = (torch.randn(LAYERS, 1, KV_HEADS, D, generator=torch.Generator().manual_seed(8))).to(torch.bfloat16).pin_memory()
    v_host = (torch.randn(LAYERS, 1, KV_HEADS, D, generator=torch.Generator().manual_seed(9))).to(torch.bfloat16).pin_memory()
    out_host = torch.zeros(LAYERS, 1, Q_HEADS * D, dtype=torch.bfloat16).pin_memory()
    q_dev, k_dev, v_dev = q_host.to(dev), k_host.to(dev), v_host.to(dev)
    q_rot = torch.empty_like(q_dev)
    out_dev = torch.zeros(LAYERS, 1, Q_HEADS * D, dtype=torch.bfloat16, device=dev)
    if world > 1:
        part = torch.zeros(LAYERS, Q_HEADS * D + Q_HEADS, dtype=torch.float32, device=dev)  # [O | lse] per layer
        gathered = torch.zeros(LAYERS, world, Q_HEADS * D + Q_HEADS, dtype=torch.float32, device=dev)
        o_parts = torch.zeros(world, Q_HEADS, D, dtype=torch.float32, device=dev)
        l_parts = torch.zeros(world, Q_HEADS, dtype=torch.float32, device=dev)

    xchg = None
    if world > 1 and args.exchange == "fused":
        xchg = paged.Exchange(local_rank, rank, world, 1, KV_HEADS)
        handles = [None] * world
        dist.all_gather_object(handles, xchg.handle())
        xchg.connect(handles)
        dist.barrier()

    state = {"global_len": ctx, "launches": 0}
    # A fused step is ONE cooperative launch of decode_step_kernel when the library takes that path
    # (the pool counts those steps); otherwise it is one decode_kernel launch per layer.

    def step(qs, ks, vs, outs):
        """One token: every layer appends and attends over the whole context."""
        state["global_len"] += 1
        g = state["global_len"]
        if rank == owner:
            pool.reserve(seq, pool.length(seq) + 1)
        if world == 1:
            pool.batch_set([seq])
            pool.decode_step(0, LAYERS, qs, ks, vs, Q_HEADS * D, KV_HEADS * D, cos, sin, q_rot, outs,
                             Q_HEADS * D, Q_HEADS * D)
            state["fused_steps"] = state.get("fused_steps", 0) + 1
            return
        pool.batch_set_sharded([seq], [1 if rank == owner else 0], [1], [g - 1], [lo])
        if xchg is not None:
            # fused exchange: partials pushed to every rank by the decode kernel's epilogue
            paged.decode_step_sharded(pool, xchg, 0, LAYERS, qs, ks if rank == owner else None,
                                      vs if rank == owner else None, Q_HEADS * D, KV_HEADS * D, cos, sin,
                                      q_rot, outs, Q_HEADS * D, Q_HEADS * D)
            state["fused_steps"] = state.get("fused_steps", 0) + 1
            return
        for layer in range(LAYERS):
            pool.append(layer, qs[layer], ks[layer], vs[layer], cos, sin, q_rot[layer])
            pool.decode(layer, q_rot[layer], None, 0, part[layer, :Q_HEADS * D], part[layer, Q_HEADS * D:])
            dist.all_gather_into_tensor(gathered[layer].view(-1), part[layer])
            o_parts.copy_(gathered[layer, :, :Q_HEADS * D].reshape(world, Q_HEADS, D))
            l_parts.copy_(gathered[layer, :, Q_HEADS * D:])
            paged.merge_partials(o_parts, l_parts, world, Q_HEADS, outs[layer])
            state["launches"] += 3

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def resident_step():
        step(q_dev, k_dev, v_dev, out_dev)

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        k_dev.copy_(k_host, non_blocking=True)
        v_dev.copy_(v_host, non_blocking=True)
        step(q_dev, k_dev, v_dev, out_dev)
        out_host.copy_(out_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result every step

    m0 = sampler.mark()  # clock samples from here on are taken under load
    for _ in range(args.warmup):
        resident_step()
    len_before = state["global_len"]
    state["launches"] = 0
    state["fused_steps"] = 0
    one_launch_before = pool.step_launches()
    ms = timed(resident_step, args.steps)
    one_launch = pool.step_launches() - one_launch_before
    launches = state["launches"] + one_launch + (state["fused_steps"] - one_launch) * LAYERS
    len_after = state["global_len"]
    bytes_timed = sum(LAYERS * decode_bytes(L) for L in range(len_before + 1, len_after + 1))
    value = bytes_timed / (ms * 1e-3) / 1e9

    len_before = state["global_len"]
    ms_e2e = timed(e2e_step, args.steps)
    bytes_e2e = sum(LAYERS * decode_bytes(L) for L in range(len_before + 1, state["global_len"] + 1))
    e2e_value = bytes_e2e / (ms_e2e * 1e-3) / 1e9
    h2d = (q_host.numel() + k_host.numel() + v_host.numel()) * 2
    d2h = out_host.numel() * 2

    # ---- dominant kernel alone: 16 back-to-back decode launches (one per layer) per event pair
    pool.batch_set_sharded([seq], [0], [1], [state["global_len"] - 1], [lo])
    L_local = pool.length(seq)
    local_out = out_dev if world == 1 else torch.zeros_like(out_dev)  # N>1: keep the merged rows

    def decode_only():
        for layer in range(LAYERS):
            pool.decode(layer, q_rot[layer], local_out[layer], Q_HEADS * D, None, None)

    decode_only()
    reps = max(3, args.steps)
    ms_iso = timed(decode_only, reps) / (reps * LAYERS)  # plain launches, nothing overlapped
    ms_k = ms_iso
    if world == 1:
        # the step's own launch (decode_step_kernel: all layers, append fused in), without the
        # host's table work
        pool.batch_set([seq])

        def step_kernels():
            pool.decode_step(0, LAYERS, q_dev, k_dev, v_dev, Q_HEADS * D, KV_HEADS * D, cos, sin, q_rot,
                             out_dev, Q_HEADS * D, Q_HEADS * D)

        step_kernels()
        ms_k = timed(step_kernels, reps) / (reps * LAYERS)
    kern_bytes = decode_bytes(L_local)
    achieved = kern_bytes / (ms_k * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    pool.check()
    m1 = sampler.mark()
    xchg_check = None
    if world > 1:
        # the last step's merged layer-0 row against an NCCL all-gather + merge of the same partials
        pool.decode(0, q_rot[0], None, 0, part[0, :Q_HEADS * D], part[0, Q_HEADS * D:])
        dist.all_gather_into_tensor(gathered[0].view(-1), part[0])
        o_parts.copy_(gathered[0, :, :Q_HEADS * D].reshape(world, Q_HEADS, D))
        l_parts.copy_(gathered[0, :, Q_HEADS * D:])
        chk = torch.zeros(1, Q_HEADS * D, dtype=torch.bfloat16, device=dev)
        paged.merge_partials(o_parts, l_parts, world, Q_HEADS, chk)
        torch.cuda.synchronize()
        xchg_check = float((chk.float() - out_dev[0].float()).abs().max().item())

    line = None
    if rank == 0:
        clocks = sampler.stop(m0, m1)
        line = {
            "metric": "paged_decode_attn_hbm_gbs", "value": round(value, 1), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 4),
            "us_per_token": round(ms / args.steps * 1e3, 2),
            "us_per_token_per_layer": round(ms / args.steps * 1e3 / LAYERS, 2),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl["name"], "context": ctx, "layers": LAYERS, "batch": 1,
                       "q_heads": Q_HEADS, "kv_heads": KV_HEADS, "head_dim": D, "block_tokens": BLOCK,
                       "block_table": "seeded random permutation over a pool 25% larger than the sequence",
                       "parallelism": "1 GPU" if world == 1 else (
                           f"sequence range split over {world} GPUs; one launch per step, per layer the combining CTAs "
                           f"push (O, LSE) to every rank over NVLink (peer stores of value+step words) and merge locally"
                           if xchg is not None else
                           f"sequence range split over {world} GPUs, NCCL all-gather of (O, LSE) per layer + merge"),
                       "l2": f"inputs larger than L2 ({decode_bytes(ctx) * LAYERS / 1e9:.2f} GB streamed per step)"},
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(ms_e2e / args.steps, 4)},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": ({"bound": "hbm", "kernel": "decode_step_kernel", "achieved": round(achieved, 1),
                          "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                          "peak_source": f"of {peak_kind}", "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                          "us_per_launch": round(ms_k * 1e3 * LAYERS, 2), "bytes_per_launch": kern_bytes * LAYERS,
                          "layers_per_launch": LAYERS, "us_per_layer": round(ms_k * 1e3, 2),
                          "us_per_layer_plain_decode_kernel": round(ms_iso * 1e3, 2),
                          "how": f"CUDA events around the step's one launch (all {LAYERS} layers, append fused in)",
                          "traffic": (NCU_TRAFFIC_BYTES[args.workload] * LAYERS
                                      if NCU_TRAFFIC_BYTES.get(args.workload) else None),
                          "traffic_note": "ncu capture of a 2-layer decode_step_kernel launch, per layer x layers"}
                         if world == 1 and LAYERS >= 2 else
                         {"bound": "hbm", "kernel": "decode_kernel", "achieved": round(achieved, 1),
                          "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                          "peak_source": f"of {peak_kind}", "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                          "us_per_launch": round(ms_k * 1e3, 2), "bytes_per_launch": kern_bytes,
                          "how": f"CUDA events around {LAYERS} plain decode_kernel launches on this rank's range, / {LAYERS}",
                          "traffic": NCU_TRAFFIC_BYTES.get(args.workload)}),
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline(pool, seq, q_rot, out_dev, L_local)
        else:
            line["exchange_vs_allgather_max_abs_diff"] = xchg_check
        print(json.dumps(line), flush=True)
    barrier()
    if xchg is not None:
        xchg.close()
    pool.close()
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(pool, seq, q_rot, out_dev, L):
    """The CPU oracle (fp32 naive attention, OpenMP) on a bounded sample: layer
    0 of this workload, repeated for about ten seconds; its answer is also the
    check of the GPU output of that layer."""
    import torch

    from oracle import oracle as orc

    dev = q_rot.device
    k = torch.zeros(KV_HEADS, L, D, dtype=torch.bfloat16, device=dev)
    v = torch.zeros_like(k)
    pool.gather_kv(0, seq, k, v, L)
    torch.cuda.synchronize()
    k_h = k.view(torch.int16).cpu().numpy().view(np.uint16)
    v_h = v.view(torch.int16).cpu().numpy().view(np.uint16)
    q_h = q_rot[0].view(torch.int16).cpu().numpy().view(np.uint16).reshape(Q_HEADS, 1, D)
    del k, v
    t0 = time.perf_counter()
    O, _ = orc.attention(q_h, k_h, v_h, L)
    t1 = time.perf_counter() - t0
    reps = 1
    budget = 10.0
    while t1 * reps < budget and reps < 64:
        orc.attention(q_h, k_h, v_h, L)
        reps += 1
    total = time.perf_counter() - t0
    got = orc.bf16_to_f32(out_dev[0].view(torch.int16).cpu().numpy().view(np.uint16)).reshape(-1)
    err = float(np.max(np.abs(got - O[:, 0].reshape(-1))))
    return {"value": round(decode_bytes(L) * reps / total / 1e9, 3), "unit": "GB/s",
            "cores": orc.num_threads(), "kind": "port",
            "sample": f"layer 0 of the workload (context {L}), {reps} passes of the fp32 CPU oracle",
            "gpu_vs_cpu_max_abs_err": err}


# =============================================================================
# reference arm: the reference's own CUDA kernels (oracle/_ref/libref.so) on this GPU
# =============================================================================
def run_reference(args):
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    from oracle import oracle as orc

    if not orc.ref_available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built (no reference checkout at build time)"}))
        return
    import torch

    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    ref = orc.ref()
    wl = WORKLOADS[args.workload]
    ctx = wl["ctx"]
    total_steps = args.warmup + 2 * args.steps + 4
    max_seq = ctx + total_steps + 1
    gen = torch.Generator(device=dev)
    gen.manual_seed(4321)
    # the reference's cache: per layer K and V [8, max_seq, 64], zero-initialised
    kc = torch.zeros(LAYERS, KV_HEADS, max_seq, D, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    for layer in range(LAYERS):
        kc[layer, :, :ctx] = (torch.randn(KV_HEADS, ctx, D, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
        vc[layer, :, :ctx] = (torch.randn(KV_HEADS, ctx, D, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    cos_h, sin_h = orc.build_rope_tables(max_seq)
    cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
    q_host = torch.randn(LAYERS, 1, Q_HEADS, D, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).pin_memory()
    k_host = torch.randn(LAYERS, 1, KV_HEADS, D, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).pin_memory()
    v_host = torch.randn(LAYERS, 1, KV_HEADS, D, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).pin_memory()
    out_host = torch.zeros(LAYERS, 1, Q_HEADS * D, dtype=torch.bfloat16).pin_memory()
    q_dev, k_dev, v_dev = q_host.to(dev), k_host.to(dev), v_host.to(dev)
    qf = torch.empty(Q_HEADS, 1, D, dtype=torch.bfloat16, device=dev)
    kf = torch.empty(KV_HEADS, 1, D, dtype=torch.bfloat16, device=dev)
    vf = torch.empty(KV_HEADS, 1, D, dtype=torch.bfloat16, device=dev)
    of = torch.empty(Q_HEADS, 1, D, dtype=torch.bfloat16, device=dev)
    out_dev = torch.zeros(LAYERS, 1, Q_HEADS * D, dtype=torch.bfloat16, device=dev)
    state = {"len": ctx}

    def step():
        """What Attention::forward does per layer for one token (steps 5-7):
        launch_rope_qkv, the 128-byte append copies, launch_flash_attention with
        q_seq_len 1, launch_flash_output_layout."""
        pos = state["len"]
        state["len"] += 1
        for layer in range(LAYERS):
            ref.ref_rope_qkv(q_dev[layer].data_ptr(), qf.data_ptr(), k_dev[layer].data_ptr(), kf.data_ptr(),
                             v_dev[layer].data_ptr(), vf.data_ptr(), cos.data_ptr(), sin.data_ptr(), 1, pos)
            ref.ref_append_memcpy_loop(kc[layer].data_ptr(), vc[layer].data_ptr(), kf.data_ptr(), vf.data_ptr(),
                                       max_seq, pos, 1)
            ref.ref_flash_attention(qf.data_ptr(), kc[layer].data_ptr(), vc[layer].data_ptr(), of.data_ptr(),
                                    None, 1, Q_HEADS, KV_HEADS, 1, pos + 1, max_seq, 0.125, 1, None)
            ref.ref_flash_output_layout(of.data_ptr(), out_dev[layer].data_ptr(), 1)

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        k_dev.copy_(k_host, non_blocking=True)
        v_dev.copy_(v_host, non_blocking=True)
        step()
        out_host.copy_(out_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = state["len"]
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        b = sum(LAYERS * decode_bytes(L) for L in range(l0 + 1, state["len"] + 1))
        return e0.elapsed_time(e1), b

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    ms, b = timed(step, args.steps)
    clocks = sampler.stop()
    ms2, b2 = timed(e2e_step, args.steps)
    value = b / (ms * 1e-3) / 1e9
    e2e = b2 / (ms2 * 1e-3) / 1e9
    print(json.dumps({
        "impl": "reference", "metric": "paged_decode_attn_hbm_gbs", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
        "us_per_token": round(ms / args.steps * 1e3, 2), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl["name"], "context": ctx, "layers": LAYERS, "batch": 1,
                   "note": "the reference's own CUDA kernels (flashattention.cu, rope.cu, layout.cu compiled "
                           "unmodified for sm_100a) on this GPU, contiguous cache, single GPU only"},
        "e2e": {"value": round(e2e, 2), "unit": "GB/s",
                "h2d_bytes_per_step": (q_host.numel() + k_host.numel() + v_host.numel()) * 2,
                "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": round(ms2 / args.steps, 4)},
        "gpu_launches": args.steps * LAYERS * 5, "clocks": clocks,
        "cpu_baseline": {"value": round(value, 2), "unit": "GB/s", "cores": 0, "kind": "reference",
                         "sample": "whole workload; the reference has no CPU implementation of this path, "
                                   "so its CUDA kernels run on the GPU (host cores only drive the launches)"},
    }), flush=True)


# =============================================================================
# batched decode workload (config 5): 64 ragged sequences, shared fragmented pool
# =============================================================================
def run_batch(args):
    """64 sequences with context lengths seeded-uniform in [1024, 32768], one
    shared free-block pool; before timing, rounds of freeing and re-creating
    sequences interleave their tables.  One step = every sequence appends one
    token and attends over its cache, 16 layers.  With N GPUs the 8 KV heads are
    sharded (8/N per GPU, each with the 4*8/N query heads of its groups); every
    layer ends with an all-gather of the head outputs into [64, 2048] on every
    rank.  Strong scaling: the same batch is split N ways."""
    import torch
    import torch.distributed as dist

    from llama_transformer_runtime_b200 import paged

    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "the reference is single-sequence and contiguous; this workload has no reference arm "
                              "(see the decode128k and prefill2k workloads)"}))
        return
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    n_seqs = args.seqs
    kvh = KV_HEADS // world
    qh = 4 * kvh
    rng = np.random.default_rng(2024)  # the same allocator decisions on every rank
    lens = rng.integers(1024, 32769, n_seqs).astype(int)
    total_steps = args.warmup + 2 * args.steps + 8
    cap = int(lens.max()) + total_steps + 64
    blocks_needed = int(sum((l + total_steps + 15) // 16 for l in lens))
    num_blocks = blocks_needed + blocks_needed // 8 + 64
    pool = paged.KVPool(LAYERS, num_blocks, kvh, n_seqs, (cap + 15) // 16, device=local_rank)
    pool.set_free_order(rng.permutation(num_blocks))

    gen = torch.Generator(device=dev)
    gen.manual_seed(777 + rank)
    max_len = int(lens.max())
    ones = torch.ones(max_len + 1, 32, dtype=torch.float32, device=dev)
    zeros = torch.zeros(max_len + 1, 32, dtype=torch.float32, device=dev)

    def fill(seq, L):
        for c0 in range(0, L, 8192):
            n = min(8192, L - c0)
            pool.reserve(seq, c0 + n)
            pool.batch_set([seq], [n])
            for layer in range(LAYERS):
                kv = (torch.randn(2, n, kvh, D, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
                pool.append(layer, None, kv[0], kv[1], ones, zeros, None)

    # sequences created in a seeded order, then a third of them freed and re-created
    # twice, so that tables interleave across the pool (fragmentation)
    seqs = {}
    for i in range(n_seqs):
        s = pool.create_seq()
        fill(s, int(lens[i]))
        seqs[s] = int(lens[i])
    for rnd in range(2):
        victims = rng.choice(sorted(seqs), n_seqs // 3, replace=False)
        new_lens = rng.integers(1024, 32769, len(victims)).astype(int)
        for s in victims:
            pool.free_seq(int(s))
            del seqs[int(s)]
        for L in new_lens:
            if (int(L) + total_steps + 15) // 16 + 8 > pool.free_blocks():
                L = 1024
            s = pool.create_seq()
            fill(s, int(L))
            seqs[s] = int(L)
    torch.cuda.synchronize()
    del ones, zeros
    ids = sorted(seqs)
    cos_h, sin_h = paged.build_rope_tables(max(seqs.values()) + total_steps + 2)
    cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)

    g7 = torch.Generator().manual_seed(7)
    q_host = torch.randn(LAYERS, n_seqs, qh, D, generator=g7).to(torch.bfloat16).pin_memory()
    k_host = torch.randn(LAYERS, n_seqs, kvh, D, generator=g7).to(torch.bfloat16).pin_memory()
    v_host = torch.randn(LAYERS, n_seqs, kvh, D, generator=g7).to(torch.bfloat16).pin_memory()
    q_dev, k_dev, v_dev = q_host.to(dev), k_host.to(dev), v_host.to(dev)
    q_rot = torch.empty_like(q_dev)
    # [layers][seqs][2048] on every rank; a rank's decode writes its own column slice
    out_full = torch.zeros(LAYERS, n_seqs, Q_HEADS * D, dtype=torch.bfloat16, device=dev)
    out_local = torch.zeros(LAYERS, n_seqs, qh * D, dtype=torch.bfloat16, device=dev)
    gath = torch.zeros(LAYERS, world, n_seqs, qh * D, dtype=torch.bfloat16, device=dev)
    out_host = torch.zeros(LAYERS, n_seqs, Q_HEADS * D, dtype=torch.bfloat16).pin_memory()
    state = {"launches": 0, "bytes": 0, "rows": None}
    hg = None
    if world > 1 and args.exchange == "fused":
        import ctypes
        cudart = ctypes.CDLL("libcudart.so.12")
        hg = paged.HeadGather(local_rank, rank, world, n_seqs, LAYERS, kvh)
        handles = [None] * world
        dist.all_gather_object(handles, hg.handle())
        hg.connect(handles)
        dist.barrier()

    def step():
        for s in ids:
            seqs[s] += 1
            pool.reserve(s, seqs[s])
        pool.batch_set(ids)
        state["bytes"] += LAYERS * sum(decode_bytes(seqs[s]) for s in ids)
        if world == 1:
            pool.decode_step(0, LAYERS, q_dev, k_dev, v_dev, n_seqs * qh * D, n_seqs * kvh * D, cos, sin, q_rot,
                             out_full, Q_HEADS * D, n_seqs * Q_HEADS * D)
            state["launches"] += LAYERS  # one fused kernel per layer
            return
        if hg is not None:
            # one fused kernel per layer; its epilogue stores this rank's columns into every
            # rank's rows (peer stores over NVLink); one arrival wait at the end of the step
            state["rows"] = hg.step(pool, q_dev, k_dev, v_dev, n_seqs * qh * D, n_seqs * kvh * D, cos, sin, q_rot)
            state["launches"] += LAYERS + 1
            return
        for layer in range(LAYERS):
            pool.append(layer, q_dev[layer], k_dev[layer], v_dev[layer], cos, sin, q_rot[layer])
            pool.decode(layer, q_rot[layer], out_local[layer], qh * D)
            dist.all_gather_into_tensor(gath[layer].view(-1), out_local[layer].view(-1))
            out_full[layer].view(n_seqs, world, qh * D).copy_(gath[layer].permute(1, 0, 2))
            state["launches"] += 2

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        k_dev.copy_(k_host, non_blocking=True)
        v_dev.copy_(v_host, non_blocking=True)
        step()
        if hg is not None:  # the rows live in the gather's buffer: device-to-host on the same stream
            assert cudart.cudaMemcpyAsync(ctypes.c_void_p(out_host.data_ptr()), ctypes.c_void_p(state["rows"]),
                                          ctypes.c_size_t(out_host.numel() * 2), 2, None) == 0
        else:
            out_host.copy_(out_full, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        state["bytes"] = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, state["bytes"]

    m0 = sampler.mark()
    for _ in range(args.warmup):
        step()
    state["launches"] = 0
    ms, nbytes = timed(step, args.steps)
    launches = state["launches"]
    ms_e2e, nbytes_e2e = timed(e2e_step, args.steps)

    # dominant kernel alone (this rank's heads), one launch per layer
    pool.batch_set(ids, [0] * n_seqs)

    def decode_only():
        for layer in range(LAYERS):
            pool.decode(layer, q_rot[layer], out_local[layer], qh * D)

    decode_only()
    reps = max(3, args.steps // 2)
    ms_k, _ = timed(decode_only, reps)
    ms_k /= reps * LAYERS
    kern_bytes = sum(decode_bytes(seqs[s]) for s in ids) // world
    achieved = kern_bytes / (ms_k * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    pool.check()
    m1 = sampler.mark()
    gather_check = None
    if hg is not None:
        # layer 0 of the last fused step against an NCCL all-gather of the same decode
        dist.all_gather_into_tensor(gath[0].view(-1), out_local[0].view(-1))
        want = gath[0].permute(1, 0, 2).reshape(n_seqs, Q_HEADS * D)
        got = torch.empty(n_seqs, Q_HEADS * D, dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        assert cudart.cudaMemcpy(ctypes.c_void_p(got.data_ptr()), ctypes.c_void_p(state["rows"]),
                                 ctypes.c_size_t(got.numel() * 2), 3) == 0
        gather_check = float((got.float() - want.float()).abs().max().item())
    if rank == 0:
        line = {
            "fused_gather_vs_allgather_max_abs_diff": gather_check,
            "metric": "paged_decode_attn_hbm_gbs", "value": round(nbytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
            "us_per_token": round(ms / args.steps * 1e3 / n_seqs, 2),
            "us_per_step_per_layer": round(ms / args.steps * 1e3 / LAYERS, 2),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"decode_batch{n_seqs}_ctxU1024-32768_x{LAYERS}layers", "sequences": n_seqs,
                       "tokens_in_cache": int(sum(seqs.values())), "layers": LAYERS, "block_tokens": BLOCK,
                       "block_table": "shared pool, seeded free order, a third of the sequences freed and "
                                      "re-created twice before timing",
                       "parallelism": "1 GPU" if world == 1 else
                                      (f"{kvh} KV head(s) per GPU over {world} GPUs; the decode epilogue stores each "
                                       f"rank's head outputs into every rank's rows over NVLink, one arrival wait per step"
                                       if hg is not None else
                                       f"{kvh} KV head(s) per GPU over {world} GPUs, NCCL all-gather of head outputs per layer"),
                       "l2": "inputs larger than L2"},
            "e2e": {"value": round(nbytes_e2e / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s",
                    "h2d_bytes_per_step": (q_host.numel() + k_host.numel() + v_host.numel()) * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": round(ms_e2e / args.steps, 4)},
            "gpu_launches": launches, "clocks": sampler.stop(m0, m1),
            "roofline": {"bound": "hbm", "kernel": "decode_kernel", "achieved": round(achieved, 1), "peak": peak,
                         "unit": "GB/s", "frac": round(achieved / peak, 4), "peak_source": f"of {peak_kind}",
                         "us_per_launch": round(ms_k * 1e3, 2), "bytes_per_launch": kern_bytes, "traffic": None},
        }
        print(json.dumps(line), flush=True)
    barrier()
    if hg is not None:
        hg.close()
    pool.close()
    if world > 1:
        dist.destroy_process_group()


# =============================================================================
# prefill workload (config 3): 2048 tokens x 16 layers, causal, batch 1
# =============================================================================
PREFILL_TOKENS = 2048


def run_qkv(args):
    """Q/K/V projections of a decode step (the producer in front of the attention path): batch 1,
    hidden 2048 -> q 2048 + k 512 + v 512 columns, all layers of the step.  A step reads every layer's
    weights once (12.6 MB per layer), so the metric is achieved HBM GB/s.  N>1: independent replicas."""
    import torch
    import torch.distributed as dist

    from llama_transformer_runtime_b200 import paged

    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    if args.impl == "reference" and rank != 0:
        return
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    H, NQ, NKV, rows = 2048, 2048, 512, 1
    gen = torch.Generator(device=dev)
    gen.manual_seed(99 + rank)
    # 8 rotating weight sets (1.6 GB) so that no step finds its weights in L2 (126 MB)
    SETS = 8 if args.impl == "ours" else 2
    wq = [(torch.randn(LAYERS, H, NQ, generator=gen, device=dev) * 0.03).to(torch.bfloat16) for _ in range(SETS)]
    wk = [(torch.randn(LAYERS, H, NKV, generator=gen, device=dev) * 0.03).to(torch.bfloat16) for _ in range(SETS)]
    wv = [(torch.randn(LAYERS, H, NKV, generator=gen, device=dev) * 0.03).to(torch.bfloat16) for _ in range(SETS)]
    x_host = torch.randn(LAYERS, rows, H, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    q = torch.zeros(LAYERS, rows, NQ, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(LAYERS, rows, NKV, dtype=torch.bfloat16, device=dev)
    v = torch.zeros(LAYERS, rows, NKV, dtype=torch.bfloat16, device=dev)
    out_host = torch.zeros(LAYERS, rows, NQ + 2 * NKV, dtype=torch.bfloat16).pin_memory()
    bytes_layer = (H * (NQ + 2 * NKV) + rows * H + rows * (NQ + 2 * NKV)) * 2
    state = {"i": 0}

    if args.impl == "reference":
        from oracle import oracle as orc
        ref = orc.ref()

        def step():
            # as Attention::forward drives it (src/runtime/attention.cu:138-191): three GEMM launches
            # per layer, a device synchronisation after each
            s = state["i"] % SETS
            state["i"] += 1
            for l in range(LAYERS):
                for w, o, n in ((wq[s], q, NQ), (wk[s], k, NKV), (wv[s], v, NKV)):
                    ref.ref_gemm(x_dev[l].data_ptr(), w[l].data_ptr(), o[l].data_ptr(), rows, n, H)
                    torch.cuda.synchronize()
        launches_per_step = 3 * LAYERS
    else:
        # weights repacked once, at load time, into the tile images both projection kernels read
        pq = [paged.pack_projection_weights(w) for w in wq]
        pk = [paged.pack_projection_weights(w) for w in wk]
        pv = [paged.pack_projection_weights(w) for w in wv]
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()

        def step():
            s = state["i"] % SETS
            state["i"] += 1
            if (not args.qkv_packed):
                paged.qkv_project(x_dev, wq[s], wk[s], wv[s], q, k, v, rows, LAYERS)
            else:
                paged.qkv_project_packed(x_dev, pq[s], pk[s], pv[s], q, k, v, rows, status, LAYERS)
        launches_per_step = 1

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        step()
        out_host[:, :, :NQ].copy_(q, non_blocking=True)
        out_host[:, :, NQ:NQ + NKV].copy_(k, non_blocking=True)
        out_host[:, :, NQ + NKV:].copy_(v, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1 and args.impl == "ours":
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1 and args.impl == "ours":
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    m0 = sampler.mark()
    for _ in range(args.warmup):
        step()
    ms = timed(step, args.steps)
    ms_e2e = timed(e2e_step, args.steps)
    m1 = sampler.mark()
    n_rep = world if args.impl == "ours" else 1
    value = n_rep * LAYERS * bytes_layer * args.steps / (ms * 1e-3) / 1e9
    e2e_value = n_rep * LAYERS * bytes_layer * args.steps / (ms_e2e * 1e-3) / 1e9
    if rank == 0:
        peak, peak_kind = measured_peak()
        line = {
            "metric": "qkv_project_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
            "us_per_layer": round(ms / args.steps * 1e3 / LAYERS, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"qkv_projection_decode_batch1_x{LAYERS}layers", "hidden": H, "q_cols": NQ,
                       "kv_cols": NKV, "rows": rows, "layers": LAYERS,
                       "parallelism": "1 GPU" if world == 1 else f"{world} independent replicas",
                       "l2": f"{SETS} weight sets in rotation ({SETS * LAYERS * bytes_layer / 1e9:.2f} GB), larger than L2"},
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": round(ms_e2e / args.steps, 4)},
            "gpu_launches": launches_per_step * args.steps, "clocks": sampler.stop(m0, m1),
        }
        if args.impl == "reference":
            line["impl"] = "reference"
            line["cpu_baseline"] = {"value": line["value"], "unit": "GB/s", "cores": os.cpu_count(), "kind": "reference",
                                    "sample": "the reference has no CPU implementation of its GEMMs: its own CUDA "
                                              "kernels (gemm_2048x2048.cu, gemm_2048x512.cu) run on the GPU, driven "
                                              "as Attention::forward drives them"}
            line["e2e"]["h2d_bytes_per_step"] = 0
            line["e2e"]["d2h_bytes_per_step"] = 0
            line["e2e"]["value"] = line["value"]
        else:
            line["roofline"] = {"bound": "hbm", "kernel": "qkv_project_kernel" if (not args.qkv_packed) else "qkv_project_packed_kernel", "achieved": round(value / n_rep, 1),
                                "peak": peak, "unit": "GB/s", "frac": round(value / n_rep / peak, 4),
                                "peak_source": f"of {peak_kind}", "us_per_launch": round(ms / args.steps * 1e3, 2),
                                "bytes_per_launch": LAYERS * bytes_layer, "traffic": None}
            # CPU baseline: the oracle's GEMM restatement (double accumulation, OpenMP) on layer 0
            from oracle import oracle as orc
            import time
            xs = x_host[0].view(torch.int16).numpy().view(np.uint16)
            ws = [w[0][0].cpu().view(torch.int16).numpy().view(np.uint16) for w in (wq, wk, wv)]
            t0 = time.perf_counter()
            reps = 0
            while time.perf_counter() - t0 < 10.0:
                outs = [orc.gemm_bf16(xs, w) for w in ws]
                reps += 1
            dt = (time.perf_counter() - t0) / reps
            got = torch.cat([q[0], k[0], v[0]], dim=1).cpu().view(torch.int16).numpy().view(np.uint16)
            # the last timed step used weight set (i - 1) % SETS; recompute layer 0 with set 0 for the check
            if (not args.qkv_packed):
                paged.qkv_project(x_dev, wq[0], wk[0], wv[0], q, k, v, rows, LAYERS)
            else:
                paged.qkv_project_packed(x_dev, pq[0], pk[0], pv[0], q, k, v, rows, status, LAYERS)
            torch.cuda.synchronize()
            assert (not args.qkv_packed) or int(status.item()) == 0
            got = torch.cat([q[0], k[0], v[0]], dim=1).cpu().view(torch.int16).numpy().view(np.uint16)
            want = np.concatenate(outs, axis=1)
            err = float(np.abs(orc.bf16_to_f32(got) - orc.bf16_to_f32(want)).max())
            line["cpu_baseline"] = {"value": round(bytes_layer / dt / 1e9, 2), "unit": "GB/s",
                                    "cores": orc.num_threads(), "kind": "port",
                                    "sample": f"layer 0 of the workload, {reps} repetitions in {dt * reps:.1f} s",
                                    "gpu_vs_cpu_max_abs_err": err}
        print(json.dumps(line), flush=True)
    barrier()
    if world > 1 and dist.is_initialized():
        dist.destroy_process_group()



def run_qkv_prefill(args):
    """Q/K/V projections of a 2048-token prompt, 16 layers: x [2048, 2048] times Wq, Wk, Wv, RoPE on Q and
    K, K/V appended to the paged cache.  Ours: one tcgen05 GEMM launch per layer with RoPE and the append
    as its epilogue.  Reference arm: its 3 GEMM launches (a device synchronisation after each, as
    Attention::forward does), its RoPE/transpose kernels and the strided form of its append copies."""
    import torch

    rank, local_rank, world = dist_env()
    if rank != 0:
        return  # independent replicas only
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    S, H, NQ, NKV = PREFILL_TOKENS, 2048, Q_HEADS * D, KV_HEADS * D
    sampler = ClockSampler(local_rank)
    sampler.start()
    gen = torch.Generator(device=dev)
    gen.manual_seed(123)
    x = torch.randn(LAYERS, S, H, generator=gen, device=dev).to(torch.bfloat16)
    wq = (torch.randn(LAYERS, H, NQ, generator=gen, device=dev) * 0.03).to(torch.bfloat16)
    wk = (torch.randn(LAYERS, H, NKV, generator=gen, device=dev) * 0.03).to(torch.bfloat16)
    wv = (torch.randn(LAYERS, H, NKV, generator=gen, device=dev) * 0.03).to(torch.bfloat16)
    x_host = x.cpu().pin_memory()
    q_rot = torch.zeros(LAYERS, S, NQ, dtype=torch.bfloat16, device=dev)
    q_host = torch.zeros(S, NQ, dtype=torch.bfloat16).pin_memory()
    burst, sustained, kind = measured_tflops()
    flops_layer = 2.0 * S * H * (NQ + 2 * NKV)

    if args.impl == "reference":
        from oracle import oracle as orc
        if not orc.ref_available():
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built"}))
            return
        ref = orc.ref()
        cos_h, sin_h = orc.build_rope_tables(S)
        cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
        ql = torch.empty(S, NQ, dtype=torch.bfloat16, device=dev)
        kl = torch.empty(S, NKV, dtype=torch.bfloat16, device=dev)
        vl = torch.empty(S, NKV, dtype=torch.bfloat16, device=dev)
        qf = torch.empty(Q_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        kf = torch.empty(KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vf = torch.empty_like(kf)
        kc = torch.zeros(LAYERS, KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)

        def step():
            for l in range(LAYERS):
                for w, o, n in ((wq, ql, NQ), (wk, kl, NKV), (wv, vl, NKV)):
                    ref.ref_gemm(x[l].data_ptr(), w[l].data_ptr(), o.data_ptr(), S, n, H)
                    torch.cuda.synchronize()
                ref.ref_rope_qkv(ql.data_ptr(), qf.data_ptr(), kl.data_ptr(), kf.data_ptr(), vl.data_ptr(),
                                 vf.data_ptr(), cos.data_ptr(), sin.data_ptr(), S, 0)
                ref.ref_append_strided(kc[l].data_ptr(), vc[l].data_ptr(), kf.data_ptr(), vf.data_ptr(), S, 0, S, None)
        launches_per_step = LAYERS * 8
    else:
        from llama_transformer_runtime_b200 import paged
        nb = (S + BLOCK - 1) // BLOCK
        num_blocks = nb + nb // 4 + 8
        pool = paged.KVPool(LAYERS, num_blocks, KV_HEADS, 1, nb + 1, device=local_rank)
        pool.set_free_order(np.random.default_rng(5).permutation(num_blocks))
        seq = pool.create_seq()
        pool.reserve(seq, S)
        pool.reserve_rows(S, H)
        pool.batch_set([seq], [S])
        cos_h, sin_h = paged.build_rope_tables(S)
        cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)

        # weights are repacked once, at load time, into the tile image the GEMM bulk-copies
        pq, pk, pv = (paged.pack_projection_weights(w) for w in (wq, wk, wv))
        torch.cuda.synchronize()

        def step():
            # the same prompt positions are rewritten every step (the table is fixed)
            for l in range(LAYERS):
                pool.qkv_project_append(l, x[l], pq[l], pk[l], pv[l], cos, sin, q_rot[l], H)
        launches_per_step = LAYERS

    def e2e_step():
        x.copy_(x_host, non_blocking=True)
        step()
        if args.impl != "reference":
            q_host.copy_(q_rot[LAYERS - 1], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    m0 = sampler.mark()
    for _ in range(args.warmup):
        step()
    ms = timed(step, args.steps) / args.steps
    ms_e2e = timed(e2e_step, args.steps) / args.steps
    value = flops_layer * LAYERS / (ms * 1e-3) / 1e12
    line = {
        "metric": "qkv_project_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "us_per_layer": round(ms * 1e3 / LAYERS, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"qkv_projection_rope_append_{S}tokens_x{LAYERS}layers", "tokens": S, "hidden": H,
                   "q_cols": NQ, "kv_cols": NKV, "layers": LAYERS, "flops": "2*tokens*hidden*(q_cols+2*kv_cols) per layer",
                   "l2": "per-layer inputs and weights are distinct tensors (20.6 MB per layer, 330 MB per step)"},
        "e2e": {"value": round(flops_layer * LAYERS / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": 0 if args.impl == "reference" else q_host.numel() * 2,
                "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": launches_per_step * args.steps,
    }
    if args.impl == "reference":
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                "sample": "whole workload on the GPU: the reference has no CPU implementation of its GEMMs"}
        line["e2e"]["h2d_bytes_per_step"] = 0
        line["e2e"]["value"] = line["value"]
    else:
        line["roofline"] = {"bound": "tensor", "kernel": "qkv_gemm_kernel", "achieved": round(value, 2), "peak": burst,
                            "unit": "TFLOP/s", "frac": round(value / burst, 4),
                            "peak_source": f"of {kind} (cuBLAS bf16 burst)", "us_per_launch": round(ms * 1e3 / LAYERS, 2),
                            "flops_per_launch": flops_layer, "traffic": None}
        pool.check()
        # CPU baseline and check: the oracle's GEMM on the first 64 rows of layer 0, q columns
        from oracle import oracle as orc
        import time
        rows = 64
        xs = x_host[0, :rows].contiguous().view(torch.int16).numpy().view(np.uint16)
        ws = wq[0].cpu().view(torch.int16).numpy().view(np.uint16)
        t0 = time.perf_counter()
        lin = orc.gemm_bf16(xs, ws)
        dt = time.perf_counter() - t0
        want = orc.rope(lin.reshape(rows, Q_HEADS, D), cos_h, sin_h, 0, 1, out_token_major=True).reshape(rows, NQ)
        got = q_rot[0, :rows].cpu().view(torch.int16).numpy().view(np.uint16)
        err = float(np.abs(orc.bf16_to_f32(got) - orc.bf16_to_f32(want)).max())
        line["cpu_baseline"] = {"value": round(2.0 * rows * H * NQ / dt / 1e12, 5), "unit": "TFLOP/s",
                                "cores": orc.num_threads(), "kind": "port",
                                "sample": f"{rows} rows x {NQ} columns of layer 0 (double accumulation), {dt:.2f} s",
                                "gpu_vs_cpu_max_abs_err": err}
        pool.close()
    line["clocks"] = sampler.stop(m0, None)
    print(json.dumps(line), flush=True)


def prefill_flops(S: int) -> float:
    """Causal-useful flops of one layer: 4 * Hq * D * S (S + 1) / 2."""
    return 4.0 * Q_HEADS * D * S * (S + 1) / 2.0


def measured_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            j = json.load(open(path))
            return float(j["bf16_tflops"]), float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), "measured"
        except Exception:
            pass
    return 1590.0, 1400.0, "fallback"


def run_prefill(args):
    """One step = one 2048-token prompt through 16 layers: per layer fused RoPE +
    paged append of the prompt's K/V, then causal GQA attention over the cache,
    output [2048, 2048] bf16.  Both arms: ours (pa_append + pa_prefill) and the
    reference's kernels (rope kernels + append copies + flash kernel + layout)."""
    import torch

    rank, local_rank, world = dist_env()
    if rank != 0:
        return  # independent replicas only: prefill is not sharded here
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    S = PREFILL_TOKENS
    sampler = ClockSampler(local_rank)
    sampler.start()
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)
    # per-layer inputs differ so that no layer finds its operands in L2 from the previous one
    q_in = torch.randn(LAYERS, S, Q_HEADS, D, generator=gen, device=dev).to(torch.bfloat16)
    k_in = torch.randn(LAYERS, S, KV_HEADS, D, generator=gen, device=dev).to(torch.bfloat16)
    v_in = torch.randn(LAYERS, S, KV_HEADS, D, generator=gen, device=dev).to(torch.bfloat16)
    out = torch.zeros(LAYERS, S, Q_HEADS * D, dtype=torch.bfloat16, device=dev)
    q_host, k_host, v_host = q_in.cpu().pin_memory(), k_in.cpu().pin_memory(), v_in.cpu().pin_memory()
    out_host = torch.zeros(S, Q_HEADS * D, dtype=torch.bfloat16).pin_memory()
    burst, sustained, kind = measured_tflops()

    if args.impl == "reference":
        from oracle import oracle as orc
        if not orc.ref_available():
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built"}))
            return
        ref = orc.ref()
        cos_h, sin_h = orc.build_rope_tables(S)
        cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
        kc = torch.zeros(LAYERS, KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        qf = torch.empty(Q_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        kf = torch.empty(KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vf = torch.empty_like(kf)
        of = torch.empty(Q_HEADS, S, D, dtype=torch.bfloat16, device=dev)

        def step():
            for layer in range(LAYERS):
                ref.ref_rope_qkv(q_in[layer].data_ptr(), qf.data_ptr(), k_in[layer].data_ptr(), kf.data_ptr(),
                                 v_in[layer].data_ptr(), vf.data_ptr(), cos.data_ptr(), sin.data_ptr(), S, 0)
                # the reference's own append is 2*8*2048 copies of 128 bytes per layer; the
                # strided form moves the same bytes in 16 calls (kernel-to-kernel comparison)
                if args.ref_literal_append:
                    ref.ref_append_memcpy_loop(kc[layer].data_ptr(), vc[layer].data_ptr(), kf.data_ptr(),
                                               vf.data_ptr(), S, 0, S)
                else:
                    ref.ref_append_strided(kc[layer].data_ptr(), vc[layer].data_ptr(), kf.data_ptr(),
                                           vf.data_ptr(), S, 0, S, None)
                ref.ref_flash_attention(qf.data_ptr(), kc[layer].data_ptr(), vc[layer].data_ptr(), of.data_ptr(),
                                        None, 1, Q_HEADS, KV_HEADS, S, S, S, 0.125, 1, None)
                ref.ref_flash_output_layout(of.data_ptr(), out[layer].data_ptr(), S)
        launches_per_step = LAYERS * 5
        kernel_name = "flash_attention_fat_kernel (reference)"
    else:
        from llama_transformer_runtime_b200 import paged
        nb = (S + BLOCK - 1) // BLOCK
        num_blocks = nb + nb // 4 + 8
        pool = paged.KVPool(LAYERS, num_blocks, KV_HEADS, 1, nb + 1, device=local_rank)
        pool.set_free_order(np.random.default_rng(5).permutation(num_blocks))
        seq = pool.create_seq()
        pool.reserve(seq, S)
        pool.batch_set([seq], [S])
        cos_h, sin_h = paged.build_rope_tables(S)
        cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
        q_rot = torch.empty_like(q_in)

        def step():
            # the same prompt positions are rewritten every step (the table is fixed)
            for layer in range(LAYERS):
                pool.append(layer, q_in[layer], k_in[layer], v_in[layer], cos, sin, q_rot[layer])
                pool.prefill(layer, q_rot[layer], out[layer], None, 0.125)
        launches_per_step = LAYERS * 2
        kernel_name = "prefill_kernel"

    def e2e_step():
        q_in.copy_(q_host, non_blocking=True)
        k_in.copy_(k_host, non_blocking=True)
        v_in.copy_(v_host, non_blocking=True)
        step()
        out_host.copy_(out[LAYERS - 1], non_blocking=True)  # the last layer's attention output
        torch.cuda.current_stream().synchronize()

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    m0 = sampler.mark()
    for _ in range(args.warmup):
        step()
    ms = timed(step, args.steps) / args.steps
    ms_e2e = timed(e2e_step, args.steps) / args.steps
    flops = prefill_flops(S) * LAYERS
    value = flops / (ms * 1e-3) / 1e12
    line = {
        "metric": "prefill_attn_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "us_per_layer": round(ms * 1e3 / LAYERS, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"prefill_{S}tokens_x{LAYERS}layers_batch1_causal", "tokens": S, "layers": LAYERS,
                   "q_heads": Q_HEADS, "kv_heads": KV_HEADS, "head_dim": D,
                   "flops": "causal-useful 4*Hq*D*S(S+1)/2 per layer",
                   "dense_count_tflops": round(4.0 * Q_HEADS * D * S * S * LAYERS / (ms * 1e-3) / 1e12, 2),
                   "l2": "per-layer inputs are distinct tensors (24 MiB per layer, 384 MiB per step)"},
        "e2e": {"value": round(flops / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": (q_host.numel() + k_host.numel() + v_host.numel()) * 2,
                "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": launches_per_step * args.steps,
    }
    if args.impl == "reference":
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                "sample": "whole workload on the GPU: the reference has no CPU implementation of this path"}
    else:
        # dominant kernel alone
        def attn_only():
            for layer in range(LAYERS):
                pool.prefill(layer, q_rot[layer], out[layer], None, 0.125)
        attn_only()
        reps = max(3, args.steps)
        ms_k = timed(attn_only, reps) / (reps * LAYERS)
        achieved = prefill_flops(S) / (ms_k * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor", "kernel": kernel_name, "achieved": round(achieved, 2),
                            "peak": burst, "unit": "TFLOP/s", "frac": round(achieved / burst, 4),
                            "peak_source": f"of {kind} (cuBLAS bf16 burst)", "us_per_launch": round(ms_k * 1e3, 2),
                            "flops_per_launch": prefill_flops(S), "traffic": None}
        pool.check()
        line["cpu_baseline"] = prefill_cpu_baseline(q_rot, out, pool, seq, S)
        pool.close()
    line["clocks"] = sampler.stop(m0, None)
    print(json.dumps(line), flush=True)


def prefill_cpu_baseline(q_rot, out, pool, seq, S):
    """fp32 CPU oracle on a bounded sample: the first 512 query rows of layer 0
    (all 32 heads) against their causal keys; also checks the GPU output."""
    import torch

    from oracle import oracle as orc

    n = 512
    k = torch.zeros(KV_HEADS, S, D, dtype=torch.bfloat16, device=q_rot.device)
    v = torch.zeros_like(k)
    pool.gather_kv(0, seq, k, v, S)
    torch.cuda.synchronize()
    to_u16 = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    qh = to_u16(q_rot[0][:n].permute(1, 0, 2))  # [32, n, 64]
    kh, vh = to_u16(k[:, :n]), to_u16(v[:, :n])
    t0 = time.perf_counter()
    O, _ = orc.attention(qh, kh, vh, n, causal=True)
    reps = 1
    while time.perf_counter() - t0 < 10.0 and reps < 200:
        orc.attention(qh, kh, vh, n, causal=True)
        reps += 1
    total = time.perf_counter() - t0
    got = orc.bf16_to_f32(to_u16(out[0][:n]))
    err = float(np.max(np.abs(got - orc.output_layout(O))))
    return {"value": round(prefill_flops(n) * reps / total / 1e12, 4), "unit": "TFLOP/s", "cores": orc.num_threads(),
            "kind": "port", "sample": f"first {n} query rows of layer 0, {reps} passes of the fp32 CPU oracle",
            "gpu_vs_cpu_max_abs_err": err}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode128k", choices=sorted(WORKLOADS) + ["prefill2k", "batch64", "qkv_decode", "qkv_prefill"])
    ap.add_argument("--seqs", type=int, default=64, help="batch64: number of sequences")
    ap.add_argument("--layers", type=int, default=16, help="fewer layers make a small case for profiling")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N>1: partials pushed by the decode epilogue over NVLink (fused) or NCCL all-gather")
    ap.add_argument("--chunk-blocks", type=int, default=0, help="decode: blocks per split-KV chunk (0 = planner)")
    ap.add_argument("--combiners", type=int, default=0, help="decode: combining CTAs per (sequence, head) in the one-launch step (0 = planner)")
    ap.add_argument("--decode-shape", default="", help="decode: WARPSxSTAGES, e.g. 8x4 (empty = planner)")
    ap.add_argument("--qkv-packed", action="store_true",
                    help="qkv_decode: the kernel that reads the packed weight tiles (shared with the prefill GEMM) "
                         "instead of the reference's row-major weights")
    ap.add_argument("--ref-literal-append", action="store_true",
                    help="prefill reference arm: the reference's literal 2*8*tokens 128-byte copies")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global LAYERS
    LAYERS = args.layers
    if args.workload == "qkv_decode":
        run_qkv(args)
    elif args.workload == "qkv_prefill":
        run_qkv_prefill(args)
    elif args.workload == "prefill2k":
        run_prefill(args)
    elif args.workload == "batch64":
        run_batch(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
