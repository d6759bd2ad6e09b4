"""Benchmark of the paged KV-cache attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (decode128k): long-context decode, batch 1, context 131072 x 16 layers (about
4.3 GB of bf16 paged KV, 16-token blocks, seeded random fragmented block table), KV values
N(0,1)*0.5.  One step = one new token: per layer a fused RoPE + paged append, then paged GQA decode
attention over the whole cache.  With N GPUs the sequence is split by token range over the ranks
(strong scaling); every layer ends with an exchange of the ranks' (O, LSE) partials and a
log-sum-exp merge, both inside the decode kernel.

metric  paged_decode_attn_hbm_gbs = algorithmic cache bytes streamed per second, sum over ranks:
        steps x layers x (2048 L + 8192 + 4 ceil(L/16)) / time.  The line also carries
        us_per_token (time per step).
value   inputs resident in HBM; the K timed steps are repeated `--repeats` times (default 15) and
        the median block is reported, so the region under load lasts a few tenths of a second.
e2e     host buffers: per step the new token's q/k/v for all layers go host->device from pinned
        memory and the attention outputs come back, inside the timed region.
dependent_layers
        the same step with the layers strictly one after the other (layer l+1 starts when layer
        l's rows are final): what a forward pass whose layers depend on each other can use.  The
        headline value lets the layers of a step overlap, which needs every layer's q/k/v up front.
The cache is 4.3 GB per step (268 MB per layer): larger than L2, no flush needed.

The default run (one GPU) also measures, after the main region, the other parts of the metric as
sub-blocks of the same JSON line: decode4k (context 4096), prefill (2048 tokens, TFLOP/s), append
(the fused RoPE + append kernel alone), out_project and qkv (the projections either side of the
path), decode_chain (projections -> attention -> output projection per layer with the true data
flow), each with its roofline and the reference's own kernels timed in the same run.  With more
than one GPU it adds batch64 (64 ragged sequences, KV heads sharded over the ranks).
"""
from __future__ import annotations

import argparse
import ctypes
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
HIDDEN = 2048
WORKLOADS = {
    "decode128k": dict(ctx=131072, name="decode_ctx131072_x16layers_batch1"),
    "decode4k": dict(ctx=4096, name="decode_ctx4096_x16layers_batch1"),
}
PREFILL_TOKENS = 2048
ROW_REL = 2.0 ** -7  # scale-aware bar: max error of a 64-wide head row over the row's largest value


def decode_bytes(L: int) -> int:
    """Algorithmic bytes of one layer's decode over a context of L tokens:
    K+V read once, Q read, O written, block table read."""
    return 2 * KV_HEADS * L * D * 2 + 2 * Q_HEADS * D * 2 + 4 * ((L + BLOCK - 1) // BLOCK)


def prefill_flops(S: int) -> float:
    """Causal-useful flops of one layer: 4 * Hq * D * S (S + 1) / 2."""
    return 4.0 * Q_HEADS * D * S * (S + 1) / 2.0


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return json.load(open(path)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def measured_peak():
    j, kind = _peaks()
    return float(j["hbm_gbs"]), kind


def measured_tflops():
    j, kind = _peaks()
    return float(j["bf16_tflops"]), float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), kind


# ncu captures (profiles/): dram read+write bytes per layer of a workload's dominant kernel.
# decode128k: the 2-layer decode_step_kernel capture read 537.10 MB and wrote 6.58 MB.
NCU_TRAFFIC_BYTES = {"decode128k": 271840128, "decode4k": None}
# one 2048-token append_kernel launch: 13.12 MB read from DRAM, 0 written inside the kernel's window (the
# 12.6 MB it writes are still in L2 when it ends)
NCU_APPEND_TRAFFIC = 13116416


def row_rel_err(got: np.ndarray, want: np.ndarray, row: int = 64) -> float:
    """max over 64-wide head rows of max|got - want| / max|want|."""
    err = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)).reshape(-1, row).max(axis=1)
    m = np.abs(np.asarray(want, np.float64)).reshape(-1, row).max(axis=1)
    return float(np.max(err / np.maximum(m, 1e-30)))


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

    def summary(self, lo: int = 0, hi: int | None = None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        rows = [r for r in self.rows[lo:hi] if len(r) >= 6] or [r for r in self.rows if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": float(rows[0][1]) if rows[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(rows)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def token_ranges(L: int, n: int):
    """Split [0, L) into n contiguous ranges on 16-token block borders."""
    blocks = (L + BLOCK - 1) // BLOCK
    cuts = [min(L, (blocks * r // n) * BLOCK) for r in range(n)] + [L]
    return [(cuts[r], cuts[r + 1]) for r in range(n)]


class Env:
    """Rank, device, process group and clock sampler of this process."""

    def __init__(self, want_group: bool):
        import torch
        self.torch = torch
        self.rank, self.local_rank, self.world = dist_env()
        torch.cuda.set_device(self.local_rank)
        self.dev = f"cuda:{self.local_rank}"
        self.dist = None
        if self.world > 1 and want_group:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device(self.dev))
            self.dist = dist
        self.sampler = ClockSampler(self.local_rank)
        if self.rank == 0:
            self.sampler.start()

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, n: int) -> float:
        """n calls of fn between a barrier + synchronize on both sides; CUDA events on the launching
        stream; max over ranks.  Milliseconds."""
        torch = self.torch
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1)
        if self.dist is not None:
            t = torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()
            self.dist = None


def local_timed(torch, fn, n: int) -> float:
    """n calls of fn on this GPU alone: synchronize on both sides, CUDA events.  Milliseconds."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def _u16(t):
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def decode_config(wl, ctx, world, exchange):
    return {"workload": wl["name"], "context": ctx, "layers": LAYERS, "batch": 1,
            "q_heads": Q_HEADS, "kv_heads": KV_HEADS, "head_dim": D, "block_tokens": BLOCK,
            "block_table": "seeded random permutation over a pool 25% larger than the sequence",
            "parallelism": "1 GPU" if world == 1 else (
                f"sequence range split over {world} GPUs; one launch per step, per layer the combining CTAs "
                f"push (O, LSE) to every rank over NVLink (peer stores of value+step words) and merge locally"
                if exchange == "fused" else
                f"sequence range split over {world} GPUs, NCCL all-gather of (O, LSE) per layer + merge"),
            "l2": f"inputs larger than L2 ({decode_bytes(ctx) * LAYERS / 1e9:.2f} GB streamed per step)"}


# =============================================================================
# decode, one sequence, range-sharded over the ranks (decode128k, decode4k)
# =============================================================================
def run_decode(env: Env, args, workload: str, sub: bool = False):
    torch, dist = env.torch, env.dist
    from llama_transformer_runtime_b200 import paged

    rank, local_rank, world, dev = env.rank, env.local_rank, env.world, env.dev
    wl = WORKLOADS[workload]
    if getattr(args, "ctx", 0) and not sub:  # another context length on the same workload (planner experiments)
        wl = dict(ctx=args.ctx, name=f"decode_ctx{args.ctx}_x{LAYERS}layers_batch1")
    ctx = wl["ctx"]
    steps = args.steps
    repeats = 5 if sub else max(1, args.repeats)
    e2e_repeats = 2 if sub else min(5, repeats)
    total_steps = args.warmup + steps * (repeats + e2e_repeats + 6) + 16
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

    state = {"global_len": ctx, "launches": 0, "fused_steps": 0}

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
            state["fused_steps"] += 1
            return
        pool.batch_set_sharded([seq], [1 if rank == owner else 0], [1], [g - 1], [lo])
        if xchg is not None:
            paged.decode_step_sharded(pool, xchg, 0, LAYERS, qs, ks if rank == owner else None,
                                      vs if rank == owner else None, Q_HEADS * D, KV_HEADS * D, cos, sin,
                                      q_rot, outs, Q_HEADS * D, Q_HEADS * D)
            state["fused_steps"] += 1
            return
        for layer in range(LAYERS):
            pool.append(layer, qs[layer], ks[layer], vs[layer], cos, sin, q_rot[layer])
            pool.decode(layer, q_rot[layer], None, 0, part[layer, :Q_HEADS * D], part[layer, Q_HEADS * D:])
            dist.all_gather_into_tensor(gathered[layer].view(-1), part[layer])
            o_parts.copy_(gathered[layer, :, :Q_HEADS * D].reshape(world, Q_HEADS, D))
            l_parts.copy_(gathered[layer, :, Q_HEADS * D:])
            paged.merge_partials(o_parts, l_parts, world, Q_HEADS, outs[layer])
            state["launches"] += 3

    def resident_step():
        step(q_dev, k_dev, v_dev, out_dev)

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        k_dev.copy_(k_host, non_blocking=True)
        v_dev.copy_(v_host, non_blocking=True)
        step(q_dev, k_dev, v_dev, out_dev)
        out_host.copy_(out_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result every step

    def block(fn):
        """One timed block of `steps` steps -> (ms, algorithmic bytes of those steps)."""
        l0 = state["global_len"]
        ms = env.timed(fn, steps)
        return ms, sum(LAYERS * decode_bytes(L) for L in range(l0 + 1, state["global_len"] + 1))

    m0 = env.sampler.mark()  # clock samples from here on are taken under load
    for _ in range(args.warmup):
        resident_step()
    state["launches"] = 0
    state["fused_steps"] = 0
    one_launch_before = pool.step_launches()
    blocks = [block(resident_step) for _ in range(repeats)]
    one_launch = pool.step_launches() - one_launch_before
    launches = (state["launches"] + one_launch + (state["fused_steps"] - one_launch) * LAYERS) // repeats
    rates = sorted(b / (ms * 1e-3) / 1e9 for ms, b in blocks)
    value = statistics.median(rates)
    ms = statistics.median(m for m, _ in blocks)

    e2e_blocks = [block(e2e_step) for _ in range(e2e_repeats)]
    e2e_value = statistics.median(b / (m * 1e-3) / 1e9 for m, b in e2e_blocks)
    ms_e2e = statistics.median(m for m, _ in e2e_blocks)
    h2d = (q_host.numel() + k_host.numel() + v_host.numel()) * 2
    d2h = out_host.numel() * 2

    # ---- the same step with layers strictly one after the other (no shared launch, no overlap)
    pool.set_layer_overlap(False)
    resident_step()
    dep_blocks = [block(resident_step) for _ in range(2 if sub else 3)]
    pool.set_layer_overlap(True)
    dep_value = statistics.median(b / (m * 1e-3) / 1e9 for m, b in dep_blocks)
    dep_ms = statistics.median(m for m, _ in dep_blocks)

    # ---- dominant kernel alone
    pool.batch_set_sharded([seq], [0], [1], [state["global_len"] - 1], [lo])
    L_local = pool.length(seq)
    local_out = torch.zeros_like(out_dev)

    def decode_only():
        for layer in range(LAYERS):
            pool.decode(layer, q_rot[layer], local_out[layer], Q_HEADS * D, None, None)

    decode_only()
    reps = max(3, steps)
    ms_iso = env.timed(decode_only, reps) / (reps * LAYERS)  # plain launches of one layer each

    # the step's own launch on this rank's range without the host's table work and without the
    # cross-rank exchange (decode_step_kernel: all layers, query rotation fused in)
    def step_kernels():
        pool.decode_step(0, LAYERS, q_dev, None, None, Q_HEADS * D, KV_HEADS * D, cos, sin, q_rot,
                         local_out, Q_HEADS * D, Q_HEADS * D)

    step_kernels()
    ms_k = env.timed(step_kernels, reps) / (reps * LAYERS)
    kern_bytes = decode_bytes(L_local)
    achieved = kern_bytes / (ms_k * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    pool.check()
    m1 = env.sampler.mark()

    # ---- checks of the last step's rows (one more one-launch step so they come from that path)
    resident_step()
    torch.cuda.synchronize()
    pool.check()
    checks = {}
    if world > 1:
        # every layer: the merged rows against an NCCL all-gather + merge of the same partials
        pool.batch_set_sharded([seq], [0], [1], [state["global_len"] - 1], [lo])
        worst = 0.0
        for layer in range(LAYERS):
            pool.decode(layer, q_rot[layer], None, 0, part[layer, :Q_HEADS * D], part[layer, Q_HEADS * D:])
            dist.all_gather_into_tensor(gathered[layer].view(-1), part[layer])
            o_parts.copy_(gathered[layer, :, :Q_HEADS * D].reshape(world, Q_HEADS, D))
            l_parts.copy_(gathered[layer, :, Q_HEADS * D:])
            chk = torch.zeros(1, Q_HEADS * D, dtype=torch.bfloat16, device=dev)
            paged.merge_partials(o_parts, l_parts, world, Q_HEADS, chk)
            torch.cuda.synchronize()
            worst = max(worst, float((chk.float() - out_dev[layer].float()).abs().max().item()))
        t = torch.tensor([worst], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        checks["exchange_vs_allgather_max_abs_diff_all_layers"] = float(t.item())
    cpu = cpu_check_and_baseline(env, pool, seq, q_rot, out_dev, pool.length(seq), budget_s=(2.0 if sub else 10.0))

    line = None
    if rank == 0:
        clocks = env.sampler.summary(m0, m1)
        roof = {"bound": "hbm", "kernel": "decode_step_kernel", "achieved": round(achieved, 1),
                "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                "peak_source": f"of {peak_kind}", "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                "us_per_launch": round(ms_k * 1e3 * LAYERS, 2), "bytes_per_launch": kern_bytes * LAYERS,
                "layers_per_launch": LAYERS, "us_per_layer": round(ms_k * 1e3, 2),
                "us_per_layer_plain_decode_kernel": round(ms_iso * 1e3, 2),
                "how": (f"CUDA events around this rank's one-launch step over its own token range (all {LAYERS} layers, "
                        f"no cross-rank exchange), {reps} launches"),
                "traffic": (NCU_TRAFFIC_BYTES[workload] * LAYERS
                            if world == 1 and NCU_TRAFFIC_BYTES.get(workload) and LAYERS >= 2 else None)}
        if world == 1:
            roof["traffic_note"] = "ncu capture of a 2-layer decode_step_kernel launch, per layer x layers"
        else:
            # what the exchange adds per layer on top of this rank's own stream + combine
            roof["per_rank_gbs_in_the_step"] = round(value / world, 1)
            roof["exchange_share"] = round(max(0.0, 1.0 - (ms_k * LAYERS) / (ms / steps)), 4)
        line = {
            "metric": "paged_decode_attn_hbm_gbs", "value": round(value, 1), "unit": "GB/s",
            "n_gpus": world, "steps": steps, "warmup": args.warmup,
            "ms_per_step": round(ms / steps, 4),
            "us_per_token": round(ms / steps * 1e3, 2),
            "us_per_token_per_layer": round(ms / steps * 1e3 / LAYERS, 2),
            "repeats": repeats, "value_min": round(rates[0], 1), "value_max": round(rates[-1], 1),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": decode_config(wl, ctx, world, args.exchange),
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(ms_e2e / steps, 4)},
            "dependent_layers": {"value": round(dep_value, 1), "unit": "GB/s", "ms_per_step": round(dep_ms / steps, 4),
                                 "us_per_token_per_layer": round(dep_ms / steps * 1e3 / LAYERS, 2),
                                 "how": "one kernel per layer, layer l+1 launched behind layer l with no overlap "
                                        "(pa_pool_set_layer_overlap(pool, 0)); the exchange and merge stay in the kernel"},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": roof,
            "checks": {**checks, **{k: v for k, v in cpu.items() if k.startswith("oracle_")}},
        }
        if world == 1:
            line["cpu_baseline"] = {k: v for k, v in cpu.items() if not k.startswith("oracle_")}
    env.barrier()
    if xchg is not None:
        xchg.close()
    pool.close()
    return line


def cpu_check_and_baseline(env: Env, pool, seq, q_rot, out_dev, L, budget_s=10.0):
    """The CPU oracle (fp32 naive attention, OpenMP) on layer 0 of this rank's token range.  Every
    rank computes its partial (O, LSE); the partials are merged on the host with the oracle's
    log-sum-exp merge and compared with the GPU's merged row.  On one GPU the same passes, repeated
    for about `budget_s` seconds, are also the timed CPU baseline."""
    torch, dist = env.torch, env.dist
    from oracle import oracle as orc

    dev = q_rot.device
    q_h = _u16(q_rot[0]).reshape(Q_HEADS, 1, D)
    reps, total = 1, 0.0
    if L > 0:
        k = torch.zeros(KV_HEADS, L, D, dtype=torch.bfloat16, device=dev)
        v = torch.zeros_like(k)
        pool.gather_kv(0, seq, k, v, L)
        torch.cuda.synchronize()
        k_h, v_h = _u16(k), _u16(v)
        del k, v
        t0 = time.perf_counter()
        O, lse = orc.attention(q_h, k_h, v_h, L, causal=False)
        t1 = time.perf_counter() - t0
        if env.world == 1:
            while t1 * reps < budget_s and reps < 64:
                orc.attention(q_h, k_h, v_h, L, causal=False)
                reps += 1
        total = time.perf_counter() - t0
    else:
        O = np.zeros((Q_HEADS, 1, D), np.float32)
        lse = np.full((Q_HEADS, 1), -np.inf, np.float32)
    if env.world > 1:
        mine = torch.from_numpy(np.concatenate([O[:, 0].reshape(-1), lse[:, 0]]).astype(np.float32)).to(dev)
        allp = torch.zeros(env.world, mine.numel(), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(allp.view(-1), mine)
        a = allp.cpu().numpy()
        want, _ = orc.lse_merge(a[:, :Q_HEADS * D].reshape(env.world, Q_HEADS, D), a[:, Q_HEADS * D:])
        want = want.reshape(-1)
    else:
        want = O[:, 0].reshape(-1)
    got = orc.bf16_to_f32(_u16(out_dev[0])).reshape(-1)
    res = {"oracle_layer0_max_abs_err": float(np.max(np.abs(got - want))),
           "oracle_layer0_max_row_rel_err": row_rel_err(got, want),
           "oracle_row_rel_bar": ROW_REL}
    res["oracle_layer0_ok"] = bool(res["oracle_layer0_max_row_rel_err"] <= ROW_REL)
    if env.world == 1:
        res.update({"value": round(decode_bytes(L) * reps / total / 1e9, 3), "unit": "GB/s",
                    "cores": orc.num_threads(), "kind": "port",
                    "sample": f"layer 0 of the workload (context {L}), {reps} passes of the fp32 CPU oracle",
                    "gpu_vs_cpu_max_abs_err": res["oracle_layer0_max_abs_err"]})
    return res


# =============================================================================
# reference arm: the reference's own CUDA kernels (oracle/_ref/libref.so) on this GPU
# =============================================================================
def reference_decode(env: Env, workload: str, steps: int, warmup: int, with_e2e: bool = True):
    """What Attention::forward does per layer for one token (steps 5-7): launch_rope_qkv, the
    128-byte append copies, launch_flash_attention with q_seq_len 1, launch_flash_output_layout.
    Returns a dict of rates and times, or None when the reference kernels were not built."""
    from oracle import oracle as orc
    torch = env.torch
    if not orc.ref_available():
        return None
    dev = env.dev
    ref = orc.ref()
    ctx = WORKLOADS[workload]["ctx"]
    total_steps = warmup + 2 * steps + 4
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
        l0 = state["len"]
        ms = local_timed(torch, fn, n)
        return ms, sum(LAYERS * decode_bytes(L) for L in range(l0 + 1, state["len"] + 1))

    for _ in range(warmup):
        step()
    ms, b = timed(step, steps)
    res = {"value": b / (ms * 1e-3) / 1e9, "ms_per_step": ms / steps,
           "h2d": (q_host.numel() + k_host.numel() + v_host.numel()) * 2, "d2h": out_host.numel() * 2}
    if with_e2e:
        ms2, b2 = timed(e2e_step, steps)
        res.update({"e2e_value": b2 / (ms2 * 1e-3) / 1e9, "e2e_ms_per_step": ms2 / steps})
    return res


def run_reference(env: Env, args, workload: str):
    if env.rank != 0:
        return None
    m0 = env.sampler.mark()
    time.sleep(0.2)
    r = reference_decode(env, workload, args.steps, args.warmup)
    if r is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built (no reference checkout at build time)"}
    wl = WORKLOADS[workload]
    cfg = decode_config(wl, wl["ctx"], 1, "fused")
    cfg["note"] = ("the reference's own CUDA kernels (flashattention.cu, rope.cu, layout.cu compiled unmodified for "
                   "sm_100a) on this GPU, contiguous cache, single GPU only")
    return {
        "impl": "reference", "metric": "paged_decode_attn_hbm_gbs", "value": round(r["value"], 2), "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(r["ms_per_step"], 4),
        "us_per_token": round(r["ms_per_step"] * 1e3, 2), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
        "e2e": {"value": round(r["e2e_value"], 2), "unit": "GB/s", "h2d_bytes_per_step": r["h2d"],
                "d2h_bytes_per_step": r["d2h"], "ms_per_step": round(r["e2e_ms_per_step"], 4)},
        "gpu_launches": args.steps * LAYERS * 5, "clocks": env.sampler.summary(m0, None),
        "cpu_baseline": {"value": round(r["value"], 2), "unit": "GB/s", "cores": 0, "kind": "reference",
                         "sample": "whole workload; the reference has no CPU implementation of this path, "
                                   "so its CUDA kernels run on the GPU (host cores only drive the launches)"},
    }


# =============================================================================
# batched decode workload: 64 ragged sequences, shared fragmented pool, KV heads sharded
# =============================================================================
def run_batch(env: Env, args, sub: bool = False):
    """64 sequences with context lengths seeded-uniform in [1024, 32768], one shared free-block
    pool; before timing, rounds of freeing and re-creating sequences interleave their tables.  One
    step = every sequence appends one token and attends over its cache, 16 layers.  With N GPUs the
    8 KV heads are sharded (8/N per GPU, each with the 4*8/N query heads of its groups); every
    layer's head outputs are gathered into [64, 2048] on every rank by the decode kernel's own
    peer stores.  Strong scaling: the same batch is split N ways."""
    torch, dist = env.torch, env.dist
    from llama_transformer_runtime_b200 import paged

    rank, local_rank, world, dev = env.rank, env.local_rank, env.world, env.dev
    if args.impl == "reference":
        return {"impl": "reference", "unavailable":
                "the reference is single-sequence and contiguous; this workload has no reference arm "
                "(see the decode128k and prefill2k workloads)"} if rank == 0 else None
    n_seqs = args.seqs
    steps = max(2, args.steps // 4) if sub else args.steps
    warmup = 3 if sub else args.warmup
    kvh = KV_HEADS // world
    qh = 4 * kvh
    rng = np.random.default_rng(2024)  # the same allocator decisions on every rank
    lens = rng.integers(1024, 32769, n_seqs).astype(int)
    total_steps = warmup + 2 * steps + 8
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
    cudart = ctypes.CDLL("libcudart.so.12")
    if world > 1 and args.exchange == "fused":
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

    def timed(fn, n):
        state["bytes"] = 0
        ms = env.timed(fn, n)
        return ms, state["bytes"]

    m0 = env.sampler.mark()
    for _ in range(warmup):
        step()
    state["launches"] = 0
    ms, nbytes = timed(step, steps)
    launches = state["launches"]
    ms_e2e, nbytes_e2e = timed(e2e_step, steps)

    # dominant kernel alone (this rank's heads), one launch per layer
    pool.batch_set(ids, [0] * n_seqs)

    def decode_only():
        for layer in range(LAYERS):
            pool.decode(layer, q_rot[layer], out_local[layer], qh * D)

    decode_only()
    reps = max(3, steps // 2)
    ms_k, _ = timed(decode_only, reps)
    ms_k /= reps * LAYERS
    kern_bytes = sum(decode_bytes(seqs[s]) for s in ids) // world
    achieved = kern_bytes / (ms_k * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    pool.check()
    m1 = env.sampler.mark()
    gather_check = None
    if hg is not None:
        # every layer of the last fused step against an NCCL all-gather of the same decode
        gather_check = 0.0
        torch.cuda.synchronize()
        got_all = torch.empty(LAYERS, n_seqs, Q_HEADS * D, dtype=torch.bfloat16, device=dev)
        assert cudart.cudaMemcpy(ctypes.c_void_p(got_all.data_ptr()), ctypes.c_void_p(state["rows"]),
                                 ctypes.c_size_t(got_all.numel() * 2), 3) == 0
        for layer in range(LAYERS):
            dist.all_gather_into_tensor(gath[layer].view(-1), out_local[layer].view(-1))
            want = gath[layer].permute(1, 0, 2).reshape(n_seqs, Q_HEADS * D)
            gather_check = max(gather_check, float((got_all[layer].float() - want.float()).abs().max().item()))
    # CPU oracle on this rank's heads of a few sequences of layer 0
    from oracle import oracle as orc
    worst_rel, worst_abs = 0.0, 0.0
    for i in (0, n_seqs // 2, n_seqs - 1):
        s, L = ids[i], seqs[ids[i]]
        kk = torch.zeros(kvh, L, D, dtype=torch.bfloat16, device=dev)
        vv = torch.zeros_like(kk)
        pool.gather_kv(0, s, kk, vv, L)
        torch.cuda.synchronize()
        O, _ = orc.attention(_u16(q_rot[0, i]).reshape(qh, 1, D), _u16(kk), _u16(vv), L, causal=False)
        got = orc.bf16_to_f32(_u16(out_local[0, i])).reshape(-1)
        worst_rel = max(worst_rel, row_rel_err(got, O[:, 0].reshape(-1)))
        worst_abs = max(worst_abs, float(np.max(np.abs(got - O[:, 0].reshape(-1)))))
    line = None
    if rank == 0:
        line = {
            "metric": "paged_decode_attn_hbm_gbs", "value": round(nbytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 4),
            "us_per_token": round(ms / steps * 1e3 / n_seqs, 2),
            "us_per_step_per_layer": round(ms / steps * 1e3 / LAYERS, 2),
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
                    "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": round(ms_e2e / steps, 4)},
            "gpu_launches": launches, "clocks": env.sampler.summary(m0, m1),
            "roofline": {"bound": "hbm", "kernel": "decode_kernel", "achieved": round(achieved, 1), "peak": peak,
                         "unit": "GB/s", "frac": round(achieved / peak, 4), "peak_source": f"of {peak_kind}",
                         "us_per_launch": round(ms_k * 1e3, 2), "bytes_per_launch": kern_bytes, "traffic": None},
            "checks": {"fused_gather_vs_allgather_max_abs_diff_all_layers": gather_check,
                       "oracle_layer0_max_abs_err": worst_abs, "oracle_layer0_max_row_rel_err": worst_rel,
                       "oracle_row_rel_bar": ROW_REL, "oracle_layer0_ok": bool(worst_rel <= ROW_REL)},
        }
    env.barrier()
    if hg is not None:
        hg.close()
    pool.close()
    return line


# =============================================================================
# Q/K/V projections of a decode step, output projection (weight streams)
# =============================================================================
def run_qkv(env: Env, args, sub: bool = False, which: str = "qkv"):
    """which == "qkv": Q/K/V projections of a decode step (the producer in front of the attention
    path): batch 1, hidden 2048 -> q 2048 + k 512 + v 512 columns, all layers of the step.
    which == "out": the output projection + residual behind it (2048 -> 2048).  A step reads every
    layer's weights once, so the metric is achieved HBM GB/s.  N>1: independent replicas."""
    torch = env.torch
    from llama_transformer_runtime_b200 import paged
    from oracle import oracle as orc

    rank, world, dev = env.rank, env.world, env.dev
    ref_arm = args.impl == "reference" and not sub
    if ref_arm and rank != 0:
        return None
    steps = max(5, args.steps // 2) if sub else args.steps
    warmup = 3 if sub else args.warmup
    H, NQ, NKV, rows = HIDDEN, 2048, 512, 1
    gen = torch.Generator(device=dev)
    gen.manual_seed(99 + rank)
    # rotating weight sets so that no step finds its weights in L2 (126 MB)
    SETS = 2 if ref_arm else (4 if sub else 8)
    x_host = torch.randn(LAYERS, rows, H, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    state = {"i": 0}
    ref = orc.ref() if orc.ref_available() else None
    if ref_arm and ref is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built"}
    if which == "qkv":
        wq = [(torch.randn(LAYERS, H, NQ, generator=gen, device=dev) * 0.03).to(torch.bfloat16) for _ in range(SETS)]
        wk = [(torch.randn(LAYERS, H, NKV, generator=gen, device=dev) * 0.03).to(torch.bfloat16) for _ in range(SETS)]
        wv = [(torch.randn(LAYERS, H, NKV, generator=gen, device=dev) * 0.03).to(torch.bfloat16) for _ in range(SETS)]
        q = torch.zeros(LAYERS, rows, NQ, dtype=torch.bfloat16, device=dev)
        k = torch.zeros(LAYERS, rows, NKV, dtype=torch.bfloat16, device=dev)
        v = torch.zeros(LAYERS, rows, NKV, dtype=torch.bfloat16, device=dev)
        out_host = torch.zeros(LAYERS, rows, NQ + 2 * NKV, dtype=torch.bfloat16).pin_memory()
        bytes_layer = (H * (NQ + 2 * NKV) + rows * H + rows * (NQ + 2 * NKV)) * 2
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        if args.qkv_packed:
            pq = [paged.pack_projection_weights(w) for w in wq]
            pk = [paged.pack_projection_weights(w) for w in wk]
            pv = [paged.pack_projection_weights(w) for w in wv]
            torch.cuda.synchronize()

        def ours_step(s):
            if not args.qkv_packed:
                paged.qkv_project(x_dev, wq[s], wk[s], wv[s], q, k, v, rows, LAYERS)
            else:
                paged.qkv_project_packed(x_dev, pq[s], pk[s], pv[s], q, k, v, rows, status, LAYERS)

        def ref_step(s):
            # as Attention::forward drives it (src/runtime/attention.cu:138-191): three GEMM launches
            # per layer, a device synchronisation after each
            for l in range(LAYERS):
                for w, o, n in ((wq[s], q, NQ), (wk[s], k, NKV), (wv[s], v, NKV)):
                    ref.ref_gemm(x_dev[l].data_ptr(), w[l].data_ptr(), o[l].data_ptr(), rows, n, H)
                    torch.cuda.synchronize()

        def copy_out():
            out_host[:, :, :NQ].copy_(q, non_blocking=True)
            out_host[:, :, NQ:NQ + NKV].copy_(k, non_blocking=True)
            out_host[:, :, NQ + NKV:].copy_(v, non_blocking=True)
        ref_launches, kernel = 3 * LAYERS, ("qkv_project_kernel" if not args.qkv_packed else "qkv_project_packed_kernel")
        metric, wname = "qkv_project_hbm_gbs", f"qkv_projection_decode_batch1_x{LAYERS}layers"
    else:
        wo = [(torch.randn(LAYERS, H, H, generator=gen, device=dev) * 0.03).to(torch.bfloat16) for _ in range(SETS)]
        res = (torch.randn(LAYERS, rows, H, generator=gen, device=dev)).to(torch.bfloat16)
        o = torch.zeros(LAYERS, rows, H, dtype=torch.bfloat16, device=dev)
        lin = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)
        out_host = torch.zeros(LAYERS, rows, H, dtype=torch.bfloat16).pin_memory()
        bytes_layer = (H * H + 3 * rows * H) * 2

        def ours_step(s):
            paged.out_project(x_dev, wo[s], res, o, rows, LAYERS)

        def ref_step(s):
            # o_proj GEMM + synchronisation (src/runtime/attention.cu:367-375), then the residual add
            # of TransformerBlock::forward (src/runtime/transformer_block.cu:76-81)
            for l in range(LAYERS):
                ref.ref_gemm(x_dev[l].data_ptr(), wo[s][l].data_ptr(), lin.data_ptr(), rows, H, H)
                torch.cuda.synchronize()
                ref.ref_residual_add(res[l].data_ptr(), lin.data_ptr(), o[l].data_ptr(), rows * H)
                torch.cuda.synchronize()

        def copy_out():
            out_host.copy_(o, non_blocking=True)
        ref_launches, kernel = 2 * LAYERS, "qkv_project_kernel (output projection + residual epilogue)"
        metric, wname = "out_project_hbm_gbs", f"out_projection_residual_decode_batch1_x{LAYERS}layers"

    def make_step(fn):
        def step():
            s = state["i"] % SETS
            state["i"] += 1
            fn(s)
        return step

    def make_e2e(step):
        def e2e_step():
            x_dev.copy_(x_host, non_blocking=True)
            step()
            copy_out()
            torch.cuda.current_stream().synchronize()
        return e2e_step

    grouped = env.dist is not None and not ref_arm and not sub

    def timed(fn, n):
        return env.timed(fn, n) if grouped else local_timed(torch, fn, n)

    m0 = env.sampler.mark()
    step = make_step(ref_step if ref_arm else ours_step)
    for _ in range(warmup):
        step()
    ms = timed(step, steps)
    ms_e2e = timed(make_e2e(step), steps)
    m1 = env.sampler.mark()
    n_rep = world if grouped else 1
    value = n_rep * LAYERS * bytes_layer * steps / (ms * 1e-3) / 1e9
    e2e_value = n_rep * LAYERS * bytes_layer * steps / (ms_e2e * 1e-3) / 1e9
    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    line = {
        "metric": metric, "value": round(value, 1), "unit": "GB/s", "n_gpus": n_rep,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 4),
        "us_per_layer": round(ms / steps * 1e3 / LAYERS, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wname, "hidden": H, "q_cols": NQ, "kv_cols": NKV, "rows": rows, "layers": LAYERS,
                   "parallelism": "1 GPU" if n_rep == 1 else f"{world} independent replicas",
                   "l2": f"{SETS} weight sets in rotation ({SETS * LAYERS * bytes_layer / 1e9:.2f} GB), larger than L2"},
        "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": round(ms_e2e / steps, 4)},
        "gpu_launches": (ref_launches if ref_arm else 1) * steps, "clocks": env.sampler.summary(m0, m1),
    }
    if ref_arm:
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "GB/s", "cores": os.cpu_count(), "kind": "reference",
                                "sample": "the reference has no CPU implementation of its GEMMs: its own CUDA "
                                          "kernels run on the GPU, driven as Attention::forward drives them"}
        line["e2e"].update({"h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "value": line["value"]})
        return line
    line["roofline"] = {"bound": "hbm", "kernel": kernel, "achieved": round(value / n_rep, 1),
                        "peak": peak, "unit": "GB/s", "frac": round(value / n_rep / peak, 4),
                        "peak_source": f"of {peak_kind}", "us_per_launch": round(ms / steps * 1e3, 2),
                        "bytes_per_launch": LAYERS * bytes_layer, "traffic": None}
    # check + CPU baseline: the oracle's GEMM restatement (double accumulation, OpenMP) on layer 0 with set 0
    ours_step(0)
    torch.cuda.synchronize()
    if which == "qkv" and args.qkv_packed:
        assert int(status.item()) == 0
    xs = _u16(x_host[0])
    t0 = time.perf_counter()
    reps = 0
    budget = 2.0 if sub else 10.0
    while True:
        if which == "qkv":
            outs = [orc.gemm_bf16(xs, _u16(w[0][0])) for w in (wq, wk, wv)]
        else:
            outs = [orc.gemm_bf16(xs, _u16(wo[0][0]))]
        reps += 1
        if time.perf_counter() - t0 >= budget:
            break
    dt = (time.perf_counter() - t0) / reps
    if which == "qkv":
        got = np.concatenate([_u16(q[0]), _u16(k[0]), _u16(v[0])], axis=1)
        want = np.concatenate(outs, axis=1)
    else:
        got = _u16(o[0])
        want = orc.f32_to_bf16(orc.bf16_to_f32(_u16(res[0])) + orc.bf16_to_f32(outs[0]))
    err = float(np.abs(orc.bf16_to_f32(got) - orc.bf16_to_f32(want)).max())
    line["cpu_baseline"] = {"value": round(bytes_layer / dt / 1e9, 2), "unit": "GB/s",
                            "cores": orc.num_threads(), "kind": "port",
                            "sample": f"layer 0 of the workload, {reps} repetitions in {dt * reps:.1f} s",
                            "gpu_vs_cpu_max_abs_err": err}
    if sub and ref is not None:
        rstep = make_step(ref_step)
        rstep()
        rn = 2
        rms = local_timed(torch, rstep, rn)
        line["reference"] = {"value": round(LAYERS * bytes_layer * rn / (rms * 1e-3) / 1e9, 2), "unit": "GB/s",
                             "us_per_layer": round(rms / rn * 1e3 / LAYERS, 2),
                             "how": "the reference's GEMM kernels with its device synchronisation after each, same weights"}
    return line


def run_qkv_prefill(env: Env, args, sub: bool = False):
    """Q/K/V projections of a 2048-token prompt, 16 layers: x [2048, 2048] times Wq, Wk, Wv, RoPE on Q
    and K, K/V appended to the paged cache.  Ours: one tcgen05 GEMM launch per layer with RoPE and the
    append as its epilogue.  Reference arm: its 3 GEMM launches (a device synchronisation after each,
    as Attention::forward does), its RoPE/transpose kernels and the strided form of its append copies."""
    torch = env.torch
    if env.rank != 0:
        return None  # independent replicas only
    from oracle import oracle as orc
    dev = env.dev
    S, H, NQ, NKV = PREFILL_TOKENS, HIDDEN, Q_HEADS * D, KV_HEADS * D
    steps = max(3, args.steps // 5) if sub else args.steps
    warmup = 3 if sub else args.warmup
    ref_arm = args.impl == "reference" and not sub
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
    ref = orc.ref() if orc.ref_available() else None
    if ref_arm and ref is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built"}
    cos_h, sin_h = orc.build_rope_tables(S)
    cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)

    if ref is not None:
        ql = torch.empty(S, NQ, dtype=torch.bfloat16, device=dev)
        kl = torch.empty(S, NKV, dtype=torch.bfloat16, device=dev)
        vl = torch.empty(S, NKV, dtype=torch.bfloat16, device=dev)
        qf = torch.empty(Q_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        kf = torch.empty(KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vf = torch.empty_like(kf)
        kc = torch.zeros(LAYERS, KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)

    def ref_step():
        for l in range(LAYERS):
            for w, o, n in ((wq, ql, NQ), (wk, kl, NKV), (wv, vl, NKV)):
                ref.ref_gemm(x[l].data_ptr(), w[l].data_ptr(), o.data_ptr(), S, n, H)
                torch.cuda.synchronize()
            ref.ref_rope_qkv(ql.data_ptr(), qf.data_ptr(), kl.data_ptr(), kf.data_ptr(), vl.data_ptr(),
                             vf.data_ptr(), cos.data_ptr(), sin.data_ptr(), S, 0)
            ref.ref_append_strided(kc[l].data_ptr(), vc[l].data_ptr(), kf.data_ptr(), vf.data_ptr(), S, 0, S, None)

    pool = None
    if not ref_arm:
        from llama_transformer_runtime_b200 import paged
        nb = (S + BLOCK - 1) // BLOCK
        num_blocks = nb + nb // 4 + 8
        pool = paged.KVPool(LAYERS, num_blocks, KV_HEADS, 1, nb + 1, device=env.local_rank)
        pool.set_free_order(np.random.default_rng(5).permutation(num_blocks))
        seq = pool.create_seq()
        pool.reserve(seq, S)
        pool.batch_set([seq], [S])
        # weights are repacked once, at load time, into the tile image the GEMM bulk-copies
        pq, pk, pv = (paged.pack_projection_weights(w) for w in (wq, wk, wv))
        torch.cuda.synchronize()

    def ours_step():
        # the same prompt positions are rewritten every step (the table is fixed)
        for l in range(LAYERS):
            pool.qkv_project_append(l, x[l], pq[l], pk[l], pv[l], cos, sin, q_rot[l], H)

    step = ref_step if ref_arm else ours_step
    launches_per_step = LAYERS * 8 if ref_arm else LAYERS * 2

    def e2e_step():
        x.copy_(x_host, non_blocking=True)
        step()
        if not ref_arm:
            q_host.copy_(q_rot[LAYERS - 1], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    m0 = env.sampler.mark()
    for _ in range(warmup):
        step()
    ms = local_timed(torch, step, steps) / steps
    ms_e2e = local_timed(torch, e2e_step, steps) / steps
    m1 = env.sampler.mark()
    value = flops_layer * LAYERS / (ms * 1e-3) / 1e12
    line = {
        "metric": "qkv_project_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "us_per_layer": round(ms * 1e3 / LAYERS, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"qkv_projection_rope_append_{S}tokens_x{LAYERS}layers", "tokens": S, "hidden": H,
                   "q_cols": NQ, "kv_cols": NKV, "layers": LAYERS, "flops": "2*tokens*hidden*(q_cols+2*kv_cols) per layer",
                   "l2": "per-layer inputs and weights are distinct tensors (20.6 MB per layer, 330 MB per step)"},
        "e2e": {"value": round(flops_layer * LAYERS / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": 0 if ref_arm else q_host.numel() * 2,
                "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": launches_per_step * steps, "clocks": env.sampler.summary(m0, m1),
    }
    if ref_arm:
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                "sample": "whole workload on the GPU: the reference has no CPU implementation of its GEMMs"}
        line["e2e"].update({"h2d_bytes_per_step": 0, "value": line["value"]})
        return line
    line["roofline"] = {"bound": "tensor", "kernel": "qkv_gemm_kernel", "achieved": round(value, 2), "peak": burst,
                        "unit": "TFLOP/s", "frac": round(value / burst, 4),
                        "peak_source": f"of {kind} (cuBLAS bf16 burst)", "us_per_launch": round(ms * 1e3 / LAYERS, 2),
                        "flops_per_launch": flops_layer, "traffic": None}
    pool.check()
    # CPU baseline and check: the oracle's GEMM on the first 64 rows of layer 0, q columns
    rows = 64
    xs = _u16(x_host[0, :rows])
    ws = _u16(wq[0])
    t0 = time.perf_counter()
    lin = orc.gemm_bf16(xs, ws)
    dt = time.perf_counter() - t0
    want = orc.rope(lin.reshape(rows, Q_HEADS, D), cos_h, sin_h, 0, 1, out_token_major=True).reshape(rows, NQ)
    got = _u16(q_rot[0, :rows])
    err = float(np.abs(orc.bf16_to_f32(got) - orc.bf16_to_f32(want)).max())
    line["cpu_baseline"] = {"value": round(2.0 * rows * H * NQ / dt / 1e12, 5), "unit": "TFLOP/s",
                            "cores": orc.num_threads(), "kind": "port",
                            "sample": f"{rows} rows x {NQ} columns of layer 0 (double accumulation), {dt:.2f} s",
                            "gpu_vs_cpu_max_abs_err": err}
    if sub and ref is not None:
        ref_step()
        rms = local_timed(torch, ref_step, 1)
        line["reference"] = {"value": round(flops_layer * LAYERS / (rms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                             "us_per_layer": round(rms * 1e3 / LAYERS, 2),
                             "how": "the reference's 3 GEMM launches + synchronisations, RoPE kernels and strided append copies"}
    pool.close()
    return line


# =============================================================================
# prefill attention (2048 tokens x 16 layers, causal, batch 1) and the append kernel alone
# =============================================================================
def run_prefill(env: Env, args, sub: bool = False, append_only: bool = False):
    """One step = one 2048-token prompt through 16 layers: per layer fused RoPE + paged append of the
    prompt's K/V, then causal GQA attention over the cache, output [2048, 2048] bf16.  Both arms: ours
    (pa_append + pa_prefill) and the reference's kernels (rope kernels + append copies + flash kernel
    + layout).  append_only: only the RoPE + append part, an HBM stream of
    tokens x (4096 + 2 x 1024 read, 4096 + 2 x 1024 written) bytes per layer."""
    torch = env.torch
    if env.rank != 0:
        return None  # independent replicas only: prefill is not sharded here
    from oracle import oracle as orc
    dev = env.dev
    S = PREFILL_TOKENS
    steps = max(3, args.steps // 5) if sub else args.steps
    warmup = 3 if sub else args.warmup
    ref_arm = args.impl == "reference" and not sub
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
    ref = orc.ref() if orc.ref_available() else None
    if ref_arm and ref is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built"}
    cos_h, sin_h = orc.build_rope_tables(S)
    cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)

    if ref is not None:
        kc = torch.zeros(LAYERS, KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        qf = torch.empty(Q_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        kf = torch.empty(KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vf = torch.empty_like(kf)
        of = torch.empty(Q_HEADS, S, D, dtype=torch.bfloat16, device=dev)

    def ref_step():
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
            if append_only:
                continue
            ref.ref_flash_attention(qf.data_ptr(), kc[layer].data_ptr(), vc[layer].data_ptr(), of.data_ptr(),
                                    None, 1, Q_HEADS, KV_HEADS, S, S, S, 0.125, 1, None)
            ref.ref_flash_output_layout(of.data_ptr(), out[layer].data_ptr(), S)

    pool = None
    if not ref_arm:
        from llama_transformer_runtime_b200 import paged
        nb = (S + BLOCK - 1) // BLOCK
        num_blocks = nb + nb // 4 + 8
        pool = paged.KVPool(LAYERS, num_blocks, KV_HEADS, 1, nb + 1, device=env.local_rank)
        pool.set_free_order(np.random.default_rng(5).permutation(num_blocks))
        seq = pool.create_seq()
        pool.reserve(seq, S)
        pool.batch_set([seq], [S])
        q_rot = torch.empty_like(q_in)

    def ours_step():
        # the same prompt positions are rewritten every step (the table is fixed)
        for layer in range(LAYERS):
            pool.append(layer, q_in[layer], k_in[layer], v_in[layer], cos, sin, q_rot[layer])
            if not append_only:
                pool.prefill(layer, q_rot[layer], out[layer], None, 0.125)

    step = ref_step if ref_arm else ours_step
    if append_only:
        launches_per_step = LAYERS * 19 if ref_arm else LAYERS
    else:
        launches_per_step = LAYERS * 5 if ref_arm else LAYERS * 2

    def e2e_step():
        q_in.copy_(q_host, non_blocking=True)
        k_in.copy_(k_host, non_blocking=True)
        v_in.copy_(v_host, non_blocking=True)
        step()
        if append_only:
            if not ref_arm:
                out_host.copy_(q_rot[LAYERS - 1].view(S, Q_HEADS * D), non_blocking=True)
        else:
            out_host.copy_(out[LAYERS - 1], non_blocking=True)  # the last layer's attention output
        torch.cuda.current_stream().synchronize()

    m0 = env.sampler.mark()
    for _ in range(warmup):
        step()
    ms = local_timed(torch, step, steps) / steps
    ms_e2e = local_timed(torch, e2e_step, steps) / steps
    m1 = env.sampler.mark()
    append_bytes = S * ((Q_HEADS + 2 * KV_HEADS) * D * 2) * 2  # read q, k, v rows; write rotated q and the cache tiles
    if append_only:
        work, unit, metric = append_bytes * LAYERS / 1e9, "GB/s", "rope_append_hbm_gbs"
        wname = f"rope_append_{S}tokens_x{LAYERS}layers_batch1"
    else:
        work, unit, metric = prefill_flops(S) * LAYERS / 1e12, "TFLOP/s", "prefill_attn_tflops"
        wname = f"prefill_{S}tokens_x{LAYERS}layers_batch1_causal"
    value = work / (ms * 1e-3)
    line = {
        "metric": metric, "value": round(value, 2), "unit": unit, "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "us_per_layer": round(ms * 1e3 / LAYERS, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wname, "tokens": S, "layers": LAYERS,
                   "q_heads": Q_HEADS, "kv_heads": KV_HEADS, "head_dim": D,
                   "l2": "per-layer inputs are distinct tensors (24 MiB per layer, 384 MiB per step)"},
        "e2e": {"value": round(work / (ms_e2e * 1e-3), 2), "unit": unit,
                "h2d_bytes_per_step": (q_host.numel() + k_host.numel() + v_host.numel()) * 2,
                "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": launches_per_step * steps, "clocks": env.sampler.summary(m0, m1),
    }
    if append_only:
        line["config"]["bytes"] = "tokens x (4096 + 2 x 1024) read + the same written, per layer"
    else:
        line["config"]["flops"] = "causal-useful 4*Hq*D*S(S+1)/2 per layer"
        line["config"]["dense_count_tflops"] = round(4.0 * Q_HEADS * D * S * S * LAYERS / (ms * 1e-3) / 1e12, 2)
    if ref_arm:
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": unit, "cores": 0, "kind": "reference",
                                "sample": "whole workload on the GPU: the reference has no CPU implementation of this path"}
        return line
    # dominant kernel alone
    if append_only:
        def kern_only():
            for layer in range(LAYERS):
                pool.append(layer, q_in[layer], k_in[layer], v_in[layer], cos, sin, q_rot[layer])
        kern_only()
        reps = max(3, steps)
        ms_k = local_timed(torch, kern_only, reps) / (reps * LAYERS)
        peak, pk = measured_peak()
        achieved = append_bytes / (ms_k * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "kernel": "append_kernel", "achieved": round(achieved, 1), "peak": peak,
                            "unit": "GB/s", "frac": round(achieved / peak, 4), "peak_source": f"of {pk}",
                            "us_per_launch": round(ms_k * 1e3, 2), "bytes_per_launch": append_bytes,
                            "traffic": NCU_APPEND_TRAFFIC,
                            "traffic_note": "ncu capture of one 2048-token append_kernel launch (profiles/): DRAM reads; the rows it "
                                            "writes are still in L2 when the kernel ends"}
        # check: rotated Q rows of layer 0 against the oracle, bit for bit (first 64 tokens); the CPU
        # baseline is the oracle's RoPE + placement of those tokens
        t0 = time.perf_counter()
        want = orc.rope(_u16(q_in[0, :64]), cos_h, sin_h, 0, 1, out_token_major=True)
        orc.rope(_u16(k_in[0, :64]), cos_h, sin_h, 0, 1)
        dt = time.perf_counter() - t0
        line["checks"] = {"rotated_q_bit_exact_vs_oracle": bool(np.array_equal(_u16(q_rot[0, :64]), want))}
        line["cpu_baseline"] = {"value": round(64 * ((Q_HEADS + KV_HEADS) * D * 2) * 2 / dt / 1e9, 4), "unit": "GB/s",
                                "cores": 1, "kind": "port", "sample": "RoPE of 64 tokens' Q and K rows of layer 0 (scalar C loop)"}
    else:
        def attn_only():
            for layer in range(LAYERS):
                pool.prefill(layer, q_rot[layer], out[layer], None, 0.125)
        attn_only()
        reps = max(3, steps)
        ms_k = local_timed(torch, attn_only, reps) / (reps * LAYERS)
        achieved = prefill_flops(S) / (ms_k * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor", "kernel": "prefill_kernel", "achieved": round(achieved, 2),
                            "peak": burst, "unit": "TFLOP/s", "frac": round(achieved / burst, 4),
                            "peak_source": f"of {kind} (cuBLAS bf16 burst)", "us_per_launch": round(ms_k * 1e3, 2),
                            "flops_per_launch": prefill_flops(S), "traffic": None}
        line["cpu_baseline"] = prefill_cpu_baseline(q_rot, out, pool, seq, S, budget_s=(2.0 if sub else 10.0))
    pool.check()
    if sub and ref is not None:
        ref_step()
        rms = local_timed(torch, ref_step, 2) / 2
        line["reference"] = {"value": round(work / (rms * 1e-3), 2), "unit": unit,
                             "us_per_layer": round(rms * 1e3 / LAYERS, 2),
                             "how": "the reference's RoPE kernels + strided append copies" +
                                    ("" if append_only else " + attention kernel + layout kernel")}
    pool.close()
    return line


def prefill_cpu_baseline(q_rot, out, pool, seq, S, budget_s=10.0):
    """fp32 CPU oracle on a bounded sample: the first 512 query rows of layer 0
    (all 32 heads) against their causal keys; also checks the GPU output."""
    import torch

    from oracle import oracle as orc

    n = 512
    k = torch.zeros(KV_HEADS, S, D, dtype=torch.bfloat16, device=q_rot.device)
    v = torch.zeros_like(k)
    pool.gather_kv(0, seq, k, v, S)
    torch.cuda.synchronize()
    qh = _u16(q_rot[0][:n].permute(1, 0, 2))  # [32, n, 64]
    kh, vh = _u16(k[:, :n]), _u16(v[:, :n])
    t0 = time.perf_counter()
    O, _ = orc.attention(qh, kh, vh, n, causal=True)
    reps = 1
    while time.perf_counter() - t0 < budget_s and reps < 200:
        orc.attention(qh, kh, vh, n, causal=True)
        reps += 1
    total = time.perf_counter() - t0
    got = orc.bf16_to_f32(_u16(out[0][:n]))
    want = orc.output_layout(O)
    err = float(np.max(np.abs(got - want)))
    return {"value": round(prefill_flops(n) * reps / total / 1e12, 4), "unit": "TFLOP/s", "cores": orc.num_threads(),
            "kind": "port", "sample": f"first {n} query rows of layer 0, {reps} passes of the fp32 CPU oracle",
            "gpu_vs_cpu_max_abs_err": err, "gpu_vs_cpu_max_row_rel_err": row_rel_err(got, want)}



# =============================================================================
# the decode step with its true data flow: projections -> attention -> output projection per layer
# =============================================================================
def run_chain(env: Env, args, sub: bool = False, ffn: bool = False, token: bool = False):
    """token=True (workload token): a whole decode step of the model, the body of the reference's
    LlamaRuntime::decode_forward — token id -> embedding row -> 16 blocks -> final RMSNorm + language-model
    head (vocabulary 128256) -> greedy token, the id staying on the device from one step to the next
    (pa_decode_token); one GPU.
    ffn=True (workload block_chain): whole transformer blocks — the attention block below followed by
    the feed-forward block (RMSNorm, gate and up projections 2048 -> 8192, SiLU(gate) * up, down
    projection, residual): two more launches and 100.7 MB more weights per layer.
    ffn=False (workload decode_chain): one token through 16 attention blocks, each layer fed by the one before it (no FFN in between:
    x_{l+1} = x_l + attention(RMSNorm(x_l)) W_o): per layer RMSNorm + Q/K/V projections (one launch),
    RoPE + append + paged decode attention (one launch), output projection + residual (one launch),
    chained by programmatic dependent launch.  Context 4096 by default (--chain-ctx).  Per layer the
    step reads the projection weights (21 MB) and the layer's cache once: the metric is HBM GB/s over
    those bytes.  With N GPUs the cache is split by token range (weights replicated, every rank
    projects the same rows), partials exchanged and merged in the decode kernel.
    Reference arm: the reference's own kernels in the order of Attention::forward +
    TransformerBlock's residual add, with its device synchronisations."""
    torch, dist = env.torch, env.dist
    from oracle import oracle as orc
    rank, local_rank, world, dev = env.rank, env.local_rank, env.world, env.dev
    if token:
        ffn = True
        if rank != 0:
            return None  # independent replicas only
        world = 1
    ctx = args.chain_ctx
    steps = max(5, args.steps // 2) if sub else args.steps
    warmup = 3 if sub else args.warmup
    ref_arm = args.impl == "reference" and not sub
    if ref_arm and rank != 0:
        return None
    H, NQ, NKV = HIDDEN, Q_HEADS * D, KV_HEADS * D
    gen = torch.Generator(device=dev)
    gen.manual_seed(31)  # the same weights on every rank
    SETS = 2 if (sub or ref_arm) else 4  # weight sets in rotation: 2 x 16 x 21 MB is already larger than L2
    mk = lambda *shape, s=0.03: (torch.randn(*shape, generator=gen, device=dev) * s).to(torch.bfloat16)
    Ws = [dict(nw=mk(LAYERS, H, s=0.7), wq=mk(LAYERS, H, NQ), wk=mk(LAYERS, H, NKV), wv=mk(LAYERS, H, NKV),
               wo=mk(LAYERS, NQ, H)) for _ in range(SETS)]
    INTER = 8192
    if ffn:
        for w in Ws:
            w.update(fn=mk(LAYERS, H, s=0.7), wg=mk(LAYERS, H, INTER), wu=mk(LAYERS, H, INTER), wd=mk(LAYERS, INTER, H, s=0.02))
    x_host = torch.randn(1, H, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).pin_memory()
    y_host = torch.zeros(1, H, dtype=torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    y_dev = torch.zeros(1, H, dtype=torch.bfloat16, device=dev)
    weight_bytes = (H * (NQ + 2 * NKV) + NQ * H + H) * 2 + ((3 * H * INTER + H) * 2 if ffn else 0)
    VOC = 128256
    # per token outside the layers: the embedding row read and written, head weight + norm weight read,
    # logits written, logits read by the argmax
    head_bytes = (2 * H * 2 + (H * VOC + H + VOC) * 2 + VOC * 2) if token else 0
    if token:
        embed = mk(VOC, H, s=1.0)
        w_lm = mk(H, VOC)
        final_norm = mk(H, s=0.7)
        tok_host = torch.tensor([1234], dtype=torch.int32).pin_memory()
        tok_dev = tok_host.to(dev)
        logits_dev = torch.zeros(1, VOC, dtype=torch.bfloat16, device=dev)
    total_steps = warmup + 2 * steps + 12
    state = {"len": ctx, "i": 0}
    ref = orc.ref() if orc.ref_available() else None
    if ref_arm and ref is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built"}
    cos_h, sin_h = orc.build_rope_tables(ctx + total_steps + 2)
    cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
    kvgen = torch.Generator(device=dev)
    kvgen.manual_seed(4321 + rank)

    pool = xchg = None
    lo = 0
    if not ref_arm:
        from llama_transformer_runtime_b200 import paged
        lo, hi = token_ranges(ctx, world)[rank]
        local_len = hi - lo
        owner = world - 1
        need_blocks = (local_len + (total_steps if rank == owner else 0) + BLOCK - 1) // BLOCK
        num_blocks = need_blocks + need_blocks // 4 + 8
        pool = paged.KVPool(LAYERS, num_blocks, KV_HEADS, 1, need_blocks + 1, device=local_rank)
        pool.set_free_order(np.random.default_rng(1234 + rank).permutation(num_blocks))
        if getattr(args, "decode_cluster", 0):
            pool.set_decode_cluster(args.decode_cluster)
        seq = pool.create_seq()
        ones = torch.ones(local_len + 1, 32, dtype=torch.float32, device=dev)
        zeros = torch.zeros(local_len + 1, 32, dtype=torch.float32, device=dev)
        for c0 in range(0, local_len, 8192):
            n = min(8192, local_len - c0)
            pool.reserve(seq, c0 + n)
            pool.batch_set([seq], [n])
            for layer in range(LAYERS):
                k = (torch.randn(n, KV_HEADS, D, generator=kvgen, device=dev) * 0.5).to(torch.bfloat16)
                v = (torch.randn(n, KV_HEADS, D, generator=kvgen, device=dev) * 0.5).to(torch.bfloat16)
                pool.append(layer, None, k, v, ones, zeros, None)
        torch.cuda.synchronize()
        del ones, zeros
        descs = [paged.attention_weights(w["nw"], w["wq"], w["wk"], w["wv"], w["wo"]) for w in Ws]
        fdescs = [paged.ffn_weights(w["fn"], w["wg"], w["wu"], w["wd"]) for w in Ws] if ffn else None
        models = [paged.model_weights(embed, descs[i], fdescs[i], final_norm, w_lm) for i in range(SETS)] if token else None

        def run_layers(s, l0, l1, xin, xout):
            if ffn:
                paged.block_step(pool, descs[s], fdescs[s], l0, l1, xin, xout, cos, sin, xchg=xchg)
            else:
                paged.attention_step(pool, descs[s], l0, l1, xin, xout, cos, sin, add_residual=True, xchg=xchg)
        if world > 1:
            xchg = paged.Exchange(local_rank, rank, world, 1, KV_HEADS)
            handles = [None] * world
            dist.all_gather_object(handles, xchg.handle())
            xchg.connect(handles)
            dist.barrier()

        def ours_step():
            state["len"] += 1
            s = state["i"] % SETS
            state["i"] += 1
            if rank == owner:
                pool.reserve(seq, pool.length(seq) + 1)
            if world == 1:
                pool.batch_set([seq])
            else:
                pool.batch_set_sharded([seq], [1 if rank == owner else 0], [1], [state["len"] - 1], [lo])
            if token:
                paged.decode_token(pool, models[s], tok_dev, tok_dev, logits_dev, cos, sin, chained=True)
            else:
                run_layers(s, 0, LAYERS, x_dev, y_dev)

    if ref is not None and (ref_arm or sub) and rank == 0:
        max_seq = ctx + total_steps + 2
        kc = torch.zeros(LAYERS, KV_HEADS, max_seq, D, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        for layer in range(LAYERS):
            kc[layer, :, :ctx] = (torch.randn(KV_HEADS, ctx, D, generator=kvgen, device=dev) * 0.5).to(torch.bfloat16)
            vc[layer, :, :ctx] = (torch.randn(KV_HEADS, ctx, D, generator=kvgen, device=dev) * 0.5).to(torch.bfloat16)
        bufs = {n: torch.zeros(1, c, dtype=torch.bfloat16, device=dev) for n, c in
                (("xn", H), ("q", NQ), ("k", NKV), ("v", NKV), ("arow", NQ), ("lin", H), ("xa", H), ("xb", H), ("xm", H),
                 ("g", INTER), ("u", INTER), ("h", INTER), ("emb", H))}
        qf = torch.empty(Q_HEADS, 1, D, dtype=torch.bfloat16, device=dev)
        kf = torch.empty(KV_HEADS, 1, D, dtype=torch.bfloat16, device=dev)
        vf = torch.empty(KV_HEADS, 1, D, dtype=torch.bfloat16, device=dev)
        of = torch.empty(Q_HEADS, 1, D, dtype=torch.bfloat16, device=dev)
        rstate = {"len": ctx, "i": 0}

        def ref_step():
            pos = rstate["len"]
            rstate["len"] += 1
            w = Ws[rstate["i"] % SETS]
            rstate["i"] += 1
            cur = x_dev
            if token:  # decode_forward: blocking copy of the id, embedding kernel, synchronisation
                tok_dev.copy_(tok_host)
                ref.ref_embedding(tok_dev.data_ptr(), embed.data_ptr(), bufs["emb"].data_ptr(), 1)
                torch.cuda.synchronize()
                cur = bufs["emb"]
            for l in range(LAYERS):
                ref.ref_rmsnorm(cur.data_ptr(), w["nw"][l].data_ptr(), bufs["xn"].data_ptr(), 1, 1e-5)
                torch.cuda.synchronize()
                for wm, o, n in ((w["wq"], bufs["q"], NQ), (w["wk"], bufs["k"], NKV), (w["wv"], bufs["v"], NKV)):
                    ref.ref_gemm(bufs["xn"].data_ptr(), wm[l].data_ptr(), o.data_ptr(), 1, n, H)
                    torch.cuda.synchronize()
                ref.ref_rope_qkv(bufs["q"].data_ptr(), qf.data_ptr(), bufs["k"].data_ptr(), kf.data_ptr(),
                                 bufs["v"].data_ptr(), vf.data_ptr(), cos.data_ptr(), sin.data_ptr(), 1, pos)
                ref.ref_append_memcpy_loop(kc[l].data_ptr(), vc[l].data_ptr(), kf.data_ptr(), vf.data_ptr(), max_seq, pos, 1)
                ref.ref_flash_attention(qf.data_ptr(), kc[l].data_ptr(), vc[l].data_ptr(), of.data_ptr(), None, 1,
                                        Q_HEADS, KV_HEADS, 1, pos + 1, max_seq, 0.125, 1, None)
                torch.cuda.synchronize()
                ref.ref_flash_output_layout(of.data_ptr(), bufs["arow"].data_ptr(), 1)
                torch.cuda.synchronize()
                ref.ref_gemm(bufs["arow"].data_ptr(), w["wo"][l].data_ptr(), bufs["lin"].data_ptr(), 1, H, NQ)
                torch.cuda.synchronize()
                nxt = bufs["xa"] if l % 2 == 0 else bufs["xb"]
                if not ffn:
                    ref.ref_residual_add(cur.data_ptr(), bufs["lin"].data_ptr(), nxt.data_ptr(), H)
                    torch.cuda.synchronize()
                    cur = nxt
                    continue
                # FeedForward::forward (one synchronisation, at its end) and the block's second residual add
                ref.ref_residual_add(cur.data_ptr(), bufs["lin"].data_ptr(), bufs["xm"].data_ptr(), H)
                torch.cuda.synchronize()
                ref.ref_rmsnorm(bufs["xm"].data_ptr(), w["fn"][l].data_ptr(), bufs["xn"].data_ptr(), 1, 1e-5)
                ref.ref_gemm(bufs["xn"].data_ptr(), w["wg"][l].data_ptr(), bufs["g"].data_ptr(), 1, INTER, H)
                ref.ref_gemm(bufs["xn"].data_ptr(), w["wu"][l].data_ptr(), bufs["u"].data_ptr(), 1, INTER, H)
                ref.ref_silu_mul(bufs["g"].data_ptr(), bufs["u"].data_ptr(), bufs["h"].data_ptr(), 1)
                ref.ref_gemm(bufs["h"].data_ptr(), w["wd"][l].data_ptr(), bufs["lin"].data_ptr(), 1, H, INTER)
                torch.cuda.synchronize()
                ref.ref_residual_add(bufs["xm"].data_ptr(), bufs["lin"].data_ptr(), nxt.data_ptr(), H)
                torch.cuda.synchronize()
                cur = nxt
            if not token:
                y_dev.copy_(cur)
                return
            torch.cuda.synchronize()  # after transformer_->forward
            ref.ref_rmsnorm(cur.data_ptr(), final_norm.data_ptr(), bufs["xn"].data_ptr(), 1, 1e-5)
            torch.cuda.synchronize()
            ref.ref_gemm(bufs["xn"].data_ptr(), w_lm.data_ptr(), logits_dev.data_ptr(), 1, VOC, H)
            torch.cuda.synchronize()
            t = torch.empty(1, dtype=torch.int32, device=dev)  # the loop's per-token cudaMalloc / cudaFree
            ref.ref_argmax(logits_dev.data_ptr(), t.data_ptr())
            tok_host.copy_(t)  # blocking copy
            del t
            torch.cuda.synchronize()

    step = ref_step if ref_arm else ours_step

    def e2e_step():
        if token:  # a generation loop that reads every token on the host (the reference's own arm does already)
            if ref_arm:
                return step()
            tok_dev.copy_(tok_host, non_blocking=True)
            step()
            tok_host.copy_(tok_dev, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return
        x_dev.copy_(x_host, non_blocking=True)
        step()
        y_host.copy_(y_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def block(fn, n):
        st = rstate if ref_arm else state
        l0 = st["len"]
        ms = local_timed(torch, fn, n) if ref_arm else env.timed(fn, n)
        return ms, sum(LAYERS * (decode_bytes(L) + weight_bytes) + head_bytes for L in range(l0 + 1, st["len"] + 1))

    m0 = env.sampler.mark()
    for _ in range(warmup):
        step()
    ms, nbytes = block(step, steps)
    ms_e2e, nbytes_e2e = block(e2e_step, steps)
    m1 = env.sampler.mark()
    value = nbytes / (ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    line = None
    if rank == 0:
        line = {
            "metric": "decode_token_hbm_gbs" if token else "block_chain_hbm_gbs" if ffn else "decode_chain_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": 1 if ref_arm else world,
            "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 4),
            "us_per_token": round(ms / steps * 1e3, 2), "us_per_layer": round(ms / steps * 1e3 / LAYERS, 2),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"token_ctx{ctx}_x{LAYERS}layers_vocab{VOC}_batch1" if token else
                                   f"{'block' if ffn else 'decode'}_chain_ctx{ctx}_x{LAYERS}layers_batch1", "context": ctx, "layers": LAYERS,
                       "batch": 1, "hidden": H, "bytes": "per layer: Wq, Wk, Wv, Wo, norm weight" + (", Wgate, Wup, Wdown, FFN norm weight" if ffn else "") + " + the layer's cache (2048 L + ...)" +
                                (f"; per token: embedding row, final norm + head weight [{H}, {VOC}], logits written and read" if token else ""),
                       "parallelism": "1 GPU" if world == 1 or ref_arm else
                                      f"cache split by token range over {world} GPUs, weights replicated",
                       "l2": f"{SETS} weight sets in rotation ({SETS * LAYERS * weight_bytes / 1e9:.2f} GB) + "
                             f"{LAYERS * decode_bytes(ctx) / 1e9:.2f} GB of cache per step"},
            "e2e": {"value": round(nbytes_e2e / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s",
                    "h2d_bytes_per_step": 4 if token else x_host.numel() * 2,
                    "d2h_bytes_per_step": 4 if token else y_host.numel() * 2,
                    "ms_per_step": round(ms_e2e / steps, 4)},
            "gpu_launches": ((LAYERS * (17 if ffn else 11) + (4 if token else 0)) if ref_arm else
                             LAYERS * (5 if ffn else 3) + (3 if token else 0)) * steps,
            "clocks": env.sampler.summary(m0, m1),
        }
        if token:
            line["tokens_per_s"] = round(steps / (ms * 1e-3), 1)
            line["e2e"]["tokens_per_s"] = round(steps / (ms_e2e * 1e-3), 1)
    if ref_arm:
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "GB/s", "cores": 0, "kind": "reference",
                                "sample": "whole workload on the GPU: the reference has no CPU implementation of this path"}
        line["e2e"].update({"h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "value": line["value"]})
        return line
    # ---- check (one GPU): layer 0 of one more step against the oracle layer on the same input, and
    # the final row against the oracle's 16-layer chain (reported; roundings build up over layers)
    if world == 1:
        w = Ws[0]
        L0 = pool.length(seq)
        kk = torch.zeros(KV_HEADS, L0 + 1, D, dtype=torch.bfloat16, device=dev)
        vv = torch.zeros_like(kk)
        caches = []
        for l in range(LAYERS):
            pool.gather_kv(l, seq, kk, vv, L0 + 1)
            torch.cuda.synchronize()
            caches.append((_u16(kk), _u16(vv)))
        pool.reserve(seq, L0 + 1)
        pool.batch_set([seq])
        y0 = torch.zeros(1, H, dtype=torch.bfloat16, device=dev)
        run_layers(0, 0, 1, x_dev, y0)
        run_layers(0, 1, LAYERS, y0, y_dev)
        torch.cuda.synchronize()
        pool.check()
        t0 = time.perf_counter()
        cur = _u16(x_host)
        first = None
        for l in range(LAYERS):
            K, V = caches[l]
            xn = orc.rmsnorm(cur, _u16(w["nw"][l]), 1e-5)
            q = orc.gemm_bf16(xn, _u16(w["wq"][l])).reshape(1, Q_HEADS, D)
            k = orc.gemm_bf16(xn, _u16(w["wk"][l])).reshape(1, KV_HEADS, D)
            v = orc.gemm_bf16(xn, _u16(w["wv"][l])).reshape(1, KV_HEADS, D)
            K[:, L0] = orc.rope(k, cos_h, sin_h, L0, 1)[:, 0]
            V[:, L0] = v[0]
            O, _ = orc.attention(orc.rope(q, cos_h, sin_h, L0, 1), K, V, L0 + 1)
            lin = orc.gemm_bf16(orc.f32_to_bf16(O[:, 0].reshape(1, NQ)), _u16(w["wo"][l]))
            cur = orc.f32_to_bf16(orc.bf16_to_f32(cur) + orc.bf16_to_f32(lin))
            if ffn:
                cur = orc.ffn(cur, _u16(w["fn"][l]), _u16(w["wg"][l]), _u16(w["wu"][l]), _u16(w["wd"][l]), 1e-5, True)
            if l == 0:
                first = cur
        dt = time.perf_counter() - t0
        e0 = row_rel_err(orc.bf16_to_f32(_u16(y0)), orc.bf16_to_f32(first), row=H)
        e15 = row_rel_err(orc.bf16_to_f32(_u16(y_dev)), orc.bf16_to_f32(cur), row=H)
        line["checks"] = {"oracle_layer0_max_err_over_row_max": e0, "oracle_layer0_ok": bool(e0 <= (2.0 ** -5 if ffn else 2.0 ** -6)),
                          "oracle_16_layer_chain_max_err_over_row_max": e15}
        if token:
            # the head on the GPU's own final row against the oracle on that row; the last timed step's token
            # against the reference kernel's rule on the logits that step produced
            last_logits, last_tok = _u16(logits_dev), int(tok_dev.cpu().item())
            chk = torch.zeros(1, VOC, dtype=torch.bfloat16, device=dev)
            paged.lm_head(y_dev, final_norm, w_lm, chk, 1)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            want = orc.gemm_bf16(orc.rmsnorm(_u16(y_dev), _u16(final_norm), 1e-5), _u16(w_lm))
            dt += time.perf_counter() - t1
            eh = row_rel_err(orc.bf16_to_f32(_u16(chk)), orc.bf16_to_f32(want), row=VOC)
            line["checks"].update({"head_logits_max_err_over_row_max": eh, "head_logits_ok": bool(eh <= 2.0 ** -7),
                                   "token": last_tok, "token_is_the_reference_rule_on_its_logits":
                                       bool(last_tok == int(orc.argmax_reference_rule(last_logits)[0]))})
        line["cpu_baseline"] = {"value": round((LAYERS * (decode_bytes(L0 + 1) + weight_bytes) + head_bytes) / dt / 1e9, 3), "unit": "GB/s",
                                "cores": orc.num_threads(), "kind": "port",
                                "sample": f"one token through all {LAYERS} layers" + (" and the head" if token else "") +
                                          f" with the CPU oracle chain, {dt:.2f} s"}
        n_launch = 5 if ffn else 3
        line["roofline"] = {"bound": "hbm", "kernel": ("embedding_rows_kernel + " if token else "") +
                                                       "qkv_project_kernel + decode_kernel + qkv_project_kernel" +
                                                       (" + ffn_gate_up_kernel + ffn_down_kernel" if ffn else "") +
                                                       f" ({n_launch} launches per layer)" +
                                                       (" + qkv_project_kernel (head) + argmax_rows_kernel" if token else ""),
                            "achieved": round(value, 1), "peak": peak, "unit": "GB/s", "frac": round(value / peak, 4),
                            "peak_source": f"of {peak_kind}", "us_per_launch": round(ms / steps * 1e3 / LAYERS / n_launch, 2),
                            "bytes_per_launch": (decode_bytes(ctx) + weight_bytes) // n_launch, "traffic": None}
        if sub and ref is not None:
            ref_step()
            rms = local_timed(torch, ref_step, 2) / 2
            rb = LAYERS * (decode_bytes(ctx) + weight_bytes) + head_bytes
            line["reference"] = {"value": round(rb / (rms * 1e-3) / 1e9, 2), "unit": "GB/s",
                                 "us_per_layer": round(rms * 1e3 / LAYERS, 2), "us_per_token": round(rms * 1e3, 2),
                                 "how": "the reference's RMSNorm, 3 GEMMs, RoPE kernels, append copies, attention kernel, "
                                        "layout kernel, output GEMM and residual add" +
                                        (", then RMSNorm, gate and up GEMMs, SiLU*up kernel, down GEMM and residual add" if ffn else "") +
                                        " per layer, with its synchronisations" +
                                        ("; around them the blocking id copy, embedding kernel, final RMSNorm, head GEMM, "
                                         "argmax with its allocation and blocking copy" if token else "")}
    env.barrier()
    if xchg is not None:
        xchg.close()
    if pool is not None:
        pool.close()
    return line

def run_lm_head(env: Env, args, sub: bool = False):
    """The end of a decode step: final RMSNorm + language-model head (hidden 2048 -> 128256 logits, a
    525 MB weight stream) + greedy sampling, batch 1.  Ours: one weight-streaming launch and one argmax
    launch.  Reference arm: its RMSNorm, launch_gemm_2048x128256 and launch_argmax with the
    synchronisations, the per-token cudaMalloc/cudaFree and the blocking copy of its decode loop
    (src/runtime/llama_runtime.cu:880-930)."""
    torch = env.torch
    if env.rank != 0:
        return None  # independent replicas only
    from oracle import oracle as orc
    dev = env.dev
    H, V = HIDDEN, 128256
    steps = max(5, args.steps // 2) if sub else args.steps
    warmup = 3 if sub else args.warmup
    ref_arm = args.impl == "reference" and not sub
    gen = torch.Generator(device=dev)
    gen.manual_seed(321)
    w = (torch.randn(H, V, generator=gen, device=dev) * 0.03).to(torch.bfloat16)  # 525 MB: larger than L2
    nw = (torch.randn(H, generator=gen, device=dev) * 0.7).to(torch.bfloat16)
    x_host = torch.randn(1, H, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).pin_memory()
    x = x_host.to(dev)
    logits = torch.zeros(1, V, dtype=torch.bfloat16, device=dev)
    token = torch.zeros(1, dtype=torch.int32, device=dev)
    token_host = torch.zeros(1, dtype=torch.int32).pin_memory()
    nbytes = (H * V + H + V) * 2
    ref = orc.ref() if orc.ref_available() else None
    if ref_arm and ref is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built"}
    xn = torch.zeros(1, H, dtype=torch.bfloat16, device=dev)

    def ref_step():
        ref.ref_rmsnorm(x.data_ptr(), nw.data_ptr(), xn.data_ptr(), 1, 1e-5)
        torch.cuda.synchronize()
        ref.ref_gemm(xn.data_ptr(), w.data_ptr(), logits.data_ptr(), 1, V, H)
        torch.cuda.synchronize()
        t = torch.empty(1, dtype=torch.int32, device=dev)  # the loop's per-token cudaMalloc / cudaFree
        ref.ref_argmax(logits.data_ptr(), t.data_ptr())
        token_host.copy_(t)  # blocking copy
        del t
        torch.cuda.synchronize()

    if not ref_arm:
        from llama_transformer_runtime_b200 import paged

        def ours_step():
            paged.lm_head(x, nw, w, logits, 1)
            paged.argmax(logits, token, 1)

    step = ref_step if ref_arm else ours_step

    def e2e_step():
        x.copy_(x_host, non_blocking=True)
        step()
        if not ref_arm:
            token_host.copy_(token, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    m0 = env.sampler.mark()
    for _ in range(warmup):
        step()
    ms = local_timed(torch, step, steps)
    ms_e2e = local_timed(torch, e2e_step, steps)
    m1 = env.sampler.mark()
    value = nbytes * steps / (ms * 1e-3) / 1e9
    peak, pk = measured_peak()
    line = {
        "metric": "lm_head_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms / steps, 4), "us_per_token": round(ms / steps * 1e3, 2), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "lm_head_2048x128256_argmax_batch1", "hidden": H, "vocab": V, "batch": 1,
                   "l2": "the weight (525 MB) is larger than L2"},
        "e2e": {"value": round(nbytes * steps / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s", "h2d_bytes_per_step": H * 2,
                "d2h_bytes_per_step": 4, "ms_per_step": round(ms_e2e / steps, 4)},
        "gpu_launches": (3 if ref_arm else 2) * steps, "clocks": env.sampler.summary(m0, m1),
    }
    if ref_arm:
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "GB/s", "cores": 0, "kind": "reference",
                                "sample": "whole workload on the GPU: the reference has no CPU implementation of this path"}
        line["e2e"].update({"h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "value": line["value"]})
        return line
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    want = orc.gemm_bf16(orc.rmsnorm(_u16(x_host), _u16(nw), 1e-5), _u16(w))
    dt = time.perf_counter() - t0
    got = _u16(logits)
    err = row_rel_err(orc.bf16_to_f32(got), orc.bf16_to_f32(want), row=V)
    tok = int(token.cpu().item())
    line["checks"] = {"logits_max_err_over_row_max": err, "logits_ok": bool(err <= 2.0 ** -7),
                      "token": tok, "token_is_the_reference_rule_on_these_logits": bool(tok == int(orc.argmax_reference_rule(got)[0]))}
    line["cpu_baseline"] = {"value": round(nbytes / dt / 1e9, 3), "unit": "GB/s", "cores": orc.num_threads(), "kind": "port",
                            "sample": f"one token: RMSNorm + 2048 x 128256 product with the CPU oracle, {dt:.2f} s"}
    line["roofline"] = {"bound": "hbm", "kernel": "qkv_project_kernel (language-model head)", "achieved": round(value, 1),
                        "peak": peak, "unit": "GB/s", "frac": round(value / peak, 4), "peak_source": f"of {pk}",
                        "us_per_launch": round(ms / steps * 1e3, 2), "bytes_per_launch": nbytes, "traffic": None}
    if sub and ref is not None:
        ref_step()
        rms = local_timed(torch, ref_step, 3) / 3
        line["reference"] = {"value": round(nbytes / (rms * 1e-3) / 1e9, 2), "unit": "GB/s", "us_per_token": round(rms * 1e3, 2),
                             "how": "the reference's RMSNorm, launch_gemm_2048x128256 and launch_argmax with the "
                                    "synchronisations, allocation and blocking copy of its decode loop"}
    return line


# =============================================================================
# a whole prompt through the 16 blocks (the prompt path of runtime::Transformer)
# =============================================================================
def run_prompt(env: Env, args, sub: bool = False):
    """A 2048-token prompt through 16 transformer blocks, as Transformer::forward runs it for
    seq_len > 1 (src/runtime/transformer.cu:47-89, transformer_block.cu:24-123): per layer RMSNorm,
    Q/K/V projections + RoPE + cache append, causal attention, output projection + residual, RMSNorm,
    gate/up projections, SiLU(gate) * up, down projection + residual.  Ours: pa_rmsnorm,
    pa_qkv_project_append, pa_prefill, pa_out_project_rows, pa_ffn_rows (7 launches per layer, the
    GEMMs on tcgen05, gate and up as one with SiLU * up in its epilogue).  Reference arm: the reference's kernels in the order of its classes, with their
    synchronisations.  Metric: TFLOP/s over 2*tokens*(weights of the layer) + the causal attention."""
    torch = env.torch
    if env.rank != 0:
        return None  # independent replicas only
    from oracle import oracle as orc
    dev = env.dev
    S, H, NQ, NKV, INTER = PREFILL_TOKENS, HIDDEN, Q_HEADS * D, KV_HEADS * D, 8192
    steps = max(3, args.steps // 5) if sub else args.steps
    warmup = 3 if sub else args.warmup
    ref_arm = args.impl == "reference" and not sub
    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    mk = lambda *shape, s=0.03: (torch.randn(*shape, generator=gen, device=dev) * s).to(torch.bfloat16)
    W = dict(nw=mk(LAYERS, H, s=0.7), wq=mk(LAYERS, H, NQ), wk=mk(LAYERS, H, NKV), wv=mk(LAYERS, H, NKV), wo=mk(LAYERS, NQ, H),
             fn=mk(LAYERS, H, s=0.7), wg=mk(LAYERS, H, INTER), wu=mk(LAYERS, H, INTER), wd=mk(LAYERS, INTER, H, s=0.02))
    x_host = torch.randn(S, H, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    y_dev = torch.zeros(S, H, dtype=torch.bfloat16, device=dev)
    y_host = torch.zeros(1, H, dtype=torch.bfloat16).pin_memory()  # the last row is what the head reads
    flops_layer = 2.0 * S * (H * (NQ + 2 * NKV) + NQ * H + 3 * H * INTER) + prefill_flops(S)
    burst, sustained, kind = measured_tflops()
    ref = orc.ref() if orc.ref_available() else None
    if ref_arm and ref is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libref.so was not built"}
    cos_h, sin_h = orc.build_rope_tables(S)
    cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
    rows = lambda c: torch.zeros(S, c, dtype=torch.bfloat16, device=dev)

    if ref is not None and (ref_arm or sub):
        rb = {n: rows(c) for n, c in (("xn", H), ("q", NQ), ("k", NKV), ("v", NKV), ("arow", NQ), ("lin", H), ("xa", H),
                                       ("xb", H), ("xm", H), ("g", INTER), ("u", INTER), ("h", INTER))}
        qf = torch.empty(Q_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        kf = torch.empty(KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vf = torch.empty_like(kf)
        of = torch.empty_like(qf)
        kc = torch.zeros(LAYERS, KV_HEADS, S, D, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)

        def ref_step():
            cur = x_dev
            for l in range(LAYERS):
                ref.ref_rmsnorm(cur.data_ptr(), W["nw"][l].data_ptr(), rb["xn"].data_ptr(), S, 1e-5)
                torch.cuda.synchronize()
                for wm, o, n in ((W["wq"], rb["q"], NQ), (W["wk"], rb["k"], NKV), (W["wv"], rb["v"], NKV)):
                    ref.ref_gemm(rb["xn"].data_ptr(), wm[l].data_ptr(), o.data_ptr(), S, n, H)
                    torch.cuda.synchronize()
                ref.ref_rope_qkv(rb["q"].data_ptr(), qf.data_ptr(), rb["k"].data_ptr(), kf.data_ptr(), rb["v"].data_ptr(),
                                 vf.data_ptr(), cos.data_ptr(), sin.data_ptr(), S, 0)
                ref.ref_append_strided(kc[l].data_ptr(), vc[l].data_ptr(), kf.data_ptr(), vf.data_ptr(), S, 0, S, None)
                ref.ref_flash_attention(qf.data_ptr(), kc[l].data_ptr(), vc[l].data_ptr(), of.data_ptr(), None, 1,
                                        Q_HEADS, KV_HEADS, S, S, S, 0.125, 1, None)
                torch.cuda.synchronize()
                ref.ref_flash_output_layout(of.data_ptr(), rb["arow"].data_ptr(), S)
                torch.cuda.synchronize()
                ref.ref_gemm(rb["arow"].data_ptr(), W["wo"][l].data_ptr(), rb["lin"].data_ptr(), S, H, NQ)
                torch.cuda.synchronize()
                ref.ref_residual_add(cur.data_ptr(), rb["lin"].data_ptr(), rb["xm"].data_ptr(), S * H)
                torch.cuda.synchronize()
                ref.ref_rmsnorm(rb["xm"].data_ptr(), W["fn"][l].data_ptr(), rb["xn"].data_ptr(), S, 1e-5)
                ref.ref_gemm(rb["xn"].data_ptr(), W["wg"][l].data_ptr(), rb["g"].data_ptr(), S, INTER, H)
                ref.ref_gemm(rb["xn"].data_ptr(), W["wu"][l].data_ptr(), rb["u"].data_ptr(), S, INTER, H)
                ref.ref_silu_mul(rb["g"].data_ptr(), rb["u"].data_ptr(), rb["h"].data_ptr(), S)
                ref.ref_gemm(rb["h"].data_ptr(), W["wd"][l].data_ptr(), rb["lin"].data_ptr(), S, H, INTER)
                torch.cuda.synchronize()
                nxt = rb["xa"] if l % 2 == 0 else rb["xb"]
                ref.ref_residual_add(rb["xm"].data_ptr(), rb["lin"].data_ptr(), nxt.data_ptr(), S * H)
                torch.cuda.synchronize()
                cur = nxt
            y_dev.copy_(cur)

    pool = None
    if not ref_arm:
        from llama_transformer_runtime_b200 import paged
        nb = (S + BLOCK - 1) // BLOCK
        num_blocks = nb + nb // 4 + 8
        pool = paged.KVPool(LAYERS, num_blocks, KV_HEADS, 1, nb + 1, device=env.local_rank)
        pool.set_free_order(np.random.default_rng(5).permutation(num_blocks))
        seq = pool.create_seq()
        pool.reserve(seq, S)
        pool.batch_set([seq], [S])
        P = {n: paged.pack_projection_weights(W[n]) for n in ("wq", "wk", "wv", "wo", "wg", "wu", "wd")}
        F = paged.ffn_weights(W["fn"], P["wg"], P["wu"], P["wd"])
        xn, q_rot, attn, mid = rows(H), rows(NQ), rows(NQ), rows(H)
        pp = [rows(H), rows(H)]
        scratch = torch.zeros(S * (H + INTER), dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()

        def ours_step(last=None):
            # the same prompt positions are rewritten every step (the table is fixed)
            cur = x_dev
            for l in range(LAYERS if last is None else last):
                out = y_dev if l == LAYERS - 1 else pp[l & 1]
                paged.rmsnorm(cur, W["nw"][l], xn, S, H)
                pool.qkv_project_append(l, xn, P["wq"][l], P["wk"][l], P["wv"][l], cos, sin, q_rot, H)
                pool.prefill(l, q_rot, attn)
                pool.out_project_rows(attn, P["wo"][l], cur, mid, S, H)
                paged.ffn_rows(pool, F, l, mid, scratch, out, S, add_residual=True)
                cur = out
            return cur

    step = ref_step if ref_arm else ours_step

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        step()
        y_host.copy_(y_dev[S - 1:S], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    m0 = env.sampler.mark()
    for _ in range(warmup):
        step()
    ms = local_timed(torch, step, steps) / steps
    ms_e2e = local_timed(torch, e2e_step, steps) / steps
    m1 = env.sampler.mark()
    value = flops_layer * LAYERS / (ms * 1e-3) / 1e12
    line = {
        "metric": "prompt_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "us_per_layer": round(ms * 1e3 / LAYERS, 2), "tokens_per_s": round(S / (ms * 1e-3), 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"prompt_{S}tokens_x{LAYERS}blocks", "tokens": S, "hidden": H, "inter": INTER, "layers": LAYERS,
                   "flops": "per layer 2*tokens*(Wq+Wk+Wv+Wo+Wgate+Wup+Wdown elements) + 4*32*64*S(S+1)/2",
                   "l2": "per-layer weights are distinct tensors (122 MB per layer)"},
        "e2e": {"value": round(flops_layer * LAYERS / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": (LAYERS * 19 if ref_arm else LAYERS * 7) * steps, "clocks": env.sampler.summary(m0, m1),
    }
    if ref_arm:
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                "sample": "whole workload on the GPU: the reference has no CPU implementation of this path"}
        line["e2e"].update({"h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "value": line["value"]})
        return line
    line["roofline"] = {"bound": "tensor", "kernel": "qkv_gemm_kernel (4 of the 7 launches of a layer) + prefill_kernel",
                        "achieved": round(value, 2), "peak": burst, "unit": "TFLOP/s", "frac": round(value / burst, 4),
                        "peak_source": f"of {kind} (cuBLAS bf16 burst)", "us_per_launch": round(ms * 1e3 / LAYERS / 7, 2),
                        "flops_per_launch": flops_layer / 7, "traffic": None}
    pool.check()
    # check and CPU baseline: the first block's output rows 0..31 against the oracle chain on the same input
    # (causal: these rows attend to themselves only)
    r = 32
    first = ours_step(last=1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    xs = _u16(x_host[:r])
    xn_o = orc.rmsnorm(xs, _u16(W["nw"][0]), 1e-5)
    q = orc.gemm_bf16(xn_o, _u16(W["wq"][0])).reshape(r, Q_HEADS, D)
    k = orc.gemm_bf16(xn_o, _u16(W["wk"][0])).reshape(r, KV_HEADS, D)
    v = orc.gemm_bf16(xn_o, _u16(W["wv"][0])).reshape(r, KV_HEADS, D)
    K = orc.rope(k, cos_h, sin_h, 0, 1)  # [heads, rows, 64]
    V = np.ascontiguousarray(v.transpose(1, 0, 2))
    O, _ = orc.attention(orc.rope(q, cos_h, sin_h, 0, 1), K, V, r)
    lin = orc.gemm_bf16(orc.f32_to_bf16(O.transpose(1, 0, 2).reshape(r, NQ)), _u16(W["wo"][0]))
    a = orc.f32_to_bf16(orc.bf16_to_f32(xs) + orc.bf16_to_f32(lin))
    want = orc.ffn(a, _u16(W["fn"][0]), _u16(W["wg"][0]), _u16(W["wu"][0]), _u16(W["wd"][0]), 1e-5, True)
    dt = time.perf_counter() - t0
    err = row_rel_err(orc.bf16_to_f32(_u16(first[:r])), orc.bf16_to_f32(want), row=H)
    line["checks"] = {"oracle_block0_rows0_31_max_err_over_row_max": err, "oracle_block0_ok": bool(err <= 2.0 ** -5)}
    line["cpu_baseline"] = {"value": round(2.0 * r * (H * (NQ + 2 * NKV) + NQ * H + 3 * H * INTER) / dt / 1e12, 5), "unit": "TFLOP/s",
                            "cores": orc.num_threads(), "kind": "port",
                            "sample": f"{r} rows through block 0 with the CPU oracle chain, {dt:.2f} s"}
    if sub and ref is not None:
        ref_step()
        rms = local_timed(torch, ref_step, 1)
        line["reference"] = {"value": round(flops_layer * LAYERS / (rms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                             "us_per_layer": round(rms * 1e3 / LAYERS, 2), "tokens_per_s": round(S / (rms * 1e-3), 1),
                             "how": "the reference's RMSNorm, GEMM, RoPE, append, attention, layout, residual and SiLU kernels "
                                    "in the order of its Attention, FeedForward and TransformerBlock classes, with their synchronisations"}
    pool.close()
    return line


# =============================================================================
# a whole decode step for several sequences at once
# =============================================================================
def run_token_batch(env: Env, args):
    """pa_decode_token for --seqs sequences (1 to 8) of context --chain-ctx in one step: the weights are
    read once for all of them (the tensor-core weight stream multiplies up to 8 rows per pass), each
    sequence reads its own cache.  The reference has no batched step: a Transformer object holds one
    sequence's cache and decode_forward takes one token, so B sequences cost it B steps; its arm here is
    the single-sequence step of workload `token`."""
    torch = env.torch
    if env.rank != 0:
        return None  # independent replicas only
    if args.impl == "reference":
        line = run_chain(env, args, token=True)
        if line and "config" in line:
            line["config"]["note"] = ("the reference has no batched decode step: this is its single-sequence step; "
                                      "B sequences cost it B of them")
        return line
    from oracle import oracle as orc
    from llama_transformer_runtime_b200 import paged
    dev = env.dev
    B = max(1, min(8, args.seqs if args.seqs != 64 else 8))
    ctx, H, NQ, NKV, INTER, VOC = args.chain_ctx, HIDDEN, Q_HEADS * D, KV_HEADS * D, 8192, 128256
    steps, warmup = args.steps, args.warmup
    gen = torch.Generator(device=dev)
    gen.manual_seed(41)
    mk = lambda *shape, s=0.03: (torch.randn(*shape, generator=gen, device=dev) * s).to(torch.bfloat16)
    W = dict(nw=mk(LAYERS, H, s=0.7), wq=mk(LAYERS, H, NQ), wk=mk(LAYERS, H, NKV), wv=mk(LAYERS, H, NKV), wo=mk(LAYERS, NQ, H),
             fn=mk(LAYERS, H, s=0.7), wg=mk(LAYERS, H, INTER), wu=mk(LAYERS, H, INTER), wd=mk(LAYERS, INTER, H, s=0.02))
    embed, w_lm, final_norm = mk(VOC, H, s=1.0), mk(H, VOC), mk(H, s=0.7)
    total_steps = warmup + 2 * steps + 8
    cos_h, sin_h = orc.build_rope_tables(ctx + total_steps + 2)
    cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
    need = (ctx + total_steps + BLOCK - 1) // BLOCK
    num_blocks = B * need + B * need // 4 + 8
    pool = paged.KVPool(LAYERS, num_blocks, KV_HEADS, B, need + 1, device=env.local_rank)
    pool.set_free_order(np.random.default_rng(77).permutation(num_blocks))
    seqs = [pool.create_seq() for _ in range(B)]
    ones = torch.ones(ctx, 32, dtype=torch.float32, device=dev)
    zeros = torch.zeros(ctx, 32, dtype=torch.float32, device=dev)
    kvgen = torch.Generator(device=dev)
    kvgen.manual_seed(99)
    for sq in seqs:  # every sequence its own cache contents, blocks interleaved in the shared pool
        pool.reserve(sq, ctx)
        pool.batch_set([sq], [ctx])
        for layer in range(LAYERS):
            k = (torch.randn(ctx, KV_HEADS, D, generator=kvgen, device=dev) * 0.5).to(torch.bfloat16)
            v = (torch.randn(ctx, KV_HEADS, D, generator=kvgen, device=dev) * 0.5).to(torch.bfloat16)
            pool.append(layer, None, k, v, ones, zeros, None)
    torch.cuda.synchronize()
    del ones, zeros
    WA = paged.attention_weights(W["nw"], W["wq"], W["wk"], W["wv"], W["wo"])
    WF = paged.ffn_weights(W["fn"], W["wg"], W["wu"], W["wd"])
    M = paged.model_weights(embed, WA, WF, final_norm, w_lm)
    tok_host = torch.arange(1000, 1000 + B, dtype=torch.int32).pin_memory()
    tok_dev = tok_host.to(dev)
    logits = torch.zeros(B, VOC, dtype=torch.bfloat16, device=dev)
    state = {"len": ctx}

    def step():
        state["len"] += 1
        for sq in seqs:
            pool.reserve(sq, state["len"])
        pool.batch_set(seqs)
        paged.decode_token(pool, M, tok_dev, tok_dev, logits, cos, sin, chained=True)

    def e2e_step():
        tok_dev.copy_(tok_host, non_blocking=True)
        step()
        tok_host.copy_(tok_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    weight_bytes = LAYERS * ((H * (NQ + 2 * NKV) + NQ * H + H) * 2 + (3 * H * INTER + H) * 2) + (H * VOC + H) * 2
    def nbytes(l0, l1):
        return sum(weight_bytes + B * (LAYERS * decode_bytes(L) + 2 * H * 2 + 2 * VOC * 2) for L in range(l0 + 1, l1 + 1))

    m0 = env.sampler.mark()
    for _ in range(warmup):
        step()
    l0 = state["len"]
    ms = local_timed(torch, step, steps)
    b1 = nbytes(l0, state["len"])
    l0 = state["len"]
    ms_e2e = local_timed(torch, e2e_step, steps)
    b2 = nbytes(l0, state["len"])
    m1 = env.sampler.mark()
    pool.check()
    value = b1 / (ms * 1e-3) / 1e9
    peak, pk = measured_peak()
    got = _u16(logits)
    toks = tok_dev.cpu().numpy()
    line = {
        "metric": "decode_token_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms / steps, 4), "us_per_step": round(ms / steps * 1e3, 2),
        "tokens_per_s": round(B * steps / (ms * 1e-3), 1), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"token_batch{B}_ctx{ctx}_x{LAYERS}layers_vocab{VOC}", "sequences": B, "context": ctx,
                   "layers": LAYERS, "bytes": "the model's weights once per step + every sequence's cache, embedding row and logits",
                   "l2": f"{weight_bytes / 1e9:.2f} GB of weights per step"},
        "e2e": {"value": round(b2 / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 4 * B, "ms_per_step": round(ms_e2e / steps, 4),
                "tokens_per_s": round(B * steps / (ms_e2e * 1e-3), 1)},
        "gpu_launches": (LAYERS * 5 + 3) * steps, "clocks": env.sampler.summary(m0, m1),
        "checks": {"logits_finite": bool(np.isfinite(orc.bf16_to_f32(got)).all()),
                   "tokens_are_the_reference_rule_on_their_logits": bool(np.array_equal(toks, orc.argmax_reference_rule(got)))},
        "roofline": {"bound": "hbm", "kernel": "the 83 launches of pa_decode_token", "achieved": round(value, 1), "peak": peak,
                     "unit": "GB/s", "frac": round(value / peak, 4), "peak_source": f"of {pk}",
                     "us_per_launch": round(ms / steps * 1e3 / (LAYERS * 5 + 3), 2), "bytes_per_launch": b1 // steps // (LAYERS * 5 + 3),
                     "traffic": None},
        "cpu_baseline": None,
    }
    pool.close()
    return line


# =============================================================================
def decode4k_sub(env: Env, args):
    line = run_decode(env, args, "decode4k", sub=True)
    r = reference_decode(env, "decode4k", 3, 2, with_e2e=False)
    if line is not None and r is not None:
        line["reference"] = {"value": round(r["value"], 2), "unit": "GB/s",
                             "us_per_token_per_layer": round(r["ms_per_step"] * 1e3 / LAYERS, 2),
                             "how": "the reference's RoPE kernels, 16 append copies, attention kernel at q_seq_len 1 "
                                    "and layout kernel per layer, as Attention::forward drives them"}
    return line


SUB_BLOCKS = {
    "decode4k": decode4k_sub,
    "prefill": lambda env, a: run_prefill(env, a, sub=True),
    "append": lambda env, a: run_prefill(env, a, sub=True, append_only=True),
    "out_project": lambda env, a: run_qkv(env, a, sub=True, which="out"),
    "qkv_decode": lambda env, a: run_qkv(env, a, sub=True, which="qkv"),
    "qkv_prefill": lambda env, a: run_qkv_prefill(env, a, sub=True),
    "decode_chain": lambda env, a: run_chain(env, a, sub=True),
    "block_chain": lambda env, a: run_chain(env, a, sub=True, ffn=True),
    "lm_head": lambda env, a: run_lm_head(env, a, sub=True),
    "token": lambda env, a: run_chain(env, a, sub=True, token=True),
    "prompt": lambda env, a: run_prompt(env, a, sub=True),
}


def compact(line):
    """A sub-block of the default line: the full line minus the keys the outer line already carries."""
    if line is None:
        return None
    drop = {"higher_is_better", "vs_baseline", "dtype", "data", "n_gpus", "warmup"}
    return {k: v for k, v in line.items() if k not in drop}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=15, help="decode: timed blocks of --steps steps; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode128k",
                    choices=sorted(WORKLOADS) + ["prefill2k", "append2k", "batch64", "qkv_decode", "out_project", "qkv_prefill",
                                                  "decode_chain", "block_chain", "lm_head", "token", "token_batch", "prompt"])
    ap.add_argument("--chain-ctx", type=int, default=4096, help="decode_chain: context length")
    ap.add_argument("--ctx", type=int, default=0, help="decode128k / decode4k: another context length (0 = the workload's own)")
    ap.add_argument("--no-sub", action="store_true", help="default workload: skip the sub-blocks")
    ap.add_argument("--sub", default="", help="default workload: comma-separated sub-blocks to run (default: all)")
    ap.add_argument("--seqs", type=int, default=64, help="batch64: number of sequences")
    ap.add_argument("--layers", type=int, default=16, help="fewer layers make a small case for profiling")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N>1: partials pushed by the decode epilogue over NVLink (fused) or NCCL all-gather")
    ap.add_argument("--chunk-blocks", type=int, default=0, help="decode: blocks per split-KV chunk (0 = planner)")
    ap.add_argument("--combiners", type=int, default=0,
                    help="decode: combining CTAs per (sequence, head) in the one-launch step (0 = planner)")
    ap.add_argument("--decode-cluster", type=int, default=0,
                    help="decode_chain / block_chain: cluster form of the one-layer decode kernel "
                         "(0 = planner, -1 = never, 2/4/8/16 = that cluster size)")
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
    rank, _, world = dist_env()
    if args.impl == "reference" and rank != 0:
        return  # the reference is single-GPU: rank 0 alone runs it
    sharded = args.workload in WORKLOADS or args.workload in ("batch64", "qkv_decode", "out_project", "decode_chain", "block_chain")
    env = Env(want_group=(args.impl == "ours" and sharded))
    line = None
    if args.workload in WORKLOADS:
        if args.impl == "reference":
            line = run_reference(env, args, args.workload)
        else:
            line = run_decode(env, args, args.workload)
            default = args.workload == "decode128k" and not args.no_sub and LAYERS == 16
            if default and world == 1:
                names = [n for n in (args.sub.split(",") if args.sub else SUB_BLOCKS) if n in SUB_BLOCKS]
                line["sub"] = {}
                for n in names:
                    try:
                        line["sub"][n] = compact(SUB_BLOCKS[n](env, args))
                    except Exception as exc:  # a failing sub-block must not lose the main line
                        line["sub"][n] = {"error": f"{type(exc).__name__}: {exc}"}
            elif default and world > 1:
                try:
                    b = run_batch(env, args, sub=True)
                except Exception as exc:
                    b = {"error": f"{type(exc).__name__}: {exc}"}
                if rank == 0:
                    line["batch64"] = compact(b)
    elif args.workload == "qkv_decode":
        line = run_qkv(env, args, which="qkv")
    elif args.workload == "out_project":
        line = run_qkv(env, args, which="out")
    elif args.workload == "qkv_prefill":
        line = run_qkv_prefill(env, args)
    elif args.workload == "prefill2k":
        line = run_prefill(env, args)
    elif args.workload == "append2k":
        line = run_prefill(env, args, append_only=True)
    elif args.workload == "batch64":
        line = run_batch(env, args)
    elif args.workload == "decode_chain":
        line = run_chain(env, args)
    elif args.workload == "block_chain":
        line = run_chain(env, args, ffn=True)
    elif args.workload == "lm_head":
        line = run_lm_head(env, args)
    elif args.workload == "token":
        line = run_chain(env, args, token=True)
    elif args.workload == "prompt":
        line = run_prompt(env, args)
    elif args.workload == "token_batch":
        line = run_token_batch(env, args)
    if rank == 0 and line is not None:
        print(json.dumps(line), flush=True)
    env.sampler.stop()
    env.close()


if __name__ == "__main__":
    main()
