"""The sharded decode step on TWO real GPUs, one process per GPU, against the CPU oracle: the
one-launch step (pa_decode_step_sharded: word exchange over NVLink peer stores, merge in the
kernel) and the data-chained step (pa_attention_step with an exchange: one kernel per layer).
Skipped where fewer than two GPUs are visible; the same step body runs on one GPU in
tests/test_sharded_step_gpu.py with the ranks co-located in one launch.

The ranks are child processes; they meet through a gloo group (handles of the exchange buffers,
results) and NCCL is not involved.  A rank leaves only after a final barrier, with nothing in
flight."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_q):
    import torch.distributed as dist

    from llama_transformer_runtime_b200 import paged
    from oracle import oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"

    def to_dev(u16):
        return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).view(torch.bfloat16).to(dev)

    def to_u16(t):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)

    rng = np.random.default_rng(5150)  # the same data on every rank
    layers, steps, L = 4, 6, 1000
    cuts = [0, 496, L]
    lo, hi = cuts[rank], cuts[rank + 1]
    owner = world - 1
    cos, sin = orc.build_rope_tables(L + steps + 1)
    cos_d, sin_d = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
    K = [orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)]
    V = [orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)]
    nb = (hi - lo + steps + 15) // 16 + 4
    pool = paged.KVPool(layers, nb, 8, 1, device=rank)
    pool.set_free_order(np.random.default_rng(rank).permutation(nb))
    s = pool.create_seq()
    n = hi - lo
    pool.reserve(s, n)
    pool.batch_set([s], [n])
    ones = torch.ones(n, 32, dtype=torch.float32, device=dev)
    zeros = torch.zeros(n, 32, dtype=torch.float32, device=dev)
    for l in range(layers):
        pool.append(l, None, to_dev(K[l][:, lo:hi].transpose(1, 0, 2)), to_dev(V[l][:, lo:hi].transpose(1, 0, 2)),
                    ones, zeros, None)
    xchg = paged.Exchange(rank, rank, world, 1, 8)
    handles = [None] * world
    dist.all_gather_object(handles, xchg.handle())
    xchg.connect(handles)
    dist.barrier()
    ok, worst = True, 0.0
    try:
        # ---- part 1: the one-launch step, several steps in a row
        for step in range(steps):
            pos = L + step
            q_new = orc.randn_bf16(rng, (layers, 1, 32, 64))
            k_new = orc.randn_bf16(rng, (layers, 1, 8, 64))
            v_new = orc.randn_bf16(rng, (layers, 1, 8, 64))
            qd, kd, vd = to_dev(q_new), to_dev(k_new), to_dev(v_new)
            q_rot = torch.zeros_like(qd)
            out = torch.full((layers, 1, 2048), 9.0, dtype=torch.bfloat16, device=dev)
            if rank == owner:
                pool.reserve(s, pool.length(s) + 1)
            pool.batch_set_sharded([s], [1 if rank == owner else 0], [1], [pos], [lo])
            before = pool.step_launches()
            paged.decode_step_sharded(pool, xchg, 0, layers, qd, kd if rank == owner else None,
                                      vd if rank == owner else None, 2048, 512, cos_d, sin_d, q_rot, out, 2048, 2048)
            torch.cuda.synchronize()
            pool.check()
            ok = ok and pool.step_launches() == before + 1
            for l in range(layers):
                K[l][:, pos] = orc.rope(k_new[l], cos, sin, pos, 1)[:, 0]
                V[l][:, pos] = v_new[l, 0]
                O, _ = orc.attention(orc.rope(q_new[l], cos, sin, pos, 1), K[l], V[l], pos + 1)
                got = orc.bf16_to_f32(to_u16(out[l, 0])).astype(np.float64).reshape(32, 64)
                want = O[:, 0].astype(np.float64)
                rel = float(np.max(np.abs(got - want).max(axis=1) / np.abs(want).max(axis=1)))
                worst = max(worst, rel)
                ok = ok and rel <= 2.0 ** -7
            rows = [None] * world
            dist.all_gather_object(rows, to_u16(out).tobytes())
            ok = ok and all(r == rows[0] for r in rows)  # every rank merged the same bits
        # ---- part 2: the data-chained step (one kernel per layer, exchange inside the decode kernel),
        # each layer fed the GPU's own previous rows and compared with the oracle layer on that input
        pos = L + steps
        nw = orc.randn_bf16(rng, (layers, 2048), 0.7)
        wq = orc.randn_bf16(rng, (layers, 2048, 2048), 0.03)
        wk = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
        wv = orc.randn_bf16(rng, (layers, 2048, 512), 0.03)
        wo = orc.randn_bf16(rng, (layers, 2048, 2048), 0.03)
        tens = [to_dev(a) for a in (nw, wq, wk, wv, wo)]
        W = paged.attention_weights(*tens)
        cos2, sin2 = orc.build_rope_tables(pos + 2)
        cos2_d, sin2_d = torch.from_numpy(cos2).to(dev), torch.from_numpy(sin2).to(dev)
        Kx = [np.concatenate([k, np.zeros((8, 1, 64), np.uint16)], axis=1) for k in K]
        Vx = [np.concatenate([v, np.zeros((8, 1, 64), np.uint16)], axis=1) for v in V]
        if rank == owner:
            pool.reserve(s, pool.length(s) + 1)
        pool.batch_set_sharded([s], [1 if rank == owner else 0], [1], [pos], [lo])
        cur = to_dev(orc.randn_bf16(rng, (1, 2048), 1.0))
        for l in range(2):
            y = torch.zeros(1, 2048, dtype=torch.bfloat16, device=dev)
            paged.attention_step(pool, W, l, l + 1, cur, y, cos2_d, sin2_d, xchg=xchg)
            torch.cuda.synchronize()
            pool.check()
            x_u = to_u16(cur)
            xn = orc.rmsnorm(x_u, nw[l], 1e-5)
            q = orc.gemm_bf16(xn, wq[l]).reshape(1, 32, 64)
            k = orc.gemm_bf16(xn, wk[l]).reshape(1, 8, 64)
            v = orc.gemm_bf16(xn, wv[l]).reshape(1, 8, 64)
            Kx[l][:, pos] = orc.rope(k, cos2, sin2, pos, 1)[:, 0]
            Vx[l][:, pos] = v[0]
            O, _ = orc.attention(orc.rope(q, cos2, sin2, pos, 1), Kx[l], Vx[l], pos + 1)
            lin = orc.gemm_bf16(orc.f32_to_bf16(O[:, 0].reshape(1, 2048)), wo[l])
            want = orc.bf16_to_f32(orc.f32_to_bf16(orc.bf16_to_f32(x_u) + orc.bf16_to_f32(lin))).astype(np.float64)
            got = orc.bf16_to_f32(to_u16(y)).astype(np.float64)
            rel = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
            ok = ok and rel <= 2.0 ** -6
            rows = [None] * world
            dist.all_gather_object(rows, to_u16(y).tobytes())
            ok = ok and all(r == rows[0] for r in rows)
            cur = y
    except Exception as exc:  # report instead of leaving the peer waiting
        ok = False
        worst = repr(exc)
    flags = [None] * world
    dist.all_gather_object(flags, (ok, worst))
    torch.cuda.synchronize()
    dist.barrier()
    xchg.close()
    pool.close()
    if rank == 0:
        result_q.put(flags)
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_step_on_two_gpus_matches_the_oracle():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    flags = q.get(timeout=10)
    assert all(f[0] for f in flags), flags
