#!/usr/bin/env python
"""Benchmark of the decode-time retrieval-attention step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one fused decode step of one layer over one batch: group-mean query -> score
scan over every cached key -> exact top-k -> softmax attention over top-k + sink + window
(+ the new token).  The workload at every N is configuration 1 of the baseline (batch 16,
32 query / 8 KV heads, head_dim 128, 131072-token context, bf16, top-k 2048 + 64 sink + 512
window) on synthetic seeded inputs; with N > 1 every rank runs its own batch (the
(batch, kv-head) problems are independent, so there is no data-path collective) and the
reported value is the aggregate over ranks: weak scaling.

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
reference engine's exact-scan path (the Rust crate cannot be built here) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from diffcache_b200 import synth  # noqa: E402

METRIC = "decode attention steps/sec at 128K ctx"
UNIT = "steps/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, smax = [], set(), None
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax = float(parts[2])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=smax, reasons=sorted(reasons), samples=len(sm))
        return out


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return world, rank, local


def build_step_inputs(cfg: synth.StepConfig, seed: int, device):
    """Engine + resident buffers + per-step inputs for one rank, all resident in HBM."""
    from diffcache_b200 import DiffCacheGPU

    dt = synth.torch_dtype(cfg.dtype)
    n_r = cfg.n_retrieval
    eng = DiffCacheGPU(cfg.batch, cfg.q_heads, cfg.kv_heads, cfg.head_dim, max_ctx_len=n_r, dtype=cfg.dtype,
                       device=device.index, use_bruteforce=True)
    # sequence = [sink | retrieval region | window]; the newest window token is the step's new token
    k, v = synth.make_kv(cfg.batch, cfg.kv_heads, cfg.context, cfg.head_dim, seed, cfg.dtype, device=device)
    q = synth.make_query(k[:, :, cfg.sink:cfg.sink + n_r], cfg.group, seed).contiguous()
    eng.prefill(k[:, :, cfg.sink:cfg.sink + n_r], v[:, :, cfg.sink:cfg.sink + n_r])
    res_rows = cfg.sink + cfg.window - 1
    res_k = torch.zeros((cfg.batch, cfg.kv_heads, cfg.sink + cfg.window + 8, cfg.head_dim), dtype=dt, device=device)
    res_v = torch.zeros_like(res_k)
    for dst, src in ((res_k, k), (res_v, v)):
        dst[:, :, :cfg.sink] = src[:, :, :cfg.sink]
        dst[:, :, cfg.sink:res_rows] = src[:, :, cfg.sink + n_r:cfg.context - 1]
    k_new = k[:, :, -1].contiguous()
    v_new = v[:, :, -1].contiguous()
    torch.cuda.synchronize()
    host = dict(k=k, v=v)  # kept only until the caller drops it (CPU baseline sample)
    return eng, q, res_k, res_v, res_rows, k_new, v_new, host


def cpu_reference_step_rate(cfg: synth.StepConfig, k_dev, v_dev, q_dev, budget_s: float, max_steps: int,
                            sample_batch: int):
    """Times the CPU restatement of DataLayer::query (brute force) + attention on a sample of the
    batch and scales to whole-batch steps/s."""
    import oracle

    oracle.build()
    code = 0 if cfg.dtype == "bf16" else 1
    sb = min(sample_batch, cfg.batch)
    n_r, D, G = cfg.n_retrieval, cfg.head_dim, cfg.group
    P = sb * cfg.kv_heads

    def u16(t):
        return t.detach().cpu().contiguous().view(torch.uint16).numpy()

    ks = u16(k_dev[:sb, :, cfg.sink:cfg.sink + n_r]).reshape(P, n_r, D)
    vs = u16(v_dev[:sb, :, cfg.sink:cfg.sink + n_r]).reshape(P, n_r, D)
    res_k = np.concatenate([u16(k_dev[:sb, :, :cfg.sink]), u16(k_dev[:sb, :, cfg.sink + n_r:])], axis=2).reshape(P, -1, D)
    res_v = np.concatenate([u16(v_dev[:sb, :, :cfg.sink]), u16(v_dev[:sb, :, cfg.sink + n_r:])], axis=2).reshape(P, -1, D)
    qh = u16(q_dev[:sb]).reshape(P * G, D)
    threads = oracle.max_threads()
    times = []
    t_end = time.time() + budget_s
    for _ in range(max_steps):
        t0 = time.perf_counter()
        qm = oracle.group_mean(qh, G, code)
        res = oracle.query(ks, vs, qm, cfg.topk, code, exact=False, n_threads=threads)
        kk = np.ascontiguousarray(np.concatenate([res["keys"], res_k], axis=1))
        vv = np.ascontiguousarray(np.concatenate([res["vals"], res_v], axis=1))
        oracle.attend(kk, vv, qh, G, D ** -0.5, code, n_threads=threads)
        times.append(time.perf_counter() - t0)
        if time.time() > t_end and len(times) >= 2:
            break
    per_sample = float(np.median(times))
    per_step = per_sample * (cfg.batch / sb)
    return dict(value=1.0 / per_step, unit=UNIT, cores=threads, kind="port",
                sample=f"{sb} of {cfg.batch} sequences ({P} of {cfg.n_prob} (batch, kv-head) problems) per timed pass, "
                       f"{len(times)} passes, median {per_sample * 1e3:.1f} ms, scaled x{cfg.batch / sb:g}; "
                       f"C restatement of DataLayer::query (exact scan, fp32 SIMD-shaped dot) + attention, OpenMP"), \
        per_step


def run_reference(args, cfg):
    """`--impl reference`: the reference's CPU path (restated in C, see oracle/) on the host cores."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1 and rank != 0:
        return
    use_cuda = torch.cuda.is_available()
    dev = torch.device("cuda", 0) if use_cuda else torch.device("cpu")
    sb = 2
    k, v = synth.make_kv(sb, cfg.kv_heads, cfg.context, cfg.head_dim, 1000, cfg.dtype, device=dev)
    q = synth.make_query(k[:, :, cfg.sink:cfg.sink + cfg.n_retrieval], cfg.group, 1000)
    sub = synth.StepConfig(cfg.name, cfg.batch, cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.context, cfg.topk,
                           cfg.sink, cfg.window, cfg.dtype)
    # warm-up passes, then `steps` timed passes (each pass = a bounded sample of the batch)
    cpu_reference_step_rate(sub, k, v, q, budget_s=0.0, max_steps=max(1, min(args.warmup, 2)), sample_batch=sb)
    base, per_step = cpu_reference_step_rate(sub, k, v, q, budget_s=60.0, max_steps=max(2, args.steps), sample_batch=sb)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": cfg.dtype, "data": "synthetic",
        "config": workload_config(cfg, args.gpus), "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_seq_sharded(cfg, world, rank, device, steps, warmup):
    """Configuration 3: ONE long sequence, retrieval region sharded by rows over the ranks (strong
    scaling).  Local scan + top-k per rank, all-gather of candidates, identical merge select,
    attention over owned rows, all-gather of partials, log-sum-exp merge.  Returns a dict (rank 0)."""
    import torch.distributed as dist

    from diffcache_b200 import DiffCacheGPU, sharded

    dt = synth.torch_dtype(cfg.dtype)
    n_r = cfg.n_retrieval
    start, length = sharded.shard_rows(n_r, world)[rank]
    eng = DiffCacheGPU(cfg.batch, cfg.q_heads, cfg.kv_heads, cfg.head_dim, max_ctx_len=max(length, 1), dtype=cfg.dtype,
                       device=device.index, use_bruteforce=True)
    k, v = synth.make_kv(cfg.batch, cfg.kv_heads, length, cfg.head_dim, 3000 + rank, cfg.dtype, device=device,
                         pos_offset=cfg.sink + start, total=cfg.context)
    eng.prefill(k, v)
    q = synth.make_query(k, cfg.group, 3000).contiguous()
    if world > 1:
        dist.broadcast(q, src=0)
    res_k = res_v = k_new = v_new = None
    res_len = 0
    if rank == 0 or rank == world - 1:
        rows = (cfg.sink if rank == 0 else 0) + (cfg.window - 1 if rank == world - 1 else 0)
        rk, rv = synth.make_kv(cfg.batch, cfg.kv_heads, rows + 9, cfg.head_dim, 4000 + rank, cfg.dtype, device=device)
        res_k, res_v, res_len = rk, rv, rows
        if rank == world - 1:
            k_new, v_new = rk[:, :, -1].contiguous(), rv[:, :, -1].contiguous()
    del k, v
    backend = sharded.GpuShardBackend(eng, start, res_k, res_v, res_len, k_new, v_new)
    step = sharded.SequenceShardedStep(backend, cfg.topk)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        step.step(q)
    eng.check_status()

    def timed(fn):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            res = fn()
        e1.record()
        barrier()
        t_ms = e0.elapsed_time(e1)
        if world > 1:
            tt = torch.tensor([t_ms], dtype=torch.float64, device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t_ms = float(tt[0])
        return t_ms, res

    ms_stream, out = timed(lambda: step.step(q))
    # the whole step (kernels and both NCCL all-gathers) captured once and replayed
    ms_graph = None
    try:
        g = torch.cuda.CUDAGraph()
        cs = torch.cuda.Stream()
        cs.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cs):
            with torch.cuda.graph(g, stream=cs):
                out_g = step.step(q)
        torch.cuda.current_stream().wait_stream(cs)
        for _ in range(3):
            g.replay()
        ms_graph, _ = timed(lambda: g.replay())
        out = out_g
    except Exception as exc:
        print(f"# cfg3 graph capture skipped on rank {rank}: {exc}", file=sys.stderr)
    ok = torch.tensor([1.0 if ms_graph else 0.0], device=device)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    ms = ms_graph if (ms_graph and float(ok[0]) > 0) else ms_stream
    checksum = float(out.float().abs().sum())
    eng.close()
    peak, _ = measured_peaks()
    per_step = ms / steps
    gbs = cfg.algorithmic_bytes() / (per_step * 1e-3) / 1e9
    return {"workload": f"{cfg.name}: batch 1, context {cfg.context}, top-k {cfg.topk} + {cfg.sink} sink + {cfg.window} "
                        f"window, rows sharded over {world} GPU(s)",
            "value": 1e3 / per_step, "unit": UNIT, "ms_per_step": per_step, "scaling": "strong", "n_gpus": world,
            "algorithmic_bytes_per_step": cfg.algorithmic_bytes(), "aggregate_gbs": gbs,
            "frac_of_measured_hbm_x_gpus": gbs / (peak * world), "collectives_per_step": 0 if world == 1 else 2,
            "ms_per_step_stream_launch": ms_stream / steps, "ms_per_step_cuda_graph": (ms_graph / steps) if ms_graph else None,
            "out_checksum": checksum}


def _time_loop(fn, steps, warmup, world, device):
    """warmup + `steps` timed calls between barriers; CUDA events on the current stream; max over ranks."""
    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    return ms / steps


def run_cfg0(cfg, device, steps, warmup):
    """Configuration 0 (batch 1, fp16, 32K context): K+V of one input set (134 MB) is about the size of
    L2, so the step rotates over 4 independent input sets; launch-bound (72 MB of algorithmic bytes)."""
    sets = [build_step_inputs(cfg, 100 + i, device) for i in range(4)]
    outs = [torch.empty_like(s[1]) for s in sets]
    state = {"i": 0}

    def step():
        eng, q, res_k, res_v, res_rows, k_new, v_new, _ = sets[state["i"] % 4]
        eng.decode_attend(q, outs[state["i"] % 4], cfg.topk, res_k=res_k, res_v=res_v, res_len=res_rows, k_new=k_new,
                          v_new=v_new)
        state["i"] += 1

    per = _time_loop(step, steps, warmup, 1, device)
    graph_per = None
    try:  # the same four steps captured once in a CUDA graph (launch-bound case)
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                for _ in range(4):
                    step()
        torch.cuda.current_stream().wait_stream(s)
        graph_per = _time_loop(g.replay, max(1, steps // 4), warmup, 1, device) / 4
    except Exception as exc:  # capture is an optimisation, not a requirement
        graph_per = None
        print(f"# cfg0 graph capture skipped: {exc}", file=sys.stderr)
    for st in sets:
        st[0].check_status()
        st[0].close()
    best = min(per, graph_per) if graph_per else per
    return {"value": 1e3 / best, "ms_per_step": best, "ms_per_step_stream_launch": per, "ms_per_step_cuda_graph": graph_per,
            "l2_policy": "4 input sets rotated (each 134 MB of K+V, total 537 MB > L2)", "gpu_launches_per_step": 4}


def run_cfg2(cfg, world, rank, device, steps, warmup, n_layers=32, hidden=4096):
    """Configuration 2: 32-layer Llama-3-8B-shaped attention stack, KV-head sharded over the ranks."""
    from diffcache_b200.stack import AttentionStack

    stack = AttentionStack(n_layers, hidden, cfg.batch, cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.context, cfg.topk,
                           cfg.sink, cfg.window, cfg.dtype, device=device)
    gen = torch.Generator(device=device).manual_seed(7)
    x = torch.randn((cfg.batch, hidden), generator=gen, device=device).to(synth.torch_dtype(cfg.dtype))
    out = {}

    def step():
        out["y"] = stack.step(x)

    per_stream = _time_loop(step, steps, warmup, world, device)
    per_graph = None
    try:  # all layers (projections, our kernels, the per-layer all-gather) captured once and replayed
        g = torch.cuda.CUDAGraph()
        cs = torch.cuda.Stream()
        cs.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cs):
            with torch.cuda.graph(g, stream=cs):
                step()
        torch.cuda.current_stream().wait_stream(cs)
        per_graph = _time_loop(g.replay, steps, warmup, world, device)
    except Exception as exc:
        print(f"# cfg2 graph capture skipped on rank {rank}: {exc}", file=sys.stderr)
    ok = torch.tensor([1.0 if per_graph else 0.0], device=device)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    per = per_graph if (per_graph and float(ok[0]) > 0) else per_stream
    for e in stack.engines:
        e.check_status()
    finite = bool(torch.isfinite(out["y"].float()).all())
    stack.close()
    return {"value": 1e3 / per, "ms_per_step": per, "ms_per_step_stream_launch": per_stream,
            "ms_per_step_cuda_graph": per_graph, "layers": n_layers, "hidden": hidden, "output_finite": finite,
            "algorithmic_bytes_per_step": n_layers * cfg.algorithmic_bytes(),
            "parallelism": f"kv-head sharded x{world}; one all-gather of the attention output per layer" if world > 1
            else "single GPU", "gpu_launches_per_step": 4 * n_layers}


def run_cfg4(cfg, device, steps, warmup, n_sub=16, n_cand=4096):
    """Configuration 4: product-quantised keys, ADC scan -> top-4096 candidates -> exact rerank -> top-2048
    -> sparse attention over the selected rows."""
    from diffcache_b200 import _lib, pq

    lib = _lib.load()
    P, n, D, G = cfg.n_prob, cfg.context, cfg.head_dim, cfg.group
    k, v = synth.make_kv(cfg.batch, cfg.kv_heads, n, D, 4000, cfg.dtype, device=device)
    q = synth.make_query(k, G, 4000).contiguous()
    kd, vd = k.view(P, n, D), v.view(P, n, D)
    book = torch.cat([pq.train_codebooks(kd[p:p + 4], n_sub=n_sub, iters=6, seed=11 + p, sample=16384)
                      for p in range(0, P, 4)])
    codes = pq.encode(kd, book, chunk=4096)
    ws = pq.PQWorkspace(P, n, n_sub, n_cand, cfg.topk, device)
    out = torch.empty_like(q)
    scratch = torch.zeros(int(lib.dc_attend_scratch_bytes(P, G, D)), dtype=torch.uint8, device=device)
    st = int(torch.cuda.current_stream().cuda_stream)

    def step():
        sel_idx, _ = pq.adc_rerank_topk(kd, codes, book, q, G, n_cand, cfg.topk, ws)
        _lib.check(lib.dc_sparse_attend(kd.data_ptr(), vd.data_ptr(), n * D, n, P, cfg.kv_heads, G, D, 0, q.data_ptr(),
                                        sel_idx.data_ptr(), cfg.topk, cfg.topk, 0, None, None, None, None, 0, 0, 0, 0.0,
                                        out.data_ptr(), None, None, None, scratch.data_ptr(), st))

    per = _time_loop(step, steps, warmup, 1, device)
    # recall of the PQ pipeline against the exact scan (informational: PQ is approximate by design)
    eng_bits = torch.empty((P, n), dtype=torch.int32, device=device)
    mm = torch.tensor([[-1, 0]] * P, dtype=torch.int32, device=device)
    _lib.check(lib.dc_score_scan(kd.data_ptr(), n * D, P, n, D, 0, q.data_ptr(), 1, G, eng_bits.data_ptr(), n,
                                 mm.data_ptr(), st))
    ex_idx = torch.empty((P, cfg.topk), dtype=torch.int32, device=device)
    _lib.check(lib.dc_topk_select(eng_bits.data_ptr(), None, n, P, n, cfg.topk, mm.data_ptr(), None, ex_idx.data_ptr(),
                                  cfg.topk, ws.status.data_ptr(), st))
    torch.cuda.synchronize()
    a, b = ws.sel_idx.cpu().numpy(), ex_idx.cpu().numpy()
    recall = float(np.mean([len(set(a[p]) & set(b[p])) / cfg.topk for p in range(P)]))
    alg = P * n * n_sub + P * n_sub * 256 * 4 + P * n_cand * D * 2 + 2 * P * cfg.topk * D * 2
    return {"value": 1e3 / per, "ms_per_step": per, "n_sub": n_sub, "n_candidates": n_cand,
            "recall_vs_exact_scan": recall, "algorithmic_bytes_per_step": alg,
            "aggregate_gbs": alg / (per * 1e-3) / 1e9, "gpu_launches_per_step": 8}


def run_other_workload(args, cfg, world, rank, device):
    if args.workload == "cfg0":
        res = run_cfg0(cfg, device, args.steps, args.warmup)
    elif args.workload == "cfg2_layer":
        res = run_cfg2(cfg, world, rank, device, args.steps, args.warmup, n_layers=args.layers)
    elif args.workload == "cfg4":
        res = run_cfg4(cfg, device, args.steps, args.warmup)
    else:
        res = run_seq_sharded(cfg, world, rank, device, args.steps, args.warmup)
    if rank == 0:
        peak, kind = measured_peaks()
        alg = res.get("algorithmic_bytes_per_step", cfg.algorithmic_bytes())
        gbs = alg / (res["ms_per_step"] * 1e-3) / 1e9
        line = {"metric": f"decode attention steps/sec ({cfg.name})", "value": res["value"], "unit": UNIT,
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
                "dtype": cfg.dtype, "data": "synthetic",
                "config": {"workload": f"{cfg.name}: batch {cfg.batch}, context {cfg.context}, top-k {cfg.topk} + "
                                       f"{cfg.sink} sink + {cfg.window} window"},
                "step_roofline": {"achieved": gbs, "unit": "GB/s", "frac_of_measured": gbs / (peak * world),
                                  "frac_of_8tbs_nominal": gbs / (8000.0 * world), "algorithmic_bytes_per_step": alg},
                "detail": res}
        print(json.dumps(line), flush=True)


def workload_config(cfg, n_gpus):
    return {
        "workload": f"{cfg.name}: batch {cfg.batch} x {cfg.q_heads}q/{cfg.kv_heads}kv heads x head_dim {cfg.head_dim}, "
                    f"context {cfg.context}, top-k {cfg.topk} + {cfg.sink} sink + {cfg.window} window, one layer",
        "per_gpu_batch": cfg.batch, "global_batch": cfg.batch * n_gpus, "context": cfg.context,
        "parallelism": f"independent batch replica per GPU x{n_gpus} (no data-path collective)",
        "l2_policy": "inputs (4.28 GB of keys scanned per step) are larger than L2; no flush needed",
        "algorithmic_bytes_per_step": cfg.algorithmic_bytes(),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=sorted(synth.CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=32, help="layers of the configuration-2 stack")
    ap.add_argument("--seq-sharded", action="store_true",
                    help="also time configuration 3 (1M-token sequence sharded by rows over the ranks) and report "
                         "it under the key seq_sharded_cfg3")
    ap.add_argument("--profile", action="store_true",
                    help="only the device-resident loop (for profiler captures): no e2e leg, no CPU baseline, "
                         "no clock sampling, warm-up taken as given")
    args = ap.parse_args()
    cfg = synth.CONFIGS[args.workload]
    if args.impl == "ours" and not args.profile:
        args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference(args, cfg)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the CUDA path has no CPU fallback")
    world, rank, local = dist_setup(args.gpus)
    device = torch.device("cuda", local if world > 1 else 0)
    if args.workload not in ("cfg1", "cfg1_b2"):
        run_other_workload(args, cfg, world, rank, device)
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
            dist.destroy_process_group()
        return
    eng, q, res_k, res_v, res_rows, k_new, v_new, host = build_step_inputs(cfg, 1000 + rank, device)
    out = torch.empty_like(q)
    idx = torch.zeros((cfg.batch, cfg.kv_heads, cfg.topk), dtype=torch.int32, device=device)

    def step():
        eng.decode_attend(q, out, cfg.topk, res_k=res_k, res_v=res_v, res_len=res_rows, k_new=k_new, v_new=v_new,
                          out_idx=idx)

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing (value) ----
    for _ in range(args.warmup):
        step()
    eng.check_status()
    sampler = ClockSampler(device.index)
    barrier()
    if rank == 0 and not args.profile:
        sampler.start()
        time.sleep(0.15)
    eng.set_phase_timing(args.steps)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    phases = eng.phase_times()
    eng.set_phase_timing(0)

    # ---- the same step replayed from a CUDA graph (no phase events, no launch gaps) ----
    graph_ms = None
    try:
        g = torch.cuda.CUDAGraph()
        cs = torch.cuda.Stream()
        cs.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cs):
            with torch.cuda.graph(g, stream=cs):
                step()
        torch.cuda.current_stream().wait_stream(cs)
        for _ in range(3):
            g.replay()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps):
            g.replay()
        g1.record()
        barrier()
        graph_ms = g0.elapsed_time(g1) / args.steps
    except Exception as exc:
        print(f"# CUDA graph replay skipped: {exc}", file=sys.stderr)

    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": cfg.name, "ms_per_step": elapsed_ms / args.steps,
                              "graph_ms_per_step": graph_ms, "phases": phases}), flush=True)
        eng.close()
        return

    # ---- end to end through the public API with host buffers (e2e) ----
    # q, k_new and v_new of a step leave the host as ONE packed pinned buffer (the layout a fused qkv
    # projection produces) and land in one device buffer; the three tensors are views into it
    nq, nk = q.numel(), k_new.numel()
    in_h = torch.cat([q.reshape(-1), k_new.reshape(-1), v_new.reshape(-1)]).cpu().pin_memory()
    in_d = torch.empty_like(in_h, device=device)
    q_d = in_d[:nq].view_as(q)
    kn_d, vn_d = in_d[nq:nq + nk].view_as(k_new), in_d[nq + nk:].view_as(v_new)
    out_h = torch.empty_like(q, device="cpu").pin_memory()

    def e2e_step():
        in_d.copy_(in_h, non_blocking=True)
        eng.decode_attend(q_d, out, cfg.topk, res_k=res_k, res_v=res_v, res_len=res_rows, k_new=kn_d, v_new=vn_d)
        out_h.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller consumes the result of every step

    for _ in range(3):
        e2e_step()
    barrier()
    # the same call sequence (copies in, step, copy out) captured once; each step still ends with the
    # host waiting for its result
    e2e_call = e2e_step
    try:
        ge = torch.cuda.CUDAGraph()
        es = torch.cuda.Stream()
        es.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(es):
            with torch.cuda.graph(ge, stream=es):
                in_d.copy_(in_h, non_blocking=True)
                eng.decode_attend(q_d, out, cfg.topk, res_k=res_k, res_v=res_v, res_len=res_rows, k_new=kn_d, v_new=vn_d)
                out_h.copy_(out, non_blocking=True)
        torch.cuda.current_stream().wait_stream(es)

        def e2e_graph_step():
            ge.replay()
            torch.cuda.current_stream().synchronize()

        for _ in range(3):
            e2e_graph_step()
        e2e_call = e2e_graph_step
    except Exception as exc:
        print(f"# e2e graph capture skipped: {exc}", file=sys.stderr)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_call()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None
    eng.check_status()

    # ---- max over ranks ----
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        peak, peak_kind = measured_peaks()
        stream_ms = elapsed_ms / args.steps
        # headline = the step replayed from a CUDA graph (how the reference drives its decode layers,
        # src/diffcache/base.py:116-155); the stream-launch loop with phase events is kept beside it
        ms_per_step = graph_ms if graph_ms else stream_ms
        value = world * 1e3 / ms_per_step
        scan_ms = phases["scan_ms"] / max(1, phases["steps"])
        scan_gbs = cfg.scan_bytes() / (scan_ms * 1e-3) / 1e9 if scan_ms > 0 else 0.0
        step_gbs = cfg.algorithmic_bytes() / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": cfg.dtype, "data": "synthetic", "config": workload_config(cfg, world),
            "roofline": {
                "bound": "hbm", "kernel": "score_scan_wide_kernel", "achieved": scan_gbs, "peak": peak, "unit": "GB/s",
                "frac": scan_gbs / peak, "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})",
                "frac_of_8tbs_nominal": scan_gbs / 8000.0,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch: ncu capture of the 2-sequence case
                # (534.55 MB + 9.54 MB, profiles/score_scan_cfg1_b2.md) scaled by the 8x rows of this workload
                "traffic": int(8 * (534.55e6 + 9.54e6)) if cfg.name == "cfg1" else None,
                "algorithmic_bytes_per_launch": cfg.scan_bytes(), "avg_launch_ms": scan_ms,
            },
            "step_roofline": {"achieved": step_gbs, "frac_of_measured": step_gbs / peak,
                              "frac_of_8tbs_nominal": step_gbs / 8000.0, "unit": "GB/s",
                              "algorithmic_bytes_per_step": cfg.algorithmic_bytes()},
            "phases_ms": {"scan": scan_ms, "select": phases["select_ms"] / max(1, phases["steps"]),
                          "attend": phases["attend_ms"] / max(1, phases["steps"])},
            "e2e": {"value": world * args.steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": int(in_h.numel() * 2),
                    "d2h_bytes_per_step": int(out_h.numel() * 2), "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": 4 * args.steps,
            "timing": {"headline": "cuda_graph_replay" if graph_ms else "stream_launch",
                       "cuda_graph_replay_ms_per_step": graph_ms, "stream_launch_ms_per_step": stream_ms},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            base, _ = cpu_reference_step_rate(cfg, host["k"], host["v"], q, budget_s=15.0, max_steps=20, sample_batch=2)
            line["cpu_baseline"] = base
    else:
        line = None
    eng.close()
    del host, eng, res_k, res_v
    torch.cuda.empty_cache()
    if args.seq_sharded:
        seq = run_seq_sharded(synth.CONFIGS["cfg3"], world, rank, device, args.steps, args.warmup)
        if rank == 0:
            line["seq_sharded_cfg3"] = seq
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
