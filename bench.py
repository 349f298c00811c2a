"""Benchmark of the ragged paged-attention step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2] [--impl ours|reference]

A step is one pass of the hot path over one packed batch: batch metadata + paged KV write of
the step's new rows + attention.  The default workload is c2 (Llama-3-8B-shaped decode, 64
sequences, 8-bit affine KV); see easymlx_b200/workloads.py for the five configurations.
Under torchrun every rank owns its own sequences and page pool (partition by sequence, no
collective; c4 alone shards KV heads and all-gathers the output), the timed region is
bracketed by barriers and the maximum over ranks is reported.  Prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "attended_kv_tokens_per_s"
UNIT = "tokens/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    source="measured (MEASURED_PEAKS.json)")
    return dict(hbm_gbs=6650.0, bf16_tflops=1400.0, source="fallback (6.65 TB/s, 1.4 PFLOP/s sustained)")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            text, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            text = ""
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in text.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            self.summary = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)),
                            "reasons": sorted(reasons), "samples": len(sm)}


def _dist():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


# ----------------------------------------------------------------------------- CPU arm

def _pick_sample(w, budget_tokens):
    order = np.argsort(w.kv_lens, kind="stable")
    picked, total = [], 0
    for s in order[::max(1, len(order) // 8)]:
        if total and total + w.kv_lens[s] * max(1, w.qlens[s]) > budget_tokens:
            continue
        picked.append(int(s)); total += int(w.kv_lens[s] * max(1, w.qlens[s]))
    return np.asarray(sorted(picked or [int(order[0])]), dtype=np.int64)


def _cpu_pool_for(w, seqs, seed):
    """NumPy-built pool holding only the sampled sequences (same distributions as the GPU workload)."""
    from oracle import kv_quant

    rng = np.random.default_rng(seed)
    kv = w.kv_lens.astype(np.int32)
    n_pages = int(sum(-(-int(kv[s]) // 128) for s in seqs))
    bt = -np.ones((len(kv), int(max(1, (-(-kv // 128)).max()))), dtype=np.int32)
    cursor = 0
    for s in seqs:
        n = -(-int(kv[s]) // 128)
        bt[s, :n] = np.arange(cursor, cursor + n)
        cursor += n
    shape = (n_pages, 128, w.hkv, w.d)
    kc = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
    vc = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
    host = dict(block_tables=bt, kv_lens=kv,
                query_start_loc=np.concatenate([[0], np.cumsum(w.qlens)]).astype(np.int32))
    if w.bits:
        kcodes, ks, kb = kv_quant.quantize_rows(kc, w.bits)
        vcodes, vs, vb = kv_quant.quantize_rows(vc, w.bits)
        host.update(key_cache=kv_quant.pack_codes(kcodes, w.bits),
                    value_cache=kv_quant.pack_codes(np.ascontiguousarray(np.transpose(vcodes, (0, 2, 3, 1))), w.bits),
                    k_scale=np.ascontiguousarray(np.transpose(ks, (0, 2, 1, 3))),
                    k_bias=np.ascontiguousarray(np.transpose(kb, (0, 2, 1, 3))),
                    v_scale=np.ascontiguousarray(np.transpose(vs, (0, 2, 1, 3))),
                    v_bias=np.ascontiguousarray(np.transpose(vb, (0, 2, 1, 3))))
    else:
        host.update(key_cache=kc, value_cache=vc)
    q = rng.standard_normal((w.total_tokens, w.hq, w.d), dtype=np.float32).astype(np.float16)
    return host, q


_FORK_STATE = {}


def _fork_worker(seq):
    w, host, q = _FORK_STATE["w"], _FORK_STATE["host"], _FORK_STATE["q"]
    from oracle import kv_quant, paged_attention as opa

    kv = int(host["kv_lens"][seq])
    pages = host["block_tables"][seq, : -(-kv // 128)]
    sub = dict(host)
    # one sequence: gather (and dequantise) only its pages, as the reference's per-sequence loop does
    kc, vc = host["key_cache"][pages], host["value_cache"][pages]
    if w.bits:
        kc = kv_quant.dequantize_key_pool(kc, host["k_scale"][pages], host["k_bias"][pages], w.bits)
        vc = kv_quant.dequantize_value_pool(vc, host["v_scale"][pages], host["v_bias"][pages], w.bits)
    bt = -np.ones_like(host["block_tables"])
    bt[seq, : len(pages)] = np.arange(len(pages))
    sub.update(key_cache=kc, value_cache=vc, block_tables=bt)
    opa.paged_attention_rows(q, kc, vc, bt, host["kv_lens"], host["query_start_loc"], softmax_scale=w.d ** -0.5,
                             seq_subset=[seq])
    return kv


def run_reference(args):
    """The reference's CPU algorithm for this op (its NumPy path, restated in oracle/) on the host cores.
    The reference project itself cannot run here: it needs Apple's MLX, which has no Linux/py3.12 wheel."""
    world, rank, _ = _dist()
    if rank != 0:
        return
    import multiprocessing as mp

    from easymlx_b200 import workloads

    os.environ.setdefault("OMP_NUM_THREADS", "1")
    w = workloads.describe(args.config)
    cores = len(os.sched_getaffinity(0))
    seqs = _pick_sample(w, budget_tokens=args.cpu_budget_tokens * max(1, cores // 2))
    host, q = _cpu_pool_for(w, seqs, seed=1234)
    _FORK_STATE.update(w=w, host=host, q=q)
    ctx = mp.get_context("fork")
    times = []
    with ctx.Pool(min(cores, len(seqs))) as pool:
        budget_s, t_start = 150.0, time.perf_counter()
        for it in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            tokens = sum(pool.map(_fork_worker, [int(s) for s in seqs], chunksize=1))
            dt = time.perf_counter() - t0
            if it >= args.warmup:
                times.append(dt)
            if time.perf_counter() - t_start > budget_s and len(times) >= 1:
                break
    per_step = float(np.mean(times))
    value = tokens / per_step
    sample = (f"{len(seqs)} of {len(w.qlens)} sequences of {args.config} ({tokens} attended KV tokens per step), "
              f"{len(times)} timed steps, sequences spread over a fork pool")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times),
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.config}: {w.description}", "note": "reference algorithm on host cores; "
                   + ("affine KV has no reference path: oracle dequantise-then-attend" if w.bits else "fp16 KV")},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": min(cores, len(seqs)), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _cpu_baseline_single_core(w, config, budget_tokens):
    """The oracle on one core over a bounded sample of the same workload (rank 0, N=1 only)."""
    seqs = _pick_sample(w, budget_tokens=budget_tokens)
    host, q = _cpu_pool_for(w, seqs, seed=4321)
    _FORK_STATE.update(w=w, host=host, q=q)
    _fork_worker(int(seqs[0]))  # warm-up
    t0 = time.perf_counter()
    tokens, passes = 0, 0
    while True:  # whole passes over the sample until about ten seconds of CPU work
        tokens += sum(_fork_worker(int(s)) for s in seqs)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= 10.0 or passes >= 50:
            break
    return {"value": tokens / dt, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"{len(seqs)} of {len(w.qlens)} sequences of {config}, {passes} passes ({tokens} attended KV tokens), "
                      f"{dt:.1f} s of NumPy oracle (dequantise + attend), BLAS threads pinned to 1"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    import easymlx_b200 as emlx
    from easymlx_b200 import _native as nv, workloads
    from easymlx_b200.runtime import AttentionStep

    world, rank, local = _dist()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    base = workloads.describe(args.config)
    head_shard = args.config == "c4" and world > 1 and base.hkv % world == 0
    if head_shard:
        per = base.hkv // world
        w = workloads.materialize(base, dev, seed=0, kv_head_slice=slice(rank * per, (rank + 1) * per))
    else:
        # weak scaling: the global batch is `world` draws of the configuration (different lengths per draw), partitioned
        # by sequence, longest first, so that every rank attends about the same number of KV tokens; every rank owns
        # the page pool of its own sequences
        if world == 1:
            w = workloads.materialize(base, dev, seed=0)
        else:
            draws = [workloads.describe(args.config, seed=None if r == 0 else 1000 * r + 7) for r in range(world)]
            whole = workloads.describe(args.config)
            whole.qlens = np.concatenate([d.qlens for d in draws])
            whole.prior = np.concatenate([d.prior for d in draws])
            mine = workloads.partition_by_sequence(whole, world)[rank]
            w = workloads.materialize(whole, dev, seed=rank, seq_subset=mine)
    if args.attn_only:
        # profiling aid: a few bare attention launches over the written pool, nothing else
        from easymlx_b200.operations.kernels.unified_attention import AttentionCall

        c = w.cache
        extra = dict(k_scale=c.k_scales, v_scale=c.v_scales, k_bias=c.k_biases, v_bias=c.v_biases) if w.bits else {}
        call = AttentionCall(w.q, c.key_cache, c.value_cache, c.block_tables,
                             torch.from_numpy(w.kv_lens.astype(np.int32)).to(dev),
                             emlx.build_query_start_loc(w.qlens.tolist(), device=dev),
                             max_query_len=int(w.qlens.max()), **extra).plan()
        for _ in range(args.attn_only):
            call.launch()
        torch.cuda.synchronize()
        print(json.dumps({"attn_only": args.attn_only, "config": args.config}))
        return
    step = AttentionStep(w.cache, w.q, w.k, w.v, w.qlens.tolist(), w.slot_ids)
    gathered = None
    if head_shard:
        gathered = torch.empty((world,) + tuple(w.q.shape), dtype=w.q.dtype, device=dev)

    def one_step():
        out = step.step()
        if head_shard:
            dist.all_gather_into_tensor(gathered.view(-1, *out.shape[1:]), out)
        return out

    for _ in range(2):
        step._eager()
    torch.cuda.synchronize()
    layers = 1 if args.no_graph else max(1, args.layers_per_graph)
    if args.steps % layers:
        layers = 1
    if not args.no_graph:
        step.capture(warmup=2, steps_per_graph=layers)
    for _ in range(max(3, args.warmup)):
        one_step()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        barrier()
        ms = start.elapsed_time(stop)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # ---- device-resident steps
    with ClockSampler(local) as clocks:
        ms_total = timed(one_step, args.steps // layers)
        # the timed region lasts a few milliseconds, shorter than nvidia-smi's sampling period: the same step keeps
        # replaying (untimed) for about half a second so that the clock record holds several samples under this load
        t_end = time.perf_counter() + 0.5
        while time.perf_counter() < t_end:
            for _ in range(20):
                one_step()
            torch.cuda.synchronize()
    ms_step = ms_total / args.steps
    tokens_rank = torch.tensor([float(w.attended_kv_tokens)], device=dev)
    if world > 1 and not head_shard:
        dist.all_reduce(tokens_rank)
    tokens_all = float(tokens_rank.item())
    value = tokens_all / (ms_step * 1e-3)

    # ---- end to end: pinned host q/k/v in, host output back, every step
    # q, k and v travel as one packed host buffer (one copy per step instead of three); the device side of the
    # end-to-end step reads them through views of the packed device buffer
    parts = (w.q, w.k, w.v)
    sizes = [t.numel() for t in parts]
    hqkv = torch.cat([t.reshape(-1).cpu() for t in parts]).pin_memory()
    dqkv = torch.empty_like(hqkv, device=dev)
    dqkv.copy_(hqkv)
    dq, dk, dv = (v.view(t.shape) for v, t in zip(torch.split(dqkv, sizes), parts))
    hout = torch.empty_like(w.q, device="cpu").pin_memory()

    # the end-to-end loop copies inputs and output every single step: one step per graph
    step1 = AttentionStep(w.cache, dq, dk, dv, w.qlens.tolist(), w.slot_ids).capture(warmup=2)

    def e2e_step():
        dqkv.copy_(hqkv, non_blocking=True)
        out = step1.step()
        if head_shard:
            dist.all_gather_into_tensor(gathered.view(-1, *out.shape[1:]), out)
        hout.copy_(gathered[rank] if head_shard else out, non_blocking=True)

    for _ in range(3):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps) / args.steps
    h2d = hqkv.numel() * hqkv.element_size()
    d2h = hout.numel() * hout.element_size()

    # ---- the dominant kernel alone (attention over the already written pool), for the roofline
    meta_lens = torch.from_numpy(w.kv_lens.astype(np.int32)).to(dev)
    qsl = emlx.build_query_start_loc(w.qlens.tolist(), device=dev)
    extra = {}
    if w.bits:
        c = w.cache
        extra = dict(k_scale=c.k_scales, v_scale=c.v_scales, k_bias=c.k_biases, v_bias=c.v_biases)
    from easymlx_b200.operations.kernels.unified_attention import AttentionCall

    call = AttentionCall(w.q, w.cache.key_cache, w.cache.value_cache, w.cache.block_tables, meta_lens, qsl,
                         max_query_len=int(w.qlens.max()), query_len_set=sorted(set(int(x) for x in w.qlens if x > 0)), **extra)
    call.plan()
    call.launch()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    reps = 10  # launches per graph, so that the gap between graph launches does not count as kernel time
    with torch.cuda.graph(g):
        for _ in range(reps):
            call.launch()
    for _ in range(3):
        g.replay()
    n_replays = max(1, args.steps // reps)
    ms_attn = timed(g.replay, n_replays) / (n_replays * reps)

    peaks = _peaks()
    attn_bytes = w.attention_bytes()
    achieved = attn_bytes / (ms_attn * 1e-3) / 1e9
    line = None
    if rank == 0:
        traffic = None
        tpath = os.path.join(ROOT, "profiles", f"traffic_{args.config}.json")
        if os.path.exists(tpath) and not head_shard:  # captured on one GPU holding every KV head
            traffic = json.load(open(tpath)).get("dram_bytes_per_launch")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_step, "us_per_batch": ms_step * 1e3, "higher_is_better": True,
            "scaling": "strong" if head_shard else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {
                "workload": f"{args.config}: {base.description}",
                "kv_format": {0: "fp16", 8: "affine8 group-64", 4: "affine4 group-64"}[w.bits],
                "step": (f"batch metadata + work list + paged KV write + attention; {layers} consecutive steps per CUDA "
                         "graph, as an engine step holds one per layer") if not args.no_graph
                        else "batch metadata + work list + paged KV write + attention, eager launches",
                "parallelism": ("kv-head shard + NCCL all-gather" if head_shard else f"sequence partition x{world}"),
                "l2": "per-step KV working set exceeds L2 (no flush needed)" if attn_bytes > 3 * 126e6
                      else "working set smaller than L2: numbers are L2-assisted",
                "sequences_per_gpu": int(len(w.qlens)), "tokens_per_gpu": int(w.total_tokens),
                "attended_kv_tokens_per_gpu": int(w.attended_kv_tokens),
            },
            "clocks": dict(clocks.summary, window="timed steps + 0.5 s of the same step replayed"),
            "e2e": {"value": tokens_all / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "us_per_batch": ms_e2e * 1e3},
            "gpu_launches": int(step.launches_per_step * args.steps),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "frac_of_8TBs_nominal": achieved / 8000.0,
                         "traffic": traffic, "kernel": "attention (all launches of emlx_attn_unified)",
                         "algorithmic_bytes_per_launch": int(attn_bytes), "us_per_launch": ms_attn * 1e3,
                         "peak_source": peaks["source"]},
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = _cpu_baseline_single_core(base, args.config, args.cpu_budget_tokens)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--layers-per-graph", type=int, default=10)
    ap.add_argument("--attn-only", type=int, default=0, help="run this many bare attention launches and exit (for ncu)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-budget-tokens", type=int, default=120000)
    args = ap.parse_args()
    os.environ.setdefault("OMP_NUM_THREADS", "1")
    os.environ.setdefault("OPENBLAS_NUM_THREADS", "1")
    os.environ.setdefault("MKL_NUM_THREADS", "1")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
