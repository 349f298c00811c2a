"""Benchmark of the ragged paged-attention step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2] [--impl ours|reference]

A step is one pass of the hot path over one packed batch: batch metadata + paged KV write of
the step's new rows + attention.  The headline workload is c2 (Llama-3-8B-shaped decode, 64
sequences, 8-bit affine KV); the same JSON line carries all five configurations of
easymlx_b200/workloads.py under "configs" (one GPU), and under torchrun the strong-scaling runs
of c3 / c5 (the same global batch partitioned by sequence) and c4 sharded by KV head with its
NCCL all-gather.  Under torchrun every rank owns its own sequences and page pool (no collective
on the data path except c4's all-gather), every timed region is bracketed by barriers and the
maximum over ranks is reported.  Prints one JSON line.
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
ALL_CONFIGS = ("c1", "c2", "c3", "c4", "c5")
BAD_CLOCK_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    bf16_tflops_burst=float(p["bf16_tflops"]), source="measured (MEASURED_PEAKS.json)")
    return dict(hbm_gbs=6650.0, bf16_tflops=1400.0, bf16_tflops_burst=1590.0,
                source="fallback (6.65 TB/s, 1.4 PFLOP/s sustained)")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
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


def _kv_format(bits):
    return {0: "fp16", 8: "affine8 group-64", 4: "affine4 group-64"}[bits]


def headline_config(name, world, layers):
    """The `config` object of the JSON line; both arms print the same one for the same command line."""
    from easymlx_b200 import workloads

    base = workloads.describe(name)
    return {
        "workload": f"{name}: {base.description}",
        "kv_format": _kv_format(base.bits),
        "step": (f"batch metadata + work list + paged KV write + attention; {layers} consecutive steps per CUDA "
                 "graph, as an engine step holds one per layer"),
        "parallelism": f"sequence partition x{world}" + (" (each rank one draw of the configuration)" if world > 1 else ""),
        "l2": "per-step KV working set exceeds L2 (no flush needed)",
        "sequences_per_gpu": int(len(base.qlens)), "tokens_per_gpu": int(base.total_tokens),
        "attended_kv_tokens_per_gpu": int(base.attended_kv_tokens),
    }


# ----------------------------------------------------------------------------- CPU arm

def _cpu_pool_for(w, seqs, seed):
    """NumPy-built pool holding only the listed sequences (same distributions as the GPU workload)."""
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
    host = dict(block_tables=bt, kv_lens=kv,
                query_start_loc=np.concatenate([[0], np.cumsum(w.qlens)]).astype(np.int32))
    parts = {}
    for p0 in range(0, n_pages, 128):  # in pieces, so that the fp32 temporaries of the quantiser stay small
        shape = (min(128, n_pages - p0), 128, w.hkv, w.d)
        kc = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
        vc = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
        if w.bits:
            kcodes, ks, kb = kv_quant.quantize_rows(kc, w.bits)
            vcodes, vs, vb = kv_quant.quantize_rows(vc, w.bits)
            piece = dict(key_cache=kv_quant.pack_codes(kcodes, w.bits),
                         value_cache=kv_quant.pack_codes(np.ascontiguousarray(np.transpose(vcodes, (0, 2, 3, 1))), w.bits),
                         k_scale=np.transpose(ks, (0, 2, 1, 3)), k_bias=np.transpose(kb, (0, 2, 1, 3)),
                         v_scale=np.transpose(vs, (0, 2, 1, 3)), v_bias=np.transpose(vb, (0, 2, 1, 3)))
        else:
            piece = dict(key_cache=kc, value_cache=vc)
        for name, a in piece.items():
            parts.setdefault(name, []).append(np.ascontiguousarray(a))
    host.update({name: np.concatenate(chunks) for name, chunks in parts.items()})
    q = rng.standard_normal((w.total_tokens, w.hq, w.d), dtype=np.float32).astype(np.float16)
    return host, q


_FORK_STATE = {}


def _fork_worker(seq):
    w, host, q = _FORK_STATE["w"], _FORK_STATE["host"], _FORK_STATE["q"]
    from oracle import kv_quant, paged_attention as opa

    kv = int(host["kv_lens"][seq])
    pages = host["block_tables"][seq, : -(-kv // 128)]
    # one sequence: gather (and dequantise) only its pages, as the reference's per-sequence loop does
    kc, vc = host["key_cache"][pages], host["value_cache"][pages]
    if w.bits:
        kc = kv_quant.dequantize_key_pool(kc, host["k_scale"][pages], host["k_bias"][pages], w.bits)
        vc = kv_quant.dequantize_value_pool(vc, host["v_scale"][pages], host["v_bias"][pages], w.bits)
    bt = -np.ones_like(host["block_tables"])
    bt[seq, : len(pages)] = np.arange(len(pages))
    opa.paged_attention_rows(q, kc, vc, bt, host["kv_lens"], host["query_start_loc"], softmax_scale=w.d ** -0.5,
                             seq_subset=[seq])
    return kv


def run_reference(args):
    """The reference's CPU algorithm for this op (its NumPy path, restated in oracle/) on the host cores, over the
    whole batch of the configuration (one draw of it when the GPU arm runs several).  The reference project itself
    cannot run on the measurement box: it needs Apple's MLX (no Linux wheel) and its sources do not travel."""
    world, rank, _ = _dist()
    if rank != 0:
        return
    import multiprocessing as mp

    from easymlx_b200 import workloads

    os.environ.setdefault("OMP_NUM_THREADS", "1")
    w = workloads.describe(args.config)
    cores = len(os.sched_getaffinity(0))
    # longest first, so that the pool's workers finish together
    seqs = np.argsort(-(w.kv_lens * np.maximum(w.qlens, 1)), kind="stable")
    host, q = _cpu_pool_for(w, seqs, seed=1234)
    _FORK_STATE.update(w=w, host=host, q=q)
    ctx = mp.get_context("fork")
    times = []
    with ctx.Pool(min(cores, len(seqs))) as pool:
        budget_s, t_start = 240.0, time.perf_counter()
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
    layers = _layers_per_graph(args)
    sample = (f"all {len(seqs)} sequences of one draw of {args.config} ({tokens} attended KV tokens per step), "
              f"{len(times)} timed steps, sequences spread over a fork pool of {min(cores, len(seqs))} processes; "
              + ("affine KV has no path in the reference: the oracle dequantises, then attends with the reference's "
                 "NumPy algorithm" if w.bits else "fp16 KV, the reference's NumPy algorithm"))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times),
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(args.config, world, layers),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": min(cores, len(seqs)), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _cpu_baseline_single_core(w, config, budget_tokens):
    """The oracle on one core over a bounded sample of the same workload (rank 0, N=1 only)."""
    order = np.argsort(w.kv_lens, kind="stable")
    picked, total = [], 0
    for s in order[::max(1, len(order) // 8)]:
        if total and total + w.kv_lens[s] * max(1, w.qlens[s]) > budget_tokens:
            continue
        picked.append(int(s)); total += int(w.kv_lens[s] * max(1, w.qlens[s]))
    seqs = np.asarray(sorted(picked or [int(order[0])]), dtype=np.int64)
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


# ----------------------------------------------------------------------------- GPU arm

def _layers_per_graph(args):
    layers = 1 if args.no_graph else max(1, args.layers_per_graph)
    return 1 if args.steps % layers else layers


class Bench:
    """Timing helpers bound to one rank."""

    def __init__(self, args, dev, world, rank, local):
        import torch

        self.torch, self.args, self.dev = torch, args, dev
        self.world, self.rank, self.local = world, rank, local
        self.peaks = _peaks()

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, steps, finish=None):
        """Milliseconds for `steps` calls of fn: CUDA events on the launching stream, barrier + synchronise on both
        sides, maximum over ranks.  `finish()` runs before the closing event (work on other streams joins there)."""
        torch = self.torch
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        start.record()
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()
        stop.record()
        self.barrier()
        ms = start.elapsed_time(stop)
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([ms], device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def graph_time(self, launch, reps, steps):
        """Average milliseconds of one `launch` replayed from a CUDA graph that holds `reps` of them."""
        torch = self.torch
        launch()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                launch()
        for _ in range(3):
            g.replay()
        n = max(1, steps // reps)
        return self.timed(g.replay, n) / (n * reps)

    def all_sum(self, x):
        if self.world == 1:
            return float(x)
        import torch.distributed as dist
        t = self.torch.tensor([float(x)], device=self.dev, dtype=self.torch.float64)
        dist.all_reduce(t)
        return float(t.item())

    # ------------------------------------------------------------------ one workload on this rank
    def measure(self, w, label, *, after_step=None, gather_target=None, parts=True, e2e=True):
        """Step time (device-resident), end-to-end step time and the attention launch alone for workload `w`.
        `after_step(out)` runs after every step (the KV-head shard's NCCL all-gather; one step per graph then, so that
        every step pays for its collective); `gather_target` makes the attention kernels store their heads into every
        rank's output instead (the step's output is then the gathered one)."""
        import easymlx_b200 as emlx
        from easymlx_b200 import _native as nv
        from easymlx_b200.operations.kernels.unified_attention import AttentionCall
        from easymlx_b200.runtime import AttentionStep

        torch, args, dev = self.torch, self.args, self.dev
        layers = 1 if after_step is not None else _layers_per_graph(args)
        step = AttentionStep(w.cache, w.q, w.k, w.v, w.qlens.tolist(), w.slot_ids, gather=gather_target)

        def one_step():
            out = step.step()
            if after_step is not None:
                after_step(out)
            return out

        for _ in range(2):
            step._eager()
        torch.cuda.synchronize()
        if not args.no_graph:
            step.capture(warmup=2, steps_per_graph=layers)
        if gather_target is not None:
            self.barrier()  # ranks wait for one another inside these kernels: start the replays together
        for _ in range(max(3, args.warmup)):
            one_step()
        torch.cuda.synchronize()

        ms_total, clocks = None, None
        for attempt in range(2):  # a run that saw a thermal / hardware slowdown is taken again, once
            with ClockSampler(self.local) as sampler:
                ms_total = self.timed(one_step, args.steps // layers)
                # the timed region lasts a few milliseconds, shorter than nvidia-smi's sampling period: the same step
                # keeps replaying (untimed) for a moment so that the clock record holds samples under this load
                # (a count, not a deadline: `ms_total` is the maximum over ranks, so every rank replays the same number
                # of steps, which steps that hold a collective or wait for the other ranks need)
                for _ in range(int(min(400, max(1, 500.0 / max(ms_total, 1e-3) * (args.steps // layers) / 20)))):
                    for _ in range(20):
                        one_step()
                    torch.cuda.synchronize()
            clocks = dict(sampler.summary, window="timed steps + 0.5 s of the same step replayed", attempts=attempt + 1)
            if not any(r in BAD_CLOCK_REASONS for r in clocks["reasons"]):
                break
        ms_step = ms_total / args.steps
        sharded = after_step is not None or gather_target is not None   # every rank works on the same batch
        tokens_all = float(w.attended_kv_tokens) if sharded else self.all_sum(w.attended_kv_tokens)
        result = {
            "label": label, "kv_format": _kv_format(w.bits), "us_per_batch": ms_step * 1e3,
            "value": tokens_all / (ms_step * 1e-3), "unit": UNIT,
            "attended_kv_tokens": int(tokens_all), "sequences_this_rank": int(len(w.qlens)),
            "tokens_this_rank": int(w.total_tokens), "gpu_launches_per_step": int(step.launches_per_step),
            "clocks": clocks,
        }

        # ---- end to end through the public host-facing call: pinned host q/k/v in, host output back, every step (one
        # packed upload per step); the upload of the next step and the download of the previous one run on their own
        # streams beside the kernels (HostStepPipeline), and the closing event waits for the last download
        if e2e:
            from easymlx_b200.runtime import HostStepPipeline
            # (a gathering call writes the one output buffer the ranks share: its steps cannot overlap their downloads)
            pipe = HostStepPipeline(w.cache, (w.q.cpu(), w.k.cpu(), w.v.cpu()), w.qlens.tolist(), w.slot_ids,
                                    depth=1 if gather_target is not None else 2, gather=gather_target, after_step=after_step)
            if gather_target is not None:
                self.barrier()
            for _ in range(4):
                pipe.submit()
            pipe.drain()
            ms_e2e = self.timed(pipe.submit, args.steps, finish=pipe.drain) / args.steps
            result["e2e"] = {"value": tokens_all / (ms_e2e * 1e-3), "unit": UNIT,
                             "h2d_bytes_per_step": pipe.h2d_bytes_per_step, "d2h_bytes_per_step": pipe.d2h_bytes_per_step,
                             "us_per_batch": ms_e2e * 1e3,
                             "overlap": "upload of step n+1 and download of step n-1 run beside the kernels of step n "
                                        "(two buffer sets, one stream per direction)"}
            del pipe

        # ---- the attention launch alone (over the already written pool), for the roofline
        c = w.cache
        lens_dev = torch.from_numpy(w.kv_lens.astype(np.int32)).to(dev)
        qsl = emlx.build_query_start_loc(w.qlens.tolist(), device=dev)
        extra = dict(k_scale=c.k_scales, v_scale=c.v_scales, k_bias=c.k_biases, v_bias=c.v_biases) if w.bits else {}
        lens_set = sorted(set(int(x) for x in w.qlens if x > 0))

        long_seqs = int((w.qlens * (w.hq // w.hkv) > 16).sum()) if w.bits else 0  # affine pools: rows for the tcgen05 route

        def attention_call(len_set):
            return AttentionCall(w.q, c.key_cache, c.value_cache, c.block_tables, lens_dev, qsl,
                                 max_query_len=int(w.qlens.max()), query_len_set=len_set, long_seqs=long_seqs, **extra).plan()

        call = attention_call(lens_set)
        ms_attn = self.graph_time(call.launch, 10, args.steps)
        attn_bytes = w.attention_bytes()
        achieved = attn_bytes / (ms_attn * 1e-3) / 1e9
        hbm = self.peaks["hbm_gbs"]
        roof = {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                "frac_of_8TBs_nominal": achieved / 8000.0, "kernel": "attention (all launches of emlx_attn_unified)",
                "algorithmic_bytes_per_launch": int(attn_bytes), "us_per_launch": ms_attn * 1e3,
                "peak_source": self.peaks["source"],
                "l2": "KV working set exceeds L2" if attn_bytes > 3 * 126e6 else
                      "working set comparable to the 126 MB L2: the figure is L2-assisted"}
        result["step_frac_of_hbm_peak"] = attn_bytes / (ms_step * 1e-3) / 1e9 / hbm
        result["roofline"] = roof

        # ---- mixed batches: the prefill-chunk launch (tensor-bound) and the short-row launches (HBM-bound) alone
        lib = nv.lib()
        fmt = w.bits if w.bits else nv.KV_FLOAT
        cls_of = {q: int(lib.emlx_attn_row_class(fmt, w.hq, w.hkv, w.d, q)) for q in lens_set}
        long_lens = [q for q in lens_set if cls_of[q] == 3]
        short_lens = [q for q in lens_set if cls_of[q] != 3]
        if parts and long_lens and self.world == 1:  # (ranks may hold different row classes: no collective timing here)
            is_long = np.isin(w.qlens, long_lens)
            flops = 4 * w.hq * w.d * int(sum(int(q) * int(p) + int(q) * (int(q) + 1) // 2
                                             for q, p in zip(w.qlens[is_long], w.prior[is_long])))
            ms_pf = self.graph_time(attention_call(long_lens).launch, 5, args.steps)
            tf = flops / (ms_pf * 1e-3) / 1e12
            roof["tensor"] = {"kernel": "attn_prefill_kernel (128-row units, tcgen05), timed alone", "flops": int(flops),
                              "us_per_launch": ms_pf * 1e3, "achieved_tflops": tf,
                              "peak_sustained_tflops": self.peaks["bf16_tflops"],
                              "frac_of_sustained": tf / self.peaks["bf16_tflops"],
                              "frac_of_burst": tf / self.peaks["bf16_tflops_burst"]}
            if short_lens:
                ms_dec = self.graph_time(attention_call(short_lens).launch, 5, args.steps)
                kv_short = int(w.kv_lens[~is_long].sum()) * 2 * w.hkv * w.row_bytes()
                roof["decode_part"] = {"kernel": "short-row launches timed alone", "us_per_launch": ms_dec * 1e3,
                                       "kv_bytes": kv_short, "achieved_gbs": kv_short / (ms_dec * 1e-3) / 1e9,
                                       "frac": kv_short / (ms_dec * 1e-3) / 1e9 / hbm}
                roof["bound_of_the_whole_launch_us"] = max(attn_bytes / hbm / 1e3, flops / self.peaks["bf16_tflops"] / 1e6)
        del step
        return result


def run_ours(args):
    import torch
    import torch.distributed as dist

    from easymlx_b200 import workloads
    from easymlx_b200.distributed import all_gather_heads

    world, rank, local = _dist()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    bench = Bench(args, dev, world, rank, local)
    layers = _layers_per_graph(args)
    head = args.config

    if args.attn_only:
        # profiling aid: a few bare attention launches over the written pool, nothing else
        import easymlx_b200 as emlx
        from easymlx_b200.operations.kernels.unified_attention import AttentionCall

        w = workloads.materialize(workloads.describe(head), dev, seed=0)
        c = w.cache
        extra = dict(k_scale=c.k_scales, v_scale=c.v_scales, k_bias=c.k_biases, v_bias=c.v_biases) if w.bits else {}
        call = AttentionCall(w.q, c.key_cache, c.value_cache, c.block_tables,
                             torch.from_numpy(w.kv_lens.astype(np.int32)).to(dev),
                             emlx.build_query_start_loc(w.qlens.tolist(), device=dev),
                             max_query_len=int(w.qlens.max()),
                             query_len_set=sorted(set(int(x) for x in w.qlens if x > 0)), **extra).plan()
        for _ in range(args.attn_only):
            call.launch()
        torch.cuda.synchronize()
        print(json.dumps({"attn_only": args.attn_only, "config": head}))
        return

    def weak_workload(name):
        """N draws of the configuration, partitioned by sequence, longest first, so that every rank attends about
        the same number of KV tokens; every rank owns the page pool of its own sequences."""
        base = workloads.describe(name)
        if world == 1:
            return workloads.materialize(base, dev, seed=0)
        draws = [workloads.describe(name, seed=None if r == 0 else 1000 * r + 7) for r in range(world)]
        whole = workloads.describe(name)
        whole.qlens = np.concatenate([d.qlens for d in draws])
        whole.prior = np.concatenate([d.prior for d in draws])
        mine = workloads.partition_by_sequence(whole, world)[rank]
        return workloads.materialize(whole, dev, seed=rank, seq_subset=mine)

    # ---- headline: weak scaling of the chosen configuration
    w = weak_workload(head)
    headline = bench.measure(w, f"{head}, {'one GPU' if world == 1 else f'weak scaling over {world} GPUs'}")
    base = workloads.describe(head)
    w = None
    torch.cuda.empty_cache()

    # ---- one GPU: all five configurations
    configs = None
    if world == 1 and not args.headline_only:
        configs = {}
        for name in ALL_CONFIGS:
            if name == head:
                configs[name] = headline
                continue
            wl = workloads.materialize(workloads.describe(name), dev, seed=0)
            configs[name] = bench.measure(wl, f"{name}, one GPU")
            wl = None
            torch.cuda.empty_cache()
        # beside BASELINE.json's five: the mixed batch of c3 over an 8-bit pool (prefill chunks on the tcgen05 kernel through
        # expanded pages, decode rows on the fused-dequant kernel)
        import dataclasses
        wl = workloads.materialize(dataclasses.replace(workloads.describe("c3"), bits=8), dev, seed=0)
        configs["c3_shape_affine8"] = bench.measure(wl, "c3's batch over an 8-bit affine pool (not a BASELINE.json configuration), one GPU",
                                                    parts=False, e2e=False)
        wl = None
        torch.cuda.empty_cache()

    # ---- several GPUs: the same global batch split over the ranks (strong scaling), and c4 sharded by KV head
    strong, c4_shard = None, None
    if world > 1 and not args.headline_only:
        strong = {}
        for name in ("c3", "c5"):
            whole = workloads.describe(name)
            mine = workloads.partition_by_sequence(whole, world)[rank]
            wl = workloads.materialize(whole, dev, seed=0, seq_subset=mine)
            r = bench.measure(wl, f"{name}: the one-GPU batch partitioned by sequence over {world} GPUs", parts=False, e2e=False)
            r["scaling"] = "strong"
            r["attended_kv_tokens_all_ranks"] = int(whole.attended_kv_tokens)
            strong[name] = r
            wl = None
            torch.cuda.empty_cache()
        whole = workloads.describe("c4")
        if whole.hkv % world == 0:
            per = whole.hkv // world
            wl = workloads.materialize(whole, dev, seed=0, kv_head_slice=slice(rank * per, (rank + 1) * per))
            gathered = torch.empty((world,) + tuple(wl.q.shape), dtype=wl.q.dtype, device=dev)

            def gather(out):
                dist.all_gather_into_tensor(gathered.view(-1, *out.shape[1:]), out)

            # parity first: the gathered heads against one rank attending all heads of the same pool
            from easymlx_b200.runtime import AttentionStep
            out = AttentionStep(wl.cache, wl.q, wl.k, wl.v, wl.qlens.tolist(), wl.slot_ids)._eager()
            full = all_gather_heads(out)
            parity = None
            if rank == 0:
                ref_w = workloads.materialize(whole, dev, seed=0)
                ref = AttentionStep(ref_w.cache, ref_w.q, ref_w.k, ref_w.v, ref_w.qlens.tolist(), ref_w.slot_ids)._eager()
                err = (full.float() - ref.float()).abs()
                bound = 2e-3 + 1e-2 * ref.float().abs()
                parity = {"max_abs_err": float(err.max().item()), "within_2e-3_plus_1e-2_rel": bool((err <= bound).all().item()),
                          "shape": list(full.shape)}
                if not parity["within_2e-3_plus_1e-2_rel"]:
                    print(f"c4: the gathered shards differ from the unsharded output: {parity}", file=sys.stderr, flush=True)
                ref_w = ref = None
                torch.cuda.empty_cache()
            r = bench.measure(wl, f"c4: KV heads sharded over {world} GPUs + NCCL all-gather of the outputs after every step",
                              after_step=gather, parts=False)
            # the same step with the gather done by the attention kernels: every rank's heads are stored into every
            # rank's output through peer-mapped memory (no collective call)
            try:
                from easymlx_b200.distributed import PeerGather
                peers = PeerGather(int(wl.total_tokens), whole.hq, whole.d, wl.q.dtype, dev, poll_limit=1 << 24)
            except Exception as exc:  # the ranks fail together (see PeerGather)
                peers, peer_store = None, {"unavailable": str(exc)[:300]}
            if peers is not None:
                got = AttentionStep(wl.cache, wl.q, wl.k, wl.v, wl.qlens.tolist(), wl.slot_ids, gather=peers.target)._eager()
                torch.cuda.synchronize()
                same = torch.tensor([int(torch.equal(got, full))], device=dev)
                dist.all_reduce(same, op=dist.ReduceOp.MIN)
                rp = bench.measure(wl, f"c4: KV heads sharded over {world} GPUs, heads stored into every rank's output "
                                       "by the attention kernels (peer-mapped memory, no collective call)",
                                   gather_target=peers.target, parts=False)
                from easymlx_b200.operations.kernels import unified_attention as ua
                status = max(int(t.view(torch.int32)[0].item()) for k, t in ua._scratch.buffers.items() if k[2] == "status")
                peer_store = {"us_per_batch": rp["us_per_batch"], "value": rp["value"], "unit": UNIT,
                              "e2e_us_per_batch": rp["e2e"]["us_per_batch"], "clocks": rp["clocks"],
                              "gpu_launches_per_step": rp["gpu_launches_per_step"],
                              "identical_to_all_gather_on_every_rank": bool(same.item()), "device_status": status}
                peers.close()
            r["scaling"] = "strong"
            r["peer_store"] = peer_store
            r["attn_us"] = r["roofline"]["us_per_launch"]
            dummy = wl.q.clone()
            r["allgather_us"] = bench.graph_time(lambda: gather(dummy), 10, args.steps) * 1e3
            r["allgather_bytes_per_rank"] = int(dummy.numel() * dummy.element_size())
            r["parity_vs_unsharded"] = parity
            c4_shard = r
            wl = None
            torch.cuda.empty_cache()

    if rank == 0:
        roof = dict(headline["roofline"])
        if world == 1:
            tpath = os.path.join(ROOT, "profiles", f"traffic_{head}.json")
            if os.path.exists(tpath):
                roof["traffic"] = json.load(open(tpath)).get("dram_bytes_per_launch")
                roof["traffic_source"] = f"ncu capture of this launch on one GPU (profiles/traffic_{head}.json), not measured in this run"
            else:
                roof["traffic"] = None
        else:
            roof["traffic"] = None
        line = {
            "metric": METRIC, "value": headline["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": headline["us_per_batch"] / 1e3,
            "us_per_batch": headline["us_per_batch"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": headline_config(head, world, layers),
            "clocks": headline["clocks"], "e2e": headline["e2e"],
            "gpu_launches": int(headline["gpu_launches_per_step"] * args.steps),
            "roofline": roof, "step_frac_of_hbm_peak": headline["step_frac_of_hbm_peak"],
        }
        if configs is not None:
            line["configs"] = configs
        if strong is not None:
            line["strong"] = strong
        if c4_shard is not None:
            line["c4_head_shard"] = c4_shard
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = _cpu_baseline_single_core(base, head, args.cpu_budget_tokens)
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
    ap.add_argument("--config", default="c2", choices=list(ALL_CONFIGS), help="headline configuration")
    ap.add_argument("--headline-only", action="store_true", help="skip the other configurations / scaling variants")
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
