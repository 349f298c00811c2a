"""One attention-layer step (KV write + metadata + attention) as a replayable CUDA graph.

The reference compiles its single-token decode closure per (slots, query lengths) key with
``mx.compile`` (``inference/esurge/runners/model_runner.py:744-856``) to get rid of per-launch host
overhead; here the same role is played by capturing the step's kernels once in a CUDA graph and
replaying it.  Inputs live in static device tensors that the caller overwrites between replays.
"""

from __future__ import annotations

import torch

from . import _native as nv
from .caching.paged.cache import PageCacheView, PageMetadata, build_query_start_loc
from .layers.attention import AttentionPerformer


class AttentionStep:
    """``step()`` = restore the slots' lengths, write the new K/V rows, attend.

    ``rewind=True`` leaves the cache's ``kv_lens`` at their values (the step's rows are written and attended,
    the lengths are not advanced), so that the same batch can be replayed any number of times (benchmarks); a
    serving loop passes ``rewind=False``.
    """

    def __init__(self, cache: PageCacheView, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, query_lens,
                 slot_ids, *, scale: float | None = None, sliding_window: int | None = None, rewind: bool = True,
                 gather=None):
        self.cache = cache
        self.q, self.k, self.v = q, k, v
        self.query_lens = tuple(int(x) for x in query_lens)
        self.slot_ids = tuple(int(x) for x in slot_ids)
        self.performer = AttentionPerformer(scale=scale if scale is not None else float(q.shape[-1]) ** -0.5)
        self.rewind = rewind
        self.gather = gather   # distributed.GatherTarget: KV heads sharded over GPUs, output gathered by the kernels
        self._base_lens = cache.kv_lens.clone()
        single = len(self.query_lens) == q.shape[0] and all(x == 1 for x in self.query_lens)
        self._meta = PageMetadata(query_start_loc=build_query_start_loc(self.query_lens), slot_ids=self.slot_ids,
                                  sliding_window=sliding_window, is_single_token_decode=single)
        self._meta_lens = None if single else self.query_lens
        self.out: torch.Tensor | None = None
        self.graph: torch.cuda.CUDAGraph | None = None
        self.launches_per_step = 0
        self.steps_per_graph = 1

    def _eager(self) -> torch.Tensor:
        # rewind: the slots' lengths are left as they were, so the same batch can be replayed
        _, kc, vc, meta = self.cache.concatenate_to_cache(self.q, self.k, self.v, cache_metadata=self._meta,
                                                          slot_ids=self.slot_ids, query_lens=self.query_lens,
                                                          advance=not self.rewind)
        if self.gather is not None:
            from .operations.kernels.unified_attention import paged_attention

            extra = {}
            if self.cache.is_affine:
                extra = dict(k_scale=self.cache.k_scales, v_scale=self.cache.v_scales, k_bias=self.cache.k_biases,
                             v_bias=self.cache.v_biases)
            return paged_attention(self.q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc,
                                   softmax_scale=self.performer.scale, sliding_window=meta.sliding_window,
                                   single_token_decode=meta.is_single_token_decode,
                                   max_query_len=int(getattr(meta, "max_query_len", 0) or 0),
                                   plan=getattr(meta, "plan", None), query_len_set=getattr(meta, "query_len_set", None),
                                   gather=self.gather, **extra)
        op = self.performer.executor.mixin_impl
        return op(query=self.q, key=kc, value=vc, cache_metadata=meta, cache_view=self.cache,
                  scale=self.performer.scale).attention_outputs

    def capture(self, warmup: int = 3, steps_per_graph: int = 1) -> "AttentionStep":
        """Run the step eagerly a few times on a side stream, then record it into a CUDA graph.

        ``steps_per_graph`` > 1 records that many consecutive steps in one graph, the way an engine step holds
        one attention step per transformer layer; ``step()`` then advances by that many steps per call."""
        side = torch.cuda.Stream(device=self.q.device)
        side.wait_stream(torch.cuda.current_stream(self.q.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                self.out = self._eager()
        torch.cuda.current_stream(self.q.device).wait_stream(side)
        torch.cuda.synchronize(self.q.device)
        graph = torch.cuda.CUDAGraph()
        before = nv.launch_count()
        with torch.cuda.graph(graph):
            for _ in range(max(1, steps_per_graph)):
                self.out = self._eager()
        self.steps_per_graph = max(1, steps_per_graph)
        self.launches_per_step = (nv.launch_count() - before) // self.steps_per_graph
        self.graph = graph
        return self

    def step(self) -> torch.Tensor:
        if self.graph is not None:
            self.graph.replay()
            return self.out
        before = nv.launch_count()
        self.out = self._eager()
        self.launches_per_step = nv.launch_count() - before
        return self.out


class HostStepPipeline:
    """Steps whose q / k / v arrive in pinned host memory and whose output goes back to pinned host memory.

    A step's upload, its kernels and its download depend on one another, but the upload of step n+1 and the download
    of step n-1 do not depend on the kernels of step n: with ``depth`` buffer sets (device inputs, a captured
    ``AttentionStep`` over them, a pinned host output) and one stream per direction, the three overlap and a step costs
    the slowest of them instead of their sum.  q, k and v travel as one packed buffer (one copy per step).

    ``submit()`` enqueues one step and returns the index of the buffer set it used; ``result(i)`` is that set's host
    output (wait for ``downloaded[i]`` before reading it); ``drain()`` makes the calling stream wait for every download,
    so that an event recorded after it covers all submitted work.
    """

    def __init__(self, cache: PageCacheView, host_qkv, query_lens, slot_ids, *, depth: int = 2, gather=None,
                 after_step=None, scale: float | None = None, sliding_window: int | None = None):
        hq, hk, hv = host_qkv
        dev = cache.key_cache.device
        self.device, self.depth, self.after_step = dev, max(1, int(depth)), after_step
        parts = (hq, hk, hv)
        sizes = [t.numel() for t in parts]
        self.host_in = torch.cat([t.reshape(-1) for t in parts]).pin_memory()
        self.dev_in, self.steps, self.host_out = [], [], []
        for _ in range(self.depth):
            packed = torch.empty_like(self.host_in, device=dev)
            packed.copy_(self.host_in)
            dq, dk, dv = (v.view(t.shape) for v, t in zip(torch.split(packed, sizes), parts))
            step = AttentionStep(cache, dq, dk, dv, query_lens, slot_ids, scale=scale, sliding_window=sliding_window,
                                 gather=gather).capture(warmup=2)
            self.dev_in.append(packed)
            self.steps.append(step)
            self.host_out.append(torch.empty_like(step.out, device="cpu").pin_memory())
        self.up, self.down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        make = lambda: [torch.cuda.Event() for _ in range(self.depth)]
        self.uploaded, self.computed, self.downloaded = make(), make(), make()
        self.submitted = 0
        torch.cuda.synchronize(dev)

    @property
    def h2d_bytes_per_step(self) -> int:
        return int(self.host_in.numel() * self.host_in.element_size())

    @property
    def d2h_bytes_per_step(self) -> int:
        return int(self.host_out[0].numel() * self.host_out[0].element_size())

    def submit(self) -> int:
        i = self.submitted % self.depth
        reused = self.submitted >= self.depth
        cur = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.up):
            if reused:
                self.up.wait_event(self.computed[i])       # the kernels that read this input buffer have finished
            else:
                self.up.wait_stream(cur)
            self.dev_in[i].copy_(self.host_in, non_blocking=True)
            self.uploaded[i].record(self.up)
        cur.wait_event(self.uploaded[i])
        if reused:
            cur.wait_event(self.downloaded[i])             # the previous result of this set has left the device
        out = self.steps[i].step()
        if self.after_step is not None:
            self.after_step(out)
        self.computed[i].record(cur)
        with torch.cuda.stream(self.down):
            self.down.wait_event(self.computed[i])
            self.host_out[i].copy_(out, non_blocking=True)
            self.downloaded[i].record(self.down)
        self.submitted += 1
        return i

    def result(self, i: int) -> torch.Tensor:
        return self.host_out[i]

    def drain(self) -> None:
        cur = torch.cuda.current_stream(self.device)
        for i in range(min(self.depth, self.submitted)):
            cur.wait_event(self.downloaded[i])


__all__ = ("AttentionStep", "HostStepPipeline")
