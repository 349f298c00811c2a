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


__all__ = ("AttentionStep",)
