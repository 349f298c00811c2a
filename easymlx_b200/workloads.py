"""Seeded synthetic batches with the shapes of the five benchmark configurations.

No dataset is involved: the configurations name model *shapes* only.  Lengths come from
``numpy.random.default_rng(1000 + index)``; K/V/Q contents are N(0,1) drawn on the GPU
from a seeded torch generator (rounded to fp16), and affine pools are filled by running
those rows through the library's own KV-write kernel.

  c1  Llama-3.2-1B shape, fp16 : 32/8 heads, D 64;  2 prefill chunks of 512 + 6 decode rows (ctx 256..2048)
  c2  Llama-3-8B decode, 8-bit : 32/8 heads, D 128; 64 rows, context 1024..8192
  c3  Qwen3-32B mixed, fp16    : 64/8 heads, D 128; 240 decode rows (Zipf 1.2, 64..16384) + 4 chunks = 4096 tokens
  c4  Llama-3-70B decode, 4-bit: 64/8 heads, D 128; 16 rows at 32768 (one KV head per GPU when sharded)
  c5  spec-verify, fp16        : 32/8 heads, D 128; 128 rows x 5 tokens after 512..8192, pool 2x oversized

"Context" counts the keys a row attends to after this step's write: ``kv_len = prior + q_len``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from . import _native as nv
from .caching.paged.cache import PageCacheView

PAGE = 128


@dataclass
class Workload:
    name: str
    hq: int
    hkv: int
    d: int
    bits: int                       # 0 = fp16 pool
    qlens: np.ndarray               # [S] new tokens per sequence
    prior: np.ndarray               # [S] tokens already cached
    oversize: float = 1.0
    description: str = ""
    cache: PageCacheView | None = None
    q: torch.Tensor | None = None
    k: torch.Tensor | None = None
    v: torch.Tensor | None = None
    slot_ids: tuple = field(default_factory=tuple)

    @property
    def kv_lens(self) -> np.ndarray:
        return self.prior + self.qlens

    @property
    def total_tokens(self) -> int:
        return int(self.qlens.sum())

    @property
    def attended_kv_tokens(self) -> int:
        return int(self.kv_lens.sum())

    def row_bytes(self) -> int:
        """Stored bytes of one K (or V) row of one head."""
        return 2 * self.d if self.bits == 0 else self.d * self.bits // 8 + 4 * (self.d // 64)

    def attention_bytes(self) -> int:
        """Algorithmic HBM bytes of the attention call: every live KV row of every head once per sequence,
        queries in, outputs out, the page ids and the lengths."""
        kv = int(self.kv_lens.sum()) * 2 * self.hkv * self.row_bytes()
        qo = 2 * self.total_tokens * self.hq * self.d * 2
        pages = int(np.ceil(self.kv_lens / PAGE).sum()) * 4
        return kv + qo + pages + 4 * (2 * len(self.qlens) + 1)

    def write_bytes(self) -> int:
        return self.total_tokens * self.hkv * (2 * 2 * self.d + 2 * self.row_bytes())

    def attention_flops(self) -> int:
        pairs = int(sum(int(q) * int(c) + int(q) * (int(q) + 1) // 2 for q, c in zip(self.qlens, self.prior)))
        return 4 * self.hq * self.d * pairs


def _lengths(name: str, seed: int | None = None):
    idx = {"c1": 1, "c2": 2, "c3": 3, "c4": 4, "c5": 5}[name]
    r = np.random.default_rng(1000 + idx if seed is None else seed)
    if name == "c1":
        ctx = r.integers(256, 2049, 6)
        return dict(hq=32, hkv=8, d=64, bits=0, qlens=[512, 512] + [1] * 6, prior=[0, 0] + list(ctx - 1),
                    description="Llama-3.2-1B-shaped mixed batch, fp16 KV")
    if name == "c2":
        ctx = r.integers(1024, 8193, 64)
        return dict(hq=32, hkv=8, d=128, bits=8, qlens=[1] * 64, prior=list(ctx - 1),
                    description="Llama-3-8B-shaped decode, 64 seqs, ctx U[1024,8192], 8-bit affine KV")
    if name == "c3":
        dec = np.clip(r.zipf(1.2, 240), 64, 16384)
        cuts = np.sort(r.choice(np.arange(1, 3856), 3, replace=False))
        chunks = np.diff(np.concatenate([[0], cuts, [3856]]))
        pctx = r.integers(0, 4097, 4)
        return dict(hq=64, hkv=8, d=128, bits=0, qlens=list(chunks) + [1] * 240, prior=list(pctx) + list(dec - 1),
                    description="Qwen3-32B-shaped mixed batch, 240 decode (Zipf) + 4 prefill chunks = 4096 tokens, fp16 KV")
    if name == "c4":
        return dict(hq=64, hkv=8, d=128, bits=4, qlens=[1] * 16, prior=[32767] * 16,
                    description="Llama-3-70B-shaped long decode, 16 seqs x 32768, 4-bit affine KV")
    if name == "c5":
        ctx = r.integers(512, 8193, 128)
        return dict(hq=32, hkv=8, d=128, bits=0, qlens=[5] * 128, prior=list(ctx), oversize=2.0,
                    description="spec-verify, 128 seqs x 5 tokens after ctx U[512,8192], fp16 KV, 2x pool")
    raise ValueError(f"unknown workload {name}")


def describe(name: str, seed: int | None = None) -> Workload:
    """Lengths and geometry only; no device memory."""
    spec = _lengths(name, seed)
    spec["qlens"] = np.asarray(spec["qlens"], dtype=np.int64)
    spec["prior"] = np.asarray(spec["prior"], dtype=np.int64)
    return Workload(name=name, **spec)


def fill_rows(cache: PageCacheView, slots: torch.Tensor, keys: torch.Tensor, values: torch.Tensor) -> None:
    """Write ``keys/values[n, Hkv, D]`` at flat pool slots ``page*bs + offset`` with the KV-write kernel."""
    pool = cache.native_pool()
    nv.check(nv.lib().emlx_kv_write(nv.ptr(keys), nv.ptr(values), nv.dtype_code(keys.dtype), int(keys.shape[0]),
                                    nv.ptr(slots), pool, nv.ptr(cache.status), nv.stream_ptr(keys.device)))


def materialize(w: Workload, device="cuda", seed: int = 0, kv_head_slice: slice | None = None,
                seq_subset: np.ndarray | None = None) -> Workload:
    """Allocate and fill the pool, page tables and the step's q/k/v on ``device``.

    ``seq_subset`` keeps only some sequences (sequence partitioning across GPUs); ``kv_head_slice``
    keeps only some KV heads and their query heads (KV-head sharding).
    """
    dev = torch.device(device)
    qlens, prior = w.qlens, w.prior
    if seq_subset is not None:
        qlens, prior = qlens[seq_subset], prior[seq_subset]
    hq, hkv = w.hq, w.hkv
    if kv_head_slice is not None:
        group = hq // hkv
        hkv = len(range(*kv_head_slice.indices(w.hkv)))
        hq = hkv * group
    out = Workload(name=w.name, hq=hq, hkv=hkv, d=w.d, bits=w.bits, qlens=qlens, prior=prior, oversize=w.oversize,
                   description=w.description)
    kv = prior + qlens
    pages = -(-kv // PAGE)
    s = len(kv)
    mb = int(max(1, pages.max()))
    nb = int(np.ceil(max(1, int(pages.sum())) * w.oversize))
    rng = np.random.default_rng(seed + 17)
    perm = rng.permutation(nb)
    bt = -np.ones((s, mb), dtype=np.int32)
    cursor = 0
    for i, n in enumerate(pages):
        bt[i, :n] = perm[cursor:cursor + n]
        cursor += int(n)
    cache = PageCacheView.init(num_seqs=s, max_seq_len=mb * PAGE, num_kv_heads=hkv, head_dim=w.d, block_size=PAGE,
                               dtype=torch.float16, cache_bits=w.bits or None,
                               cache_dtype="affine" if w.bits else None, device=dev, num_blocks=nb)
    cache.block_tables.copy_(torch.from_numpy(bt))
    cache.kv_lens.copy_(torch.from_numpy(prior.astype(np.int32)))
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + 1)
    heads = kv_head_slice if kv_head_slice is not None else slice(None)
    qheads = slice(None)
    if kv_head_slice is not None:
        lo, hi, _ = kv_head_slice.indices(w.hkv)
        qheads = slice(lo * (w.hq // w.hkv), hi * (w.hq // w.hkv))
    if w.bits == 0 and kv_head_slice is None:
        cache.key_cache.normal_(generator=gen)
        cache.value_cache.normal_(generator=gen)
    else:
        # rows are drawn at the full head count and sliced, so that a KV-head shard holds exactly the heads it would
        # hold in the unsharded pool (same seed on every rank)
        chunk_pages = 256
        for p0 in range(0, nb, chunk_pages):
            p1 = min(nb, p0 + chunk_pages)
            n = (p1 - p0) * PAGE
            k = torch.randn((n, w.hkv, w.d), generator=gen, device=dev, dtype=torch.float32).half()[:, heads].contiguous()
            v = torch.randn((n, w.hkv, w.d), generator=gen, device=dev, dtype=torch.float32).half()[:, heads].contiguous()
            if w.bits == 0:
                cache.key_cache[p0:p1] = k.view(p1 - p0, PAGE, hkv, w.d)
                cache.value_cache[p0:p1] = v.view(p1 - p0, PAGE, hkv, w.d)
            else:
                slots = torch.arange(p0 * PAGE, p1 * PAGE, dtype=torch.int64, device=dev)
                fill_rows(cache, slots, k, v)
    t = int(qlens.sum())
    out.q = torch.randn((t, w.hq, w.d), generator=gen, device=dev, dtype=torch.float32).half()[:, qheads].contiguous()
    out.k = torch.randn((t, w.hkv, w.d), generator=gen, device=dev, dtype=torch.float32).half()[:, heads].contiguous()
    out.v = torch.randn((t, w.hkv, w.d), generator=gen, device=dev, dtype=torch.float32).half()[:, heads].contiguous()
    out.cache = cache
    out.slot_ids = tuple(range(s))
    return out


def partition_by_sequence(w: Workload, world: int) -> list[np.ndarray]:
    """The sequences of ``w`` assigned to ``world`` ranks (``distributed.partition_by_sequence``: greedy, longest
    first, balancing attended KV tokens)."""
    from .distributed import partition_by_sequence as _partition

    return _partition(w.qlens, w.kv_lens, world)
