"""Rotary position embeddings for the paged path.

Mirrors the factory of easymlx ``layers/rotary/_rotary.py`` (``get_rope`` ``:327-415``): every variant there ends
in ``mx.fast.rope(x, dims, traditional, base | freqs, scale, offset)``, i.e. a table of per-pair periods, a
position scale and an optional magnitude scale.  ``RotaryEmbedding`` holds exactly that (``LongRopeEmbedding`` holds two
of them and picks one by sequence length); ``PageCacheView.
concatenate_to_cache(rope=...)`` hands it to the CUDA write kernel, which rotates K while storing it and Q in the
same launch.  Calling the object rotates a tensor on its own (``rope(x, offset=...)``, ``x`` ``[B, H, L, D]`` or
``[T, H, D]``).
"""

from __future__ import annotations

import math
import typing as tp

import numpy as np
import torch

from .. import _native as nv


class RotaryEmbedding:
    def __init__(self, dims: int, base: float = 10000.0, traditional: bool = False, scale: float = 1.0,
                 freqs: tp.Sequence[float] | np.ndarray | None = None, mscale: float = 1.0):
        if dims <= 0 or dims % 2:
            raise ValueError("dims must be positive and even")
        self.dims, self.traditional, self.scale, self.mscale = int(dims), bool(traditional), float(scale), float(mscale)
        if freqs is None:
            freqs = np.float32(base) ** (np.arange(0, dims, 2, dtype=np.float32) / np.float32(dims))
        self.freqs = np.asarray(freqs, dtype=np.float32)
        if self.freqs.shape != (dims // 2,):
            raise ValueError("freqs must have dims / 2 entries")
        self._inv_freq: dict[str, torch.Tensor] = {}

    def inv_freq(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self._inv_freq:
            self._inv_freq[key] = torch.from_numpy((np.float32(1.0) / self.freqs).astype(np.float32)).to(device)
        return self._inv_freq[key]

    def native(self, device, head_dim: int = 0) -> nv.Rope:
        r = nv.Rope()
        r.inv_freq = self.inv_freq(device).data_ptr()
        r.dims, r.traditional = self.dims, int(self.traditional)
        r.position_scale, r.mscale = self.scale, self.mscale
        r.head_dim_if_no_pool = int(head_dim)
        return r

    def __call__(self, x: torch.Tensor, offset: int | torch.Tensor = 0) -> torch.Tensor:
        """Rotate ``x`` (``[B, H, L, D]`` with positions ``offset + arange(L)``, or ``[T, H, D]`` with ``offset`` a
        tensor of T positions)."""
        nv.require_cuda(x)
        if x.ndim == 4:
            b, h, l, d = x.shape
            flat = x.permute(0, 2, 1, 3).reshape(b * l, h, d).contiguous()
            off = torch.as_tensor(offset, device=x.device, dtype=torch.int32).reshape(-1, 1).expand(b, 1) if \
                torch.is_tensor(offset) or not isinstance(offset, int) else torch.full((b, 1), int(offset), dtype=torch.int32, device=x.device)
            pos = (off + torch.arange(l, dtype=torch.int32, device=x.device)[None, :]).reshape(-1).contiguous()
            return self._apply(flat, pos).reshape(b, l, h, d).permute(0, 2, 1, 3)
        if x.ndim != 3:
            raise ValueError("x must be [B, H, L, D] or [T, H, D]")
        pos = torch.as_tensor(offset, device=x.device, dtype=torch.int32).reshape(-1).contiguous()
        if pos.numel() == 1:
            pos = pos.expand(x.shape[0]).contiguous()
        return self._apply(x.contiguous(), pos)

    def _apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        t, h, d = x.shape
        if t == 0:
            return out
        rope = self.native(x.device, head_dim=d)
        nv.check(nv.lib().emlx_kv_write_rope(nv.ptr(x), nv.ptr(out), h, None, None, nv.dtype_code(x.dtype), t, None,
                                             nv.ptr(positions), rope, None, None, nv.stream_ptr(x.device)))
        return out


class LongRopeEmbedding:
    """Su-scaled ("longrope") rotary embedding: two period tables, one for sequences up to
    ``original_max_position_embeddings`` tokens and one for longer ones, each with its magnitude scale
    (easymlx ``layers/rotary/_rotary.py:36-131``).

    The reference chooses per call from ``offset + length``.  Here the choice is made on the host, once per call or
    per packed batch: ``select(total_len)`` returns the ``RotaryEmbedding`` for a sequence that is ``total_len``
    tokens long after the step.  ``PageCacheView.concatenate_to_cache`` calls it with the longest scheduled
    sequence (``PageMetadata.max_kv_len`` when the runner supplies it, else one device read), so a batch that mixes
    sequences on both sides of the threshold is rotated with the long table throughout.
    """

    def __init__(self, dims: int, base: float = 10000.0, max_position_embeddings: int = 131072,
                 original_max_position_embeddings: int = 4096, short_factor: tp.Sequence[float] | float = 1.0,
                 long_factor: tp.Sequence[float] | float = 1.0, short_mscale: float | None = None,
                 long_mscale: float | None = None):
        self.dims = int(dims)
        self.original_max_position_embeddings = int(original_max_position_embeddings)
        freqs = np.float32(base) ** (np.arange(0, dims, 2, dtype=np.float32) / np.float32(dims))
        factor = max_position_embeddings / original_max_position_embeddings
        default = 1.0 if factor <= 1.0 else math.sqrt(1 + math.log(factor) / math.log(original_max_position_embeddings))
        self.short = RotaryEmbedding(self.dims, freqs=np.asarray(short_factor, dtype=np.float32) * freqs,
                                     mscale=short_mscale or default)
        self.long = RotaryEmbedding(self.dims, freqs=np.asarray(long_factor, dtype=np.float32) * freqs,
                                    mscale=long_mscale or default)

    def select(self, total_len: int) -> RotaryEmbedding:
        return self.long if int(total_len) > self.original_max_position_embeddings else self.short

    def __call__(self, x: torch.Tensor, offset: int | torch.Tensor = 0) -> torch.Tensor:
        length = int(x.shape[-2]) if x.ndim == 4 else 1
        last = int(torch.as_tensor(offset).max().item()) if torch.is_tensor(offset) else int(offset)
        return self.select(last + length)(x, offset=offset)


def _llama3_freqs(dims, base, cfg) -> np.ndarray:
    factor = cfg["factor"]
    low, high = cfg.get("low_freq_factor", 1.0), cfg.get("high_freq_factor", 4.0)
    old_len = cfg.get("original_max_position_embeddings", 8192)
    freqs = (np.float32(base) ** (np.arange(0, dims, 2, dtype=np.float32) / np.float32(dims))).astype(np.float64)
    wavelens = 2 * math.pi * freqs
    scaled = np.where(wavelens > old_len / low, freqs * factor, freqs)
    smooth = (old_len / wavelens - low) / (high - low)
    mid = scaled / ((1 - smooth) / factor + smooth)
    return np.where((wavelens > old_len / high) & (wavelens < old_len / low), mid, scaled).astype(np.float32)


def _yarn(dims, base, factor, original_max=4096, beta_fast=32, beta_slow=1, mscale=1, mscale_all_dim=0):
    def correction_dim(rotations):
        return dims * math.log(original_max / (rotations * 2 * math.pi)) / (2 * math.log(base))

    def magnitude(scale, m):
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

    lo, hi = max(math.floor(correction_dim(beta_fast)), 0), min(math.ceil(correction_dim(beta_slow)), dims - 1)
    if lo == hi:
        hi += 0.001
    ramp = np.clip((np.arange(dims // 2, dtype=np.float32) - lo) / (hi - lo), 0, 1)
    extra = np.float32(base) ** (np.arange(0, dims, 2, dtype=np.float32) / np.float32(dims))
    inter = factor * extra
    mask = 1.0 - ramp
    freqs = (inter * extra) / (inter * mask + extra * (1 - mask))
    return freqs.astype(np.float32), magnitude(factor, mscale) / magnitude(factor, mscale_all_dim)


def get_rope(dims: int, base: float, traditional: bool, scaling_config: dict | None = None,
             max_position_embeddings: int | None = None) -> RotaryEmbedding:
    """Same arguments and variant names as the reference factory."""
    kind = "default"
    if scaling_config is not None:
        kind = scaling_config.get("type") or scaling_config.get("rope_type", "default")
    if kind in ("default", "linear", "mrope"):
        scale = 1 / scaling_config["factor"] if kind == "linear" else 1.0
        return RotaryEmbedding(int(dims), base=base, traditional=traditional, scale=scale)
    if kind == "llama3":
        return RotaryEmbedding(int(dims), traditional=traditional, freqs=_llama3_freqs(int(dims), base, scaling_config))
    if kind == "yarn":
        keys = ("original_max_position_embeddings", "beta_fast", "beta_slow", "mscale", "mscale_all_dim")
        kw = {k: scaling_config[k] for k in keys if k in scaling_config}
        if "original_max_position_embeddings" in kw:
            kw["original_max"] = kw.pop("original_max_position_embeddings")
        freqs, mscale = _yarn(int(dims), base, scaling_config["factor"], **kw)
        return RotaryEmbedding(int(dims), traditional=traditional, freqs=freqs, mscale=mscale)
    if kind == "longrope":
        return LongRopeEmbedding(int(dims), base=base, max_position_embeddings=int(max_position_embeddings or 131072),
                                 original_max_position_embeddings=scaling_config["original_max_position_embeddings"],
                                 short_factor=scaling_config["short_factor"], long_factor=scaling_config["long_factor"])
    raise ValueError(f"Unsupported RoPE type {kind}")


__all__ = ("LongRopeEmbedding", "RotaryEmbedding", "get_rope")
