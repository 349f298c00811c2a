"""CPU oracle for the rotary embedding fused into the KV write.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

PARITY UNPINNED: in the reference the rotation itself is ``mlx.core.fast.rope`` (mlx 0.31.1, third party, not
in the reference tree; call sites ``layers/rotary/_rotary.py:123-131,213-221,369-370``), and the only reference
test compares against the same call.  This file restates the published rotation
(angle = position * scale / freqs[i]; pairs (i, i + dims/2), or (2i, 2i + 1) in the "traditional" layout) and
the frequency tables the reference builds for its variants (``_rotary.py:94-98,179-193,291-300``).
"""

from __future__ import annotations

import math

import numpy as np


def default_freqs(dims: int, base: float) -> np.ndarray:
    return (np.float32(base) ** (np.arange(0, dims, 2, dtype=np.float32) / np.float32(dims))).astype(np.float32)


def llama3_freqs(dims, base, factor, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192):
    freqs = default_freqs(dims, base).astype(np.float64)
    wavelens = 2 * math.pi * freqs
    low_wl, high_wl = original_max_position_embeddings / low_freq_factor, original_max_position_embeddings / high_freq_factor
    scaled = np.where(wavelens > low_wl, freqs * factor, freqs)
    smooth = (original_max_position_embeddings / wavelens - low_freq_factor) / (high_freq_factor - low_freq_factor)
    mid = scaled / ((1 - smooth) / factor + smooth)
    return np.where((wavelens > high_wl) & (wavelens < low_wl), mid, scaled).astype(np.float32)


def rotate(x, positions, freqs, dims, *, traditional=False, scale=1.0, mscale=1.0):
    """``x[T, H, D]`` rotated at ``positions[T]``; fp32 arithmetic, result in the dtype of ``x``."""
    x32 = np.asarray(x, dtype=np.float32).copy()
    inv = (np.float32(1.0) / np.asarray(freqs, dtype=np.float32)).astype(np.float32)
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * np.float32(scale)) * inv[None, :]   # [T, dims/2]
    cs, sn = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    head = x32[..., :dims] * np.float32(mscale)
    if traditional:
        a, b = head[..., 0::2], head[..., 1::2]
        out = np.empty_like(head)
        out[..., 0::2] = a * cs - b * sn
        out[..., 1::2] = a * sn + b * cs
    else:
        a, b = head[..., : dims // 2], head[..., dims // 2:]
        out = np.concatenate([a * cs - b * sn, a * sn + b * cs], axis=-1)
    x32[..., :dims] = out
    return x32.astype(np.asarray(x).dtype)
