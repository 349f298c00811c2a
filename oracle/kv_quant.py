"""CPU oracle for the affine group-64 KV quantiser.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

PARITY UNPINNED: the reference has no affine-quantised KV cache.  Its only affine
quantiser is ``mlx.core.quantize(..., mode="affine")`` from the third-party package
mlx 0.31.1 (pinned in the reference's ``uv.lock``), called for *weights* at
``infra/mixins/bridge.py:304,361`` and ``layers/linears/_linear_moe.py:113-121``; MLX is
not installed here, its source is not part of the reference tree, and no reference test
holds a quantisation vector.  The specification below is therefore this build's own
("min-max over each group of 64 along head_dim, fp16 scale and bias"), and "bit-exact"
means CUDA kernel == this file on the same inputs.

Specification, per (token, kv head, group g of 64 consecutive head_dim elements), all
arithmetic IEEE fp32 round-to-nearest-even unless a cast is named:

    lo, hi = min(x), max(x)                       x converted to fp32 first
    scale  = fp16( (hi - lo) / (2**bits - 1) )    replaced by fp16(1) when that cast is 0
    bias   = fp16( lo )
    code   = clamp( rint( (x - fp32(bias)) / fp32(scale) ), 0, 2**bits - 1 )
    x'     = fp32(scale) * code + fp32(bias)      (dequantised value, fp32)

Storage.  Key codes are bytes ``[NB, bs, Hkv, D*bits/8]`` (token-major; with 4 bits element
``2i`` sits in the low nibble of byte ``i``).  Value codes are bytes ``[NB, Hkv, D, bs*bits/8]``:
transposed inside a page, so that the tokens of one head_dim element are contiguous (with 4
bits token ``2i`` sits in the low nibble of byte ``i``).  ``scale`` and ``bias`` are fp16
``[NB, Hkv, bs, D/64]`` for keys and for values (head-major inside a page, so the 128 tokens
of one (page, head) tile are contiguous).
"""

from __future__ import annotations

import numpy as np

GROUP = 64


def quantize_rows(x, bits):
    """``x[..., D]`` -> ``(codes[..., D] uint8 (unpacked), scale[..., D/64] f16, bias[..., D/64] f16)``."""
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    x = np.asarray(x).astype(np.float32)
    d = x.shape[-1]
    if d % GROUP:
        raise ValueError("head_dim must be a multiple of 64")
    levels = np.float32((1 << bits) - 1)
    g = x.reshape(x.shape[:-1] + (d // GROUP, GROUP))
    lo = g.min(axis=-1)
    hi = g.max(axis=-1)
    scale = ((hi - lo) / levels).astype(np.float16)
    scale = np.where(scale == 0, np.float16(1.0), scale).astype(np.float16)
    bias = lo.astype(np.float16)
    code = np.rint((g - bias.astype(np.float32)[..., None]) / scale.astype(np.float32)[..., None])
    code = np.clip(code, 0, levels).astype(np.uint8)
    return code.reshape(x.shape), scale, bias


def pack_codes(codes, bits):
    """Unpacked ``uint8[..., D]`` -> stored bytes ``uint8[..., D*bits/8]``."""
    if bits == 8:
        return np.ascontiguousarray(codes, dtype=np.uint8)
    c = np.asarray(codes, dtype=np.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


def unpack_codes(stored, bits):
    if bits == 8:
        return np.asarray(stored, dtype=np.uint8)
    s = np.asarray(stored, dtype=np.uint8)
    out = np.empty(s.shape[:-1] + (s.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = s & 0xF
    out[..., 1::2] = s >> 4
    return out


def dequantize_rows(codes, scale, bias):
    """Unpacked codes ``[..., D]`` with ``scale/bias[..., D/64]`` -> fp32 ``[..., D]``."""
    d = codes.shape[-1]
    g = codes.reshape(codes.shape[:-1] + (d // GROUP, GROUP)).astype(np.float32)
    x = scale.astype(np.float32)[..., None] * g + bias.astype(np.float32)[..., None]
    return x.reshape(codes.shape)


def dequantize_key_pool(code_cache, scale, bias, bits):
    """Key pool ``[NB, bs, Hkv, D*bits/8]`` + ``scale/bias[NB, Hkv, bs, D/64]`` -> fp32 ``[NB, bs, Hkv, D]``."""
    codes = unpack_codes(code_cache, bits)
    s = np.transpose(scale, (0, 2, 1, 3))
    b = np.transpose(bias, (0, 2, 1, 3))
    return dequantize_rows(codes, s, b)


def dequantize_value_pool(code_cache, scale, bias, bits):
    """Value pool ``[NB, Hkv, D, bs*bits/8]`` + ``scale/bias[NB, Hkv, bs, D/64]`` -> fp32 ``[NB, bs, Hkv, D]``."""
    codes = unpack_codes(code_cache, bits)               # [NB, Hkv, D, bs]
    codes = np.ascontiguousarray(np.transpose(codes, (0, 3, 1, 2)))  # [NB, bs, Hkv, D]
    s = np.transpose(scale, (0, 2, 1, 3))
    b = np.transpose(bias, (0, 2, 1, 3))
    return dequantize_rows(codes, s, b)
