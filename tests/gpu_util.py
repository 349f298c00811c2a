"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

from oracle import kv_quant, kv_write

ATOL, RTOL = 2e-3, 1e-2  # the op's stated tolerance: max-abs 2e-3 / rel 1e-2 at fp32 accumulation


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def assert_close(actual, expected, atol=ATOL, rtol=RTOL):
    a = actual.float().cpu().numpy() if isinstance(actual, torch.Tensor) else np.asarray(actual, dtype=np.float32)
    e = np.asarray(expected, dtype=np.float32)
    assert a.shape == e.shape
    err = np.abs(a - e)
    bound = atol + rtol * np.abs(e)
    worst = float((err - bound).max()) if err.size else 0.0
    assert worst <= 0, f"max abs err {err.max():.3e}, worst excess over atol+rtol*|ref| {worst:.3e}"


def quantized_pool_from_float(kc, vc, bits):
    """Quantise a float pool ``[NB, bs, Hkv, D]`` with the oracle; returns the stored arrays."""
    nb, bs, hkv, d = kc.shape
    slots = np.arange(nb * bs, dtype=np.int64)
    kcode = np.zeros((nb, bs, hkv, d * bits // 8), np.uint8)
    vcode = np.zeros((nb, hkv, d, bs * bits // 8), np.uint8)
    sb = lambda: np.zeros((nb, hkv, bs, d // 64), np.float16)
    ks, kb, vs, vb = sb(), sb(), sb(), sb()
    kv_write.write_key_rows_quantized(kcode, ks, kb, kc.reshape(nb * bs, hkv, d), slots, bits)
    vcodes, s, b = kv_quant.quantize_rows(vc, bits)          # [NB, bs, Hkv, D]
    vcode[:] = kv_quant.pack_codes(np.ascontiguousarray(np.transpose(vcodes, (0, 2, 3, 1))), bits)
    vs[:] = np.transpose(s, (0, 2, 1, 3))
    vb[:] = np.transpose(b, (0, 2, 1, 3))
    return kcode, vcode, ks, kb, vs, vb
