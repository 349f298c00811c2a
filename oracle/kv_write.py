"""CPU oracle for batch metadata and the paged KV write.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Restates, with paths relative to ``lib/python/easymlx``:

* ``build_query_start_loc``          -> ``caching/paged/cache.py:1448-1465``
* ``batch_metadata``                 -> the index arithmetic of
  ``PageCacheView.concatenate_to_cache`` (``caching/paged/cache.py:1123-1169,1214-1261,1300-1305``):
  per-row base length, per-token position, page id, in-page offset, flat slot
  ``page*bs + offset``, the new lengths and the gathered rows handed to attention.
* ``write_rows``                     -> the scatter itself (``cache.py:1186-1190,1278-1282``),
  including the cast to the pool dtype (``cache.py:830-832``).
* ``append``                         -> ``PageCacheView.append`` (``cache.py:834-872``).
* ``write_key_rows_quantized`` / ``write_value_rows_quantized`` -> this build's affine extension (see ``kv_quant.py``;
  PARITY UNPINNED), same placement rule.

One deliberate difference from the reference, which applies to caller errors only: a
position whose page id is negative is skipped here (slot -1), as ``append`` does
(``cache.py:861-862``); the reference's fancy-index scatter would wrap to the pool's
last page.  The fixtures never contain that situation.

Pinned by ``tests/golden/write_*.npz`` and ``ref_write_seed2.npz`` (outputs of the
reference's own ``concatenate_to_cache``).
"""

from __future__ import annotations

import numpy as np

from . import kv_quant


def build_query_start_loc(query_lens):
    out = np.zeros(len(query_lens) + 1, dtype=np.int32)
    np.cumsum(np.asarray(query_lens, dtype=np.int64), out=out[1:])
    return out


def batch_metadata(query_lens, slot_ids, block_tables_all, kv_lens_all, block_size):
    """Everything the write and the attention need for one packed batch.

    Returns a dict with ``query_start_loc[S+1]``, ``slot_mapping[T]`` (int64, -1 = skip),
    ``kv_lens_all`` after the step, and the gathered ``block_tables[S, MB]`` / ``kv_lens[S]``.
    Rows with ``query_len <= 0`` write nothing and keep their length.
    """
    q_lens = np.maximum(np.asarray(query_lens, dtype=np.int64), 0)
    slots = np.asarray(slot_ids, dtype=np.int64)
    bt = np.asarray(block_tables_all)
    base = np.asarray(kv_lens_all, dtype=np.int64)[slots]
    qsl = build_query_start_loc(q_lens)
    total = int(qsl[-1])
    token_row = np.repeat(np.arange(len(slots)), q_lens)
    token_pos = base[token_row] + (np.arange(total) - qsl[:-1].astype(np.int64)[token_row])
    page_idx = token_pos // block_size
    in_range = page_idx < bt.shape[1]
    page = np.where(in_range, bt[slots[token_row], np.minimum(page_idx, bt.shape[1] - 1)], -1).astype(np.int64)
    slot_mapping = np.where(page >= 0, page * block_size + token_pos % block_size, -1)
    new_lens = np.asarray(kv_lens_all, dtype=np.int32).copy()
    new_lens[slots] = (base + q_lens).astype(np.int32)
    return dict(
        query_start_loc=qsl,
        slot_mapping=slot_mapping.astype(np.int64),
        token_positions=token_pos.astype(np.int32),
        kv_lens_all=new_lens,
        block_tables=bt[slots].astype(np.int32),
        kv_lens=new_lens[slots],
    )


def write_rows(key_cache, value_cache, keys, values, slot_mapping):
    """In-place scatter of ``keys/values[T, Hkv, D]`` into ``[NB, bs, Hkv, D]`` pools."""
    kc = key_cache.reshape((-1,) + key_cache.shape[2:])
    vc = value_cache.reshape((-1,) + value_cache.shape[2:])
    ok = slot_mapping >= 0
    kc[slot_mapping[ok]] = np.asarray(keys)[ok].astype(key_cache.dtype)
    vc[slot_mapping[ok]] = np.asarray(values)[ok].astype(value_cache.dtype)


def write_key_rows_quantized(code_cache, scale, bias, rows, slot_mapping, bits):
    """Quantise ``rows[T, Hkv, D]`` and scatter into a key pool (layouts in ``kv_quant``)."""
    nb, bs, hkv, _ = code_cache.shape
    codes, s, b = kv_quant.quantize_rows(rows, bits)
    packed = kv_quant.pack_codes(codes, bits)
    flat_codes = code_cache.reshape(nb * bs, hkv, -1)
    ok = slot_mapping >= 0
    slots = slot_mapping[ok]
    flat_codes[slots] = packed[ok]
    page, off = slots // bs, slots % bs
    for h in range(hkv):
        scale[page, h, off] = s[ok][:, h]
        bias[page, h, off] = b[ok][:, h]


def write_value_rows_quantized(code_cache, scale, bias, rows, slot_mapping, bits):
    """Quantise ``rows[T, Hkv, D]`` and scatter into a value pool ``[NB, Hkv, D, bs*bits/8]``."""
    nb, hkv, d, _ = code_cache.shape
    bs = scale.shape[2]
    codes, s, b = kv_quant.quantize_rows(rows, bits)      # [T, Hkv, D]
    for t in np.nonzero(slot_mapping >= 0)[0]:
        page, off = int(slot_mapping[t]) // bs, int(slot_mapping[t]) % bs
        if bits == 8:
            code_cache[page, :, :, off] = codes[t]
        else:
            col = code_cache[page, :, :, off // 2]
            if off & 1:
                code_cache[page, :, :, off // 2] = (col & 0x0F) | (codes[t] << 4)
            else:
                code_cache[page, :, :, off // 2] = (col & 0xF0) | codes[t]
        scale[page, :, off] = s[t]
        bias[page, :, off] = b[t]


def append(key_cache, value_cache, block_tables_all, kv_lens_all, slot, keys, values, block_size):
    """One sequence's rows at its current end; pages with a negative id are skipped."""
    start = int(kv_lens_all[slot])
    for i in range(keys.shape[0]):
        pos = start + i
        page = int(block_tables_all[slot, pos // block_size])
        if page < 0:
            continue
        key_cache[page, pos % block_size] = keys[i].astype(key_cache.dtype)
        value_cache[page, pos % block_size] = values[i].astype(value_cache.dtype)
    kv_lens_all[slot] = start + keys.shape[0]
