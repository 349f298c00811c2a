"""Seeded input builders shared by ``make_golden.py`` (which feeds them to the
easymlx reference and stores what it returns) and by the tests (which rebuild
the same inputs and compare the oracle / the CUDA path with the stored outputs).

Only NumPy.  Every builder is a pure function of its arguments; the fixture
files store a digest of the inputs so that a drift in the generator is caught.
"""

from __future__ import annotations

import hashlib

import numpy as np


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        a = np.ascontiguousarray(a)
        h.update(str(a.dtype).encode())
        h.update(str(a.shape).encode())
        h.update(a.tobytes())
    return h.hexdigest()


# --------------------------------------------------------------------------- attention inputs

def attention_inputs(seed, *, hq, hkv, d, bs, ctx, qlens, window=0, dtype="float16", pool_extra=3, scale=None):
    """Random pool, permuted and -1 padded page tables; kv_len = ctx + q_len for scheduled rows."""
    rng = np.random.default_rng(seed)
    dtype = np.dtype(dtype)
    ctx = np.asarray(ctx, dtype=np.int64)
    qlens = np.asarray(qlens, dtype=np.int64)
    kv = np.where(qlens > 0, ctx + qlens, ctx)
    pages = (kv + bs - 1) // bs
    nb = int(pages.sum()) + pool_extra
    mb = int(max(1, pages.max())) + 2
    perm = rng.permutation(nb)
    bt = -np.ones((len(kv), mb), dtype=np.int32)
    cursor = 0
    for i, n in enumerate(pages):
        bt[i, :n] = perm[cursor:cursor + n]
        cursor += n
    kc = rng.standard_normal((nb, bs, hkv, d)).astype(dtype)
    vc = rng.standard_normal((nb, bs, hkv, d)).astype(dtype)
    q = rng.standard_normal((int(qlens.sum()), hq, d)).astype(dtype)
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    return dict(
        q=q, key_cache=kc, value_cache=vc, block_tables=bt, kv_lens=kv.astype(np.int32), query_start_loc=qsl,
        scale=float(scale) if scale is not None else float(1.0 / np.sqrt(d)), window=int(window),
    )


ATTENTION_CASES = {
    "attn_f16_decode_d128": dict(seed=101, hq=32, hkv=8, d=128, bs=128, ctx=[300, 1, 127, 128, 129, 700], qlens=[1] * 6),
    "attn_f16_decode_d64": dict(seed=102, hq=32, hkv=8, d=64, bs=128, ctx=[255, 256, 511, 40], qlens=[1] * 4),
    "attn_f16_mixed_d128": dict(seed=103, hq=16, hkv=4, d=128, bs=128, ctx=[0, 200, 37, 0, 130], qlens=[150, 1, 5, 0, 64]),
    "attn_f16_mixed_d64": dict(seed=104, hq=32, hkv=8, d=64, bs=128, ctx=[0, 0, 300, 511], qlens=[130, 7, 1, 1]),
    "attn_f16_specverify": dict(seed=105, hq=32, hkv=8, d=128, bs=128, ctx=[126, 250, 600], qlens=[5, 5, 5]),
    "attn_f16_window": dict(seed=106, hq=8, hkv=2, d=128, bs=128, ctx=[400, 90, 0, 260], qlens=[1, 6, 140, 1], window=100),
    "attn_f16_gqa8": dict(seed=107, hq=64, hkv=8, d=128, bs=128, ctx=[70, 513, 0], qlens=[1, 1, 40]),
    "attn_f16_mha_smallpage": dict(seed=108, hq=4, hkv=4, d=32, bs=16, ctx=[20, 0, 33], qlens=[1, 9, 3], scale=0.25),
    "attn_f32_d256": dict(seed=109, hq=4, hkv=2, d=256, bs=8, ctx=[10, 0], qlens=[1, 12], dtype="float32"),
    "attn_f16_empty_rows": dict(seed=110, hq=8, hkv=2, d=64, bs=128, ctx=[0, 50, 0], qlens=[0, 1, 0]),
}

# One sequence, several query tokens: the reference routes these through a dense masked
# softmax that rounds the probabilities to the value dtype before the PV product.
DENSE_SINGLE_CASES = {
    "dense_single_f16": dict(seed=201, hq=8, hkv=2, d=128, bs=128, ctx=[200], qlens=[5], pool_extra=2),
    "dense_single_f32_window": dict(seed=202, hq=4, hkv=2, d=64, bs=16, ctx=[40], qlens=[9], window=16,
                                    dtype="float32", pool_extra=2),
}


# --------------------------------------------------------------------------- write inputs

def write_inputs(seed, *, num_seqs, max_seq_len, hkv, hq, d, bs, initial_lens, slot_ids, qlens,
                 dtype="float16", in_dtype=None, shuffle_tables=True):
    """A pool pre-filled with random data, per-slot lengths, and one packed batch of new rows.

    The pool geometry is the reference allocator's: ``ceil(max_seq_len/bs)`` pages per slot,
    ``num_seqs`` slots.  With ``shuffle_tables`` the page ids are a random permutation.
    """
    rng = np.random.default_rng(seed)
    dtype = np.dtype(dtype)
    in_dtype = np.dtype(in_dtype or dtype)
    mb = -(-max_seq_len // bs)
    nb = mb * num_seqs
    bt = np.arange(nb, dtype=np.int32).reshape(num_seqs, mb)
    if shuffle_tables:
        bt = rng.permutation(nb).astype(np.int32).reshape(num_seqs, mb)
    kc = rng.standard_normal((nb, bs, hkv, d)).astype(dtype)
    vc = rng.standard_normal((nb, bs, hkv, d)).astype(dtype)
    t = int(np.sum(qlens))
    q = rng.standard_normal((t, hq, d)).astype(in_dtype)
    k = rng.standard_normal((t, hkv, d)).astype(in_dtype)
    v = rng.standard_normal((t, hkv, d)).astype(in_dtype)
    return dict(
        key_cache=kc, value_cache=vc, block_tables=bt, kv_lens=np.asarray(initial_lens, dtype=np.int32),
        q=q, k=k, v=v, slot_ids=np.asarray(slot_ids, dtype=np.int32), query_lens=np.asarray(qlens, dtype=np.int32),
        block_size=int(bs),
    )


WRITE_CASES = {
    # decode fast path of the reference (every row one token, query_lens passed explicitly)
    "write_decode_f16": dict(seed=301, num_seqs=6, max_seq_len=512, hkv=8, hq=32, d=128, bs=128,
                             initial_lens=[127, 128, 0, 300, 5, 255], slot_ids=[4, 0, 3, 1, 5], qlens=[1, 1, 1, 1, 1]),
    # ragged path, page-boundary crossings, an empty row, non-identity slot order
    "write_ragged_f16": dict(seed=302, num_seqs=5, max_seq_len=640, hkv=4, hq=16, d=64, bs=128,
                             initial_lens=[120, 0, 255, 3, 0], slot_ids=[2, 4, 0, 3], qlens=[5, 200, 17, 0]),
    # fp32 inputs cast to an fp16 pool
    "write_ragged_cast": dict(seed=303, num_seqs=3, max_seq_len=64, hkv=2, hq=4, d=32, bs=16,
                              initial_lens=[15, 0, 31], slot_ids=[0, 1, 2], qlens=[3, 20, 2], in_dtype="float32"),
    # spec-verify shape: 5 rows per sequence straddling a page edge
    "write_specverify_f16": dict(seed=304, num_seqs=4, max_seq_len=384, hkv=8, hq=32, d=128, bs=128,
                                 initial_lens=[126, 250, 0, 128], slot_ids=[3, 1, 0, 2], qlens=[5, 5, 5, 5]),
}
WRITE_DECODE_HINT = {"write_decode_f16"}
