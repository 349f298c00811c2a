"""Generate the golden fixtures in this directory from the easymlx reference.

Run once, on a machine that has the reference checkout:

    python tests/golden/make_golden.py --reference <easymlx checkout>

The script imports the reference's own ``PageCacheView`` / ``paged_attention`` /
``UnifiedAttention`` (through the NumPy stand-in for ``mlx.core`` in
``mlx_shim/``) and records what the reference returned.  The fixtures pin the
CPU oracle in ``oracle/`` and, through it, the CUDA path.

Fixture kinds:

  ref_*.npz          replays of the reference's own seeded tests; inputs are built in
                     the reference's order (its ``append``) and stored whole (they are tiny):
                       ref_attn_seed0/1/11  tests/operations/test_unified_attention.py:86-145,148-208,211-265
                       ref_write_seed2      tests/operations/test_unified_attention.py:268-345
                       ref_performer_seed0  tests/layers/test_attention_performer.py:114-170
  attn_*.npz         ``paged_attention(..., use_metal=False)`` = the reference's NumPy path
                     (operations/kernels/unified_attention.py:187-281) on inputs from
                     ``cases.attention_inputs``; only the output and an input digest are stored.
  dense_single_*.npz one sequence with several query tokens through
                     ``UnifiedAttention.forward_native`` (unified_attention.py:1658-1673 ->
                     page_attention.py:84-133).
  write_*.npz        ``PageCacheView.concatenate_to_cache`` (caching/paged/cache.py:1088-1306)
                     on inputs from ``cases.write_inputs``; stored as the list of pool rows that
                     changed, their new contents, the new lengths and the returned metadata.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def _import_reference(reference_root: str):
    sys.path.insert(0, os.path.join(HERE, "mlx_shim"))
    sys.path.insert(1, os.path.join(reference_root, "lib", "python"))
    import mlx.core as mx  # the stand-in
    from easymlx.caching.paged.cache import PageCacheView, PageMetadata, build_query_start_loc
    from easymlx.operations.kernels.unified_attention import UnifiedAttention, paged_attention

    return mx, PageCacheView, PageMetadata, build_query_start_loc, UnifiedAttention, paged_attention


def _null_packed(cache):
    # The engine drops the packed side caches before use (esurge_engine.py:1367-1379);
    # without this the ragged write calls a Metal-only kernel.
    cache.page_key_cache = None
    cache.page_value_cache = None
    cache.page_vec_size = 0
    return cache


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the easymlx checkout")
    args = ap.parse_args()
    mx, PageCacheView, PageMetadata, build_qsl, UnifiedAttention, paged_attention = _import_reference(args.reference)

    def save(name, **arrays):
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(f"{name}: {os.path.getsize(path)} bytes; " + ", ".join(f"{k}{tuple(np.shape(v))}" for k, v in arrays.items()))

    # ---------------------------------------------------------------- replays of the reference's tests
    def replay_attention(name, seed, seq_lens, query_lens, hq, hkv, d, bs, q_per_seq):
        rng = np.random.default_rng(seed)
        cache = PageCacheView.allocate(num_seqs=len(seq_lens), max_seq_len=max(seq_lens), num_kv_heads=hkv,
                                       head_dim=d, block_size=bs, dtype=mx.float32)
        for i, n in enumerate(seq_lens):
            k = mx.array(rng.standard_normal((n, hkv, d)).astype(np.float32))
            v = mx.array(rng.standard_normal((n, hkv, d)).astype(np.float32))
            cache.append(i, k, v)
        if q_per_seq:
            q = np.concatenate([rng.standard_normal((n, hq, d)).astype(np.float32) for n in query_lens], axis=0)
        else:
            q = rng.standard_normal((sum(query_lens), hq, d)).astype(np.float32)
        qsl = build_qsl(query_lens)
        scale = 1.0 / np.sqrt(d)
        out = paged_attention(mx.array(q), cache.key_cache, cache.value_cache, cache.block_tables, cache.kv_lens,
                              qsl, softmax_scale=scale, sliding_window=0, use_metal=False)
        save(name, q=q, key_cache=np.asarray(cache.key_cache), value_cache=np.asarray(cache.value_cache),
             block_tables=np.asarray(cache.block_tables), kv_lens=np.asarray(cache.kv_lens),
             query_start_loc=np.asarray(qsl), scale=np.float32(scale), window=np.int32(0), out=np.asarray(out))

    replay_attention("ref_attn_seed0", 0, [5, 3], [2, 1], 2, 1, 4, 4, True)
    replay_attention("ref_attn_seed1", 1, [6, 4], [2, 1], 4, 2, 8, 4, True)
    replay_attention("ref_attn_seed11", 11, [5, 7, 3], [1, 1, 1], 4, 2, 8, 4, False)

    def replay_write_seed2():
        rng = np.random.default_rng(2)
        cache = _null_packed(PageCacheView.allocate(num_seqs=3, max_seq_len=8, num_kv_heads=1, head_dim=4,
                                                    block_size=4, dtype=mx.float32))
        for slot, n in enumerate([1, 0, 2]):
            if n == 0:
                continue
            k = mx.array(rng.standard_normal((n, 1, 4)).astype(np.float32))
            v = mx.array(rng.standard_normal((n, 1, 4)).astype(np.float32))
            cache.append(slot, k, v)
        before = dict(key_cache_before=np.asarray(cache.key_cache).copy(),
                      value_cache_before=np.asarray(cache.value_cache).copy(),
                      kv_lens_before=np.asarray(cache.kv_lens).copy(),
                      block_tables_all=np.asarray(cache.block_tables).copy())
        qlens = [2, 0, 3]
        qsl = build_qsl(qlens)
        q = rng.standard_normal((5, 2, 4)).astype(np.float32)
        k = rng.standard_normal((5, 1, 4)).astype(np.float32)
        v = rng.standard_normal((5, 1, 4)).astype(np.float32)
        pq, kc, vc, meta = cache.concatenate_to_cache(mx.array(q), mx.array(k), mx.array(v),
                                                      cache_metadata=PageMetadata(query_start_loc=qsl),
                                                      slot_ids=[0, 1, 2])
        save("ref_write_seed2", q=q, k=k, v=v, slot_ids=np.asarray([0, 1, 2], dtype=np.int32),
             query_lens=np.asarray(qlens, dtype=np.int32), block_size=np.int32(4), **before,
             key_cache_after=np.asarray(kc), value_cache_after=np.asarray(vc),
             kv_lens_after=np.asarray(cache.kv_lens), prepared_queries=np.asarray(pq),
             meta_block_tables=np.asarray(meta.block_tables), meta_kv_lens=np.asarray(meta.kv_lens))

    replay_write_seed2()

    def replay_performer_seed0():
        rng = np.random.default_rng(0)
        hq, hkv, d = 2, 1, 4
        cache = _null_packed(PageCacheView.allocate(num_seqs=2, max_seq_len=8, num_kv_heads=hkv, head_dim=d,
                                                    block_size=4, dtype=mx.float32))
        k0 = rng.standard_normal((2, hkv, d)).astype(np.float32)
        v0 = rng.standard_normal((2, hkv, d)).astype(np.float32)
        k1 = rng.standard_normal((1, hkv, d)).astype(np.float32)
        v1 = rng.standard_normal((1, hkv, d)).astype(np.float32)
        cache.append(0, mx.array(k0), mx.array(v0))
        cache.append(1, mx.array(k1), mx.array(v1))
        before = dict(key_cache_before=np.asarray(cache.key_cache).copy(),
                      value_cache_before=np.asarray(cache.value_cache).copy(),
                      kv_lens_before=np.asarray(cache.kv_lens).copy(),
                      block_tables_all=np.asarray(cache.block_tables).copy())
        qlens = [2, 1]
        q = rng.standard_normal((3, hq, d)).astype(np.float32)
        k = rng.standard_normal((3, hkv, d)).astype(np.float32)
        v = rng.standard_normal((3, hkv, d)).astype(np.float32)
        qsl = build_qsl(qlens)
        pq, kc, vc, meta = cache.concatenate_to_cache(
            mx.array(q), mx.array(k), mx.array(v), cache_metadata=PageMetadata(query_start_loc=qsl, slot_ids=(0, 1)))
        scale = 1.0 / np.sqrt(d)
        # two sequences: the op goes to paged_attention (unified_attention.py:1675-1683)
        res = UnifiedAttention(use_metal=False)(query=pq, key=kc, value=vc, cache_metadata=meta, cache_view=cache,
                                                scale=scale)
        save("ref_performer_seed0", q=q, k=k, v=v, slot_ids=np.asarray([0, 1], dtype=np.int32),
             query_lens=np.asarray(qlens, dtype=np.int32), block_size=np.int32(4), scale=np.float32(scale), **before,
             key_cache_after=np.asarray(kc), value_cache_after=np.asarray(vc),
             kv_lens_after=np.asarray(cache.kv_lens), out=np.asarray(res.attention_outputs))

    replay_performer_seed0()

    # ---------------------------------------------------------------- seeded attention cases
    for name, spec in cases.ATTENTION_CASES.items():
        x = cases.attention_inputs(**spec)
        out = paged_attention(mx.array(x["q"]), mx.array(x["key_cache"]), mx.array(x["value_cache"]),
                              mx.array(x["block_tables"]), mx.array(x["kv_lens"]), mx.array(x["query_start_loc"]),
                              softmax_scale=x["scale"], sliding_window=x["window"], use_metal=False)
        save(name, out=np.asarray(out), input_digest=np.asarray(cases.digest(
            x["q"], x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"], x["query_start_loc"])))

    for name, spec in cases.DENSE_SINGLE_CASES.items():
        x = cases.attention_inputs(**spec)
        meta = PageMetadata(query_start_loc=mx.array(x["query_start_loc"]), block_tables=mx.array(x["block_tables"]),
                            kv_lens=mx.array(x["kv_lens"]), block_size=spec["bs"], sliding_window=x["window"],
                            is_single_token_decode=False)
        res = UnifiedAttention()(query=mx.array(x["q"]), key=mx.array(x["key_cache"]), value=mx.array(x["value_cache"]),
                                 cache_metadata=meta, cache_view=None, scale=x["scale"])
        save(name, out=np.asarray(res.attention_outputs), input_digest=np.asarray(cases.digest(
            x["q"], x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"], x["query_start_loc"])))

    # ---------------------------------------------------------------- seeded write cases
    mxdt = {np.dtype(np.float32): mx.float32, np.dtype(np.float16): mx.float16}
    for name, spec in cases.WRITE_CASES.items():
        x = cases.write_inputs(**spec)
        cache = _null_packed(PageCacheView(
            key_cache=mx.array(x["key_cache"]), value_cache=mx.array(x["value_cache"]),
            block_tables=mx.array(x["block_tables"]), kv_lens=mx.array(x["kv_lens"]), block_size=x["block_size"],
            num_kv_heads=spec["hkv"], head_dim=spec["d"]))
        assert cache.key_cache.dtype == mxdt[x["key_cache"].dtype]
        qsl = build_qsl(x["query_lens"].tolist())
        pq, kc, vc, meta = cache.concatenate_to_cache(
            mx.array(x["q"]), mx.array(x["k"]), mx.array(x["v"]), cache_metadata=PageMetadata(query_start_loc=qsl),
            slot_ids=x["slot_ids"].tolist(),
            query_lens=x["query_lens"].tolist() if name in cases.WRITE_DECODE_HINT else None)
        kc = np.asarray(kc).reshape(-1, spec["hkv"], spec["d"])
        vc = np.asarray(vc).reshape(-1, spec["hkv"], spec["d"])
        k0 = x["key_cache"].reshape(kc.shape)
        v0 = x["value_cache"].reshape(vc.shape)
        changed = np.nonzero(np.any(kc != k0, axis=(1, 2)) | np.any(vc != v0, axis=(1, 2)))[0]
        assert np.array_equal(np.asarray(pq), x["q"])  # no RoPE: queries pass through
        save(name, changed_rows=changed.astype(np.int64), key_rows=kc[changed], value_rows=vc[changed],
             kv_lens_after=np.asarray(cache.kv_lens), meta_block_tables=np.asarray(meta.block_tables),
             meta_kv_lens=np.asarray(meta.kv_lens), query_start_loc=np.asarray(qsl),
             input_digest=np.asarray(cases.digest(x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"],
                                                  x["k"], x["v"], x["slot_ids"], x["query_lens"])))


if __name__ == "__main__":
    main()
