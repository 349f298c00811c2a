"""The single-launch cache step (``emlx_kv_write_step`` / ``emlx_kv_write_decode``) against the oracle and against the
two-launch path (``emlx_build_metadata`` + ``emlx_kv_write``).

The reference has the same split: ``PageCacheView.concatenate_to_cache`` takes a fast path when every scheduled
sequence brings exactly one token (``caching/paged/cache.py:1155-1206``) and a ragged path otherwise
(``:1208-1306``); both must place the same rows at the same slots and return the same metadata.
"""

import numpy as np
import pytest
import torch

import cases
from gpu_util import assert_close, dev
from oracle import kv_quant, kv_write, paged_attention as opa, rope as orope

pytestmark = pytest.mark.gpu


def _decode_batch(seed, num_slots, max_seq_len, hkv, hq, d, sched, lens, bits=0):
    """A cache with random page tables and ``lens`` tokens per slot, plus one new token for each slot in ``sched``."""
    import easymlx_b200 as emlx

    rng = np.random.default_rng(seed)
    bs = 128
    cache = emlx.PageCacheView.init(num_seqs=num_slots, max_seq_len=max_seq_len, num_kv_heads=hkv, head_dim=d,
                                    block_size=bs, cache_bits=bits or None, cache_dtype="affine" if bits else None)
    mb = cache.blocks_per_seq
    bt = rng.permutation(num_slots * mb).astype(np.int32).reshape(num_slots, mb)
    cache.block_tables.copy_(torch.from_numpy(bt))
    cache.kv_lens.copy_(torch.from_numpy(np.asarray(lens, dtype=np.int32)))
    for a in (cache.key_cache, cache.value_cache):  # stale contents everywhere
        if a.dtype == torch.uint8:
            a.copy_(torch.from_numpy(rng.integers(0, 256, tuple(a.shape), dtype=np.uint8)))
        else:
            a.copy_(torch.from_numpy(rng.standard_normal(tuple(a.shape)).astype(np.float16)))
    if bits:
        for a in (cache.k_scales, cache.k_biases, cache.v_scales, cache.v_biases):
            a.copy_(torch.from_numpy(rng.standard_normal(tuple(a.shape)).astype(np.float16)))
    t = len(sched)
    q = rng.standard_normal((t, hq, d)).astype(np.float16)
    k = rng.standard_normal((t, hkv, d)).astype(np.float16)
    v = rng.standard_normal((t, hkv, d)).astype(np.float16)
    return cache, bt, q, k, v


def _snapshot(cache):
    arrays = [cache.key_cache, cache.value_cache, cache.kv_lens]
    if cache.is_affine:
        arrays += [cache.k_scales, cache.k_biases, cache.v_scales, cache.v_biases]
    return [a.clone() for a in arrays]


def _step(cache, q, k, v, sched, hint=True, rope=None):
    import easymlx_b200 as emlx

    meta = emlx.PageMetadata(query_start_loc=emlx.build_query_start_loc([1] * len(sched)))
    return cache.concatenate_to_cache(dev(q), dev(k), dev(v), cache_metadata=meta, slot_ids=list(sched),
                                      query_lens=[1] * len(sched) if hint else None, rope=rope)


@pytest.mark.parametrize("bits", [0, 8, 4])
@pytest.mark.parametrize("shape", ["small", "many"])
def test_fused_decode_step_equals_the_two_launch_path(bits, shape, monkeypatch):
    from easymlx_b200.caching.paged import cache as cache_mod

    rng = np.random.default_rng(21)
    if shape == "small":
        num_slots, hkv, hq, d, max_len = 6, 8, 32, 128, 512
        lens, sched = [127, 128, 0, 300, 5, 255], [4, 0, 3, 1, 5]
    else:  # several write CTAs, slots scheduled out of order, some on a page edge
        num_slots, hkv, hq, d, max_len = 331, 2, 8, 64, 640
        lens = rng.integers(0, 639, num_slots)
        lens[:7] = [0, 127, 128, 255, 256, 511, 512]
        sched = rng.permutation(num_slots)[:300].tolist()
    results = []
    for fused in (True, False):
        cache, bt, q, k, v = _decode_batch(7, num_slots, max_len, hkv, hq, d, sched, lens, bits)
        monkeypatch.setattr(cache_mod, "_FUSED_STEP_MAX_SEQS", 2048 if fused else 0)
        pq, kc, vc, meta = _step(cache, q, k, v, sched)
        cache.check()
        assert int(cache.ticket.item()) == 0
        results.append((_snapshot(cache), meta, cache))
    (a, ma, ca), (b, mb_, cb) = results
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    for name in ("query_start_loc", "block_tables", "kv_lens"):
        assert torch.equal(getattr(ma, name), getattr(mb_, name)), name
    # and against the oracle: placement of the new rows and the lengths
    m = kv_write.batch_metadata([1] * len(sched), sched, bt, lens, 128)
    np.testing.assert_array_equal(ca.kv_lens.cpu().numpy(), m["kv_lens_all"])
    np.testing.assert_array_equal(ma.kv_lens.cpu().numpy(), m["kv_lens"])
    np.testing.assert_array_equal(ma.block_tables.cpu().numpy(), m["block_tables"])
    slots = torch.from_numpy(m["slot_mapping"]).cuda()
    if bits == 0:
        np.testing.assert_array_equal(ca.key_cache.reshape(-1, hkv, d)[slots].cpu().numpy(), k)
        np.testing.assert_array_equal(ca.value_cache.reshape(-1, hkv, d)[slots].cpu().numpy(), v)
    else:
        kcodes, ks, kb = kv_quant.quantize_rows(k, bits)
        got = ca.key_cache.reshape(-1, hkv, d * bits // 8)[slots].cpu().numpy()
        np.testing.assert_array_equal(got, kv_quant.pack_codes(kcodes, bits))
        pg, of = slots // 128, slots % 128
        np.testing.assert_array_equal(ca.k_scales[pg, :, of].cpu().numpy().view(np.uint16), ks.view(np.uint16))
        np.testing.assert_array_equal(ca.k_biases[pg, :, of].cpu().numpy().view(np.uint16), kb.view(np.uint16))
    # the work list built inside the fused launch drives the same attention result as the stand-alone one
    import easymlx_b200 as emlx
    extra = dict(k_scale=ca.k_scales, v_scale=ca.v_scales, k_bias=ca.k_biases, v_bias=ca.v_biases) if bits else {}
    with_plan = emlx.paged_attention(dev(q), ca.key_cache, ca.value_cache, ma.block_tables, ma.kv_lens, ma.query_start_loc,
                                     max_query_len=1, plan=ma.plan, **extra)
    own_plan = emlx.paged_attention(dev(q), ca.key_cache, ca.value_cache, ma.block_tables, ma.kv_lens, ma.query_start_loc,
                                    max_query_len=1, **extra)
    assert torch.equal(with_plan, own_plan)


def test_two_fused_decode_steps_back_to_back():
    """No host synchronisation between the steps: the second launch must see the lengths the first one advanced."""
    num_slots, hkv, hq, d = 5, 4, 16, 64
    lens, sched = [126, 127, 0, 383, 200], [3, 0, 1, 4]
    cache, bt, q, k, v = _decode_batch(3, num_slots, 512, hkv, hq, d, sched, lens)
    kc0, vc0 = cache.key_cache.cpu().numpy().copy(), cache.value_cache.cpu().numpy().copy()
    rng = np.random.default_rng(4)
    k2, v2 = rng.standard_normal(k.shape).astype(np.float16), rng.standard_normal(v.shape).astype(np.float16)
    _step(cache, q, k, v, sched)
    _, _, _, meta2 = _step(cache, q, k2, v2, sched)
    cache.check()
    m1 = kv_write.batch_metadata([1] * 4, sched, bt, lens, 128)
    kv_write.write_rows(kc0, vc0, k, v, m1["slot_mapping"])
    m2 = kv_write.batch_metadata([1] * 4, sched, bt, m1["kv_lens_all"], 128)
    kv_write.write_rows(kc0, vc0, k2, v2, m2["slot_mapping"])
    np.testing.assert_array_equal(cache.key_cache.cpu().numpy(), kc0)
    np.testing.assert_array_equal(cache.value_cache.cpu().numpy(), vc0)
    np.testing.assert_array_equal(cache.kv_lens.cpu().numpy(), m2["kv_lens_all"])
    np.testing.assert_array_equal(meta2.kv_lens.cpu().numpy(), m2["kv_lens"])


def test_fused_decode_step_leaves_a_full_row_alone():
    num_slots, hkv, hq, d = 3, 2, 8, 64
    lens, sched = [256, 100, 255], [0, 1, 2]   # slot 0 is full (2 pages of 128)
    cache, bt, q, k, v = _decode_batch(9, num_slots, 256, hkv, hq, d, sched, lens)
    before = cache.key_cache.clone()
    with pytest.raises(RuntimeError, match="outgrows"):
        _step(cache, q, k, v, sched)
    np.testing.assert_array_equal(cache.kv_lens.cpu().numpy(), [256, 101, 256])
    # nothing of slot 0 was touched
    assert torch.equal(cache.key_cache[torch.from_numpy(bt[0]).long().cuda()], before[torch.from_numpy(bt[0]).long().cuda()])


@pytest.mark.parametrize("traditional", [False, True])
def test_fused_decode_step_with_rotary_embedding(traditional):
    from easymlx_b200.layers import RotaryEmbedding

    num_slots, hkv, hq, d = 4, 2, 8, 128
    lens, sched = [127, 300, 0, 41], [2, 0, 3, 1]
    cache, bt, q, k, v = _decode_batch(13, num_slots, 512, hkv, hq, d, sched, lens)
    rope = RotaryEmbedding(64, base=10000.0, traditional=traditional, scale=0.5, mscale=1.25)
    pq, kc, vc, meta = _step(cache, q, k, v, sched, rope=rope)
    cache.check()
    m = kv_write.batch_metadata([1] * 4, sched, bt, lens, 128)
    want_q = orope.rotate(q, m["token_positions"], rope.freqs, 64, traditional=traditional, scale=0.5, mscale=1.25)
    want_k = orope.rotate(k, m["token_positions"], rope.freqs, 64, traditional=traditional, scale=0.5, mscale=1.25)
    np.testing.assert_allclose(pq.float().cpu().numpy(), want_q.astype(np.float32), atol=4e-3, rtol=2e-3)
    slots = torch.from_numpy(m["slot_mapping"]).cuda()
    np.testing.assert_allclose(kc.reshape(-1, hkv, d)[slots].float().cpu().numpy(), want_k.astype(np.float32), atol=4e-3, rtol=2e-3)
    np.testing.assert_array_equal(vc.reshape(-1, hkv, d)[slots].cpu().numpy(), v)


def test_decode_batch_without_host_lengths_attends_like_the_oracle():
    """write + attention through the performer for a decode batch, checked end to end against the oracle."""
    import easymlx_b200 as emlx

    num_slots, hkv, hq, d = 6, 8, 32, 128
    lens, sched = [127, 128, 0, 300, 5, 255], [4, 0, 3, 1, 5]
    cache, bt, q, k, v = _decode_batch(17, num_slots, 512, hkv, hq, d, sched, lens)
    kc0, vc0 = cache.key_cache.cpu().numpy().copy(), cache.value_cache.cpu().numpy().copy()
    meta = emlx.PageMetadata(query_start_loc=emlx.build_query_start_loc([1] * 5), slot_ids=tuple(sched),
                             is_single_token_decode=True)
    out = emlx.AttentionPerformer(scale=d ** -0.5)(dev(q), dev(k), dev(v), cache_view=cache, cache_metadata=meta)
    m = kv_write.batch_metadata([1] * 5, sched, bt, lens, 128)
    kv_write.write_rows(kc0, vc0, k, v, m["slot_mapping"])
    want = opa.paged_attention_rows(q, kc0, vc0, m["block_tables"], m["kv_lens"], m["query_start_loc"], softmax_scale=d ** -0.5)
    assert_close(out, want)


@pytest.mark.parametrize("bits", [0, 8, 4])
@pytest.mark.parametrize("name", ["write_ragged_f16", "write_specverify_f16", "write_ragged_cast", "write_decode_f16"])
def test_ragged_single_launch_step_equals_the_two_launch_path(name, bits, monkeypatch):
    """Ragged batches (page-edge crossings, an empty row, fp32 inputs cast on the way) through both routes: same pool,
    same lengths, same metadata, and a work list that drives the same attention output."""
    import easymlx_b200 as emlx
    from easymlx_b200.caching.paged import cache as cache_mod

    spec = cases.WRITE_CASES[name]
    x = cases.write_inputs(**spec)
    hkv, hq, d, bs = spec["hkv"], spec["hq"], spec["d"], x["block_size"]
    if bits and (d % 64 or bs != 128):
        pytest.skip("affine pools need head_dim % 64 == 0 and 128-token pages here")
    results = []
    for fused in (True, False):
        monkeypatch.setattr(cache_mod, "_FUSED_STEP_MAX_SEQS", 2048 if fused else 0)
        cache = emlx.PageCacheView.init(num_seqs=spec["num_seqs"], max_seq_len=spec["max_seq_len"], num_kv_heads=hkv, head_dim=d,
                                        block_size=bs, cache_bits=bits or None, cache_dtype="affine" if bits else None)
        rng = np.random.default_rng(11)
        for a in (cache.key_cache, cache.value_cache):
            if a.dtype == torch.uint8:
                a.copy_(torch.from_numpy(rng.integers(0, 256, tuple(a.shape), dtype=np.uint8)))
            else:
                a.copy_(torch.from_numpy(rng.standard_normal(tuple(a.shape)).astype(np.float16)))
        if bits:
            for a in (cache.k_scales, cache.k_biases, cache.v_scales, cache.v_biases):
                a.copy_(torch.from_numpy(rng.standard_normal(tuple(a.shape)).astype(np.float16)))
        cache.block_tables.copy_(dev(x["block_tables"]))
        cache.kv_lens.copy_(dev(x["kv_lens"]))
        qlens = x["query_lens"].tolist()
        meta = emlx.PageMetadata(query_start_loc=emlx.build_query_start_loc(qlens))
        _, kc, vc, resolved = cache.concatenate_to_cache(dev(x["q"]), dev(x["k"]), dev(x["v"]), cache_metadata=meta,
                                                         slot_ids=x["slot_ids"].tolist(), query_lens=qlens)
        cache.check()
        assert int(cache.ticket.item()) == 0
        results.append((_snapshot(cache), resolved, cache))
    (a, ma, ca), (b, mb_, _) = results
    for u, w in zip(a, b):
        assert torch.equal(u, w)
    for field in ("query_start_loc", "block_tables", "kv_lens"):
        assert torch.equal(getattr(ma, field), getattr(mb_, field)), field
    m = kv_write.batch_metadata(x["query_lens"], x["slot_ids"], x["block_tables"], x["kv_lens"], bs)
    np.testing.assert_array_equal(ca.kv_lens.cpu().numpy(), m["kv_lens_all"])
    np.testing.assert_array_equal(ma.query_start_loc.cpu().numpy(), m["query_start_loc"])
    if bs == 128 and d in (64, 128) and x["q"].dtype == np.float16:
        extra = dict(k_scale=ca.k_scales, v_scale=ca.v_scales, k_bias=ca.k_biases, v_bias=ca.v_biases) if bits else {}
        args = (dev(x["q"]), ca.key_cache, ca.value_cache, ma.block_tables, ma.kv_lens, ma.query_start_loc)
        with_plan = emlx.paged_attention(*args, max_query_len=int(max(qlens)), plan=ma.plan, **extra)
        own_plan = emlx.paged_attention(*args, max_query_len=int(max(qlens)), **extra)
        assert torch.equal(with_plan, own_plan)


def test_single_launch_step_reports_a_token_count_that_does_not_match():
    import easymlx_b200 as emlx

    cache = emlx.PageCacheView.init(num_seqs=2, max_seq_len=256, num_kv_heads=2, head_dim=64, block_size=128)
    k = torch.zeros((5, 2, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="query_lens"):
        cache.concatenate_to_cache(k.repeat(1, 2, 1), k, k, cache_metadata=emlx.PageMetadata(
            query_start_loc=emlx.build_query_start_loc([2, 2])), slot_ids=[0, 1], query_lens=[2, 2])
