"""Rotary embedding: oracle properties on CPU; fused write kernel vs the oracle on GPU."""

import numpy as np
import pytest
import torch

import cases
from oracle import kv_quant, kv_write, rope as orope


def test_oracle_rotation_is_norm_preserving_and_relative():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((6, 2, 64)).astype(np.float32)
    y = rng.standard_normal((6, 2, 64)).astype(np.float32)
    freqs = orope.default_freqs(64, 10000.0)
    for trad in (False, True):
        p = np.array([0, 1, 5, 17, 300, 4000])
        rx = orope.rotate(x, p, freqs, 64, traditional=trad)
        np.testing.assert_allclose(np.linalg.norm(rx, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-5)
        # scores depend on the position difference only
        ry = orope.rotate(y, p + 7, freqs, 64, traditional=trad)
        rx2, ry2 = orope.rotate(x, p + 100, freqs, 64, traditional=trad), orope.rotate(y, p + 107, freqs, 64, traditional=trad)
        np.testing.assert_allclose((rx * ry).sum(-1), (rx2 * ry2).sum(-1), atol=2e-3)
    np.testing.assert_array_equal(orope.rotate(x, np.zeros(6), freqs, 64), x)


def test_factory_tables_match_the_oracle_restatement():
    from easymlx_b200.layers import get_rope

    r = get_rope(128, 500000.0, False, {"type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                        "original_max_position_embeddings": 8192}, 131072)
    np.testing.assert_allclose(r.freqs, orope.llama3_freqs(128, 500000.0, 8.0), rtol=1e-6)
    lin = get_rope(64, 10000.0, True, {"type": "linear", "factor": 4.0})
    assert lin.scale == 0.25 and lin.traditional
    with pytest.raises(ValueError):
        get_rope(64, 10000.0, False, {"type": "nope"})


def test_longrope_picks_its_table_by_sequence_length():
    """Su-scaled rotary embedding (layers/rotary/_rotary.py:36-131 of the reference): periods are the base periods
    times the short or the long factors, the magnitude scale is sqrt(1 + ln(factor) / ln(original_max)), and the long
    table applies to sequences of more than original_max tokens."""
    import math

    from easymlx_b200.layers import LongRopeEmbedding, get_rope

    short, long_ = [1.0 + 0.01 * i for i in range(16)], [2.0 + 0.5 * i for i in range(16)]
    r = get_rope(32, 10000.0, False, {"type": "longrope", "original_max_position_embeddings": 4096,
                                      "short_factor": short, "long_factor": long_}, 131072)
    assert isinstance(r, LongRopeEmbedding)
    base = np.float32(10000.0) ** (np.arange(0, 32, 2, dtype=np.float32) / np.float32(32))
    np.testing.assert_allclose(r.short.freqs, np.asarray(short, np.float32) * base, rtol=1e-6)
    np.testing.assert_allclose(r.long.freqs, np.asarray(long_, np.float32) * base, rtol=1e-6)
    want = math.sqrt(1 + math.log(131072 / 4096) / math.log(4096))
    assert abs(r.short.mscale - want) < 1e-12 and abs(r.long.mscale - want) < 1e-12
    assert r.select(4096) is r.short and r.select(4097) is r.long
    same = get_rope(32, 10000.0, False, {"rope_type": "longrope", "original_max_position_embeddings": 4096,
                                         "short_factor": short, "long_factor": long_}, 4096)
    assert same.short.mscale == 1.0  # no length extension: no magnitude change


@pytest.mark.gpu
def test_longrope_in_the_cache_write_uses_the_long_table_past_the_threshold():
    import easymlx_b200 as emlx
    from easymlx_b200.layers import get_rope

    long_ = [1.0 + 0.25 * i for i in range(32)]
    rope = get_rope(64, 10000.0, False, {"type": "longrope", "original_max_position_embeddings": 256,
                                         "short_factor": [1.0] * 32, "long_factor": long_}, 1024)
    hkv, hq, d, bs = 2, 4, 64, 128
    rng = np.random.default_rng(1)
    for base_len, table in ((100, rope.short), (300, rope.long)):
        cache = emlx.PageCacheView.init(num_seqs=1, max_seq_len=512, num_kv_heads=hkv, head_dim=d, block_size=bs)
        cache.kv_lens.fill_(base_len)
        q = rng.standard_normal((3, hq, d)).astype(np.float16)
        k = rng.standard_normal((3, hkv, d)).astype(np.float16)
        meta = emlx.PageMetadata(query_start_loc=emlx.build_query_start_loc([3]))
        pq, kc, _, _ = cache.concatenate_to_cache(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                                                  torch.from_numpy(k).cuda(), cache_metadata=meta, slot_ids=[0],
                                                  query_lens=[3], rope=rope)
        pos = base_len + np.arange(3)
        want_q = orope.rotate(q, pos, table.freqs, 64, mscale=table.mscale)
        np.testing.assert_allclose(pq.float().cpu().numpy(), want_q.astype(np.float32), atol=4e-3, rtol=2e-3)
        x = torch.from_numpy(q).cuda()
        assert torch.equal(rope(x.reshape(1, 3, hq, d).permute(0, 2, 1, 3), offset=base_len).permute(0, 2, 1, 3).reshape(3, hq, d), pq)


@pytest.mark.gpu
@pytest.mark.parametrize("traditional", [False, True])
@pytest.mark.parametrize("bits", [0, 8])
def test_fused_rope_write_matches_oracle(traditional, bits):
    import easymlx_b200 as emlx
    from easymlx_b200.layers import RotaryEmbedding

    spec = cases.WRITE_CASES["write_specverify_f16"]
    x = cases.write_inputs(**spec)
    hkv, d, bs = spec["hkv"], spec["d"], x["block_size"]
    rope = RotaryEmbedding(64, base=10000.0, traditional=traditional, scale=0.5, mscale=1.25)  # partial rotation: 64 of 128
    cache = emlx.PageCacheView.init(num_seqs=spec["num_seqs"], max_seq_len=spec["max_seq_len"], num_kv_heads=hkv,
                                    head_dim=d, block_size=bs, cache_bits=bits or None, cache_dtype="affine" if bits else None)
    cache.block_tables.copy_(torch.from_numpy(x["block_tables"]))
    cache.kv_lens.copy_(torch.from_numpy(x["kv_lens"]))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    meta = emlx.PageMetadata(query_start_loc=emlx.build_query_start_loc(x["query_lens"].tolist()))
    pq, kc, vc, resolved = cache.concatenate_to_cache(dev(x["q"]), dev(x["k"]), dev(x["v"]), cache_metadata=meta,
                                                      slot_ids=x["slot_ids"].tolist(), rope=rope)
    cache.check()
    m = kv_write.batch_metadata(x["query_lens"], x["slot_ids"], x["block_tables"], x["kv_lens"], bs)
    want_q = orope.rotate(x["q"], m["token_positions"], rope.freqs, 64, traditional=traditional, scale=0.5, mscale=1.25)
    want_k = orope.rotate(x["k"], m["token_positions"], rope.freqs, 64, traditional=traditional, scale=0.5, mscale=1.25)
    np.testing.assert_allclose(pq.float().cpu().numpy(), want_q.astype(np.float32), atol=4e-3, rtol=2e-3)
    slots = torch.from_numpy(m["slot_mapping"]).cuda()
    if bits == 0:
        got_k = kc.reshape(-1, hkv, d)[slots].float().cpu().numpy()
        got_v = vc.reshape(-1, hkv, d)[slots].cpu().numpy()
        np.testing.assert_allclose(got_k, want_k.astype(np.float32), atol=4e-3, rtol=2e-3)
        np.testing.assert_array_equal(got_v, x["v"])            # values are not rotated
    else:
        page, off = m["slot_mapping"] // bs, m["slot_mapping"] % bs
        codes = kc.reshape(-1, hkv, d)[slots].cpu().numpy()
        pg, of = torch.from_numpy(page).cuda(), torch.from_numpy(off).cuda()
        deq = kv_quant.dequantize_rows(codes, cache.k_scales[pg, :, of].cpu().numpy(), cache.k_biases[pg, :, of].cpu().numpy())
        step = cache.k_scales[pg, :, of].float().cpu().numpy().max()
        np.testing.assert_allclose(deq, want_k.astype(np.float32), atol=0.6 * step + 4e-3)
    # the stand-alone call rotates the same way
    alone = rope(dev(x["q"]), offset=dev(m["token_positions"]))
    assert torch.equal(alone, pq)
    b4 = rope(dev(x["q"][:6]).reshape(1, 6, -1, d).permute(0, 2, 1, 3), offset=11)
    want4 = orope.rotate(x["q"][:6], 11 + np.arange(6), rope.freqs, 64, traditional=traditional, scale=0.5, mscale=1.25)
    np.testing.assert_allclose(b4.permute(0, 2, 1, 3).reshape(6, -1, d).float().cpu().numpy(), want4.astype(np.float32),
                               atol=4e-3, rtol=2e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("traditional", [False, True])
def test_rotation_at_long_context_positions(traditional):
    """Positions up to 131 071 with the llama3 table: the angle reaches 1e5 rad, where a fast sine would be off by
    several per cent; the kernel and the oracle both reduce the fp32 angle exactly."""
    from easymlx_b200.layers import get_rope

    rope = get_rope(128, 500000.0, traditional, {"type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                 "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}, 131072)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((64, 4, 128)).astype(np.float16)
    pos = np.concatenate([rng.integers(100_000, 131_072, size=60), [0, 1, 131_071, 65_536]]).astype(np.int32)
    got = rope(torch.from_numpy(x).cuda(), offset=torch.from_numpy(pos).cuda())
    want = orope.rotate(x, pos, rope.freqs, 128, traditional=traditional, scale=rope.scale, mscale=rope.mscale)
    np.testing.assert_allclose(got.float().cpu().numpy(), want.astype(np.float32), atol=4e-3, rtol=2e-3)
