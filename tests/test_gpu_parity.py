"""CUDA path vs the reference's stored outputs and vs the CPU oracle (run with -m gpu on a B200)."""

import numpy as np
import pytest
import torch

import cases
from gpu_util import assert_close, dev, quantized_pool_from_float
from oracle import kv_quant, kv_write, paged_attention as opa

pytestmark = pytest.mark.gpu

KERNELS = ["generic", None]  # None = what a caller gets (tiled where the geometry allows)


def _run(x, kernel, **kw):
    from easymlx_b200 import paged_attention

    return paged_attention(dev(x["q"]), dev(x["key_cache"]), dev(x["value_cache"]), dev(x["block_tables"]),
                           dev(x["kv_lens"]), dev(x["query_start_loc"]), softmax_scale=x["scale"],
                           sliding_window=x["window"], kernel=kernel, **kw)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", ["ref_attn_seed0", "ref_attn_seed1", "ref_attn_seed11"])
def test_reference_test_shapes(golden, name, kernel):
    g = golden(name)
    x = dict(g, scale=float(g["scale"]), window=int(g["window"]))
    out = _run(x, kernel)
    # fp32 in, fp32 out: the reference's own test tolerance
    assert_close(out, g["out"], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", sorted(cases.ATTENTION_CASES))
def test_attention_golden(golden, name, kernel):
    g = golden(name)
    x = cases.attention_inputs(**cases.ATTENTION_CASES[name])
    out = _run(x, kernel)
    assert out.dtype == dev(x["q"]).dtype and out.shape == x["q"].shape
    assert_close(out, g["out"])


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", sorted(cases.DENSE_SINGLE_CASES))
def test_single_sequence_multi_token_golden(golden, name, kernel):
    g = golden(name)
    x = cases.attention_inputs(**cases.DENSE_SINGLE_CASES[name])
    assert_close(_run(x, kernel), g["out"])


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("name", ["attn_f16_decode_d128", "attn_f16_decode_d64", "attn_f16_specverify",
                                  "attn_f16_mixed_d128", "attn_f16_gqa8", "attn_f16_window"])
def test_attention_affine_pool(name, bits, kernel):
    x = cases.attention_inputs(**cases.ATTENTION_CASES[name])
    kcode, vcode, ks, kb, vs, vb = quantized_pool_from_float(x["key_cache"], x["value_cache"], bits)
    kf = kv_quant.dequantize_key_pool(kcode, ks, kb, bits)
    vf = kv_quant.dequantize_value_pool(vcode, vs, vb, bits)
    expect = opa.paged_attention_rows(x["q"], kf, vf, x["block_tables"], x["kv_lens"], x["query_start_loc"],
                                      softmax_scale=x["scale"], sliding_window=x["window"])
    xq = dict(x, key_cache=kcode, value_cache=vcode)
    out = _run(xq, kernel, k_scale=dev(ks), k_bias=dev(kb), v_scale=dev(vs), v_bias=dev(vb))
    assert_close(out, expect)


def test_zero_tokens_returns_zeros():
    from easymlx_b200 import paged_attention

    q = torch.zeros((0, 8, 64), dtype=torch.float16, device="cuda")
    kc = torch.zeros((2, 128, 2, 64), dtype=torch.float16, device="cuda")
    out = paged_attention(q, kc, kc, torch.zeros((0, 1), dtype=torch.int32, device="cuda"),
                          torch.zeros(0, dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda"))
    assert out.shape == q.shape


def test_shape_errors_match_reference():
    from easymlx_b200 import paged_attention

    q = torch.zeros((1, 8, 64), dtype=torch.float16, device="cuda")
    kc = torch.zeros((2, 128, 2, 64), dtype=torch.float16, device="cuda")
    bt = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    lens = torch.ones(1, dtype=torch.int32, device="cuda")
    qsl = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="rank-3"):
        paged_attention(q[0], kc, kc, bt, lens, qsl)
    with pytest.raises(ValueError, match="divisible"):
        paged_attention(q[:, :3], kc, kc, bt, lens, qsl)
    with pytest.raises(ValueError, match="num_seqs \\+ 1"):
        paged_attention(q, kc, kc, bt, lens, qsl[:1])
    with pytest.raises(ValueError, match="head_dim"):
        paged_attention(q[:, :, :32], kc, kc, bt, lens, qsl)


# --------------------------------------------------------------------------- write + metadata

def _cache_from(x, spec):
    from easymlx_b200 import PageCacheView

    return PageCacheView(key_cache=dev(x["key_cache"]), value_cache=dev(x["value_cache"]),
                         block_tables=dev(x["block_tables"]), kv_lens=dev(x["kv_lens"]), block_size=x["block_size"],
                         num_kv_heads=spec["hkv"], head_dim=spec["d"])


@pytest.mark.parametrize("name", sorted(cases.WRITE_CASES))
def test_write_golden(golden, name):
    from easymlx_b200 import PageMetadata, build_query_start_loc

    g = golden(name)
    spec = cases.WRITE_CASES[name]
    x = cases.write_inputs(**spec)
    cache = _cache_from(x, spec)
    qsl = build_query_start_loc(x["query_lens"].tolist())
    hint = x["query_lens"].tolist() if name in cases.WRITE_DECODE_HINT else None
    pq, kc, vc, meta = cache.concatenate_to_cache(dev(x["q"]), dev(x["k"]), dev(x["v"]),
                                                  cache_metadata=PageMetadata(query_start_loc=qsl),
                                                  slot_ids=x["slot_ids"].tolist(), query_lens=hint)
    cache.check()
    exp_k = x["key_cache"].reshape(-1, spec["hkv"], spec["d"]).copy()
    exp_v = x["value_cache"].reshape(-1, spec["hkv"], spec["d"]).copy()
    exp_k[g["changed_rows"]] = g["key_rows"]
    exp_v[g["changed_rows"]] = g["value_rows"]
    np.testing.assert_array_equal(kc.cpu().numpy().reshape(exp_k.shape), exp_k)   # bit-exact placement
    np.testing.assert_array_equal(vc.cpu().numpy().reshape(exp_v.shape), exp_v)
    np.testing.assert_array_equal(cache.kv_lens.cpu().numpy(), g["kv_lens_after"])
    np.testing.assert_array_equal(meta.kv_lens.cpu().numpy(), g["meta_kv_lens"])
    np.testing.assert_array_equal(meta.block_tables.cpu().numpy(), g["meta_block_tables"])
    np.testing.assert_array_equal(meta.query_start_loc.cpu().numpy(), g["query_start_loc"])
    assert torch.equal(pq, dev(x["q"]))


def test_write_reference_seed2_and_performer(golden):
    from easymlx_b200 import AttentionPerformer, PageCacheView, PageMetadata, build_query_start_loc

    g = golden("ref_write_seed2")
    cache = PageCacheView(key_cache=dev(g["key_cache_before"]), value_cache=dev(g["value_cache_before"]),
                          block_tables=dev(g["block_tables_all"]), kv_lens=dev(g["kv_lens_before"]),
                          block_size=int(g["block_size"]), num_kv_heads=1, head_dim=4)
    _, kc, vc, meta = cache.concatenate_to_cache(
        dev(g["q"]), dev(g["k"]), dev(g["v"]),
        cache_metadata=PageMetadata(query_start_loc=build_query_start_loc(g["query_lens"].tolist())), slot_ids=[0, 1, 2])
    np.testing.assert_array_equal(kc.cpu().numpy(), g["key_cache_after"])
    np.testing.assert_array_equal(vc.cpu().numpy(), g["value_cache_after"])
    np.testing.assert_array_equal(meta.kv_lens.cpu().numpy(), g["meta_kv_lens"])
    np.testing.assert_array_equal(meta.block_tables.cpu().numpy(), g["meta_block_tables"])

    g = golden("ref_performer_seed0")
    cache = PageCacheView(key_cache=dev(g["key_cache_before"]), value_cache=dev(g["value_cache_before"]),
                          block_tables=dev(g["block_tables_all"]), kv_lens=dev(g["kv_lens_before"]),
                          block_size=int(g["block_size"]), num_kv_heads=1, head_dim=4)
    performer = AttentionPerformer(scale=float(g["scale"]))
    meta = PageMetadata(query_start_loc=build_query_start_loc(g["query_lens"].tolist()), slot_ids=(0, 1))
    out = performer(dev(g["q"]), dev(g["k"]), dev(g["v"]), cache_view=cache, cache_metadata=meta)
    assert_close(out, g["out"], atol=1e-5, rtol=1e-5)
    np.testing.assert_array_equal(cache.kv_lens.cpu().numpy(), g["kv_lens_after"])
    np.testing.assert_array_equal(cache.key_cache.cpu().numpy(), g["key_cache_after"])


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("name", ["write_decode_f16", "write_specverify_f16", "write_ragged_f16"])
def test_affine_write_is_bit_exact(name, bits):
    from easymlx_b200 import PageCacheView, PageMetadata, build_query_start_loc

    spec = cases.WRITE_CASES[name]
    x = cases.write_inputs(**spec)
    hkv, d, bs = spec["hkv"], spec["d"], x["block_size"]
    nb = x["key_cache"].shape[0]
    cache = PageCacheView.init(num_seqs=spec["num_seqs"], max_seq_len=spec["max_seq_len"], num_kv_heads=hkv,
                               head_dim=d, block_size=bs, cache_bits=bits, cache_dtype="affine")
    rng = np.random.default_rng(7)
    # stale contents everywhere: the kernel must replace exactly the addressed codes / nibbles
    kcode = rng.integers(0, 256, cache.key_cache.shape, dtype=np.uint8)
    vcode = rng.integers(0, 256, cache.value_cache.shape, dtype=np.uint8)
    sb = [rng.standard_normal(cache.k_scales.shape).astype(np.float16) for _ in range(4)]
    cache.key_cache.copy_(dev(kcode)); cache.value_cache.copy_(dev(vcode))
    for t, a in zip((cache.k_scales, cache.k_biases, cache.v_scales, cache.v_biases), sb):
        t.copy_(dev(a))
    cache.block_tables.copy_(dev(x["block_tables"])); cache.kv_lens.copy_(dev(x["kv_lens"]))
    cache.concatenate_to_cache(dev(x["q"]), dev(x["k"]), dev(x["v"]),
                               cache_metadata=PageMetadata(query_start_loc=build_query_start_loc(x["query_lens"].tolist())),
                               slot_ids=x["slot_ids"].tolist())
    cache.check()
    meta = kv_write.batch_metadata(x["query_lens"], x["slot_ids"], x["block_tables"], x["kv_lens"], bs)
    ks, kb, vs, vb = [a.copy() for a in sb]
    kv_write.write_key_rows_quantized(kcode, ks, kb, x["k"], meta["slot_mapping"], bits)
    kv_write.write_value_rows_quantized(vcode, vs, vb, x["v"], meta["slot_mapping"], bits)
    assert nb == cache.num_blocks
    np.testing.assert_array_equal(cache.key_cache.cpu().numpy(), kcode)
    np.testing.assert_array_equal(cache.value_cache.cpu().numpy(), vcode)
    for t, a in zip((cache.k_scales, cache.k_biases, cache.v_scales, cache.v_biases), (ks, kb, vs, vb)):
        np.testing.assert_array_equal(t.cpu().numpy().view(np.uint16), a.view(np.uint16))
    np.testing.assert_array_equal(cache.kv_lens.cpu().numpy(), meta["kv_lens_all"])


def test_two_appends_in_a_row_and_strided_inputs():
    """Launch ordering: every kernel waits for the launch before it, so a second append right behind the first sees the
    advanced length, and rows that a copy kernel has only just made contiguous (views into a fused QKV projection)
    are complete when the write reads them.  Bit-exact against the oracle."""
    from easymlx_b200 import PageCacheView, PageMetadata, build_query_start_loc

    rng = np.random.default_rng(5)
    hkv, hq, d, bs = 4, 8, 64, 128
    cache = PageCacheView.init(num_seqs=3, max_seq_len=512, num_kv_heads=hkv, head_dim=d, block_size=bs)
    bt = rng.permutation(12).astype(np.int32).reshape(3, 4)
    cache.block_tables.copy_(torch.from_numpy(bt))
    kc = np.zeros((12, bs, hkv, d), np.float16)
    vc = np.zeros_like(kc)
    lens = np.zeros(3, np.int32)
    for n in (100, 60, 3, 130):  # back to back on slot 1, crossing a page edge, no synchronisation in between
        k = rng.standard_normal((n, hkv, d)).astype(np.float16)
        v = rng.standard_normal((n, hkv, d)).astype(np.float16)
        cache.append(1, dev(k), dev(v))
        kv_write.append(kc, vc, bt, lens, 1, k, v, bs)
    # a packed batch whose K and V are strided views of one [T, Hq + 2 Hkv, D] projection output
    qlens, slots = [7, 1, 30], [2, 1, 0]
    t = sum(qlens)
    qkv = dev(rng.standard_normal((t, hq + 2 * hkv, d)).astype(np.float16))
    q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
    assert not k.is_contiguous()
    cache.concatenate_to_cache(q, k, v, cache_metadata=PageMetadata(query_start_loc=build_query_start_loc(qlens)),
                               slot_ids=slots, query_lens=qlens)
    cache.check()
    m = kv_write.batch_metadata(qlens, slots, bt, lens, bs)
    kv_write.write_rows(kc, vc, k.cpu().numpy(), v.cpu().numpy(), m["slot_mapping"])
    np.testing.assert_array_equal(cache.key_cache.cpu().numpy(), kc)
    np.testing.assert_array_equal(cache.value_cache.cpu().numpy(), vc)
    np.testing.assert_array_equal(cache.kv_lens.cpu().numpy(), m["kv_lens_all"])


def test_bad_slot_and_overflow_are_flagged():
    from easymlx_b200 import PageCacheView, PageMetadata, build_query_start_loc

    cache = PageCacheView.init(num_seqs=2, max_seq_len=256, num_kv_heads=2, head_dim=64, block_size=128)
    k = torch.zeros((3, 2, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="slot id"):
        cache.concatenate_to_cache(k.repeat(1, 2, 1), k, k, cache_metadata=PageMetadata(
            query_start_loc=build_query_start_loc([3])), slot_ids=[5])
        cache.check()
    big = torch.zeros((300, 2, 64), dtype=torch.float16, device="cuda")
    before = cache.key_cache.clone()
    with pytest.raises(RuntimeError, match="outgrows"):
        cache.concatenate_to_cache(big.repeat(1, 2, 1), big, big, cache_metadata=PageMetadata(
            query_start_loc=build_query_start_loc([300])), slot_ids=[1])
        cache.check()
    cache.check()  # reported once, then clear
    # the sequence that would not fit is left alone: length unchanged, nothing written (the reference raises before
    # it touches the cache)
    assert cache.kv_lens.cpu().tolist() == [0, 0] and torch.equal(cache.key_cache, before)


def test_bounded_wait_reports_a_timeout_and_leaves_the_context_usable():
    """Failure detection without a fault: a wait that nothing satisfies runs out and is reported through the status
    word; afterwards the same context runs a normal batch."""
    from easymlx_b200 import _native as nv

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib, stream = nv.lib(), nv.stream_ptr(status.device)
    nv.check(lib.emlx_selftest_wait_timeout(nv.ptr(status), 4096, stream))
    rc = lib.emlx_read_status(nv.ptr(status), stream)
    assert rc == nv.EMLX_ERR_DEVICE and b"timed out" in lib.emlx_last_error()
    x = cases.attention_inputs(**cases.ATTENTION_CASES["attn_f16_decode_d64"])
    assert torch.isfinite(_run(x, None)).all()


@pytest.mark.parametrize("name", ["attn_f16_decode_d128", "attn_f16_mixed_d128", "attn_f16_specverify", "attn_f16_mixed_d64"])
def test_bfloat16_queries_and_pool(name):
    from easymlx_b200 import paged_attention

    x = cases.attention_inputs(**cases.ATTENTION_CASES[name])
    q = torch.from_numpy(x["q"]).float().bfloat16().cuda()
    kc = torch.from_numpy(x["key_cache"]).float().bfloat16().cuda()
    vc = torch.from_numpy(x["value_cache"]).float().bfloat16().cuda()
    out = paged_attention(q, kc, vc, dev(x["block_tables"]), dev(x["kv_lens"]), dev(x["query_start_loc"]),
                          softmax_scale=x["scale"], sliding_window=x["window"])
    assert out.dtype == torch.bfloat16
    want = opa.paged_attention_rows(q.float().cpu().numpy(), kc.float().cpu().numpy(), vc.float().cpu().numpy(),
                                    x["block_tables"], x["kv_lens"], x["query_start_loc"], softmax_scale=x["scale"],
                                    sliding_window=x["window"])
    # bf16 keeps 8 significant bits: probabilities and outputs are rounded to 2^-9 relative
    assert_close(out, want, atol=4e-3, rtol=2e-2)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("name", ["attn_f16_decode_d128", "attn_f16_decode_d64", "attn_f16_specverify", "attn_f16_mixed_d128"])
def test_bfloat16_queries_over_an_affine_pool(name, bits):
    """bf16 models with a quantised cache: the queries are converted to fp16 inside the fast kernels (the codes are
    multiplied on the fp16 tensor path), the output comes back as bf16."""
    from easymlx_b200 import paged_attention

    x = cases.attention_inputs(**cases.ATTENTION_CASES[name])
    kcode, vcode, ks, kb, vs, vb = quantized_pool_from_float(x["key_cache"], x["value_cache"], bits)
    kf = kv_quant.dequantize_key_pool(kcode, ks, kb, bits)
    vf = kv_quant.dequantize_value_pool(vcode, vs, vb, bits)
    q = torch.from_numpy(x["q"]).float().bfloat16().cuda()
    expect = opa.paged_attention_rows(q.float().cpu().numpy(), kf, vf, x["block_tables"], x["kv_lens"], x["query_start_loc"],
                                      softmax_scale=x["scale"], sliding_window=x["window"])
    out = paged_attention(q, dev(kcode), dev(vcode), dev(x["block_tables"]), dev(x["kv_lens"]), dev(x["query_start_loc"]),
                          softmax_scale=x["scale"], sliding_window=x["window"], kernel="tiled",
                          k_scale=dev(ks), k_bias=dev(kb), v_scale=dev(vs), v_bias=dev(vb))
    assert out.dtype == torch.bfloat16
    # the output is rounded to bf16 (8 significant bits)
    assert_close(out, expect, atol=4e-3, rtol=2e-2)
