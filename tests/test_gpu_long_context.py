"""Shapes that stretch the work split: one unit spread over every CTA of the grid (merge of more than a hundred
partial results), prefill items with far more than 64 KV tiles (several page-id batches in the producer), and the
same with a sliding window.  The fast kernels are compared with the coverage kernel (independent code path) and
must repeat bit for bit."""

import numpy as np
import pytest
import torch

from gpu_util import assert_close

pytestmark = pytest.mark.gpu


def _pool(hkv, d, lens, bits, seed, block_size=128, dtype=torch.float16):
    from easymlx_b200 import PageCacheView
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages = [-(-int(n) // block_size) for n in lens]
    cache = PageCacheView.init(num_seqs=len(lens), max_seq_len=max(pages) * block_size, num_kv_heads=hkv, head_dim=d,
                               block_size=block_size, dtype=dtype, cache_dtype=(f"affine{bits}" if bits else None), device="cuda")
    for a in (cache.key_cache, cache.value_cache):
        if a.dtype == torch.uint8:
            a.copy_(torch.randint(0, 256, a.shape, device="cuda", generator=g, dtype=torch.uint8))
        else:
            a.copy_(torch.randn(a.shape, device="cuda", generator=g).to(a.dtype))
    if bits:
        for a in (cache.k_scales, cache.v_scales):
            a.copy_((torch.rand(a.shape, device="cuda", generator=g) * 0.05 + 0.01).to(a.dtype))
        for a in (cache.k_biases, cache.v_biases):
            a.copy_((torch.rand(a.shape, device="cuda", generator=g) - 0.5).to(a.dtype))
    return cache


def _run(cache, q, qlens, kv_lens, kernel, window=None):
    import easymlx_b200 as emlx
    extra = dict(k_scale=cache.k_scales, v_scale=cache.v_scales, k_bias=cache.k_biases, v_bias=cache.v_biases) \
        if cache.is_affine else {}
    return emlx.paged_attention(q, cache.key_cache, cache.value_cache, cache.block_tables,
                                torch.tensor(kv_lens, dtype=torch.int32, device="cuda"),
                                emlx.build_query_start_loc(qlens, device="cuda"), max_query_len=max(qlens),
                                sliding_window=window, kernel=kernel, **extra)


@pytest.mark.parametrize("bits", [0, 8, 4])
def test_one_decode_row_over_the_whole_grid(bits):
    # 150 000 keys of one KV head: 1172 tiles over 148 CTAs, every CTA holds one part of the same unit
    hq, hkv, d, kv = 4, 1, 128, 150_000
    cache = _pool(hkv, d, [kv], bits, seed=bits)
    q = torch.randn(1, hq, d, device="cuda", dtype=torch.float16)
    fast = _run(cache, q, [1], [kv], None)
    ref = _run(cache, q, [1], [kv], "generic")
    assert_close(fast, ref.float().cpu().numpy())
    assert torch.equal(fast, _run(cache, q, [1], [kv], None))


@pytest.mark.parametrize("bits", [0, 8, 4])
@pytest.mark.parametrize("group", [4, 8, 16])
def test_few_long_sequences_share_their_final_merge(bits, group):
    # 8 units of about 300 tiles on the whole grid: every unit ends in a merge of some twenty parts, which the
    # consumer warps of the last CTA to arrive share when they are free and one warp does alone when they are not;
    # both ways fold the parts in the same order with the same arithmetic, so repeated runs must agree bit for bit
    hkv, d = 2, 128
    lens = [40_000, 37_003, 39_111, 36_500]
    cache = _pool(hkv, d, lens, bits, seed=40 + bits)
    q = torch.randn(len(lens), hkv * group, d, device="cuda", dtype=torch.float16)
    first = _run(cache, q, [1] * len(lens), lens, None)
    assert_close(first, _run(cache, q, [1] * len(lens), lens, "generic").float().cpu().numpy())
    for _ in range(6):
        assert torch.equal(first, _run(cache, q, [1] * len(lens), lens, None))


@pytest.mark.parametrize("window", [None, 5000])
def test_prefill_chunk_after_a_long_context(window):
    # 256 new tokens after 20 000 cached ones: 32 x 128-row units x 2 KV heads, up to 159 KV tiles per item
    hq, hkv, d, q_len, prior = 16, 2, 128, 256, 20_000
    cache = _pool(hkv, d, [prior + q_len], 0, seed=11)
    q = torch.randn(q_len, hq, d, device="cuda", dtype=torch.float16)
    fast = _run(cache, q, [q_len], [prior + q_len], None, window)
    ref = _run(cache, q, [q_len], [prior + q_len], "generic", window)
    assert_close(fast, ref.float().cpu().numpy())
    assert torch.equal(fast, _run(cache, q, [q_len], [prior + q_len], None, window))


def test_mixed_lengths_with_empty_and_single_token_sequences():
    # query lengths 0, 1, 3 (one 8-row unit ... 24 rows), 40 and 130 tokens in one batch, ragged contexts
    hq, hkv, d = 16, 2, 128
    qlens = [1, 0, 3, 40, 1, 130]
    prior = [700, 0, 129, 5, 4000, 300]
    kv = [a + b for a, b in zip(qlens, prior)]
    cache = _pool(hkv, d, [max(n, 1) for n in kv], 0, seed=5)
    q = torch.randn(sum(qlens), hq, d, device="cuda", dtype=torch.float16)
    fast = _run(cache, q, qlens, kv, None)
    ref = _run(cache, q, qlens, kv, "generic")
    assert_close(fast, ref.float().cpu().numpy())


@pytest.mark.parametrize("bits", [0, 8])
def test_output_does_not_depend_on_where_the_pages_live(bits):
    """Same logical K/V, pages shuffled through the pool: the rows must come out bit for bit the same (the work split
    depends on lengths only, and the split merge runs in a fixed order)."""
    import easymlx_b200 as emlx
    hq, hkv, d = 8, 2, 128
    qlens = [1, 1, 1, 9]
    kv = [3000, 130, 777, 2000]
    cache = _pool(hkv, d, kv, bits, seed=21)
    q = torch.randn(sum(qlens), hq, d, device="cuda", dtype=torch.float16)
    first = _run(cache, q, qlens, kv, None)
    # move every page to a new place
    nb = cache.num_blocks
    perm = torch.randperm(nb, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(nb, device="cuda")
    arrays = [cache.key_cache, cache.value_cache]
    if cache.is_affine:
        arrays += [cache.k_scales, cache.k_biases, cache.v_scales, cache.v_biases]
    for a in arrays:
        a.copy_(a[inv].clone())  # page p of the old pool is page perm[p] of the new one
    cache.block_tables.copy_(perm[cache.block_tables.long()].to(torch.int32))
    second = _run(cache, q, qlens, kv, None)
    assert torch.equal(first, second)


@pytest.mark.parametrize("block_size", [16, 32, 64])
@pytest.mark.parametrize("d,dtype", [(128, torch.float16), (64, torch.bfloat16)])
def test_small_pages_take_the_fast_kernels(block_size, d, dtype):
    """Pages of 16 / 32 / 64 tokens (the reference's default is 16): a 128-token tile is assembled from several pages.
    Decode rows, a 3-token row and a prefill chunk; page order scrambled; fast path against the coverage kernel."""
    import easymlx_b200 as emlx
    hq, hkv = 8, 2
    qlens = [1, 3, 1, 150, 1]
    prior = [1000, 77, 0, 300, 2049]
    kv = [a + b for a, b in zip(qlens, prior)]
    cache = _pool(hkv, d, kv, 0, seed=block_size, block_size=block_size, dtype=dtype)
    # scatter the pages: every row of the table is a random set of distinct pages
    g = torch.Generator(device="cuda").manual_seed(9)
    perm = torch.randperm(cache.num_blocks, device="cuda", generator=g).to(torch.int32)
    cache.block_tables.copy_(perm.reshape(cache.block_tables.shape))
    q = torch.randn(sum(qlens), hq, d, device="cuda", generator=g).to(dtype)
    args = (q, cache.key_cache, cache.value_cache, cache.block_tables, torch.tensor(kv, dtype=torch.int32, device="cuda"),
            emlx.build_query_start_loc(qlens, device="cuda"))
    fast = emlx.paged_attention(*args, max_query_len=max(qlens), kernel="tiled")
    ref = emlx.paged_attention(*args, kernel="generic")
    assert_close(fast, ref.float().cpu().numpy(), atol=(2e-3 if dtype == torch.float16 else 8e-3), rtol=(1e-2 if dtype == torch.float16 else 2e-2))
    assert torch.equal(fast, emlx.paged_attention(*args, max_query_len=max(qlens), query_len_set=qlens))


def test_step_with_more_sequences_than_the_metadata_kernel_keeps_on_chip():
    """2 500 decode sequences in one step: the prefix sums, lengths and unit table of the metadata kernel no longer fit
    its shared-memory staging (2 048 sequences / 4 096 units), and the scan runs in three passes of 1 024."""
    import easymlx_b200 as emlx
    from oracle import kv_write
    hq, hkv, d, s = 8, 2, 64, 2500
    rng = np.random.default_rng(12)
    prior = rng.integers(0, 300, size=s).astype(np.int32)
    qlens = np.ones(s, dtype=np.int64)
    qlens[::97] = 3  # a few multi-token rows among the decode rows
    cache = emlx.PageCacheView.init(num_seqs=s, max_seq_len=384, num_kv_heads=hkv, head_dim=d, block_size=128, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(12)
    cache.key_cache.copy_(torch.randn(cache.key_cache.shape, device="cuda", generator=g).half())
    cache.value_cache.copy_(torch.randn(cache.value_cache.shape, device="cuda", generator=g).half())
    cache.kv_lens.copy_(torch.from_numpy(prior))
    t = int(qlens.sum())
    q, k, v = (torch.randn(t, h, d, device="cuda", generator=g).half() for h in (hq, hkv, hkv))
    slots = tuple(range(s))
    meta = emlx.PageMetadata(query_start_loc=emlx.build_query_start_loc(qlens.tolist()), slot_ids=slots)
    want_meta = kv_write.batch_metadata(qlens, np.arange(s), cache.block_tables.cpu().numpy(), prior, 128)
    _, kc, vc, resolved = cache.concatenate_to_cache(q, k, v, cache_metadata=meta, slot_ids=slots, query_lens=qlens.tolist())
    cache.check()
    kv = (prior + qlens).astype(np.int32)
    np.testing.assert_array_equal(resolved.kv_lens.cpu().numpy(), kv)
    np.testing.assert_array_equal(resolved.query_start_loc.cpu().numpy(), np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32))
    slot_map = torch.from_numpy(want_meta["slot_mapping"]).cuda()
    assert torch.equal(kc.reshape(-1, hkv, d)[slot_map], k) and torch.equal(vc.reshape(-1, hkv, d)[slot_map], v)
    fast = emlx.AttentionPerformer(scale=d ** -0.5).executor.mixin_impl(
        query=q, key=kc, value=vc, cache_metadata=resolved, cache_view=cache, scale=d ** -0.5).attention_outputs
    ref = emlx.paged_attention(q, kc, vc, resolved.block_tables, resolved.kv_lens, resolved.query_start_loc, kernel="generic")
    assert_close(fast, ref.float().cpu().numpy())


@pytest.mark.parametrize("qlens,kv", [([1, 1], [700, 300]), ([200], [600])])
def test_unassigned_page_inside_a_live_range_reads_as_zero_rows_and_is_reported(qlens, kv):
    """A page id of -1 below kv_len: the fp16 kernels attend zero K/V rows there (as the reference's NumPy path does) and
    raise the bad-page flag; decode kernel and 128-row kernel alike."""
    import easymlx_b200 as emlx
    hq, hkv, d = 8, 2, 128
    cache = _pool(hkv, d, kv, 0, seed=33)
    cache.block_tables[0, 1] = -1
    q = torch.randn(sum(qlens), hq, d, device="cuda", dtype=torch.float16)
    args = (q, cache.key_cache, cache.value_cache, cache.block_tables, torch.tensor(kv, dtype=torch.int32, device="cuda"),
            emlx.build_query_start_loc(qlens, device="cuda"))
    outs = {}
    for kernel in ("tiled", "generic"):
        call = emlx.operations.kernels.unified_attention.AttentionCall(*args, max_query_len=max(qlens), kernel=kernel).plan()
        with pytest.raises(RuntimeError, match="page id out of range"):  # the tests run with device-side checks reported
            call.launch()
        outs[kernel] = call.out
    assert_close(outs["tiled"], outs["generic"].float().cpu().numpy())


@pytest.mark.parametrize("bits", [8, 4])
def test_tail_of_a_long_peaked_row_over_an_affine_pool(bits):
    """30 000 keys whose values all sit well above zero, scores spread widely: in most rows one key takes most of the
    weight and the others share a few per cent, each with weight * scale below the fp16 subnormal step.  Rounding
    those weights away lowers every channel of the row by the same amount; the decode rows, a 40-token chunk (32-row
    units) and the coverage kernel must agree element by element and in the mean over each row."""
    hq, hkv, d = 16, 2, 64
    qlens, prior = [40, 1, 1], [30_000, 30_000, 12_345]
    kv = [a + b for a, b in zip(qlens, prior)]
    cache = _pool(hkv, d, kv, bits, seed=31)
    q = torch.randn(sum(qlens), hq, d, device="cuda", dtype=torch.float16)
    fast = _run(cache, q, qlens, kv, None)
    ref = _run(cache, q, qlens, kv, "generic")
    assert_close(fast, ref.float().cpu().numpy())
    row_shift = (fast.float() - ref.float()).mean(dim=-1).abs().max().item()
    assert row_shift <= 1e-3, f"rows shifted by up to {row_shift:.2e}"


def test_tail_of_a_long_peaked_row_over_an_fp16_pool():
    """One key holds nearly all the weight of a row and 131 000 others sit 2^-25.5 below it.  As plain fp16 numbers
    those weights would all round to zero (half the smallest subnormal is 2^-25) and the row would lose everything the
    others contribute, 5e-3 in every channel; the kernels therefore scale the weights up before the 16-bit cast.  The
    128-row chunk runs on the tcgen05 kernel (one thread follows a row over all of its keys, so the whole tail is at
    stake), the decode row on the split-KV kernel.  Expected values are exact: scores are 0 except for the first
    key, values are 2 except for the first key's 0."""
    import easymlx_b200 as emlx
    hq, hkv, d = 4, 1, 128
    qlens, prior = [32, 1], [131_072, 131_072]
    kv = [a + b for a, b in zip(qlens, prior)]
    cache = _pool(hkv, d, kv, 0, seed=5)
    cache.key_cache.zero_()
    cache.value_cache.fill_(2.0)
    for s in range(2):
        first_page = int(cache.block_tables[s, 0])
        cache.key_cache[first_page, 0] = 1.25
        cache.value_cache[first_page, 0] = 0.0
    q = torch.full((sum(qlens), hq, d), 1.25, device="cuda", dtype=torch.float16)
    fast = _run(cache, q, qlens, kv, None)
    ref = _run(cache, q, qlens, kv, "generic")
    gap = 1.25 * 1.25 * d / np.sqrt(d)                      # score of the first key; every other score is 0
    others = np.concatenate([prior[0] + np.arange(qlens[0]), [prior[1]]]).astype(np.float64)  # keys besides the first
    tail = others * np.exp(-gap)
    expect = 2.0 * tail / (1.0 + tail)                       # per packed row, the same in every head and channel
    assert 4e-3 < expect.min() < 7e-3
    got = fast.float().cpu().numpy().astype(np.float64)
    assert np.abs(got - expect[:, None, None]).max() <= 3e-4, np.abs(got - expect[:, None, None]).max()
    assert_close(fast, ref.float().cpu().numpy())
