"""Prefill chunks over an affine (8/4-bit) pool: with the host's query lengths known, rows of more than 16 go to the
tcgen05 kernel over pages expanded to 16-bit rows; results must agree with the coverage kernel, which reads the codes
itself, and with the short-row route."""

import numpy as np
import pytest
import torch

import easymlx_b200 as emlx
from easymlx_b200 import workloads
from easymlx_b200.operations.kernels.unified_attention import AttentionCall
from gpu_util import assert_close

pytestmark = pytest.mark.gpu


def _batch(bits, hq=32, hkv=8, qlens=(200, 1, 5, 1, 37, 1), prior=(3000, 500, 129, 0, 0, 7000)):
    whole = workloads.Workload(name="affine-mixed", hq=hq, hkv=hkv, d=128, bits=bits, qlens=np.asarray(qlens, np.int64),
                               prior=np.asarray(prior, np.int64))
    return workloads.materialize(whole, "cuda", seed=21 + bits)


def _after_write(w):
    c = w.cache
    q, kc, vc, meta = c.concatenate_to_cache(w.q, w.k, w.v, cache_metadata=emlx.PageMetadata(
        query_start_loc=emlx.build_query_start_loc(w.qlens.tolist()), slot_ids=tuple(w.slot_ids)),
        slot_ids=tuple(w.slot_ids), query_lens=tuple(int(x) for x in w.qlens), advance=False)
    extra = dict(k_scale=c.k_scales, v_scale=c.v_scales, k_bias=c.k_biases, v_bias=c.v_biases)
    return q, kc, vc, meta, extra


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("hq,hkv", [(32, 8), (16, 2), (8, 8)])
def test_long_rows_over_an_affine_pool_take_the_128_row_kernel(bits, hq, hkv):
    w = _batch(bits, hq, hkv)
    q, kc, vc, meta, extra = _after_write(w)
    group = hq // hkv
    assert meta.long_seqs == sum(1 for x in w.qlens if x * group > 16)
    assert int(meta.plan[3]) & 1, "the step's work list holds 128-row units"
    fast = AttentionCall(q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, plan=meta.plan,
                         max_query_len=meta.max_query_len, query_len_set=meta.query_len_set, long_seqs=meta.long_seqs, **extra)
    assert fast.planned and fast.args.row_class_mask & 8
    out = fast.launch()
    ref = emlx.paged_attention(q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, kernel="generic", **extra)
    assert_close(out, ref.float().cpu().numpy())
    # the route without the hint (32-row units on the short-row kernels) gives the same rows within tolerance
    slow = emlx.paged_attention(q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, **extra)
    assert_close(slow, ref.float().cpu().numpy())
    # twice in a row: the scratch-page counter is back at zero
    assert torch.equal(out, fast.launch())


@pytest.mark.parametrize("bits", [8, 4])
def test_long_rows_with_a_sliding_window(bits):
    # the 128-row kernel applies the window itself; the expansion leaves out the pages before the window of the
    # sequence's first query token (17 of the 3200-key sequence's 25 pages here)
    w = _batch(bits)
    q, kc, vc, meta, extra = _after_write(w)
    ref = emlx.paged_attention(q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, kernel="generic",
                               sliding_window=700, **extra)
    call = AttentionCall(q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, sliding_window=700,
                         max_query_len=meta.max_query_len, query_len_set=meta.query_len_set, long_seqs=meta.long_seqs, **extra)
    assert call.plan_flags & 1
    assert_close(call.plan().launch(), ref.float().cpu().numpy())


@pytest.mark.parametrize("bits", [8, 4])
def test_bfloat16_queries_go_through_fp16_copies(bits):
    # the expanded rows are fp16 and the tensor core multiplies operands of one type: the queries of the sequences
    # served by the 128-row kernel are converted to fp16 on the way in, their output rows back to bf16 on the way out
    w = _batch(bits)
    q, kc, vc, meta, extra = _after_write(w)
    qb = q.bfloat16()
    call = AttentionCall(qb, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, max_query_len=meta.max_query_len,
                         query_len_set=meta.query_len_set, long_seqs=meta.long_seqs, sliding_window=900, **extra)
    assert call.plan_flags & 1
    out = call.plan().launch()
    assert out.dtype == torch.bfloat16
    ref = emlx.paged_attention(qb, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, kernel="generic",
                               sliding_window=900, **extra)
    assert_close(out, ref.float().cpu().numpy(), atol=8e-3, rtol=2e-2)
    assert torch.equal(out, call.launch())


def test_expansion_scratch_too_small_is_reported():
    w = _batch(8, qlens=(200, 1, 40, 37), prior=(3000, 500, 3000, 3100))
    q, kc, vc, meta, extra = _after_write(w)
    call = AttentionCall(q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, max_query_len=meta.max_query_len,
                         query_len_set=meta.query_len_set, long_seqs=1, **extra).plan()  # three sequences have long rows
    with pytest.raises(RuntimeError, match="overflow|outgrow|capacity|status"):
        call.launch()
    torch.cuda.synchronize()
    good = AttentionCall(q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, max_query_len=meta.max_query_len,
                         query_len_set=meta.query_len_set, long_seqs=meta.long_seqs, **extra).plan().launch()
    ref = emlx.paged_attention(q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, kernel="generic", **extra)
    assert_close(good, ref.float().cpu().numpy())


def test_short_verify_rows_keep_the_32_row_route():
    # 5 tokens x 8 heads = 40 rows per sequence: expanding every page would cost more than it saves
    w = _batch(8, qlens=(5, 5, 5, 5), prior=(3000, 500, 129, 0))
    q, kc, vc, meta, extra = _after_write(w)
    assert meta.long_seqs == 0 and not int(meta.plan[3]) & 1


def test_performer_path_uses_the_hint():
    from easymlx_b200.runtime import AttentionStep

    w = _batch(8)
    out = AttentionStep(w.cache, w.q, w.k, w.v, w.qlens.tolist(), w.slot_ids)._eager()
    q, kc, vc, meta, extra = _after_write(w)
    ref = emlx.paged_attention(q, kc, vc, meta.block_tables, meta.kv_lens, meta.query_start_loc, kernel="generic", **extra)
    assert_close(out, ref.float().cpu().numpy())
