"""The five benchmark configurations at full size (run with -m gpu on a B200).

The CPU oracle cannot attend 10^5..10^6 keys per row in seconds, so the checks here are the
size-independent ones: the tiled kernels against the coverage kernel (same inputs, independent code path:
one warp per row walking keys one by one), bit-identical repeat runs (deterministic split merge), the oracle
on a few sampled sequences, and bit-exact placement/codes of the step's new rows read back from the pool.
"""

import numpy as np
import pytest
import torch

from gpu_util import ATOL, RTOL, assert_close
from oracle import kv_quant, kv_write, paged_attention as opa

pytestmark = pytest.mark.gpu

CONFIGS = ["c1", "c2", "c3", "c4", "c5"]


@pytest.fixture(scope="module", params=CONFIGS)
def workload(request):
    from easymlx_b200 import workloads

    w = workloads.materialize(workloads.describe(request.param), "cuda", seed=3)
    yield w
    del w
    torch.cuda.empty_cache()


def _attend(w, kernel, kv_lens):
    import easymlx_b200 as emlx

    c = w.cache
    extra = dict(k_scale=c.k_scales, v_scale=c.v_scales, k_bias=c.k_biases, v_bias=c.v_biases) if w.bits else {}
    return emlx.paged_attention(w.q, c.key_cache, c.value_cache, c.block_tables, kv_lens,
                                emlx.build_query_start_loc(w.qlens.tolist(), device="cuda"),
                                max_query_len=int(w.qlens.max()), kernel=kernel, **extra)


def test_step_matches_coverage_kernel_and_oracle(workload):
    import easymlx_b200 as emlx

    w = workload
    c = w.cache
    prior = c.kv_lens.clone()
    meta = emlx.PageMetadata(query_start_loc=emlx.build_query_start_loc(w.qlens.tolist()), slot_ids=w.slot_ids)
    performer = emlx.AttentionPerformer(scale=w.d ** -0.5)
    _, kc, vc, resolved = c.concatenate_to_cache(w.q, w.k, w.v, cache_metadata=meta, slot_ids=w.slot_ids,
                                                 query_lens=w.qlens.tolist())
    c.check()
    np.testing.assert_array_equal(resolved.kv_lens.cpu().numpy(), w.kv_lens.astype(np.int32))
    np.testing.assert_array_equal(c.kv_lens.cpu().numpy(), w.kv_lens.astype(np.int32))

    # ---- the step's new rows, read back: bit-exact placement (and codes / scale / bias for affine pools)
    m = kv_write.batch_metadata(w.qlens, np.arange(len(w.qlens)), c.block_tables.cpu().numpy(), prior.cpu().numpy(), 128)
    rng = np.random.default_rng(0)
    sample = rng.choice(w.total_tokens, size=min(64, w.total_tokens), replace=False)
    slots = m["slot_mapping"][sample]
    k_new, v_new = w.k[sample].cpu().numpy(), w.v[sample].cpu().numpy()
    page, off = slots // 128, slots % 128
    if w.bits == 0:
        got_k = c.key_cache.reshape(-1, w.hkv, w.d)[torch.from_numpy(slots).cuda()].cpu().numpy()
        got_v = c.value_cache.reshape(-1, w.hkv, w.d)[torch.from_numpy(slots).cuda()].cpu().numpy()
        np.testing.assert_array_equal(got_k, k_new)
        np.testing.assert_array_equal(got_v, v_new)
    else:
        kcodes, ks, kb = kv_quant.quantize_rows(k_new, w.bits)
        vcodes, vs, vb = kv_quant.quantize_rows(v_new, w.bits)
        got_k = c.key_cache.reshape(-1, w.hkv, w.d * w.bits // 8)[torch.from_numpy(slots).cuda()].cpu().numpy()
        np.testing.assert_array_equal(got_k, kv_quant.pack_codes(kcodes, w.bits))
        pg, of = torch.from_numpy(page).cuda(), torch.from_numpy(off).cuda()
        np.testing.assert_array_equal(c.k_scales[pg, :, of].cpu().numpy().view(np.uint16), ks.view(np.uint16))
        np.testing.assert_array_equal(c.k_biases[pg, :, of].cpu().numpy().view(np.uint16), kb.view(np.uint16))
        np.testing.assert_array_equal(c.v_scales[pg, :, of].cpu().numpy().view(np.uint16), vs.view(np.uint16))
        np.testing.assert_array_equal(c.v_biases[pg, :, of].cpu().numpy().view(np.uint16), vb.view(np.uint16))
        vstore = c.value_cache[pg].cpu().numpy()                       # [n, Hkv, D, bs*bits/8]
        vun = kv_quant.unpack_codes(vstore, w.bits)                    # [n, Hkv, D, bs]
        got_v = vun[np.arange(len(off)), :, :, off]                    # [n, Hkv, D]
        np.testing.assert_array_equal(got_v, vcodes)

    # ---- attention: tiled kernels vs the coverage kernel, twice (determinism)
    out = _attend(w, None, resolved.kv_lens)
    again = _attend(w, None, resolved.kv_lens)
    assert torch.equal(out, again), "two runs of the same batch differ: the split merge is not deterministic"
    ref = _attend(w, "generic", resolved.kv_lens)
    assert_close(out, ref.float().cpu().numpy(), atol=ATOL, rtol=RTOL)
    assert not torch.isnan(out).any()

    # ---- and the CPU oracle on the rows that are hardest to get right: the shortest, the median and a long sequence,
    # the LONGEST decode sequence of the batch, and of every prefill chunk its first row, its last row and eight
    # random ones (a row of a chunk costs the oracle microseconds per thousand keys, a whole chunk would cost minutes)
    order = np.argsort(w.kv_lens * np.maximum(w.qlens, 1), kind="stable")
    picks = {int(order[0]), int(order[len(order) // 2]), int(order[min(len(order) - 1, (3 * len(order)) // 4)])}
    decode_like = np.flatnonzero(w.qlens <= 8)
    if len(decode_like):
        picks.add(int(decode_like[np.argmax(w.kv_lens[decode_like])]))
    row_subset = {}
    rng_rows = np.random.default_rng(5)
    for s_idx in np.flatnonzero(w.qlens > 32):
        n = int(w.qlens[s_idx])
        picks.add(int(s_idx))
        row_subset[int(s_idx)] = np.unique(np.concatenate([[0, n - 1], rng_rows.integers(0, n, 8)]))
    picks = sorted(picks)
    bt = c.block_tables.cpu().numpy()
    pages = np.unique(np.concatenate([bt[s, : -(-int(w.kv_lens[s]) // 128)] for s in picks]))
    remap = -np.ones(c.num_blocks, dtype=np.int64)
    remap[pages] = np.arange(len(pages))
    idx = torch.from_numpy(pages).cuda()
    if w.bits == 0:
        kf, vf = c.key_cache[idx].cpu().numpy(), c.value_cache[idx].cpu().numpy()
    else:
        kf = kv_quant.dequantize_key_pool(c.key_cache[idx].cpu().numpy(), c.k_scales[idx].cpu().numpy(),
                                          c.k_biases[idx].cpu().numpy(), w.bits)
        vf = kv_quant.dequantize_value_pool(c.value_cache[idx].cpu().numpy(), c.v_scales[idx].cpu().numpy(),
                                            c.v_biases[idx].cpu().numpy(), w.bits)
    sub_bt = np.where(bt >= 0, remap[np.maximum(bt, 0)], -1).astype(np.int32)
    qsl = np.concatenate([[0], np.cumsum(w.qlens)]).astype(np.int32)
    want = opa.paged_attention_rows(w.q.cpu().numpy(), kf, vf, sub_bt, w.kv_lens.astype(np.int32), qsl,
                                    softmax_scale=w.d ** -0.5, seq_subset=picks, row_subset=row_subset)
    rows = np.concatenate([qsl[s] + row_subset[s] if s in row_subset else np.arange(qsl[s], qsl[s + 1]) for s in picks])
    assert_close(out[torch.from_numpy(rows).cuda()], want[rows].astype(np.float32), atol=ATOL, rtol=RTOL)
    del performer
