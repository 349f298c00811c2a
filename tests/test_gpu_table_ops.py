"""CUDA batch / page-table kernels against the CPU oracle (bit-exact: byte and index work)."""

import os
from collections import namedtuple

import numpy as np
import pytest
import torch

from oracle import page_table as ot

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "table_ops.npz"))
Seq = namedtuple("Seq", "token_ids")


def _golden_view():
    from easymlx_b200 import PageCacheView
    k0, v0 = GOLD["k0"], GOLD["v0"]
    return PageCacheView(key_cache=torch.from_numpy(k0.copy()).cuda(), value_cache=torch.from_numpy(v0.copy()).cuda(),
                         block_tables=torch.from_numpy(GOLD["bt0"].copy()).cuda(),
                         kv_lens=torch.from_numpy(GOLD["lens0"].copy()).cuda(), block_size=k0.shape[1],
                         num_kv_heads=k0.shape[2], head_dim=k0.shape[3])


def _runner(view):
    from easymlx_b200.inference.esurge import PageTableRunner
    return PageTableRunner([view])


def test_row_operations_match_the_reference_vectors():
    v = _golden_view(); r = _runner(v)
    r._assign_row_mapping(2, [7, 3, 9], cached_tokens=5)
    r._assign_row_mapping(4, [1, 2, 3, 4, 5, 6, 7], cached_tokens=-3)
    np.testing.assert_array_equal(v.block_tables.cpu().numpy(), GOLD["assign_bt"])
    np.testing.assert_array_equal(v.kv_lens.cpu().numpy(), GOLD["assign_lens"])
    with pytest.raises(RuntimeError):
        r._assign_row_mapping(v.num_seqs, [1])

    v = _golden_view(); r = _runner(v)
    r._move_cache_row(1, 4)
    r._move_cache_row(3, 3)
    np.testing.assert_array_equal(v.block_tables.cpu().numpy(), GOLD["swap_bt"])
    np.testing.assert_array_equal(v.kv_lens.cpu().numpy(), GOLD["swap_lens"])

    v = _golden_view(); r = _runner(v)
    moves = [tuple(m) for m in GOLD["compact_moves"].tolist()]
    assert r.compact_rows(moves) == moves
    np.testing.assert_array_equal(v.block_tables.cpu().numpy(), GOLD["compact_bt"])
    np.testing.assert_array_equal(v.kv_lens.cpu().numpy(), GOLD["compact_lens"])

    v = _golden_view(); r = _runner(v)
    r._clear_row_mapping(2)
    r._clear_row_mapping(99)  # past the table: ignored, as in the reference
    np.testing.assert_array_equal(v.block_tables.cpu().numpy(), GOLD["clear_bt"])
    np.testing.assert_array_equal(v.kv_lens.cpu().numpy(), GOLD["clear_lens"])
    v.check()


def test_zero_pages_matches_the_reference_vectors():
    v = _golden_view(); r = _runner(v)
    r._zero_pages(GOLD["zero_ids"].tolist())
    np.testing.assert_array_equal(v.key_cache.cpu().numpy(), GOLD["zero_k"])
    np.testing.assert_array_equal(v.value_cache.cpu().numpy(), GOLD["zero_v"])


def test_packed_ids_and_last_tokens_match_the_reference_vectors():
    from easymlx_b200.inference.esurge import extract_last_tokens
    from easymlx_b200 import PageMetadata
    lens = GOLD["ids_lens"].tolist(); flat = GOLD["ids_flat"]
    seqs, at = [], 0
    for n in lens:
        seqs.append(Seq(flat[at:at + n].tolist())); at += n
    r = _runner(_golden_view())
    got_flat, got_lens = r._flatten_sequence_tokens(seqs, device="cuda")
    np.testing.assert_array_equal(got_flat.cpu().numpy(), flat)
    padded, got_lens2 = r._pad_batch_token_ids(seqs)
    assert got_lens == lens and got_lens2 == lens
    np.testing.assert_array_equal(padded.cpu().numpy(), GOLD["ids_padded"])
    empty, _ = r._pad_batch_token_ids([])
    assert tuple(empty.shape) == (0, 0)

    hidden = torch.from_numpy(GOLD["last_hidden"]).cuda()
    meta = PageMetadata(query_start_loc=torch.from_numpy(GOLD["last_qsl"]).cuda(), is_single_token_decode=False)
    np.testing.assert_array_equal(extract_last_tokens(hidden, meta).cpu().numpy(), GOLD["last_out"])
    single = PageMetadata(query_start_loc=torch.from_numpy(GOLD["last_qsl"]).cuda(), is_single_token_decode=True)
    assert extract_last_tokens(hidden, single) is hidden
    assert extract_last_tokens(hidden, None) is hidden


@pytest.mark.parametrize("hidden_size,dtype", [(4096, torch.float16), (1023, torch.float32), (7, torch.bfloat16)])
def test_last_tokens_larger_batches(hidden_size, dtype):
    from easymlx_b200.inference.esurge import extract_last_tokens
    from easymlx_b200 import PageMetadata
    rng = np.random.default_rng(3)
    lens = rng.integers(0, 40, size=300); lens[0] = 3
    qsl = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    hidden = torch.randn(int(qsl[-1]), hidden_size, device="cuda").to(dtype)
    got = extract_last_tokens(hidden, PageMetadata(query_start_loc=torch.from_numpy(qsl).cuda()))
    want = hidden[torch.from_numpy((qsl[1:] - 1).astype(np.int64)).cuda()]
    assert torch.equal(got, want)


def test_pad_ids_larger_batch():
    rng = np.random.default_rng(4)
    lens = rng.integers(0, 600, size=257).tolist()
    seqs = [Seq(rng.integers(0, 128000, size=n).tolist()) for n in lens]
    r = _runner(_golden_view())
    padded, _ = r._pad_batch_token_ids(seqs)
    flat, _ = ot.flatten_sequence_tokens([s.token_ids for s in seqs])
    np.testing.assert_array_equal(padded.cpu().numpy(), ot.pad_batch_token_ids(flat, lens))


def _pool_arrays(view):
    arrs = [view.key_cache, view.value_cache]
    if view.is_affine:
        arrs += [view.k_scales, view.k_biases, view.v_scales, view.v_biases]
    return arrs


@pytest.mark.parametrize("bits", [0, 8, 4])
@pytest.mark.parametrize("mapping,host", [
    ([[0, 1], [2, 3], [4, 9]], True),            # independent pairs: one in-place launch
    ([[0, 1], [1, 2], [5, 0], [7, 7]], True),    # chained: staged, reads see the old pool
    ([[0, 1], [1, 2], [5, 0]], False),           # device-resident mapping: staged
])
def test_copy_blocks_all_pool_arrays(bits, mapping, host):
    from easymlx_b200 import PageCacheView
    v = PageCacheView.init(num_seqs=4, max_seq_len=1024, num_kv_heads=2, head_dim=128, block_size=128,
                           cache_dtype=(f"affine{bits}" if bits else None), device="cuda")
    g = torch.Generator(device="cuda").manual_seed(bits)
    for a in _pool_arrays(v):
        if a.dtype == torch.uint8:
            a.copy_(torch.randint(0, 256, a.shape, device="cuda", generator=g, dtype=torch.uint8))
        else:
            a.copy_(torch.randn(a.shape, device="cuda", generator=g).to(a.dtype))
    want = [a.cpu().numpy().copy() for a in _pool_arrays(v)]
    ot.copy_blocks(want, mapping)
    arg = mapping if host else torch.tensor(mapping, dtype=torch.int32, device="cuda")
    v.copy_blocks(arg)
    for a, w in zip(_pool_arrays(v), want):
        np.testing.assert_array_equal(a.cpu().numpy().view(np.uint8), w.view(np.uint8))


def test_copy_blocks_validation():
    from easymlx_b200 import PageCacheView, PageCache
    v = PageCacheView.init(num_seqs=2, max_seq_len=256, num_kv_heads=2, head_dim=64, block_size=128, device="cuda")
    with pytest.raises(ValueError):
        v.copy_blocks(torch.zeros(3, dtype=torch.int32, device="cuda"))
    v.copy_blocks(torch.zeros((0, 2), dtype=torch.int32, device="cuda"))  # no pairs: nothing to do
    before = v.key_cache.clone()
    with pytest.raises(RuntimeError):
        v.copy_blocks([[0, v.num_blocks + 3]])  # a page past the pool: skipped and reported
    assert torch.equal(v.key_cache, before)
    PageCache([v]).copy_blocks([[0, 1]])


def test_prepare_step_drives_write_and_attention():
    """Scheduler selection -> bound rows, packed ids / positions, metadata -> KV write + attention, against the oracle."""
    from easymlx_b200 import AttentionPerformer, PageCacheView
    from easymlx_b200.inference.esurge import PageTableRunner, ScheduledSequence, extract_last_tokens, prepare_step
    from oracle import paged_attention as opa

    hq, hkv, d, bs = 8, 2, 64, 128
    cache = PageCacheView.init(num_seqs=4, max_seq_len=512, num_kv_heads=hkv, head_dim=d, block_size=bs, device="cuda",
                               num_blocks=16)
    cache.block_tables.fill_(-1)
    runner = PageTableRunner([cache])
    seqs = [ScheduledSequence("a", 2, list(range(40)), 0, page_ids=(5, 9)),       # a 40-token prefill chunk in row 2
            ScheduledSequence("b", 0, [7], 0, page_ids=(3,))]                      # a first decode token in row 0
    batch = prepare_step(runner, seqs)
    assert batch.query_lens == [40, 1] and batch.slot_ids == (2, 0)
    np.testing.assert_array_equal(batch.token_ids.cpu().numpy(), np.asarray(list(range(40)) + [7], dtype=np.int32))
    np.testing.assert_array_equal(batch.positions.cpu().numpy(), np.asarray(list(range(40)) + [0], dtype=np.int32))
    np.testing.assert_array_equal(cache.block_tables[2, :3].cpu().numpy(), [5, 9, -1])
    np.testing.assert_array_equal(cache.block_tables[0, :2].cpu().numpy(), [3, -1])

    g = torch.Generator(device="cuda").manual_seed(1)
    t = sum(batch.query_lens)
    q = torch.randn(t, hq, d, device="cuda", generator=g).half()
    k = torch.randn(t, hkv, d, device="cuda", generator=g).half()
    v = torch.randn(t, hkv, d, device="cuda", generator=g).half()
    out = AttentionPerformer(scale=d ** -0.5)(q, k, v, cache_view=cache, cache_metadata=batch.cache_metadata)
    cache.check()
    want = opa.paged_attention_rows(q.cpu().numpy(), cache.key_cache.cpu().numpy(), cache.value_cache.cpu().numpy(),
                                    cache.block_tables[[2, 0]].cpu().numpy(), np.asarray([40, 1], dtype=np.int32),
                                    np.asarray([0, 40, 41], dtype=np.int32), softmax_scale=d ** -0.5)
    from gpu_util import assert_close
    assert_close(out, want)
    hidden = out.reshape(t, hq * d)
    last = extract_last_tokens(hidden, batch.cache_metadata)
    assert torch.equal(last, hidden[[39, 40]])


@pytest.mark.parametrize("bits", [0, 8, 4])
def test_gather_and_dequantize_kv_cache(bits):
    """PageCacheView.gather_kv_cache / dequantize_kv_cache against the oracle's gather and dequantisation."""
    from easymlx_b200 import PageCacheView
    from oracle import kv_quant, paged_attention as opa
    hkv, d, bs = 2, 128, 128
    v = PageCacheView.init(num_seqs=3, max_seq_len=512, num_kv_heads=hkv, head_dim=d, block_size=bs,
                           cache_dtype=(f"affine{bits}" if bits else None), device="cuda")
    g = torch.Generator(device="cuda").manual_seed(40 + bits)
    for a in _pool_arrays(v):
        if a.dtype == torch.uint8:
            a.copy_(torch.randint(0, 256, a.shape, device="cuda", generator=g, dtype=torch.uint8))
        else:
            a.copy_(torch.randn(a.shape, device="cuda", generator=g).to(a.dtype))
    if bits:
        kf = kv_quant.dequantize_key_pool(v.key_cache.cpu().numpy(), v.k_scales.cpu().numpy(), v.k_biases.cpu().numpy(), bits)
        vf = kv_quant.dequantize_value_pool(v.value_cache.cpu().numpy(), v.v_scales.cpu().numpy(), v.v_biases.cpu().numpy(), bits)
    else:
        kf, vf = v.key_cache.float().cpu().numpy(), v.value_cache.float().cpu().numpy()
    table = np.asarray([[7, 2, 9, -1], [0, -1, -1, -1], [11, 3, 5, 1]], dtype=np.int32)
    lens = [300, 0, 512]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    k_out, v_out = v.gather_kv_cache(table, cu, out_dtype=torch.float32)
    want_k = np.concatenate([opa.gather_sequence(kf, table[s], lens[s], bs) for s in range(3)])
    want_v = np.concatenate([opa.gather_sequence(vf, table[s], lens[s], bs) for s in range(3)])
    np.testing.assert_array_equal(k_out.cpu().numpy(), want_k)
    np.testing.assert_array_equal(v_out.cpu().numpy(), want_v)
    dk, dv = v.dequantize_kv_cache(v.key_cache, v.value_cache, out_dtype=torch.float32)
    if bits:
        np.testing.assert_array_equal(dk.cpu().numpy(), kf)
        np.testing.assert_array_equal(dv.cpu().numpy(), vf)
    else:
        assert dk is v.key_cache and dv is v.value_cache


@pytest.mark.parametrize("seed", range(6))
def test_random_sequences_of_row_and_page_operations(seed):
    """Twenty random operations in a row (assign, exchange, compaction with chained moves, clear, page zeroing,
    copy-on-write page copies with chained mappings) on one cache; table, lengths and every pool array against the oracle
    after each of them."""
    from easymlx_b200 import PageCacheView
    rng = np.random.default_rng(4200 + seed)
    bits = int(rng.choice([0, 8, 4]))
    slots, mb, bs = int(rng.choice([3, 8, 33])), int(rng.choice([2, 5, 9])), int(rng.choice([16, 128]))
    v = PageCacheView.init(num_seqs=slots, max_seq_len=mb * bs, num_kv_heads=int(rng.choice([1, 2])), head_dim=64,
                           block_size=bs, cache_dtype=(f"affine{bits}" if bits else None), device="cuda")
    g = torch.Generator(device="cuda").manual_seed(seed)
    for a in _pool_arrays(v):
        if a.dtype == torch.uint8:
            a.copy_(torch.randint(0, 256, a.shape, device="cuda", generator=g, dtype=torch.uint8))
        else:
            a.copy_(torch.randn(a.shape, device="cuda", generator=g).to(a.dtype))
    nb = v.num_blocks
    bt = rng.integers(-1, nb, size=(slots, mb)).astype(np.int32)
    lens = rng.integers(0, mb * bs, size=slots).astype(np.int32)
    v.block_tables.copy_(torch.from_numpy(bt)); v.kv_lens.copy_(torch.from_numpy(lens))
    arrays = [a.cpu().numpy().copy() for a in _pool_arrays(v)]
    r = _runner(v)
    for step in range(20):
        op = str(rng.choice(["assign", "swap", "compact", "clear", "zero", "copy"]))
        if op == "assign":
            row, pages = int(rng.integers(0, slots)), rng.integers(0, nb, size=int(rng.integers(0, mb + 3))).tolist()
            cached = int(rng.integers(-4, mb * bs))
            r._assign_row_mapping(row, pages, cached_tokens=cached)
            ot.assign_row(bt, lens, row, pages, cached)
        elif op == "swap":
            a, b = int(rng.integers(0, slots)), int(rng.integers(0, slots))
            r._move_cache_row(a, b)
            ot.swap_rows(bt, lens, a, b)
        elif op == "compact":
            # holes are filled from the back, and a later move may read a row that an earlier one wrote
            moves = [(int(rng.integers(0, slots)), int(rng.integers(0, slots))) for _ in range(int(rng.integers(1, 5)))]
            r.compact_rows(moves)
            ot.compact_rows(bt, lens, moves)
        elif op == "clear":
            row = int(rng.integers(0, slots))
            r._clear_row_mapping(row)
            ot.clear_row(bt, lens, row)
        elif op == "zero":
            ids = rng.integers(-2, nb + 3, size=int(rng.integers(1, 6))).tolist()
            r._zero_pages(ids)
            ot.zero_pages(arrays, ids)
        else:
            n = int(rng.integers(1, min(nb, 6) + 1))
            dst = rng.permutation(nb)[:n]                      # one writer per destination page
            mapping = [[int(rng.integers(0, nb)), int(d)] for d in dst]
            v.copy_blocks(mapping if rng.random() < 0.5 else torch.tensor(mapping, dtype=torch.int32, device="cuda"))
            ot.copy_blocks(arrays, mapping)
        label = f"seed {seed} step {step} {op}"
        np.testing.assert_array_equal(v.block_tables.cpu().numpy(), bt, err_msg=label)
        np.testing.assert_array_equal(v.kv_lens.cpu().numpy(), lens, err_msg=label)
        for a, w in zip(_pool_arrays(v), arrays):
            np.testing.assert_array_equal(a.cpu().numpy().view(np.uint8), w.view(np.uint8), err_msg=label)
    v.check()
