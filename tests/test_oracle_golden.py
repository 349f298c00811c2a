"""The CPU oracle against outputs of the easymlx reference (tests/golden/*.npz)."""

import numpy as np
import pytest

import cases
from oracle import kv_write, paged_attention as opa

REF_ATTN = ["ref_attn_seed0", "ref_attn_seed1", "ref_attn_seed11"]


@pytest.mark.parametrize("name", REF_ATTN)
@pytest.mark.parametrize("fn", [opa.paged_attention_loop, opa.paged_attention_rows])
def test_reference_test_replays(golden, name, fn):
    g = golden(name)
    out = fn(g["q"], g["key_cache"], g["value_cache"], g["block_tables"], g["kv_lens"], g["query_start_loc"],
             softmax_scale=float(g["scale"]), sliding_window=int(g["window"]))
    # tolerance of the reference's own tests (tests/operations/test_unified_attention.py:145)
    np.testing.assert_allclose(out, g["out"], atol=1e-5, rtol=1e-5)


def _attn_inputs(spec, g):
    x = cases.attention_inputs(**spec)
    assert cases.digest(x["q"], x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"],
                        x["query_start_loc"]) == str(g["input_digest"]), "input generator drifted"
    return x


@pytest.mark.parametrize("name", sorted(cases.ATTENTION_CASES))
def test_loop_oracle_is_bit_identical_to_reference(golden, name):
    g = golden(name)
    x = _attn_inputs(cases.ATTENTION_CASES[name], g)
    out = opa.paged_attention_loop(x["q"], x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"],
                                   x["query_start_loc"], softmax_scale=x["scale"], sliding_window=x["window"])
    assert out.dtype == g["out"].dtype
    np.testing.assert_array_equal(out, g["out"])


@pytest.mark.parametrize("name", sorted(cases.ATTENTION_CASES))
def test_rows_oracle_matches_reference(golden, name):
    g = golden(name)
    x = _attn_inputs(cases.ATTENTION_CASES[name], g)
    out = opa.paged_attention_rows(x["q"], x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"],
                                   x["query_start_loc"], softmax_scale=x["scale"], sliding_window=x["window"])
    np.testing.assert_allclose(out.astype(np.float32), g["out"].astype(np.float32), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("name", sorted(cases.DENSE_SINGLE_CASES))
def test_dense_single_sequence(golden, name):
    g = golden(name)
    spec = cases.DENSE_SINGLE_CASES[name]
    x = _attn_inputs(spec, g)
    out = opa.dense_single_sequence(x["q"], x["key_cache"], x["value_cache"], block_tables=x["block_tables"],
                                    kv_lens=x["kv_lens"], query_start_loc=x["query_start_loc"],
                                    block_size=spec["bs"], softmax_scale=x["scale"], sliding_window=x["window"])
    np.testing.assert_allclose(out.astype(np.float32), g["out"].astype(np.float32), atol=1e-6, rtol=1e-6)
    # the ragged formulation agrees with the dense route within the op's tolerance
    ragged = opa.paged_attention_rows(x["q"], x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"],
                                      x["query_start_loc"], softmax_scale=x["scale"], sliding_window=x["window"])
    np.testing.assert_allclose(ragged.astype(np.float32), g["out"].astype(np.float32), atol=2e-3, rtol=1e-2)


def test_dense_single_sequence_declines_like_reference():
    x = cases.attention_inputs(**cases.ATTENTION_CASES["attn_f16_decode_d64"])
    assert opa.dense_single_sequence(x["q"], x["key_cache"], x["value_cache"], block_tables=x["block_tables"],
                                     kv_lens=x["kv_lens"], query_start_loc=x["query_start_loc"], block_size=128) is None


@pytest.mark.parametrize("name", sorted(cases.WRITE_CASES))
def test_write_placement(golden, name):
    g = golden(name)
    spec = cases.WRITE_CASES[name]
    x = cases.write_inputs(**spec)
    assert cases.digest(x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"], x["k"], x["v"],
                        x["slot_ids"], x["query_lens"]) == str(g["input_digest"])
    meta = kv_write.batch_metadata(x["query_lens"], x["slot_ids"], x["block_tables"], x["kv_lens"], x["block_size"])
    kc, vc = x["key_cache"].copy(), x["value_cache"].copy()
    kv_write.write_rows(kc, vc, x["k"], x["v"], meta["slot_mapping"])
    exp_k = x["key_cache"].reshape(-1, spec["hkv"], spec["d"]).copy()
    exp_v = x["value_cache"].reshape(-1, spec["hkv"], spec["d"]).copy()
    exp_k[g["changed_rows"]] = g["key_rows"]
    exp_v[g["changed_rows"]] = g["value_rows"]
    np.testing.assert_array_equal(kc.reshape(exp_k.shape), exp_k)
    np.testing.assert_array_equal(vc.reshape(exp_v.shape), exp_v)
    np.testing.assert_array_equal(np.sort(meta["slot_mapping"]), g["changed_rows"])
    np.testing.assert_array_equal(meta["kv_lens_all"], g["kv_lens_after"])
    np.testing.assert_array_equal(meta["block_tables"], g["meta_block_tables"])
    np.testing.assert_array_equal(meta["kv_lens"], g["meta_kv_lens"])
    np.testing.assert_array_equal(meta["query_start_loc"], g["query_start_loc"])


def test_write_reference_seed2(golden):
    g = golden("ref_write_seed2")
    meta = kv_write.batch_metadata(g["query_lens"], g["slot_ids"], g["block_tables_all"], g["kv_lens_before"],
                                   int(g["block_size"]))
    kc, vc = g["key_cache_before"].copy(), g["value_cache_before"].copy()
    kv_write.write_rows(kc, vc, g["k"], g["v"], meta["slot_mapping"])
    np.testing.assert_array_equal(kc, g["key_cache_after"])
    np.testing.assert_array_equal(vc, g["value_cache_after"])
    np.testing.assert_array_equal(meta["kv_lens_all"], g["kv_lens_after"])
    np.testing.assert_array_equal(meta["block_tables"], g["meta_block_tables"])
    np.testing.assert_array_equal(meta["kv_lens"], g["meta_kv_lens"])
    np.testing.assert_array_equal(g["prepared_queries"], g["q"])


def test_performer_reference_seed0(golden):
    g = golden("ref_performer_seed0")
    bs = int(g["block_size"])
    meta = kv_write.batch_metadata(g["query_lens"], g["slot_ids"], g["block_tables_all"], g["kv_lens_before"], bs)
    kc, vc = g["key_cache_before"].copy(), g["value_cache_before"].copy()
    kv_write.write_rows(kc, vc, g["k"], g["v"], meta["slot_mapping"])
    np.testing.assert_array_equal(kc, g["key_cache_after"])
    out = opa.paged_attention_loop(g["q"], kc, vc, meta["block_tables"], meta["kv_lens"], meta["query_start_loc"],
                                   softmax_scale=float(g["scale"]))
    np.testing.assert_allclose(out, g["out"], atol=1e-5, rtol=1e-5)


def test_append_matches_batch_write():
    x = cases.write_inputs(**cases.WRITE_CASES["write_ragged_f16"])
    meta = kv_write.batch_metadata(x["query_lens"], x["slot_ids"], x["block_tables"], x["kv_lens"], x["block_size"])
    kc, vc = x["key_cache"].copy(), x["value_cache"].copy()
    kv_write.write_rows(kc, vc, x["k"], x["v"], meta["slot_mapping"])
    kc2, vc2, lens2 = x["key_cache"].copy(), x["value_cache"].copy(), x["kv_lens"].copy()
    qsl = meta["query_start_loc"]
    for i, slot in enumerate(x["slot_ids"]):
        kv_write.append(kc2, vc2, x["block_tables"], lens2, int(slot), x["k"][qsl[i]:qsl[i + 1]],
                        x["v"][qsl[i]:qsl[i + 1]], x["block_size"])
    np.testing.assert_array_equal(kc, kc2)
    np.testing.assert_array_equal(vc, vc2)
    np.testing.assert_array_equal(meta["kv_lens_all"], lens2)


def test_merge_splits_equals_unsplit_softmax():
    rng = np.random.default_rng(5)
    n, d, parts = 700, 16, 5
    s = rng.standard_normal(n).astype(np.float32) * 3
    v = rng.standard_normal((n, d)).astype(np.float32)
    full = (np.exp(s - s.max())[:, None] * v).sum(0) / np.exp(s - s.max()).sum()
    cuts = [0, 100, 100, 350, 699, 700]  # includes an empty part
    po, pm, pl = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        if a == b:
            po.append(np.zeros(d, np.float32)); pm.append(np.float32(-np.inf)); pl.append(np.float32(0))
            continue
        m = s[a:b].max()
        e = np.exp(s[a:b] - m)
        po.append((e[:, None] * v[a:b]).sum(0)); pm.append(m); pl.append(e.sum())
    got = opa.merge_splits(np.stack(po), np.asarray(pm), np.asarray(pl))
    np.testing.assert_allclose(got, full, atol=1e-5, rtol=1e-5)
