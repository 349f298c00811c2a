"""Properties of the oracle that hold at any size: its two attention restatements against a float64 attention written
per (token, head) from the definition, the merge of split partial results, and the affine quantiser's round trip."""

import numpy as np
import pytest

from oracle import kv_quant, paged_attention as opa


def _random_batch(rng, hq, hkv, d, bs, qlens, priors, spare_pages=3, dtype=np.float16):
    kv = [p + q for p, q in zip(priors, qlens)]
    pages_per_seq = [(n + bs - 1) // bs for n in kv]
    mb = max(pages_per_seq) + 1
    nb = sum(pages_per_seq) + spare_pages
    perm = rng.permutation(nb)
    bt = np.full((len(kv), mb), -1, np.int32)
    at = 0
    for s, n in enumerate(pages_per_seq):
        bt[s, :n] = perm[at:at + n]
        at += n
    kc = rng.standard_normal((nb, bs, hkv, d)).astype(dtype)
    vc = rng.standard_normal((nb, bs, hkv, d)).astype(dtype)
    q = rng.standard_normal((sum(qlens), hq, d)).astype(dtype)
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    return q, kc, vc, bt, np.asarray(kv, np.int32), qsl


def _attention_from_the_definition(q, kc, vc, bt, kv_lens, qsl, scale, window):
    """float64, one (token, q head) at a time: keys ctx+i-window+1 .. ctx+i of the sequence's contiguous history."""
    t, hq, d = q.shape
    bs, hkv = kc.shape[1], kc.shape[2]
    group = hq // hkv
    out = np.zeros((t, hq, d), np.float64)
    for s in range(len(kv_lens)):
        n, q0, q1 = int(kv_lens[s]), int(qsl[s]), int(qsl[s + 1])
        ctx = n - (q1 - q0)
        for i in range(q1 - q0):
            last = min(n - 1, ctx + i)
            first = max(0, last - window + 1) if window > 0 else 0
            if last < first:
                continue
            pos = np.arange(first, last + 1)
            pages = bt[s, pos // bs]
            for h in range(hq):
                k = kc[pages, pos % bs, h // group].astype(np.float64)
                v = vc[pages, pos % bs, h // group].astype(np.float64)
                sc = k @ (q[q0 + i, h].astype(np.float64) * scale)
                w = np.exp(sc - sc.max())
                out[q0 + i, h] = (w / w.sum()) @ v
    return out


@pytest.mark.parametrize("seed,hq,hkv,d,bs,window", [
    (0, 4, 2, 32, 16, 0), (1, 8, 1, 64, 8, 0), (2, 6, 2, 16, 128, 0), (3, 4, 4, 32, 16, 9), (4, 12, 4, 64, 48, 40),
    (5, 3, 1, 96, 16, 1),
])
def test_both_restatements_follow_the_definition(seed, hq, hkv, d, bs, window):
    rng = np.random.default_rng(seed)
    qlens = [int(x) for x in rng.integers(1, 12, size=5)]
    priors = [int(x) for x in rng.integers(0, 70, size=5)]
    priors[1] = 0                      # a sequence that starts with this chunk
    qlens[2] = 1                       # a decode row
    q, kc, vc, bt, kv_lens, qsl = _random_batch(rng, hq, hkv, d, bs, qlens, priors, dtype=np.float32)
    scale = d ** -0.5
    want = _attention_from_the_definition(q, kc, vc, bt, kv_lens, qsl, scale, window)
    loop = opa.paged_attention_loop(q, kc, vc, bt, kv_lens, qsl, softmax_scale=scale, sliding_window=window)
    rows = opa.paged_attention_rows(q, kc, vc, bt, kv_lens, qsl, softmax_scale=scale, sliding_window=window)
    np.testing.assert_allclose(loop, want, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(rows, want, rtol=2e-5, atol=2e-6)


def test_rows_of_idle_and_empty_sequences_stay_zero():
    rng = np.random.default_rng(7)
    q, kc, vc, bt, kv_lens, qsl = _random_batch(rng, 4, 2, 32, 16, [3, 2, 4], [5, 0, 9], dtype=np.float32)
    kv_lens[1] = 0                     # scheduled, but nothing stored: the reference leaves such rows at zero
    out = opa.paged_attention_rows(q, kc, vc, bt, kv_lens, qsl, softmax_scale=0.2)
    assert not out[qsl[1]:qsl[2]].any()
    assert out[qsl[0]:qsl[1]].any() and out[qsl[2]:qsl[3]].any()
    np.testing.assert_array_equal(out, opa.paged_attention_rows(q, kc, vc, bt, kv_lens, qsl, softmax_scale=0.2,
                                                                seq_subset=[0, 1, 2]))


def test_unassigned_pages_read_as_zero_rows():
    rng = np.random.default_rng(8)
    q, kc, vc, bt, kv_lens, qsl = _random_batch(rng, 2, 1, 16, 8, [1], [30], dtype=np.float32)
    holed = bt.copy()
    holed[0, 1] = -1                   # keys 8..15 are lost
    zeroed_k, zeroed_v = kc.copy(), vc.copy()
    zeroed_k[bt[0, 1]] = 0
    zeroed_v[bt[0, 1]] = 0
    a = opa.paged_attention_loop(q, kc, vc, holed, kv_lens, qsl, softmax_scale=0.25)
    b = opa.paged_attention_loop(q, zeroed_k, zeroed_v, bt, kv_lens, qsl, softmax_scale=0.25)
    np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("parts", [2, 5, 18])
def test_merge_of_any_split_equals_the_whole(parts):
    rng = np.random.default_rng(parts)
    n, d = 400, 24
    s = rng.standard_normal(n) * 6
    v = rng.standard_normal((n, d))
    w = np.exp(s - s.max())
    whole = (w / w.sum()) @ v
    cuts = np.sort(rng.choice(np.arange(1, n), size=parts - 1, replace=False))
    outs, maxs, sums = [], [], []
    for lo, hi in zip(np.concatenate([[0], cuts]), np.concatenate([cuts, [n]])):
        m = s[lo:hi].max()
        e = np.exp(s[lo:hi] - m)
        outs.append(e @ v[lo:hi])          # un-normalised accumulator of the part
        maxs.append(m)
        sums.append(e.sum())
    got = opa.merge_splits(np.asarray(outs), np.asarray(maxs), np.asarray(sums))
    np.testing.assert_allclose(got, whole, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("bits", [8, 4])
def test_quantiser_round_trip_is_within_half_a_step_and_stable(bits):
    rng = np.random.default_rng(bits)
    x = (rng.standard_normal((50, 3, 128)) * np.exp(rng.uniform(-4, 3, size=(50, 3, 1)))).astype(np.float16)
    x[0, 0, :64] = 0.75                # a constant group: scale falls back to 1, every code 0
    codes, scale, bias = kv_quant.quantize_rows(x, bits)
    assert codes.max() <= (1 << bits) - 1 and scale.dtype == np.float16 and bias.dtype == np.float16
    assert not codes[0, 0, :64].any() and scale[0, 0, 0] == 1 and bias[0, 0, 0] == np.float16(0.75)
    back = kv_quant.dequantize_rows(codes, scale, bias)
    step = np.repeat(scale.astype(np.float32), 64, axis=-1)
    # half a step, plus what rounding scale and bias to fp16 can move the top of the range by
    slack = 0.5 * step + ((1 << bits) - 1) * step * 2.0 ** -10 + np.abs(x.astype(np.float32)) * 2.0 ** -10
    assert (np.abs(back - x.astype(np.float32)) <= slack).all()
    # stored bytes survive pack / unpack, and the codes of the dequantised rows' own grid are the codes
    np.testing.assert_array_equal(kv_quant.unpack_codes(kv_quant.pack_codes(codes, bits), bits), codes)
    grid = scale.astype(np.float32)[..., None] * codes.reshape(50, 3, 2, 64) + bias.astype(np.float32)[..., None]
    again = np.clip(np.rint((grid - bias.astype(np.float32)[..., None]) / scale.astype(np.float32)[..., None]), 0,
                    (1 << bits) - 1).astype(np.uint8)
    np.testing.assert_array_equal(again.reshape(codes.shape), codes)
