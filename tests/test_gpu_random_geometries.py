"""Seeded random batches: head counts, group sizes, page sizes, pool formats, dtypes, windows and length mixes that
the hand-written cases do not enumerate.  Attention: the automatic kernel choice against the coverage kernel (an
independent code path that the golden-vector tests pin to the oracle), and bit-for-bit repeatability.  Cache write:
pools, scales, biases, lengths and gathered tables against the oracle, bit for bit."""

import numpy as np
import pytest
import torch

from gpu_util import ATOL, RTOL, dev
from oracle import kv_write

pytestmark = pytest.mark.gpu

_QLEN_CHOICES = {
    "decode": [1],
    "spec": list(range(1, 9)),
    "prefill": [0, 1, 16, 127, 128, 129, 300, 513],
    "mixed": [0, 1, 1, 1, 2, 3, 7, 8, 9, 33, 100, 257],
}


def _draw_attention_case(rng):
    d = int(rng.choice([64, 128]))
    hkv = int(rng.choice([1, 2, 3, 4, 8]))
    hq = hkv * int(rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 12, 16]))
    bits = int(rng.choice([0, 0, 8, 4]))
    dtype = torch.float16 if rng.random() < 0.6 else torch.bfloat16
    bs = 128 if bits else int(rng.choice([16, 32, 64, 128, 128]))
    nseq = int(rng.choice([1, 2, 3, 5, 17, 64, 200]))
    style = str(rng.choice(sorted(_QLEN_CHOICES)))
    qlens = [int(rng.choice(_QLEN_CHOICES[style])) for _ in range(nseq)]
    longest = [0, 1, 130, 1000, 5000] + ([40000] if nseq <= 17 else [])
    prior = [int(rng.integers(0, int(rng.choice(longest)) + 1)) for _ in range(nseq)]
    if sum(qlens) == 0:
        qlens[0] = 1
    window = None if rng.random() < 0.7 else int(rng.choice([1, 17, 128, 1000]))
    hints = bool(rng.random() < 0.5)
    return d, hq, hkv, bits, dtype, bs, qlens, prior, window, hints


def _random_pool(hkv, d, lens, bits, seed, block_size, dtype):
    """Pool with values well away from zero (codes uniform, scales 0.01 - 0.06) and every table row a random set of pages."""
    from easymlx_b200 import PageCacheView
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages = max(-(-int(n) // block_size) for n in lens)
    cache = PageCacheView.init(num_seqs=len(lens), max_seq_len=max(pages, 1) * block_size, num_kv_heads=hkv, head_dim=d,
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
    perm = torch.randperm(cache.num_blocks, device="cuda", generator=g).to(torch.int32)
    cache.block_tables.copy_(perm[: cache.block_tables.numel()].reshape(cache.block_tables.shape))
    return cache


def _attend(cache, q, qlens, kv, kernel, window, hints):
    import easymlx_b200 as emlx
    extra = dict(k_scale=cache.k_scales, v_scale=cache.v_scales, k_bias=cache.k_biases, v_bias=cache.v_biases) \
        if cache.is_affine else {}
    if hints and kernel is None:
        extra.update(max_query_len=max(qlens), query_len_set=sorted(set(qlens)))
        # with the count of sequences of more than 16 rows an affine pool serves them on the tcgen05 kernel through
        # expanded pages (when the head geometry allows); without it they stay on the 32-row units
        group = q.shape[1] // cache.num_kv_heads
        extra.update(long_seqs=sum(1 for n in qlens if n * group > 16))
    return emlx.paged_attention(q, cache.key_cache, cache.value_cache, cache.block_tables,
                                torch.tensor(kv, dtype=torch.int32, device="cuda"),
                                emlx.build_query_start_loc(qlens, device="cuda"), sliding_window=window, kernel=kernel, **extra)


@pytest.mark.parametrize("block", range(8))
def test_attention_over_random_batches(block):
    failures = []
    for case in range(block * 40, block * 40 + 40):
        rng = np.random.default_rng(90_000 + case)
        d, hq, hkv, bits, dtype, bs, qlens, prior, window, hints = _draw_attention_case(rng)
        if sum(qlens) > 6000:
            continue
        kv = [a + b for a, b in zip(qlens, prior)]
        cache = _random_pool(hkv, d, [max(n, 1) for n in kv], bits, case, bs, dtype)
        q = torch.randn(sum(qlens), hq, d, device="cuda", generator=torch.Generator(device="cuda").manual_seed(case + 5)).to(dtype)
        fast = _attend(cache, q, qlens, kv, None, window, hints)
        ref = _attend(cache, q, qlens, kv, "generic", window, hints)
        a, e = fast.float(), ref.float()
        # bf16 keeps 8 bits of the weights and of the output: the stated fp16 tolerance, widened by that much
        atol, rtol = (ATOL, RTOL) if dtype == torch.float16 else (8e-3, 2e-2)
        excess = ((a - e).abs() - (atol + rtol * e.abs())).max().item()
        what = dict(case=case, d=d, hq=hq, hkv=hkv, bits=bits, dtype=str(dtype), page=bs, window=window, hints=hints,
                    qlens=qlens[:8], prior=prior[:8])
        if not torch.isfinite(a).all():
            failures.append(("non-finite output", what))
        elif excess > 0:
            failures.append((f"excess over the tolerance {excess:.2e}", what))
        elif not torch.equal(fast, _attend(cache, q, qlens, kv, None, window, hints)):
            failures.append(("not repeatable bit for bit", what))
    assert not failures, failures


def _draw_rows(rng, t, h, d, kind):
    x = rng.standard_normal((t, h, d)).astype(np.float32)
    if kind == "big":
        x *= 300.0
    elif kind == "tiny":
        x *= 1e-4
    elif kind == "offset":
        x += 5.0
    elif kind == "mixed":
        x *= np.exp(rng.uniform(-8, 6, size=(t, h, 1))).astype(np.float32)
        x[rng.integers(0, t)] = 0.0        # a constant row: scale 0
        x[rng.integers(0, t)] = 1.25
    return x.astype(np.float16)


@pytest.mark.parametrize("block", range(4))
def test_cache_write_over_random_batches(block):
    from easymlx_b200 import PageCacheView, PageMetadata, build_query_start_loc
    for case in range(block * 10, block * 10 + 10):
        rng = np.random.default_rng(70_000 + case)
        d, hkv, bits = int(rng.choice([64, 128, 256])), int(rng.choice([1, 2, 3, 8])), int(rng.choice([0, 8, 4]))
        bs, slots = int(rng.choice([16, 32, 64, 128])), int(rng.choice([1, 3, 9, 40, 300]))
        max_len = int(rng.choice([130, 700, 3000]))
        kind = str(rng.choice(["normal", "big", "tiny", "mixed", "offset"]))
        slot_ids = rng.permutation(slots)[: int(rng.integers(1, slots + 1))]
        style = str(rng.choice(["decode", "spec", "ragged"]))
        prior_all = rng.integers(0, max_len, size=slots).astype(np.int32)
        pick = {"decode": [1], "spec": list(range(1, 9)), "ragged": [0, 1, 2, 17, 128, 333]}[style]
        qlens = np.asarray([min(int(rng.choice(pick)), max_len - int(prior_all[s])) for s in slot_ids], dtype=np.int64)
        t = int(qlens.sum())
        if t == 0 or t > 20000:
            continue
        cache = PageCacheView.init(num_seqs=slots, max_seq_len=max_len, num_kv_heads=hkv, head_dim=d, block_size=bs,
                                   cache_dtype=(f"affine{bits}" if bits else None), device="cuda")
        # stale contents everywhere and a scrambled table: exactly the addressed rows may change
        if bits:
            kc0 = rng.integers(0, 256, size=tuple(cache.key_cache.shape), dtype=np.uint8)
            vc0 = rng.integers(0, 256, size=tuple(cache.value_cache.shape), dtype=np.uint8)
            sb0 = [rng.standard_normal(tuple(cache.k_scales.shape)).astype(np.float16) for _ in range(4)]
            for tensor, a in zip((cache.k_scales, cache.k_biases, cache.v_scales, cache.v_biases), sb0):
                tensor.copy_(dev(a))
        else:
            kc0 = rng.standard_normal(tuple(cache.key_cache.shape)).astype(np.float16)
            vc0 = rng.standard_normal(tuple(cache.value_cache.shape)).astype(np.float16)
        cache.key_cache.copy_(dev(kc0))
        cache.value_cache.copy_(dev(vc0))
        bt = rng.permutation(cache.num_blocks)[: cache.block_tables.numel()].reshape(tuple(cache.block_tables.shape)).astype(np.int32)
        cache.block_tables.copy_(dev(bt))
        cache.kv_lens.copy_(dev(prior_all))
        q, k, v = _draw_rows(rng, t, 2 * hkv, d, "normal"), _draw_rows(rng, t, hkv, d, kind), _draw_rows(rng, t, hkv, d, kind)
        hint = qlens.tolist() if rng.random() < 0.5 else None
        _, _, _, meta = cache.concatenate_to_cache(
            dev(q), dev(k), dev(v), cache_metadata=PageMetadata(query_start_loc=build_query_start_loc(qlens.tolist())),
            slot_ids=slot_ids.tolist(), query_lens=hint)
        cache.check()
        want = kv_write.batch_metadata(qlens, slot_ids, bt, prior_all, bs)
        label = f"case {case}: d={d} hkv={hkv} bits={bits} page={bs} slots={slots} {style} {kind} T={t}"
        if bits:
            ks, kb, vs, vb = [a.copy() for a in sb0]
            kv_write.write_key_rows_quantized(kc0, ks, kb, k, want["slot_mapping"], bits)
            kv_write.write_value_rows_quantized(vc0, vs, vb, v, want["slot_mapping"], bits)
            for tensor, a in zip((cache.k_scales, cache.k_biases, cache.v_scales, cache.v_biases), (ks, kb, vs, vb)):
                np.testing.assert_array_equal(tensor.cpu().numpy().view(np.uint16), a.view(np.uint16), err_msg=label)
        else:
            kv_write.write_rows(kc0, vc0, k, v, want["slot_mapping"])
        word = np.uint8 if bits else np.uint16
        np.testing.assert_array_equal(cache.key_cache.cpu().numpy().view(word), kc0.view(word), err_msg=label)
        np.testing.assert_array_equal(cache.value_cache.cpu().numpy().view(word), vc0.view(word), err_msg=label)
        np.testing.assert_array_equal(cache.kv_lens.cpu().numpy(), want["kv_lens_all"], err_msg=label)
        np.testing.assert_array_equal(meta.kv_lens.cpu().numpy(), want["kv_lens"], err_msg=label)
        np.testing.assert_array_equal(meta.block_tables.cpu().numpy(), want["block_tables"], err_msg=label)


@pytest.mark.parametrize("block", range(4))
def test_small_random_batches_against_the_oracle(block):
    """Both routes against the oracle itself on batches small enough for it: head sizes and page sizes that only the
    coverage kernel takes (32, 96, 256; pages of 8 or 48 tokens), fp32 and fp16 queries, 8- and 4-bit pools built by the
    oracle's quantiser, negative page ids past the sequence end."""
    from easymlx_b200 import paged_attention
    from gpu_util import assert_close, quantized_pool_from_float
    from oracle import kv_quant, paged_attention as opa
    for case in range(block * 8, block * 8 + 8):
        rng = np.random.default_rng(50_000 + case)
        d = int(rng.choice([32, 64, 96, 128, 256]))
        hkv = int(rng.choice([1, 2, 3]))
        hq = hkv * int(rng.choice([1, 2, 4, 7]))
        bs = int(rng.choice([8, 16, 48, 128]))
        bits = int(rng.choice([0, 0, 8, 4])) if d % 64 == 0 else 0
        f32 = bits == 0 and rng.random() < 0.3
        nseq = int(rng.integers(1, 7))
        qlens = [int(rng.choice([0, 1, 1, 2, 5, 19, 140])) for _ in range(nseq)]
        prior = [int(rng.integers(0, 400)) for _ in range(nseq)]
        if sum(qlens) == 0:
            qlens[0] = 1
        kv = np.asarray([a + b for a, b in zip(qlens, prior)], dtype=np.int32)
        window = 0 if rng.random() < 0.6 else int(rng.choice([1, 9, 200]))
        mb = max(1, -(-int(kv.max()) // bs)) + 1
        nb = nseq * mb
        bt = rng.permutation(nb).reshape(nseq, mb).astype(np.int32)
        for s in range(nseq):                       # entries past the last page of a sequence are -1, as an engine leaves them
            bt[s, -(-int(kv[s]) // bs):] = -1
        np_dtype = np.float32 if f32 else np.float16
        kc = rng.standard_normal((nb, bs, hkv, d)).astype(np_dtype)
        vc = rng.standard_normal((nb, bs, hkv, d)).astype(np_dtype)
        q = rng.standard_normal((sum(qlens), hq, d)).astype(np_dtype)
        qsl = kv_write.build_query_start_loc(qlens)
        scale = float(d) ** -0.5
        label = f"case {case}: d={d} hq={hq} hkv={hkv} page={bs} bits={bits} f32={f32} window={window} qlens={qlens} prior={prior}"
        extra = {}
        if bits:
            kcode, vcode, ks, kb, vs, vb = quantized_pool_from_float(kc, vc, bits)
            kf = kv_quant.dequantize_key_pool(kcode, ks, kb, bits)
            vf = kv_quant.dequantize_value_pool(vcode, vs, vb, bits)
            pools = (dev(kcode), dev(vcode))
            extra = dict(k_scale=dev(ks), k_bias=dev(kb), v_scale=dev(vs), v_bias=dev(vb))
        else:
            kf, vf, pools = kc, vc, (dev(kc), dev(vc))
        expect = opa.paged_attention_rows(q, kf, vf, bt, kv, qsl, softmax_scale=scale, sliding_window=window)
        for kernel in ("generic", None):
            out = paged_attention(dev(q), *pools, dev(bt), dev(kv), dev(qsl), softmax_scale=scale,
                                  sliding_window=(window or None), kernel=kernel, **extra)
            try:
                assert_close(out, expect, **(dict(atol=1e-5, rtol=1e-5) if f32 else {}))
            except AssertionError as err:
                raise AssertionError(f"{label} kernel={kernel}: {err}") from None
