"""The allocation-free decode entry point against the regular one, through the C ABI.

``emlx_attn_decode_static`` serves embedders that cannot allocate device memory around the call (their
allocator owns all of HBM already, or they must avoid the device-wide synchronisation an allocation
implies): its work list and split-KV workspace sit in an array built into the library.  The file name
sorts last on purpose, so a run that stops at the first failure has already run every other test.
"""

import ctypes as C

import numpy as np
import pytest
import torch

import cases
from gpu_util import ATOL, RTOL, assert_close, dev, quantized_pool_from_float

pytestmark = pytest.mark.gpu


def _both(x, extra):
    from easymlx_b200 import _native as nv
    from easymlx_b200.operations.kernels.unified_attention import AttentionCall

    call = AttentionCall(dev(x["q"]), dev(x["key_cache"]), dev(x["value_cache"]), dev(x["block_tables"]),
                         dev(x["kv_lens"]), dev(x["query_start_loc"]), softmax_scale=x["scale"],
                         sliding_window=x["window"], kernel="decode", max_query_len=1, **extra)
    expected = call.plan().launch().clone()
    lib, stream = nv.lib(), nv.stream_ptr(call.device)
    outs = []
    for _ in range(2):  # two calls in a row share the built-in scratch
        out = torch.full_like(call.queries, float("nan"))
        args = nv.AttnArgs()
        C.memmove(C.byref(args), C.byref(call.args), C.sizeof(args))
        args.out = out.data_ptr()
        args.plan, args.plan_bytes, args.workspace, args.workspace_bytes = None, 0, None, 0
        nv.check(lib.emlx_attn_decode_static(args, call.pool, stream))
        torch.cuda.synchronize()
        outs.append(out)
    return expected, outs


@pytest.mark.parametrize("name", ["attn_f16_decode_d128", "attn_f16_decode_d64"])
def test_static_scratch_matches_regular_entry_fp16(name, golden):
    x = cases.attention_inputs(**cases.ATTENTION_CASES[name])
    expected, outs = _both(x, {})
    stored = golden(name)["out"]  # what the reference itself returned for these inputs
    for out in outs:
        assert not torch.isnan(out).any()
        assert_close(out, expected.float().cpu().numpy(), atol=ATOL, rtol=RTOL)
        assert_close(out, stored, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("qlens,hq,hkv", [([1, 1, 1], 64, 2), ([5, 1, 5], 16, 4)])
def test_static_scratch_with_wide_groups_and_a_row_class_hint(qlens, hq, hkv):
    """A GQA group of 32 (a single token already has more rows than the 16-row classes hold) and 5-token rows with a
    caller's row-class hint that was computed for a different kind of work list: the built-in entry point builds
    its own list, serves every row and ignores the hint.  Checked against the coverage kernel."""
    import easymlx_b200 as emlx
    from easymlx_b200 import _native as nv
    from easymlx_b200.operations.kernels.unified_attention import AttentionCall

    x = cases.attention_inputs(seed=77, hq=hq, hkv=hkv, d=128, bs=128, ctx=[300, 127, 513], qlens=qlens)
    args_t = (dev(x["q"]), dev(x["key_cache"]), dev(x["value_cache"]), dev(x["block_tables"]), dev(x["kv_lens"]),
              dev(x["query_start_loc"]))
    want = emlx.paged_attention(*args_t, softmax_scale=x["scale"], kernel="generic")
    call = AttentionCall(*args_t, softmax_scale=x["scale"], kernel="decode", max_query_len=max(qlens),
                         query_len_set=sorted(set(qlens)))
    lib, stream = nv.lib(), nv.stream_ptr(call.device)
    for _ in range(2):
        out = torch.full_like(call.queries, float("nan"))
        args = nv.AttnArgs()
        C.memmove(C.byref(args), C.byref(call.args), C.sizeof(args))
        args.out = out.data_ptr()
        args.plan, args.plan_bytes, args.workspace, args.workspace_bytes = None, 0, None, 0
        args.plan_flags = 1                      # speaks for a work list with 128-row units; the entry point drops it
        args.row_class_mask = 1 << 3             # "only class 3 occurs": true for such a list, wrong for the built-in one
        nv.check(lib.emlx_attn_decode_static(args, call.pool, stream))
        torch.cuda.synchronize()
        assert not torch.isnan(out).any()
        assert_close(out, want.float().cpu().numpy(), atol=ATOL, rtol=RTOL)
    # the regular decode entry with a 128-row work list cannot serve a 32-row group and says so instead of returning OK
    if hq // hkv == 32:
        args.plan, args.plan_bytes = call.args.plan, call.args.plan_bytes
        args.workspace, args.workspace_bytes = call.args.workspace, call.args.workspace_bytes
        args.row_class_mask = 0
        assert lib.emlx_attn_decode(args, call.pool, stream) == nv.EMLX_ERR_UNSUPPORTED


def test_static_scratch_matches_regular_entry_affine8():
    x = cases.attention_inputs(**cases.ATTENTION_CASES["attn_f16_decode_d128"])
    kcode, vcode, ks, kb, vs, vb = quantized_pool_from_float(x["key_cache"], x["value_cache"], 8)
    xq = dict(x, key_cache=kcode, value_cache=vcode)
    expected, outs = _both(xq, dict(k_scale=dev(ks), k_bias=dev(kb), v_scale=dev(vs), v_bias=dev(vb)))
    for out in outs:
        assert_close(out, expected.float().cpu().numpy(), atol=ATOL, rtol=RTOL)


def test_static_scratch_rejects_oversized_batches():
    from easymlx_b200 import _native as nv

    args, pool = nv.AttnArgs(), nv.Pool()
    args.total_tokens, args.num_seqs, args.num_q_heads = 1 << 20, 1 << 20, 32
    pool.num_kv_heads, pool.head_dim, pool.block_size = 8, 128, 128
    rc = nv.lib().emlx_attn_decode_static(args, pool, None)
    assert rc == nv.EMLX_ERR_WORKSPACE
    assert b"limit" in nv.lib().emlx_last_error()
