"""The C-ABI library builds, loads without a GPU and exports every symbol the header declares."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    from easymlx_b200 import build

    return build.build()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "easymlx_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(emlx_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(built_lib):
    handle = ctypes.CDLL(built_lib)
    names = _declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"


def test_binding_covers_the_header(built_lib):
    from easymlx_b200 import _native

    assert sorted(_native.SIGNATURES) == _declared_symbols()
    assert _native.lib().emlx_abi_version() >= 1


def test_struct_layouts_match_the_header():
    from easymlx_b200 import _native

    # 6 pointers + int64 + 6 int32; 5 pointers + 6 int32 + float + 3 int32 + 2x(pointer,size_t) + pointer
    assert ctypes.sizeof(_native.Pool) == 6 * 8 + 8 + 6 * 4
    assert ctypes.sizeof(_native.AttnArgs) == 5 * 8 + 10 * 4 + 4 * 8 + 8
    assert _native.AttnArgs.plan_flags.offset == 76 and _native.AttnArgs.plan.offset == 80


def test_per_device_setup_bookkeeping(built_lib):
    from easymlx_b200 import _native

    assert _native.lib().emlx_selftest_device_once() == 0


def test_host_side_validation_needs_no_gpu(built_lib):
    from easymlx_b200 import _native

    lib = _native.lib()
    pool = _native.Pool()
    rc = lib.emlx_kv_write(None, None, 0, 4, None, pool, None, None)
    assert rc == _native.EMLX_ERR_INVALID
    with pytest.raises(ValueError):
        _native.check(rc)
    assert b"key_cache" in lib.emlx_last_error()


def test_registry_and_requirements():
    import easymlx_b200 as emlx
    from easymlx_b200.operations import MetadataField

    for alias in ("unified_attention", "unified", "paged", "full_attention", "linear_attention"):
        assert emlx.OperationRegistry.get(alias) is emlx.UnifiedAttention
    req = emlx.UnifiedAttention.get_requirements()
    assert req.required_metadata == (MetadataField.QUERY_START_LOC | MetadataField.BLOCK_TABLES
                                     | MetadataField.KV_LENS | MetadataField.BLOCK_SIZE)
    assert req.optional_metadata == MetadataField.SLIDING_WINDOW
    assert req.requires_cache and req.cache_view_cls is emlx.PageCacheView
    with pytest.raises(KeyError):
        emlx.OperationRegistry.get("nope")
    with pytest.raises(ValueError, match="requires cache_metadata"):
        emlx.UnifiedAttention()(query=None, key=None, value=None)


def test_cpu_tensors_are_refused():
    import torch

    import easymlx_b200 as emlx

    q = torch.zeros((1, 2, 64), dtype=torch.float16)
    kc = torch.zeros((1, 128, 1, 64), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        emlx.paged_attention(q, kc, kc, torch.zeros((1, 1), dtype=torch.int32), torch.ones(1, dtype=torch.int32),
                             torch.tensor([0, 1], dtype=torch.int32))


def test_expanded_page_scratch_size_is_host_arithmetic(built_lib):
    """emlx_attn_dequant_bytes: scratch page table + two pools of MB pages per long sequence (+ fp16 copies of the
    queries and the output for bf16 queries); zero when the pool is not affine or nothing is long."""
    from easymlx_b200 import _native

    lib = _native.lib()
    pool = _native.Pool()
    pool.num_kv_heads, pool.head_dim, pool.block_size, pool.kv_format = 8, 128, 128, 8
    s, mb, n, t, hq = 244, 160, 4, 4096, 64
    page = 128 * 8 * 128 * 2
    header = -(-s * mb * 4 // 256) * 256
    assert lib.emlx_attn_dequant_bytes(pool, s, mb, n, t, hq, _native.F16) == header + 2 * page * n * mb
    rows = -(-t * hq * 128 * 2 // 256) * 256
    assert lib.emlx_attn_dequant_bytes(pool, s, mb, n, t, hq, _native.BF16) == header + 2 * rows + 2 * page * n * mb
    assert lib.emlx_attn_dequant_bytes(pool, s, mb, 0, t, hq, _native.F16) == 0
    pool.kv_format = _native.KV_FLOAT
    assert lib.emlx_attn_dequant_bytes(pool, s, mb, n, t, hq, _native.F16) == 0


def test_gather_arguments_are_checked_on_the_host(built_lib):
    from easymlx_b200 import _native

    lib = _native.lib()
    block = ctypes.create_string_buffer(512)
    outs = (ctypes.c_void_p * 2)(ctypes.addressof(block), ctypes.addressof(block))
    flags = (ctypes.c_void_p * 2)(ctypes.addressof(block), ctypes.addressof(block))
    assert lib.emlx_gather_init(None, outs, flags, 2, 0, 0, None) == _native.EMLX_ERR_INVALID
    assert lib.emlx_gather_init(ctypes.addressof(block), outs, flags, 9, 0, 0, None) == _native.EMLX_ERR_INVALID
    assert lib.emlx_gather_init(ctypes.addressof(block), outs, flags, 2, 2, 0, None) == _native.EMLX_ERR_INVALID
    other = ctypes.create_string_buffer(512)
    wrong = (ctypes.c_void_p * 2)(ctypes.addressof(other), ctypes.addressof(block))
    assert lib.emlx_gather_init(ctypes.addressof(block), outs, wrong, 2, 0, 0, None) == _native.EMLX_ERR_INVALID  # flags[rank] != own block
    assert lib.emlx_attn_decode_gather(None, None, None, 64, 0, None) == _native.EMLX_ERR_INVALID


def test_wide_unit_geometry_rule():
    from easymlx_b200.caching.paged.cache import wide_units_geometry

    assert wide_units_geometry(32, 8, 128) and wide_units_geometry(64, 8, 64) and wide_units_geometry(8, 8, 128)
    assert not wide_units_geometry(24, 8, 128)      # group of 3 does not divide 128
    assert not wide_units_geometry(32, 8, 256)      # head_dim outside {64, 128}
    assert not wide_units_geometry(30, 8, 128)      # not a whole group


def test_expanded_page_hint():
    from easymlx_b200.caching.paged.cache import expanded_page_hint

    assert expanded_page_hint(None, 4) == 0                     # lengths not known on the host
    assert expanded_page_hint((1,) * 128, 8) == 0               # decode rows only
    assert expanded_page_hint((1, 1, 512, 2030), 4) == 2        # prefill chunks beside decode rows
    assert expanded_page_hint((5,) * 64, 4) == 0                # spec-verify: 20 rows each, expansion does not pay
    assert expanded_page_hint((5,) * 64 + (2048,), 4) == 65     # one long chunk lifts the average above 64 rows
    assert expanded_page_hint((4,), 4) == 0                     # 16 rows fit the short-row classes
    assert expanded_page_hint((16,), 4) == 1                    # 64 rows
