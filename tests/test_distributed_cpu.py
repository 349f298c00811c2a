"""World-size-2 gloo runs on CPU of the multi-GPU host logic: sequence partition, output reassembly and the
KV-head all-gather.  The per-rank attention is played by the CPU oracle (the CUDA kernels are covered by the
GPU tests); what is checked here is that sharding + gathering reproduces the unsharded batch exactly."""

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from oracle import paged_attention as opa


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _subset(x, seqs):
    """The batch restricted to some sequences (own queries, own table rows; the pool is shared read-only here)."""
    from easymlx_b200.distributed import local_token_index

    qlens = np.diff(x["query_start_loc"])
    tok = local_token_index(qlens, seqs)
    return dict(q=x["q"][tok], block_tables=x["block_tables"][seqs], kv_lens=x["kv_lens"][seqs],
                query_start_loc=np.concatenate([[0], np.cumsum(qlens[seqs])]).astype(np.int32))


def _seq_worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from easymlx_b200.distributed import gather_packed_outputs, partition_by_sequence

    x = cases.attention_inputs(**cases.ATTENTION_CASES["attn_f16_mixed_d64"])
    qlens = np.diff(x["query_start_loc"])
    parts = partition_by_sequence(qlens, x["kv_lens"], world)
    sub = _subset(x, parts[rank])
    local = opa.paged_attention_rows(sub["q"], x["key_cache"], x["value_cache"], sub["block_tables"], sub["kv_lens"],
                                     sub["query_start_loc"], softmax_scale=x["scale"])
    full = gather_packed_outputs(torch.from_numpy(local), qlens, parts)
    if rank == 0:
        result.put(full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_sequence_partition_reassembles_the_batch():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_seq_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = cases.attention_inputs(**cases.ATTENTION_CASES["attn_f16_mixed_d64"])
    want = opa.paged_attention_rows(x["q"], x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"],
                                    x["query_start_loc"], softmax_scale=x["scale"])
    np.testing.assert_array_equal(got, want)


def _head_worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from easymlx_b200.distributed import all_gather_heads

    x = cases.attention_inputs(**cases.ATTENTION_CASES["attn_f16_decode_d64"])
    hq, hkv = x["q"].shape[1], x["key_cache"].shape[2]
    g, per = hq // hkv, hkv // world
    kv_slice = slice(rank * per, (rank + 1) * per)
    local = opa.paged_attention_rows(x["q"][:, rank * per * g:(rank + 1) * per * g], x["key_cache"][:, :, kv_slice],
                                     x["value_cache"][:, :, kv_slice], x["block_tables"], x["kv_lens"],
                                     x["query_start_loc"], softmax_scale=x["scale"])
    full = all_gather_heads(torch.from_numpy(local))
    if rank == 0:
        result.put(full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_kv_head_shard_all_gather():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_head_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = cases.attention_inputs(**cases.ATTENTION_CASES["attn_f16_decode_d64"])
    want = opa.paged_attention_rows(x["q"], x["key_cache"], x["value_cache"], x["block_tables"], x["kv_lens"],
                                    x["query_start_loc"], softmax_scale=x["scale"])
    np.testing.assert_array_equal(got, want)


def test_partition_is_a_balanced_cover():
    from easymlx_b200 import workloads
    from easymlx_b200.distributed import partition_by_sequence

    for name in ("c2", "c3", "c5"):
        w = workloads.describe(name)
        for world in (2, 4, 8):
            parts = partition_by_sequence(w.qlens, w.kv_lens, world)
            flat = np.sort(np.concatenate(parts))
            np.testing.assert_array_equal(flat, np.arange(len(w.qlens)))
            load = np.array([w.kv_lens[p].sum() + 64 * w.qlens[p].sum() for p in parts], dtype=np.float64)
            assert load.max() <= 1.25 * load.mean() + w.kv_lens.max()
