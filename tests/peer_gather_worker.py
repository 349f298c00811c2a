"""Worker of ``test_two_processes_exchange_their_heads`` (launched with torch.distributed.run, one process per GPU):
KV heads sharded over the ranks, the attention kernels store their heads into every rank's output through peer-mapped
memory; every rank compares what it received with the unsharded result."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from easymlx_b200 import workloads  # noqa: E402
from easymlx_b200.distributed import PeerGather, all_gather_heads  # noqa: E402
from easymlx_b200.operations.kernels import unified_attention as ua  # noqa: E402
from easymlx_b200.runtime import AttentionStep  # noqa: E402


def close(a, b):
    err = (a.float() - b.float()).abs()
    return bool((err <= 2e-3 + 1e-2 * b.float().abs()).all().item()), float(err.max().item())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    failures = []
    for bits, qlens, prior in ((4, [1] * 6, [9000, 300, 129, 0, 2047, 5555]), (0, [1, 3, 1, 5], [700, 1000, 40, 4000])):
        whole = workloads.Workload(name="shard", hq=32, hkv=4, d=128, bits=bits, qlens=np.asarray(qlens, np.int64),
                                   prior=np.asarray(prior, np.int64))
        per = whole.hkv // world
        ref_w = workloads.materialize(whole, dev, seed=3)
        ref = AttentionStep(ref_w.cache, ref_w.q, ref_w.k, ref_w.v, ref_w.qlens.tolist(), ref_w.slot_ids)._eager()
        shard = workloads.materialize(whole, dev, seed=3, kv_head_slice=slice(rank * per, (rank + 1) * per))
        t = int(whole.total_tokens)
        # the NCCL route, for comparison
        local = AttentionStep(shard.cache, shard.q, shard.k, shard.v, shard.qlens.tolist(), shard.slot_ids)._eager()
        ok, err = close(all_gather_heads(local), ref)
        if not ok:
            failures.append(f"bits {bits}: all-gather route differs ({err})")
        peers = PeerGather(t, whole.hq, whole.d, torch.float16, dev, poll_limit=1 << 24)
        step = AttentionStep(shard.cache, shard.q, shard.k, shard.v, shard.qlens.tolist(), shard.slot_ids,
                             gather=peers.target)
        for i in range(5):
            out = step._eager()
            torch.cuda.synchronize()
            ok, err = close(out, ref)
            if not ok:
                failures.append(f"bits {bits}: eager call {i} differs ({err})")
            peers.output(t).add_(1000.0)  # a stale row would show in the next call
        dist.barrier()
        step.capture(warmup=2, steps_per_graph=4)
        dist.barrier()
        for i in range(3):
            out = step.step()
            torch.cuda.synchronize()
            ok, err = close(out, ref)
            if not ok:
                failures.append(f"bits {bits}: graph replay {i} differs ({err})")
        status = int(ua._scratch.get(dev, "status", 4, zero=True).view(torch.int32)[0].item())
        if status:
            failures.append(f"bits {bits}: device status {status}")
        peers.close()
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    if failures:
        print(f"rank {rank}: " + "; ".join(failures), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if int(flag.item()):
        sys.exit(1)
    if rank == 0:
        print("peer gather ok", flush=True)


if __name__ == "__main__":
    main()
