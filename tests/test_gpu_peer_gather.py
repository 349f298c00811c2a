"""KV heads sharded over ranks with the output gathered by the attention kernels themselves
(``emlx_attn_decode_gather``): every rank stores its heads into every rank's full output and flags tell when.

One GPU plays the ranks one after the other.  Kernels that wait for one another must never be separate launches
on one GPU, so every flag another rank would send is put in place by the host before a rank's call; what the test
checks is the addressing (head offset and stride of the full output, stores into the other ranks' buffers), the flags
a call sends, the epoch bookkeeping and the bounded wait.  The real exchange between processes runs in
``test_two_processes_exchange_their_heads`` when the machine has two GPUs.
"""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from easymlx_b200 import _native as nv
from easymlx_b200 import workloads
from easymlx_b200.distributed import PEER_FLAG_BYTES, GatherTarget
from easymlx_b200.runtime import AttentionStep
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu

READY, DONE, EPOCH, TICKET = 0, 8, 16, 17   # int32 slots of a flag block (csrc/peer.cuh)
FAR = 1 << 20


def _batch(bits, qlens, prior):
    return workloads.Workload(name="shard", hq=32, hkv=4, d=128, bits=bits, qlens=np.asarray(qlens, np.int64),
                              prior=np.asarray(prior, np.int64), description="4 KV heads, one per rank")


def _step(w, gather=None):
    return AttentionStep(w.cache, w.q, w.k, w.v, w.qlens.tolist(), w.slot_ids, gather=gather)._eager()


@pytest.mark.parametrize("bits", [0, 8, 4])
@pytest.mark.parametrize("qlens,prior", [([1, 1, 1, 1, 1], [5000, 300, 129, 0, 2047]),      # decode rows, split and whole units
                                         ([1, 3, 1, 5], [700, 1000, 40, 4000])])             # 8-, 24- and 40-row units
def test_ranks_in_turn_fill_every_output(bits, qlens, prior):
    world, dev = 4, torch.device("cuda")
    whole = _batch(bits, qlens, prior)
    ref = _step(workloads.materialize(whole, dev, seed=3))
    t = int(whole.total_tokens)
    outs = [torch.full((t + 2, whole.hq, whole.d), float("nan"), dtype=torch.float16, device=dev) for _ in range(world)]
    flags = [torch.zeros(PEER_FLAG_BYTES // 4, dtype=torch.int32, device=dev) for _ in range(world)]
    for epoch in (1, 2):
        for o in outs:
            o.fill_(float("nan"))
        for r in range(world):
            flags[r][READY:READY + 8] = FAR      # "the others are ready and done": they are not running
            flags[r][DONE:DONE + 8] = FAR
            shard = workloads.materialize(whole, dev, seed=3, kv_head_slice=slice(r, r + 1))
            target = GatherTarget.local(outs, flags, r, head_offset=r * (whole.hq // world))
            got = _step(shard, gather=target)
            torch.cuda.synchronize()
            assert got.data_ptr() == outs[r].data_ptr() and got.shape == (t, whole.hq, whole.d)
            f = flags[r].cpu().numpy()
            assert f[EPOCH] == epoch and f[TICKET] == 0
            for peer in range(world):
                if peer != r:   # what rank r told the others
                    g = flags[peer].cpu().numpy()
                    assert g[READY + r] == epoch and g[DONE + r] == epoch
        for o in outs:
            assert_close(o[:t], ref.float().cpu().numpy())
            assert torch.isnan(o[t:]).all()      # nothing past the batch's tokens is touched


def test_wait_for_a_rank_that_never_answers_gives_up():
    world, dev = 2, torch.device("cuda")
    whole = _batch(8, [1, 1], [3000, 200])
    ref = _step(workloads.materialize(whole, dev, seed=5))
    t = int(whole.total_tokens)
    outs = [torch.zeros((t, whole.hq, whole.d), dtype=torch.float16, device=dev) for _ in range(world)]
    flags = [torch.zeros(PEER_FLAG_BYTES // 4, dtype=torch.int32, device=dev) for _ in range(world)]
    shard = workloads.materialize(whole, dev, seed=5, kv_head_slice=slice(0, 2))
    target = GatherTarget.local(outs, flags, 0, head_offset=0, poll_limit=50)   # rank 1 never runs
    from easymlx_b200.operations.kernels import unified_attention as ua

    status = ua._scratch.get(dev, "status", 4, zero=True)
    status.zero_()
    with pytest.raises(RuntimeError, match="wait timed out"):   # tests run with the device status checked per call
        _step(shard, gather=target)
    torch.cuda.synchronize()                       # the kernel returned: nothing hangs, nothing faults
    assert int(status.view(torch.int32)[0].item()) == 0          # reported once, then cleared
    got = outs[0]
    assert int(flags[0][EPOCH].item()) == 1 and int(flags[0][TICKET].item()) == 0
    # the rows were computed and stored all the same, and the context is still usable
    assert_close(got[:, :16], ref[:, :16].float().cpu().numpy())
    assert_close(outs[1][:, :16], ref[:, :16].float().cpu().numpy())
    again = _step(workloads.materialize(whole, dev, seed=5))
    assert_close(again, ref.float().cpu().numpy())


def test_gather_entry_point_rejects_what_it_cannot_serve():
    import ctypes as C

    dev = torch.device("cuda")
    whole = _batch(0, [1, 1], [300, 200])
    w = workloads.materialize(whole, dev, seed=1)
    flags = torch.zeros(PEER_FLAG_BYTES // 4, dtype=torch.int32, device=dev)
    out = torch.zeros((2, whole.hq, whole.d), dtype=torch.float16, device=dev)
    lib = nv.lib()
    ptrs = (C.c_void_p * 1)(out.data_ptr())
    fl = (C.c_void_p * 1)(flags.data_ptr())
    assert lib.emlx_gather_init(flags.data_ptr(), ptrs, fl, 9, 0, 0, None) == nv.EMLX_ERR_INVALID      # > 8 ranks
    assert lib.emlx_gather_init(flags.data_ptr(), ptrs, fl, 1, 1, 0, None) == nv.EMLX_ERR_INVALID      # rank out of range
    with pytest.raises(ValueError):
        AttentionStep(w.cache, w.q, w.k, w.v, w.qlens.tolist(), w.slot_ids,
                      gather=GatherTarget.local([out[:1]], [flags], 0, head_offset=0))._eager()        # too few tokens


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_exchange_their_heads():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.pop("EASYMLX_B200_CHECK", None)   # the worker records CUDA graphs; a status read per call synchronises the stream
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29741", os.path.join(root, "tests", "peer_gather_worker.py")]
    done = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert "peer gather ok" in done.stdout
