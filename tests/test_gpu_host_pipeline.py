"""``HostStepPipeline``: steps fed from pinned host memory with uploads, kernels and downloads overlapped over two
buffer sets must return, step after step, what the plain step returns."""

import numpy as np
import pytest
import torch

from easymlx_b200 import workloads
from easymlx_b200.runtime import AttentionStep, HostStepPipeline

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [0, 8])
@pytest.mark.parametrize("depth", [1, 2, 3])
def test_pipelined_steps_return_the_plain_result(bits, depth):
    whole = workloads.Workload(name="pipe", hq=16, hkv=4, d=128, bits=bits, qlens=np.asarray([1, 4, 1, 7], np.int64),
                               prior=np.asarray([900, 130, 0, 2000], np.int64))
    w = workloads.materialize(whole, "cuda", seed=9)
    ref = AttentionStep(w.cache, w.q, w.k, w.v, w.qlens.tolist(), w.slot_ids)._eager().cpu()
    pipe = HostStepPipeline(w.cache, (w.q.cpu(), w.k.cpu(), w.v.cpu()), w.qlens.tolist(), w.slot_ids, depth=depth)
    assert pipe.h2d_bytes_per_step == 2 * (w.q.numel() + w.k.numel() + w.v.numel())
    for n in range(7):
        i = pipe.submit()
        assert i == n % depth
        if n % 3 == 2:  # read a result while later steps are in flight
            pipe.downloaded[i].synchronize()
            assert torch.equal(pipe.result(i), ref)
            pipe.result(i).zero_()
    pipe.drain()
    torch.cuda.synchronize()
    last = (7 - 1) % depth
    assert torch.equal(pipe.result(last), ref)
