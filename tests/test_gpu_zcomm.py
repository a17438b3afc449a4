"""The library's communicator when a rank never joins: a host-side deadline, no GPU fault (one GPU is enough)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _lonely_rank(ret):
    """Rank 0 of a world of two whose partner never starts."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import floneum_b200 as fb
    from floneum_b200 import FusorCudaError, _lib
    from floneum_b200.sharding import Communicator
    import time
    dev = fb.Device.gpu(0)
    t0 = time.time()
    try:
        Communicator(dev, 0, 2, timeout_ms=3000, unique_id=Communicator.make_unique_id())
        ret["code"] = "joined"
    except FusorCudaError as e:
        ret["code"], ret["msg"], ret["seconds"] = e.code, e.message, time.time() - t0
    # the context is intact: a kernel still runs on it
    q = np.ones((1, 2, 4, 16), np.float32)
    out = fb.Tensor.from_slice(dev, q.shape, q).flash_attention(fb.Tensor.from_slice(dev, q.shape, q), fb.Tensor.from_slice(dev, q.shape, q), 0.25)
    ret["after"] = float(np.abs(out.as_slice() - 1.0).max())
    ret["timeout_code"] = _lib.TIMEOUT


def test_communicator_init_times_out_when_a_rank_never_joins():
    """Failure detection on the host: the second rank of the communicator is never started.  The non-blocking
    initialisation is polled against the deadline, the communicator is aborted, the caller gets TIMEOUT and the context
    still computes.  Runs in a child process (an aborted communicator stays behind in the library's state)."""
    import torch
    if torch.cuda.device_count() < 1:
        pytest.skip("needs a GPU")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    p = ctx.Process(target=_lonely_rank, args=(ret,))
    p.start()
    p.join(120)
    if p.is_alive():
        p.terminate()
        pytest.fail("the lonely rank did not come back")
    assert ret.get("code") == ret.get("timeout_code"), dict(ret)
    assert "did not complete within 3000 ms" in ret["msg"] and 2.5 <= ret["seconds"] <= 60
    assert ret["after"] < 1e-6
