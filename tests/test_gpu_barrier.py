"""
The bounded cross-GPU barrier kernel. A wait that nobody satisfies must run out, report status 4 through the device
status word and leave the context usable. Nothing here faults or hangs a GPU: the "missing" peer is simply a flag that
no one sets, and the deadline is a few milliseconds.
"""

import ctypes

import pytest
import torch

from olmo_core_b200.testing import requires_multi_gpu, run_distributed_test

pytestmark = pytest.mark.gpu


def test_barrier_wait_expires_and_reports_status():
    from olmo_core_b200.ops import _lib

    dev = torch.device("cuda", 0)
    L = _lib.lib()
    words = L.ocb_peer_barrier_flag_words()
    mine = torch.zeros(words, dtype=torch.int32, device=dev)
    absent = torch.zeros(words, dtype=torch.int32, device=dev)  # stands in for a rank that never arrives
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
    st = _lib.status_buffer(dev)
    _lib.check_device_status(dev)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    assert L.ocb_peer_barrier(ptrs, 2, 0, 0, 1, 5, -1, st.data_ptr(), _lib.stream_ptr()) == 0
    stop.record()
    torch.cuda.synchronize()
    assert 4.0 < start.elapsed_time(stop) < 500.0  # gave up after the 5 ms deadline, not earlier and not much later
    with pytest.raises(_lib.KernelError, match="another rank"):
        _lib.check_device_status(dev)
    # this rank's own signal did go out, and the context still works
    assert int(absent[0].item()) == 1 and int(mine[0].item()) == 1
    _lib.check_device_status(dev)
    # a world of one completes at once
    one = (ctypes.c_void_p * 1)(mine.data_ptr())
    assert L.ocb_peer_barrier(one, 1, 0, 1, 1, 5, -1, st.data_ptr(), _lib.stream_ptr()) == 0
    torch.cuda.synchronize()
    _lib.check_device_status(dev)


def _withheld_signal_worker():
    import torch.distributed as dist

    from olmo_core_b200.ops import _lib
    from olmo_core_b200.parallel.symmetric import SymmetricBuffer

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    buf = SymmetricBuffer(1024, torch.float32, dev, dist.group.WORLD)
    # a normal barrier carries data: rank r writes into its peer's buffer, the peer reads it after the barrier
    peer = 1 - rank
    buf.barrier()
    buf.tensor.fill_(float(rank + 1))
    buf.barrier()
    torch.cuda.synchronize()
    _lib.check_device_status(dev)
    # rank 1 withholds its signal from rank 0 once: rank 0's wait runs out, rank 1's does not
    buf.barrier(timeout_ms=200, _skip_signal_rank=0 if rank == 1 else -1)
    torch.cuda.synchronize()
    if rank == 0:
        with pytest.raises(_lib.KernelError, match="another rank"):
            _lib.check_device_status(dev)
    else:
        _lib.check_device_status(dev)
    # epochs only grow, so the next barrier works again for both
    dist.barrier()
    buf.barrier()
    torch.cuda.synchronize()
    _lib.check_device_status(dev)
    assert peer in (0, 1)


@requires_multi_gpu
def test_barrier_two_gpus_withheld_signal(monkeypatch):
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    monkeypatch.setenv("OLMO_CORE_B200_MULTIMEM", "0")
    run_distributed_test(_withheld_signal_worker, world_size=2, backend="cuda:nccl,cpu:gloo")
