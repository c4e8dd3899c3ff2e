"""A device-side wait that runs out: the kernel returns an error status, the context stays usable.

No fault, trap or endless loop is involved: the peer-flag barrier is launched for a world of two
whose second rank does not exist (its flag word is a local buffer nothing ever writes), with a
50 microsecond budget. The kernel must come back by itself with status word 5, the host-side
check must raise, and the next launch on the same context must work.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_barrier_gives_up_with_a_status_and_the_context_survives():
    from shadowspill_b200.ops import _lib
    from shadowspill_b200.parallel import collectives  # noqa: F401  (registers the signatures)
    lib = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    mine = torch.zeros(64, dtype=torch.int32, device=dev)      # flags written by the peers
    theirs = torch.zeros(64, dtype=torch.int32, device=dev)    # stands for rank 1's flag words
    ptrs = (C.c_void_p * 2)(mine.data_ptr(), theirs.data_ptr())
    status = _lib.status_word(dev)
    status.zero_()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    rc = lib.ss_peer_barrier_timed(ptrs, 0, 2, 1, 50_000, status.data_ptr(), _lib.stream_ptr())
    stop.record()
    assert rc == 0
    torch.cuda.synchronize()                                   # the kernel ended by itself
    assert start.elapsed_time(stop) < 100.0                    # far below the 2 s default
    assert int(theirs[0]) == 1                                 # this rank did signal its peer
    assert int(status.item()) == 5                             # KS_TIMEOUT_PEER
    with pytest.raises(RuntimeError, match="peer flag"):
        _lib.check_status(dev)                                 # the host learns of it and clears it
    assert int(status.item()) == 0
    # the context is intact: a barrier whose peer word is already set passes cleanly
    mine[1] = 2
    rc = lib.ss_peer_barrier_timed(ptrs, 0, 2, 2, 50_000, status.data_ptr(), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
