"""Failure detection without a faulting GPU: a device-side wait for another rank is made to run out.

The barrier between GPUs polls signal slots that the other ranks write.  Here a two-rank barrier is
launched on ONE GPU with a second rank that does not exist: its slot is ordinary local memory that
nobody ever writes.  With a poll budget of about a millisecond the kernel must give up and return,
the status word must report the timeout (and clear), and the library must keep working."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sgq():
    from __graft_entry__ import load_package
    return load_package()


def test_peer_wait_runs_out_and_is_reported(sgq):
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    sig = torch.zeros(2, 8, dtype=torch.int64, device="cuda")          # the signal arrays of "rank 0" and of a rank that never runs
    epoch = torch.zeros(2, dtype=torch.int64, device="cuda")
    signals = (C.c_void_p * 2)(sig[0].data_ptr(), sig[1].data_ptr())
    assert sgq.device_status() == 0
    prev = sgq.lib.sgq_set_peer_wait_budget(4096)                       # about a millisecond of polling
    try:
        sgq.check(sgq.lib.sgq_peer_barrier(signals, 0, 2, epoch.data_ptr(), stream))
        torch.cuda.synchronize()                                       # the kernel returned by itself
    finally:
        sgq.lib.sgq_set_peer_wait_budget(prev)
    word = C.c_uint(0)
    assert sgq.lib.sgq_device_status(C.byref(word), 1) == 9            # SGQ_ERR_TIMEOUT, read and cleared
    assert word.value >> 24 == 5                                       # a wait for a peer
    assert b"status word" in sgq.lib.sgq_last_error()
    assert sgq.device_status() == 0                                    # cleared
    assert int(epoch[0]) == 1 and int(sig[0, 0]) == 1 and int(sig[1, 0]) == 1     # this rank did publish its epoch
    # the context is intact: an ordinary forward afterwards is correct
    g = torch.Generator(device="cuda").manual_seed(0)
    w = torch.randn(64, 512, device="cuda", generator=g) * 0.02
    x = torch.randn(2, 512, device="cuda", generator=g)
    q = sgq.quantize_int4(w, 32)
    y = sgq.quantized_matmul(x, q, None, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV)
    y_ref = sgq.quantized_matmul(x, q, None, layout=sgq.LAYOUT_NK, path=sgq.PATH_SIMT)
    assert float((y - y_ref).abs().max() / y_ref.abs().max()) <= 1e-3
    assert sgq.device_status() == 0


def test_deferred_exchange_wait_runs_out_and_is_reported(sgq):
    """The same for the wait in the prologue of the deferred fused all-gather: rank 0 of a two-rank exchange
    whose peer never signals.  The first forward has nothing to wait for; the second waits for the peer's
    signal of the first, gives up, reports, and still stores its own (incomplete) result."""
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    M, K, N = 1, 512, 64
    g = torch.Generator(device="cuda").manual_seed(1)
    q = sgq.quantize_int4(torch.randn(N, K, device="cuda", generator=g) * 0.02, 32)
    x = torch.randn(M, K, device="cuda", generator=g)
    y = torch.zeros(2, M, 2 * N, device="cuda")                          # two "ranks'" full-width outputs, both local
    sig = torch.zeros(2, 8, dtype=torch.int64, device="cuda")
    state = torch.zeros(2, dtype=torch.int64, device="cuda")
    y_ranks = (C.c_void_p * 2)(y[0].data_ptr(), y[1].data_ptr())
    signals = (C.c_void_p * 2)(sig[0].data_ptr(), sig[1].data_ptr())
    call = lambda: sgq.lib.sgq_linear_int4_allgather_deferred(x.data_ptr(), M, K, N, q.qdata.data_ptr(), q.scales.data_ptr(), None,  # noqa: E731
                                                             y_ranks, 2, 2 * N, 0, None, 0, signals, 0, state.data_ptr(), stream)
    prev = sgq.lib.sgq_set_peer_wait_budget(4096)
    try:
        sgq.check(call())
        torch.cuda.synchronize()
        assert sgq.device_status() == 0                                  # nothing to wait for yet
        sgq.check(call())
        torch.cuda.synchronize()
    finally:
        sgq.lib.sgq_set_peer_wait_budget(prev)
    word = C.c_uint(0)
    assert sgq.lib.sgq_device_status(C.byref(word), 1) == 9
    assert word.value >> 24 == 5
    want = sgq.quantized_matmul(x, q, None, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV)
    assert torch.equal(y[0, :, :N], want) and torch.equal(y[1, :, :N], want)      # both copies of this rank's slice
    # the signals count arrivals of CTAs: two launches of N / 16 = 4 CTAs each, sent to both slots of this rank
    assert int(state[0]) == 2 * (N // 16) and int(sig[0, 0]) == 2 * (N // 16) and int(sig[0, 1]) == 0
