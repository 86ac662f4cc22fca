"""The allocation-free decode entry point, sgq_linear_int4_decode_noalloc.

It serves callers that cannot get device memory at call time (a plugin inside a host that owns
every allocation, a process with a frozen pool, a token loop that must not touch the allocator),
so its scratch is a fixed array inside the library.  The test calls it through the C ABI only,
with buffers made beforehand, twice in a row, and compares with the regular entry point that takes
a caller workspace.  The file sorts last so that a run stopping at the first failure has already
run everything else; it also passes on its own in a fresh process.
"""
import ctypes as C

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sgq():
    from __graft_entry__ import load_package
    return load_package()


@pytest.mark.parametrize("M,K,N", [(8, 4096, 1024), (16, 2048, 272), (1, 1024, 64)])
def test_noalloc_matches_workspace_entry_point(sgq, M, K, N):
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    b = torch.randn(N, device="cuda", generator=g)
    q = sgq.quantize_int4(w, 32)
    xs = [torch.randn(M, K, device="cuda", generator=g) for _ in range(2)]
    need = sgq.linear_workspace_bytes(4, M, K, N, sgq.LAYOUT_NK, sgq.PATH_GEMV)
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
    want = [torch.empty(M, N, device="cuda") for _ in range(2)]
    got = [torch.full((M, N), float("nan"), device="cuda") for _ in range(2)]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for i in range(2):   # the regular entry point, caller workspace
        sgq.check(sgq.lib.sgq_linear_int4(xs[i].data_ptr(), M, K, N, q.qdata.data_ptr(), q.scales.data_ptr(), sgq.LAYOUT_NK, 32,
                                          b.data_ptr(), want[i].data_ptr(), N, sgq.PATH_GEMV, ws.data_ptr() if need else None,
                                          ws.numel() if need else 0, stream))
    # one warm-up call: the first call on a device looks up the scratch array's address and loads the kernel
    sgq.check(sgq.lib.sgq_linear_int4_decode_noalloc(xs[0].data_ptr(), M, K, N, q.qdata.data_ptr(), q.scales.data_ptr(),
                                                     b.data_ptr(), got[0].data_ptr(), N, stream))
    torch.cuda.synchronize()
    got[0].fill_(float("nan"))
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]        # the driver's own count: also sees a cudaMalloc made by the library
    for i in range(2):   # two calls in a row share the built-in scratch; the second must not see the first's leftovers
        sgq.check(sgq.lib.sgq_linear_int4_decode_noalloc(xs[i].data_ptr(), M, K, N, q.qdata.data_ptr(), q.scales.data_ptr(),
                                                         b.data_ptr(), got[i].data_ptr(), N, stream))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated during the calls"
    assert sgq.device_status() == 0
    for i in range(2):
        # same kernels, same order of operations: within the 1e-3 bound of the fp32 paths (in fact equal)
        err = ((got[i] - want[i]).abs() / want[i].abs().clamp_min(want[i].pow(2).mean().sqrt())).max().item()
        assert err <= 1e-3, err
        assert torch.equal(got[i], want[i])


def test_noalloc_rejects_what_exceeds_the_builtin_scratch(sgq):
    M, K, N = 16, 16384, 32                      # needs 16384/32 * (6 * 288 + 16) bytes > 448 KiB
    one = torch.zeros(M * K, device="cuda")
    rc = sgq.lib.sgq_linear_int4_decode_noalloc(one.data_ptr(), M, K, N, one.data_ptr(), one.data_ptr(), None, one.data_ptr(), N, None)
    assert rc == 5                               # SGQ_ERR_WORKSPACE: too large for the built-in scratch
    assert sgq.lib.sgq_linear_int4_decode_noalloc(None, 1, 256, 16, None, None, None, None, 16, None) == 1   # null pointers
    assert sgq.lib.sgq_linear_int4_decode_noalloc(None, 0, 256, 16, None, None, None, None, 16, None) == 0   # empty batch
