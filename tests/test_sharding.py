"""Host-side logic of the column-sharded linear on CPU ranks (gloo, world_size 2 and 4): slice
bounds, all-gather assembly, per-tensor scale sharing.  The local compute is the oracle here; the
GPU tests cover the kernels, and test_gpu_linear.py::test_column_slices_reassemble covers
slice-writing on one device."""
import importlib.util
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from __graft_entry__ import PKG_DIR, ROOT


def load_sharding():
    spec = importlib.util.spec_from_file_location("sgq_sharding_cpu", os.path.join(PKG_DIR, "sharding.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_shard_bounds():
    sh = load_sharding()
    for n, world in [(11008, 8), (28672, 8), (2048, 8), (5632, 8), (32000, 8), (11008, 2), (96, 4), (100, 3)]:
        edges = [sh.shard_bounds(n, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
            assert a1 == b0 and a0 % 32 == 0 and b0 % 32 == 0
    assert sh.shard_bounds(11008, 8, 3) == (4128, 5504)       # 11008 / 8 = 1376 = 43 * 32
    assert sh.shard_bounds(100, 3, 2) == (96, 100)            # ragged tail goes to the last rank
    with pytest.raises(ValueError):
        sh.shard_bounds(64, 2, 2)


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, M, K, N, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import oracle
    import cases
    sh = load_sharding()
    port_oracle = oracle.Port()
    x = cases.normal(1, (M, K))
    w = cases.weight_with_outliers(2, (N, K))
    b = cases.normal(3, (N,), 0.1)
    n0, n1 = sh.shard_bounds(N, world, rank)
    # INT4: quantize the local rows only — groups never cross a slice
    packed, scales = port_oracle.quantize_int4(w[n0:n1], 32)
    full_packed, full_scales = port_oracle.quantize_int4(w, 32)
    assert np.array_equal(packed, full_packed[n0 * K // 2: n1 * K // 2])
    assert scales.tobytes() == full_scales[n0 * K // 32: n1 * K // 32].tobytes()

    def local_forward(xt, out):
        y = port_oracle.qlinear_int4(xt.numpy(), packed, scales, K, n1 - n0, oracle.LAYOUT_NK, 32, b[n0:n1])
        out.copy_(torch.from_numpy(y))

    def interleave(gathered, M_, n_local, y):
        y.copy_(gathered.permute(1, 0, 2).reshape(M_, -1))
        return y

    lin = sh.ShardedLinear(N, local_forward, interleave)
    y = lin(torch.from_numpy(x)).numpy()
    want = port_oracle.qlinear_int4(x, full_packed, full_scales, K, N, oracle.LAYOUT_NK, 32, b)
    assert np.array_equal(y, want), "sharded result must equal the single-device result bit for bit"

    # INT8 per tensor: the absmax is global.  Local quantization would pick a different scale...
    codes_local, scale_local = port_oracle.quantize_int8(w[n0:n1], oracle.PER_TENSOR)
    codes_full, scale_full = port_oracle.quantize_int8(w, oracle.PER_TENSOR)
    local_max = torch.tensor([float(np.abs(w[n0:n1]).max())])
    dist.all_reduce(local_max, op=dist.ReduceOp.MAX)
    assert np.float32(local_max.item()) / np.float32(127.0) == scale_full[0]      # ...the all-reduced absmax gives it back
    # ...so the weight is quantized before slicing: every rank holds the same scale and its rows
    y8 = port_oracle.qlinear_int8(x, codes_full[n0:n1], scale_full, K, n1 - n0, oracle.LAYOUT_NK, oracle.PER_TENSOR, b[n0:n1])
    gathered = [torch.empty(M, n1 - n0) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(y8))
    want8 = port_oracle.qlinear_int8(x, codes_full, scale_full, K, N, oracle.LAYOUT_NK, oracle.PER_TENSOR, b)
    assert np.array_equal(torch.cat(gathered, dim=1).numpy(), want8)
    if rank == 0:
        open(os.path.join(out_dir, "ok"), "w").write("ok")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,N", [(2, 128), (4, 256)])
def test_sharded_linear_gloo(tmp_path, world, N):
    mp.spawn(worker, args=(world, free_port(), 3, 96, N, str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "ok").read_text() == "ok"


def test_unequal_slices_are_rejected():
    sh = load_sharding()

    class FakeDist:
        pass
    lin = sh.ShardedLinear(96, lambda x, out: None)       # world 1: always fine
    assert (lin.n0, lin.n1) == (0, 96)
