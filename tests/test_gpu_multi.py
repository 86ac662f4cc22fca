"""Column-sharded forward on 2 GPUs over NCCL: gathered result == single-GPU result, bit for bit."""
import os
import socket
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, out_dir):
    import importlib
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from __graft_entry__ import load_package
    sgq = load_package()
    sh = importlib.import_module("sgq_b200.sharding")
    g = torch.Generator(device="cuda").manual_seed(7)          # same seed on every rank: same tensors
    for (M, K, N, path) in [(1, 1024, 512, sgq.PATH_GEMV), (4, 2048, 1024, sgq.PATH_GEMV), (16, 1024, 256, sgq.PATH_AUTO),
                            (130, 512, 512, sgq.PATH_SIMT)]:
        x = torch.randn(M, K, device="cuda", generator=g)
        w = torch.randn(N, K, device="cuda", generator=g) * 0.02
        b = torch.randn(N, device="cuda", generator=g)
        q_full = sgq.quantize_int4(w, 32)
        want = sgq.quantized_matmul(x, q_full, b, layout=sgq.LAYOUT_NK, path=path)
        n0, n1 = sh.shard_bounds(N, world, rank)
        q_local = sgq.quantize_int4(w[n0:n1].contiguous(), 32)
        sliced = sh.slice_quantized(q_full, n0, n1)
        assert torch.equal(q_local.qdata, sliced.qdata) and torch.equal(q_local.scales, sliced.scales)
        lin = sh.cuda_sharded_linear(q_local, b[n0:n1].contiguous(), N, path=path)
        y = lin(x)
        assert torch.equal(y, want), (M, K, N)
        # INT8 per tensor: one global scale -> quantize, then slice
        q8 = sgq.quantize_int8(w, sgq.PER_TENSOR)
        want8 = sgq.quantized_matmul(x, q8, b, layout=sgq.LAYOUT_NK, path=sgq.PATH_SIMT)
        lin8 = sh.cuda_sharded_linear(sh.slice_quantized(q8, n0, n1), b[n0:n1].contiguous(), N, path=sgq.PATH_SIMT)
        assert torch.equal(lin8(x), want8)
    # fused all-gather: peer stores from the decode kernel + the barrier kernel, no NCCL on the data path
    # (16 rows at K = 8192: the planes do not fit in shared memory, so two blocks of 8 rows converted by a kernel in front)
    for (M, K, N) in [(1, 1024, 512), (8, 2048, 1024), (16, 1024, 256), (16, 8192, 512)]:
        x = torch.randn(M, K, device="cuda", generator=g)
        w = torch.randn(N, K, device="cuda", generator=g) * 0.02
        b = torch.randn(N, device="cuda", generator=g)
        q_full = sgq.quantize_int4(w, 32)
        n0, n1 = sh.shard_bounds(N, world, rank)
        ex = sh.PeerExchange(M, N, torch.device("cuda", rank))
        for fused in (True, False):                              # barrier in the kernel's tail / as its own kernel
            lin = sh.PeerShardedLinear(sh.slice_quantized(q_full, n0, n1), b[n0:n1].contiguous(), N, ex, fused_barrier=fused)
            for rep in range(5):                                 # alternates between the two output sets
                xr = x * (rep + 1)
                want = sgq.quantized_matmul(xr, q_full, b, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV)
                y = lin(xr)
                torch.cuda.synchronize()
                assert torch.equal(y, want), ("peer", M, K, N, rep, fused)
        # deferred form: a forward only signals, the next one waits in its prologue; a barrier ends the sequence
        lin = sh.PeerShardedLinear(sh.slice_quantized(q_full, n0, n1), b[n0:n1].contiguous(), N, ex, deferred=True)
        ys, wants = [], []
        for rep in range(6):
            xr = x * (rep + 1)
            wants.append(sgq.quantized_matmul(xr, q_full, b, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV))
            ys.append(lin(xr))           # a buffer is whole only after a later forward's wait or the barrier below
        ex.barrier()
        torch.cuda.synchronize()
        assert torch.equal(ys[5], wants[5]), ("deferred, last", M, K, N)
        assert torch.equal(ex.local[(ex.turn + 0) % 2], wants[4]), ("deferred, one before last", M, K, N)
    # prefill-sized batches: the tcgen05 GEMM's epilogue stores its tiles into every rank's output, a barrier kernel
    # follows; every output element is accumulated in the same order as on one GPU, so the bits agree
    for (M, K, N) in [(128, 512, 512), (300, 1024, 1536)]:
        x = torch.randn(M, K, device="cuda", generator=g)
        w = torch.randn(N, K, device="cuda", generator=g) * 0.02
        b = torch.randn(N, device="cuda", generator=g)
        q_full = sgq.quantize_int4(w, 32)
        n0, n1 = sh.shard_bounds(N, world, rank)
        ex = sh.PeerExchange(M, N, torch.device("cuda", rank), n_buffers=1)
        lin = sh.PeerShardedLinear(sh.slice_quantized(q_full, n0, n1), b[n0:n1].contiguous(), N, ex)
        for overlap in (0, 1):
            prev = sgq.set_stream_overlap(overlap)
            try:
                for rep in range(3):
                    xr = x * (rep + 1)
                    want = sgq.quantized_matmul(xr, q_full, b, layout=sgq.LAYOUT_NK, path=sgq.PATH_TC_BF16)
                    y = lin(xr)
                    torch.cuda.synchronize()
                    assert torch.equal(y, want), ("tensor-core peer stores", M, K, N, rep, overlap)
                    dist.barrier()
            finally:
                sgq.set_stream_overlap(prev)
    # the sharded decoder (heads, SwiGLU columns, wo / w_down outputs and the vocabulary split by column) against
    # the same model on one GPU: every output element is computed by the same instructions, so logits are equal
    nl = importlib.import_module("sgq_b200.nanollama")
    cfg = nl.NanoLlamaConfig(dim=256, n_layers=2, n_heads=2, hidden=512, vocab=512, max_seq=64)
    prompt = torch.randint(0, cfg.vocab, (2, 9), generator=torch.Generator().manual_seed(3))
    single = nl.NanoLlamaInt4(cfg, "cuda", 2, seed=11)
    tok1, log1 = single.generate(prompt, 6, use_graph=False, keep_logits=True)
    for exchange in ("peer", "nccl"):
        sharded = nl.NanoLlamaInt4(cfg, "cuda", 2, seed=11, rank=rank, world=world, exchange=exchange)
        tok2, log2 = sharded.generate(prompt, 6, use_graph=False, keep_logits=True)
        assert torch.equal(tok2, tok1), exchange
        for a, b2 in zip(log1, log2):
            assert torch.equal(a, b2), exchange
        if exchange == "peer":                       # the sharded decode step as one CUDA graph
            tok3 = sharded.generate(prompt, 6, use_graph=True)
            assert torch.equal(tok3, tok1)
            tok4 = sharded.generate(prompt, 6, use_graph=True)
            assert torch.equal(tok4, tok1)
        torch.cuda.synchronize()
        dist.barrier()
    # a prompt of 64 rows or more: the tensor-core GEMMs of the sharded model store into every rank's buffers
    long_prompt = torch.randint(0, cfg.vocab, (2, 40), generator=torch.Generator().manual_seed(5))
    single = nl.NanoLlamaInt4(cfg, "cuda", 2, seed=11)
    tok1, log1 = single.generate(long_prompt, 4, use_graph=False, keep_logits=True)
    sharded = nl.NanoLlamaInt4(cfg, "cuda", 2, seed=11, rank=rank, world=world, exchange="peer")
    tok2, log2 = sharded.generate(long_prompt, 4, use_graph=False, keep_logits=True)
    assert sharded._prompt_sites, "the prompt pass did not take the peer exchange"
    assert torch.equal(tok2, tok1)
    for a, b2 in zip(log1, log2):
        assert torch.equal(a, b2)
    torch.cuda.synchronize()
    dist.barrier()
    assert sgq.device_status() == 0
    dist.barrier()
    if rank == 0:
        open(os.path.join(out_dir, "ok"), "w").write("ok")
    dist.destroy_process_group()


def test_sharded_forward_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    mp.spawn(worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").read_text() == "ok"
