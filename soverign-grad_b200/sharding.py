"""Column (N) sharding of a quantized linear across the GPUs of one box.

The reference has no distributed code at all (its nn::DataParallel, include/sovereigngrad/nn.hpp:
1006-1053, is an OpenMP loop on one device).  Here every rank owns a contiguous slice of output
features — rows [n0, n1) of a weight stored [N, K] — with its packed codes, scales and bias slice,
sees the whole activation, computes y[:, n0:n1] with the same kernels as the single-GPU path and
the slices are exchanged with ONE collective, an all-gather over NVLink.  Because each output
element is produced by exactly one rank running the same instructions, the gathered result equals
the single-GPU result.

Slices are multiples of 32 rows so that an INT4 group (32 consecutive k of one row) never crosses
a rank.  INT8 per-tensor weights carry ONE scale for the whole tensor: quantize before slicing
(`slice_quantized`) so that every rank uses the identical scale.

torch.distributed is plumbing here (process group, NCCL all-gather); the compute is the C ABI.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int, multiple: int = 32) -> tuple[int, int]:
    """Rows [n0, n1) of rank `rank`: equal slices when n divides evenly, else the first ranks get one
    more block of `multiple` rows.  Every slice except possibly the last is a multiple of `multiple`."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    blocks = (n + multiple - 1) // multiple
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * multiple, n), min(b1 * multiple, n)


def slice_quantized(q, n0: int, n1: int):
    """Rows [n0, n1) of an already quantized [N, K] weight (same scales -> same bytes as one GPU)."""
    from . import PER_TENSOR, QuantizedTensor  # late import: this module is also used by CPU-only tests
    N, K = q.original_shape
    if q.bits == 4:
        if (n0 * K) % (2 * q.group_size) or (K % q.group_size):
            raise ValueError("INT4 slices must start on a group boundary")
        qdata = q.qdata[n0 * K // 2: n1 * K // 2]
        scales = q.scales[n0 * K // q.group_size: n1 * K // q.group_size]
    else:
        qdata = q.qdata[n0:n1]
        per_tensor = q.scheme == PER_TENSOR or q.scales.numel() == 1
        scales = q.scales if per_tensor else q.scales[n0:n1]
    return QuantizedTensor(qdata.contiguous(), scales.contiguous(), q.scheme, (n1 - n0, K), q.group_size, q.bits)


class ShardedLinear:
    """y[M, N] = x[M, K] * W^T + b with W[N, K] split by rows over the ranks of `group`.

    local_forward(x, out) computes this rank's [M, n_local] slice into `out`;
    interleave(gathered, M, n_local) turns the all-gather order [world][M][n_local] into row-major
    [M, world * n_local].  Both default to the CUDA kernels; CPU tests inject stand-ins.
    Slices must have equal width (all-gather of equal pieces): N % (32 * world) == 0.
    """

    def __init__(self, n_total: int, local_forward: Callable, interleave: Optional[Callable] = None,
                 group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_total = n_total
        self.n0, self.n1 = shard_bounds(n_total, self.world, self.rank)
        widths = {shard_bounds(n_total, self.world, r)[1] - shard_bounds(n_total, self.world, r)[0] for r in range(self.world)}
        if len(widths) != 1:
            raise ValueError(f"N={n_total} does not split into {self.world} equal slices of 32-row blocks")
        self.n_local = self.n1 - self.n0
        self.local_forward = local_forward
        self.interleave = interleave
        self._bufs = {}

    def _buffers(self, M: int, device):
        key = (M, str(device))
        if key not in self._bufs:
            self._bufs[key] = (torch.empty(M, self.n_local, dtype=torch.float32, device=device),
                               torch.empty(self.world, M, self.n_local, dtype=torch.float32, device=device),
                               torch.empty(M, self.n_total, dtype=torch.float32, device=device))
        return self._bufs[key]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        M = x.shape[0]
        y_local, gathered, y = self._buffers(M, x.device)
        self.local_forward(x, y_local)
        if self.world == 1:
            return y_local
        dist.all_gather_into_tensor(gathered.view(self.world * M, self.n_local), y_local, group=self.group)
        if self.interleave is not None:
            return self.interleave(gathered, M, self.n_local, y)
        from . import interleave_slices
        return interleave_slices(gathered, self.world, M, self.n_local, y)

    __call__ = forward


class PeerExchange:
    """Symmetric memory for the fused all-gather: `n_buffers` full-width outputs [M, n_total] per
    rank that every rank can store into, plus the barrier's signal slots.  torch's symmetric-memory
    allocator does the mapping (plumbing); the stores and the barrier are this library's kernels."""

    def __init__(self, M: int, n_total: int, device, group=None, n_buffers: int = 2):
        import ctypes as C
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # plain peer stores only: no multicast object is bound
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.M, self.n_total, self.n_buffers = M, n_total, n_buffers
        per = ((M * n_total + 63) // 64) * 64
        self._out = symm.empty(n_buffers * per, dtype=torch.float32, device=device)
        self._sig = symm.empty(64, dtype=torch.int64, device=device)
        self._out.zero_()
        self._sig.zero_()
        h_out = symm.rendezvous(self._out, self.group)
        h_sig = symm.rendezvous(self._sig, self.group)
        torch.cuda.synchronize()
        dist.barrier(self.group)                       # every rank's signals are zero before anyone signals
        self.local = [self._out[i * per: i * per + M * n_total].view(M, n_total) for i in range(n_buffers)]
        out_ptrs = [int(p) for p in h_out.buffer_ptrs]
        self._y_ranks = [(C.c_void_p * self.world)(*[p + i * per * 4 for p in out_ptrs]) for i in range(n_buffers)]
        self._signals = (C.c_void_p * self.world)(*[int(p) for p in h_sig.buffer_ptrs])
        self._epoch = torch.zeros(2, dtype=torch.int64, device=device)       # {epoch, finished-CTA counter} of the barrier
        self._handles = (h_out, h_sig)
        self.turn = 0

    def next_buffer(self) -> int:
        i = self.turn
        self.turn = (self.turn + 1) % self.n_buffers
        return i

    def y_ranks(self, i: int):
        return self._y_ranks[i]

    def barrier(self):
        from . import _ptr, _stream, check, lib
        check(lib.sgq_peer_barrier(self._signals, self.rank, self.world, _ptr(self._epoch), _stream()), "sgq_peer_barrier")


class PeerShardedLinear:
    """Column-sharded forward with the all-gather fused into the kernel's epilogue: every rank's kernel (the
    decode kernel up to 16 rows, the tcgen05 GEMM from 64 rows on) stores its [M, n_local] slice into all
    ranks' [M, n_total] outputs; the barrier between the ranks runs in the decode kernel's own tail
    (fused_barrier) or as a second small kernel.  No collective library on the data path."""

    def __init__(self, q_local, bias_local, n_total: int, exchange: PeerExchange, fused_barrier: bool = True,
                 deferred: bool = False):
        from . import Workspace
        # deferred: the kernel only signals at its end and the NEXT forward on this exchange waits in its prologue
        # (sgq_linear_int4_allgather_deferred); the caller ends a sequence with exchange.barrier()
        self.fused_barrier, self.deferred = fused_barrier or deferred, deferred
        self.q, self.bias, self.n_total, self.ex = q_local, bias_local, n_total, exchange
        self.n_local = q_local.original_shape[0]
        self.n0, self.n1 = shard_bounds(n_total, exchange.world, exchange.rank)
        if self.n1 - self.n0 != self.n_local:
            raise ValueError("local weight does not match this rank's slice")
        self.ws = Workspace(q_local.qdata.device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import LAYOUT_NK, PATH_AUTO, _ptr, _stream, check, lib, linear_workspace_bytes
        M, K = x.shape
        i = self.ex.next_buffer()
        # decode batches: the decode kernel's planes; from 64 rows on the tensor-core GEMM's operands (its epilogue
        # stores the tiles into every rank's output, the barrier kernel follows it)
        need = linear_workspace_bytes(4, M, K, self.n_local, LAYOUT_NK, PATH_AUTO)
        ws = self.ws.get(need) if need else None
        fn = lib.sgq_linear_int4_allgather_deferred if self.deferred else lib.sgq_linear_int4_allgather
        check(fn(_ptr(x), M, K, self.n_local, _ptr(self.q.qdata), _ptr(self.q.scales), _ptr(self.bias),
                 self.ex.y_ranks(i), self.ex.world, self.n_total, self.n0,
                 _ptr(ws) if ws is not None else None, ws.numel() if ws is not None else 0,
                 self.ex._signals if self.fused_barrier else None, self.ex.rank, _ptr(self.ex._epoch), _stream()),
              "sgq_linear_int4_allgather")
        if not self.fused_barrier:
            self.ex.barrier()
        return self.ex.local[i]

    __call__ = forward


def cuda_sharded_linear(q_local, bias_local, n_total: int, path: int = 0, group=None) -> ShardedLinear:
    """The product path: the local slice runs through sgq_linear_* on this rank's GPU."""
    from . import LAYOUT_NK, Workspace, quantized_matmul
    ws = Workspace(q_local.qdata.device)

    def local_forward(x, out):
        quantized_matmul(x, q_local, bias_local, layout=LAYOUT_NK, path=path, out=out, workspace=ws)

    return ShardedLinear(n_total, local_forward, None, group)
