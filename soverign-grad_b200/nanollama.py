"""NanoLLaMA-INT4: greedy decoding of a LLaMA-style decoder whose every Linear is an INT4 (group 32)
QuantizedLinear4Bit served by the C ABI.

The reference's NanoLLaMA (include/sovereigngrad/models.hpp:193-305) is a toy: no batch, no heads,
no rotary call, no KV cache, and generate() re-runs the whole context for each new token
(models.hpp:262-300).  The model here is the benchmarked configuration — dim 2048, 16 blocks,
16 heads of 128, SwiGLU hidden 5632, RMSNorm (eps 1e-5), RoPE base 1e4, vocab 32000 — assembled from
the reference's operators: nn::RMSNorm (nn.hpp:67-85), nn::RotaryEmbedding (nn.hpp:583-612),
nn::CausalSelfAttention (nn.hpp:503-560), nn::SwiGLU (nn.hpp:138-160), nn::Embedding (nn.hpp:390-410)
and greedy selection (models.hpp:286-298: first index of the strict maximum).

What runs where: every Linear goes through sgq_linear_int4 (decode kernel for the M = batch steps,
tcgen05 kernel for the prefill); RMSNorm, RoPE + KV-cache store, cache attention and the SiLU gate
the prompt's causal attention, the embedding lookup and the greedy argmax are the sgqd_* kernels of
include/sgq_decoder.h; torch supplies device memory only.  A decode step touches no host state — the
cache position lives in device memory — so one step is recorded into a CUDA graph and replayed.

Sharding (world > 1): heads, SwiGLU columns, output features of wo / w_down and the vocabulary are
split by column over the ranks; each split output is all-gathered over NCCL and re-interleaved
(`sharding.ShardedLinear` has the single-layer version of the same scheme).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

import contextlib
import ctypes as C

from . import (LAYOUT_NK, PATH_AUTO, PATH_GEMV, PATH_TC_BF16, QuantizedTensor, Workspace, _ptr, _stream, check, interleave_slices, lib,
               linear_int4_prepared, prepared_x_bytes, quantize_int4, quantized_matmul, set_stream_overlap)


@dataclass
class NanoLlamaConfig:
    dim: int = 2048
    n_layers: int = 16
    n_heads: int = 16
    hidden: int = 5632
    vocab: int = 32000
    max_seq: int = 640
    rope_base: float = 10000.0
    eps: float = 1e-5
    group: int = 32

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads


LAYER_WEIGHTS = ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")


def weight_shape(cfg: NanoLlamaConfig, name: str) -> tuple[int, int]:
    """[out, in] of a float weight; `embed` and `lm_head` are [vocab, dim]."""
    if name in ("wq", "wk", "wv", "wo"):
        return cfg.dim, cfg.dim
    if name in ("w_gate", "w_up"):
        return cfg.hidden, cfg.dim
    if name == "w_down":
        return cfg.dim, cfg.hidden
    if name in ("embed", "lm_head"):
        return cfg.vocab, cfg.dim
    raise KeyError(name)


def default_init(cfg: NanoLlamaConfig, device, seed: int) -> Callable[[str, int], torch.Tensor]:
    """Random weights with the reference's initialisers: nn::Linear N(0, sqrt(2 / (in + out)))
    (nn.hpp:23-26), nn::Embedding N(0, sqrt(1 / dim)) (nn.hpp:396-400)."""
    gen = torch.Generator(device=device).manual_seed(seed)

    def make(name: str, layer: int) -> torch.Tensor:
        out_f, in_f = weight_shape(cfg, name)
        std = (1.0 / cfg.dim) ** 0.5 if name == "embed" else (2.0 / (in_f + out_f)) ** 0.5
        return torch.randn(out_f, in_f, device=device, generator=gen) * std
    return make


def rope_tables(cfg: NanoLlamaConfig, device):
    """nn::RotaryEmbedding (nn.hpp:583-607): float32 inv_freq and theta, tables [max_seq, head_dim/2]."""
    half = cfg.head_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(cfg.rope_base, dtype=torch.float32), (2.0 * i) / float(cfg.head_dim))
    theta = torch.arange(cfg.max_seq, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(theta.double()).float().to(device).contiguous(), torch.sin(theta.double()).float().to(device).contiguous()


def _rows(w: torch.Tensor, r0: int, r1: int) -> torch.Tensor:
    return w[r0:r1]


class _Linear:
    """One column slice of an INT4 linear: rows [n0, n1) of the [N, K] weight on this rank."""

    def __init__(self, w_local: torch.Tensor, group: int, ws: Workspace):
        self.q: QuantizedTensor = quantize_int4(w_local.contiguous(), group)
        self.n_local, self.k = w_local.shape
        self.ws = ws

    def __call__(self, x: torch.Tensor, out: torch.Tensor, path: int) -> torch.Tensor:
        return quantized_matmul(x, self.q, None, layout=LAYOUT_NK, path=path, out=out, workspace=self.ws)

    def prepared(self, planes: torch.Tensor, M: int, out: torch.Tensor) -> torch.Tensor:
        return linear_int4_prepared(planes, M, self.q, None, out)


class _PeerSites:
    """Full-width symmetric buffers of one decode step (attention output, wo output, SiLU gate output,
    w_down output, logits) that every rank stores its column slice into, and one signal/epoch space for
    the barriers.  One buffer per site is enough: a rank can run at most one exchange ahead of another,
    and a site is reused only four exchanges later."""

    def __init__(self, cfg: NanoLlamaConfig, M: int, device, group, with_logits: bool = True):
        import ctypes as C
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        widths = {"attn": cfg.dim, "o": cfg.dim, "act": cfg.hidden, "d": cfg.dim}
        if with_logits:
            widths["logits"] = cfg.vocab
        offs, total = {}, 0
        for k, w in widths.items():
            offs[k] = total
            total += (M * w + 63) // 64 * 64
        self._buf = symm.empty(total, dtype=torch.float32, device=device)
        self._sig = symm.empty(64, dtype=torch.int64, device=device)
        self._buf.zero_()
        self._sig.zero_()
        h_buf, h_sig = symm.rendezvous(self._buf, self.group), symm.rendezvous(self._sig, self.group)
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self.local = {k: self._buf[offs[k]: offs[k] + M * w].view(M, w) for k, w in widths.items()}
        self.y_ranks = {k: (C.c_void_p * self.world)(*[int(p) + offs[k] * 4 for p in h_buf.buffer_ptrs]) for k in widths}
        self.width = widths
        self.signals = (C.c_void_p * self.world)(*[int(p) for p in h_sig.buffer_ptrs])
        self.state = torch.zeros(2, dtype=torch.int64, device=device)
        self._handles = (h_buf, h_sig)


class NanoLlamaInt4:
    def __init__(self, cfg: NanoLlamaConfig, device, batch: int, *, seed: int = 0,
                 init: Optional[Callable[[str, int], torch.Tensor]] = None, rank: int = 0, world: int = 1, group=None,
                 decode_path: int = PATH_AUTO, prefill_path: int = PATH_AUTO, overlap: int = 1,
                 exchange: str = "peer"):
        if cfg.n_heads % world or cfg.hidden % (32 * world) or cfg.dim % (32 * world) or cfg.vocab % (32 * world):
            raise ValueError("heads, hidden, dim and vocab must split into equal 32-row slices per rank")
        self.cfg, self.device, self.batch = cfg, torch.device(device), batch
        self.rank, self.world, self.group = rank, world, group
        self.decode_path, self.prefill_path = decode_path, prefill_path
        # consecutive kernels overlap (sgq_set_stream_overlap): legal here because no weight is ever
        # written by the kernel in front of the linear that reads it
        self.overlap = overlap
        # world > 1, decode steps: "peer" = slices stored into every rank's buffers by this library's kernels +
        # sgq_peer_barrier (graph-capturable); "nccl" = all-gather + interleave (eager).  A prompt pass of fewer
        # than 64 rows, or one held to the fp32 contract, uses NCCL in both cases.
        self.exchange = exchange if world > 1 else "none"
        self._sites = None
        self._prompt_sites = {}
        init = init or default_init(cfg, self.device, seed)
        dev = self.device
        self.ws = Workspace(dev)
        hd, H = cfg.head_dim, cfg.n_heads
        self.h_local = H // world
        self.dim_local = self.h_local * hd
        self.hid_local = cfg.hidden // world
        self.voc_local = cfg.vocab // world
        d0, d1 = rank * self.dim_local, (rank + 1) * self.dim_local
        f0, f1 = rank * self.hid_local, (rank + 1) * self.hid_local
        v0, v1 = rank * self.voc_local, (rank + 1) * self.voc_local

        self.embed = init("embed", -1).to(dev).float().contiguous()
        self.layers = []
        for li in range(cfg.n_layers):
            w = {n: init(n, li).to(dev).float() for n in LAYER_WEIGHTS}
            qkv = torch.cat([_rows(w["wq"], d0, d1), _rows(w["wk"], d0, d1), _rows(w["wv"], d0, d1)], 0)
            gu = torch.cat([_rows(w["w_gate"], f0, f1), _rows(w["w_up"], f0, f1)], 0)
            self.layers.append({
                "qkv": _Linear(qkv, cfg.group, self.ws), "wo": _Linear(_rows(w["wo"], d0, d1), cfg.group, self.ws),
                "gu": _Linear(gu, cfg.group, self.ws), "down": _Linear(_rows(w["w_down"], d0, d1), cfg.group, self.ws),
                "attn_norm": torch.ones(cfg.dim, device=dev), "ffn_norm": torch.ones(cfg.dim, device=dev)})
            del w, qkv, gu
        self.final_norm = torch.ones(cfg.dim, device=dev)
        self.lm_head = _Linear(_rows(init("lm_head", -1).to(dev).float(), v0, v1), cfg.group, self.ws)

        self.cos, self.sin = rope_tables(cfg, dev)
        shape = (cfg.n_layers, batch, self.h_local, cfg.max_seq, hd)
        self.k_cache = torch.zeros(shape, device=dev)
        self.v_cache = torch.zeros(shape, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self._bufs = {}
        self._graph = None
        self.tok = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.launches_per_decode_step = 0

    # ---- buffers -------------------------------------------------------------------------
    def _buffers(self, M: int):
        if M not in self._bufs:
            c, dev, W = self.cfg, self.device, self.world
            f = lambda *s: torch.empty(*s, device=dev)  # noqa: E731
            b = {"h": f(M, c.dim), "n": f(M, c.dim), "qkv": f(M, 3 * self.dim_local), "attn": f(M, self.dim_local),
                 "o": f(M, c.dim // W), "gu": f(M, 2 * self.hid_local), "act": f(M, self.hid_local), "d": f(M, c.dim // W)}
            use_prep = self.decode_path in (PATH_AUTO, PATH_GEMV)
            for key, width in (("p_dim", c.dim), ("p_hid", c.hidden)):
                nb = prepared_x_bytes(M, width) if use_prep else 0
                b[key] = torch.empty(nb, dtype=torch.uint8, device=dev) if nb else None
            if W > 1:
                b["p_hid"] = None          # the SiLU gate output is a column slice per rank: converted after the gather
                b.update({"g_attn": f(W, M, self.dim_local), "g_o": f(W, M, c.dim // W), "g_act": f(W, M, self.hid_local),
                          "attn_full": f(M, c.dim), "o_full": f(M, c.dim), "act_full": f(M, c.hidden), "d_full": f(M, c.dim)})
            self._bufs[M] = b
        return self._bufs[M]

    def _peer(self, M: int):
        """The symmetric buffers, if this pass exchanges through peer stores: the decode steps of a sharded model,
        and a prompt pass of 64 rows or more on the tensor-core path (the GEMM's epilogue stores into every rank's
        buffers).  The logits always belong to the decode-sized set."""
        if self.exchange != "peer":
            return None
        if M == self.batch:
            if self._sites is None:
                self._sites = _PeerSites(self.cfg, M, self.device, self.group)
            return self._sites
        if M < 64 or self.prefill_path not in (PATH_AUTO, PATH_TC_BF16) or self.cfg.dim % 64 or self.cfg.hidden % 64:
            return None
        if M not in self._prompt_sites:
            self._prompt_sites[M] = _PeerSites(self.cfg, M, self.device, self.group, with_logits=False)
        return self._prompt_sites[M]

    def _barrier(self, sites):
        check(lib.sgq_peer_barrier(sites.signals, self.rank, self.world, _ptr(sites.state), _stream()), "sgq_peer_barrier")
        self._count()

    def _gather(self, local: torch.Tensor, gathered: torch.Tensor, full: torch.Tensor, site: Optional[str] = None) -> torch.Tensor:
        """[M, n_local] slices of every rank -> row-major [M, world * n_local]; identity on one GPU."""
        if self.world == 1:
            return local
        sites = self._peer(local.shape[0]) if site else None
        if sites is not None:
            M, n_local = local.shape
            check(lib.sgq_peer_scatter(_ptr(local), M, n_local, sites.y_ranks[site], self.world, sites.width[site],
                                       self.rank * n_local, _stream()), "sgq_peer_scatter")
            self._count()
            self._barrier(sites)
            return sites.local[site]
        import torch.distributed as dist
        M, n_local = local.shape
        dist.all_gather_into_tensor(gathered.view(self.world * M, n_local), local, group=self.group)
        self._count(1)
        return interleave_slices(gathered, self.world, M, n_local, full)

    def _count(self, n: int = 1):
        self._launches += n

    # ---- the C-ABI operators ---------------------------------------------------------------
    def _add_rmsnorm(self, h, delta, gamma, out, planes=None):
        check(lib.sgqd_add_rmsnorm(_ptr(h), _ptr(delta), _ptr(gamma), self.cfg.eps, h.shape[0], h.shape[1], _ptr(out),
                                   _ptr(planes), planes.numel() if planes is not None else 0, _stream()), "sgqd_add_rmsnorm")
        self._count()

    def _linear_gathered(self, lin: _Linear, x, out, path, gathered, full, site: str):
        """A column-sharded linear whose full-width output every rank needs: on the peer exchange the decode
        kernel stores its slice into all ranks' buffers itself (fused all-gather), then the barrier."""
        sites = self._peer(x.shape[0]) if self.world > 1 else None
        if sites is None:
            self._linear(lin, x, out, path)
            return self._gather(out, gathered, full)
        M, K = x.shape
        need = int(lib.sgq_linear_workspace_bytes(4, M, K, lin.n_local, LAYOUT_NK, PATH_AUTO))
        ws = self.ws.get(need) if need else None
        check(lib.sgq_linear_int4_allgather(_ptr(x), M, K, lin.n_local, _ptr(lin.q.qdata), _ptr(lin.q.scales), None,
                                            sites.y_ranks[site], self.world, sites.width[site], self.rank * lin.n_local,
                                            _ptr(ws), ws.numel() if ws is not None else 0, None, self.rank, None, _stream()),
              "sgq_linear_int4_allgather")
        self._count(2 if (M > 16 or M * (K // 8) > 1024) else 1)
        self._barrier(sites)
        return sites.local[site]

    def _linear(self, lin: _Linear, x, out, path, planes=None):
        """planes: x already in the decode kernel's prepared form (written by the operator before)."""
        if planes is not None:
            lin.prepared(planes, x.shape[0], out)
            self._count()
            return
        lin(x, out, path)
        M, K = x.shape
        # the decode kernel converts activations inside its CTAs up to 1024 eight-value chunks; larger
        # batches and the tensor-core path run a conversion kernel first
        self._count(2 if (M > 16 or M * (K // 8) > 1024) else 1)

    # ---- one pass over t_new new tokens per sequence ---------------------------------------
    def _forward(self, tokens: torch.Tensor, t_new: int, path: int) -> torch.Tensor:
        """tokens [batch * t_new] (sequence-major).  Returns the final-normed hidden state [M, dim]."""
        c, B = self.cfg, self.batch
        M = B * t_new
        b = self._buffers(M)
        h, n = b["h"], b["n"]
        # nn::Embedding lookup; an id outside the vocabulary gives a row of zeros, as in the reference
        check(lib.sgqd_embedding(_ptr(self.embed), c.vocab, c.dim, _ptr(tokens), M, _ptr(h), _stream()), "sgqd_embedding")
        self._count()
        delta = None
        p_dim, p_hid = b["p_dim"], b["p_hid"]          # None for batches the decode kernel does not take
        if path not in (PATH_AUTO, PATH_GEMV):
            p_dim = p_hid = None
        for li, L in enumerate(self.layers):
            self._add_rmsnorm(h, delta, L["attn_norm"], n, p_dim)
            self._linear(L["qkv"], n, b["qkv"], path, p_dim)
            kc, vc = self.k_cache[li], self.v_cache[li]
            p_attn = None
            sites = self._peer(M) if self.world > 1 else None
            attn = None
            if t_new == 1 and sites is not None:
                # sharded: the kernel stores this rank's heads into every rank's full-width buffer itself
                check(lib.sgqd_attn_decode_allgather(_ptr(b["qkv"]), 3 * self.dim_local, B, self.h_local, c.head_dim, _ptr(self.cos),
                                                     _ptr(self.sin), _ptr(kc), _ptr(vc), c.max_seq, _ptr(self.pos),
                                                     sites.y_ranks["attn"], self.world, sites.width["attn"],
                                                     self.rank * self.dim_local, _stream()), "sgqd_attn_decode_allgather")
                self._count()
                self._barrier(sites)
                attn = sites.local["attn"]
            elif t_new == 1:     # rotary embedding, cache append and attention of the new token in one kernel
                # unsharded: the kernel also emits the prepared form of its output for the output projection
                # (the planes of the normed hidden state have been consumed by the q/k/v projection by then)
                p_attn = p_dim if self.world == 1 else None
                check(lib.sgqd_attn_decode(_ptr(b["qkv"]), 3 * self.dim_local, B, self.h_local, c.head_dim, _ptr(self.cos),
                                           _ptr(self.sin), _ptr(kc), _ptr(vc), c.max_seq, _ptr(self.pos), _ptr(b["attn"]),
                                           self.dim_local, _ptr(p_attn), p_attn.numel() if p_attn is not None else 0, _stream()),
                      "sgqd_attn_decode")
                self._count()
            else:
                check(lib.sgqd_rope_kv_store(_ptr(b["qkv"]), B, t_new, self.h_local, c.head_dim, _ptr(self.cos), _ptr(self.sin),
                                             _ptr(self.pos), _ptr(kc), _ptr(vc), c.max_seq, _stream()), "sgqd_rope_kv_store")
                self._count()
                self._prefill_attention(b["qkv"], kc, vc, t_new, b["attn"], bf16=path in (PATH_AUTO, PATH_TC_BF16) and M >= 64)
            if attn is None:
                attn = self._gather(b["attn"], b.get("g_attn"), b.get("attn_full"), "attn")
            if p_attn is not None:
                self._linear(L["wo"], attn, b["o"], path, p_attn)
                o = b["o"]
            else:
                o = self._linear_gathered(L["wo"], attn, b["o"], path, b.get("g_o"), b.get("o_full"), "o")
            self._add_rmsnorm(h, o, L["ffn_norm"], n, p_dim)
            self._linear(L["gu"], n, b["gu"], path, p_dim)
            if sites is not None:
                check(lib.sgqd_silu_mul_allgather(_ptr(b["gu"]), M, self.hid_local, sites.y_ranks["act"], self.world,
                                                  sites.width["act"], self.rank * self.hid_local, _stream()), "sgqd_silu_mul_allgather")
                self._count()
                self._barrier(sites)
                act = sites.local["act"]
            else:
                check(lib.sgqd_silu_mul(_ptr(b["gu"]), M, self.hid_local, _ptr(b["act"]), _ptr(p_hid),
                                        p_hid.numel() if p_hid is not None else 0, _stream()), "sgqd_silu_mul")
                self._count()
                act = self._gather(b["act"], b.get("g_act"), b.get("act_full"), "act")
            if self.world == 1:
                self._linear(L["down"], act, b["d"], path, p_hid)
                delta = b["d"]
            else:
                delta = self._linear_gathered(L["down"], act, b["d"], path, b.get("g_o"), b.get("d_full"), "d")
        self._add_rmsnorm(h, delta, self.final_norm, n, p_dim)
        self._final_planes = p_dim
        return n

    def _prefill_attention(self, qkv, kc, vc, T: int, out, bf16: bool = False):
        """Causal attention of the prompt: q from the rotated qkv rows, k and v from the cache rows just written.
        bf16: the pass runs its linears on the bf16 tensor cores (2e-2 contract), so the attention does too."""
        fn = lib.sgqd_attn_prefill_bf16 if (bf16 and self.cfg.head_dim == 128) else lib.sgqd_attn_prefill
        check(fn(_ptr(qkv), 3 * self.dim_local, self.batch, T, self.h_local, self.cfg.head_dim, _ptr(kc), _ptr(vc),
                 self.cfg.max_seq, _ptr(self.pos), _ptr(out), self.dim_local, _stream()), "sgqd_attn_prefill")
        self._count()

    def _logits(self, n_rows: torch.Tensor, path: int, planes=None) -> torch.Tensor:
        M = n_rows.shape[0]
        key = ("logits", M)
        if key not in self._bufs:
            f = lambda *s: torch.empty(*s, device=self.device)  # noqa: E731
            self._bufs[key] = (f(M, self.voc_local), f(self.world, M, self.voc_local) if self.world > 1 else None,
                               f(M, self.cfg.vocab) if self.world > 1 else None)
        loc, g, full = self._bufs[key]
        if self.world > 1:
            return self._linear_gathered(self.lm_head, n_rows, loc, path, g, full, "logits")
        self._linear(self.lm_head, n_rows, loc, path, planes)
        return loc

    @contextlib.contextmanager
    def _overlapped(self):
        prev = set_stream_overlap(int(self.overlap))
        try:
            yield
        finally:
            set_stream_overlap(prev)

    # ---- public ---------------------------------------------------------------------------
    def reset(self):
        self.pos.zero_()

    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        """prompt [batch, P] int64 at positions 0..P-1.  Returns the logits of the last position [batch, vocab]."""
        B, P = prompt.shape
        if B != self.batch or P > self.cfg.max_seq:
            raise ValueError("prompt shape does not fit the model's batch / max_seq")
        self._launches = 0
        self.reset()
        with self._overlapped():
            n = self._forward(prompt.reshape(-1).to(self.device, dtype=torch.int64).contiguous(), P, self.prefill_path)
            last = n.view(B, P, self.cfg.dim)[:, -1].contiguous()
            logits = self._logits(last, self.decode_path)
        self.pos.fill_(P)
        return logits

    def decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [batch] int64: the token at position *pos of every sequence.  Appends it to the cache,
        advances the position and returns the logits of the next token [batch, vocab]."""
        self._launches = 0
        with self._overlapped():
            n = self._forward(tokens.to(self.device, dtype=torch.int64).contiguous(), 1, self.decode_path)
            logits = self._logits(n, self.decode_path, self._final_planes)
        self.pos.add_(1)
        self._count()
        return logits

    def _greedy_step(self):
        logits = self.decode_step(self.tok)
        self._argmax(logits)
        self._count()
        self.launches_per_decode_step = self._launches
        return logits

    def _argmax(self, logits: torch.Tensor):
        """Greedy choice into self.tok: first index of the strict maximum (models.hpp:291-298)."""
        check(lib.sgqd_argmax_rows(_ptr(logits), logits.shape[0], logits.shape[1], logits.stride(0), _ptr(self.tok), _stream()),
              "sgqd_argmax_rows")

    def capture_decode_graph(self):
        """Records one greedy decode step (token buffer -> next token buffer) into a CUDA graph."""
        if self.world > 1 and self.exchange != "peer":
            raise RuntimeError("NCCL collectives are launched eagerly; use exchange='peer' to record the sharded step")
        saved_pos, saved_tok = self.pos.clone(), self.tok.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._greedy_step()                          # eager once: lazy kernel loading
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._greedy_step()
        self._graph = graph
        self.pos.copy_(saved_pos)
        self.tok.copy_(saved_tok)
        torch.cuda.synchronize()

    def generate(self, prompt: torch.Tensor, n_new: int, *, use_graph: bool = True, keep_logits: bool = False):
        """Greedy generation.  Returns tokens [batch, n_new] (and the list of per-step logits)."""
        B, P = prompt.shape
        if P + n_new > self.cfg.max_seq + 1:
            raise ValueError("prompt + new tokens exceed max_seq")
        logits = self.prefill(prompt)
        out = torch.empty(B, n_new, dtype=torch.int64, device=self.device)
        kept = [logits.clone()] if keep_logits else None
        self._argmax(logits)
        out[:, 0].copy_(self.tok)
        use_graph = use_graph and (self.world == 1 or self.exchange == "peer") and not keep_logits
        if use_graph and self._graph is None:
            self.capture_decode_graph()
        for s in range(1, n_new):
            if use_graph:
                self._graph.replay()
            else:
                lg = self._greedy_step()
                if keep_logits:
                    kept.append(lg.clone())
            out[:, s].copy_(self.tok)
        # A bounded device-side wait that ran out (a rank that never arrived at an exchange, a pipeline stall)
        # leaves incomplete outputs behind: it must reach the caller as an error, not as tokens.
        word = C.c_uint(0)
        if lib.sgq_device_status(C.byref(word), 1) != 0:
            raise RuntimeError(f"a device-side wait timed out during generation (status word 0x{word.value:08x}); the output is invalid")
        return (out, kept) if keep_logits else out
