"""Host-side mirror of the reference's xLSTM-Large (xLSTM-7B architecture) forward and greedy decode.

The reference drives the cell kernels from ``xlstm/xlstm_large/model.py`` (embedding -> blocks of
[RMSNorm, mLSTM layer, residual, RMSNorm, SwiGLU FFN, residual] -> RMSNorm -> lm_head -> soft cap,
``model.py:126-153, 379-452, 499-510``) and ``generate.py:27-90``.  That file runs unchanged on the
kernels of this package (through ``xlstm_b200.integration``); this mirror exists because benchmarks and GPU tests must
run where the reference checkout is not available, and because it adds what the reference has no code
for: head-parallel execution over several GPUs (one process per GPU, NCCL all-reduce after the
row-parallel projections) and slot-indexed states.

It consumes a state dict with the reference's "single" weight-mode key names
(``backbone.blocks.{i}.mlstm_layer.q.weight`` ...), so real checkpoints and the reference's own
modules are interchangeable with it.  Dense layers are plain library GEMMs (``torch.nn.functional.linear``);
the recurrent cell is the only part computed by this package's CUDA kernels.
"""
from __future__ import annotations

import hashlib
import math
from contextlib import nullcontext as _nullcontext
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from . import ops


@dataclass
class LargeConfig:
    """Subset of ``xLSTMLargeConfig`` (``model.py:30-109``) that determines the computation."""
    embedding_dim: int
    num_heads: int
    num_blocks: int
    vocab_size: int
    qk_dim_factor: float = 0.5
    v_dim_factor: float = 1.0
    ffn_proj_factor: float = 2.6667
    ffn_round_up_to_multiple_of: int = 64
    gate_soft_cap: float = 15.0
    output_logit_soft_cap: float = 30.0
    norm_eps: float = 1e-6
    eps: float = 1e-6

    @property
    def qk_dim(self):
        return int(self.embedding_dim * self.qk_dim_factor)

    @property
    def v_dim(self):
        return int(self.embedding_dim * self.v_dim_factor)

    @property
    def ffn_dim(self):
        m = self.ffn_round_up_to_multiple_of
        return int(math.ceil(self.embedding_dim * self.ffn_proj_factor / m) * m)


def parameter_shapes(cfg: LargeConfig) -> dict:
    D, NH, F_, V = cfg.embedding_dim, cfg.num_heads, cfg.ffn_dim, cfg.vocab_size
    shapes = {"embedding.weight": (V, D), "backbone.out_norm.weight": (D,), "lm_head.weight": (V, D)}
    for i in range(cfg.num_blocks):
        b = f"backbone.blocks.{i}."
        shapes.update({
            b + "norm_mlstm.weight": (D,), b + "norm_ffn.weight": (D,),
            b + "mlstm_layer.q.weight": (cfg.qk_dim, D), b + "mlstm_layer.k.weight": (cfg.qk_dim, D),
            b + "mlstm_layer.v.weight": (cfg.v_dim, D), b + "mlstm_layer.ogate_preact.weight": (cfg.v_dim, D),
            b + "mlstm_layer.igate_preact.weight": (NH, D), b + "mlstm_layer.igate_preact.bias": (NH,),
            b + "mlstm_layer.fgate_preact.weight": (NH, D), b + "mlstm_layer.fgate_preact.bias": (NH,),
            b + "mlstm_layer.multihead_norm.weight": (cfg.v_dim,), b + "mlstm_layer.out_proj.weight": (D, cfg.v_dim),
            b + "ffn.proj_up_gate.weight": (F_, D), b + "ffn.proj_up.weight": (F_, D), b + "ffn.proj_down.weight": (D, F_),
        })
    return shapes


def procedural_state_dict(cfg: LargeConfig, seed: int = 0, dtype=torch.float32, device="cpu", gen_device="cpu") -> dict:
    """Random-init weights that depend only on (seed, parameter name, shape): the same tensors can be produced in
    any process without shipping a checkpoint.  Linear weights ~ N(0, 1/fan_in), norm weights 1 + small noise,
    forget-gate biases around +3 (long memory), input-gate biases around 0."""
    out = {}
    for name, shape in parameter_shapes(cfg).items():
        h = int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") % (2 ** 63)
        # values are drawn on `gen_device`: "cpu" gives bit-identical tensors everywhere (fixtures), a CUDA device is
        # much faster for multi-billion-parameter shapes (benchmarks) but yields a different stream of numbers
        g = torch.Generator(device=gen_device).manual_seed(h)
        if name.endswith("norm.weight") or "norm_" in name:
            t = 1.0 + 0.05 * torch.randn(shape, generator=g, device=gen_device)
        elif name.endswith("fgate_preact.bias"):
            t = 3.0 + torch.randn(shape, generator=g, device=gen_device)
        elif name.endswith("bias"):
            t = 0.5 * torch.randn(shape, generator=g, device=gen_device)
        elif name == "embedding.weight":
            t = torch.randn(shape, generator=g, device=gen_device)
        else:
            t = torch.randn(shape, generator=g, device=gen_device) / math.sqrt(shape[-1])
        out[name] = t.to(dtype).to(device)
    return out


def _soft_cap(x, cap):
    return cap * torch.tanh(x / cap)


def _rms_norm(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class LargeModel:
    """Inference-only mirror.  With ``tp_world > 1`` each rank holds ``num_heads / tp_world`` heads (column-parallel
    q/k/v/o-gate/gate projections, per-head norm, row-parallel out_proj).

    Prefill (many tokens, compute-bound) keeps the residual stream SHARDED OVER TOKENS: the partial sums of the
    row-parallel out_proj are reduce-scattered over the token axis, the residual add, both RMSNorms and the whole FFN run
    on the rank's own tokens with the full FFN weights, and the normed activations are all-gathered in front of the next
    block's projections -- one reduce-scatter + one all-gather per block, the traffic of ONE all-reduce, instead of the
    two all-reduces of the classic scheme.  The batch rows are cut into groups that are issued alternately on two
    streams, so that one group's collectives run under the other group's GEMMs and cell kernels.

    Decode (one token per stream, bound by streaming the weights) shards the FFN over its WIDTH instead, so that every
    rank streams 1/tp_world of every weight; that costs a second small all-reduce per block, which a replay of the
    captured step graph includes.  Every rank therefore holds the full FFN weights; its decode slice is a view of them."""

    def __init__(self, cfg: LargeConfig, state_dict: dict, device, dtype=torch.bfloat16, tp_rank: int = 0,
                 tp_world: int = 1, group=None, cell_ops=ops, fused_adjacent: bool = True):
        # `cell_ops` provides mlstm_sequence / mlstm_step; the default is this package's CUDA kernels (the test
        # suite substitutes the CPU oracle to check the dense part of this mirror against the reference on a CPU)
        self.cell = cell_ops
        # residual add + RMSNorm, per-head norm + output gate and the soft caps as single kernels of this package (CUDA only)
        self.fused = bool(fused_adjacent) and torch.device(device).type == "cuda" and cell_ops is ops
        if cfg.num_heads % tp_world or cfg.ffn_dim % tp_world:
            raise ValueError("num_heads and the FFN width must be divisible by the tensor-parallel world size")
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.tp_rank, self.tp_world, self.group = tp_rank, tp_world, group
        NH, NHl = cfg.num_heads, cfg.num_heads // tp_world
        self.nh_local = NHl
        dq, dv = cfg.qk_dim // NH, cfg.v_dim // NH
        self.dq, self.dv = dq, dv
        h0, h1 = tp_rank * NHl, (tp_rank + 1) * NHl
        # zero rows behind the 2 * NHl gate rows of the stacked projection weight: its output rows then are a multiple of
        # 16 elements long, which keeps every column slice (q, k, v, o) on the 16-byte alignment TMA and vector loads need
        self.gate_pad = (-2 * NHl) % 16
        f0, f1 = tp_rank * cfg.ffn_dim // tp_world, (tp_rank + 1) * cfg.ffn_dim // tp_world

        def W(name):
            return state_dict[name].to(self.device, dtype)

        self.embedding, self.out_norm, self.lm_head = W("embedding.weight"), W("backbone.out_norm.weight"), W("lm_head.weight")
        self.blocks = []
        for i in range(cfg.num_blocks):
            b = f"backbone.blocks.{i}."
            # one stacked weight for q | k | v | o-gate | i-gate | f-gate: the views below share its memory, and the fused
            # path runs all six projections as ONE GEMM (the gate bias is added by the soft-cap kernel)
            qkvo_if = torch.cat([W(b + "mlstm_layer.q.weight")[h0 * dq:h1 * dq], W(b + "mlstm_layer.k.weight")[h0 * dq:h1 * dq],
                                 W(b + "mlstm_layer.v.weight")[h0 * dv:h1 * dv], W(b + "mlstm_layer.ogate_preact.weight")[h0 * dv:h1 * dv],
                                 W(b + "mlstm_layer.igate_preact.weight")[h0:h1], W(b + "mlstm_layer.fgate_preact.weight")[h0:h1],
                                 torch.zeros(self.gate_pad, cfg.embedding_dim, device=self.device, dtype=dtype)], 0).contiguous()
            n_qkvo = 2 * NHl * dq + 2 * NHl * dv
            blk = dict(
                norm_mlstm=W(b + "norm_mlstm.weight"), norm_ffn=W(b + "norm_ffn.weight"), qkvo_if=qkvo_if,
                qkvo=qkvo_if[:n_qkvo], if_w=qkvo_if[n_qkvo:n_qkvo + 2 * NHl],
                if_b=torch.cat([W(b + "mlstm_layer.igate_preact.bias")[h0:h1], W(b + "mlstm_layer.fgate_preact.bias")[h0:h1]], 0).contiguous(),
                mh_norm=W(b + "mlstm_layer.multihead_norm.weight")[h0 * dv:h1 * dv].contiguous(),
                out_proj=W(b + "mlstm_layer.out_proj.weight")[:, h0 * dv:h1 * dv].contiguous(),
                up=torch.cat([W(b + "ffn.proj_up_gate.weight")[f0:f1], W(b + "ffn.proj_up.weight")[f0:f1]], 0).contiguous(),
                down=W(b + "ffn.proj_down.weight")[:, f0:f1].contiguous(),
            )
            if tp_world > 1:   # token-parallel prefill runs the whole FFN on the rank's own tokens
                blk["up_full"] = torch.cat([W(b + "ffn.proj_up_gate.weight"), W(b + "ffn.proj_up.weight")], 0).contiguous()
                blk["down_full"] = W(b + "ffn.proj_down.weight").contiguous()
            self.blocks.append(blk)
        self.comm_ms = None        # set by forward(..., time_collectives=True): CUDA-event time inside collectives
        self.comm_bytes = 0
        self.peer = None           # PeerReducer of the decode step (enable_peer_reduce)
        self.peer_unavailable = None

    # ------------------------------------------------------------------------------------------------
    def _all_reduce(self, x):
        if self.tp_world > 1:
            torch.distributed.all_reduce(x, group=self.group)
        return x

    def _mlstm_layer(self, blk, x, state, cu_seqlens, slot, reduce: bool = True):
        cfg, NHl, dq, dv = self.cfg, self.nh_local, self.dq, self.dv
        B, S, _ = x.shape
        if self.fused:   # one GEMM for all six projections; the gates are capped in fp32 (they enter exponentials in the cell)
            allp = F.linear(x, blk["qkvo_if"])
            q, k, v, o, gpre, _ = torch.split(allp, [NHl * dq, NHl * dq, NHl * dv, NHl * dv, 2 * NHl, self.gate_pad], dim=-1)
            if S == 1 and cu_seqlens is None and self.cell is ops and dv <= 1024:
                # decode: gate cap, cell step, per-head norm and output gate in one kernel
                c, n, m = state if state is not None else (None, None, None)
                hg, new_state = ops.mlstm_decode_cell(q.reshape(B, NHl, dq), k.reshape(B, NHl, dq), v.reshape(B, NHl, dv), gpre, blk["if_b"],
                                                      cfg.gate_soft_cap, o, blk["mh_norm"], c, n, m, slot=slot, eps=cfg.eps,
                                                      norm_eps=cfg.norm_eps)
                y = F.linear(hg.reshape(B, 1, NHl * dv), blk["out_proj"])
                return (self._all_reduce(y) if reduce else y), new_state
            gates = ops.soft_cap(gpre, cfg.gate_soft_cap, out_float32=True, float32_math=True, bias=blk["if_b"])
        else:
            qkvo = F.linear(x, blk["qkvo"])
            q, k, v, o = torch.split(qkvo, [NHl * dq, NHl * dq, NHl * dv, NHl * dv], dim=-1)
            gates = _soft_cap(F.linear(x, blk["if_w"], blk["if_b"]).float(), cfg.gate_soft_cap)   # (B,S,2*NHl) fp32
        ig, fg = gates[..., :NHl].transpose(1, 2), gates[..., NHl:].transpose(1, 2)          # (B,NHl,S) views
        q = q.reshape(B, S, NHl, dq).transpose(1, 2)     # strided views, no copies (model.py:415-417)
        k = k.reshape(B, S, NHl, dq).transpose(1, 2)
        v = v.reshape(B, S, NHl, dv).transpose(1, 2)
        if S == 1 and cu_seqlens is None:
            c, n, m = state if state is not None else (None, None, None)
            h, new_state = self.cell.mlstm_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], ig, fg, c, n, m, slot=slot, eps=cfg.eps)
            h = h[:, :, None]
        else:
            c, n, m = state if state is not None else (None, None, None)
            h, new_state = self.cell.mlstm_sequence(q, k, v, ig, fg, c, n, m, cu_seqlens=cu_seqlens, eps=cfg.eps)
        if self.fused:
            hg = ops.headnorm_gate(h, o, blk["mh_norm"], eps=cfg.norm_eps)
            y = F.linear(hg, blk["out_proj"])
            return (self._all_reduce(y) if reduce else y), new_state
        h = h.transpose(1, 2)                            # (B,S,NHl,dv)
        hf = h.float()
        hn = (hf - hf.mean(-1, keepdim=True)) * torch.rsqrt(hf.var(-1, keepdim=True, unbiased=False) + cfg.norm_eps)
        hn = hn.to(x.dtype).reshape(B, S, NHl * dv) * blk["mh_norm"]
        y = F.linear(torch.sigmoid(o) * hn, blk["out_proj"])
        return (self._all_reduce(y) if reduce else y), new_state

    def _swiglu(self, gz):
        """silu(gate) * up on the output of the stacked up-projection (``model.py:268-277``)."""
        if self.fused:
            return ops.swiglu(gz)
        g, z = gz.chunk(2, dim=-1)
        return F.silu(g) * z

    def enable_peer_reduce(self, rows_max: int = 256) -> bool:
        """Tensor-parallel decode without NCCL launches: the all-reduce of each row-parallel projection's partial sums is
        fused with the residual add and the following RMSNorm into one kernel over peer memory (``peer.PeerReducer``).
        Every rank must call this; returns False (and keeps NCCL) where symmetric memory cannot be set up."""
        if self.tp_world == 1 or not self.fused:
            return False
        if self.peer is None and self.peer_unavailable is None:
            from .peer import PeerReducer
            self.peer, self.peer_unavailable = PeerReducer.create(self.group, self.device, rows_max, self.cfg.embedding_dim, self.dtype)
            # all ranks or none: a rank that failed makes the others fall back too
            okt = torch.tensor([1 if self.peer is not None else 0], device=self.device)
            torch.distributed.all_reduce(okt, op=torch.distributed.ReduceOp.MIN, group=self.group)
            if int(okt.item()) == 0:
                self.peer = None
                self.peer_unavailable = self.peer_unavailable or "another rank could not set up symmetric memory"
        return self.peer is not None

    def _reduce_add_norm(self, x, y_partial, w):
        """``_add_norm`` on the SUM over ranks of `y_partial`: one peer-memory kernel when it is enabled and the rows fit,
        an all-reduce followed by the add + norm kernel otherwise."""
        if y_partial is None or self.tp_world == 1:
            return self._add_norm(x, y_partial, w)
        rows = x.numel() // x.shape[-1]
        if self.peer is not None and rows <= self.peer.rows_max and x.is_contiguous():
            return self.peer.reduce_add_rmsnorm(y_partial, x, w, self.cfg.norm_eps)
        return self._add_norm(x, self._all_reduce(y_partial), w)

    def _add_norm(self, x, y, w):
        """x + y (y may be None) and its RMSNorm, as the reference's block does with two operators (model.py:499-510)."""
        if self.fused:
            return ops.add_rmsnorm(x, w, y, eps=self.cfg.norm_eps, inplace=True)
        if y is not None:
            x = x + y
        return x, _rms_norm(x, w, self.cfg.norm_eps)

    # ------------------------------------------------------------------------------------------------ token-parallel prefill
    def _gather_tokens(self, x_shard):
        """(T/world, D) -> (T, D): every rank's tokens, in rank order."""
        out = torch.empty((x_shard.shape[0] * self.tp_world, x_shard.shape[1]), dtype=x_shard.dtype, device=x_shard.device)
        torch.distributed.all_gather_into_tensor(out, x_shard.contiguous(), group=self.group)
        return out

    def _scatter_sum(self, y_full):
        """(T, D) partial sums -> (T/world, D): the sum over ranks of this rank's tokens."""
        T = y_full.shape[0]
        n = T // self.tp_world
        if torch.distributed.get_backend(self.group) == "gloo":   # (CPU tests: gloo has no reduce-scatter)
            y = y_full.clone()
            torch.distributed.all_reduce(y, group=self.group)
            return y[self.tp_rank * n:(self.tp_rank + 1) * n].contiguous()
        out = torch.empty((n, y_full.shape[1]), dtype=y_full.dtype, device=y_full.device)
        torch.distributed.reduce_scatter_tensor(out, y_full.contiguous(), group=self.group)
        return out

    def _timed(self, fn, x, record):
        if record is None:
            return fn(x)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        y = fn(x)
        e1.record()
        record.append((e0, e1, x.numel() * x.element_size() if fn == self._scatter_sum else y.numel() * y.element_size()))
        return y

    def _side_stream(self):
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side

    def token_parallel_ok(self, tokens, state, cu_seqlens, slot) -> bool:
        return (self.tp_world > 1 and tokens.shape[1] > 1 and slot is None
                and (tokens.shape[0] * tokens.shape[1]) % self.tp_world == 0)

    def _forward_token_parallel(self, tokens, state, cu_seqlens, last_only, groups: int = 2, time_collectives: bool = False,
                                greedy: bool = False):
        """Prefill with the residual stream sharded over tokens (see the class docstring).  Batch rows are cut into
        `groups` independent pieces; piece g runs on stream g % 2, so its collectives overlap the other piece's compute."""
        cfg, W, dev = self.cfg, self.tp_world, self.device
        B, S = tokens.shape
        if cu_seqlens is not None or B % groups or ((B // groups) * S) % W:
            groups = 1
        Bg = B // groups
        n = Bg * S // W                                   # tokens of a piece that live on this rank
        cuda = dev.type == "cuda"
        streams = ([torch.cuda.current_stream(dev)] + ([self._side_stream()] if groups > 1 else [])) if cuda else [None]
        record = [] if (time_collectives and cuda) else None
        if cuda and len(streams) > 1:
            streams[1].wait_stream(streams[0])
        pieces = []
        for g in range(groups):
            flat = tokens[g * Bg:(g + 1) * Bg].reshape(-1)
            pieces.append(dict(x=self.embedding[flat[self.tp_rank * n:(self.tp_rank + 1) * n]], pending=None, state={}))
        for i, blk in enumerate(self.blocks):
            for g, pc in enumerate(pieces):
                ctx = torch.cuda.stream(streams[g % len(streams)]) if cuda else _nullcontext()
                with ctx:
                    pc["x"], xn = self._add_norm(pc["x"], pc["pending"], blk["norm_mlstm"])
                    xn_full = self._timed(self._gather_tokens, xn, record).reshape(Bg, S, -1)
                    st_in = None if state is None else tuple(t[g * Bg:(g + 1) * Bg] for t in state[i])
                    y, st = self._mlstm_layer(blk, xn_full, st_in, cu_seqlens, None, reduce=False)
                    pc["state"][i] = st
                    y = self._timed(self._scatter_sum, y.reshape(Bg * S, -1), record)
                    pc["x"], xn = self._add_norm(pc["x"], y, blk["norm_ffn"])
                    pc["pending"] = F.linear(self._swiglu(F.linear(xn, blk["up_full"])), blk["down_full"])
        outs = []
        for g, pc in enumerate(pieces):
            ctx = torch.cuda.stream(streams[g % len(streams)]) if cuda else _nullcontext()
            with ctx:
                pc["x"], xn = self._add_norm(pc["x"], pc["pending"], self.out_norm)
                xn_full = self._timed(self._gather_tokens, xn, record).reshape(Bg, S, -1)
                if last_only:
                    xn_full = xn_full[:, -1:]
                outs.append(self._head(xn_full, greedy))
        if cuda and len(streams) > 1:
            streams[0].wait_stream(streams[1])
        logits = outs[0] if groups == 1 else torch.cat(outs, 0)
        new_state = {}
        for i in range(len(self.blocks)):
            parts = [pc["state"][i] for pc in pieces]
            new_state[i] = parts[0] if groups == 1 else tuple(torch.cat([p_[k] for p_ in parts], 0) for k in range(3))
        if record is not None:
            torch.cuda.synchronize(dev)
            self.comm_ms = sum(a.elapsed_time(b_) for a, b_, _ in record)
            self.comm_bytes = sum(nb for _, _, nb in record)
            self.comm_calls = len(record)
        return logits, new_state

    def _head(self, xn, greedy: bool):
        """lm_head and soft cap; with `greedy` the argmax of the last position as well (``generate.py:13-15``), on CUDA in
        one kernel behind the GEMM."""
        cfg = self.cfg
        logits = F.linear(xn, self.lm_head)
        if greedy:
            if self.fused:
                return ops.softcap_argmax(logits[:, -1], cfg.output_logit_soft_cap)[:, None]
            return torch.argmax(_soft_cap(logits[:, -1:], cfg.output_logit_soft_cap), dim=-1)
        return ops.soft_cap(logits, cfg.output_logit_soft_cap) if self.fused else _soft_cap(logits, cfg.output_logit_soft_cap)

    def forward(self, tokens, state: Optional[dict] = None, cu_seqlens=None, slot=None, last_only: bool = False,
                time_collectives: bool = False, positions=None, greedy: bool = False):
        """tokens (B,S) int64 -> logits (B,S,V) (or (B,1,V) with ``last_only``) and the per-block state dict
        ``{i: (c,n,m)}`` exactly as ``xLSTMLarge.forward`` returns it (``model.py:126-153``).  With ``cu_seqlens`` every
        interval of the flattened (B*S) token axis is a document of its own and the states have one row per document;
        ``positions`` (flat token indices) restricts the logits to those tokens, returned as (len(positions), 1, V) --
        a packed prefill only needs the last token of every document.  ``greedy`` returns the greedy token of the last
        position, (rows, 1) int64, in place of the logits."""
        if positions is None and self.token_parallel_ok(tokens, state, cu_seqlens, slot):
            return self._forward_token_parallel(tokens, state, cu_seqlens, last_only or greedy, time_collectives=time_collectives,
                                                greedy=greedy)
        cfg = self.cfg
        x = self.embedding[tokens]
        new_state = {}
        pending = None   # output of the previous sub-block (a PARTIAL sum under tensor parallelism): reduced over the ranks
        # and added to the residual stream by the next norm call
        for i, blk in enumerate(self.blocks):
            x, xn = self._reduce_add_norm(x, pending, blk["norm_mlstm"])
            y, st = self._mlstm_layer(blk, xn, None if state is None else state[i], cu_seqlens, slot, reduce=False)
            new_state[i] = st
            x, xn = self._reduce_add_norm(x, y, blk["norm_ffn"])
            pending = F.linear(self._swiglu(F.linear(xn, blk["up"])), blk["down"])
        if positions is not None:
            x = x.reshape(-1, x.shape[-1])[positions][:, None]
            pending = None if pending is None else pending.reshape(-1, pending.shape[-1])[positions][:, None]
        elif last_only or greedy:
            x = x[:, -1:]
            pending = None if pending is None else pending[:, -1:]
        if pending is not None and not x.is_contiguous():
            x, pending = x.contiguous(), pending.contiguous()
        x, xn = self._reduce_add_norm(x, pending, self.out_norm)
        return self._head(xn, greedy), new_state

    # ------------------------------------------------------------------------------------------------
    def _capture_decode_graph(self, state, batch: int, slot_map=None):
        """Capture one decode step (all blocks, lm_head, argmax) in a CUDA graph.  ``slot_map`` (int32, one entry per
        row: the row's own index, or -1 while the row is free) makes the step kernel skip free rows, so an idle slot
        costs no state traffic.  The reference's decode loop
        (``generate.py:79-85``) launches every small operator from the host for every token; replaying a graph
        removes that launch cost.  State lives in static buffers: C is updated in place by the step kernel, n and m
        are copied back into their buffers inside the graph, and the sampled token feeds the next replay."""
        dev = self.device
        if self.tp_world > 1:
            self.enable_peer_reduce(max(batch, 256))   # (keeps NCCL where symmetric memory is not available)
        self._g_state = {i: tuple(t for t in st) for i, st in state.items()}
        self._g_tok = torch.zeros(batch, 1, dtype=torch.long, device=dev)

        self._g_slot = slot_map

        def body():
            nxt, st = self.forward(self._g_tok, self._g_state, greedy=True, slot=self._g_slot)
            dsts, srcs = [], []
            for i, (c, n, m) in st.items():
                assert c is self._g_state[i][0]
                dsts += [self._g_state[i][1], self._g_state[i][2]]
                srcs += [n, m.reshape(self._g_state[i][2].shape)]
            torch._foreach_copy_(dsts, srcs)   # one multi-tensor launch instead of two small copies per block
            self._g_tok.copy_(nxt)

        snapshot = {i: tuple(t.clone() for t in st) for i, st in self._g_state.items()}
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):   # warm-up outside capture (lazy initialisations, allocator pools)
                body()
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        # With tensor parallelism the graph holds NCCL all-reduces: their communicator is warm (the warm-up runs above)
        # and the capture must not be global, or the watchdog thread's event queries would invalidate it.
        mode = "thread_local" if self.tp_world > 1 else "global"
        with torch.cuda.graph(graph, capture_error_mode=mode):
            body()
        for i, st in snapshot.items():   # undo the state changes of the warm-up and capture runs
            for dst, src in zip(self._g_state[i], st):
                dst.copy_(src)
        self._graph, self._graph_batch = graph, batch

    def parameters_on_device(self):
        """Every weight tensor this rank holds (its share under tensor parallelism)."""
        out = [self.embedding, self.out_norm, self.lm_head]
        for blk in self.blocks:
            out += [v for k, v in blk.items() if isinstance(v, torch.Tensor) and k not in ("qkvo", "if_w")]   # (views of qkvo_if)
        return out

    def release_graph(self):
        """Drop the captured decode graph and its static buffers.  With tensor parallelism call this before the process
        group is destroyed: a live graph that holds NCCL kernels keeps the communicator from shutting down."""
        self._graph = None
        self._g_state = None
        self._g_tok = None
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    @torch.no_grad()
    def generate(self, prefill_tokens, max_length: int, state=None, use_cuda_graph: bool = False):
        """Greedy decoding as ``generate_tokens`` does it (``generate.py:79-85``): the first iteration consumes the
        prefill, every iteration appends argmax of the last position.  With ``use_cuda_graph`` the single-token
        iterations replay a captured graph (same arithmetic, far fewer host launches)."""
        out = torch.empty(prefill_tokens.shape[0], max_length, dtype=torch.long, device=self.device)
        last = prefill_tokens
        for i in range(max_length):
            if use_cuda_graph and i >= 1:
                if i == 1:
                    B = prefill_tokens.shape[0]
                    if getattr(self, "_graph", None) is None or self._graph_batch != B:
                        self._capture_decode_graph(state, B)
                    else:   # load the fresh prefill state into the graph's static buffers
                        for j, st in state.items():
                            for dst, src in zip(self._g_state[j], st):
                                dst.copy_(src.reshape(dst.shape))
                    self._g_tok.copy_(last)
                self._graph.replay()
                out[:, i:i + 1] = self._g_tok
                continue
            last, state = self.forward(last, state, greedy=True)
            out[:, i:i + 1] = last
        if use_cuda_graph and max_length > 1:
            state = self._g_state
        if self.device.type == "cuda" and self.cell is ops:
            ops.check_device_status(self.device)   # synchronises; surfaces a kernel whose bounded wait expired
        return out, state


class ContinuousDecoder:
    """Continuous-batch greedy decoding over a fixed pool of state slots with refill.

    Every stream owns one row of the per-block state pool; a decode step advances all ACTIVE rows at once (on CUDA by
    replaying the captured graph of ``LargeModel``, whose static state buffers ARE the pool; rows of free slots are
    marked -1 in the slot map the step kernel reads and cost no state traffic).  When a stream has its tokens the host
    frees the slot (``sharding.SlotPool``) and queued documents take free slots over.

    Admission is a PACKED prefill: the waiting documents are packed into rows of ``row_len`` tokens
    (``sharding.pack_documents``), one forward with ``cu_seqlens`` runs them all -- the cell kernels reset their state at
    every document boundary and emit every document's own final state -- and those states are scattered into the
    documents' slots, their first tokens into the slots' token cells.  The reference's loop (``generate.py:27-90``) has no
    refill: it decodes one fixed batch to the end.  Token by token a stream computes what ``LargeModel.generate`` computes
    for it alone.  ``packed_admission=False`` prefills every document on its own (the CPU tests use it with the oracle
    cell, which knows no document offsets)."""

    def __init__(self, model: LargeModel, num_slots: int, use_cuda_graph: Optional[bool] = None, row_len: int = 32768,
                 max_rows_per_prefill: int = 4, packed_admission: Optional[bool] = None):
        from .sharding import SlotPool
        self.model, self.num_slots = model, num_slots
        cfg, dev = model.cfg, model.device
        self.graphed = (dev.type == "cuda") if use_cuda_graph is None else use_cuda_graph
        self.packed = (dev.type == "cuda" and model.cell is ops) if packed_admission is None else packed_admission
        self.row_len, self.max_rows = row_len, max_rows_per_prefill
        self.state = {i: (torch.zeros(num_slots, model.nh_local, model.dq, model.dv, device=dev),
                          torch.zeros(num_slots, model.nh_local, model.dq, device=dev),
                          torch.zeros(num_slots, model.nh_local, 1, device=dev)) for i in range(cfg.num_blocks)}
        self.tok = torch.zeros(num_slots, 1, dtype=torch.long, device=dev)
        self.slots = SlotPool(num_slots)
        self.slot_map = torch.full((num_slots,), -1, dtype=torch.int32, device=dev) if dev.type == "cuda" and model.cell is ops else None
        self.prefill_calls = 0
        if self.graphed:
            if self.slot_map is not None:
                self.slot_map.copy_(torch.arange(num_slots, dtype=torch.int32, device=dev))   # capture with every row live
            model._capture_decode_graph(self.state, num_slots, slot_map=self.slot_map)   # the graph's static buffers are this pool
            self.state, self.tok = model._g_state, model._g_tok
            if self.slot_map is not None:
                self.slot_map.fill_(-1)

    # ------------------------------------------------------------------------------------------------ admission
    @torch.no_grad()
    def _admit_single(self, slot: int, prompt: torch.Tensor) -> None:
        first, st = self.model.forward(prompt.reshape(1, -1).to(self.model.device), greedy=True)
        self.prefill_calls += 1
        for i, (c, n, m) in st.items():
            self.state[i][0][slot].copy_(c[0])
            self.state[i][1][slot].copy_(n[0])
            self.state[i][2][slot].copy_(m[0].reshape(self.state[i][2][slot].shape))
        self.tok[slot].copy_(first[0])

    @torch.no_grad()
    def _admit_packed(self, slots, prompts) -> None:
        """slots[i] receives prompts[i].  Documents longer than a row get a row of their own length."""
        from .sharding import pack_documents
        dev = self.model.device
        lengths = [int(p.numel()) for p in prompts]
        # rows of row_len tokens; a batch that is shorter than one row gets one row of its own size, a document that is
        # longer than a row widens the rows
        row_len = max(max(lengths), min(self.row_len, -(-sum(lengths) // 8) * 8))
        packed = pack_documents(lengths, row_len)
        # rows in groups of at most max_rows: one forward per group
        for r0 in range(0, packed.rows, self.max_rows):
            r1 = min(packed.rows, r0 + self.max_rows)
            lo, hi = r0 * packed.row_len, r1 * packed.row_len
            first = next(k for k, c in enumerate(packed.cu_seqlens) if c >= lo)
            last = max(k for k, c in enumerate(packed.cu_seqlens) if c <= hi)
            cu = [c - lo for c in packed.cu_seqlens[first:last + 1]]
            ids = packed.doc_ids[first:last]
            tokens = torch.zeros((r1 - r0) * packed.row_len, dtype=torch.long, device=dev)
            docs, rows_of_state, ends = [], [], []
            for k, d in enumerate(ids):
                if d < 0:
                    continue
                tokens[cu[k]:cu[k + 1]] = prompts[d].to(dev)
                docs.append(d); rows_of_state.append(k); ends.append(cu[k + 1] - 1)
            first, st = self.model.forward(tokens.reshape(r1 - r0, packed.row_len), cu_seqlens=cu, greedy=True,
                                           positions=torch.tensor(ends, dtype=torch.long, device=dev))
            self.prefill_calls += 1
            dst = torch.tensor([slots[d] for d in docs], dtype=torch.long, device=dev)
            src = torch.tensor(rows_of_state, dtype=torch.long, device=dev)
            for i, (c, n, m) in st.items():
                self.state[i][0].index_copy_(0, dst, c.index_select(0, src))
                self.state[i][1].index_copy_(0, dst, n.index_select(0, src))
                self.state[i][2].index_copy_(0, dst, m.index_select(0, src).reshape(len(docs), *self.state[i][2].shape[1:]))
            self.tok.index_copy_(0, dst, first)

    def _admit(self, slots, prompts) -> None:
        if self.packed:
            self._admit_packed(slots, prompts)
        else:
            for s_, p_ in zip(slots, prompts):
                self._admit_single(s_, p_)
        if self.slot_map is not None:
            idx = torch.tensor(slots, dtype=torch.long, device=self.model.device)
            self.slot_map.index_copy_(0, idx, idx.to(torch.int32))

    @torch.no_grad()
    def _step(self) -> None:
        if self.graphed:
            self.model._graph.replay()
            return
        nxt, st = self.model.forward(self.tok, self.state, greedy=True, slot=self.slot_map)
        for i, (c, n, m) in st.items():
            for dst, src in zip(self.state[i], (c, n, m)):
                if dst is not src:
                    dst.copy_(src.reshape(dst.shape))
        self.tok.copy_(nxt)

    # ------------------------------------------------------------------------------------------------ eviction
    @torch.no_grad()
    def _evict(self, slot: int, park_on_host: bool):
        """Takes a running stream out of its slot: its whole recurrent state (C, n, m of every block -- constant size, no
        cache that grows) and its pending token are copied to a parking buffer, the slot is marked inactive."""
        def park(t):
            return t.to("cpu", non_blocking=False) if park_on_host else t.clone()
        parcel = ({i: tuple(park(x[slot]) for x in self.state[i]) for i in self.state}, park(self.tok[slot]))
        if self.slot_map is not None:
            self.slot_map[slot] = -1
        return parcel

    @torch.no_grad()
    def _resume(self, slot: int, parcel) -> None:
        st, tok = parcel
        for i, parts in st.items():
            for dst, src in zip(self.state[i], parts):
                dst[slot].copy_(src.to(dst.device))
        self.tok[slot].copy_(tok.to(self.tok.device))
        if self.slot_map is not None:
            self.slot_map[slot] = slot

    @torch.no_grad()
    def run(self, prompts, new_tokens, quantum: Optional[int] = None, park_on_host: bool = False):
        """prompts: sequence of 1-D int64 tensors; new_tokens: int or per-document counts (>= 1).  Returns the list of
        generated token tensors in the order of ``prompts``.

        ``quantum``: with documents waiting and no slot free, a stream that has decoded ``quantum`` tokens since it was
        (re)admitted is EVICTED -- state and pending token parked (on the device, or on the host with ``park_on_host``) --
        and queues up behind the waiting documents; it later resumes from the parked state in whatever slot is free,
        without a second prefill.  Tokens are the same with and without eviction."""
        counts = [int(new_tokens)] * len(prompts) if isinstance(new_tokens, int) else [int(x) for x in new_tokens]
        if len(counts) != len(prompts) or any(c < 1 for c in counts):
            raise ValueError("one positive token count per prompt")
        if quantum is not None and quantum < 1:
            raise ValueError("quantum must be positive")
        queue = list(range(len(prompts)))[::-1]
        parked = {}          # document -> parcel of an evicted stream
        left = dict(enumerate(counts))   # document -> tokens still to produce
        active = {}          # slot -> [document, position of the first token of this residency in `hist`, steps in this residency]
        hist = []            # token column of every step (device tensors; read back once at the end)
        spans = {d: [] for d in range(len(prompts))}   # document -> [(slot, first, count)] in order
        self.evictions = 0
        while queue or active:
            if queue and self.slots.free:
                fresh, back = [], []
                while queue and self.slots.free:
                    d = queue.pop()
                    (back if d in parked else fresh).append((self.slots.acquire(d), d))
                if fresh:
                    self._admit([s_ for s_, _ in fresh], [prompts[d] for _, d in fresh])
                for s_, d in back:
                    self._resume(s_, parked.pop(d))
                for s_, d in fresh + back:
                    active[s_] = [d, len(hist), 0]
            hist.append(self.tok[:, 0].clone())      # the token every active slot has just produced
            freed = []
            for s_ in list(active):
                d = active[s_][0]
                left[d] -= 1
                active[s_][2] += 1
                if left[d] == 0:
                    _, first, n = active.pop(s_)
                    spans[d].append((s_, first, n))
                    self.slots.release(s_)
                    freed.append(s_)
            if freed and self.slot_map is not None:
                self.slot_map.index_fill_(0, torch.tensor(freed, dtype=torch.long, device=self.model.device), -1)
            if active:
                self._step()
            # eviction: between steps, with nothing in flight for the stream (its state and next token are complete)
            if quantum is not None and queue and not self.slots.free:
                waiting = len(queue)
                for s_ in sorted(active, key=lambda k: -active[k][2]):
                    if waiting == 0 or active[s_][2] < quantum:
                        break
                    d, first, n = active.pop(s_)
                    spans[d].append((s_, first, n))
                    parked[d] = self._evict(s_, park_on_host)
                    self.slots.release(s_)
                    queue.insert(0, d)          # behind every document that is waiting now
                    self.evictions += 1
                    waiting -= 1
        cols = torch.stack(hist, dim=1).cpu()          # (slots, steps)
        if self.model.device.type == "cuda" and self.model.cell is ops:
            ops.check_device_status(self.model.device)
        return [torch.cat([cols[s_, first:first + n] for s_, first, n in spans[d]]).clone() for d in range(len(prompts))]
