"""Drop-in for ``mlstm_kernels.torch.backend_module`` restricted to the sm_100a kernels.

The reference's ``xlstm/xlstm_large/model.py:3-14`` imports seven names from that third-party
module and drives the cell through them (config built at ``model.py:477-487``, call at
``model.py:425-434``).  This module exports the same seven names with the same semantics:

* ``mLSTMBackendConfig`` -- dataclass with the fields the reference passes by keyword;
* ``mLSTMBackend`` -- ``nn.Module`` whose ``forward(q,k,v,i,f,c_initial,n_initial,m_initial)``
  returns ``(h, (c,n,m))`` in inference mode, ``h`` or ``(h, state)`` in the training modes
  exactly as documented at ``model.py:56-91``;
* the five ``Literal`` aliases used for type annotations.

Kernel names are looked up in three registries.  This package registers only its own CUDA
kernels (``chunkwise--b200``, ``native_sequence__b200``, ``b200``); nothing here computes the cell
in PyTorch.  Other kernels can be added with :func:`register_kernel` (the test-suite registers the
CPU oracle under the upstream ``native`` names that way).

Packed ragged batches and slot-indexed decode cannot be expressed through the reference's
``forward(x, state)`` signature, so that metadata travels through a side channel:
``with packed_batch(cu_seqlens): model(x)`` and ``with decode_slots(slot): model(x, state)``.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Callable, Literal, Optional

import torch
from torch import nn

from . import ops

ChunkwiseKernelType = str
SequenceKernelType = str
StepKernelType = str
DtypeType = Literal["float32", "bfloat16", "float16"]
BackendModeType = Literal["train", "train_with_padding", "inference"]

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}

_registry: dict[str, dict[str, Callable]] = {"chunkwise": {}, "sequence": {}, "step": {}}


def register_kernel(kind: str, name: str, fn: Callable) -> None:
    """kind in {"chunkwise","sequence","step"}.  Signatures:
    chunkwise/sequence: fn(q,k,v,i,f,c_initial,n_initial,m_initial,chunk_size=,eps=,return_last_states=) -> (h,(c,n,m))
    step:               fn(q,k,v,i,f,c,n,m,eps=) -> (h,(c,n,m)) with q,k,v (B,NH,D), i,f (B,NH,1)
    A chunkwise kernel that also handles a trailing partial chunk sets ``fn.handles_any_length = True``."""
    _registry[kind][name] = fn


def get_available_mlstm_kernels() -> list[str]:
    return sorted(_registry["chunkwise"])


def get_available_mlstm_sequence_kernels() -> list[str]:
    return sorted(_registry["sequence"])


def get_available_mlstm_step_kernels() -> list[str]:
    return sorted(_registry["step"])


# ------------------------------------------------------------------------------------------------
# side channel for what the reference's forward signature cannot carry
# ------------------------------------------------------------------------------------------------
class _SideChannel:
    cu_seqlens = None        # document offsets on the flattened (B*S) axis
    doc_states: Optional[list] = None   # filled with per-layer (c,n,m), one row per document
    slot = None              # (B,) int32 rows of the state pool for decode


_side = _SideChannel()


@contextlib.contextmanager
def packed_batch(cu_seqlens, collect_document_states: bool = True):
    """Inside this context the b200 prefill kernel treats every ``cu_seqlens`` interval as its own
    document (state reset at each boundary, inside the kernel).  The backend still returns a
    (B,NH,...) state -- the state of the LAST document of each row -- to keep the reference's
    contract; all per-document final states are appended to the yielded list, one entry per call."""
    prev = (_side.cu_seqlens, _side.doc_states)
    _side.cu_seqlens = cu_seqlens
    _side.doc_states = [] if collect_document_states else None
    try:
        yield _side.doc_states
    finally:
        _side.cu_seqlens, _side.doc_states = prev


@contextlib.contextmanager
def decode_slots(slot: torch.Tensor):
    """Inside this context the b200 step kernel reads and writes row ``slot[b]`` of the state tensors
    for stream b, so finished streams can be replaced without moving state."""
    prev = _side.slot
    _side.slot = slot
    try:
        yield
    finally:
        _side.slot = prev


# ------------------------------------------------------------------------------------------------
# the sm_100a kernels behind the registry names
# ------------------------------------------------------------------------------------------------
def _b200_sequence_impl(kernel):
    def fn(q, k, v, i, f, c_initial=None, n_initial=None, m_initial=None, chunk_size: int = 64, eps: float = 1e-6,
           return_last_states: bool = True, **_):
        B, NH, S, _ = q.shape
        cu = _side.cu_seqlens
        if cu is not None and c_initial is not None:
            raise ValueError("a packed batch starts every document from the zero state; do not pass an initial state")
        h, (c, n, m) = ops.mlstm_sequence(q, k, v, i, f, c_initial, n_initial, m_initial, cu_seqlens=cu, eps=eps,
                                          kernel=kernel)
        if cu is not None:
            if _side.doc_states is not None:
                _side.doc_states.append((c, n, m))
            # last document of each row = the document that ends at (b+1)*S
            cu_t = cu if torch.is_tensor(cu) else torch.tensor(list(cu))
            ends = torch.arange(1, B + 1, device=cu_t.device, dtype=cu_t.dtype) * S
            last = (torch.searchsorted(cu_t.contiguous(), ends, right=False) - 1).to(c.device).long()
            c, n, m = c[last], n[last], m[last]
        return h, (c, n, m)

    fn.handles_any_length = True
    return fn


def _b200_step(q, k, v, i, f, c=None, n=None, m=None, eps: float = 1e-6, **_):
    return ops.mlstm_step(q, k, v, i, f, c, n, m, slot=_side.slot, eps=eps, inplace=True)


register_kernel("chunkwise", "chunkwise--b200", _b200_sequence_impl("auto"))
register_kernel("sequence", "native_sequence__b200", _b200_sequence_impl("recurrent"))
register_kernel("step", "b200", _b200_step)


# ------------------------------------------------------------------------------------------------
# the interface the reference imports
# ------------------------------------------------------------------------------------------------
@dataclass
class mLSTMBackendConfig:
    """Same fields as the upstream config.  The b200 kernels are FORWARD ONLY: the modes 'train' and
    'train_with_padding' run them without an autograd graph, and ``mLSTMBackend.forward`` raises if an input
    requires a gradient while gradients are enabled."""
    chunkwise_kernel: ChunkwiseKernelType = "chunkwise--b200"
    sequence_kernel: SequenceKernelType = "native_sequence__b200"
    step_kernel: StepKernelType = "b200"
    mode: BackendModeType = "train"
    chunk_size: int = 64
    return_last_states: bool = True
    autocast_kernel_dtype: DtypeType = "bfloat16"
    eps: float = 1e-6
    inference_state_dtype: DtypeType = "float32"

    def __post_init__(self):
        if self.return_last_states and "parallel" in self.chunkwise_kernel:
            raise ValueError("return_last_states=True is not supported by parallel kernels")
        if self.mode not in ("train", "train_with_padding", "inference"):
            raise ValueError(f"unknown mode {self.mode!r}")
        if self.mode == "inference":
            self.return_last_states = True


class mLSTMBackend(nn.Module):
    config_class = mLSTMBackendConfig

    def __init__(self, config: mLSTMBackendConfig):
        super().__init__()
        self.config = config
        for kind, name in (("chunkwise", config.chunkwise_kernel), ("sequence", config.sequence_kernel),
                           ("step", config.step_kernel)):
            if name not in _registry[kind]:
                raise ValueError(f"unknown mLSTM {kind} kernel {name!r}; available: {sorted(_registry[kind])}")
        self.chunkwise_kernel_fn = _registry["chunkwise"][config.chunkwise_kernel]
        self.sequence_kernel_fn = _registry["sequence"][config.sequence_kernel]
        self.step_kernel_fn = _registry["step"][config.step_kernel]

    def extra_repr(self) -> str:
        return f"{self.config}"

    # -- helpers ---------------------------------------------------------------------------------
    def _cast_state(self, state):
        dt = _TORCH_DTYPES[self.config.inference_state_dtype]
        return tuple(None if s is None else s.to(dt) for s in state)

    def _chunkwise(self, q, k, v, i, f, c, n, m, return_last_states=True):
        return self.chunkwise_kernel_fn(q, k, v, i, f, c_initial=c, n_initial=n, m_initial=m,
                                        chunk_size=self.config.chunk_size, eps=self.config.eps,
                                        return_last_states=return_last_states)

    def forward(self, q, k, v, i, f, c_initial=None, n_initial=None, m_initial=None, return_last_states=None,
                mode=None):
        mode = self.config.mode if mode is None else mode
        if return_last_states is None:
            return_last_states = self.config.return_last_states
        S = q.shape[2]
        L = self.config.chunk_size
        if mode != "inference" and torch.is_grad_enabled() and any(
                t is not None and t.requires_grad for t in (q, k, v, i, f, c_initial, n_initial, m_initial)):
            if not getattr(self.chunkwise_kernel_fn, "differentiable", False):
                raise RuntimeError(
                    f"mLSTM kernel {self.config.chunkwise_kernel!r} is forward only (no backward kernel): run it under "
                    "torch.no_grad() or detach the inputs; training needs a differentiable kernel")
        if mode == "train":
            if S % L != 0 and not getattr(self.chunkwise_kernel_fn, "handles_any_length", False):
                raise ValueError(f"sequence length {S} is not a multiple of chunk_size {L}; use train_with_padding")
            h, state = self._chunkwise(q, k, v, i, f, c_initial, n_initial, m_initial, return_last_states)
            return (h, state) if return_last_states else h
        if mode == "train_with_padding":
            if return_last_states:
                raise ValueError("train_with_padding does not return states")
            if getattr(self.chunkwise_kernel_fn, "handles_any_length", False):
                h, _ = self._chunkwise(q, k, v, i, f, c_initial, n_initial, m_initial, False)
                return h
            pad = (-S) % L
            if pad:
                q, k, v = (torch.nn.functional.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
                i = torch.nn.functional.pad(i, (0, pad))
                f = torch.nn.functional.pad(f, (0, pad))
            h, _ = self._chunkwise(q, k, v, i, f, c_initial, n_initial, m_initial, False)
            return h[:, :, :S]
        # ---- inference: arbitrary S, always returns the last state
        if S == 1:
            h, state = self.step_kernel_fn(q[:, :, 0], k[:, :, 0], v[:, :, 0], i[:, :, 0:1], f[:, :, 0:1],
                                           c_initial, n_initial, m_initial, eps=self.config.eps)
            return h[:, :, None, :], self._cast_state(state)
        if getattr(self.chunkwise_kernel_fn, "handles_any_length", False):
            h, state = self._chunkwise(q, k, v, i, f, c_initial, n_initial, m_initial)
            return h, self._cast_state(state)
        S0 = (S // L) * L
        parts, state = [], (c_initial, n_initial, m_initial)
        if S0 > 0:
            h0, state = self._chunkwise(q[:, :, :S0], k[:, :, :S0], v[:, :, :S0], i[:, :, :S0], f[:, :, :S0], *state)
            parts.append(h0)
        if S0 < S:
            h1, state = self.sequence_kernel_fn(q[:, :, S0:], k[:, :, S0:], v[:, :, S0:], i[:, :, S0:], f[:, :, S0:],
                                                c_initial=state[0], n_initial=state[1], m_initial=state[2],
                                                eps=self.config.eps, return_last_states=True)
            parts.append(h1)
        h = parts[0] if len(parts) == 1 else torch.cat(parts, dim=2)
        return h, self._cast_state(state)
