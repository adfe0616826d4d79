"""Hooks that put the sm_100a kernels behind the reference package's own selectors.

``install_mlstm_backend()``  makes ``import mlstm_kernels.torch.backend_module`` resolve to
:mod:`xlstm_b200.backend_module` when the upstream package is not installed, or adds the b200
kernel names to the upstream registries when it is.  After that
``xLSTMLargeConfig(chunkwise_kernel="chunkwise--b200", sequence_kernel="native_sequence__b200",
step_kernel="b200", mode="inference")`` selects the CUDA kernels and ``xlstm/xlstm_large/model.py``
runs unchanged.

``install_slstm_backend()`` teaches ``xlstm.blocks.slstm.cell.sLSTMCell`` the backend name
``"b200"`` (the switch at ``cell.py:777-788``), so ``sLSTMLayerConfig(backend="b200")`` and
``xLSTMBlockStack`` run unchanged.

``pack_aware_slstm_layers(stack)`` swaps, in every sLSTM layer of a built model, the causal
convolution + SiLU in front of the cell for the kernel that knows document boundaries, and
``set_document_offsets(stack, cu_seqlens)`` hands the boundaries of a packed batch to those
convolutions and to the b200 cells behind them.
"""
from __future__ import annotations

import importlib
import importlib.util
import sys
import types

import torch

from . import backend_module, ops


def install_mlstm_backend() -> str:
    """Returns "shim" when this package now provides ``mlstm_kernels.torch.backend_module`` and
    "registered" when the b200 kernels were added to an installed upstream package."""
    existing = sys.modules.get("mlstm_kernels.torch.backend_module")
    if existing is backend_module:
        return "shim"
    if existing is None and importlib.util.find_spec("mlstm_kernels") is not None:
        # The upstream package is installed.  Its registries are keyed differently (module and function name split on
        # "--"), so the b200 names are only reported as registered once they resolve through upstream's own
        # config validation; otherwise this package's module takes the place of upstream's backend module.
        try:
            up = importlib.import_module("mlstm_kernels.torch")
            for attr, kind in (("_mlstm_chunkwise_kernel_registry", "chunkwise"), ("_mlstm_sequence_kernel_registry", "sequence"),
                               ("_mlstm_step_kernel_registry", "step")):
                reg = getattr(up, attr, None)
                if isinstance(reg, dict):
                    reg.update({n: f for n, f in backend_module._registry[kind].items() if "b200" in n})
            upbm = importlib.import_module("mlstm_kernels.torch.backend_module")
            upbm.mLSTMBackend(upbm.mLSTMBackendConfig(chunkwise_kernel="chunkwise--b200", sequence_kernel="native_sequence__b200",
                                                      step_kernel="b200", mode="inference"))
            return "registered"
        except Exception:
            sys.modules.pop("mlstm_kernels.torch.backend_module", None)
    pkg = types.ModuleType("mlstm_kernels")
    pkg.__path__ = []  # mark as package
    sub = types.ModuleType("mlstm_kernels.torch")
    sub.__path__ = []
    sub.backend_module = backend_module
    sub.get_available_mlstm_kernels = backend_module.get_available_mlstm_kernels
    sub.get_available_mlstm_step_kernels = backend_module.get_available_mlstm_step_kernels
    sub.get_available_mlstm_sequence_kernels = backend_module.get_available_mlstm_sequence_kernels
    pkg.torch = sub
    sys.modules["mlstm_kernels"] = pkg
    sys.modules["mlstm_kernels.torch"] = sub
    sys.modules["mlstm_kernels.torch.backend_module"] = backend_module
    return "shim"


_slstm_installed = False


def install_slstm_backend():
    """Adds backend="b200" to the reference's sLSTMCell switch and returns the new cell class."""
    global _slstm_installed
    cell_mod = importlib.import_module("xlstm.blocks.slstm.cell")
    if _slstm_installed:
        return cell_mod.sLSTMCell_b200

    class sLSTMCell_b200(cell_mod.sLSTMCellBase):
        """sLSTM cell on the persistent sm_100a kernel.  Parameters keep the reference's external layout
        (R: (NH, DH_in, 4, DH_out), bias: (NH, 4, DH); ``cell.py:234-261``), which is also what the kernel
        reads, so the four layout converters are the identity."""

        config_class = cell_mod.sLSTMCellConfig

        def __init__(self, config, skip_backend_init: bool = False):
            super().__init__(config)
            if config.function != "slstm":
                raise ValueError("the b200 backend implements function='slstm' only")
            self._cu_seqlens = None

        def set_document_offsets(self, cu_seqlens):
            """Document boundaries on the flattened (B*S) axis for the next forward calls (None to clear);
            h, c, n, m are reset inside the kernel at each boundary."""
            self._cu_seqlens = cu_seqlens

        def _cast_inputs(self, x, state):
            if self.config.input_shape != "BSGNH" or self.config.output_shape != "BNSH":
                raise ValueError("the b200 backend supports input_shape='BSGNH' and output_shape='BNSH'")
            wdt = self.config.torch_dtype_w
            if wdt != torch.bfloat16:
                raise ValueError("the b200 sLSTM kernel computes on bfloat16 inputs: use dtype='bfloat16'")
            R = self._recurrent_kernel_.reshape(self.config.num_heads, self.head_dim, self.config.num_gates, self.head_dim)
            b = self._bias_.reshape(self.config.num_heads, self.config.num_gates, self.head_dim)
            return x.to(wdt), R.to(wdt), b.float(), (None if state is None else state.float())

        def forward(self, input, state=None, lengths=None):
            self._check_input(input)
            if state is not None:
                assert state.shape == (self.config.num_states, input.shape[0], self.config.hidden_size)
            x, R, b, s0 = self._cast_inputs(input, state)
            if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (x, R, b, s0)):
                # training: the cache-writing forward with the backward-through-time kernel behind it
                # (sLSTMCellFunction, cell.py:543-598)
                if self._cu_seqlens is not None:
                    raise ValueError("the b200 sLSTM backward pass takes no document offsets")
                out, last = ops.SlstmFunction.apply(x, R, b, s0)
            else:
                out, last = ops.slstm_forward(x, R, b, s0, cu_seqlens=self._cu_seqlens)
            if torch.is_autocast_enabled():
                return out, last
            return out.to(input.dtype), last.to(input.dtype)

        def step(self, input, state):
            out, last = self.forward(input, state)
            return out, last

        def _impl(self, training, input, state):
            raise NotImplementedError("the b200 backend overrides forward(); it never materialises all states")

        _impl_step = _impl

    cell_mod.sLSTMCell_b200 = sLSTMCell_b200
    original_new = cell_mod.sLSTMCell.__new__

    def __new__(cls, config, skip_backend_init: bool = False):
        if config.backend == "b200":
            return sLSTMCell_b200(config, skip_backend_init=skip_backend_init)
        return original_new(cls, config, skip_backend_init=skip_backend_init)

    cell_mod.sLSTMCell.__new__ = staticmethod(__new__)
    _slstm_installed = True
    return sLSTMCell_b200


def _needs_grad(*tensors) -> bool:
    """True when autograd would record an operator on these tensors: the forward-only kernels then step aside for the
    reference's own differentiable operators."""
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


class PackAwareCausalConv1d(torch.nn.Module):
    """Stands in for the pair ``CausalConv1d`` + ``SiLU`` at the front of the reference's sLSTM layer
    (xlstm/blocks/slstm/layer.py:133-142).  It owns the SAME ``nn.Conv1d`` parameters (state dicts stay compatible) and
    computes convolution and activation in one kernel; with document offsets set, no tap reaches across a document
    boundary -- the reference's module pads per batch row only (xlstm/components/conv.py:110-129), so in a packed row
    it mixes the last tokens of one document into the first tokens of the next although the cell restarts there.
    Single-token ``step`` calls go to the reference module (the activation is applied here, since the layer's own
    activation module is replaced by an identity)."""

    def __init__(self, reference_conv):
        super().__init__()
        self.ref = reference_conv
        self.config = reference_conv.config
        self._cu_seqlens = None

    def set_document_offsets(self, cu_seqlens):
        self._cu_seqlens = cu_seqlens

    def reset_parameters(self, **kwargs):
        self.ref.reset_parameters(**kwargs)

    def forward(self, x, conv_state=None, return_last_state: bool = False):
        if self.config.kernel_size == 0:
            return x
        if _needs_grad(x, conv_state, self.ref.conv.weight, self.ref.conv.bias):
            # training: the reference's module (the kernel has no backward pass)
            if self._cu_seqlens is not None:
                raise ValueError("the convolution kernel with document offsets is forward only")
            if return_last_state:
                y, state = self.ref(x, conv_state, return_last_state=True)
                return torch.nn.functional.silu(y), state
            return torch.nn.functional.silu(self.ref(x, conv_state, return_last_state=False))
        if conv_state is not None:
            if self._cu_seqlens is not None:
                raise ValueError("a packed batch starts every document from an empty convolution state")
            xx = torch.cat([conv_state, x], dim=1)
            y = ops.causal_conv1d(xx, self.ref.conv.weight, self.ref.conv.bias, silu=True)[:, conv_state.shape[1]:]
        else:
            y = ops.causal_conv1d(x, self.ref.conv.weight, self.ref.conv.bias, cu_seqlens=self._cu_seqlens, silu=True)
        if return_last_state:
            full = x if conv_state is None else torch.cat([conv_state, x], dim=1)
            return y, full[:, -(self.config.kernel_size - 1):]
        return y

    def step(self, x, conv_state=None):
        y, state = self.ref.step(x, conv_state=conv_state)
        return torch.nn.functional.silu(y), state


class HeadGroupNorm(torch.nn.Module):
    """Stands in for the ``MultiHeadLayerNorm`` behind the sLSTM cell (xlstm/blocks/slstm/layer.py:157;
    xlstm/components/ln.py:52-68): the per-head group norm of the cell output in one kernel that reads the cell's
    (B, NH, S, DH) layout through its strides and writes (B, S, NH*DH) -- the transposes on either side of the reference
    module become views.  It owns the same parameters (``weight`` is the reference's residual weight; 1 + weight is
    applied), eps included."""

    def __init__(self, reference_norm):
        super().__init__()
        if reference_norm.bias is not None:
            raise ValueError("the kernel covers the bias-free norm the sLSTM layer builds")
        self.ref = reference_norm

    def reset_parameters(self):
        self.ref.reset_parameters()

    def forward(self, x):
        B, NH, S, DH = x.shape
        w = self.ref.weight_proxy
        if _needs_grad(x, w):
            return self.ref(x)      # training: the reference's module (the kernel has no backward pass)
        w = torch.ones(NH * DH, dtype=x.dtype, device=x.device) if w is None else w.to(x.dtype)
        out = ops.headnorm_gate(x, None, w, eps=self.ref.eps)            # (B, S, NH*DH)
        return out.view(B, S, NH, DH).transpose(1, 2)                   # the caller transposes back and flattens: views


def _slstm_layer_forward_fused(self, x, conv_state=None, slstm_state=None, return_last_state=False, **kwargs):
    """``sLSTMLayer.forward`` (xlstm/blocks/slstm/layer.py:123-162) with the four headwise gate projections and their
    concatenation done by ONE kernel that writes the cell's (B, S, 4, NH, DH) input directly (`xl_headwise_proj`); every
    other step calls the layer's own sub-modules as the reference does."""
    B, S, _ = x.shape
    if self.config.conv1d_kernel_size > 0:
        if return_last_state:
            x_conv, conv_state = self.conv1d(x, conv_state, return_last_state=True)
        else:
            x_conv = self.conv1d(x, conv_state, return_last_state=False)
        x_conv = self.conv_act_fn(x_conv)
    else:
        x_conv = x
    gates = (self.fgate, self.igate, self.zgate, self.ogate)   # the order in which the reference concatenates them
    DH = gates[0].weight.shape[-1]
    fusable = (x.is_cuda and x.dtype == torch.bfloat16 and DH in (64, 128, 256)
               and not _needs_grad(x, x_conv, *(g.weight for g in gates))     # forward-only kernel
               and all(g.bias is None and g.weight.shape[1] == DH and g.weight.dtype == torch.bfloat16 for g in gates))
    if fusable:
        wx = ops.headwise_proj([x, x_conv], [g.weight for g in gates], [1, 1, 0, 0])
    else:
        wx = torch.cat([self.fgate(x_conv), self.igate(x_conv), self.zgate(x), self.ogate(x)], dim=-1)
    y, slstm_state = self.slstm_cell(wx, state=slstm_state)
    y = self.dropout(y)
    out = self.group_norm(y).transpose(1, 2).view(B, S, -1)
    if return_last_state:
        return out, {"conv_state": conv_state, "slstm_state": slstm_state}
    return out


def fuse_slstm_gate_projections(model) -> int:
    """Gives every ``sLSTMLayer`` instance below `model` a forward that computes its four gate projections with one
    kernel (the class and its parameters are untouched: state dicts load and save as before); returns how many."""
    layer_mod = importlib.import_module("xlstm.blocks.slstm.layer")
    n = 0
    for m in model.modules():
        if isinstance(m, layer_mod.sLSTMLayer) and "forward" not in m.__dict__:
            m.forward = types.MethodType(_slstm_layer_forward_fused, m)
            n += 1
    return n


def pack_aware_slstm_layers(model) -> int:
    """Replaces conv1d + conv_act_fn in front of the cell, and the group norm behind it, in every ``sLSTMLayer`` below
    `model`; returns how many layers were changed."""
    layer_mod = importlib.import_module("xlstm.blocks.slstm.layer")
    n = 0
    for m in model.modules():
        if isinstance(m, layer_mod.sLSTMLayer) and not isinstance(m.group_norm, HeadGroupNorm):
            if m.config.conv1d_kernel_size > 0:
                m.conv1d = PackAwareCausalConv1d(m.conv1d)
                m.conv_act_fn = torch.nn.Identity()
            if m.group_norm.bias is None:
                m.group_norm = HeadGroupNorm(m.group_norm)
            n += 1
    return n


def set_document_offsets(model, cu_seqlens) -> None:
    """Document boundaries (offsets on the flattened (B*S) token axis, or None to clear) for every pack-aware
    convolution and every b200 sLSTM cell below `model`."""
    for m in model.modules():
        if isinstance(m, PackAwareCausalConv1d) or type(m).__name__ == "sLSTMCell_b200":
            m.set_document_offsets(cu_seqlens)
