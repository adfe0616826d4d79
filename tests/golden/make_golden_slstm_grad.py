"""Gradient fixtures for the sLSTM cell from the REFERENCE's vanilla backend (plain PyTorch, differentiated by autograd).

    python tests/golden/make_golden_slstm_grad.py [/path/to/reference]     (default: $XLSTM_REFERENCE)

Writes ``slstm_grad.npz`` / ``slstm_grad_state.npz``: inputs, the loss weights, and the gradients of
``sum(out * gh) + sum(last_h * gl)`` with respect to wx, the recurrent matrix and the bias (both in the cell's external
layouts) and the initial h, c, n.  The loss reads h only: the reference's own backward kernel gives the stabiliser
state no gradient, and a loss on h does not depend on it.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    sys.path.insert(0, ref_root)
    from xlstm.blocks.slstm.cell import sLSTMCell, sLSTMCellConfig

    def case(seed, hidden, heads, B, S, with_state):
        torch.manual_seed(seed)
        cfg = sLSTMCellConfig(hidden_size=hidden, num_heads=heads, backend="vanilla", recurrent_weight_init="standard",
                              bias_init="standard", dtype="float32")
        cell = sLSTMCell(cfg).float()
        wx = torch.randn(B, S, 4 * hidden, requires_grad=True)
        st = None
        if with_state:
            st = torch.randn(4, B, hidden)
            st[2] = st[2].abs() + 0.5
            st.requires_grad_()
        out, last = cell(wx, st)
        gh = torch.randn_like(out)
        gl = torch.randn_like(last[0])
        loss = (out * gh).sum() + (last[0] * gl).sum()
        loss.backward()
        d = dict(wx=wx.detach(), gh=gh, gl=gl, out=out.detach(),
                 R=cell._recurrent_kernel_int2ext(cell._recurrent_kernel_.data),
                 bias=cell._bias_int2ext(cell._bias_.data),
                 dwx=wx.grad, dR=cell._recurrent_kernel_int2ext(cell._recurrent_kernel_.grad),
                 dbias=cell._bias_int2ext(cell._bias_.grad))
        if st is not None:
            d["state0"] = st.detach()
            d["dstate0"] = st.grad
        return {k: v.detach().float().numpy() for k, v in d.items()}

    for name, d in (("slstm_grad", case(51, 64, 4, 3, 24, False)), ("slstm_grad_state", case(52, 128, 2, 2, 17, True))):
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)
        print(name, {k: v.shape for k, v in d.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["XLSTM_REFERENCE"])
