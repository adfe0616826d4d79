"""Generate the golden fixtures in this directory from the REFERENCE's own code.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's pure-PyTorch implementations
(``xlstm/blocks/mlstm/backends.py`` and the vanilla sLSTM cell), feeds them
seeded inputs and stores inputs + outputs as small ``.npz`` files.  A third,
independent implementation (the native fallback inside the installed
``transformers`` package, which supports DHQK != DHV) is recorded as a
cross-check.  The fixtures are what pins the CPU oracle; the GPU tests never
need the reference checkout.
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(**kw):
    return {k: (v.detach().cpu().numpy() if torch.is_tensor(v) else np.asarray(v)) for k, v in kw.items()}


def mlstm_inputs(seed, B, NH, S, DHQK, DHV, f_mean=3.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, NH, S, DHQK, generator=g)
    k = torch.randn(B, NH, S, DHQK, generator=g)
    v = torch.randn(B, NH, S, DHV, generator=g)
    i = torch.randn(B, NH, S, generator=g)
    f = torch.randn(B, NH, S, generator=g) + f_mean
    return q, k, v, i, f


def hf_cross_check():
    # must run BEFORE the reference is put on sys.path (transformers probes for an `xlstm` package)
    import transformers.models.xlstm.modeling_xlstm as M
    out = {}
    q, k, v, i, f = mlstm_inputs(11, 1, 2, 192, 32, 64)
    h, (c, n, m) = M.mlstm_chunkwise_native_autograd(q, k, v, i, f, chunk_size=64, return_last_states=True)
    out["chunk"] = _np(q=q, k=k, v=v, i=i, f=f, h=h, c=c, n=n, m=m)
    # recurrent sequence with an initial state
    g = torch.Generator().manual_seed(12)
    c0 = torch.randn(1, 2, 32, 64, generator=g); n0 = torch.randn(1, 2, 32, generator=g); m0 = torch.randn(1, 2, 1, generator=g)
    q, k, v, i, f = mlstm_inputs(13, 1, 2, 37, 32, 64, f_mean=1.0)
    h, (c, n, m) = M.mlstm_recurrent_sequence_native(q, k, v, i, f, c_initial=c0, n_initial=n0, m_initial=m0,
                                                      return_last_states=True)
    out["seq"] = _np(q=q, k=k, v=v, i=i, f=f, c0=c0, n0=n0, m0=m0, h=h, c=c, n=n, m=m)
    return out


def main(ref_root):
    hf = None
    try:
        hf = hf_cross_check()
    except Exception as e:  # cross-check only; the reference fixtures below are the pin
        print("transformers cross-check unavailable:", repr(e))
    sys.path.insert(0, ref_root)
    from xlstm.blocks.mlstm.backends import chunkwise_simple, recurrent_step_stabilized_simple
    from xlstm.blocks.slstm.cell import sLSTMCell, sLSTMCellConfig

    fx = {}
    # ---- mLSTM chunkwise, zero initial state (reference needs DHQK == DHV)
    q, k, v, i, f = mlstm_inputs(1, 2, 2, 128, 32, 32)
    h, (c, n, m) = chunkwise_simple(q, k, v, i, f, chunk_size=64, return_last_state=True)
    fx["mlstm_chunk_zero"] = _np(q=q, k=k, v=v, i=i, f=f, h=h, c=c, n=n, m=m[..., 0, 0])
    # ---- with an initial state and harsher forget gates
    q, k, v, i, f = mlstm_inputs(2, 1, 3, 192, 16, 16, f_mean=0.0)
    g = torch.Generator().manual_seed(3)
    c0 = torch.randn(1, 3, 16, 16, generator=g); n0 = torch.randn(1, 3, 16, generator=g); m0 = torch.randn(1, 3, 1, generator=g)
    h, (c, n, m) = chunkwise_simple(q, k, v, i, f, initial_C=c0, initial_n=n0, initial_m=m0[..., 0], chunk_size=64,
                                    return_last_state=True)
    fx["mlstm_chunk_init"] = _np(q=q, k=k, v=v, i=i, f=f, c0=c0, n0=n0, m0=m0, h=h, c=c, n=n, m=m[..., 0, 0])
    # ---- recurrent step chain (reference scales k, not q: C and n carry 1/sqrt(DH))
    q, k, v, i, f = mlstm_inputs(4, 2, 2, 20, 32, 32, f_mean=1.0)
    DH = 32
    c = torch.zeros(2, 2, DH, DH); n = torch.zeros(2, 2, DH, 1); m = torch.zeros(2, 2, 1, 1)
    hs = []
    for t in range(20):
        h, (c, n, m) = recurrent_step_stabilized_simple(
            c, n, m, q[:, :, t:t + 1].clone(), k[:, :, t:t + 1].clone(), v[:, :, t:t + 1].clone(),
            i[:, :, t, None, None], f[:, :, t, None, None])
        hs.append(h)
    fx["mlstm_step_chain"] = _np(q=q, k=k, v=v, i=i, f=f, h=torch.cat(hs, dim=2), c_kscaled=c, n_kscaled=n[..., 0],
                                 m=m[..., 0, 0])
    if hf is not None:
        for name, d in hf.items():
            fx["hf_" + name] = d

    # ---- sLSTM vanilla cell
    def slstm_case(seed, hidden, heads, B, S, with_state, dtype=torch.float32):
        torch.manual_seed(seed)
        cfg = sLSTMCellConfig(hidden_size=hidden, num_heads=heads, backend="vanilla",
                              recurrent_weight_init="standard", bias_init="standard",
                              dtype="float32" if dtype == torch.float32 else "bfloat16")
        cell = sLSTMCell(cfg).to(dtype)
        wx = torch.randn(B, S, 4 * hidden).to(dtype)
        st = (torch.randn(4, B, hidden).to(dtype)) if with_state else None
        if st is not None:
            st[2] = st[2].abs() + 0.5  # a normaliser state is positive
        with torch.no_grad():
            out, last = cell(wx, st)
        R_ext = cell.recurrent_kernel.data if hasattr(cell.recurrent_kernel, "data") else cell.recurrent_kernel[...]
        b_ext = cell.bias.data if hasattr(cell.bias, "data") else cell.bias[...]
        d = dict(wx=wx.float(), out=out.float(), last=last.float(),
                 R=cell._recurrent_kernel_int2ext(cell._recurrent_kernel_.data).float(),
                 bias=cell._bias_int2ext(cell._bias_.data).float())
        if st is not None:
            d["state0"] = st.float()
        return _np(**d)

    fx["slstm_zero"] = slstm_case(42, 64, 4, 3, 24, False)
    fx["slstm_state"] = slstm_case(43, 64, 4, 2, 17, True)
    fx["slstm_b1s1"] = slstm_case(42, 64, 4, 1, 1, False)
    fx["slstm_bf16"] = slstm_case(44, 128, 2, 4, 32, False, dtype=torch.bfloat16)

    for name, d in fx.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)
        print(name, {k: v.shape for k, v in d.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["XLSTM_REFERENCE"])
