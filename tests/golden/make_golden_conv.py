"""Generate ``conv.npz`` from the REFERENCE's own ``CausalConv1d`` module followed by ``nn.SiLU`` (the front of
``sLSTMLayer.forward``, xlstm/blocks/slstm/layer.py:133-142).

    python tests/golden/make_golden_conv.py /path/to/reference

Two cases per dtype: plain rows, and rows packed from several documents, for which the reference module is run ONCE
PER DOCUMENT (its own padding then is the document's) and the pieces are put back together.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CU = [0, 5, 5, 30, 48, 48 + 1, 48 + 4, 96]   # two rows of 48 tokens: documents of 5, 0, 25, 18 | 1, 3, 44 tokens


def main(ref_root):
    spec = importlib.util.spec_from_file_location("ref_conv", os.path.join(ref_root, "xlstm", "components", "conv.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = {"cu": np.array(CU, dtype=np.int64)}
    act = torch.nn.SiLU()
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        torch.manual_seed(7)
        B, S, F_, K = 2, 48, 64, 4
        conv = mod.CausalConv1d(mod.CausalConv1dConfig(feature_dim=F_, kernel_size=K)).to(dt)
        with torch.no_grad():
            conv.conv.weight.copy_(torch.randn(F_, 1, K).to(dt))
            conv.conv.bias.copy_((0.5 * torch.randn(F_)).to(dt))
        x = (2.0 * torch.randn(B, S, F_)).to(dt)
        with torch.no_grad():
            rows = act(conv(x))
            flat = x.reshape(1, B * S, F_)
            pieces = [act(conv(flat[:, a:e])) for a, e in zip(CU[:-1], CU[1:]) if e > a]
            packed = torch.cat(pieces, dim=1).reshape(B, S, F_)
        out.update({f"{tag}_x": x.float().numpy(), f"{tag}_w": conv.conv.weight[:, 0, :].detach().float().numpy(),
                    f"{tag}_b": conv.conv.bias.detach().float().numpy(), f"{tag}_rows": rows.float().numpy(),
                    f"{tag}_packed": packed.float().numpy()})
    np.savez_compressed(os.path.join(HERE, "conv.npz"), **out)
    print("wrote conv.npz with", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["XLSTM_REFERENCE"])
