"""Generate ``layer_ops.npz`` from the REFERENCE's own norm modules.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden_layer.py /path/to/reference

It imports ``xlstm/xlstm_large/components.py`` (RMSNorm, MultiHeadLayerNorm, soft_cap), feeds seeded inputs in fp32 and
bf16 and stores inputs and outputs (bf16 tensors as their fp32 images, which is exact).  The residual add and the
output gate are the eager expressions of ``xlstm/xlstm_large/model.py:445-449, 499-510``.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    spec = importlib.util.spec_from_file_location("ref_components", os.path.join(ref_root, "xlstm", "xlstm_large", "components.py"))
    comp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(comp)
    out = {}
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        g = torch.Generator().manual_seed(5)
        # residual add + RMSNorm
        rows, D = 6, 512
        x = (2.0 * torch.randn(rows, D, generator=g)).to(dt)
        y = torch.randn(rows, D, generator=g).to(dt)
        w = (1.0 + 0.1 * torch.randn(D, generator=g)).to(dt)
        norm = comp.RMSNorm(num_features=D, eps=1e-6, use_weight=True, use_bias=False, force_float32_reductions=True)
        with torch.no_grad():
            norm.weight.copy_(w.float())
        norm = norm.to(dt)
        xn = x + y
        with torch.no_grad():
            normed = norm(xn)
        out.update({f"rms_{tag}_x": x.float().numpy(), f"rms_{tag}_y": y.float().numpy(), f"rms_{tag}_w": w.float().numpy(),
                    f"rms_{tag}_xnew": xn.float().numpy(), f"rms_{tag}_normed": normed.float().numpy()})
        # per-head LayerNorm + output gate
        B, NH, S, DH = 2, 4, 5, 128
        h = (3.0 * torch.randn(B, NH, S, DH, generator=g) + 0.5).to(dt)
        o = (2.0 * torch.randn(B, S, NH * DH, generator=g)).to(dt)
        w2 = (1.0 + 0.1 * torch.randn(NH * DH, generator=g)).to(dt)
        mh = comp.MultiHeadLayerNorm(num_heads=NH, head_dim=DH, eps=1e-6, use_weight=True, use_bias=False,
                                     force_float32_reductions=True)
        with torch.no_grad():
            mh.weight.copy_(w2.float())
        mh = mh.to(dt)
        with torch.no_grad():
            h_norm = mh(h.transpose(1, 2)).reshape(B, S, -1)
            gated = torch.sigmoid(o) * h_norm
        out.update({f"hng_{tag}_h": h.float().numpy(), f"hng_{tag}_o": o.float().numpy(), f"hng_{tag}_w": w2.float().numpy(),
                    f"hng_{tag}_out": gated.float().numpy()})
        # soft cap (gate pre-activations use 15, logits 30)
        v = (20.0 * torch.randn(4, 333, generator=g)).to(dt)
        out.update({f"cap_{tag}_x": v.float().numpy(), f"cap_{tag}_15": comp.soft_cap(v, 15.0).float().numpy(),
                    f"cap_{tag}_30": comp.soft_cap(v, 30.0).float().numpy()})
    np.savez_compressed(os.path.join(HERE, "layer_ops.npz"), **out)
    print("wrote layer_ops.npz with", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["XLSTM_REFERENCE"])
