"""Generate ``headwise.npz`` from the REFERENCE's own ``LinearHeadwiseExpand`` modules, used the way
``sLSTMLayer.forward`` uses them (xlstm/blocks/slstm/layer.py:145-154): four bias-free projections, the first two of the
convolved input and the last two of the plain one, concatenated.  Arrays hold bfloat16 bit patterns (uint16).

    python tests/golden/make_golden_headwise.py /path/to/reference
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    spec = importlib.util.spec_from_file_location("ref_lhw", os.path.join(ref_root, "xlstm", "components", "linear_headwise.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = {}
    for tag, (B, S, NH, DH) in (("a", (2, 37, 4, 64)), ("b", (1, 70, 1, 128))):
        torch.manual_seed(11)
        D = NH * DH
        gates = [mod.LinearHeadwiseExpand(mod.LinearHeadwiseExpandConfig(in_features=D, num_heads=NH, bias=False)).bfloat16()
                 for _ in range(4)]
        with torch.no_grad():
            for g in gates:
                g.weight.copy_((torch.randn(NH, DH, DH) / DH ** 0.5).bfloat16())
        x = torch.randn(B, S, D).bfloat16()
        xc = torch.randn(B, S, D).bfloat16()
        with torch.no_grad():
            y = torch.cat([gates[0](xc), gates[1](xc), gates[2](x), gates[3](x)], dim=-1)
        bits = lambda t: t.detach().contiguous().view(torch.int16).numpy().view(np.uint16)   # bf16 bit patterns: half the bytes
        out.update({f"{tag}_x": bits(x), f"{tag}_xc": bits(xc), f"{tag}_y": bits(y)})
        for i, g in enumerate(gates):
            out[f"{tag}_w{i}"] = bits(g.weight)
    np.savez_compressed(os.path.join(HERE, "headwise.npz"), **out)
    print("wrote headwise.npz with", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["XLSTM_REFERENCE"])
