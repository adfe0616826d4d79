"""Golden outputs of the REFERENCE xLSTMLarge model (xlstm/xlstm_large/model.py, unchanged) for the small
CPU-runnable configuration: embedding_dim=512, num_heads=4, num_blocks=6, vocab_size=2048, fp32, inference mode with the native
kernel triple (served by the CPU oracle through the drop-in backend module), input ids (3,256), then 32 greedy
tokens.  Weights are procedural (xlstm_b200.large_model.procedural_state_dict, seed 0) so that no checkpoint has
to be shipped.

    python tests/golden/make_golden_model.py /path/to/reference
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main(ref_root):
    from xlstm_b200.integration import install_mlstm_backend
    from xlstm_b200.large_model import LargeConfig, procedural_state_dict
    install_mlstm_backend()
    from test_boundary_cpu import _register_native_oracle
    _register_native_oracle()
    sys.path.insert(0, ref_root)
    from xlstm.xlstm_large.model import xLSTMLarge, xLSTMLargeConfig

    cfg = LargeConfig(embedding_dim=512, num_heads=4, num_blocks=6, vocab_size=2048)
    sd = procedural_state_dict(cfg, seed=0)
    ref = xLSTMLarge(xLSTMLargeConfig(embedding_dim=512, num_heads=4, num_blocks=6, vocab_size=2048, mode="inference",
                                      return_last_states=True, chunkwise_kernel="chunkwise--native_autograd",
                                      sequence_kernel="native_sequence__native", step_kernel="native")).eval()
    missing = ref.load_state_dict(sd, strict=True)
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, 2048, (3, 256), generator=g)
    with torch.no_grad():
        logits, state = ref(tokens)
        gen, _ = ref.generate(tokens, max_length=32)
    out = dict(tokens=tokens.numpy(), logits_last=logits[:, -1].numpy(), logits_sub=logits[:, ::37, ::16].numpy(),
               c5=state[5][0].numpy(), n5=state[5][1].numpy(), m5=state[5][2].numpy(), generated=gen.numpy())
    np.savez_compressed(os.path.join(HERE, "model_config1.npz"), **out)
    print({k: v.shape for k, v in out.items()}, missing)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["XLSTM_REFERENCE"])
