"""xlstm_b200: sm_100a kernels for xLSTM's recurrent cells behind the reference's selector API."""
from .ops import (add_rmsnorm, causal_conv1d, check_device_status, headnorm_gate, headwise_proj, mlstm_sequence, mlstm_sequence_from_host,  # noqa: F401
                  mlstm_step, slstm_forward, soft_cap, softcap_argmax, swiglu)

__all__ = ["mlstm_sequence", "mlstm_sequence_from_host", "mlstm_step", "slstm_forward", "add_rmsnorm", "headnorm_gate", "soft_cap", "causal_conv1d", "softcap_argmax", "swiglu", "headwise_proj",
           "check_device_status"]
