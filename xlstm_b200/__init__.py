"""xlstm_b200: sm_100a kernels for xLSTM's recurrent cells behind the reference's selector API."""
from .ops import check_device_status, mlstm_sequence, mlstm_sequence_from_host, mlstm_step, slstm_forward  # noqa: F401

__all__ = ["mlstm_sequence", "mlstm_sequence_from_host", "mlstm_step", "slstm_forward", "check_device_status"]
