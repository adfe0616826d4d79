"""ctypes binding of the C-ABI library declared in include/xlstm_b200.h.

There is deliberately no fallback: if the shared library is missing or a call
fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libxlstm_b200.so")

XL_F32, XL_BF16 = 0, 1

EXPORTS = (
    "xl_strerror", "xl_last_cuda_error", "xl_abi_version",
    "xl_mlstm_chunkwise", "xl_mlstm_recurrent", "xl_mlstm_step", "xl_slstm_forward",
    "xl_add_rmsnorm", "xl_headnorm_gate", "xl_soft_cap", "xl_causal_conv1d",
    "xl_softcap_argmax", "xl_softcap_argmax_scratch_bytes", "xl_swiglu",
    "xl_softcap_argmax_noalloc", "xl_softcap_argmax_noalloc_max_rows", "xl_peer_reduce_add_rmsnorm", "xl_headwise_proj", "xl_mlstm_decode_cell",
    "xl_slstm_backward", "xl_slstm_cache_bytes",
)


class MlstmSeqParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("h", C.c_void_p),
        ("igate", C.c_void_p), ("fgate", C.c_void_p),
        ("c0", C.c_void_p), ("n0", C.c_void_p), ("m0", C.c_void_p),
        ("c_out", C.c_void_p), ("n_out", C.c_void_p), ("m_out", C.c_void_p),
        ("cu_seqlens", C.c_void_p), ("status", C.c_void_p),
        ("B", C.c_int32), ("NH", C.c_int32), ("S", C.c_int32), ("DHQK", C.c_int32), ("DHV", C.c_int32),
        ("num_docs", C.c_int32),
        ("q_sb", C.c_int64), ("q_sh", C.c_int64), ("q_st", C.c_int64),
        ("k_sb", C.c_int64), ("k_sh", C.c_int64), ("k_st", C.c_int64),
        ("v_sb", C.c_int64), ("v_sh", C.c_int64), ("v_st", C.c_int64),
        ("h_sb", C.c_int64), ("h_sh", C.c_int64), ("h_st", C.c_int64),
        ("g_sb", C.c_int64), ("g_sh", C.c_int64), ("g_st", C.c_int64),
        ("eps", C.c_float), ("dtype", C.c_int32),
    ]


class MlstmStepParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("h", C.c_void_p),
        ("igate", C.c_void_p), ("fgate", C.c_void_p),
        ("c_in", C.c_void_p), ("n_in", C.c_void_p), ("m_in", C.c_void_p),
        ("c_out", C.c_void_p), ("n_out", C.c_void_p), ("m_out", C.c_void_p),
        ("slot", C.c_void_p), ("status", C.c_void_p),
        ("B", C.c_int32), ("NH", C.c_int32), ("DHQK", C.c_int32), ("DHV", C.c_int32), ("n_slots", C.c_int32),
        ("q_sb", C.c_int64), ("q_sh", C.c_int64), ("k_sb", C.c_int64), ("k_sh", C.c_int64),
        ("v_sb", C.c_int64), ("v_sh", C.c_int64), ("h_sb", C.c_int64), ("h_sh", C.c_int64),
        ("g_sb", C.c_int64), ("g_sh", C.c_int64),
        ("eps", C.c_float), ("dtype", C.c_int32),
    ]


class SlstmParams(C.Structure):
    _fields_ = [
        ("wx", C.c_void_p), ("R", C.c_void_p), ("bias", C.c_void_p), ("state0", C.c_void_p),
        ("h_out", C.c_void_p), ("state_out", C.c_void_p), ("cu_seqlens", C.c_void_p), ("status", C.c_void_p),
        ("B", C.c_int32), ("S", C.c_int32), ("NH", C.c_int32), ("DH", C.c_int32),
        ("num_docs", C.c_int32), ("dtype", C.c_int32), ("train_cache", C.c_void_p),
    ]


class SlstmBwdParams(C.Structure):
    _fields_ = [
        ("cache", C.c_void_p), ("R", C.c_void_p), ("dh", C.c_void_p), ("dstate_out", C.c_void_p),
        ("state0", C.c_void_p), ("dwx", C.c_void_p), ("dstate0", C.c_void_p), ("status", C.c_void_p),
        ("B", C.c_int32), ("S", C.c_int32), ("NH", C.c_int32), ("DH", C.c_int32), ("dtype", C.c_int32),
    ]


class AddRmsnormParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("y", C.c_void_p), ("weight", C.c_void_p), ("x_out", C.c_void_p), ("normed", C.c_void_p),
        ("rows", C.c_int64), ("D", C.c_int32),
        ("x_sr", C.c_int64), ("y_sr", C.c_int64), ("xo_sr", C.c_int64), ("n_sr", C.c_int64),
        ("eps", C.c_float), ("dtype", C.c_int32),
    ]


class HeadnormGateParams(C.Structure):
    _fields_ = [
        ("h", C.c_void_p), ("o", C.c_void_p), ("weight", C.c_void_p), ("out", C.c_void_p),
        ("B", C.c_int32), ("NH", C.c_int32), ("S", C.c_int32), ("DH", C.c_int32),
        ("h_sb", C.c_int64), ("h_sh", C.c_int64), ("h_st", C.c_int64), ("o_sb", C.c_int64), ("o_st", C.c_int64),
        ("eps", C.c_float), ("dtype", C.c_int32),
    ]


class SoftCapParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("out", C.c_void_p), ("n", C.c_int64), ("cap", C.c_float), ("dtype", C.c_int32),
                ("out_f32", C.c_int32), ("cols", C.c_int64), ("x_row_stride", C.c_int64), ("bias", C.c_void_p)]


class SwigluParams(C.Structure):
    _fields_ = [("gz", C.c_void_p), ("out", C.c_void_p), ("rows", C.c_int64), ("F", C.c_int32), ("gz_row_stride", C.c_int64),
                ("dtype", C.c_int32)]


class Conv1dParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("weight", C.c_void_p), ("bias", C.c_void_p), ("out", C.c_void_p), ("cu_seqlens", C.c_void_p),
        ("B", C.c_int32), ("S", C.c_int32), ("F", C.c_int32), ("K", C.c_int32), ("num_docs", C.c_int32), ("act", C.c_int32),
        ("x_sb", C.c_int64), ("x_st", C.c_int64), ("o_sb", C.c_int64), ("o_st", C.c_int64),
        ("dtype", C.c_int32),
    ]


class MlstmDecodeCellParams(C.Structure):
    _fields_ = [
        ("step", MlstmStepParams),
        ("gates_raw", C.c_void_p), ("gate_bias", C.c_void_p), ("ogate", C.c_void_p), ("norm_weight", C.c_void_p), ("hg", C.c_void_p),
        ("gr_sb", C.c_int64), ("o_sb", C.c_int64), ("hg_sb", C.c_int64),
        ("gate_cap", C.c_float), ("norm_eps", C.c_float),
    ]


class HeadwiseParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p * 2), ("w", C.c_void_p * 4), ("out", C.c_void_p), ("status", C.c_void_p),
        ("in_sel", C.c_int32 * 4),
        ("rows", C.c_int64), ("NH", C.c_int32), ("DH", C.c_int32), ("n_slots", C.c_int32), ("dtype", C.c_int32),
        ("x_row_stride", C.c_int64 * 2), ("out_row_stride", C.c_int64),
    ]


class GreedyParams(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("tokens", C.c_void_p), ("scratch", C.c_void_p), ("scratch_bytes", C.c_int64),
        ("rows", C.c_int32), ("V", C.c_int32), ("row_stride", C.c_int64), ("cap", C.c_float), ("dtype", C.c_int32),
    ]


class PeerReduceParams(C.Structure):
    _fields_ = [
        ("partial", C.c_void_p), ("peer_recv", C.c_void_p), ("recv_local", C.c_void_p), ("peer_flags", C.c_void_p),
        ("flags_local", C.c_void_p), ("epoch", C.c_void_p), ("x", C.c_void_p), ("weight", C.c_void_p), ("x_out", C.c_void_p),
        ("normed", C.c_void_p), ("status", C.c_void_p),
        ("rank", C.c_int32), ("world", C.c_int32), ("rows", C.c_int32), ("D", C.c_int32), ("rows_max", C.c_int32),
        ("partial_sr", C.c_int64), ("x_sr", C.c_int64), ("xo_sr", C.c_int64), ("n_sr", C.c_int64),
        ("eps", C.c_float), ("dtype", C.c_int32),
    ]


_lib = None


def lib() -> C.CDLL:
    """Load (once) and return the library; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m xlstm_b200.build` "
                "(there is no fallback implementation)")
        l = C.CDLL(LIB_PATH)
        l.xl_strerror.restype = C.c_char_p
        l.xl_strerror.argtypes = [C.c_int]
        l.xl_last_cuda_error.restype = C.c_char_p
        l.xl_abi_version.restype = C.c_int
        for name, ptype in (("xl_mlstm_chunkwise", MlstmSeqParams), ("xl_mlstm_recurrent", MlstmSeqParams),
                            ("xl_mlstm_step", MlstmStepParams), ("xl_slstm_forward", SlstmParams),
                            ("xl_add_rmsnorm", AddRmsnormParams), ("xl_headnorm_gate", HeadnormGateParams),
                            ("xl_soft_cap", SoftCapParams), ("xl_causal_conv1d", Conv1dParams),
                            ("xl_softcap_argmax", GreedyParams), ("xl_swiglu", SwigluParams),
                            ("xl_softcap_argmax_noalloc", GreedyParams), ("xl_peer_reduce_add_rmsnorm", PeerReduceParams),
                            ("xl_slstm_backward", SlstmBwdParams)):
            fn = getattr(l, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(ptype), C.c_void_p]
        l.xl_softcap_argmax_scratch_bytes.restype = C.c_int64
        l.xl_softcap_argmax_scratch_bytes.argtypes = [C.c_int32]
        l.xl_softcap_argmax_noalloc_max_rows.restype = C.c_int32
        l.xl_slstm_cache_bytes.restype = C.c_int64
        l.xl_slstm_cache_bytes.argtypes = [C.c_int32] * 4
        _lib = l
    return _lib


class XlError(RuntimeError):
    def __init__(self, code: int, where: str):
        l = lib()
        msg = l.xl_strerror(code).decode()
        if code == -7:
            msg += ": " + l.xl_last_cuda_error().decode()
        super().__init__(f"{where} failed with status {code}: {msg}")
        self.code = code


def check(code: int, where: str) -> None:
    if code != 0:
        raise XlError(code, where)
