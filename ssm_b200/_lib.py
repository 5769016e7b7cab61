"""ctypes binding of ``libssm_b200.so`` (declarations mirror ``include/ssm_b200.h``).

There is no fallback: if the shared library is missing or an entry point is absent the
import of the operators fails with a clear error, and every call that the library rejects
raises.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libssm_b200.so"

F32, BF16, F16 = 0, 1, 2
ABI_VERSION = 3  # SSM_B200_ABI_VERSION of include/ssm_b200.h this binding mirrors
i32, i64, vp, fp = C.c_int32, C.c_int64, C.c_void_p, C.c_void_p


class ScanFwdArgs(C.Structure):
    _fields_ = [
        ("batch", i32), ("dim", i32), ("len", i32), ("nstate", i32),
        ("io_dtype", i32), ("bc_dtype", i32), ("last_dtype", i32), ("delta_softplus", i32),
        ("u", vp), ("delta", vp), ("z", vp), ("A", fp), ("Bm", vp), ("Cm", vp),
        ("bc_groups", i32), ("reserved0", i32),
        ("b_sb", i64), ("b_sg", i64), ("b_sn", i64), ("b_st", i64),
        ("c_sb", i64), ("c_sg", i64), ("c_sn", i64), ("c_st", i64),
        ("D", fp), ("dt_bias", fp), ("initial_state", fp),
        ("out", vp), ("last_state", vp), ("checkpoints", fp),
        ("row_sb", i64), ("row_sd", i64),
        ("split_scratch", fp), ("split_segments", i32), ("reserved1", i32),
    ]


class ScanBwdArgs(C.Structure):
    _fields_ = [
        ("fwd", ScanFwdArgs),
        ("dout", vp), ("dlast_state", fp), ("du", vp), ("ddelta", vp), ("dz", vp),
        ("dA", fp), ("dB", fp), ("dC", fp),
        ("db_sb", i64), ("db_sg", i64), ("db_sn", i64), ("db_st", i64),
        ("dc_sb", i64), ("dc_sg", i64), ("dc_sn", i64), ("dc_st", i64),
        ("dD", fp), ("ddt_bias", fp), ("dinitial_state", fp),
    ]


class StepArgs(C.Structure):
    _fields_ = [
        ("batch", i32), ("dim", i32), ("nstate", i32), ("io_dtype", i32),
        ("bc_dtype", i32), ("bc_groups", i32), ("dt_softplus", i32), ("param_heads", i32),
        ("state", fp), ("x", vp), ("dt", vp), ("z", vp), ("A", fp), ("Bm", vp), ("Cm", vp),
        ("b_sb", i64), ("b_sg", i64), ("b_sn", i64),
        ("c_sb", i64), ("c_sg", i64), ("c_sn", i64),
        ("D", fp), ("dt_bias", fp), ("out", vp),
    ]


class StepBwdArgs(C.Structure):
    _fields_ = [
        ("fwd", StepArgs),
        ("dout", vp), ("dnew_state", fp), ("dstate", fp), ("dx", vp), ("ddt", vp), ("dz", vp),
        ("dA", fp), ("dB", fp), ("dC", fp), ("dD", fp), ("ddt_bias", fp),
    ]


class Bcast4(C.Structure):
    _fields_ = [("ptr", vp), ("sb", i64), ("st", i64), ("sh", i64), ("sq", i64)]


class ChunkArgs(C.Structure):
    _fields_ = [
        ("batch", i32), ("len", i32), ("heads", i32), ("proj", i32),
        ("io_dtype", i32), ("par_dtype", i32), ("reserved0", i32), ("typed_grads", i32),
        ("X", vp), ("dt", vp),
        ("A", Bcast4), ("Bm", Bcast4), ("Cm", Bcast4), ("D", Bcast4), ("z", Bcast4), ("initial", Bcast4),
        ("seq_lens", vp), ("Y", vp), ("final_state", fp), ("scratch", fp),
        ("chunk_size", i32), ("reserved2", i32),
    ]


class ChunkBwdArgs(C.Structure):
    _fields_ = [
        ("fwd", ChunkArgs),
        ("dY", vp), ("dX", vp), ("ddt", fp),
        ("dA", Bcast4), ("dB", Bcast4), ("dC", Bcast4), ("dD", Bcast4), ("dz", Bcast4), ("dinitial", Bcast4),
        ("history", fp), ("scratch", fp),
    ]


class ConvArgs(C.Structure):
    _fields_ = [
        ("batch", i32), ("channels", i32), ("len", i32), ("width", i32),
        ("io_dtype", i32), ("channels_first", i32), ("silu", i32), ("reserved0", i32),
        ("x", vp), ("weight", fp), ("bias", fp), ("halo", fp), ("y", vp),
        ("row_sb", i64), ("row_sc", i64),
    ]


class ConvBwdArgs(C.Structure):
    _fields_ = [("fwd", ConvArgs), ("dy", vp), ("dx", vp), ("dweight", fp), ("dbias", fp)]


class ConvUpdateArgs(C.Structure):
    _fields_ = [
        ("batch", i32), ("channels", i32), ("width", i32), ("io_dtype", i32),
        ("silu", i32), ("reserved0", i32),
        ("conv_state", fp), ("x", vp), ("weight", fp), ("bias", fp), ("out", vp),
    ]


class NormArgs(C.Structure):
    _fields_ = [
        ("rows", i64),
        ("hidden", i32), ("io_dtype", i32), ("res_dtype", i32), ("resout_dtype", i32),
        ("is_rms", i32), ("prenorm", i32), ("reserved0", i32), ("reserved2", i32),
        ("eps", C.c_float), ("reserved1", C.c_float),
        ("x", vp), ("residual", vp), ("weight", fp), ("bias", fp), ("y", vp), ("residual_out", vp),
    ]


class NormBwdArgs(C.Structure):
    _fields_ = [("fwd", NormArgs), ("dy", vp), ("dx", vp), ("dresidual", vp), ("dweight", fp), ("dbias", fp), ("partial", fp), ("dresidual_out", vp)]


class SsdArgs(C.Structure):
    _fields_ = [
        ("batch", i32), ("len", i32), ("heads", i32), ("headdim", i32),
        ("nstate", i32), ("groups", i32), ("chunk_size", i32), ("io_dtype", i32),
        ("dt_softplus", i32), ("d_has_p", i32), ("phase", i32), ("dt_mode", i32),
        ("X", vp), ("dt", vp), ("A", fp), ("Bm", vp), ("Cm", vp), ("D", fp), ("z", vp), ("dt_bias", fp),
        ("initial_states", fp), ("Y", vp), ("final_states", fp),
        ("ws_dt", fp), ("ws_cum", fp), ("ws_state", fp), ("ws_state_in", vp), ("status", vp),
        ("row_dots", fp), ("row_scale", fp), ("bc_width", i32), ("x_heads", i32),
        ("ws_state_in_f32", fp),
    ]


class SsdBwdArgs(C.Structure):
    _fields_ = [
        ("batch", i32), ("len", i32), ("len_valid", i32), ("heads", i32),
        ("headdim", i32), ("io_dtype", i32), ("d_has_p", i32), ("reserved0", i32),
        ("gY", vp), ("z", vp), ("X", vp), ("y_plain", vp), ("dx_rev", vp), ("D", fp),
        ("dy", vp), ("dy_rev", vp), ("dX", vp), ("dz", vp), ("dD", fp),
    ]


# entry point -> (restype, argtypes); every name here is declared in include/ssm_b200.h
ENTRY_POINTS = {
    "ssm_b200_abi_version": (C.c_int, []),
    "ssm_b200_last_error": (C.c_char_p, []),
    "ssm_scan_checkpoint_interval": (C.c_int, []),
    "ssm_scan_split_segments": (C.c_int, [i32, i32, i32, i32]),
    "ssm_selective_scan_fwd": (C.c_int, [C.POINTER(ScanFwdArgs), vp]),
    "ssm_selective_scan_bwd": (C.c_int, [C.POINTER(ScanBwdArgs), vp]),
    "ssm_selective_state_step": (C.c_int, [C.POINTER(StepArgs), vp]),
    "ssm_selective_state_step_bwd": (C.c_int, [C.POINTER(StepBwdArgs), vp]),
    "ssm_chunk_scan_scratch_floats": (C.c_int64, [i32, i32, i32, i32, i32]),
    "ssm_chunk_scan_fwd": (C.c_int, [C.POINTER(ChunkArgs), vp]),
    "ssm_chunk_scan_bwd_scratch_floats": (C.c_int64, [i32, i32, i32, i32, i32]),
    "ssm_chunk_scan_bwd": (C.c_int, [C.POINTER(ChunkBwdArgs), vp]),
    "ssm_dw_causal_conv_fwd": (C.c_int, [C.POINTER(ConvArgs), vp]),
    "ssm_dw_causal_conv_bwd": (C.c_int, [C.POINTER(ConvBwdArgs), vp]),
    "ssm_dw_causal_conv_update": (C.c_int, [C.POINTER(ConvUpdateArgs), vp]),
    "ssm_fused_add_norm_fwd": (C.c_int, [C.POINTER(NormArgs), vp]),
    "ssm_norm_bwd_scratch_floats": (C.c_int64, [i64, i32]),
    "ssm_fused_add_norm_bwd": (C.c_int, [C.POINTER(NormBwdArgs), vp]),
    "ssm_fused_add_norm_bwd_noalloc": (C.c_int, [C.POINTER(NormBwdArgs), vp]),
    "ssm_ssd_supported": (C.c_int, [i32, i32, i32, i32]),
    "ssm_ssd_wait_selftest": (C.c_int, [vp, i32, vp]),
    "ssm_ssd_scratch_bytes": (C.c_int64, [i32, i32, i32]),
    "ssm_ssd_state_scratch_bytes": (C.c_int64, [i32, i32, i32]),
    "ssm_ssd_bwd_gate": (C.c_int, [C.POINTER(SsdBwdArgs), vp]),
    "ssm_ssd_bwd_finish": (C.c_int, [C.POINTER(SsdBwdArgs), vp]),
    "ssm_time_flip": (C.c_int, [vp, vp, i32, i32, i32, C.c_int64, vp]),
    "ssm_ssd_bwd_group_sum": (C.c_int, [vp, fp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp]),
    "ssm_ssd_bwd_spread": (C.c_int, [vp, vp, C.c_int64, i32, i32, C.c_int64, vp]),
    "ssm_ssd_state_dot": (C.c_int, [vp, vp, fp, i32, i32, i32, i32, i32, vp]),
    "ssm_ssd_fwd": (C.c_int, [C.POINTER(SsdArgs), vp]),
    "ssm_ssd_shard_summary_floats": (C.c_int64, [i32, i32]),
    "ssm_ssd_fold_shards": (C.c_int, [vp, i32, i32, i32, i32, vp, vp, vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it or any declared symbol is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run `python -m ssm_b200.build`); there is no CPU or PyTorch fallback."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in ENTRY_POINTS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise RuntimeError(f"{LIB_PATH} does not export {name}; rebuild the library") from exc
        fn.restype, fn.argtypes = res, args
    if lib.ssm_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libssm_b200.so has an unexpected ABI version; rebuild the library")
    _lib = lib
    return lib


class BackendError(RuntimeError):
    """The library rejected a call (``code`` < 0) or a launch failed (``code`` > 0)."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


def check(code: int) -> None:
    if code != 0:
        msg = load().ssm_b200_last_error().decode("utf-8", "replace")
        raise BackendError(code, msg or f"libssm_b200 error {code}")
