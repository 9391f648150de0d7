"""ctypes binding of libflamia_b200.so (the C ABI declared in include/flamia_b200.h).

The library is the only compute path: there is no CPU or PyTorch fallback. If it is missing the import of the kernels
fails loudly with the command that builds it.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libflamia_b200.so")

# status codes (csrc/sm100.cuh)
ABI_VERSION = 8
FL_OK, FL_ERR_BAD_ARG, FL_ERR_CUDA, FL_ERR_UNSUPPORTED, FL_ERR_TOO_LARGE = 0, 1, 2, 3, 4
FL_DEV_WAIT_TIMEOUT = 0x100
FL_DEV_BAD_TABLE = 0x200
ERR_NAMES = {1: "bad argument", 2: "CUDA error", 3: "unsupported configuration", 4: "size beyond the supported maximum"}

FL_Q_HADAMARD, FL_Q_TOKEN_LOCAL, FL_Q_HADAMARD_NVFP4_ONLY, FL_Q_O_PACKED, FL_Q_LEGACY = 1, 2, 4, 8, 16
FL_MODE_FP8, FL_MODE_FP4 = 0, 1
FL_A_CAUSAL, FL_A_OUT_F16, FL_A_TOKEN_LOCAL, FL_A_DQ_ROWLOCAL, FL_A_HAD_DQ, FL_A_HAD_DK, FL_A_P_GROUP = 1, 2, 4, 8, 16, 32, 64

vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


class QuantArgs(C.Structure):
    _fields_ = [(n, vp) for n in ("x", "o", "lse", "codes", "codes_t", "e_tab", "fac", "sf_tok", "sf_dim",
                                  "token_factors", "x4", "sf4", "d_out", "lse_log2", "zero_acc", "tile_stats")] + \
               [(n, i32) for n in ("b", "s", "h", "d", "flags", "in_f16")] + [("lse_shift", f32), ("d_multiplier", f32),
                                                                            ("status", vp), ("wait_cycles", i64),
                                                                            ("slot_src", vp), ("slot_rows", vp), ("src_rows", i32),
                                                                            ("row_stat", vp), ("row_stat_kind", i32)]


class AttnArgs(C.Structure):
    _fields_ = [(n, vp) for n in ("q_codes", "k_codes", "v_codes", "do_codes", "fac_q", "fac_k", "fac_v", "fac_do", "q4",
                                  "k4", "sfq4", "sfk4", "out", "lse", "lse_log2", "d_rows", "dq_acc", "dq_scale", "dk",
                                  "dv", "doc_start", "doc_len")] + \
               [(n, i32) for n in ("n_docs", "b", "s_q", "s_k", "h", "h_kv", "d")] + [("softmax_scale", f32)] + \
               [(n, i32) for n in ("mode", "flags")] + [("status", vp), ("wait_cycles", i64)] + \
               [(n, i32) for n in ("window_left_p1", "window_right_p1")] + [("seqused_k", vp), ("softcap", f32), ("dq_order", vp), ("dq_scale_rows", vp), ("o_mult", vp), ("dk_mult", vp), ("slot_src", vp), ("slot_rows", vp), ("out_rows", i32), ("tok_lg_v", vp), ("tok_rcp_v", vp)]


EXPORTS = {
    "fl_abi_version": (i32, []),
    "fl_quant_blocks": (i32, [C.POINTER(QuantArgs), vp]),
    "fl_fwd": (i32, [C.POINTER(AttnArgs), vp]),
    "fl_bwd": (i32, [C.POINTER(AttnArgs), vp]),
    "fl_dq_prescale": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp, vp]),
    "fl_bwd_static_acc": (i32, [C.POINTER(AttnArgs), vp, f32, vp, vp]),
    "fl_dq_post": (i32, [vp, vp, f32, vp, i32, i32, i32, i32, i32, i32, vp]),
    "fl_dq_post_rows": (i32, [vp, vp, f32, vp, i32, i32, i32, i32, i32, i32, vp]),
    "fl_dq_post_ex": (i32, [vp, vp, i32, vp, f32, vp, i32, i32, i32, i32, i32, i32, vp]),
    "fl_code_stats": (i32, [vp, vp, i32, i32, i32, i32, vp, vp]),
    "fl_token_aux": (i32, [vp, C.c_int64, vp, vp, vp]),
    "fl_dq_post_packed": (i32, [vp, vp, f32, vp, i32, i32, i32, i32, i32, vp, vp, vp]),
    "fl_dq_prescale_rows": (i32, [vp, vp, vp, i32, i32, f32, vp, vp, vp]),
    "fl_pack_rows": (i32, [vp, vp, vp, i32, i32, vp]),
    "fl_unpack_rows": (i32, [vp, vp, vp, i32, i32, vp]),
    "fl_selftest_mma": (i32, [i32, vp, vp, vp, vp, vp, vp, i64, vp]),
    "fl_read_status": (i32, [vp, C.POINTER(i32), vp]),
    "fl_last_cuda_error": (i32, [C.c_char_p, i32]),
}

_lib = None


def load():
    """The loaded library (cached). Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m flamia_blackwell_attention_b200.build` "
                          "(nvcc, sm_100a). There is no fallback path.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc != 0:
        detail = ""
        if rc == FL_ERR_CUDA:
            buf = C.create_string_buffer(256)
            load().fl_last_cuda_error(buf, 256)
            detail = ": " + buf.value.decode(errors="replace")
        raise RuntimeError(f"{what} failed: {ERR_NAMES.get(rc, rc)} (code {rc}){detail}")


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())
