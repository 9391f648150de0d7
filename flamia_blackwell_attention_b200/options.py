"""Option objects of flash_attn_fp8 / flash_attn_fp4.

Same class names, field names, defaults and construction-time validation as the reference's
flash_attn/cute/lowprec/options.py (FP4AttnOptions :39, FP8AttnOptions :210, KernelTuning :325-501): an options object is
a frozen value that is hashed into the resolved plan, and an illegal value raises ValueError naming the field and the
allowed values when the object is built. Fields that configure routes this library does not build keep their place so
that reference-style call sites construct; the plan refuses their non-default values by name instead of ignoring them.
Nothing here reads the environment or any global state.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Optional

__all__ = ["FP4AttnOptions", "FP8AttnOptions", "KernelTuning", "TUNING_FIELDS"]

# measured-constant knobs of the reference kernels (not API there either); accepted as names, refused when set
TUNING_FIELDS = tuple("""fp4_q_stage qk_split_pipe qk_split_causal qk_split_seqused fp8_generic_e2e fp8_e2e8_min_sk
fp8_e2e8_max_sk fwd_mask_loops fwd_softmax_fused fwd_max_tmem fwd_o_regstore fwd_o_regstore_min_sk fwd_causal_persistent
fwd_causal_persistent_max_sk fwd_nc_persistent q_dbuf corr_empty_early corr_rescale_batch qk_split_bprefetch
qk_split_late_p0 split_lean mxfp4_split mxfp4_directp fp8_pv_use_explicit_pack fp8_pv_zero_fill_regs fp8_pv_kv_stage_cap
fp8_pv_p_split_num fp8_pv_p_split_den fp4_pv_p_split_num fp4_pv_p_split_den fp4_pv_tmem_store_rep fp8_pv_tmem_store_rep
e2e_freq e2e_start_frg force_e2e mxfp8_use_inline_ptx ldred_rowmax fp4_group_max_first fp4_pv_log2_quant
fp4_exp2_emulation_every fp8_pv_p_log2_offset fp8_pv_rescale_threshold fp4_pv_tile_frame_drop token_block_forward
varlen_fwd_list varlen_fwd_tma_o varlen_fwd_stage_skip varlen_l2_sections varlen_fwd_sched varlen_fwd_sched_stages
varlen_fwd_sched_jit varlen_fwd_sched_early fwd_ptxas fwd_exp bwd_fp4_ds_fold bwd_dq_f16 bwd_fp4_ld_rep
bwd_fp4_sload_early bwd_fp4_warp_sync bwd_fp4_causal_diag bwd_fp4_dp_ld2 bwd_fp4_do_stage bwd_fp4_q_stage
bwd_fp4_q_dyn_issue bwd_fp4_stat_shfl bwd_fp4_reduce_chunked bwd_fp4_dq_ncol bwd_fp4_dq_stages bwd_fp4_dq_post
varlen_bwd_list bwd_fp4_det_gqa_rot two_cta8_warp_sync two_cta8_mx_xw two_cta8_regs two_cta8_causal_diag two_cta8_ld_rep
two_cta8_q_stage two_cta8_dq_ncol two_cta8_dq_stages two_cta8_lpt_l2 two_cta8_dq_zero bwd_2cta_gqa bwd_fp4q_qrow_cap
bwd_fp4q_sr_dither bwd_fp4q_post bwd_fp4q_dk_sr_blk32 fp4_d_do8 fp4_fused_ds_bound qk_hadamard_e4m3
qk_hadamard_rotation_method fp4_qk_sf_vec""".split())


class _Tuning:
    """Measured performance constants of the reference's kernels. Every field defaults to None ('the measured rule').
    This library has its own kernels and no tuning surface: a non-None field is refused by the plan (rule 'B2')."""

    def __init__(self, **kw):
        for n in TUNING_FIELDS:
            object.__setattr__(self, n, None)
        for n, v in kw.items():
            if n not in TUNING_FIELDS:
                raise TypeError(f"KernelTuning got an unexpected field {n!r}")
            object.__setattr__(self, n, v)

    def __setattr__(self, name, value):
        raise AttributeError("KernelTuning is frozen")

    def non_default(self) -> dict:
        return {n: getattr(self, n) for n in TUNING_FIELDS if getattr(self, n) is not None}

    def _key(self):
        return tuple(sorted(self.non_default().items()))

    def __eq__(self, other):
        return isinstance(other, _Tuning) and self._key() == other._key()

    def __hash__(self):
        return hash(self._key())

    def __repr__(self):
        return "KernelTuning(" + ", ".join(f"{k}={v!r}" for k, v in self.non_default().items()) + ")"


KernelTuning = _Tuning
KernelTuning.__name__ = KernelTuning.__qualname__ = "KernelTuning"


def _validate(obj, choices: dict, bools=()):
    owner = type(obj).__name__
    for name, allowed in choices.items():
        value = getattr(obj, name)
        if value not in allowed:
            raise ValueError(f"{owner}.{name} must be one of {', '.join(repr(a) for a in allowed)}; got {value!r}.")
    for name in bools:
        if not isinstance(getattr(obj, name), bool):
            raise ValueError(f"{owner}.{name} must be a bool; got {getattr(obj, name)!r}.")
    if obj.tuning is not None and not isinstance(obj.tuning, KernelTuning):
        raise ValueError(f"{owner}.tuning must be a KernelTuning or None; got {type(obj.tuning).__name__}.")


_ON_OFF = ("auto", "on", "off")
_SCALING = ("auto", "token_block", "block_32x32", "per_tensor", "token_local")


@dataclass(frozen=True)
class FP8AttnOptions:
    """Advanced options of flash_attn_fp8; every default is the certified 8-bit configuration.

    Served here: operand_scaling 'auto' | 'token_block' | 'token_local'; ds_scaling 'auto' | 'block_32x32';
    ds_dq_rowlocal 'off' | 'all'; p_scaling 'row'; grad_format 'e4m3'; softmax_exp 'exp2'; forward_kernel 'auto' | 'fork';
    two_cta 'auto' | 'off'; forward_two_cta 'auto' | 'off'; p_hat_frame 'auto' | 'row'. Anything else is refused by name."""
    operand_scaling: str = "auto"
    per_tensor_scale: str = "exact"
    ds_scaling: str = "auto"
    ds_dq_rowlocal: str = "off"
    per_tensor_ds_source: Optional[str] = None
    p_scaling: str = "row"
    grad_format: str = "e4m3"
    softmax_exp: str = "exp2"
    forward_kernel: str = "auto"
    two_cta: str = "auto"
    forward_two_cta: str = "auto"
    p_hat_frame: str = "auto"
    tuning: Optional[Any] = None

    def __post_init__(self):
        _validate(self, {
            "operand_scaling": _SCALING, "per_tensor_scale": ("exact", "power_of_two"),
            "ds_scaling": ("auto", "block_32x32", "per_tensor", "row_local", "row_1x32", "block_32x64", "tile_128"),
            "ds_dq_rowlocal": ("off", "diagonal", "all"), "per_tensor_ds_source": (None, "recompute", "forward_bound"),
            "p_scaling": ("row", "block_1x32"), "grad_format": ("e4m3", "e5m2"), "softmax_exp": ("exp2", "mitchell"),
            "forward_kernel": ("auto", "fork", "upstream"), "two_cta": _ON_OFF, "forward_two_cta": _ON_OFF,
            "p_hat_frame": ("auto", "row", "group")})


@dataclass(frozen=True)
class FP4AttnOptions:
    """Advanced options of flash_attn_fp4 (NVFP4 Q.K^T, E4M3 elsewhere); every default is the certified configuration.

    Served here: the defaults, operand_scaling 'auto' | 'token_block', ds_dq_rowlocal 'off' | 'all', two_cta /
    forward_two_cta 'auto' | 'off'. The fields of the all-4-bit route and of the 4-bit P.V (option A) keep their names and
    defaults; a non-default value is refused by name."""
    operand_scaling: str = "auto"
    per_tensor_scale: str = "exact"
    ds_scaling: str = "auto"
    ds_dq_rowlocal: str = "off"
    fp4_ds_multiplier: str = "auto"
    p_scaling: str = "row"
    p_frame: str = "two_level"
    p_hat_frame: str = "auto"
    softmax_exp: str = "auto"
    k_channel: str = "fold"
    q_block_2d: bool = False
    v_hadamard: bool = False
    all_fp4_stabiliser: str = "sr"
    sr_ds: bool = False
    sr_dk_operand: bool = True
    sr_dv_operand: bool = False
    fp4_backward_dkdv: str = "e4m3"
    dq_operand: str = "fp4"
    two_cta: str = "auto"
    forward_two_cta: str = "auto"
    seqused_k_group_aligned: bool = False
    save_bf16_inputs: bool = True
    p_consistency: str = "reproduce_forward_p"
    do_rounding: str = "rtn"
    exp_mix: str = "auto"
    tuning: Optional[Any] = None

    def __post_init__(self):
        _validate(self, {
            "operand_scaling": _SCALING, "per_tensor_scale": ("exact", "power_of_two"),
            "ds_scaling": ("auto", "block_32x32", "per_tensor"), "ds_dq_rowlocal": ("off", "diagonal", "all"),
            "fp4_ds_multiplier": ("auto", "global", "global_row_boost", "row_local"),
            "p_scaling": ("row", "block_1x32"), "p_frame": ("two_level", "per_tile", "single_level"),
            "p_hat_frame": ("auto", "row", "group"), "softmax_exp": ("auto", "exp2", "mitchell"),
            "k_channel": ("fold", "cut", "all", "open"), "all_fp4_stabiliser": ("sr", "rtn", "eden_rht"),
            "fp4_backward_dkdv": ("e4m3", "fp4"), "dq_operand": ("fp4", "e4m3"), "two_cta": _ON_OFF,
            "forward_two_cta": _ON_OFF, "p_consistency": ("reproduce_forward_p", "none"), "do_rounding": ("rtn", "sr")},
            bools=("q_block_2d", "v_hadamard", "sr_ds", "sr_dk_operand", "sr_dv_operand", "seqused_k_group_aligned",
                   "save_bf16_inputs"))


def non_default_fields(opts) -> dict:
    """{field: value} of every option that differs from its default."""
    return {f.name: getattr(opts, f.name) for f in fields(opts) if getattr(opts, f.name) != f.default}
