"""Plan resolution: resolve_fp8 / resolve_fp4 turn a call's arguments and tensor METADATA into one immutable AttnPlan
before anything is quantised or launched, or refuse the call.

Mirrors the contract of the reference's flash_attn/cute/lowprec/plan.py (resolve_fp4 :973, resolve_fp8 :1504, AttnPlan
:166, _fail :76): every invalid or unserved combination raises ValueError / NotImplementedError / TypeError carrying a
`.rule` attribute ("refused rather than ignored"); "auto" values are resolved once with a reason recorded in
plan.log(); the plan is a pure function of the arguments (works on device="meta" tensors) and the only configuration
the backward sees. Rule ids and message prefixes follow the reference's table (tests/cute/test_lowprec_api.py:55-213) for
the rules that apply to the two routes built here; features of routes this library does not build are refused under
rule ids "B1".."B9" that name the missing piece.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Optional, Tuple

import torch

from .options import FP4AttnOptions, FP8AttnOptions, KernelTuning, non_default_fields

__all__ = ["AttnPlan", "CallShape", "FwdSpec", "BwdSpec", "resolve_fp4", "resolve_fp8"]


def _fail(rule, exc_cls, msg):
    e = exc_cls(msg)
    e.rule = rule
    raise e


@dataclass(frozen=True)
class CallShape:
    b: int
    s_q: int
    s_k: int
    h: int
    h_kv: int
    d: int
    dtype: str
    varlen: bool
    aligned_varlen: bool
    requires_grad: bool
    tot_q: int
    tot_k: int

    @property
    def mha(self) -> bool:
        return self.h == self.h_kv


@dataclass(frozen=True)
class FwdSpec:
    kernel: str            # fwd_sm100 (this library's forward kernel)
    qk_format: str         # e4m3 | nvfp4
    pv_operand: str        # e4m3
    operand_scaling: str   # token_block | token_local
    p_hat_frame: str       # row | group
    softmax_exp: str       # exp2
    qk_hadamard: bool
    causal: bool
    varlen: bool
    aligned_varlen: bool
    ragged_documents: bool
    return_lse: bool
    window: Optional[tuple] = None
    softcap: float = 0.0
    seqused_k: bool = False
    two_cta: bool = False


@dataclass(frozen=True)
class BwdSpec:
    kernel: str            # 1cta | none
    operand_scaling: str
    ds_scaling: str        # block_32x32
    ds_dq_rowlocal: str    # off | all
    p_scaling: str         # row
    grad_format: str       # e4m3
    deterministic: bool
    dq_prescale: str       # row | causal_tile | causal_row


@dataclass(frozen=True)
class AttnPlan:
    entry: str                                        # fp8 | fp4
    route: str                                        # fp8 | fp4.e4m3_pv
    softmax_scale: float
    shape: CallShape
    fwd: FwdSpec
    bwd: BwdSpec
    tuning: Optional[KernelTuning]
    prequant: bool
    q_scale_fused: bool
    resolution_log: Tuple[Tuple[str, str, str], ...]
    options: object = field(compare=True)
    pad_from: int = 0                                 # the call's own head dim when the kernels run it padded (else 0)

    def log(self) -> str:
        return "\n".join(f"{f} = {v}: {r}" for f, v, r in self.resolution_log)


# ---------------------------------------------------------------------------------------------------------------------
def _shape_of(entry, q, k, v, cu_q, cu_k, seqused_q, seqused_k, max_q, max_k):
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor):
            _fail("B9", TypeError, f"flash_attn_{entry}: {name} must be a torch.Tensor; got {type(t).__name__}")
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        _fail("B9", TypeError, f"flash_attn_{entry}: q, k, v must share the dtype bfloat16 or float16; got "
                               f"{q.dtype}, {k.dtype}, {v.dtype}")
    varlen = cu_q is not None or cu_k is not None
    if varlen:
        if cu_q is None or cu_k is None:
            _fail("B9", ValueError, f"flash_attn_{entry}: cu_seqlens_q and cu_seqlens_k must be supplied together")
        if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
            _fail("B9", ValueError, f"flash_attn_{entry}: packed q, k, v are (total, heads, head_dim) with cu_seqlens_*")
        b = int(cu_q.shape[0]) - 1
        tot_q, h, d = q.shape
        tot_k, h_kv, _ = k.shape
        aligned = seqused_q is not None and seqused_k is not None
        if (seqused_q is None) != (seqused_k is None):
            _fail("B9", ValueError, f"flash_attn_{entry}: the aligned varlen form takes seqused_q AND seqused_k")
        s_q = int(max_q) if max_q is not None else int(tot_q)
        s_k = int(max_k) if max_k is not None else int(tot_k)
    else:
        if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
            _fail("B9", ValueError, f"flash_attn_{entry}: q, k, v are (batch, seqlen, heads, head_dim)")
        b, s_q, h, d = q.shape
        _, s_k, h_kv, _ = k.shape
        tot_q, tot_k, aligned = s_q, s_k, False
        if seqused_q is not None:
            _fail("B9", ValueError, f"flash_attn_{entry}: seqused_q belongs to the aligned varlen form (with cu_seqlens)")
    if tuple(k.shape) != tuple(v.shape):
        _fail("B9", ValueError, f"flash_attn_{entry}: k and v must have the same shape; got {tuple(k.shape)} and "
                                f"{tuple(v.shape)}")
    if k.shape[-1] != d or (not varlen and k.shape[0] != b):
        _fail("B9", ValueError, f"flash_attn_{entry}: q and k disagree on batch or head_dim")
    if h_kv <= 0 or h % h_kv:
        _fail("B9", ValueError, f"flash_attn_{entry}: heads ({h}) must be a multiple of kv heads ({h_kv})")
    rg = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v))
    return CallShape(int(b), int(s_q), int(s_k), int(h), int(h_kv), int(d), str(q.dtype).replace("torch.", ""),
                     bool(varlen), bool(aligned), bool(rg), int(tot_q), int(tot_k))


def scaling_request(o):
    return getattr(o, "operand_scaling", "auto")


def _common(entry, shape, log, *, causal, window_size, softcap, score_mod, score_mod_bwd, mask_mod, seqused_k,
            deterministic, qk_hadamard, opts, two_cta_fields=True):
    """Rules shared by both entries; returns (qk_hadamard, operand_scaling, ds_dq_rowlocal, ragged)."""
    o = opts
    if o.tuning is not None and o.tuning.non_default():
        _fail("B2", ValueError, f"KernelTuning {sorted(o.tuning.non_default())} configures the reference's CuTe-DSL "
                                "kernels; this library has its own kernels and no tuning surface")
    if score_mod is not None and score_mod_bwd is None and shape.requires_grad:
        _fail(28, ValueError, "score_mod needs score_mod_bwd when an input requires grad")
    if mask_mod is not None and (causal or tuple(window_size) != (None, None)):
        _fail(28, ValueError, "mask_mod with causal / window_size: express the whole mask in the mask_mod")
    if score_mod is not None or score_mod_bwd is not None or mask_mod is not None:
        _fail("B3", NotImplementedError, "score_mod / mask_mod are CuTe-DSL callables of the reference's kernels; "
                                         "this library takes causal and dense masks")
    wl, wr = tuple(window_size)
    for w in (wl, wr):
        if w is not None and (not isinstance(w, int) or w < -1):
            _fail(28, ValueError, f"window_size entries are None, -1 (unlimited) or a non-negative int; got {window_size}")
    if softcap:
        if not isinstance(softcap, (int, float)) or softcap < 0:
            _fail(28, ValueError, f"softcap is a non-negative float (0 = off); got {softcap!r}")
        if scaling_request(o) == "token_local" or o.ds_dq_rowlocal == "all":
            _fail("B4", NotImplementedError, "softcap is built on the default route (token-block operands, shared "
                                             "dS-hat exponents), not with operand_scaling='token_local' / "
                                             "ds_dq_rowlocal='all'")
    if seqused_k is not None and not shape.aligned_varlen:
        if shape.varlen:
            _fail("B9", ValueError, f"flash_attn_{entry}: the aligned varlen form takes seqused_q AND seqused_k")
        if shape.s_q % 128 or shape.s_k % 128:
            _fail("B4", NotImplementedError, "batched seqused_k with lengths that are no multiple of 128 is not built "
                                             f"(those run as documents); got {shape.s_q} / {shape.s_k}")
        if scaling_request(o) == "token_local":
            _fail("B4", NotImplementedError, "batched seqused_k with operand_scaling='token_local' is not built")
        if isinstance(seqused_k, torch.Tensor) and (seqused_k.dim() != 1 or seqused_k.shape[0] != shape.b or
                                                    seqused_k.dtype != torch.int32):
            _fail("B9", ValueError, f"flash_attn_{entry}: seqused_k is an int32 tensor of shape (batch,); got "
                                    f"{tuple(seqused_k.shape)} {seqused_k.dtype}")
    if deterministic:
        if (softcap or 0.0) > 0.0 or scaling_request(o) == "token_local" or o.ds_dq_rowlocal == "all":
            _fail("B5", NotImplementedError, "deterministic=True (ordered dQ reduction) is built on the default backward "
                                             "only: without softcap, operand_scaling='token_local' or "
                                             "ds_dq_rowlocal='all'")
        log("deterministic", "ordered", "the key tiles add their f16 dQ partial sums in ascending key order (bounded waits)")
    # ---- dS
    if o.ds_scaling == "per_tensor":
        _fail(33, ValueError, f"ds_scaling='per_tensor' was removed from flash_attn_{entry}: sizing a per-tensor dS needs "
                              "either an extra full pass or the forward's loose P_max bound, and it is a global causal "
                              "channel")
    if o.ds_scaling not in ("auto", "block_32x32"):
        _fail("B6", NotImplementedError, f"ds_scaling={o.ds_scaling!r} is not built: block_32x32 is the dS-hat scaling")
    log("ds_scaling", "block_32x32", "auto" if o.ds_scaling == "auto" else "explicit")
    if o.ds_dq_rowlocal == "diagonal":
        _fail("B6", NotImplementedError, "ds_dq_rowlocal='diagonal' is not built (measured not to close the channel); "
                                         "use 'all'")
    if o.p_scaling != "row":
        _fail(16, ValueError, f"flash_attn_{entry}: operand_scaling='auto' resolves to token blocks, which cannot serve "
                              f"this call: p_scaling={o.p_scaling!r}")
    if o.softmax_exp == "mitchell":
        _fail(21, ValueError, "Mitchell P-hat on an E4M3 P.V was removed: the E4M3 P-hat is formed with exp2")
    if o.per_tensor_scale != "exact":
        _fail(16, ValueError, "per_tensor_scale configures per-tensor operands, which this library does not build")
    # ---- head dim / lengths
    if shape.d not in (64, 128):
        if shape.d > 128 and entry == "fp8":
            _fail("E13", NotImplementedError, f"flash_attn_fp8 serves head_dim <= 128; got {shape.d}")
        _fail("E13", NotImplementedError, f"flash_attn_{entry} serves head_dim <= 128 (a multiple of 16; 64 and 128 "
                                          f"natively, the others padded); got {shape.d}")
    # ---- operand scaling
    scaling = o.operand_scaling
    if scaling in ("block_32x32", "per_tensor"):
        _fail(16, ValueError, f"operand_scaling={scaling!r} cannot serve this call: this library builds token-block and "
                              "token-local operands (a per-tensor scale is a global causal channel)")
    if scaling == "auto":
        scaling = "token_block"
        log("operand_scaling", "token_block", "auto: one UE8M0 exponent per 32 tokens x the whole head dim")
    else:
        log("operand_scaling", scaling, "explicit")
    rowlocal = o.ds_dq_rowlocal
    if scaling == "token_local":
        if rowlocal != "all":
            _fail(16, ValueError, "operand_scaling='token_local' needs ds_dq_rowlocal='all' (the shared block exponent "
                                  "of dS-hat would reopen the channel it closes)")
        if shape.varlen:
            _fail(16, ValueError, "operand_scaling='token_local' runs the fold forward, which takes no varlen documents")
        if causal and shape.s_q > shape.s_k:
            _fail(16, ValueError, f"operand_scaling='token_local' with causal s_q > s_k ({shape.s_q} vs {shape.s_k})")
        if qk_hadamard is True:
            _fail(16, ValueError, "operand_scaling='token_local' has no rotated quantiser: qk_hadamard=True cannot be "
                                  "served")
    # ---- Hadamard
    had = qk_hadamard
    if had is True and shape.d != 128:
        _fail(4, NotImplementedError, f"qk_hadamard is built for head_dim 128; got {shape.d}")
    if had is None:
        if shape.d != 128:
            had = False
            log("qk_hadamard", "off", f"auto: built for head_dim 128, this call has {shape.d}")
        elif scaling == "token_local":
            had = False
            log("qk_hadamard", "off", "auto: no rotated token-local quantiser exists")
        else:
            had = True
            log("qk_hadamard", "on", "auto: ON wherever it runs (d = 128)")
    else:
        log("qk_hadamard", "on" if had else "off", "explicit")
    # ---- kernels
    if o.two_cta == "on":
        why = f"head_dim {shape.d}" if shape.d != 128 else "this library builds the 1-CTA backward only"
        _fail(15, ValueError, f"two_cta='on' but the 2-CTA backward cannot serve this call: {why}")
    if o.forward_two_cta == "on":
        _fail(15, ValueError, "forward_two_cta='on' but the forward on CTA pairs is not built here")
    ragged = (not shape.varlen) and (shape.s_q % 128 != 0 or shape.s_k % 128 != 0)
    if scaling == "token_local" and ragged:
        _fail(16, ValueError, "operand_scaling='token_local' runs the fold forward, which takes no documents: lengths that "
                              f"are no multiple of 128 run as documents; got {shape.s_q} / {shape.s_k}")
    if shape.d != 128 and shape.requires_grad and (rowlocal == "all" or scaling == "token_local"):
        _fail("B6", NotImplementedError, "ds_dq_rowlocal='all' (and with it operand_scaling='token_local') is built in "
                                         f"the head_dim 128 backward; this call runs at head_dim {shape.d}")
    return bool(had), scaling, rowlocal, ragged


def _finish(entry, route, qk_format, shape, log_rows, opts, *, softmax_scale, causal, return_lse, had, scaling, rowlocal,
            ragged, dq_causal, window_size=(None, None), p_frame="row", seqused_k=False, softcap=0.0,
            deterministic=False, pad_from=0):
    sc = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(shape.d)
    # sliding window (left, right): None / -1 = unlimited on that side; causal caps the right side at 0 in the kernels
    win = tuple(None if (w is None or w < 0) else int(w) for w in tuple(window_size))
    fwd = FwdSpec("fwd_sm100", qk_format, "e4m3", scaling, p_frame, "exp2", had, bool(causal), shape.varlen,
                  shape.aligned_varlen, ragged, bool(return_lse), None if win == (None, None) else win,
                  softcap=float(softcap or 0.0), seqused_k=bool(seqused_k))
    bwd = BwdSpec("1cta" if shape.requires_grad else "none", scaling, "block_32x32", rowlocal, "row", "e4m3",
                  bool(deterministic), dq_causal if isinstance(dq_causal, str) else ("causal_tile" if dq_causal else "row"))
    return AttnPlan(entry, route, sc, shape, fwd, bwd, opts.tuning, False, False, tuple(log_rows), opts, int(pad_from))


def resolve_fp8(q, k, v, *, softmax_scale=None, causal=False, window_size=(None, None), softcap=0.0, score_mod=None,
                score_mod_bwd=None, mask_mod=None, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=None,
                max_seqlen_k=None, seqused_k=None, seqused_q=None, deterministic=False, return_lse=False,
                qk_hadamard=None, q_quantized=None, k_quantized=None, q_scale_fused=False, options=None) -> AttnPlan:
    """The plan of a flash_attn_fp8 call (same arguments); launches nothing."""
    o = options if options is not None else FP8AttnOptions()
    if not isinstance(o, FP8AttnOptions):
        _fail("B9", TypeError, f"flash_attn_fp8: options must be an FP8AttnOptions; got {type(o).__name__}")
    if (q_quantized is None) != (k_quantized is None):
        _fail(32, ValueError, "flash_attn_fp8: q_quantized and k_quantized must be supplied together")
    if q_scale_fused and q_quantized is None:
        _fail(32, ValueError, "q_scale_fused=True needs q_quantized")
    if q_quantized is not None:
        _fail("B7", NotImplementedError, "pre-quantised Q / K (per-tensor E4M3) are not built: this library quantises "
                                         "token blocks itself")
    if o.per_tensor_ds_source is not None:
        _fail(33, ValueError, f"per_tensor_ds_source={o.per_tensor_ds_source!r} was removed with the per-tensor dS")
    if o.grad_format == "e5m2":
        _fail(16, ValueError, "grad_format='e5m2' is a per-tensor option (one scale over all of dO); token blocks use "
                              "E4M3")
    if o.forward_kernel == "upstream":
        _fail(16, ValueError, "flash_attn_fp8: operand_scaling='auto' resolves to token blocks, which cannot serve this "
                              "call: forward_kernel='upstream'")
    shape = _shape_of("fp8", q, k, v, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k, max_seqlen_q, max_seqlen_k)
    rows = []

    def log(f, val, why):
        rows.append((f, str(val), why))
        return val
    # head dims 16, 32, 48, 80, 96, 112 run padded to the next of 64 / 128 (the reference's rule E13,
    # flash_attn/cute/lowprec/plan.py:1529-1541): zero columns add nothing to S / dP and move no block exponent
    pad_from = 0
    if shape.d not in (64, 128) and 0 < shape.d < 128 and shape.d % 16 == 0:
        pad_from = shape.d
        d_pad = 64 if shape.d < 64 else 128
        if qk_hadamard is True:
            _fail(4, NotImplementedError, f"qk_hadamard is built for head_dim 128 (the rotation is 128-point); got {shape.d}")
        if scaling_request(o) == "token_local":
            _fail("E13", NotImplementedError, f"head_dim {shape.d} runs padded on token-block operands; "
                                              "operand_scaling='token_local' serves 64 and 128")
        log("head_dim_padding", d_pad, f"head_dim {shape.d}: the kernels run it padded to {d_pad} with zero columns; "
                                       "O / dQ / dK / dV are the first head_dim columns")
        had_why = "explicit" if qk_hadamard is False else f"auto: built for head_dim 128, this call has {shape.d}"
        qk_hadamard = False
        if softmax_scale is None:
            softmax_scale = 1.0 / math.sqrt(shape.d)
        shape = replace(shape, d=d_pad)
    had, scaling, rowlocal, ragged = _common("fp8", shape, log, causal=causal, window_size=window_size, softcap=softcap,
                                             score_mod=score_mod, score_mod_bwd=score_mod_bwd, mask_mod=mask_mod,
                                             seqused_k=seqused_k, deterministic=deterministic, qk_hadamard=qk_hadamard,
                                             opts=o)
    if pad_from:
        rows[:] = [(f, val, had_why) if f == "qk_hadamard" else (f, val, why) for f, val, why in rows]
    p_frame = _p_frame("fp8", o, shape, scaling, default="row")
    log("p_hat_frame", p_frame, "auto: the 8-bit default" if o.p_hat_frame == "auto" else "explicit")
    log("backward_kernel", "1cta", "the 1-CTA backward (key-stationary, GQA in the same accumulators)")
    from . import interface_bwd_fp4
    dq_causal = bool(interface_bwd_fp4.DQ_CAUSAL_PRESCALE) and bool(causal) and not shape.varlen and shape.s_q == shape.s_k
    gran = str(interface_bwd_fp4.DQ_CAUSAL_GRANULARITY)
    if gran not in ("tile", "row"):
        _fail("B9", ValueError, f"interface_bwd_fp4.DQ_CAUSAL_GRANULARITY is 'tile' or 'row'; got {gran!r}")
    if dq_causal and gran == "row" and (scaling == "token_local" or window_size not in ((None, None), (-1, -1))
                                        or seqused_k is not None or (softcap or 0.0) > 0.0 or ragged):
        gran = "tile"          # the per-row form serves the plain causal square call, like the reference's
    dq_causal = "causal_row" if (dq_causal and gran == "row") else ("causal_tile" if dq_causal else False)
    log("dq_prescale", dq_causal or "row", "per query row from per-token statistics and running maxima over the keys j <= i"
        if dq_causal == "causal_row" else ("per query tile from the prefix of key tiles"
        if dq_causal else "one power of two per batch row / document"))
    return _finish("fp8", "fp8", "e4m3", shape, rows, o, softmax_scale=softmax_scale, causal=causal,
                   return_lse=return_lse, had=had, scaling=scaling, rowlocal=rowlocal, ragged=ragged, dq_causal=dq_causal,
                   window_size=window_size, p_frame=p_frame,
                   seqused_k=seqused_k is not None and not shape.aligned_varlen, softcap=softcap,
                   deterministic=deterministic, pad_from=pad_from)


def _p_frame(entry, o, shape, scaling, default):
    """The frame of the E4M3 P-hat: 'row' (one frame per query row) or 'group' (one UE8M0 exponent per row and 32 keys)."""
    frame = default if o.p_hat_frame == "auto" else o.p_hat_frame
    if frame == "group" and (shape.d != 128 or scaling == "token_local"):
        if o.p_hat_frame == "auto":
            return "row"
        _fail("B6", NotImplementedError, f"p_hat_frame='group' is built for head_dim 128 with token-block operands (flash_attn_{entry})"
                                         "")
    return frame


def resolve_fp4(q, k, v, *, softmax_scale=None, causal=False, window_size=(None, None), softcap=0.0, score_mod=None,
                score_mod_bwd=None, mask_mod=None, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=None,
                max_seqlen_k=None, seqused_k=None, seqused_q=None, deterministic=False, return_lse=False,
                pv_precision="fp8", backward="e4m3", causal_safety="auto", qk_hadamard=None, options=None) -> AttnPlan:
    """The plan of a flash_attn_fp4 call (same arguments); launches nothing."""
    o = options if options is not None else FP4AttnOptions()
    if not isinstance(o, FP4AttnOptions):
        _fail("B9", TypeError, f"flash_attn_fp4: options must be an FP4AttnOptions; got {type(o).__name__}")
    if pv_precision not in ("fp8", "fp4") or backward not in ("e4m3", "fp4"):
        _fail("B9", ValueError, "pv_precision must be 'fp8' | 'fp4' and backward 'e4m3' | 'fp4'")
    if backward == "fp4" and pv_precision != "fp4":
        _fail(1, ValueError, "backward='fp4' is the query-row backward of the all-4-bit route: it needs pv_precision='fp4'")
    if pv_precision == "fp4":
        _fail("B1", NotImplementedError, "pv_precision='fp4' (the 4-bit P.V routes: option A and the all-4-bit step) is "
                                         "not built: flash_attn_fp4 runs NVFP4 Q.K^T with an E4M3 P.V here")
    if causal_safety not in ("auto", "key_local", "diagonal", "off"):
        _fail("B9", ValueError, f"causal_safety must be 'auto' | 'key_local' | 'diagonal' | 'off'; got {causal_safety!r}")
    if causal_safety in ("key_local", "diagonal"):
        _fail(7, ValueError, f"causal_safety={causal_safety!r} applies to a 4-bit P.V; this call's P.V is E4M3")
    for name, (rule, msg) in {
        "q_block_2d": (2, "q_block_2d shares one scale per 16 queries x 16 d and is not built"),
        "v_hadamard": ("B1", "v_hadamard configures the all-4-bit route"),
        "sr_ds": ("B6", "sr_ds (stochastic rounding of dS-hat) is not built"),
        "fp4_backward_dkdv": (29, "fp4_backward_dkdv configures the all-4-bit backward"),
        "dq_operand": (29, "dq_operand configures the all-4-bit backward"),
        "fp4_ds_multiplier": (29, "fp4_ds_multiplier configures the all-4-bit backward"),
        "all_fp4_stabiliser": (29, "all_fp4_stabiliser configures the all-4-bit backward"),
        "k_channel": (11, "k_channel selects how the diagonal route closes dQ's K channel (all-4-bit route)"),
        "p_frame": (23, "p_frame frames the 4-bit P-hat of option A"),
        "seqused_k_group_aligned": (26, "seqused_k_group_aligned applies to seqused_k with a 4-bit P.V, which no route "
                                        "takes"),
        "save_bf16_inputs": (34, "save_bf16_inputs=False cannot serve this call: the codes are all that is saved already"),
        "p_consistency": ("B1", "p_consistency configures option A"),
        "do_rounding": ("E1", "do_rounding configures option A"),
        "exp_mix": ("B1", "exp_mix configures the 4-bit P-hat"),
        "sr_dk_operand": ("B1", "sr_dk_operand configures the all-4-bit backward"),
        "sr_dv_operand": ("B1", "sr_dv_operand configures the all-4-bit backward"),
    }.items():
        if name in non_default_fields(o):
            _fail(rule, ValueError, msg + f"; got {name}={getattr(o, name)!r}")
    shape = _shape_of("fp4", q, k, v, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k, max_seqlen_q, max_seqlen_k)
    if shape.d != 128:
        _fail("E13", NotImplementedError, f"flash_attn_fp4 serves head_dim 128 here; got {shape.d}")
    if not shape.varlen and (shape.s_q % 128 or shape.s_k % 128):
        _fail(27, ValueError, f"flash_attn_fp4 needs seqlen % 128 == 0; got {shape.s_q} / {shape.s_k}")
    rows = []

    def log(f, val, why):
        rows.append((f, str(val), why))
        return val
    had, scaling, rowlocal, ragged = _common("fp4", shape, log, causal=causal, window_size=window_size, softcap=softcap,
                                             score_mod=score_mod, score_mod_bwd=score_mod_bwd, mask_mod=mask_mod,
                                             seqused_k=seqused_k, deterministic=deterministic, qk_hadamard=qk_hadamard,
                                             opts=o)
    if scaling == "token_local":
        _fail("B6", NotImplementedError, "operand_scaling='token_local' is built on flash_attn_fp8 only")
    p_frame = _p_frame("fp4", o, shape, scaling, default="group")
    log("p_hat_frame", p_frame, "auto: one UE8M0 exponent per query row and 32 keys of P-hat" if o.p_hat_frame == "auto"
        else "explicit")
    log("backward_kernel", "1cta", "the 1-CTA backward; S recomputed from the forward's NVFP4 codes")
    return _finish("fp4", "fp4.e4m3_pv", "nvfp4", shape, rows, o, softmax_scale=softmax_scale, causal=causal,
                   return_lse=return_lse, had=had, scaling=scaling, rowlocal=rowlocal, ragged=ragged, dq_causal=False,
                   window_size=window_size, p_frame=p_frame,
                   seqused_k=seqused_k is not None and not shape.aligned_varlen, softcap=softcap,
                   deterministic=deterministic)
