"""Public entry points flash_attn_fp8 / flash_attn_fp4: same signatures, defaults, return values and refusal convention
as the reference's flash_attn/cute/lowprec/api.py (flash_attn_fp4 :169, flash_attn_fp8 :270). Each call resolves one
immutable plan (cached per argument values and tensor metadata) before anything is quantised or launched, then runs the
registered op lowbit_attn::fp8 / ::fp4, whose autograd node carries the plan handle to the backward.
"""
from __future__ import annotations

import functools
import warnings
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch

from . import _op
from .options import FP4AttnOptions, FP8AttnOptions
from .plan import AttnPlan, _fail, resolve_fp4, resolve_fp8

__all__ = ["flash_attn_fp4", "flash_attn_fp8"]

_REPACK_WARNED = False
REPACK_WARNING = (
    "flash_attn_{entry} got cu_seqlens_q / cu_seqlens_k without seqused_q / seqused_k. No tensor is copied (the kernels "
    "read and write the packed rows in place), but the document tables are rebuilt on the device on every call (a dozen "
    "small launches) and the intermediates take a padded buffer of up to 127 extra rows per document. Build the tables "
    "once with DocMaps.from_cu_seqlens(...) and pass doc_maps=, or lay the documents out at starts that are multiples of "
    "128 and pass the true lengths as seqused_q / seqused_k. (Warned once.)")


@dataclass(frozen=True)
class _TensorFacts:
    """What plan resolution may look at in a tensor argument: nothing but metadata."""
    shape: Tuple[int, ...]
    dtype: torch.dtype
    requires_grad: bool

    @staticmethod
    def of(t):
        return _TensorFacts(tuple(t.shape), t.dtype, bool(t.requires_grad)) if isinstance(t, torch.Tensor) else t

    def stand_in(self):
        grad = self.requires_grad and self.dtype.is_floating_point
        return torch.empty(self.shape, dtype=self.dtype, device="meta", requires_grad=grad)


@dataclass(frozen=True)
class _CallFacts:
    """Hashable description of one call: everything a plan depends on and nothing else."""
    entry: str
    grad_mode: bool
    dq_causal_prescale: Tuple[bool, str]      # the module switches the resolver reads: (on, granularity)
    q: _TensorFacts
    k: _TensorFacts
    v: _TensorFacts
    keywords: Tuple[Tuple[str, object], ...]


@functools.lru_cache(maxsize=1024)
def _plan_of(facts: _CallFacts) -> AttnPlan:
    # plans are pure functions of argument values and tensor metadata, so they are resolved on meta stand-ins; a refusal
    # raises out of here and is not remembered
    resolve = resolve_fp8 if facts.entry == "fp8" else resolve_fp4
    kw = {n: (x.stand_in() if isinstance(x, _TensorFacts) else x) for n, x in facts.keywords}
    with torch.set_grad_enabled(facts.grad_mode):
        return resolve(facts.q.stand_in(), facts.k.stand_in(), facts.v.stand_in(), **kw)


def _cached_plan(resolve, q, k, v, kw) -> AttnPlan:
    from . import interface_bwd_fp4
    entry = "fp8" if resolve is resolve_fp8 else "fp4"
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v)):
        return resolve(q, k, v, **kw)           # the resolver words the refusal
    facts = _CallFacts(entry, torch.is_grad_enabled(),
                       (bool(interface_bwd_fp4.DQ_CAUSAL_PRESCALE), str(interface_bwd_fp4.DQ_CAUSAL_GRANULARITY)), _TensorFacts.of(q),
                       _TensorFacts.of(k), _TensorFacts.of(v), tuple(sorted((n, _TensorFacts.of(x)) for n, x in kw.items())))
    try:
        return _plan_of(facts)
    except TypeError as exc:
        if getattr(exc, "rule", None) is not None:
            raise
        return resolve(q, k, v, **kw)           # an unhashable argument (e.g. a callable object): resolve uncached


def _doc_maps_args(maps, q, cu_q, cu_k, su_q, su_k):
    """doc_maps= stands for the varlen arguments: the plan is resolved as for cu_seqlens = maps.cu."""
    from .docmaps import DocMaps
    if not isinstance(maps, DocMaps):
        _fail("B9", TypeError, f"doc_maps must be a DocMaps; got {type(maps).__name__}")
    if cu_q is not None or cu_k is not None or su_q is not None or su_k is not None:
        _fail("B9", ValueError, "doc_maps carries the documents: do not pass cu_seqlens_* / seqused_* with it")
    if isinstance(q, torch.Tensor) and (q.dim() != 3 or q.shape[0] != maps.total):
        _fail("B9", ValueError, f"doc_maps describes {maps.total} packed rows; q is {tuple(q.shape)}")
    if isinstance(q, torch.Tensor) and q.is_cuda and maps.device != q.device:
        _fail("B9", ValueError, f"doc_maps is on {maps.device}, q on {q.device}: move the maps with .to(device)")
    return maps.cu, maps.cu, maps.max_seqlen, maps.max_seqlen


def _run(plan, q, k, v, cu_q, cu_k, su_q, su_k, return_lse, doc_maps=None):
    global _REPACK_WARNED
    if not q.is_cuda:
        raise RuntimeError(f"flash_attn_{plan.entry}: q, k, v must be CUDA tensors (this library has no CPU path)")
    sh = plan.shape
    if sh.varlen and sh.tot_q != sh.tot_k:
        _fail("B8", NotImplementedError, "packed documents are self-attention documents here: q and k must share "
                                         "cu_seqlens (total_q == total_k)")
    if sh.varlen:
        # the kernels walk ONE document table (built from cu_seqlens_q / seqused_q): the key side must be the same
        # tensor, otherwise a call with different key documents would silently run as self-attention over q's table
        for a, b_, name in ((cu_q, cu_k, "cu_seqlens"), (su_q, su_k, "seqused")):
            if a is None or b_ is None or a is b_:
                continue
            if tuple(a.shape) != tuple(b_.shape) or a.data_ptr() != b_.data_ptr():
                _fail("B8", NotImplementedError, f"packed documents are self-attention documents here: pass the SAME tensor "
                                                 f"as {name}_q and {name}_k (distinct query / key tables are not built)")
    if plan.fwd.ragged_documents and sh.s_q != sh.s_k:
        _fail("B8", NotImplementedError, "lengths that are no multiple of 128 run the batch rows as self-attention "
                                         f"documents: s_q must equal s_k; got {sh.s_q} and {sh.s_k}")
    if sh.varlen and not sh.aligned_varlen and doc_maps is None and not _REPACK_WARNED:
        _REPACK_WARNED = True
        warnings.warn(REPACK_WARNING.format(entry=plan.entry), UserWarning, stacklevel=3)
    if doc_maps is not None:
        docs = doc_maps.tensors()           # cu, start, len, row_map, slot_src, slot_rows: nothing is computed per call
    else:
        docs = [t for t in (cu_q, cu_k, su_q, su_k) if t is not None] if sh.varlen else \
            ([su_k.contiguous()] if plan.fwd.seqused_k else [])
    if plan.pad_from:
        # head dim below the kernels' 64 / 128: zero columns on the way in (differentiable: the gradients of the pad
        # are the first head_dim columns of dQ / dK / dV), the first head_dim columns of O on the way out
        extra = sh.d - plan.pad_from
        q, k, v = (torch.nn.functional.pad(t, (0, extra)) for t in (q, k, v))
    out, lse = _op.op_apply(plan, q, k, v, docs)
    if plan.pad_from:
        out = out[..., :plan.pad_from].contiguous()
    if return_lse:
        if lse.numel() == 0:
            _fail("B8", ValueError, "return_lse is served on the batched and the aligned varlen forms, not under "
                                    "repacked documents")
        return out, lse
    return out


def flash_attn_fp8(q, k, v, *, softmax_scale: Optional[float] = None, causal: bool = False,
                   window_size: Tuple[Optional[int], Optional[int]] = (None, None), softcap: float = 0.0,
                   score_mod: Optional[Callable] = None, score_mod_bwd: Optional[Callable] = None,
                   mask_mod: Optional[Callable] = None, aux_tensors: Optional[tuple] = None,
                   cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q: Optional[int] = None,
                   max_seqlen_k: Optional[int] = None, seqused_k=None, seqused_q=None, deterministic: bool = False,
                   return_lse: bool = False, qk_hadamard: Optional[bool] = None, q_quantized=None, k_quantized=None,
                   q_scale_fused: bool = False, options: Optional[FP8AttnOptions] = None, q_descale=None, k_descale=None,
                   v_descale=None, grad_proxies=None, doc_maps=None):
    """8-bit (MXFP8) attention, forward and backward, on B200.

    q: (b, s, h, d); k, v: (b, s, h_kv, d); bf16 or f16; h % h_kv == 0; d in {64, 128}, or another multiple of 16 below
    128 (run padded with zero columns to the next of 64 / 128). Packed (total, h, d) with
    cu_seqlens_q / cu_seqlens_k (repacked), or with seqused_q / seqused_k as well (aligned, zero-copy: starts multiples of
    128). Returns out (dtype and shape of q); with return_lse=True (out, lse) with lse (b, h, s) float32 in nats,
    non-differentiable ((h, total_q) in the caller's row order on the packed forms). causal is bottom-right aligned.
    E4M3 Q, K, V, dO with one UE8M0 exponent per 32 tokens x the whole head dim; qk_hadamard=None turns the random-sign
    Hadamard rotation of Q / K on at d = 128. Every unserved combination raises with a `.rule` before any launch."""
    if doc_maps is not None:
        cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k = _doc_maps_args(doc_maps, q, cu_seqlens_q, cu_seqlens_k,
                                                                                seqused_q, seqused_k)
    if aux_tensors is not None:
        _fail("B3", NotImplementedError, "aux_tensors belong to score_mod / mask_mod, which this library does not take")
    if q_descale is not None or k_descale is not None or v_descale is not None or grad_proxies is not None or \
            (isinstance(q, torch.Tensor) and q.dtype == torch.float8_e4m3fn):
        if doc_maps is not None:
            _fail("B7", NotImplementedError, "pre-quantised E4M3 inputs are served on the batched form, not with doc_maps")
        from .prequant_fa3 import flash_attn_fp8_prequant
        return flash_attn_fp8_prequant(resolve_fp8, q, k, v, q_descale, k_descale, v_descale, grad_proxies, dict(
            softmax_scale=softmax_scale, causal=causal, window_size=tuple(window_size), softcap=softcap,
            score_mod=score_mod, score_mod_bwd=score_mod_bwd, mask_mod=mask_mod, cu_seqlens_q=cu_seqlens_q,
            cu_seqlens_k=cu_seqlens_k, max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k, seqused_k=seqused_k,
            seqused_q=seqused_q, deterministic=deterministic, return_lse=return_lse, qk_hadamard=qk_hadamard,
            q_quantized=q_quantized, k_quantized=k_quantized, q_scale_fused=q_scale_fused, options=options), return_lse)
    plan = _cached_plan(resolve_fp8, q, k, v, dict(
        softmax_scale=softmax_scale, causal=causal, window_size=tuple(window_size), softcap=softcap, score_mod=score_mod,
        score_mod_bwd=score_mod_bwd, mask_mod=mask_mod, cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k,
        max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k, seqused_k=seqused_k, seqused_q=seqused_q,
        deterministic=deterministic, return_lse=return_lse, qk_hadamard=qk_hadamard, q_quantized=q_quantized,
        k_quantized=k_quantized, q_scale_fused=q_scale_fused, options=options))
    return _run(plan, q, k, v, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k, return_lse, doc_maps)


def flash_attn_fp4(q, k, v, *, softmax_scale: Optional[float] = None, causal: bool = False,
                   window_size: Tuple[Optional[int], Optional[int]] = (None, None), softcap: float = 0.0,
                   score_mod: Optional[Callable] = None, score_mod_bwd: Optional[Callable] = None,
                   mask_mod: Optional[Callable] = None, aux_tensors: Optional[tuple] = None,
                   cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q: Optional[int] = None,
                   max_seqlen_k: Optional[int] = None, seqused_k=None, seqused_q=None, deterministic: bool = False,
                   return_lse: bool = False, pv_precision: str = "fp8", backward: str = "e4m3",
                   causal_safety: str = "auto", qk_hadamard: Optional[bool] = None,
                   options: Optional[FP4AttnOptions] = None, q_descale=None, k_descale=None, v_descale=None,
                   doc_maps=None):
    """Mixed NVFP4 / FP8 attention, forward and backward, on B200: Q.K^T and its recomputation in the backward on NVFP4
    codes (E2M1, one E4M3 scale per 16 along d); P.V, dP, dV, dK, dQ on E4M3 token blocks. Arguments, shapes and returns
    as flash_attn_fp8; d = 128. With qk_hadamard on (default) the NVFP4 codes are of the rotated rows, the E4M3 copies of
    the rows as given."""
    if doc_maps is not None:
        cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k = _doc_maps_args(doc_maps, q, cu_seqlens_q, cu_seqlens_k,
                                                                                seqused_q, seqused_k)
    if q_descale is not None or k_descale is not None or v_descale is not None or \
            any(isinstance(t, torch.Tensor) and t.dtype == torch.float8_e4m3fn for t in (q, k, v)):
        _fail("B7", TypeError, "flash_attn_fp4 takes bf16 / f16 inputs: pre-quantised E4M3 inputs are a flash_attn_fp8 "
                               "feature of the reference and are not built here")
    if aux_tensors is not None:
        _fail("B3", NotImplementedError, "aux_tensors belong to score_mod / mask_mod, which this library does not take")
    plan = _cached_plan(resolve_fp4, q, k, v, dict(
        softmax_scale=softmax_scale, causal=causal, window_size=tuple(window_size), softcap=softcap, score_mod=score_mod,
        score_mod_bwd=score_mod_bwd, mask_mod=mask_mod, cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k,
        max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k, seqused_k=seqused_k, seqused_q=seqused_q,
        deterministic=deterministic, return_lse=return_lse, pv_precision=pv_precision, backward=backward,
        causal_safety=causal_safety, qk_hadamard=qk_hadamard, options=options))
    return _run(plan, q, k, v, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k, return_lse, doc_maps)
