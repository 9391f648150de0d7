"""flash_attn_fp8 on operands that are already E4M3 (FlashAttention-3's convention), at the reference's module name
(flash_attn/cute/lowprec/prequant_fa3.py; docs/lowprec.md:97-137).

    flash_attn_fp8(q8, k8, v8, q_descale=dq, k_descale=dk, v_descale=dv, grad_proxies=(q, k, v), causal=True)

x ~= code * descale[b, kv_head]: one float32 (or float64) scale per (batch row, kv head); the q heads of a GQA group share
their kv head's q_descale. No Q / K / V quantiser runs: the kernels read the caller's codes, the descales fill the
factor tables (the score scale takes them as floats; a block-scaled product takes a factor's exponent, and its mantissa
is multiplied in afterwards: on O for V, on dK for Q, on dQ for K). dO is quantised by the library, in the launch that also
writes D, the shifted LSE and the zeroed f16 dQ accumulator; the f16 dQ pre-scale is sized from one read of the K / V codes.
E4M3 leaves cannot take gradients: pass detached codes and grad_proxies=(q, k, v) (bf16 / f16, the codes' shapes), whose
.grad receives the straight-through gradient.

Served: the batched (b, s, h, d) form with s_q % 128 == 0 and s_k % 128 == 0, head_dim 64 / 128, causal or dense, sliding
window, softcap, batched seqused_k, deterministic, MHA / GQA, return_lse. Refused, each with its rule: packed forms,
token-local / row-local options, qk_hadamard=True (the codes are unrotated), q_quantized / q_scale_fused beside the descales.
"""
from __future__ import annotations

import dataclasses

import torch

from . import _routes
from .plan import _fail


def _validate(q, k, v, descs, proxies):
    for n, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor) or t.dtype != torch.float8_e4m3fn:
            _fail(32, TypeError, f"flash_attn_fp8 with q_descale / k_descale / v_descale takes q, k, v as "
                                 f"torch.float8_e4m3fn codes; {n} is {getattr(t, 'dtype', type(t).__name__)}")
        if t.requires_grad:
            _fail(32, ValueError, f"E4M3 {n} requires grad: PyTorch would cast its gradient to E4M3. Pass detached codes "
                                  "and grad_proxies=(q, k, v)")
    if any(d is None for d in descs):
        _fail(32, ValueError, "pre-quantised E4M3 inputs need q_descale, k_descale and v_descale (all three)")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        _fail("B7", NotImplementedError, "pre-quantised E4M3 inputs are served on the batched (b, s, h, d) form")
    b, h_kv = q.shape[0], k.shape[2]
    for n, d in zip(("q_descale", "k_descale", "v_descale"), descs):
        if not isinstance(d, torch.Tensor) or d.dtype not in (torch.float32, torch.float64) or tuple(d.shape) != (b, h_kv):
            _fail(32, ValueError, f"{n} is a float32 / float64 tensor of shape (batch, kv heads) = ({b}, {h_kv}); got "
                                  f"{tuple(d.shape) if isinstance(d, torch.Tensor) else type(d).__name__} "
                                  f"{getattr(d, 'dtype', '')}")
        if d.device != q.device:
            _fail(32, ValueError, f"{n} is on {d.device}, the codes on {q.device}")
    if proxies is not None:
        if not isinstance(proxies, (tuple, list)) or len(proxies) != 3:
            _fail(32, ValueError, "grad_proxies is a tuple (q, k, v) of bf16 / f16 tensors of the codes' shapes")
        for n, p_, t in zip(("q", "k", "v"), proxies, (q, k, v)):
            if not isinstance(p_, torch.Tensor) or p_.dtype not in (torch.bfloat16, torch.float16) or p_.shape != t.shape:
                _fail(32, ValueError, f"grad_proxies[{n}] must be bf16 / f16 of shape {tuple(t.shape)}")
        if len({p_.dtype for p_ in proxies}) != 1:
            _fail(32, ValueError, "grad_proxies must share one dtype")


def mantissa(f):
    """f / 2^floor(log2 f) in [1, 2): what is left of a factor once a block-scaled product has taken its exponent."""
    m, _e = torch.frexp(f.float())          # f = m 2^e, m in [0.5, 1)
    return (m * 2.0).contiguous()


class _PrequantAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pq, pk, pv, q8, k8, v8, qd, kd, vd, plan, seqused_k):
        out, lse, state = _routes.forward(plan, q8, k8, v8, None, seqused_k, prequant=(qd, kd, vd))
        ctx.plan = plan
        ctx.save_for_backward(*state)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        dq, dk, dv = _routes.backward(ctx.plan, list(ctx.saved_tensors), dout.contiguous(), None)
        return dq, dk, dv, None, None, None, None, None, None, None, None


def flash_attn_fp8_prequant(resolve, q, k, v, q_descale, k_descale, v_descale, grad_proxies, kw, return_lse):
    """The body of a flash_attn_fp8 call with E4M3 inputs. kw: the call's remaining keyword arguments for the resolver."""
    _validate(q, k, v, (q_descale, k_descale, v_descale), grad_proxies)
    if kw.get("cu_seqlens_q") is not None or kw.get("cu_seqlens_k") is not None or kw.get("seqused_q") is not None:
        _fail("B7", NotImplementedError, "pre-quantised E4M3 inputs are served on the batched form, not with cu_seqlens")
    if kw.get("qk_hadamard"):
        _fail(32, ValueError, "qk_hadamard=True with pre-quantised inputs: the codes are unrotated (None resolves to off)")
    if kw.get("q_quantized") is not None or kw.get("k_quantized") is not None or kw.get("q_scale_fused"):
        _fail(32, ValueError, "q_quantized / k_quantized / q_scale_fused do not go with q_descale / k_descale / v_descale")
    if q.shape[1] % 128 or k.shape[1] % 128:
        _fail("B7", NotImplementedError, "pre-quantised E4M3 inputs need s_q % 128 == 0 and s_k % 128 == 0; got "
                                         f"{q.shape[1]} and {k.shape[1]}")
    want_grad = grad_proxies is not None and torch.is_grad_enabled() and any(p_.requires_grad for p_ in grad_proxies)
    dt = grad_proxies[0].dtype if grad_proxies is not None else torch.bfloat16
    meta = [torch.empty(t.shape, dtype=dt, device="meta", requires_grad=want_grad) for t in (q, k, v)]
    kw = dict(kw, qk_hadamard=False)
    plan = resolve(*meta, **kw)
    if plan.pad_from:
        _fail("B7", NotImplementedError, f"pre-quantised E4M3 inputs are served at head_dim 64 / 128; got {plan.pad_from}")
    if plan.fwd.operand_scaling != "token_block" or plan.bwd.ds_dq_rowlocal != "off":
        _fail(32, ValueError, "block-scaled operand_scaling / ds_dq_rowlocal options do not go with pre-quantised inputs: "
                              "the operands' scaling is the caller's")
    bwd = plan.bwd if plan.bwd.dq_prescale != "causal_row" else dataclasses.replace(plan.bwd, dq_prescale="causal_tile")
    plan = dataclasses.replace(plan, prequant=True, bwd=bwd)
    if not q.is_cuda:
        raise RuntimeError("flash_attn_fp8: q, k, v must be CUDA tensors (this library has no CPU path)")
    qd, kd, vd = (d.to(torch.float32).contiguous() for d in (q_descale, k_descale, v_descale))
    su_k = kw.get("seqused_k")
    su_k = su_k.contiguous() if plan.fwd.seqused_k else None
    pq, pk, pv = grad_proxies if want_grad else (None, None, None)
    out, lse = _PrequantAttn.apply(pq, pk, pv, q.contiguous(), k.contiguous(), v.contiguous(), qd, kd, vd, plan, su_k)
    return (out, lse) if return_lse else out
