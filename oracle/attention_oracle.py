"""CPU oracle of the attention path (TEST INFRASTRUCTURE, not product code).

Restates, in plain PyTorch on the CPU, the two pieces the reference composes for its "quantise-dequantise emulation":

  * fp32 attention forward + backward with a bottom-right aligned causal mask and GQA by repeating K / V
    -- benchmarks/benchmark_lowprec_attn.py:889-922 (`reference`) and, for packed documents,
       benchmarks/benchmark_packed_docs.py:75-114 (`reference_docs`) of the reference;
  * the accuracy figures of the reference benchmark -- benchmarks/benchmark_lowprec_attn.py:935-939 (`accuracy`) --
    plus the relative L2 error.

qdq_attention() = quantise Q, K, V, dO with the quantiser oracle (token-block MXFP8, optionally NVFP4 for the S operands)
-> dequantise -> fp32 attention. The roundings of P-hat and dS-hat inside the kernels are not emulated (fp32 softmax).
Parity pin: the quantiser part is pinned byte-for-byte by tests/test_oracle_golden.py; attention_fp32,
attention_docs_fp32 and accuracy are pinned by tests/test_oracle_attention.py against tests/golden/attention_small.npz,
written by tests/golden/make_golden_attention.py from the reference's own `reference`, `reference_docs`, `accuracy`
and (rectangular / bottom-right causal cases) tests/cute/test_lowprec_api.py:1346 `_ref_bottom_right`, run on CPU.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import quant_oracle as Q


def attention_fp32(q, k, v, g=None, causal=False, softmax_scale=None, chunk=1024, q_grad=None, k_grad=None,
                   window=None, seqused_k=None, softcap=0.0):
    """q (b, s_q, h, d), k / v (b, s_k, h_kv, d) float32 CPU tensors -> (o, lse, dq, dk, dv); lse (b, h, s_q) in nats.
    Causal: key j visible to query i iff j <= i + (s_k - s_q). g = dO or None (forward only).
    q_grad / k_grad: the copies of Q / K used as operands of dK = dS^T Q and dQ = dS K when they differ from the S
    operands (the mixed route: S from the NVFP4 copies, gradient GEMMs from the E4M3 copies).
    window = (left, right), None = unlimited: key j visible iff i + off - left <= j <= i + off + right (causal caps the
    right side at 0). seqused_k: per batch row the number of valid keys (keys at or past it are masked; the causal
    alignment keeps using s_k - s_q), as tests/cute/test_lowprec_api.py:1346 `_ref_bottom_right` of the reference.
    softcap c > 0: the scaled scores become c tanh(score / c) before masking, and dS takes the factor 1 - tanh^2
    (flash_attn/cute/utils.py:167-187, tests/cute/test_lowprec_api.py:1118 `_ref_attn`)."""
    q, k, v = q.float(), k.float(), v.float()
    qg = q if q_grad is None else q_grad.float()
    kg = k if k_grad is None else k_grad.float()
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    grp = h // hk
    sc = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)
    kr, vr = k.repeat_interleave(grp, 2), v.repeat_interleave(grp, 2)
    kgr = kg.repeat_interleave(grp, 2)
    o = torch.zeros_like(q)
    lse = torch.zeros(b, h, sq)
    bwd = g is not None
    dq = torch.zeros_like(q) if bwd else None
    dk = torch.zeros(b, sk, h, d) if bwd else None
    dv = torch.zeros(b, sk, h, d) if bwd else None
    off = sk - sq
    for bi in range(b):
        for hi in range(h):
            Qm, Km, Vm = q[bi, :, hi], kr[bi, :, hi], vr[bi, :, hi]
            for r0 in range(0, sq, chunk):
                S = (Qm[r0:r0 + chunk] @ Km.T) * sc
                dcap = None
                if softcap:
                    th = torch.tanh(S / float(softcap))
                    S = float(softcap) * th
                    dcap = 1.0 - th * th
                wl, wr = (None, None) if window is None else window
                if causal:
                    wr = 0
                if wl is not None or wr is not None:
                    rr = torch.arange(r0, r0 + S.shape[0])[:, None]
                    cc = torch.arange(sk)[None, :]
                    if wr is not None:
                        S = S.masked_fill(cc > rr + off + wr, float("-inf"))
                    if wl is not None:
                        S = S.masked_fill(cc < rr + off - wl, float("-inf"))
                if seqused_k is not None:
                    S = S.masked_fill(torch.arange(sk)[None, :] >= int(seqused_k[bi]), float("-inf"))
                L = torch.logsumexp(S, -1)
                lse[bi, hi, r0:r0 + chunk] = L
                P = torch.exp(S - torch.where(torch.isinf(L), torch.zeros_like(L), L)[:, None])
                P = torch.where(torch.isinf(L)[:, None], torch.zeros_like(P), P)
                O = P @ Vm
                o[bi, r0:r0 + chunk, hi] = O
                if bwd:
                    dO = g[bi, r0:r0 + chunk, hi].float()
                    dS = P * (dO @ Vm.T - (dO * O).sum(-1, keepdim=True))
                    if dcap is not None:
                        dS = dS * dcap
                    dq[bi, r0:r0 + chunk, hi] = (dS @ kgr[bi, :, hi]) * sc
                    dk[bi, :, hi] += (dS.T @ qg[bi, r0:r0 + chunk, hi]) * sc
                    dv[bi, :, hi] += P.T @ dO
    if bwd and grp > 1:
        dk, dv = (t.view(b, sk, hk, grp, d).sum(3) for t in (dk, dv))
    return o, lse, dq, dk, dv


def attention_docs_fp32(q, k, v, g, lengths, causal=True, softmax_scale=None):
    """Packed (total, h, d) tensors with documents of the given lengths: attention inside each document only."""
    outs = [torch.zeros_like(q.float()), torch.zeros(q.shape[1], q.shape[0]), *(torch.zeros_like(t.float()) for t in (q, k, v))]
    pos = 0
    for n in lengths:
        sl = slice(pos, pos + n)
        r = attention_fp32(q[None, sl], k[None, sl], v[None, sl], None if g is None else g[None, sl], causal, softmax_scale)
        outs[0][sl] = r[0][0]
        outs[1][:, sl] = r[1][0]
        if g is not None:
            outs[2][sl], outs[3][sl], outs[4][sl] = r[2][0], r[3][0], r[4][0]
        pos += n
    return tuple(outs)


def _qdq8(x, rotate=False, token_local=False):
    r = Q.fp8_token_blocks(x.float().numpy(), rotate=rotate, token_local=token_local)
    if token_local:
        sc = r["token_factors"].transpose(0, 2, 1)[..., None]          # (b, s, h, 1)
        deq = Q.e4m3_decode(r["codes"]) * sc
    else:
        deq = Q.fp8_dequant(r["codes"], r["e"])
    return torch.from_numpy(np.ascontiguousarray(deq, dtype=np.float32))


def _qdq4(x, rotate=False):
    r = Q.nvfp4_rows(x.float().numpy(), rotate=rotate)
    return torch.from_numpy(Q.nvfp4_dequant(r["codes"], r["sf_table"]))


def qdq_attention(q, k, v, g=None, *, causal=False, softmax_scale=None, fp4_qk=False, rotate_qk=False,
                  token_local=False, window=None, seqused_k=None, softcap=0.0):
    """The quantise-dequantise emulation: MXFP8 (token-block) Q, K, V, dO -> fp32 attention. fp4_qk: the S operands are
    the NVFP4 codes of Q, K instead (the mixed route's forward and S recompute; dP / dV / dK / dQ keep the E4M3 copies --
    emulated here by using the NVFP4 values for S and the E4M3 values for the gradient GEMMs' Q / K operands).
    rotate_qk: the Q / K operands are quantised after the Hadamard rotation; (QR)(KR)^T = QK^T, so the emulation rotates
    back after dequantising. Inputs bf16 / fp32 CPU tensors (b, s, h, d)."""
    def back(t):
        return torch.from_numpy(Q.hadamard_unrotate(t.numpy())) if rotate_qk else t
    q8 = back(_qdq8(q, rotate_qk, token_local))
    k8 = back(_qdq8(k, rotate_qk, token_local))
    v8 = _qdq8(v, False, token_local)
    g8 = _qdq8(g, False, token_local) if g is not None else None
    if not fp4_qk:
        return attention_fp32(q8, k8, v8, g8, causal, softmax_scale, window=window, seqused_k=seqused_k, softcap=softcap)
    q4, k4 = back(_qdq4(q, rotate_qk)), back(_qdq4(k, rotate_qk))
    # forward and P from the 4-bit S operands; with rotation on only the 4-bit copies are rotated on this route, so the
    # E4M3 copies for the gradient GEMMs are those of the unrotated rows
    q8u, k8u = (q8, k8) if not rotate_qk else (_qdq8(q, False, token_local), _qdq8(k, False, token_local))
    return attention_fp32(q4, k4, v8, g8, causal, softmax_scale, q_grad=q8u, k_grad=k8u, window=window, seqused_k=seqused_k,
                          softcap=softcap)


def accuracy(x, ref):
    """cosine, norm ratio, max / mean relative error with the floor 1e-3 * max|ref| (the reference benchmark's four figures),
    plus the relative L2 error and the largest absolute error in units of max|ref| (`max_abs`)."""
    p, r = x.detach().float().flatten().double(), ref.detach().float().flatten().double()
    floor = max(float(r.abs().max()) * 1e-3, 1e-30)
    rel = (p - r).abs() / r.abs().clamp_min(floor)
    return dict(cos=float(p @ r / (p.norm() * r.norm() + 1e-30)), norm_ratio=float(p.norm() / (r.norm() + 1e-30)),
                max_rel_err=float(rel.max()), mean_rel_err=float(rel.mean()),
                rel_l2=float((p - r).norm() / (r.norm() + 1e-30)),
                max_abs=float((p - r).abs().max() / (r.abs().max() + 1e-30)))
