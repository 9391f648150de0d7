"""GPU: the benchmark configurations at their full sizes, through size-independent properties.

The oracle cannot finish these sizes in seconds, so the checks are: (1) sharding invariance -- every (batch, kv-head
group) is an independent problem with scales local to it, so running one slice alone must reproduce O, LSE, dK and dV of
the full run bit for bit (this is also what makes the multi-GPU split exact) and dQ up to the f16 reduce-add order;
(2) run-to-run determinism of O / LSE / dK / dV; (3) everything finite; (4) one (batch row, kv group) slice of every
configuration, and two documents of the packed one, against the oracle AT THAT SIZE: the quantise-dequantise emulation
(rel-L2 bounds of tests/test_gpu_bwd.py) and fp32 attention on the unquantised inputs (1.05 x the error implied by the
reference's published cosines, docs/lowprec.md:583, and the max-abs bounds MAX_ABS below)."""
import math

import pytest
import torch

from inputs import attention_inputs, packed_doc_lengths
from oracle import attention_oracle as A

pytestmark = pytest.mark.gpu

# reference's published cosines against fp32 attention at b4 s4096 h16 d128 causal (docs/lowprec.md:583), per route
PUBLISHED_COS = {"fp8": dict(o=0.9988, dq=0.9979, dk=0.9979, dv=0.9987), "fp4": dict(o=0.9920, dq=0.9906, dk=0.9906, dv=0.9919)}
# stated max-abs bounds: largest |x - fp32 reference| in units of max|reference|, per route (N(0, 1) inputs)
MAX_ABS = {"fp8": 0.10, "fp4": 0.20}


def _against_oracles(route, got, q, k, v, g, *, rotate=True, token_local=False, qdq_tol=5e-2, published=True):
    """got = (o, dq, dk, dv) of one slice; q, k, v, g its CPU inputs (b, s, h, d)."""
    names = ("o", "dq", "dk", "dv")
    r32 = A.attention_fp32(q.float(), k.float(), v.float(), g.float(), True)
    rq = A.qdq_attention(q, k, v, g, causal=True, rotate_qk=rotate, fp4_qk=route == "fp4", token_local=token_local)
    for n, x, a32, aq in zip(names, got, (r32[0], r32[2], r32[3], r32[4]), (rq[0], rq[2], rq[3], rq[4])):
        x = x.float().cpu()
        e_q, e_32 = A.accuracy(x, aq), A.accuracy(x, a32)
        print(f"full-size {route} {n}: vs QDQ rel_l2 {e_q['rel_l2']:.4f}; vs fp32 rel_l2 {e_32['rel_l2']:.4f} cos {e_32['cos']:.5f} "
              f"max_abs {e_32['max_abs']:.4f}")
        assert e_q["rel_l2"] < qdq_tol, (n, e_q)
        if published:
            assert e_32["rel_l2"] <= 1.05 * math.sqrt(2 * (1 - PUBLISHED_COS[route][n])), (n, e_32)
            assert e_32["max_abs"] <= MAX_ABS[route], (n, e_32)


def _run(fn, q, k, v, g, **kw):
    qc, kc, vc = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out = fn(qc, kc, vc, **kw)
    out.backward(g)
    torch.cuda.synchronize()
    return out.detach(), qc.grad, kc.grad, vc.grad


def _close(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-30))


@pytest.mark.parametrize("route,causal", [("fp8", True), ("fp8", False), ("fp4", True)])
def test_headline_cell_sharding_invariance(route, causal):
    """b4 s4096 h16 d128 (configurations 2 and 3)."""
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    q, k, v, g = (t.cuda() for t in attention_inputs(4, 4096, 16, 16, 128, seed=0))
    o, dq, dk, dv = _run(fn, q, k, v, g, causal=causal)
    o2, dq2, dk2, dv2 = _run(fn, q, k, v, g, causal=causal)
    assert torch.equal(o, o2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)
    assert _close(dq, dq2) < 5e-3       # f16 adds in arrival order, then a bf16 rounding (2^-9) that may flip
    for t in (o, dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    # one (batch row, head) alone: same bytes
    bi, hi = 2, 5
    sl = lambda t: t[bi:bi + 1, :, hi:hi + 1].contiguous()
    os_, dqs, dks, dvs = _run(fn, sl(q), sl(k), sl(v), sl(g), causal=causal)
    assert torch.equal(os_, sl(o)) and torch.equal(dks, sl(dk)) and torch.equal(dvs, sl(dv))
    assert _close(dqs, sl(dq)) < 8e-3      # the f16 pre-scale is per batch row over all heads: a different power of two
    if causal:      # configurations 2 and 3 at their own size: one (batch row, head) against both oracles
        _against_oracles(route, (os_, dqs, dks, dvs), *(sl(t).cpu() for t in (q, k, v, g)))


def test_gqa_token_local_configuration_full_size():
    """b2 s8192 h32 h_kv8 d128 causal, token-local scales, row-local dQ side, causal dQ pre-scale, 1 % of the
    (head, channel) pairs of Q and K scaled x20 (configuration 4)."""
    import flamia_blackwell_attention_b200 as F
    import flamia_blackwell_attention_b200.interface_bwd_fp4 as I
    q, k, v, g = (t.cuda() for t in attention_inputs(2, 8192, 32, 8, 128, seed=0, outlier_channels=True))
    opts = F.FP8AttnOptions(operand_scaling="token_local", ds_dq_rowlocal="all")
    old = I.DQ_CAUSAL_PRESCALE
    I.DQ_CAUSAL_PRESCALE = True
    try:
        o, dq, dk, dv = _run(F.flash_attn_fp8, q, k, v, g, causal=True, options=opts)
        o2, dq2, dk2, dv2 = _run(F.flash_attn_fp8, q, k, v, g, causal=True, options=opts)
        # one kv head with its four query heads, one batch row
        bi, hk = 1, 3
        qs, gs = (t[bi:bi + 1, :, 4 * hk:4 * hk + 4].contiguous() for t in (q, g))
        ks, vs = (t[bi:bi + 1, :, hk:hk + 1].contiguous() for t in (k, v))
        os_, dqs, dks, dvs = _run(F.flash_attn_fp8, qs, ks, vs, gs, causal=True, options=opts)
    finally:
        I.DQ_CAUSAL_PRESCALE = old
    assert torch.equal(o, o2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)
    for t in (o, dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    assert torch.equal(os_, o[bi:bi + 1, :, 4 * hk:4 * hk + 4])
    assert torch.equal(dks, dk[bi:bi + 1, :, hk:hk + 1]) and torch.equal(dvs, dv[bi:bi + 1, :, hk:hk + 1])
    assert _close(dqs, dq[bi:bi + 1, :, 4 * hk:4 * hk + 4]) < 8e-3
    # the slice at its own size against the oracle's token-local emulation (outlier channels make near one-hot rows, where
    # the E4M3 roundings of P-hat / dS-hat weigh more: the bound is the small-case bound of tests/test_gpu_api.py)
    _against_oracles("fp8", (os_, dqs, dks, dvs), *(t.cpu() for t in (qs, ks, vs, gs)), rotate=False, token_local=True,
                     qdq_tol=9e-2, published=False)


@pytest.mark.parametrize("route", ["fp8", "fp4"])
def test_packed_documents_full_size(route):
    """16384 tokens in seeded log-uniform documents, h16 d128 causal (configuration 5): every document must reproduce the
    batched run of that document alone (scales are document-local)."""
    import warnings
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    lens = packed_doc_lengths()
    total = sum(lens)
    starts = [sum(lens[:i]) for i in range(len(lens))]
    h, d = 16, 128
    q, k, v, g = (t[0].cuda() for t in attention_inputs(1, total, h, h, d, seed=5))
    cu = torch.tensor(starts + [total], dtype=torch.int32, device="cuda")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        o, dq, dk, dv = _run(fn, q, k, v, g, causal=True, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens),
                             max_seqlen_k=max(lens))
        for t in (o, dq, dk, dv):
            assert torch.isfinite(t.float()).all()
        for i in (2, 5, 10):       # 736, 690 and 64 tokens
            sl = slice(starts[i], starts[i] + lens[i])
            if route == "fp8":
                od, dqd, dkd, dvd = (t[0] for t in _run(fn, q[None, sl], k[None, sl], v[None, sl], g[None, sl], causal=True))
            else:      # the mixed route's batched form takes multiples of 128 only: the document alone, packed
                cu1 = torch.tensor([0, lens[i]], dtype=torch.int32, device="cuda")
                od, dqd, dkd, dvd = _run(fn, q[sl], k[sl], v[sl], g[sl], causal=True, cu_seqlens_q=cu1, cu_seqlens_k=cu1,
                                         max_seqlen_q=lens[i], max_seqlen_k=lens[i])
            assert torch.equal(od, o[sl]), i
            assert torch.equal(dkd, dk[sl]) and torch.equal(dvd, dv[sl]), i
            assert _close(dqd, dq[sl]) < 8e-3, i
        # two documents against the oracle: the document alone, zero-padded to a multiple of 128 as in the repacked buffer
        for i in (2, 5):
            n = lens[i]
            pad = (n + 127) // 128 * 128
            sl = slice(starts[i], starts[i] + n)
            qd, kd, vd, gd = (torch.nn.functional.pad(t[sl].cpu(), (0, 0, 0, 0, 0, pad - n))[None] for t in (q, k, v, g))
            rq = A.qdq_attention(qd, kd, vd, gd, causal=True, rotate_qk=True, fp4_qk=route == "fp4")
            for name, x, ref in (("o", o[sl], rq[0]), ("dq", dq[sl], rq[2]), ("dk", dk[sl], rq[3]), ("dv", dv[sl], rq[4])):
                acc = A.accuracy(x.float().cpu(), ref[0, :n])
                print(f"packed {route} doc {i} {name}: vs QDQ rel_l2 {acc['rel_l2']:.4f}")
                assert acc["rel_l2"] < 5e-2, (route, i, name, acc)
