"""GPU: the public entry points end to end (plan -> custom op -> autograd) against the CPU oracle: batched, GQA, f16,
lengths that are no multiple of 128, repacked and aligned packed documents. Tolerances as tests/test_gpu_bwd.py."""
import math

import pytest
import torch

from inputs import attention_inputs, packed_doc_lengths
from oracle import attention_oracle as A

pytestmark = pytest.mark.gpu


def _step(fn, q, k, v, g, **kw):
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = fn(qc, kc, vc, **kw)
    lse = None
    if isinstance(out, tuple):
        out, lse = out
    out.backward(g.cuda())
    torch.cuda.synchronize()
    return out.detach().float().cpu(), qc.grad.float().cpu(), kc.grad.float().cpu(), vc.grad.float().cpu(), lse


def _check(got, ref, tol=5e-2, names=("o", "dq", "dk", "dv")):
    for n, a, r in zip(names, got, ref):
        acc = A.accuracy(a, r)
        assert acc["rel_l2"] < tol, (n, acc)


def test_fp8_batched_autograd_default_route():
    from flamia_blackwell_attention_b200 import flash_attn_fp8
    q, k, v, g = attention_inputs(2, 512, 4, 2, 128, seed=4)
    o, dq, dk, dv, lse = _step(flash_attn_fp8, q, k, v, g, causal=True, return_lse=True)
    ro, rl, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=True, rotate_qk=True)
    _check((o, dq, dk, dv), (ro, rdq, rdk, rdv))
    assert lse.shape == (2, 4, 512) and not lse.requires_grad
    assert float((lse.cpu() - rl).abs().max()) < 2e-3


def test_fp8_f16_inputs_and_d64():
    from flamia_blackwell_attention_b200 import flash_attn_fp8
    q, k, v, g = (t.half() for t in attention_inputs(1, 512, 4, 4, 64, seed=5))
    o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, causal=True)
    ro, _, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=True)
    _check((o, dq, dk, dv), (ro, rdq, rdk, rdv))


def test_fp8_forward_only_under_no_grad():
    from flamia_blackwell_attention_b200 import flash_attn_fp8
    q, k, v, _ = attention_inputs(1, 256, 2, 2, 128, seed=6)
    with torch.no_grad():
        o = flash_attn_fp8(q.cuda(), k.cuda(), v.cuda())
    ro, *_ = A.qdq_attention(q, k, v, causal=False, rotate_qk=True)
    assert A.accuracy(o.float().cpu(), ro)["rel_l2"] < 3.2e-2


def test_fp8_lengths_that_are_no_multiple_of_128():
    from flamia_blackwell_attention_b200 import flash_attn_fp8
    q, k, v, g = attention_inputs(2, 300, 2, 2, 128, seed=7)
    o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, causal=True)
    ro, _, rdq, rdk, rdv = A.attention_fp32(q.float(), k.float(), v.float(), g.float(), True)
    _check((o, dq, dk, dv), (ro, rdq, rdk, rdv), tol=7e-2)       # vs fp32 on the unquantised inputs


@pytest.mark.parametrize("aligned", [False, True])
def test_fp8_packed_documents(aligned):
    from flamia_blackwell_attention_b200 import flash_attn_fp8
    lens = [300, 128, 77, 515]
    h, d = 2, 128
    if aligned:
        starts, pos = [], 0
        for n in lens:
            starts.append(pos)
            pos += (n + 127) // 128 * 128
        total = pos
    else:
        starts = [sum(lens[:i]) for i in range(len(lens))]
        total = sum(lens)
    q, k, v, g = (t[0] for t in attention_inputs(1, total, h, h, d, seed=8))
    if aligned:      # padding rows are zero by contract
        mask = torch.zeros(total, dtype=torch.bool)
        for s0, n in zip(starts, lens):
            mask[s0:s0 + n] = True
        q, k, v, g = (t * mask[:, None, None] for t in (q, k, v, g))
    cu = torch.tensor(starts + [total], dtype=torch.int32, device="cuda")
    kw = dict(causal=True, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    if aligned:
        su = torch.tensor(lens, dtype=torch.int32, device="cuda")
        kw.update(seqused_q=su, seqused_k=su)
    from flamia_blackwell_attention_b200 import api
    api._REPACK_WARNED = False                   # the notice is given once per process: make this call the first
    with pytest.warns(UserWarning) if not aligned else _nullcontext():
        o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, **kw)
    for s0, n in zip(starts, lens):
        sl = slice(s0, s0 + n)
        ro, _, rdq, rdk, rdv = A.attention_fp32(q[None, sl].float(), k[None, sl].float(), v[None, sl].float(),
                                                g[None, sl].float(), True)
        _check((o[sl], dq[sl], dk[sl], dv[sl]), (ro[0], rdq[0], rdk[0], rdv[0]), tol=7e-2)


class _nullcontext:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


def test_inputs_are_not_mutated_and_no_host_sync():
    from flamia_blackwell_attention_b200 import flash_attn_fp8
    q, k, v, g = (t.cuda() for t in attention_inputs(1, 256, 2, 2, 128, seed=9))
    q0, k0, v0, g0 = (t.clone() for t in (q, k, v, g))
    qc, kc, vc = (t.requires_grad_(True) for t in (q, k, v))
    flash_attn_fp8(qc, kc, vc, causal=True).backward(g)        # warm: plan cache, library load
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        flash_attn_fp8(qc, kc, vc, causal=True).backward(g)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    for a, b in ((q, q0), (k, k0), (v, v0), (g, g0)):
        assert torch.equal(a.detach(), b)


def test_fp4_batched_autograd_default_route():
    """flash_attn_fp4 defaults: NVFP4 S operands of the rotated rows, E4M3 P.V and gradient products."""
    from flamia_blackwell_attention_b200 import flash_attn_fp4
    q, k, v, g = attention_inputs(2, 512, 4, 2, 128, seed=14)
    o, dq, dk, dv, lse = _step(flash_attn_fp4, q, k, v, g, causal=True, return_lse=True)
    ro, rl, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=True, fp4_qk=True, rotate_qk=True)
    _check((o, dq, dk, dv), (ro, rdq, rdk, rdv))
    assert lse.shape == (2, 4, 512)
    assert float((lse.cpu() - rl).abs().max()) < 2e-3


def test_fp4_forward_only_and_dense():
    from flamia_blackwell_attention_b200 import flash_attn_fp4
    q, k, v, _ = attention_inputs(1, 384, 2, 2, 128, seed=15)
    with torch.no_grad():
        o = flash_attn_fp4(q.cuda(), k.cuda(), v.cuda())
    ro, *_ = A.qdq_attention(q, k, v, causal=False, fp4_qk=True, rotate_qk=True)
    assert A.accuracy(o.float().cpu(), ro)["rel_l2"] < 3.2e-2


def test_fp4_packed_documents():
    from flamia_blackwell_attention_b200 import flash_attn_fp4
    lens = [300, 128, 77, 515]
    h, d = 2, 128
    starts = [sum(lens[:i]) for i in range(len(lens))]
    total = sum(lens)
    q, k, v, g = (t[0] for t in attention_inputs(1, total, h, h, d, seed=16))
    cu = torch.tensor(starts + [total], dtype=torch.int32, device="cuda")
    kw = dict(causal=True, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    import warnings
    with warnings.catch_warnings():          # the repacking notice is issued once per process
        warnings.simplefilter("ignore")
        o, dq, dk, dv, _ = _step(flash_attn_fp4, q, k, v, g, **kw)
    for s0, n in zip(starts, lens):
        sl = slice(s0, s0 + n)
        ro, _, rdq, rdk, rdv = A.attention_fp32(q[None, sl].float(), k[None, sl].float(), v[None, sl].float(),
                                                g[None, sl].float(), True)
        _check((o[sl], dq[sl], dk[sl], dv[sl]), (ro[0], rdq[0], rdk[0], rdv[0]), tol=0.17)   # 4-bit S operands vs fp32


def test_fp8_token_local_rowlocal_causal_prescale_gqa():
    """The GQA configuration's options: token-local operand scales, dQ-side row-local dS-hat, causal dQ pre-scale, with
    1 % of the Q / K channels scaled x20."""
    from flamia_blackwell_attention_b200 import flash_attn_fp8, FP8AttnOptions
    import flamia_blackwell_attention_b200.interface_bwd_fp4 as I
    q, k, v, g = attention_inputs(1, 1024, 8, 2, 128, seed=17, outlier_channels=True)
    opts = FP8AttnOptions(operand_scaling="token_local", ds_dq_rowlocal="all")
    old = I.DQ_CAUSAL_PRESCALE
    I.DQ_CAUSAL_PRESCALE = True
    try:
        o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, causal=True, options=opts)
    finally:
        I.DQ_CAUSAL_PRESCALE = old
    # bound: the default route's own error on the same inputs (outlier channels make near one-hot rows, where the E4M3
    # roundings of P-hat / dS-hat weigh more whatever the operand scaling)
    ro, _, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=True, token_local=True)
    base = _step(flash_attn_fp8, q, k, v, g, causal=True)
    bo, _, bdq, bdk, bdv = A.qdq_attention(q, k, v, g, causal=True, rotate_qk=True)
    for n, a, r, ba, br in zip(("o", "dq", "dk", "dv"), (o, dq, dk, dv), (ro, rdq, rdk, rdv), base[:4], (bo, bdq, bdk, bdv)):
        e_new, e_base = A.accuracy(a, r)["rel_l2"], A.accuracy(ba, br)["rel_l2"]
        print("token-local", n, e_new, "default route", e_base)
        assert e_new <= 1.15 * e_base + 1e-3, (n, e_new, e_base)


WINDOW_CASES = [
    # s_q, s_k, causal, window, route
    (512, 512, True, (200, 0), "fp8"),
    (1024, 1024, True, (256, None), "fp8"),        # the right side is capped by causal
    (640, 640, False, (100, 50), "fp8"),
    (384, 768, False, (None, 64), "fp8"),          # only a right limit, s_q != s_k
    (768, 768, True, (300, 0), "fp4"),
    (300, 300, True, (64, 0), "fp8"),              # a length that is no multiple of 128 (repacked internally)
]


@pytest.mark.parametrize("sq,sk,causal,window,route", WINDOW_CASES)
def test_sliding_window(sq, sk, causal, window, route):
    """window_size=(left, right): key j visible iff i + off - left <= j <= i + off + right."""
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    s = max(sq, sk)
    q, k, v, g = attention_inputs(2, s, 4, 2, 128, seed=21)
    q, g, k, v = q[:, :sq], g[:, :sq], k[:, :sk], v[:, :sk]
    o, dq, dk, dv, _ = _step(fn, q, k, v, g, causal=causal, window_size=window)
    if sq % 128 == 0:
        ro, _, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=causal, rotate_qk=True, fp4_qk=route == "fp4", window=window)
        _check((o, dq, dk, dv), (ro, rdq, rdk, rdv))
    else:
        ro, _, rdq, rdk, rdv = A.attention_fp32(q.float(), k.float(), v.float(), g.float(), causal, window=window)
        _check((o, dq, dk, dv), (ro, rdq, rdk, rdv), tol=7e-2)
    # rows / keys outside every window get exact zeros
    assert torch.isfinite(o).all() and torch.isfinite(dq).all()


@pytest.mark.parametrize("form", ["batched_fp8", "batched_fp4", "token_local", "ragged", "packed", "aligned"])
def test_state_matches_its_spec(form):
    """The saved state of the registered forward op has exactly the shapes and dtypes the fake implementation announces
    (flamia_blackwell_attention_b200/_routes.py::state_spec)."""
    import flamia_blackwell_attention_b200 as F
    from flamia_blackwell_attention_b200 import _op, _routes
    h, hk, d = 4, 2, 128
    kw = dict(causal=True)
    entry = "fp4" if form == "batched_fp4" else "fp8"
    docs, n_docs = [], 0
    if form in ("packed", "aligned"):
        lens = [300, 128, 77, 515]
        if form == "aligned":
            starts = [0, 384, 512, 640]
            total = 1280
            su = torch.tensor(lens, dtype=torch.int32, device="cuda")
            kw.update(seqused_q=su, seqused_k=su)
        else:
            starts = [sum(lens[:i]) for i in range(4)]
            total = sum(lens)
        q, k, v, _ = (t[0].cuda() for t in attention_inputs(1, total, h, hk, d, seed=31))
        cu = torch.tensor(starts + [total], dtype=torch.int32, device="cuda")
        kw.update(cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
        docs = [cu, cu] + ([su, su] if form == "aligned" else [])
        n_docs = len(lens)
    else:
        s = 300 if form == "ragged" else 384
        q, k, v, _ = (t.cuda() for t in attention_inputs(2, s, h, hk, d, seed=31))
        if form == "token_local":
            kw["options"] = F.FP8AttnOptions(operand_scaling="token_local", ds_dq_rowlocal="all")
    for t in (q, k, v):
        t.requires_grad_(True)
    plan = (F.resolve_fp4 if entry == "fp4" else F.resolve_fp8)(q, k, v, **kw)
    pid = _op.register_plan(plan)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out, lse, state = getattr(torch.ops.lowbit_attn, entry)(q.detach(), k.detach(), v.detach(), docs, pid, 0)
    spec = _routes.state_spec(plan, n_docs, q.dtype)
    is_docs = plan.shape.varlen or plan.fwd.ragged_documents
    # O / LSE leave as the op's outputs; repacked documents keep the aligned buffer's LSE in the state
    want = (spec[1:] if (is_docs and not plan.shape.aligned_varlen) else spec[2:]) + [((), torch.int64)]
    assert [(tuple(t.shape), t.dtype) for t in state] == [(tuple(sh), dt) for sh, dt in want]
    assert out.shape == q.shape


def test_fp8_d64_packed_documents_and_window():
    """Head dimension 64 through the packed form (repacked documents) and with a sliding window."""
    import warnings
    from flamia_blackwell_attention_b200 import flash_attn_fp8
    lens = [300, 128, 77, 515]
    h, d = 4, 64
    starts = [sum(lens[:i]) for i in range(len(lens))]
    total = sum(lens)
    q, k, v, g = (t[0] for t in attention_inputs(1, total, h, 2, d, seed=41))
    cu = torch.tensor(starts + [total], dtype=torch.int32, device="cuda")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, causal=True, cu_seqlens_q=cu, cu_seqlens_k=cu,
                                 max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    for s0, n in zip(starts, lens):
        sl = slice(s0, s0 + n)
        ro, _, rdq, rdk, rdv = A.attention_fp32(q[None, sl].float(), k[None, sl].float(), v[None, sl].float(),
                                                g[None, sl].float(), True)
        _check((o[sl], dq[sl], dk[sl], dv[sl]), (ro[0], rdq[0], rdk[0], rdv[0]), tol=7e-2)
    q, k, v, g = attention_inputs(2, 512, 4, 2, d, seed=42)
    o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, causal=True, window_size=(150, 0))
    ro, _, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=True, window=(150, 0))
    _check((o, dq, dk, dv), (ro, rdq, rdk, rdv))


@pytest.mark.parametrize("route", ["fp8", "fp4"])
def test_f16_inputs_d128(route):
    """float16 inputs and gradients at head dimension 128 on both routes."""
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    q, k, v, g = (t.half() for t in attention_inputs(2, 384, 4, 2, 128, seed=51))
    o, dq, dk, dv, _ = _step(fn, q, k, v, g, causal=True)
    assert o.dtype == torch.float32 and dq.shape == q.shape          # _step returns float copies
    ro, _, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=True, rotate_qk=True, fp4_qk=route == "fp4")
    _check((o, dq, dk, dv), (ro, rdq, rdk, rdv))


@pytest.mark.parametrize("dist", ["logit3", "outlier", "zeros", "tiny", "near_min_normal", "mixed", "subnorm_sf"])
def test_extreme_input_families(dist):
    """The quantiser test's input families through the whole fwd+bwd call: zeros, values near the bottom of the float range,
    scattered x1000 outliers, per-group exponents spread over 2^+-60 (in V and dO). Outputs must be finite and track the
    oracle's quantise-dequantise emulation of the same inputs (against fp32 attention the x1000 outliers alone cost 40 %:
    that is the format, not the kernels). One known limit, shared with the reference: the f16 dQ accumulator's pre-scale
    exponent is clamped to +-40, so gradients beyond 65504 * 2^40 (the 'mixed' family reaches 1e34) overflow it."""
    from flamia_blackwell_attention_b200 import flash_attn_fp8
    from inputs import make
    b, s, h, d = 1, 384, 2, 128
    q, k, v, g = (make((b, s, h, d), dist, seed=60 + i) for i in range(4))
    if dist == "mixed":      # keep the scores representable: the spread goes to V and dO only
        q, k = make((b, s, h, d), "n01", seed=70), make((b, s, h, d), "n01", seed=71)
    o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, causal=True)
    ro, _, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=True, rotate_qk=True)
    for name, t, r in (("o", o, ro), ("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        if dist == "mixed" and name == "dq":
            continue
        assert torch.isfinite(t).all(), (dist, name)
        if torch.isfinite(r).all() and float(r.abs().max()) > 0:
            assert A.accuracy(t, r)["rel_l2"] < 6e-2, (dist, name, A.accuracy(t, r))


@pytest.mark.parametrize("route,causal,sq,sk", [("fp8", True, 512, 512), ("fp8", False, 256, 640), ("fp4", True, 384, 384)])
def test_batched_seqused_k(route, causal, sq, sk):
    """seqused_k on the batched form: keys at or past seqused_k[b] are masked, their dK / dV rows come back zero, rows that
    see no key give a zero output row (tests/cute/test_lowprec_api.py:1346 of the reference states the semantics)."""
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    s = max(sq, sk)
    q, k, v, g = attention_inputs(3, s, 4, 2, 128, seed=91)
    q, g, k, v = q[:, :sq], g[:, :sq], k[:, :sk], v[:, :sk]
    used = [sk, 200, 129]
    su = torch.tensor(used, dtype=torch.int32, device="cuda")
    o, dq, dk, dv, _ = _step(fn, q, k, v, g, causal=causal, seqused_k=su)
    ro, _, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=causal, rotate_qk=True, fp4_qk=route == "fp4", seqused_k=used)
    _check((o, dq, dk, dv), (ro, rdq, rdk, rdv))
    for b_, n in enumerate(used):
        assert float(dk[b_, n:].abs().max() if n < sk else 0.0) == 0.0 and float(dv[b_, n:].abs().max() if n < sk else 0.0) == 0.0
    assert torch.isfinite(o).all() and torch.isfinite(dq).all()


@pytest.mark.parametrize("route,d,causal,window", [("fp8", 128, True, None), ("fp8", 64, False, None), ("fp4", 128, True, (200, 0)),
                                                   ("fp8", 128, True, (100, 0))])
def test_softcap(route, d, causal, window):
    """softcap c: score -> c tanh(score / c) before masking, dS takes 1 - tanh^2 (flash_attn/cute/utils.py:167-187 of the
    reference). Scores are made large enough (Q x 3) for the cap to bite."""
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    q, k, v, g = attention_inputs(2, 512, 4, 2, d, seed=93)
    q = (q.float() * 3.0).to(torch.bfloat16)
    kw = dict(causal=causal, softcap=2.0)
    if window is not None:
        kw["window_size"] = window
    o, dq, dk, dv, _ = _step(fn, q, k, v, g, **kw)
    ro, _, rdq, rdk, rdv = A.qdq_attention(q, k, v, g, causal=causal, rotate_qk=d == 128, fp4_qk=route == "fp4", window=window,
                                           softcap=2.0)
    _check((o, dq, dk, dv), (ro, rdq, rdk, rdv))
    # the cap does something: the uncapped result differs
    o2, *_ = _step(fn, q, k, v, g, causal=causal, **({} if window is None else dict(window_size=window)))
    assert A.accuracy(o2, ro)["rel_l2"] > 0.05


@pytest.mark.parametrize("d,hk", [(96, 2), (32, 4), (112, 1)])
def test_fp8_padded_head_dims(d, hk):
    """Head dims that are multiples of 16 below 128 run padded with zero columns to the next of 64 / 128 (the reference's
    rule E13, flash_attn/cute/lowprec/plan.py:1529-1541): same numbers, bit for bit, as the padded call made by hand with
    the call's own softmax scale, and within the usual tolerance of the oracle at the true head dim."""
    from flamia_blackwell_attention_b200 import flash_attn_fp8
    q, k, v, g = attention_inputs(2, 384, 4, hk, d, seed=21)
    o, dq, dk, dv, lse = _step(flash_attn_fp8, q, k, v, g, causal=True, return_lse=True)
    assert o.shape == q.shape and dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    dp = 64 if d < 64 else 128
    pad = lambda t: torch.nn.functional.pad(t, (0, dp - d))      # noqa: E731
    o2, dq2, dk2, dv2, lse2 = _step(flash_attn_fp8, pad(q), pad(k), pad(v), pad(g), causal=True, return_lse=True,
                                    softmax_scale=1.0 / math.sqrt(d), qk_hadamard=False)
    assert torch.equal(o, o2[..., :d]) and torch.equal(lse.cpu(), lse2.cpu())
    assert torch.equal(dk, dk2[..., :d]) and torch.equal(dv, dv2[..., :d])
    assert float((dq - dq2[..., :d]).abs().max()) <= 2e-3 * float(dq2.abs().max())     # f16 reduction order only
    assert float(o2[..., d:].abs().max()) == 0.0
    # the oracle's quantiser takes 64 / 128 columns: zero columns move no block maximum, so the padded oracle call is the
    # definition at the true head dim; the fp32 reference is taken at the true head dim itself
    ro, rl, rdq, rdk, rdv = A.qdq_attention(pad(q), pad(k), pad(v), pad(g), causal=True, softmax_scale=1.0 / math.sqrt(d))
    _check((o, dq, dk, dv), (ro[..., :d], rdq[..., :d], rdk[..., :d], rdv[..., :d]))
    assert float((lse.cpu() - rl).abs().max()) < 2e-3
    fo, _fl, fdq, fdk, fdv = A.attention_fp32(q, k, v, g, causal=True)
    _check((o, dq, dk, dv), (fo, fdq, fdk, fdv), tol=1e-1)


@pytest.mark.parametrize("b,s,h,hk,d", [(3, 256, 3, 3, 128), (2, 129, 21, 3, 96), (1, 384, 20, 5, 64), (2, 31, 7, 1, 32)])
def test_fp8_odd_head_counts_and_lengths(b, s, h, hk, d):
    """Head counts that are no power of two, GQA ratios 1 / 4 / 7, lengths 31 and 129 (documents of the batch rows), padded
    head dims: against fp32 attention at the true shapes (the quantisation's own error is about 5e-2 on ragged lengths,
    where the rotation is off)."""
    from flamia_blackwell_attention_b200 import flash_attn_fp8, check_status
    q, k, v, g = attention_inputs(b, s, h, hk, d, seed=31)
    o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, causal=True)
    check_status()
    fo, _fl, fdq, fdk, fdv = A.attention_fp32(q, k, v, g, causal=True)
    _check((o, dq, dk, dv), (fo, fdq, fdk, fdv), tol=1e-1)
    assert all(torch.isfinite(t).all() for t in (o, dq, dk, dv))


def test_single_token_and_empty_key_ranges():
    """One query and one key per row: O is the V row, dV the dO row, dQ = dK = 0 (P = 1 has no gradient); a batch row
    whose seqused_k is 0 sees no key at all: zero output rows, zero gradients, nothing non-finite."""
    from flamia_blackwell_attention_b200 import flash_attn_fp8, check_status
    q, k, v, g = attention_inputs(2, 1, 4, 2, 64, seed=32)
    o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, causal=True)
    assert A.accuracy(o, v.float().repeat_interleave(2, dim=2))["rel_l2"] < 3e-2
    assert A.accuracy(dv, g.float().reshape(2, 1, 2, 2, 64).sum(3))["rel_l2"] < 3e-2
    assert float(dq.abs().max()) < 1e-2 and float(dk.abs().max()) < 1e-2
    q, k, v, g = attention_inputs(2, 256, 2, 2, 128, seed=33)
    su = torch.tensor([0, 256], dtype=torch.int32)
    o, dq, dk, dv, _ = _step(flash_attn_fp8, q, k, v, g, causal=True, seqused_k=su.cuda())
    check_status()
    assert all(torch.isfinite(t).all() for t in (o, dq, dk, dv))
    assert float(o[0].abs().max()) == 0.0 and float(dq[0].abs().max()) == 0.0
    assert float(dk[0].abs().max()) == 0.0 and float(dv[0].abs().max()) == 0.0
    ro, _, rdq, rdk, rdv = A.qdq_attention(q[1:], k[1:], v[1:], g[1:], causal=True, rotate_qk=True)
    _check((o[1:], dq[1:], dk[1:], dv[1:]), (ro, rdq, rdk, rdv))


@pytest.mark.parametrize("route", ["fp8", "fp4"])
def test_lse_of_repacked_documents_and_ragged_batch_rows(route):
    """return_lse on the forms that run as repacked documents: (h, total) in the caller's packed row order under
    cu_seqlens / doc_maps, (b, h, s) for batch rows whose length is no multiple of 128 -- each row's value is that of
    its own document."""
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    lens, h, hk, d = [200, 128, 37, 300], 4, 2, 128
    total = sum(lens)
    q, k, v, g = (t[0] for t in attention_inputs(1, total, h, hk, d, seed=41))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    ref = torch.empty(h, total)
    s0 = 0
    for n in lens:
        sl = slice(s0, s0 + n)
        _, rl, *_ = A.attention_fp32(q[None, sl].float(), k[None, sl].float(), v[None, sl].float(), None, True)
        ref[:, sl] = rl[0]
        s0 += n
    # against fp32 attention: a row with few keys takes the quantisation error of its few scores in full (up to 0.1 on
    # the 8-bit route), long rows average it out: bound the worst row and the typical one
    tol, typ = (0.2, 1e-2) if route == "fp8" else (0.5, 4e-2)
    for kw in (dict(cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens)),
               dict(doc_maps=F.DocMaps.from_cu_seqlens(cu.cpu()).to("cuda"))):
        with torch.no_grad():
            out, lse = fn(q.cuda(), k.cuda(), v.cuda(), causal=True, return_lse=True, **kw)
        assert lse.shape == (h, total) and lse.dtype == torch.float32
        err = (lse.cpu() - ref).abs()
        assert float(err.max()) < tol and float(err.median()) < typ
    if route == "fp8":                               # batch rows of 200 tokens run as documents
        q, k, v, g = attention_inputs(3, 200, h, hk, d, seed=42)
        with torch.no_grad():
            out, lse = fn(q.cuda(), k.cuda(), v.cuda(), causal=True, return_lse=True)
        _, rl, *_ = A.attention_fp32(q.float(), k.float(), v.float(), None, True)
        err = (lse.cpu() - rl).abs()
        assert lse.shape == (3, h, 200) and float(err.max()) < tol and float(err.median()) < typ
