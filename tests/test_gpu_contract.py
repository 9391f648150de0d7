"""GPU: run-time contracts of the public call and robustness of the document forms.

  * the f16 dQ pre-scale tables of fl_dq_prescale, bit for bit against the pinned scale oracle (row and causal-tile modes,
    unit != 1, zero / overflowing / tiny statistics);
  * packed and ragged documents stay finite when the caching allocator hands out memory full of NaN;
  * a document table that does not fit its buffer is clamped and reported through the status word;
  * check_status() raises for a status word that records a wait that ran out;
  * distinct query / key document tables are refused;
  * the backward runs on another thread with the plan of ITS forward (two plans interleaved);
  * a captured CUDA graph of the public fwd+bwd call replays to the eager result (O, LSE, dK, dV bitwise);
  * causal safety: future K / V / dO rows do not move earlier rows of O, LSE and dQ.
The last three follow the reference's tests/cute/test_lowprec_api.py:831-883, :977-1000 and
tests/cute/test_lowprec_causal_safe_v.py.
"""
import math
import threading
import warnings

import numpy as np
import pytest
import torch

from inputs import attention_inputs, scale_stats
from oracle import attention_oracle as A
from oracle import scales_oracle as S

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------------------------ dQ pre-scale tables
@pytest.mark.parametrize("kind", ["plain", "zeros", "huge", "tiny"])
@pytest.mark.parametrize("shape", [(2, 4, 2, 3, 3), (1, 2, 2, 5, 5), (3, 8, 1, 2, 4)])
@pytest.mark.parametrize("unit", [1.0, 256.0])
def test_dq_prescale_tables_bitwise(kind, shape, unit):
    from flamia_blackwell_attention_b200 import kernels as K
    b, hq, hk, tq, tk = shape
    dn, vn, km = scale_stats(b, hq, hk, tq, tk, kind, seed=b * 100 + tq)
    st_do = torch.zeros(b, hq, tq, 2)
    st_v = torch.zeros(b, hk, tk, 2)
    st_k = torch.zeros(b, hk, tk, 2)
    st_do[..., 1] = dn.view(b, hq, tq)      # max row sum of squares of dO
    st_v[..., 1] = vn.view(b, hk, tk)       # max row sum of squares of V
    st_k[..., 0] = km.view(b, hk, tk)       # amax of K
    for mode in ("row", "causal_tile"):
        if mode == "causal_tile" and tq != tk:
            continue
        ks, ps = K.dq_prescale(st_do.cuda(), st_v.cuda(), st_k.cuda(), causal_local=mode == "causal_tile", unit=unit)
        fn = S.dq_prescale_rows if mode == "row" else S.dq_prescale_causal_tiles
        want_k, want_p = fn(dn.numpy(), vn.numpy(), km.numpy(), b, hq, hk, tq, tk, unit=unit, base=1.0, num=1.0)
        assert np.array_equal(ks.cpu().numpy().reshape(-1).view(np.uint32), want_k.view(np.uint32)), (mode, kind)
        assert np.array_equal(ps.cpu().numpy().reshape(-1).view(np.uint32), want_p.view(np.uint32)), (mode, kind)


@pytest.mark.parametrize("rotate", [False, True])
def test_dq_prescale_rows_bitwise(rotate):
    """The per-query-row causal pre-scale (the reference's CAUSAL == 2 table, flash_attn/cute/device_scales.py:256-268):
    per-token statistics from the quantisers (maximum over the heads), running maxima over the keys, and the table
    against the oracle's restatement, bit for bit."""
    from flamia_blackwell_attention_b200 import kernels as K
    b, s, h, hk, d = 2, 1280, 4, 2, 128
    q, k, v, g = (t.cuda() for t in attention_inputs(b, s, h, hk, d, seed=93))
    k = k * torch.linspace(0.2, 3.0, s, device="cuda").view(1, s, 1, 1).to(k.dtype)       # statistics that grow and shrink
    v = v * (1.0 + torch.sin(torch.arange(s, device="cuda") / 50.0)).view(1, s, 1, 1).to(v.dtype)
    rk, rv, rdo = (torch.zeros(b, s, dtype=torch.float32, device="cuda") for _ in range(3))
    K.quantize_fp8_blocks(k, apply_hadamard_rotation=rotate, row_stat=("norm2" if rotate else "amax", rk))
    K.quantize_fp8_blocks(v, row_stat=("sumsq", rv))
    K.quantize_fp8_blocks(g, row_stat=("sumsq", rdo))
    # the statistics themselves: maximum over the heads of the row's own figure (fp32 sums in the kernel's order: close)
    want_k = (k.float().norm(dim=-1) if rotate else k.float().abs().amax(dim=-1)).amax(dim=-1)
    torch.testing.assert_close(rk, want_k, rtol=2e-3, atol=1e-6)
    torch.testing.assert_close(rv, v.float().pow(2).sum(-1).amax(-1), rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(rdo, g.float().pow(2).sum(-1).amax(-1), rtol=1e-4, atol=1e-6)
    vn_prefix = torch.cummax(rv, dim=1).values.cpu().numpy()
    km_prefix = torch.cummax(rk, dim=1).values.cpu().numpy()
    dn = rdo.cpu().numpy()
    pv, pk = rv.clone(), rk.clone()
    ks, ps = K.dq_prescale_rows(rdo, pv, pk)
    assert np.array_equal(pv.cpu().numpy(), vn_prefix) and np.array_equal(pk.cpu().numpy(), km_prefix)
    want_ks, want_ps = S.dq_prescale_causal_rows(dn.reshape(-1), vn_prefix.reshape(-1), km_prefix.reshape(-1))
    assert np.array_equal(ks.cpu().numpy().reshape(-1).view(np.uint32), want_ks.view(np.uint32))
    assert np.array_equal(ps.cpu().numpy().reshape(-1).view(np.uint32), want_ps.view(np.uint32))


# ------------------------------------------------------------------------------------------------ NaN-filled allocator
def _poison_allocator(nbytes=192 << 20):
    """Allocate, fill with NaN bit patterns (as f32 and as bf16) and free: the caching allocator hands these blocks out
    again to the next torch.empty calls."""
    blocks = [torch.full((nbytes // 16,), float("nan"), dtype=torch.float32, device="cuda") for _ in range(3)]
    blocks += [torch.full((nbytes // 64,), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(8)]
    torch.cuda.synchronize()
    del blocks


@pytest.mark.parametrize("form", ["ragged", "packed", "aligned"])
@pytest.mark.parametrize("route", ["fp8", "fp4"])
def test_documents_stay_finite_on_poisoned_memory(form, route):
    import flamia_blackwell_attention_b200 as F
    if route == "fp4" and form == "ragged":
        pytest.skip("flash_attn_fp4 takes lengths that are multiples of 128 on the batched form")
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    h, d = 2, 128
    kw = dict(causal=True)
    if form == "ragged":
        q, k, v, g = attention_inputs(2, 300, h, h, d, seed=81)
    else:
        lens = [300, 128, 77, 515]
        if form == "aligned":
            starts, total = [0, 384, 512, 640], 1280 + 256       # two unused tail tiles
            su = torch.tensor(lens, dtype=torch.int32, device="cuda")
            kw.update(seqused_q=su, seqused_k=su)
        else:
            starts, total = [sum(lens[:i]) for i in range(4)], sum(lens)
        q, k, v, g = (t[0] for t in attention_inputs(1, total, h, h, d, seed=82))
        cu = torch.tensor(starts + [total], dtype=torch.int32, device="cuda")
        kw.update(cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    gc = g.cuda()
    _poison_allocator()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = fn(qc, kc, vc, **kw)
        _poison_allocator()
        out.backward(gc)
    torch.cuda.synchronize()
    if form == "aligned":      # rows between documents are the caller's padding: only document rows are defined
        rows = torch.zeros(total, dtype=torch.bool)
        for s0, n in zip(starts, lens):
            rows[s0:s0 + n] = True
        rows = rows.cuda()
        for name, t in (("o", out), ("dq", qc.grad), ("dk", kc.grad), ("dv", vc.grad)):
            assert torch.isfinite(t[rows]).all(), (form, route, name)
    else:
        for name, t in (("o", out), ("dq", qc.grad), ("dk", kc.grad), ("dv", vc.grad)):
            assert torch.isfinite(t).all(), (form, route, name)
    assert F.check_status() == 0


# ------------------------------------------------------------------------------------------------ status word
def test_document_table_that_does_not_fit_is_clamped_and_reported():
    """seqused beyond the end of the buffer: the kernels cut the document at the buffer's end, touch nothing outside it
    and leave FL_DEV_BAD_TABLE in the status word, which check_status() turns into an error."""
    import flamia_blackwell_attention_b200 as F
    from flamia_blackwell_attention_b200 import _lib as L
    h, d, total = 2, 128, 512
    q, k, v, g = (t[0] for t in attention_inputs(1, total, h, h, d, seed=83))
    cu = torch.tensor([0, 256, total], dtype=torch.int32, device="cuda")
    su = torch.tensor([200, 900], dtype=torch.int32, device="cuda")          # the second document claims 900 of 256 rows
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = F.flash_attn_fp8(qc, kc, vc, causal=True, cu_seqlens_q=cu, cu_seqlens_k=cu, seqused_q=su, seqused_k=su,
                           max_seqlen_q=256, max_seqlen_k=256)
    out.backward(g.cuda())
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="document table"):
        F.check_status()
    assert torch.isfinite(out[:200]).all() and torch.isfinite(out[256:]).all()
    # the first document is untouched by its neighbour's bad entry
    ro, *_ = A.attention_fp32(q[None, :200].float(), k[None, :200].float(), v[None, :200].float(), None, True)
    assert A.accuracy(out[:200].float().cpu(), ro[0])["rel_l2"] < 7e-2
    assert L.FL_DEV_BAD_TABLE == 0x200
    with torch.no_grad():      # a clean call: the status word of the last call is fine again
        F.flash_attn_fp8(qc[:256].detach()[None], kc[:256].detach()[None], vc[:256].detach()[None], causal=True)
    assert F.check_status() == 0


def test_check_status_raises_for_a_wait_that_ran_out():
    import flamia_blackwell_attention_b200 as F
    from flamia_blackwell_attention_b200 import _routes
    q, k, v, _ = (t.cuda() for t in attention_inputs(1, 256, 2, 2, 128, seed=84))
    with torch.no_grad():
        F.flash_attn_fp8(q, k, v, causal=True)
    assert F.check_status() == 0
    _routes._note_status(torch.tensor([0x100 | 23], dtype=torch.int32, device="cuda"))    # what a kernel would leave
    with pytest.raises(RuntimeError, match="site 23"):
        F.check_status()
    with torch.no_grad():
        F.flash_attn_fp8(q, k, v, causal=True)
    assert F.check_status() == 0


def test_distinct_key_table_is_refused():
    import flamia_blackwell_attention_b200 as F
    q, k, v, _ = (t[0].cuda() for t in attention_inputs(1, 512, 2, 2, 128, seed=85))
    cu_q = torch.tensor([0, 200, 512], dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0, 300, 512], dtype=torch.int32, device="cuda")
    with pytest.raises(NotImplementedError) as e:
        F.flash_attn_fp8(q, k, v, causal=True, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, max_seqlen_q=312, max_seqlen_k=312)
    assert e.value.rule == "B8"


# ------------------------------------------------------------------------------------------------ threads and graphs
def _eager(fn, q, k, v, g, **kw):
    qc, kc, vc = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out, lse = fn(qc, kc, vc, return_lse=True, **kw)
    out.backward(g)
    torch.cuda.synchronize()
    return out.detach(), lse, qc.grad, kc.grad, vc.grad


def _cos(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(a @ b / (a.norm() * b.norm() + 1e-30))


def test_backward_on_another_thread_uses_the_plan_of_its_forward():
    """forward A (row-local dQ side), forward B (defaults), backward B, backward A, each backward on a fresh thread: every
    gradient equals the one of the same call made alone on the main thread."""
    import flamia_blackwell_attention_b200 as F
    q, k, v, g = (t.cuda() for t in attention_inputs(1, 512, 4, 2, 128, seed=86))
    opt_a = F.FP8AttnOptions(ds_dq_rowlocal="all")
    alone_a = _eager(F.flash_attn_fp8, q, k, v, g, causal=True, options=opt_a)
    alone_b = _eager(F.flash_attn_fp8, q, k, v, g, causal=True)
    assert not torch.equal(alone_a[2], alone_b[2])          # the two plans do differ in dQ
    leaves = {}

    def fwd(tag, **kw):
        leaves[tag] = tuple(t.detach().clone().requires_grad_(True) for t in (q, k, v))
        return F.flash_attn_fp8(*leaves[tag], causal=True, **kw)
    o_a = fwd("a", options=opt_a)
    o_b = fwd("b")
    for o in (o_b, o_a):
        t = threading.Thread(target=lambda o=o: o.backward(g))
        t.start()
        t.join()
    torch.cuda.synchronize()
    for tag, alone in (("a", alone_a), ("b", alone_b)):
        qg, kg, vg = (t.grad for t in leaves[tag])
        assert torch.equal(kg, alone[3]) and torch.equal(vg, alone[4]), tag
        assert _cos(qg, alone[2]) > 0.99999, tag           # f16 partial sums are added in arrival order


def test_library_call_as_first_cuda_work_of_a_thread():
    """A thread that has made no CUDA runtime call has no context bound, and tensor-map encoding is a driver call: the
    library binds the primary context itself instead of failing."""
    from flamia_blackwell_attention_b200 import kernels as K
    x = attention_inputs(1, 256, 2, 2, 128, seed=88)[0].cuda()
    want = K.quantize_fp8_blocks(x)["codes"].view(torch.uint8)
    torch.cuda.synchronize()
    got = {}

    a, keep = _raw_quant_args(x)                              # allocated here: the thread makes the library call only

    def work():
        got["rc"] = __import__("flamia_blackwell_attention_b200")._lib.load().fl_quant_blocks(a, None)
        got["keep"] = keep
    t = threading.Thread(target=work)
    t.start()
    t.join()
    torch.cuda.synchronize()
    assert got["rc"] == 0
    assert torch.equal(got["keep"][0], want)


def _raw_quant_args(x):
    import ctypes as C
    from flamia_blackwell_attention_b200 import _lib as L
    b, s, h, d = x.shape
    codes = torch.empty(b, s, h, d, dtype=torch.uint8, device=x.device)
    e = torch.empty(b, h, s // 32, d // 32, dtype=torch.uint8, device=x.device)
    fac = torch.empty(b, h, s // 32, dtype=torch.float32, device=x.device)
    a = L.QuantArgs()
    a.x, a.codes, a.e_tab, a.fac = L.ptr(x), L.ptr(codes), L.ptr(e), L.ptr(fac)
    a.b, a.s, a.h, a.d = b, s, h, d
    return C.byref(a), (codes, e, fac, a)


@pytest.mark.parametrize("route,kw", [("fp8", dict(causal=True)), ("fp4", dict(causal=True)),
                                      ("fp8", dict(causal=False)), ("fp8", dict(causal=True, window_size=(300, 0)))])
def test_deterministic_dq_is_bitwise_reproducible(route, kw):
    """deterministic=True: the key tiles add their partial sums in ascending key order, so dQ is the same bits from call to
    call (the reference's deterministic mode, flash_attn/cute/flash_bwd_sm100_fp4.py:4119-4215), and it agrees with the
    arrival-order result to f16 rounding."""
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    q, k, v, g = (t.cuda() for t in attention_inputs(2, 1536, 4, 2, 128, seed=91))
    runs = [_eager(fn, q, k, v, g, deterministic=True, **kw) for _ in range(3)]
    for r in runs[1:]:
        for a, b in zip(runs[0], r):
            assert torch.equal(a, b)
    loose = _eager(fn, q, k, v, g, **kw)
    assert torch.equal(loose[3], runs[0][3]) and torch.equal(loose[4], runs[0][4])      # dK, dV do not depend on it
    assert _cos(loose[2], runs[0][2]) > 0.99999
    assert F.check_status() == 0


def test_deterministic_order_wait_is_bounded():
    """An order table that never reaches a key tile's turn (here: pre-filled with a value no tile counts to): the wait
    gives up after its budget, the status word names the site, and the context stays usable."""
    from flamia_blackwell_attention_b200 import kernels as K
    b, s, h, d = 1, 256, 2, 128
    sc = 1.0 / math.sqrt(d)
    q, k, v, g = (t.cuda() for t in attention_inputs(b, s, h, h, d, seed=92))
    qq = K.quantize_fp8_blocks(q)
    kq = K.quantize_fp8_blocks(k, output_tile_stats=True)
    vq = K.quantize_fp8_blocks(v, output_tile_stats=True)
    out, lse, st = K.attn_fwd(qq, kq, vq, causal=True, softmax_scale=sc)
    acc = torch.empty(b, h, s, d, dtype=torch.float16, device="cuda")
    gq = K.quantize_fp8_blocks(g, compute_d_with_output=out, shifted_log2_lse_from=lse, log2_lse_shift=8.0,
                               d_multiplier=-2.0 ** -8, zero_accumulator=acc, output_tile_stats=True)
    ks, _ps = K.dq_prescale(gq["tile_stats"], vq["tile_stats"], kq["tile_stats"])
    order = torch.full((b, h, s // 128, 2), 1000, dtype=torch.int32, device="cuda")
    st2 = K.new_status(q.device)
    K.attn_bwd(qq, kq, vq, gq, lse_log2=gq["lse_log2"], d_rows=gq["D"], dq_acc=acc, dq_scale=ks, causal=True,
               softmax_scale=sc, status=st2, wait_cycles=2_000_000, dq_order=order)
    torch.cuda.synchronize()
    code = K.read_status(st2)
    assert code & 0x100 and (code & 0xFF) in (44, 40, 41, 42, 22, 23, 24, 31, 32, 33, 36, 21, 10, 11), hex(code)
    # the same call with a zeroed table runs to the end
    order.zero_()
    st3 = K.new_status(q.device)
    acc.zero_()
    K.attn_bwd(qq, kq, vq, gq, lse_log2=gq["lse_log2"], d_rows=gq["D"], dq_acc=acc, dq_scale=ks, causal=True,
               softmax_scale=sc, status=st3, dq_order=order)
    torch.cuda.synchronize()
    assert K.read_status(st3) == 0
    assert order.view(-1, 2)[:, 0].tolist() == [1, 2, 1, 2]          # (head, query tile): key tiles that see it


@pytest.mark.parametrize("route", ["fp8", "fp4"])
def test_graph_replay_equals_eager(route):
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    q, k, v, g = (t.cuda() for t in attention_inputs(2, 512, 4, 2, 128, seed=87))
    eager = _eager(fn, q, k, v, g, causal=True)
    sq, sk, sv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn(sq, sk, sv, causal=True).backward(g)
            sq.grad = sk.grad = sv.grad = None
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        go, glse = fn(sq, sk, sv, causal=True, return_lse=True)
        go.backward(g)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(go, eager[0]) and torch.equal(glse, eager[1])
    assert torch.equal(sk.grad, eager[3]) and torch.equal(sv.grad, eager[4])
    assert _cos(sq.grad, eager[2]) > 0.99999
    assert F.check_status() == 0


# ------------------------------------------------------------------------------------------------ causal safety
@pytest.mark.parametrize("route,opts", [("fp8", None), ("fp8", "token_local"), ("fp4", None)])
def test_future_rows_do_not_move_earlier_rows(route, opts):
    """Causal calls: K, V and dO rows from K0 on (K0 a multiple of 128, so no visible row shares a scale block with them)
    are replaced by large values; O, LSE and dQ of the rows before K0 must not move: O and LSE bitwise, dQ up to the
    arrival order of its f16 partial sums. With the causal dQ pre-scale the scale of an earlier query tile is sized from
    the keys it may see only, so dQ keeps its rounding too."""
    import flamia_blackwell_attention_b200 as F
    import flamia_blackwell_attention_b200.interface_bwd_fp4 as I
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    kw = dict(causal=True)
    if opts == "token_local":
        kw["options"] = F.FP8AttnOptions(operand_scaling="token_local", ds_dq_rowlocal="all")
    s, k0 = 1024, 640
    q, k, v, g = (t.cuda() for t in attention_inputs(1, s, 4, 2, 128, seed=88))
    k2, v2, g2 = k.clone(), v.clone(), g.clone()
    gen = torch.Generator(device="cuda").manual_seed(7)
    for t in (k2, v2, g2):
        t[:, k0:k0 + 40] = torch.randn(t[:, k0:k0 + 40].shape, generator=gen, device="cuda").sign().to(t.dtype) * 60.0
    old = I.DQ_CAUSAL_PRESCALE
    I.DQ_CAUSAL_PRESCALE = route == "fp8"
    try:
        base = _eager(fn, q, k, v, g, **kw)
        again = _eager(fn, q, k, v, g, **kw)
        pert = _eager(fn, q, k2, v2, g2, **kw)
    finally:
        I.DQ_CAUSAL_PRESCALE = old
    assert not torch.equal(base[0][:, k0:], pert[0][:, k0:])                 # the probe is not blind
    assert torch.equal(base[0][:, :k0], pert[0][:, :k0])
    assert torch.equal(base[1][..., :k0], pert[1][..., :k0])
    if route == "fp8":
        noise = float((base[2][:, :k0].float() - again[2][:, :k0].float()).abs().max())
        moved = float((base[2][:, :k0].float() - pert[2][:, :k0].float()).abs().max())
        ulp = float(base[2][:, :k0].float().abs().max()) * 2.0 ** -7
        assert moved <= max(noise, ulp), (moved, noise, ulp)


def test_row_wise_causal_prescale_is_exactly_causal():
    """DQ_CAUSAL_GRANULARITY = 'row' with the ordered reduction: dQ of the rows before K0 keeps every bit when later K, V
    and dO rows change (K0 need not be a multiple of the query tile here: the pre-scale is per query row), and the
    gradients agree with the per-tile form to f16 rounding."""
    import flamia_blackwell_attention_b200 as F
    import flamia_blackwell_attention_b200.interface_bwd_fp4 as I
    s, k0 = 1024, 672                                   # a multiple of 32 (the operands' scale blocks), not of 128
    q, k, v, g = (t.cuda() for t in attention_inputs(2, s, 4, 2, 128, seed=94))
    k2, v2, g2 = k.clone(), v.clone(), g.clone()
    gen = torch.Generator(device="cuda").manual_seed(8)
    for t in (k2, v2, g2):
        t[:, k0:k0 + 40] = torch.randn(t[:, k0:k0 + 40].shape, generator=gen, device="cuda").sign().to(t.dtype) * 60.0
    old = I.DQ_CAUSAL_PRESCALE, I.DQ_CAUSAL_GRANULARITY
    try:
        I.DQ_CAUSAL_PRESCALE, I.DQ_CAUSAL_GRANULARITY = True, "tile"
        tile = _eager(F.flash_attn_fp8, q, k, v, g, causal=True, deterministic=True)
        I.DQ_CAUSAL_GRANULARITY = "row"
        assert F.resolve_fp8(q, k, v, causal=True).bwd.dq_prescale == "causal_row"
        base = _eager(F.flash_attn_fp8, q, k, v, g, causal=True, deterministic=True)
        pert = _eager(F.flash_attn_fp8, q, k2, v2, g2, causal=True, deterministic=True)
    finally:
        I.DQ_CAUSAL_PRESCALE, I.DQ_CAUSAL_GRANULARITY = old
    assert torch.equal(base[0], tile[0]) and torch.equal(base[3], tile[3]) and torch.equal(base[4], tile[4])
    assert _cos(base[2], tile[2]) > 0.99999
    assert not torch.equal(base[2][:, k0:], pert[2][:, k0:])                 # the probe is not blind
    assert torch.equal(base[2][:, :k0], pert[2][:, :k0])
    assert F.check_status() == 0
