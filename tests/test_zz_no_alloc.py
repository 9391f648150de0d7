"""fl_bwd_static_acc (backward pass with the library-held dQ accumulator) against fl_bwd + fl_dq_post with a caller
buffer, through the C ABI. Collected last (file name) so that it also runs after every other GPU test has used the
library; it passes alone as well."""
import math

import pytest
import torch

from tests.inputs import attention_inputs

pytestmark = pytest.mark.gpu


def _operands(b, s, h, d, seed, rotate=True, fp4=False):
    from flamia_blackwell_attention_b200 import kernels as K, _lib as L
    q, k, v, g = (t.cuda() for t in attention_inputs(b, s, h, h, d, seed=seed))
    sc = 1.0 / math.sqrt(d)
    kw = dict(apply_hadamard_rotation=rotate)
    if fp4:     # the mixed route: rotated NVFP4 copies feed S, the E4M3 codes stay unrotated
        kw.update(also_make_nvfp4_copy=True, hadamard_rotation_scope="nvfp4_copy")
    qq = K.quantize_fp8_blocks(q, **kw)
    kq = K.quantize_fp8_blocks(k, output_tile_stats=True, **kw)
    vq = K.quantize_fp8_blocks(v, output_tile_stats=True)
    st = K.new_status(q.device)
    out, lse, _ = K.attn_fwd(qq, kq, vq, causal=True, softmax_scale=sc, status=st,
                             mode=L.FL_MODE_FP4 if fp4 else L.FL_MODE_FP8)
    acc = torch.empty(b, h, s, d, dtype=torch.float16, device="cuda")
    gq = K.quantize_fp8_blocks(g, compute_d_with_output=out, shifted_log2_lse_from=lse, log2_lse_shift=8.0,
                               d_multiplier=-2.0 ** -8, zero_accumulator=acc, output_tile_stats=True)
    ks, ps = K.dq_prescale(gq["tile_stats"], vq["tile_stats"], kq["tile_stats"])
    return K, qq, kq, vq, gq, acc, ks, ps, sc, st


@pytest.mark.parametrize("b,s,h", [(1, 128, 2), (2, 512, 4), (1, 1024, 3)])
def test_static_accumulator_matches_caller_buffer(b, s, h):
    d = 128
    K, qq, kq, vq, gq, acc, ks, ps, sc, st = _operands(b, s, h, d, seed=11)
    dk0, dv0, _ = K.attn_bwd(qq, kq, vq, gq, lse_log2=gq["lse_log2"], d_rows=gq["D"], dq_acc=acc, dq_scale=ks,
                             causal=True, softmax_scale=sc, had_dk=True, status=st)
    dq0 = K.dq_post(acc, ps, sc, b=b, s=s, h=h, d=d, unrotate=True)
    for call in range(2):      # two calls in a row: the second starts from the array the first one left behind
        dq1, dk1, dv1, _ = K.attn_bwd_static_acc(qq, kq, vq, gq, lse_log2=gq["lse_log2"], d_rows=gq["D"], dq_scale=ks,
                                                 post_scale=ps, mult=sc, causal=True, softmax_scale=sc, had_dk=True,
                                                 had_dq=True, status=st)
        torch.cuda.synchronize()
        assert K.read_status(st) == 0
        assert torch.equal(dk1, dk0) and torch.equal(dv1, dv0), f"call {call}"
        if s == 128:           # one key tile per query tile: a single add per accumulator element, order-free
            assert torch.equal(dq1, dq0), f"call {call}"
        else:                  # several f16 adds per element arrive in a run-dependent order
            err = (dq1.float() - dq0.float()).norm() / dq0.float().norm()
            assert err < 2e-3, f"call {call}: {err}"
        assert torch.isfinite(dq1.float()).all()


@pytest.mark.parametrize("d,fp4", [(64, False), (128, True)])
def test_static_accumulator_other_kernels(d, fp4):
    """The same comparison on the head_dim 64 kernel (accumulator laid out (b, h, s, d)) and on the mixed NVFP4 / FP8
    route (FL_MODE_FP4), neither with rotated E4M3 codes."""
    from flamia_blackwell_attention_b200 import _lib as L
    b, s, h = 2, 384, 3
    mode = L.FL_MODE_FP4 if fp4 else L.FL_MODE_FP8
    K, qq, kq, vq, gq, acc, ks, ps, sc, st = _operands(b, s, h, d, seed=12, rotate=fp4, fp4=fp4)
    dk0, dv0, _ = K.attn_bwd(qq, kq, vq, gq, lse_log2=gq["lse_log2"], d_rows=gq["D"], dq_acc=acc, dq_scale=ks,
                             causal=True, softmax_scale=sc, status=st, mode=mode)
    dq0 = K.dq_post(acc, ps, sc, b=b, s=s, h=h, d=d)
    for call in range(2):
        dq1, dk1, dv1, _ = K.attn_bwd_static_acc(qq, kq, vq, gq, lse_log2=gq["lse_log2"], d_rows=gq["D"], dq_scale=ks,
                                                 post_scale=ps, mult=sc, causal=True, softmax_scale=sc, status=st, mode=mode)
        torch.cuda.synchronize()
        assert K.read_status(st) == 0
        assert torch.equal(dk1, dk0) and torch.equal(dv1, dv0), f"call {call}"
        err = (dq1.float() - dq0.float()).norm() / dq0.float().norm()
        assert err < 2e-3 and torch.isfinite(dq1.float()).all(), f"call {call}: {err}"


def test_static_accumulator_limit():
    """A problem beyond FL_STATIC_ACC_MAX_ELEMS is refused before anything is enqueued."""
    import ctypes as C
    from flamia_blackwell_attention_b200 import _lib as L
    a = L.AttnArgs()
    a.b, a.h, a.s_q, a.d = 4, 16, 4096, 128          # 32 Mi elements > 8 Mi
    one = torch.zeros(1, device="cuda")
    rc = L.load().fl_bwd_static_acc(C.byref(a), L.ptr(one), 1.0, L.ptr(one), None)
    assert rc == 4
