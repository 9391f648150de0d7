"""Pre-quantised E4M3 inputs (FlashAttention-3's q_descale / k_descale / v_descale convention; the reference's
flash_attn/cute/lowprec/prequant_fa3.py, docs/lowprec.md:97-137). CPU: the refusals. GPU: outputs and straight-through
gradients against fp32 attention on the DEQUANTISED codes: what is left is the kernels' own E4M3 rounding of P-hat, dS-hat
and dO and the f16 accumulation of dQ (rel-L2 below 3.2e-2 forward, 5e-2 backward, as for operands the library quantises)."""
import pytest
import torch

from inputs import attention_inputs
from oracle import attention_oracle as A


def _prequantise(x, h_kv, pow2=False):
    """codes (E4M3) and descale (b, h_kv) with x ~= codes * descale[b, kv head of the head]."""
    b, s, h, d = x.shape
    g = h // h_kv
    amax = x.float().abs().reshape(b, s, h_kv, g * d).amax(dim=(1, 3))                # (b, h_kv)
    scale = amax / 448.0
    if pow2:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    codes = (x.float() / scale.repeat_interleave(g, dim=1)[:, None, :, None]).to(torch.float8_e4m3fn)
    return codes, scale.float()


def _deq(codes, scale):
    g = codes.shape[2] // scale.shape[1]
    return codes.float() * scale.repeat_interleave(g, dim=1)[:, None, :, None]


def test_refusals_name_their_rule():
    import flamia_blackwell_attention_b200 as F
    q = torch.zeros(1, 128, 2, 128).to(torch.float8_e4m3fn)
    d = torch.ones(1, 2)
    cases = [
        (dict(q_descale=d, k_descale=d), 32, "pre-quantised E4M3 inputs need"),
        (dict(q_descale=d, k_descale=d, v_descale=torch.ones(2, 2)), 32, "v_descale is a float32"),
        (dict(q_descale=d, k_descale=d, v_descale=d, qk_hadamard=True), 32, "qk_hadamard=True"),
        (dict(q_descale=d, k_descale=d, v_descale=d, grad_proxies=(q, q, q)), 32, "grad_proxies[q]"),
        (dict(q_descale=d, k_descale=d, v_descale=d,
              options=F.FP8AttnOptions(operand_scaling="token_local", ds_dq_rowlocal="all")), 32, "block-scaled"),
    ]
    for kw, rule, prefix in cases:
        with pytest.raises(Exception) as ei:
            F.flash_attn_fp8(q, q, q, causal=True, **kw)
        assert getattr(ei.value, "rule", None) == rule and str(ei.value).startswith(prefix), (kw.keys(), ei.value)
    with pytest.raises(Exception) as ei:
        F.flash_attn_fp8(torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16), q, q, q_descale=d, k_descale=d, v_descale=d)
    assert ei.value.rule == 32
    with pytest.raises(Exception) as ei:
        F.flash_attn_fp4(q, q, q, q_descale=d, k_descale=d, v_descale=d)
    assert ei.value.rule == "B7"


@pytest.mark.gpu
@pytest.mark.parametrize("b,s_q,s_k,h,hk,d,causal,pow2", [
    (2, 512, 512, 4, 2, 128, True, False),
    (1, 384, 384, 2, 2, 64, False, False),
    (1, 256, 640, 4, 1, 128, True, True),
])
def test_prequant_against_fp32_attention_on_the_dequantised_codes(b, s_q, s_k, h, hk, d, causal, pow2):
    import flamia_blackwell_attention_b200 as F
    q, _, _, g = attention_inputs(b, s_q, h, hk, d, seed=101)
    _, k, v, _ = attention_inputs(b, s_k, h, hk, d, seed=102)
    k = k * 1.7                                               # different scales per operand
    v = v * 0.3
    q8, qd = _prequantise(q, hk, pow2)
    k8, kd = _prequantise(k, hk, pow2)
    v8, vd = _prequantise(v, hk, pow2)
    want = A.attention_fp32(_deq(q8, qd), _deq(k8, kd), _deq(v8, vd), g.float(), causal=causal)
    pq, pk, pv = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out, lse = F.flash_attn_fp8(q8.cuda(), k8.cuda(), v8.cuda(), q_descale=qd.cuda(), k_descale=kd.cuda().double(),
                                v_descale=vd.cuda(), grad_proxies=(pq, pk, pv), causal=causal, return_lse=True)
    assert out.dtype == torch.bfloat16 and out.shape == q.shape
    out.backward(g.cuda())
    torch.cuda.synchronize()
    assert F.check_status() == 0
    got = (out.detach(), lse, pq.grad, pk.grad, pv.grad)
    for name, a, r, tol in zip(("o", "lse", "dq", "dk", "dv"), got, want, (3.2e-2, 2e-3, 5e-2, 5e-2, 5e-2)):
        a, r = a.float().cpu(), r.float()
        fin = torch.isfinite(r)
        assert torch.equal(torch.isfinite(a), fin), name
        err = float((a[fin] - r[fin]).norm() / (r[fin].norm() + 1e-30))
        print(name, err)
        assert err < tol, (name, err)
    # no gradient wanted: the same output, no state kept
    with torch.no_grad():
        out2 = F.flash_attn_fp8(q8.cuda(), k8.cuda(), v8.cuda(), q_descale=qd.cuda(), k_descale=kd.cuda(),
                                v_descale=vd.cuda(), causal=causal)
    assert torch.equal(out2, out.detach())


@pytest.mark.gpu
def test_prequant_with_power_of_two_descales_equals_float_path():
    """Power-of-two descales have mantissa 1: the multipliers are exact ones, and scaling every descale by 2 moves O and
    the gradients by exact powers of two."""
    import flamia_blackwell_attention_b200 as F
    b, s, h, hk, d = 1, 256, 2, 2, 128
    q, k, v, g = attention_inputs(b, s, h, hk, d, seed=103)
    q8, qd = _prequantise(q, hk, True)
    k8, kd = _prequantise(k, hk, True)
    v8, vd = _prequantise(v, hk, True)

    def run(qd_, kd_, vd_, scale):
        p = tuple(t.cuda().requires_grad_(True) for t in (q, k, v))
        o = F.flash_attn_fp8(q8.cuda(), k8.cuda(), v8.cuda(), q_descale=qd_.cuda(), k_descale=kd_.cuda(), v_descale=vd_.cuda(),
                             grad_proxies=p, causal=True, softmax_scale=scale, deterministic=True)
        o.backward(g.cuda())
        torch.cuda.synchronize()
        return o.detach(), p[0].grad, p[1].grad, p[2].grad
    base = run(qd, kd, vd, 0.125)
    # q descale x 2 with the softmax scale halved: the scores are the same; V descale x 4: O x 4
    moved = run(qd * 2, kd, vd * 4, 0.0625)
    assert torch.equal(moved[0].float(), base[0].float() * 4)
    assert torch.equal(moved[3].float(), base[3].float())                  # dV = P^T dO does not see V's scale
    assert torch.allclose(moved[2].float(), base[2].float() * 4, rtol=2e-2, atol=1e-6)   # dK ~ dS^T Q: dS x 4, q x 2, scale / 2
