"""CPU: option validation and the plan's refusal rules, on device="meta" tensors (no CUDA work). Follows the shape of the
reference's rule table (tests/cute/test_lowprec_api.py:55-213): exception type, `.rule` id and message prefix, for the
rules that apply to the routes this library builds, plus this build's own refusals of unbuilt routes."""
import pytest
import torch

from flamia_blackwell_attention_b200 import (FP4AttnOptions as O4, FP8AttnOptions as O8, KernelTuning, resolve_fp4,
                                             resolve_fp8)
from flamia_blackwell_attention_b200 import interface_bwd_fp4

BF16 = torch.bfloat16


def M(b=1, s=1024, h=4, hk=None, d=128, rg=True):
    return torch.empty(b, s, h if hk is None else hk, d, dtype=BF16, device="meta").requires_grad_(rg)


def qkv(b=1, s=1024, h=4, hk=None, d=128, s_k=None, rg=True):
    return M(b, s, h, None, d, rg), M(b, s if s_k is None else s_k, h, hk or h, d, rg), \
        M(b, s if s_k is None else s_k, h, hk or h, d, rg)


R4, R8 = resolve_fp4, resolve_fp8
_I32 = lambda n: torch.empty(n, dtype=torch.int32, device="meta")  # noqa: E731

RULES = [
    ("r01", R4, dict(backward="fp4"), {}, ValueError, 1, "backward='fp4' is the query-row backward"),
    ("r04", R4, dict(qk_hadamard=True), dict(d=64), NotImplementedError, "E13", "flash_attn_fp4 serves head_dim 128"),
    ("r04b", R8, dict(qk_hadamard=True), dict(d=64), NotImplementedError, 4, "qk_hadamard is built for head_dim 128"),
    ("r07", R4, dict(causal_safety="key_local"), {}, ValueError, 7, "causal_safety='key_local' applies to a 4-bit P.V"),
    ("r15", R8, dict(options=O8(two_cta="on")), dict(d=64), ValueError, 15,
     "two_cta='on' but the 2-CTA backward cannot serve this call: head_dim 64"),
    ("r15b", R4, dict(options=O4(two_cta="on")), {}, ValueError, 15, "two_cta='on' but the 2-CTA backward cannot serve"),
    ("r16", R8, dict(options=O8(operand_scaling="per_tensor")), {}, ValueError, 16,
     "operand_scaling='per_tensor' cannot serve this call"),
    ("r16b", R8, dict(options=O8(grad_format="e5m2")), {}, ValueError, 16, "grad_format='e5m2' is a per-tensor option"),
    ("r16h", R8, dict(options=O8(forward_kernel="upstream")), {}, ValueError, 16,
     "flash_attn_fp8: operand_scaling='auto' resolves to token blocks, which cannot serve this call: "
     "forward_kernel='upstream'"),
    ("r16i", R4, dict(options=O4(p_scaling="block_1x32")), {}, ValueError, 16,
     "flash_attn_fp4: operand_scaling='auto' resolves to token blocks, which cannot serve this call: "
     "p_scaling='block_1x32'"),
    ("r16k", R8, dict(causal=True, options=O8(operand_scaling="token_local", ds_dq_rowlocal="all")),
     dict(s=1024, s_k=512), ValueError, 16, "operand_scaling='token_local' with causal s_q > s_k"),
    ("r16m", R8, dict(options=O8(operand_scaling="token_local")), {}, ValueError, 16,
     "operand_scaling='token_local' needs ds_dq_rowlocal='all'"),
    ("r21", R4, dict(options=O4(softmax_exp="mitchell")), {}, ValueError, 21, "Mitchell P-hat on an E4M3 P.V"),
    ("r21b", R8, dict(options=O8(softmax_exp="mitchell")), dict(rg=False), ValueError, 21,
     "Mitchell P-hat on an E4M3 P.V was removed"),
    ("r23", R4, dict(options=O4(p_frame="per_tile")), {}, ValueError, 23, "p_frame frames the 4-bit P-hat"),
    ("r26", R4, dict(options=O4(seqused_k_group_aligned=True)), {}, ValueError, 26,
     "seqused_k_group_aligned applies to seqused_k with a 4-bit P.V, which no route takes"),
    ("r27", R4, {}, dict(s=1000), ValueError, 27, "flash_attn_fp4 needs seqlen % 128 == 0"),
    ("r28c", R8, dict(score_mod=lambda *a: a[0]), {}, ValueError, 28, "score_mod needs score_mod_bwd"),
    ("r28d", R8, dict(mask_mod=lambda *a: True, causal=True), {}, ValueError, 28, "mask_mod with causal / window_size"),
    ("r29", R4, dict(options=O4(dq_operand="e4m3")), {}, ValueError, 29, "dq_operand configures the all-4-bit backward"),
    ("r29b", R4, dict(options=O4(fp4_ds_multiplier="global")), {}, ValueError, 29,
     "fp4_ds_multiplier configures the all-4-bit backward"),
    ("r32", R8, dict(q_quantized=(torch.empty(1, device="meta"), 1.0)), {}, ValueError, 32,
     "flash_attn_fp8: q_quantized and k_quantized must be supplied together"),
    ("r32b", R8, dict(q_scale_fused=True), {}, ValueError, 32, "q_scale_fused=True needs q_quantized"),
    ("r33", R8, dict(options=O8(ds_scaling="per_tensor")), {}, ValueError, 33,
     "ds_scaling='per_tensor' was removed from flash_attn_fp8"),
    ("r33b", R8, dict(options=O8(per_tensor_ds_source="recompute")), {}, ValueError, 33,
     "per_tensor_ds_source='recompute' was removed with the per-tensor dS"),
    ("r33f", R4, dict(options=O4(ds_scaling="per_tensor")), {}, ValueError, 33,
     "ds_scaling='per_tensor' was removed from flash_attn_fp4"),
    ("r34", R4, dict(options=O4(save_bf16_inputs=False)), {}, ValueError, 34, "save_bf16_inputs=False cannot serve this call"),
    ("rE13c", R8, {}, dict(d=256, rg=False), NotImplementedError, "E13", "flash_attn_fp8 serves head_dim <= 128"),
    ("rE13b", R4, {}, dict(d=192), NotImplementedError, "E13", "flash_attn_fp4 serves head_dim 128"),
    ("rE13d", R8, {}, dict(d=72, rg=False), NotImplementedError, "E13", "flash_attn_fp8 serves head_dim <= 128 (a multiple of 16"),
    ("rE13e", R8, dict(options=O8(operand_scaling="token_local", ds_dq_rowlocal="all")), dict(d=96), NotImplementedError,
     "E13", "head_dim 96 runs padded on token-block operands"),
    ("r04c", R8, dict(qk_hadamard=True), dict(d=96), NotImplementedError, 4, "qk_hadamard is built for head_dim 128"),
    ("rB6c", R8, dict(options=O8(ds_dq_rowlocal="all")), dict(d=64), NotImplementedError, "B6",
     "ds_dq_rowlocal='all' (and with it operand_scaling='token_local') is built in the head_dim 128 backward"),
    ("rB6d", R8, dict(options=O8(operand_scaling="token_local", ds_dq_rowlocal="all")), dict(d=64), NotImplementedError, "B6",
     "ds_dq_rowlocal='all' (and with it operand_scaling='token_local') is built in the head_dim 128 backward"),
    ("r16t", R8, dict(options=O8(operand_scaling="token_local", ds_dq_rowlocal="all")), dict(s=200), ValueError, 16,
     "operand_scaling='token_local' runs the fold forward, which takes no documents"),
    # this build's own refusals: routes and features it does not build
    ("rB1", R4, dict(pv_precision="fp4", causal=True), {}, NotImplementedError, "B1", "pv_precision='fp4'"),
    ("rB2", R8, dict(options=O8(tuning=KernelTuning(bwd_fp4_ld_rep=64))), {}, ValueError, "B2", "KernelTuning"),
    ("r28w", R8, dict(window_size=(-5, 0)), {}, ValueError, 28, "window_size entries"),
    ("rB5", R8, dict(deterministic=True, softcap=30.0), {}, NotImplementedError, "B5", "deterministic=True"),
    ("rB4b", R8, dict(softcap=30.0, options=O8(ds_dq_rowlocal="all")), {}, NotImplementedError, "B4", "softcap"),
    ("rB4c", R8, dict(seqused_k=_I32(2), options=O8(operand_scaling="token_local", ds_dq_rowlocal="all")), {},
     NotImplementedError, "B4", "batched seqused_k"),
    ("rB6", R8, dict(options=O8(ds_scaling="row_local")), {}, NotImplementedError, "B6", "ds_scaling='row_local'"),
    ("rB6b", R8, dict(options=O8(p_hat_frame="group", operand_scaling="token_local", ds_dq_rowlocal="all")), {},
     NotImplementedError, "B6", "p_hat_frame='group'"),
    ("rB7", R8, dict(q_quantized=(1, 1.0), k_quantized=(1, 1.0)), {}, NotImplementedError, "B7", "pre-quantised Q / K"),
]


@pytest.mark.parametrize("rid,fn,kw,shape,exc,rule,prefix", RULES, ids=[r[0] for r in RULES])
def test_rule(rid, fn, kw, shape, exc, rule, prefix):
    q, k, v = qkv(**shape)
    with pytest.raises(exc) as ei:
        fn(q, k, v, **kw)
    assert type(ei.value) is exc
    assert getattr(ei.value, "rule", None) == rule, (getattr(ei.value, "rule", None), str(ei.value))
    assert str(ei.value).startswith(prefix), str(ei.value)


def test_defaults_resolved():
    q, k, v = qkv(b=4, s=4096, h=16)
    p = R8(q, k, v, causal=True)
    assert (p.entry, p.route, p.fwd.qk_format, p.fwd.operand_scaling, p.fwd.qk_hadamard) == \
        ("fp8", "fp8", "e4m3", "token_block", True)
    assert (p.bwd.kernel, p.bwd.ds_scaling, p.bwd.ds_dq_rowlocal, p.bwd.dq_prescale) == ("1cta", "block_32x32", "off", "row")
    assert abs(p.softmax_scale - 128 ** -0.5) < 1e-12 and "qk_hadamard = on" in p.log()
    p4 = R4(q, k, v, causal=True)
    assert (p4.route, p4.fwd.qk_format, p4.fwd.pv_operand) == ("fp4.e4m3_pv", "nvfp4", "e4m3")
    # GQA config of the benchmark set: token-local operands turn the rotation off and say so
    q, k, v = qkv(b=2, s=8192, h=32, hk=8)
    p = R8(q, k, v, causal=True, options=O8(operand_scaling="token_local", ds_dq_rowlocal="all"))
    assert p.fwd.operand_scaling == "token_local" and not p.fwd.qk_hadamard and p.bwd.ds_dq_rowlocal == "all"
    assert "no rotated token-local quantiser" in p.log()
    # no gradient required: no backward kernel in the plan
    q, k, v = qkv(rg=False)
    assert R8(q, k, v).bwd.kernel == "none"


def test_causal_dq_prescale_switch_is_read_at_resolution():
    q, k, v = qkv()
    assert R8(q, k, v, causal=True).bwd.dq_prescale == "row"
    interface_bwd_fp4.DQ_CAUSAL_PRESCALE = True
    try:
        assert R8(q, k, v, causal=True).bwd.dq_prescale == "causal_tile"
        assert R8(q, k, v, causal=False).bwd.dq_prescale == "row"
    finally:
        interface_bwd_fp4.DQ_CAUSAL_PRESCALE = False


def test_options_validate_at_construction_and_hash():
    with pytest.raises(ValueError, match="FP8AttnOptions.ds_scaling must be one of"):
        O8(ds_scaling="nope")
    with pytest.raises(ValueError, match="FP4AttnOptions.q_block_2d must be a bool"):
        O4(q_block_2d=1)
    with pytest.raises(ValueError, match="tuning must be a KernelTuning"):
        O8(tuning=3)
    with pytest.raises(TypeError):
        KernelTuning(not_a_field=1)
    assert O8() == O8() and hash(O8(two_cta="off")) == hash(O8(two_cta="off")) and O8() != O8(two_cta="off")
    with pytest.raises(Exception):
        O8().two_cta = "on"      # frozen


def test_varlen_shapes_resolve():
    q = torch.empty(3000, 4, 128, dtype=BF16, device="meta").requires_grad_(True)
    cu = _I32(5)
    p = R8(q, q, q, causal=True, cu_seqlens_q=cu, cu_seqlens_k=cu)
    assert p.shape.varlen and not p.shape.aligned_varlen and p.shape.b == 4 and p.shape.tot_q == 3000
    p = R8(q, q, q, causal=True, cu_seqlens_q=cu, cu_seqlens_k=cu, seqused_q=_I32(4), seqused_k=_I32(4))
    assert p.shape.aligned_varlen
    q2 = torch.empty(2, 1000, 4, 128, dtype=BF16, device="meta")
    assert R8(q2, q2, q2).fwd.ragged_documents


@pytest.mark.parametrize("d,d_pad", [(16, 64), (48, 64), (80, 128), (96, 128)])
def test_padded_head_dims_resolve(d, d_pad):
    """Rule E13 of the reference (flash_attn/cute/lowprec/plan.py:1529-1541): multiples of 16 below 128 are served padded
    to the next of 64 / 128, with the softmax scale of the call's own head dim and the rotation off."""
    plan = resolve_fp8(*qkv(d=d), causal=True)
    assert plan.pad_from == d and plan.shape.d == d_pad and abs(plan.softmax_scale - d ** -0.5) < 1e-12
    assert not plan.fwd.qk_hadamard
    rows = {f: (val, why) for f, val, why in plan.resolution_log}
    assert rows["head_dim_padding"][0] == str(d_pad) and rows["qk_hadamard"] == ("off", f"auto: built for head_dim 128, this call has {d}")
    assert resolve_fp8(*qkv(d=d_pad), causal=True).pad_from == 0
    assert resolve_fp8(*qkv(d=d), softmax_scale=0.25).softmax_scale == 0.25
