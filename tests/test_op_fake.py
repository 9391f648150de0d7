"""The registered ops' fake (meta) implementations: shapes and dtypes of every output, saved state included, without a
GPU (FakeTensorMode creates device-less CUDA tensors). The same expectations are checked against the real ops on a GPU in
tests/test_gpu_api.py::test_state_matches_its_spec."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import flamia_blackwell_attention_b200 as F
from flamia_blackwell_attention_b200 import _op, _routes


def _expected(plan, n_docs, dtype):
    spec = _routes.state_spec(plan, n_docs, dtype)
    is_docs = plan.shape.varlen or plan.fwd.ragged_documents
    # O / LSE leave as the op's outputs; repacked documents keep the aligned buffer's LSE in the state
    return (spec[1:] if (is_docs and not plan.shape.aligned_varlen) else spec[2:]) + [((), torch.int64)]


CASES = [
    ("fp8", dict(causal=True), (2, 256, 4, 2, 128), False, None),
    ("fp8", dict(causal=True), (2, 256, 4, 2, 128), True, None),
    ("fp4", dict(causal=True), (1, 384, 2, 2, 128), True, None),
    ("fp8", dict(causal=True, options="tl"), (1, 256, 4, 1, 128), True, None),
    ("fp8", dict(causal=True), (2, 300, 2, 2, 128), True, None),               # ragged: runs as documents
    ("fp8", dict(causal=True), (1, 1020, 2, 2, 128), True, [300, 128, 77, 515]),  # packed, repacked
]


@pytest.mark.parametrize("entry,kw,shape,grad,lens", CASES)
def test_fake_forward_and_backward_shapes(entry, kw, shape, grad, lens):
    b, s, h, hk, d = shape
    kw = dict(kw)
    if kw.get("options") == "tl":
        kw["options"] = F.FP8AttnOptions(operand_scaling="token_local", ds_dq_rowlocal="all")
    resolve = F.resolve_fp8 if entry == "fp8" else F.resolve_fp4
    op = getattr(torch.ops.lowbit_attn, entry)
    op_bwd = getattr(torch.ops.lowbit_attn, entry + "_bwd")
    with FakeTensorMode():
        if lens is None:
            q = torch.empty(b, s, h, d, dtype=torch.bfloat16, device="cuda", requires_grad=grad)
            k = torch.empty(b, s, hk, d, dtype=torch.bfloat16, device="cuda", requires_grad=grad)
            v = torch.empty(b, s, hk, d, dtype=torch.bfloat16, device="cuda", requires_grad=grad)
            docs = []
        else:
            q = torch.empty(s, h, d, dtype=torch.bfloat16, device="cuda", requires_grad=grad)
            k = torch.empty(s, hk, d, dtype=torch.bfloat16, device="cuda", requires_grad=grad)
            v = torch.empty(s, hk, d, dtype=torch.bfloat16, device="cuda", requires_grad=grad)
            cu = torch.empty(len(lens) + 1, dtype=torch.int32, device="cuda")
            docs = [cu, cu]
            kw.update(cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
        plan = resolve(q, k, v, **kw)
        pid = _op.register_plan(plan)
        out, lse, state = op(q.detach(), k.detach(), v.detach(), docs, pid, 0)
        assert out.shape == q.shape and out.dtype == q.dtype
        want = _expected(plan, 0 if lens is None else len(lens), q.dtype)
        assert [(tuple(t.shape), t.dtype) for t in state] == [(tuple(sh), dt) for sh, dt in want]
        if grad:
            entry_id = _op._register_entry(pid, None)
            dq, dk, dv = op_bwd(torch.empty_like(out), list(state), entry_id)
            assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
