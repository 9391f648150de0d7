"""DocMaps (precomputed document tables): the numpy construction, the device construction and the tables the cu_seqlens
form builds per call agree; the GPU test runs the public call with doc_maps= and compares it bit for bit with the
cu_seqlens form. Follows tests/cute/test_lowprec_docmaps.py of the reference (same outputs either way)."""
import numpy as np
import pytest
import torch

from inputs import attention_inputs


LENS = [300, 128, 77, 515, 1, 127, 129]


def _cu(lens):
    return torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)


def test_numpy_tables_equal_the_per_call_tables():
    from flamia_blackwell_attention_b200 import DocMaps
    from flamia_blackwell_attention_b200._routes import Docs
    cu = _cu(LENS)
    total = int(cu[-1])
    ref = Docs(cu, cu[1:] - cu[:-1], total, False)              # what a cu_seqlens call builds (here on CPU tensors)
    m = DocMaps.from_cu_seqlens(cu, padded_size=ref.capacity)
    for name in ("start", "len", "row_map", "slot_src", "slot_rows"):
        assert torch.equal(getattr(m, name), getattr(ref, name)), name
    assert (m.total, m.max_seqlen, m.padded_size, m.max_num_documents) == (total, max(LENS), ref.capacity, len(LENS))
    # every packed row appears exactly once, in order, inside its document's aligned slot
    rm = m.row_map.numpy()
    assert sorted(rm[rm >= 0].tolist()) == list(range(total))
    for d, (s0, n) in enumerate(zip(m.start.tolist(), m.len.tolist())):
        assert s0 % 128 == 0 and rm[s0:s0 + n].tolist() == list(range(int(cu[d]), int(cu[d]) + n))


def test_fixed_capacity_and_padding_documents():
    from flamia_blackwell_attention_b200 import DocMaps
    from flamia_blackwell_attention_b200.docmaps import default_padded_size
    cu = _cu(LENS)
    m = DocMaps.from_cu_seqlens(cu, max_num_documents=16, max_seqlen=2048)
    assert m.max_num_documents == 16 and m.padded_size == default_padded_size(int(cu[-1]), 16) and m.max_seqlen == 2048
    assert m.len[len(LENS):].sum() == 0 and int(m.cu[-1]) == int(cu[-1])
    m2 = DocMaps.from_cu_seqlens(_cu([5, 1000]), max_num_documents=16, max_seqlen=2048, padded_size=m.padded_size)
    m.copy_(m2)                                                  # same shapes: an in-place refresh
    assert m.total == 1005 and m.len[:2].tolist() == [5, 1000]
    with pytest.raises(ValueError):
        DocMaps.from_cu_seqlens(cu, max_num_documents=3)
    with pytest.raises(ValueError):
        DocMaps.from_cu_seqlens(cu, padded_size=1024)


def test_plan_of_a_doc_maps_call_is_the_varlen_plan():
    import flamia_blackwell_attention_b200 as F
    cu = _cu(LENS)
    m = F.DocMaps.from_cu_seqlens(cu, max_num_documents=8, max_seqlen=1024)
    q = torch.empty(int(cu[-1]), 4, 128, dtype=torch.bfloat16, device="meta")
    p = F.resolve_fp8(q, q, q, causal=True, cu_seqlens_q=m.cu.to("meta"), cu_seqlens_k=m.cu.to("meta"), max_seqlen_q=m.max_seqlen,
                      max_seqlen_k=m.max_seqlen)
    assert p.shape.varlen and not p.shape.aligned_varlen and p.shape.b == 8


@pytest.mark.gpu
@pytest.mark.parametrize("route", ["fp8", "fp4"])
@pytest.mark.parametrize("where", ["cpu_built", "cuda_built"])
def test_doc_maps_call_equals_cu_seqlens_call(route, where):
    import warnings
    import flamia_blackwell_attention_b200 as F
    fn = F.flash_attn_fp8 if route == "fp8" else F.flash_attn_fp4
    lens = LENS
    cu = _cu(lens)
    total, h, d = int(cu[-1]), 4, 128
    q, k, v, g = (t[0].cuda() for t in attention_inputs(1, total, h, 2, d, seed=71))
    cu_d = cu.cuda()

    def run(**kw):
        qc, kc, vc = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        out = fn(qc, kc, vc, causal=True, **kw)
        out.backward(g)
        torch.cuda.synchronize()
        return out.detach(), qc.grad, kc.grad, vc.grad
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ref = run(cu_seqlens_q=cu_d, cu_seqlens_k=cu_d, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    cap = ((total + 127 * len(lens) + 127) // 128) * 128        # the cu_seqlens form's buffer: same rows, same bits
    if where == "cpu_built":
        maps = F.DocMaps.from_cu_seqlens(cu, padded_size=cap).pin_memory().to("cuda", non_blocking=True)
    else:
        maps = F.DocMaps.from_cu_seqlens(cu_d, padded_size=cap, total_q=total, max_seqlen=max(lens))
    torch.cuda.set_sync_debug_mode("error")                      # nothing on the maps path reads a device value
    try:
        got = run(doc_maps=maps)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    assert torch.equal(got[0], ref[0]) and torch.equal(got[2], ref[2]) and torch.equal(got[3], ref[3])
    a, b = got[1].double().flatten(), ref[1].double().flatten()
    assert float(a @ b / (a.norm() * b.norm())) > 0.99999        # f16 partial sums are added in arrival order
    # a larger, fixed capacity with padding documents gives the same rows
    maps2 = F.DocMaps.from_cu_seqlens(cu, max_num_documents=12, max_seqlen=1024).to("cuda")
    got2 = run(doc_maps=maps2)
    assert torch.equal(got2[0], ref[0]) and torch.equal(got2[2], ref[2]) and torch.equal(got2[3], ref[3])
    with pytest.raises(ValueError):
        fn(q, k, v, causal=True, doc_maps=maps, cu_seqlens_q=cu_d, cu_seqlens_k=cu_d)
