"""The attention call as registered torch ops, so that selective activation checkpointing can save it and torch.compile
can trace it. Same op names and schemas as the reference's flash_attn/cute/lowprec/_op.py (:12-16, 428-476):

    lowbit_attn::fp8(Tensor q, Tensor k, Tensor v, Tensor[] docs, int plan, int docs_id) -> (Tensor, Tensor, Tensor[])
    lowbit_attn::fp8_bwd(Tensor dout, Tensor[] state, int entry) -> (Tensor, Tensor, Tensor)          (and ::fp4)

`plan` is a process-local integer handle into an append-only registry of resolved plans; `docs` carries the varlen
tensors (cu_seqlens_q, cu_seqlens_k[, seqused_q, seqused_k]). The saved state is codes + factor tables + O + LSE, not the
bf16 inputs. LSE and the state are non-differentiable; gradients are not materialised for unused outputs.
"""
from __future__ import annotations

import threading
from typing import List

import torch

from . import _routes

_REG_LOCK = threading.Lock()
_PLANS: list = []          # handle -> AttnPlan
_PLAN_HANDLES: dict = {}   # AttnPlan (by value: plans are frozen) -> handle
_ENTRIES: list = []        # backward entry handle -> (plan handle, docs meta)
_ENTRY_HANDLES: dict = {}  # (plan handle, docs meta) -> backward entry handle


def register_plan(plan) -> int:
    """Handle of a plan. Equal plans share one handle, so the registry grows with the number of DISTINCT plans a
    process resolves, not with the number of calls or of cache evictions."""
    with _REG_LOCK:
        h = _PLAN_HANDLES.get(plan)
        if h is None:
            h = _PLAN_HANDLES[plan] = len(_PLANS)
            _PLANS.append(plan)
        return h


def _register_entry(plan_id, docs_meta) -> int:
    key = (plan_id, docs_meta)
    with _REG_LOCK:
        h = _ENTRY_HANDLES.get(key)
        if h is None:
            h = _ENTRY_HANDLES[key] = len(_ENTRIES)
            _ENTRIES.append(key)
        return h


def _fwd_impl(q, k, v, docs: List[torch.Tensor], plan: int, docs_id: int):
    p = _PLANS[plan]
    seqused_k = None
    if p.fwd.seqused_k:           # batched form: docs = [seqused_k]
        seqused_k, docs = docs[0], []
    if len(docs) == 6:            # precomputed maps: cu, start, len, row_map, slot_src, slot_rows
        d = _routes.Docs.from_tables(docs[1], docs[2], docs[3], docs[4], docs[5], docs[3].numel())
    else:
        cu_q = docs[0] if len(docs) > 0 else None
        cu_k = docs[1] if len(docs) > 1 else None
        su_q = docs[2] if len(docs) > 2 else None
        su_k = docs[3] if len(docs) > 3 else None
        d = _routes.docs_of(p, q, cu_q, cu_k, su_q, su_k)
    out, lse, state = _routes.forward(p, q, k, v, d, seqused_k)
    meta = None if d is None else (d.capacity, d.aligned)
    entry = _register_entry(plan, meta)
    # The kernels' O (and LSE, except under repacked documents, whose LSE keeps the aligned buffer's rows and is not
    # returned) ARE the op's outputs, up to a view: the autograd node saves those itself and the backward rebuilds the
    # kernels' shapes from them, because an op output may not alias another.
    # The entry handle rides along as a 0-d tensor so that the backward op needs no Python object.
    keep_lse = d is not None and not d.aligned
    state = list(state[1:] if keep_lse else state[2:]) + [torch.tensor(entry, dtype=torch.int64)]
    return out, lse, state


def _bwd_impl(dout, state: List[torch.Tensor], entry: int):
    plan_id, meta = _ENTRIES[entry]
    return _routes.backward(_PLANS[plan_id], state[:-1], dout, meta)     # state = [out_k, lse_k, codes..., entry]


def _fake_fwd(q, k, v, docs, plan, docs_id):
    p = _PLANS[plan]
    sh = p.shape
    is_docs = sh.varlen or p.fwd.ragged_documents
    if sh.aligned_varlen or (is_docs and sh.varlen and p.fwd.return_lse):
        lse_shape = (sh.h, sh.tot_q)
    elif is_docs and not p.fwd.return_lse:
        lse_shape = (0,)
    else:
        lse_shape = (sh.b, sh.h, sh.s_q)
    n_docs = int(docs[0].shape[0]) - 1 if (len(docs) > 0 and not p.fwd.seqused_k) else 0
    spec = _routes.state_spec(p, n_docs, q.dtype, capacity=int(docs[3].numel()) if len(docs) == 6 else None)
    # as _fwd_impl: O / LSE leave as the op's outputs; repacked documents keep the aligned buffer's LSE in the state
    state = [q.new_empty(shape, dtype=dt) for shape, dt in (spec[1:] if (is_docs and not sh.aligned_varlen) else spec[2:])]
    state.append(torch.empty((), dtype=torch.int64))
    return torch.empty_like(q), q.new_empty(lse_shape, dtype=torch.float32), state


def _fake_bwd(dout, state, entry):
    plan_id, _ = _ENTRIES[entry]
    sh = _PLANS[plan_id].shape
    if sh.varlen:
        kshape = (sh.tot_k, sh.h_kv, sh.d)
    else:
        kshape = (sh.b, sh.s_k, sh.h_kv, sh.d)
    return torch.empty_like(dout), dout.new_empty(kshape), dout.new_empty(kshape)


def _define(entry: str):
    name = f"lowbit_attn::{entry}"
    torch.library.define(name, "(Tensor q, Tensor k, Tensor v, Tensor[] docs, int plan, int docs_id) -> "
                               "(Tensor, Tensor, Tensor[])")
    torch.library.define(name + "_bwd", "(Tensor dout, Tensor[] state, int entry) -> (Tensor, Tensor, Tensor)")
    torch.library.impl(name, "CUDA")(_fwd_impl)
    torch.library.impl(name + "_bwd", "CUDA")(_bwd_impl)
    torch.library.register_fake(name)(_fake_fwd)
    torch.library.register_fake(name + "_bwd")(_fake_bwd)

    def setup_context(ctx, inputs, output):
        out, lse, state = output
        ctx.n_docs = len(inputs[3])
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(lse, *state)
        ctx.save_for_backward(out, lse, *state)

    def backward(ctx, dout, dlse, dstate):
        saved = list(ctx.saved_tensors)
        nodocs = [None] * ctx.n_docs
        if dout is None:
            return None, None, None, nodocs, None, None
        entry_id = int(saved[-1])
        meta = _ENTRIES[entry_id][1]
        if meta is None:                     # batched: the outputs are the kernels' O / LSE
            state = saved
        else:                                # documents: the kernels saw one batch entry of (rows, h, d)
            o = saved[0].reshape(1, -1, saved[0].shape[-2], saved[0].shape[-1])
            state = [o, saved[1].unsqueeze(0)] + saved[2:] if meta[1] else [o] + saved[2:]
        dq, dk, dv = getattr(torch.ops.lowbit_attn, entry + "_bwd")(dout.contiguous(), state, entry_id)
        return dq, dk, dv, nodocs, None, None

    torch.library.register_autograd(name, backward, setup_context=setup_context)


for _e in ("fp8", "fp4"):
    _define(_e)


def op_apply(plan, q, k, v, docs_tensors):
    """Runs the registered op of the plan's entry; returns (out, lse)."""
    handle = register_plan(plan)
    op = getattr(torch.ops.lowbit_attn, plan.entry)
    out, lse, _state = op(q, k, v, list(docs_tensors), handle, 0)
    return out, lse
