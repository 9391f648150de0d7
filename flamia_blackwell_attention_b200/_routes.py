"""Route bodies: what one resolved plan launches, forward and backward. Host glue only (allocation, views, the order
of the C-ABI calls); mirrors the launch sequence of the reference's flash_attn/cute/lowprec/_routes.py (_fp8_forward_mx
:709, _fp8_backward_mx :911, _e4pv_forward_blk32 :308, run_documents :1388):

  forward   3 quantiser launches (Q, K [rotated], V) + 1 forward kernel
  backward  1 fused prologue (dO quantiser + D + shifted LSE + zeroed accumulator) + 1 pre-scale + 1 main kernel
            + 1 dQ postprocess
No host synchronisation anywhere; everything is enqueued on the current stream.
"""
from __future__ import annotations

import os

import torch

from . import _lib as L
from . import kernels as K

P_SHIFT_LOG2 = 8.0     # the backward recomputes P' = 2^8 P (its E4M3 P-hat then uses the normal range)


def backward_scalars(softmax_scale, dq_boost=1.0):
    """The eight kernel scalars of the reference's 8-bit backward (flash_attn/cute/device_scales.py:734-743, slots 0-7)
    as this library uses them. Block-scaled operands carry their scales with the codes, so every operand descale is 1
    and the scalars are constants: [0] softmax scale of S, [1] dP-sum scale, [2] dS boost 2^-8 (with P' = 2^8 P), [3] dV
    scale 2^-8 (folded into the dV epilogue), [4] dK scale (the dK epilogue), [5] the f16 dQ pre-scale (per query tile on
    the device: fl_dq_prescale; `dq_boost` stands for it here), [6] the D fold multiplier -2^-8 (applied by the dO
    quantiser launch), [7] the dQ postprocess scale softmax_scale / pre-scale."""
    import numpy as np
    f = np.float32
    p_shift = f(2.0 ** P_SHIFT_LOG2)
    sm = f(softmax_scale)
    return (sm, f(1.0), f(1.0) / p_shift, f(1.0) / p_shift, sm, f(dq_boost), -(f(1.0) / p_shift), sm / f(dq_boost))


# --------------------------------------------------------------------------------------------------------------- status
# Every device-side wait of the kernels is bounded; one that runs out writes 0x100 | site into the call's status word and
# the kernel drains, leaving its outputs partly written. Reading the word costs a host synchronisation, so the hot path
# never does it: the device's word is remembered here for check_status(), and the environment variable
# FLAMIA_B200_CHECK_STATUS=1 makes every forward and backward check it (a debugging mode).
_LAST_STATUS: dict = {}
_DEVICE_STATUS: dict = {}


def _status_word(device):
    """The device's status word: one persistent int32 per device, zeroed when it is made and again by check_status()
    after it reported a code (kernels only ever write it when something went wrong), so a call launches no fill kernel.
    A first call made inside a stream capture gets a word of the capture's own."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _DEVICE_STATUS.get(idx)
    if st is None:
        if torch.cuda.is_current_stream_capturing():
            return K.new_status(device)
        st = _DEVICE_STATUS[idx] = K.new_status(device)
    return st


def _note_status(status):
    _LAST_STATUS[status.device.index] = status
    if os.environ.get("FLAMIA_B200_CHECK_STATUS", "0") not in ("", "0"):
        check_status(status.device)


def check_status(device=None) -> int:
    """Synchronises `device` (default: the current one) and raises RuntimeError if a flash_attn_fp8 / flash_attn_fp4 call
    there (forward or backward) since the last check gave up a device-side wait or met a bad document table; returns 0
    otherwise. The word is cleared when a code has been reported."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    st = _LAST_STATUS.get(idx)
    if st is None:
        return 0
    with torch.cuda.device(idx):
        code = K.read_status(st)
    if code:
        with torch.cuda.device(idx):
            st.zero_()
        what = f"a bounded wait ran out at site {code & 0xFF}" if code & L.FL_DEV_WAIT_TIMEOUT else \
            (f"the document table is inconsistent (code {code:#x})" if code & L.FL_DEV_BAD_TABLE else f"code {code:#x}")
        raise RuntimeError(f"flamia_blackwell_attention_b200: an attention call on cuda:{idx} did not complete: "
                           f"{what}; its outputs are not valid")
    return 0


# --------------------------------------------------------------------------------------------------------------- docs
class Docs:
    """Packed documents laid out at 128-aligned starts of one padded buffer. Built on the device without a host sync:
    the padded capacity is the host-known bound total + 127 * n_docs rounded up to 128. The quantisers read the packed
    rows in place through the slot tables (slot_src / slot_rows: first source row and number of real rows of every
    128-row slot of the buffer); outputs are scattered back through row_map."""

    def __init__(self, cu, lens, total, aligned, capacity=None):
        dev = cu.device
        self.n = int(lens.numel())
        self.len = lens.to(torch.int32).contiguous()
        self.aligned = aligned
        self.slot_src = self.slot_rows = None
        if aligned:
            self.start = cu[:-1].to(torch.int32).contiguous()
            self.capacity = int(total)
            self.row_map = None
            return
        padded = ((self.len + 127) // 128) * 128
        ends = torch.cumsum(padded, 0)
        self.start = (ends - padded).to(torch.int32).contiguous()
        self.capacity = int(capacity) if capacity is not None else ((int(total) + 127 * self.n + 127) // 128) * 128
        rows = torch.arange(self.capacity, device=dev, dtype=torch.int32)
        doc = torch.searchsorted(ends.to(torch.int32), rows, right=True).clamp_(max=self.n - 1)
        off = rows - self.start[doc]
        src = cu[:-1].to(torch.int32)[doc] + off
        live = (off >= 0) & (off < self.len[doc])
        self.row_map = torch.where(live, src, torch.full_like(src, -1)).contiguous()
        first = slice(0, self.capacity, 128)
        self.slot_src = self.row_map[first].contiguous()                     # a slot's first row is real or the slot is empty
        self.slot_rows = torch.where(live[first], (self.len[doc] - off)[first].clamp(max=128),
                                     torch.zeros_like(off[first])).to(torch.int32).contiguous()

    @classmethod
    def from_tables(cls, start, lens, row_map, slot_src, slot_rows, capacity):
        """A Docs over precomputed tables (DocMaps): nothing is computed."""
        d = object.__new__(cls)
        d.n, d.len, d.start, d.aligned = int(lens.numel()), lens, start, False
        d.capacity, d.row_map, d.slot_src, d.slot_rows = int(capacity), row_map, slot_src, slot_rows
        return d

    def slots(self):
        """The quantisers' packed-source argument, or None on the aligned form (the rows are in place already)."""
        return None if self.aligned else (self.slot_src, self.slot_rows, self.capacity)

    def pack(self, x):
        """(total, h, d) -> (1, capacity, h, d) with zero padding rows."""
        if self.aligned:
            return x.unsqueeze(0)
        x = x.contiguous()
        out = torch.empty(1, self.capacity, *x.shape[1:], dtype=x.dtype, device=x.device)
        rb = x.shape[1] * x.shape[2] * x.element_size()
        L.check(L.load().fl_pack_rows(L.ptr(x), L.ptr(out), L.ptr(self.row_map), self.capacity, rb, K._stream()),
                "fl_pack_rows")
        return out

    def unpack(self, y, total):
        """(1, capacity, h, d) -> (total, h, d)."""
        if self.aligned:
            return y.squeeze(0)
        out = torch.empty(total, *y.shape[2:], dtype=y.dtype, device=y.device)
        rb = y.shape[2] * y.shape[3] * y.element_size()
        L.check(L.load().fl_unpack_rows(L.ptr(y), L.ptr(out), L.ptr(self.row_map), self.capacity, rb, K._stream()),
                "fl_unpack_rows")
        return out


def docs_of(plan, q, cu_q, cu_k, seqused_q, seqused_k):
    """The document table of a call, or None for the batched form."""
    sh = plan.shape
    if sh.varlen:
        if sh.aligned_varlen:
            return Docs(cu_q, seqused_q, sh.tot_q, True)
        lens = (cu_q[1:] - cu_q[:-1])
        return Docs(cu_q, lens, sh.tot_q, False)
    if plan.fwd.ragged_documents:     # batch rows of a length that is no multiple of 128 run as documents
        b, s = sh.b, sh.s_q
        cu = torch.arange(0, (b + 1) * s, s, device=q.device, dtype=torch.int32)
        return Docs(cu, torch.full((b,), s, device=q.device, dtype=torch.int32), b * s, False)
    return None


def state_spec(plan, n_docs=0, dtype=torch.bfloat16, capacity=None):
    """Shapes and dtypes of the tensors forward() returns as `state`, in order, from the plan alone (n_docs = number of
    documents of a packed call). The fake implementations of the registered ops are built from this, and a GPU test
    checks it against the real state."""
    sh, f = plan.shape, plan.fwd
    fp4 = plan.entry == "fp4"
    tl = f.operand_scaling == "token_local"
    need_bwd = plan.bwd.kernel != "none"
    f8, u8, f32, i32 = torch.float8_e4m3fn, torch.uint8, torch.float32, torch.int32
    docs = sh.varlen or f.ragged_documents
    if docs:
        if sh.aligned_varlen:
            n, cap = n_docs, sh.tot_q
        else:
            n, tot = (n_docs, sh.tot_q) if sh.varlen else (sh.b, sh.b * sh.s_q)
            cap = capacity if capacity is not None else ((tot + 127 * n + 127) // 128) * 128
        b, s_q, s_k = 1, cap, cap
    else:
        b, s_q, s_k = sh.b, sh.s_q, sh.s_k
    h, hk, d = sh.h, sh.h_kv, sh.d
    o_rows = s_q
    if docs and not sh.aligned_varlen:      # repacked documents: O has the caller's packed rows
        o_rows = sh.tot_q if sh.varlen else sh.b * sh.s_q
    spec = [((b, o_rows, h, d), dtype), ((b, h, s_q), f32),                                    # O, LSE of the kernels
            ((b, s_q, h, d), f8), ((b, h, s_q // 32), f32), ((b, s_k, hk, d), f8), ((b, hk, s_k // 32), f32),
            ((b, s_k, hk, d), f8), ((b, hk, s_k // 32), f32), ((1,), i32)]                     # codes, factors, status
    if need_bwd:      # K / V statistics of the f16 dQ pre-scale: per 128-row tile and head, or per token
        spec += [((b, s_k), f32)] * 2 if plan.bwd.dq_prescale == "causal_row" else [((b, hk, s_k // 128, 2), f32)] * 2
    if fp4:
        spec += [((b, s_q, h, d // 2), u8), ((b, h, s_q // 128, d // 64, 32, 4, 4), u8),
                 ((b, s_k, hk, d // 2), u8), ((b, hk, s_k // 128, d // 64, 32, 4, 4), u8)]
    if tl:
        spec += [((b, h, s_q), f32), ((b, hk, s_k), f32), ((b, hk, s_k), f32)]
    if f.seqused_k:
        spec += [((b,), i32)]
    if docs:
        spec += [((n,), i32), ((n,), i32)] + ([] if sh.aligned_varlen else [((cap,), i32), ((cap // 128,), i32), ((cap // 128,), i32)])
    return spec


# --------------------------------------------------------------------------------------------------------------- forward
def _forward_prequant(plan, q8, k8, v8, descales, seqused_k):
    """forward() for operands that are already E4M3 codes with one float descale per (batch row, kv head): no quantiser
    runs; the descales fill the factor tables, and V's mantissa goes on the output rows."""
    from .prequant_fa3 import mantissa
    sh, f = plan.shape, plan.fwd
    qd, kd, vd = descales
    grp = sh.h // sh.h_kv
    need_bwd = plan.bwd.kernel != "none"
    status = _status_word(q8.device)

    def table(dsc, heads_rep, s):
        return dsc.repeat_interleave(heads_rep, dim=1)[:, :, None].expand(sh.b, dsc.shape[1] * heads_rep, s // 32).contiguous()
    qq = dict(codes=q8, fac=table(qd, grp, sh.s_q))
    kq = dict(codes=k8, fac=table(kd, 1, sh.s_k))
    vq = dict(codes=v8, fac=table(vd, 1, sh.s_k))
    out, lse, _ = K.attn_fwd(qq, kq, vq, causal=f.causal, softmax_scale=plan.softmax_scale,
                             out_dtype=torch.float16 if sh.dtype == "float16" else torch.bfloat16, status=status,
                             window=f.window, seqused_k=seqused_k, softcap=f.softcap, o_mult=mantissa(vd))
    state = [out, lse, q8, qq["fac"], k8, kq["fac"], v8, vq["fac"], status]
    if need_bwd:
        state += [K.code_stats(k8, kd), K.code_stats(v8, vd)]
    if seqused_k is not None:
        state += [seqused_k]
    state += [qd, kd]
    _note_status(status)
    return out, lse, state


def forward(plan, q, k, v, docs, seqused_k=None, prequant=None):
    """Returns (out, lse, state): out / lse in the caller's layout, state = the tensors the backward needs.
    seqused_k: the batched form's (b,) int32 valid-key counts, or None. prequant: (q_descale, k_descale, v_descale) when
    q, k, v are E4M3 codes already."""
    if prequant is not None:
        return _forward_prequant(plan, q, k, v, prequant, seqused_k)
    sh, f = plan.shape, plan.fwd
    fp4 = plan.entry == "fp4"
    mode = L.FL_MODE_FP4 if fp4 else L.FL_MODE_FP8
    tl = f.operand_scaling == "token_local"
    slots = None
    if docs is not None:
        qp = q.reshape(sh.b * sh.s_q, sh.h, sh.d) if q.dim() == 4 else q
        kp = k.reshape(-1, sh.h_kv, sh.d) if k.dim() == 4 else k
        vp = v.reshape(-1, sh.h_kv, sh.d) if v.dim() == 4 else v
        slots = docs.slots()                  # repacked documents: the quantisers gather the packed rows themselves
        if slots is None:
            qp, kp, vp = qp.unsqueeze(0), kp.unsqueeze(0), vp.unsqueeze(0)
    else:
        qp, kp, vp = q, k, v
    need_bwd = plan.bwd.kernel != "none"
    # rotation: the 8-bit route rotates the E4M3 codes; the mixed route rotates only the NVFP4 S operands
    qk_kw = dict(apply_hadamard_rotation=f.qk_hadamard, hadamard_rotation_scope="nvfp4_copy" if fp4 else "all",
                 also_make_nvfp4_copy=fp4, token_local_exponents=tl, packed_slots=slots)
    status = _status_word(q.device)
    rows = need_bwd and plan.bwd.dq_prescale == "causal_row"      # per-token K / V statistics instead of per-tile ones
    k_rows = v_rows = None
    if rows:
        k_rows, v_rows = torch.zeros(2, sh.b, sh.s_k, dtype=torch.float32, device=q.device).unbind(0)
    qq = K.quantize_fp8_blocks(qp, status=status, **qk_kw)
    # max |K_j| of the codes' values; where those are rotated, the rotation-invariant 2-norm bounds it
    kq = K.quantize_fp8_blocks(kp, output_tile_stats=need_bwd and not rows, status=status,
                               row_stat=("norm2" if (f.qk_hadamard and not fp4) else "amax", k_rows) if rows else None, **qk_kw)
    vq = K.quantize_fp8_blocks(vp, output_tile_stats=need_bwd and not rows, token_local_exponents=tl, status=status,
                               packed_slots=slots, row_stat=("sumsq", v_rows) if rows else None)
    # repacked documents: the kernel writes the caller's packed rows itself (out is (1, total, h, d))
    total = (sh.tot_q if sh.varlen else sh.b * sh.s_q) if slots is not None else None
    out, lse, _ = K.attn_fwd(qq, kq, vq, causal=f.causal, softmax_scale=plan.softmax_scale, out_dtype=q.dtype, mode=mode,
                             status=status, token_local=tl, window=f.window, p_group=f.p_hat_frame == "group",
                             seqused_k=seqused_k, softcap=f.softcap,
                             packed_out=None if slots is None else (slots[0], slots[1], total),
                             doc_start=None if docs is None else docs.start, doc_len=None if docs is None else docs.len)
    state = [out, lse, qq["codes"], qq["fac"], kq["codes"], kq["fac"], vq["codes"], vq["fac"], status]
    if need_bwd:
        state += [k_rows, v_rows] if rows else [kq["tile_stats"], vq["tile_stats"]]
    if fp4:
        state += [qq["x4"], qq["sf4_raw"], kq["x4"], kq["sf4_raw"]]
    if tl:
        state += [qq["token_factors"], kq["token_factors"], vq["token_factors"]]
    if seqused_k is not None:
        state += [seqused_k]
    if docs is not None:
        state += [docs.start, docs.len] + ([] if docs.row_map is None else [docs.row_map, docs.slot_src, docs.slot_rows])
        out_user = out[0]                        # aligned: in place; repacked: the kernel wrote the packed rows
        if not sh.varlen:
            out_user = out_user.reshape(sh.b, sh.s_q, sh.h, sh.d)
        if sh.aligned_varlen:
            lse_user = lse[0]                    # (h, total_q): the caller's rows are the kernels' rows
        elif f.return_lse:
            # repacked documents: the kernels' LSE has the aligned buffer's rows; its live rows go to the caller's packed
            # rows (padding rows to a spare column), no host synchronisation
            tot = sh.tot_q if sh.varlen else sh.b * sh.s_q
            idx = torch.where(docs.row_map >= 0, docs.row_map, torch.full_like(docs.row_map, tot)).long()
            buf = lse.new_zeros(sh.h, tot + 1)
            buf.index_copy_(1, idx, lse[0])
            lse_user = buf[:, :tot].contiguous() if sh.varlen else \
                buf[:, :tot].reshape(sh.h, sh.b, sh.s_q).permute(1, 0, 2).contiguous()
        else:
            lse_user = lse.new_zeros(0)
    else:
        out_user, lse_user = out, lse
    _note_status(status)
    return out_user, lse_user, state


# --------------------------------------------------------------------------------------------------------------- backward
def backward(plan, state, dout, docs_meta):
    """dq, dk, dv in the caller's layout. state as returned by forward(); docs_meta = (capacity, aligned) or None."""
    sh, f, bw = plan.shape, plan.fwd, plan.bwd
    fp4 = plan.entry == "fp4"
    tl = f.operand_scaling == "token_local"
    it = iter(state)
    out, lse, qc, qf, kc, kf, vc, vf, status, kstats, vstats = (next(it) for _ in range(11))
    qq, kq, vq = dict(codes=qc, fac=qf), dict(codes=kc, fac=kf), dict(codes=vc, fac=vf)
    if fp4:
        qq["x4"], qq["sf4_raw"], kq["x4"], kq["sf4_raw"] = (next(it) for _ in range(4))
    if tl:
        qq["token_factors"], kq["token_factors"], vq["token_factors"] = (next(it) for _ in range(3))
    seqused_k = next(it) if f.seqused_k else None
    dk_mult = dq_mult = None
    if plan.prequant:       # float descales: the mantissas the block-scaled dK / dQ products left out
        from .prequant_fa3 import mantissa
        qd, kd = next(it), next(it)
        dk_mult, dq_mult = mantissa(qd), mantissa(kd).repeat_interleave(sh.h // sh.h_kv, dim=1).contiguous()
    docs = None
    if docs_meta is not None:
        docs = object.__new__(Docs)
        docs.start, docs.len = next(it), next(it)
        docs.capacity, docs.aligned = docs_meta
        docs.n = int(docs.len.numel())
        docs.row_map, docs.slot_src, docs.slot_rows = (None, None, None) if docs.aligned else (next(it), next(it), next(it))
        gp = (dout.reshape(-1, sh.h, sh.d) if dout.dim() == 4 else dout).contiguous()
        if docs.aligned:
            gp = gp.unsqueeze(0)
    else:
        gp = dout.contiguous()
    b, s_q, h, d = qc.shape                      # (the aligned buffer's rows; out has the packed rows under repacked documents)
    acc = torch.empty(b, h, s_q, d, dtype=torch.float16, device=out.device)
    packed_out = None
    if docs is not None and not docs.aligned:
        packed_out = (docs.slot_src, docs.slot_rows, int(out.shape[1]))
    rows = bw.dq_prescale == "causal_row"
    do_rows = torch.zeros(b, s_q, dtype=torch.float32, device=out.device) if rows else None
    gq = K.quantize_fp8_blocks(gp, compute_d_with_output=out, shifted_log2_lse_from=lse, log2_lse_shift=P_SHIFT_LOG2,
                               d_multiplier=float(backward_scalars(plan.softmax_scale)[6]), zero_accumulator=acc,
                               output_tile_stats=not rows, token_local_exponents=tl, status=status,
                               packed_slots=None if docs is None else docs.slots(),
                               row_stat=("sumsq", do_rows) if rows else None)
    if rows:      # kstats / vstats are the per-token tables here; the prefix maxima go into copies (the state is read-only)
        ks, ps = K.dq_prescale_rows(do_rows, vstats.clone(), kstats.clone())
    else:
        ks, ps = K.dq_prescale(gq["tile_stats"], vstats, kstats, causal_local=bw.dq_prescale == "causal_tile")
    had8 = f.qk_hadamard and not fp4           # only the 8-bit route's E4M3 codes are rotated
    dk, dv, _ = K.attn_bwd(qq, kq, vq, gq, lse_log2=gq["lse_log2"], d_rows=gq["D"], dq_acc=acc,
                           dq_scale=None if rows else ks, dq_scale_rows=ks if rows else None,
                           causal=f.causal, softmax_scale=plan.softmax_scale, out_dtype=out.dtype,
                           mode=L.FL_MODE_FP4 if fp4 else L.FL_MODE_FP8, had_dk=had8, status=status,
                           token_local=tl, dq_rowlocal=bw.ds_dq_rowlocal == "all", window=f.window, seqused_k=seqused_k,
                           softcap=f.softcap, dk_mult=dk_mult, packed_out=packed_out,
                           dq_order=torch.zeros(b, h, s_q // 128, 2, dtype=torch.int32, device=out.device)
                           if bw.deterministic else None,
                           doc_start=None if docs is None else docs.start, doc_len=None if docs is None else docs.len)
    dq = K.dq_post(acc, ps, plan.softmax_scale, b=b, s=s_q, h=h, d=d, unrotate=had8, out_dtype=out.dtype, per_row=rows,
                   head_mult=dq_mult, packed_out=packed_out)
    _note_status(status)
    if docs is not None:
        dq, dk, dv = dq[0], dk[0], dv[0]         # aligned: in place; repacked: the kernels wrote the packed rows
        if not sh.varlen:
            dq = dq.reshape(sh.b, sh.s_q, sh.h, sh.d)
            dk, dv = dk.reshape(sh.b, sh.s_k, sh.h_kv, sh.d), dv.reshape(sh.b, sh.s_k, sh.h_kv, sh.d)
    return dq, dk, dv
