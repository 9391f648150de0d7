"""Thin PyTorch wrappers over the C ABI: they allocate outputs with torch, pass raw device pointers and the current
stream, and return tensors. No arithmetic happens here.

quantize_fp8_blocks mirrors the reference's quant.fp8.quantize_fp8_blocks (flash_attn/cute/quant/fp8.py:2512): same
argument names for the features this build serves, same output keys.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this library has no CPU path")


def new_status(device):
    return torch.zeros(1, dtype=torch.int32, device=device)


def read_status(status) -> int:
    """Host value of a device status word (synchronises the current stream)."""
    v = C.c_int32(0)
    L.check(L.load().fl_read_status(L.ptr(status), C.byref(v), _stream()), "fl_read_status")
    return int(v.value)


def quantize_fp8_blocks(x, *, apply_hadamard_rotation=False, hadamard_rotation_scope="all", token_local_exponents=False,
                        make_channel_major_copy=False, output_exponent_table=True, output_token_block_factors=True,
                        output_sf_atoms=False, also_make_nvfp4_copy=False, compute_d_with_output=None,
                        shifted_log2_lse_from=None, log2_lse_shift=0.0, d_multiplier=1.0, zero_accumulator=None,
                        output_tile_stats=False, status=None, wait_cycles=0, packed_slots=None, row_stat=None,
                        legacy_kernel=False):
    """Token-block MXFP8 quantiser of x (b, s, h, d) bf16 / f16 (s % 128 == 0, d in {64, 128}).
    packed_slots = (slot_src, slot_rows, padded_rows): x is a packed (total, h, d) tensor of documents stored back to back
    and the outputs are those of the 128-aligned buffer (1, padded_rows, h, d): slot_src[i] = first row of x of output
    rows [128 i, 128 i + 128) (-1 = empty), slot_rows[i] = how many of them are real. Nothing is copied.
    Returns a dict: codes (b,s,h,d) float8_e4m3fn; e (b,h,s/32,d/32) uint8; fac (b,h,s/32) f32; optionally codes_t,
    sf_tok_raw, sf_dim_raw, token_factors, x4 / sf4_raw (NVFP4 copy), D, lse_log2, tile_stats.
    hadamard_rotation_scope: "all" (codes and NVFP4 copy of the rotated rows) | "nvfp4_copy" (only the NVFP4 copy).
    row_stat = (kind, table): table (b, s) f32, zero on entry, takes per token the maximum over the heads of the row's
    "sumsq" | "amax" | "norm2" (the statistics of the per-query-row causal dQ pre-scale)."""
    _require_cuda(x, "x")
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("x must be bf16 or f16")
    x = x.contiguous()
    a = L.QuantArgs()
    if packed_slots is not None:
        slot_src, slot_rows, padded_rows = packed_slots
        assert x.dim() == 3 and padded_rows % 128 == 0 and slot_src.numel() == padded_rows // 128
        (total, h, d), b, s = x.shape, 1, int(padded_rows)
        a.slot_src, a.slot_rows, a.src_rows = L.ptr(slot_src), L.ptr(slot_rows), int(total)
    else:
        b, s, h, d = x.shape
    dev = x.device
    u8 = dict(dtype=torch.uint8, device=dev)
    out = {}
    a.x = L.ptr(x)
    a.b, a.s, a.h, a.d = b, s, h, d
    a.in_f16 = int(x.dtype == torch.float16)
    flags = 0
    if apply_hadamard_rotation:
        flags |= L.FL_Q_HADAMARD if hadamard_rotation_scope == "all" else L.FL_Q_HADAMARD_NVFP4_ONLY
    if token_local_exponents:
        flags |= L.FL_Q_TOKEN_LOCAL
    if legacy_kernel:       # the four-lanes-per-row kernel even where the one-thread-per-row kernel serves (same bits)
        flags |= L.FL_Q_LEGACY
    a.flags = flags
    out["codes"] = torch.empty(b, s, h, d, **u8)
    a.codes = L.ptr(out["codes"])
    if make_channel_major_copy:
        out["codes_t"] = torch.empty(b, h, d, s, **u8)
        a.codes_t = L.ptr(out["codes_t"])
    if output_exponent_table:
        out["e"] = torch.empty(b, h, s // 32, d // 32, **u8)
        a.e_tab = L.ptr(out["e"])
    if output_token_block_factors:
        out["fac"] = torch.empty(b, h, s // 32, dtype=torch.float32, device=dev)
        a.fac = L.ptr(out["fac"])
    if output_sf_atoms:
        out["sf_tok_raw"] = torch.empty(b, h, s // 128, 1, 32, 4, 4, **u8)
        out["sf_dim_raw"] = torch.empty(b, h, 1, s // 128, 32, 4, 4, **u8)
        a.sf_tok, a.sf_dim = L.ptr(out["sf_tok_raw"]), L.ptr(out["sf_dim_raw"])
    if token_local_exponents:
        out["token_factors"] = torch.empty(b, h, s, dtype=torch.float32, device=dev)
        a.token_factors = L.ptr(out["token_factors"])
    if also_make_nvfp4_copy:
        out["x4"] = torch.empty(b, s, h, d // 2, **u8)
        out["sf4_raw"] = torch.empty(b, h, s // 128, d // 64, 32, 4, 4, **u8)
        a.x4, a.sf4 = L.ptr(out["x4"]), L.ptr(out["sf4_raw"])
    keep = []
    if compute_d_with_output is not None:
        o = compute_d_with_output.contiguous()
        if packed_slots is not None and o.numel() == x.numel():      # the forward output has x's packed rows
            a.flags = flags | L.FL_Q_O_PACKED
        else:
            assert tuple(o.shape) == (b, s, h, d)
        assert o.dtype == x.dtype
        keep.append(o)
        a.o = L.ptr(o)
        out["D"] = torch.empty(b, h, s, dtype=torch.float32, device=dev)
        a.d_out = L.ptr(out["D"])
    if shifted_log2_lse_from is not None:
        lse = shifted_log2_lse_from.contiguous().float()
        assert lse.shape == (b, h, s)
        keep.append(lse)
        a.lse = L.ptr(lse)
        out["lse_log2"] = torch.empty(b, h, s, dtype=torch.float32, device=dev)
        a.lse_log2 = L.ptr(out["lse_log2"])
    if zero_accumulator is not None:
        assert zero_accumulator.dtype == torch.float16 and zero_accumulator.numel() == b * h * s * d
        a.zero_acc = L.ptr(zero_accumulator)
    if output_tile_stats:
        out["tile_stats"] = torch.empty(b, h, s // 128, 2, dtype=torch.float32, device=dev)
        a.tile_stats = L.ptr(out["tile_stats"])
    if row_stat is not None:
        kind, table = row_stat
        assert table.dtype == torch.float32 and tuple(table.shape) == (b, s) and table.is_contiguous()
        a.row_stat, a.row_stat_kind = L.ptr(table), {"sumsq": 1, "amax": 2, "norm2": 3}[kind]
    a.lse_shift, a.d_multiplier = float(log2_lse_shift), float(d_multiplier)
    a.status, a.wait_cycles = L.ptr(status), int(wait_cycles)      # status: the call's device status word or None
    L.check(L.load().fl_quant_blocks(C.byref(a), _stream()), "fl_quant_blocks")
    out["codes"] = out["codes"].view(torch.float8_e4m3fn)
    if "codes_t" in out:
        out["codes_t"] = out["codes_t"].view(torch.float8_e4m3fn)
    return out


def attn_args(q, k, v, *, causal, softmax_scale, mode=L.FL_MODE_FP8, flags=0, status=None, doc_start=None, doc_len=None,
              wait_cycles=0, token_local=False, window=None, seqused_k=None, softcap=0.0):
    """AttnArgs from quantiser outputs q / k / v (dicts with codes, fac [, x4, sf4_raw, token_factors])."""
    qc, kc, vc = q["codes"], k["codes"], v["codes"]
    b, s_q, h, d = qc.shape
    s_k, h_kv = kc.shape[1], kc.shape[2]
    a = L.AttnArgs()
    a.q_codes, a.k_codes, a.v_codes = L.ptr(qc), L.ptr(kc), L.ptr(vc)
    fkey = "token_factors" if token_local else "fac"
    a.fac_q, a.fac_k, a.fac_v = L.ptr(q[fkey]), L.ptr(k[fkey]), L.ptr(v[fkey])
    if token_local:
        flags |= L.FL_A_TOKEN_LOCAL
    if mode == L.FL_MODE_FP4:
        a.q4, a.k4, a.sfq4, a.sfk4 = L.ptr(q["x4"]), L.ptr(k["x4"]), L.ptr(q["sf4_raw"]), L.ptr(k["sf4_raw"])
    a.b, a.s_q, a.s_k, a.h, a.h_kv, a.d = b, s_q, s_k, h, h_kv, d
    a.softmax_scale = float(softmax_scale)
    a.mode = mode
    a.flags = flags | (L.FL_A_CAUSAL if causal else 0)
    if doc_start is not None:
        a.doc_start, a.doc_len, a.n_docs = L.ptr(doc_start), L.ptr(doc_len), int(doc_len.numel())
    a.status = L.ptr(status)
    a.wait_cycles = int(wait_cycles)
    if window is not None:      # (left, right), None = unlimited; stored as window + 1 (0 = unlimited)
        a.window_left_p1 = 0 if window[0] is None else int(window[0]) + 1
        a.window_right_p1 = 0 if window[1] is None else int(window[1]) + 1
    a.seqused_k = L.ptr(seqused_k)      # batched form: (b,) int32 valid keys per batch row, or None
    a.softcap = float(softcap or 0.0)
    return a


def attn_fwd(q, k, v, *, causal, softmax_scale, out_dtype=torch.bfloat16, mode=L.FL_MODE_FP8, status=None,
             doc_start=None, doc_len=None, wait_cycles=0, token_local=False, window=None, p_group=False, seqused_k=None,
             softcap=0.0, o_mult=None, packed_out=None):
    """Forward kernel on quantised operands. Returns (out (b, s_q, h, d), lse (b, h, s_q) float32, status).
    p_group: group-frame P-hat (one UE8M0 exponent per query row and 32 keys) instead of the row frame.
    o_mult: (b, h_kv) f32 factor on the output rows (the mantissa of a V factor that is no power of two).
    packed_out = (slot_src, slot_rows, total): documents; out is (1, total, h, d) with the documents stored back to back
    (the kernel writes the caller's packed rows itself); lse keeps the aligned buffer's rows."""
    qc = q["codes"]
    b, s_q, h, d = qc.shape
    dev = qc.device
    if status is None:
        status = new_status(dev)
    # documents: the kernel writes only the rows of its documents; padding rows and unused tail tiles must read as
    # zeros afterwards (the backward prologue forms rowsum(O * dO) for every row of the buffer)
    alloc = torch.empty if doc_start is None else torch.zeros
    out = torch.empty(1, int(packed_out[2]), h, d, dtype=out_dtype, device=dev) if packed_out is not None else \
        alloc(b, s_q, h, d, dtype=out_dtype, device=dev)
    lse = alloc(b, h, s_q, dtype=torch.float32, device=dev)
    a = attn_args(q, k, v, causal=causal, softmax_scale=softmax_scale, mode=mode,
                  flags=(L.FL_A_OUT_F16 if out_dtype == torch.float16 else 0) | (L.FL_A_P_GROUP if p_group else 0),
                  status=status, doc_start=doc_start,
                  doc_len=doc_len, wait_cycles=wait_cycles, token_local=token_local, window=window, seqused_k=seqused_k,
                  softcap=softcap)
    a.out, a.lse = L.ptr(out), L.ptr(lse)
    if packed_out is not None:
        a.slot_src, a.slot_rows, a.out_rows = L.ptr(packed_out[0]), L.ptr(packed_out[1]), int(packed_out[2])
    if o_mult is not None:
        assert o_mult.dtype == torch.float32 and o_mult.numel() == b * k["codes"].shape[2] and o_mult.is_contiguous()
        a.o_mult = L.ptr(o_mult)
    if token_local:     # log2 f_V and 1 / f_V per key, which the forward applies to every score
        lg, rcp = token_aux(v["token_factors"])
        a.tok_lg_v, a.tok_rcp_v = L.ptr(lg), L.ptr(rcp)
    L.check(L.load().fl_fwd(C.byref(a), _stream()), "fl_fwd")
    return out, lse, status


def token_aux(factors):
    """(log2 f, 1 / f) float32 tables of a power-of-two factor table (the quantiser's token_factors)."""
    f = factors.contiguous()
    assert f.dtype == torch.float32
    lg, rcp = torch.empty_like(f), torch.empty_like(f)
    L.check(L.load().fl_token_aux(L.ptr(f), int(f.numel()), L.ptr(lg), L.ptr(rcp), _stream()), "fl_token_aux")
    return lg, rcp


def selftest_mma(which, a, b, sfa=None, sfb=None, wait_cycles=0):
    """One 128x128x128 product through the library's tensor-core helpers; returns (d (128,128) f32, status value)."""
    dev = a.device if a is not None else torch.device("cuda")
    d = torch.zeros(128, 128, dtype=torch.float32, device=dev)
    status = new_status(dev)
    L.check(L.load().fl_selftest_mma(int(which), L.ptr(a), L.ptr(b), L.ptr(sfa), L.ptr(sfb), L.ptr(d), L.ptr(status),
                                     int(wait_cycles), _stream()), "fl_selftest_mma")
    return d, read_status(status)


def dq_prescale(stats_do, stats_v, stats_k, *, causal_local=False, unit=1.0):
    """Power-of-two pre-scale of the f16 dQ accumulator per (batch row, query tile) from the quantisers' tile statistics
    (b, heads, tiles, 2). Returns (kernel_scale, post_scale), each (b, s_q / 128) float32."""
    b, h, nt_q, _ = stats_do.shape
    h_kv, nt_k = stats_v.shape[1], stats_v.shape[2]
    dev = stats_do.device
    ks = torch.empty(b, nt_q, dtype=torch.float32, device=dev)
    ps = torch.empty(b, nt_q, dtype=torch.float32, device=dev)
    L.check(L.load().fl_dq_prescale(L.ptr(stats_do), L.ptr(stats_v), L.ptr(stats_k), b, h, h_kv, nt_q, nt_k,
                                    int(bool(causal_local)), float(unit), L.ptr(ks), L.ptr(ps), _stream()),
            "fl_dq_prescale")
    return ks, ps


def dq_prescale_rows(row_do, row_v, row_k, *, unit=1.0):
    """Power-of-two pre-scale of the f16 dQ accumulator per QUERY ROW of a causal square batched call, from the
    quantisers' per-token statistics (b, s): row i's own dO statistic and the running maxima of the V / K statistics over
    the keys j <= i (row_v / row_k are replaced by those prefix maxima). Returns (kernel_rows, post_rows), each (b, s)."""
    b, s = row_do.shape
    assert row_v.shape == row_do.shape == row_k.shape
    ks = torch.empty(b, s, dtype=torch.float32, device=row_do.device)
    ps = torch.empty(b, s, dtype=torch.float32, device=row_do.device)
    L.check(L.load().fl_dq_prescale_rows(L.ptr(row_do), L.ptr(row_v), L.ptr(row_k), b, s, float(unit), L.ptr(ks),
                                         L.ptr(ps), _stream()), "fl_dq_prescale_rows")
    return ks, ps


def dq_post(acc, post_scale, mult, *, b, s, h, d, unrotate=False, out_dtype=torch.bfloat16, per_row=False,
            head_mult=None, packed_out=None):
    """dq (b, s, h, d) = cast(acc * post_scale[b, s / 128] * mult) (per_row: post_scale[b, s]; head_mult: times a (b, h)
    factor), optionally rotated back. acc is the f16 accumulator in the backward kernel's layout: (b, h, d, s) at
    d = 128, (b, h, s, d) at d = 64."""
    if packed_out is not None:      # documents: dq (1, total, h, d) takes the packed rows (see attn_fwd)
        assert b == 1 and not per_row and head_mult is None
        dq = torch.empty(1, int(packed_out[2]), h, d, dtype=out_dtype, device=acc.device)
        L.check(L.load().fl_dq_post_packed(L.ptr(acc), L.ptr(post_scale), float(mult), L.ptr(dq), s, h, d, int(bool(unrotate)),
                                           int(out_dtype == torch.float16), L.ptr(packed_out[0]), L.ptr(packed_out[1]),
                                           _stream()), "fl_dq_post_packed")
        return dq
    dq = torch.empty(b, s, h, d, dtype=out_dtype, device=acc.device)
    assert post_scale.numel() == (b * s if per_row else b * (s // 128))
    if head_mult is not None:
        assert head_mult.dtype == torch.float32 and head_mult.numel() == b * h and head_mult.is_contiguous()
    L.check(L.load().fl_dq_post_ex(L.ptr(acc), L.ptr(post_scale), int(bool(per_row)), L.ptr(head_mult), float(mult),
                                   L.ptr(dq), b, s, h, d, int(bool(unrotate)), int(out_dtype == torch.float16), _stream()),
            "fl_dq_post_ex")
    return dq


def code_stats(codes, descale):
    """Tile statistics (b, h, s / 128, 2) of E4M3 codes (b, s, h, d) times descale (b, h): largest magnitude and largest
    row sum of squares per 128-row tile, what the quantiser writes for operands it quantises itself."""
    b, s, h, d = codes.shape
    assert codes.element_size() == 1 and codes.is_contiguous() and descale.dtype == torch.float32 and descale.numel() == b * h
    out = torch.empty(b, h, s // 128, 2, dtype=torch.float32, device=codes.device)
    L.check(L.load().fl_code_stats(L.ptr(codes), L.ptr(descale), b, s, h, d, L.ptr(out), _stream()), "fl_code_stats")
    return out


def attn_bwd(q, k, v, do, *, lse_log2, d_rows, dq_acc, dq_scale, causal, softmax_scale, out_dtype=torch.bfloat16,
             mode=L.FL_MODE_FP8, had_dk=False, status=None, doc_start=None, doc_len=None, wait_cycles=0,
             token_local=False, dq_rowlocal=False, window=None, seqused_k=None, softcap=0.0, dq_order=None,
             dq_scale_rows=None, dk_mult=None, packed_out=None):
    """Backward main kernel on quantised operands. q / k / v / do: quantiser outputs (codes, fac). Adds the pre-scaled
    dQ partials into the f16 accumulator dq_acc of b * h * s_q * d elements ((b, h, d, s_q) at d = 128, (b, h, s_q, d)
    at d = 64) and returns (dk, dv, status), each (b, s_k, h_kv, d). dq_order: a zeroed (b, h, s_q / 128, 2) int32 table
    makes the key tiles add their partial sums in ascending key order (bitwise reproducible dQ)."""
    kc = k["codes"]
    b, s_k, h_kv, d = kc.shape
    dev = kc.device
    if status is None:
        status = new_status(dev)
    rows_out = s_k if packed_out is None else int(packed_out[2])      # packed_out: dk, dv (1, total, h_kv, d), see attn_fwd
    dk = torch.empty(b, rows_out, h_kv, d, dtype=out_dtype, device=dev)
    dv = torch.empty(b, rows_out, h_kv, d, dtype=out_dtype, device=dev)
    flags = (L.FL_A_OUT_F16 if out_dtype == torch.float16 else 0) | (L.FL_A_HAD_DK if had_dk else 0) | \
        (L.FL_A_DQ_ROWLOCAL if dq_rowlocal else 0)
    a = attn_args(q, k, v, causal=causal, softmax_scale=softmax_scale, mode=mode, flags=flags, status=status,
                  doc_start=doc_start, doc_len=doc_len, wait_cycles=wait_cycles, token_local=token_local, window=window,
                  seqused_k=seqused_k, softcap=softcap)
    if packed_out is not None:
        a.slot_src, a.slot_rows, a.out_rows = L.ptr(packed_out[0]), L.ptr(packed_out[1]), int(packed_out[2])
    a.do_codes, a.fac_do = L.ptr(do["codes"]), L.ptr(do["token_factors" if token_local else "fac"])
    a.lse_log2, a.d_rows, a.dq_acc, a.dq_scale = L.ptr(lse_log2), L.ptr(d_rows), L.ptr(dq_acc), L.ptr(dq_scale)
    a.dk, a.dv = L.ptr(dk), L.ptr(dv)
    if dq_scale_rows is not None:      # one pre-scale per query row instead of dq_scale per query tile
        assert dq_scale_rows.dtype == torch.float32 and dq_scale_rows.numel() == b * q["codes"].shape[1]
        a.dq_scale_rows = L.ptr(dq_scale_rows)
    if dk_mult is not None:             # the mantissa of a Q factor that is no power of two, per (batch row, kv head)
        assert dk_mult.dtype == torch.float32 and dk_mult.numel() == b * h_kv and dk_mult.is_contiguous()
        a.dk_mult = L.ptr(dk_mult)
    if dq_order is not None:
        assert dq_order.dtype == torch.int32 and dq_order.numel() == b * q["codes"].shape[2] * (q["codes"].shape[1] // 128) * 2
        a.dq_order = L.ptr(dq_order)
    L.check(L.load().fl_bwd(C.byref(a), _stream()), "fl_bwd")
    return dk, dv, status


def attn_bwd_static_acc(q, k, v, do, *, lse_log2, d_rows, dq_scale, post_scale, mult, causal, softmax_scale,
                        out_dtype=torch.bfloat16, had_dk=False, had_dq=False, status=None, wait_cycles=0,
                        mode=L.FL_MODE_FP8):
    """fl_bwd_static_acc: backward main kernel + dQ postprocess with the f16 accumulator held in the library's fixed
    device array (nothing is allocated inside the call; b * h * s_q * d is limited to FL_STATIC_ACC_MAX_ELEMS and a
    larger problem raises). Returns (dq, dk, dv, status). Calls on one device must not overlap in time."""
    kc = k["codes"]
    b, s_k, h_kv, d = kc.shape
    _, s_q, h, _ = q["codes"].shape
    dev = kc.device
    if status is None:
        status = new_status(dev)
    dq = torch.empty(b, s_q, h, d, dtype=out_dtype, device=dev)
    dk = torch.empty(b, s_k, h_kv, d, dtype=out_dtype, device=dev)
    dv = torch.empty(b, s_k, h_kv, d, dtype=out_dtype, device=dev)
    flags = (L.FL_A_OUT_F16 if out_dtype == torch.float16 else 0) | (L.FL_A_HAD_DK if had_dk else 0) | \
        (L.FL_A_HAD_DQ if had_dq else 0)
    a = attn_args(q, k, v, causal=causal, softmax_scale=softmax_scale, mode=mode, flags=flags, status=status,
                  wait_cycles=wait_cycles)
    a.do_codes, a.fac_do = L.ptr(do["codes"]), L.ptr(do["fac"])
    a.lse_log2, a.d_rows, a.dq_scale = L.ptr(lse_log2), L.ptr(d_rows), L.ptr(dq_scale)
    a.dk, a.dv = L.ptr(dk), L.ptr(dv)
    L.check(L.load().fl_bwd_static_acc(C.byref(a), L.ptr(post_scale), float(mult), L.ptr(dq), _stream()),
            "fl_bwd_static_acc")
    return dq, dk, dv, status
