"""CPU oracle of the backward pass's scalars and of the f16 dQ pre-scale tables (TEST INFRASTRUCTURE, not product code).

numpy float32 restatements, operation by operation in the reference's order (every product / quotient / square root
rounded to float32 once, no fused multiply-add), of

  * flash_attn/cute/device_scales.py:124-132  `_dq_bound_pow2`: bound = ((((4 unit) 2) sqrt(dn2)) sqrt(vn2)) kmax,
    B = the largest power of two <= 65504 / bound with its exponent clamped to [-40, 40] (:40-45 `_pow2_floor_clamped`);
  * :158-184 `_dq_row_bound` and :234-319 `_dq_tile_table`: one B per batch row (from every query / key tile of the row),
    one per (row, query tile) from that tile's dO rows and the PREFIX of key tiles 0..t (CAUSAL = 1), one per query row
    from per-row statistics (CAUSAL = 2); kernel scale = base B, postprocess scale = num / (unit B);
  * :734-743 `_bwd1_fp8_ref`: the eight kernel scalars of the 8-bit backward (softmax scale, dP-sum scale, dS boost, dV
    scale, dK scale, dQ scale, D fold multiplier, dQ postprocess scale) for given operand descales.

Parity pin: tests/test_oracle_attention.py checks every function here against tests/golden/scales_small.json, which
tests/golden/make_golden_attention.py wrote by running the reference's own definitions (the Triton kernel under Triton's
CPU interpreter, the `_host` functions as they are).
"""
from __future__ import annotations

import numpy as np

F = np.float32


def pow2_floor_clamped(y, lo=-40, hi=40):
    """Largest power of two <= y (y >= 0 float32), exponent clamped to [lo, hi]: the float32 exponent field
    (0 / subnormal -> 2^lo, inf / NaN -> 2^hi)."""
    y = np.asarray(y, dtype=np.float32)
    e = ((y.view(np.int32) >> 23) & 0xFF) - 127
    e = np.minimum(np.maximum(e, lo), hi)
    return ((e + 127).astype(np.int32) << 23).view(np.float32)


def dq_bound_pow2(dn2, vn2, kmax, unit):
    """B of one row from max ||dO_q||^2, max ||V_k||^2, max|K| and the route's fixed factor `unit`."""
    with np.errstate(over="ignore", divide="ignore", invalid="ignore"):
        dn2, vn2, kmax = (np.asarray(t, dtype=np.float32) for t in (dn2, vn2, kmax))
        bnd = F(4.0) * F(unit)
        bnd = F(bnd * F(2.0))
        bnd = (bnd * np.sqrt(dn2, dtype=np.float32)).astype(np.float32)
        bnd = (bnd * np.sqrt(vn2, dtype=np.float32)).astype(np.float32)
        bnd = (bnd * kmax).astype(np.float32)
        return pow2_floor_clamped((F(65504.0) / bnd).astype(np.float32))


def _tables(b_pow2, base, num, unit):
    with np.errstate(over="ignore", divide="ignore"):
        kern = (F(base) * b_pow2).astype(np.float32)
        post = (F(num) / (F(unit) * b_pow2).astype(np.float32)).astype(np.float32)
    return kern, post


def dq_prescale_rows(dn, vn, km, b, hq, hk, tq, tk, unit=1.0, base=1.0, num=1.0):
    """One B per batch row, written for each of its tq query tiles: (kernel (b tq,), post (b tq,))."""
    dn = np.asarray(dn, np.float32).reshape(b, hq * tq)
    vn = np.asarray(vn, np.float32).reshape(b, hk * tk)
    km = np.asarray(km, np.float32).reshape(b, hk * tk)
    bb = dq_bound_pow2(dn.max(1), vn.max(1), km.max(1), unit)
    kern, post = _tables(bb, base, num, unit)
    return np.repeat(kern, tq), np.repeat(post, tq)


def dq_prescale_causal_tiles(dn, vn, km, b, hq, hk, tq, tk, unit=1.0, base=1.0, num=1.0):
    """One B per (batch row, query tile t): that tile's own dO statistics over the q heads, key tiles 0 .. min(t + 1, tk)
    over the kv heads."""
    dn = np.asarray(dn, np.float32).reshape(b, hq, tq)
    vn = np.asarray(vn, np.float32).reshape(b, hk, tk)
    km = np.asarray(km, np.float32).reshape(b, hk, tk)
    kern = np.empty((b, tq), np.float32)
    post = np.empty((b, tq), np.float32)
    for t in range(tq):
        hi = min(t + 1, tk)
        bb = dq_bound_pow2(dn[:, :, t].max(1), vn[:, :, :hi].reshape(b, -1).max(1), km[:, :, :hi].reshape(b, -1).max(1), unit)
        kern[:, t], post[:, t] = _tables(bb, base, num, unit)
    return kern.reshape(-1), post.reshape(-1)


def dq_prescale_causal_rows(dn_row, vn_prefix, km_prefix, unit=1.0, base=1.0, num=1.0):
    """One B per query row from per-row statistics: max ||dO_i||^2 and the running maxima of ||V_j||^2, max|K_j| over the keys
    j <= i (already prefix maxima)."""
    return _tables(dq_bound_pow2(dn_row, vn_prefix, km_prefix, unit), base, num, unit)


def bwd1_fp8_scalars(softmax, p_shift, dq_boost, sq=1.0, sk=1.0, sv=1.0, sdo=1.0, s_ds=None):
    """The 8-bit backward's kernel scalars, slots 0-7, for operand descales sq, sk, sv, sdo (all 1 with block-scaled
    operands, whose scales travel with the codes) and a block-scaled dS-hat (s_ds None)."""
    softmax, p_shift, dq_boost = F(softmax), F(p_shift), F(dq_boost)
    sq, sk, sv, sdo = F(sq), F(sk), F(sv), F(sdo)
    ds_boost = F(1.0) if s_ds is None else F(F(sv * sdo) / F(s_ds))
    r = F(F(sv * sdo) / ds_boost)
    m = -F(F(ds_boost / p_shift) / F(sv * sdo))
    return (F(F(softmax * sq) * sk), F(F(1.0) / F(sv * sdo)), F(ds_boost / p_shift), F(sdo / p_shift),
            F(F(softmax * sq) * r), F(F(r * sk) * dq_boost), m, F(softmax / dq_boost))
