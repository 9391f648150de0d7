"""CPU oracle of the block-scaled quantisers (TEST INFRASTRUCTURE, not product code).

A numpy restatement, written from the format definitions, of the reference's quantiser contracts:

  * token-block MXFP8 (E4M3 codes, one UE8M0 exponent per 32 tokens x the whole head dim), its side tables and the
    fused backward-prologue outputs          -- tests/cute/quant_reference.py:687-703, 714-798 (fp8_blocks_reference,
                                                ue8m0_exponent, lse_log2_reference) of the reference
  * NVFP4 rows (E2M1 codes, E4M3 scale / 16) -- tests/cute/quant_reference.py:62-89, 179-216, 270-369
                                                (e2m1_encode_rn, pack_nibbles, _nvfp4_scale, _encode_groups,
                                                fp4_rows_reference)
  * the 128 x 4 scale-factor atom            -- tests/cute/quant_reference.py:163-175, 706-710
  * the random-sign Hadamard rotation        -- tests/cute/quant_reference.py:129-140, 633-648 and
                                                flash_attn/cute/quant/_rotations.py:107-115 (sign vector)
  * D = rowsum(O * dequant(dO)) in the kernels' fixed fp32 tree order -- tests/cute/test_quant_fp8.py:77-92

Parity pin: tests/test_oracle_golden.py compares every function here, byte for byte, with fixtures under
tests/golden/ that were produced by importing the reference's own quant_reference.py (tests/golden/make_golden.py).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may import this package. The product
(flamia_blackwell_attention_b200) never does and has no CPU fallback.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
U32 = np.uint32
FLT_MIN = F32(2.0 ** -126)

# signs[i] = -1 where bit i is set: torch CPU generator, manual_seed(4321), randint(0, 2, (128,)) * 2 - 1
_HADAMARD_NEG_MASK_4321 = 0x75954FED45809F07E0D9F0E210D2E03E
E2M1_GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def hadamard_signs(d: int = 128) -> np.ndarray:
    """(d,) float32 +-1 sign vector of the fixed rotation (seed 4321)."""
    assert d == 128
    return np.array([-1.0 if (_HADAMARD_NEG_MASK_4321 >> i) & 1 else 1.0 for i in range(128)], dtype=np.float32)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32."""
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (round to nearest even), uint16."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (r >> np.uint32(16)).astype(np.uint16)


# ------------------------------------------------------------------------------------------------ element formats
def e4m3_encode(y: np.ndarray) -> np.ndarray:
    """float32 -> E4M3 (fn) byte: clamp to +-448 (satfinite), round to nearest even; -0.0 -> 0x80."""
    y = np.ascontiguousarray(y, dtype=np.float32)
    sign = (y.view(np.uint32) >> np.uint32(24)) & np.uint32(0x80)
    a = np.minimum(np.abs(y), F32(448.0))
    bits = a.view(np.uint32)
    # normal range |y| >= 2^-6: round the 23-bit mantissa to 3 bits
    r = bits + np.uint32(0x7FFFF) + ((bits >> np.uint32(20)) & np.uint32(1))
    normal = (r >> np.uint32(20)).astype(np.int64) - ((127 - 7) << 3)
    # subnormal range: multiples of 2^-9, rint = ties to even (8 = the smallest normal, same code space)
    sub = np.rint(a.astype(np.float64) * 512.0).astype(np.int64)
    code = np.where(a >= F32(2.0 ** -6), normal, sub)
    code = np.where(np.isnan(y), 0x7F, code)
    return (code.astype(np.uint32) | sign).astype(np.uint8)


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    c = code.astype(np.int64)
    e = (c >> 3) & 0xF
    m = c & 7
    v = np.where(e == 0, m * 2.0 ** -9, (8 + m) * np.exp2((e - 10).astype(np.float64)))
    v = np.where((c & 0x7F) == 0x7F, np.nan, v)
    return np.where(c & 0x80, -v, v).astype(np.float32)


def e2m1_encode(y: np.ndarray) -> np.ndarray:
    """float32 -> E2M1 nibble (sign in bit 3): nearest grid point, ties to the even code, |y| > 6 -> 6, NaN -> 7."""
    y = np.ascontiguousarray(y, dtype=np.float32)
    nan = np.isnan(y)
    a = np.where(nan, F32(6.0), np.minimum(np.abs(y), F32(6.0))).astype(np.float64)
    # midpoints between neighbouring grid values; a tie goes to the even code index
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    idx = np.zeros(a.shape, dtype=np.int64)
    for k, m in enumerate(mids):           # code k -> k+1 when above the midpoint, or at it when k+1 is even
        up = (a > m) | ((a == m) & ((k + 1) % 2 == 0))
        idx = np.where(up & (idx == k), k + 1, idx)
    neg = np.signbit(y) & ~nan
    return (idx + 8 * neg).astype(np.uint8)


def e2m1_decode(code: np.ndarray) -> np.ndarray:
    c = code.astype(np.int64)
    v = E2M1_GRID[c & 7]
    return np.where(c & 8, -v, v).astype(np.float32)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    c = codes.astype(np.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << np.uint8(4))).astype(np.uint8)


def flush_subnormals(x: np.ndarray) -> np.ndarray:
    """fp32 subnormals -> zero of the same sign."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return np.where(np.abs(x) < FLT_MIN, x * F32(0.0), x).astype(np.float32)


# ------------------------------------------------------------------------------------------------ UE8M0 selector
def ue8m0_select(amax: np.ndarray, fmax_is_448: bool = True):
    """Round-up power-of-two selector: the smallest e with 448 * 2^e >= amax. Returns (byte = e + 127, scale = 2^e);
    byte 0 / scale 0 for a block whose fp32(amax * fp32(1/448)) is below the smallest normal (zero included)."""
    assert fmax_is_448
    amax = np.ascontiguousarray(amax, dtype=np.float32)
    m, k = np.frexp(amax.astype(np.float64))            # amax = m * 2^k, m in [0.5, 1)
    # amax / 448 = (m / 0.875) * 2^(k - 9);  448 = 0.875 * 2^9
    e = np.where(m <= 0.875, k - 9, k - 8).astype(np.int64)
    r = (amax * F32(1.0 / 448.0)).astype(np.float32)
    pos = r >= FLT_MIN
    byte = np.where(pos, e + 127, 0).astype(np.uint8)
    scale = np.where(pos, np.exp2(e.astype(np.float64)), 0.0).astype(np.float32)
    return byte, scale


# ------------------------------------------------------------------------------------------------ SF atom
def sf_atoms(table: np.ndarray) -> np.ndarray:
    """(b, h, R, G) bytes (row r, K group g; R % 128 == 0, G % 4 == 0) -> (b, h, R/128, G/4, 32, 4, 4): the SM100
    128 x 4 atom, byte (r % 32) * 16 + ((r // 32) % 4) * 4 + g % 4 of atom (r // 128, g // 4)."""
    b, h, R, G = table.shape
    t = table.reshape(b, h, R // 128, 4, 32, G // 4, 4)     # row = rt*128 + j*32 + i
    return np.ascontiguousarray(t.transpose(0, 1, 2, 5, 4, 3, 6))


# ------------------------------------------------------------------------------------------------ Hadamard
def hadamard_rotate(x: np.ndarray) -> np.ndarray:
    """(x * signs) H_128 / sqrt(128) along the last dim, fp32, butterfly levels 1, 2, ..., 64 with (a, b) -> (a+b, a-b),
    then one multiply by fp32(1/sqrt(128))."""
    y = (np.ascontiguousarray(x, dtype=np.float32) * hadamard_signs()).astype(np.float32)
    shape = y.shape
    h = 1
    while h < 128:
        y = y.reshape(*shape[:-1], 128 // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = np.stack(((a + b).astype(np.float32), (a - b).astype(np.float32)), -2).reshape(shape)
        h *= 2
    return (y * F32(1.0 / np.sqrt(128.0))).astype(np.float32)


def hadamard_unrotate(y: np.ndarray) -> np.ndarray:
    """The inverse map used on dQ / dK: (y H_128 / sqrt(128)) * signs, same butterfly order."""
    z = np.ascontiguousarray(y, dtype=np.float32)
    shape = z.shape
    h = 1
    while h < 128:
        z = z.reshape(*shape[:-1], 128 // (2 * h), 2, h)
        a, b = z[..., 0, :], z[..., 1, :]
        z = np.stack(((a + b).astype(np.float32), (a - b).astype(np.float32)), -2).reshape(shape)
        h *= 2
    return ((z * F32(1.0 / np.sqrt(128.0))).astype(np.float32) * hadamard_signs()).astype(np.float32)


# ------------------------------------------------------------------------------------------------ D tree order
def row_dot_tree(a: np.ndarray, o: np.ndarray) -> np.ndarray:
    """sum_c a_c o_c over the last dim (128, shorter rows zero-padded) in the fixed fp32 order: first
    fma(a_c, o_c, fl(a_{c+2} o_{c+2})) for c with bit 1 clear, then pairwise adds over column bits 2, 3, 0, 6, 5, 4."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    o = np.ascontiguousarray(o, dtype=np.float32)
    d = a.shape[-1]
    if d < 128:
        pad = [(0, 0)] * (a.ndim - 1) + [(0, 128 - d)]
        a, o = np.pad(a, pad), np.pad(o, pad)
    idx = np.arange(128)
    lo = idx[((idx >> 1) & 1) == 0]
    hi_prod = (a[..., lo + 2] * o[..., lo + 2]).astype(np.float32)
    v = (a[..., lo].astype(np.float64) * o[..., lo].astype(np.float64) + hi_prod.astype(np.float64)).astype(np.float32)
    cols = lo
    for bit in (2, 3, 0, 6, 5, 4):
        keep = ((cols >> bit) & 1) == 0
        pos = np.full(128, -1)
        pos[cols] = np.arange(cols.size)
        partner = pos[cols[keep] | (1 << bit)]
        v = (v[..., keep] + v[..., partner]).astype(np.float32)
        cols = cols[keep]
    return v[..., 0]


# ------------------------------------------------------------------------------------------------ NVFP4 rows
def nvfp4_rows(x: np.ndarray, rotate: bool = False) -> dict:
    """x (b, s, h, d) float32 values (bf16-representable) -> NVFP4 'qk_operand' codes: per 16 along d, SF =
    E4M3_rn(amax * fp32(1/6)) with fp32 subnormals flushed first; codes = E2M1_rn(flush(x * m)), m = fp32(1/SF) for
    SF > 0, +inf when SF rounds to 0 while amax * fp32(1/6) > 0, 0 for an all-zero group.
    Returns codes (b, s, h, d/2) uint8 (element 0 in the low nibble) and sf (b, h, s/128, d/64, 32, 4, 4)."""
    b, s, h, d = x.shape
    xf = np.ascontiguousarray(x, dtype=np.float32)
    if rotate:
        xf = hadamard_rotate(xf)
    g = flush_subnormals(xf).reshape(b, s, h, d // 16, 16)
    a = np.abs(g)
    amax = np.where(np.isnan(a), F32(0), a).max(-1)
    u = (amax * F32(1.0 / 6.0)).astype(np.float32)
    sfb = e4m3_encode(u)
    sfv = e4m3_decode(sfb)
    with np.errstate(divide="ignore"):
        mult = np.where(sfv > 0, (F32(1.0) / np.where(sfv > 0, sfv, F32(1))).astype(np.float32),
                        np.where(u > 0, F32(np.inf), F32(0.0))).astype(np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        y = flush_subnormals((g * mult[..., None]).astype(np.float32))
    codes = e2m1_encode(y).reshape(b, s, h, d)
    table = np.ascontiguousarray(sfb.transpose(0, 2, 1, 3))               # (b, h, s, d/16)
    return dict(codes=pack_nibbles(codes), sf=sf_atoms(table), sf_table=table)


def nvfp4_dequant(codes: np.ndarray, sf_table: np.ndarray) -> np.ndarray:
    """packed codes (b, s, h, d/2) + sf_table (b, h, s, d/16) -> float32 (b, s, h, d)."""
    c = codes.astype(np.uint8)
    nib = np.stack([c & 0xF, c >> 4], -1).reshape(*c.shape[:-1], -1)
    val = e2m1_decode(nib)
    sfv = e4m3_decode(sf_table).transpose(0, 2, 1, 3)                     # (b, s, h, d/16)
    return (val.reshape(*val.shape[:-1], -1, 16) * sfv[..., None]).reshape(val.shape).astype(np.float32)


# ------------------------------------------------------------------------------------------------ MXFP8 blocks
def fp8_token_blocks(x: np.ndarray, *, rotate: bool = False, token_local: bool = False,
                     d_with_output: np.ndarray | None = None, lse: np.ndarray | None = None,
                     lse_shift: float = 0.0, d_multiplier: float = 1.0, nvfp4_copy: bool = False) -> dict:
    """Token-block MXFP8 of x (b, s, h, d) float32 (values of a bf16 tensor), s % 128 == 0, d in {64, 128}.

    Per 32 tokens x d block: amax (fp32 subnormals are zero) -> UE8M0 byte (ue8m0_select) -> codes =
    E4M3_rn(clamp(x * 2^-e, +-448)) (all zero for a byte-0 block).
    token_local: codes / sf_tok use each token's own exponent; e / fac / sf_dim the block's (sf_dim is the unit byte 127
    on the token-local route is the caller's choice and not produced here).
    Outputs (names follow the reference's quantize_fp8_blocks): codes (b,s,h,d) u8, codes_t (b,h,d,s) u8,
    e (b,h,s/32,d/32) u8, fac (b,h,s/32) f32, sf_tok_raw (b,h,s/128,1,32,4,4) u8, sf_dim_raw (b,h,1,s/128,32,4,4) u8,
    token_factors (b,h,s) f32 [token_local], D (b,h,s) f32 = d_multiplier * row_dot_tree(dequant, O), lse_log2 (b,h,s),
    x4 / sf4 (NVFP4 copy of the same, possibly rotated, values)."""
    b, s, h, d = x.shape
    assert s % 128 == 0 and d in (64, 128)
    xf = np.ascontiguousarray(x, dtype=np.float32)
    if rotate:
        assert d == 128
        xf = hadamard_rotate(xf)
    xq = flush_subnormals(xf)
    a = np.abs(xq).transpose(0, 2, 1, 3)                                  # (b, h, s, d)
    blk = a.reshape(b, h, s // 32, 32 * d).max(-1)                        # (b, h, s/32)
    byte, scale = ue8m0_select(blk)
    sc_tok = np.repeat(scale, 32, axis=2)                                 # (b, h, s)
    by_tok = np.repeat(byte, 32, axis=2)
    out = {}
    if token_local:
        tbyte, tscale = ue8m0_select(a.max(-1))                           # (b, h, s)
        sc_tok = tscale
        out["token_factors"] = np.where(tscale > 0, tscale, F32(1.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(sc_tok > 0, 1.0 / sc_tok.astype(np.float64), 0.0)
    y = (xq.transpose(0, 2, 1, 3).astype(np.float64) * inv[..., None]).astype(np.float32)   # (b, h, s, d)
    codes_bh = e4m3_encode(y)
    out["codes"] = np.ascontiguousarray(codes_bh.transpose(0, 2, 1, 3))
    out["codes_t"] = np.ascontiguousarray(codes_bh.transpose(0, 1, 3, 2))
    ng = d // 32
    e_tab = np.repeat(byte[..., None], ng, axis=-1)                       # (b, h, s/32, d/32)
    out["e"] = np.ascontiguousarray(e_tab)
    # factor row: 2^(e-127); an all-zero block takes its 128-token tile's largest factor, 1 for an all-zero tile
    e0 = byte.astype(np.int64)
    tile_max = np.repeat(e0.reshape(b, h, s // 128, 4).max(-1), 4, axis=-1)
    e0 = np.where(e0 > 0, e0, tile_max)
    out["fac"] = np.where(e0 > 0, np.exp2((e0 - 127).astype(np.float64)), 1.0).astype(np.float32)
    k = (tbyte if token_local else by_tok)[..., None].repeat(ng, -1)      # (b, h, s, d/32)
    if ng < 4:
        k = np.tile(k, (1, 1, 1, 4 // ng))
    out["sf_tok_raw"] = sf_atoms(np.ascontiguousarray(k))
    t = np.repeat(byte[:, :, None, :], 128, axis=2)                       # (b, h, 128 rows (d, repeated), s/32)
    out["sf_dim_raw"] = sf_atoms(np.ascontiguousarray(t))
    if d_with_output is not None:
        deq = (e4m3_decode(codes_bh).astype(np.float64) * sc_tok[..., None].astype(np.float64)).astype(np.float32)
        o = np.ascontiguousarray(d_with_output, dtype=np.float32).transpose(0, 2, 1, 3)
        out["D"] = (row_dot_tree(deq, o) * F32(d_multiplier)).astype(np.float32)
        out["D_f64"] = (deq.astype(np.float64) * o.astype(np.float64)).sum(-1)
    if lse is not None:
        out["lse_log2"] = lse_log2(lse, lse_shift)
    if nvfp4_copy:
        r4 = nvfp4_rows(xf)            # the same (possibly rotated) values, 'raw' scaling
        out["x4"], out["sf4"], out["sf4_table"] = r4["codes"], r4["sf"], r4["sf_table"]
    return out


def fp8_dequant(codes: np.ndarray, e: np.ndarray) -> np.ndarray:
    """codes (b, s, h, d) + exponent table (b, h, s/32, d/32) -> float32 (b, s, h, d); byte 0 = zero block."""
    b, s, h, d = codes.shape
    sc = np.where(e[..., 0] == 0, 0.0, np.exp2(e[..., 0].astype(np.float64) - 127.0))     # (b, h, s/32)
    sc = np.repeat(sc, 32, axis=2).transpose(0, 2, 1)[..., None]                         # (b, s, h, 1)
    return (e4m3_decode(codes).astype(np.float64) * sc).astype(np.float32)


def lse_log2(lse: np.ndarray, shift: float) -> np.ndarray:
    """where(lse == -inf, 0, fp32(lse * fp32(log2 e))) - fp32(shift), fp32 operations."""
    lse = np.ascontiguousarray(lse, dtype=np.float32)
    with np.errstate(invalid="ignore"):
        prod = (lse * F32(1.4426950408889634)).astype(np.float32)
    return (np.where(np.isneginf(lse), F32(0.0), prod) - F32(shift)).astype(np.float32)
