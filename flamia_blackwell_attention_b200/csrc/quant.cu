// Fused block-scaled quantiser (token-block MXFP8, optional NVFP4 S-operand copy, optional Hadamard rotation) and the
// fused backward prologue (D = rowsum(O * dequant(dO)), shifted log2 LSE, zeroed f16 dQ accumulator).
//
// Replaces the reference's quantize_fp8_blocks launch (flash_attn/cute/quant/fp8.py:2512, kernel_stream :1639; its input
// staging :262-300) and the fused NVFP4 copy (flash_attn/cute/quant/_fp8_nvfp4.py:121-158). Outputs are byte-identical to
// the reference's eager definitions (tests/cute/quant_reference.py:714-798, 270-369).
//
// Persistent CTAs (512 threads) walk the (128-token tile, head) pairs of the tensor, heads fastest, so the CTAs running
// at any moment read one contiguous stretch of the (b, s, h, d) input. Each CTA keeps STAGES tiles in flight: one thread
// issues the TMA loads of tile t + STAGES (plain cp.async.bulk.tensor, never multicast) as soon as every thread has read
// tile t out of its stage, so the memory system stays busy while the butterflies and conversions of the current tile run.
// Four lanes share a token row: lane q of the row holds the 16-byte chunks c = 4 j + q (8 elements each); element index
// i = 32 j + 8 q + e, so the Hadamard levels 1, 2, 4 and 32, 64 are in-thread and levels 8, 16 are two lane exchanges:
// the same order of operations as a one-thread-per-row butterfly, hence the same bits. The butterflies run as packed
// f32x2 instructions on register pairs (chunk j, chunk j + 2): one issue slot per two additions, same rounding.
// Bound: HBM (2 B read + 1 B written per element, plus the optional copies).
#include "flamia_internal.h"

namespace fl {

static constexpr int QT = 128;        // tokens per tile
static constexpr int QTHREADS = 512;  // four lanes per token
static constexpr int QSTAGES = 3;

struct QuantParams {
  const float* lse;       // (b, h, s) or null
  uint8_t* codes;         // (b, s, h, d)
  uint8_t* codes_t;       // (b, h, d, s) or null
  uint8_t* e_tab;         // (b, h, s/32, d/32) or null
  float* fac;             // (b, h, s/32) or null
  uint8_t* sf_tok;        // (b, h, s/128, 512) or null
  uint8_t* sf_dim;        // (b, h, s/128, 512) or null
  float* token_factors;   // (b, h, s) or null
  uint8_t* x4;            // (b, s, h, d/2) or null
  uint8_t* sf4;           // (b, h, s/128, d/64, 512) or null
  float* d_out;           // (b, h, s) or null
  float* lse_log2;        // (b, h, s) or null
  uint16_t* zero_acc;     // f16 accumulator of b * h * s * d elements or null
  float* tile_stats;      // (b, h, s/128, 2): [amax of the values quantised, max row sum of squares] or null
  uint32_t* row_stat;     // (b, s) per-token maximum over the heads (float bits, zero on entry) or null
  int row_stat_kind;      // 1 = sum of squares, 2 = largest magnitude, 3 = 2-norm
  int o_packed;           // packed source: the forward output o has the packed rows of x (else the outputs' rows)
  int b, s, h;
  const int32_t* slot_src;   // packed source: first source row of each 128-row slot of the output (-1: an empty slot), or null
  const int32_t* slot_rows;  // packed source: valid rows of each slot (the rest of the slot reads as zero)
  int n_tiles;            // b * (s / 128) * h
  int token_local;
  int in_f16;
  float lse_shift, d_multiplier;
  DevCtl ctl;
};

__device__ __forceinline__ float flush_sub(float v) { return fabsf(v) < 1.17549435e-38f ? v * 0.0f : v; }
// packed pairs: a + b, a - b, and a * b with subnormal inputs and results flushed to zero (the product and its flush in
// one instruction); each half rounds exactly as the scalar instruction does
__device__ __forceinline__ uint64_t mul2_ftz(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint4 lds_u4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// UE8M0 round-up selector: smallest e with 448 * 2^e >= amax; byte 0 when fp32(amax * fp32(1/448)) is subnormal / zero
__device__ __forceinline__ uint32_t ue8m0_byte(float amax) {
  float r = __fmul_rn(amax, 1.0f / 448.0f);
  if (!(r >= 1.17549435e-38f)) return 0;
  uint32_t bits = __float_as_uint(amax);
  uint32_t E = bits >> 23, man = bits & 0x7FFFFF;
  return man <= 0x600000 ? E - 8 : E - 7;   // 448 = 1.75 * 2^8
}
__device__ __forceinline__ float pow2_from_field(int field) { return __uint_as_float((uint32_t)field << 23); }

// two E4M3 codes (low byte first) -> their exact values
__device__ __forceinline__ float2 e4m3x2_to_f32(uint16_t v) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(v));
  return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}

// MODE bits: 1 = the E4M3 codes are of the rotated rows, 2 = also write the NVFP4 copy, 4 = rotate only the NVFP4 copy
// PK: packed source (slot tables); a template flag, so that the batched form pays nothing for it
template <int D, int MODE, bool PRO, bool PK>
__global__ void __launch_bounds__(QTHREADS, PRO ? 1 : 2)
quant_blocks_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_o,
                    const QuantParams p) {
  constexpr bool ROT = (MODE & 1) != 0, NV4 = (MODE & 2) != 0, ROT4 = (MODE & 4) != 0;
  constexpr int NJ = D / 32;                     // 16-byte chunks per lane
  constexpr int NE = 8 * NJ;                     // elements per lane
  constexpr int TILE_B = QT * D * 2;             // bytes of one 16-bit input tile
  constexpr int STAGE_B = PRO ? 2 * TILE_B : TILE_B;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_codes = smem + QSTAGES * STAGE_B;   // channel-major copy only (present when codes_t is asked for)
  __shared__ __align__(8) uint64_t full[QSTAGES];
  __shared__ float s_wmax[2][16];                // per-warp (8 rows) maximum, double-buffered by tile parity
  __shared__ float s_wsq[2][16];                 // per-warp maximum row sum of squares
  __shared__ __align__(16) uint32_t s_sign[4][4][4];   // [lane of the row][chunk][word]: sign bits of the rotation
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // lane -> (row of the warp's eight, lane of the row). The two rows of a quarter warp differ in bit 2, so that with
  // the 128-byte swizzle their 16-byte chunks fall into different bank groups (conflict-free 128-bit loads).
  const int q = lane & 3;
  const int r = warp * 8 + ((lane >> 2) & 1) * 4 + (lane >> 3);      // token row of the tile
  const int G = gridDim.x;
  const int ntile = p.s / QT;
  volatile int* abortp = &abort_s;

  auto issue = [&](int L, int st) {              // one thread: the loads of linear tile L into stage st
    const int head = L % p.h, tile = (L / p.h) % ntile, bat = L / (p.h * ntile);
    uint8_t* dst = smem + st * STAGE_B;
    // packed source (documents stored back to back): the slot's rows start at an arbitrary row of the (1, total, h, d)
    // tensor; only the innermost TMA coordinate has an alignment rule. An empty slot loads nothing of x.
    const int xrow = PK ? p.slot_src[tile] : tile * QT;
    mbar_arrive_expect_tx(&full[st], (xrow >= 0 ? TILE_B : 0) + ((PRO && (xrow >= 0 || !(PK && p.o_packed))) ? TILE_B : 0));
    if (xrow >= 0) {
      tma_load_4d(dst, &tm_x, &full[st], 0, head, xrow, bat);
      if (D == 128) tma_load_4d(dst + TILE_B / 2, &tm_x, &full[st], 64, head, xrow, bat);
    }
    if (PRO) {
      // (packed source: the forward output has the packed rows too; an empty slot's stage keeps what it held, and its
      // rows read as zero below)
      const int orow = (PK && p.o_packed) ? xrow : tile * QT;
      if (orow >= 0) {
        tma_load_4d(dst + TILE_B, &tm_o, &full[st], 0, head, orow, bat);
        if (D == 128) tma_load_4d(dst + TILE_B + TILE_B / 2, &tm_o, &full[st], 64, head, orow, bat);
      }
    }
  };
  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < QSTAGES; ++i) mbar_init(&full[i], 1);
    fence_barrier_init();
    tma_prefetch_desc(&tm_x);
    if (PRO) tma_prefetch_desc(&tm_o);
    for (int i = 0; i < QSTAGES; ++i)
      if (blockIdx.x + i * G < p.n_tiles) issue(blockIdx.x + i * G, i);
  }
  if ((ROT || ROT4) && tid < 16) {               // sign words: bit 15 / 31 of word k = sign of element 2 k / 2 k + 1
    constexpr uint32_t NEG[4] = {0x10D2E03Eu, 0xE0D9F0E2u, 0x45809F07u, 0x75954FEDu};
    const int qq = tid >> 2, j = tid & 3;
    const uint32_t m = (NEG[j] >> (8 * qq)) & 0xFF;
#pragma unroll
    for (int k = 0; k < 4; ++k) s_sign[qq][j][k] = (((m >> (2 * k)) & 1) << 15) | (((m >> (2 * k + 1)) & 1) << 31);
  }
  __syncthreads();

  // raw 16-byte chunk j of this thread's row (global chunk 4 j + q) from a staged tile
  bool row_live = true;                          // packed source: false for the rows of a slot past its document's end
  auto lds_chunk = [&](uint32_t tile_addr, int j) -> uint4 {
    const int g = 4 * j + q;
    const uint32_t box = (D == 128) ? (uint32_t)(g >> 3) * (TILE_B / 2) : 0u;
    return lds_u4(tile_addr + box + r * 128 + (((g & 7) ^ (r & 7)) << 4));
  };
  // the same for a chunk of x: rows that do not belong to the slot's document (or an empty slot, whose stage holds
  // whatever was there) read as zero
  auto lds_chunk_x = [&](uint32_t tile_addr, int j) -> uint4 {
    uint4 v = lds_chunk(tile_addr, j);
    if (PK && !row_live) v = make_uint4(0, 0, 0, 0);
    return v;
  };
  auto to_f32 = [&](const uint4& v, float* dst) {      // 8 elements of one chunk
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    if (p.in_f16) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
        dst[2 * k] = f.x;
        dst[2 * k + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        dst[2 * k] = __uint_as_float(w[k] << 16);
        dst[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
      }
    }
  };
  // (y * signs) H_128 / sqrt(128): butterfly levels 1, 2, ..., 64 with (a, b) -> (a + b, a - b), then the scaling with
  // subnormal results flushed. Reads the staged tile, leaves the rotated row in y.
  auto load_rotated = [&](uint32_t tile_addr, float* y) {
    if constexpr (D == 128) {
      float t[32];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v = lds_chunk_x(tile_addr, j);
        const uint4 sg = *reinterpret_cast<const uint4*>(&s_sign[q][j][0]);
        v.x ^= sg.x; v.y ^= sg.y; v.z ^= sg.z; v.w ^= sg.w;
        to_f32(v, t + 8 * j);
      }
      uint64_t Y[16];                              // Y[8 jp + e] = (element (jp, e), element (jp + 2, e))
#pragma unroll
      for (int k = 0; k < 16; ++k) Y[k] = pack2(t[k], t[k + 16]);
#pragma unroll
      for (int hs = 1; hs < 8; hs <<= 1) {         // element bits 0..2: inside one chunk
#pragma unroll
        for (int k = 0; k < 16; ++k)
          if ((k & hs) == 0) {
            const uint64_t a = Y[k], b2 = Y[k + hs];
            Y[k] = add2(a, b2);
            Y[k + hs] = sub2(a, b2);
          }
      }
#pragma unroll
      for (int lb = 1; lb < 4; lb <<= 1) {         // element bits 3, 4 = the lane of the row
        // low lane: y + other; high lane: other - y. Both are other + (+-1) y: one fma (the product is exact)
        const float sg = (q & lb) ? -1.0f : 1.0f;
        const uint64_t sg2 = pack2(sg, sg);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          float lo, hi;
          unpack2(Y[k], lo, hi);
          const uint64_t other = pack2(__shfl_xor_sync(0xFFFFFFFFu, lo, lb), __shfl_xor_sync(0xFFFFFFFFu, hi, lb));
          Y[k] = fma2(Y[k], sg2, other);
        }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {                // element bit 5 = chunk bit 0
        const uint64_t a = Y[k], b2 = Y[k + 8];
        Y[k] = add2(a, b2);
        Y[k + 8] = sub2(a, b2);
      }
      const uint64_t c2 = pack2(0.08838834764831845f, 0.08838834764831845f);
#pragma unroll
      for (int k = 0; k < 16; ++k) {               // element bit 6 = chunk bit 1: the two halves of a pair
        float lo, hi;
        unpack2(Y[k], lo, hi);
        const uint64_t s2 = mul2_ftz(pack2(__fadd_rn(lo, hi), __fsub_rn(lo, hi)), c2);   // scaled and flushed
        unpack2(s2, y[k], y[k + 16]);
      }
    }
  };
  auto load_plain = [&](uint32_t tile_addr, float* y) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) to_f32(lds_chunk_x(tile_addr, j), y + 8 * j);
  };

  int it = 0;
  for (int L = blockIdx.x; L < p.n_tiles; L += G, ++it) {
    const int st = it % QSTAGES, par = it & 1;
    const int head = L % p.h, tile = (L / p.h) % ntile, bat = L / (p.h * ntile);
    const int t0 = tile * QT;
    const size_t row_off = (((size_t)bat * p.s + t0 + r) * p.h + head) * D;     // this row in a (b, s, h, D) tensor
    const size_t bh = (size_t)bat * p.h + head;
    const size_t ri = bh * p.s + t0 + r;
    const uint32_t tile_addr = smem_u32(smem + st * STAGE_B);
    bool ok = mbar_wait(&full[st], (it / QSTAGES) & 1, p.ctl, abortp, 50);
    if (PK) row_live = r < p.slot_rows[tile];

    if (p.zero_acc) {   // this tile's share of the accumulator: 128 * D f16 = 32 D 16-byte chunks, contiguous
      uint4* z = reinterpret_cast<uint4*>(p.zero_acc + (bh * p.s + t0) * D);
      const uint4 zero = make_uint4(0, 0, 0, 0);
      for (int i = tid; i < QT * D / 8; i += QTHREADS) z[i] = zero;
    }

    // NVFP4 copy of y: per 16 along d (two neighbouring lanes): SF = E4M3_rn(amax * f32(1/6)); codes = E2M1_rn(ftz(y * m)),
    // m = 1 / SF | +inf (SF rounds to 0, amax > 0) | 0
    auto nvfp4_row = [&](const float* y) {
      uint32_t sfpack = 0;                         // this lane's scale bytes: chunk j in byte j
      uint8_t* x4row = p.x4 + row_off / 2;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        float am = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float a = fabsf(flush_sub(y[8 * j + e]));
          am = (a > am) ? a : am;                  // a NaN never wins
        }
        const float oth = __shfl_xor_sync(0xFFFFFFFFu, am, 1);
        am = (oth > am) ? oth : am;
        const float u = __fmul_rn(am, 1.0f / 6.0f);
        const uint32_t sfb = cvt_e4m3x2(u, 0.f) & 0xFF;
        const float sfv = e4m3x2_to_f32((uint16_t)sfb).x;
        const float m = sfv > 0.f ? __frcp_rn(sfv) : (u > 0.f ? __int_as_float(0x7F800000) : 0.f);
        uint32_t packed = 0;
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float a0 = flush_sub(__fmul_rn(flush_sub(y[8 * j + e]), m));
          const float a1 = flush_sub(__fmul_rn(flush_sub(y[8 * j + e + 1]), m));
          uint16_t c2;
          asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}" : "=h"(c2) : "f"(a1), "f"(a0));
          packed |= (uint32_t)(c2 & 0xFF) << (e * 4);
        }
        *reinterpret_cast<uint32_t*>(x4row + (4 * j + q) * 4) = packed;
        sfpack |= sfb << (8 * j);
      }
      // group g = 2 j + (q >> 1): atom g / 4 = j / 2, byte g % 4 = 2 (j & 1) + (q >> 1); lane 0 of the row assembles
      const uint32_t hi = __shfl_down_sync(0xFFFFFFFFu, sfpack, 2);
      if (p.sf4 && q == 0) {
        uint8_t* atom = p.sf4 + ((bh * ntile + tile) * (D / 64)) * 512;
#pragma unroll
        for (int a = 0; a < D / 64; ++a) {
          const uint32_t lo0 = (sfpack >> (16 * a)) & 0xFF, lo1 = (sfpack >> (16 * a + 8)) & 0xFF;
          const uint32_t hi0 = (hi >> (16 * a)) & 0xFF, hi1 = (hi >> (16 * a + 8)) & 0xFF;
          *reinterpret_cast<uint32_t*>(atom + a * 512 + (r & 31) * 16 + (r >> 5) * 4) = lo0 | (hi0 << 8) | (lo1 << 16) | (hi1 << 24);
        }
      }
    };

    float x[NE];
    if (ROT4) {          // NVFP4 codes of the rotated row, E4M3 codes of the row as read
      load_rotated(tile_addr, x);
      nvfp4_row(x);
      load_plain(tile_addr, x);
    } else if (ROT) {
      load_rotated(tile_addr, x);
      if (NV4) nvfp4_row(x);
    } else {
      load_plain(tile_addr, x);
      if (NV4) nvfp4_row(x);
    }
    uint4 o_raw[NJ];     // prologue: the forward output's row, kept as read until the codes exist
    if (PRO) {
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        o_raw[j] = lds_chunk(tile_addr + TILE_B, j);
        if (PK && p.o_packed && !row_live) o_raw[j] = make_uint4(0, 0, 0, 0);
      }
    }

    // ---- exponents: per token (4 lanes) and per 32-token block (4 warps)
    float amax = 0.f, sumsq = 0.f;
    if (!ROT || ROT4) {  // subnormal -> zero of the same sign (rotated rows were flushed by their scaling)
#pragma unroll
      for (int i = 0; i < NE; i += 2) {
        const uint64_t f2 = mul2_ftz(pack2(x[i], x[i + 1]), pack2(1.0f, 1.0f));
        unpack2(f2, x[i], x[i + 1]);
      }
    }
#pragma unroll
    for (int i = 0; i < NE; i += 2) amax = fmaxf(fmaxf(amax, fabsf(x[i])), fabsf(x[i + 1]));
    if (p.tile_stats || p.row_stat) {     // the row norm is only wanted with the statistics (K, V, dO)
      float sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < NE; ++i) sq[i & 3] = fmaf(x[i], x[i], sq[i & 3]);
      sumsq = (sq[0] + sq[1]) + (sq[2] + sq[3]);
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));      // the token's maximum
    sumsq += __shfl_xor_sync(0xFFFFFFFFu, sumsq, 1);
    sumsq += __shfl_xor_sync(0xFFFFFFFFu, sumsq, 2);
    if (p.row_stat && q == 0 && (!PK || row_live)) {     // non-negative floats order as their bit patterns
      const float v = p.row_stat_kind == 2 ? amax : (p.row_stat_kind == 3 ? __fsqrt_rn(sumsq) : sumsq);
      atomicMax(p.row_stat + (size_t)bat * p.s + t0 + r, __float_as_uint(v));
    }
    float wmax = amax, wsq = sumsq;
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      wmax = fmaxf(wmax, __shfl_xor_sync(0xFFFFFFFFu, wmax, o));
      wsq = fmaxf(wsq, __shfl_xor_sync(0xFFFFFFFFu, wsq, o));
    }
    if (lane == 0) { s_wmax[par][warp] = wmax; s_wsq[par][warp] = wsq; }
    // every thread has read the stage: it can take tile it + STAGES. A wait that ran out leaves the loop here, all
    // threads together.
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (!ok) break;
    if (tid == 0 && L + QSTAGES * G < p.n_tiles) issue(L + QSTAGES * G, st);

    const float* wm = s_wmax[par];
    const int blk = r >> 5;                                         // 32-token block of the tile
    const float bmax = fmaxf(fmaxf(wm[4 * blk], wm[4 * blk + 1]), fmaxf(wm[4 * blk + 2], wm[4 * blk + 3]));
    const uint32_t bbyte = ue8m0_byte(bmax);
    const bool tl = p.token_local != 0;
    const uint32_t tbyte = tl ? ue8m0_byte(amax) : bbyte;
    const float inv = tbyte ? pow2_from_field(254 - (int)tbyte) : 0.f;
    const float scale = tbyte ? pow2_from_field((int)tbyte) : 0.f;

    uint32_t cw[2 * NJ];
    {
      const uint64_t inv2 = pack2(inv, inv);
#pragma unroll
      for (int i = 0; i < 2 * NJ; ++i) {
        float a0, a1, a2, a3;
        unpack2(mul2(pack2(x[4 * i], x[4 * i + 1]), inv2), a0, a1);
        unpack2(mul2(pack2(x[4 * i + 2], x[4 * i + 3]), inv2), a2, a3);
        cw[i] = cvt_e4m3x4(a0, a1, a2, a3);
      }
      uint8_t* crow = p.codes + row_off;
#pragma unroll
      for (int j = 0; j < NJ; ++j)
        *reinterpret_cast<uint2*>(crow + (4 * j + q) * 8) = make_uint2(cw[2 * j], cw[2 * j + 1]);
    }

    // ---- prologue: D in the fixed tree order (column bits 1 (fma), 2, 3, 0, 6, 5, 4), shifted log2 LSE
    if (PRO) {
      float o[NE];
#pragma unroll
      for (int j = 0; j < NJ; ++j) to_f32(o_raw[j], o + 8 * j);
      float v[4 * NJ];                               // columns with bit 1 clear: index (j, e bit 2, e bit 0)
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        // the chunk's eight codes back as floats: the hardware conversion E4M3 -> f16 is exact (two codes per instruction)
        float c8[8];
#pragma unroll
        for (int hw = 0; hw < 4; ++hw) {
          const float2 f = e4m3x2_to_f32((uint16_t)(cw[2 * j + (hw >> 1)] >> (16 * (hw & 1))));
          c8[2 * hw] = f.x;
          c8[2 * hw + 1] = f.y;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int e = ((k >> 1) << 2) | (k & 1);   // 0, 1, 4, 5
          const float a0 = __fmul_rn(c8[e], scale);
          const float a2 = __fmul_rn(c8[e + 2], scale);
          v[4 * j + k] = __fmaf_rn(a0, o[8 * j + e], __fmul_rn(a2, o[8 * j + e + 2]));
        }
      }
#pragma unroll
      for (int j = 0; j < NJ; ++j) {                 // bit 2
        v[4 * j + 0] = __fadd_rn(v[4 * j + 0], v[4 * j + 2]);
        v[4 * j + 1] = __fadd_rn(v[4 * j + 1], v[4 * j + 3]);
      }
#pragma unroll
      for (int j = 0; j < NJ; ++j) {                 // bit 3 = lane bit 0
        v[4 * j + 0] = __fadd_rn(v[4 * j + 0], __shfl_xor_sync(0xFFFFFFFFu, v[4 * j + 0], 1));
        v[4 * j + 1] = __fadd_rn(v[4 * j + 1], __shfl_xor_sync(0xFFFFFFFFu, v[4 * j + 1], 1));
      }
      float w4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) w4[j] = j < NJ ? __fadd_rn(v[4 * (j < NJ ? j : 0) + 0], v[4 * (j < NJ ? j : 0) + 1]) : 0.f;   // bit 0
      const float w2a = __fadd_rn(w4[0], w4[2]), w2b = __fadd_rn(w4[1], w4[3]);                  // bit 6
      float w1 = __fadd_rn(w2a, w2b);                                                            // bit 5
      w1 = __fadd_rn(w1, __shfl_xor_sync(0xFFFFFFFFu, w1, 2));                                   // bit 4 = lane bit 1
      if (q == 0 && p.d_out) p.d_out[ri] = __fmul_rn(w1, p.d_multiplier);
    }
    if (p.lse && p.lse_log2 && q == 0) {
      const float l = p.lse[ri];
      p.lse_log2[ri] = __fsub_rn((l == -INFINITY) ? 0.f : __fmul_rn(l, 1.4426950408889634f), p.lse_shift);
    }

    // ---- side tables
    const uint32_t b0 = ue8m0_byte(fmaxf(fmaxf(wm[0], wm[1]), fmaxf(wm[2], wm[3])));
    const uint32_t b1 = ue8m0_byte(fmaxf(fmaxf(wm[4], wm[5]), fmaxf(wm[6], wm[7])));
    const uint32_t b2 = ue8m0_byte(fmaxf(fmaxf(wm[8], wm[9]), fmaxf(wm[10], wm[11])));
    const uint32_t b3 = ue8m0_byte(fmaxf(fmaxf(wm[12], wm[13]), fmaxf(wm[14], wm[15])));
    if ((tid & 127) == 0) {                          // one thread per 32-token block (tid 128 k: row 32 k, lane 0 of it)
      if (p.e_tab) {
        uint8_t* e = p.e_tab + (bh * (p.s / 32) + tile * 4 + blk) * (D / 32);
#pragma unroll
        for (int g = 0; g < D / 32; ++g) e[g] = (uint8_t)bbyte;
      }
      if (p.fac) {
        const uint32_t tm = max(max(b0, b1), max(b2, b3));
        const uint32_t e0 = bbyte ? bbyte : tm;
        p.fac[bh * (p.s / 32) + tile * 4 + blk] = e0 ? pow2_from_field((int)e0) : 1.0f;
      }
    }
    if (q == 0) {
      if (p.token_factors) p.token_factors[ri] = tbyte ? scale : 1.0f;
      if (p.sf_tok)
        *reinterpret_cast<uint32_t*>(p.sf_tok + (bh * ntile + tile) * 512 + (r & 31) * 16 + (r >> 5) * 4) = tbyte * 0x01010101u;
    }
    if (p.sf_dim && tid < 128)
      *reinterpret_cast<uint32_t*>(p.sf_dim + (bh * ntile + tile) * 512 + tid * 4) = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
    if (p.tile_stats && tid == 0) {
      float a = 0.f, sq = 0.f;
#pragma unroll
      for (int w = 0; w < 16; ++w) { a = fmaxf(a, wm[w]); sq = fmaxf(sq, s_wsq[par][w]); }
      p.tile_stats[(bh * ntile + tile) * 2] = a;
      p.tile_stats[(bh * ntile + tile) * 2 + 1] = sq;
    }

    // ---- channel-major copy (b, h, d, s): through shared memory, thread c gathers column c
    if (p.codes_t) {
      constexpr int CROWB = D + 16;
#pragma unroll
      for (int j = 0; j < NJ; ++j)
        *reinterpret_cast<uint2*>(s_codes + r * CROWB + (4 * j + q) * 8) = make_uint2(cw[2 * j], cw[2 * j + 1]);
      __syncthreads();
      for (int i = tid; i < D * 8; i += QTHREADS) {  // (channel, 16-token group)
        const int c = i >> 3, rg = (i & 7) * 16;
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          w[k] = (uint32_t)s_codes[(rg + 4 * k) * CROWB + c] | ((uint32_t)s_codes[(rg + 4 * k + 1) * CROWB + c] << 8) |
                 ((uint32_t)s_codes[(rg + 4 * k + 2) * CROWB + c] << 16) | ((uint32_t)s_codes[(rg + 4 * k + 3) * CROWB + c] << 24);
        *reinterpret_cast<uint4*>(p.codes_t + (bh * D + c) * (size_t)p.s + t0 + rg) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      __syncthreads();                               // the staging rows are rewritten by the next tile
    }
  }
  // a CTA that gave up must not exit while loads into its shared memory may still land
  if (abort_s) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

// ------------------------------------------------------------------------------------------------ one thread per row
// The plain launches at head_dim 128 (and, unrotated, 64) (codes, exponent / factor tables, statistics; no
// prologue, no token-local exponents, no packed source) run with ONE THREAD PER TOKEN ROW: CTA = 128 threads = one
// 128-token tile, warp = one 32-token block, so the block maximum is a warp reduction, the Hadamard butterflies need no
// shuffles, and one barrier per tile remains (it hands the input stage back to the loader and the codes to a TMA store).
// Every floating-point operation is the one the four-lanes-per-row kernel above performs on the same operands in the same
// order, so the two kernels' outputs are bit-identical (tests/test_gpu_quant.py compares them).
static constexpr int QR_STAGES = 2;

// MODE as in the four-lane kernel: bit 0 = the E4M3 codes are of the rotated row, bit 1 = also the NVFP4 copy, bit 2 =
// rotate only the NVFP4 copy.
template <int MODE, int D = 128>
__global__ void __launch_bounds__(128, 2)
quant_rows_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_c, const QuantParams p) {
  static_assert(D == 128 || (D == 64 && MODE == 0), "head_dim 64 has no rotation and no NVFP4 copy");
  constexpr int QR_TILE_B = QT * D * 2;            // one 16-bit input tile (boxes of 64 columns: 128-byte rows)
  constexpr int QR_CODE_B = QT * D;                // its codes (rows of D bytes, the swizzle of that width)
  constexpr bool ROT = (MODE & 1) != 0, NV4 = (MODE & 2) != 0, ROT4 = (MODE & 4) != 0;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_out = smem + QR_STAGES * QR_TILE_B;   // two code tiles (128 rows x 128 B, 128 B swizzle)
  __shared__ __align__(8) uint64_t full[QR_STAGES];
  __shared__ float s_wmax[2][4], s_wsq[2][4];
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = tid;                               // token row of the tile
  const int G = gridDim.x;
  const int ntile = p.s / QT;
  volatile int* abortp = &abort_s;

  auto issue = [&](int L, int st) {
    const int head = L % p.h, tile = (L / p.h) % ntile, bat = L / (p.h * ntile);
    uint8_t* dst = smem + st * QR_TILE_B;
    mbar_arrive_expect_tx(&full[st], QR_TILE_B);
    tma_load_4d(dst, &tm_x, &full[st], 0, head, tile * QT, bat);
    if (D == 128) tma_load_4d(dst + QR_TILE_B / 2, &tm_x, &full[st], 64, head, tile * QT, bat);
  };
  if (tid == 0) {
    abort_s = 0;
    for (int i = 0; i < QR_STAGES; ++i) mbar_init(&full[i], 1);
    fence_barrier_init();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_c);
    for (int i = 0; i < QR_STAGES; ++i)
      if (blockIdx.x + i * G < p.n_tiles) issue(blockIdx.x + i * G, i);
  }
  __syncthreads();

  int it = 0;
  for (int L = blockIdx.x; L < p.n_tiles; L += G, ++it) {
    const int st = it % QR_STAGES, par = it & 1;
    const int head = L % p.h, tile = (L / p.h) % ntile, bat = L / (p.h * ntile);
    const int t0 = tile * QT;
    const size_t bh = (size_t)bat * p.h + head;
    const uint32_t tile_addr = smem_u32(smem + st * QR_TILE_B);
    bool ok = mbar_wait(&full[st], (it / QR_STAGES) & 1, p.ctl, abortp, 51);

    // ---- the row: D / 8 chunks of 8 elements (element 8 g + e in chunk g), rotation signs applied to the raw bits
    float x[D];
    auto load_row = [&](bool signs) {
      constexpr uint32_t NEG[4] = {0x10D2E03Eu, 0xE0D9F0E2u, 0x45809F07u, 0x75954FEDu};
#pragma unroll
      for (int g = 0; g < D / 8; ++g) {
        const uint32_t box = (uint32_t)(g >> 3) * (QR_TILE_B / 2);
        uint4 v = lds_u4(tile_addr + box + r * 128 + (((g & 7) ^ (r & 7)) << 4));
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (signs) {
            const int i0 = 8 * g + 2 * k, i1 = i0 + 1;
            const uint32_t m = (((NEG[i0 >> 5] >> (i0 & 31)) & 1u) << 15) | (((NEG[i1 >> 5] >> (i1 & 31)) & 1u) << 31);
            w[k] ^= m;
          }
          if (p.in_f16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
            x[8 * g + 2 * k] = f.x;
            x[8 * g + 2 * k + 1] = f.y;
          } else {
            x[8 * g + 2 * k] = __uint_as_float(w[k] << 16);
            x[8 * g + 2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
          }
        }
      }
    };
    // (y * signs) H_128 / sqrt(128): butterfly levels 1, 2, ..., 64 with (a, b) -> (a + b, a - b), the last one with the
    // scaling, subnormal results flushed
    auto rotate_row = [&]() {
      if constexpr (D == 128) {
      uint64_t Y[D / 2];
#pragma unroll
      for (int k = 0; k < D / 2; ++k) Y[k] = pack2(__fadd_rn(x[2 * k], x[2 * k + 1]), __fsub_rn(x[2 * k], x[2 * k + 1]));
#pragma unroll
      for (int hs = 1; hs < D / 4; hs <<= 1) {
#pragma unroll
        for (int k = 0; k < D / 2; ++k)
          if ((k & hs) == 0) {
            const uint64_t a = Y[k], b2 = Y[k + hs];
            Y[k] = add2(a, b2);
            Y[k + hs] = sub2(a, b2);
          }
      }
      const uint64_t c2 = pack2(0.08838834764831845f, 0.08838834764831845f);
#pragma unroll
      for (int k = 0; k < D / 4; ++k) {
        const uint64_t a = Y[k], b2 = Y[k + D / 4];
        unpack2(mul2_ftz(add2(a, b2), c2), x[2 * k], x[2 * k + 1]);
        unpack2(mul2_ftz(sub2(a, b2), c2), x[2 * k + D / 2], x[2 * k + D / 2 + 1]);
      }
      }
    };
    // NVFP4 copy of x: per 16 along d: SF = E4M3_rn(amax * f32(1/6)); codes = E2M1_rn(ftz(x * m)), m = 1 / SF | +inf (SF
    // rounds to 0, amax > 0) | 0. Scale bytes: group g of the row = byte g % 4 of the row's word in atom g / 4.
    auto nvfp4_row = [&]() {
      const size_t row_off = (((size_t)bat * p.s + t0 + r) * p.h + head) * D;
      uint8_t* x4row = p.x4 + row_off / 2;
      uint32_t sfw[2] = {0u, 0u};
#pragma unroll
      for (int g2 = 0; g2 < D / 32; ++g2) {           // two groups of 16 elements = one 16-byte store
        uint32_t pk[4];
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {
          const int g = 2 * g2 + gg;
          // the largest flushed magnitude = the flushed largest magnitude (flushing is monotone; a NaN never wins a max)
          float am = 0.f;
#pragma unroll
          for (int e = 0; e < 16; e += 2) am = fmax3_abs(am, x[16 * g + e], x[16 * g + e + 1]);
          am = flush_sub(am);
          const float u = __fmul_rn(am, 1.0f / 6.0f);
          const uint32_t sfb = cvt_e4m3x2(u, 0.f) & 0xFF;
          const float sfv = e4m3x2_to_f32((uint16_t)sfb).x;
          const float m = sfv > 0.f ? __frcp_rn(sfv) : (u > 0.f ? __int_as_float(0x7F800000) : 0.f);
          const uint64_t m2 = pack2(m, m);
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {            // eight elements -> one word, low nibble first
            float a[8];
#pragma unroll
            for (int k = 0; k < 4; ++k)               // the product with subnormal inputs and results flushed, two at a time
              unpack2(mul2_ftz(pack2(x[16 * g + 8 * hh + 2 * k], x[16 * g + 8 * hh + 2 * k + 1]), m2), a[2 * k], a[2 * k + 1]);
            uint32_t w;
            asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
                "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\tcvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
                "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\tcvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
                "mov.b32 %0, {t0, t1, t2, t3};\n\t}"
                : "=r"(w)
                : "f"(a[0]), "f"(a[1]), "f"(a[2]), "f"(a[3]), "f"(a[4]), "f"(a[5]), "f"(a[6]), "f"(a[7]));
            pk[2 * gg + hh] = w;
          }
          sfw[g >> 2] |= sfb << (8 * (g & 3));
        }
        *reinterpret_cast<uint4*>(x4row + g2 * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      if (p.sf4) {
        uint8_t* atom = p.sf4 + ((bh * ntile + tile) * (D / 64)) * 512;
#pragma unroll
        for (int a = 0; a < D / 64; ++a) *reinterpret_cast<uint32_t*>(atom + a * 512 + (r & 31) * 16 + (r >> 5) * 4) = sfw[a];
      }
    };
    if (ROT4) {          // NVFP4 codes of the rotated row, E4M3 codes of the row as read
      load_row(true);
      rotate_row();
      nvfp4_row();
      load_row(false);
    } else if (ROT) {
      load_row(true);
      rotate_row();
      if (NV4) nvfp4_row();
    } else {
      load_row(false);
      if (NV4) nvfp4_row();
    }
    if (!ROT || ROT4) {  // subnormal -> zero of the same sign (rotated rows were flushed by their scaling)
#pragma unroll
      for (int i = 0; i < D; i += 2) unpack2(mul2_ftz(pack2(x[i], x[i + 1]), pack2(1.0f, 1.0f)), x[i], x[i + 1]);
    }

    // ---- the row's maximum and (with the statistics) its sum of squares, in the four-lane kernel's summation order
    float amax = 0.f, sumsq = 0.f;
    {
      float aq[4] = {0.f, 0.f, 0.f, 0.f};          // per quarter q: elements 32 j + 8 q + e
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < D / 32; ++j)
#pragma unroll
          for (int e = 0; e < 8; e += 2)
            aq[q] = fmax3_abs(aq[q], x[32 * j + 8 * q + e], x[32 * j + 8 * q + e + 1]);
      amax = fmaxf(fmaxf(aq[0], aq[1]), fmaxf(aq[2], aq[3]));
      if (p.tile_stats || p.row_stat) {
        float lq[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int j = 0; j < D / 32; ++j)
#pragma unroll
            for (int e = 0; e < 8; ++e) sq[e & 3] = fmaf(x[32 * j + 8 * q + e], x[32 * j + 8 * q + e], sq[e & 3]);
          lq[q] = (sq[0] + sq[1]) + (sq[2] + sq[3]);
        }
        sumsq = (lq[0] + lq[1]) + (lq[2] + lq[3]);
      }
    }
    if (p.row_stat) {
      const float v = p.row_stat_kind == 2 ? amax : (p.row_stat_kind == 3 ? __fsqrt_rn(sumsq) : sumsq);
      atomicMax(p.row_stat + (size_t)bat * p.s + t0 + r, __float_as_uint(v));
    }
    // the 32-token block = this warp (non-negative floats order as their bit patterns)
    uint32_t bm_bits, bs_bits;
    asm volatile("redux.sync.max.u32 %0, %1, 0xffffffff;" : "=r"(bm_bits) : "r"(__float_as_uint(amax)));
    // (a row whose sum of squares is NaN does not take part, as with the NaN-ignoring maximum of the four-lane kernel)
    asm volatile("redux.sync.max.u32 %0, %1, 0xffffffff;" : "=r"(bs_bits) : "r"(sumsq == sumsq ? __float_as_uint(sumsq) : 0u));
    const float bmax = __uint_as_float(bm_bits);
    if (lane == 0) { s_wmax[par][warp] = bmax; s_wsq[par][warp] = __uint_as_float(bs_bits); }
    const uint32_t bbyte = ue8m0_byte(bmax);
    const float inv = bbyte ? pow2_from_field(254 - (int)bbyte) : 0.f;

    // ---- codes -> this tile's staging buffer (rows of D bytes, the swizzle of that width)
    {
      const uint64_t inv2 = pack2(inv, inv);
      const uint32_t orow = smem_u32(s_out + par * QR_CODE_B) + r * D;
      const int swz = D == 128 ? (r & 7) : ((r >> 1) & 3);
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {            // 16 codes per 16-byte chunk
        uint32_t cw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float a0, a1, a2, a3;
          unpack2(mul2(pack2(x[16 * c + 4 * k], x[16 * c + 4 * k + 1]), inv2), a0, a1);
          unpack2(mul2(pack2(x[16 * c + 4 * k + 2], x[16 * c + 4 * k + 3]), inv2), a2, a3);
          cw[k] = cvt_e4m3x4(a0, a1, a2, a3);
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(orow + ((c ^ swz) << 4)), "r"(cw[0]), "r"(cw[1]),
                     "r"(cw[2]), "r"(cw[3]) : "memory");
      }
    }
    fence_proxy_async();
    // the store of the previous tile has read its staging buffer (the other one): the next tile may write it
    if (tid == 0) tma_store_wait_read<0>();
    // every thread has read the stage and written its codes; a wait that ran out leaves the loop here, all threads together
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (!ok) break;
    if (tid == 0) {
      if (L + QR_STAGES * G < p.n_tiles) issue(L + QR_STAGES * G, st);
      tma_store_4d(&tm_c, s_out + par * QR_CODE_B, 0, head, t0, bat);
      tma_store_commit();
    }
    // ---- side tables
    const float* wm = s_wmax[par];
    if (lane == 0) {
      const uint32_t b0 = ue8m0_byte(wm[0]), b1 = ue8m0_byte(wm[1]), b2 = ue8m0_byte(wm[2]), b3 = ue8m0_byte(wm[3]);
      if (p.e_tab) {
        uint8_t* e = p.e_tab + (bh * (p.s / 32) + tile * 4 + warp) * (D / 32);
#pragma unroll
        for (int g = 0; g < D / 32; ++g) e[g] = (uint8_t)bbyte;
      }
      if (p.fac) {
        const uint32_t tm = max(max(b0, b1), max(b2, b3));
        const uint32_t e0 = bbyte ? bbyte : tm;
        p.fac[bh * (p.s / 32) + tile * 4 + warp] = e0 ? pow2_from_field((int)e0) : 1.0f;
      }
    }
    if (p.tile_stats && tid == 0) {
      p.tile_stats[(bh * ntile + tile) * 2] = fmaxf(fmaxf(wm[0], wm[1]), fmaxf(wm[2], wm[3]));
      p.tile_stats[(bh * ntile + tile) * 2 + 1] = fmaxf(fmaxf(s_wsq[par][0], s_wsq[par][1]), fmaxf(s_wsq[par][2], s_wsq[par][3]));
    }
  }
  // the staging buffers must outlive the stores that read them; a CTA that gave up must not exit while loads may still land
  if (tid == 0) tma_store_wait_read<0>();
  if (abort_s) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

template <int MODE, int D = 128>
static int launch_quant_rows(const CUtensorMap& mx, const CUtensorMap& mc, const QuantParams& p, cudaStream_t st) {
  const int smem = QR_STAGES * QT * D * 2 + 2 * QT * D + 1024;
  auto kern = quant_rows_kernel<MODE, D>;
  if (cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); e != cudaSuccess)
    return cuda_fail((int)e, "fl_quant_blocks: cudaFuncSetAttribute");
  const int grid = min(p.n_tiles, sm_count() * 2);
  kern<<<grid, 128, smem, st>>>(mx, mc, p);
  return FL_OK;
}

template <int D, int MODE, bool PRO, bool PK>
static int launch_quant_pk(const CUtensorMap& mx, const CUtensorMap& mo, const QuantParams& p, bool want_t, cudaStream_t st) {
  constexpr int TILE_B = QT * D * 2;
  const int smem = QSTAGES * (PRO ? 2 : 1) * TILE_B + 1024 + (want_t ? QT * (D + 16) : 0);
  auto kern = quant_blocks_kernel<D, MODE, PRO, PK>;
  if (cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); e != cudaSuccess)
      return cuda_fail((int)e, "fl_quant_blocks: cudaFuncSetAttribute");
  const int per_sm = (PRO || want_t) ? 1 : 2;
  const int grid = min(p.n_tiles, sm_count() * per_sm);
  kern<<<grid, QTHREADS, smem, st>>>(mx, mo, p);
  return FL_OK;
}

template <int D, int MODE, bool PRO>
static int launch_quant(const CUtensorMap& mx, const CUtensorMap& mo, const QuantParams& p, bool want_t, cudaStream_t st) {
  return p.slot_src ? launch_quant_pk<D, MODE, PRO, true>(mx, mo, p, want_t, st)
                    : launch_quant_pk<D, MODE, PRO, false>(mx, mo, p, want_t, st);
}

}  // namespace fl

extern "C" int fl_quant_blocks(const fl_quant_args* a, void* stream) {
  using namespace fl;
  if (!a || !a->x || !a->codes) return FL_ERR_BAD_ARG;
  if (a->b <= 0 || a->s <= 0 || a->h <= 0 || (a->s % 128) != 0) return FL_ERR_BAD_ARG;
  if (a->d != 64 && a->d != 128) return FL_ERR_UNSUPPORTED;
  if ((a->flags & (FL_Q_HADAMARD | FL_Q_HADAMARD_NVFP4_ONLY)) && a->d != 128) return FL_ERR_UNSUPPORTED;
  if ((a->flags & FL_Q_HADAMARD) && (a->flags & FL_Q_TOKEN_LOCAL)) return FL_ERR_UNSUPPORTED;
  if ((a->flags & FL_Q_HADAMARD_NVFP4_ONLY) && !a->x4) return FL_ERR_BAD_ARG;
  if (a->h > 65535 || a->b > 65535) return FL_ERR_TOO_LARGE;
  const long long n_tiles = (long long)a->b * (a->s / 128) * a->h;
  if (n_tiles > 0x7FFFFFFF) return FL_ERR_TOO_LARGE;
  const bool pro = a->d_out != nullptr && a->o != nullptr;
  const bool rot = (a->flags & FL_Q_HADAMARD) != 0, rot4 = (a->flags & FL_Q_HADAMARD_NVFP4_ONLY) != 0;
  const bool nv4 = a->x4 != nullptr;
  if (pro && (rot || rot4 || nv4)) return FL_ERR_UNSUPPORTED;     // the prologue rides on the dO launch, which does neither
  QuantParams p;
  p.lse = a->lse; p.codes = a->codes; p.codes_t = a->codes_t; p.e_tab = a->e_tab; p.fac = a->fac; p.sf_tok = a->sf_tok;
  p.sf_dim = a->sf_dim; p.token_factors = a->token_factors; p.x4 = a->x4; p.sf4 = a->sf4; p.d_out = a->d_out;
  p.lse_log2 = a->lse_log2; p.zero_acc = (uint16_t*)a->zero_acc; p.tile_stats = a->tile_stats;
  p.row_stat = (uint32_t*)a->row_stat; p.row_stat_kind = a->row_stat_kind;
  if (a->row_stat && (a->row_stat_kind < 1 || a->row_stat_kind > 3)) return FL_ERR_BAD_ARG;
  p.b = a->b; p.s = a->s; p.h = a->h; p.n_tiles = (int)n_tiles;
  p.slot_src = a->slot_src; p.slot_rows = a->slot_rows;
  const bool packed = a->slot_src != nullptr;
  if (packed && (!a->slot_rows || a->b != 1 || a->src_rows <= 0)) return FL_ERR_BAD_ARG;
  p.token_local = (a->flags & FL_Q_TOKEN_LOCAL) ? 1 : 0;
  p.in_f16 = a->in_f16;
  p.lse_shift = a->lse_shift; p.d_multiplier = a->d_multiplier;
  p.ctl.status = a->status;
  p.ctl.wait_cycles = a->wait_cycles > 0 ? a->wait_cycles : kDefaultWaitCycles;
  CUtensorMap mx, mo;
  int rc;
  if ((rc = make_rows_map_16(&mx, a->x, a->b, packed ? a->src_rows : a->s, a->h, a->d, 128))) return rc;
  p.o_packed = (packed && (a->flags & FL_Q_O_PACKED)) ? 1 : 0;
  if ((rc = make_rows_map_16(&mo, pro ? a->o : a->x, a->b, p.o_packed ? a->src_rows : a->s, a->h, a->d, 128))) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const bool wt = a->codes_t != nullptr;
  // the plain launches of the 8-bit route: one thread per row (same bits, fewer instructions, no shuffles)
  if ((a->d == 128 || (a->d == 64 && !rot && !rot4 && !nv4)) && !pro && !wt && !packed && !p.token_local && !a->sf_tok &&
      !a->sf_dim && !a->token_factors && !a->zero_acc && !a->lse_log2 && !(a->flags & FL_Q_LEGACY)) {
    CUtensorMap mc;
    if ((rc = make_rows_map(&mc, a->codes, a->b, a->s, a->h, a->d, 128))) return rc;
    if (a->d == 64) rc = launch_quant_rows<0, 64>(mx, mc, p, st);
    else if (rot4) rc = launch_quant_rows<6>(mx, mc, p, st);
    else if (rot) rc = nv4 ? launch_quant_rows<3>(mx, mc, p, st) : launch_quant_rows<1>(mx, mc, p, st);
    else rc = nv4 ? launch_quant_rows<2>(mx, mc, p, st) : launch_quant_rows<0>(mx, mc, p, st);
    if (rc) return rc;
    return launch_result("fl_quant_blocks: kernel launch");
  }
  if (a->d == 64) {
    if (pro) rc = launch_quant<64, 0, true>(mx, mo, p, wt, st);
    else rc = nv4 ? launch_quant<64, 2, false>(mx, mo, p, wt, st) : launch_quant<64, 0, false>(mx, mo, p, wt, st);
  } else if (pro) {
    rc = launch_quant<128, 0, true>(mx, mo, p, wt, st);
  } else if (rot4) {
    rc = launch_quant<128, 6, false>(mx, mo, p, wt, st);
  } else if (rot) {
    rc = nv4 ? launch_quant<128, 3, false>(mx, mo, p, wt, st) : launch_quant<128, 1, false>(mx, mo, p, wt, st);
  } else {
    rc = nv4 ? launch_quant<128, 2, false>(mx, mo, p, wt, st) : launch_quant<128, 0, false>(mx, mo, p, wt, st);
  }
  if (rc) return rc;
  return launch_result("fl_quant_blocks: kernel launch");
}
