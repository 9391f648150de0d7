// Fused block-scaled quantiser (token-block MXFP8, optional NVFP4 S-operand copy, optional Hadamard rotation) and the
// fused backward prologue (D = rowsum(O * dequant(dO)), shifted log2 LSE, zeroed f16 dQ accumulator).
//
// Replaces the reference's quantize_fp8_blocks launch (flash_attn/cute/quant/fp8.py:2512, kernel_stream :1639) and the
// fused NVFP4 copy (flash_attn/cute/quant/_fp8_nvfp4.py:121-158). Outputs are byte-identical to the reference's eager
// definitions (tests/cute/quant_reference.py:714-798, 270-369).
//
// One CTA (512 threads) per (128-token tile, head, batch). Four lanes share a token row: lane q of the row holds the
// 16-byte chunks c = 4 j + q (8 elements each), so every global access of a row is 64 contiguous bytes per instruction
// and no staging through shared memory is needed. Element index i = 32 j + 8 q + e: the Hadamard levels 1, 2, 4 and
// 32, 64 are in-thread, levels 8, 16 are two lane exchanges; the same order of operations as the one-thread-per-row
// butterfly, hence the same bits. The kernel is HBM-bound (2 B read + 1 B written per element, plus optional copies).
#include "flamia_internal.h"

namespace fl {

static constexpr int QT = 128;       // tokens per tile
static constexpr int QTHREADS = 512; // four lanes per token

struct QuantParams {
  const uint16_t* x;
  const uint16_t* o;      // prologue: forward output (same layout as x) or null
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
  int b, s, h, d;
  int flags;
  int in_f16;
  float lse_shift, d_multiplier;
};

__device__ __forceinline__ float in_to_f32(uint32_t v16, int f16) {
  return f16 ? __half2float(__ushort_as_half((uint16_t)v16)) : __uint_as_float(v16 << 16);
}
__device__ __forceinline__ float flush_sub(float v) { return fabsf(v) < 1.17549435e-38f ? v * 0.0f : v; }
// a * b rounded to nearest with subnormal inputs and results flushed to zero (the product and its flush in one instruction)
__device__ __forceinline__ float mul_ftz(float a, float b) {
  float r;
  asm("mul.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
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

__device__ __forceinline__ float e4m3_byte_to_f32(uint32_t c) {
  uint32_t e = (c >> 3) & 0xF, m = c & 7;
  float v = e ? __uint_as_float(((e + 120) << 23) | (m << 20)) : (float)m * 0.001953125f;
  return (c & 0x80) ? -v : v;
}

template <int D>
__global__ void __launch_bounds__(QTHREADS) quant_blocks_kernel(const QuantParams p) {
  constexpr int NJ = D / 32;                     // 16-byte chunks per lane
  constexpr int NE = 8 * NJ;                     // elements per lane
  __shared__ float s_wmax[16];                   // per-warp (8 rows) maximum
  __shared__ float s_wsq[16];                    // per-warp maximum row sum of squares
  __shared__ __align__(16) uint8_t s_codes[QT * (D + 16)];   // channel-major copy only

  const int tile = blockIdx.x, head = blockIdx.y, bat = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = tid >> 2, q = tid & 3;           // token row of the tile, lane of the row
  const int t0 = tile * QT;
  const size_t row_stride = (size_t)p.h * D;     // elements between consecutive tokens
  const size_t row_off = ((size_t)bat * p.s + t0 + r) * row_stride + (size_t)head * D;
  const bool prologue = p.d_out != nullptr && p.o != nullptr;

  float x[NE];
  auto load_row = [&](const uint16_t* base, float* dst) {
    const uint4* src = reinterpret_cast<const uint4*>(base + row_off) + q;
    uint4 v[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) v[j] = src[4 * j];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        dst[8 * j + 2 * k] = in_to_f32(w[k] & 0xFFFF, p.in_f16);
        dst[8 * j + 2 * k + 1] = in_to_f32(w[k] >> 16, p.in_f16);
      }
    }
  };
  load_row(p.x, x);
  if (p.zero_acc) {   // this tile's share of the accumulator: 128 * D f16 = 32 D 16-byte chunks, contiguous
    uint4* z = reinterpret_cast<uint4*>(p.zero_acc + (((size_t)bat * p.h + head) * p.s + t0) * D);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int i = tid; i < QT * D / 8; i += QTHREADS) z[i] = zero;
  }

  const bool rotate = (p.flags & (FL_Q_HADAMARD | FL_Q_HADAMARD_NVFP4_ONLY)) != 0;
  const bool rot_only4 = (p.flags & FL_Q_HADAMARD_NVFP4_ONLY) != 0;
  const bool want4 = p.x4 != nullptr;

  // (y * signs) H_128 / sqrt(128): butterfly levels 1, 2, ..., 64 with (a, b) -> (a + b, a - b)
  auto rotate_row = [&](float* y) {
    if constexpr (D == 128) {
      constexpr uint32_t NEG[4] = {0x10D2E03Eu, 0xE0D9F0E2u, 0x45809F07u, 0x75954FEDu};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t m = NEG[j] >> (8 * q);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if ((m >> e) & 1) y[8 * j + e] = -y[8 * j + e];
      }
#pragma unroll
      for (int hs = 1; hs < 8; hs <<= 1) {       // element bits 0..2: inside one chunk
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if ((i & hs) == 0) {
            const float a = y[i], b2 = y[i + hs];
            y[i] = __fadd_rn(a, b2);
            y[i + hs] = __fsub_rn(a, b2);
          }
      }
#pragma unroll
      for (int lb = 1; lb < 4; lb <<= 1) {       // element bits 3, 4 = the lane of the row
        // low lane: y + other; high lane: other - y. Both are other + (+-1) y: one fma (the product is exact)
        const float sg = (q & lb) ? -1.0f : 1.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float other = __shfl_xor_sync(0xFFFFFFFFu, y[i], lb);
          y[i] = __fmaf_rn(y[i], sg, other);
        }
      }
#pragma unroll
      for (int jb = 1; jb < 4; jb <<= 1) {       // element bits 5, 6 = the chunk index j
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (((i >> 3) & jb) == 0) {
            const float a = y[i], b2 = y[i + 8 * jb];
            y[i] = __fadd_rn(a, b2);
            y[i + 8 * jb] = __fsub_rn(a, b2);
          }
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) y[i] = mul_ftz(y[i], 0.08838834764831845f);   // scaled and flushed
    }
  };

  // NVFP4 copy of y: per 16 along d (two neighbouring lanes): SF = E4M3_rn(amax * f32(1/6)); codes = E2M1_rn(ftz(y * m)),
  // m = 1 / SF | +inf (SF rounds to 0, amax > 0) | 0
  auto nvfp4_row = [&](const float* y) {
    uint32_t sfpack = 0;                         // this lane's scale bytes: chunk j in byte j
    uint8_t* x4row = p.x4 + (((size_t)bat * p.s + t0 + r) * p.h + head) * (D / 2);
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
      const float sfv = e4m3_byte_to_f32(sfb);
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
      uint8_t* atom = p.sf4 + ((((size_t)bat * p.h + head) * (p.s / QT) + tile) * (D / 64)) * 512;
#pragma unroll
      for (int a = 0; a < D / 64; ++a) {
        const uint32_t lo0 = (sfpack >> (16 * a)) & 0xFF, lo1 = (sfpack >> (16 * a + 8)) & 0xFF;
        const uint32_t hi0 = (hi >> (16 * a)) & 0xFF, hi1 = (hi >> (16 * a + 8)) & 0xFF;
        *reinterpret_cast<uint32_t*>(atom + a * 512 + (r & 31) * 16 + (r >> 5) * 4) = lo0 | (hi0 << 8) | (lo1 << 16) | (hi1 << 24);
      }
    }
  };

  if (want4 && rotate && rot_only4) {   // NVFP4 codes of the rotated row, E4M3 codes of the row as read
    rotate_row(x);
    nvfp4_row(x);
    load_row(p.x, x);
  } else if (rotate) {
    rotate_row(x);
  }
  if (want4 && !(rotate && rot_only4)) nvfp4_row(x);

  // ---- exponents: per token (4 lanes) and per 32-token block (4 warps)
  float amax = 0.f, sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < NE; ++i) {
    x[i] = mul_ftz(x[i], 1.0f);      // subnormal -> zero of the same sign (rotated rows were flushed by their scaling)
    amax = fmaxf(amax, fabsf(x[i]));
  }
  if (p.tile_stats) {     // the row norm is only wanted with the tile statistics (K, V, dO)
#pragma unroll
    for (int i = 0; i < NE; ++i) sumsq = fmaf(x[i], x[i], sumsq);
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));      // the token's maximum
  sumsq += __shfl_xor_sync(0xFFFFFFFFu, sumsq, 1);
  sumsq += __shfl_xor_sync(0xFFFFFFFFu, sumsq, 2);
  float wmax = amax, wsq = sumsq;
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    wmax = fmaxf(wmax, __shfl_xor_sync(0xFFFFFFFFu, wmax, o));
    wsq = fmaxf(wsq, __shfl_xor_sync(0xFFFFFFFFu, wsq, o));
  }
  if (lane == 0) { s_wmax[warp] = wmax; s_wsq[warp] = wsq; }
  __syncthreads();
  const int blk = r >> 5;                                         // 32-token block of the tile
  const float bmax = fmaxf(fmaxf(s_wmax[4 * blk], s_wmax[4 * blk + 1]), fmaxf(s_wmax[4 * blk + 2], s_wmax[4 * blk + 3]));
  const uint32_t bbyte = ue8m0_byte(bmax);
  const bool tl = (p.flags & FL_Q_TOKEN_LOCAL) != 0;
  const uint32_t tbyte = tl ? ue8m0_byte(amax) : bbyte;
  const float inv = tbyte ? pow2_from_field(254 - (int)tbyte) : 0.f;
  const float scale = tbyte ? pow2_from_field((int)tbyte) : 0.f;

  uint32_t cw[2 * NJ];
#pragma unroll
  for (int i = 0; i < 2 * NJ; ++i)
    cw[i] = cvt_e4m3x4(__fmul_rn(x[4 * i], inv), __fmul_rn(x[4 * i + 1], inv), __fmul_rn(x[4 * i + 2], inv),
                       __fmul_rn(x[4 * i + 3], inv));
  {
    uint8_t* crow = p.codes + row_off;
#pragma unroll
    for (int j = 0; j < NJ; ++j)
      *reinterpret_cast<uint2*>(crow + (4 * j + q) * 8) = make_uint2(cw[2 * j], cw[2 * j + 1]);
  }

  const size_t bh = (size_t)bat * p.h + head;
  const size_t ri = bh * p.s + t0 + r;
  // ---- prologue: D in the fixed tree order (column bits 1 (fma), 2, 3, 0, 6, 5, 4), shifted log2 LSE
  if (prologue) {
    float o[NE];
    load_row(p.o, o);
    float v[4 * NJ];                               // columns with bit 1 clear: index (j, e bit 2, e bit 0)
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int e = ((k >> 1) << 2) | (k & 1);   // 0, 1, 4, 5
        const float a0 = __fmul_rn(e4m3_byte_to_f32((cw[2 * j + (e >> 2)] >> (8 * (e & 3))) & 0xFF), scale);
        const float a2 = __fmul_rn(e4m3_byte_to_f32((cw[2 * j + ((e + 2) >> 2)] >> (8 * ((e + 2) & 3))) & 0xFF), scale);
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
    if (q == 0) p.d_out[ri] = __fmul_rn(w1, p.d_multiplier);
  }
  if (p.lse && p.lse_log2 && q == 0) {
    const float l = p.lse[ri];
    p.lse_log2[ri] = __fsub_rn((l == -INFINITY) ? 0.f : __fmul_rn(l, 1.4426950408889634f), p.lse_shift);
  }

  // ---- side tables
  const int ntile = p.s / QT;
  const uint32_t b0 = ue8m0_byte(fmaxf(fmaxf(s_wmax[0], s_wmax[1]), fmaxf(s_wmax[2], s_wmax[3])));
  const uint32_t b1 = ue8m0_byte(fmaxf(fmaxf(s_wmax[4], s_wmax[5]), fmaxf(s_wmax[6], s_wmax[7])));
  const uint32_t b2 = ue8m0_byte(fmaxf(fmaxf(s_wmax[8], s_wmax[9]), fmaxf(s_wmax[10], s_wmax[11])));
  const uint32_t b3 = ue8m0_byte(fmaxf(fmaxf(s_wmax[12], s_wmax[13]), fmaxf(s_wmax[14], s_wmax[15])));
  if ((tid & 127) == 0) {                          // one thread per 32-token block
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
    for (int w = 0; w < 16; ++w) { a = fmaxf(a, s_wmax[w]); sq = fmaxf(sq, s_wsq[w]); }
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
  }
}

}  // namespace fl

extern "C" int fl_quant_blocks(const fl_quant_args* a, void* stream) {
  using namespace fl;
  if (!a || !a->x || !a->codes) return FL_ERR_BAD_ARG;
  if (a->b <= 0 || a->s <= 0 || a->h <= 0 || (a->s % 128) != 0) return FL_ERR_BAD_ARG;
  if (a->d != 64 && a->d != 128) return FL_ERR_UNSUPPORTED;
  if ((a->flags & (FL_Q_HADAMARD | FL_Q_HADAMARD_NVFP4_ONLY)) && a->d != 128) return FL_ERR_UNSUPPORTED;
  if ((a->flags & FL_Q_HADAMARD) && (a->flags & FL_Q_TOKEN_LOCAL)) return FL_ERR_UNSUPPORTED;
  if (a->h > 65535 || a->b > 65535) return FL_ERR_TOO_LARGE;
  QuantParams p;
  p.x = (const uint16_t*)a->x; p.o = (const uint16_t*)a->o; p.lse = a->lse;
  p.codes = a->codes; p.codes_t = a->codes_t; p.e_tab = a->e_tab; p.fac = a->fac; p.sf_tok = a->sf_tok;
  p.sf_dim = a->sf_dim; p.token_factors = a->token_factors; p.x4 = a->x4; p.sf4 = a->sf4; p.d_out = a->d_out;
  p.lse_log2 = a->lse_log2; p.zero_acc = (uint16_t*)a->zero_acc; p.tile_stats = a->tile_stats;
  p.b = a->b; p.s = a->s; p.h = a->h; p.d = a->d; p.flags = a->flags; p.in_f16 = a->in_f16;
  p.lse_shift = a->lse_shift; p.d_multiplier = a->d_multiplier;
  dim3 grid(a->s / 128, a->h, a->b);
  cudaStream_t st = (cudaStream_t)stream;
  if (a->d == 128) quant_blocks_kernel<128><<<grid, QTHREADS, 0, st>>>(p);
  else quant_blocks_kernel<64><<<grid, QTHREADS, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? FL_OK : FL_ERR_CUDA;
}
