// Fused block-scaled quantiser (token-block MXFP8, optional NVFP4 S-operand copy, optional Hadamard rotation) and the
// fused backward prologue (D = rowsum(O * dequant(dO)), shifted log2 LSE, zeroed f16 dQ accumulator).
//
// Replaces the reference's quantize_fp8_blocks launch (flash_attn/cute/quant/fp8.py:2512, kernel_stream :1639) and the
// fused NVFP4 copy (flash_attn/cute/quant/_fp8_nvfp4.py:121-158). Outputs are byte-identical to the reference's eager
// definitions (tests/cute/quant_reference.py:714-798, 270-369).
//
// One CTA per (128-token tile, head, batch); thread r owns token row r, warp w owns the 32-token block w, so the block
// maximum is one warp reduction. The tile is staged through shared memory with 16-byte coalesced accesses on both sides:
// the kernel is HBM-bound (2 B read + 1 B written per element, plus the optional copies).
#include "flamia_internal.h"

namespace fl {

static constexpr int QT = 128;  // tokens per tile = threads per CTA

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
  uint16_t* zero_acc;     // (b, h, s, d) f16 or null
  float* tile_stats;      // (b, h, s/128, 2): [amax of the values quantised, max row sum of squares] or null
  int b, s, h, d;
  int flags;
  int in_f16;
  float lse_shift, d_multiplier;
};

__device__ __forceinline__ float in_to_f32(uint16_t v, int f16) {
  return f16 ? __half2float(__ushort_as_half(v)) : __uint_as_float((uint32_t)v << 16);
}
__device__ __forceinline__ float flush_sub(float v) { return fabsf(v) < 1.17549435e-38f ? v * 0.0f : v; }

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
__global__ void __launch_bounds__(QT) quant_blocks_kernel(const QuantParams p) {
  constexpr int ROWB = D * 2 + 16;               // padded bf16 row in shared memory
  constexpr int CROWB = D + 16;                  // padded code row
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* sx = smem;                            // QT * ROWB  input tile (kept intact)
  uint8_t* sc = smem + QT * ROWB;                // QT * CROWB staging of codes / packed NVFP4 codes
  uint8_t* so = sc + QT * CROWB;                 // QT * ROWB  forward output tile (prologue only)
  __shared__ uint32_t s_bytes[4];

  const int tile = blockIdx.x, head = blockIdx.y, bat = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = tile * QT;
  const size_t row_stride = (size_t)p.h * D;     // elements between consecutive tokens
  const uint16_t* xg = p.x + ((size_t)bat * p.s + t0) * row_stride + (size_t)head * D;
  const bool prologue = p.d_out != nullptr && p.o != nullptr;

  // ---- stage the tile: 16 B per thread per step, D/8 threads per row
  constexpr int TPR = D / 8;                     // threads per row
  constexpr int RPS = QT / TPR;                  // rows per step
  {
    const int c = tid % TPR, r0 = tid / TPR;
#pragma unroll 4
    for (int r = r0; r < QT; r += RPS) {
      uint4 v = *reinterpret_cast<const uint4*>(xg + (size_t)r * row_stride + c * 8);
      *reinterpret_cast<uint4*>(sx + r * ROWB + c * 16) = v;
    }
    if (prologue) {
      const uint16_t* og = p.o + ((size_t)bat * p.s + t0) * row_stride + (size_t)head * D;
#pragma unroll 4
      for (int r = r0; r < QT; r += RPS) {
        uint4 v = *reinterpret_cast<const uint4*>(og + (size_t)r * row_stride + c * 8);
        *reinterpret_cast<uint4*>(so + r * ROWB + c * 16) = v;
      }
    }
  }
  if (p.zero_acc) {   // the tile's slice of the (b, h, s, d) f16 accumulator is contiguous
    uint4* z = reinterpret_cast<uint4*>(p.zero_acc + (((size_t)bat * p.h + head) * p.s + t0) * D);
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll 4
    for (int i = tid; i < QT * D / 8; i += QT) z[i] = zero;
  }
  __syncthreads();

  // ---- this thread's row in registers
  float x[D];
  auto load_row = [&]() {
    const uint8_t* rowp = sx + tid * ROWB;
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
      uint4 v = *reinterpret_cast<const uint4*>(rowp + c * 16);
      uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        x[c * 8 + 2 * j] = in_to_f32((uint16_t)(w[j] & 0xFFFF), p.in_f16);
        x[c * 8 + 2 * j + 1] = in_to_f32((uint16_t)(w[j] >> 16), p.in_f16);
      }
    }
  };
  load_row();

  const bool rotate = (p.flags & (FL_Q_HADAMARD | FL_Q_HADAMARD_NVFP4_ONLY)) != 0;
  const bool rot_only4 = (p.flags & FL_Q_HADAMARD_NVFP4_ONLY) != 0;
  const bool want4 = p.x4 != nullptr;

  // ---- NVFP4 copy first when it needs rotated values but the E4M3 copy does not (two passes over the registers)
  auto rotate_row = [&](float* y) {
    if constexpr (D == 128) {
      constexpr uint32_t NEG[4] = {0x10D2E03Eu, 0xE0D9F0E2u, 0x45809F07u, 0x75954FEDu};
#pragma unroll
      for (int i = 0; i < 128; ++i)
        if ((NEG[i >> 5] >> (i & 31)) & 1) y[i] = -y[i];
#pragma unroll
      for (int hs = 1; hs < 128; hs <<= 1) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          if ((i & hs) == 0) {
            float a = y[i], b2 = y[i + hs];
            y[i] = __fadd_rn(a, b2);
            y[i + hs] = __fsub_rn(a, b2);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 128; ++i) y[i] = __fmul_rn(y[i], 0.08838834764831845f);
    }
  };

  auto nvfp4_row = [&](const float* y) {
    // per 16 along d: SF = E4M3_rn(amax * f32(1/6)); codes = E2M1_rn(ftz(x * m)), m = 1/SF | +inf | 0
    uint8_t* x4row = sc + tid * CROWB;   // D/2 bytes staged for the coalesced store
    uint32_t sfw[D / 64];
#pragma unroll
    for (int a = 0; a < D / 64; ++a) sfw[a] = 0;
#pragma unroll
    for (int g = 0; g < D / 16; ++g) {
      float am = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float a = fabsf(flush_sub(y[g * 16 + j]));
        am = (a > am) ? a : am;          // a NaN never wins
      }
      float u = __fmul_rn(am, 1.0f / 6.0f);
      uint32_t sfb = cvt_e4m3x2(u, 0.f) & 0xFF;
      float sfv = e4m3_byte_to_f32(sfb);
      float m = sfv > 0.f ? __frcp_rn(sfv) : (u > 0.f ? __int_as_float(0x7F800000) : 0.f);
      uint32_t packed[2] = {0, 0};
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        float a0 = flush_sub(__fmul_rn(flush_sub(y[g * 16 + j]), m));
        float a1 = flush_sub(__fmul_rn(flush_sub(y[g * 16 + j + 1]), m));
        uint16_t c2;
        asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}"
            : "=h"(c2)
            : "f"(a1), "f"(a0));
        packed[j >> 3] |= (uint32_t)(c2 & 0xFF) << ((j & 7) * 4);
      }
      *reinterpret_cast<uint2*>(x4row + g * 8) = make_uint2(packed[0], packed[1]);
      sfw[g >> 2] |= sfb << ((g & 3) * 8);
    }
    if (p.sf4) {
      uint8_t* atom = p.sf4 + ((((size_t)bat * p.h + head) * (p.s / QT) + tile) * (D / 64)) * 512;
#pragma unroll
      for (int a = 0; a < D / 64; ++a)
        *reinterpret_cast<uint32_t*>(atom + a * 512 + (tid & 31) * 16 + (tid >> 5) * 4) = sfw[a];
    }
  };

  auto store_x4 = [&]() {   // QT rows of D/2 bytes from the staging area, coalesced
    __syncthreads();
    constexpr int TPR4 = D / 32;   // 16-byte chunks per row
    uint8_t* g4 = p.x4 + (((size_t)bat * p.s + t0) * p.h + head) * (D / 2);
    for (int i = tid; i < QT * TPR4; i += QT) {
      int r = i / TPR4, c = i % TPR4;
      *reinterpret_cast<uint4*>(g4 + (size_t)r * p.h * (D / 2) + c * 16) =
          *reinterpret_cast<const uint4*>(sc + r * CROWB + c * 16);
    }
    __syncthreads();
  };

  if (want4 && rotate && rot_only4) {   // NVFP4 codes of the rotated row, E4M3 codes of the row as read
    rotate_row(x);
    nvfp4_row(x);
    store_x4();
    load_row();
  } else if (rotate) {
    rotate_row(x);
  }
  if (want4 && !(rotate && rot_only4)) {
    nvfp4_row(x);
    store_x4();
  }

  // ---- token-block exponent
  float amax = 0.f, sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < D; ++i) {
    x[i] = flush_sub(x[i]);
    float a = fabsf(x[i]);
    amax = fmaxf(amax, a);
    sumsq = fmaf(x[i], x[i], sumsq);
  }
  float bmax = amax;
#pragma unroll
  for (int o = 16; o; o >>= 1) bmax = fmaxf(bmax, __shfl_xor_sync(0xFFFFFFFFu, bmax, o));
  const uint32_t bbyte = ue8m0_byte(bmax);
  const bool tl = (p.flags & FL_Q_TOKEN_LOCAL) != 0;
  const uint32_t tbyte = tl ? ue8m0_byte(amax) : bbyte;
  const float inv = tbyte ? pow2_from_field(254 - (int)tbyte) : 0.f;
  const float scale = tbyte ? pow2_from_field((int)tbyte) : 0.f;

  uint32_t cw[D / 4];
#pragma unroll
  for (int i = 0; i < D / 4; ++i)
    cw[i] = cvt_e4m3x4(__fmul_rn(x[4 * i], inv), __fmul_rn(x[4 * i + 1], inv), __fmul_rn(x[4 * i + 2], inv),
                       __fmul_rn(x[4 * i + 3], inv));

  // ---- prologue: D in the fixed tree order, shifted log2 LSE
  if (prologue) {
    float a[D];
#pragma unroll
    for (int i = 0; i < D / 4; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) a[4 * i + j] = __fmul_rn(e4m3_byte_to_f32((cw[i] >> (8 * j)) & 0xFF), scale);
    }
    const uint8_t* orow = so + tid * ROWB;
    float v[64];
#pragma unroll
    for (int k = 0; k < 64; ++k) {
      const int c = ((k >> 1) << 2) | (k & 1);   // columns with bit 1 clear
      float prod = 0.f, acc = 0.f;
      if (c < D) {
        float o0 = in_to_f32(*reinterpret_cast<const uint16_t*>(orow + c * 2), p.in_f16);
        float o2 = in_to_f32(*reinterpret_cast<const uint16_t*>(orow + (c + 2) * 2), p.in_f16);
        prod = __fmul_rn(a[c + 2 < D ? c + 2 : 0], o2);
        acc = __fmaf_rn(a[c], o0, prod);
      }
      v[k] = acc;
    }
    // v index k <-> column c(k); column bits (2,3,0,6,5,4) <-> k bits (1,2,0,5,4,3)
    constexpr int KB[6] = {1, 2, 0, 5, 4, 3};
#pragma unroll
    for (int st = 0; st < 6; ++st) {
      const int bit = 1 << KB[st];
#pragma unroll
      for (int k = 0; k < 64; ++k)
        if ((k & bit) == 0) v[k] = __fadd_rn(v[k], v[k | bit]);
    }
    const size_t ri = ((size_t)bat * p.h + head) * p.s + t0 + tid;
    p.d_out[ri] = __fmul_rn(v[0], p.d_multiplier);
    if (p.lse && p.lse_log2) {
      float l = p.lse[ri];
      float pr = __fmul_rn(l, 1.4426950408889634f);
      p.lse_log2[ri] = __fsub_rn((l == -INFINITY) ? 0.f : pr, p.lse_shift);
    }
  } else if (p.lse && p.lse_log2) {
    const size_t ri = ((size_t)bat * p.h + head) * p.s + t0 + tid;
    float l = p.lse[ri];
    p.lse_log2[ri] = __fsub_rn((l == -INFINITY) ? 0.f : __fmul_rn(l, 1.4426950408889634f), p.lse_shift);
  }

  // ---- side tables
  if (lane == 0) s_bytes[warp] = bbyte;
  {
    uint8_t* crow = sc + tid * CROWB;
#pragma unroll
    for (int i = 0; i < D / 16; ++i)
      *reinterpret_cast<uint4*>(crow + i * 16) = make_uint4(cw[4 * i], cw[4 * i + 1], cw[4 * i + 2], cw[4 * i + 3]);
  }
  __syncthreads();
  const size_t bh = (size_t)bat * p.h + head;
  const int ntile = p.s / QT;
  if (p.e_tab && lane == 0) {
    uint8_t* e = p.e_tab + (bh * (p.s / 32) + tile * 4 + warp) * (D / 32);
#pragma unroll
    for (int g = 0; g < D / 32; ++g) e[g] = (uint8_t)bbyte;
  }
  if (p.fac && lane == 0) {
    uint32_t tm = max(max(s_bytes[0], s_bytes[1]), max(s_bytes[2], s_bytes[3]));
    uint32_t e0 = bbyte ? bbyte : tm;
    p.fac[bh * (p.s / 32) + tile * 4 + warp] = e0 ? pow2_from_field((int)e0) : 1.0f;
  }
  if (p.token_factors) p.token_factors[bh * p.s + t0 + tid] = tbyte ? scale : 1.0f;
  if (p.sf_tok)
    *reinterpret_cast<uint32_t*>(p.sf_tok + (bh * ntile + tile) * 512 + lane * 16 + warp * 4) = tbyte * 0x01010101u;
  if (p.sf_dim) {
    uint32_t w = s_bytes[0] | (s_bytes[1] << 8) | (s_bytes[2] << 16) | (s_bytes[3] << 24);
    *reinterpret_cast<uint32_t*>(p.sf_dim + (bh * ntile + tile) * 512 + tid * 4) = w;
  }
  if (p.tile_stats) {
    float a = bmax, q = sumsq;
#pragma unroll
    for (int o = 16; o; o >>= 1) q = fmaxf(q, __shfl_xor_sync(0xFFFFFFFFu, q, o));
    __shared__ float s_st[8];
    if (lane == 0) { s_st[warp] = a; s_st[4 + warp] = q; }
    __syncthreads();
    if (tid == 0) {
      p.tile_stats[(bh * ntile + tile) * 2] = fmaxf(fmaxf(s_st[0], s_st[1]), fmaxf(s_st[2], s_st[3]));
      p.tile_stats[(bh * ntile + tile) * 2 + 1] = fmaxf(fmaxf(s_st[4], s_st[5]), fmaxf(s_st[6], s_st[7]));
    }
  }

  // ---- codes (b, s, h, d): coalesced 16 B stores
  {
    constexpr int TPRC = D / 16;
    uint8_t* cg = p.codes + ((size_t)bat * p.s + t0) * row_stride + (size_t)head * D;
    for (int i = tid; i < QT * TPRC; i += QT) {
      int r = i / TPRC, c = i % TPRC;
      *reinterpret_cast<uint4*>(cg + (size_t)r * row_stride + c * 16) =
          *reinterpret_cast<const uint4*>(sc + r * CROWB + c * 16);
    }
  }
  // ---- channel-major copy (b, h, d, s): thread c gathers column c
  if (p.codes_t) {
    for (int c = tid; c < D; c += QT) {
      uint8_t* dst = p.codes_t + (bh * D + c) * (size_t)p.s + t0;
#pragma unroll 2
      for (int r = 0; r < QT; r += 16) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          w[j] = (uint32_t)sc[(r + 4 * j) * CROWB + c] | ((uint32_t)sc[(r + 4 * j + 1) * CROWB + c] << 8) |
                 ((uint32_t)sc[(r + 4 * j + 2) * CROWB + c] << 16) | ((uint32_t)sc[(r + 4 * j + 3) * CROWB + c] << 24);
        *reinterpret_cast<uint4*>(dst + r) = make_uint4(w[0], w[1], w[2], w[3]);
      }
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
  if (a->s / 128 > 65535 * 64 || a->h > 65535 || a->b > 65535) return FL_ERR_TOO_LARGE;
  QuantParams p;
  p.x = (const uint16_t*)a->x; p.o = (const uint16_t*)a->o; p.lse = a->lse;
  p.codes = a->codes; p.codes_t = a->codes_t; p.e_tab = a->e_tab; p.fac = a->fac; p.sf_tok = a->sf_tok;
  p.sf_dim = a->sf_dim; p.token_factors = a->token_factors; p.x4 = a->x4; p.sf4 = a->sf4; p.d_out = a->d_out;
  p.lse_log2 = a->lse_log2; p.zero_acc = (uint16_t*)a->zero_acc; p.tile_stats = a->tile_stats;
  p.b = a->b; p.s = a->s; p.h = a->h; p.d = a->d; p.flags = a->flags; p.in_f16 = a->in_f16;
  p.lse_shift = a->lse_shift; p.d_multiplier = a->d_multiplier;
  dim3 grid(a->s / 128, a->h, a->b);
  cudaStream_t st = (cudaStream_t)stream;
  const bool pro = p.d_out && p.o;
  if (a->d == 128) {
    size_t sm = 128 * (128 * 2 + 16) * (pro ? 2 : 1) + 128 * (128 + 16);
    if (cudaFuncSetAttribute(quant_blocks_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm) !=
        cudaSuccess)
      return FL_ERR_CUDA;
    quant_blocks_kernel<128><<<grid, 128, sm, st>>>(p);
  } else {
    size_t sm = 128 * (64 * 2 + 16) * (pro ? 2 : 1) + 128 * (64 + 16);
    if (cudaFuncSetAttribute(quant_blocks_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm) !=
        cudaSuccess)
      return FL_ERR_CUDA;
    quant_blocks_kernel<64><<<grid, 128, sm, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? FL_OK : FL_ERR_CUDA;
}
