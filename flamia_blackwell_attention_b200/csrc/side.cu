// HBM-bound side kernels of the backward: f16 dQ pre-scale table, dQ postprocess, packed-row gather / scatter.
#include "flamia_internal.h"

namespace fl {

// ------------------------------------------------------------------------------------------------ dQ pre-scale
// Restates flash_attn/cute/device_scales.py:124-132 (_dq_bound_pow2) and :158-184, 234-319 (_dq_row_bound,
// _dq_tile_table) of the reference: bound = ((((4 unit) 2) sqrt(dn2)) sqrt(vn2)) kmax in fp32 (mul.rn / sqrt.rn / div.rn
// only), B = the largest power of two <= 65504 / bound with its exponent clamped to [-40, 40].
__device__ __forceinline__ float pow2_floor_clamped(float x, int lo, int hi) {
  int e = (int)((__float_as_uint(x) >> 23) & 0xFF) - 127;
  e = max(lo, min(hi, e));
  return __uint_as_float((uint32_t)(e + 127) << 23);
}

__global__ void dq_prescale_kernel(const float* __restrict__ st_do, const float* __restrict__ st_v,
                                   const float* __restrict__ st_k, int h, int h_kv, int nt_q, int nt_k, int causal_local,
                                   float unit, float* kernel_scale, float* post_scale) {
  const int bq = blockIdx.y, t = blockIdx.x, tid = threadIdx.x;
  const int q_lo = causal_local ? t : 0, q_hi = causal_local ? t + 1 : nt_q;
  const int k_lo = 0, k_hi = causal_local ? min(t + 1 + max(nt_k - nt_q, 0), nt_k) : nt_k;
  float dn = 0.f, vn = 0.f, km = 0.f;
  const int nq = q_hi - q_lo, nk = k_hi - k_lo;
  for (int j = tid; j < h * nq; j += blockDim.x)
    dn = fmaxf(dn, st_do[(((size_t)bq * h + j / nq) * nt_q + q_lo + j % nq) * 2 + 1]);
  for (int j = tid; j < h_kv * nk; j += blockDim.x) {
    const size_t o = (((size_t)bq * h_kv + j / nk) * nt_k + k_lo + j % nk) * 2;
    vn = fmaxf(vn, st_v[o + 1]);
    km = fmaxf(km, st_k[o]);
  }
  __shared__ float red[3][32];
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    dn = fmaxf(dn, __shfl_xor_sync(0xFFFFFFFFu, dn, o));
    vn = fmaxf(vn, __shfl_xor_sync(0xFFFFFFFFu, vn, o));
    km = fmaxf(km, __shfl_xor_sync(0xFFFFFFFFu, km, o));
  }
  if ((tid & 31) == 0) { red[0][tid >> 5] = dn; red[1][tid >> 5] = vn; red[2][tid >> 5] = km; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
      dn = fmaxf(dn, red[0][w]); vn = fmaxf(vn, red[1][w]); km = fmaxf(km, red[2][w]);
    }
    float bnd = __fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(4.0f, unit), 2.0f), __fsqrt_rn(dn)), __fsqrt_rn(vn)), km);
    float bb = pow2_floor_clamped(__fdiv_rn(65504.0f, bnd), -40, 40);
    kernel_scale[(size_t)bq * nt_q + t] = bb;
    post_scale[(size_t)bq * nt_q + t] = __fdiv_rn(1.0f, __fmul_rn(unit, bb));
  }
}

// Per query row i of a causal square batched call: B_i from the row's own dO statistic and the running maxima of the V / K
// statistics over the keys j <= i (flash_attn/cute/device_scales.py:256-268, CAUSAL == 2). One CTA per batch row walks
// the sequence in chunks of its size, carrying the running maxima; the prefix maxima overwrite row_v / row_k.
__global__ void __launch_bounds__(1024) dq_prescale_rows_kernel(const float* __restrict__ row_do, float* row_v, float* row_k,
                                                                int s, float unit, float* kernel_rows, float* post_rows) {
  __shared__ float sv[32], sk[32];
  const int bat = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t base = (size_t)bat * s;
  float run_v = 0.f, run_k = 0.f;
  for (int i0 = 0; i0 < s; i0 += blockDim.x) {
    const int i = i0 + tid;
    float v = i < s ? row_v[base + i] : 0.f, k = i < s ? row_k[base + i] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {             // inclusive prefix maximum inside the warp
      const float ov = __shfl_up_sync(0xFFFFFFFFu, v, o), okk = __shfl_up_sync(0xFFFFFFFFu, k, o);
      if (lane >= o) { v = fmaxf(v, ov); k = fmaxf(k, okk); }
    }
    if (lane == 31) { sv[warp] = v; sk[warp] = k; }
    __syncthreads();
    float pv = run_v, pk = run_k;                  // everything before this warp: earlier chunks and earlier warps
    for (int w = 0; w < warp; ++w) { pv = fmaxf(pv, sv[w]); pk = fmaxf(pk, sk[w]); }
    v = fmaxf(v, pv);
    k = fmaxf(k, pk);
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { run_v = fmaxf(run_v, sv[w]); run_k = fmaxf(run_k, sk[w]); }
    if (i < s) {
      row_v[base + i] = v;
      row_k[base + i] = k;
      const float dn = row_do[base + i];
      const float bnd = __fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(4.0f, unit), 2.0f), __fsqrt_rn(dn)), __fsqrt_rn(v)), k);
      const float bb = pow2_floor_clamped(__fdiv_rn(65504.0f, bnd), -40, 40);
      kernel_rows[base + i] = bb;
      post_rows[base + i] = __fdiv_rn(1.0f, __fmul_rn(unit, bb));
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------ dQ postprocess
// dq[b, q, h, :] = cast(f32(acc) * post[b, q / 128] * mult), optionally rotated back: (y H_128 / sqrt(128)) * signs in the
// quantiser's butterfly order. Replaces the reference's DQPostprocess (flash_attn/cute/dq_postprocess_cute.py:46-124).
// HBM-bound: 2 B read + 2 B written per element.
__device__ __forceinline__ uint32_t cvt_out2(float a, float b, int out_f16) {
  if (out_f16) { __half2 hh = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&hh); }
  return pack_bf16x2(a, b);
}

// head dim 64: the accumulator is (b, h, s, 64); a straight scaled copy into the (b, s, h, 64) gradient
__global__ void __launch_bounds__(128) dq_post_rows64_kernel(const __half* __restrict__ acc, const float* __restrict__ post,
                                                             uint16_t* __restrict__ dq, int s, int h, float mult,
                                                             int out_f16, int per_row, const float* __restrict__ head_mult,
                                                             const int32_t* __restrict__ slot_src,
                                                             const int32_t* __restrict__ slot_rows) {
  constexpr int D = 64, CPR = D / 8;
  const int tile = blockIdx.x, head = blockIdx.y, bat = blockIdx.z, tid = threadIdx.x;
  const int t0 = tile * 128;
  if (head_mult) mult *= head_mult[(size_t)bat * h + head];
  const __half* src = acc + (((size_t)bat * h + head) * s + t0) * D;
  const float sc_tile = per_row ? 0.f : post[(size_t)bat * (s / 128) + tile] * mult;
  // packed output: the tile's rows go to the packed rows slot_src[tile] .. + slot_rows[tile] of dq
  const int n_rows = slot_src ? (slot_src[tile] >= 0 ? min(slot_rows[tile], 128) : 0) : 128;
  uint16_t* dst = dq + (((size_t)bat * s + (slot_src ? (n_rows ? slot_src[tile] : 0) : t0)) * h + head) * D;
  const size_t row_stride = (size_t)h * D;
  for (int i = tid; i < 128 * CPR; i += 128) {
    const int r = i / CPR, c = i % CPR;
    if (r >= n_rows) continue;
    const float sc = per_row ? post[(size_t)bat * s + t0 + r] * mult : sc_tile;
    uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)r * D + c * 8);
    const __half2* hv = reinterpret_cast<const __half2*>(&v);
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __half22float2(hv[j]);
      w[j] = cvt_out2(f.x * sc, f.y * sc, out_f16);
    }
    *reinterpret_cast<uint4*>(dst + (size_t)r * row_stride + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// head dim 128: the accumulator is (b, h, 128, s) (the backward produces transposed dQ tiles). One CTA per (128-token tile,
// head): the 128 x 128 f16 tile comes in as two TMA boxes of 64 tokens (128-byte rows, 128 B swizzle), thread t gathers
// token t's column from shared memory, optionally rotates it back, and the rows leave through a padded staging buffer
// as coalesced 16-byte stores.
__global__ void __launch_bounds__(128) dq_post_t128_kernel(const __grid_constant__ CUtensorMap tm_acc,
                                                           const float* __restrict__ post, uint16_t* __restrict__ dq,
                                                           int s, int h, float mult, int unrotate, int out_f16,
                                                           int per_row, const float* __restrict__ head_mult,
                                                           const int32_t* __restrict__ slot_src,
                                                           const int32_t* __restrict__ slot_rows) {
  constexpr int D = 128, ROWB = D * 2 + 16, CPR = D / 8;
  extern __shared__ __align__(1024) uint8_t sm_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sm_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_in = sm;                  // 2 boxes x 128 head-dim rows x 128 B
  uint8_t* s_out = sm + 32768;         // 128 token rows x (256 + 16) B
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_s;
  const int tile = blockIdx.x, head = blockIdx.y, bat = blockIdx.z, tid = threadIdx.x;
  const int t0 = tile * 128;
  if (tid == 0) {
    abort_s = 0;
    mbar_init(&bar, 1);
    fence_barrier_init();
    mbar_arrive_expect_tx(&bar, 32768);
    tma_load_4d(s_in, &tm_acc, &bar, t0, 0, head, bat);
    tma_load_4d(s_in + 16384, &tm_acc, &bar, t0 + 64, 0, head, bat);
  }
  if (head_mult) mult *= head_mult[(size_t)bat * h + head];
  const float sc = (per_row ? post[(size_t)bat * s + t0 + tid] : post[(size_t)bat * (s / 128) + tile]) * mult;   // thread = token
  __syncthreads();
  const DevCtl ctl = {nullptr, kDefaultWaitCycles};
  bool ok = mbar_wait(&bar, 0, ctl, &abort_s, 60);
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  if (ok) {
    float y[128];
    {
      const int tt = tid & 63;
      const uint32_t base = smem_u32(s_in) + (tid >> 6) * 16384 + (tt & 7) * 2;
#pragma unroll
      for (int c = 0; c < 128; ++c) {
        uint16_t hv;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(hv) : "r"(base + c * 128 + ((((uint32_t)tt >> 3) ^ (c & 7)) << 4)));
        y[c] = __half2float(__ushort_as_half(hv)) * sc;
      }
    }
    // pairs of neighbouring head-dim columns in one 64-bit register: one instruction per pair
    uint64_t Y[64];
    if (unrotate) {      // (y H_128 / sqrt(128)) * signs: butterfly levels 1, 2, ..., 64, then the scaling with the signs
#pragma unroll
      for (int i = 0; i < 64; ++i) Y[i] = pack2(__fadd_rn(y[2 * i], y[2 * i + 1]), __fsub_rn(y[2 * i], y[2 * i + 1]));
#pragma unroll
      for (int hs = 1; hs < 64; hs <<= 1) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          if ((i & hs) == 0) {
            const uint64_t a = Y[i], b2 = Y[i + hs];
            Y[i] = add2(a, b2);
            Y[i + hs] = sub2(a, b2);
          }
        }
      }
      constexpr uint32_t NEG[4] = {0x10D2E03Eu, 0xE0D9F0E2u, 0x45809F07u, 0x75954FEDu};
      constexpr float CP = 0.08838834764831845f;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const bool n0 = (NEG[(2 * i) >> 5] >> ((2 * i) & 31)) & 1, n1 = (NEG[(2 * i + 1) >> 5] >> ((2 * i + 1) & 31)) & 1;
        Y[i] = mul2(Y[i], pack2(n0 ? -CP : CP, n1 ? -CP : CP));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) Y[i] = pack2(y[2 * i], y[2 * i + 1]);
    }
    uint8_t* rowo = s_out + tid * ROWB;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a, b2;
        unpack2(Y[c * 4 + j], a, b2);
        w[j] = cvt_out2(a, b2, out_f16);
      }
      *reinterpret_cast<uint4*>(rowo + c * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    __syncthreads();
    // packed output: the tile's rows go to the packed rows slot_src[tile] .. + slot_rows[tile] of dq
    const int n_rows = slot_src ? (slot_src[tile] >= 0 ? min(slot_rows[tile], 128) : 0) : 128;
    uint16_t* dst = dq + (((size_t)bat * s + (slot_src ? (n_rows ? slot_src[tile] : 0) : t0)) * h + head) * D;
    const size_t row_stride = (size_t)h * D;
    for (int i = tid; i < 128 * CPR; i += 128) {
      const int r = i / CPR, c = i % CPR;
      if (r < n_rows)
        *reinterpret_cast<uint4*>(dst + (size_t)r * row_stride + c * 8) = *reinterpret_cast<const uint4*>(s_out + r * ROWB + c * 16);
    }
  } else {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);     // loads into this CTA's shared memory may still land
  }
}

// ------------------------------------------------------------------------------------------------ statistics of codes
// One CTA per (128-row tile, head, batch row), thread = row: the largest magnitude and the largest row sum of squares of
// codes * descale[b, h] (fp32 sums in column order).
__device__ __forceinline__ float e4m3_to_f32(uint32_t c) {
  const uint32_t e = (c >> 3) & 0xF, m = c & 7;
  const float v = e ? __uint_as_float(((e + 120) << 23) | (m << 20)) : (float)m * 0.001953125f;
  return (c & 0x80) ? -v : v;
}
__global__ void __launch_bounds__(128) code_stats_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ descale,
                                                         int s, int h, int d, float* __restrict__ tile_stats) {
  const int tile = blockIdx.x, head = blockIdx.y, bat = blockIdx.z, tid = threadIdx.x;
  const uint8_t* row = codes + (((size_t)bat * s + tile * 128 + tid) * h + head) * d;
  const float f = descale[(size_t)bat * h + head];
  float am = 0.f, sq = 0.f;
  for (int c = 0; c < d; c += 16) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float x = e4m3_to_f32((w[k >> 2] >> (8 * (k & 3))) & 0xFF) * f;
      am = fmaxf(am, fabsf(x));
      sq = fmaf(x, x, sq);
    }
  }
  __shared__ float red[2][4];
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, o));
    sq = fmaxf(sq, __shfl_xor_sync(0xFFFFFFFFu, sq, o));
  }
  if ((tid & 31) == 0) { red[0][tid >> 5] = am; red[1][tid >> 5] = sq; }
  __syncthreads();
  if (tid == 0) {
    float* o = tile_stats + ((((size_t)bat * h + head) * (s / 128)) + tile) * 2;
    o[0] = fmaxf(fmaxf(red[0][0], red[0][1]), fmaxf(red[0][2], red[0][3]));
    o[1] = fmaxf(fmaxf(red[1][0], red[1][1]), fmaxf(red[1][2], red[1][3]));
  }
}

// ------------------------------------------------------------------------------------------------ packed rows
__global__ void pack_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int32_t* __restrict__ map,
                                 int n_rows, int chunks) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_rows * chunks) return;
  const int r = (int)(i / chunks), c = (int)(i % chunks);
  const int sr = map[r];
  dst[i] = sr >= 0 ? src[(size_t)sr * chunks + c] : make_uint4(0, 0, 0, 0);
}
__global__ void unpack_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int32_t* __restrict__ map,
                                   int n_rows, int chunks) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_rows * chunks) return;
  const int r = (int)(i / chunks), c = (int)(i % chunks);
  const int dr = map[r];
  if (dr >= 0) dst[(size_t)dr * chunks + c] = src[i];
}

}  // namespace fl

extern "C" int fl_dq_prescale(const float* stats_do, const float* stats_v, const float* stats_k, int32_t b, int32_t h,
                              int32_t h_kv, int32_t nt_q, int32_t nt_k, int32_t causal_local, float unit,
                              float* kernel_scale, float* post_scale, void* stream) {
  using namespace fl;
  if (!stats_do || !stats_v || !stats_k || !kernel_scale || !post_scale || b <= 0 || nt_q <= 0 || nt_k <= 0)
    return FL_ERR_BAD_ARG;
  dq_prescale_kernel<<<dim3(nt_q, b), 128, 0, (cudaStream_t)stream>>>(stats_do, stats_v, stats_k, h, h_kv, nt_q, nt_k,
                                                                      causal_local, unit, kernel_scale, post_scale);
  return launch_result("fl_dq_prescale: kernel launch");
}

// The accumulator layout follows the backward kernel that filled it: (b, h, d, s) for head_dim 128 (pipelined kernel,
// transposed dQ tiles), (b, h, s, d) for head_dim 64.
static int dq_post_launch(const void* dq_acc, const float* post_scale, float mult, void* dq, int32_t b, int32_t s,
                          int32_t h, int32_t d, int32_t unrotate, int32_t out_f16, int per_row, const float* head_mult,
                          void* stream, const int32_t* slot_src = nullptr, const int32_t* slot_rows = nullptr) {
  using namespace fl;
  if (!dq_acc || !post_scale || !dq || b <= 0 || s <= 0 || (s % 128) || h <= 0) return FL_ERR_BAD_ARG;
  if ((d != 64 && d != 128) || (unrotate && d != 128)) return FL_ERR_UNSUPPORTED;
  if (h > 65535 || b > 65535) return FL_ERR_TOO_LARGE;
  dim3 grid(s / 128, h, b);
  cudaStream_t st = (cudaStream_t)stream;
  if (d == 128) {
    CUtensorMap macc;
    int rc = make_acc_t_map_16(&macc, dq_acc, b, h, d, s);
    if (rc) return rc;
    const int sm = 32768 + 128 * 272 + 1024;
    if (cudaError_t e = cudaFuncSetAttribute(dq_post_t128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sm); e != cudaSuccess)
      return cuda_fail((int)e, "fl_dq_post: cudaFuncSetAttribute");
    dq_post_t128_kernel<<<grid, 128, sm, st>>>(macc, post_scale, (uint16_t*)dq, s, h, mult, unrotate, out_f16, per_row,
                                               head_mult, slot_src, slot_rows);
  } else {
    dq_post_rows64_kernel<<<grid, 128, 0, st>>>((const __half*)dq_acc, post_scale, (uint16_t*)dq, s, h, mult, out_f16,
                                                per_row, head_mult, slot_src, slot_rows);
  }
  return launch_result("fl_dq_post: kernel launch");
}

extern "C" int fl_dq_post(const void* dq_acc, const float* post_scale, float mult, void* dq, int32_t b, int32_t s,
                          int32_t h, int32_t d, int32_t unrotate, int32_t out_f16, void* stream) {
  return dq_post_launch(dq_acc, post_scale, mult, dq, b, s, h, d, unrotate, out_f16, 0, nullptr, stream);
}

extern "C" int fl_dq_post_ex(const void* dq_acc, const float* post_scale, int32_t per_row, const float* head_mult, float mult,
                             void* dq, int32_t b, int32_t s, int32_t h, int32_t d, int32_t unrotate, int32_t out_f16,
                             void* stream) {
  return dq_post_launch(dq_acc, post_scale, mult, dq, b, s, h, d, unrotate, out_f16, per_row ? 1 : 0, head_mult, stream);
}

extern "C" int fl_dq_post_rows(const void* dq_acc, const float* post_scale_rows, float mult, void* dq, int32_t b, int32_t s,
                               int32_t h, int32_t d, int32_t unrotate, int32_t out_f16, void* stream) {
  return dq_post_launch(dq_acc, post_scale_rows, mult, dq, b, s, h, d, unrotate, out_f16, 1, nullptr, stream);
}

extern "C" int fl_dq_post_packed(const void* dq_acc, const float* post_scale, float mult, void* dq, int32_t s, int32_t h,
                                 int32_t d, int32_t unrotate, int32_t out_f16, const int32_t* slot_src,
                                 const int32_t* slot_rows, void* stream) {
  if (!slot_src || !slot_rows) return fl::FL_ERR_BAD_ARG;
  return dq_post_launch(dq_acc, post_scale, mult, dq, 1, s, h, d, unrotate, out_f16, 0, nullptr, stream, slot_src, slot_rows);
}

extern "C" int fl_dq_prescale_rows(const float* row_do, float* row_v, float* row_k, int32_t b, int32_t s, float unit,
                                   float* kernel_rows, float* post_rows, void* stream) {
  using namespace fl;
  if (!row_do || !row_v || !row_k || !kernel_rows || !post_rows || b <= 0 || s <= 0) return FL_ERR_BAD_ARG;
  dq_prescale_rows_kernel<<<b, 1024, 0, (cudaStream_t)stream>>>(row_do, row_v, row_k, s, unit, kernel_rows, post_rows);
  return launch_result("fl_dq_prescale_rows: kernel launch");
}

namespace fl {
// lg = log2 f, rcp = 1 / f for power-of-two factors: exponent-field arithmetic, exact
__global__ void token_aux_kernel(const float* __restrict__ f, long long n, float* __restrict__ lg, float* __restrict__ rcp) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t bits = __float_as_uint(f[i]) & 0x7F800000u;
  lg[i] = (float)((int)(bits >> 23) - 127);
  rcp[i] = __uint_as_float((254u << 23) - bits);
}
}  // namespace fl

extern "C" int fl_token_aux(const float* factors, int64_t n, float* lg, float* rcp, void* stream) {
  using namespace fl;
  if (!factors || !lg || !rcp || n <= 0) return FL_ERR_BAD_ARG;
  if ((n + 255) / 256 > 0x7FFFFFFF) return FL_ERR_TOO_LARGE;
  token_aux_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(factors, (long long)n, lg, rcp);
  return launch_result("fl_token_aux: kernel launch");
}

extern "C" int fl_code_stats(const void* codes, const float* descale, int32_t b, int32_t s, int32_t h, int32_t d,
                             float* tile_stats, void* stream) {
  using namespace fl;
  if (!codes || !descale || !tile_stats || b <= 0 || s <= 0 || (s % 128) || h <= 0) return FL_ERR_BAD_ARG;
  if (d != 64 && d != 128) return FL_ERR_UNSUPPORTED;
  if (h > 65535 || b > 65535) return FL_ERR_TOO_LARGE;
  code_stats_kernel<<<dim3(s / 128, h, b), 128, 0, (cudaStream_t)stream>>>((const uint8_t*)codes, descale, s, h, d, tile_stats);
  return launch_result("fl_code_stats: kernel launch");
}

extern "C" int fl_pack_rows(const void* src, void* dst, const int32_t* row_map, int32_t n_dst_rows, int32_t row_bytes,
                            void* stream) {
  using namespace fl;
  if (!src || !dst || !row_map || n_dst_rows <= 0 || row_bytes <= 0 || (row_bytes % 16)) return FL_ERR_BAD_ARG;
  const int chunks = row_bytes / 16;
  const size_t n = (size_t)n_dst_rows * chunks;
  pack_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, row_map,
                                                                                  n_dst_rows, chunks);
  return launch_result("fl_pack_rows: kernel launch");
}

extern "C" int fl_unpack_rows(const void* src, void* dst, const int32_t* row_map, int32_t n_src_rows, int32_t row_bytes,
                              void* stream) {
  using namespace fl;
  if (!src || !dst || !row_map || n_src_rows <= 0 || row_bytes <= 0 || (row_bytes % 16)) return FL_ERR_BAD_ARG;
  const int chunks = row_bytes / 16;
  const size_t n = (size_t)n_src_rows * chunks;
  unpack_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst,
                                                                                    row_map, n_src_rows, chunks);
  return launch_result("fl_unpack_rows: kernel launch");
}
