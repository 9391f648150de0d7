// One 128 x 128 x 128 tensor-core product per launch through the library's descriptor, TMA and TMEM helpers, in each of
// the operand paths the attention kernels use. The unit tests compare the result with a CPU product, which pins the
// shared-memory / instruction descriptor encodings, the TMEM operand packing and the scale-factor placement.
#include "flamia_internal.h"

namespace fl {

struct SelfTestParams {
  const uint8_t* a;
  const uint8_t* b;
  const uint8_t* sfa;
  const uint8_t* sfb;
  float* d;
  int which;
  DevCtl ctl;
};

static constexpr int ST_COL_D = 0, ST_COL_A = 128, ST_COL_SFA = 160, ST_COL_SFB = 168;

__global__ void __launch_bounds__(128) selftest_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                        const __grid_constant__ CUtensorMap tm_b,
                                                        const SelfTestParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                 // 16 KB
  uint8_t* sB = smem + 16384;         // 16 KB
  uint8_t* sSF = smem + 32768;        // 4 x 512 B scale atoms (NVFP4)
  __shared__ __align__(8) uint64_t bar_load, bar_mma, bar_never;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int which = p.which;
  if (tid == 0) {
    abort_s = 0;
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    mbar_init(&bar_never, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  if (which == FL_ST_WAIT_TIMEOUT) {
    if (tid == 0) mbar_wait(&bar_never, 0, p.ctl, &abort_s, 1);
  } else {
    const bool nvf4 = which == FL_ST_NVF4 || which == FL_ST_NVF4_N64_HI;
    const bool hi64 = which == FL_ST_NVF4_N64_HI;
    const bool dqt = which == FL_ST_MX8_MN_N64;
    const bool a2 = which == FL_ST_MX8_A_MN_2X64;      // A = two 64-byte-row blocks side by side along M
    const bool a_tmem = which == FL_ST_F8_A_TMEM || which == FL_ST_MX8_TS;
    const bool scaled8 = which == FL_ST_MX8_SS || which == FL_ST_MX8_TS || dqt || a2;
    const uint32_t tile_bytes = nvf4 ? 8192u : 16384u;
    if (tid == 0) {
      uint32_t tx = (a_tmem ? 0u : tile_bytes) + ((dqt || a2) ? 8192u : tile_bytes) + (nvf4 ? 2048u : 0u);
      mbar_arrive_expect_tx(&bar_load, tx);
      if (a2) {                       // columns [0, 64) and [64, 128) of A as two 128 x 64-byte blocks, 8 KB apart
        tma_load_2d(sA, &tm_a, &bar_load, 0, 0);
        tma_load_2d(sA + 8192, &tm_a, &bar_load, 64, 0);
      } else if (!a_tmem) tma_load_2d(sA, &tm_a, &bar_load, 0, 0);
      tma_load_2d(sB, &tm_b, &bar_load, 0, 0);
      if (nvf4) {
        bulk_load(sSF, p.sfa, 1024, &bar_load);
        bulk_load(sSF + 1024, p.sfb, 1024, &bar_load);
      }
    }
    // operands that live in tensor memory are written by the thread that owns the row (lane = row)
    const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
    if (a_tmem) {
      uint32_t w[32];
      const uint32_t* src = reinterpret_cast<const uint32_t*>(p.a + (size_t)tid * 128);
#pragma unroll
      for (int i = 0; i < 32; ++i) w[i] = src[i];
      FL_TMEM_ST_32(lane_addr + ST_COL_A, w);
    }
    if (scaled8) {
      uint32_t wa[4], wb[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        wa[c] = *reinterpret_cast<const uint32_t*>(p.sfa + (size_t)(32 * c + lane) * 4);
        wb[c] = *reinterpret_cast<const uint32_t*>(p.sfb + (size_t)(32 * c + lane) * 4);
      }
      FL_TMEM_ST_4(lane_addr + ST_COL_SFA, wa);
      FL_TMEM_ST_4(lane_addr + ST_COL_SFB, wb);
    }
    tc_wait_st();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      if (mbar_wait(&bar_load, 0, p.ctl, &abort_s, 2)) {
        const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
        if (nvf4) {
          // scale atoms: 32 rows x 16 B, no swizzle, 8-row core matrices 128 B apart
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            tmem_cp_sf_atom(tmem + ST_COL_SFA + 4 * i, smem_desc(smem_u32(sSF) + 512 * i, 0, 128, SWZ_NONE));
            tmem_cp_sf_atom(tmem + ST_COL_SFB + 4 * i, smem_desc(smem_u32(sSF) + 1024 + 512 * i, 0, 128, SWZ_NONE));
          }
          // rows of 64 bytes (128 E2M1), 64 B swizzle; K = 64 elements = 32 bytes per instruction
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            if (hi64) {
              // N = 64: rows 64..127 of the B tile (4 KB further down); their scales are columns 2, 3 of each atom
              umma_nvf4_ss(tmem + ST_COL_D, smem_desc(a0 + 32 * k, 16, 512, SWZ_64),
                           smem_desc(b0 + 4096 + 32 * k, 16, 512, SWZ_64), idesc_bs(128, 64, 1, 1, 0, 0, 0, 0, 0),
                           tmem + ST_COL_SFA + 4 * k, tmem + ST_COL_SFB + 4 * k + 2, k > 0);
            } else {
              umma_nvf4_ss(tmem + ST_COL_D, smem_desc(a0 + 32 * k, 16, 512, SWZ_64), smem_desc(b0 + 32 * k, 16, 512, SWZ_64),
                           idesc_bs(128, 128, 1, 1, 0, 0, 0, 0, 0), tmem + ST_COL_SFA + 4 * k, tmem + ST_COL_SFB + 4 * k,
                           k > 0);
            }
          }
        } else if (a2) {
#pragma unroll
          for (int k = 0; k < 4; ++k)   // A MN-major: 32 K rows of 64 B per step, second M block 8 KB further (leading byte offset)
            umma_mxf8_ss(tmem + ST_COL_D, smem_desc(a0 + 2048 * k, 8192, 512, SWZ_64),
                         smem_desc(b0 + 2048 * k, 16, 512, SWZ_64), idesc_bs(128, 64, 0, 0, 1, 1, 1, k, k),
                         tmem + ST_COL_SFA, tmem + ST_COL_SFB, k > 0);
        } else if (dqt) {
#pragma unroll
          for (int k = 0; k < 4; ++k)   // A: 32 K rows of 128 B further down; B: 32 K rows of 64 B (64 B swizzle, 512 B atoms)
            umma_mxf8_ss(tmem + ST_COL_D, smem_desc(a0 + 4096 * k, 16, 1024, SWZ_128),
                         smem_desc(b0 + 2048 * k, 16, 512, SWZ_64), idesc_bs(128, 64, 0, 0, 1, 1, 1, k, k),
                         tmem + ST_COL_SFA, tmem + ST_COL_SFB, k > 0);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // K-major: 32 bytes further along the 128-byte row; MN-major: 32 rows (4 KB) further down
            const uint64_t ad_k = smem_desc(a0 + 32 * k, 16, 1024, SWZ_128);
            const uint64_t ad_mn = smem_desc(a0 + 4096 * k, 16, 1024, SWZ_128);
            const uint64_t bd_k = smem_desc(b0 + 32 * k, 16, 1024, SWZ_128);
            const uint64_t bd_mn = smem_desc(b0 + 4096 * k, 16, 1024, SWZ_128);
            const uint32_t acc = k > 0;
            switch (which) {
              case FL_ST_F8_KMAJOR:
                umma_f8_ss(tmem + ST_COL_D, ad_k, bd_k, idesc_f8(128, 128, 0, 0), acc);
                break;
              case FL_ST_F8_B_MNMAJOR:
                umma_f8_ss(tmem + ST_COL_D, ad_k, bd_mn, idesc_f8(128, 128, 0, 1), acc);
                break;
              case FL_ST_F8_A_MNMAJOR:
                umma_f8_ss(tmem + ST_COL_D, ad_mn, bd_k, idesc_f8(128, 128, 1, 0), acc);
                break;
              case FL_ST_F8_A_TMEM:
                umma_f8_ts(tmem + ST_COL_D, tmem + ST_COL_A + 8 * k, bd_mn, idesc_f8(128, 128, 0, 1), acc);
                break;
              case FL_ST_MX8_SS:
                umma_mxf8_ss(tmem + ST_COL_D, ad_k, bd_mn, idesc_bs(128, 128, 0, 0, 0, 1, 1, k, k), tmem + ST_COL_SFA,
                             tmem + ST_COL_SFB, acc);
                break;
              case FL_ST_MX8_TS:
                umma_mxf8_ts(tmem + ST_COL_D, tmem + ST_COL_A + 8 * k, bd_mn, idesc_bs(128, 128, 0, 0, 0, 1, 1, k, k),
                             tmem + ST_COL_SFA, tmem + ST_COL_SFB, acc);
                break;
              default:
                break;
            }
          }
        }
        tc_commit(&bar_mma);
      }
    }
    __syncwarp();
    if (mbar_wait(&bar_mma, 0, p.ctl, &abort_s, 3)) {
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < ((which == FL_ST_MX8_MN_N64 || which == FL_ST_NVF4_N64_HI || which == FL_ST_MX8_A_MN_2X64) ? 2 : 4); ++c) {
        uint32_t v[32];
        FL_TMEM_LD_32(lane_addr + ST_COL_D + 32 * c, v);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) p.d[(size_t)tid * 128 + 32 * c + i] = __uint_as_float(v[i]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace fl

extern "C" int fl_selftest_mma(int32_t which, const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                               float* d, int32_t* status, int64_t wait_cycles, void* stream) {
  using namespace fl;
  if (which < 0 || which > FL_ST_MX8_A_MN_2X64 || !status) return FL_ERR_BAD_ARG;
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return FL_ERR_CUDA;
  CUtensorMap ma, mb;
  const bool nvf4 = which == FL_ST_NVF4 || which == FL_ST_NVF4_N64_HI;
  if (which != FL_ST_WAIT_TIMEOUT) {
    if (!a || !b || !d) return FL_ERR_BAD_ARG;
    const cuuint64_t rowb = nvf4 ? 64 : 128;
    cuuint64_t dims[2] = {rowb, 128};
    cuuint64_t strides[1] = {rowb};
    cuuint32_t box[2] = {(cuuint32_t)rowb, 128};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = nvf4 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
    const bool a2x64 = which == FL_ST_MX8_A_MN_2X64;
    if (a2x64) box[0] = 64;
    if (enc(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(a), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, a2x64 ? CU_TENSOR_MAP_SWIZZLE_64B : sw, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return FL_ERR_CUDA;
    box[0] = (cuuint32_t)rowb;
    const bool b64 = which == FL_ST_MX8_MN_N64 || which == FL_ST_MX8_A_MN_2X64;     // B tile with 64-byte rows
    if (b64) { dims[0] = 64; strides[0] = 64; box[0] = 64; }
    if (enc(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(b), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, b64 ? CU_TENSOR_MAP_SWIZZLE_64B : sw, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return FL_ERR_CUDA;
  } else {
    memset(&ma, 0, sizeof(ma));
    memset(&mb, 0, sizeof(mb));
  }
  SelfTestParams p;
  p.a = a; p.b = b; p.sfa = sfa; p.sfb = sfb; p.d = d; p.which = which;
  p.ctl.status = status;
  p.ctl.wait_cycles = wait_cycles > 0 ? wait_cycles : kDefaultWaitCycles;
  const int smem = 32768 + 2048 + 1024;
  if (cudaFuncSetAttribute(selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return FL_ERR_CUDA;
  selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? FL_OK : FL_ERR_CUDA;
}
