// sm_100a building blocks: mbarrier, TMA (cp.async.bulk.tensor, never multicast), tcgen05 (TMEM allocation, UMMA issue,
// TMEM load / store / copy), shared-memory and instruction descriptors, and the bounded-wait protocol.
//
// Every wait in this library is bounded: a spin that exceeds its cycle budget records a code in the kernel's global
// status word, raises the CTA's abort flag and returns false; the caller unwinds to the common exit where TMEM is
// released. A kernel therefore always terminates and the host reads the status word through fl_read_status().
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fl {

// ---------------------------------------------------------------------------------------------------- status codes
enum : int {
  FL_OK = 0,
  FL_ERR_BAD_ARG = 1,
  FL_ERR_CUDA = 2,
  FL_ERR_UNSUPPORTED = 3,
  FL_ERR_TOO_LARGE = 4,
  // device-side (written to the status word by a bounded wait): 0x100 | site
  FL_DEV_WAIT_TIMEOUT = 0x100,
  // a packed-document table entry that does not fit the buffer (start negative, not a multiple of 128 or past the end,
  // or start + length past the end): the entry is clamped, nothing out of bounds is touched, and this code is recorded
  FL_DEV_BAD_TABLE = 0x200,
};

struct DevCtl {
  int* status;              // global status word (0 = ok)
  long long wait_cycles;    // budget of one wait
};

// One entry of a packed-document table, made safe: a start that is not a tile-aligned row of the buffer gives an empty
// document, a length that runs past the buffer is cut; either way the status word says so.
__device__ __forceinline__ void doc_entry(const int32_t* doc_start, const int32_t* doc_len, int i, int total, int* status,
                                          int& start, int& len) {
  start = doc_start[i];
  len = doc_len[i];
  const bool bad_start = start < 0 || (start & 127) != 0 || start >= total;
  if (bad_start || len < 0 || len > total - start) {
    if (status) atomicCAS(status, 0, FL_DEV_BAD_TABLE);
    if (bad_start) { start = 0; len = 0; }
    else len = max(0, min(len, total - start));
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. `abort` is a CTA-shared int; `site` identifies the wait for the status word.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const DevCtl& ctl, volatile int* abort,
                                          int site) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xFF) == 0) {
      if (*abort) return false;
      if (clock64() - t0 > ctl.wait_cycles) {
        *abort = 1;
        if (ctl.status) atomicCAS(ctl.status, 0, FL_DEV_WAIT_TIMEOUT | site);
        return false;
      }
    }
  }
  return true;
}

// Warp-level forms for a CONVERGED warp: one lane polls / arrives for the warp (32 lanes polling the same mbarrier
// serialise in the barrier unit and cost hundreds of cycles per wait). __syncwarp orders the other lanes' accesses.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, const DevCtl& ctl, volatile int* abort,
                                               int site) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, ctl, abort, site) ? 1 : 0;
  return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
}
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* src, int x, int y, int z, int w) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, const void* src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// plain (untiled) bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// one lane of a converged warp (the others skip); the UMMA issuer keeps the whole warp converged around its waits and
// address arithmetic so that those stay warp-uniform, and elects a lane only for the issue itself
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], dense 8-bit float kind
__device__ __forceinline__ void umma_f8_ss(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_f8_ts(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d),
      "r"(a), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// block-scaled MXFP8 (UE8M0 scale per 32 along K)
__device__ __forceinline__ void umma_mxf8_ss(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                             uint32_t sfb, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_mxf8_ts(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                             uint32_t sfb, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], [%1], %2, %3, [%4], [%5], p;\n\t}" ::"r"(
          d),
      "r"(a), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
      : "memory");
}
// block-scaled NVFP4 (E2M1 codes, UE4M3 scale per 16 along K; K = 64 per instruction)
__device__ __forceinline__ void umma_nvf4_ss(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                             uint32_t sfb, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
      : "memory");
}
// 512-byte scale-factor atom (128 rows x 4 bytes, 32 x 16 B) from shared memory into 4 TMEM columns of all four lane
// quadrants
__device__ __forceinline__ void tmem_cp_sf_atom(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

#define FL_TMEM_ST_16(taddr, v)                                                                                        \
  asm volatile(                                                                                                        \
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, " \
      "%16};" ::"r"(taddr),                                                                                            \
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),     \
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])                                           \
      : "memory")

#define FL_TMEM_LD_32(taddr, v)                                                                                        \
  asm volatile(                                                                                                        \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "  \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                        \
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),     \
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),         \
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),        \
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])                      \
      : "r"(taddr)                                                                                                     \
      : "memory")

#define FL_TMEM_ST_32(taddr, v)                                                                                        \
  asm volatile(                                                                                                        \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, " \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),            \
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),     \
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),      \
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),      \
      "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])                                                                   \
      : "memory")

#define FL_TMEM_ST_8(taddr, v)                                                                                         \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),           \
               "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])                   \
               : "memory")

#define FL_TMEM_ST_4(taddr, v)                                                                                         \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v[0]), "r"(v[1]),     \
               "r"(v[2]), "r"(v[3])                                                                                    \
               : "memory")

// ---------------------------------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor (sm_100 version field = 1). Addresses and offsets in bytes.
//   K-major, swizzled:  rows of SW bytes (SW = 128 / 64 / 32), 8-row atoms; sbo = bytes between 8-row groups.
//   MN-major, swizzled: rows (one per K index) of SW bytes holding SW contiguous MN elements; sbo = bytes between groups
//                       of 8 K rows; lbo = bytes between MN atoms (unused when the tile is one atom wide).
enum : uint64_t { SWZ_128 = 2, SWZ_64 = 4, SWZ_32 = 6, SWZ_NONE = 0 };
__host__ __device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint64_t swz) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46) | (swz << 61);
}
// A descriptor whose start address is `bytes` further (bytes % 16 == 0; the 14-bit address field must not wrap, which
// holds for offsets inside one CTA's shared memory window below 256 KB). The UMMA issuer is a single thread whose own
// instruction latency bounds the tensor pipe's issue rate, so descriptors are built once and only advanced in loops.
__host__ __device__ __forceinline__ uint64_t desc_adv(uint64_t d, uint32_t bytes) { return d + (uint64_t)(bytes >> 4); }
// Instruction descriptor, kind::f8f6f4 with E4M3 x E4M3 -> F32.
__host__ __device__ constexpr uint32_t idesc_f8(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}
// Block-scaled descriptor: a_fmt / b_fmt 0 = E4M3 (mxf8f6f4), 1 = E2M1 (mxf4nvf4); ue8m0 = scale format bit.
__host__ __device__ constexpr uint32_t idesc_bs(int M, int N, int a_fmt, int b_fmt, int a_mn_major, int b_mn_major,
                                                int ue8m0, int sfa_id, int sfb_id) {
  return ((uint32_t)sfb_id << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)ue8m0 << 23) |
         ((uint32_t)(M >> 4) << 24) | ((uint32_t)sfa_id << 29);
}

// ---------------------------------------------------------------------------------------------------- small math
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// max(a, |b|, |c|)
__device__ __forceinline__ float fmax3_abs(float a, float b, float c) {
  float d;
  asm("{\n\t.reg .f32 x, y;\n\tabs.f32 x, %2;\n\tabs.f32 y, %3;\n\tmax.f32 %0, %1, x, y;\n\t}" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^(-x)
__device__ __forceinline__ float ex2_neg(float x) {
  float y;
  asm("{\n\t.reg .f32 t;\n\tneg.f32 t, %1;\n\tex2.approx.ftz.f32 %0, t;\n\t}" : "=f"(y) : "f"(x));
  return y;
}
// Packed pairs of floats in one 64-bit register (fma / add .f32x2: one issue slot for two elements).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for two arguments on the FMA pipe instead of the transcendental unit (one warp instruction per 8 clocks and
// scheduler, shared by the two softmax warpgroups): n = round(x) through the 1.5 * 2^23 trick, f = x - n in [-0.5, 0.5],
// 2^f by a degree-3 polynomial (weighted least-squares fit of the relative error on Chebyshev nodes: max 7.5e-5),
// then n is added into the exponent field. Arguments below -126 give 2^-126.
__device__ __forceinline__ void ex2_poly2(float x0, float x1, float& r0, float& r1) {
  constexpr float MAGIC = 12582912.f;
  const uint64_t x = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t xr = add2(x, pack2(MAGIC, MAGIC));
  const uint64_t n = add2(xr, pack2(-MAGIC, -MAGIC));
  const uint64_t f = fma2(n, pack2(-1.f, -1.f), x);
  uint64_t p = fma2(f, pack2(0.0551716685295105f, 0.0551716685295105f), pack2(0.2426111251115799f, 0.2426111251115799f));
  p = fma2(p, f, pack2(0.6932609677314758f, 0.6932609677314758f));
  p = fma2(p, f, pack2(0.9999280571937561f, 0.9999280571937561f));
  float a0, a1, b0, b1;
  unpack2(p, a0, a1);
  unpack2(xr, b0, b1);
  r0 = __uint_as_float(__float_as_uint(a0) + (__float_as_uint(b0) << 23));
  r1 = __uint_as_float(__float_as_uint(a1) + (__float_as_uint(b1) << 23));
}
// two floats -> two E4M3 bytes (lo in bits 0-7), round to nearest even, saturating
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return (uint32_t)r;
}
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  uint32_t r;      // two conversions and one register pack
  asm("{\n\t.reg .b16 lo, hi;\n\tcvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\tcvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(r)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

}  // namespace fl
