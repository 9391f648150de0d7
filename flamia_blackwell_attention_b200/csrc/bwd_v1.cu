// Backward main kernel for sm_100a, first form (whole 128-query tiles, roles strictly in sequence). Serves head_dim 64;
// head_dim 128 runs the pipelined kernel of bwd.cu.
//
// dK, dV and the pre-scaled f16 dQ accumulator from block-scaled operands.
//
// Replaces the reference's FlashAttentionBackwardSm100FP4 (flash_attn/cute/flash_bwd_sm100_fp4.py:82; driver
// flash_attn/cute/interface_bwd_fp4.py:1207) for the E4M3 backward of both routes. Per (key tile n, query tile m):
//   S^T  = K Q^T            kind::f8f6f4 (token-block factors folded into the exponent argument)
//   P'   = 2^(S^T c - lse_log2) = 2^8 P            -> P-hat = E4M3(P')                  [tensor memory]
//   dV  += P-hat^T dO-hat   kind::mxf8f6f4.block_scale, B scale = dO's UE8M0 per 32 queries
//   dP^T = V dO^T           kind::f8f6f4
//   dS   = P' (b dP^T + D''), b = f_V f_dO 2^-8, D'' = -2^-8 rowsum(O dO)                (true units)
//   dS-hat: one UE8M0 exponent per 32 keys x 32 queries, E4M3 codes (the same codes feed dK and dQ)
//   dK  += dS-hat^T Q-hat   block-scaled, A from tensor memory, A scale = dS exponent, B scale = Q's
//   dQ_m = dS-hat K-hat     block-scaled, A = dS-hat from shared memory (MN-major), B = K tile (MN-major)
//   dQ_m * B_m -> f16 -> reduce-add into the (b, h, s, d) accumulator with a TMA reduction
//
// One CTA per (128-key tile, kv head, batch | document); it loops over the query tiles that see the key tile and over
// the query heads of the GQA group, keeping dK / dV in tensor memory.
//   warps 0-3 / 4-7  compute (thread = key row; the two warpgroups split the 128 query columns)
//   warps 8-11       dQ reduction (thread = query row)          warp 12 UMMA issuer      warp 13 TMA producer
// TMEM: [0,128) S^T, then P-hat [0,32), dS-hat [32,64), scale tiles [64,88); [128,256) dV; [256,384) dP^T, then dQ_m;
// [384,512) dK.  Every wait is bounded (sm100.cuh).
#include "flamia_internal.h"

namespace fl {
namespace v1 {

struct BwdParams {
  const float* fac_q;
  const float* fac_k;
  const float* fac_v;
  const float* fac_do;
  const float* lse_log2;
  const float* d_rows;
  const float* dq_scale;
  void* dk;
  void* dv;
  const int32_t* doc_start;
  const int32_t* doc_len;
  int n_docs;
  int b, s_q, s_k, h, h_kv;
  float scale_log2;
  float softmax_scale;
  int causal;
  int win_l, win_r;      // sliding window sides, -1 = unlimited (causal: the right side is 0)
  int out_f16;
  int had_dk;
  DevCtl ctl;
};

struct BTile {
  int bat;     // batch coordinate of the tensor maps
  int k0;      // first key row of this CTA (row inside the batch entry)
  int nk;      // valid keys of the tile (<= 128)
  int krel;    // document-relative index of key row k0
  int q0;      // first query row of the document
  int sq;      // queries of the document
  int off;     // key j visible to query i iff j <= i + off (document-relative)
};

enum { BB_KV = 0, BB_QFULL = 1, BB_QEMPTY = 3, BB_S = 5, BB_DP = 6, BB_P = 7, BB_DS = 8, BB_DQFULL = 9, BB_DQEMPTY = 10,
       BB_ACC = 11, BB_X1 = 12, BB_X2 = 13, BB_R1 = 14, BB_R2 = 15, BB_COUNT = 16 };

// TMEM columns
enum { TC_S = 0, TC_P = 0, TC_DS = 32, TC_SFA_P = 64, TC_SFB_DO = 68, TC_SFA_DK = 72, TC_SFB_Q = 76, TC_SFA_DQ = 80,
       TC_SFB_K = 84, TC_DV = 128, TC_DP = 256, TC_DQ = 256, TC_DK = 384 };

__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
  uint32_t r;
  asm volatile("redux.sync.max.u32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
  return r;
}
template <int N>
__device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

template <int D>
__global__ void __launch_bounds__(512, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
           const __grid_constant__ CUtensorMap tm_acc, const BwdParams p) {
  constexpr int TILE_BYTES = 128 * D;
  constexpr uint64_t SWZ = (D == 128) ? SWZ_128 : SWZ_64;
  constexpr uint32_t SBO = 8 * D;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                                  // 1 tile
  uint8_t* sV = sK + TILE_BYTES;                       // 1 tile
  uint8_t* sQ = sV + TILE_BYTES;                       // 2 stages
  uint8_t* sDO = sQ + 2 * TILE_BYTES;                  // 2 stages
  uint8_t* sDS = sDO + 2 * TILE_BYTES;                 // 128 key rows x 128 query bytes (MN-major A of the dQ product)
  uint8_t* sDQ = sDS + 16384;                          // f16 staging of the dQ tile: D/64 boxes of 128 rows x 128 B
  float* sVec = reinterpret_cast<float*>(sDQ + 128 * D * 2);   // 2 stages x {lse_log2[128], D''[128]}
  __shared__ __align__(8) uint64_t bars[BB_COUNT];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ BTile tile_s;
  __shared__ uint32_t sE[4];                           // dS exponent bytes: sE[key block] = bytes of query blocks 0..3

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // causal: grid = (kv heads, batch rows, key tiles), so key tiles with the same number of query tiles are dispatched
  // together, longest first. Otherwise grid = (key tiles, kv heads, batch rows): the CTAs of one head run together and
  // share its Q / dO tiles in L2.
  const int hkv = p.causal ? blockIdx.x : blockIdx.y;
  const int tile_id = p.causal ? blockIdx.z : blockIdx.x, bat_id = p.causal ? blockIdx.y : blockIdx.z;
  const int grp = p.h / p.h_kv;

  if (tid == 0) {
    abort_s = 0;
    mbar_init(&bars[BB_KV], 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[BB_QFULL + i], 1); mbar_init(&bars[BB_QEMPTY + i], 1); }
    mbar_init(&bars[BB_S], 1);
    mbar_init(&bars[BB_DP], 1);
    mbar_init(&bars[BB_P], 256);
    mbar_init(&bars[BB_DS], 256);
    mbar_init(&bars[BB_DQFULL], 1);
    mbar_init(&bars[BB_DQEMPTY], 128);
    mbar_init(&bars[BB_ACC], 1);
    mbar_init(&bars[BB_X1], 256);
    mbar_init(&bars[BB_X2], 256);
    mbar_init(&bars[BB_R1], 128);
    mbar_init(&bars[BB_R2], 128);
    fence_barrier_init();
    BTile t;
    if (p.doc_start == nullptr) {
      t.bat = bat_id; t.k0 = tile_id * 128; t.nk = min(128, p.s_k - t.k0); t.krel = t.k0; t.q0 = 0; t.sq = p.s_q;
      t.off = p.s_k - p.s_q;
    } else {
      int x = tile_id, dsel = -1;
      for (int dI = 0; dI < p.n_docs; ++dI) {
        const int nb = (p.doc_len[dI] + 127) / 128;
        if (x < nb) { dsel = dI; break; }
        x -= nb;
      }
      if (dsel < 0) { t.nk = 0; t.bat = 0; t.k0 = 0; t.krel = 0; t.q0 = 0; t.sq = 0; t.off = 0; }
      else {
        const int len = p.doc_len[dsel], st = p.doc_start[dsel];
        t.bat = 0; t.k0 = st + x * 128; t.nk = min(128, len - x * 128); t.krel = x * 128; t.q0 = st; t.sq = len; t.off = 0;
      }
    }
    tile_s = t;
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const BTile T = tile_s;
  volatile int* abortp = &abort_s;

  // query tiles that see this key tile: m in [m_lo, m_hi)
  int m_hi = (T.sq + 127) / 128;
  int m_lo = 0;
  if (p.win_r >= 0 && T.krel - T.off - p.win_r > 0) m_lo = (T.krel - T.off - p.win_r) / 128;
  if (p.win_l >= 0) m_hi = min(m_hi, max(0, T.krel + T.nk - 1 - T.off + p.win_l) / 128 + 1);
  const int n_m = (T.nk > 0 && m_hi > m_lo) ? (m_hi - m_lo) : 0;
  const int n_it = n_m * grp;                                // iterations: query heads of the group x query tiles
  const bool early_out = (T.nk <= 0) || (*p.ctl.status != 0);

  if (!early_out) {
    if (warp >= 12) reg_dealloc<48>();       // the whole warpgroup 12-15 gives its registers back
    if (warp == 13) {
      // =================================================================== TMA producer
      if (lane == 0) {
        tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_do);
        mbar_arrive_expect_tx(&bars[BB_KV], 2 * TILE_BYTES);
        tma_load_4d(sK, &tm_k, &bars[BB_KV], 0, hkv, T.k0, T.bat);
        tma_load_4d(sV, &tm_v, &bars[BB_KV], 0, hkv, T.k0, T.bat);
        for (int it = 0; it < n_it; ++it) {
          const int st = it & 1, u = it >> 1;
          const int head = hkv * grp + it / n_m, m = m_lo + it % n_m;
          if (it >= 2 && !mbar_wait(&bars[BB_QEMPTY + st], (u & 1) ^ 1, p.ctl, abortp, 10)) break;
          mbar_arrive_expect_tx(&bars[BB_QFULL + st], 2 * TILE_BYTES + 1024);
          tma_load_4d(sQ + st * TILE_BYTES, &tm_q, &bars[BB_QFULL + st], 0, head, T.q0 + m * 128, T.bat);
          tma_load_4d(sDO + st * TILE_BYTES, &tm_do, &bars[BB_QFULL + st], 0, head, T.q0 + m * 128, T.bat);
          const size_t ro = ((size_t)T.bat * p.h + head) * p.s_q + T.q0 + m * 128;
          bulk_load(sVec + st * 256, p.lse_log2 + ro, 512, &bars[BB_QFULL + st]);
          bulk_load(sVec + st * 256 + 128, p.d_rows + ro, 512, &bars[BB_QFULL + st]);
        }
      }
    } else if (warp == 12) {
      // =================================================================== UMMA issuer
      // The whole warp stays converged through the waits and the descriptor arithmetic (warp-uniform values); one elected
      // lane issues. Descriptors are built once; the loop only adds byte offsets (the issuing thread's own instruction
      // latency is what bounds the tensor pipe's issue rate).
      {
        constexpr uint32_t ID_KK = idesc_f8(128, 128, 0, 0);
        const uint32_t tm = __shfl_sync(0xFFFFFFFFu, tmem, 0);
        const int nit = __shfl_sync(0xFFFFFFFFu, n_it, 0);
        const uint64_t dK0 = smem_desc(smem_u32(sK), 16, SBO, SWZ), dV0 = smem_desc(smem_u32(sV), 16, SBO, SWZ),
                       dQ0 = smem_desc(smem_u32(sQ), 16, SBO, SWZ), dDO0 = smem_desc(smem_u32(sDO), 16, SBO, SWZ),
                       dDS0 = smem_desc(smem_u32(sDS), 16, 1024, SWZ_128);
        bool ok = mbar_wait(&bars[BB_KV], 0, p.ctl, abortp, 20);
        for (int it = 0; ok && it < nit; ++it) {
          const int st = it & 1, u = it >> 1;
          const uint64_t dQs = desc_adv(dQ0, st * TILE_BYTES), dDOs = desc_adv(dDO0, st * TILE_BYTES);
          const uint32_t accum = it > 0;
          if (!(ok = mbar_wait(&bars[BB_QFULL + st], u & 1, p.ctl, abortp, 21))) break;
          tc_fence_after();
          if (elect_one()) {   // S^T = K Q^T
#pragma unroll
            for (int k = 0; k < D / 32; ++k) umma_f8_ss(tm + TC_S, desc_adv(dK0, 32 * k), desc_adv(dQs, 32 * k), ID_KK, k > 0);
            tc_commit(&bars[BB_S]);
          }
          __syncwarp();
          // dP^T = V dO^T (its columns are the previous dQ tile's: wait until that one has been read out)
          if (it > 0 && !(ok = mbar_wait(&bars[BB_DQEMPTY], (it - 1) & 1, p.ctl, abortp, 22))) break;
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < D / 32; ++k) umma_f8_ss(tm + TC_DP, desc_adv(dV0, 32 * k), desc_adv(dDOs, 32 * k), ID_KK, k > 0);
            tc_commit(&bars[BB_DP]);
          }
          __syncwarp();
          // dV += P-hat^T dO-hat
          if (!(ok = mbar_wait(&bars[BB_P], it & 1, p.ctl, abortp, 23))) break;
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_mxf8_ts(tm + TC_DV, tm + TC_P + 8 * kk, desc_adv(dDOs, kk * 32 * D), idesc_bs(128, D, 0, 0, 0, 1, 1, kk, kk),
                           tm + TC_SFA_P, tm + TC_SFB_DO, accum | kk);
          }
          __syncwarp();
          // dK += dS-hat^T Q-hat ; dQ_m = dS-hat K-hat
          if (!(ok = mbar_wait(&bars[BB_DS], it & 1, p.ctl, abortp, 24))) break;
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_mxf8_ts(tm + TC_DK, tm + TC_DS + 8 * kk, desc_adv(dQs, kk * 32 * D), idesc_bs(128, D, 0, 0, 0, 1, 1, kk, kk),
                           tm + TC_SFA_DK, tm + TC_SFB_Q, accum | kk);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_mxf8_ss(tm + TC_DQ, desc_adv(dDS0, kk * 4096), desc_adv(dK0, kk * 32 * D), idesc_bs(128, D, 0, 0, 1, 1, 1, kk, kk),
                           tm + TC_SFA_DQ, tm + TC_SFB_K, kk > 0);
            tc_commit(&bars[BB_DQFULL]);
            tc_commit(&bars[BB_QEMPTY + st]);
          }
          __syncwarp();
        }
        if (ok && elect_one()) tc_commit(&bars[BB_ACC]);
        __syncwarp();
      }
    } else if (warp >= 8 && warp < 12) {
      reg_dealloc<96>();
      // =================================================================== dQ reduction (thread = query row)
      const int r = tid & 127;
      const uint32_t t_dq = tmem + TC_DQ + ((uint32_t)((warp & 3) * 32) << 16);
      bool ok = true;
      for (int it = 0; it < n_it; ++it) {
        const int head = hkv * grp + it / n_m, m = m_lo + it % n_m;
        const float sc = p.dq_scale[(size_t)T.bat * (p.s_q / 128) + (T.q0 / 128) + m];
        if (!(ok = mbar_wait(&bars[BB_DQFULL], it & 1, p.ctl, abortp, 40))) break;
        tc_fence_after();
        // the previous tile's reduction must have finished reading the staging buffer
        if (tid == 256) tma_store_wait_read<0>();
        mbar_arrive(&bars[BB_R1]);
        if (!(ok = mbar_wait(&bars[BB_R1], it & 1, p.ctl, abortp, 41))) break;
#pragma unroll 1
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t v[32];
          FL_TMEM_LD_32(t_dq + 32 * cc, v);
          tc_wait_ld();
          // 32 f32 -> 32 f16 = 64 bytes = 4 chunks of 16 B inside box (cc / 2), swizzled by the row
          uint8_t* box = sDQ + (cc >> 1) * 16384 + r * 128;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __half2 hh = __floats2half2_rn(__uint_as_float(v[8 * q4 + 2 * e]) * sc, __uint_as_float(v[8 * q4 + 2 * e + 1]) * sc);
              w[e] = *reinterpret_cast<uint32_t*>(&hh);
            }
            const int chunk = ((cc & 1) * 4 + q4) ^ (r & 7);
            *reinterpret_cast<uint4*>(box + chunk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        tc_fence_before();
        mbar_arrive(&bars[BB_DQEMPTY]);
        fence_proxy_async();
        mbar_arrive(&bars[BB_R2]);
        if (!(ok = mbar_wait(&bars[BB_R2], it & 1, p.ctl, abortp, 42))) break;
        if (tid == 256) {
#pragma unroll
          for (int bx = 0; bx < D / 64; ++bx)
            tma_reduce_add_4d(&tm_acc, sDQ + bx * 16384, bx * 64, T.q0 + m * 128, head, T.bat);
          tma_store_commit();
        }
      }
      if (tid == 256) tma_store_wait<0>();
    } else if (warp < 8) {
      reg_alloc<184>();
      // =================================================================== compute (thread = key row)
      const int hc = warp >> 2;                        // which half of the 128 query columns
      const int wq = warp & 3;                         // lane quadrant = 32-key block of the tile
      const int r = wq * 32 + lane;                    // key row of the tile = TMEM lane
      const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16);
      const int krel = T.krel + r;
      const bool key_valid = r < T.nk;
      const size_t bh_k = (size_t)T.bat * p.h_kv + hkv;
      const int kblk = (T.k0 + r) / 32;
      const float fk = p.fac_k[bh_k * (p.s_k / 32) + kblk] * p.scale_log2;
      const float fv8 = p.fac_v[bh_k * (p.s_k / 32) + kblk] * 0.00390625f;   // f_V 2^-8
      uint32_t ek_word = 0;                            // UE8M0 bytes of the tile's four key blocks (B scale of dQ)
#pragma unroll
      for (int kb = 0; kb < 4; ++kb)
        ek_word |= ((__float_as_uint(p.fac_k[bh_k * (p.s_k / 32) + T.k0 / 32 + kb]) >> 23) & 0xFF) << (8 * kb);
      bool ok = true;
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1, u = it >> 1;
        const int head = hkv * grp + it / n_m, m = m_lo + it % n_m;
        const size_t bh_q = (size_t)T.bat * p.h + head;
        const float* fq_t = p.fac_q + bh_q * (p.s_q / 32) + (T.q0 + m * 128) / 32;
        const float* fdo_t = p.fac_do + bh_q * (p.s_q / 32) + (T.q0 + m * 128) / 32;
        float c[2], b8[2];
        uint32_t eq_word = 0, edo_word = 0;
#pragma unroll
        for (int qb = 0; qb < 4; ++qb) {
          const float fqv = fq_t[qb], fdv = fdo_t[qb];
          eq_word |= ((__float_as_uint(fqv) >> 23) & 0xFF) << (8 * qb);
          edo_word |= ((__float_as_uint(fdv) >> 23) & 0xFF) << (8 * qb);
          if ((qb >> 1) == hc) { c[qb & 1] = fk * fqv; b8[qb & 1] = fv8 * fdv; }
        }
        if (!(ok = mbar_wait(&bars[BB_QFULL + st], u & 1, p.ctl, abortp, 30))) break;   // lse / D'' vectors visible
        const float* lse2 = sVec + st * 256 + hc * 64;
        const float* dpp = sVec + st * 256 + 128 + hc * 64;
        // element (key r, query column hc*64 + j) is live iff the key is valid, the query exists and sees the key
        const int q_first = m * 128 + hc * 64;                            // document-relative query of column 0
        const int vis_from = p.win_r >= 0 ? (krel - T.off - p.win_r) : 0;  // queries in [vis_from, vis_to] see this key
        const int vis_to = p.win_l >= 0 ? (krel - T.off + p.win_l) : 0x7FFFFFFF;
        const bool full = key_valid && (q_first >= vis_from) && (q_first + 63 <= vis_to) && (q_first + 64 <= T.sq);

        if (!(ok = mbar_wait(&bars[BB_S], it & 1, p.ctl, abortp, 31))) break;
        tc_fence_after();
        uint32_t pv[64];
        FL_TMEM_LD_32(lane_base + TC_S + hc * 64, pv);
        FL_TMEM_LD_32(lane_base + TC_S + hc * 64 + 32, (pv + 32));
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(&bars[BB_X1]);       // every S^T column has been read: its tensor-memory columns may be rewritten
        if (!(ok = mbar_wait(&bars[BB_X1], it & 1, p.ctl, abortp, 35))) break;
        tc_fence_after();
        float pf[64];
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          float x = fmaf(__uint_as_float(pv[j]), c[j >> 5], -lse2[j]);
          float e = ex2(x);
          if (!full) {
            const int qi = q_first + j;
            e = (key_valid && qi >= vis_from && qi <= vis_to && qi < T.sq) ? e : 0.f;
          }
          pf[j] = e;
        }
        {
          uint32_t pw[16];
#pragma unroll
          for (int w = 0; w < 16; ++w) pw[w] = cvt_e4m3x4(pf[4 * w], pf[4 * w + 1], pf[4 * w + 2], pf[4 * w + 3]);
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
              "%15, %16};" ::"r"(lane_base + TC_P + hc * 16),
              "r"(pw[0]), "r"(pw[1]), "r"(pw[2]), "r"(pw[3]), "r"(pw[4]), "r"(pw[5]), "r"(pw[6]), "r"(pw[7]), "r"(pw[8]),
              "r"(pw[9]), "r"(pw[10]), "r"(pw[11]), "r"(pw[12]), "r"(pw[13]), "r"(pw[14]), "r"(pw[15])
              : "memory");
          if (hc == 0) {   // scale tiles of the dV product: A = 1, B = dO's exponent per 32 queries
            uint32_t sf[8] = {0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, edo_word, edo_word, edo_word, edo_word};
            FL_TMEM_ST_8(lane_base + TC_SFA_P, sf);
          }
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&bars[BB_P]);

        // ---- dS = P' (b dP + D''), block exponent per (this warp's 32 keys, 32 queries)
        if (!(ok = mbar_wait(&bars[BB_DP], it & 1, p.ctl, abortp, 32))) break;
        tc_fence_after();
        FL_TMEM_LD_32(lane_base + TC_DP + hc * 64, pv);
        FL_TMEM_LD_32(lane_base + TC_DP + hc * 64 + 32, (pv + 32));
        tc_wait_ld();
        uint32_t ebyte[2];
#pragma unroll
        for (int qh = 0; qh < 2; ++qh) {
          float am = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int jj = qh * 32 + j;
            const float ds = pf[jj] * fmaf(__uint_as_float(pv[jj]), b8[qh], dpp[jj]);
            pf[jj] = ds;
            am = fmaxf(am, fabsf(ds));
          }
          const uint32_t wm = warp_max_u32(__float_as_uint(am));          // non-negative floats order as integers
          int e = (int)((wm + 0x00200000u) >> 23) - 8;                     // smallest e with 448 * 2^(e-127) >= amax
          e = max(e, 1);
          e = min(e, 254);
          ebyte[qh] = (uint32_t)e;
        }
        if (lane == 0) {
          // sE[key block] holds the bytes of query blocks 0..3; this warp owns two of them
          uint16_t two = (uint16_t)(ebyte[0] | (ebyte[1] << 8));
          reinterpret_cast<uint16_t*>(&sE[wq])[hc] = two;
        }
        uint32_t dsw[16];
#pragma unroll
        for (int qh = 0; qh < 2; ++qh) {
          const float inv = __uint_as_float((uint32_t)(254 - (int)ebyte[qh]) << 23);   // 2^(127 - e)
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            const int j0 = qh * 32 + 4 * w;
            dsw[qh * 8 + w] = cvt_e4m3x4(pf[j0] * inv, pf[j0 + 1] * inv, pf[j0 + 2] * inv, pf[j0 + 3] * inv);
          }
        }
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
            "%15, %16};" ::"r"(lane_base + TC_DS + hc * 16),
            "r"(dsw[0]), "r"(dsw[1]), "r"(dsw[2]), "r"(dsw[3]), "r"(dsw[4]), "r"(dsw[5]), "r"(dsw[6]), "r"(dsw[7]),
            "r"(dsw[8]), "r"(dsw[9]), "r"(dsw[10]), "r"(dsw[11]), "r"(dsw[12]), "r"(dsw[13]), "r"(dsw[14]), "r"(dsw[15])
            : "memory");
        {   // the same codes as the MN-major A operand of dQ_m: row = key, 64 bytes = 4 chunks of 16 B, 128 B swizzle
          uint8_t* rowp = sDS + r * 128;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int chunk = (hc * 4 + q4) ^ (r & 7);
            *reinterpret_cast<uint4*>(rowp + chunk * 16) =
                make_uint4(dsw[4 * q4], dsw[4 * q4 + 1], dsw[4 * q4 + 2], dsw[4 * q4 + 3]);
          }
        }
        mbar_arrive(&bars[BB_X2]);       // all eight warps have published their exponent bytes
        if (!(ok = mbar_wait(&bars[BB_X2], it & 1, p.ctl, abortp, 36))) break;
        if (hc == 1) {
          // scale tiles: dK: A[key lane, column = key block] = bytes over query blocks; B = Q's exponents
          //              dQ: A[query lane, column = query block] = bytes over key blocks;  B = K's exponents
          const uint32_t e0 = sE[0], e1 = sE[1], e2 = sE[2], e3 = sE[3];
          uint32_t sf[16];
          sf[0] = e0; sf[1] = e1; sf[2] = e2; sf[3] = e3;
          sf[4] = sf[5] = sf[6] = sf[7] = eq_word;
#pragma unroll
          for (int qb = 0; qb < 4; ++qb)
            sf[8 + qb] = ((e0 >> (8 * qb)) & 0xFF) | (((e1 >> (8 * qb)) & 0xFF) << 8) | (((e2 >> (8 * qb)) & 0xFF) << 16) |
                         (((e3 >> (8 * qb)) & 0xFF) << 24);
          sf[12] = sf[13] = sf[14] = sf[15] = ek_word;
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
              "%15, %16};" ::"r"(lane_base + TC_SFA_DK),
              "r"(sf[0]), "r"(sf[1]), "r"(sf[2]), "r"(sf[3]), "r"(sf[4]), "r"(sf[5]), "r"(sf[6]), "r"(sf[7]), "r"(sf[8]),
              "r"(sf[9]), "r"(sf[10]), "r"(sf[11]), "r"(sf[12]), "r"(sf[13]), "r"(sf[14]), "r"(sf[15])
              : "memory");
        }
        tc_wait_st();
        fence_proxy_async();             // the dS-hat tile in shared memory is read by the tensor core (async proxy)
        tc_fence_before();
        mbar_arrive(&bars[BB_DS]);
      }
      // ---- epilogue: warpgroup 0 writes dV, warpgroup 1 writes dK (full rows)
      if (ok && n_it > 0) ok = mbar_wait(&bars[BB_ACC], 0, p.ctl, abortp, 33);
      if (ok) {
        tc_fence_after();
        const uint32_t t_acc = lane_base + (hc == 0 ? TC_DV : TC_DK);
        const float mult = (hc == 0) ? 0.00390625f : p.softmax_scale;      // dV carries 2^8 (P'), dK the softmax scale
        float y[D];
        if (n_it > 0) {
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t v[32];
            FL_TMEM_LD_32(t_acc + 32 * cc, v);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) y[32 * cc + e] = __uint_as_float(v[e]) * mult;
          }
        } else {
#pragma unroll
          for (int e = 0; e < D; ++e) y[e] = 0.f;
        }
        if constexpr (D == 128) {
          if (hc == 1 && p.had_dk) {      // dK of rotated operands: (y H / sqrt(128)) * signs
#pragma unroll
            for (int hs = 1; hs < 128; hs <<= 1) {
#pragma unroll
              for (int i = 0; i < 128; ++i) {
                if ((i & hs) == 0) {
                  const float a = y[i], b2 = y[i + hs];
                  y[i] = a + b2;
                  y[i + hs] = a - b2;
                }
              }
            }
            constexpr uint32_t NEG[4] = {0x10D2E03Eu, 0xE0D9F0E2u, 0x45809F07u, 0x75954FEDu};
#pragma unroll
            for (int i = 0; i < 128; ++i) {
              y[i] *= 0.08838834764831845f;
              if ((NEG[i >> 5] >> (i & 31)) & 1) y[i] = -y[i];
            }
          }
        }
        if (key_valid) {
          uint16_t* orow = reinterpret_cast<uint16_t*>(hc == 0 ? p.dv : p.dk) +
                           (((size_t)T.bat * p.s_k + T.k0 + r) * p.h_kv + hkv) * D;
#pragma unroll
          for (int c8 = 0; c8 < D / 8; ++c8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float a = y[8 * c8 + 2 * e], b2 = y[8 * c8 + 2 * e + 1];
              if (p.out_f16) {
                __half2 hh = __floats2half2_rn(a, b2);
                w[e] = *reinterpret_cast<uint32_t*>(&hh);
              } else {
                w[e] = pack_bf16x2(a, b2);
              }
            }
            *reinterpret_cast<uint4*>(orow + 8 * c8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  if (abort_s) {
    for (int it = 0; it < 200; ++it) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace v1
}  // namespace fl

int fl_bwd_v1(const fl_attn_args* a, void* stream) {
  using namespace fl;
  using namespace fl::v1;
  if (!a || !a->q_codes || !a->k_codes || !a->v_codes || !a->do_codes || !a->status) return FL_ERR_BAD_ARG;
  if (!a->fac_q || !a->fac_k || !a->fac_v || !a->fac_do || !a->lse_log2 || !a->d_rows || !a->dq_acc || !a->dq_scale ||
      !a->dk || !a->dv)
    return FL_ERR_BAD_ARG;
  if (a->d != 64 && a->d != 128) return FL_ERR_UNSUPPORTED;
  if (a->mode != FL_MODE_FP8) return FL_ERR_UNSUPPORTED;
  if (a->flags & (FL_A_TOKEN_LOCAL | FL_A_DQ_ROWLOCAL)) return FL_ERR_UNSUPPORTED;
  if (a->h <= 0 || a->h_kv <= 0 || a->h % a->h_kv) return FL_ERR_BAD_ARG;
  if ((a->s_q % 128) || (a->s_k % 128) || a->s_q <= 0 || a->s_k <= 0 || a->b <= 0) return FL_ERR_BAD_ARG;
  if (a->doc_start && (a->b != 1 || a->n_docs <= 0 || !a->doc_len || a->s_q != a->s_k)) return FL_ERR_BAD_ARG;
  CUtensorMap mq, mk, mv, mdo, macc;
  int rc;
  if ((rc = make_rows_map(&mq, a->q_codes, a->b, a->s_q, a->h, a->d, 128))) return rc;
  if ((rc = make_rows_map(&mk, a->k_codes, a->b, a->s_k, a->h_kv, a->d, 128))) return rc;
  if ((rc = make_rows_map(&mv, a->v_codes, a->b, a->s_k, a->h_kv, a->d, 128))) return rc;
  if ((rc = make_rows_map(&mdo, a->do_codes, a->b, a->s_q, a->h, a->d, 128))) return rc;
  if ((rc = make_acc_map_16(&macc, a->dq_acc, a->b, a->h, a->s_q, a->d, 128))) return rc;
  BwdParams p;
  p.fac_q = a->fac_q; p.fac_k = a->fac_k; p.fac_v = a->fac_v; p.fac_do = a->fac_do; p.lse_log2 = a->lse_log2;
  p.d_rows = a->d_rows; p.dq_scale = a->dq_scale; p.dk = a->dk; p.dv = a->dv;
  p.doc_start = a->doc_start; p.doc_len = a->doc_len; p.n_docs = a->n_docs;
  p.b = a->b; p.s_q = a->s_q; p.s_k = a->s_k; p.h = a->h; p.h_kv = a->h_kv;
  p.softmax_scale = a->softmax_scale;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.causal = (a->flags & FL_A_CAUSAL) ? 1 : 0;
  p.win_l = a->window_left_p1 - 1;
  p.win_r = p.causal ? 0 : a->window_right_p1 - 1;
  p.out_f16 = (a->flags & FL_A_OUT_F16) ? 1 : 0;
  p.had_dk = (a->flags & FL_A_HAD_DK) ? 1 : 0;
  p.ctl.status = a->status;
  p.ctl.wait_cycles = a->wait_cycles > 0 ? a->wait_cycles : kDefaultWaitCycles;
  const int ntile = a->doc_start ? (a->s_k / 128 + a->n_docs) : a->s_k / 128;
  const int nb = a->doc_start ? 1 : a->b;
  dim3 grid = p.causal ? dim3(a->h_kv, nb, ntile) : dim3(ntile, a->h_kv, nb);
  const int smem = 6 * 128 * a->d + 16384 + 128 * a->d * 2 + 2048 + 1024;
  cudaStream_t st = (cudaStream_t)stream;
  if (a->d == 128) {
    if (cudaFuncSetAttribute(bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return FL_ERR_CUDA;
    bwd_kernel<128><<<grid, 512, smem, st>>>(mq, mk, mv, mdo, macc, p);
  } else {
    if (cudaFuncSetAttribute(bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return FL_ERR_CUDA;
    bwd_kernel<64><<<grid, 512, smem, st>>>(mq, mk, mv, mdo, macc, p);
  }
  return cudaGetLastError() == cudaSuccess ? FL_OK : FL_ERR_CUDA;
}
