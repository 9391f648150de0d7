// Backward main kernel for sm_100a (head_dim 128 or 64): dK, dV and the pre-scaled f16 dQ accumulator from block-scaled
// operands, software-pipelined over 64-query half tiles.
//
// Replaces the reference's FlashAttentionBackwardSm100FP4 (flash_attn/cute/flash_bwd_sm100_fp4.py:82; driver
// flash_attn/cute/interface_bwd_fp4.py:1207) for the E4M3 backward. One CTA per (128-key tile, kv head, batch | document);
// it walks the query tiles that see the key tile (x the query heads of the GQA group), each as two 64-query halves
// x = 0, 1 that run one step apart, so the tensor core works on one half while the other half's elementwise math runs:
//   S^T_x  = K Q_x^T                  kind::f8f6f4, N = 64 (token-block factors folded into the exponent argument)
//   P'     = 2^(S^T c - lse_log2) = 2^8 P        -> P-hat = E4M3(P')                   [tensor memory]
//   dV    += P-hat^T dO_x             kind::mxf8f6f4.block_scale, B scale = dO's UE8M0 per 32 queries
//   dP^T_x = V dO_x^T                 kind::f8f6f4
//   dS     = P' (b dP^T + D''), b = f_V f_dO 2^-8, D'' = -2^-8 rowsum(O dO)
//   dS-hat : one UE8M0 exponent per 32 keys x 32 queries, E4M3 codes (the same codes feed dK and dQ)
//   dK    += dS-hat^T Q_x             block-scaled, A from tensor memory
//   dQ^T_x = K^T dS-hat^T             block-scaled, M = head dim, N = 64 queries; A = K tile and B = dS-hat (shared
//                                     memory) both MN-major; the f16 pre-scale B_m is folded into the A scale bytes
//   dQ^T_x -> f16 -> TMA reduce-add into the (b, h, d, s) accumulator
//   d = 64: block-scaled products need M = 128, so the product is taken the other way round, dQ_x = dS-hat_x K with
//   A = dS-hat (shared memory, MN-major; its second 64-row block is whatever follows in memory and only fills the
//   unused rows 64..127 of the result) and B = the K tile; rows = queries, accumulator layout (b, h, s, d)
//   warps 0-3 compute half 0, warps 4-7 compute half 1 (thread = key row = TMEM lane, 64 query columns)
//   warps 8-11 dQ reduction (thread = head-dim row)      warp 12 UMMA issuer      warp 13 TMA producer
// TMEM: [0,64) / [64,128) S^T_x, then P-hat +0, dS-hat +16, six scale tiles +32..+56; [128,256) dV;
//       [256,320) / [320,384) dP^T_x, then dQ^T_x; [384,512) dK.  Every wait is bounded (sm100.cuh).
// FL_MODE_FP4 (the mixed route): S^T_x is recomputed at the forward's precision, K4 Q4_x^T with
// kind::mxf4nvf4.block_scale.scale_vec::4X on the NVFP4 copies; everything after P' is the E4M3 path above. The 16 scale
// columns of that product (tcgen05.cp of the K and Q atoms) are parked in the half's own dP^T columns: they are free
// once the previous dQ^T_x has been read out, and the dP^T_x product that overwrites them is issued right after S^T_x
// (the tensor pipe runs in issue order). The second half's Q scales are columns 2, 3 of each atom.
// VAR = 1 (FL_A_DQ_ROWLOCAL, the reference's ds_dq_rowlocal="all", flash_bwd_sm100_fp4.py:3637-3642): the dQ side of
// dS-hat gets its own codes with one exponent per (query row, 32-key block) instead of sharing the 32 x 32 block's.
// VAR = 2 (FL_A_TOKEN_LOCAL + row-local, flash_bwd_sm100_fp4.py:152-158): every token of Q, K, V, dO carries its own
// power-of-two factor. Per-key factors are per-thread scalars here, per-query factors are read per element; S and dP
// take f_K f_Q and f_V f_dO in the elementwise math; dV takes f_dO inside a block-scaled P-hat (one exponent per key row
// x 32 queries); dK takes f_Q inside its dS-hat codes, dQ takes f_K inside its own; the operand scale tiles are unit.
#include "flamia_internal.h"

namespace fl {

struct BwdParams {
  const float* fac_q;
  const float* fac_k;
  const float* fac_v;
  const float* fac_do;
  const float* lse_log2;
  const float* d_rows;
  const float* dq_scale;
  const uint8_t* sfq4;   // FL_MODE_FP4: E4M3 scale atoms of the NVFP4 Q / K copies (1 KB per 128-row tile)
  const uint8_t* sfk4;
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
  int bat;    // batch coordinate of the tensor maps (0 for packed documents)
  int k0;     // first key row of the tile (row index inside the batch entry)
  int nk;     // valid keys of the tile (<= 128)
  int krel;   // document-relative index of key row k0
  int q0;     // first query row of the document (row index inside the batch entry)
  int sq;     // queries of the document
  int off;    // causal alignment: key j (document-relative) is visible to query i iff j <= i + off
};

enum { BB_KV = 0, BB_QFULL = 1, BB_QEMPTY = 3, BB_S = 5, BB_DP = 7, BB_P = 9, BB_DS = 11, BB_EX = 13, BB_DQF = 15,
       BB_DQE = 17, BB_R1 = 19, BB_R2 = 20, BB_ACC = 21, BB_EP = 22, BB_COUNT = 24 };
// TMEM columns; the per-half regions are at + 64 * x
enum { TC_S = 0, TO_P = 0, TO_DS = 16, TO_SFA_P = 32, TO_SFB_DO = 36, TO_SFA_DK = 40, TO_SFB_Q = 44, TO_SFA_DQ = 48,
       TO_SFB_DQ = 52, TC_DV = 128, TC_DP = 256, TC_DK = 384 };

// Timeline tracing of one CTA (development aid, compiled out unless FL_TRACE is defined): clock64 stamps per role, step
// and event into a caller-provided buffer of [8 roles][256 steps][8 events] int64.
#ifdef FL_TRACE
__device__ long long* g_trace = nullptr;
#define TRACE_INIT() long long* const trace_p = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? g_trace : nullptr
#define TRACE(role, step, ev)                                                                                     \
  do {                                                                                                            \
    if (trace_p && (step) < 256) trace_p[(((role) * 256) + (step)) * 8 + (ev)] = clock64();                       \
  } while (0)
#else
#define TRACE_INIT()
#define TRACE(role, step, ev)
#endif

__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
  uint32_t r;
  asm volatile("redux.sync.max.u32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
  return r;
}
template <int N>
__device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// 448 * 2^(e - 127) >= amax for the returned UE8M0 byte (bits = the non-negative float's pattern), clamped to [1, 254]
__device__ __forceinline__ uint32_t exp448(uint32_t bits) {
  const int e = (int)((bits + 0x00200000u) >> 23) - 8;
  return (uint32_t)min(max(e, 1), 254);
}
__device__ __forceinline__ float pow2_inv(uint32_t ebyte) { return __uint_as_float((uint32_t)(254 - (int)ebyte) << 23); }

template <int D, bool FP4, int VAR>
__global__ void __launch_bounds__(512, 1)
bwd_kernel_pipelined(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_acc, const __grid_constant__ CUtensorMap tm_q4,
                     const __grid_constant__ CUtensorMap tm_k4, const __grid_constant__ CUtensorMap tm_dk,
                     const __grid_constant__ CUtensorMap tm_dv, const BwdParams p) {
  constexpr int TILE_BYTES = 128 * D;
  constexpr uint64_t OP_SWZ = (D == 128) ? SWZ_128 : SWZ_64;     // operand tiles: rows of D bytes
  constexpr uint32_t OP_SBO = 8 * D;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                                  // 1 tile
  uint8_t* sV = sK + TILE_BYTES;                       // 1 tile
  uint8_t* sQ = sV + TILE_BYTES;                       // 2 stages
  uint8_t* sDO = sQ + 2 * TILE_BYTES;                  // 2 stages
  uint8_t* sDS = sDO + 2 * TILE_BYTES;                 // per half: 128 key rows x 64 query bytes, 64 B swizzle
  uint8_t* sDQ = sDS + 2 * 8192;                       // per half: 128 head-dim rows x 64 queries f16, 128 B swizzle
  float* sVec = reinterpret_cast<float*>(sDQ + 2 * 16384);   // 2 stages x {lse_log2[128], D''[128]}
  // FP4 only: NVFP4 K tile (8 KB), two Q4 stages (8 KB each), scale atoms K 1 KB + Q 2 x 1 KB
  uint8_t* sK4 = reinterpret_cast<uint8_t*>(sVec) + 2048;
  uint8_t* sQ4 = sK4 + 8192;
  uint8_t* sSF = sQ4 + 2 * 8192;
  __shared__ __align__(8) uint64_t bars[BB_COUNT];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ BTile tile_s;
  __shared__ uint32_t sE[2][4];                        // [half][key block] = exponent bytes of the half's two query blocks
  __shared__ uint32_t sEP[2][128];                     // VAR 2: [half][key row] = P-hat exponent bytes of the two query blocks
  __shared__ __align__(4) uint8_t sEQ[2][64][4];       // VAR >= 1: [half][query][key block] = dQ-side dS-hat exponents
  constexpr bool RL = VAR >= 1, TL = VAR == 2;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // causal: grid = (kv heads, batch rows, key tiles), so key tiles with the same number of query tiles are dispatched
  // together, longest first. Otherwise grid = (key tiles, kv heads, batch rows): the CTAs of one head run together and
  // share its Q / dO tiles in L2.
  const int hkv = p.causal ? blockIdx.x : blockIdx.y;
  const int tile_id = p.causal ? blockIdx.z : blockIdx.x, bat_id = p.causal ? blockIdx.y : blockIdx.z;
  const int grp = p.h / p.h_kv;
  TRACE_INIT();
  if (tid == 0) TRACE(6, 0, 0);

  // Set-up by the TMA thread itself, which then starts the first loads (K, V and the first Q / dO tile) before the CTA-wide
  // barrier: they fly while tensor memory is allocated and the other warps arrive (~1300 clocks earlier first scores).
  if (tid == 13 * 32) {
    abort_s = 0;
    mbar_init(&bars[BB_KV], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[BB_QFULL + i], 1); mbar_init(&bars[BB_QEMPTY + i], 1);
      mbar_init(&bars[BB_S + i], 1); mbar_init(&bars[BB_DP + i], 1);
      mbar_init(&bars[BB_P + i], 4); mbar_init(&bars[BB_DS + i], 4); mbar_init(&bars[BB_EX + i], 4);      // one arrival per warp
      mbar_init(&bars[BB_DQF + i], 1); mbar_init(&bars[BB_DQE + i], 4);
      mbar_init(&bars[BB_EP + i], 4);
    }
    mbar_init(&bars[BB_R1], 4);
    mbar_init(&bars[BB_R2], 4);
    mbar_init(&bars[BB_ACC], 1);
    fence_barrier_init();
    BTile t;
    if (p.doc_start == nullptr) {
      t.bat = bat_id; t.k0 = tile_id * 128; t.nk = min(128, p.s_k - t.k0); t.krel = t.k0; t.q0 = 0; t.sq = p.s_q;
      t.off = p.s_k - p.s_q;
    } else {
      int x = tile_id, dsel = -1, len = 0, st = 0;
      for (int dI = 0; dI < p.n_docs; ++dI) {
        doc_entry(p.doc_start, p.doc_len, dI, p.s_k, p.ctl.status, st, len);
        const int nb = (len + 127) / 128;
        if (x < nb) { dsel = dI; break; }
        x -= nb;
      }
      if (dsel < 0) { t.nk = 0; t.bat = 0; t.k0 = 0; t.krel = 0; t.q0 = 0; t.sq = 0; t.off = 0; }
      else {
        t.bat = 0; t.k0 = st + x * 128; t.nk = min(128, len - x * 128); t.krel = x * 128; t.q0 = st; t.sq = len; t.off = 0;
      }
    }
    tile_s = t;
    int mh = (t.sq + 127) / 128, ml = 0;      // as below: the query tiles that see this key tile
    if (p.win_r >= 0 && t.krel - t.off - p.win_r > 0) ml = (t.krel - t.off - p.win_r) / 128;
    if (p.win_l >= 0) mh = min(mh, max(0, t.krel + t.nk - 1 - t.off + p.win_l) / 128 + 1);
    if (t.nk > 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_do);
      mbar_arrive_expect_tx(&bars[BB_KV], 2 * TILE_BYTES + (FP4 ? 8192 + 1024 : 0));
      tma_load_4d(sK, &tm_k, &bars[BB_KV], 0, hkv, t.k0, t.bat);
      tma_load_4d(sV, &tm_v, &bars[BB_KV], 0, hkv, t.k0, t.bat);
      if (FP4) {
        tma_load_4d(sK4, &tm_k4, &bars[BB_KV], 0, hkv, t.k0, t.bat);
        bulk_load(sSF, p.sfk4 + (((size_t)t.bat * p.h_kv + hkv) * (p.s_k / 128) + t.k0 / 128) * 1024, 1024, &bars[BB_KV]);
      }
      if (mh > ml) {       // iteration 0: first head of the group, first query tile
        const int head = hkv * grp, m = ml;
        mbar_arrive_expect_tx(&bars[BB_QFULL + 0], 2 * TILE_BYTES + 1024 + (FP4 ? 8192 + 1024 : 0));
        tma_load_4d(sQ, &tm_q, &bars[BB_QFULL + 0], 0, head, t.q0 + m * 128, t.bat);
        if (FP4) {
          tma_load_4d(sQ4, &tm_q4, &bars[BB_QFULL + 0], 0, head, t.q0 + m * 128, t.bat);
          bulk_load(sSF + 1024, p.sfq4 + (((size_t)t.bat * p.h + head) * (p.s_q / 128) + (t.q0 + m * 128) / 128) * 1024, 1024,
                    &bars[BB_QFULL + 0]);
        }
        tma_load_4d(sDO, &tm_do, &bars[BB_QFULL + 0], 0, head, t.q0 + m * 128, t.bat);
        const size_t ro = ((size_t)t.bat * p.h + head) * p.s_q + t.q0 + m * 128;
        bulk_load(sVec, p.lse_log2 + ro, 512, &bars[BB_QFULL + 0]);
        bulk_load(sVec + 128, p.d_rows + ro, 512, &bars[BB_QFULL + 0]);
      }
    }
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

  // query tiles that see this key tile: the first query that sees its first key, the last one that sees its last key
  int m_hi = (T.sq + 127) / 128;
  int m_lo = 0;
  if (p.win_r >= 0 && T.krel - T.off - p.win_r > 0) m_lo = (T.krel - T.off - p.win_r) / 128;
  if (p.win_l >= 0) m_hi = min(m_hi, max(0, T.krel + T.nk - 1 - T.off + p.win_l) / 128 + 1);
  const int n_m = (T.nk > 0 && m_hi > m_lo) ? (m_hi - m_lo) : 0;
  const int n_it = n_m * grp;                                          // tile iterations: GQA heads x query tiles
  // (a status word already set by an earlier launch is not looked at: the first loads are in flight by now, and a
  // kernel that runs after one that gave up does no harm)
  const bool early_out = T.nk <= 0;
  if (tid == 0) TRACE(6, 0, 1);

  if (!early_out) {
    if (warp >= 12) reg_dealloc<80>();     // register budget per warpgroup: 176 / 176 / 80 / 80 (x 128 threads = 64 K)
    if (warp == 13) {
      // =================================================================== TMA producer
      if (lane == 0) {
        for (int it = 1; it < n_it; ++it) {      // K, V and iteration 0 were started during set-up
          const int st = it & 1, u = it >> 1;
          const int head = hkv * grp + it / n_m, m = m_lo + it % n_m;
          if (it >= 2 && !mbar_wait(&bars[BB_QEMPTY + st], (u & 1) ^ 1, p.ctl, abortp, 10)) break;
          mbar_arrive_expect_tx(&bars[BB_QFULL + st], 2 * TILE_BYTES + 1024 + (FP4 ? 8192 + 1024 : 0));
          tma_load_4d(sQ + st * TILE_BYTES, &tm_q, &bars[BB_QFULL + st], 0, head, T.q0 + m * 128, T.bat);
          if (FP4) {
            tma_load_4d(sQ4 + st * 8192, &tm_q4, &bars[BB_QFULL + st], 0, head, T.q0 + m * 128, T.bat);
            bulk_load(sSF + 1024 + st * 1024,
                      p.sfq4 + (((size_t)T.bat * p.h + head) * (p.s_q / 128) + (T.q0 + m * 128) / 128) * 1024, 1024,
                      &bars[BB_QFULL + st]);
          }
          tma_load_4d(sDO + st * TILE_BYTES, &tm_do, &bars[BB_QFULL + st], 0, head, T.q0 + m * 128, T.bat);
          const size_t ro = ((size_t)T.bat * p.h + head) * p.s_q + T.q0 + m * 128;
          bulk_load(sVec + st * 256, p.lse_log2 + ro, 512, &bars[BB_QFULL + st]);
          bulk_load(sVec + st * 256 + 128, p.d_rows + ro, 512, &bars[BB_QFULL + st]);
        }
      }
    } else if (warp == 12) {
      // =================================================================== UMMA issuer
      // The whole warp stays converged through the waits and the descriptor arithmetic (warp-uniform values); one elected
      // lane issues. Descriptors are built once; the loop only adds byte offsets.
      {
        constexpr uint32_t ID_N64 = idesc_f8(128, 64, 0, 0);
        const uint32_t tm = __shfl_sync(0xFFFFFFFFu, tmem, 0);
        const int n_steps = 2 * __shfl_sync(0xFFFFFFFFu, n_it, 0);
        const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ), do_addr = smem_u32(sDO),
                       ds_addr = smem_u32(sDS);
        const uint64_t dK_k = smem_desc(k_addr, 16, OP_SBO, OP_SWZ), dV_k = smem_desc(v_addr, 16, OP_SBO, OP_SWZ),
                       dQ0 = smem_desc(q_addr, 16, OP_SBO, OP_SWZ), dDO0 = smem_desc(do_addr, 16, OP_SBO, OP_SWZ),
                       dDS_A = smem_desc(ds_addr, 8192, 512, SWZ_64),   // d = 64: dS-hat as A, next M block 8 KB further
                       dDS0 = smem_desc(ds_addr, 16, 512, SWZ_64);
        const uint64_t dK4 = smem_desc(smem_u32(sK4), 16, 512, SWZ_64), dQ40 = smem_desc(smem_u32(sQ4), 16, 512, SWZ_64),
                       dSF0 = smem_desc(smem_u32(sSF), 0, 128, SWZ_NONE);
        bool ok = mbar_wait(&bars[BB_KV], 0, p.ctl, abortp, 20);
        for (int t = 0; ok && t <= n_steps; ++t) {
          if (t < n_steps) {
            // ---- front end of step t: S^T_x and dP^T_x
            const int it = t >> 1, x = t & 1, st = it & 1;
            if (x == 0 && !(ok = mbar_wait(&bars[BB_QFULL + st], (it >> 1) & 1, p.ctl, abortp, 21))) break;
            tc_fence_after();
            const uint64_t qx = desc_adv(dQ0, st * TILE_BYTES + x * 64 * D), dox = desc_adv(dDO0, st * TILE_BYTES + x * 64 * D);
            if (FP4) {
              // the scale columns go into the half's dP^T region: its previous dQ^T must have been read out first
              if (it > 0 && !(ok = mbar_wait(&bars[BB_DQE + x], (it - 1) & 1, p.ctl, abortp, 22))) break;
              tc_fence_after();
            }
            if (elect_one()) {
              if (FP4) {
                const uint32_t park = tm + TC_DP + 64 * x;
                const uint64_t q4x = desc_adv(dQ40, st * 8192 + x * 4096);
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                  tmem_cp_sf_atom(park + 4 * k, desc_adv(dSF0, 512 * k));
                  tmem_cp_sf_atom(park + 8 + 4 * k, desc_adv(dSF0, 1024 + st * 1024 + 512 * k));
                }
#pragma unroll
                for (int k = 0; k < 2; ++k)   // K = 64 elements = 32 bytes per instruction
                  umma_nvf4_ss(tm + TC_S + 64 * x, desc_adv(dK4, 32 * k), desc_adv(q4x, 32 * k),
                               idesc_bs(128, 64, 1, 1, 0, 0, 0, 0, 0), park + 4 * k, park + 8 + 4 * k + 2 * x, k > 0);
              } else {
#pragma unroll
                for (int k = 0; k < D / 32; ++k)
                  umma_f8_ss(tm + TC_S + 64 * x, desc_adv(dK_k, 32 * k), desc_adv(qx, 32 * k), ID_N64, k > 0);
              }
              tc_commit(&bars[BB_S + x]);
              TRACE(0, t, 0);
            }
            __syncwarp();
            // the half's dP^T columns hold its previous dQ^T until the reduction warps have read it
            if (!FP4 && it > 0 && !(ok = mbar_wait(&bars[BB_DQE + x], (it - 1) & 1, p.ctl, abortp, 22))) break;
            tc_fence_after();
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < D / 32; ++k)
                umma_f8_ss(tm + TC_DP + 64 * x, desc_adv(dV_k, 32 * k), desc_adv(dox, 32 * k), ID_N64, k > 0);
              tc_commit(&bars[BB_DP + x]);
              TRACE(0, t, 1);
            }
            __syncwarp();
          }
          if (t >= 1) {
            // ---- back end of step t - 1: dV, dK, dQ^T of half y
            const int tb = t - 1, it = tb >> 1, y = tb & 1, st = it & 1;
            const uint32_t sx = tm + TC_S + 64 * y;
            const uint64_t qy = desc_adv(dQ0, st * TILE_BYTES + y * 64 * D), doy = desc_adv(dDO0, st * TILE_BYTES + y * 64 * D);
            const uint32_t accum = tb > 0;
            if (!(ok = mbar_wait(&bars[BB_P + y], it & 1, p.ctl, abortp, 23))) break;
            tc_fence_after();
            if (elect_one()) {
              TRACE(0, tb, 2);
#pragma unroll
              for (int kk = 0; kk < 2; ++kk)     // K = 64 queries: two instructions of 32
                umma_mxf8_ts(tm + TC_DV, sx + TO_P + 8 * kk, desc_adv(doy, kk * 32 * D),
                             idesc_bs(128, D, 0, 0, 0, 1, 1, kk, kk), sx + TO_SFA_P, sx + TO_SFB_DO, accum | kk);
              TRACE(0, tb, 3);
            }
            __syncwarp();
            if (!(ok = mbar_wait(&bars[BB_DS + y], it & 1, p.ctl, abortp, 24))) break;
            tc_fence_after();
            if (elect_one()) {
              TRACE(0, tb, 4);
#pragma unroll
              for (int kk = 0; kk < 2; ++kk)
                umma_mxf8_ts(tm + TC_DK, sx + TO_DS + 8 * kk, desc_adv(qy, kk * 32 * D),
                             idesc_bs(128, D, 0, 0, 0, 1, 1, kk, kk), sx + TO_SFA_DK, sx + TO_SFB_Q, accum | kk);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {   // K = 128 keys
                if (D == 128)      // A = K tile (M = head dim), B = dS-hat half (N = 64 queries)
                  umma_mxf8_ss(tm + TC_DP + 64 * y, desc_adv(dK_k, kk * 32 * D), desc_adv(dDS0, y * 8192 + kk * 2048),
                               idesc_bs(128, 64, 0, 0, 1, 1, 1, kk, kk), sx + TO_SFA_DQ, sx + TO_SFB_DQ, kk > 0);
                else               // A = dS-hat half (M = 64 queries + 64 unused rows), B = K tile (N = head dim)
                  umma_mxf8_ss(tm + TC_DP + 64 * y, desc_adv(dDS_A, y * 8192 + kk * 2048), desc_adv(dK_k, kk * 32 * D),
                               idesc_bs(128, 64, 0, 0, 1, 1, 1, kk, kk), sx + TO_SFB_DQ, sx + TO_SFA_DQ, kk > 0);
              }
              tc_commit(&bars[BB_DQF + y]);
              TRACE(0, tb, 5);
              if (y == 1) tc_commit(&bars[BB_QEMPTY + st]);
            }
            __syncwarp();
          }
        }
        if (ok && elect_one()) tc_commit(&bars[BB_ACC]);
        __syncwarp();
      }
    } else if (warp >= 8 && warp < 12) {
      reg_dealloc<80>();
      // =================================================================== dQ reduction (thread = head-dim row)
      const int r = tid & 127;
      const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
      bool ok = true;
      const int n_steps = 2 * n_it;
      for (int t = 0; t < n_steps; ++t) {
        const int it = t >> 1, y = t & 1;
        const int head = hkv * grp + it / n_m, m = m_lo + it % n_m;
        // the staging buffer of this half was last read by the reduction of step t - 2
        if (tid == 256) tma_store_wait_read<1>();
        mbar_arrive_warp(&bars[BB_R1]);
        if (!(ok = mbar_wait(&bars[BB_R1], t & 1, p.ctl, abortp, 41))) break;
        if (r == 0) TRACE(3, t, 0);
        if (!(ok = mbar_wait(&bars[BB_DQF + y], it & 1, p.ctl, abortp, 40))) break;
        if (r == 0) TRACE(3, t, 1);
        tc_fence_after();
        const uint32_t rowp = smem_u32(sDQ) + y * 16384 + r * 128;
        // d = 128: thread = head-dim row of dQ^T, 64 query columns. d = 64: thread = query row (the first 64 lanes; the
        // other two warps hold the product's unused rows), 64 head-dim columns. Either way 64 f16 = one 128-byte row.
        if (D == 128 || warp < 10) {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            uint32_t v[32];
            FL_TMEM_LD_32(lane_base + TC_DP + 64 * y + 32 * cc, v);
            tc_wait_ld();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {     // 8 f16 = 16 bytes per chunk; 128 B swizzle by the row
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __half2 hh = __floats2half2_rn(__uint_as_float(v[8 * q4 + 2 * e]), __uint_as_float(v[8 * q4 + 2 * e + 1]));
                w[e] = *reinterpret_cast<uint32_t*>(&hh);
              }
              sts128(rowp + (((cc * 4 + q4) ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
            }
          }
        }
        tc_fence_before();
        mbar_arrive_warp(&bars[BB_DQE + y]);
        if (r == 0) TRACE(3, t, 2);
        fence_proxy_async();
        mbar_arrive_warp(&bars[BB_R2]);
        if (!(ok = mbar_wait(&bars[BB_R2], t & 1, p.ctl, abortp, 42))) break;
        if (tid == 256) {
          if (D == 128) tma_reduce_add_4d(&tm_acc, sDQ + y * 16384, T.q0 + m * 128 + 64 * y, 0, head, T.bat);
          else tma_reduce_add_4d(&tm_acc, sDQ + y * 16384, 0, T.q0 + m * 128 + 64 * y, head, T.bat);
          tma_store_commit();
        }
      }
      if (tid == 256) tma_store_wait<0>();
    } else if (warp < 8) {
      reg_alloc<176>();
      // =================================================================== compute (thread = key row, 64 query columns)
      const int x = warp >> 2;                         // the half this warpgroup owns
      const int wq = warp & 3;                         // lane quadrant = 32-key block of the tile
      const int r = wq * 32 + lane;                    // key row of the tile = TMEM lane
      const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16);
      const uint32_t t_sx = lane_base + TC_S + 64 * x, t_dpx = lane_base + TC_DP + 64 * x;
      const int krel = T.krel + r;
      const bool key_valid = r < T.nk;
      const size_t bh_k = (size_t)T.bat * p.h_kv + hkv;
      const int kblk = (T.k0 + r) / 32;
      // token-local: this key's own factors; otherwise its 32-key block's
      const float fk_true = TL ? p.fac_k[bh_k * p.s_k + T.k0 + r] : p.fac_k[bh_k * (p.s_k / 32) + kblk];
      const float fk = fk_true * p.scale_log2;
      const float fv8 = (TL ? p.fac_v[bh_k * p.s_k + T.k0 + r] : p.fac_v[bh_k * (p.s_k / 32) + kblk]) * 0.00390625f;   // f_V 2^-8
      uint32_t ek_word = TL ? 0x7F7F7F7Fu : 0u;        // UE8M0 bytes of the tile's four key blocks (unit when token-local)
      if (!TL) {
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
          ek_word |= ((__float_as_uint(p.fac_k[bh_k * (p.s_k / 32) + T.k0 / 32 + kb]) >> 23) & 0xFF) << (8 * kb);
      }
      const uint32_t ds_row = smem_u32(sDS) + x * 8192 + r * 64;
      const int vis_from = p.win_r >= 0 ? (krel - T.off - p.win_r) : 0;    // queries in [vis_from, vis_to] see this key
      const int vis_to = p.win_l >= 0 ? (krel - T.off + p.win_l) : 0x7FFFFFFF;
      bool ok = true;
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1, u = it >> 1;
        const int head = hkv * grp + it / n_m, m = m_lo + it % n_m;
        const size_t bh_q = (size_t)T.bat * p.h + head;
        const int qb0 = (T.q0 + m * 128) / 32 + 2 * x;                     // first of the half's two 32-query blocks
        const float fq0 = TL ? 1.f : p.fac_q[bh_q * (p.s_q / 32) + qb0], fq1 = TL ? 1.f : p.fac_q[bh_q * (p.s_q / 32) + qb0 + 1];
        const float fd0 = TL ? 1.f : p.fac_do[bh_q * (p.s_q / 32) + qb0], fd1 = TL ? 1.f : p.fac_do[bh_q * (p.s_q / 32) + qb0 + 1];
        // token-local: the 64 per-query factors of the half (same addresses for every thread: broadcast loads)
        const float4* fq_vec = reinterpret_cast<const float4*>(p.fac_q + (TL ? bh_q * p.s_q + T.q0 + m * 128 + 64 * x : 0));
        const float4* fdo_vec = reinterpret_cast<const float4*>(p.fac_do + (TL ? bh_q * p.s_q + T.q0 + m * 128 + 64 * x : 0));
        const float bsc = p.dq_scale[(size_t)T.bat * (p.s_q / 128) + T.q0 / 128 + m];
        // FP4: the block scales of S were applied by the tensor core; only the softmax scale remains
        const float c[2] = {FP4 ? p.scale_log2 : fk * fq0, FP4 ? p.scale_log2 : fk * fq1}, b8[2] = {fv8 * fd0, fv8 * fd1};
        // token-local: fq0 = fq1 = fd0 = fd1 = 1, i.e. unit scale bytes for the Q and dO operands
        const uint32_t eq2 = ((__float_as_uint(fq0) >> 23) & 0xFF) | (((__float_as_uint(fq1) >> 23) & 0xFF) << 8);
        const uint32_t edo2 = ((__float_as_uint(fd0) >> 23) & 0xFF) | (((__float_as_uint(fd1) >> 23) & 0xFF) << 8);
        // K's exponent bytes with the power-of-two f16 pre-scale of this query tile folded in (A scale of dQ^T)
        const uint32_t lb = (uint32_t)((int)((__float_as_uint(bsc) >> 23) & 0xFF) - 127) & 0xFF;
        const uint32_t ekb_word = __vadd4(ek_word, lb * 0x01010101u);
        if (!(ok = mbar_wait(&bars[BB_QFULL + st], u & 1, p.ctl, abortp, 30))) break;   // lse / D'' vectors visible
        const uint32_t v_lse = smem_u32(sVec) + (st * 256 + 64 * x) * 4, v_dpp = v_lse + 512;
        const int q_first = m * 128 + 64 * x;                              // document-relative query of column 0
        const bool full = key_valid && (q_first >= vis_from) && (q_first + 63 <= vis_to) && (q_first + 64 <= T.sq);

        // ---- P' = 2^(s c - lse2)
        if (r == 0) TRACE(1 + x, it, 0);
        if (!(ok = mbar_wait(&bars[BB_S + x], it & 1, p.ctl, abortp, 31))) break;
        if (r == 0) TRACE(1 + x, it, 1);
        tc_fence_after();
        uint32_t pv[64];
        FL_TMEM_LD_32(t_sx, pv);
        FL_TMEM_LD_32(t_sx + 32, (pv + 32));
        tc_wait_ld();
        float pf[64];
#pragma unroll
        for (int j4 = 0; j4 < 16; ++j4) {
          const float4 l4 = lds128(v_lse + 16 * j4);
          const float cc = c[j4 >> 3];
          float4 c4 = make_float4(cc, cc, cc, cc);
          if (TL) {
            const float4 f4 = __ldg(fq_vec + j4);
            c4 = make_float4(fk * f4.x, fk * f4.y, fk * f4.z, fk * f4.w);
          }
          pf[4 * j4 + 0] = ex2(fmaf(__uint_as_float(pv[4 * j4 + 0]), c4.x, -l4.x));
          pf[4 * j4 + 1] = ex2(fmaf(__uint_as_float(pv[4 * j4 + 1]), c4.y, -l4.y));
          pf[4 * j4 + 2] = ex2(fmaf(__uint_as_float(pv[4 * j4 + 2]), c4.z, -l4.z));
          pf[4 * j4 + 3] = ex2(fmaf(__uint_as_float(pv[4 * j4 + 3]), c4.w, -l4.w));
        }
        if (!full) {      // diagonal / tail tiles only
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            const int qi = q_first + j;
            pf[j] = (key_valid && qi >= vis_from && qi <= vis_to && qi < T.sq) ? pf[j] : 0.f;
          }
        }
        if (TL) {
          // block-scaled P-hat carrying f_dO(query): one exponent per (this key row, 32 queries)
          uint32_t pw[16], ep[2];
#pragma unroll
          for (int qh = 0; qh < 2; ++qh) {
            float t[32];
            float am = 0.f;
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              const float4 f4 = __ldg(fdo_vec + qh * 8 + j4);
              const int j = qh * 32 + 4 * j4;
              t[4 * j4 + 0] = pf[j + 0] * f4.x; t[4 * j4 + 1] = pf[j + 1] * f4.y;
              t[4 * j4 + 2] = pf[j + 2] * f4.z; t[4 * j4 + 3] = pf[j + 3] * f4.w;
              am = fmaxf(am, fmaxf(fmaxf(t[4 * j4], t[4 * j4 + 1]), fmaxf(t[4 * j4 + 2], t[4 * j4 + 3])));
            }
            ep[qh] = exp448(__float_as_uint(am));
            const float inv = pow2_inv(ep[qh]);
#pragma unroll
            for (int w = 0; w < 8; ++w)
              pw[qh * 8 + w] = cvt_e4m3x4(t[4 * w] * inv, t[4 * w + 1] * inv, t[4 * w + 2] * inv, t[4 * w + 3] * inv);
          }
          FL_TMEM_ST_16(t_sx + TO_P, pw);
          // every lane quadrant holds the whole A scale tile: column = key block, lane = row of the block
          sEP[x][r] = ep[0] | (ep[1] << 8);
          mbar_arrive_warp(&bars[BB_EP + x]);
          if (!(ok = mbar_wait(&bars[BB_EP + x], it & 1, p.ctl, abortp, 37))) break;
          uint32_t sf[8] = {sEP[x][lane], sEP[x][32 + lane], sEP[x][64 + lane], sEP[x][96 + lane],
                            0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu};
          FL_TMEM_ST_8(t_sx + TO_SFA_P, sf);
        } else {
          uint32_t pw[16];
#pragma unroll
          for (int w = 0; w < 16; ++w) pw[w] = cvt_e4m3x4(pf[4 * w], pf[4 * w + 1], pf[4 * w + 2], pf[4 * w + 3]);
          FL_TMEM_ST_16(t_sx + TO_P, pw);
          // scale tiles of the dV product: A = 1, B = dO's exponent per 32 queries (bytes = the half's two K steps)
          uint32_t sf[8] = {0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, edo2, edo2, edo2, edo2};
          FL_TMEM_ST_8(t_sx + TO_SFA_P, sf);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive_warp(&bars[BB_P + x]);
        if (r == 0) TRACE(1 + x, it, 2);

        // ---- dS = P' (b dP + D''), block exponent per (this warp's 32 keys, 32 queries)
        if (!(ok = mbar_wait(&bars[BB_DP + x], it & 1, p.ctl, abortp, 32))) break;
        if (r == 0) TRACE(1 + x, it, 3);
        tc_fence_after();
        FL_TMEM_LD_32(t_dpx, pv);
        FL_TMEM_LD_32(t_dpx + 32, (pv + 32));
        tc_wait_ld();
        uint32_t ebyte[2];
#pragma unroll
        for (int qh = 0; qh < 2; ++qh) {
          float am = 0.f;
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 d4 = lds128(v_dpp + 16 * (qh * 8 + j4));
            const int j = qh * 32 + 4 * j4;
            float4 b4 = make_float4(b8[qh], b8[qh], b8[qh], b8[qh]);
            float4 q4 = make_float4(1.f, 1.f, 1.f, 1.f);
            if (TL) {
              const float4 f4 = __ldg(fdo_vec + qh * 8 + j4);
              b4 = make_float4(fv8 * f4.x, fv8 * f4.y, fv8 * f4.z, fv8 * f4.w);
              q4 = __ldg(fq_vec + qh * 8 + j4);
            }
            pf[j + 0] *= fmaf(__uint_as_float(pv[j + 0]), b4.x, d4.x);
            pf[j + 1] *= fmaf(__uint_as_float(pv[j + 1]), b4.y, d4.y);
            pf[j + 2] *= fmaf(__uint_as_float(pv[j + 2]), b4.z, d4.z);
            pf[j + 3] *= fmaf(__uint_as_float(pv[j + 3]), b4.w, d4.w);
            if (!full) {
              // masked entries hold P' = 0, but their dP^T or D'' may come from rows outside the document (padding or
              // whatever the buffer held: possibly Inf / NaN), and 0 * NaN is NaN: select, do not multiply
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int qi = q_first + j + e;
                pf[j + e] = (key_valid && qi >= vis_from && qi <= vis_to && qi < T.sq) ? pf[j + e] : 0.f;
              }
            }
            // the dK side carries f_Q(query) when the operands are token-local
            am = fmaxf(am, fmaxf(fmaxf(fabsf(pf[j] * q4.x), fabsf(pf[j + 1] * q4.y)),
                                 fmaxf(fabsf(pf[j + 2] * q4.z), fabsf(pf[j + 3] * q4.w))));
          }
          const uint32_t wm = warp_max_u32(__float_as_uint(am));          // non-negative floats order as integers
          ebyte[qh] = exp448(wm);                                          // 448 * 2^(e-127) >= amax
        }
        if (lane == 0) sE[x][wq] = ebyte[0] | (ebyte[1] << 8);
        if (!RL) mbar_arrive_warp(&bars[BB_EX + x]);
        uint32_t dsw[16];
#pragma unroll
        for (int qh = 0; qh < 2; ++qh) {
          const float inv = pow2_inv(ebyte[qh]);                           // 2^(127 - e)
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            const int j0 = qh * 32 + 4 * w;
            float4 q4 = make_float4(inv, inv, inv, inv);
            if (TL) {
              const float4 f4 = __ldg(fq_vec + qh * 8 + w);
              q4 = make_float4(f4.x * inv, f4.y * inv, f4.z * inv, f4.w * inv);   // powers of two: exact, in range
            }
            dsw[qh * 8 + w] = cvt_e4m3x4(pf[j0] * q4.x, pf[j0 + 1] * q4.y, pf[j0 + 2] * q4.z, pf[j0 + 3] * q4.w);
          }
        }
        FL_TMEM_ST_16(t_sx + TO_DS, dsw);
        if (RL) {
          // the dQ side's own codes: one exponent per (query, this warp's 32 keys); token-local: they carry f_K(key)
          // per column: t = the exponent field of 2^(e - 119), e the UE8M0 byte with 448 * 2^(e - 127) >= amax, floored
          // at e = 1; 2^(127 - e) is then the field 262 - (e + 8). (Integer and min / max instructions issue at half rate:
          // the fewer per column the better.)
          uint32_t mine[2] = {9u << 23, 9u << 23};
#pragma unroll
          for (int w = 0; w < 16; ++w) {
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j = 4 * w + e;
              const float a = TL ? pf[j] * fk_true : pf[j];
              const uint32_t wm = warp_max_u32(__float_as_uint(a) & 0x7FFFFFFFu);
              const uint32_t t = max((wm + 0x00200000u) & 0x7F800000u, 9u << 23);
              if (lane == (j & 31)) mine[j >> 5] = t;
              v[e] = a * __uint_as_float(0x83000000u - t);
            }
            dsw[w] = cvt_e4m3x4(v[0], v[1], v[2], v[3]);
          }
          sEQ[x][lane][wq] = (uint8_t)((mine[0] >> 23) - 8);
          sEQ[x][32 + lane][wq] = (uint8_t)((mine[1] >> 23) - 8);
          mbar_arrive_warp(&bars[BB_EX + x]);
        }
        // the dQ^T product's MN-major B operand: row = key, 64 bytes = 4 chunks of 16 B, 64 B swizzle
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          sts128(ds_row + ((q4 ^ ((r >> 1) & 3)) << 4), dsw[4 * q4], dsw[4 * q4 + 1], dsw[4 * q4 + 2], dsw[4 * q4 + 3]);
        if (r == 0) TRACE(1 + x, it, 4);
        if (!(ok = mbar_wait(&bars[BB_EX + x], it & 1, p.ctl, abortp, 36))) break;
        if (r == 0) TRACE(1 + x, it, 5);
        {
          // dK:   A[key lane, column = key block]  bytes = the half's two query blocks;  B = Q's exponents
          // dQ^T: A[head-dim lane] = K's exponents (+ pre-scale) per key block; B[query lane, column = query block of
          //       the half] bytes = the four key blocks
          const uint32_t e0 = sE[x][0], e1 = sE[x][1], e2 = sE[x][2], e3 = sE[x][3];
          uint32_t sf[16];
          sf[0] = e0; sf[1] = e1; sf[2] = e2; sf[3] = e3;
          sf[4] = sf[5] = sf[6] = sf[7] = eq2;
          sf[8] = sf[9] = sf[10] = sf[11] = ekb_word;
          if (RL) {   // B[query lane, column = query block] bytes = that query's exponents over the four key blocks
            sf[12] = *reinterpret_cast<const uint32_t*>(&sEQ[x][lane][0]);
            sf[13] = *reinterpret_cast<const uint32_t*>(&sEQ[x][32 + lane][0]);
          } else {
            sf[12] = (e0 & 0xFF) | ((e1 & 0xFF) << 8) | ((e2 & 0xFF) << 16) | ((e3 & 0xFF) << 24);
            sf[13] = ((e0 >> 8) & 0xFF) | (((e1 >> 8) & 0xFF) << 8) | (((e2 >> 8) & 0xFF) << 16) | (((e3 >> 8) & 0xFF) << 24);
          }
          sf[14] = sf[15] = 0x7F7F7F7Fu;
          FL_TMEM_ST_16(t_sx + TO_SFA_DK, sf);
        }
        tc_wait_st();
        fence_proxy_async();             // the dS-hat tile in shared memory is read by the tensor core (async proxy)
        tc_fence_before();
        mbar_arrive_warp(&bars[BB_DS + x]);
        if (r == 0) TRACE(1 + x, it, 6);
      }
      // ---- epilogue: warpgroup 0 writes dV, warpgroup 1 writes dK (full rows)
      if (r == 0) TRACE(6, 0, 2 + 3 * x);
      if (ok) ok = mbar_wait(&bars[BB_ACC], 0, p.ctl, abortp, 33);
      if (r == 0) TRACE(6, 0, 3 + 3 * x);
      if (ok) {
        tc_fence_after();
        const uint32_t t_acc = lane_base + (x == 0 ? TC_DV : TC_DK);
        const float mult = (x == 0) ? 0.00390625f : p.softmax_scale;       // dV carries 2^8 (P'), dK the softmax scale
        float y[D];
        if (n_it > 0) {                  // (CTA-uniform: the tensor-memory loads are warp-collective)
          uint32_t v[D];                 // all four loads in flight, one wait
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) FL_TMEM_LD_32(t_acc + 32 * cc, (v + 32 * cc));
          tc_wait_ld();
          const float mk = key_valid ? mult : 0.f;     // rows past the end of the document store zeros
#pragma unroll
          for (int e = 0; e < D; ++e) y[e] = __uint_as_float(v[e]) * mk;
        } else {                         // no query tile saw this key tile
#pragma unroll
          for (int e = 0; e < D; ++e) y[e] = 0.f;
        }
        if (D == 128 && x == 1 && p.had_dk) {       // dK of rotated operands: (y H / sqrt(128)) * signs
#pragma unroll
          for (int hs = 1; hs < D; hs <<= 1) {
#pragma unroll
            for (int i = 0; i < D; ++i) {
              if ((i & hs) == 0) {
                const float a = y[i], b2 = y[i + hs];
                y[i] = a + b2;
                y[i + hs] = a - b2;
              }
            }
          }
          constexpr uint32_t NEG[4] = {0x10D2E03Eu, 0xE0D9F0E2u, 0x45809F07u, 0x75954FEDu};
#pragma unroll
          for (int i = 0; i < D; ++i) {
            y[i] *= 0.08838834764831845f;
            if ((NEG[i >> 5] >> (i & 31)) & 1) y[i] = -y[i];
          }
        }
        // rows -> shared memory (two boxes of 64 elements, 128 B swizzle) -> one TMA store per box: a thread's own 256-byte
        // row written straight to global memory costs 32 separate 128-byte lines per warp instruction
        uint8_t* stage = (x == 0) ? sQ : sDO;            // the operand stages are dead: every product has completed
        const uint32_t srow = smem_u32(stage) + r * 128;
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
          sts128(srow + (c8 >> 3) * 16384 + (((c8 & 7) ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
        }
        fence_proxy_async();
        mbar_arrive_warp(&bars[BB_EX + x]);              // the warpgroup's four warps; phase n_it of that barrier
        if (mbar_wait(&bars[BB_EX + x], n_it & 1, p.ctl, abortp, 38) && r == 0) {
          const CUtensorMap* tm_out = (x == 0) ? &tm_dv : &tm_dk;
          tma_store_4d(tm_out, stage, 0, hkv, T.k0, T.bat);
          if (D == 128) tma_store_4d(tm_out, stage + 16384, 64, hkv, T.k0, T.bat);
          tma_store_commit();
          tma_store_wait_read<0>();      // the shared-memory source must outlive the copy; the writes complete with the grid
        }
      }
    }
  }
  if (tid == 0 || tid == 128) TRACE(6, 0, 4 + 3 * (tid >> 7));
  if (abort_s) {
    for (int it = 0; it < 200; ++it) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0) TRACE(6, 1, 0);
}

}  // namespace fl

#ifdef FL_TRACE
extern "C" int fl_debug_set_trace(void* buf) {
  return cudaMemcpyToSymbol(fl::g_trace, &buf, sizeof(buf)) == cudaSuccess ? 0 : 2;
}
#endif

extern "C" int fl_bwd(const fl_attn_args* a, void* stream) {
  using namespace fl;
  if (!a || !a->q_codes || !a->k_codes || !a->v_codes || !a->do_codes || !a->status) return FL_ERR_BAD_ARG;
  if (!a->fac_q || !a->fac_k || !a->fac_v || !a->fac_do || !a->lse_log2 || !a->d_rows || !a->dq_acc || !a->dq_scale ||
      !a->dk || !a->dv)
    return FL_ERR_BAD_ARG;
  if (a->d != 128 && a->d != 64) return FL_ERR_UNSUPPORTED;
  if (a->mode != FL_MODE_FP8 && a->mode != FL_MODE_FP4) return FL_ERR_UNSUPPORTED;
  const bool fp4 = a->mode == FL_MODE_FP4;
  if (fp4 && (!a->q4 || !a->k4 || !a->sfq4 || !a->sfk4)) return FL_ERR_BAD_ARG;
  const bool tl = (a->flags & FL_A_TOKEN_LOCAL) != 0, rl = (a->flags & FL_A_DQ_ROWLOCAL) != 0;
  if (tl && (!rl || fp4 || a->doc_start)) return FL_ERR_UNSUPPORTED;   // token-local needs the dQ side's own codes
  if (a->d == 64 && (fp4 || rl || tl)) return FL_ERR_UNSUPPORTED;       // d = 64: the default 8-bit route only
  if (a->h <= 0 || a->h_kv <= 0 || a->h % a->h_kv) return FL_ERR_BAD_ARG;
  if ((a->s_q % 128) || (a->s_k % 128) || a->s_q <= 0 || a->s_k <= 0 || a->b <= 0) return FL_ERR_BAD_ARG;
  if (a->doc_start && (a->b != 1 || a->n_docs <= 0 || !a->doc_len || a->s_q != a->s_k)) return FL_ERR_BAD_ARG;
  CUtensorMap mq, mk, mv, mdo, macc, mq4, mk4, mdk, mdv;
  int rc;
  if ((rc = make_rows_map(&mq, a->q_codes, a->b, a->s_q, a->h, a->d, 128))) return rc;
  if ((rc = make_rows_map(&mk, a->k_codes, a->b, a->s_k, a->h_kv, a->d, 128))) return rc;
  if ((rc = make_rows_map(&mv, a->v_codes, a->b, a->s_k, a->h_kv, a->d, 128))) return rc;
  if ((rc = make_rows_map(&mdo, a->do_codes, a->b, a->s_q, a->h, a->d, 128))) return rc;
  if (a->d == 128) rc = make_acc_t_map_16(&macc, a->dq_acc, a->b, a->h, a->d, a->s_q);
  else rc = make_acc_map_16(&macc, a->dq_acc, a->b, a->h, a->s_q, a->d, 64);       // (b, h, s, d): boxes of 64 query rows
  if (rc) return rc;
  // the NVFP4 copies (64-byte rows); the 8-bit route passes the E4M3 maps again, which the kernel never touches
  if ((rc = make_rows_map(&mq4, fp4 ? (const void*)a->q4 : (const void*)a->q_codes, a->b, a->s_q, a->h, fp4 ? 64 : a->d, 128)))
    return rc;
  if ((rc = make_rows_map(&mk4, fp4 ? (const void*)a->k4 : (const void*)a->k_codes, a->b, a->s_k, a->h_kv, fp4 ? 64 : a->d,
                          128)))
    return rc;
  if ((rc = make_rows_map_16(&mdk, a->dk, a->b, a->s_k, a->h_kv, a->d, 128))) return rc;
  if ((rc = make_rows_map_16(&mdv, a->dv, a->b, a->s_k, a->h_kv, a->d, 128))) return rc;
  BwdParams p;
  p.fac_q = a->fac_q; p.fac_k = a->fac_k; p.fac_v = a->fac_v; p.fac_do = a->fac_do; p.lse_log2 = a->lse_log2;
  p.d_rows = a->d_rows; p.dq_scale = a->dq_scale; p.dk = a->dk; p.dv = a->dv;
  p.sfq4 = a->sfq4; p.sfk4 = a->sfk4;
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
  const int smem = 6 * 128 * a->d + 2 * 8192 + 2 * 16384 + 2048 + 1024 + (fp4 ? 3 * 8192 + 3 * 1024 : 0);
  auto launch = [&](auto kern) -> int {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FL_ERR_CUDA;
    kern<<<grid, 512, smem, (cudaStream_t)stream>>>(mq, mk, mv, mdo, macc, mq4, mk4, mdk, mdv, p);
    return FL_OK;
  };
  if (a->d == 64) rc = launch(bwd_kernel_pipelined<64, false, 0>);
  else if (fp4) rc = rl ? launch(bwd_kernel_pipelined<128, true, 1>) : launch(bwd_kernel_pipelined<128, true, 0>);
  else if (tl) rc = launch(bwd_kernel_pipelined<128, false, 2>);
  else rc = rl ? launch(bwd_kernel_pipelined<128, false, 1>) : launch(bwd_kernel_pipelined<128, false, 0>);
  if (rc) return rc;
  return cudaGetLastError() == cudaSuccess ? FL_OK : FL_ERR_CUDA;
}
