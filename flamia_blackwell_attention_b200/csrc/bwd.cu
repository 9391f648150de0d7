// Backward main kernel for sm_100a (head_dim 128 or 64): dK, dV and the pre-scaled f16 dQ accumulator from block-scaled
// operands, software-pipelined over 64-query half tiles, on a persistent grid.
//
// Replaces the reference's FlashAttentionBackwardSm100FP4 (flash_attn/cute/flash_bwd_sm100_fp4.py:82; driver
// flash_attn/cute/interface_bwd_fp4.py:1207) for the E4M3 backward. One CTA per SM walks a static list of work items
// (128-key tile, kv head, batch | document): under the causal mask the items are ordered longest first and dealt out in
// zigzag rounds (round k gives CTA c item k G + c or k G + G - 1 - c), so every CTA gets nearly the same number of query
// tiles. All pipelines run ACROSS items: the K / V tiles of the next item are loaded into a second buffer while the
// current item's last query tiles are processed, the first S^T / dP^T products of the next item are issued while the
// compute warpgroups write the current item's dK / dV, and barriers, tensor memory and tensor maps are set up once per CTA.
// An item walks the query tiles that see its key tile (x the query heads of the GQA group), each as two 64-query halves
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
// Item epilogue: the compute warpgroups read dV (warpgroup 0) / dK (warpgroup 1) out of tensor memory, release the
// accumulators to the next item's products, and write their rows through the finished item's K / V tile buffers (dead by
// then) with TMA stores, 64 columns at a time; only then may the producer refill those buffers (two items ahead).
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
  const float* dq_scale_rows;   // (b, s_q) per query row instead of dq_scale per query tile, or null
  const float* dk_mult;         // (b, h_kv) factor on dK (Q's mantissa with float descales), or null
  const int32_t* slot_src;      // packed output: packed row of each 128-row slot of the aligned buffer (-1: empty), or null
  const int32_t* slot_rows;     // packed output: real rows of each slot
  const uint8_t* sfq4;   // FL_MODE_FP4: E4M3 scale atoms of the NVFP4 Q / K copies (1 KB per 128-row tile)
  const uint8_t* sfk4;
  void* dk;
  void* dv;
  const int32_t* doc_start;
  const int32_t* doc_len;
  const int32_t* seqused_k;   // batched form: valid keys per batch row, or null
  int32_t* dq_order;     // deterministic dQ: (b, h, s_q / 128, 2) counters, zero on entry, or null
  int n_docs;
  int b, s_q, s_k, h, h_kv;
  float scale_log2;
  float softmax_scale;
  float cap_a, cap_b;    // soft cap c: x = cap_a tanh(s * factor * cap_b) in log2 units, cap_a = c log2 e, cap_b = 1 / cap_a
  int causal;
  int win_l, win_r;      // sliding window sides, -1 = unlimited (causal: the right side is 0)
  int out_f16;
  int had_dk;
  int n_items;           // work items: key tiles x kv heads x batch rows (documents: tile slots x kv heads)
  int n_tile;            // key tiles per batch row (documents: tile slots of the packed buffer)
  int zigzag;            // deal the items out in zigzag rounds (causal: they are ordered longest first)
  DevCtl ctl;
};

struct BTile {
  int bat;    // batch coordinate of the tensor maps (0 for packed documents)
  int hkv;    // kv head
  int k0;     // first key row of the tile (row index inside the batch entry)
  int nk;     // key rows of the tile inside the document / batch row (<= 128; 0 = an empty tile slot)
  int nv;     // of those, the keys that take part (fewer under seqused_k; <= 0: none, the tile's gradients are zero)
  int krel;   // document-relative index of key row k0
  int q0;     // first query row of the document (row index inside the batch entry)
  int sq;     // queries of the document
  int off;    // causal alignment: key j (document-relative) is visible to query i iff j <= i + off
  int m_lo;   // first query tile that sees this key tile
  int n_m;    // number of query tiles that see it
};

// barriers; [2] = one per half, stage or buffer
enum { BB_KV = 0, BB_KVE = 2, BB_QFULL = 4, BB_QEMPTY = 6, BB_S = 8, BB_DP = 10, BB_P = 12, BB_DS = 14, BB_EX = 16,
       BB_DQF = 18, BB_DQE = 20, BB_EP = 22, BB_EPI = 24, BB_R1 = 26, BB_R2 = 27, BB_ACC = 28, BB_ACCFREE = 29,
       BB_COUNT = 30 };
// TMEM columns; the per-half regions are at + 64 * x
enum { TC_S = 0, TO_P = 0, TO_DS = 16, TO_SFA_P = 32, TO_SFB_DO = 36, TO_SFA_DK = 40, TO_SFB_Q = 44, TO_SFA_DQ = 48,
       TO_SFB_DQ = 52, TC_DV = 128, TC_DP = 256, TC_DK = 384 };

// bits of the warp's largest |v| (the f32 form of the instruction is faster than masking the sign and reducing integers:
// -8 % on the row-local backward, which runs it once per dS column)
__device__ __forceinline__ uint32_t warp_max_abs_f32(float v) {
  float r;
  asm volatile("redux.sync.max.abs.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return __float_as_uint(r);
}
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

// k-th work item of CTA c on a grid of G CTAs (>= n_items: the CTA is done)
__device__ __forceinline__ int bwd_item(int k, int G, int c, int zigzag) {
  return k * G + ((zigzag && (k & 1)) ? (G - 1 - c) : c);
}

// Work item L -> its key tile. Causal: tiles slowest, so that the item index orders the items longest first (a key tile
// near the start of the sequence is seen by the most query tiles). Otherwise tiles fastest: the CTAs that run at the same
// time work on one head and share its Q / dO tiles in L2.
__device__ __forceinline__ void bwd_decode(const BwdParams& p, int L, BTile& t) {
  if (p.doc_start == nullptr) {
    int tile, rem;
    if (p.causal) { tile = L / (p.h_kv * p.b); rem = L % (p.h_kv * p.b); }
    else { tile = L % p.n_tile; rem = L / p.n_tile; }
    t.hkv = rem % p.h_kv; t.bat = rem / p.h_kv;
    t.k0 = tile * 128; t.nk = min(128, p.s_k - t.k0); t.krel = t.k0; t.q0 = 0; t.sq = p.s_q; t.off = p.s_k - p.s_q;
    t.nv = p.seqused_k ? min(t.nk, p.seqused_k[t.bat] - t.k0) : t.nk;
  } else {
    // documents sit at 128-aligned starts of one packed batch entry; tile slot x -> (document, key tile of it)
    int x = L / p.h_kv, dsel = -1, len = 0, st = 0;
    t.hkv = L % p.h_kv;
    for (int dI = 0; dI < p.n_docs; ++dI) {
      doc_entry(p.doc_start, p.doc_len, dI, p.s_k, p.ctl.status, st, len);
      const int nb = (len + 127) / 128;
      if (x < nb) { dsel = dI; break; }
      x -= nb;
    }
    if (dsel < 0) { t.nk = 0; t.bat = 0; t.k0 = 0; t.krel = 0; t.q0 = 0; t.sq = 0; t.off = 0; }
    else { t.bat = 0; t.k0 = st + x * 128; t.nk = min(128, len - x * 128); t.krel = x * 128; t.q0 = st; t.sq = len; t.off = 0; }
    t.nv = t.nk;
  }
  // query tiles that see this key tile: the first query that sees its first key, the last one that sees its last key
  int m_hi = (t.sq + 127) / 128, m_lo = 0;
  if (p.win_r >= 0 && t.krel - t.off - p.win_r > 0) m_lo = (t.krel - t.off - p.win_r) / 128;
  if (p.win_l >= 0) m_hi = min(m_hi, max(0, t.krel + t.nk - 1 - t.off + p.win_l) / 128 + 1);
  t.m_lo = m_lo;
  t.n_m = (t.nv > 0 && m_hi > m_lo) ? (m_hi - m_lo) : 0;
}

// Deterministic dQ: how many key tiles before this one also see query tile m of the document (they add their partial sums
// first). The key tiles that see a query tile are a contiguous range; without a left window it starts at key tile 0.
__device__ __forceinline__ int bwd_order_rank(const BwdParams& p, const BTile& t, int m) {
  const int kt = t.krel / 128;
  if (p.win_l < 0) return kt;
  // first key tile whose last query tile is not below m (key tiles are full except the document's last one)
  int klo = 0;
  while (klo < kt && max(0, klo * 128 + 127 - t.off + p.win_l) / 128 < m) ++klo;
  return kt - klo;
}
__device__ __forceinline__ int ld_acquire_gpu(const int32_t* ptr) {
  int v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int32_t* ptr, int v) {
  asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}

// FULL: the variants that also serve the rarer call forms (deterministic dQ order, per-query-row pre-scale, packed
// outputs, the dK mantissa factor), each behind a run-time check of its pointer. A template flag, so that the kernels
// of the plain calls carry none of that code: the loop is sensitive to every register and instruction added to it.
template <int D, bool FP4, int VAR, bool SC, bool FULL = false>
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
  uint8_t* sK = smem;                                  // 2 buffers (items alternate)
  uint8_t* sV = sK + 2 * TILE_BYTES;                   // 2 buffers
  uint8_t* sQ = sV + 2 * TILE_BYTES;                   // 2 stages
  uint8_t* sDO = sQ + 2 * TILE_BYTES;                  // 2 stages
  uint8_t* sDS = sDO + 2 * TILE_BYTES;                 // per half: 128 key rows x 64 query bytes, 64 B swizzle
  uint8_t* sDQ = sDS + 2 * 8192;                       // per half: 128 head-dim rows x 64 queries f16, 128 B swizzle
  float* sVec = reinterpret_cast<float*>(sDQ + 2 * 16384);   // 2 stages x {lse_log2[128], D''[128]}
  // d = 64 only: the gradient rows' way out (2 x 16 KB; at d = 128 the finished item's K / V buffers serve)
  uint8_t* sOut64 = reinterpret_cast<uint8_t*>(sVec) + 2048;
  // FP4 only: NVFP4 K tiles (2 x 8 KB), Q4 stages (2 x 8 KB), scale atoms K 2 x 1 KB + Q 2 x 1 KB
  uint8_t* sK4 = sOut64 + (D == 64 ? 2 * 16384 : 0);
  uint8_t* sQ4 = sK4 + 2 * 8192;
  uint8_t* sSF = sQ4 + 2 * 8192;
  // d = 128, 8-bit route: a second way out for the gradient rows (2 x 16 KB), see the item epilogue
  constexpr bool EPI2 = (D == 128) && !FP4;
  uint8_t* sOut2 = sOut64;
  __shared__ __align__(8) uint64_t bars[BB_COUNT];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ BTile tile_s[2];                          // the items in flight (written by the producer, item k in slot k & 1)
  __shared__ uint32_t sE[2][4];                        // [half][key block] = exponent bytes of the half's two query blocks
  __shared__ uint32_t sEP[2][128];                     // VAR 2: [half][key row] = P-hat exponent bytes of the two query blocks
  __shared__ __align__(4) uint8_t sEQ[2][64][4];       // VAR >= 1: [half][query][key block] = dQ-side dS-hat exponents
  constexpr bool RL = VAR >= 1, TL = VAR == 2;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int grp = p.h / p.h_kv;

  if (tid == 13 * 32) {
    abort_s = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[BB_KV + i], 1); mbar_init(&bars[BB_KVE + i], 2);      // released by one thread of each compute warpgroup
      mbar_init(&bars[BB_QFULL + i], 1); mbar_init(&bars[BB_QEMPTY + i], 1);
      mbar_init(&bars[BB_S + i], 1); mbar_init(&bars[BB_DP + i], 1);
      mbar_init(&bars[BB_P + i], 4); mbar_init(&bars[BB_DS + i], 4); mbar_init(&bars[BB_EX + i], 4);      // one arrival per warp
      mbar_init(&bars[BB_DQF + i], 1); mbar_init(&bars[BB_DQE + i], 4);
      mbar_init(&bars[BB_EP + i], 4); mbar_init(&bars[BB_EPI + i], 4);
    }
    mbar_init(&bars[BB_R1], 4);
    mbar_init(&bars[BB_R2], 4);
    mbar_init(&bars[BB_ACC], 1);
    mbar_init(&bars[BB_ACCFREE], 8);
    fence_barrier_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_acc); tma_prefetch_desc(&tm_dk); tma_prefetch_desc(&tm_dv);
    if (FP4) { tma_prefetch_desc(&tm_q4); tma_prefetch_desc(&tm_k4); }
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  volatile int* abortp = &abort_s;
  // (a status word already set by an earlier launch is not looked at: a kernel that runs after one that gave up does no harm)

  if (warp >= 12) reg_dealloc<80>();     // register budget per warpgroup: 176 / 176 / 80 / 80 (x 128 threads = 64 K)
  if (warp == 13) {
    // =================================================================== TMA producer
    if (lane == 0) {
      int gi = 0;                          // query-tile iterations issued so far, over all items
      bool ok = true;
      for (int k = 0; ok; ++k) {
        const int L = bwd_item(k, G, cta, p.zigzag);
        if (L >= p.n_items) break;
        const int kb = k & 1;
        // the buffers of item k - 2 (and its slot of tile_s) are free once both compute warpgroups have written its
        // gradient rows out of them
        if (k >= 2 && !(ok = mbar_wait(&bars[BB_KVE + kb], ((k >> 1) - 1) & 1, p.ctl, abortp, 11))) break;
        BTile t;
        bwd_decode(p, L, t);
        tile_s[kb] = t;
        if (t.nk > 0) {
          mbar_arrive_expect_tx(&bars[BB_KV + kb], 2 * TILE_BYTES + (FP4 ? 8192 + 1024 : 0));
          tma_load_4d(sK + kb * TILE_BYTES, &tm_k, &bars[BB_KV + kb], 0, t.hkv, t.k0, t.bat);
          tma_load_4d(sV + kb * TILE_BYTES, &tm_v, &bars[BB_KV + kb], 0, t.hkv, t.k0, t.bat);
          if (FP4) {
            tma_load_4d(sK4 + kb * 8192, &tm_k4, &bars[BB_KV + kb], 0, t.hkv, t.k0, t.bat);
            bulk_load(sSF + kb * 1024, p.sfk4 + (((size_t)t.bat * p.h_kv + t.hkv) * (p.s_k / 128) + t.k0 / 128) * 1024, 1024,
                      &bars[BB_KV + kb]);
          }
        } else {
          mbar_arrive(&bars[BB_KV + kb]);  // an empty tile slot: the phase still completes, every role moves on
        }
        const int n_it = t.n_m * grp;
        for (int it = 0; it < n_it; ++it, ++gi) {
          const int st = gi & 1;
          const int head = t.hkv * grp + it / t.n_m, m = t.m_lo + it % t.n_m;
          if (gi >= 2 && !(ok = mbar_wait(&bars[BB_QEMPTY + st], ((gi >> 1) - 1) & 1, p.ctl, abortp, 10))) break;
          mbar_arrive_expect_tx(&bars[BB_QFULL + st], 2 * TILE_BYTES + 1024 + (FP4 ? 8192 + 1024 : 0));
          tma_load_4d(sQ + st * TILE_BYTES, &tm_q, &bars[BB_QFULL + st], 0, head, t.q0 + m * 128, t.bat);
          if (FP4) {
            tma_load_4d(sQ4 + st * 8192, &tm_q4, &bars[BB_QFULL + st], 0, head, t.q0 + m * 128, t.bat);
            bulk_load(sSF + 2048 + st * 1024,
                      p.sfq4 + (((size_t)t.bat * p.h + head) * (p.s_q / 128) + (t.q0 + m * 128) / 128) * 1024, 1024,
                      &bars[BB_QFULL + st]);
          }
          tma_load_4d(sDO + st * TILE_BYTES, &tm_do, &bars[BB_QFULL + st], 0, head, t.q0 + m * 128, t.bat);
          const size_t ro = ((size_t)t.bat * p.h + head) * p.s_q + t.q0 + m * 128;
          bulk_load(sVec + st * 256, p.lse_log2 + ro, 512, &bars[BB_QFULL + st]);
          bulk_load(sVec + st * 256 + 128, p.d_rows + ro, 512, &bars[BB_QFULL + st]);
        }
      }
    }
  } else if (warp == 12) {
    // =================================================================== UMMA issuer
    // The whole warp stays converged through the waits and the descriptor arithmetic (warp-uniform values); one elected
    // lane issues. Descriptors are built once; the loops only add byte offsets.
    constexpr uint32_t ID_N64 = idesc_f8(128, 64, 0, 0);
    const uint32_t tm = __shfl_sync(0xFFFFFFFFu, tmem, 0);
    const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ), do_addr = smem_u32(sDO),
                   ds_addr = smem_u32(sDS);
    const uint64_t dQ0 = smem_desc(q_addr, 16, OP_SBO, OP_SWZ), dDO0 = smem_desc(do_addr, 16, OP_SBO, OP_SWZ),
                   dDS_A = smem_desc(ds_addr, 8192, 512, SWZ_64),   // d = 64: dS-hat as A, next M block 8 KB further
                   dDS0 = smem_desc(ds_addr, 16, 512, SWZ_64);
    const uint32_t k4_addr = smem_u32(sK4);
    const uint64_t dQ40 = smem_desc(smem_u32(sQ4), 16, 512, SWZ_64), dSF0 = smem_desc(smem_u32(sSF), 0, 128, SWZ_NONE);
    int gi = 0;
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int L = bwd_item(k, G, cta, p.zigzag);
      if (L >= p.n_items) break;
      const int kb = k & 1;
      if (!(ok = mbar_wait(&bars[BB_KV + kb], (k >> 1) & 1, p.ctl, abortp, 20))) break;
      const int n_it = tile_s[kb].n_m * grp;
      const int n_steps = 2 * n_it;
      const uint64_t dK_k = smem_desc(k_addr + kb * TILE_BYTES, 16, OP_SBO, OP_SWZ),
                     dV_k = smem_desc(v_addr + kb * TILE_BYTES, 16, OP_SBO, OP_SWZ),
                     dK4 = smem_desc(k4_addr + kb * 8192, 16, 512, SWZ_64);
      for (int t = 0; ok && t <= n_steps; ++t) {
        if (t < n_steps) {
          // ---- front end of step t: S^T_x and dP^T_x
          const int g = gi + (t >> 1), x = t & 1, st = g & 1;
          if (x == 0 && !(ok = mbar_wait(&bars[BB_QFULL + st], (g >> 1) & 1, p.ctl, abortp, 21))) break;
          tc_fence_after();
          const uint64_t qx = desc_adv(dQ0, st * TILE_BYTES + x * 64 * D), dox = desc_adv(dDO0, st * TILE_BYTES + x * 64 * D);
          if (FP4) {
            // the scale columns go into the half's dP^T region: its previous dQ^T must have been read out first
            if (g > 0 && !(ok = mbar_wait(&bars[BB_DQE + x], (g - 1) & 1, p.ctl, abortp, 22))) break;
            tc_fence_after();
          }
          if (elect_one()) {
            if (FP4) {
              const uint32_t park = tm + TC_DP + 64 * x;
              const uint64_t q4x = desc_adv(dQ40, st * 8192 + x * 4096);
#pragma unroll
              for (int kk = 0; kk < 2; ++kk) {
                tmem_cp_sf_atom(park + 4 * kk, desc_adv(dSF0, kb * 1024 + 512 * kk));
                tmem_cp_sf_atom(park + 8 + 4 * kk, desc_adv(dSF0, 2048 + st * 1024 + 512 * kk));
              }
#pragma unroll
              for (int kk = 0; kk < 2; ++kk)   // K = 64 elements = 32 bytes per instruction
                umma_nvf4_ss(tm + TC_S + 64 * x, desc_adv(dK4, 32 * kk), desc_adv(q4x, 32 * kk),
                             idesc_bs(128, 64, 1, 1, 0, 0, 0, 0, 0), park + 4 * kk, park + 8 + 4 * kk + 2 * x, kk > 0);
            } else {
#pragma unroll
              for (int kk = 0; kk < D / 32; ++kk)
                umma_f8_ss(tm + TC_S + 64 * x, desc_adv(dK_k, 32 * kk), desc_adv(qx, 32 * kk), ID_N64, kk > 0);
            }
            tc_commit(&bars[BB_S + x]);
          }
          __syncwarp();
          // the half's dP^T columns hold its previous dQ^T until the reduction warps have read it
          if (!FP4 && g > 0 && !(ok = mbar_wait(&bars[BB_DQE + x], (g - 1) & 1, p.ctl, abortp, 22))) break;
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < D / 32; ++kk)
              umma_f8_ss(tm + TC_DP + 64 * x, desc_adv(dV_k, 32 * kk), desc_adv(dox, 32 * kk), ID_N64, kk > 0);
            tc_commit(&bars[BB_DP + x]);
          }
          __syncwarp();
        }
        if (t >= 1) {
          // ---- back end of step t - 1: dV, dK, dQ^T of half y
          const int tb = t - 1, g = gi + (tb >> 1), y = tb & 1, st = g & 1;
          const uint32_t sx = tm + TC_S + 64 * y;
          const uint64_t qy = desc_adv(dQ0, st * TILE_BYTES + y * 64 * D), doy = desc_adv(dDO0, st * TILE_BYTES + y * 64 * D);
          const uint32_t accum = tb > 0;
          // the first products of an item overwrite dV / dK: the previous item's rows must have left tensor memory
          if (tb == 0 && k > 0 && !(ok = mbar_wait(&bars[BB_ACCFREE], (k - 1) & 1, p.ctl, abortp, 25))) break;
          if (!(ok = mbar_wait(&bars[BB_P + y], g & 1, p.ctl, abortp, 23))) break;
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 2; ++kk)     // K = 64 queries: two instructions of 32
              umma_mxf8_ts(tm + TC_DV, sx + TO_P + 8 * kk, desc_adv(doy, kk * 32 * D),
                           idesc_bs(128, D, 0, 0, 0, 1, 1, kk, kk), sx + TO_SFA_P, sx + TO_SFB_DO, accum | kk);
          }
          __syncwarp();
          if (!(ok = mbar_wait(&bars[BB_DS + y], g & 1, p.ctl, abortp, 24))) break;
          tc_fence_after();
          if (elect_one()) {
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
            if (y == 1) tc_commit(&bars[BB_QEMPTY + st]);
          }
          __syncwarp();
        }
      }
      if (!ok) break;
      // an item without query tiles issues nothing, but its accumulator hand-over still takes place once
      if (n_steps == 0 && k > 0 && !(ok = mbar_wait(&bars[BB_ACCFREE], (k - 1) & 1, p.ctl, abortp, 25))) break;
      if (elect_one()) tc_commit(&bars[BB_ACC]);       // every product of the item has completed when this arrives
      __syncwarp();
      gi += n_it;
    }
  } else if (warp >= 8 && warp < 12) {
    reg_dealloc<80>();
    // =================================================================== dQ reduction (thread = head-dim row)
    const int r = tid & 127;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    bool ok = true;
    int gi = 0, gt = 0;                     // iterations and half steps so far, over all items
    for (int k = 0; ok; ++k) {
      const int L = bwd_item(k, G, cta, p.zigzag);
      if (L >= p.n_items) break;
      const int kb = k & 1;
      if (!(ok = mbar_wait(&bars[BB_KV + kb], (k >> 1) & 1, p.ctl, abortp, 43))) break;
      const BTile T = tile_s[kb];
      const int n_it = T.n_m * grp;
      for (int t = 0; t < 2 * n_it; ++t, ++gt) {
        const int it = t >> 1, y = t & 1, g = gi + it;
        const int head = T.hkv * grp + it / T.n_m, m = T.m_lo + it % T.n_m;
        // the staging buffer of this half was last read by the reduction of step gt - 2
        if (tid == 256) tma_store_wait_read<1>();
        mbar_arrive_warp(&bars[BB_R1]);
        if (!(ok = mbar_wait(&bars[BB_R1], gt & 1, p.ctl, abortp, 41))) break;
        if (!(ok = mbar_wait(&bars[BB_DQF + y], g & 1, p.ctl, abortp, 40))) break;
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
        fence_proxy_async();
        mbar_arrive_warp(&bars[BB_R2]);
        if (!(ok = mbar_wait(&bars[BB_R2], gt & 1, p.ctl, abortp, 42))) break;
        const bool det = FULL && p.dq_order != nullptr;
        if (!det) {
          if (tid == 256) {
            if (D == 128) tma_reduce_add_4d(&tm_acc, sDQ + y * 16384, T.q0 + m * 128 + 64 * y, 0, head, T.bat);
            else tma_reduce_add_4d(&tm_acc, sDQ + y * 16384, 0, T.q0 + m * 128 + 64 * y, head, T.bat);
            tma_store_commit();
          }
        } else if (warp == 8) {                 // (the whole warp stays converged: lane 0 works, the others follow its result)
          int go = 1;
          int32_t* order = nullptr;
          int rank = 0;
          {
            // deterministic order: the key tiles before this one have added their partial sums of this half
            order = p.dq_order + ((((size_t)T.bat * p.h + head) * (p.s_q / 128) + T.q0 / 128 + m) * 2 + y);
            rank = bwd_order_rank(p, T, m);
            if (lane == 0) {
              const long long t_start = clock64();
              while (ld_acquire_gpu(order) != rank) {
                if (*abortp || clock64() - t_start > p.ctl.wait_cycles) {
                  if (p.ctl.status) atomicCAS(p.ctl.status, 0, FL_DEV_WAIT_TIMEOUT | 44);
                  *abortp = 1;
                  go = 0;
                  break;
                }
              }
            }
            go = __shfl_sync(0xFFFFFFFFu, go, 0);
          }
          if (go && lane == 0) {
            if (D == 128) tma_reduce_add_4d(&tm_acc, sDQ + y * 16384, T.q0 + m * 128 + 64 * y, 0, head, T.bat);
            else tma_reduce_add_4d(&tm_acc, sDQ + y * 16384, 0, T.q0 + m * 128 + 64 * y, head, T.bat);
            tma_store_commit();
            if (order) {
              tma_store_wait<0>();                // the addition has completed, not only read its source
              __threadfence();
              st_release_gpu(order, rank + 1);
            }
          }
          __syncwarp();
          if (!go) ok = false;           // the other warps of the group see the flag at their next wait
        }
        if (!ok) break;
      }
      gi += n_it;
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
    const uint32_t ds_row = smem_u32(sDS) + x * 8192 + r * 64;
    bool ok = true;
    int gi = 0, epi = 0;                             // iterations so far; uses of the epilogue barrier so far
    int pending_kve = -1;                            // the K / V buffer whose gradient stores are still to be confirmed
    for (int k = 0; ok; ++k) {
      const int L = bwd_item(k, G, cta, p.zigzag);
      if (L >= p.n_items) break;
      const int kb = k & 1;
      if (!(ok = mbar_wait(&bars[BB_KV + kb], (k >> 1) & 1, p.ctl, abortp, 39))) break;
      // token-local variant: short of registers, so the tile is read from its slot where needed (the slot stays valid until
      // this item's buffers are released); otherwise a register copy
      const BTile Tcopy = tile_s[kb];
      const BTile& T = TL ? tile_s[kb] : Tcopy;
      const int hkv = T.hkv, n_m = T.n_m, m_lo = T.m_lo;
      const int n_it = n_m * grp;
      const int krel = T.krel + r;
      const bool key_valid = r < T.nv;
      const size_t bh_k = (size_t)T.bat * p.h_kv + hkv;
      const int kblk = (T.k0 + r) / 32;
      // token-local: this key's own factors; otherwise its 32-key block's
      const float fk_true = TL ? p.fac_k[bh_k * p.s_k + T.k0 + r] : p.fac_k[bh_k * (p.s_k / 32) + kblk];
      const float fk = fk_true * p.scale_log2;
      const float fv8 = (TL ? p.fac_v[bh_k * p.s_k + T.k0 + r] : p.fac_v[bh_k * (p.s_k / 32) + kblk]) * 0.00390625f;   // f_V 2^-8
      uint32_t ek_word = TL ? 0x7F7F7F7Fu : 0u;        // UE8M0 bytes of the tile's four key blocks (unit when token-local)
      if (!TL) {
#pragma unroll
        for (int kbk = 0; kbk < 4; ++kbk)
          ek_word |= ((__float_as_uint(p.fac_k[bh_k * (p.s_k / 32) + T.k0 / 32 + kbk]) >> 23) & 0xFF) << (8 * kbk);
      }
      const int vis_from = p.win_r >= 0 ? (krel - T.off - p.win_r) : 0;    // queries in [vis_from, vis_to] see this key
      const int vis_to = p.win_l >= 0 ? (krel - T.off + p.win_l) : 0x7FFFFFFF;
      for (int it = 0; it < n_it; ++it) {
        const int g = gi + it, st = g & 1, u = g >> 1;
        const int head = hkv * grp + it / n_m, m = m_lo + it % n_m;
        if (it == 1 && pending_kve >= 0) {
          // the previous item's gradient stores have long read their shared-memory source: its K / V buffer goes back
          if (r == 0) { tma_store_wait_read<0>(); mbar_arrive(&bars[BB_KVE + pending_kve]); }
          pending_kve = -1;
        }
        const size_t bh_q = (size_t)T.bat * p.h + head;
        const int qb0 = (T.q0 + m * 128) / 32 + 2 * x;                     // first of the half's two 32-query blocks
        const float fq0 = TL ? 1.f : p.fac_q[bh_q * (p.s_q / 32) + qb0], fq1 = TL ? 1.f : p.fac_q[bh_q * (p.s_q / 32) + qb0 + 1];
        const float fd0 = TL ? 1.f : p.fac_do[bh_q * (p.s_q / 32) + qb0], fd1 = TL ? 1.f : p.fac_do[bh_q * (p.s_q / 32) + qb0 + 1];
        // token-local: the 64 per-query factors of the half (same addresses for every thread: broadcast loads)
        const float4* fq_vec = reinterpret_cast<const float4*>(p.fac_q + (TL ? bh_q * p.s_q + T.q0 + m * 128 + 64 * x : 0));
        const float4* fdo_vec = reinterpret_cast<const float4*>(p.fac_do + (TL ? bh_q * p.s_q + T.q0 + m * 128 + 64 * x : 0));
        // the f16 pre-scale: one power of two per query tile (folded into K's exponent bytes below), or one per query row
        // (folded into the dQ side's B scale bytes, whose lanes are the queries)
        const bool pre_rows = FULL && p.dq_scale_rows != nullptr;
        const float bsc = pre_rows ? 1.0f : p.dq_scale[(size_t)T.bat * (p.s_q / 128) + T.q0 / 128 + m];
        [[maybe_unused]] uint32_t lq0 = 0, lq1 = 0;
        if (pre_rows) {
          const float* rp = p.dq_scale_rows + (size_t)T.bat * p.s_q + T.q0 + m * 128 + 64 * x;
          lq0 = ((uint32_t)((int)((__float_as_uint(rp[lane]) >> 23) & 0xFF) - 127) & 0xFF) * 0x01010101u;
          lq1 = ((uint32_t)((int)((__float_as_uint(rp[32 + lane]) >> 23) & 0xFF) - 127) & 0xFF) * 0x01010101u;
        }
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
        if (!(ok = mbar_wait(&bars[BB_S + x], g & 1, p.ctl, abortp, 31))) break;
        tc_fence_after();
        uint32_t pv[64];
        FL_TMEM_LD_32(t_sx, pv);
        FL_TMEM_LD_32(t_sx + 32, (pv + 32));
        tc_wait_ld();
        float pf[64];
        [[maybe_unused]] uint32_t pw_sc[SC ? 16 : 1];
        if constexpr (SC) {
          // soft cap: x = cap_a tanh(s c cap_b); P-hat is taken from P' right here, and what stays in pf is
          // P' (1 - tanh^2), the factor dS needs (the reference's score_mod_bwd, flash_attn/cute/utils.py:178-187)
#pragma unroll
          for (int j4 = 0; j4 < 16; ++j4) {
            const float4 l4 = lds128(v_lse + 16 * j4);
            const float cc = c[j4 >> 3];
            const float l[4] = {l4.x, l4.y, l4.z, l4.w};
            float pp[4], df[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float th = tanh_fast(__uint_as_float(pv[4 * j4 + e]) * (cc * p.cap_b));
              pp[e] = ex2(fmaf(p.cap_a, th, -l[e]));
              df[e] = fmaf(-th, th, 1.0f);
              if (!full) {
                const int qi = q_first + 4 * j4 + e;
                pp[e] = (key_valid && qi >= vis_from && qi <= vis_to && qi < T.sq) ? pp[e] : 0.f;
              }
            }
            pw_sc[j4] = cvt_e4m3x4(pp[0], pp[1], pp[2], pp[3]);
#pragma unroll
            for (int e = 0; e < 4; ++e) pf[4 * j4 + e] = pp[e] * df[e];
          }
        } else {
#pragma unroll
          for (int j4 = 0; j4 < 16; ++j4) {
            const float4 l4 = lds128(v_lse + 16 * j4);
            const float cc = c[j4 >> 3];
            if (TL) {
              // t = lse2 - s f_K f_Q(query), two columns per instruction
              const float4 f4 = __ldg(fq_vec + j4);
              const uint64_t nfk2 = pack2(-fk, -fk);
              float t0, t1, t2, t3;
              unpack2(fma2(pack2(__uint_as_float(pv[4 * j4 + 0]), __uint_as_float(pv[4 * j4 + 1])),
                           mul2(pack2(f4.x, f4.y), nfk2), pack2(l4.x, l4.y)), t0, t1);
              unpack2(fma2(pack2(__uint_as_float(pv[4 * j4 + 2]), __uint_as_float(pv[4 * j4 + 3])),
                           mul2(pack2(f4.z, f4.w), nfk2), pack2(l4.z, l4.w)), t2, t3);
              pf[4 * j4 + 0] = ex2_neg(t0);
              pf[4 * j4 + 1] = ex2_neg(t1);
              pf[4 * j4 + 2] = ex2_neg(t2);
              pf[4 * j4 + 3] = ex2_neg(t3);
            } else {
              // two columns per instruction: t = lse2 - s c, P' = 2^-t
              const uint64_t nc2 = pack2(-cc, -cc);
              float t0, t1, t2, t3;
              unpack2(fma2(pack2(__uint_as_float(pv[4 * j4 + 0]), __uint_as_float(pv[4 * j4 + 1])), nc2, pack2(l4.x, l4.y)), t0, t1);
              unpack2(fma2(pack2(__uint_as_float(pv[4 * j4 + 2]), __uint_as_float(pv[4 * j4 + 3])), nc2, pack2(l4.z, l4.w)), t2, t3);
              pf[4 * j4 + 0] = ex2_neg(t0);
              pf[4 * j4 + 1] = ex2_neg(t1);
              pf[4 * j4 + 2] = ex2_neg(t2);
              pf[4 * j4 + 3] = ex2_neg(t3);
            }
          }
        }
        if (!SC && !full) {      // diagonal / tail tiles only
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
              unpack2(mul2(pack2(pf[j + 0], pf[j + 1]), pack2(f4.x, f4.y)), t[4 * j4 + 0], t[4 * j4 + 1]);
              unpack2(mul2(pack2(pf[j + 2], pf[j + 3]), pack2(f4.z, f4.w)), t[4 * j4 + 2], t[4 * j4 + 3]);
              am = fmax3_abs(fmax3_abs(am, t[4 * j4], t[4 * j4 + 1]), t[4 * j4 + 2], t[4 * j4 + 3]);   // all >= 0
            }
            ep[qh] = exp448(__float_as_uint(am));
            const float inv = pow2_inv(ep[qh]);
            const uint64_t inv2 = pack2(inv, inv);
#pragma unroll
            for (int w = 0; w < 8; ++w) {
              float a0, a1, a2, a3;
              unpack2(mul2(pack2(t[4 * w], t[4 * w + 1]), inv2), a0, a1);
              unpack2(mul2(pack2(t[4 * w + 2], t[4 * w + 3]), inv2), a2, a3);
              pw[qh * 8 + w] = cvt_e4m3x4(a0, a1, a2, a3);
            }
          }
          FL_TMEM_ST_16(t_sx + TO_P, pw);
          // every lane quadrant holds the whole A scale tile: column = key block, lane = row of the block
          sEP[x][r] = ep[0] | (ep[1] << 8);
          mbar_arrive_warp(&bars[BB_EP + x]);
          if (!(ok = mbar_wait(&bars[BB_EP + x], g & 1, p.ctl, abortp, 37))) break;
          uint32_t sf[8] = {sEP[x][lane], sEP[x][32 + lane], sEP[x][64 + lane], sEP[x][96 + lane],
                            0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu};
          FL_TMEM_ST_8(t_sx + TO_SFA_P, sf);
        } else {
          uint32_t pw[16];
#pragma unroll
          for (int w = 0; w < 16; ++w) {
            if constexpr (SC) pw[w] = pw_sc[w];
            else pw[w] = cvt_e4m3x4(pf[4 * w], pf[4 * w + 1], pf[4 * w + 2], pf[4 * w + 3]);
          }
          FL_TMEM_ST_16(t_sx + TO_P, pw);
          // scale tiles of the dV product: A = 1, B = dO's exponent per 32 queries (bytes = the half's two K steps)
          uint32_t sf[8] = {0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, edo2, edo2, edo2, edo2};
          FL_TMEM_ST_8(t_sx + TO_SFA_P, sf);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive_warp(&bars[BB_P + x]);

        // ---- dS = P' (b dP + D''), block exponent per (this warp's 32 keys, 32 queries)
        if (!(ok = mbar_wait(&bars[BB_DP + x], g & 1, p.ctl, abortp, 32))) break;
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
            if (TL) {
              // b = f_V(key) f_dO(query) per column; the dK side's maximum carries f_Q(query)
              const float4 f4 = __ldg(fdo_vec + qh * 8 + j4);
              const float4 q4 = __ldg(fq_vec + qh * 8 + j4);
              const uint64_t fv2 = pack2(fv8, fv8);
              const uint64_t u01 = fma2(pack2(__uint_as_float(pv[j + 0]), __uint_as_float(pv[j + 1])),
                                        mul2(pack2(f4.x, f4.y), fv2), pack2(d4.x, d4.y));
              const uint64_t u23 = fma2(pack2(__uint_as_float(pv[j + 2]), __uint_as_float(pv[j + 3])),
                                        mul2(pack2(f4.z, f4.w), fv2), pack2(d4.z, d4.w));
              const uint64_t p01 = mul2(pack2(pf[j + 0], pf[j + 1]), u01), p23 = mul2(pack2(pf[j + 2], pf[j + 3]), u23);
              unpack2(p01, pf[j + 0], pf[j + 1]);
              unpack2(p23, pf[j + 2], pf[j + 3]);
              float w0, w1, w2, w3;
              unpack2(mul2(p01, pack2(q4.x, q4.y)), w0, w1);
              unpack2(mul2(p23, pack2(q4.z, q4.w)), w2, w3);
              am = fmax3_abs(fmax3_abs(am, w0, w1), w2, w3);
            } else {
              // two columns per instruction
              const uint64_t b2 = pack2(b8[qh], b8[qh]);
              const uint64_t u01 = fma2(pack2(__uint_as_float(pv[j + 0]), __uint_as_float(pv[j + 1])), b2, pack2(d4.x, d4.y));
              const uint64_t u23 = fma2(pack2(__uint_as_float(pv[j + 2]), __uint_as_float(pv[j + 3])), b2, pack2(d4.z, d4.w));
              unpack2(mul2(pack2(pf[j + 0], pf[j + 1]), u01), pf[j + 0], pf[j + 1]);
              unpack2(mul2(pack2(pf[j + 2], pf[j + 3]), u23), pf[j + 2], pf[j + 3]);
              am = fmax3_abs(fmax3_abs(am, pf[j], pf[j + 1]), pf[j + 2], pf[j + 3]);
            }
          }
          const uint32_t wm = warp_max_u32(__float_as_uint(am));          // non-negative floats order as integers
          ebyte[qh] = exp448(wm);                                          // 448 * 2^(e-127) >= amax
        }
        if (!full) {      // diagonal / tail tiles only
          // masked entries hold P' = 0, but their dP^T or D'' may come from rows outside the document (padding or whatever
          // the buffer held: possibly Inf / NaN), and 0 * NaN is NaN: select again after the multiply. (The maxima above
          // ignore NaN, so the block exponents are those of the visible entries.)
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            const int qi = q_first + j;
            pf[j] = (key_valid && qi >= vis_from && qi <= vis_to && qi < T.sq) ? pf[j] : 0.f;
          }
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
            const uint64_t inv2 = pack2(inv, inv);
            float a0, a1, a2, a3;
            if (TL) {
              const float4 f4 = __ldg(fq_vec + qh * 8 + w);      // f_Q(query) 2^(127 - e): powers of two, exact, in range
              unpack2(mul2(pack2(pf[j0], pf[j0 + 1]), mul2(pack2(f4.x, f4.y), inv2)), a0, a1);
              unpack2(mul2(pack2(pf[j0 + 2], pf[j0 + 3]), mul2(pack2(f4.z, f4.w), inv2)), a2, a3);
              dsw[qh * 8 + w] = cvt_e4m3x4(a0, a1, a2, a3);
            } else {
              unpack2(mul2(pack2(pf[j0], pf[j0 + 1]), inv2), a0, a1);
              unpack2(mul2(pack2(pf[j0 + 2], pf[j0 + 3]), inv2), a2, a3);
              dsw[qh * 8 + w] = cvt_e4m3x4(a0, a1, a2, a3);
            }
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
              const uint32_t wm = warp_max_abs_f32(a);
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
        if (!(ok = mbar_wait(&bars[BB_EX + x], g & 1, p.ctl, abortp, 36))) break;
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
          if constexpr (FULL) {
            sf[12] = __vadd4(sf[12], lq0);
            sf[13] = __vadd4(sf[13], lq1);
          }
          sf[14] = sf[15] = 0x7F7F7F7Fu;
          FL_TMEM_ST_16(t_sx + TO_SFA_DK, sf);
        }
        tc_wait_st();
        fence_proxy_async();             // the dS-hat tile in shared memory is read by the tensor core (async proxy)
        tc_fence_before();
        mbar_arrive_warp(&bars[BB_DS + x]);
      }
      if (!ok) break;
      gi += n_it;

      // ---- item epilogue: warpgroup 0 writes dV, warpgroup 1 writes dK (full rows)
      if (!(ok = mbar_wait(&bars[BB_ACC], k & 1, p.ctl, abortp, 33))) break;
      tc_fence_after();
      {
        const uint32_t t_acc = lane_base + (x == 0 ? TC_DV : TC_DK);
        // dV carries 2^8 (P'), dK the softmax scale (and the mantissa of a Q factor that is no power of two)
        const float mult = (x == 0) ? 0.00390625f : p.softmax_scale * ((FULL && p.dk_mult) ? p.dk_mult[bh_k] : 1.0f);
        const float mk = key_valid ? mult : 0.f;       // rows past the end of the document store zeros
        uint32_t v[D];
        if (n_it > 0) {                  // (CTA-uniform: the tensor-memory loads are warp-collective)
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) FL_TMEM_LD_32(t_acc + 32 * cc, (v + 32 * cc));   // all loads in flight, one wait
          tc_wait_ld();
        } else {                         // no query tile saw this key tile
#pragma unroll
          for (int e = 0; e < D; ++e) v[e] = 0;
        }
        // the accumulators are in registers: the next item's products may overwrite them
        tc_fence_before();
        mbar_arrive_warp(&bars[BB_ACCFREE]);
        // pairs of neighbouring columns in one 64-bit register: every step below is one instruction per pair
        uint64_t Y[D / 2];
        if (D == 128 && x == 1 && p.had_dk) {       // dK of rotated operands: (y H / sqrt(128)) * signs
#pragma unroll
          for (int i = 0; i < D / 2; ++i) {         // butterfly level 1: the two halves of a pair
            const float a = __uint_as_float(v[2 * i]), b2 = __uint_as_float(v[2 * i + 1]);
            Y[i] = pack2(a + b2, a - b2);
          }
#pragma unroll
          for (int hs = 1; hs < D / 2; hs <<= 1) {  // levels 2 .. D / 2: whole pairs
#pragma unroll
            for (int i = 0; i < D / 2; ++i) {
              if ((i & hs) == 0) {
                const uint64_t a = Y[i], b2 = Y[i + hs];
                Y[i] = add2(a, b2);
                Y[i + hs] = sub2(a, b2);
              }
            }
          }
          constexpr uint32_t NEG[4] = {0x10D2E03Eu, 0xE0D9F0E2u, 0x45809F07u, 0x75954FEDu};
          const float cp = 0.08838834764831845f * mk, cn = -cp;
#pragma unroll
          for (int i = 0; i < D / 2; ++i) {
            const bool n0 = (NEG[(2 * i) >> 5] >> ((2 * i) & 31)) & 1, n1 = (NEG[(2 * i + 1) >> 5] >> ((2 * i + 1) & 31)) & 1;
            Y[i] = mul2(Y[i], pack2(n0 ? cn : cp, n1 ? cn : cp));
          }
        } else {
          const uint64_t mk2 = pack2(mk, mk);
#pragma unroll
          for (int i = 0; i < D / 2; ++i) Y[i] = mul2(pack2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])), mk2);
        }
        // rows -> shared memory (boxes of 64 elements, 128 B swizzle) -> one TMA store per box: a thread's own row
        // written straight to global memory costs 32 separate 128-byte lines per warp instruction. At d = 128 the first
        // box goes through the finished item's K (warpgroup 0) / V (warpgroup 1) buffer: every product that read it has
        // completed. The second box has a buffer of its own where shared memory allows (the 8-bit route), so that both
        // stores are issued together and nobody waits for them here: the thread that issued them confirms that they have
        // read their source, and only then hands the K / V buffer back to the producer, one query tile into the next item.
        if (pending_kve >= 0) {          // (an item with fewer than two query tiles came in between)
          if (r == 0) { tma_store_wait_read<0>(); mbar_arrive(&bars[BB_KVE + pending_kve]); }
          pending_kve = -1;
          mbar_arrive_warp(&bars[BB_EPI + x]);
          if (!(ok = mbar_wait(&bars[BB_EPI + x], epi & 1, p.ctl, abortp, 38))) break;
          ++epi;
        }
        uint8_t* stage0 = (D == 128) ? ((x == 0 ? sK : sV) + kb * TILE_BYTES) : (sOut64 + x * 16384);
        uint8_t* stage1 = EPI2 ? (sOut2 + x * 16384) : stage0;
        const CUtensorMap* tm_out = (x == 0) ? &tm_dv : &tm_dk;
        // packed output: the key tile is slot T.k0 / 128 of the aligned buffer; its rows go to the packed rows out_row ..
        // + out_n of the caller's tensor: a full slot as TMA stores, a document's last rows row by row
        int out_row = T.k0, out_n = T.nk > 0 ? 128 : 0;
        if (FULL && p.slot_src) {
          out_row = T.nk > 0 ? p.slot_src[T.k0 / 128] : -1;
          out_n = (T.nk > 0 && out_row >= 0) ? min(p.slot_rows[T.k0 / 128], 128) : 0;
        }
        const bool by_rows = FULL && p.slot_src && out_n < 128;   // (CTA-uniform)
        uint16_t* out_base = reinterpret_cast<uint16_t*>(x == 0 ? p.dv : p.dk);
#pragma unroll
        for (int pass = 0; pass < D / 64; ++pass) {
          uint8_t* stage = pass == 0 ? stage0 : stage1;
          const uint32_t srow = smem_u32(stage) + r * 128;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float a, b2;
              unpack2(Y[32 * pass + 4 * c8 + e], a, b2);
              if (p.out_f16) {
                __half2 hh = __floats2half2_rn(a, b2);
                w[e] = *reinterpret_cast<uint32_t*>(&hh);
              } else {
                w[e] = pack_bf16x2(a, b2);
              }
            }
            if (by_rows) {
              if (r < out_n)
                *reinterpret_cast<uint4*>(out_base + ((size_t)(out_row + r) * p.h_kv + hkv) * D + 64 * pass + 8 * c8) =
                    make_uint4(w[0], w[1], w[2], w[3]);
            } else {
              sts128(srow + ((c8 ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
            }
          }
          if (by_rows) continue;
          const bool last = pass + 1 == D / 64;
          if (EPI2 && !last) continue;                    // both boxes are announced together
          fence_proxy_async();
          mbar_arrive_warp(&bars[BB_EPI + x]);            // the warpgroup's four warps have written their rows
          if (!(ok = mbar_wait(&bars[BB_EPI + x], epi & 1, p.ctl, abortp, 38))) break;
          ++epi;
          if (r == 0 && out_n == 128) {
            if (EPI2) tma_store_4d(tm_out, stage0, 0, hkv, out_row, T.bat);
            tma_store_4d(tm_out, stage, 64 * pass, hkv, out_row, T.bat);
            tma_store_commit();
            if (!last) tma_store_wait_read<0>();          // the one buffer is written again by the next pass
          }
          if (!last) {
            mbar_arrive_warp(&bars[BB_EPI + x]);
            if (!(ok = mbar_wait(&bars[BB_EPI + x], epi & 1, p.ctl, abortp, 38))) break;
            ++epi;
          }
        }
        if (!ok) break;
        pending_kve = kb;
      }
    }
    // the shared-memory sources of the last stores must outlive the copies (the writes complete with the grid)
    if (r == 0) tma_store_wait_read<0>();
  }
  if (abort_s) {
    for (int it = 0; it < 200; ++it) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace fl

extern "C" int fl_bwd(const fl_attn_args* a, void* stream) {
  using namespace fl;
  if (!a || !a->q_codes || !a->k_codes || !a->v_codes || !a->do_codes || !a->status) return FL_ERR_BAD_ARG;
  if (!a->fac_q || !a->fac_k || !a->fac_v || !a->fac_do || !a->lse_log2 || !a->d_rows || !a->dq_acc || (!a->dq_scale && !a->dq_scale_rows) ||
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
  if (a->seqused_k && a->doc_start) return FL_ERR_UNSUPPORTED;      // documents carry their own lengths
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
  if ((rc = make_rows_map_16(&mdk, a->dk, a->b, a->slot_src ? a->out_rows : a->s_k, a->h_kv, a->d, 128))) return rc;
  if ((rc = make_rows_map_16(&mdv, a->dv, a->b, a->slot_src ? a->out_rows : a->s_k, a->h_kv, a->d, 128))) return rc;
  BwdParams p;
  p.fac_q = a->fac_q; p.fac_k = a->fac_k; p.fac_v = a->fac_v; p.fac_do = a->fac_do; p.lse_log2 = a->lse_log2;
  p.d_rows = a->d_rows; p.dq_scale = a->dq_scale; p.dq_scale_rows = a->dq_scale_rows; p.dk = a->dk; p.dv = a->dv;
  p.dk_mult = a->dk_mult;
  if (a->dk_mult && a->doc_start) return FL_ERR_UNSUPPORTED;            // per-(batch row, head) factors: the batched form
  p.slot_src = a->slot_src; p.slot_rows = a->slot_rows;
  if (a->slot_src && (!a->doc_start || !a->slot_rows || a->out_rows <= 0)) return FL_ERR_BAD_ARG;
  if (a->dq_scale_rows && a->doc_start) return FL_ERR_UNSUPPORTED;      // per-row pre-scale: the batched form
  p.sfq4 = a->sfq4; p.sfk4 = a->sfk4;
  p.doc_start = a->doc_start; p.doc_len = a->doc_len; p.n_docs = a->n_docs;
  p.seqused_k = a->seqused_k;
  p.dq_order = a->dq_order;
  p.b = a->b; p.s_q = a->s_q; p.s_k = a->s_k; p.h = a->h; p.h_kv = a->h_kv;
  p.softmax_scale = a->softmax_scale;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  const bool sc = a->softcap > 0.f;
  if (sc && (tl || rl)) return FL_ERR_UNSUPPORTED;     // soft cap: the default dS-hat route only
  p.cap_a = sc ? a->softcap * 1.4426950408889634f : 0.f;
  p.cap_b = sc ? 1.0f / p.cap_a : 0.f;
  p.causal = (a->flags & FL_A_CAUSAL) ? 1 : 0;
  p.win_l = a->window_left_p1 - 1;
  p.win_r = p.causal ? 0 : a->window_right_p1 - 1;
  p.out_f16 = (a->flags & FL_A_OUT_F16) ? 1 : 0;
  p.had_dk = (a->flags & FL_A_HAD_DK) ? 1 : 0;
  p.ctl.status = a->status;
  p.ctl.wait_cycles = a->wait_cycles > 0 ? a->wait_cycles : kDefaultWaitCycles;
  const int ntile = a->doc_start ? (a->s_k / 128 + a->n_docs) : a->s_k / 128;
  const int nb = a->doc_start ? 1 : a->b;
  p.n_tile = ntile;
  const long long n_items = (long long)ntile * a->h_kv * nb;
  if (n_items > 0x3FFFFFFF) return FL_ERR_TOO_LARGE;
  p.n_items = (int)n_items;
  p.zigzag = (p.causal && !a->doc_start) ? 1 : 0;
  const int grid = (int)(n_items < sm_count() ? n_items : sm_count());     // one persistent CTA per SM
  const int smem = 8 * 128 * a->d + 2 * 8192 + 2 * 16384 + 2048 + ((a->d == 64 || !fp4) ? 2 * 16384 : 0) + 1024 +
                   (fp4 ? 4 * 8192 + 4 * 1024 : 0);
  auto launch = [&](auto kern) -> int {
    if (cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); e != cudaSuccess)
      return cuda_fail((int)e, "fl_bwd: cudaFuncSetAttribute");
    kern<<<grid, 512, smem, (cudaStream_t)stream>>>(mq, mk, mv, mdo, macc, mq4, mk4, mdk, mdv, p);
    return FL_OK;
  };
  const bool det = a->dq_order != nullptr;
  if (det && (sc || rl || tl)) return FL_ERR_UNSUPPORTED;     // ordered dQ: the default dS-hat route only
  // the lean kernels serve the plain calls; any of the rarer forms takes the full variant of the same kernel
  const bool full = det || a->dq_scale_rows || a->slot_src || a->dk_mult;
#define FL_BWD_LAUNCH(D_, FP4_, VAR_, SC_) \
  (full ? launch(bwd_kernel_pipelined<D_, FP4_, VAR_, SC_, true>) : launch(bwd_kernel_pipelined<D_, FP4_, VAR_, SC_, false>))
  if (sc) {
    if (a->d == 64) rc = FL_BWD_LAUNCH(64, false, 0, true);
    else rc = fp4 ? FL_BWD_LAUNCH(128, true, 0, true) : FL_BWD_LAUNCH(128, false, 0, true);
  } else if (a->d == 64) {
    rc = FL_BWD_LAUNCH(64, false, 0, false);
  } else if (fp4) {
    rc = rl ? FL_BWD_LAUNCH(128, true, 1, false) : FL_BWD_LAUNCH(128, true, 0, false);
  } else if (tl) {
    rc = FL_BWD_LAUNCH(128, false, 2, false);
  } else {
    rc = rl ? FL_BWD_LAUNCH(128, false, 1, false) : FL_BWD_LAUNCH(128, false, 0, false);
  }
#undef FL_BWD_LAUNCH
  if (rc) return rc;
  return launch_result("fl_bwd: kernel launch");
}
