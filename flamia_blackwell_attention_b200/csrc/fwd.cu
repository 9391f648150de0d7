// Forward attention kernel for sm_100a: O = softmax(scale * Q K^T + mask) V and LSE on block-scaled operands, on a
// persistent grid.
//
// Replaces the reference's FlashAttentionForwardSm100 (flash_attn/cute/flash_fwd_sm100_fp4.py:370), its driver
// _flash_attn_fwd (flash_attn/cute/interface_fwd_fp4.py:301) and its persistent longest-first tile scheduling
// (interface_fwd_fp4.py:1148-1166, 1203-1208) for the two in-scope routes:
//   FL_MODE_FP8: S = E4M3 x E4M3 (kind::f8f6f4); the power-of-two token-block factors f_Q[row/32] * f_K[key/32] are
//                folded into the softmax scale (exact); P.V = kind::mxf8f6f4.block_scale with V's UE8M0 exponent per
//                32 keys as the B scale.
//   FL_MODE_FP4: S = NVFP4 x NVFP4 (kind::mxf4nvf4.block_scale.scale_vec::4X), same P.V.
//   softcap c:   score = scale q.k becomes c tanh(score / c) before masking (flash_attn/cute/utils.py:167-175).
//   FL_A_TOKEN_LOCAL (the reference's "fold forward", flash_attn/cute/lowprec/_routes.py:749-786): every token of Q, K,
//                V has its own power-of-two factor; f_Q f_K multiplies each score, log2 f_V(key) is added to the exponent
//                argument of P-hat (so P.V runs with unit scales) and the row sum takes P / f_V(key) back out.
// P-hat frames (the A operand of P.V, E4M3):
//   row frame    P-hat = E4M3(2^(x - m + 4)) with a constant-one A scale: one frame per query row.
//   group frame  (FL_A_P_GROUP; the reference's _fused_log2_group_quant, flash_fwd_sm100_fp4.py:5426-5600): per 32 keys
//                g of a row, bias_g = ceil(max(m_g, -100) - log2 448) with m_g the group's largest x - m + log2 448;
//                P-hat = E4M3(2^(x - m + log2 448 - bias_g)), in (224, 448] at the group's maximum; A scale byte
//                127 + bias_g per (row, 32 keys); row sum += 2^bias_g * sum of the group; the LSE takes log2 448 back out
//                (flash_fwd_sm100_fp4.py:6433-6437).
//
// Masks: bottom-right aligned causal and / or a sliding window (query i sees keys i + off - left .. i + off + right); a block
// starts at the first key tile any of its rows can see and only boundary tiles are masked element by element.
//
// One CTA per SM walks a static list of work items = 256 query rows (two 128-row stages) of one (batch | document, head):
// under the causal mask the items are ordered longest first and dealt out in zigzag rounds. All pipelines run across
// items: the K / V ring never drains, the next item's Q tiles land in a second buffer and its first S products are issued
// while the softmax warps still write the current item's output.
//   warps 0-3   softmax stage 0 (thread r owns query row r: TMEM lane r)      warp 8  TMA producer
//   warps 4-7   softmax stage 1                                               warp 9  UMMA issuer
//   warps 10-11 idle: they complete the third warpgroup, which hands its registers to the softmax warpgroups
//   (setmaxnreg 216 / 216 / 72 of a 168-register launch: a softmax thread keeps 128 scores and 32 packed words live)
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P-hat overlays columns [0,32) of its S, the
// P.V scale factors columns [32,40).
// Output rows leave through the finished item's own Q tile buffer (dead once the stage's last product has completed): 64
// columns at a time -> shared memory (128 B swizzle) -> TMA store; only then may the producer refill that Q buffer.
// FL_MODE_FP4: all 512 columns are taken, so the 16 scale columns of an S product (Q and K atoms, tcgen05.cp from shared
// memory) are parked in columns [64,80) of the OTHER stage's S region once that stage's softmax warps have read their
// latest scores into registers (B_SDRAIN), and in O1 for the two products of the very first key tile of the CTA (nothing
// lives there yet). The tensor pipe runs in issue order, so the next product that overwrites the parked columns starts
// after the reader. All waits are bounded (sm100.cuh); a kernel that gives up writes a code to the status word and drains.
#include "flamia_internal.h"

namespace fl {

static constexpr int KV_STAGES = 3;
static constexpr int Q_STRIDE = 16384;            // bytes between Q tile buffers (also the output staging: 128 rows x 128 B)
static constexpr float P_LOG2_OFFSET = 4.0f;      // row frame: P-hat = 2^(x - m + 4) keeps small probabilities out of E4M3 subnormals
static constexpr float P_LOG2_448 = 8.807354922057604f;   // group frame: the row maximum sits at 448 before the group bias
static constexpr long long STAGE_SKEW_CLOCKS = 2000;   // about half a softmax period; see the UMMA issuer's prologue
static constexpr float RESCALE_THRESHOLD = 4.0f;  // the running maximum is refreshed only when it grew by more than this

struct FwdParams {
  const float* fac_q;
  const float* fac_k;
  const float* fac_v;
  const float* tok_lg_v;   // token-local: log2 f_V(key) and 1 / f_V(key), (b, h_kv, s_k)
  const float* tok_rcp_v;
  const uint8_t* sfq4;   // FL_MODE_FP4: E4M3 scale atoms of the NVFP4 Q / K copies, 1 KB per 128-row tile at d = 128
  const uint8_t* sfk4;
  float* lse;
  const int32_t* doc_start;
  const int32_t* doc_len;
  const int32_t* seqused_k;   // batched form: valid keys per batch row, or null
  const float* o_mult;        // (b, h_kv) factor on the output rows (V's mantissa with float descales), or null
  const int32_t* slot_src;    // packed output: packed row of each 128-row slot of the aligned buffer (-1: empty), or null
  const int32_t* slot_rows;   // packed output: real rows of each slot
  void* out;                  // packed output: the (out_rows, h, d) tensor (row stores of a document's last rows)
  int n_docs;
  int b, s_q, s_k, h, h_kv;
  float scale_log2;
  float cap_a, cap_b;    // soft cap c: x = cap_a tanh(s * factor * cap_b) in log2 units, cap_a = c log2 e, cap_b = 1 / cap_a
  int causal;
  int win_l, win_r;      // sliding window sides, -1 = unlimited (causal: the right side is 0)
  int out_f16;
  int n_items;           // work items: 256-row blocks x heads x batch rows (documents: block slots x heads)
  int n_blk;             // blocks per batch row (documents: block slots of the packed buffer)
  int zigzag;            // deal the items out in zigzag rounds (causal: they are ordered longest first)
  DevCtl ctl;
};

struct Tile {
  int bat;    // batch coordinate of the tensor maps (0 for packed documents)
  int head;   // query head
  int q0;     // first query row (row index inside the batch entry)
  int nq;     // valid query rows of this item (<= 256; 0 = an empty block slot)
  int k0;     // first key row this item loads (row index inside the batch entry)
  int sk;     // keys of the document
  int off;    // causal alignment: key j (document-relative) is visible to query i iff j <= i + off
  int qrel;   // document-relative index of row q0
  int kofs;   // document-relative key of the first key row this item loads (a multiple of 128; > 0 under a left window)
  int n[2];   // key tiles stage 0 / 1 walks: keys [kofs, kmax_i), n_i = ceil((kmax_i - kofs) / 128)
};

// barrier indices
enum { B_Q = 0, B_QE = 2, B_KFULL = 4, B_KEMPTY = B_KFULL + KV_STAGES, B_VFULL = B_KEMPTY + KV_STAGES,
       B_VEMPTY = B_VFULL + KV_STAGES, B_SFULL = B_VEMPTY + KV_STAGES, B_PFULL = B_SFULL + 2, B_PVDONE = B_PFULL + 2,
       B_SDRAIN = B_PVDONE + 2, B_EPI = B_SDRAIN + 2, B_COUNT = B_EPI + 2 };

template <int N>
__device__ __forceinline__ void fwd_reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void fwd_reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
__device__ __forceinline__ void fwd_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// k-th work item of CTA c on a grid of G CTAs (>= n_items: the CTA is done)
__device__ __forceinline__ int fwd_item(int k, int G, int c, int zigzag) {
  return k * G + ((zigzag && (k & 1)) ? (G - 1 - c) : c);
}

// Work item L -> its block. Causal: blocks slowest and last block first, so that the item index orders the items longest
// first; heads fastest, so the query heads of a kv group run together and share its K / V tiles in L2. Otherwise blocks
// fastest: neighbours share their K / V tiles in L2 and every block costs the same.
__device__ __forceinline__ void fwd_decode(const FwdParams& p, int L, Tile& t) {
  if (p.doc_start == nullptr) {
    int blk, rem;
    if (p.causal) { blk = p.n_blk - 1 - L / (p.h * p.b); rem = L % (p.h * p.b); }
    else { blk = L % p.n_blk; rem = L / p.n_blk; }
    t.head = rem % p.h; t.bat = rem / p.h;
    t.q0 = blk * 256; t.nq = min(256, p.s_q - t.q0); t.k0 = 0; t.sk = p.s_k;
    if (p.seqused_k) t.sk = max(0, min(p.s_k, p.seqused_k[t.bat]));      // keys past it are masked like a document's end
    t.off = p.s_k - p.s_q; t.qrel = t.q0;
  } else {
    // documents sit at 128-aligned starts of one packed batch entry; block slot x -> (document, 256-row block)
    int x = L / p.h, dsel = -1, blk = 0, len = 0, st = 0;
    t.head = L % p.h;
    for (int dI = 0; dI < p.n_docs; ++dI) {
      doc_entry(p.doc_start, p.doc_len, dI, p.s_q, p.ctl.status, st, len);
      const int nb = (len + 255) / 256;
      if (x < nb) { dsel = dI; blk = x; break; }
      x -= nb;
    }
    if (dsel < 0) { t.nq = 0; t.bat = 0; t.q0 = 0; t.k0 = 0; t.sk = 0; t.off = 0; t.qrel = 0; }
    else {
      if (p.causal) blk = (len + 255) / 256 - 1 - blk;
      t.bat = 0; t.q0 = st + blk * 256; t.nq = min(256, len - blk * 256); t.k0 = st; t.sk = len; t.off = 0;
      t.qrel = blk * 256;
    }
  }
  // left window: the first key any row of this block can see; both stages start at that key tile
  t.kofs = 0;
  if (p.win_l >= 0 && t.nq > 0) t.kofs = (max(0, t.qrel + t.off - p.win_l) / 128) * 128;
  t.k0 += t.kofs;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rows = min(128, t.nq - 128 * i);             // valid rows of the stage (<= 0: stage absent)
    int kmax = t.sk;
    if (p.win_r >= 0) kmax = min(t.sk, t.qrel + 128 * i + rows + t.off + p.win_r);
    t.n[i] = (rows > 0 && kmax > t.kofs) ? (kmax - t.kofs + 127) / 128 : 0;
  }
}

// FULL: the variants that also serve packed outputs and the output-row factor, each behind a run-time check of its
// pointer. A template flag, so that the kernels of the plain calls carry none of that code (-2 % kernel time).
template <int D, bool FP4, bool TL, bool GF, bool SC, bool FULL = false>
__global__ void __launch_bounds__(384, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const FwdParams p) {
  constexpr int TILE_BYTES = 128 * D;
  constexpr uint64_t SWZ = (D == 128) ? SWZ_128 : SWZ_64;
  constexpr uint32_t SBO = 8 * D;                       // bytes between 8-row groups
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                   // [item buffer 2][stage 2] x Q_STRIDE
  uint8_t* sK = sQ + 4 * Q_STRIDE;                      // KV_STAGES tiles
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;            // KV_STAGES tiles
  uint8_t* sSF = sV + KV_STAGES * TILE_BYTES;           // FP4: scale atoms, Q [item buffer 2] x 2 KB then K KV_STAGES x 1 KB
  constexpr int SF_K = 4096;                            // offset of the K atoms inside sSF
  constexpr int OP_BYTES = FP4 ? TILE_BYTES / 2 : TILE_BYTES;   // bytes of one Q / K operand tile (4-bit codes: half)
  __shared__ __align__(8) uint64_t bars[B_COUNT];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ Tile tile_s[2];                            // the items in flight (written by the producer, item k in slot k & 1)
  // group frame: [stage][tile parity] one scale atom (32 rows x 16 B: row r at word (r % 32) * 4 + r / 32) = P-hat's four
  // exponent bytes per row; the issuer copies it into the A scale columns right before the stage's P.V product
  __shared__ __align__(16) uint32_t s_sfp[2][2][128];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int grp = p.h / p.h_kv;

  if (tid == 8 * 32) {
    abort_s = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[B_Q + i], 1);
      mbar_init(&bars[B_QE + i], 2);         // released by one thread of each softmax warpgroup
      mbar_init(&bars[B_SFULL + i], 1);
      mbar_init(&bars[B_PFULL + i], 4);      // one arrival per softmax warp
      mbar_init(&bars[B_PVDONE + i], 1);
      mbar_init(&bars[B_SDRAIN + i], 4);
      mbar_init(&bars[B_EPI + i], 4);
    }
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(&bars[B_KFULL + i], 1);
      mbar_init(&bars[B_KEMPTY + i], 1);
      mbar_init(&bars[B_VFULL + i], 1);
      mbar_init(&bars[B_VEMPTY + i], 1);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_o);
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

  if (warp >= 8) fwd_reg_dealloc<72>();
  if (warp == 8) {
    // =================================================================== TMA producer
    if (lane == 0) {
      int gj = 0;                          // key tiles issued so far, over all items (the K / V ring never restarts)
      bool ok = true;
      for (int k = 0; ok; ++k) {
        const int L = fwd_item(k, G, cta, p.zigzag);
        if (L >= p.n_items) break;
        const int kb = k & 1;
        // the Q buffer of item k - 2 (and its slot of tile_s) is free once both softmax warpgroups have written its
        // output rows out of it
        if (k >= 2 && !(ok = mbar_wait(&bars[B_QE + kb], ((k >> 1) - 1) & 1, p.ctl, abortp, 12))) break;
        Tile t;
        fwd_decode(p, L, t);
        tile_s[kb] = t;
        const int hkv = t.head / grp;
        if (t.nq > 0) {
          const bool two = t.nq > 128;
          mbar_arrive_expect_tx(&bars[B_Q + kb], 2 * OP_BYTES + (FP4 ? (two ? 2048 : 1024) : 0));
          tma_load_4d(sQ + (2 * kb) * Q_STRIDE, &tm_q, &bars[B_Q + kb], 0, t.head, t.q0, t.bat);
          tma_load_4d(sQ + (2 * kb + 1) * Q_STRIDE, &tm_q, &bars[B_Q + kb], 0, t.head, t.q0 + 128, t.bat);
          if (FP4)
            bulk_load(sSF + kb * 2048, p.sfq4 + (((size_t)t.bat * p.h + t.head) * (p.s_q / 128) + t.q0 / 128) * 1024,
                      two ? 2048 : 1024, &bars[B_Q + kb]);
        } else {
          mbar_arrive(&bars[B_Q + kb]);    // an empty block slot: the phase still completes, every role moves on
        }
        const int n_max = max(t.n[0], t.n[1]);
        for (int j = 0; j < n_max; ++j, ++gj) {
          const int st = gj % KV_STAGES, ph = (gj / KV_STAGES) & 1;
          if (gj >= KV_STAGES && !(ok = mbar_wait(&bars[B_KEMPTY + st], ph ^ 1, p.ctl, abortp, 10))) break;
          mbar_arrive_expect_tx(&bars[B_KFULL + st], OP_BYTES + (FP4 ? 1024 : 0));
          tma_load_4d(sK + st * TILE_BYTES, &tm_k, &bars[B_KFULL + st], 0, hkv, t.k0 + j * 128, t.bat);
          if (FP4)
            bulk_load(sSF + SF_K + st * 1024,
                      p.sfk4 + (((size_t)t.bat * p.h_kv + hkv) * (p.s_k / 128) + t.k0 / 128 + j) * 1024, 1024,
                      &bars[B_KFULL + st]);
          if (gj >= KV_STAGES && !(ok = mbar_wait(&bars[B_VEMPTY + st], ph ^ 1, p.ctl, abortp, 11))) break;
          mbar_arrive_expect_tx(&bars[B_VFULL + st], TILE_BYTES);
          tma_load_4d(sV + st * TILE_BYTES, &tm_v, &bars[B_VFULL + st], 0, hkv, t.k0 + j * 128, t.bat);
        }
      }
    }
  } else if (warp == 9) {
    // =================================================================== UMMA issuer
    // The whole warp stays converged through the waits and the descriptor arithmetic (warp-uniform values); one elected
    // lane issues. Descriptors are built once; the loops only add byte offsets.
    constexpr uint32_t ID_S = idesc_f8(128, 128, 0, 0);
    const uint32_t tm = __shfl_sync(0xFFFFFFFFu, tmem, 0);
    const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
    // FP4: rows of D / 2 bytes (64 B swizzle at d = 128), K = 64 elements = 32 bytes per instruction
    const uint64_t dq0 = FP4 ? smem_desc(q_addr, 16, 512, SWZ_64) : smem_desc(q_addr, 16, SBO, SWZ),
                   dk0 = FP4 ? smem_desc(k_addr, 16, 512, SWZ_64) : smem_desc(k_addr, 16, SBO, SWZ),
                   dv0 = smem_desc(v_addr, 16, SBO, SWZ);
    const uint64_t dsf0 = smem_desc(smem_u32(sSF), 0, 128, SWZ_NONE);   // scale atoms: 32 rows x 16 B, unswizzled
    int gj = 0;                            // key tiles consumed so far, over all items
    int cs0 = 0, cs1 = 0;                  // S products issued so far, per stage
    bool first_s = true;                   // FP4: the very first key tile of the CTA parks its scale columns in O1
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int L = fwd_item(k, G, cta, p.zigzag);
      if (L >= p.n_items) break;
      const int kb = k & 1;
      if (!(ok = mbar_wait(&bars[B_Q + kb], (k >> 1) & 1, p.ctl, abortp, 20))) break;
      const int n0 = tile_s[kb].n[0], n1 = tile_s[kb].n[1];
      const int nmax = max(n0, n1);
      // issue_s(i, st): S of stage i against the K tile in ring slot st
      auto issue_s = [&](int i, int st, bool park_o1) {
        const uint64_t a = desc_adv(dq0, (2 * kb + i) * Q_STRIDE), b = desc_adv(dk0, st * TILE_BYTES);
        if (FP4) {
          constexpr uint32_t ID_S4 = idesc_bs(128, 128, 1, 1, 0, 0, 0, 0, 0);
          const uint32_t park = park_o1 ? (tm + 384 + 16 * i) : (tm + 128 * (1 - i) + 64);
#pragma unroll
          for (int kk = 0; kk < D / 64; ++kk) {
            tmem_cp_sf_atom(park + 4 * kk, desc_adv(dsf0, kb * 2048 + i * 1024 + 512 * kk));
            tmem_cp_sf_atom(park + 8 + 4 * kk, desc_adv(dsf0, SF_K + st * 1024 + 512 * kk));
          }
#pragma unroll
          for (int kk = 0; kk < D / 64; ++kk)
            umma_nvf4_ss(tm + 128 * i, desc_adv(a, 32 * kk), desc_adv(b, 32 * kk), ID_S4, park + 4 * kk, park + 8 + 4 * kk, kk > 0);
        } else {
#pragma unroll
          for (int kk = 0; kk < D / 32; ++kk) umma_f8_ss(tm + 128 * i, desc_adv(a, 32 * kk), desc_adv(b, 32 * kk), ID_S, kk > 0);
        }
      };
      // FP4: the other stage's latest scores must have been read before their region takes the scale columns
      auto drained = [&](int i) -> bool {
        if (!FP4) return true;
        const int cy = i == 0 ? cs1 : cs0;
        if (cy == 0) return true;
        return mbar_wait(&bars[B_SDRAIN + (1 - i)], (cy - 1) & 1, p.ctl, abortp, 26 + i);
      };
      auto issue_pv = [&](int i, int st, uint32_t accum, int par) {
        const uint64_t b = desc_adv(dv0, st * TILE_BYTES);
        const uint32_t ts = tm + 128 * i;
        if (GF) tmem_cp_sf_atom(ts + 32, smem_desc(smem_u32(&s_sfp[i][par][0]), 0, 128, SWZ_NONE));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)   // 32 keys per instruction: 32 rows of the V tile (MN-major operand)
          umma_mxf8_ts(tm + 256 + 128 * i, ts + 8 * kk, desc_adv(b, kk * 32 * D), idesc_bs(128, D, 0, 0, 0, 1, 1, kk, kk),
                       ts + 32, ts + 36, accum | kk);
      };
      if (nmax > 0) {
        const int st0 = gj % KV_STAGES, ph0 = (gj / KV_STAGES) & 1;
        if (!(ok = mbar_wait(&bars[B_KFULL + st0], ph0, p.ctl, abortp, 21))) break;
        tc_fence_after();
        const bool o1 = first_s;
        if (n0 > 0) {
          if (!o1 && !(ok = drained(0))) break;
          if (FP4) tc_fence_after();
          if (elect_one()) { issue_s(0, st0, o1); tc_commit(&bars[B_SFULL + 0]); }
          __syncwarp();
          ++cs0;
        }
        // Start the second stage about half a softmax period after the first: the two softmax warpgroups share each
        // scheduler's transcendental unit, which saturates when their exponential phases coincide and idles while
        // both wait for the tensor core. Nothing pulls the phases apart later, so the offset is set once per CTA.
        if (k == 0 && n0 > 0 && n1 > 0) {
          const long long t_skew = clock64();
          while (clock64() - t_skew < STAGE_SKEW_CLOCKS) {}
        }
        if (n1 > 0) {
          if (!o1 && !(ok = drained(1))) break;
          if (FP4) tc_fence_after();
          if (elect_one()) { issue_s(1, st0, o1); tc_commit(&bars[B_SFULL + 1]); }
          __syncwarp();
          ++cs1;
        }
        if (elect_one()) tc_commit(&bars[B_KEMPTY + st0]);   // K tile 0 is free once both S(0) products have completed
        __syncwarp();
        first_s = false;
      }
      for (int j = 0; ok && j < nmax; ++j) {
        const int g = gj + j;
        const int st = g % KV_STAGES, ph = (g / KV_STAGES) & 1;
        const int stn = (g + 1) % KV_STAGES, phn = ((g + 1) / KV_STAGES) & 1;
        if (!(ok = mbar_wait(&bars[B_VFULL + st], ph, p.ctl, abortp, 22))) break;
        bool k_next_ready = false;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int n_i = i == 0 ? n0 : n1;
          if (j >= n_i) continue;
          // P-hat(j) of stage i belongs to the stage's latest S product (number cs_i - 1)
          const int ci = i == 0 ? cs0 : cs1;
          if (!(ok = mbar_wait(&bars[B_PFULL + i], (ci - 1) & 1, p.ctl, abortp, 23 + i))) break;
          tc_fence_after();
          // P.V(j) completes before S(j + 1) does (issue order), which the softmax threads wait for anyway: a
          // separate completion signal is needed only after the stage's last tile (each commit costs the issuer ~60 clocks)
          if (elect_one()) { issue_pv(i, st, j > 0, (ci - 1) & 1); if (j + 1 == n_i) tc_commit(&bars[B_PVDONE + i]); }
          __syncwarp();
          if (j + 1 < n_i) {
            if (!k_next_ready) {
              if (!(ok = mbar_wait(&bars[B_KFULL + stn], phn, p.ctl, abortp, 25))) break;
              k_next_ready = true;
              tc_fence_after();
            }
            if (!(ok = drained(i))) break;
            if (FP4) tc_fence_after();
            if (elect_one()) { issue_s(i, stn, false); tc_commit(&bars[B_SFULL + i]); }
            __syncwarp();
            if (i == 0) ++cs0; else ++cs1;
          }
        }
        if (!ok) break;
        // every MMA that reads K tile j+1 / V tile j has been issued: release the stages when they complete
        if (elect_one()) {
          if (j + 1 < nmax) tc_commit(&bars[B_KEMPTY + stn]);
          tc_commit(&bars[B_VEMPTY + st]);
        }
        __syncwarp();
      }
      gj += nmax;
    }
  } else if (warp < 8) {
    // =================================================================== softmax + correction + epilogue
    fwd_reg_alloc<216>();
    const int i = warp >> 2;                          // stage
    const int r = tid & 127;                          // row of the stage = TMEM lane
    const uint32_t t_s = tmem + 128 * i + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t t_o = tmem + 256 + 128 * i + ((uint32_t)((warp & 3) * 32) << 16);
    int cs = 0;                                       // tiles of this stage so far, over all items
    int cd = 0;                                       // items of this stage that ended with a P.V so far
    int epi = 0, gfn = 0;                             // uses of the epilogue barrier / group-frame scale atoms so far
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int L = fwd_item(k, G, cta, p.zigzag);
      if (L >= p.n_items) break;
      const int kb = k & 1;
      if (!(ok = mbar_wait(&bars[B_Q + kb], (k >> 1) & 1, p.ctl, abortp, 36))) break;
      const Tile T = tile_s[kb];
      const int head = T.head, hkv = head / grp;
      const int n_i = T.n[i];
      const int qrow = T.q0 + 128 * i + r;              // row inside the batch entry
      const int qrel = T.qrel + 128 * i + r;            // row inside the document
      const bool row_valid = (128 * i + r) < T.nq;
      const size_t bh_q = (size_t)T.bat * p.h + head, bh_k = (size_t)T.bat * p.h_kv + hkv;
      const float fq = !row_valid ? 0.f
                       : FP4     ? p.scale_log2
                       : TL      ? p.fac_q[bh_q * p.s_q + qrow] * p.scale_log2
                                 : p.fac_q[bh_q * (p.s_q / 32) + qrow / 32] * p.scale_log2;
      const float* fk_row = p.fac_k + bh_k * (p.s_k / 32) + T.k0 / 32;
      const float* fv_row = p.fac_v + bh_k * (p.s_k / 32) + T.k0 / 32;
      const int col_limit = p.win_r >= 0 ? min(qrel + T.off + p.win_r, T.sk - 1) : T.sk - 1;   // last visible key of this row
      const int col_first = p.win_l >= 0 ? qrel + T.off - p.win_l : 0;                          // first visible key
      constexpr float P_OFF = GF ? P_LOG2_448 : P_LOG2_OFFSET;

      float m_used = -INFINITY, l_sum = 0.f;
      for (int j = 0; j < n_i; ++j, ++cs) {
        float c[4];
        uint32_t sfv = 0;
#pragma unroll
        for (int kbk = 0; kbk < 4; ++kbk) {
          if (TL) continue;
          c[kbk] = FP4 ? fq : fq * fk_row[j * 4 + kbk];      // FP4: the block scales were applied by the tensor core
          sfv |= ((__float_as_uint(fv_row[j * 4 + kbk]) >> 23) & 0xFF) << (8 * kbk);
        }
        // token-local: the tile's 128 per-key factors (same addresses for every thread: broadcast loads through L1;
        // staging them in shared memory was twice as slow: 384 broadcast reads per thread and tile saturate the
        // shared-memory port that the tensor core's operand reads also go through)
        const float4* fk4 = reinterpret_cast<const float4*>(p.fac_k + (TL ? bh_k * p.s_k + T.k0 + j * 128 : 0));
        const float4* lg4 = reinterpret_cast<const float4*>(TL ? p.tok_lg_v + bh_k * p.s_k + T.k0 + j * 128 : p.fac_v);
        const float4* rc4 = reinterpret_cast<const float4*>(TL ? p.tok_rcp_v + bh_k * p.s_k + T.k0 + j * 128 : p.fac_v);
        if (TL) {
          sfv = 0x7F7F7F7Fu;
#pragma unroll
          for (int kbk = 0; kbk < 4; ++kbk) c[kbk] = 1.f;
        }
        if (!(ok = mbar_wait(&bars[B_SFULL + i], cs & 1, p.ctl, abortp, 30 + i))) break;
        tc_fence_after();
        uint32_t su[128];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) FL_TMEM_LD_32(t_s + 32 * cc, (su + 32 * cc));
        tc_wait_ld();
        if (FP4) {      // the scores are in registers: this S region may take the other stage's scale columns
          tc_fence_before();
          mbar_arrive_warp(&bars[B_SDRAIN + i]);
        }
        float s[128];
#pragma unroll
        for (int e = 0; e < 128; ++e) s[e] = __uint_as_float(su[e]);
        if (TL) {   // y = s f_Q f_K(key) scale + log2 f_V(key)
#pragma unroll
          for (int e4 = 0; e4 < 32; ++e4) {
            // two columns per instruction; log2 f_V comes from a table (derived here it cost three integer instructions
            // per score on loops that are issue-bound)
            const float4 k4 = __ldg(fk4 + e4), l4 = __ldg(lg4 + e4);
            const uint64_t fq2 = pack2(fq, fq);
            unpack2(fma2(pack2(s[4 * e4 + 0], s[4 * e4 + 1]), mul2(pack2(k4.x, k4.y), fq2), pack2(l4.x, l4.y)),
                    s[4 * e4 + 0], s[4 * e4 + 1]);
            unpack2(fma2(pack2(s[4 * e4 + 2], s[4 * e4 + 3]), mul2(pack2(k4.z, k4.w), fq2), pack2(l4.z, l4.w)),
                    s[4 * e4 + 2], s[4 * e4 + 3]);
          }
        }
        if (SC) {   // soft cap: the capped score in log2 units; the factors are used up here
#pragma unroll
          for (int e = 0; e < 128; ++e) s[e] = p.cap_a * tanh_fast(s[e] * (c[e >> 5] * p.cap_b));
#pragma unroll
          for (int kbk = 0; kbk < 4; ++kbk) c[kbk] = 1.f;
        }
        const int kb0 = T.kofs + j * 128;                       // document-relative key of column 0
        const bool need_mask = (kb0 + 127 > col_limit) || (kb0 < col_first);    // only on boundary tiles
        if (need_mask) {   // scale first, then mask: the factor product may underflow to zero and 0 * inf is NaN
#pragma unroll
          for (int e = 0; e < 128; ++e)
            s[e] = (kb0 + e > col_limit || kb0 + e < col_first) ? -INFINITY : s[e] * c[e >> 5];
#pragma unroll
          for (int kbk = 0; kbk < 4; ++kbk) c[kbk] = 1.f;
        }
        float mx = -INFINITY;
        float gm[4];                                             // the four 32-key groups' maxima (scaled)
#pragma unroll
        for (int kbk = 0; kbk < 4; ++kbk) {
          // eight independent chains of three-input maxima, then a tree: a serial chain would cost its latency 31 times
          float a[8];
#pragma unroll
          for (int t = 0; t < 8; ++t)
            a[t] = fmaxf(fmax3(s[32 * kbk + 4 * t], s[32 * kbk + 4 * t + 1], s[32 * kbk + 4 * t + 2]), s[32 * kbk + 4 * t + 3]);
          const float m8 = fmax3(fmax3(a[0], a[1], a[2]), fmax3(a[3], a[4], a[5]), fmaxf(a[6], a[7]));
          gm[kbk] = m8 * c[kbk];
          mx = fmaxf(mx, gm[kbk]);
        }
        // lazy refresh of the running maximum
        float alpha = 1.f;
        const bool refresh = mx > m_used + RESCALE_THRESHOLD;
        if (refresh) {
          alpha = ex2(m_used - mx);     // 0 on the first tile (m_used = -inf)
          m_used = mx;
        }
        if (j > 0 && __any_sync(0xFFFFFFFFu, refresh)) {
          // rescale this row of O in tensor memory once the previous P.V has finished
          // P.V(j - 1) has completed: S(j), which this thread has read, was issued after it
#pragma unroll 1
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t ov[32];
            FL_TMEM_LD_32(t_o + 32 * cc, ov);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
            FL_TMEM_ST_32(t_o + 32 * cc, ov);
          }
        }
        const float mb = (m_used == -INFINITY) ? 0.f : (m_used - P_OFF);
        // group frame: per 32 keys the exponent argument is lowered by the group's own integer bias
        float gb[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t sfp = 0x7F7F7F7Fu;
        if (GF) {
          sfp = 0;
#pragma unroll
          for (int kbk = 0; kbk < 4; ++kbk) {
            gb[kbk] = ceilf(fmaxf(gm[kbk] - mb, -100.0f) - P_LOG2_448);
            sfp |= ((uint32_t)(127 + (int)gb[kbk]) & 0xFF) << (8 * kbk);
          }
        }
        float ps[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};     // independent partial sums (group frame: two per group)
        [[maybe_unused]] uint64_t ps2[4] = {0ull, 0ull, 0ull, 0ull};  // the same as packed pairs (default route)
        uint32_t pw[32];
#pragma unroll
        for (int w = 0; w < 32; ++w) {
          const float cw = c[w >> 3];
          const float mbw = GF ? mb + gb[w >> 3] : mb;
          // exponent arguments: two columns per instruction
          float a0, a1, a2, a3;
          {
            const uint64_t cw2 = pack2(cw, cw), nm2 = pack2(-mbw, -mbw);
            unpack2(fma2(pack2(s[4 * w], s[4 * w + 1]), cw2, nm2), a0, a1);
            unpack2(fma2(pack2(s[4 * w + 2], s[4 * w + 3]), cw2, nm2), a2, a3);
          }
          float p0 = ex2(a0), p1 = ex2(a1);
          float p2, p3;
          if (w & 1) {    // one pair in four on the FMA pipe (none: +4 % kernel time causal, +8 % dense; three in eight: the same)
            ex2_poly2(a2, a3, p2, p3);
          } else {
            p2 = ex2(a2);
            p3 = ex2(a3);
          }
          if (TL) {     // the row sum is that of the probabilities: take f_V(key) back out
            const float4 r4 = __ldg(rc4 + w);
            ps2[w & 3] = fma2(pack2(p0, p1), pack2(r4.x, r4.y), ps2[w & 3]);
            ps2[w & 3] = fma2(pack2(p2, p3), pack2(r4.z, r4.w), ps2[w & 3]);
          } else if (GF) {  // packed: (p0 + p2, p1 + p3) into the group's pair accumulator
            ps2[w >> 3] = add2(ps2[w >> 3], add2(pack2(p0, p1), pack2(p2, p3)));
          } else {          // the same into one of four pair accumulators
            ps2[w & 3] = add2(ps2[w & 3], add2(pack2(p0, p1), pack2(p2, p3)));
          }
          pw[w] = cvt_e4m3x4(p0, p1, p2, p3);
        }
        float psum;
        if (GF) {   // each group's sum weighs 2^bias_g
          float pg[4];
#pragma unroll
          for (int kbk = 0; kbk < 4; ++kbk) unpack2(ps2[kbk], ps[2 * kbk], ps[2 * kbk + 1]);
#pragma unroll
          for (int kbk = 0; kbk < 4; ++kbk)
            pg[kbk] = (ps[2 * kbk] + ps[2 * kbk + 1]) * __uint_as_float((uint32_t)(127 + (int)gb[kbk]) << 23);
          psum = (pg[0] + pg[1]) + (pg[2] + pg[3]);
        } else {
#pragma unroll
          for (int t = 0; t < 4; ++t) unpack2(ps2[t], ps[2 * t], ps[2 * t + 1]);
          psum = ((ps[0] + ps[1]) + (ps[2] + ps[3])) + ((ps[4] + ps[5]) + (ps[6] + ps[7]));
        }
        l_sum = fmaf(l_sum, alpha, psum);
        FL_TMEM_ST_32(t_s, pw);
        if (GF) {
          // the A scale tile (every lane quadrant holds all 128 rows' exponent words: lane = row % 32, column = row / 32)
          // is copied from this atom by the issuer; only the B scale columns are stored from here
          s_sfp[i][gfn & 1][(r & 31) * 4 + (r >> 5)] = sfp;
          ++gfn;
          fence_proxy_async();             // the atom is read by tcgen05.cp (async proxy)
          uint32_t sf[8] = {0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, sfv, sfv, sfv, sfv};
          FL_TMEM_ST_8(t_s + 32, sf);
        } else {
          uint32_t sf[8] = {0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, sfv, sfv, sfv, sfv};
          FL_TMEM_ST_8(t_s + 32, sf);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive_warp(&bars[B_PFULL + i]);
      }
      if (!ok) break;
      // ---- item epilogue: O / l -> bf16 rows through this stage's Q tile buffer, LSE
      if (n_i > 0) {
        if (!(ok = mbar_wait(&bars[B_PVDONE + i], cd & 1, p.ctl, abortp, 34 + i))) break;
        ++cd;
      }
      tc_fence_after();
      const bool stage_present = T.nq > 128 * i;        // (warpgroup-uniform) an absent stage's rows belong to someone else
      const float inv_l = ((l_sum > 0.f) ? 1.0f / l_sum : 0.f) * ((FULL && p.o_mult) ? p.o_mult[bh_k] : 1.0f);
      uint8_t* stage = sQ + (2 * kb + i) * Q_STRIDE;
      const uint32_t srow = smem_u32(stage) + r * 128;
      // packed output: this stage's 128 rows are slot (T.q0 + 128 i) / 128 of the aligned buffer; they go to the packed
      // rows out_row .. + out_n of the caller's tensor: a full slot as TMA stores, a document's last rows row by row
      int out_row = T.q0 + 128 * i, out_n = stage_present ? 128 : 0;
      if (FULL && p.slot_src) {
        const int slot = (T.q0 + 128 * i) / 128;
        out_row = stage_present ? p.slot_src[slot] : -1;
        out_n = (stage_present && out_row >= 0) ? min(p.slot_rows[slot], 128) : 0;
      }
      const bool by_rows = FULL && p.slot_src && out_n < 128;    // (warpgroup-uniform)
#pragma unroll 1
      for (int pass = 0; pass < D / 64; ++pass) {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t ov[32];
          if (n_i > 0) {                 // (warpgroup-uniform: the tensor-memory loads are warp-collective)
            FL_TMEM_LD_32(t_o + 64 * pass + 32 * cc, ov);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] = 0;
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // rows past the end of the document store zeros (a select: what tensor memory holds there is arbitrary)
              float a, b2;
              unpack2(mul2(pack2(__uint_as_float(ov[8 * q4 + 2 * e]), __uint_as_float(ov[8 * q4 + 2 * e + 1])),
                           pack2(inv_l, inv_l)), a, b2);
              a = row_valid ? a : 0.f;
              b2 = row_valid ? b2 : 0.f;
              if (p.out_f16) {
                __half2 hh = __floats2half2_rn(a, b2);
                w[e] = *reinterpret_cast<uint32_t*>(&hh);
              } else {
                w[e] = pack_bf16x2(a, b2);
              }
            }
            if (by_rows) {
              if (r < out_n)
                *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) +
                                          ((size_t)(out_row + r) * p.h + head) * D + 64 * pass + 8 * (cc * 4 + q4)) =
                    make_uint4(w[0], w[1], w[2], w[3]);
            } else {
              fwd_sts128(srow + (((cc * 4 + q4) ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
            }
          }
        }
        if (by_rows) continue;
        fence_proxy_async();
        mbar_arrive_warp(&bars[B_EPI + i]);             // the warpgroup's four warps have written their rows
        if (!(ok = mbar_wait(&bars[B_EPI + i], epi & 1, p.ctl, abortp, 38))) break;
        ++epi;
        if (r == 0 && out_n == 128) {
          tma_store_4d(&tm_o, stage, 64 * pass, head, out_row, T.bat);
          tma_store_commit();
          tma_store_wait_read<0>();      // the shared-memory source must outlive the copy; the writes complete with the grid
        }
        mbar_arrive_warp(&bars[B_EPI + i]);             // the buffer has been read: the next pass / the producer may take it
        if (!(ok = mbar_wait(&bars[B_EPI + i], epi & 1, p.ctl, abortp, 38))) break;
        ++epi;
      }
      if (!ok) break;
      if (row_valid && p.lse) {
        // l carries 2^P_OFF: lse = ln2 * (m - P_OFF + log2 l)
        float v = (l_sum > 0.f) ? (m_used - P_OFF + lg2(l_sum)) * 0.6931471805599453f : -INFINITY;
        p.lse[bh_q * p.s_q + qrow] = v;
      }
      tc_fence_before();                 // this stage's output has left tensor memory before the next item's P-hat is announced
      if (r == 0) mbar_arrive(&bars[B_QE + kb]);
    }
  }
  // ---- common exit: nothing of this CTA may still be in flight when tensor memory is released
  if (abort_s) {
    for (int it = 0; it < 200; ++it) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace fl

extern "C" int fl_fwd(const fl_attn_args* a, void* stream) {
  using namespace fl;
  if (!a || !a->q_codes || !a->k_codes || !a->v_codes || !a->out || !a->status) return FL_ERR_BAD_ARG;
  if (!a->fac_q || !a->fac_k || !a->fac_v) return FL_ERR_BAD_ARG;
  if (a->d != 64 && a->d != 128) return FL_ERR_UNSUPPORTED;
  if (a->mode != FL_MODE_FP8 && a->mode != FL_MODE_FP4) return FL_ERR_UNSUPPORTED;
  const bool fp4 = a->mode == FL_MODE_FP4;
  if (fp4 && a->d != 128) return FL_ERR_UNSUPPORTED;
  if (fp4 && (!a->q4 || !a->k4 || !a->sfq4 || !a->sfk4)) return FL_ERR_BAD_ARG;
  const bool tl = (a->flags & FL_A_TOKEN_LOCAL) != 0, gf = (a->flags & FL_A_P_GROUP) != 0;
  if (tl && (a->doc_start || a->mode != FL_MODE_FP8)) return FL_ERR_UNSUPPORTED;   // token-local: batched 8-bit route
  if (tl && (!a->tok_lg_v || !a->tok_rcp_v)) return FL_ERR_BAD_ARG;                 // tables of fl_token_aux over V's factors
  if (gf && (tl || a->d != 128)) return FL_ERR_UNSUPPORTED;                        // group frame: d = 128, block factors
  if (a->h <= 0 || a->h_kv <= 0 || a->h % a->h_kv) return FL_ERR_BAD_ARG;
  if ((a->s_q % 128) || (a->s_k % 128) || a->s_q <= 0 || a->s_k <= 0 || a->b <= 0) return FL_ERR_BAD_ARG;
  if (a->doc_start && (a->b != 1 || a->n_docs <= 0 || !a->doc_len || a->s_q != a->s_k)) return FL_ERR_BAD_ARG;
  if (a->seqused_k && a->doc_start) return FL_ERR_UNSUPPORTED;      // documents carry their own lengths
  CUtensorMap mq, mk, mv, mo;
  int rc;
  if ((rc = make_rows_map(&mq, fp4 ? a->q4 : a->q_codes, a->b, a->s_q, a->h, fp4 ? a->d / 2 : a->d, 128))) return rc;
  if ((rc = make_rows_map(&mk, fp4 ? a->k4 : a->k_codes, a->b, a->s_k, a->h_kv, fp4 ? a->d / 2 : a->d, 128))) return rc;
  if ((rc = make_rows_map(&mv, a->v_codes, a->b, a->s_k, a->h_kv, a->d, 128))) return rc;
  if ((rc = make_rows_map_16(&mo, a->out, a->b, a->slot_src ? a->out_rows : a->s_q, a->h, a->d, 128))) return rc;
  FwdParams p;
  p.fac_q = a->fac_q; p.fac_k = a->fac_k; p.fac_v = a->fac_v; p.lse = a->lse;
  p.sfq4 = a->sfq4; p.sfk4 = a->sfk4;
  p.tok_lg_v = a->tok_lg_v; p.tok_rcp_v = a->tok_rcp_v;
  p.doc_start = a->doc_start; p.doc_len = a->doc_len; p.n_docs = a->n_docs;
  p.seqused_k = a->seqused_k;
  p.o_mult = a->o_mult;
  if (a->o_mult && a->doc_start) return FL_ERR_UNSUPPORTED;      // per-(batch row, head) factors: the batched form
  p.slot_src = a->slot_src; p.slot_rows = a->slot_rows; p.out = a->out;
  if (a->slot_src && (!a->doc_start || !a->slot_rows || a->out_rows <= 0)) return FL_ERR_BAD_ARG;
  p.b = a->b; p.s_q = a->s_q; p.s_k = a->s_k; p.h = a->h; p.h_kv = a->h_kv;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.causal = (a->flags & FL_A_CAUSAL) ? 1 : 0;
  p.win_l = a->window_left_p1 - 1;
  p.win_r = p.causal ? 0 : a->window_right_p1 - 1;
  p.out_f16 = (a->flags & FL_A_OUT_F16) ? 1 : 0;
  p.ctl.status = a->status;
  p.ctl.wait_cycles = a->wait_cycles > 0 ? a->wait_cycles : kDefaultWaitCycles;
  // packed documents: at most one extra 256-row block per document beyond total / 256
  const int nblk = a->doc_start ? (a->s_q / 256 + a->n_docs + 1) : (a->s_q + 255) / 256;
  const int nb = a->doc_start ? 1 : a->b;
  p.n_blk = nblk;
  const long long n_items = (long long)nblk * a->h * nb;
  if (n_items > 0x3FFFFFFF) return FL_ERR_TOO_LARGE;
  p.n_items = (int)n_items;
  p.zigzag = (p.causal && !a->doc_start) ? 1 : 0;
  const int grid = (int)(n_items < sm_count() ? n_items : sm_count());     // one persistent CTA per SM
  const int smem = 4 * Q_STRIDE + 2 * KV_STAGES * 128 * a->d + 1024 + (fp4 ? 4096 + KV_STAGES * 1024 : 0);
  cudaStream_t st = (cudaStream_t)stream;
  auto launch = [&](auto kern) -> int {
    if (cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); e != cudaSuccess)
      return cuda_fail((int)e, "fl_fwd: cudaFuncSetAttribute");
    kern<<<grid, 384, smem, st>>>(mq, mk, mv, mo, p);
    return FL_OK;
  };
  const bool sc = a->softcap > 0.f;
  if (sc && tl) return FL_ERR_UNSUPPORTED;
  p.cap_a = sc ? a->softcap * 1.4426950408889634f : 0.f;
  p.cap_b = sc ? 1.0f / p.cap_a : 0.f;
  // the lean kernels serve the plain calls; packed outputs and the output-row factor take the full variant
  const bool full = a->slot_src != nullptr || a->o_mult != nullptr;
#define FL_FWD_LAUNCH(D_, FP4_, TL_, GF_, SC_) \
  (full ? launch(fwd_kernel<D_, FP4_, TL_, GF_, SC_, true>) : launch(fwd_kernel<D_, FP4_, TL_, GF_, SC_, false>))
  if (sc) {
    if (fp4) rc = gf ? FL_FWD_LAUNCH(128, true, false, true, true) : FL_FWD_LAUNCH(128, true, false, false, true);
    else if (a->d == 128) rc = gf ? FL_FWD_LAUNCH(128, false, false, true, true) : FL_FWD_LAUNCH(128, false, false, false, true);
    else rc = FL_FWD_LAUNCH(64, false, false, false, true);
  } else if (fp4) {
    rc = gf ? FL_FWD_LAUNCH(128, true, false, true, false) : FL_FWD_LAUNCH(128, true, false, false, false);
  } else if (a->d == 128) {
    rc = tl ? FL_FWD_LAUNCH(128, false, true, false, false)
            : (gf ? FL_FWD_LAUNCH(128, false, false, true, false) : FL_FWD_LAUNCH(128, false, false, false, false));
  } else {
    rc = tl ? FL_FWD_LAUNCH(64, false, true, false, false) : FL_FWD_LAUNCH(64, false, false, false, false);
  }
#undef FL_FWD_LAUNCH
  if (rc) return rc;
  return launch_result("fl_fwd: kernel launch");
}
