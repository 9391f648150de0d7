/* C ABI of the B200 microscaling-attention hot path (libflamia_b200.so).
 *
 * Plain pointers and sizes only; every pointer is a CUDA device pointer unless stated otherwise; every function
 * enqueues on the given cudaStream_t (passed as void*), never synchronises the host, never allocates device memory,
 * and returns 0 or a positive FL_ERR_* code. Device-side problems (a bounded wait that ran out) are reported through
 * the int status word the caller passes in (0 = ok) and can be read with fl_read_status(): 0x100 | site = that wait
 * gave up and the kernel drained with its outputs partly written; 0x200 = an entry of the packed-document table did not
 * fit the buffer and was clamped (nothing out of bounds was touched).
 *
 * The reference has no C ABI on this path: its boundary is Python over CuTe-DSL JIT kernels. Each entry point below
 * names the reference interface it replaces (paths inside the reference repository).
 */
#ifndef FLAMIA_B200_H
#define FLAMIA_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FL_ABI_VERSION 8

/* fl_quant_args.flags */
#define FL_Q_HADAMARD 1            /* rotate rows by diag(signs) H_128 / sqrt(128) before quantising (d = 128) */
#define FL_Q_TOKEN_LOCAL 2         /* codes / sf_tok from each token's own exponent */
#define FL_Q_HADAMARD_NVFP4_ONLY 4 /* rotate only the values of the NVFP4 copy; the E4M3 codes stay unrotated */
#define FL_Q_O_PACKED 8            /* packed source with the prologue: o has x's packed rows (else the outputs' rows) */
#define FL_Q_LEGACY 16             /* keep the four-lanes-per-row kernel where the one-thread-per-row kernel would serve
                                      (the two are bit-identical; for tests that compare them) */

/* Fused block-scaled quantiser + backward prologue.
 * Replaces flash_attn/cute/quant/fp8.py:2512 quantize_fp8_blocks (kernel :1639), the fused NVFP4 S-operand copy
 * flash_attn/cute/quant/_fp8_nvfp4.py:121-158, and the fused backward preprocess (compute_d_with_output,
 * shifted_log2_lse_from, zero_accumulator: quant/fp8.py:1980-2032). Any output pointer may be NULL = not produced. */
typedef struct fl_quant_args {
  const void* x;        /* (b, s, h, d) bf16 (in_f16 = 0) or f16 (1), contiguous, 16-byte aligned; s % 128 == 0; d = 64 | 128 */
  const void* o;        /* prologue: forward output, same layout / dtype as x */
  const float* lse;     /* (b, h, s) natural-log LSE */
  uint8_t* codes;       /* (b, s, h, d) E4M3 */
  uint8_t* codes_t;     /* (b, h, d, s) channel-major copy */
  uint8_t* e_tab;       /* (b, h, s/32, d/32) UE8M0 bytes (0 = all-zero block) */
  float* fac;           /* (b, h, s/32) 2^(e-127), zero blocks take their tile's largest factor (1 if none) */
  uint8_t* sf_tok;      /* (b, h, s/128, 512) SM100 128x4 atoms, rows = tokens, K = d/32 */
  uint8_t* sf_dim;      /* (b, h, s/128, 512) atoms, rows = d, K = tokens/32 */
  float* token_factors; /* (b, h, s) 2^(e_token-127) (1 for an all-zero token) */
  uint8_t* x4;          /* (b, s, h, d/2) NVFP4 E2M1 codes, element 0 in the low nibble */
  uint8_t* sf4;         /* (b, h, s/128, d/64, 512) E4M3 scale atoms, rows = tokens, K = d/16 */
  float* d_out;         /* (b, h, s): d_multiplier * rowsum(O * dequant(codes)) in the fixed tree order */
  float* lse_log2;      /* (b, h, s): (lse == -inf ? 0 : lse * log2 e) - lse_shift */
  void* zero_acc;       /* f16 dQ accumulator of b * h * s * d elements, zero-filled (a flat fill: its layout is the backward's,
                           (b, h, d, s) at d = 128 and (b, h, s, d) at d = 64, see fl_attn_args.dq_acc) */
  float* tile_stats;    /* (b, h, s/128, 2): amax and max row sum of squares of the values quantised */
  int32_t b, s, h, d;
  int32_t flags;
  int32_t in_f16;
  float lse_shift;
  float d_multiplier;
  int32_t* status;      /* device int, 0 on entry, or NULL: a wait of the kernel's load pipeline that gave up writes a code */
  int64_t wait_cycles;  /* budget of one device-side wait in SM clocks; 0 = default (2^31) */
  /* Packed source (documents stored back to back, b = 1): x is (src_rows, h, d) and the outputs are the 128-aligned buffer
   * of s rows; slot_src[i] = first row of x that goes to rows [128 i, 128 i + 128) of the outputs (-1: the slot is
   * empty), slot_rows[i] = how many of them are real (the others quantise as zeros). Replaces the row gather of
   * flash_attn/cute/lp_docmaps.py (the quantisers read Q / K / V / dO through the row map). NULL = x has the outputs' rows. */
  const int32_t* slot_src;
  const int32_t* slot_rows;
  int32_t src_rows;
  /* Per-token statistic for the per-query-row causal dQ pre-scale (flash_attn/cute/interface_bwd_fp4.py:950-987
   * dq_causal_kv_rows / dq_causal_rows): (b, s) float, ZERO on entry, or NULL. Each (token, head) takes the maximum into
   * its token's entry (over the heads of one launch): row_stat_kind 1 = the row's sum of squares, 2 = its largest
   * magnitude, 3 = its 2-norm (of the values quantised, i.e. after the rotation where there is one). */
  float* row_stat;
  int32_t row_stat_kind;
} fl_quant_args;

int fl_quant_blocks(const fl_quant_args* args, void* stream);

/* fl_attn_args.mode */
#define FL_MODE_FP8 0   /* S = E4M3 x E4M3 with the token-block factors folded into the softmax */
#define FL_MODE_FP4 1   /* S = NVFP4 x NVFP4 block-scaled (kind::mxf4nvf4, scale_vec::4X) */
/* fl_attn_args.flags */
#define FL_A_CAUSAL 1        /* bottom-right aligned causal mask */
#define FL_A_OUT_F16 2       /* outputs / gradients are f16 instead of bf16 */
#define FL_A_TOKEN_LOCAL 4   /* per-token factor tables instead of per-32-token ones */
#define FL_A_DQ_ROWLOCAL 8   /* backward: the dQ side of dS-hat gets one exponent per query row of each 32-key block */
#define FL_A_HAD_DQ 16       /* backward: dQ accumulator holds rotated rows (post kernel rotates back) */
#define FL_A_HAD_DK 32       /* backward: rotate dK back in the epilogue */
#define FL_A_P_GROUP 64      /* forward: group-frame P-hat (one UE8M0 exponent per query row and 32 keys) instead of the row frame */

/* One attention problem. Operands are the quantiser's outputs; q / k / v / dO codes are (b, s, heads, d) E4M3. */
typedef struct fl_attn_args {
  const uint8_t* q_codes;
  const uint8_t* k_codes;
  const uint8_t* v_codes;
  const uint8_t* do_codes;   /* backward only */
  const float* fac_q;        /* (b, h, s_q/32)    [token_local: (b, h, s_q)] */
  const float* fac_k;        /* (b, h_kv, s_k/32) [token_local: (b, h_kv, s_k)] */
  const float* fac_v;        /* (b, h_kv, s_k/32) [token_local: (b, h_kv, s_k)] */
  const float* fac_do;       /* (b, h, s_q/32) backward only */
  const uint8_t* q4;         /* FL_MODE_FP4: (b, s_q, h, d/2) */
  const uint8_t* k4;         /* (b, s_k, h_kv, d/2) */
  const uint8_t* sfq4;       /* (b, h, s_q/128, d/64, 512) */
  const uint8_t* sfk4;       /* (b, h_kv, s_k/128, d/64, 512) */
  void* out;                 /* forward: (b, s_q, h, d) bf16 | f16 */
  float* lse;                /* forward: (b, h, s_q) natural log */
  const float* lse_log2;     /* backward: (b, h, s_q) lse * log2 e - 8 */
  const float* d_rows;       /* backward: (b, h, s_q) -2^-8 * rowsum(O * dO) */
  void* dq_acc;              /* backward: f16, zeroed by the prologue; reduce-added here. Layout (b, h, d, s_q) at d = 128,
                                (b, h, s_q, d) at d = 64; fl_dq_post reads the same layout */
  const float* dq_scale;     /* backward: (b, s_q/128) pre-scale of the f16 accumulator per query tile (power of two) */
  void* dk;                  /* backward: (b, s_k, h_kv, d) */
  void* dv;                  /* backward: (b, s_k, h_kv, d) */
  const int32_t* doc_start;  /* packed documents: (n_docs + 1) tile-aligned row starts, or NULL = batched */
  const int32_t* doc_len;    /* (n_docs) true lengths */
  int32_t n_docs;
  int32_t b, s_q, s_k, h, h_kv, d;
  float softmax_scale;
  int32_t mode;
  int32_t flags;
  int32_t* status;           /* device int, 0 on entry; a kernel that gives up a wait writes a nonzero code */
  int64_t wait_cycles;       /* budget of one device-side wait in SM clocks; 0 = default (2^31) */
  /* Sliding window (the reference's window_size=(left, right), flash_attn/cute/lowprec/api.py:270): query i sees key j
   * iff i + off - left <= j <= i + off + right, off = s_k - s_q. Stored as window + 1; 0 = unlimited on that side, so
   * a zero-filled struct means no window. FL_A_CAUSAL caps the right side at 0. */
  int32_t window_left_p1;
  int32_t window_right_p1;
  /* Batched form only: (b) int32, the number of valid keys of each batch row (keys at or past it are masked; dK / dV rows
   * there come back zero), or NULL. The reference's batched seqused_k (flash_attn/cute/lowprec/api.py:270). The causal
   * alignment keeps using s_k - s_q. */
  const int32_t* seqused_k;
  /* Soft cap of the scaled scores: c > 0 turns score = softmax_scale q.k into c tanh(score / c) before masking, and dS takes
   * the factor 1 - tanh^2 (the reference's softcap, flash_attn/cute/utils.py:167-187); 0 = off. Default P-hat route only
   * (no token-local / row-local variants). */
  float softcap;
  /* Backward, deterministic dQ (the reference's deterministic=True: semaphore-ordered dQ reduction,
   * flash_attn/cute/flash_bwd_sm100_fp4.py:4119-4215): (b, h, s_q/128, 2) int32, ZERO on entry, or NULL = the partial
   * sums are added in arrival order. With the table, the key tiles that see a query tile add their f16 partial sums in
   * ascending key order: each waits (bounded by wait_cycles; status 0x100 | 44 when it gives up) until the table entry of
   * its (head, query tile, 64-query half) has counted the key tiles before it, adds, waits for the addition to complete
   * and counts itself. dQ is then bitwise reproducible from call to call; the other outputs always are. */
  int32_t* dq_order;
  /* Backward: (b, s_q) power-of-two pre-scale of the f16 accumulator per QUERY ROW (the reference's row-wise causal
   * pre-scale of its 1-CTA kernels, flash_attn/cute/device_scales.py:256-268), or NULL = dq_scale per query tile. With
   * it dq_scale is not read. Batched form only. */
  const float* dq_scale_rows;
  /* Operands whose factor tables are not powers of two (pre-quantised E4M3 inputs with float descales, the reference's
   * flash_attn/cute/lowprec/prequant_fa3.py): a block-scaled product takes only the exponent of a factor, so the mantissa
   * (factor / 2^floor(log2 factor), in [1, 2)) is multiplied in afterwards. Forward: o_mult (b, h_kv) = V's mantissa, on
   * the output rows. Backward: dk_mult (b, h_kv) = Q's mantissa, on dK (dQ takes K's in fl_dq_post_ex). NULL = 1. */
  const float* o_mult;
  const float* dk_mult;
  /* Packed documents whose outputs go straight to the caller's packed tensors (with doc_start / doc_len; the counterpart
   * of fl_quant_args.slot_src on the way out): out (forward) and dk, dv (backward) are (out_rows, heads, d) with the
   * documents stored back to back; slot_src[i] = the packed row of row 128 i of the aligned buffer the kernels work in
   * (-1: an empty slot), slot_rows[i] = how many rows of that slot are real. A full slot leaves as one TMA store, a
   * document's last rows as row stores. NULL = the outputs have the aligned buffer's rows. lse keeps those rows. */
  const int32_t* slot_src;
  const int32_t* slot_rows;
  int32_t out_rows;
  /* fl_fwd with FL_A_TOKEN_LOCAL: log2 f_V(key) and 1 / f_V(key) as float tables (b, h_kv, s_k), from fl_token_aux over
   * V's token_factors. The forward folds log2 f_V into the scores and takes f_V back out of the row sums for every score:
   * read from tables this is one load each, derived from f_V in the kernel it was three integer instructions per score. */
  const float* tok_lg_v;
  const float* tok_rcp_v;
} fl_attn_args;

/* Forward: O = softmax(scale Q K^T + mask) V, LSE.
 * Replaces flash_attn/cute/interface_fwd_fp4.py:301 _flash_attn_fwd -> flash_fwd_sm100_fp4.py:370
 * FlashAttentionForwardSm100. */
int fl_fwd(const fl_attn_args* args, void* stream);

/* Backward main kernel: dK, dV and the pre-scaled f16 dQ accumulator.
 * Replaces flash_attn/cute/interface_bwd_fp4.py:1207 _flash_attn_bwd_fp4 -> flash_bwd_sm100_fp4.py:82
 * FlashAttentionBackwardSm100FP4 (and the 2-CTA variant flash_bwd_sm100_2cta8.py:74). */
int fl_bwd(const fl_attn_args* args, void* stream);

/* f16 dQ pre-scale per query tile from the quantisers' tile statistics.
 * Replaces flash_attn/cute/device_scales.py:124-155, 234-319 (_dq_bound_pow2, _dq_prescale, _dq_tile_table). */
int fl_dq_prescale(const float* stats_do, const float* stats_v, const float* stats_k, int32_t b, int32_t h, int32_t h_kv,
                   int32_t nt_q, int32_t nt_k, int32_t causal_local, float unit, float* kernel_scale, float* post_scale,
                   void* stream);

/* The same per QUERY ROW of a causal square batched call (the reference's dq_tile_causal = 2,
 * flash_attn/cute/device_scales.py:256-268): row i's pre-scale from its own statistic and the running maxima over the
 * keys j <= i. row_do / row_v / row_k: (b, s) per-token statistics of the quantisers (fl_quant_args.row_stat: kind 1, 1
 * and 2 or 3); row_v and row_k are replaced by their prefix maxima. kernel_rows / post_rows: (b, s). */
int fl_dq_prescale_rows(const float* row_do, float* row_v, float* row_k, int32_t b, int32_t s, float unit,
                        float* kernel_rows, float* post_rows, void* stream);

/* dQ postprocess: dq[b, s, h, c] = cast(acc(b, h, s, c) * post_scale[b, s/128] * mult) with optional Hadamard
 * back-rotation, where acc(b, h, s, c) is element [b, h, c, s] of the (b, h, d, s) accumulator at d = 128 (the backward
 * kernel produces transposed dQ tiles) and element [b, h, s, c] of the (b, h, s, d) accumulator at d = 64.
 * Replaces flash_attn/cute/dq_postprocess_cute.py:46 DQPostprocess / bwd_2cta8_side.dq_postprocess_2cta8. */
/* fl_dq_post_ex: the general form. per_row: post_scale is (b, s) instead of (b, s/128); head_mult: (b, h) extra factor per
 * head or NULL (the mantissa of K's factor with pre-quantised inputs). */
int fl_dq_post_ex(const void* dq_acc, const float* post_scale, int32_t per_row, const float* head_mult, float mult, void* dq,
                  int32_t b, int32_t s, int32_t h, int32_t d, int32_t unrotate, int32_t out_f16, void* stream);
/* fl_dq_post_packed: b = 1, the accumulator has the aligned buffer's s rows, dq is the caller's packed (out_rows, h, d)
 * tensor: rows of slot i go to slot_src[i] .. + slot_rows[i] (see fl_attn_args.slot_src). */
int fl_dq_post_packed(const void* dq_acc, const float* post_scale, float mult, void* dq, int32_t s, int32_t h, int32_t d,
                      int32_t unrotate, int32_t out_f16, const int32_t* slot_src, const int32_t* slot_rows, void* stream);
/* Tile statistics of E4M3 codes times a factor per (batch row, head): tile_stats (b, h, s/128, 2) = the largest
 * magnitude and the largest row sum of squares of codes * descale[b, h] per 128-row tile, the figures the quantiser
 * writes for operands it quantises itself (the reference sizes the f16 dQ pre-scale of pre-quantised inputs from one
 * read of the V codes, flash_attn/cute/lowprec/prequant_fa3.py:386-470). */
int fl_code_stats(const void* codes, const float* descale, int32_t b, int32_t s, int32_t h, int32_t d, float* tile_stats,
                  void* stream);
/* lg[i] = log2 f[i], rcp[i] = 1 / f[i] for n power-of-two factors (fl_quant_args.token_factors): the tables of
 * fl_attn_args.tok_lg_v / tok_rcp_v. The reference keeps such per-token rows in its (6, b, h, s) token table
 * (flash_attn/cute/lowprec/_routes.py:749-755). */
int fl_token_aux(const float* factors, int64_t n, float* lg, float* rcp, void* stream);
/* fl_dq_post_rows: post_scale_rows is (b, s), one value per query row. */
int fl_dq_post_rows(const void* dq_acc, const float* post_scale_rows, float mult, void* dq, int32_t b, int32_t s,
                    int32_t h, int32_t d, int32_t unrotate, int32_t out_f16, void* stream);
int fl_dq_post(const void* dq_acc, const float* post_scale, float mult, void* dq, int32_t b, int32_t s, int32_t h,
               int32_t d, int32_t unrotate, int32_t out_f16, void* stream);

/* Backward pass with the f16 dQ accumulator held in a fixed device array of the library (no counterpart in the
 * reference, which always takes torch-allocated buffers). For callers that cannot allocate device memory where the
 * backward runs: a pool sized before this operator was known, a serving loop that keeps the allocator off its hot
 * path, a C / cgo / JNI embedder without an allocator. Runs fl_bwd with args->dq_acc replaced by that array (the field
 * is ignored), then fl_dq_post into dq (b, s_q, h, d) with unrotate = (flags & FL_A_HAD_DQ), out_f16 =
 * (flags & FL_A_OUT_F16). Calls no allocating routine. Limit: b * h * s_q * d <= FL_STATIC_ACC_MAX_ELEMS, otherwise
 * FL_ERR_TOO_LARGE (4) is returned and nothing is enqueued. The used part of the array is cleared on the stream by
 * every call. The first call on a device resolves the array's address (cudaGetSymbolAddress): make it before any
 * stream capture starts. One array per device: calls that overlap in time on one device race on it. */
#define FL_STATIC_ACC_MAX_ELEMS (1 << 23)   /* 16 MiB of f16: e.g. b1 h16 s4096 d128 */
int fl_bwd_static_acc(const fl_attn_args* args, const float* post_scale, float mult, void* dq, void* stream);

/* Row gather / scatter between a packed (total, h, d) tensor and its 128-aligned repacked buffer.
 * Replaces flash_attn/cute/lp_varlen.py:421 pack_rows / unpack_rows. row_map[i] = source row of padded row i or -1. */
int fl_pack_rows(const void* src, void* dst, const int32_t* row_map, int32_t n_dst_rows, int32_t row_bytes, void* stream);
int fl_unpack_rows(const void* src, void* dst, const int32_t* row_map, int32_t n_src_rows, int32_t row_bytes,
                   void* stream);

/* Building-block self test: one 128 x 128 x 128 tensor-core product through the library's own descriptor / TMEM helpers.
 * `which` selects the operand path (see FL_ST_*); used by the unit tests to pin the descriptor encodings. */
#define FL_ST_F8_KMAJOR 0      /* A, B K-major from shared memory, kind::f8f6f4 */
#define FL_ST_F8_B_MNMAJOR 1   /* B MN-major */
#define FL_ST_F8_A_TMEM 2      /* A from tensor memory, B MN-major */
#define FL_ST_MX8_SS 3         /* block-scaled MXFP8, A K-major, B MN-major, scales written with tcgen05.st */
#define FL_ST_MX8_TS 4         /* block-scaled MXFP8, A from tensor memory */
#define FL_ST_NVF4 5           /* block-scaled NVFP4, scale atoms copied with tcgen05.cp */
#define FL_ST_F8_A_MNMAJOR 6   /* A MN-major from shared memory */
#define FL_ST_WAIT_TIMEOUT 7   /* a wait that nothing completes: returns through the bounded-wait path */
#define FL_ST_MX8_MN_N64 8     /* block-scaled MXFP8, A MN-major (128 B rows), B MN-major with N = 64 (64 B rows) */
#define FL_ST_NVF4_N64_HI 9     /* NVFP4 with N = 64: rows 64..127 of B, whose scales are columns 2, 3 of each atom */
#define FL_ST_MX8_A_MN_2X64 10  /* block-scaled MXFP8, A MN-major as two 64-byte-row blocks (M = 2 x 64), B MN-major N = 64 */
int fl_selftest_mma(int32_t which, const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, float* d,
                    int32_t* status, int64_t wait_cycles, void* stream);

/* Copies the device status word to the host (synchronises the stream). */
int fl_read_status(const int32_t* status, int32_t* host_value, void* stream);

/* Detail of the last FL_ERR_CUDA this host thread got from the library: writes "<failing call>: <CUDA error name and
 * text>" into text (a host buffer of text_bytes bytes, may be null) and returns the CUDA error code (10000 + CUresult
 * for a driver call, -1 where there is no code, 0 if no call has failed). No reference counterpart. */
int fl_last_cuda_error(char* text, int32_t text_bytes);

int fl_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif
