/*
 * hot_b200 -- C ABI of the B200 (sm_100a) implementation of the HOT linear-layer backward.
 *
 * Every entry point takes raw DEVICE pointers, sizes and a CUDA stream, launches its
 * kernels on that stream and returns without synchronising (except where stated).  No
 * entry point allocates device memory: the caller owns every buffer, including the
 * workspaces whose sizes the *_workspace_bytes() queries return.  The return value is a
 * hot_status; hot_status_string() turns it into text.
 *
 * Each declaration names the piece of the reference (sungonuni/HOT) it stands in for,
 * as file:line within that project.
 */
#ifndef HOT_B200_H
#define HOT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* hot_stream_t; /* a cudaStream_t; NULL is the legacy default stream */

enum hot_status {
  HOT_OK = 0,
  HOT_ERR_ARG = 1,         /* null pointer, non-positive size, misaligned pointer or pitch      */
  HOT_ERR_UNSUPPORTED = 2, /* a size or mode the kernels do not cover (message names it)        */
  HOT_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed; see hot_last_error()           */
  HOT_ERR_TIMEOUT = 4,     /* a bounded device-side wait ran out (reported via the status word) */
  HOT_ERR_WORKSPACE = 5    /* workspace too small                                               */
};

enum hot_dtype { HOT_F32 = 0, HOT_BF16 = 1, HOT_I32 = 2 };
enum hot_rounding { HOT_ROUND_NEAREST = 0, HOT_ROUND_STOCH_PHILOX = 1, HOT_ROUND_STOCH_NOISE = 2 };
/* TENSOR / ROW: s = absmax / qmax over the tensor / each row.  SAWB (hot_col_ht_quant only, nearest
 * rounding): one scale from clip = 12.1 * sqrt(mean(y^2)) - 12.2 * mean(|y|), values clamped to
 * +-clip first (sawb_quantizer, utils/quant_matmul.py:40-55). */
enum hot_scale_mode { HOT_SCALE_TENSOR = 0, HOT_SCALE_ROW = 1, HOT_SCALE_SAWB = 2 };
/* INT4: two codes per byte.  The packed dim is cut into runs of 16 codes (8 bytes; a last partial run is
 * zero-filled): byte j of a run holds code j in its low nibble and code j + 8 in its high nibble, so each
 * half of a run expands to consecutive int8 codes with one shift or mask. */
enum hot_storage { HOT_STORE_INT8 = 0, HOT_STORE_INT4 = 1 };
enum hot_layout { HOT_LAYOUT_NATURAL = 0, HOT_LAYOUT_TRANSPOSED = 1 };

/* How one operand is quantised.  Codes lie in [-(2^(bits-1)-1), 2^(bits-1)-1]. */
typedef struct hot_quant {
  int32_t bits;       /* 2..8; HOT_STORE_INT4 needs bits <= 4                                      */
  int32_t storage;    /* hot_storage                                                             */
  int32_t rounding;   /* hot_rounding                                                            */
  int32_t scale_mode; /* hot_scale_mode                                                          */
  uint64_t seed;      /* Philox key   (HOT_ROUND_STOCH_PHILOX)                                   */
  uint64_t offset;    /* Philox stream offset: a different value per quantiser call              */
  const float* noise; /* HOT_ROUND_STOCH_NOISE: uniforms in [0,1), one per code, in the layout   */
                      /* the quantiser sees (see each function); a code rounds up iff u < frac   */
} hot_quant_t;

const char* hot_status_string(int status);

/*
 * Bounded waits.  Every wait inside a kernel (on an mbarrier that a bulk copy, the tensor core or
 * another warp completes) gives up after a time limit: the kernel then ORs one of the bits below
 * into the caller's status word, stops issuing work, releases what it holds and returns normally;
 * the context stays usable and the outputs of that launch are incomplete.  The status word is a
 * device uint32 the caller zeroes and reads back; hot_check_status turns a value read back into a
 * hot_status (HOT_OK for 0, else HOT_ERR_TIMEOUT with the kernels named in hot_last_error()).
 * hot_set_wait_limit_ns sets the limit for launches made after it (process-wide; 0 restores the
 * default of 1.5 s).  hot_wait_probe launches one warp that waits on a barrier nothing arrives on,
 * so that the give-up path can be exercised: it needs a limit of at most 100 ms.
 * The reference has no counterpart (its kernels have no waits: cuda_measure/HLQ_backward_kernel.cu
 * synchronises the device between stages, :525-552).
 */
/*
 * The GEMM and the fused grad_out kernels are persistent: one CTA per SM of the device.  A caller whose
 * communication library runs kernels beside them (the grad_w all-reduce of a data-parallel step) can ask
 * for `sms` SMs to be left out of those grids, so that the collective's CTAs find room at once instead of
 * queueing behind a persistent CTA; 0 (the default) uses every SM.  Process-wide, for launches made after it.
 * The reference has no counterpart (DistributedDataParallel schedules its own kernels, ViT_main.py:284-286).
 */
void hot_set_sm_margin(int sms);

enum hot_status_bits { HOT_STATUS_GEMM = 1, HOT_STATUS_GO_DUAL = 2, HOT_STATUS_GO_DUAL_TC = 4, HOT_STATUS_PROBE = 8 };
void hot_set_wait_limit_ns(uint64_t limit_ns);
uint64_t hot_get_wait_limit_ns(void);
int hot_wait_probe(uint32_t* status_word, hot_stream_t stream);
int hot_check_status(uint32_t status_value);
/* Text of the most recent failure on the calling thread ("" if none). */
const char* hot_last_error(void);
/* Library ABI version (bumped on any signature change). */
int hot_abi_version(void);

/*
 * Fused block-Hadamard transform along the LAST (contiguous) dim + quantisation.
 *   x      [rows, cols] row-major, pitch ldx elements, dtype HOT_F32 | HOT_BF16
 *   order  Hadamard block order: 1, 2, 4, ..., 64; cols % max(order, 16) == 0
 *   codes  HOT_STORE_INT8: [rows, cols] int8, pitch ld_codes bytes
 *          HOT_STORE_INT4: [rows, cols/2] bytes (cols is a multiple of 16: whole runs), pitch ld_codes bytes
 *   scales [1] (HOT_SCALE_TENSOR) or [rows] (HOT_SCALE_ROW): s = absmax / (2^(bits-1)-1)
 *   absmax_ws  one 32-bit word of scratch, used in HOT_SCALE_TENSOR mode only
 * noise / Philox element index: row * cols + col.
 * Stands in for lowering_matmul_front (utils/hadamard_matmul.py:121-141) followed by
 * stoch_quantizer / int_quantizer / norm_quantizer (utils/quant_matmul.py:19-37,86-122),
 * and for fwht_kernel + find_scale_kernel + quant_int4_kernel / quant_int4_per_token_kernel /
 * quant_int8_kernel (cuda_measure/HLQ_backward_kernel.cu:39-178,282-307).
 */
int hot_row_ht_quant(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order,
                     const hot_quant_t* q, void* codes, int64_t ld_codes, float* scales,
                     uint32_t* absmax_ws, hot_stream_t stream);

/*
 * hot_row_ht_quant on a batch of samples with ONE SCALE PER SAMPLE, in one pair of launches:
 *   x      [batch, rows, cols] (sample b at row b * rows of a [batch * rows, cols] matrix, pitch ldx)
 *   codes  same layout as x; scales [batch]; absmax_ws  `batch` 32-bit words of scratch
 * q->scale_mode must be HOT_SCALE_TENSOR (per-row scales do not depend on the batch: use
 * hot_row_ht_quant).  noise / Philox element index: (b * rows + row) * cols + col.
 * Stands in for the vmapped quantisers (torch.vmap(stoch_quantizer_BWD / int_quantizer_BWD),
 * utils/quant_matmul.py:102-106,117-122) the reference applies to 3-D [B, L, O] tensors after
 * lowering_matmul_front (utils/hadamard_matmul.py:121-141).
 */
int hot_row_ht_quant_batched(const void* x, int dtype, int64_t batch, int64_t rows, int64_t cols, int64_t ldx,
                             int order, const hot_quant_t* q, void* codes, int64_t ld_codes, float* scales,
                             uint32_t* absmax_ws, hot_stream_t stream);

/*
 * Fused block Walsh-Hadamard transform along the FIRST dim with row selection (the
 * Hadamard low-rank projection; all rows kept = plain Hadamard) + quantisation, written
 * TRANSPOSED so that the transformed dim becomes the contiguous (contraction) dim.
 *   x      [rows, cols] row-major, pitch ldx elements; rows % order == 0
 *   order  n = 2..64 (power of two)
 *   sel    HOST array of r natural-order row indices of the Sylvester matrix H_n, in
 *          output order (out row b*r+j = sum_t H_n[sel[j], t] * x[b*n+t, :])
 *   codes_t [cols, rows*r/n] codes (int8, or packed int4 along the transformed dim),
 *          pitch ld_codes bytes, a multiple of 16
 *   scales [1] (HOT_SCALE_TENSOR) or [cols] (HOT_SCALE_ROW: one scale per row of the
 *          transposed output, i.e. per input column)
 *   absmax_ws  scratch, hot_col_ht_quant_scratch_words() 32-bit words: 1 (TENSOR), cols (ROW), or
 *          two doubles per CTA (SAWB; 8-byte aligned)
 *   logical_layout  layout in which the reference's quantiser sees the tensor, which fixes
 *          the noise / Philox element index: HOT_LAYOUT_NATURAL [rows*r/n, cols] or
 *          HOT_LAYOUT_TRANSPOSED [cols, rows*r/n]
 * Stands in for lowering_matmul_back (utils/hadamard_matmul.py:143-161) with the matrices
 * of make_hadamard / make_WHT (:57-59,209-226) followed by a quantiser, as used at
 * utils/quant_matmul.py:189-204 (activation buffer), :269-285 (weight), :300-320 (g_w side
 * of grad_output); and for the transpose + "first L/2 rows" stand-in at
 * cuda_measure/HLQ_backward_kernel.cu:536-549,587-611.
 */
int hot_col_ht_quant(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order,
                     const int32_t* sel, int r, const hot_quant_t* q, int logical_layout,
                     void* codes_t, int64_t ld_codes, float* scales, uint32_t* absmax_ws,
                     hot_stream_t stream);
/*
 * hot_col_ht_quant on a batch of samples with ONE SCALE PER SAMPLE:
 *   x        [batch, rows, cols]: sample b is rows b * rows .. of a [batch * rows, cols] matrix;
 *            the transform runs along the rows of each sample (rows % order == 0)
 *   codes_t  [cols, batch * sample_pitch] INT8: sample b's rows * r / order codes start
 *            b * sample_pitch bytes into each output row and are followed by zeros up to the next
 *            sample (sample_pitch a multiple of 16; a multiple of 128 for hot_gemm_i8_grouped)
 *   scales [batch];  absmax_ws  `batch` words of scratch (HOT_SCALE_SAWB: batch times the words
 *            hot_col_ht_quant_scratch_words gives for one sample, 8-byte aligned)
 * HOT_SCALE_TENSOR, HOT_SCALE_SAWB (the clip of each sample from its own moments, as the vmapped
 * sawb_quantizer gives, utils/quant_matmul.py:51-55) or HOT_SCALE_ROW (scales [batch, cols]: one per
 * sample and output row, the vmapped norm_quantizer; batch * cols words of scratch); HOT_STORE_INT8 only.  noise element index: b * (rows*r/order * cols) + the index
 * hot_col_ht_quant would use within the sample; Philox element index: the byte position in codes_t
 * counted with a row pitch of batch * sample_pitch (column c, sample b, code l: (c * batch + b) *
 * sample_pitch + l).
 * Stands in for lowering_matmul_back on a 3-D tensor (utils/hadamard_matmul.py:143-161, the
 * middle-dim case) followed by a vmapped quantiser, as FLinearQ uses them for [B, L, I]
 * activations and [B, L, O] output gradients (utils/quant_matmul.py:180-204, 300-320).
 */
int hot_col_ht_quant_batched(const void* x, int dtype, int64_t batch, int64_t rows, int64_t cols, int64_t ldx,
                             int order, const int32_t* sel, int r, const hot_quant_t* q, int logical_layout,
                             void* codes_t, int64_t ld_codes, int64_t sample_pitch, float* scales,
                             uint32_t* absmax_ws, hot_stream_t stream);
/* Scratch words hot_col_ht_quant needs for these sizes and this hot_scale_mode (0 on bad arguments). */
size_t hot_col_ht_quant_scratch_words(int dtype, int64_t rows, int64_t cols, int order, int r, int scale_mode);

/*
 * hot_col_ht_quant without a scratch argument, for callers that cannot supply device scratch
 * of their own: code running where device allocation is off limits (a host that hands the
 * library a fixed set of pre-registered buffers, an allocator-free inference/training runtime,
 * a section of the program in which cudaMalloc would synchronise or is simply forbidden).
 * The abs-max words live in a 64 KiB array inside the library's device image instead, which
 * every GPU that loads the library carries until the process exits.
 *   - Same arguments, results and errors as hot_col_ht_quant, minus absmax_ws.
 *   - Limit: the array holds 16384 words.  HOT_SCALE_TENSOR needs one (any size goes);
 *     HOT_SCALE_ROW needs one per column, so cols <= 16384; HOT_SCALE_SAWB needs four per CTA of
 *     the statistics kernel plus four, i.e. hot_col_ht_quant_scratch_words(...) <= 16384 (about
 *     4095 CTAs: in bf16 with order 16, 12608 x 3072 fits and 50432 x 3072 does not).  Beyond the limit the call
 *     fails with HOT_ERR_UNSUPPORTED and says so.
 *   - It allocates nothing (no cudaMalloc / cudaFree / allocating library call).  The first call
 *     on each device looks up the array's device address; make that first call outside any
 *     stream capture.  The device of `stream` must be the current device on EVERY call: the
 *     address is chosen by the current device.
 *   - All calls on a device share the one array, which keeps the last call's contents.  In the
 *     abs-max modes each call clears the words it uses on its stream before using them; in
 *     HOT_SCALE_SAWB mode every word that is read was written by the same call's first kernel.
 *     So calls that run one after another are independent; calls that can overlap on the GPU
 *     (different streams, no ordering between them) race on it and must be serialised by the
 *     caller.
 * This entry point has no counterpart in the reference.
 */
int hot_col_ht_quant_static(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order,
                            const int32_t* sel, int r, const hot_quant_t* q, int logical_layout,
                            void* codes_t, int64_t ld_codes, float* scales, hot_stream_t stream);

/*
 * The un-quantised projection of hot_col_ht_quant in the natural layout, and its transpose:
 *   hot_hla_project: out[b*r + j, c] = sum_t H_n[sel[j], t] * x[b*n + t, c]      x [rows, cols] -> out float32 [rows*r/n, cols]
 *   hot_hla_expand : out[b*n + t, c] = scale * sum_j H_n[sel[j], t] * in[b*r + j, c]   in float32 [rows_out*r/n, cols] -> out [rows_out, cols]
 * Same fixed butterfly order as the quantising kernels.  Pitches ldx / ldo / ldi in elements.
 * Stand in for lowering_matmul_back(h_bs, .) where its result is quantised as it stands
 * (transform_scheme low_rank / gilr_gwh, utils/quant_matmul.py:229-234) and for
 * lowering_matmul_back(h_bs.mT, grad_input) / n (utils/quant_matmul.py:334,337).
 */
int hot_hla_project(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int order, const int32_t* sel,
                    int r, float* out, int64_t ldo, hot_stream_t stream);
int hot_hla_expand(const float* in, int64_t ldi, int64_t rows_out, int64_t cols, int order, const int32_t* sel, int r,
                   float scale, void* out, int out_dtype, int64_t ldo, hot_stream_t stream);

/*
 * Integer GEMM on tcgen05 (kind::i8) with fused dequantisation:
 *   out[m, n] = ((float)(sum_k a[m,k] * b[n,k]) * sa[m or 0]) * sb[n or 0] * post
 *   a [M, K] and b [N, K]: K contiguous, pitches lda/ldb in BYTES (multiples of 16),
 *       storage HOT_STORE_INT8 or HOT_STORE_INT4 (K even, packed along K)
 *   scale_a / scale_b: device floats, [1] or per row ([M] / [N]) when *_per_row != 0;
 *       scale_a_per_row = k > 1: one scale per k consecutive rows of a ([ceil(M / k)]: the per-sample
 *       scales of a batch of k-row samples)
 *   out: HOT_F32 | HOT_BF16 [M, N] pitch ldo elements, or HOT_I32 for the raw accumulator
 *   status_word: device word the kernel ORs a non-zero code into when a bounded wait runs
 *       out (may be NULL); the caller clears and reads it
 * Stands in for CutlassSgemmNN_int4 / CutlassSgemmNN_int8 + dequantize_cuda_kernel /
 * dequantize_cuda_per_token_kernel (cuda_measure/HLQ_backward_kernel.cu:181-280,309-450)
 * and for the float matmuls on integer values at utils/quant_matmul.py:288-290,322-324.
 */
int hot_gemm_i8(const void* a, int a_storage, int64_t lda, const void* b, int b_storage, int64_t ldb,
                int64_t M, int64_t N, int64_t K, const float* scale_a, int scale_a_per_row,
                const float* scale_b, int scale_b_per_row, float post, void* out, int out_dtype,
                int64_t ldo, uint32_t* status_word, hot_stream_t stream);

/*
 * hot_gemm_i8 with a caller-owned workspace (hot_gemm_i8_workspace_bytes(M, N) bytes, 16-byte
 * aligned, contents irrelevant).  With it the kernel may cut the work into equal shares of
 * (tile, k-block) units per SM ("stream-K") instead of whole tiles: a tile shared by several CTAs
 * is summed, in exact int32 arithmetic, by the contributor that arrives last.  Results are
 * identical to hot_gemm_i8; the schedule matters when the tile count is not a multiple of the SM
 * count (few tiles, or a ragged last wave).  workspace == NULL behaves as hot_gemm_i8.
 */
size_t hot_gemm_i8_workspace_bytes(int64_t M, int64_t N);
int hot_gemm_i8_ws(const void* a, int a_storage, int64_t lda, const void* b, int b_storage, int64_t ldb,
                   int64_t M, int64_t N, int64_t K, const float* scale_a, int scale_a_per_row,
                   const float* scale_b, int scale_b_per_row, float post, void* out, int out_dtype,
                   int64_t ldo, void* workspace, size_t workspace_bytes, uint32_t* status_word,
                   hot_stream_t stream);

/*
 * Integer GEMM whose contraction axis is a batch of samples laid side by side, each with its own
 * pair of scales; the dequantised per-sample products are summed in fp32, sample 0 first:
 *   out[m, n] = (sum_g ((float)(sum_{k in group g} a[m,k] * b[n,k]) * scale_a[g]) * scale_b[g]) * post
 *   a [M, groups * group_k], b [N, groups * group_k] INT8, K contiguous, pitches in bytes
 *   group_k a multiple of 128 (pad each sample with zero codes: hot_col_ht_quant_batched does)
 *   scale_a [groups], or with scale_a_per_row != 0 [groups, M]: scale_a[g * M + m] (one scale per
 *   sample and row, what the vmapped norm_quantizer gives, utils/quant_matmul.py:19-37);  scale_b [groups]
 *   out HOT_F32 | HOT_BF16, base and pitch 16-byte aligned
 * Stands in for the batched matmul on integer values, the per-sample scales and the sum over
 * the batch that autograd applies to the [B, O, I] result (utils/quant_matmul.py:322-324).
 */
int hot_gemm_i8_grouped(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t M, int64_t N,
                        int64_t groups, int64_t group_k, const float* scale_a, int scale_a_per_row,
                        const float* scale_b, float post, void* out, int out_dtype, int64_t ldo,
                        uint32_t* status_word, hot_stream_t stream);

/*
 * Two integer GEMMs in one launch.  The g_x product of a layer leaves its last wave of tiles nearly
 * empty at ViT sizes (297 tiles of 128 x 256 on 148 SMs) and the g_w product is a few long tiles:
 * run together, the g_w tiles ride in the SMs that wave leaves idle.  Each problem is what
 * hot_gemm_i8 computes; results are identical to two hot_gemm_i8 calls, and when the shapes do not
 * suit one launch (rider tiles of 128 x 256 more than SMs, or no gain by the cost model) that is
 * what happens internally.
 *   main:  a INT8 or packed INT4, b INT8;   rider: a and b INT8.
 */
typedef struct hot_gemm_problem {
  const void* a;
  int32_t a_storage;        /* hot_storage of a (b is HOT_STORE_INT8) */
  int64_t lda;              /* bytes */
  const void* b;
  int64_t ldb;              /* bytes */
  int64_t M, N, K;
  const float* scale_a;
  int32_t scale_a_per_row;  /* as in hot_gemm_i8 */
  const float* scale_b;
  int32_t scale_b_per_row;
  float post;
  void* out;
  int32_t out_dtype;        /* hot_dtype */
  int64_t ldo;              /* elements */
} hot_gemm_problem_t;
int hot_gemm_i8_dual(const hot_gemm_problem_t* main_problem, const hot_gemm_problem_t* rider_problem,
                     uint32_t* status_word, hot_stream_t stream);

/* Per-layer configuration of the backward pass (scheme gih_gwlr, utils/quant_matmul.py:214-348). */
typedef struct hot_linear_cfg {
  int32_t dtype;      /* dtype of grad_out, w, x and of the returned gradients                  */
  int32_t order_o;    /* Hadamard block order along O (make_hadamard(O): min(16, 2-adic part))  */
  int32_t order_l;    /* low-rank block order n along tokens                                    */
  int32_t rank_l;     /* kept rows r (<= n)                                                     */
  int32_t sel_l[64];  /* the r natural-order row indices                                        */
  hot_quant_t q_gx;   /* grad_out on the g_x path   (scale_mode ROW = per token)                */
  hot_quant_t q_w;    /* weight                                                                 */
  hot_quant_t q_gw;   /* grad_out on the g_w path   (scale_mode ROW = per output channel)       */
  hot_quant_t q_x;    /* activation buffer                                                      */
} hot_linear_cfg_t;

/* Bytes of workspace hot_linear_backward / hot_abc_compress need for these sizes. */
size_t hot_linear_workspace_bytes(int64_t L, int64_t O, int64_t I, const hot_linear_cfg_t* cfg);
/* Pitch in bytes of the compressed activation buffer [I, L*r/n] for these sizes. */
int64_t hot_abc_pitch(int64_t L, const hot_linear_cfg_t* cfg);

/*
 * Activation-buffer compression (forward side): x [L, I] -> x_q_t [I, L*r/n] int8 codes
 * (pitch hot_abc_pitch) + scale_x [1].  noise layout: HOT_LAYOUT_NATURAL [L*r/n, I].
 * workspace: hot_col_ht_quant_scratch_words() words at least.  With 16 bytes or more, bf16 input, the
 * basis "8 lowest-sequency rows of H_16", L % 32 == 0, I % 128 == 0, 16-byte aligned x and pitch, and
 * nearest or Philox rounding, the tensor-core kernels of hot_go_dual_quant make the buffer (same codes
 * and scale); they use workspace words 0-3 and leave word 3 non-zero if a device-side wait ran out
 * (hot_check_status reads it).
 * Stands in for FLinearQ.setup_context (utils/quant_matmul.py:177-212).
 */
int hot_abc_compress(const void* x, int64_t L, int64_t I, int64_t ldx, const hot_linear_cfg_t* cfg,
                     void* x_q_t, float* scale_x, void* workspace, size_t workspace_bytes,
                     hot_stream_t stream);

/*
 * Both quantised operands of grad_out in two fused launches (abs-max pass + quantise pass),
 * each reading go [L, O] once through a TMA-fed shared-memory pipeline:
 *   q_go   [L, O] codes of Q(HT_O(go)) for g_x (cfg->q_gx; INT4 packed or INT8), scale(s) s_gx
 *   q_gw_t [O, L/2] INT8 codes of Q(HLA(go))^T for g_w (cfg->q_gw), scale(s) s_gw
 * bit-identical to hot_row_ht_quant + hot_col_ht_quant on the same input.  Covers the low-rank
 * basis "8 lowest-sequency rows of H_16" (cfg->order_l = 16, rank_l = 8), L % 32 == 0,
 * O % 64 == 0, INT8 storage for q_gw, nearest or Philox rounding; HOT_ERR_UNSUPPORTED otherwise.
 *   scratch  L + O + 2 words (per-token and per-channel abs-max, whichever mode is on)
 * Stands in for the same reference code as those two functions (both read grad_output:
 * utils/quant_matmul.py:237-257 and :300-320).
 */
int hot_go_dual_quant(const void* go, int64_t L, int64_t O, int64_t ldgo, const hot_linear_cfg_t* cfg,
                      void* q_go, int64_t ld_qgo, float* s_gx, void* q_gw_t, int64_t ld_qgw, float* s_gw,
                      uint32_t* scratch, uint32_t* status_word, hot_stream_t stream);

/*
 * The HOT backward of one linear layer:
 *   grad_x [L, I] = (Q(HT_O(go)) . Q(HT_O(w))) * s_go * s_w / order_o
 *   grad_w [O, I] = (Q(HLA(go))^T . x_q) * s_gw * s_x / order_l
 * go [L, O] pitch ldgo, w [O, I] pitch ldw (elements); x_q_t / scale_x from hot_abc_compress.
 * status_word: device word, non-zero after the call completes if a device-side wait ran out.
 * cfg->q_gx / q_gw take HOT_SCALE_TENSOR or HOT_SCALE_ROW (HOT_SCALE_SAWB is for q_w and q_x).
 * Where the tensor-core kernels of hot_go_dual_quant apply (bf16, order_o 16, the basis above, O % 128 == 0,
 * I % 32 == 0, one scale for the weight) the weight is transformed and quantised inside those two launches
 * and a call is three kernels on `stream`.  Otherwise the weight is quantised on a helper stream the
 * library keeps per device (one stream and one fork/join event pair): calls on one device must come
 * from one host thread and one stream at a time; the first call on a device creates them and should
 * be made outside stream capture.
 * Stands in for FLinearQ.backward (utils/quant_matmul.py:214-348) and for backward_cuda
 * (cuda_measure/HLQ_backward_kernel.cu:457-737).
 */
int hot_linear_backward(const void* go, int64_t ldgo, const void* w, int64_t ldw, const void* x_q_t,
                        const float* scale_x, int64_t L, int64_t O, int64_t I,
                        const hot_linear_cfg_t* cfg, void* grad_x, int64_t ldgx, void* grad_w,
                        int64_t ldgw, void* workspace, size_t workspace_bytes, uint32_t* status_word,
                        hot_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* HOT_B200_H */
