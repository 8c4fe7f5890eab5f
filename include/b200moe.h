/* C ABI of libb200moe.so -- the sm_100a fused-MoE path behind pyhip's `fused_moe` call surface.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle (as void*),
 * enqueues work on that stream and returns without synchronising.  Return value: 0 = ok,
 * negative = argument error (nothing was launched), positive = CUDA error code.
 * b200moe_last_error() describes the last non-zero return of the calling thread.
 * The caller provides every buffer, including the workspace; the one exception is the fixed scratch array
 * behind b200moe_forward_static (see there), which is part of the library image.
 *
 * Reference interfaces these replace (paths inside tingqli/pyhip):
 *   - kernels are reached there through ctypes + hipModuleLaunchKernel with raw data_ptr()
 *     arguments on torch's current stream (src/core/hiptools.py:10-35,88-100); the same calling
 *     convention is kept here (ctypes.CDLL, raw pointers, stream as void*).
 */
#ifndef B200MOE_H_
#define B200MOE_H_
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_VERSION 3

/* weight formats */
#define B200MOE_W_MXFP4 0 /* E2M1 pairs (low nibble = even element) + E8M0 scale per 32 along K */
#define B200MOE_W_FP8_128 1 /* e4m3 + fp32 scale per 128x128 block */
#define B200MOE_W_FP8_ROW 2 /* e4m3 + one fp32 scale per output row, w_scale [E, 2I] / [E, H]: the reference's
                               per-token-per-channel FP8 weights (tests/contrib/moe/test_moe.py:123-128); its per-tensor
                               weights (:130-137) are the same with a row's scale repeated.  The scale tensors are passed
                               in place as the *_scale_prepared arguments */
#define B200MOE_W_BF16 3 /* unquantised bf16 weights w1 [E,2I,H] / w2 [E,H,I], no scales (the *_scale arguments are
                            ignored and may be NULL): the reference wrapper's QuantType.No
                            (src/contrib/fused_moe.py:253; torch form tests/contrib/moe/test_moe.py:86-118).  Activations
                            stay bf16 (act_terms / act_quant do not apply), products accumulate in fp32 */
/* activation functions of the gate-up stage */
#define B200MOE_ACT_SILU 0   /* silu(gate) * up                        (test_moe.py:74-75) */
#define B200MOE_ACT_SWIGLU 1 /* clamped gate*sigmoid(1.702 gate)*(up+1) (test_moe.py:76-81) */

/* how the down stage returns its rows to token order */
#define B200MOE_COMBINE_GATHER 0 /* sorted rows -> workspace, then a gather-sum launch in ascending expert order:
                                    bitwise reproducible, the arithmetic of the reference's torch oracle
                                    (tests/contrib/moe/test_moe.py:107-117) */
#define B200MOE_COMBINE_FUSED 1  /* the down epilogue multiplies by the routing weight and adds into the zeroed
                                    output with packed-bf16 reductions -- the reference kernels' own epilogue
                                    (src/contrib/moe.py:703-787 global_atomic_pk_add_bf16); the order of the K
                                    bf16 additions of a token is not fixed */
/* activation operand of the FP8 (128x128-block) GEMMs */
#define B200MOE_ACTQ_TERMS 0   /* two e4m3 terms with E8M0 scales per 32 (default; exact for bf16 inputs to ~2^-9) */
#define B200MOE_ACTQ_1X128 1   /* one e4m3 value with an fp32 scale per token and 128 channels, scale = amax/448:
                                  the reference's per_1x128 activation quantiser (src/contrib/fused_moe.py:276-281,375-381) */

/* Shape of one MoE layer call.  B (rows per sorted block = token tile of the GEMMs) is a multiple
 * of 16 up to 128.  E is the number of experts whose weights are present (local experts under expert
 * parallelism); E_route is the size of the routing id space (E_route >= E; equal without a mask).
 * act_terms: how many packed-FP4 terms represent one activation row inside the MXFP4 GEMMs (1..4; 0 = default 3).
 *   1 is the plain per-1x32 MXFP4 activation format of the reference's a4w4 kernels
 *   (tests/contrib/moe/test_moe.py:665-679, src/contrib/moe_gemm_mxfp4.py:972); 3 keeps the layer within
 *   cosine 0.9999 of the bf16-activation oracle; 4 reproduces bf16 activations to ~1e-4 of the block maximum.
 * doweight_stage1: the routing weight multiplies the gate-up output instead of the down output
 *   (the aiter flag of that name, src/contrib/fused_moe.py:137). */
typedef struct b200moe_shape {
  int32_t T, K, E, E_route, H, I, B;
  int32_t weight_format;
  int32_t activation;
  float swiglu_limit;
  int32_t act_terms;
  int32_t combine_mode;
  int32_t act_quant;
  int32_t doweight_stage1;
  int32_t cta_pairs;   /* MXFP4 GEMMs on CTA pairs (tcgen05.mma.cta_group::2: two CTAs of a cluster share one token tile, each
                          fetching half of it): 0 = in the compute-bound regime (token tiles of 64 rows and more whose
                          activation terms are separate instructions), 1 = never, 2 = wherever the tile allows it */
} b200moe_shape;

/* Byte sizes and offsets of the caller-provided workspace (all offsets 1024-byte aligned). */
typedef struct b200moe_workspace {
  int64_t total_bytes;
  int64_t max_rows;          /* Lmax: worst-case padded row count, multiple of B */
  int64_t off_sorted_ids;    /* u32 [Lmax]      (k<<24)|token, sentinel (K<<24)|T            */
  int64_t off_sorted_w;      /* f32 [Lmax]                                                   */
  int64_t off_sorted_e;      /* i32 [Lmax/B]    local expert id of each block                */
  int64_t off_num_valid;     /* i32 [2]         {padded row total, T}                        */
  int64_t off_loc;           /* i32 [T*K]       sorted position of pair (t,k), -1 if dropped */
  int64_t off_status;        /* i32 [16]        device-side error words, 0 = clean           */
  int64_t off_xq;            /* u8 [terms, Lmax, Hpad/2]  layer input as packed-FP4 terms, sorted order */
  int64_t off_xsf;           /* E8M0 scale chunks of xq                                      */
  int64_t off_hq;            /* u8 [terms, Lmax, Ipad/2]  gate-up output, same form           */
  int64_t off_hsf;           /* E8M0 scale chunks of hq                                      */
  int64_t off_out2;          /* bf16 [Lmax, H]  down-projection rows in sorted order         */
  int64_t off_sort_scratch;  /* i32 scratch of the multi-CTA sort (large batches only)       */
} b200moe_workspace;

int b200moe_version(void);
const char* b200moe_last_error(void);

/* Fills *ws for `shape`.  Pure host arithmetic. */
int b200moe_workspace_layout(const b200moe_shape* shape, b200moe_workspace* ws);

/* Bytes of the prepared scale image of one weight tensor: which = 1 (w1, [E,2I,H]) or
 * 2 (w2, [E,H,I]). */
int b200moe_prepared_scale_bytes(const b200moe_shape* shape, int which, int64_t* scale_bytes);

/* One-off regrouping of a weight tensor's E8M0 scales into pairs of 128-row x 4-scale chunks in
 * tensor-memory order (the packed FP4 weights themselves are consumed in place, in their canonical
 * [E, R, Kd/2] layout).  Plays the part of the reference's e8m0_shuffle / shuffle_weight
 * pre-shuffle (src/misc.py:114-128, tests/contrib/moe/test_moe.py:167-172).
 *   w_s : u8 [E, R, Kd/32]   (R = 2I, Kd = H for which=1; R = H, Kd = I for which=2) */
int b200moe_prepare_scales(const b200moe_shape* shape, int which, const void* w_s, void* out_scale,
                           void* stream);

/* Router: fp32 logits [T, E] -> top-k ids [T, K] (descending score, ties to the lower id) and weights [T, K].
 * The reference leaves routing outside the operator (torch.topk in tests/contrib/moe/test_moe_sorting.py:81-84,
 * aiter's fused_topk in tests/contrib/moe/test_fused_moe.py:38,87); this is that step as one launch in front of
 * b200moe_sort_align.  scoring 0 = softmax, 1 = sigmoid; renormalize != 0 divides the k weights by their sum.
 * E <= 1024. */
int b200moe_route_topk(const float* logits, int32_t T, int32_t E, int32_t K, int32_t scoring,
                       int32_t renormalize, int32_t* topk_ids, float* topk_weight, void* stream);

/* Token->expert sort/align: replaces aiter.moe_sorting as called at src/contrib/fused_moe.py:283,
 * 301-305 and 368-372 (contract: fused_moe.py:56-100; ck_tile reference_moe_sorting.hpp:14-117).
 * Deterministic; only [0, num_valid[0]) of the outputs is defined.  expert_mask may be NULL.
 * loc may be NULL. */
int b200moe_sort_align(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                       int32_t E_route, int32_t B, const int32_t* expert_mask, uint32_t* sorted_ids,
                       float* sorted_weights, int32_t* sorted_expert_ids, int32_t* num_valid_ids,
                       int32_t* loc, void* stream);

/* The same with a token count that lives on the device: tokens at and beyond *num_local_tokens take no
 * part (their pairs are dropped, their loc entries read -1, num_valid_ids[1] = the live count), so a call
 * captured into a CUDA graph at a fixed, padded T serves smaller batches -- the reference's
 * num_local_tokens argument (src/contrib/fused_moe.py:48-49,63,145,304,371).  NULL = all T tokens. */
int b200moe_sort_align_dyn(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                           int32_t E_route, int32_t B, const int32_t* expert_mask,
                           const int32_t* num_local_tokens, uint32_t* sorted_ids, float* sorted_weights,
                           int32_t* sorted_expert_ids, int32_t* num_valid_ids, int32_t* loc, void* stream);

/* The same with caller scratch of b200moe_sort_scratch_bytes(E_route) bytes: from 8192 (token, expert) pairs
 * up the sort is spread over several CTAs (three chained launches; one CTA's store path limits the single-CTA
 * kernel at prefill sizes).  Outputs are bit-identical.  scratch may be NULL (single CTA). */
int b200moe_sort_scratch_bytes(int32_t E_route, int64_t* bytes);
int b200moe_sort_align_ws(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                          int32_t E_route, int32_t B, const int32_t* expert_mask,
                          const int32_t* num_local_tokens, uint32_t* sorted_ids, float* sorted_weights,
                          int32_t* sorted_expert_ids, int32_t* num_valid_ids, int32_t* loc, void* scratch,
                          int64_t scratch_bytes, void* stream);

/* Quantise bf16 rows into `terms` packed-FP4 (E2M1) terms with E8M0 scales per 32, gathered into
 * sorted-row order (stands where the reference calls aiter's per_1x32 activation quantiser
 * followed by moe_mxfp4_sort, tests/contrib/moe/test_moe.py:665-679).
 *   src_mode 0: src is [T, Kd], row = token.   src_mode 1: src is [T, K, Kd], row = token*K + k.
 *   terms 1..4.  q: u8 [terms, max_rows, Kpad/2], Kpad = Kd rounded up to 256.  sf: per (block of B sorted
 *   rows, 128-wide k-block) a group of 512-byte chunks.  Only the rows of live (token, k) pairs are
 *   written; the padding rows of a block stay as they were. */
int b200moe_quant_rows(const void* src_bf16, int32_t src_mode, const uint32_t* sorted_ids,
                       const int32_t* num_valid_ids, int32_t T, int32_t K, int32_t Kd, int32_t B,
                       int32_t terms, int64_t max_rows, void* q, void* sf, void* stream);

/* Same for FP8 128x128-block weights (weight_format B200MOE_W_FP8_128): two e4m3 terms with E8M0
 * scales per 32 (stands where the reference calls aiter's per_1x128 activation quantiser,
 * src/contrib/fused_moe.py:276-281,375-381).  Kd must be a multiple of 128.
 *   q: u8 [2, max_rows, Kd];  sf: per (block of B sorted rows, 128-wide k-block) two 512-byte chunks. */
int b200moe_quant_rows_e4m3(const void* src_bf16, int32_t src_mode, const uint32_t* sorted_ids,
                            const int32_t* num_valid_ids, int32_t T, int32_t K, int32_t Kd, int32_t B,
                            int64_t max_rows, void* q, void* sf, void* stream);

/* The reference's own FP8 activation format (act_quant B200MOE_ACTQ_1X128): one e4m3 value per element with an
 * fp32 scale = amax / 448 per row and 128 channels (1.0 for an all-zero block); stands where the reference calls
 * aiter's per_1x128 quantiser with transpose_scale (src/contrib/fused_moe.py:276-281,375-381,449-456).
 *   q: u8 [max_rows, Kd];  sf: f32 [max_rows / B][Kd / 128][B] -- the B token scales of one sorted block and
 *   k-block are contiguous (the reference's transposed scale layout, per block). */
int b200moe_quant_rows_fp8_1x128(const void* src_bf16, int32_t src_mode, const uint32_t* sorted_ids,
                                 const int32_t* num_valid_ids, int32_t T, int32_t K, int32_t Kd, int32_t B,
                                 int64_t max_rows, void* q, void* sf, void* stream);

/* Gate-up grouped GEMM + activation: replaces moe_2stage_splitk(with_silu=True) /
 * moe_gemm_mxfp4(gate_up=True) (src/contrib/moe.py:362-702, src/contrib/moe_gemm_mxfp4.py:972-1290).
 * Consumes the quantised rows in workspace (xq), the canonical packed w1 [E,2I,H/2], its prepared
 * scale image and the sort arrays.
 *   With weight_format B200MOE_W_FP8_128 (replaces moe_gemm_8wave_g1u1, src/contrib/moe_gemm_8wave.py:131-765):
 *   w1_q is e4m3 [E,2I,H] and w1_scale_prepared is the raw fp32 [E, 2I/128, H/128] scale tensor.
 *   bias1 : NULL or fp32 [E, 2I] (gate then up), added to the bf16-rounded products before the activation
 *           (the aiter argument of that name, src/contrib/fused_moe.py:151; the reference asserts it absent).
 *   With weight_format B200MOE_W_BF16 (replaces moe_2stage_splitk on bf16 weights, src/contrib/moe.py:362-702):
 *   w1_q is bf16 [E,2I,H], w1_scale_prepared is ignored, h_out must be NULL.
 *   h_out != NULL : bf16 [T, K, I] scattered by (token,k) like the reference (moe.py:651-655)
 *   h_out == NULL : the result is re-quantised (bf16 weights: stored as bf16) in sorted-row order into
 *                   workspace hq for b200moe_down (fused path). */
int b200moe_gateup(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                   const void* w1_q, const void* w1_scale_prepared, const float* bias1, void* h_out,
                   void* stream);

/* Down grouped GEMM: replaces moe_2stage_splitk(with_silu=False) / moe_gemm_mxfp4(gate_up=False)
 * (src/contrib/moe.py:703-787, src/contrib/moe_gemm_mxfp4.py:1291-1398).  Reads workspace hq.
 *   bias2 : NULL or fp32 [E, H].
 *   combine_mode GATHER: writes bf16 rows in sorted order to workspace out2 (y_bf16 is ignored; follow with
 *     b200moe_combine).
 *   combine_mode FUSED: y_bf16 [T, H] must hold zeros; every row of the result is multiplied by its routing
 *     weight (workspace sorted_w; 1 with doweight_stage1) and added into it. */
int b200moe_down(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                 const void* w2_q, const void* w2_scale_prepared, const float* bias2, void* y_bf16,
                 void* stream);

/* Weighted combine back to token order: y[t] = sum_k w[t,k] * out2[loc[t,k]] accumulated in bf16
 * in ascending expert order, the order of the reference's torch oracle
 * (tests/contrib/moe/test_moe.py:107-117); replaces moe_gemm_final_reduce_bf16
 * (src/contrib/moe_gemm_mxfp4.py:199-282) / stage2_out.sum(dim=1) (src/contrib/fused_moe.py:565).
 * With doweight_stage1 the weights are not applied again. */
int b200moe_combine(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                    const float* topk_weight, void* y_bf16, void* stream);

/* Whole layer.  Replaces the body of pyhip.contrib.fused_moe.fused_moe (src/contrib/fused_moe.py:268-576).
 *   large batches: sort_align -> quant_rows(x) -> gateup (fused re-quantisation) -> down [-> combine]
 *   at most 256 (token, expert) pairs: sort/align and the input quantiser are ONE launch (every CTA repeats
 *   the small sort in shared memory; with T = 1 this is the reference's batch-1 shortcut, src/contrib/moe.py:41-188),
 *   so a decode step with combine_mode FUSED is three launches. */
int b200moe_forward(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                    const void* x_bf16, const int32_t* topk_ids, const float* topk_weight,
                    const int32_t* expert_mask, const void* w1_q, const void* w1_scale_prepared,
                    const void* w2_q, const void* w2_scale_prepared, void* y_bf16, void* stream);

/* Whole layer with a device-side token count (see b200moe_sort_align_dyn); output rows of tokens at and
 * beyond *num_local_tokens are zero. */
int b200moe_forward_dyn(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                        const void* x_bf16, const int32_t* topk_ids, const float* topk_weight,
                        const int32_t* expert_mask, const int32_t* num_local_tokens, const void* w1_q,
                        const void* w1_scale_prepared, const void* w2_q, const void* w2_scale_prepared,
                        void* y_bf16, void* stream);

/* Whole layer with every optional tensor of the aiter-shaped signature (src/contrib/fused_moe.py:128-155):
 * expert_mask, num_local_tokens, bias1, bias2 may be NULL. */
typedef struct b200moe_io {
  const void* x_bf16;              /* [T, H] */
  const int32_t* topk_ids;         /* [T, K] */
  const float* topk_weight;        /* [T, K] */
  const int32_t* expert_mask;      /* [E_route] or NULL */
  const int32_t* num_local_tokens; /* device scalar or NULL */
  const void* w1_q;
  const void* w1_scale_prepared;
  const void* w2_q;
  const void* w2_scale_prepared;
  const float* bias1;              /* [E, 2I] or NULL */
  const float* bias2;              /* [E, H] or NULL */
  void* y_bf16;                    /* [T, H] */
} b200moe_io;
int b200moe_forward_ex(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                       const b200moe_io* io, void* stream);

/* ONE token through the MXFP4 layer: replaces moe_gemm_batch1 (src/contrib/moe.py:41-188), the reference's batch-1
 * fast path that takes its experts straight from topk_ids with no sort (src/contrib/moe.py:79-84).  Two launches
 * (gate-up + activation; down + the weighted sum over the token's K experts in ascending expert order with the
 * oracle's bf16 roundings, tests/contrib/moe/test_moe.py:107-117), no workspace, no activation quantiser: the
 * products are formed from the bf16 input itself with fp32 block accumulation, and the result is bitwise
 * reproducible.  shape.T must be 1, shape.K <= 8, weight_format MXFP4; act_terms / combine_mode / B are not used.
 *   w1_scale / w2_scale : the CANONICAL E8M0 tensors [E, 2I, H/32] / [E, H, I/32] (not the prepared images)
 *   expert_mask, num_local_tokens, bias1, bias2 : as in b200moe_forward_ex, or NULL
 *   scratch : b200moe_batch1_scratch_bytes(shape) bytes of device memory, 16-byte aligned (h [K, I] + K ids) */
int b200moe_batch1_scratch_bytes(const b200moe_shape* shape, int64_t* bytes);
int b200moe_forward_batch1(const b200moe_shape* shape, const void* x_bf16, const int32_t* topk_ids,
                           const float* topk_weight, const int32_t* expert_mask, const int32_t* num_local_tokens,
                           const void* w1_q, const void* w1_scale, const void* w2_q, const void* w2_scale,
                           const float* bias1, const float* bias2, void* scratch, void* y_bf16, void* stream);

/* Whole layer WITHOUT a caller-provided workspace.  No counterpart in the reference (pyhip's
 * wrapper lets torch allocate its intermediates on every call).  It exists for hosts that cannot
 * allocate device memory when the layer runs -- e.g. a serving process that gave all free HBM to
 * its cache pool at start-up, or a foreign-language host with no allocator binding.  The scratch
 * lives in a fixed array inside the library image: B200MOE_STATIC_SCRATCH_BYTES are held on every
 * GPU that loads the library, until it is unloaded.  A shape whose workspace layout
 * (b200moe_workspace_layout) is larger is refused with an argument error.  All calls on a device
 * share that array: calls whose GPU work may overlap must be serialised by the caller.  The first
 * call on each device performs a one-time address look-up and should be made outside stream
 * capture, with the stream's device current.  Same arguments and result as b200moe_forward otherwise;
 * allocates nothing. */
#define B200MOE_STATIC_SCRATCH_BYTES (48ll << 20)
int b200moe_forward_static(const b200moe_shape* shape, const void* x_bf16, const int32_t* topk_ids,
                           const float* topk_weight, const int32_t* expert_mask, const void* w1_q,
                           const void* w1_scale_prepared, const void* w2_q, const void* w2_scale_prepared,
                           void* y_bf16, void* stream);
/* The 16 device-side status words the latest b200moe_forward_static call with this shape left on the current
 * device, copied to host memory asynchronously on `stream` (synchronise before reading; the next call clears
 * them).  Word 0 != 0: a bounded wait inside a kernel gave up; word 2 != 0: an expert id outside the weight image.
 * No counterpart in the reference. */
int b200moe_static_status(const b200moe_shape* shape, int32_t* status_host16, void* stream);

/* Expert-parallel combine.  No counterpart in the reference, which has no dispatch/combine (expert
 * parallelism exists there only as the expert_mask input convention, src/contrib/fused_moe.py:134,210-212).
 * y[t,:] = sum over s in [0, slots) of rows[pos[t*slots + s], :] for pos >= 0, accumulated in fp32 in
 * ascending slot order (slot = owner rank = ascending expert range) and rounded to bf16 once.
 *   rows: bf16 [n, H] partial outputs returned by the owner ranks;  pos: i32 [T, slots], -1 = no row. */
int b200moe_gather_sum(const void* rows_bf16, const int32_t* pos, int32_t T, int32_t slots, int32_t H,
                       void* y_bf16, void* stream);

/* Expert-parallel dispatch plan in one launch.  No counterpart in the reference (see b200moe_gather_sum).
 * Rank d owns experts [d*experts_per_rank, (d+1)*experts_per_rank); a token travels once to every rank that
 * owns at least one of its K experts.
 *   pos    i32 [T, world]  position of the token in the rank-major send buffer (ascending rank, ascending
 *                          token within a rank), -1 where the rank owns none of its experts
 *   counts i32 [world]     tokens bound for each rank
 *   rows   i32 [T*world]   token at every send-buffer position; only [0, sum(counts)) is written
 * world <= 32.  Deterministic (no atomics). */
int b200moe_ep_plan(const int32_t* topk_ids, int32_t T, int32_t K, int32_t experts_per_rank, int32_t world,
                    int32_t* pos, int32_t* counts, int32_t* rows, void* stream);

/* Hardware known-answer probes used by the GPU test-suite and the benchmark (bounded waits).
 *   which = 1: TMA load of one 128-row x 256-element packed-FP4 tile (128-byte swizzle) from `in`
 *              (16384 bytes) -> `out` receives the 16384-byte shared-memory image.
 *   which = 2: 512 bytes `in` -> shared -> tcgen05.cp 32x128b.warpx4 -> tcgen05.ld;
 *              `out` receives u32 [128 lanes][4 columns].
 *   which = 4: whole-chip dense MMA rate: one CTA per SM issues `count` block-scaled MMAs of 128 x N x (64 for
 *              FP4, 32 for FP8) from resident shared-memory tiles; the caller times the launch with stream events.
 *              `in` = i32 {kind (0 = kind::mxf4, 1 = kind::mxf8f6f4 e4m3), N, count}; `out` = u32 [SM count][3]
 *              {issue cycles, cycles until complete, status}.
 *   which = 5: a bounded wait that is MADE to run out (a barrier nothing arrives on): `in` = i32 {limit in
 *              microseconds}; `out` = u32 {status word = 0xBEEF (the wait's id), 1 if the wait succeeded, microseconds
 *              waited}.  The kernel returns normally and the context stays usable.
 * status word: 0 = ok, non-zero = a bounded wait ran out. */
int b200moe_debug_probe(int which, const void* in, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
