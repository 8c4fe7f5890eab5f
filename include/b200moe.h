/* C ABI of libb200moe.so -- the sm_100a fused-MoE path behind pyhip's `fused_moe` call surface.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle (as void*),
 * enqueues work on that stream and returns without synchronising.  Return value: 0 = ok,
 * negative = argument error (nothing was launched), positive = CUDA error code.
 * b200moe_last_error() describes the last non-zero return of the calling thread.
 * The library owns no device memory: the caller provides every buffer, including the workspace.
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

#define B200MOE_VERSION 1

/* weight formats */
#define B200MOE_W_MXFP4 0 /* E2M1 pairs (low nibble = even element) + E8M0 scale per 32 along K */
#define B200MOE_W_FP8_128 1 /* e4m3 + fp32 scale per 128x128 block */
/* activation functions of the gate-up stage */
#define B200MOE_ACT_SILU 0   /* silu(gate) * up                        (test_moe.py:74-75) */
#define B200MOE_ACT_SWIGLU 1 /* clamped gate*sigmoid(1.702 gate)*(up+1) (test_moe.py:76-81) */

/* Shape of one MoE layer call.  B (rows per sorted block = token tile of the GEMMs) is 32, 64
 * or 128.  E is the number of experts whose weights are present (local experts under expert
 * parallelism); E_route is the size of the routing id space (E_route >= E; equal without a mask). */
typedef struct b200moe_shape {
  int32_t T, K, E, E_route, H, I, B;
  int32_t weight_format;
  int32_t activation;
  float swiglu_limit;
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
  int64_t off_xq_hi, off_xq_lo, off_xsf_hi, off_xsf_lo; /* quantised input rows, sorted order   */
  int64_t off_hq_hi, off_hq_lo, off_hsf_hi, off_hsf_lo; /* quantised gate-up output, same order */
  int64_t off_out2;          /* bf16 [Lmax, H]  down-projection rows in sorted order         */
} b200moe_workspace;

int b200moe_version(void);
const char* b200moe_last_error(void);

/* Fills *ws for `shape`.  Pure host arithmetic. */
int b200moe_workspace_layout(const b200moe_shape* shape, b200moe_workspace* ws);

/* Bytes of the prepared (device-layout) image of one weight tensor: which = 1 (w1, [E,2I,H]) or
 * 2 (w2, [E,H,I]); *data_bytes for the element image, *scale_bytes for the scale image. */
int b200moe_prepared_bytes(const b200moe_shape* shape, int which, int64_t* data_bytes, int64_t* scale_bytes);

/* One-off repack of canonical weights into the layout the GEMMs stream (K padded to 128 with
 * zero codes; scales regrouped into 128-row x 4-scale chunks in tensor-memory order).  Plays the
 * part of the reference's pre-shuffle (src/misc.py:114-128, tests/contrib/moe/test_moe.py:167-172).
 *   w_q   : u8  [E, R, Kd/2]   (R = 2I, Kd = H for which=1; R = H, Kd = I for which=2)
 *   w_s   : u8  [E, R, Kd/32]
 */
int b200moe_prepare_weights(const b200moe_shape* shape, int which, const void* w_q, const void* w_s,
                            void* out_data, void* out_scale, void* stream);

/* Token->expert sort/align: replaces aiter.moe_sorting as called at src/contrib/fused_moe.py:283,
 * 301-305 and 368-372 (contract: fused_moe.py:56-100; ck_tile reference_moe_sorting.hpp:14-117).
 * Deterministic; only [0, num_valid[0]) of the outputs is defined.  expert_mask may be NULL.
 * loc may be NULL. */
int b200moe_sort_align(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                       int32_t E_route, int32_t B, const int32_t* expert_mask, uint32_t* sorted_ids,
                       float* sorted_weights, int32_t* sorted_expert_ids, int32_t* num_valid_ids,
                       int32_t* loc, void* stream);

/* Quantise bf16 rows into the two-term e4m3 + E8M0/32 operand format, gathered into sorted-row
 * order (stands where the reference calls aiter's per_1x32 activation quantiser followed by
 * moe_mxfp4_sort, tests/contrib/moe/test_moe.py:665-679).
 *   src_mode 0: src is [T, Kd], row = token.   src_mode 1: src is [T, K, Kd], row = token*K + k.
 *   q_*: e4m3 [max_rows, Kd padded to 128]; sf_*: one 512-byte scale chunk per (block of B sorted
 *   rows, 128-wide k-block), row r of the block and scale j at byte (r%32)*16 + (r/32)*4 + j. */
int b200moe_quant_rows(const void* src_bf16, int32_t src_mode, const uint32_t* sorted_ids,
                       const int32_t* num_valid_ids, int32_t T, int32_t K, int32_t Kd, int32_t B,
                       int64_t max_rows, void* q_hi, void* q_lo, void* sf_hi, void* sf_lo, void* stream);

/* Gate-up grouped GEMM + activation: replaces moe_2stage_splitk(with_silu=True) /
 * moe_gemm_mxfp4(gate_up=True) (src/contrib/moe.py:362-702, src/contrib/moe_gemm_mxfp4.py:972-1290).
 * Consumes the quantised rows in workspace (xq_*), the prepared w1 image and the sort arrays.
 *   h_out != NULL : bf16 [T, K, I] scattered by (token,k) like the reference (moe.py:651-655)
 *   h_out == NULL : the result is re-quantised in sorted-row order into workspace hq_* for
 *                   b200moe_down (fused path). */
int b200moe_gateup(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                   const void* w1_data, const void* w1_scale, void* h_out, void* stream);

/* Down grouped GEMM: replaces moe_2stage_splitk(with_silu=False) / moe_gemm_mxfp4(gate_up=False)
 * (src/contrib/moe.py:703-787, src/contrib/moe_gemm_mxfp4.py:1291-1398).  Reads workspace hq_*,
 * writes bf16 rows in sorted order to workspace out2. */
int b200moe_down(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                 const void* w2_data, const void* w2_scale, void* stream);

/* Weighted combine back to token order: y[t] = sum_k w[t,k] * out2[loc[t,k]] accumulated in bf16
 * in ascending expert order, the order of the reference's torch oracle
 * (tests/contrib/moe/test_moe.py:107-117); replaces moe_gemm_final_reduce_bf16
 * (src/contrib/moe_gemm_mxfp4.py:199-282) / stage2_out.sum(dim=1) (src/contrib/fused_moe.py:565). */
int b200moe_combine(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                    const float* topk_weight, void* y_bf16, void* stream);

/* Whole layer: sort_align -> quant_rows(x) -> gateup (fused re-quantisation) -> down -> combine.
 * Replaces the body of pyhip.contrib.fused_moe.fused_moe (src/contrib/fused_moe.py:268-576). */
int b200moe_forward(const b200moe_shape* shape, const b200moe_workspace* ws, void* workspace,
                    const void* x_bf16, const int32_t* topk_ids, const float* topk_weight,
                    const int32_t* expert_mask, const void* w1_data, const void* w1_scale,
                    const void* w2_data, const void* w2_scale, void* y_bf16, void* stream);

/* Hardware known-answer probes used by the GPU test-suite (tiny, single CTA, bounded waits).
 *   which = 1: TMA load of one 128x128 FP4 tile (16-byte-aligned unpacking, 128-byte swizzle)
 *              from `in` (8192 bytes) -> `out` receives the 16384-byte shared-memory image.
 *   which = 2: 512 bytes `in` -> shared -> tcgen05.cp 32x128b.warpx4 -> tcgen05.ld;
 *              `out` receives u32 [128 lanes][4 columns].
 *   which = 3: tensor-core issue-rate measurement; `in` = i32 {kind (0 mxf8f6f4, 1 mxf4), N,
 *              count, accumulators}; `out` = u32 {issue cycles, cycles until complete, status}.
 * out[last] status word: 0 = ok, non-zero = a bounded wait ran out. */
int b200moe_debug_probe(int which, const void* in, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
