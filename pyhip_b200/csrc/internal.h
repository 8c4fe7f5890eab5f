// Declarations shared by the translation units of libb200moe.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200moe.h"

namespace b200moe {

int set_error(int code, const char* fmt, ...);

#define B200_CHECK_ARG(cond, ...)                      \
  do {                                                 \
    if (!(cond)) return b200moe::set_error(-1, __VA_ARGS__); \
  } while (0)

#define B200_CHECK_CUDA(expr)                                                                  \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return b200moe::set_error((int)_e, "%s failed: %s", #expr, cudaGetErrorString(_e));      \
  } while (0)

static inline int64_t round_up64(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// scale-factor chunk: 128 rows x 4 scales in tensor-memory order
constexpr int kSfChunk = 512;
__host__ __device__ static inline int sf_chunk_offset(int row_in_128, int j) {
  return (row_in_128 & 31) * 16 + (row_in_128 >> 5) * 4 + j;
}
// Activation operand layout, shared by the quantisers and the GEMM that consumes their output.
// NT terms per row.  "Merged": the terms of a block are stacked along the MMA's N (one
// instruction, N = NT*B) -- possible when that fits an instruction (<= 256) and two accumulator
// buffers of `parts` tiles fit tensor memory; otherwise every term is its own instruction.
// Scales: per (sorted block, 128-wide k-block) a group of 512-byte chunks; term t, block-local
// row r sit at virtual row v = t*TS + r (TS = B when merged, 128 otherwise): chunk v/128.
constexpr int kAccColsLimit = 416;   // TMEM columns left for accumulators (the rest holds scales)
constexpr int kKPad = 256;           // activation K is padded to the K extent of one pipeline stage
__host__ __device__ static inline bool act_merged(int B, int NT, int parts) {
  return NT * B <= 256 && 2 * parts * NT * B <= kAccColsLimit;
}
__host__ __device__ static inline int act_term_stride(int B, int NT, int parts) {
  return act_merged(B, NT, parts) ? B : 128;
}
__host__ __device__ static inline int act_sf_chunks(int NT, int TS) { return (NT * TS + 127) / 128; }
__host__ __device__ static inline int64_t act_sf_index(int64_t block, int kb, int KB, int B, int NT, int TS,
                                                       int term, int r, int j) {
  (void)B;
  const int v = term * TS + r;
  return ((block * KB + kb) * act_sf_chunks(NT, TS) + (v >> 7)) * kSfChunk + sf_chunk_offset(v & 127, j);
}

// launchers (moe_aux.cu)
int launch_sort_align(const int32_t* ids, const float* w, int T, int K, int E, int B, const int32_t* mask,
                      uint32_t* sorted_ids, float* sorted_w, int32_t* sorted_e, int32_t* num_valid,
                      int32_t* loc, const int32_t* num_local, cudaStream_t st);
constexpr int64_t kSortWideMinPairs = 8192;   // (token, expert) pairs from which the sort is spread over several CTAs
// the same over several CTAs with caller scratch of sort_scratch_bytes(E) bytes (4-byte aligned)
int64_t sort_scratch_bytes(int E);
int launch_sort_align_wide(const int32_t* ids, const float* w, int T, int K, int E, int B, const int32_t* mask,
                           uint32_t* sorted_ids, float* sorted_w, int32_t* sorted_e, int32_t* num_valid,
                           int32_t* loc, const int32_t* num_local, void* scratch, cudaStream_t st);
int launch_route_topk(const float* logits, int T, int E, int K, int scoring, int renorm, int32_t* ids, float* weights,
                      cudaStream_t st);
// zero_ptr / zero_bytes: an optional region the same launch clears (the output of the fused combine).
// loc (with src_mode 0): the sort's [T, K] table of sorted positions; when given, every token is quantised once and
// stored at its K rows instead of once per sorted row.
int launch_quant_rows(const void* src, int src_mode, const uint32_t* sorted_ids, const int32_t* num_valid,
                      int T, int K, int Kd, int B, int NT, int64_t max_rows, void* q, void* sf, void* zero_ptr,
                      int64_t zero_bytes, const int32_t* loc, cudaStream_t st);
// sort/align + input quantiser in one launch for decode-sized batches
// (fmt 0: packed-FP4 terms, 1: two e4m3 terms, 2: e4m3 with fp32 scales per 1x128)
bool sort_quant_small_ok(int T, int K, int E);
int launch_sort_quant_small(int fmt, const void* x, const int32_t* ids, const float* w, int T, int K, int E, int B,
                            const int32_t* mask, const int32_t* num_local, uint32_t* sorted_ids, float* sorted_w,
                            int32_t* sorted_e, int32_t* num_valid, int32_t* loc, int Kd, int NT, int64_t max_rows,
                            void* q, void* sf, void* zero_ptr, int64_t zero_bytes, cudaStream_t st);
int launch_ep_plan(const int32_t* ids, int T, int K, int epr, int W, int32_t* pos, int32_t* counts, int32_t* rows,
                   cudaStream_t st);
int launch_gather_sum(const void* rows, const int32_t* pos, void* y, int T, int S, int H, cudaStream_t st);
int launch_combine(const void* out2, const int32_t* loc, const float* topk_w, void* y, int T, int K, int H,
                   cudaStream_t st);
int launch_repack_scales(const void* w_s, void* out, int E, bool gateup, int rows, int Kd, cudaStream_t st);

// grouped GEMM (moe_gemm_sm100.cu)
struct GemmArgs {
  bool gateup;
  int N;               // token tile (= sort block B)
  int rows;            // weight rows per part (I for gate-up, H for down)
  int Kd;              // reduction length (H for gate-up, I for down)
  int E;               // experts in the weight image
  int topk, T;
  int activation;
  float swiglu_limit;
  int64_t max_rows;
  int NT;              // activation terms
  const void* w_data;  // canonical packed FP4 [E, parts*rows, Kd/2], used in place
  const void* w_scale; // [E, MT, KB, 2, 512]
  const void* a_q;     // [NT, max_rows, KP/2] packed FP4 terms
  const void* asf;     // [max_rows/N, KB, chunks, 512]
  const uint32_t* sorted_ids;
  const int32_t* sorted_e;
  const int32_t* num_valid;
  int32_t* status;
  // outputs
  void* h_out;         // gate-up: bf16 [T, topk, I] or null
  void* oq; void* osf;   // gate-up fused re-quantisation ([NT, max_rows, out_kp/2] + scale chunks)
  int out_kp;          // row pitch of oq_* (I padded to 128) and chunk count per row block
  void* out2;          // down: bf16 [max_rows, H]
  void* gstage;        // gate-up: scratch for per-CTA staging tiles in global memory (may be null)
  int64_t gstage_bytes;
  const float* sorted_w;   // routing weight per sorted row (weight_stage1 needs it; with y, null means weight 1)
  const float* bias;       // fp32 per-expert bias: gate-up [E, 2*rows], down [E, rows]; or null
  void* y;                 // down: zeroed bf16 [T, rows]; non-null selects the fused weighted scatter-add epilogue
  int weight_stage1;       // gate-up: apply the routing weight to h
  int act_quant;           // FP8 kernel: 0 = two e4m3 terms with E8M0 scales, 1 = one e4m3 term with fp32 scales per 1x128
  int w_row_scaled;        // FP8 kernel: w_scale holds one fp32 scale per weight row [E, parts*rows] (not per 128x128 block)
  int pair_mode;           // MXFP4 kernel: CTA pairs (cta_group::2): 0 = in the compute-bound regime, 1 = never, 2 = wherever possible
};
int launch_grouped_gemm(const GemmArgs& a, cudaStream_t st);
// FP8 128x128-block variant (moe_gemm_fp8_sm100.cu): w_data = e4m3 bytes [E, parts*rows, Kd], w_scale = fp32
// [E, parts*rows/128, Kd/128] (used in place), a_q = two e4m3 terms [2, max_rows, Kd], NT ignored
int launch_grouped_gemm_fp8(const GemmArgs& a, cudaStream_t st);
// bf16-weight variant (moe_gemm_bf16_sm100.cu): w_data = bf16 [E, parts*rows, Kd], a_q = bf16 token rows
// [max_rows, Kd] in sorted order; gate-up writes h as bf16 [max_rows, rows] to `oq`; scales and NT are ignored
int launch_grouped_gemm_bf16(const GemmArgs& a, cudaStream_t st);
// the layer input copied (bf16, no quantisation) to each token's sorted rows; also clears zero_ptr
int launch_gather_rows_bf16(const void* src, const int32_t* loc, int T, int K, int Kd, int B, int64_t max_rows, void* q,
                            void* zero_ptr, int64_t zero_bytes, cudaStream_t st);
int launch_quant_rows_e4m3(const void* src, int src_mode, const uint32_t* sorted_ids, const int32_t* num_valid,
                           int T, int K, int Kd, int B, int64_t max_rows, void* q, void* sf, void* zero_ptr,
                           int64_t zero_bytes, const int32_t* loc, cudaStream_t st);
int launch_quant_rows_fp8_1x128(const void* src, int src_mode, const uint32_t* sorted_ids, const int32_t* num_valid,
                                int T, int K, int Kd, int B, int64_t max_rows, void* q, void* sf, void* zero_ptr,
                                int64_t zero_bytes, const int32_t* loc, cudaStream_t st);
int encode_map_sw(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const cuuint64_t* dims,
                  const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle,
                  CUtensorMapL2promotion promo, const char* what);
int device_sm_count();

// Launch `kernel` so that it may begin (prologue only: every kernel of this library calls
// grid_dep_wait() before it touches global memory) while the previous kernel in the stream drains.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                          int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.numAttrs = 1;
  if (cluster_x > 1) {          // thread-block clusters of cluster_x CTAs along x (grid.x is a multiple of it)
    at[1].id = cudaLaunchAttributeClusterDimension;
    at[1].val.clusterDim.x = (unsigned)cluster_x;
    at[1].val.clusterDim.y = 1;
    at[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = at;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args&&... args) {
  return launch_chained_cluster(kernel, grid, block, smem, st, 1, static_cast<Args&&>(args)...);
}
// batch-1 path (moe_batch1.cu): one token, MXFP4 weights with their canonical E8M0 scales, no sort and no quantiser
int64_t batch1_scratch_bytes(int K, int I);
int launch_forward_batch1(const void* x, const int32_t* ids, const float* tw, const int32_t* mask, const int32_t* num_local,
                          const void* w1, const void* s1, const void* w2, const void* s2, const float* bias1,
                          const float* bias2, void* scratch, void* y, int H, int I, int K, int E, int E_route,
                          int activation, float swiglu_limit, int stage1, cudaStream_t st);
int run_debug_probe(int which, const void* in, void* out, cudaStream_t st);

}  // namespace b200moe
