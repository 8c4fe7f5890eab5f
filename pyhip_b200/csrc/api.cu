// extern "C" surface of libb200moe.so: argument validation, workspace arithmetic, weight
// preparation and the stage-by-stage / whole-layer entry points.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "internal.h"

namespace b200moe {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static bool is_fp8(const b200moe_shape* s) {
  return s->weight_format == B200MOE_W_FP8_128 || s->weight_format == B200MOE_W_FP8_ROW;
}
static bool is_bf16(const b200moe_shape* s) { return s->weight_format == B200MOE_W_BF16; }

static int check_shape(const b200moe_shape* s) {
  B200_CHECK_ARG(s != nullptr, "shape is NULL");
  B200_CHECK_ARG(s->T >= 0 && s->T < (1 << 24), "T=%d outside [0, 2^24)", s->T);
  B200_CHECK_ARG(s->K >= 1 && s->K <= 32, "K=%d outside [1,32]", s->K);
  B200_CHECK_ARG(s->E >= 1 && s->E_route >= s->E && s->E_route <= 1024, "E=%d / E_route=%d invalid", s->E,
                 s->E_route);
  B200_CHECK_ARG(s->B >= 16 && s->B <= 128 && s->B % 16 == 0, "B=%d is not a multiple of 16 in [16,128]", s->B);
  B200_CHECK_ARG(s->H >= 32 && s->H % 32 == 0, "H=%d must be a positive multiple of 32", s->H);
  B200_CHECK_ARG(s->I >= 32 && s->I % 32 == 0, "I=%d must be a positive multiple of 32", s->I);
  B200_CHECK_ARG(s->H % 8 == 0, "H must be a multiple of 8");
  B200_CHECK_ARG(s->weight_format == B200MOE_W_MXFP4 || s->weight_format == B200MOE_W_FP8_128 ||
                 s->weight_format == B200MOE_W_FP8_ROW || s->weight_format == B200MOE_W_BF16,
                 "weight_format %d unknown", s->weight_format);
  if (is_fp8(s)) {
    B200_CHECK_ARG(s->H % 128 == 0 && s->I % 128 == 0, "FP8 weights need H and I to be multiples of 128");
    B200_CHECK_ARG(s->B <= 96, "FP8 weights: B=%d exceeds 96", s->B);
  }
  B200_CHECK_ARG(s->activation == B200MOE_ACT_SILU || s->activation == B200MOE_ACT_SWIGLU,
                 "activation %d unknown", s->activation);
  B200_CHECK_ARG(s->act_terms >= 0 && s->act_terms <= 4, "act_terms=%d not in [0,4]", s->act_terms);
  B200_CHECK_ARG(s->combine_mode == B200MOE_COMBINE_GATHER || s->combine_mode == B200MOE_COMBINE_FUSED,
                 "combine_mode %d unknown", s->combine_mode);
  B200_CHECK_ARG(s->act_quant == B200MOE_ACTQ_TERMS || s->act_quant == B200MOE_ACTQ_1X128, "act_quant %d unknown",
                 s->act_quant);
  B200_CHECK_ARG(s->act_quant == B200MOE_ACTQ_TERMS || s->weight_format == B200MOE_W_FP8_128,
                 "act_quant 1x128 belongs to the FP8 128x128 weight format (MXFP4 weights take act_terms)");
  B200_CHECK_ARG(s->doweight_stage1 == 0 || s->doweight_stage1 == 1, "doweight_stage1=%d must be 0 or 1",
                 s->doweight_stage1);
  B200_CHECK_ARG(s->cta_pairs >= 0 && s->cta_pairs <= 2, "cta_pairs=%d must be 0 (auto), 1 (off) or 2 (on)", s->cta_pairs);
  return 0;
}

static int64_t kp_of(int k) { return round_up64(k, kKPad); }
static int terms_of(const b200moe_shape* s) { return s->act_terms == 0 ? 3 : s->act_terms; }

}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_version(void) { return B200MOE_VERSION; }

const char* b200moe_last_error(void) { return g_err; }

int b200moe_workspace_layout(const b200moe_shape* s, b200moe_workspace* ws) {
  if (int rc = check_shape(s)) return rc;
  B200_CHECK_ARG(ws != nullptr, "workspace descriptor is NULL");
  const bool fp8w = is_fp8(s);
  const int NT = fp8w ? 2 : terms_of(s);
  const int64_t P = (int64_t)s->T * s->K;
  const int64_t nblk = (P + (int64_t)s->E_route * (s->B - 1) + s->B - 1) / s->B;
  const int64_t L = std::max<int64_t>(nblk, 1) * s->B;
  const int64_t nb = L / s->B;   // one scale chunk group per sorted block and k-block
  const int64_t HP = kp_of(s->H), IP = kp_of(s->I);
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    int64_t o = off;
    off += round_up64(std::max<int64_t>(bytes, 16), 1024);
    return o;
  };
  memset(ws, 0, sizeof(*ws));
  ws->max_rows = L;
  ws->off_sorted_ids = take(L * 4);
  ws->off_sorted_w = take(L * 4);
  ws->off_sorted_e = take(L / s->B * 4);
  ws->off_num_valid = take(8);
  ws->off_loc = take(std::max<int64_t>(P, 1) * 4);
  ws->off_status = take(64);
  if (is_bf16(s)) {   // bf16 rows in sorted order, no scales
    ws->off_xq = take(L * s->H * 2);
    ws->off_xsf = take(16);
    ws->off_hq = take(L * s->I * 2);
    ws->off_hsf = take(16);
  } else if (fp8w) {   // two e4m3 terms, one byte per element, one scale chunk per term
    ws->off_xq = take(2 * L * s->H);
    ws->off_xsf = take(nb * (s->H / 128) * 2 * kSfChunk);
    ws->off_hq = take(2 * L * s->I);
    ws->off_hsf = take(nb * (s->I / 128) * 2 * kSfChunk);
  } else {
    ws->off_xq = take(NT * L * (HP / 2));
    ws->off_xsf = take(nb * (HP / 128) * act_sf_chunks(NT, act_term_stride(s->B, NT, 2)) * kSfChunk);
    ws->off_hq = take(NT * L * (IP / 2));
    ws->off_hsf = take(nb * (IP / 128) * act_sf_chunks(NT, act_term_stride(s->B, NT, 2)) * kSfChunk);
  }
  ws->off_out2 = take(L * s->H * 2);
  ws->off_sort_scratch = take(P >= kSortWideMinPairs ? sort_scratch_bytes(s->E_route) : 16);
  ws->total_bytes = off;
  return 0;
}

int b200moe_prepared_scale_bytes(const b200moe_shape* s, int which, int64_t* scale_bytes) {
  if (int rc = check_shape(s)) return rc;
  B200_CHECK_ARG(which == 1 || which == 2, "which=%d must be 1 or 2", which);
  B200_CHECK_ARG(scale_bytes != nullptr, "scale_bytes is NULL");
  B200_CHECK_ARG(s->weight_format == B200MOE_W_MXFP4, "FP8 128x128 scales are consumed in place: nothing to prepare");
  // two 128-row tiles per chunk pair: (gate, up) of one feature tile, or two consecutive down tiles
  const int groups = which == 1 ? (s->I + 127) / 128 : (s->H + 255) / 256;
  const int Kd = which == 1 ? s->H : s->I;
  *scale_bytes = (int64_t)s->E * groups * (kp_of(Kd) / 128) * 2 * kSfChunk;
  return 0;
}

int b200moe_prepare_scales(const b200moe_shape* s, int which, const void* w_s, void* out_scale, void* stream) {
  if (int rc = check_shape(s)) return rc;
  B200_CHECK_ARG(which == 1 || which == 2, "which=%d must be 1 or 2", which);
  B200_CHECK_ARG(w_s && out_scale, "prepare_scales: NULL pointer");
  B200_CHECK_ARG(s->weight_format == B200MOE_W_MXFP4, "FP8 128x128 scales are consumed in place: nothing to prepare");
  B200_CHECK_ARG(((uintptr_t)out_scale & 15) == 0, "prepare_scales: output must be 16-byte aligned");
  const int Kd = which == 1 ? s->H : s->I;
  return launch_repack_scales(w_s, out_scale, s->E, which == 1, which == 1 ? s->I : s->H, Kd, (cudaStream_t)stream);
}

static int sort_align_impl(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K, int32_t E_route,
                           int32_t B, const int32_t* expert_mask, const int32_t* num_local_tokens, uint32_t* sorted_ids,
                           float* sorted_weights, int32_t* sorted_expert_ids, int32_t* num_valid_ids, int32_t* loc,
                           void* scratch, int64_t scratch_bytes, void* stream) {
  B200_CHECK_ARG(T >= 0 && T < (1 << 24) && K >= 1 && K <= 255, "sort_align: T=%d K=%d out of range", T, K);
  B200_CHECK_ARG(B >= 1, "sort_align: B=%d", B);
  B200_CHECK_ARG(sorted_ids && sorted_weights && sorted_expert_ids && num_valid_ids, "sort_align: NULL output");
  B200_CHECK_ARG(T == 0 || (topk_ids && topk_weight), "sort_align: NULL input");
  // large batches: several CTAs over caller scratch (one CTA's store path limits the single-CTA kernel)
  if ((int64_t)T * K >= kSortWideMinPairs && scratch != nullptr && scratch_bytes >= sort_scratch_bytes(E_route) &&
      ((uintptr_t)scratch & 3) == 0)
    return launch_sort_align_wide(topk_ids, topk_weight, T, K, E_route, B, expert_mask, sorted_ids, sorted_weights,
                                  sorted_expert_ids, num_valid_ids, loc, num_local_tokens, scratch,
                                  (cudaStream_t)stream);
  return launch_sort_align(topk_ids, topk_weight, T, K, E_route, B, expert_mask, sorted_ids, sorted_weights,
                           sorted_expert_ids, num_valid_ids, loc, num_local_tokens, (cudaStream_t)stream);
}

int b200moe_sort_align(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K, int32_t E_route,
                       int32_t B, const int32_t* expert_mask, uint32_t* sorted_ids, float* sorted_weights,
                       int32_t* sorted_expert_ids, int32_t* num_valid_ids, int32_t* loc, void* stream) {
  return sort_align_impl(topk_ids, topk_weight, T, K, E_route, B, expert_mask, nullptr, sorted_ids, sorted_weights,
                         sorted_expert_ids, num_valid_ids, loc, nullptr, 0, stream);
}

int b200moe_sort_align_dyn(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K, int32_t E_route,
                           int32_t B, const int32_t* expert_mask, const int32_t* num_local_tokens,
                           uint32_t* sorted_ids, float* sorted_weights, int32_t* sorted_expert_ids,
                           int32_t* num_valid_ids, int32_t* loc, void* stream) {
  return sort_align_impl(topk_ids, topk_weight, T, K, E_route, B, expert_mask, num_local_tokens, sorted_ids,
                         sorted_weights, sorted_expert_ids, num_valid_ids, loc, nullptr, 0, stream);
}

int b200moe_quant_rows_fp8_1x128(const void* src_bf16, int32_t src_mode, const uint32_t* sorted_ids,
                                 const int32_t* num_valid_ids, int32_t T, int32_t K, int32_t Kd, int32_t B,
                                 int64_t max_rows, void* q, void* sf, void* stream) {
  B200_CHECK_ARG(src_mode == 0 || src_mode == 1, "quant_rows: src_mode=%d", src_mode);
  B200_CHECK_ARG(sorted_ids && num_valid_ids && q && sf, "quant_rows: NULL pointer");
  B200_CHECK_ARG(T == 0 || src_bf16, "quant_rows: NULL source");
  B200_CHECK_ARG(((uintptr_t)src_bf16 & 15) == 0 && ((uintptr_t)q & 15) == 0,
                 "quant_rows: source and destination must be 16-byte aligned");
  return launch_quant_rows_fp8_1x128(src_bf16, src_mode, sorted_ids, num_valid_ids, T, K, Kd, B, max_rows, q, sf,
                                     nullptr, 0, nullptr, (cudaStream_t)stream);
}

int b200moe_sort_scratch_bytes(int32_t E_route, int64_t* bytes) {
  B200_CHECK_ARG(E_route >= 1 && bytes != nullptr, "sort_scratch_bytes: bad argument");
  *bytes = sort_scratch_bytes(E_route);
  return 0;
}

int b200moe_sort_align_ws(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K, int32_t E_route,
                          int32_t B, const int32_t* expert_mask, const int32_t* num_local_tokens,
                          uint32_t* sorted_ids, float* sorted_weights, int32_t* sorted_expert_ids,
                          int32_t* num_valid_ids, int32_t* loc, void* scratch, int64_t scratch_bytes, void* stream) {
  return sort_align_impl(topk_ids, topk_weight, T, K, E_route, B, expert_mask, num_local_tokens, sorted_ids,
                         sorted_weights, sorted_expert_ids, num_valid_ids, loc, scratch, scratch_bytes, stream);
}

int b200moe_quant_rows(const void* src_bf16, int32_t src_mode, const uint32_t* sorted_ids,
                       const int32_t* num_valid_ids, int32_t T, int32_t K, int32_t Kd, int32_t B, int32_t terms,
                       int64_t max_rows, void* q, void* sf, void* stream) {
  B200_CHECK_ARG(src_mode == 0 || src_mode == 1, "quant_rows: src_mode=%d", src_mode);
  B200_CHECK_ARG(sorted_ids && num_valid_ids && q && sf, "quant_rows: NULL pointer");
  B200_CHECK_ARG(T == 0 || src_bf16, "quant_rows: NULL source");
  B200_CHECK_ARG(((uintptr_t)src_bf16 & 15) == 0 && ((uintptr_t)q & 15) == 0,
                 "quant_rows: source and destination must be 16-byte aligned");
  return launch_quant_rows(src_bf16, src_mode, sorted_ids, num_valid_ids, T, K, Kd, B, terms, max_rows, q, sf,
                           nullptr, 0, nullptr, (cudaStream_t)stream);
}

int b200moe_quant_rows_e4m3(const void* src_bf16, int32_t src_mode, const uint32_t* sorted_ids,
                            const int32_t* num_valid_ids, int32_t T, int32_t K, int32_t Kd, int32_t B,
                            int64_t max_rows, void* q, void* sf, void* stream) {
  B200_CHECK_ARG(src_mode == 0 || src_mode == 1, "quant_rows: src_mode=%d", src_mode);
  B200_CHECK_ARG(sorted_ids && num_valid_ids && q && sf, "quant_rows: NULL pointer");
  B200_CHECK_ARG(T == 0 || src_bf16, "quant_rows: NULL source");
  B200_CHECK_ARG(((uintptr_t)src_bf16 & 15) == 0 && ((uintptr_t)q & 15) == 0,
                 "quant_rows: source and destination must be 16-byte aligned");
  return launch_quant_rows_e4m3(src_bf16, src_mode, sorted_ids, num_valid_ids, T, K, Kd, B, max_rows, q, sf,
                                nullptr, 0, nullptr, (cudaStream_t)stream);
}

static void fill_common(GemmArgs& g, const b200moe_shape* s, const b200moe_workspace* ws, uint8_t* base) {
  g.N = s->B;
  g.act_quant = s->act_quant;
  g.pair_mode = s->cta_pairs;
  g.w_row_scaled = s->weight_format == B200MOE_W_FP8_ROW;
  g.NT = terms_of(s);
  g.E = s->E;
  g.topk = s->K;
  g.T = s->T;
  g.activation = s->activation;
  g.swiglu_limit = s->swiglu_limit > 0.f ? s->swiglu_limit : 7.0f;
  g.max_rows = ws->max_rows;
  g.sorted_ids = (const uint32_t*)(base + ws->off_sorted_ids);
  g.sorted_w = (const float*)(base + ws->off_sorted_w);
  g.sorted_e = (const int32_t*)(base + ws->off_sorted_e);
  g.num_valid = (const int32_t*)(base + ws->off_num_valid);
  g.status = (int32_t*)(base + ws->off_status);
}

int b200moe_gateup(const b200moe_shape* s, const b200moe_workspace* ws, void* workspace, const void* w1_q,
                   const void* w1_scale, const float* bias1, void* h_out, void* stream) {
  if (int rc = check_shape(s)) return rc;
  B200_CHECK_ARG(ws && workspace && w1_q && (w1_scale || is_bf16(s)), "gateup: NULL pointer");
  B200_CHECK_ARG(((uintptr_t)workspace & 1023) == 0, "gateup: workspace must be 1024-byte aligned");
  uint8_t* base = (uint8_t*)workspace;
  GemmArgs g = {};
  fill_common(g, s, ws, base);
  g.gateup = true;
  g.rows = s->I;
  g.Kd = s->H;
  g.w_data = w1_q;
  g.w_scale = w1_scale;
  g.a_q = base + ws->off_xq;
  g.asf = base + ws->off_xsf;
  g.h_out = h_out;
  g.bias = bias1;
  g.weight_stage1 = s->doweight_stage1;
  g.oq = base + ws->off_hq;
  g.osf = base + ws->off_hsf;
  if (is_bf16(s)) {
    B200_CHECK_ARG(h_out == nullptr, "gateup: bf16 weights write h in sorted-row order only (h_out must be NULL)");
    return launch_grouped_gemm_bf16(g, (cudaStream_t)stream);
  }
  if (is_fp8(s)) {
    g.out_kp = s->I;
    return launch_grouped_gemm_fp8(g, (cudaStream_t)stream);
  }
  g.out_kp = (int)kp_of(s->I);
  // the rows of the down projection are not live yet: their region serves as staging scratch of the gate-up
  g.gstage = base + ws->off_out2;
  g.gstage_bytes = ws->max_rows * (int64_t)s->H * 2;
  return launch_grouped_gemm(g, (cudaStream_t)stream);
}

int b200moe_down(const b200moe_shape* s, const b200moe_workspace* ws, void* workspace, const void* w2_q,
                 const void* w2_scale, const float* bias2, void* y_bf16, void* stream) {
  if (int rc = check_shape(s)) return rc;
  B200_CHECK_ARG(ws && workspace && w2_q && (w2_scale || is_bf16(s)), "down: NULL pointer");
  B200_CHECK_ARG(s->combine_mode != B200MOE_COMBINE_FUSED || y_bf16 != nullptr, "down: the fused combine needs y");
  B200_CHECK_ARG(((uintptr_t)workspace & 1023) == 0, "down: workspace must be 1024-byte aligned");
  uint8_t* base = (uint8_t*)workspace;
  GemmArgs g = {};
  fill_common(g, s, ws, base);
  g.gateup = false;
  g.rows = s->H;
  g.Kd = s->I;
  g.w_data = w2_q;
  g.w_scale = w2_scale;
  g.a_q = base + ws->off_hq;
  g.asf = base + ws->off_hsf;
  g.out2 = base + ws->off_out2;
  g.bias = bias2;
  g.y = s->combine_mode == B200MOE_COMBINE_FUSED ? y_bf16 : nullptr;
  if (s->doweight_stage1) g.sorted_w = nullptr;     // weights already applied upstream
  if (is_bf16(s)) return launch_grouped_gemm_bf16(g, (cudaStream_t)stream);
  if (is_fp8(s)) return launch_grouped_gemm_fp8(g, (cudaStream_t)stream);
  return launch_grouped_gemm(g, (cudaStream_t)stream);
}

int b200moe_combine(const b200moe_shape* s, const b200moe_workspace* ws, void* workspace, const float* topk_weight,
                    void* y_bf16, void* stream) {
  if (int rc = check_shape(s)) return rc;
  B200_CHECK_ARG(ws && workspace && (s->T == 0 || y_bf16), "combine: NULL pointer");
  B200_CHECK_ARG(s->T == 0 || topk_weight || s->doweight_stage1, "combine: NULL routing weights");
  if (s->doweight_stage1) topk_weight = nullptr;
  B200_CHECK_ARG(((uintptr_t)y_bf16 & 15) == 0, "combine: output must be 16-byte aligned");
  uint8_t* base = (uint8_t*)workspace;
  return launch_combine(base + ws->off_out2, (const int32_t*)(base + ws->off_loc), topk_weight, y_bf16, s->T, s->K,
                        s->H, (cudaStream_t)stream);
}

// A workspace laid out for more tokens than the call carries is fine (its offsets and row capacity are used as
// given); one that is too small in ANY region is an argument error: the layout is recomputed for the call's shape
// and every region of the caller's descriptor must be at least as large (a descriptor laid out for another K, B
// or E_route can have enough rows and still too small a scale or index region).
static int check_capacity(const b200moe_shape* s, const b200moe_workspace* ws) {
  b200moe_workspace need;
  if (int rc = b200moe_workspace_layout(s, &need)) return rc;
  B200_CHECK_ARG(ws->max_rows >= need.max_rows && ws->max_rows % s->B == 0,
                 "workspace holds %lld rows, T=%d needs %lld (blocks of %d)", (long long)ws->max_rows, s->T,
                 (long long)need.max_rows, s->B);
  static int64_t b200moe_workspace::* const kOff[] = {
      &b200moe_workspace::off_sorted_ids, &b200moe_workspace::off_sorted_w, &b200moe_workspace::off_sorted_e,
      &b200moe_workspace::off_num_valid,  &b200moe_workspace::off_loc,      &b200moe_workspace::off_status,
      &b200moe_workspace::off_xq,         &b200moe_workspace::off_xsf,      &b200moe_workspace::off_hq,
      &b200moe_workspace::off_hsf,        &b200moe_workspace::off_out2,     &b200moe_workspace::off_sort_scratch,
      &b200moe_workspace::total_bytes};
  constexpr int n = sizeof(kOff) / sizeof(kOff[0]);
  for (int i = 0; i + 1 < n; ++i) {
    const int64_t have = ws->*kOff[i + 1] - ws->*kOff[i], want = need.*kOff[i + 1] - need.*kOff[i];
    B200_CHECK_ARG(ws->*kOff[i] >= 0 && have >= want,
                   "workspace region %d holds %lld bytes, this call needs %lld (was the descriptor laid out for "
                   "another K, B or E_route?)", i, (long long)have, (long long)want);
  }
  return 0;
}

static int forward_impl(const b200moe_shape* s, const b200moe_workspace* ws, void* workspace, const b200moe_io* io,
                        void* stream) {
  if (int rc = check_shape(s)) return rc;
  B200_CHECK_ARG(ws && workspace && io, "forward: NULL workspace");
  if (s->T == 0) return 0;
  if (int rc = check_capacity(s, ws)) return rc;
  B200_CHECK_ARG(io->x_bf16 && io->topk_ids && io->topk_weight && io->y_bf16, "forward: NULL tensor");
  B200_CHECK_ARG(((uintptr_t)io->y_bf16 & 15) == 0, "forward: output must be 16-byte aligned");
  uint8_t* base = (uint8_t*)workspace;
  const bool fp8w = is_fp8(s);
  const bool fused = s->combine_mode == B200MOE_COMBINE_FUSED;
  // the fused combine accumulates into y: the quantiser launch clears it first
  void* zero_ptr = fused ? io->y_bf16 : nullptr;
  const int64_t zero_bytes = fused ? (int64_t)s->T * s->H * 2 : 0;
  uint32_t* sorted_ids = (uint32_t*)(base + ws->off_sorted_ids);
  float* sorted_w = (float*)(base + ws->off_sorted_w);
  int32_t* sorted_e = (int32_t*)(base + ws->off_sorted_e);
  int32_t* num_valid = (int32_t*)(base + ws->off_num_valid);
  int32_t* loc = (int32_t*)(base + ws->off_loc);
  int rc;
  if (sort_quant_small_ok(s->T, s->K, s->E_route)) {
    rc = launch_sort_quant_small(is_bf16(s) ? 3 : fp8w ? (s->act_quant ? 2 : 1) : 0, io->x_bf16, io->topk_ids, io->topk_weight, s->T, s->K, s->E_route, s->B,
                                 io->expert_mask, io->num_local_tokens, sorted_ids, sorted_w, sorted_e, num_valid, loc,
                                 s->H, terms_of(s), ws->max_rows, base + ws->off_xq, base + ws->off_xsf, zero_ptr,
                                 zero_bytes, (cudaStream_t)stream);
    if (rc) return rc;
  } else {
    rc = sort_align_impl(io->topk_ids, io->topk_weight, s->T, s->K, s->E_route, s->B, io->expert_mask,
                         io->num_local_tokens, sorted_ids, sorted_w, sorted_e, num_valid, loc,
                         base + ws->off_sort_scratch, sort_scratch_bytes(s->E_route), stream);
    if (rc) return rc;
    if (is_bf16(s))
      rc = launch_gather_rows_bf16(io->x_bf16, loc, s->T, s->K, s->H, s->B, ws->max_rows, base + ws->off_xq, zero_ptr,
                                   zero_bytes, (cudaStream_t)stream);
    else if (fp8w && s->act_quant)
      rc = launch_quant_rows_fp8_1x128(io->x_bf16, 0, sorted_ids, num_valid, s->T, s->K, s->H, s->B, ws->max_rows,
                                       base + ws->off_xq, base + ws->off_xsf, zero_ptr, zero_bytes, loc, (cudaStream_t)stream);
    else if (fp8w)
      rc = launch_quant_rows_e4m3(io->x_bf16, 0, sorted_ids, num_valid, s->T, s->K, s->H, s->B, ws->max_rows,
                                  base + ws->off_xq, base + ws->off_xsf, zero_ptr, zero_bytes, loc, (cudaStream_t)stream);
    else
      rc = launch_quant_rows(io->x_bf16, 0, sorted_ids, num_valid, s->T, s->K, s->H, s->B, terms_of(s), ws->max_rows,
                             base + ws->off_xq, base + ws->off_xsf, zero_ptr, zero_bytes, loc, (cudaStream_t)stream);
    if (rc) return rc;
  }
  rc = b200moe_gateup(s, ws, workspace, io->w1_q, io->w1_scale_prepared, io->bias1, nullptr, stream);
  if (rc) return rc;
  rc = b200moe_down(s, ws, workspace, io->w2_q, io->w2_scale_prepared, io->bias2, io->y_bf16, stream);
  if (rc || fused) return rc;
  return b200moe_combine(s, ws, workspace, io->topk_weight, io->y_bf16, stream);
}

int b200moe_forward_ex(const b200moe_shape* s, const b200moe_workspace* ws, void* workspace, const b200moe_io* io,
                       void* stream) {
  return forward_impl(s, ws, workspace, io, stream);
}

int b200moe_forward(const b200moe_shape* s, const b200moe_workspace* ws, void* workspace, const void* x_bf16,
                    const int32_t* topk_ids, const float* topk_weight, const int32_t* expert_mask,
                    const void* w1_q, const void* w1_scale, const void* w2_q, const void* w2_scale,
                    void* y_bf16, void* stream) {
  const b200moe_io io = {x_bf16, topk_ids, topk_weight, expert_mask, nullptr, w1_q, w1_scale, w2_q, w2_scale,
                         nullptr, nullptr, y_bf16};
  return forward_impl(s, ws, workspace, &io, stream);
}

int b200moe_forward_dyn(const b200moe_shape* s, const b200moe_workspace* ws, void* workspace, const void* x_bf16,
                        const int32_t* topk_ids, const float* topk_weight, const int32_t* expert_mask,
                        const int32_t* num_local_tokens, const void* w1_q, const void* w1_scale, const void* w2_q,
                        const void* w2_scale, void* y_bf16, void* stream) {
  const b200moe_io io = {x_bf16, topk_ids, topk_weight, expert_mask, num_local_tokens, w1_q, w1_scale, w2_q, w2_scale,
                         nullptr, nullptr, y_bf16};
  return forward_impl(s, ws, workspace, &io, stream);
}

int b200moe_batch1_scratch_bytes(const b200moe_shape* s, int64_t* bytes) {
  if (int rc = check_shape(s)) return rc;
  B200_CHECK_ARG(bytes != nullptr, "batch1_scratch_bytes: NULL pointer");
  *bytes = batch1_scratch_bytes(s->K, s->I);
  return 0;
}

int b200moe_forward_batch1(const b200moe_shape* s, const void* x_bf16, const int32_t* topk_ids, const float* topk_weight,
                           const int32_t* expert_mask, const int32_t* num_local_tokens, const void* w1_q,
                           const void* w1_scale, const void* w2_q, const void* w2_scale, const float* bias1,
                           const float* bias2, void* scratch, void* y_bf16, void* stream) {
  if (int rc = check_shape(s)) return rc;
  B200_CHECK_ARG(s->T == 1, "forward_batch1: T=%d (this entry point takes exactly one token)", s->T);
  B200_CHECK_ARG(s->weight_format == B200MOE_W_MXFP4, "forward_batch1: MXFP4 weights only");
  B200_CHECK_ARG(x_bf16 && topk_ids && topk_weight && w1_q && w1_scale && w2_q && w2_scale && scratch && y_bf16,
                 "forward_batch1: NULL pointer");
  return launch_forward_batch1(x_bf16, topk_ids, topk_weight, expert_mask, num_local_tokens, w1_q, w1_scale, w2_q,
                               w2_scale, bias1, bias2, scratch, y_bf16, s->H, s->I, s->K, s->E, s->E_route,
                               s->activation, s->swiglu_limit > 0.f ? s->swiglu_limit : 7.0f, s->doweight_stage1,
                               (cudaStream_t)stream);
}

int b200moe_route_topk(const float* logits, int32_t T, int32_t E, int32_t K, int32_t scoring, int32_t renormalize,
                       int32_t* topk_ids, float* topk_weight, void* stream) {
  B200_CHECK_ARG(T >= 0, "route_topk: T=%d", T);
  B200_CHECK_ARG(T == 0 || (logits && topk_ids && topk_weight), "route_topk: NULL pointer");
  return launch_route_topk(logits, T, E, K, scoring, renormalize, topk_ids, topk_weight, (cudaStream_t)stream);
}

int b200moe_gather_sum(const void* rows_bf16, const int32_t* pos, int32_t T, int32_t slots, int32_t H, void* y_bf16,
                       void* stream) {
  B200_CHECK_ARG(T >= 0 && slots >= 1 && H > 0, "gather_sum: bad sizes T=%d slots=%d H=%d", T, slots, H);
  if (T == 0) return 0;
  B200_CHECK_ARG(rows_bf16 && pos && y_bf16, "gather_sum: NULL pointer");
  B200_CHECK_ARG(((uintptr_t)rows_bf16 & 15) == 0 && ((uintptr_t)y_bf16 & 15) == 0, "gather_sum: 16-byte alignment");
  return launch_gather_sum(rows_bf16, pos, y_bf16, T, slots, H, (cudaStream_t)stream);
}

int b200moe_ep_plan(const int32_t* topk_ids, int32_t T, int32_t K, int32_t experts_per_rank, int32_t world,
                    int32_t* pos, int32_t* counts, int32_t* rows, void* stream) {
  B200_CHECK_ARG(pos && counts && rows && (T == 0 || topk_ids), "ep_plan: NULL pointer");
  return launch_ep_plan(topk_ids, T, K, experts_per_rank, world, pos, counts, rows, (cudaStream_t)stream);
}

int b200moe_debug_probe(int which, const void* in, void* out, void* stream) {
  B200_CHECK_ARG(in && out, "debug_probe: NULL pointer");
  return run_debug_probe(which, in, out, (cudaStream_t)stream);
}

}  // extern "C"
