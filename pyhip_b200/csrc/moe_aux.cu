// Integer / byte kernels around the grouped GEMMs: token->expert sort/align, activation
// quantise-and-gather, scale repack, weighted combine.  All HBM- or latency-bound.
#include "gemm_common.cuh"

namespace b200moe {

// =====================================================================================
// sort / align  (contract: src/contrib/fused_moe.py:56-100 of the reference; ck_tile
// reference_moe_sorting.hpp:14-117).  One CTA; every warp owns a contiguous slice of the
// flattened [T*K] id array, so slice order == the required stable token-major order.
// No atomics: ranks come from warp match/popc and per-warp counters, hence deterministic.
// =====================================================================================
constexpr int kSortWarps = 32;

__device__ __forceinline__ int sort_fetch_expert(const int32_t* ids, const int32_t* mask, int i, int P, int E) {
  if (i >= P) return -1;
  int e = ids[i];
  if (e < 0 || e >= E) return -1;
  if (mask != nullptr && mask[e] == 0) return -1;
  return e;
}

__global__ void __launch_bounds__(kSortWarps * 32, 1)
sort_align_kernel(const int32_t* __restrict__ ids, const float* __restrict__ w, int T, int K, int E, int B,
                  const int32_t* __restrict__ mask, uint32_t* __restrict__ sorted_ids,
                  float* __restrict__ sorted_w, int32_t* __restrict__ sorted_e,
                  int32_t* __restrict__ num_valid, int32_t* __restrict__ loc,
                  const int32_t* __restrict__ num_local) {
  extern __shared__ int32_t sm[];
  int32_t* cnt = sm;                        // [kSortWarps][E] per-warp counts, then running offsets
  int32_t* base = sm + kSortWarps * E;      // [E] first sorted row of the expert
  int32_t* total = base + E;                // [E]
  int32_t* lid = total + E;                 // [E] emitted (local) expert id
  unsigned long long* wsum =                // [33] scan scratch, 8-byte aligned
      reinterpret_cast<unsigned long long*>(sm + ((kSortWarps * E + 3 * E + 1) & ~1));

  grid_dep_launch();
  grid_dep_wait();     // the previous call on this stream may still read the arrays written below
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int P = T * K;
  const int seg = ((P + kSortWarps - 1) / kSortWarps + 31) & ~31;
  const int seg_lo = warp * seg, seg_hi = min(P, seg_lo + seg);
  // tokens at and beyond *num_local (a device value, for batches padded to a fixed T) take no part:
  // their pairs are dropped and their loc entries read -1
  const int T_live = (num_local != nullptr) ? min(T, max(num_local[0], 0)) : T;
  const int live_hi = min(seg_hi, T_live * K);

  for (int i = tid; i < kSortWarps * E; i += blockDim.x) cnt[i] = 0;
  __syncthreads();

  // pass 1: per-warp histogram of its slice
  for (int i0 = seg_lo; i0 < seg_hi; i0 += 32) {
    int e = sort_fetch_expert(ids, mask, i0 + lane, live_hi, E);
    unsigned same = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && lane == __ffs(same) - 1) cnt[warp * E + e] += __popc(same);
  }
  __syncthreads();

  // per-expert (one thread each, E <= blockDim.x): warp offsets inside the expert, padded
  // size, and whether the expert advances the emitted (local) expert id
  {
    const int e = tid;
    int padded = 0, live = 0;
    if (e < E) {
      int run = 0;
      for (int wv = 0; wv < kSortWarps; ++wv) {
        int c = cnt[wv * E + e];
        cnt[wv * E + e] = run;
        run += c;
      }
      total[e] = run;
      padded = (run + B - 1) / B * B;
      live = (mask == nullptr || mask[e] != 0) ? 1 : 0;
    }
    // block-wide exclusive scan of (padded, live), packed in one 64-bit word
    const unsigned long long v = ((unsigned long long)(unsigned)padded << 32) | (unsigned)live;
    unsigned long long incl = v;
    for (int d = 1; d < 32; d <<= 1) {
      unsigned long long o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const unsigned long long s = wsum[lane];
      unsigned long long si = s;
      for (int d = 1; d < 32; d <<= 1) {
        unsigned long long o = __shfl_up_sync(0xffffffffu, si, d);
        if (lane >= d) si += o;
      }
      wsum[lane] = si - s;
      if (lane == 31) wsum[32] = si;
    }
    __syncthreads();
    const unsigned long long excl = wsum[warp] + incl - v;
    if (e < E) {
      base[e] = (int)(excl >> 32);
      lid[e] = (int)(excl & 0xffffffffu);
    }
    if (tid == 0) {
      num_valid[0] = (int)(wsum[32] >> 32);
      num_valid[1] = T_live;
    }
  }
  __syncthreads();

  // pass 2: stable scatter
  const uint32_t lt_mask = (1u << lane) - 1u;
  for (int i0 = seg_lo; i0 < seg_hi; i0 += 32) {
    int i = i0 + lane;
    int e = sort_fetch_expert(ids, mask, i, live_hi, E);
    unsigned same = __match_any_sync(0xffffffffu, e);
    int pos = -1;
    if (e >= 0) pos = base[e] + cnt[warp * E + e] + __popc(same & lt_mask);
    __syncwarp();
    if (e >= 0 && lane == __ffs(same) - 1) cnt[warp * E + e] += __popc(same);
    __syncwarp();
    if (i < seg_hi) {
      if (pos >= 0) {
        sorted_ids[pos] = ((uint32_t)(i % K) << 24) | (uint32_t)(i / K);
        sorted_w[pos] = w[i];
      }
      if (loc != nullptr) loc[i] = pos;
    }
  }

  // padding rows and per-block expert ids
  const uint32_t sentinel = ((uint32_t)K << 24) | (uint32_t)T;
  for (int e = tid; e < E; e += blockDim.x) {
    int n = total[e];
    if (n == 0) continue;
    int b0 = base[e], n_pad = (n + B - 1) / B * B;
    for (int p = b0 + n; p < b0 + n_pad; ++p) {
      sorted_ids[p] = sentinel;
      sorted_w[p] = 0.f;
    }
    for (int blk = b0 / B; blk < (b0 + n_pad) / B; ++blk) sorted_e[blk] = lid[e];
  }
}

int launch_sort_align(const int32_t* ids, const float* w, int T, int K, int E, int B, const int32_t* mask,
                      uint32_t* sorted_ids, float* sorted_w, int32_t* sorted_e, int32_t* num_valid,
                      int32_t* loc, const int32_t* num_local, cudaStream_t st) {
  B200_CHECK_ARG(E >= 1 && E <= kSortWarps * 32, "sort_align: E=%d outside [1,%d]", E, kSortWarps * 32);
  size_t smem = (size_t)(kSortWarps * E + 3 * E + 2) * sizeof(int32_t) + 34 * sizeof(unsigned long long);
  B200_CHECK_ARG(smem <= 200 * 1024, "sort_align: E=%d needs %zu bytes of shared memory", E, smem);
  // the attribute belongs to the (function, device) pair and setting it is cheap: do it on every launch
  B200_CHECK_CUDA(cudaFuncSetAttribute(sort_align_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  B200_CHECK_CUDA(launch_chained(sort_align_kernel, dim3(1), dim3(kSortWarps * 32), smem, st, ids, w, T, K, E, B, mask,
                                 sorted_ids, sorted_w, sorted_e, num_valid, loc, num_local));
  return 0;
}

// =====================================================================================
// The same sort spread over several CTAs, for batches whose (token, expert) pairs number in the tens of
// thousands: one CTA's store path is the limit there (three scattered 4-byte stores per pair).  Three
// chained launches over caller scratch: per-(CTA, warp) histograms of contiguous slices -> one CTA turns them
// into offsets (slice order = the required stable order) and does the per-expert part -> every warp
// scatters its slice.  Bit-identical to the single-CTA kernel.
// scratch: int32 [slices = G*32][E] counts per warp, [G][E] counts per CTA, [G][E] offsets per CTA, then [E] first
// sorted row of each expert.
// =====================================================================================
constexpr int kSortMaxCtas = 64;

__host__ __device__ inline int sort_slice_pairs(int P, int G) {       // pairs per CTA: whole warps x 32 lanes
  return ((P + G - 1) / G + 1023) & ~1023;
}

__global__ void __launch_bounds__(kSortWarps * 32, 1)
sort_count_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ mask, int T, int K, int E,
                  const int32_t* __restrict__ num_local, int slice, int32_t* __restrict__ hist,
                  int32_t* __restrict__ ctot) {
  extern __shared__ int32_t sm[];          // [kSortWarps][E]
  grid_dep_launch();
  grid_dep_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int P = T * K;
  const int T_live = (num_local != nullptr) ? min(T, max(num_local[0], 0)) : T;
  const int per_warp = slice / kSortWarps;
  const int lo = min(P, blockIdx.x * slice + warp * per_warp), hi = min(P, lo + per_warp);
  const int live_hi = min(hi, T_live * K);
  int32_t* cnt = sm + warp * E;
  for (int e = lane; e < E; e += 32) cnt[e] = 0;
  __syncwarp();
  for (int i0 = lo; i0 < hi; i0 += 32) {
    int e = sort_fetch_expert(ids, mask, i0 + lane, live_hi, E);
    unsigned same = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && lane == __ffs(same) - 1) cnt[e] += __popc(same);
    __syncwarp();
  }
  int32_t* row = hist + ((int64_t)blockIdx.x * kSortWarps + warp) * E;
  for (int e = lane; e < E; e += 32) row[e] = cnt[e];
  __syncthreads();
  // the CTA's own total per expert: the scan launch walks one row per CTA, not one per warp
  for (int e = tid; e < E; e += blockDim.x) {
    int sum = 0;
    for (int wi = 0; wi < kSortWarps; ++wi) sum += sm[wi * E + e];
    ctot[(int64_t)blockIdx.x * E + e] = sum;
  }
}

__global__ void __launch_bounds__(kSortWarps * 32, 1)
sort_scan_kernel(const int32_t* __restrict__ hist, int32_t* __restrict__ offs, int S, int T, int K, int E, int B,
                 const int32_t* __restrict__ mask,
                 const int32_t* __restrict__ num_local, uint32_t* __restrict__ sorted_ids,
                 float* __restrict__ sorted_w, int32_t* __restrict__ sorted_e, int32_t* __restrict__ num_valid) {
  __shared__ int32_t part[kSortWarps * 32];      // partial sums [threads per expert][E]
  __shared__ int32_t total[kSortWarps * 32], base[kSortWarps * 32], lid[kSortWarps * 32];
  __shared__ unsigned long long wsum[34];
  grid_dep_launch();
  grid_dep_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // several threads per expert share the walk over the S slices
  const int tpe = max(1, (int)blockDim.x / E);
  const int e_of = tid % E, j = tid / E;
  const int chunk = (S + tpe - 1) / tpe;
  const int s0 = min(S, j * chunk), s1 = min(S, s0 + chunk);
  const bool walker = j < tpe;
  if (walker) {
    int sum = 0;
    for (int sidx = s0; sidx < s1; ++sidx) sum += hist[(int64_t)sidx * E + e_of];
    part[j * E + e_of] = sum;
  }
  __syncthreads();
  if (walker) {
    int run = 0;
    for (int jj = 0; jj < j; ++jj) run += part[jj * E + e_of];
    // counts are read from one array and offsets written to another, so the loads do not wait for the stores
    for (int sidx = s0; sidx < s1; ++sidx) {
      const int c = hist[(int64_t)sidx * E + e_of];
      offs[(int64_t)sidx * E + e_of] = run;
      run += c;
    }
    if (j == tpe - 1) total[e_of] = run;
  }
  __syncthreads();
  const int T_live = (num_local != nullptr) ? min(T, max(num_local[0], 0)) : T;
  {
    const int e = tid;
    int padded = 0, live = 0;
    if (e < E) {
      padded = (total[e] + B - 1) / B * B;
      live = (mask == nullptr || mask[e] != 0) ? 1 : 0;
    }
    const unsigned long long v = ((unsigned long long)(unsigned)padded << 32) | (unsigned)live;
    unsigned long long incl = v;
    for (int d = 1; d < 32; d <<= 1) {
      unsigned long long o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const unsigned long long sv = wsum[lane];
      unsigned long long si = sv;
      for (int d = 1; d < 32; d <<= 1) {
        unsigned long long o = __shfl_up_sync(0xffffffffu, si, d);
        if (lane >= d) si += o;
      }
      wsum[lane] = si - sv;
      if (lane == 31) wsum[32] = si;
    }
    __syncthreads();
    const unsigned long long excl = wsum[warp] + incl - v;
    if (e < E) {
      base[e] = (int)(excl >> 32);
      lid[e] = (int)(excl & 0xffffffffu);
      offs[(int64_t)S * E + e] = base[e];          // for the scatter launch
    }
    if (tid == 0) {
      num_valid[0] = (int)(wsum[32] >> 32);
      num_valid[1] = T_live;
    }
  }
  __syncthreads();
  // padding rows and per-block expert ids: all threads share the rows of all experts
  const uint32_t sentinel = ((uint32_t)K << 24) | (uint32_t)T;
  for (int e = warp; e < E; e += kSortWarps) {
    const int n = total[e];
    if (n == 0) continue;
    const int b0 = base[e], n_pad = (n + B - 1) / B * B;
    for (int p = b0 + n + lane; p < b0 + n_pad; p += 32) {
      sorted_ids[p] = sentinel;
      sorted_w[p] = 0.f;
    }
    for (int blk = b0 / B + lane; blk < (b0 + n_pad) / B; blk += 32) sorted_e[blk] = lid[e];
  }
}

__global__ void __launch_bounds__(kSortWarps * 32, 1)
sort_scatter_kernel(const int32_t* __restrict__ ids, const float* __restrict__ w, const int32_t* __restrict__ mask,
                    int T, int K, int E, const int32_t* __restrict__ num_local, int slice, int G,
                    const int32_t* __restrict__ hist, const int32_t* __restrict__ coffs,
                    uint32_t* __restrict__ sorted_ids,
                    float* __restrict__ sorted_w, int32_t* __restrict__ loc) {
  extern __shared__ int32_t sm[];          // [kSortWarps][E] running offsets, then [E] expert bases
  grid_dep_launch();
  grid_dep_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int P = T * K;
  const int T_live = (num_local != nullptr) ? min(T, max(num_local[0], 0)) : T;
  const int per_warp = slice / kSortWarps;
  const int lo = min(P, blockIdx.x * slice + warp * per_warp), hi = min(P, lo + per_warp);
  const int live_hi = min(hi, T_live * K);
  int32_t* cnt = sm + warp * E;
  int32_t* base = sm + kSortWarps * E;
  const int32_t* row = hist + ((int64_t)blockIdx.x * kSortWarps + warp) * E;
  for (int e = lane; e < E; e += 32) cnt[e] = row[e];
  __syncthreads();
  // counts of this CTA's warps -> where each warp's first row of an expert goes, relative to the expert's first row
  for (int e = tid; e < E; e += blockDim.x) {
    int run = coffs[(int64_t)blockIdx.x * E + e];
    for (int wi = 0; wi < kSortWarps; ++wi) {
      const int c = sm[wi * E + e];
      sm[wi * E + e] = run;
      run += c;
    }
    base[e] = coffs[(int64_t)G * E + e];
  }
  __syncthreads();
  const uint32_t lt_mask = (1u << lane) - 1u;
  for (int i0 = lo; i0 < hi; i0 += 32) {
    const int i = i0 + lane;
    int e = sort_fetch_expert(ids, mask, i, live_hi, E);
    unsigned same = __match_any_sync(0xffffffffu, e);
    int pos = -1;
    if (e >= 0) pos = base[e] + cnt[e] + __popc(same & lt_mask);
    __syncwarp();
    if (e >= 0 && lane == __ffs(same) - 1) cnt[e] += __popc(same);
    __syncwarp();
    if (i < hi) {
      if (pos >= 0) {
        sorted_ids[pos] = ((uint32_t)(i % K) << 24) | (uint32_t)(i / K);
        sorted_w[pos] = w[i];
      }
      if (loc != nullptr) loc[i] = pos;
    }
  }
}

int64_t sort_scratch_bytes(int E) { return (2ll * kSortMaxCtas * kSortWarps + 1) * E * (int64_t)sizeof(int32_t); }

int launch_sort_align_wide(const int32_t* ids, const float* w, int T, int K, int E, int B, const int32_t* mask,
                           uint32_t* sorted_ids, float* sorted_w, int32_t* sorted_e, int32_t* num_valid,
                           int32_t* loc, const int32_t* num_local, void* scratch, cudaStream_t st) {
  B200_CHECK_ARG(E >= 1 && E <= kSortWarps * 32, "sort_align: E=%d outside [1,%d]", E, kSortWarps * 32);
  const int P = T * K;
  const int G = std::max(1, std::min(kSortMaxCtas, (P + 2047) / 2048));
  const int slice = sort_slice_pairs(P, G);
  const int S = G * kSortWarps;
  const size_t smem = (size_t)(kSortWarps * E + E) * sizeof(int32_t);
  B200_CHECK_ARG(smem <= 200 * 1024, "sort_align: E=%d needs %zu bytes of shared memory", E, smem);
  B200_CHECK_CUDA(cudaFuncSetAttribute(sort_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  B200_CHECK_CUDA(cudaFuncSetAttribute(sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  int32_t* hist = (int32_t*)scratch;                 // [S][E] counts per warp
  int32_t* ctot = hist + (int64_t)S * E;             // [G][E] counts per CTA
  int32_t* coffs = ctot + (int64_t)G * E;            // [G][E] offsets per CTA, then [E] first row of each expert
  B200_CHECK_CUDA(launch_chained(sort_count_kernel, dim3(G), dim3(kSortWarps * 32), smem, st, ids, mask, T, K, E,
                                 num_local, slice, hist, ctot));
  B200_CHECK_CUDA(launch_chained(sort_scan_kernel, dim3(1), dim3(kSortWarps * 32), 0, st, (const int32_t*)ctot, coffs, G,
                                 T, K, E, B, mask, num_local, sorted_ids, sorted_w, sorted_e, num_valid));
  B200_CHECK_CUDA(launch_chained(sort_scatter_kernel, dim3(G), dim3(kSortWarps * 32), smem, st, ids, w, mask, T, K, E,
                                 num_local, slice, G, (const int32_t*)hist, (const int32_t*)coffs, sorted_ids, sorted_w,
                                 loc));
  return 0;
}

// =====================================================================================
// activation quantisers: bf16 row -> the operand format of the GEMMs, written in sorted-row order.
// One thread per 32-element block.
//
// Packed-FP4 terms (MXFP4 weights).  Term t quantises what the previous terms left over:
//   e = max(biased_exponent(amax(r)) - 2, 0);  q = e2m1_rne_sat(r * 2^(127-e));  r -= q * 2^(e-127)
// (amax/2^(e-127) lies in [4,8): the OCP MX scale rule; values above 6 saturate and the next
// term picks up the rest).  One term is the plain MXFP4 activation format of the reference's a4w4
// kernels; three terms reproduce a bf16 input to ~2e-3 of the block maximum, four to ~1e-4.
//
// Two e4m3 terms with E8M0 scales (FP8 128x128 weights): q [2, max_rows, Kd] bytes, one scale
// chunk per term (virtual row = term*128 + r).
// =====================================================================================
__device__ __forceinline__ void load_block32(const __nv_bfloat16* src, float (&x)[32]) {
  const uint4* p = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    uint4 u = p[v];
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float2 f = __bfloat1622float2(b2[t]);
      x[v * 8 + t * 2] = f.x;
      x[v * 8 + t * 2 + 1] = f.y;
    }
  }
}

struct QuantGeom {
  int Kd, KP, B, NT, TS;       // TS: scale row stride between the terms of a block
  int64_t max_rows;
  uint8_t* q;
  uint8_t* sf;
};

// One quantised unit = block j (32 elements) of a source row, held in registers between its computation (which
// needs only the source row) and its store (which needs the sorted row): the decode path computes the unit
// while the sort is still being worked out.
struct QuantUnit {
  uint4 q[8];        // packed-FP4 terms: q[t]; e4m3 terms: q[2t], q[2t+1]; 1x128: q[0], q[1]
  int e[4];          // E8M0 exponents of the terms
  float scale;       // 1x128: the block's fp32 scale
};

// block j of source row `srow`: packed-FP4 terms
__device__ __forceinline__ void quant_compute_fp4(const __nv_bfloat16* src, int64_t srow, int j, const QuantGeom& g,
                                                  QuantUnit& u) {
  float x[32];
  if (j * 32 < g.Kd) {
    load_block32(src + srow * g.Kd + j * 32, x);
  } else {                      // blocks of the K padding are written as zeros (finite scales)
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = 0.f;
  }
#pragma unroll
  for (int t = 0; t < 4; ++t)
    if (t < g.NT) u.e[t] = (t + 1 < g.NT) ? quant_block32_fp4<true>(x, u.q[t]) : quant_block32_fp4<false>(x, u.q[t]);
}
__device__ __forceinline__ void quant_store_fp4(int j, int64_t r, const QuantGeom& g, const QuantUnit& u) {
  const int64_t term_stride = g.max_rows * (g.KP / 2);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    if (t < g.NT) {
      *reinterpret_cast<uint4*>(g.q + t * term_stride + r * (g.KP / 2) + j * 16) = u.q[t];
      g.sf[act_sf_index(r / g.B, j >> 2, g.KP / 128, g.B, g.NT, g.TS, t, (int)(r % g.B), j & 3)] = (uint8_t)u.e[t];
    }
  }
}

// the same for two e4m3 terms (KP == Kd, a multiple of 128)
__device__ __forceinline__ void quant_compute_e4m3(const __nv_bfloat16* src, int64_t srow, int j, const QuantGeom& g,
                                                   QuantUnit& u) {
  float x[32];
  load_block32(src + srow * g.Kd + j * 32, x);
  u.e[0] = quant_block32_e4m3<true>(x, u.q[0], u.q[1]);
  u.e[1] = quant_block32_e4m3<false>(x, u.q[2], u.q[3]);
}
__device__ __forceinline__ void quant_store_e4m3(int j, int64_t r, const QuantGeom& g, const QuantUnit& u) {
  const int64_t term_stride = g.max_rows * g.Kd;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    uint4* dst = reinterpret_cast<uint4*>(g.q + t * term_stride + r * g.Kd + j * 32);
    dst[0] = u.q[2 * t];
    dst[1] = u.q[2 * t + 1];
    g.sf[act_sf_index(r / g.B, j >> 2, g.Kd / 128, g.B, 2, 128, t, (int)(r % g.B), j & 3)] = (uint8_t)u.e[t];
  }
}

// Per-token, per-128-channel e4m3 with an fp32 scale = amax / 448 (1.0 for an all-zero block): the reference's
// per_1x128 activation format (src/contrib/fused_moe.py:276-281,375-381).  Four neighbouring threads own the four
// 32-element quarters of a 128-block and share its amax through shuffles, so every lane of the warp must call the
// compute step (`live` = this thread has a unit).  q [max_rows, Kd] bytes; scales fp32 [blocks][Kd/128][B] (one
// contiguous run of B token scales per sorted block and k-block, the order the GEMM's producer copies them in).
__device__ __forceinline__ void quant_compute_fp8_1x128(const __nv_bfloat16* src, int64_t srow, int j, const QuantGeom& g,
                                                        bool live, QuantUnit& u) {
  float x[32];
  if (live) {
    load_block32(src + srow * g.Kd + j * 32, x);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
  uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const __nv_fp8x2_storage_t pk = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(x[i], scale), __fdiv_rn(x[i + 1], scale)),
                                                              __NV_SATFINITE, __NV_E4M3);
    w[i >> 2] |= (uint32_t)pk << ((i & 2) * 8);
  }
  u.q[0] = make_uint4(w[0], w[1], w[2], w[3]);
  u.q[1] = make_uint4(w[4], w[5], w[6], w[7]);
  u.scale = scale;
}
__device__ __forceinline__ void quant_store_fp8_1x128(int j, int64_t r, const QuantGeom& g, const QuantUnit& u) {
  uint4* dst = reinterpret_cast<uint4*>(g.q + r * g.Kd + j * 32);
  dst[0] = u.q[0];
  dst[1] = u.q[1];
  if ((j & 3) == 0)
    reinterpret_cast<float*>(g.sf)[((r / g.B) * (g.Kd / 128) + (j >> 2)) * g.B + (int)(r % g.B)] = u.scale;
}

// unquantised bf16 rows (bf16 weights): the unit is the 32 elements themselves, copied into sorted-row order
__device__ __forceinline__ void quant_compute_copy(const __nv_bfloat16* src, int64_t srow, int j, const QuantGeom& g,
                                                   QuantUnit& u) {
  const uint4* p = reinterpret_cast<const uint4*>(src + srow * g.Kd + j * 32);
#pragma unroll
  for (int v = 0; v < 4; ++v) u.q[v] = p[v];
}
__device__ __forceinline__ void quant_store_copy(int j, int64_t r, const QuantGeom& g, const QuantUnit& u) {
  uint4* p = reinterpret_cast<uint4*>(g.q + (r * g.Kd + j * 32) * 2);
#pragma unroll
  for (int v = 0; v < 4; ++v) p[v] = u.q[v];
}

template <int FMT>    // 0: packed-FP4 terms, 1: two e4m3 terms, 2: e4m3 with fp32 scales per 1x128, 3: bf16 as is
__device__ __forceinline__ void quant_compute(const __nv_bfloat16* src, int64_t srow, int j, const QuantGeom& g, bool live,
                                              QuantUnit& u) {
  if (FMT == 2) quant_compute_fp8_1x128(src, srow, j, g, live, u);
  else if (live) {
    if (FMT == 0) quant_compute_fp4(src, srow, j, g, u);
    else if (FMT == 1) quant_compute_e4m3(src, srow, j, g, u);
    else quant_compute_copy(src, srow, j, g, u);
  }
}
template <int FMT>
__device__ __forceinline__ void quant_store(int j, int64_t r, const QuantGeom& g, const QuantUnit& u) {
  if (FMT == 0) quant_store_fp4(j, r, g, u);
  else if (FMT == 1) quant_store_e4m3(j, r, g, u);
  else if (FMT == 2) quant_store_fp8_1x128(j, r, g, u);
  else quant_store_copy(j, r, g, u);
}

// grid-stride zero fill in 16-byte vectors (the output buffer of the fused combine)
__device__ __forceinline__ void zero_fill(uint4* ptr, int64_t nvec) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x)
    ptr[i] = make_uint4(0, 0, 0, 0);
}

template <int FMT>    // 0: packed-FP4 terms, 1: two e4m3 terms, 2: e4m3 with fp32 scales per 1x128
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ src, int src_mode, const uint32_t* __restrict__ sorted_ids,
                  const int32_t* __restrict__ num_valid, int T, int K, QuantGeom g, uint4* zero_ptr, int64_t zero_vec) {
  const int nb = g.KP / 32;
  grid_dep_launch();
  grid_dep_wait();
  zero_fill(zero_ptr, zero_vec);
  const int64_t total = min((int64_t)num_valid[0], g.max_rows) * nb;
  // block-uniform trip count: the 1x128 format shares a block maximum across four lanes with shuffles
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x; base < total; base += (int64_t)gridDim.x * blockDim.x) {
    const int64_t u = base + threadIdx.x;
    const int64_t r = min(u, total - 1) / nb;
    const int j = (int)(min(u, total - 1) % nb);
    const uint32_t id = sorted_ids[r];
    const int tok = (int)(id & 0xFFFFFFu), kk = (int)(id >> 24);
    // padding rows of a block are left unwritten: every token column of the GEMMs depends on its own row
    // only, and no kernel reads the columns of padding rows
    const bool live = u < total && kk < K && tok < T;
    const int64_t srow = (src_mode == 0) ? (int64_t)tok : ((int64_t)tok * K + kk);
    QuantUnit qu;
    quant_compute<FMT>(src, srow, j, g, live, qu);
    if (live) quant_store<FMT>(j, r, g, qu);
  }
}

// The layer input quantised once per TOKEN and stored at each of its K sorted rows (`loc[t, k]`, -1 where the pair was
// dropped): a token's row is read and quantised once instead of once per (token, expert) pair.
template <int FMT>
__global__ void __launch_bounds__(256)
quant_tokens_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ loc, int T, int K, QuantGeom g,
                    uint4* zero_ptr, int64_t zero_vec) {
  const int nb = g.KP / 32;
  grid_dep_launch();
  grid_dep_wait();
  zero_fill(zero_ptr, zero_vec);
  const int64_t total = (int64_t)T * nb;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x; base < total; base += (int64_t)gridDim.x * blockDim.x) {
    const int64_t u = base + threadIdx.x;
    const int64_t t = min(u, total - 1) / nb;
    const int j = (int)(min(u, total - 1) % nb);
    const bool live = u < total;
    QuantUnit qu;
    quant_compute<FMT>(src, t, j, g, live, qu);
    if (live) {
      for (int k = 0; k < K; ++k) {
        const int r = loc[t * K + k];
        if (r >= 0 && r < g.max_rows) quant_store<FMT>(j, r, g, qu);
      }
    }
  }
}

static int small_grid(int64_t units) { return (int)std::max<int64_t>(1, (units + 255) / 256); }   // one unit per thread
static int quant_grid(int64_t units) {
  return (int)std::max<int64_t>(1, std::min<int64_t>((units + 255) / 256, (int64_t)device_sm_count() * 16));
}

int launch_quant_rows(const void* src, int src_mode, const uint32_t* sorted_ids, const int32_t* num_valid,
                      int T, int K, int Kd, int B, int NT, int64_t max_rows, void* q, void* sf, void* zero_ptr,
                      int64_t zero_bytes, const int32_t* loc, cudaStream_t st) {
  B200_CHECK_ARG(B >= 16 && B <= 128 && B % 16 == 0, "quant_rows: B=%d is not a multiple of 16 in [16,128]", B);
  B200_CHECK_ARG(NT >= 1 && NT <= 4, "quant_rows: %d activation terms (1..4 supported)", NT);
  B200_CHECK_ARG(Kd % 32 == 0, "quant_rows: Kd=%d must be a multiple of 32", Kd);
  B200_CHECK_ARG(zero_bytes % 16 == 0 && ((uintptr_t)zero_ptr & 15) == 0, "quant_rows: zero region must be 16-byte aligned");
  const int KP = (int)round_up64(Kd, kKPad);
  QuantGeom g = {Kd, KP, B, NT, act_term_stride(B, NT, 2), max_rows, (uint8_t*)q, (uint8_t*)sf};
  if (loc != nullptr && src_mode == 0) {        // once per token, stored at its K sorted rows
    B200_CHECK_CUDA(launch_chained(quant_tokens_kernel<0>, dim3(quant_grid((int64_t)T * (KP / 32))), dim3(256), 0, st,
                                   reinterpret_cast<const __nv_bfloat16*>(src), loc, T, K, g, (uint4*)zero_ptr, zero_bytes / 16));
    return 0;
  }
  B200_CHECK_CUDA(launch_chained(quant_rows_kernel<0>, dim3(quant_grid(max_rows * (KP / 32))), dim3(256), 0, st,
                                 reinterpret_cast<const __nv_bfloat16*>(src), src_mode, sorted_ids, num_valid, T, K, g,
                                 (uint4*)zero_ptr, zero_bytes / 16));
  return 0;
}

int launch_quant_rows_e4m3(const void* src, int src_mode, const uint32_t* sorted_ids, const int32_t* num_valid,
                           int T, int K, int Kd, int B, int64_t max_rows, void* q, void* sf, void* zero_ptr,
                           int64_t zero_bytes, const int32_t* loc, cudaStream_t st) {
  B200_CHECK_ARG(B >= 16 && B <= 96 && B % 16 == 0, "quant_rows (e4m3): B=%d is not a multiple of 16 in [16,96]", B);
  B200_CHECK_ARG(Kd % 128 == 0, "quant_rows (e4m3): Kd=%d must be a multiple of 128", Kd);
  B200_CHECK_ARG(zero_bytes % 16 == 0 && ((uintptr_t)zero_ptr & 15) == 0, "quant_rows: zero region must be 16-byte aligned");
  QuantGeom g = {Kd, Kd, B, 2, 128, max_rows, (uint8_t*)q, (uint8_t*)sf};
  if (loc != nullptr && src_mode == 0) {
    B200_CHECK_CUDA(launch_chained(quant_tokens_kernel<1>, dim3(quant_grid((int64_t)T * (Kd / 32))), dim3(256), 0, st,
                                   reinterpret_cast<const __nv_bfloat16*>(src), loc, T, K, g, (uint4*)zero_ptr, zero_bytes / 16));
    return 0;
  }
  B200_CHECK_CUDA(launch_chained(quant_rows_kernel<1>, dim3(quant_grid(max_rows * (Kd / 32))), dim3(256), 0, st,
                                 reinterpret_cast<const __nv_bfloat16*>(src), src_mode, sorted_ids, num_valid, T, K, g,
                                 (uint4*)zero_ptr, zero_bytes / 16));
  return 0;
}

int launch_quant_rows_fp8_1x128(const void* src, int src_mode, const uint32_t* sorted_ids, const int32_t* num_valid,
                                int T, int K, int Kd, int B, int64_t max_rows, void* q, void* sf, void* zero_ptr,
                                int64_t zero_bytes, const int32_t* loc, cudaStream_t st) {
  B200_CHECK_ARG(B >= 16 && B <= 96 && B % 16 == 0, "quant_rows (1x128): B=%d is not a multiple of 16 in [16,96]", B);
  B200_CHECK_ARG(Kd % 128 == 0, "quant_rows (1x128): Kd=%d must be a multiple of 128", Kd);
  B200_CHECK_ARG(zero_bytes % 16 == 0 && ((uintptr_t)zero_ptr & 15) == 0 && ((uintptr_t)sf & 15) == 0,
                 "quant_rows: zero region / scales must be 16-byte aligned");
  QuantGeom g = {Kd, Kd, B, 1, 128, max_rows, (uint8_t*)q, (uint8_t*)sf};
  if (loc != nullptr && src_mode == 0) {
    B200_CHECK_CUDA(launch_chained(quant_tokens_kernel<2>, dim3(quant_grid((int64_t)T * (Kd / 32))), dim3(256), 0, st,
                                   reinterpret_cast<const __nv_bfloat16*>(src), loc, T, K, g, (uint4*)zero_ptr, zero_bytes / 16));
    return 0;
  }
  B200_CHECK_CUDA(launch_chained(quant_rows_kernel<2>, dim3(quant_grid(max_rows * (Kd / 32))), dim3(256), 0, st,
                                 reinterpret_cast<const __nv_bfloat16*>(src), src_mode, sorted_ids, num_valid, T, K, g,
                                 (uint4*)zero_ptr, zero_bytes / 16));
  return 0;
}

// bf16 weights: the layer input copied into sorted-row order, q = bf16 [max_rows, Kd] (no scales)
int launch_gather_rows_bf16(const void* src, const int32_t* loc, int T, int K, int Kd, int B, int64_t max_rows, void* q,
                            void* zero_ptr, int64_t zero_bytes, cudaStream_t st) {
  B200_CHECK_ARG(Kd % 32 == 0 && loc != nullptr, "gather_rows: Kd=%d must be a multiple of 32 and loc given", Kd);
  B200_CHECK_ARG(zero_bytes % 16 == 0 && ((uintptr_t)zero_ptr & 15) == 0, "gather_rows: zero region must be 16-byte aligned");
  QuantGeom g = {Kd, Kd, B, 1, 128, max_rows, (uint8_t*)q, nullptr};
  B200_CHECK_CUDA(launch_chained(quant_tokens_kernel<3>, dim3(quant_grid((int64_t)T * (Kd / 32))), dim3(256), 0, st,
                                 reinterpret_cast<const __nv_bfloat16*>(src), loc, T, K, g, (uint4*)zero_ptr, zero_bytes / 16));
  return 0;
}

// =====================================================================================
// Decode-sized batches (at most kSmallPairs (token, expert) pairs): sort/align and the input
// quantiser in ONE launch.  Every CTA repeats the whole sort in shared memory -- a few hundred
// integer operations -- and then quantises its share of the rows, so nothing waits for a
// single-CTA sort launch; CTA 0 also writes the sort arrays for the GEMMs.  The rank of a pair
// inside its expert is the number of earlier pairs with the same expert (token-major order), so
// the result is the same stable order as sort_align_kernel's, bit for bit, with no atomics on
// the order.  With T = 1 this is the reference's batch-1 shortcut (src/contrib/moe.py:79-84:
// blocks are taken straight from topk_ids) in this library's data layout.
// =====================================================================================
constexpr int kSmallPairs = 256;
constexpr int kSmallMaxE = 1024;

template <int FMT>
__global__ void __launch_bounds__(256)
sort_quant_small_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ ids,
                        const float* __restrict__ w, int T, int K, int E, const int32_t* __restrict__ mask,
                        const int32_t* __restrict__ num_local, uint32_t* __restrict__ sorted_ids,
                        float* __restrict__ sorted_w, int32_t* __restrict__ sorted_e,
                        int32_t* __restrict__ num_valid, int32_t* __restrict__ loc, QuantGeom g, uint4* zero_ptr,
                        int64_t zero_vec) {
  __shared__ int32_t pair_e[kSmallPairs], pair_pos[kSmallPairs];
  __shared__ int32_t cnt[kSmallMaxE], base[kSmallMaxE], lid[kSmallMaxE];
  __shared__ unsigned long long wsum[9];
  grid_dep_launch();
  grid_dep_wait();
  zero_fill(zero_ptr, zero_vec);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int P = T * K, B = g.B;
  // This thread's unit = (pair, 32-element block of the pair's token row).  Its source row is known without the
  // sort, so the row is loaded and quantised into registers first: the loads are in flight while the sort runs.
  const int nb = g.KP / 32;
  const int my_u = min(blockIdx.x * 256 + tid, P * nb - 1);
  const int my_pair = my_u / nb, my_j = my_u - my_pair * nb;
  const bool have_unit = blockIdx.x * 256 + tid < P * nb;
  QuantUnit qu;
  quant_compute<FMT>(x, my_pair / K, my_j, g, have_unit, qu);
  const int T_live = (num_local != nullptr) ? min(T, max(num_local[0], 0)) : T;
  for (int e = tid; e < E; e += 256) cnt[e] = 0;
  const int my_e = sort_fetch_expert(ids, mask, tid, min(P, T_live * K), E);
  if (tid < kSmallPairs) pair_e[tid] = my_e;
  __syncthreads();
  int rank = 0;
  if (my_e >= 0) {
    for (int i = 0; i < tid; ++i) rank += (pair_e[i] == my_e);
    atomicAdd(&cnt[my_e], 1);            // a count only: its value does not depend on the order of the adds
  }
  __syncthreads();
  // exclusive scan over the experts of (padded rows, emitted expert id); four consecutive experts per thread
  {
    unsigned long long v[4], run = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = tid * 4 + q;
      unsigned long long t = 0;
      if (e < E) {
        const unsigned padded = (unsigned)((cnt[e] + B - 1) / B * B);
        const unsigned live = (mask == nullptr || mask[e] != 0) ? 1u : 0u;
        t = ((unsigned long long)padded << 32) | live;
      }
      v[q] = run;
      run += t;
    }
    unsigned long long incl = run;
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned long long o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (tid == 0) {
      unsigned long long acc = 0;
      for (int i = 0; i < 8; ++i) { const unsigned long long t = wsum[i]; wsum[i] = acc; acc += t; }
      wsum[8] = acc;
    }
    __syncthreads();
    const unsigned long long off = wsum[warp] + incl - run;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = tid * 4 + q;
      if (e < E) {
        base[e] = (int)((off + v[q]) >> 32);
        lid[e] = (int)((off + v[q]) & 0xffffffffu);
      }
    }
  }
  __syncthreads();
  const int pos = (my_e >= 0) ? base[my_e] + rank : -1;
  if (tid < kSmallPairs) pair_pos[tid] = pos;
  if (blockIdx.x == 0) {
    if (tid < P) {
      if (pos >= 0) {
        sorted_ids[pos] = ((uint32_t)(tid % K) << 24) | (uint32_t)(tid / K);
        sorted_w[pos] = w[tid];
      }
      if (loc != nullptr) loc[tid] = pos;
    }
    const uint32_t sentinel = ((uint32_t)K << 24) | (uint32_t)T;
    for (int e = tid; e < E; e += 256) {
      const int n = cnt[e];
      if (n == 0) continue;
      const int b0 = base[e], n_pad = (n + B - 1) / B * B;
      for (int r = b0 + n; r < b0 + n_pad; ++r) {
        sorted_ids[r] = sentinel;
        sorted_w[r] = 0.f;
      }
      for (int blk = b0 / B; blk < (b0 + n_pad) / B; ++blk) sorted_e[blk] = lid[e];
    }
    if (tid == 0) {
      num_valid[0] = (int)(wsum[8] >> 32);
      num_valid[1] = T_live;
    }
  }
  __syncthreads();
  // store the unit computed above at its pair's sorted row (pairs that were dropped have none)
  const int r = pair_pos[my_pair];
  if (have_unit && r >= 0) quant_store<FMT>(my_j, r, g, qu);
}

bool sort_quant_small_ok(int T, int K, int E) { return (int64_t)T * K <= kSmallPairs && E <= kSmallMaxE && T >= 1; }

int launch_sort_quant_small(int fmt, const void* x, const int32_t* ids, const float* w, int T, int K, int E, int B,
                            const int32_t* mask, const int32_t* num_local, uint32_t* sorted_ids, float* sorted_w,
                            int32_t* sorted_e, int32_t* num_valid, int32_t* loc, int Kd, int NT, int64_t max_rows,
                            void* q, void* sf, void* zero_ptr, int64_t zero_bytes, cudaStream_t st) {
  B200_CHECK_ARG(sort_quant_small_ok(T, K, E), "sort_quant_small: T*K=%d pairs / E=%d outside the small-batch path", T * K, E);
  B200_CHECK_ARG(B >= 16 && B <= 128 && B % 16 == 0, "sort_quant_small: B=%d", B);
  B200_CHECK_ARG(zero_bytes % 16 == 0 && ((uintptr_t)zero_ptr & 15) == 0, "sort_quant_small: zero region must be 16-byte aligned");
  if (fmt == 0) {
    B200_CHECK_ARG(NT >= 1 && NT <= 4 && Kd % 32 == 0, "sort_quant_small: terms %d / Kd %d", NT, Kd);
    const int KP = (int)round_up64(Kd, kKPad);
    QuantGeom g = {Kd, KP, B, NT, act_term_stride(B, NT, 2), max_rows, (uint8_t*)q, (uint8_t*)sf};
    B200_CHECK_CUDA(launch_chained(sort_quant_small_kernel<0>, dim3(small_grid((int64_t)T * K * (KP / 32))), dim3(256), 0,
                                   st, (const __nv_bfloat16*)x, ids, w, T, K, E, mask, num_local, sorted_ids, sorted_w,
                                   sorted_e, num_valid, loc, g, (uint4*)zero_ptr, zero_bytes / 16));
  } else if (fmt == 3) {
    B200_CHECK_ARG(Kd % 32 == 0, "sort_quant_small (bf16): Kd %d", Kd);
    QuantGeom g = {Kd, Kd, B, 1, 128, max_rows, (uint8_t*)q, nullptr};
    B200_CHECK_CUDA(launch_chained(sort_quant_small_kernel<3>, dim3(small_grid((int64_t)T * K * (Kd / 32))), dim3(256), 0,
                                   st, (const __nv_bfloat16*)x, ids, w, T, K, E, mask, num_local, sorted_ids, sorted_w,
                                   sorted_e, num_valid, loc, g, (uint4*)zero_ptr, zero_bytes / 16));
  } else {
    B200_CHECK_ARG(Kd % 128 == 0 && B <= 96, "sort_quant_small (e4m3): Kd %d / B %d", Kd, B);
    QuantGeom g = {Kd, Kd, B, fmt == 1 ? 2 : 1, 128, max_rows, (uint8_t*)q, (uint8_t*)sf};
    if (fmt == 1)
      B200_CHECK_CUDA(launch_chained(sort_quant_small_kernel<1>, dim3(small_grid((int64_t)T * K * (Kd / 32))), dim3(256), 0,
                                     st, (const __nv_bfloat16*)x, ids, w, T, K, E, mask, num_local, sorted_ids, sorted_w,
                                     sorted_e, num_valid, loc, g, (uint4*)zero_ptr, zero_bytes / 16));
    else
      B200_CHECK_CUDA(launch_chained(sort_quant_small_kernel<2>, dim3(small_grid((int64_t)T * K * (Kd / 32))), dim3(256), 0,
                                     st, (const __nv_bfloat16*)x, ids, w, T, K, E, mask, num_local, sorted_ids, sorted_w,
                                     sorted_e, num_valid, loc, g, (uint4*)zero_ptr, zero_bytes / 16));
  }
  return 0;
}

// =====================================================================================
// combine: y[t,:] = sum over the token's pairs, in ascending sorted position (= ascending
// expert id), of bf16(out2[loc] * w), each partial sum rounded to bf16 -- the arithmetic of
// the reference's index_add_ loop (tests/contrib/moe/test_moe.py:107-117).
// One warp per (token, run of 32 sixteen-byte vectors): the token's K positions are ordered once per warp
// with shuffles (lane i ends up holding the i-th smallest position and its weight) instead of a K^2 rescan
// per vector, and a row is spread over several warps so that decode-sized batches still fill the machine.
// topk_w == nullptr: the routing weights were applied upstream (weight 1 here).
// =====================================================================================
constexpr int kMaxTopk = 32;

__global__ void __launch_bounds__(256)
combine_kernel(const __nv_bfloat16* __restrict__ out2, const int32_t* __restrict__ loc,
               const float* __restrict__ topk_w, __nv_bfloat16* __restrict__ y, int T, int K, int H) {
  const int vec_per_row = H / 8;
  const int chunks = (vec_per_row + 31) / 32;
  grid_dep_launch();
  grid_dep_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t u = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; u < (int64_t)T * chunks; u += warps) {
    const int t = (int)(u / chunks), c = (int)(u % chunks) * 32 + lane;
    const int p = (lane < K) ? loc[t * K + lane] : -1;
    const float wv = (lane < K) ? (topk_w != nullptr ? topk_w[t * K + lane] : 1.f) : 0.f;
    int rank = 0;
    for (int k = 0; k < K; ++k) {
      const int o = __shfl_sync(0xffffffffu, p, k);
      rank += (o >= 0 && o < p);
    }
    const int n = __popc(__ballot_sync(0xffffffffu, p >= 0));
    // lane i fetches the pair whose rank is i (positions are distinct)
    int ps = -1;
    float ws = 0.f;
    for (int k = 0; k < K; ++k) {
      const int o = __shfl_sync(0xffffffffu, p, k), r = __shfl_sync(0xffffffffu, rank, k);
      const float ow = __shfl_sync(0xffffffffu, wv, k);
      if (o >= 0 && r == lane) { ps = o; ws = ow; }
    }
    const bool active = c < vec_per_row;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int it = 0; it < n; ++it) {              // warp-uniform trip count: the shuffles need every lane
      const int pos = __shfl_sync(0xffffffffu, ps, it);
      const float wt = __shfl_sync(0xffffffffu, ws, it);
      if (active) {
        const uint4 v = *reinterpret_cast<const uint4*>(out2 + (int64_t)pos * H + c * 8);
        const __nv_bfloat16* d = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float contrib = __bfloat162float(__float2bfloat16_rn(__bfloat162float(d[i]) * wt));
          acc[i] = __bfloat162float(__float2bfloat16_rn(acc[i] + contrib));
        }
      }
    }
    if (active) {
      uint4 o;
      __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
      for (int i = 0; i < 8; ++i) ob[i] = __float2bfloat16_rn(acc[i]);
      *reinterpret_cast<uint4*>(y + (int64_t)t * H + c * 8) = o;
    }
  }
}

int launch_combine(const void* out2, const int32_t* loc, const float* topk_w, void* y, int T, int K, int H,
                   cudaStream_t st) {
  B200_CHECK_ARG(H % 8 == 0 && K <= kMaxTopk, "combine: H %% 8 != 0 or K > %d", kMaxTopk);
  if (T == 0) return 0;
  const int64_t units = (int64_t)T * ((H / 8 + 31) / 32);          // warps of work
  const int blocks = (int)std::min<int64_t>((units + 7) / 8, (int64_t)device_sm_count() * 16);
  B200_CHECK_CUDA(launch_chained(combine_kernel, dim3(blocks), dim3(256), 0, st, (const __nv_bfloat16*)out2, loc,
                                 topk_w, (__nv_bfloat16*)y, T, K, H));
  return 0;
}

// =====================================================================================
// expert-parallel combine: y[t,:] = sum over the slots s of rows[pos[t,s],:] (pos < 0: no row), added
// in fp32 in ascending slot order (slot = owner rank, i.e. ascending expert range) and rounded once.
// =====================================================================================
__global__ void __launch_bounds__(256)
gather_sum_kernel(const __nv_bfloat16* __restrict__ rows, const int32_t* __restrict__ pos,
                  __nv_bfloat16* __restrict__ y, int T, int S, int H) {
  const int vec_per_row = H / 8;
  grid_dep_launch();
  grid_dep_wait();
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < (int64_t)T * vec_per_row;
       g += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(g / vec_per_row), c = (int)(g % vec_per_row) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < S; ++s) {
      const int p = pos[(int64_t)t * S + s];
      if (p < 0) continue;
      const uint4 raw = *reinterpret_cast<const uint4*>(rows + (int64_t)p * H + c);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(b2[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    uint4 out;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(y + (int64_t)t * H + c) = out;
  }
}

int launch_gather_sum(const void* rows, const int32_t* pos, void* y, int T, int S, int H, cudaStream_t st) {
  B200_CHECK_ARG(H % 8 == 0 && S >= 1, "gather_sum: H %% 8 != 0 or no slots");
  if (T == 0) return 0;
  int64_t work = (int64_t)T * (H / 8);
  int blocks = (int)std::min<int64_t>((work + 255) / 256, device_sm_count() * 16);
  B200_CHECK_CUDA(launch_chained(gather_sum_kernel, dim3(blocks), dim3(256), 0, st, (const __nv_bfloat16*)rows, pos,
                                 (__nv_bfloat16*)y, T, S, H));
  return 0;
}

// =====================================================================================
// expert-parallel dispatch plan, one launch: which tokens travel to which rank and where they sit in
// the rank-major send buffer.  Rank d owns experts [d*epr, (d+1)*epr); token t goes to rank d once if
// any of its K experts lives there.  pos[t, d] = position of t in the send buffer (ascending rank,
// ascending token within a rank) or -1; counts[d] = tokens bound for rank d; rows[p] = token at
// send-buffer position p for p < sum(counts).  One CTA: every thread owns a contiguous run of
// tokens, per-rank running counts are scanned across the threads, so the order is fixed (no atomics).
// =====================================================================================
constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxWorld = 32;

__global__ void __launch_bounds__(kPlanThreads, 1)
ep_plan_kernel(const int32_t* __restrict__ ids, int T, int K, int epr, int W, int32_t* __restrict__ pos,
               int32_t* __restrict__ counts, int32_t* __restrict__ rows) {
  extern __shared__ int32_t cnt[];                 // [kPlanThreads][W], then offs[W]
  int32_t* offs = cnt + kPlanThreads * W;
  grid_dep_launch();
  grid_dep_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = (T + kPlanThreads - 1) / kPlanThreads;
  const int t0 = min(T, tid * chunk), t1 = min(T, t0 + chunk);
  auto needs = [&](int t) {
    uint32_t m = 0;
    for (int k = 0; k < K; ++k) {
      const int id = ids[(int64_t)t * K + k];
      const int d = min(max(id >= 0 ? id / epr : 0, 0), W - 1);
      m |= 1u << d;
    }
    return m;
  };
  for (int d = 0; d < W; ++d) cnt[tid * W + d] = 0;
  for (int t = t0; t < t1; ++t) {
    uint32_t m = needs(t);
    while (m) {
      const int d = __ffs(m) - 1;
      m &= m - 1;
      cnt[tid * W + d] += 1;
    }
  }
  __syncthreads();
  // exclusive scan over the threads, one warp per destination rank
  for (int d = warp; d < W; d += kPlanThreads / 32) {
    int run = 0;
    for (int base = 0; base < kPlanThreads; base += 32) {
      const int v = cnt[(base + lane) * W + d];
      int incl = v;
      for (int s = 1; s < 32; s <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, s);
        if (lane >= s) incl += o;
      }
      cnt[(base + lane) * W + d] = run + incl - v;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) offs[d] = run;            // total for rank d (turned into an offset below)
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int d = 0; d < W; ++d) {
      const int c = offs[d];
      counts[d] = c;
      offs[d] = run;
      run += c;
    }
  }
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const uint32_t m = needs(t);
    for (int d = 0; d < W; ++d) {
      int p = -1;
      if (m & (1u << d)) {
        p = offs[d] + cnt[tid * W + d];
        cnt[tid * W + d] += 1;
        rows[p] = t;
      }
      pos[(int64_t)t * W + d] = p;
    }
  }
}

int launch_ep_plan(const int32_t* ids, int T, int K, int epr, int W, int32_t* pos, int32_t* counts, int32_t* rows,
                   cudaStream_t st) {
  B200_CHECK_ARG(T >= 0 && K >= 1 && epr >= 1 && W >= 1 && W <= kPlanMaxWorld, "ep_plan: T=%d K=%d experts/rank=%d world=%d",
                 T, K, epr, W);
  const size_t smem = (size_t)(kPlanThreads * W + W) * sizeof(int32_t);
  B200_CHECK_CUDA(cudaFuncSetAttribute(ep_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  B200_CHECK_CUDA(launch_chained(ep_plan_kernel, dim3(1), dim3(kPlanThreads), smem, st, ids, T, K, epr, W, pos, counts, rows));
  return 0;
}

// =====================================================================================
// router: fp32 logits [T, E] -> top-k expert ids (descending score, ties to the lower id) and weights.
// One warp per token; lane l holds experts l, l+32, ...  softmax scores are exp(x - max) / sum, sigmoid
// scores 1 / (1 + exp(-x)); with `renorm` the k weights are divided by their sum (the softmax
// denominator cancels there, so it is never formed).
// =====================================================================================
constexpr int kRouteMaxPerLane = 32;          // E <= 1024

__global__ void __launch_bounds__(256)
route_topk_kernel(const float* __restrict__ logits, int T, int E, int K, int scoring, int renorm,
                  int32_t* __restrict__ ids, float* __restrict__ weights) {
  grid_dep_launch();
  grid_dep_wait();
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  for (int t = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); t < T; t += gridDim.x * warps_per_cta) {
    const float* row = logits + (int64_t)t * E;
    float v[kRouteMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      v[i] = (e < E) ? row[e] : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < E) {
        v[i] = (scoring == 0) ? expf(v[i] - mx) : 1.f / (1.f + expf(-v[i]));
        sum += v[i];
      } else {
        v[i] = -1.f;            // scores are non-negative: never selected
      }
    }
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    const float inv_all = (scoring == 0) ? 1.f / sum : 1.f;
    float wsum = 0.f, my_w = 0.f;     // lane k keeps the k-th selection
    int my_id = 0;
    for (int k = 0; k < K; ++k) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kRouteMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        if (v[i] > best) { best = v[i]; best_e = e; }     // ascending e within the lane: ties keep the lower id
      }
      for (int d = 16; d > 0; d >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, d);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, d);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
#pragma unroll
      for (int i = 0; i < kRouteMaxPerLane; ++i)
        if (lane + 32 * i == best_e) v[i] = -1.f;
      wsum += best;
      if ((k & 31) == lane) { my_w = best; my_id = best_e; }
      if ((k & 31) == 31 || k == K - 1) {          // flush a group of up to 32 selections (K > 32 is unusual)
        const int k0 = k & ~31;
        if (k0 + lane <= k) {
          ids[(int64_t)t * K + k0 + lane] = my_id;
          weights[(int64_t)t * K + k0 + lane] = my_w;      // scaled below
        }
      }
    }
    __syncwarp();
    const float scale = renorm ? 1.f / wsum : inv_all;
    for (int k = lane; k < K; k += 32) weights[(int64_t)t * K + k] *= scale;
  }
}

int launch_route_topk(const float* logits, int T, int E, int K, int scoring, int renorm, int32_t* ids, float* weights,
                      cudaStream_t st) {
  B200_CHECK_ARG(E >= 1 && E <= 32 * kRouteMaxPerLane && K >= 1 && K <= E, "route_topk: E=%d K=%d", E, K);
  B200_CHECK_ARG(scoring == 0 || scoring == 1, "route_topk: scoring=%d (0 softmax, 1 sigmoid)", scoring);
  if (T == 0) return 0;
  const int blocks = std::min((T + 7) / 8, device_sm_count() * 8);
  B200_CHECK_CUDA(launch_chained(route_topk_kernel, dim3(blocks), dim3(256), 0, st, logits, T, E, K, scoring, renorm, ids,
                                 weights));
  return 0;
}

// =====================================================================================
// weight-scale repack: [E, R, Kd/32] bytes -> [E, MT, KB, 2, 512] chunks in tensor-memory order.
// A chunk = 128 rows x 4 scales.  The two chunks of a group are the tiles one pipeline stage
// carries: gate rows [mt*128, +128) and up rows I + [mt*128, +128) of w1 (R = 2I), or rows
// [mt*256, +128) and [mt*256+128, +128) of w2 (R = H).  Rows / k-blocks that do not exist get
// exponent 127 (= 1.0).
// =====================================================================================
__global__ void __launch_bounds__(256)
repack_scales_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int E, int gateup, int rows,
                     int nsf, int MT, int KB) {
  const int64_t total = (int64_t)E * MT * KB * 2 * kSfChunk;
  const int R = gateup ? 2 * rows : rows;
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total;
       g += (int64_t)gridDim.x * blockDim.x) {
    int off = (int)(g % kSfChunk);
    int64_t c = g / kSfChunk;
    int part = (int)(c % 2); c /= 2;
    int kb = (int)(c % KB); c /= KB;
    int mt = (int)(c % MT);
    int e = (int)(c / MT);
    int r_local = (off >> 4) + 32 * ((off & 15) >> 2);
    int j = off & 3;
    int kidx = kb * 4 + j;
    int row_in = gateup ? mt * 128 + r_local : (2 * mt + part) * 128 + r_local;   // row inside its part
    int row = gateup ? part * rows + row_in : row_in;
    uint8_t v = 127;
    if (row_in < rows && kidx < nsf) v = src[((int64_t)e * R + row) * nsf + kidx];
    dst[g] = v;
  }
}

int launch_repack_scales(const void* w_s, void* out, int E, bool gateup, int rows, int Kd, cudaStream_t st) {
  const int KB = (int)round_up64(Kd, kKPad) / 128;
  const int MT = gateup ? (rows + 127) / 128 : (rows + 255) / 256;
  int64_t total = (int64_t)E * MT * KB * 2 * kSfChunk;
  int blocks = (int)std::min<int64_t>((total + 255) / 256, device_sm_count() * 32);
  repack_scales_kernel<<<blocks, 256, 0, st>>>((const uint8_t*)w_s, (uint8_t*)out, E, gateup ? 1 : 0, rows, Kd / 32,
                                               MT, KB);
  B200_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200moe
