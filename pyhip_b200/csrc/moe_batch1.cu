// Batch-1 path: ONE token through the MXFP4 layer with no sort, no activation quantiser and no tensor cores -- the
// counterpart of the reference's moe_gemm_batch1 (src/contrib/moe.py:41-188: blocks take their expert straight from
// topk_ids[k], src/contrib/moe.py:79-84).  With one token every projection is a matrix-vector product that streams
// each weight row once, so the work is done where the bytes arrive: a warp owns an output feature, every lane
// takes one 32-element block (16 bytes of packed E2M1 + one E8M0 byte) per step, and the K pairs of the token are
// independent rows of independent experts.  Two launches: gate-up + activation, then down + the weighted sum over
// the token's K experts in ascending expert order with the oracle's bf16 roundings (deterministic, no atomics).
// Selected explicitly (method "batch1" of the Python call): on the gpt-oss shape it takes 38.6 us against 31.5 us for
// the sorted tensor-core path -- expanding E2M1 codes in the integer and half-precision pipes costs about nine
// million warp instructions per launch at half of the issue rate, which is more than the 53 MB of weights cost to
// stream -- so the default stays with the tensor cores even for one token.
//
// Arithmetic.  An E2M1 code placed at bits [11:9] of a 16-bit word with its sign at bit 15 IS the fp16 number
// value * 2^-14 (codes 0 and 1 land on fp16 zero / the fp16 subnormal 2^-15 = 0.5 * 2^-14), so eight codes become four
// half2 registers with shifts, masks and byte permutes -- no conversion instructions.  The vector operand is staged in
// shared memory as fp16, scaled by a power of two so that its largest element lies in [2^14, 2^15): elements down
// to 2^-28 of the largest stay normal fp16 numbers, and the products are the true products times the token's scale.
// A lane multiplies its block with HFMA2 into two half2 accumulators (16 products each), converts the block sum to
// fp32, applies the block's E8M0 scale there and accumulates blocks in fp32: the rounding of a 32-element fp16
// partial sum (about 2^-10 of it) is far below the bf16 rounding of the result that the oracle itself applies.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "gemm_common.cuh"

namespace b200moe {

namespace {

constexpr int kB1Threads = 256;          // 8 warps
constexpr int kB1Warps = kB1Threads / 32;
constexpr int kB1MaxK = 8;               // experts per token on this path
constexpr int kB1MaxIters = 8;           // 32-lane steps along a row: rows of up to 8 * 1024 elements

struct B1Params {
  const __nv_bfloat16* x;        // [H]
  const int32_t* ids;            // [K]
  const float* tw;               // [K]
  const int32_t* mask;           // [E_route] or null
  const int32_t* num_local;      // device scalar or null
  const uint8_t* w1;             // [E, 2I, H/2]
  const uint8_t* s1;             // [E, 2I, H/32]
  const uint8_t* w2;             // [E, H, I/2]
  const uint8_t* s2;             // [E, H, I/32]
  const float* bias1;            // [E, 2I] or null
  const float* bias2;            // [E, H] or null
  __nv_bfloat16* h;              // scratch [K, I]
  int32_t* le;                   // scratch [K]: local expert id of every pair, -1 = dropped
  __nv_bfloat16* y;              // [H]
  int H, I, K, E, E_route, activation, stage1;
  float swiglu_limit;
};

// eight E2M1 codes of one 32-bit word -> four half2 holding (e0,e2) (e4,e6) (e1,e3) (e5,e7), each value * 2^-14
__device__ __forceinline__ void e2m1x8_to_half2x4(uint32_t w, __half2 (&o)[4]) {
  // byte i of `ev` / `od` = fp16 high byte of the even / odd element of byte i: (code & 7) << 1 | sign << 7
  const uint32_t ev = ((w << 1) & 0x0E0E0E0Eu) | ((w << 4) & 0x80808080u);
  const uint32_t od = ((w >> 3) & 0x0E0E0E0Eu) | (w & 0x80808080u);
  const uint32_t h0 = __byte_perm(ev, 0u, 0x1404), h1 = __byte_perm(ev, 0u, 0x3424);
  const uint32_t h2 = __byte_perm(od, 0u, 0x1404), h3 = __byte_perm(od, 0u, 0x3424);
  o[0] = *reinterpret_cast<const __half2*>(&h0);
  o[1] = *reinterpret_cast<const __half2*>(&h1);
  o[2] = *reinterpret_cast<const __half2*>(&h2);
  o[3] = *reinterpret_cast<const __half2*>(&h3);
}

// Stage `nvec` bf16 vectors of n elements each (n % 32 == 0, vector v at src + v * n) into shared memory as fp16,
// all scaled by ONE power of two 2^sh that puts the largest magnitude of all of them in [2^14, 2^15).  Layout of a
// staged vector: 16-byte piece q (0..3) of 32-element block b sits at piece index q * (n / 32) + b, so the lanes of
// a warp, which take consecutive blocks, read consecutive 16-byte pieces (no bank conflicts); inside a piece the
// eight elements stand in the order e2m1x8_to_half2x4 produces (e0 e2 e4 e6 e1 e3 e5 e7).
// Returns the fp32 factor the fp16 dot products have to be multiplied by (2^14 for the weights' placement times
// 2^-sh).  All threads of the CTA call it; `red` is a shared float[kB1Warps].
__device__ __forceinline__ float stage_vectors_fp16(const __nv_bfloat16* __restrict__ src, int n, int nvec, __half* dst,
                                                    float* red) {
  const int total = n * nvec;
  float amax = 0.f;
  for (int i = threadIdx.x * 2; i < total; i += blockDim.x * 2) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i));
    amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
  }
  for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int i = 0; i < kB1Warps; ++i) amax = fmaxf(amax, red[i]);
  // biased exponent of amax -> scale 2^(141 - exp) puts amax in [2^14, 2^15); an all-zero (or denormal) input takes 1
  const int ex = (int)((__float_as_uint(amax) >> 23) & 0xFF);
  const int sh = ex == 0 ? 0 : 141 - ex;
  const float up = __uint_as_float((uint32_t)(127 + max(-126, min(127, sh))) << 23);
  const int nb = n / 32;
  for (int i = threadIdx.x * 2; i < total; i += blockDim.x * 2) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i));
    const int v = i / n, e = i - v * n;                 // e is even: elements e and e + 1 share a block and a piece
    const int b = e >> 5, q = (e >> 3) & 3, j = e & 7;
    __half* piece = dst + (int64_t)v * n + (q * nb + b) * 8;
    piece[j >> 1] = __float2half_rn(f.x * up);           // even element j     -> slot j / 2
    piece[4 + (j >> 1)] = __float2half_rn(f.y * up);     // odd element j + 1  -> slot 4 + j / 2
  }
  __syncthreads();
  return __uint_as_float((uint32_t)(127 + max(-126, min(127, 14 - sh))) << 23);
}

// fp32 dot product of one 32-element block: 16 packed bytes of E2M1 codes against 32 staged fp16 values
__device__ __forceinline__ float block_dot(const uint4& wq, const uint4 (&xv)[4]) {
  const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
  __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    __half2 hw[4];
    e2m1x8_to_half2x4(ww[q], hw);
    const __half2* hx = reinterpret_cast<const __half2*>(&xv[q]);
    a0 = __hfma2(hw[0], hx[0], a0);
    a1 = __hfma2(hw[1], hx[1], a1);
    a0 = __hfma2(hw[2], hx[2], a0);
    a1 = __hfma2(hw[3], hx[3], a1);
  }
  const float2 f = __half22float2(__hadd2(a0, a1));
  return f.x + f.y;
}

__device__ __forceinline__ float e8m0_to_float(uint32_t b) { return __uint_as_float(b << 23); }   // 2^(b-127); b = 0 reads as 0

// Local expert id of pair k, computed by the whole CTA (every thread gets the result): -1 when the id lies outside
// the routing space, the expert is masked out on this rank, or the token is padding (num_local_tokens < 1).  With a
// mask the local id is the number of unmasked experts below it.  `cnt` is a shared int.
__device__ __forceinline__ int local_expert(const B1Params& p, int k, int* cnt) {
  if (threadIdx.x == 0) *cnt = 0;
  __syncthreads();
  const int e = p.ids[k];
  const bool live = (p.num_local == nullptr || p.num_local[0] >= 1) && e >= 0 && e < p.E_route &&
                    (p.mask == nullptr || p.mask[e] != 0);
  if (live && p.mask != nullptr) {
    int c = 0;
    for (int i = threadIdx.x; i < e; i += blockDim.x) c += p.mask[i] != 0;
    if (c) atomicAdd(cnt, c);           // a count: its value does not depend on the order of the adds
  }
  __syncthreads();
  const int le = !live ? -1 : (p.mask == nullptr ? e : *cnt);
  __syncthreads();                       // `cnt` may be reused by the next call
  return (le >= 0 && le < p.E) ? le : -1;
}

// One lane's share of NR packed weight rows: blocks lane, lane + 32, ... (ITERS of them), fetched together so that
// all loads are in flight at once; a row whose pointer is null is skipped and yields 0.
template <int ITERS, int NR>
struct RowLoads {
  uint4 q[NR][ITERS];
  uint32_t sc[NR][ITERS];
};
template <int ITERS, int NR>
__device__ __forceinline__ void load_rows(RowLoads<ITERS, NR>& L, const uint8_t* const (&wrow)[NR],
                                          const uint8_t* const (&srow)[NR], int nb, int lane) {
#pragma unroll
  for (int r = 0; r < NR; ++r) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int blk = it * 32 + lane;
      L.q[r][it] = make_uint4(0, 0, 0, 0);
      L.sc[r][it] = 0;
      if (wrow[r] != nullptr && blk < nb) {
        L.q[r][it] = __ldg(reinterpret_cast<const uint4*>(wrow[r]) + blk);
        L.sc[r][it] = __ldg(srow[r] + blk);
      }
    }
  }
}
// ... and their dot products with staged vectors (SHARED: all rows multiply the same vector, read once)
template <int ITERS, int NR, bool SHARED>
__device__ __forceinline__ void dot_rows(const RowLoads<ITERS, NR>& L, const __half* const (&vec)[NR], int nb, int lane,
                                         float (&out)[NR]) {
#pragma unroll
  for (int r = 0; r < NR; ++r) out[r] = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int blk = it * 32 + lane;
    if (blk < nb) {
      uint4 xv[4];
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        if (r == 0 || !SHARED) {
          const uint4* s = reinterpret_cast<const uint4*>(vec[r]);
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) xv[qq] = s[qq * nb + blk];
        }
        out[r] = fmaf(block_dot(L.q[r][it], xv), e8m0_to_float(L.sc[r][it]), out[r]);
      }
    }
  }
}

// ---- launch 1: h[k, f] = act(x . W1[e_k, f], x . W1[e_k, I + f]) -- grid (feature groups, K)
template <int ITERS>
__global__ void __launch_bounds__(kB1Threads)
batch1_gateup_kernel(const B1Params p, int feats_per_cta) {
  extern __shared__ __align__(16) uint8_t smem_b1[];
  __half* xs = reinterpret_cast<__half*>(smem_b1);           // [H] staged vector
  __shared__ float red[kB1Warps];
  __shared__ int cnt;
  grid_dep_launch();
  grid_dep_wait();
  const int k = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int le = local_expert(p, k, &cnt);
  if (blockIdx.x == 0 && threadIdx.x == 0) p.le[k] = le;
  if (le < 0) return;
  const float undo = stage_vectors_fp16(p.x, p.H, 1, xs, red);
  const int nb = p.H / 32;
  const int64_t row_bytes = p.H / 2;
  const uint8_t* wbase = p.w1 + (int64_t)le * 2 * p.I * row_bytes;
  const uint8_t* sbase = p.s1 + (int64_t)le * 2 * p.I * nb;
  const float tw = p.stage1 ? p.tw[k] : 1.f;
  const int f0 = blockIdx.x * feats_per_cta, f_end = min(f0 + feats_per_cta, p.I);
  const __half* const vr[2] = {xs, xs};
  auto fetch = [&](RowLoads<ITERS, 2>& L, int f) {
    const bool on = f < f_end;
    const uint8_t* const wr[2] = {on ? wbase + (int64_t)f * row_bytes : nullptr, on ? wbase + (int64_t)(p.I + f) * row_bytes : nullptr};
    const uint8_t* const sr[2] = {sbase + (int64_t)(on ? f : 0) * nb, sbase + (int64_t)(on ? p.I + f : 0) * nb};
    load_rows<ITERS, 2>(L, wr, sr, nb, lane);
  };
  for (int f = f0 + warp; f < f_end; f += kB1Warps) {
    RowLoads<ITERS, 2> cur;
    fetch(cur, f);
    float part[2];
    dot_rows<ITERS, 2, true>(cur, vr, nb, lane, part);
    float ag = part[0], au = part[1];
    for (int d = 16; d > 0; d >>= 1) {
      ag += __shfl_xor_sync(0xffffffffu, ag, d);
      au += __shfl_xor_sync(0xffffffffu, au, d);
    }
    if (lane == 0) {
      float g = ag * undo, u = au * undo;
      if (p.bias1 != nullptr) {       // the oracle's matmul returns bf16 and the bias is added to that
        g = bf16r(g) + p.bias1[(int64_t)le * 2 * p.I + f];
        u = bf16r(u) + p.bias1[(int64_t)le * 2 * p.I + p.I + f];
      }
      float v = gateup_act(g, u, p.activation, p.swiglu_limit);
      if (p.stage1) v *= tw;
      p.h[(int64_t)k * p.I + f] = __float2bfloat16_rn(v);
    }
  }
}

// ---- launch 2: y[n] = sum over the token's experts, ascending expert id, of bf16(bf16(h_k . W2[e_k, n] (+ b2)) * w_k)
template <int ITERS>
__global__ void __launch_bounds__(kB1Threads)
batch1_down_kernel(const B1Params p, int feats_per_cta) {
  extern __shared__ __align__(16) uint8_t smem_b1[];
  __half* hs = reinterpret_cast<__half*>(smem_b1);           // [K][I] staged vectors
  __shared__ float red[kB1Warps];
  __shared__ int le_s[kB1MaxK], order_s[kB1MaxK];
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K;
  if (threadIdx.x < K) le_s[threadIdx.x] = p.le[threadIdx.x];
  __syncthreads();
  // rows of dropped pairs were never written by the first launch: clear them before the common scale is taken
  for (int k = 0; k < K; ++k)
    if (le_s[k] < 0)
      for (int i = threadIdx.x; i < p.I; i += blockDim.x) p.h[(int64_t)k * p.I + i] = __float2bfloat16_rn(0.f);
  __syncthreads();
  const float undo = stage_vectors_fp16(p.h, p.I, K, hs, red);
  if (threadIdx.x == 0) {
    // the token's pairs in ascending expert id (ties keep k order): the order of the oracle's index_add_ loop
    int n = 0;
    for (int k = 0; k < K; ++k) if (le_s[k] >= 0) order_s[n++] = k;
    for (int i = 1; i < n; ++i) {
      const int kk = order_s[i];
      int j = i - 1;
      while (j >= 0 && p.ids[order_s[j]] > p.ids[kk]) { order_s[j + 1] = order_s[j]; --j; }
      order_s[j + 1] = kk;
    }
    for (int i = n; i < K; ++i) order_s[i] = -1;
  }
  __syncthreads();
  const int nb = p.I / 32;
  const int64_t row_bytes = p.I / 2;
  const int n0 = blockIdx.x * feats_per_cta, n_end = min(n0 + feats_per_cta, p.H);
  // two rows (experts) per step: few registers per thread, so that many warps stream at once
  for (int n = n0 + warp; n < n_end; n += kB1Warps) {
    float acc[kB1MaxK];
#pragma unroll
    for (int k0 = 0; k0 < kB1MaxK; k0 += 2) {
      if (k0 < K) {
        const uint8_t* wr[2];
        const uint8_t* sr[2];
        const __half* vr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int k = k0 + r;
          const bool on = k < K && le_s[k] >= 0;
          const int64_t row = on ? (int64_t)le_s[k] * p.H + n : 0;
          wr[r] = on ? p.w2 + row * row_bytes : nullptr;
          sr[r] = p.s2 + row * nb;
          vr[r] = hs + (int64_t)(on ? k : 0) * p.I;
        }
        RowLoads<ITERS, 2> L;
        load_rows<ITERS, 2>(L, wr, sr, nb, lane);
        float part[2];
        dot_rows<ITERS, 2, false>(L, vr, nb, lane, part);
#pragma unroll
        for (int r = 0; r < 2; ++r) acc[k0 + r] = part[r];
      } else {
#pragma unroll
        for (int r = 0; r < 2; ++r) acc[k0 + r] = 0.f;
      }
    }
#pragma unroll
    for (int k = 0; k < kB1MaxK; ++k) {
      if (k < K) {
        for (int d = 16; d > 0; d >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], d);
        acc[k] *= undo;
      }
    }
    if (lane == 0) {
      float y = 0.f;
      for (int i = 0; i < K; ++i) {
        const int k = order_s[i];
        if (k < 0) break;
        float o = 0.f;
#pragma unroll
        for (int kk = 0; kk < kB1MaxK; ++kk) if (kk == k) o = acc[kk];
        o = bf16r(o);
        if (p.bias2 != nullptr) o = bf16r(o + p.bias2[(int64_t)le_s[k] * p.H + n]);
        const float w = p.stage1 ? 1.f : p.tw[k];
        y = bf16r(y + bf16r(o * w));
      }
      p.y[n] = __float2bfloat16_rn(y);
    }
  }
}

}  // namespace

int64_t batch1_scratch_bytes(int K, int I) { return round_up64((int64_t)K * I * 2, 256) + 256; }

int launch_forward_batch1(const void* x, const int32_t* ids, const float* tw, const int32_t* mask, const int32_t* num_local,
                          const void* w1, const void* s1, const void* w2, const void* s2, const float* bias1,
                          const float* bias2, void* scratch, void* y, int H, int I, int K, int E, int E_route,
                          int activation, float swiglu_limit, int stage1, cudaStream_t st) {
  B200_CHECK_ARG(K >= 1 && K <= kB1MaxK, "forward_batch1: top-k %d outside [1,%d]", K, kB1MaxK);
  B200_CHECK_ARG(H % 32 == 0 && I % 32 == 0 && H <= kB1MaxIters * 1024 && I <= kB1MaxIters * 1024,
                 "forward_batch1: H=%d / I=%d must be multiples of 32 up to %d", H, I, kB1MaxIters * 1024);
  B200_CHECK_ARG(((uintptr_t)w1 & 15) == 0 && ((uintptr_t)w2 & 15) == 0 && ((uintptr_t)scratch & 15) == 0,
                 "forward_batch1: weights and scratch must be 16-byte aligned");
  B1Params p;
  memset(&p, 0, sizeof(p));
  p.x = (const __nv_bfloat16*)x; p.ids = ids; p.tw = tw; p.mask = mask; p.num_local = num_local;
  p.w1 = (const uint8_t*)w1; p.s1 = (const uint8_t*)s1; p.w2 = (const uint8_t*)w2; p.s2 = (const uint8_t*)s2;
  p.bias1 = bias1; p.bias2 = bias2;
  p.h = (__nv_bfloat16*)scratch;
  p.le = (int32_t*)((uint8_t*)scratch + round_up64((int64_t)K * I * 2, 256));
  p.y = (__nv_bfloat16*)y;
  p.H = H; p.I = I; p.K = K; p.E = E; p.E_route = E_route; p.activation = activation; p.stage1 = stage1;
  p.swiglu_limit = swiglu_limit;
  const size_t smem1 = (size_t)H * 2, smem2 = (size_t)K * I * 2;
  B200_CHECK_ARG(smem1 <= 200 * 1024 && smem2 <= 200 * 1024, "forward_batch1: vectors do not fit shared memory");
  const int sms = device_sm_count();
  // Features per CTA: the smallest multiple of the warp count for which the whole grid is resident at once (every
  // CTA stages the vector operand first, so a second wave would pay that again behind the first).
  auto launch = [&](auto kernel, int feats_total, int grid_y, size_t smem) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    int per_sm = 1;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kB1Threads, smem);
    if (e != cudaSuccess) return e;
    const int64_t cap = (int64_t)sms * std::max(per_sm, 1);
    int f = kB1Warps;
    while ((int64_t)((feats_total + f - 1) / f) * grid_y > cap && f < feats_total) f += kB1Warps;
    return launch_chained(kernel, dim3((feats_total + f - 1) / f, grid_y), dim3(kB1Threads), smem, st, p, f);
  };
  auto launch1 = [&](auto kernel) { return launch(kernel, I, K, smem1); };
  auto launch2 = [&](auto kernel) { return launch(kernel, H, 1, smem2); };
  const int it1 = (H / 32 + 31) / 32, it2 = (I / 32 + 31) / 32;      // 32-lane steps along a row of each projection
  switch (it1) {
    case 1: B200_CHECK_CUDA(launch1(batch1_gateup_kernel<1>)); break;
    case 2: B200_CHECK_CUDA(launch1(batch1_gateup_kernel<2>)); break;
    case 3: B200_CHECK_CUDA(launch1(batch1_gateup_kernel<3>)); break;
    case 4: B200_CHECK_CUDA(launch1(batch1_gateup_kernel<4>)); break;
    default: B200_CHECK_CUDA(launch1(batch1_gateup_kernel<kB1MaxIters>)); break;
  }
  switch (it2) {
    case 1: B200_CHECK_CUDA(launch2(batch1_down_kernel<1>)); break;
    case 2: B200_CHECK_CUDA(launch2(batch1_down_kernel<2>)); break;
    case 3: B200_CHECK_CUDA(launch2(batch1_down_kernel<3>)); break;
    case 4: B200_CHECK_CUDA(launch2(batch1_down_kernel<4>)); break;
    default: B200_CHECK_CUDA(launch2(batch1_down_kernel<kB1MaxIters>)); break;
  }
  B200_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200moe
