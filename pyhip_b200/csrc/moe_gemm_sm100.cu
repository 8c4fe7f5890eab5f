// Grouped GEMMs of the MoE layer on the sm_100a tensor cores.
//
// Orientation ("swap-AB"): the MMA's M side holds 128 weight rows, its N side holds the token
// tile of one sorted block (N = 32/64/128), so ragged token counts cost N-padding, never M.
//     D[128 weight rows, N tokens] += W4[128, K] * A8[N, K]^T      (tcgen05.mma kind::mxf8f6f4)
// W4: MXFP4 weights streamed by TMA straight from HBM (FP4 in memory, unpacked to the 16-byte
//     aligned shared-memory form by the copy engine), E8M0 scale per 32 along K.
// A8: activations as two e4m3 terms (value + residual), each with E8M0 scales per 32 along K;
//     both terms accumulate into the same TMEM tile, which reproduces bf16 activations to
//     ~2^-9 relative without any dequantisation arithmetic in the main loop.
// Block scales travel shared memory -> tensor memory with tcgen05.cp and are consumed by the MMA.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2-5 = epilogue (one TMEM lane quadrant each).  Persistent CTAs walk the work list
// (sorted block, 128-row weight tile) in block-major order so that the CTAs running at the same
// time share activation tiles and neighbouring blocks of an expert share weight tiles in L2.
// All barrier waits are bounded; a wait that runs out sets status[] and the CTA unwinds
// (frees its tensor memory) instead of spinning.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <mutex>

#include "internal.h"
#include "ptx_sm100.cuh"

namespace b200moe {

constexpr int kThreads = 192;
constexpr int kTileM = 128;          // weight rows per MMA
constexpr int kTileK = 128;          // K per pipeline stage (4 MMA K-steps of 32)
constexpr int kATileBytes = kTileM * kTileK;   // FP4 unpacked to one byte per element in shared memory
constexpr int kATileTxBytes = kTileM * kTileK / 2;   // the copy engine counts the packed bytes it read
constexpr int kMaxStages = 12;
constexpr int kTmemCols = 512;
constexpr int kSfCol0 = 448;         // scale columns: 2 buffers x {A0, A1, Bhi, Blo} x 4 columns
constexpr int kSmemLimit = 232448;   // 227 KB

struct GemmParams {
  CUtensorMap tmA0, tmA1, tmBhi, tmBlo;
  const uint8_t* w_scale;
  const uint8_t* asf_hi;
  const uint8_t* asf_lo;
  const uint32_t* sorted_ids;
  const int32_t* sorted_e;
  const int32_t* num_valid;
  int32_t* status;
  __nv_bfloat16* h_out;
  uint8_t* oq_hi; uint8_t* oq_lo; uint8_t* osf_hi; uint8_t* osf_lo;
  __nv_bfloat16* out2;
  int64_t max_rows;
  int N, rows, KB, MT, E, topk, T, parts, stages, out_kp, out_kb, activation;
  float swiglu_limit;
};

struct SmemCtl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_word;
};

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float gateup_act(float g, float u, int activation, float limit) {
  // the oracle's matmuls return bf16, and its activation rounds to bf16 after silu and after
  // the product (tests/contrib/moe/test_moe.py:73-83,100-106): reproduce those roundings
  g = bf16r(g);
  u = bf16r(u);
  if (activation == B200MOE_ACT_SILU) {
    float s = bf16r(g / (1.f + __expf(-g)));
    return bf16r(s * u);
  }
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return bf16r(g * (1.f / (1.f + __expf(-1.702f * g))) * (u + 1.f));
}

template <bool GATEUP>
__global__ void __launch_bounds__(kThreads, 1)
moe_grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
  constexpr int NA = GATEUP ? 2 : 1;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle atoms
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(smem);
  uint8_t* stage0 = smem + 1024;
  const int N = p.N;
  const int b_bytes = N * kTileK;
  const int stage_bytes = NA * kATileBytes + 2 * b_bytes + 4 * kSfChunk;
  const uint32_t stage_tx = NA * kATileTxBytes + 2 * b_bytes + (NA + 2) * kSfChunk;
  const int S = p.stages;
  const int acc_stride = NA * N;
  const int n_acc = (2 * acc_stride <= 256) ? 2 : 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_word = &ctl->abort_word;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[a]), 4);
    }
    ctl->abort_word = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  const int64_t rows_live = min((int64_t)p.num_valid[0], p.max_rows);
  const int n_blocks = (int)(rows_live / N);
  const int total_work = n_blocks * p.MT;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&p.tmA0);
      if (GATEUP) prefetch_tensormap(&p.tmA1);
      prefetch_tensormap(&p.tmBhi);
      prefetch_tensormap(&p.tmBlo);
      int stage = 0;
      uint32_t phase = 0;
      int64_t issued = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int b = w / p.MT, m = w % p.MT;
        int e = p.sorted_e[b];
        if (e < 0 || e >= p.E) { p.status[2] = 1; e = 0; }
        const int r0 = b * N;
        const uint8_t* sfa = p.w_scale + ((int64_t)e * p.parts * p.MT + m) * p.KB * kSfChunk;
        const uint8_t* sfb_hi = p.asf_hi + (int64_t)b * p.KB * kSfChunk;
        const uint8_t* sfb_lo = p.asf_lo + (int64_t)b * p.KB * kSfChunk;
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1, abort_word, 0x100 + stage)) { ok = false; break; }
          uint8_t* st = stage0 + (size_t)stage * stage_bytes;
          const uint32_t full = smem_u32(&ctl->full[stage]);
          mbar_expect_tx(full, stage_tx);
          tma_load_3d(smem_u32(st), &p.tmA0, full, kb * kTileK, m * kTileM, e);
          if (GATEUP) tma_load_3d(smem_u32(st + kATileBytes), &p.tmA1, full, kb * kTileK, m * kTileM, e);
          uint8_t* sb = st + NA * kATileBytes;
          tma_load_2d(smem_u32(sb), &p.tmBhi, full, kb * kTileK, r0);
          tma_load_2d(smem_u32(sb + b_bytes), &p.tmBlo, full, kb * kTileK, r0);
          uint8_t* sf = sb + 2 * b_bytes;
          bulk_load(smem_u32(sf), sfa + (int64_t)kb * kSfChunk, kSfChunk, full);
          if (GATEUP)
            bulk_load(smem_u32(sf + kSfChunk), sfa + ((int64_t)p.MT * p.KB + kb) * kSfChunk, kSfChunk, full);
          bulk_load(smem_u32(sf + 2 * kSfChunk), sfb_hi + (int64_t)kb * kSfChunk, kSfChunk, full);
          bulk_load(smem_u32(sf + 3 * kSfChunk), sfb_lo + (int64_t)kb * kSfChunk, kSfChunk, full);
          ++issued;
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok || *abort_word) {
        // unwinding: let this CTA's copies still in flight land before shared memory is released
        const int64_t first = issued > S ? issued - S : 0;
        for (int64_t i = first; i < issued; ++i) {
          const uint32_t bar = smem_u32(&ctl->full[i % S]);
          const uint32_t par = (uint32_t)((i / S) & 1);
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(bar, par) && global_timer_ns() - t0 < 200000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      uint32_t sf_buf = 0;          // scale columns alternate between two TMEM buffers
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        if (!mbar_wait(smem_u32(&ctl->tmem_empty[acc]), acc_phase ^ 1, abort_word, 0x200 + acc)) break;
        tc_fence_after_sync();
        const uint32_t d0 = tmem_base + acc * acc_stride;
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_word, 0x300 + stage)) { ok = false; break; }
          tc_fence_after_sync();
          uint8_t* st = stage0 + (size_t)stage * stage_bytes;
          const uint32_t a0 = smem_u32(st);
          const uint32_t bh = a0 + NA * kATileBytes, bl = bh + b_bytes;
          const uint32_t sf = bl + b_bytes;
          const uint32_t sfc = tmem_base + kSfCol0 + sf_buf * 16;
          sf_buf ^= 1;
          tc_copy_sf_32x128b(sfc + 0, make_desc_sf(sf));
          if (GATEUP) tc_copy_sf_32x128b(sfc + 4, make_desc_sf(sf + kSfChunk));
          tc_copy_sf_32x128b(sfc + 8, make_desc_sf(sf + 2 * kSfChunk));
          tc_copy_sf_32x128b(sfc + 12, make_desc_sf(sf + 3 * kSfChunk));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t idesc = make_idesc_block_scaled(kFmtE2M1_f8f6f4, kFmtE4M3, kTileM, N, k, k);
            const uint32_t accum = (kb | k) != 0;
            const uint64_t da0 = make_desc_sw128(a0 + k * 32);
            const uint64_t dbh = make_desc_sw128(bh + k * 32);
            const uint64_t dbl = make_desc_sw128(bl + k * 32);
            mma_mxf8f6f4(d0, da0, dbh, idesc, sfc + 0, sfc + 8, accum);
            mma_mxf8f6f4(d0, da0, dbl, idesc, sfc + 0, sfc + 12, 1);
            if (GATEUP) {
              const uint64_t da1 = make_desc_sw128(a0 + kATileBytes + k * 32);
              mma_mxf8f6f4(d0 + N, da1, dbh, idesc, sfc + 4, sfc + 8, accum);
              mma_mxf8f6f4(d0 + N, da1, dbl, idesc, sfc + 4, sfc + 12, 1);
            }
          }
          tc_commit(smem_u32(&ctl->empty[stage]));
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(smem_u32(&ctl->tmem_full[acc]));
        if (n_acc == 2) { acc ^= 1; if (acc == 0) acc_phase ^= 1; } else { acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quad = warp & 3;                 // TMEM lanes [32*quad, 32*quad+32)
    const int row_local = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
      const int b = w / p.MT, m = w % p.MT;
      const int r0 = b * N;
      const int j = m * kTileM + row_local;    // output feature of this thread
      if (!mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_phase, abort_word, 0x400 + acc)) break;
      tc_fence_after_sync();
      const uint32_t t0 = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * acc_stride;
      for (int c0 = 0; c0 < N; c0 += 32) {
        uint32_t g[32], u[32];
        tmem_ld_32x32b_x32(t0 + c0, g);
        if (GATEUP) tmem_ld_32x32b_x32(t0 + N + c0, u);
        tmem_ld_wait();
        const uint32_t my_id = p.sorted_ids[r0 + c0 + lane];
        if (GATEUP) {
          const bool j_ok = j < p.rows;
          if (p.h_out != nullptr) {
#pragma unroll
            for (int n = 0; n < 32; ++n) {
              const uint32_t id = __shfl_sync(0xffffffffu, my_id, n);
              const int tok = (int)(id & 0xFFFFFFu), kk = (int)(id >> 24);
              const float v = gateup_act(__uint_as_float(g[n]), __uint_as_float(u[n]), p.activation,
                                         p.swiglu_limit);
              if (j_ok && kk < p.topk && tok < p.T)
                p.h_out[((int64_t)tok * p.topk + kk) * p.rows + j] = __float2bfloat16_rn(v);
            }
          } else {
            // fused re-quantisation of h into the operand format of the down GEMM; the 32
            // lanes of a warp are one 32-wide scale block along the feature axis
#pragma unroll
            for (int n = 0; n < 32; ++n) {
              float v = gateup_act(__uint_as_float(g[n]), __uint_as_float(u[n]), p.activation, p.swiglu_limit);
              if (!j_ok) v = 0.f;
              const int64_t r = (int64_t)r0 + c0 + n;
              // first term
              uint32_t amax = __reduce_max_sync(0xffffffffu, __float_as_uint(v) & 0x7fffffffu);
              int e1 = max((int)(amax >> 23) - 7, 0);
              float inv = __uint_as_float((uint32_t)(254 - e1) << 23);
              __nv_fp8_storage_t q1 = __nv_cvt_float_to_fp8(v * inv, __NV_SATFINITE, __NV_E4M3);
              float back = __half2float(__half(__nv_cvt_fp8_to_halfraw(q1, __NV_E4M3)));
              float res = v - back * __uint_as_float(e1 == 0 ? 0x00400000u : ((uint32_t)e1 << 23));
              // residual term
              uint32_t amax2 = __reduce_max_sync(0xffffffffu, __float_as_uint(res) & 0x7fffffffu);
              int e2 = max((int)(amax2 >> 23) - 7, 0);
              float inv2 = __uint_as_float((uint32_t)(254 - e2) << 23);
              __nv_fp8_storage_t q2 = __nv_cvt_float_to_fp8(res * inv2, __NV_SATFINITE, __NV_E4M3);
              p.oq_hi[r * p.out_kp + j] = q1;
              p.oq_lo[r * p.out_kp + j] = q2;
              if (lane == 0) {
                const int64_t off = ((int64_t)b * p.out_kb + m) * kSfChunk + sf_chunk_offset(c0 + n, quad);
                p.osf_hi[off] = (uint8_t)e1;
                p.osf_lo[off] = (uint8_t)e2;
              }
            }
          }
        } else {
          if (j < p.rows) {
#pragma unroll
            for (int n = 0; n < 32; ++n) {
              const int64_t r = (int64_t)r0 + c0 + n;
              p.out2[r * p.rows + j] = __float2bfloat16_rn(__uint_as_float(g[n]));
            }
          }
        }
        (void)my_id;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
      if (n_acc == 2) { acc ^= 1; if (acc == 0) acc_phase ^= 1; } else { acc_phase ^= 1; }
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (threadIdx.x == 0 && ctl->abort_word != 0) {
    p.status[0] = (int32_t)ctl->abort_word;
    p.status[1] = (int32_t)blockIdx.x;
  }
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------
// host side: tensor maps and launch
// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

static int encode_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base,
                      const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
                      CUtensorMapL2promotion promo, const char* what) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return set_error(-2, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, type, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(-3, "cuTensorMapEncodeTiled(%s) failed with CUresult %d (base %p dims %llu,%llu,%llu)", what,
                     (int)r, base, (unsigned long long)dims[0], (unsigned long long)dims[1],
                     (unsigned long long)(rank > 2 ? dims[2] : 0));
  return 0;
}

static int device_sm_count() {
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int& n = sms[dev & 63];
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

int launch_grouped_gemm(const GemmArgs& a, cudaStream_t st) {
  B200_CHECK_ARG(a.N == 32 || a.N == 64 || a.N == 128, "grouped gemm: token tile %d not in {32,64,128}", a.N);
  B200_CHECK_ARG(a.Kd % 32 == 0 && a.rows > 0 && a.E > 0, "grouped gemm: bad shape");
  B200_CHECK_ARG(a.max_rows % a.N == 0, "grouped gemm: max_rows %% N != 0");
  const int KP = (int)round_up64(a.Kd, kTileK);
  const int parts = a.gateup ? 2 : 1;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.N = a.N; p.rows = a.rows; p.KB = KP / kTileK; p.MT = (a.rows + kTileM - 1) / kTileM;
  p.E = a.E; p.topk = a.topk; p.T = a.T; p.parts = parts; p.activation = a.activation;
  p.swiglu_limit = a.swiglu_limit; p.max_rows = a.max_rows;
  p.w_scale = (const uint8_t*)a.w_scale; p.asf_hi = (const uint8_t*)a.asf_hi; p.asf_lo = (const uint8_t*)a.asf_lo;
  p.sorted_ids = a.sorted_ids; p.sorted_e = a.sorted_e; p.num_valid = a.num_valid; p.status = a.status;
  p.h_out = (__nv_bfloat16*)a.h_out; p.oq_hi = (uint8_t*)a.oq_hi; p.oq_lo = (uint8_t*)a.oq_lo;
  p.osf_hi = (uint8_t*)a.osf_hi; p.osf_lo = (uint8_t*)a.osf_lo; p.out_kp = a.out_kp; p.out_kb = a.out_kp / kTileK;
  p.out2 = (__nv_bfloat16*)a.out2;
  if (a.gateup && a.h_out == nullptr)
    B200_CHECK_ARG(a.out_kp == (int)round_up64(a.rows, kTileK) && a.oq_hi && a.oq_lo && a.osf_hi && a.osf_lo,
                   "gate-up: fused output buffers missing");

  // weights: FP4 pairs in memory, [E, parts*rows, KP/2] bytes
  const cuuint64_t row_pitch = (cuuint64_t)KP / 2;
  {
    cuuint64_t dims[3] = {(cuuint64_t)KP, (cuuint64_t)a.rows, (cuuint64_t)a.E};
    cuuint64_t strides[2] = {row_pitch, row_pitch * (cuuint64_t)a.rows * parts};
    cuuint32_t box[3] = {kTileK, kTileM, 1};
    const uint8_t* base = (const uint8_t*)a.w_data;
    int rc = encode_map(&p.tmA0, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, base, dims, strides, box,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "weights part 0");
    if (rc) return rc;
    if (a.gateup) {
      rc = encode_map(&p.tmA1, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, base + row_pitch * a.rows, dims, strides,
                      box, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "weights part 1");
      if (rc) return rc;
    }
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)KP, (cuuint64_t)a.max_rows};
    cuuint64_t strides[1] = {(cuuint64_t)KP};
    cuuint32_t box[2] = {kTileK, (cuuint32_t)a.N};
    int rc = encode_map(&p.tmBhi, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.a_hi, dims, strides, box,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "activations hi");
    if (rc) return rc;
    rc = encode_map(&p.tmBlo, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.a_lo, dims, strides, box,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "activations lo");
    if (rc) return rc;
  }

  const int stage_bytes = parts * kATileBytes + 2 * a.N * kTileK + 4 * kSfChunk;
  int stages = (kSmemLimit - 2048) / stage_bytes;
  stages = std::min(stages, kMaxStages);
  B200_CHECK_ARG(stages >= 2, "grouped gemm: tile does not fit shared memory");
  p.stages = stages;
  const size_t smem = 2048 + (size_t)stages * stage_bytes;

  const int64_t max_work = (a.max_rows / a.N) * p.MT;
  const int grid = (int)std::min<int64_t>(device_sm_count(), std::max<int64_t>(max_work, 1));
  static bool attr[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& done = attr[a.gateup ? 1 : 0][dev & 63];
  if (a.gateup) {
    if (!done)
      B200_CHECK_CUDA(cudaFuncSetAttribute(moe_grouped_gemm_kernel<true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    done = true;
    moe_grouped_gemm_kernel<true><<<grid, kThreads, smem, st>>>(p);
  } else {
    if (!done)
      B200_CHECK_CUDA(cudaFuncSetAttribute(moe_grouped_gemm_kernel<false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    done = true;
    moe_grouped_gemm_kernel<false><<<grid, kThreads, smem, st>>>(p);
  }
  B200_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------
// known-answer probes of the two hardware paths the main loop depends on
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1)
probe_tma_fp4_kernel(const __grid_constant__ CUtensorMap map, uint32_t* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_word;
  for (int i = threadIdx.x; i < kATileBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0xA5A5A5A5u;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_expect_tx(smem_u32(&bar), kATileTxBytes);
    tma_load_3d(smem_u32(smem), &map, smem_u32(&bar), 0, 0, 0);
    mbar_wait(smem_u32(&bar), 0, &abort_word, 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kATileBytes / 4; i += blockDim.x) out[i] = reinterpret_cast<uint32_t*>(smem)[i];
  if (threadIdx.x == 0) out[kATileBytes / 4] = abort_word;
}

__global__ void __launch_bounds__(128, 1) probe_utccp_kernel(const uint32_t* in, uint32_t* out) {
  __shared__ __align__(1024) uint8_t chunk[kSfChunk];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot, abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  reinterpret_cast<uint32_t*>(chunk)[threadIdx.x] = in[threadIdx.x];
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  if (threadIdx.x == 0) {
    tc_copy_sf_32x128b(tbase, make_desc_sf(smem_u32(chunk)));
    tc_commit(smem_u32(&bar));
    mbar_wait(smem_u32(&bar), 0, &abort_word, 2);
  }
  __syncthreads();
  tc_fence_after_sync();
  uint32_t r[4];
  tmem_ld_32x32b_x4(tbase + ((uint32_t)(warp * 32) << 16), r);
  tmem_ld_wait();
  for (int c = 0; c < 4; ++c) out[(warp * 32 + lane) * 4 + c] = r[c];
  if (threadIdx.x == 0) out[512] = abort_word;
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 32);
}

// Issue-rate probe: `count` dependent MMAs of shape 128 x N into `nacc` alternating accumulators,
// one commit, one bounded wait; reports clock cycles.  Operand contents are irrelevant (zeros).
__global__ void __launch_bounds__(128, 1) probe_mma_rate_kernel(const int32_t* cfg, uint32_t* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot, abort_word;
  const int kind = cfg[0], N = cfg[1], count = cfg[2], nacc = cfg[3];
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < (16384 + 32768 + 1024) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t a = smem_u32(smem), b = a + 16384, sf = b + 32768;
    tc_copy_sf_32x128b(tbase + 448, make_desc_sf(sf));
    tc_copy_sf_32x128b(tbase + 452, make_desc_sf(sf + 512));
    tc_copy_sf_32x128b(tbase + 456, make_desc_sf(sf));
    const long long t0 = clock64();
    for (int i = 0; i < count; ++i) {
      const int k = i & 3;
      const uint32_t d = tbase + (i % nacc) * N;
      if (kind == 0) {
        const uint32_t idesc = make_idesc_block_scaled(kFmtE2M1_f8f6f4, kFmtE4M3, 128, N, k, k);
        mma_mxf8f6f4(d, make_desc_sw128(a + k * 32), make_desc_sw128(b + k * 32), idesc, tbase + 448, tbase + 452,
                     i >= nacc);
      } else {
        const uint32_t idesc = make_idesc_block_scaled(kFmtE2M1_mxf4, kFmtE2M1_mxf4, 128, N, (k & 1) * 2, (k & 1) * 2);
        mma_mxf4(d, make_desc_sw128(a + (k & 1) * 32), make_desc_sw128(b + (k & 1) * 32), idesc, tbase + 448,
                 tbase + 452, i >= nacc);
      }
    }
    const long long t1 = clock64();
    tc_commit(smem_u32(&bar));
    mbar_wait(smem_u32(&bar), 0, &abort_word, 3);
    const long long t2 = clock64();
    out[0] = (uint32_t)(t1 - t0);
    out[1] = (uint32_t)(t2 - t0);
    out[2] = abort_word;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

int run_debug_probe(int which, const void* in, void* out, cudaStream_t st) {
  if (which == 1) {
    CUtensorMap map;
    cuuint64_t dims[3] = {128, 128, 1};
    cuuint64_t strides[2] = {64, 64 * 128};
    cuuint32_t box[3] = {128, 128, 1};
    int rc = encode_map(&map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, in, dims, strides, box,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, "probe tile");
    if (rc) return rc;
    probe_tma_fp4_kernel<<<1, 128, kATileBytes + 1024, st>>>(map, (uint32_t*)out);
    B200_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  if (which == 2) {
    probe_utccp_kernel<<<1, 128, 0, st>>>((const uint32_t*)in, (uint32_t*)out);
    B200_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  if (which == 3) {
    static bool attr = false;
    if (!attr) {
      B200_CHECK_CUDA(cudaFuncSetAttribute(probe_mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           65536));
      attr = true;
    }
    probe_mma_rate_kernel<<<1, 128, 16384 + 32768 + 1024 + 1024, st>>>((const int32_t*)in, (uint32_t*)out);
    B200_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  return set_error(-1, "debug_probe: unknown probe %d", which);
}

}  // namespace b200moe
