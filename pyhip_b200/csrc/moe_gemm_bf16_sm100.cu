// Grouped GEMMs of the MoE layer for UNQUANTISED (bf16) expert weights: tcgen05.mma kind::f16, bf16 x bf16 with
// fp32 accumulation in tensor memory -- the arithmetic of the reference's QuantType.No path
// (src/contrib/fused_moe.py:253; torch form tests/contrib/moe/test_moe.py:86-118).
//
// Same orientation and work list as the block-scaled kernels: the MMA's M side holds 128 weight rows, its N side the
// token tile of one sorted block (B rows, a multiple of 16),
//     D[128 weight rows, tokens] += W[128, K] * A[tokens, K]^T
// and a pipeline stage (K = 64 elements = 128-byte rows = one swizzle span) carries TWO 128-row weight tiles that
// share one token tile: gate and up rows of the same features, or two consecutive row tiles of the down projection.
// A stage is two copy instructions (one 4-D TMA for the weights, one 3-D TMA for the token rows); K and row tails
// are filled with zeros by the copy engine.  The token rows are bf16 in sorted-row order: the layer input is copied
// there once per token by the launch in front, the gate-up epilogue writes h there directly (bf16, as the oracle's h).
//
// Warp roles (352 threads): warp 0 TMA producer; warps 1 and 10 MMA issuers, one per weight tile of the stage
// (warp 1 owns the tensor memory); warps 2-9 epilogue, two per TMEM lane quadrant.  Two accumulator buffers of
// 2 x B columns overlap a tile's epilogue with the next tile's main loop.  Every barrier wait is bounded; a wait
// that runs out sets status[] and the CTA unwinds and frees its tensor memory.
#include <cuda_bf16.h>

#include <algorithm>

#include "gemm_common.cuh"

namespace b200moe {

namespace {

constexpr int kThreadsH = 352;
constexpr int kMma2WarpH = 10;
constexpr int kTileMH = 128;                        // weight rows per MMA
constexpr int kTileKH = 64;                         // bf16 elements of K per stage
constexpr int kRowBytesH = kTileKH * 2;             // 128 bytes = one swizzle span
constexpr int kATileBytesH = kTileMH * kRowBytesH;  // 16 KB
constexpr int kMaxStagesH = 16;
constexpr int kTmemColsH = 512;
constexpr int kSmemLimitH = 232448;                 // 227 KB

struct Bf16Params {
  CUtensorMap tmW;     // weights: gate-up (K, I, 2, E) box (64,128,2,1); down (K, H, 1, E) box (64,256,1,1)
  CUtensorMap tmA;     // token rows (K, max_rows, 1) box (64, B, 1)
  const uint32_t* sorted_ids;
  const int32_t* sorted_e;
  const int32_t* num_valid;
  int32_t* status;
  __nv_bfloat16* h_sorted;   // gate-up output: bf16 [max_rows, rows] in sorted-row order
  __nv_bfloat16* out2;       // down output, gather form: bf16 [max_rows, rows]
  __nv_bfloat16* y;          // down output, fused combine: zeroed bf16 [T, rows]; or null
  const float* sorted_w;
  const float* bias;
  int64_t max_rows;
  int B, rows, KB, MT, E, topk, T, stages, activation, k_tail_steps, weight_stage1;
  float swiglu_limit;
};

struct SmemCtlH {
  uint64_t full[kMaxStagesH];
  uint64_t empty[kMaxStagesH];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_word;
};

// Instruction descriptor of the dense kinds: [4,6) D format (1 = f32)  [7,10) A format  [10,13) B format (1 = bf16)
// [15] A major  [16] B major (0 = K-major)  [17,23) N>>3  [24,29) M>>4
__device__ __forceinline__ uint32_t make_idesc_bf16(uint32_t M, uint32_t N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, bf16 x bf16, K = 16 per instruction
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw)
      : "memory");
}

template <bool GATEUP>
__global__ void __launch_bounds__(kThreadsH, 1)
moe_grouped_gemm_bf16_kernel(const __grid_constant__ Bf16Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemCtlH* ctl = reinterpret_cast<SmemCtlH*>(smem);
  const uint32_t stage0 = smem_u32(smem) + 1024;
  const int B = p.B, S = p.stages;
  const int a_bytes = 2 * kATileBytesH, b_bytes = B * kRowBytesH;
  const int stage_bytes = (a_bytes + b_bytes + 1023) & ~1023;
  const int ncol = B, acc_cols = 2 * B;            // two accumulators of B columns per buffer, two buffers
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_word = &ctl->abort_word;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 2);      // one commit per MMA warp
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tmem_full[a]), 2);
      mbar_init(smem_u32(&ctl->tmem_empty[a]), 8);
    }
    ctl->abort_word = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemColsH);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  grid_dep_launch();   // tensor memory is held: the next kernel's CTAs may be scheduled
  grid_dep_wait();     // predecessor complete: sort arrays and token rows are valid

  const int64_t rows_live = min((int64_t)p.num_valid[0], p.max_rows);
  const int n_blocks = (int)(rows_live / B);
  const int total_work = n_blocks * p.MT;
  const int w_first = (int)blockIdx.x, w_step = (int)gridDim.x;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&p.tmW);
      prefetch_tensormap(&p.tmA);
      int stage = 0;
      uint32_t phase = 0;
      int64_t issued = 0;
      bool ok = true;
      for (int w = w_first; w < total_work && ok; w += w_step) {
        const int b = w / p.MT, m = w - b * p.MT;
        int e = p.sorted_e[b];
        if (e < 0 || e >= p.E) { p.status[2] = 1; e = 0; }
        const int r0 = b * B;
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1, abort_word, 0x100 + stage)) { ok = false; break; }
          const uint32_t st = stage0 + (uint32_t)stage * stage_bytes;
          const uint32_t full = smem_u32(&ctl->full[stage]);
          mbar_expect_tx(full, (uint32_t)(a_bytes + b_bytes));
          tma_load_4d(st, &p.tmW, full, kb * kTileKH, m * (GATEUP ? kTileMH : 2 * kTileMH), 0, e);
          tma_load_3d(st + a_bytes, &p.tmA, full, kb * kTileKH, r0, 0);
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
  } else if (warp == 1 || warp == kMma2WarpH) {
    // ------------------------------------------------------------------ MMA issuers
    const uint32_t part = (warp == 1) ? 0u : 1u;
    const uint32_t idesc = make_idesc_bf16(kTileMH, (uint32_t)B);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // the MMAs cover only the live rows of the block (rounded up to 16); the row ids of the NEXT item are fetched
    // while the current one is multiplied
    uint32_t nid[4];
    auto fetch_ids = [&](int w, uint32_t (&r)[4]) {
      const int r0 = (w / p.MT) * B;
#pragma unroll
      for (int q = 0; q < 4; ++q) r[q] = (w < total_work && q * 32 + lane < B) ? p.sorted_ids[r0 + q * 32 + lane] : 0xFFFFFFFFu;
    };
    fetch_ids(w_first, nid);
    for (int w = w_first; w < total_work && ok; w += w_step) {
      int nlive = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q)
        nlive += __popc(__ballot_sync(0xffffffffu, (int)(nid[q] >> 24) < p.topk && (int)(nid[q] & 0xFFFFFFu) < p.T));
      fetch_ids(w + w_step, nid);
      const uint32_t n_mma = (uint32_t)min(B, max(16, (nlive + 15) & ~15));
      const uint32_t idesc_w = (idesc & ~(0x3Fu << 17)) | ((n_mma >> 3) << 17);
      if (!mbar_wait(smem_u32(&ctl->tmem_empty[acc]), acc_phase ^ 1, abort_word, 0x200 + acc)) break;
      tc_fence_after_sync();
      const uint32_t d0 = tmem_base + acc * acc_cols + part * ncol;
      for (int kb = 0; kb < p.KB; ++kb) {
        if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_word, 0x300 + stage)) { ok = false; break; }
        tc_fence_after_sync();
        __syncwarp();
        if (elect_one()) {
          const uint32_t st = stage0 + (uint32_t)stage * stage_bytes;
          const uint32_t a_lo = desc_lo_sw(st + part * kATileBytesH);
          const uint32_t b_lo = desc_lo_sw(st + a_bytes);
          const int nsteps = (kb == p.KB - 1) ? p.k_tail_steps : 4;   // skip k-steps that are all padding
#pragma unroll
          for (int s = 0; s < 4; ++s)
            if (s < nsteps) umma_bf16(d0, a_lo + 2 * s, b_lo + 2 * s, idesc_w, (kb != 0 || s != 0) ? 1u : 0u);
          tc_commit(smem_u32(&ctl->empty[stage]));
        }
        __syncwarp();
        if (++stage == S) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (lane == 0) tc_commit(smem_u32(&ctl->tmem_full[acc]));
      __syncwarp();
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    // warp w reads TMEM lanes [32*(w%4), +32); the two warps of a quadrant split the token columns in alternating
    // groups of 16.  A lane holds one output feature; a pair of lanes swaps one value per two token columns so that
    // every lane stores two neighbouring features of one token as one 4-byte word.
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int half = ew >> 2;
    const int row_local = quad * 32 + lane;
    const bool odd = lane & 1;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = w_first; w < total_work; w += w_step) {
      const int b = w / p.MT, m = w - b * p.MT;
      const int r0 = b * B;
      // output feature of this thread: gate-up pairs gate/up of feature j; down holds j and j+128
      const int j = (GATEUP ? m * kTileMH : m * 2 * kTileMH) + row_local;
      const int jp = j & ~1;
      int nvalid = 0;
      for (int q = 0; q < B; q += 32) {
        const uint32_t id = (q + lane < B) ? p.sorted_ids[r0 + q + lane] : 0xFFFFFFFFu;
        nvalid += __popc(__ballot_sync(0xffffffffu, (int)(id >> 24) < p.topk && (int)(id & 0xFFFFFFu) < p.T));
      }
      const bool ok = mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_phase, abort_word, 0x400 + acc);
      if (!epi_all(ok)) break;
      tc_fence_after_sync();
      const uint32_t t0 = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * acc_cols;
      const bool j_ok = j < p.rows;
      const bool j2_ok = !GATEUP && j + kTileMH < p.rows;
      float bias0 = 0.f, bias1 = 0.f;
      if (p.bias != nullptr) {
        int e = p.sorted_e[b];
        if (e < 0 || e >= p.E) e = 0;
        const float* be = p.bias + (int64_t)e * (GATEUP ? 2 : 1) * p.rows;
        if (j_ok) bias0 = be[j];
        if (GATEUP ? j_ok : j2_ok) bias1 = be[j + (GATEUP ? p.rows : kTileMH)];
      }
      const bool col_weights = GATEUP ? (p.weight_stage1 != 0) : (p.y != nullptr);
      for (int c0 = half * 16; c0 < nvalid; c0 += 32) {
        uint32_t g[16], u[16];
        tmem_ld_32x32b_x16(t0 + c0, g);
        tmem_ld_32x32b_x16(t0 + ncol + c0, u);
        tmem_ld_wait();
        if (p.bias != nullptr) {
          // the oracle's matmul returns bf16 and the bias is added to that (one more rounding follows below)
#pragma unroll
          for (int n = 0; n < 16; ++n) {
            g[n] = __float_as_uint(bf16r(__uint_as_float(g[n])) + bias0);
            u[n] = __float_as_uint(bf16r(__uint_as_float(u[n])) + bias1);
          }
        }
        float my_w = 1.f;      // routing weight of the chunk's token columns (lane n holds column c0 + n)
        if (col_weights && p.sorted_w != nullptr) my_w = p.sorted_w[min(r0 + c0 + (lane & 15), r0 + B - 1)];
        if (GATEUP) {
          // h = act(gate, up) with the oracle's bf16 roundings, stored bf16 at its sorted row
#pragma unroll
          for (int n = 0; n < 16; n += 2) {
            if (c0 + n < nvalid) {
              float v0 = gateup_act(__uint_as_float(g[n]), __uint_as_float(u[n]), p.activation, p.swiglu_limit);
              float v1 = gateup_act(__uint_as_float(g[n + 1]), __uint_as_float(u[n + 1]), p.activation, p.swiglu_limit);
              if (p.weight_stage1) {
                v0 *= __shfl_sync(0xffffffffu, my_w, n);
                v1 *= __shfl_sync(0xffffffffu, my_w, n + 1);
              }
              const float rv = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);
              const int col = c0 + n + (odd ? 1 : 0);
              if (col < nvalid && j_ok)
                *reinterpret_cast<__nv_bfloat162*>(p.h_sorted + ((int64_t)r0 + col) * p.rows + jp) =
                    odd ? __floats2bfloat162_rn(rv, v1) : __floats2bfloat162_rn(v0, rv);
            }
          }
        } else if (p.y == nullptr) {
#pragma unroll
          for (int n = 0; n < 16; n += 2) {
            if (c0 + n < nvalid) {
              const float rg = __shfl_xor_sync(0xffffffffu, __uint_as_float(odd ? g[n] : g[n + 1]), 1);
              const float ru = __shfl_xor_sync(0xffffffffu, __uint_as_float(odd ? u[n] : u[n + 1]), 1);
              const int col = c0 + n + (odd ? 1 : 0);
              if (col < nvalid) {
                __nv_bfloat16* row = p.out2 + ((int64_t)r0 + col) * p.rows + jp;
                if (j_ok)
                  *reinterpret_cast<__nv_bfloat162*>(row) = odd ? __floats2bfloat162_rn(rg, __uint_as_float(g[n + 1]))
                                                                : __floats2bfloat162_rn(__uint_as_float(g[n]), rg);
                if (j2_ok)
                  *reinterpret_cast<__nv_bfloat162*>(row + kTileMH) =
                      odd ? __floats2bfloat162_rn(ru, __uint_as_float(u[n + 1])) : __floats2bfloat162_rn(__uint_as_float(u[n]), ru);
              }
            }
          }
        } else {
          // fused combine: y[token, feature] += bf16(bf16(acc) * routing weight) with packed bf16x2 reductions
          // (the reference's epilogue: src/contrib/moe.py:703-787)
          const uint32_t my_id = p.sorted_ids[min(r0 + c0 + (lane & 15), r0 + B - 1)];
#pragma unroll
          for (int n = 0; n < 16; n += 2) {
            if (c0 + n < nvalid) {
              const float w0 = __shfl_sync(0xffffffffu, my_w, n), w1 = __shfl_sync(0xffffffffu, my_w, n + 1);
              const uint32_t id = __shfl_sync(0xffffffffu, my_id, n + (odd ? 1 : 0));
              const float g0 = bf16r(bf16r(__uint_as_float(g[n])) * w0), g1 = bf16r(bf16r(__uint_as_float(g[n + 1])) * w1);
              const float u0 = bf16r(bf16r(__uint_as_float(u[n])) * w0), u1 = bf16r(bf16r(__uint_as_float(u[n + 1])) * w1);
              const float rg = __shfl_xor_sync(0xffffffffu, odd ? g0 : g1, 1);
              const float ru = __shfl_xor_sync(0xffffffffu, odd ? u0 : u1, 1);
              if (c0 + n + (odd ? 1 : 0) < nvalid) {
                __nv_bfloat16* row = p.y + (int64_t)(id & 0xFFFFFFu) * p.rows + jp;
                if (j_ok)
                  atomicAdd(reinterpret_cast<__nv_bfloat162*>(row),
                            odd ? __floats2bfloat162_rn(rg, g1) : __floats2bfloat162_rn(g0, rg));
                if (j2_ok)
                  atomicAdd(reinterpret_cast<__nv_bfloat162*>(row + kTileMH),
                            odd ? __floats2bfloat162_rn(ru, u1) : __floats2bfloat162_rn(u0, ru));
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
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
  if (warp == 1) tmem_dealloc(tmem_base, kTmemColsH);
}

}  // namespace

int launch_grouped_gemm_bf16(const GemmArgs& a, cudaStream_t st) {
  B200_CHECK_ARG(a.N >= 16 && a.N <= 128 && a.N % 16 == 0, "grouped gemm (bf16): token tile %d is not a multiple of 16 in [16,128]",
                 a.N);
  B200_CHECK_ARG(a.Kd % 32 == 0 && a.rows > 0 && a.rows % 2 == 0 && a.E > 0, "grouped gemm (bf16): bad shape");
  B200_CHECK_ARG(a.max_rows % a.N == 0, "grouped gemm (bf16): max_rows %% B != 0");
  B200_CHECK_ARG(((uintptr_t)a.w_data & 15) == 0 && ((uintptr_t)a.a_q & 15) == 0,
                 "grouped gemm (bf16): operand tensors must be 16-byte aligned");
  Bf16Params p;
  memset(&p, 0, sizeof(p));
  p.B = a.N; p.rows = a.rows; p.KB = (a.Kd + kTileKH - 1) / kTileKH;
  p.MT = a.gateup ? (a.rows + kTileMH - 1) / kTileMH : (a.rows + 2 * kTileMH - 1) / (2 * kTileMH);
  p.k_tail_steps = (a.Kd - (p.KB - 1) * kTileKH + 15) / 16;
  p.E = a.E; p.topk = a.topk; p.T = a.T; p.activation = a.activation; p.swiglu_limit = a.swiglu_limit;
  p.max_rows = a.max_rows;
  p.sorted_ids = a.sorted_ids; p.sorted_e = a.sorted_e; p.num_valid = a.num_valid; p.status = a.status;
  p.h_sorted = (__nv_bfloat16*)a.oq; p.out2 = (__nv_bfloat16*)a.out2;
  p.sorted_w = a.sorted_w; p.bias = a.bias; p.y = a.gateup ? nullptr : (__nv_bfloat16*)a.y;
  p.weight_stage1 = (a.gateup && a.weight_stage1) ? 1 : 0;
  B200_CHECK_ARG(p.weight_stage1 == 0 || a.sorted_w != nullptr, "grouped gemm (bf16): routing weights missing");
  B200_CHECK_ARG(!a.gateup || p.h_sorted != nullptr, "gate-up (bf16): output rows missing");
  B200_CHECK_ARG(a.gateup || p.out2 != nullptr || p.y != nullptr, "down (bf16): output missing");
  B200_CHECK_ARG(p.y == nullptr || ((uintptr_t)p.y & 3) == 0, "grouped gemm (bf16): y must be 4-byte aligned");

  // weights: bf16 [E, parts*rows, Kd] as they sit in HBM; K and row tails are zero-filled by TMA
  const cuuint64_t row_pitch = (cuuint64_t)a.Kd * 2;
  {
    const cuuint64_t parts = a.gateup ? 2 : 1;
    cuuint64_t dims[4] = {(cuuint64_t)a.Kd, (cuuint64_t)a.rows, parts, (cuuint64_t)a.E};
    cuuint64_t strides[3] = {row_pitch, row_pitch * (cuuint64_t)a.rows, row_pitch * (cuuint64_t)a.rows * parts};
    cuuint32_t box[4] = {kTileKH, a.gateup ? (cuuint32_t)kTileMH : 2u * kTileMH, a.gateup ? 2u : 1u, 1};
    int rc = encode_map_sw(&p.tmW, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a.w_data, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "bf16 weights");
    if (rc) return rc;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)a.Kd, (cuuint64_t)a.max_rows, 1};
    cuuint64_t strides[2] = {row_pitch, row_pitch * (cuuint64_t)a.max_rows};
    cuuint32_t box[3] = {kTileKH, (cuuint32_t)a.N, 1};
    int rc = encode_map_sw(&p.tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.a_q, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "bf16 token rows");
    if (rc) return rc;
  }
  const int stage_bytes = (2 * kATileBytesH + a.N * kRowBytesH + 1023) & ~1023;
  const int stages = std::min((kSmemLimitH - 2048) / stage_bytes, kMaxStagesH);
  B200_CHECK_ARG(stages >= 2, "grouped gemm (bf16): tile does not fit shared memory");
  p.stages = stages;
  const size_t smem = 2048 + (size_t)stages * stage_bytes;
  const int64_t max_work = (a.max_rows / a.N) * p.MT;
  const int grid = (int)std::min<int64_t>(device_sm_count(), std::max<int64_t>(max_work, 1));
  void (*kernel)(Bf16Params) = a.gateup ? moe_grouped_gemm_bf16_kernel<true> : moe_grouped_gemm_bf16_kernel<false>;
  B200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimitH));
  B200_CHECK_CUDA(launch_chained(kernel, dim3(grid), dim3(kThreadsH), smem, st, p));
  B200_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200moe
