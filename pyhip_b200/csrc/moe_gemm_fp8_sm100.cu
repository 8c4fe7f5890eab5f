// Grouped GEMMs for FP8 (e4m3) expert weights with one fp32 scale per 128x128 block
// (the format of tests/contrib/moe/test_moe.py:201-260 of the reference; DeepSeek-V3 style).
//
// Same orientation and warp roles as the MXFP4 kernels (moe_gemm_sm100.cu): 128 weight rows on
// the MMA's M side, the token tile of one sorted block on N, two weight tiles per pipeline stage,
// TMA producer / MMA issuer / 8 epilogue warps / 4 scale-loader warps, bounded waits.
// What differs:
//   * tcgen05.mma kind::mxf8f6f4.block_scale, e4m3 x e4m3, K = 32 per instruction.  Activations
//     are two e4m3 terms (value + residual) with E8M0 scales per 32 -- exact for bf16 inputs up to
//     ~2^-9 of the block maximum -- applied by the tensor core; the weight operand's E8M0 scale is
//     the constant 1.0.
//   * a 128-block fp32 scale is not a power of two, so it cannot ride in the MMA.  One pipeline
//     stage is exactly one 128-wide k-block: its MMAs OVERWRITE a TMEM accumulator, the epilogue
//     warps read it, multiply by the block's weight scale (one scalar per weight tile and k-block)
//     and add into fp32 registers -- the two-level accumulation the reference's FP8 kernel does
//     with its FIFO + fmac (src/contrib/moe_gemm_8wave.py:386-405).  Two TMEM accumulator buffers
//     let the next k-block's MMAs run under the promotion of the current one.
//   * row-scaled weights (one fp32 scale per output row: the reference's per-token-per-channel and per-tensor FP8
//     weight formats, tests/contrib/moe/test_moe.py:123-138,190-200): the scale does not change along K, so the
//     MMAs accumulate over all k-blocks in tensor memory and the epilogue multiplies each accumulator row by its
//     scale once per tile -- in this orientation a thread owns one weight row, so that is one scalar per thread.
//   * act_quant 1x128 (the reference's own activation format: one e4m3 value per element with an fp32
//     scale per token and 128 channels, src/contrib/fused_moe.py:375-381): a single activation term, all
//     E8M0 scales of the MMA are 1.0, and the promotion multiplies every token column by
//     sA[token, k-block] * sB[row block, k-block] (src/contrib/moe_gemm_8wave.py:386-405 folds the two the
//     same way).  The four scale-loader warps form those products once per k-block into a small
//     shared-memory table that the epilogue warps read with broadcast loads.
#include <algorithm>
#include <mutex>

#include "gemm_common.cuh"

namespace b200moe {

namespace fp8 {

constexpr int kThreads = 512;                   // 4 warpgroups: {TMA, MMA, 2 idle}, 2 x epilogue, scale loaders
// registers per thread after reallocation: 8 epilogue warps, warpgroup 0 (producer, issuers, store warp),
// 4 scale-loader warps: 256*184 + 128*104 + 128*40 = the 64K registers of an SM
constexpr int kRegsEpilogue = 184, kRegsWg0 = 104, kRegsSf = 40;
constexpr int kTileM = 128;
constexpr int kTileK = 128;                      // one weight-scale block per stage
constexpr int kATileBytes = kTileM * kTileK;     // 16 KB (one byte per element)
constexpr int kMaxStages = 12;
constexpr int kTmemCols = 512;
constexpr int kSfCol0 = kAccColsLimit;           // scale columns: A (constant) 4, then 2 buffers x 8 for B
constexpr int kSmemLimit = 232448;
constexpr int kStagePitch = kTileM * 2 + 16;
constexpr int kMaxChunks = 3;                    // 16-column groups per epilogue warp (token tile <= 96)
constexpr int kTerms = 2;
constexpr int kCtlBytes = 4096;                  // barriers + the current tile's weight-block scales
constexpr int kMaxKB = 128;                      // k-blocks per row whose scales fit the control region

struct Params {
  CUtensorMap tmW;     // weights: gate-up (K, I, 2, E) box (128,128,2,1); down (K, H, 1, E) box (128,256,1,1), bytes
  CUtensorMap tmA;     // activations (K, max_rows, 2 terms) box (128, B, 2), bytes
  const float* w_scale;     // gate-up [E, 2I/128, K/128]; down [E, H/128, K/128]
  const uint8_t* asf;       // [blocks, KB, 2 chunks, 512]
  const uint32_t* sorted_ids;
  const int32_t* sorted_e;
  const int32_t* num_valid;
  int32_t* status;
  __nv_bfloat16* h_out;
  uint8_t* oq; uint8_t* osf;
  __nv_bfloat16* out2;
  int64_t max_rows;
  int64_t oq_term_stride;
  int B, rows, KB, MT, E, topk, T, stages, out_k, out_kb, activation;
  float swiglu_limit;
  const float* sorted_w;   // routing weight of every sorted row (fused combine, weights applied in the gate-up stage)
  const float* bias;       // per-expert bias: gate-up [E, 2*rows] (gate then up), down [E, rows]; or null
  __nv_bfloat16* y;        // down, fused combine: zeroed [T, rows] output accumulated with bf16x2 reductions; or null
  int weight_stage1;       // gate-up: multiply h by the routing weight
  int aq;                  // 1: single e4m3 activation term with fp32 scales per (token, 128 channels)
  int rowsc;               // 1: w_scale is [E, parts*rows], one scale per weight row, constant along K
};

struct SmemCtl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[4];      // [accumulator buffer * 2 + weight tile]
  uint64_t tmem_empty[4];
  uint64_t sf_full[2];
  uint64_t sf_empty[2];
  uint64_t stg_full, stg_empty;   // staging tile of the fused gate-up output: epilogue warps -> store warp
  uint32_t tmem_base;
  uint32_t abort_word;
  float wscale[2][2][kMaxKB];   // [tile parity][weight tile][k-block]
  alignas(16) float cscale[2][2][96];       // read as float4; 1x128 mode: [ring slot][weight tile][token column] = sA * sB of one k-block
};
static_assert(sizeof(SmemCtl) <= kCtlBytes, "control region");

struct StageGeom {
  int a_bytes, b_bytes, sfb_bytes, stage_bytes;
  uint32_t tx_bytes;
};
__host__ __device__ inline StageGeom stage_geom(int B, int aq) {
  StageGeom g;
  g.a_bytes = 2 * kATileBytes;
  g.b_bytes = (aq ? 1 : kTerms) * B * kTileK;
  g.sfb_bytes = aq ? B * 4 : kTerms * kSfChunk;   // fp32 per token, or one E8M0 chunk per term (virtual row = term*128 + r)
  g.stage_bytes = (g.a_bytes + g.b_bytes + g.sfb_bytes + 1023) & ~1023;
  g.tx_bytes = (uint32_t)(g.a_bytes + g.b_bytes + g.sfb_bytes);
  return g;
}

template <bool GATEUP>
__global__ void __launch_bounds__(kThreads, 1) moe_grouped_gemm_fp8_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(smem);
  const uint32_t stage0 = smem_u32(smem) + kCtlBytes;
  const int B = p.B;
  const StageGeom geo = stage_geom(B, p.aq);
  const int S = p.stages;
  const int nterms = p.aq ? 1 : kTerms;
  const int acc_cols = 2 * B;                  // two weight tiles x B token columns, per accumulator buffer

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_word = &ctl->abort_word;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      // one commit per MMA warp; in 1x128 mode the four scale-loader warps read the stage's token scales too
      mbar_init(smem_u32(&ctl->empty[s]), p.aq ? 6 : 2);
    }
    for (int a = 0; a < 2; ++a) {
      for (int h = 0; h < 2; ++h) {
        mbar_init(smem_u32(&ctl->tmem_full[2 * a + h]), 1);
        mbar_init(smem_u32(&ctl->tmem_empty[2 * a + h]), 8);
      }
      mbar_init(smem_u32(&ctl->sf_full[a]), 4);
      mbar_init(smem_u32(&ctl->sf_empty[a]), p.aq ? 8 : 2);     // consumers: the MMA warps, or (1x128) the epilogue warps
    }
    mbar_init(smem_u32(&ctl->stg_full), 8);
    mbar_init(smem_u32(&ctl->stg_empty), 1);
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
  // the epilogue warpgroups (warps 4..11) hold the promoted fp32 accumulators in registers: they take the
  // registers that the producer / issuer / scale-loader warpgroups do not need
  // (the reallocation itself is the first statement of each warpgroup's branch below)
  grid_dep_launch();   // tensor memory is held: the next kernel's CTAs may be scheduled
  grid_dep_wait();     // predecessor complete: sort arrays and quantised activations are valid

  const int64_t rows_live = min((int64_t)p.num_valid[0], p.max_rows);
  const int n_blocks = (int)(rows_live / B);
  const int total_work = n_blocks * p.MT;

  if (warp < 4) {
    // warpgroup 0: TMA producer (warp 0), MMA issuers (warps 1, 2), store warp (warp 3)
    reg_release<kRegsWg0>();
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        prefetch_tensormap(&p.tmW);
        prefetch_tensormap(&p.tmA);
        int stage = 0;
        uint32_t phase = 0;
        int64_t issued = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
          const int b = w / p.MT, m = w - b * p.MT;
          int e = p.sorted_e[b];
          if (e < 0 || e >= p.E) { p.status[2] = 1; e = 0; }
          const int r0 = b * B;
          const uint8_t* sfb = p.asf + (int64_t)b * p.KB * geo.sfb_bytes;
          for (int kb = 0; kb < p.KB; ++kb) {
            if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1, abort_word, 0x100 + stage)) { ok = false; break; }
            const uint32_t st = stage0 + (uint32_t)stage * geo.stage_bytes;
            const uint32_t full = smem_u32(&ctl->full[stage]);
            mbar_expect_tx(full, geo.tx_bytes);
            tma_load_4d(st, &p.tmW, full, kb * kTileK, m * (GATEUP ? kTileM : 2 * kTileM), 0, e);
            tma_load_3d(st + geo.a_bytes, &p.tmA, full, kb * kTileK, r0, 0);
            bulk_load(st + geo.a_bytes + geo.b_bytes, sfb, (uint32_t)geo.sfb_bytes, full);
            sfb += geo.sfb_bytes;
            ++issued;
            if (++stage == S) { stage = 0; phase ^= 1; }
          }
        }
        if (!ok || *abort_word) {
          const int64_t first = issued > S ? issued - S : 0;
          for (int64_t i = first; i < issued; ++i) {
            const uint32_t bar = smem_u32(&ctl->full[i % S]);
            const uint32_t par = (uint32_t)((i / S) & 1);
            const uint64_t t0 = global_timer_ns();
            while (!mbar_try_wait(bar, par) && global_timer_ns() - t0 < 200000000ull) {}
          }
        }
      }
    } else if (warp <= 2) {
      // ------------------------------------------------------------------ MMA issuers: warp 1 multiplies the
      // first weight tile of every stage, warp 2 the second, each into its own accumulator columns
      const uint32_t part = (uint32_t)(warp - 1);
      uint32_t idesc[4];
  #pragma unroll
      for (int k = 0; k < 4; ++k) idesc[k] = make_idesc_block_scaled(kFmtE4M3, kFmtE4M3, kTileM, (uint32_t)B, k, k);
      const uint32_t term_lo = (uint32_t)(B * kTileK) >> 4;
      const uint32_t sfa_t = tmem_base + kSfCol0;
      int stage = 0;
      uint32_t phase = 0, acc = 0, acc_phase = 0, sf_buf = 0, sf_phase = 0;
      bool ok = true;
      PROF_DECL(t_acc);
      PROF_DECL(t_full);
      PROF_DECL(t_sf);
      const long long t_begin = PROF_NOW();
      (void)t_begin;
      // The MMAs cover only the live rows of the block (rounded up to 16): padding rows that end an expert's last
      // block cost neither tensor time nor operand reads.  The row ids of the NEXT item are fetched while the
      // current one is multiplied.
      uint32_t nid[3];
      auto fetch_ids = [&](int w, uint32_t (&r)[3]) {
        const int r0 = (w / p.MT) * B;
#pragma unroll
        for (int q = 0; q < 3; ++q) r[q] = (w < total_work && q * 32 + lane < B) ? p.sorted_ids[r0 + q * 32 + lane] : 0xFFFFFFFFu;
      };
      fetch_ids((int)blockIdx.x, nid);
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int nlive = 0;
#pragma unroll
        for (int q = 0; q < 3; ++q)
          nlive += __popc(__ballot_sync(0xffffffffu, (int)(nid[q] >> 24) < p.topk && (int)(nid[q] & 0xFFFFFFu) < p.T));
        fetch_ids(w + (int)gridDim.x, nid);
        const uint32_t n_mma = (uint32_t)min(B, max(16, (nlive + 15) & ~15));
        uint32_t idesc_w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) idesc_w[k] = (idesc[k] & ~(0x3Fu << 17)) | ((n_mma >> 3) << 17);
        for (int kb = 0; kb < p.KB; ++kb) {
          // every k-block gets its own accumulator buffer: the epilogue promotes it with the
          // block's fp32 weight scale while the next k-block is being multiplied
          // (row-scaled weights: one accumulator per TILE, multiplied into across all k-blocks)
          const bool first_kb = !p.rowsc || kb == 0, last_kb = !p.rowsc || kb == p.KB - 1;
          const long long c0 = PROF_NOW();
          if (first_kb)
            ok = mbar_wait(smem_u32(&ctl->tmem_empty[2 * acc + part]), acc_phase ^ 1, abort_word, 0x200 + 2 * acc + part);
          PROF_ADD(t_acc, c0);
          const long long c1 = PROF_NOW();
          ok = ok && mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_word, 0x300 + stage);
          PROF_ADD(t_full, c1);
          const long long c2 = PROF_NOW();
          // 1x128 mode: the MMA's scale columns are constants written once by the scale-loader warps before their
          // first table is published, so only the very first MMA has to wait for that
          if (!p.aq || (w == (int)blockIdx.x && kb == 0))
            ok = ok && mbar_wait(smem_u32(&ctl->sf_full[sf_buf]), sf_phase, abort_word, 0x500 + sf_buf);
          PROF_ADD(t_sf, c2);
          if (!ok) break;
          tc_fence_after_sync();
          __syncwarp();
          if (elect_one()) {       // one issuing lane; descriptors stay in uniform registers
            const uint32_t st = stage0 + (uint32_t)stage * geo.stage_bytes;
            const uint32_t a_lo = desc_lo_sw(st + part * kATileBytes);
            const uint32_t b_lo = desc_lo_sw(st + geo.a_bytes);
            const uint32_t sfb_t = sfa_t + 4 + sf_buf * 8;
            const uint32_t d0 = tmem_base + acc * acc_cols + part * B;
  #pragma unroll
            for (int k = 0; k < 4; ++k) {
  #pragma unroll
              for (int t = 0; t < kTerms; ++t)
                if (t < nterms)
                  umma_mxf8(d0, a_lo + 2 * k, b_lo + t * term_lo + 2 * k, idesc_w[k], sfa_t, sfb_t + 4 * t,
                            (k | t) != 0 || !first_kb);
            }
            tc_commit(smem_u32(&ctl->empty[stage]));
            if (!p.aq) tc_commit(smem_u32(&ctl->sf_empty[sf_buf]));
            if (last_kb) tc_commit(smem_u32(&ctl->tmem_full[2 * acc + part]));
          }
          __syncwarp();
          if (sf_buf == 1) sf_phase ^= 1;
          sf_buf ^= 1;
          if (last_kb) {
            if (acc == 1) acc_phase ^= 1;
            acc ^= 1;
          }
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
      }
#ifdef B200MOE_PROFILE
      if (blockIdx.x == 0 && lane == 0 && part == 0) {   // kilo-cycles: issuer total, waiting for data, for an accumulator, for scales
        p.status[5] = (int32_t)((clock64() - t_begin) >> 10);
        p.status[6] = (int32_t)(t_full >> 10);
        p.status[7] = (int32_t)(t_acc >> 10);
        p.status[4] = (int32_t)(t_sf >> 10);
      }
#endif
    } else if (warp == 3) {
      // ------------------------------------------------------------------ store warp (fused gate-up only):
      // takes each finished h tile from the staging buffer, re-quantises it into two e4m3 terms with
      // E8M0 scales per 32 features and writes it out in sorted-row order, while the epilogue warps
      // are already promoting the next tile
      if (GATEUP && p.h_out == nullptr) {
        const uint32_t stg = stage0 + (uint32_t)S * geo.stage_bytes;
        uint32_t ph = 0;
        for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
          const int b = w / p.MT, m = w - b * p.MT;
          const int r0 = b * B;
          int nvalid = 0;
          for (int q = 0; q < B; q += 32) {
            const uint32_t id = (q + lane < B) ? p.sorted_ids[r0 + q + lane] : 0xFFFFFFFFu;
            nvalid += __popc(__ballot_sync(0xffffffffu, (int)(id >> 24) < p.topk && (int)(id & 0xFFFFFFu) < p.T));
          }
          if (!mbar_wait(smem_u32(&ctl->stg_full), ph, abort_word, 0x900)) break;
          for (int unit0 = 0; unit0 < nvalid * 4; unit0 += 32) {       // warp-uniform trip count (shuffles below)
            const int unit = unit0 + lane;
            const bool live = unit < nvalid * 4;
            const int n = min(unit, nvalid * 4 - 1) >> 2, q = unit & 3;
            float x[32];
  #pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              const uint4 raw = ld_shared_v4(stg + (uint32_t)n * kStagePitch + q * 64 + v4 * 16);
              const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
  #pragma unroll
              for (int t = 0; t < 4; ++t) {
                const float2 f = __bfloat1622float2(b2[t]);
                x[v4 * 8 + t * 2] = f.x;
                x[v4 * 8 + t * 2 + 1] = f.y;
              }
            }
            const int64_t r = (int64_t)r0 + n;
            if (p.weight_stage1) {
              const float wr = p.sorted_w[r];
  #pragma unroll
              for (int i = 0; i < 32; ++i) x[i] = bf16r(x[i] * wr);
            }
            if (p.aq) {
              // one fp32 scale per row and 128 features = this tile: the row's four lanes share the maximum
              float amax = 0.f;
  #pragma unroll
              for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[i]));
              amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
              amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
              const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
              uint32_t wq[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  #pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const __nv_fp8x2_storage_t pk = __nv_cvt_float2_to_fp8x2(
                    make_float2(__fdiv_rn(x[i], scale), __fdiv_rn(x[i + 1], scale)), __NV_SATFINITE, __NV_E4M3);
                wq[i >> 2] |= (uint32_t)pk << ((i & 2) * 8);
              }
              if (live) {
                uint4* dst = reinterpret_cast<uint4*>(p.oq + r * p.out_k + m * kTileM + q * 32);
                dst[0] = make_uint4(wq[0], wq[1], wq[2], wq[3]);
                dst[1] = make_uint4(wq[4], wq[5], wq[6], wq[7]);
                if (q == 0) reinterpret_cast<float*>(p.osf)[((int64_t)b * p.out_kb + m) * B + n] = scale;
              }
            } else if (live) {
  #pragma unroll
              for (int t = 0; t < kTerms; ++t) {
                uint4 q0, q1;
                const int ex = (t + 1 < kTerms) ? quant_block32_e4m3<true>(x, q0, q1) : quant_block32_e4m3<false>(x, q0, q1);
                uint4* dst = reinterpret_cast<uint4*>(p.oq + t * p.oq_term_stride + r * p.out_k + m * kTileM + q * 32);
                dst[0] = q0;
                dst[1] = q1;
                p.osf[act_sf_index(b, m, p.out_kb, B, kTerms, 128, t, n, q)] = (uint8_t)ex;
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctl->stg_empty));
          ph ^= 1;
        }
      } else if (!GATEUP) {
        // down projection: two 128-feature halves per tile, staging rows -> out2 rows as 16-byte vectors
        const uint32_t stg = stage0 + (uint32_t)S * geo.stage_bytes;
        uint32_t ph = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
          const int b = w / p.MT, m = w - b * p.MT;
          const int r0 = b * B;
          int nvalid = 0;
          for (int q = 0; q < B; q += 32) {
            const uint32_t id = (q + lane < B) ? p.sorted_ids[r0 + q + lane] : 0xFFFFFFFFu;
            nvalid += __popc(__ballot_sync(0xffffffffu, (int)(id >> 24) < p.topk && (int)(id & 0xFFFFFFu) < p.T));
          }
          for (int hf = 0; hf < 2; ++hf) {
            if (!mbar_wait(smem_u32(&ctl->stg_full), ph, abort_word, 0x901)) { ok = false; break; }
            const int f0 = m * 2 * kTileM + hf * kTileM;
            if (f0 < p.rows) {
              for (int idx = lane; idx < nvalid * 16; idx += 32) {
                const int n = idx >> 4, v = idx & 15;
                const uint4 val = ld_shared_v4(stg + (uint32_t)n * kStagePitch + v * 16);
                if (p.y == nullptr) {
                  *reinterpret_cast<uint4*>(p.out2 + ((int64_t)r0 + n) * p.rows + f0 + v * 8) = val;
                } else {
                  // fused combine: y[token] += bf16(row * routing weight), 16 bytes per reduction
                  // (the reference's weighted atomic epilogue, src/contrib/moe.py:703-787)
                  const uint32_t id = p.sorted_ids[r0 + n];
                  const float wr = p.sorted_w != nullptr ? p.sorted_w[r0 + n] : 1.f;   // null: applied upstream
                  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&val);
                  uint32_t o[4];
  #pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(b2[i]);
                    const __nv_bfloat162 c = __floats2bfloat162_rn(f.x * wr, f.y * wr);
                    o[i] = *reinterpret_cast<const uint32_t*>(&c);
                  }
                  __nv_bfloat16* dst = p.y + (int64_t)(id & 0xFFFFFFu) * p.rows + f0 + v * 8;
                  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(o[0]), "r"(o[1]),
                               "r"(o[2]), "r"(o[3])
                               : "memory");
                }
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->stg_empty));
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp >= 12) {
    reg_release<kRegsSf>();
    // ------------------------------------------------------------------ scale-loader warps
    // Weight operand: E8M0 scale 1.0 everywhere, written once.  Activation operand: the two terms'
    // scale chunks of every stage, shared memory -> registers -> this warp's TMEM lane quadrant.
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint4 ones = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
    tmem_st_32x32b_x4(tmem_base + lane_base + kSfCol0, ones);
    int stage = 0;
    uint32_t phase = 0, sf_buf = 0, sf_phase = 0;
    bool ok = true;
    if (p.aq) {
      // 1x128 activations: every E8M0 scale of the MMA is 1.0 (written once, weight and activation side); per
      // k-block these warps form c[tile][token] = sA[token, kb] * sB[tile's row block, kb] for the promotion
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_st_32x32b_x4(tmem_base + lane_base + kSfCol0 + 4 + 4 * c, ones);
      tmem_st_wait();
      tc_fence_before_sync();
      const int tcol = (warp & 3) * 32 + lane;             // token column of this thread (live when < B)
      const int row_blocks = (GATEUP ? 2 * p.rows : p.rows) / kTileM;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int b = w / p.MT, m = w - b * p.MT;
        int e = p.sorted_e[b];
        if (e < 0 || e >= p.E) e = 0;
        const int rb0 = GATEUP ? m : 2 * m;
        const int rb1 = GATEUP ? p.rows / kTileM + m : min(2 * m + 1, row_blocks - 1);
        const float* s0 = p.w_scale + ((int64_t)e * row_blocks + rb0) * p.KB;
        const float* s1 = p.w_scale + ((int64_t)e * row_blocks + rb1) * p.KB;
        float n0 = s0[0], n1 = s1[0];                      // next k-block's weight scales, fetched one step ahead
        for (int kb = 0; kb < p.KB; ++kb) {
          const float w0 = n0, w1 = n1;
          if (kb + 1 < p.KB) { n0 = s0[kb + 1]; n1 = s1[kb + 1]; }
          if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_word, 0x600 + stage) ||
              !mbar_wait(smem_u32(&ctl->sf_empty[sf_buf]), sf_phase ^ 1, abort_word, 0x700 + sf_buf)) {
            ok = false;
            break;
          }
          if (tcol < B) {
            const float sa = *reinterpret_cast<const float*>(smem + kCtlBytes + (size_t)stage * geo.stage_bytes + geo.a_bytes +
                                                             geo.b_bytes + tcol * 4);
            ctl->cscale[sf_buf][0][tcol] = sa * w0;
            ctl->cscale[sf_buf][1][tcol] = sa * w1;
          }
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(smem_u32(&ctl->sf_full[sf_buf]));     // release: the table entries above are visible to the waiters
            mbar_arrive(smem_u32(&ctl->empty[stage]));        // this warp is done with the stage's token scales
          }
          if (sf_buf == 1) sf_phase ^= 1;
          sf_buf ^= 1;
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
      }
    } else {
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_word, 0x600 + stage) ||
              !mbar_wait(smem_u32(&ctl->sf_empty[sf_buf]), sf_phase ^ 1, abort_word, 0x700 + sf_buf)) {
            ok = false;
            break;
          }
          const uint32_t sf_s = stage0 + (uint32_t)stage * geo.stage_bytes + geo.a_bytes + geo.b_bytes + lane * 16;
          const uint32_t sfb_t = tmem_base + lane_base + kSfCol0 + 4 + sf_buf * 8;
          tmem_st_32x32b_x4(sfb_t, ld_shared_v4(sf_s));
          tmem_st_32x32b_x4(sfb_t + 4, ld_shared_v4(sf_s + kSfChunk));
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctl->sf_full[sf_buf]));
          if (sf_buf == 1) sf_phase ^= 1;
          sf_buf ^= 1;
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (4..11)
    reg_acquire<kRegsEpilogue>();
    const int ew = warp - 4;
    const int quad = warp & 3;
    const int half = ew >> 2;                  // the two warps of a quadrant take alternating 16-column groups
    const int tid_e = ew * 32 + lane;
    const int row_local = quad * 32 + lane;
    const uint32_t stg = stage0 + (uint32_t)S * geo.stage_bytes;
    const bool fused = GATEUP && p.h_out == nullptr;
    const bool staged = fused || !GATEUP;      // finished tiles leave through the staging buffer and the store warp
    const int row_blocks = (GATEUP ? 2 * p.rows : p.rows) / kTileM;   // weight-scale rows per expert
    uint32_t acc = 0, acc_phase = 0;
    uint32_t cs_buf = 0, cs_phase = 0;      // 1x128 mode: ring slot of the per-column scale table
    bool alive = true;
    PROF_DECL(t_wait_epi);
    PROF_DECL(t_wait_cs);
    PROF_DECL(t_fma);
    int tile_par = 0;
    uint32_t stg_phase = 0;
    const long long t_begin_epi = PROF_NOW();
    (void)t_begin_epi;
    for (int w = blockIdx.x; w < total_work && alive; w += gridDim.x) {
      const int b = w / p.MT, m = w - b * p.MT;
      const int r0 = b * B;
      int e = p.sorted_e[b];
      if (e < 0 || e >= p.E) e = 0;
      const int j = (GATEUP ? m * kTileM : m * 2 * kTileM) + row_local;
      const int rb0 = GATEUP ? m : 2 * m;
      const int rb1 = GATEUP ? p.rows / kTileM + m : min(2 * m + 1, row_blocks - 1);
      const float* s0 = p.w_scale + ((int64_t)e * row_blocks + rb0) * p.KB;
      const float* s1 = p.w_scale + ((int64_t)e * row_blocks + rb1) * p.KB;
      // row-scaled weights: this thread's two weight rows carry one scale each for the whole tile
      float rs0 = 0.f, rs1 = 0.f;
      if (p.rowsc) {
        const float* rs = p.w_scale + (int64_t)e * (GATEUP ? 2 : 1) * p.rows;
        if (j < p.rows) rs0 = rs[j];
        if (GATEUP ? j < p.rows : j + kTileM < p.rows) rs1 = rs[j + (GATEUP ? p.rows : kTileM)];
      }
      int nvalid = 0;
      for (int q = 0; q < B; q += 32) {
        const uint32_t id = (q + lane < B) ? p.sorted_ids[r0 + q + lane] : 0xFFFFFFFFu;
        nvalid += __popc(__ballot_sync(0xffffffffu, (int)(id >> 24) < p.topk && (int)(id & 0xFFFFFFu) < p.T));
      }
      float ag[kMaxChunks * 16], au[kMaxChunks * 16];
#pragma unroll
      for (int i = 0; i < kMaxChunks * 16; ++i) { ag[i] = 0.f; au[i] = 0.f; }

      // the tile's weight-block scales go to shared memory first: a global load inside the k loop would sit
      // in front of every accumulator hand-back (the arrive has release semantics)
      float (*ws)[kMaxKB] = ctl->wscale[tile_par];
      if (!p.aq && !p.rowsc) {
        for (int i = tid_e; i < 2 * p.KB; i += 256) ws[i >= p.KB][i >= p.KB ? i - p.KB : i] = (i >= p.KB ? s1 : s0)[i >= p.KB ? i - p.KB : i];
        tile_par ^= 1;
        epi_sync();
      }
      const int kb_rounds = p.rowsc ? 1 : p.KB;        // accumulator hand-overs per tile
      for (int kb = 0; kb < kb_rounds && alive; ++kb) {
        const float sc[2] = {p.rowsc ? rs0 : (p.aq ? 0.f : ws[0][kb]), p.rowsc ? rs1 : (p.aq ? 0.f : ws[1][kb])};
        if (p.aq) {
          // the k-block's per-column scale table (token scale x weight-block scale), made by the scale-loader warps
          const long long tc0 = PROF_NOW();
          if (!mbar_wait(smem_u32(&ctl->sf_full[cs_buf]), cs_phase, abort_word, 0x480 + cs_buf)) { alive = false; break; }
          PROF_ADD(t_wait_cs, tc0);
        }
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          const long long te0 = PROF_NOW();
          const bool ok = mbar_wait(smem_u32(&ctl->tmem_full[2 * acc + part]), acc_phase, abort_word, 0x400 + 2 * acc + part);
          PROF_ADD(t_wait_epi, te0);
          if (!ok) { alive = false; break; }      // the vote after the k loop takes every warp out together
          tc_fence_after_sync();
          const uint32_t t0 = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * acc_cols + part * B;
          // this warp's 16-column groups of the tile -> registers; the accumulator is handed back to the
          // MMA warp before the values are scaled and added
          uint32_t v[kMaxChunks][16];
#pragma unroll
          for (int ci = 0; ci < kMaxChunks; ++ci)
            if ((2 * ci + half) * 16 < nvalid) tmem_ld_32x32b_x16(t0 + (2 * ci + half) * 16, v[ci]);
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[2 * acc + part]));
          if (p.aq) {
#pragma unroll
            for (int ci = 0; ci < kMaxChunks; ++ci) {
              if ((2 * ci + half) * 16 < nvalid) {
                const float4* cv = reinterpret_cast<const float4*>(&ctl->cscale[cs_buf][part][(2 * ci + half) * 16]);
#pragma unroll
                for (int n4 = 0; n4 < 4; ++n4) {
                  const float4 c = cv[n4];                  // same address in every lane: a broadcast load
                  const int n = n4 * 4;
                  if (part == 0) {
                    ffma2_pair(ag[ci * 16 + n], ag[ci * 16 + n + 1], c.x, c.y, v[ci][n], v[ci][n + 1]);
                    ffma2_pair(ag[ci * 16 + n + 2], ag[ci * 16 + n + 3], c.z, c.w, v[ci][n + 2], v[ci][n + 3]);
                  } else {
                    ffma2_pair(au[ci * 16 + n], au[ci * 16 + n + 1], c.x, c.y, v[ci][n], v[ci][n + 1]);
                    ffma2_pair(au[ci * 16 + n + 2], au[ci * 16 + n + 3], c.z, c.w, v[ci][n + 2], v[ci][n + 3]);
                  }
                }
              }
            }
          } else {
#pragma unroll
            for (int ci = 0; ci < kMaxChunks; ++ci) {
              if ((2 * ci + half) * 16 < nvalid) {
#pragma unroll
                for (int n = 0; n < 16; n += 2) {
                  if (part == 0) ffma2_scaled(ag[ci * 16 + n], ag[ci * 16 + n + 1], sc[0], v[ci][n], v[ci][n + 1]);
                  else ffma2_scaled(au[ci * 16 + n], au[ci * 16 + n + 1], sc[1], v[ci][n], v[ci][n + 1]);
                }
              }
            }
          }
        }
        if (p.aq && alive) {
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctl->sf_empty[cs_buf]));     // this warp has read the table
          if (cs_buf == 1) cs_phase ^= 1;
          cs_buf ^= 1;
        }
        if (acc == 1) acc_phase ^= 1;
        acc ^= 1;
      }
      // one vote per tile: a warp whose wait gave up has set the shared abort word, so the others'
      // waits return at once and every epilogue warp leaves before the next named barrier
      if (staged && alive) alive = mbar_wait(smem_u32(&ctl->stg_empty), stg_phase ^ 1, abort_word, 0x800);
      if (!epi_all(alive)) break;
      const long long tt0 = PROF_NOW();

      // ---- tile finished: activation / stores from the register accumulators
      const bool j_ok = j < p.rows;
      if (p.bias != nullptr) {
        // the oracle's matmul returns bf16 and the bias is added to that (the consumers below round once more)
        const float* be = p.bias + (int64_t)e * (GATEUP ? 2 : 1) * p.rows;
        const float b0 = j_ok ? be[j] : 0.f;
        const float b1 = GATEUP ? (j_ok ? be[p.rows + j] : 0.f) : (j + kTileM < p.rows ? be[j + kTileM] : 0.f);
#pragma unroll
        for (int i = 0; i < kMaxChunks * 16; ++i) {
          ag[i] = bf16r(ag[i]) + b0;
          au[i] = bf16r(au[i]) + b1;
        }
      }
#pragma unroll
      for (int ci = 0; ci < kMaxChunks; ++ci) {
        const int c0 = (2 * ci + half) * 16;
        if (c0 < nvalid) {
          if (GATEUP) {
            if (!fused) {
              const uint32_t my_id = p.sorted_ids[min(r0 + c0 + lane, r0 + B - 1)];
#pragma unroll
              for (int n = 0; n < 16; ++n) {
                const uint32_t id = __shfl_sync(0xffffffffu, my_id, n);
                if (c0 + n < nvalid) {
                  const int tok = (int)(id & 0xFFFFFFu), kk = (int)(id >> 24);
                  float v = gateup_act(ag[ci * 16 + n], au[ci * 16 + n], p.activation, p.swiglu_limit);
                  if (p.weight_stage1) v *= p.sorted_w[r0 + c0 + n];
                  if (j_ok) p.h_out[((int64_t)tok * p.topk + kk) * p.rows + j] = __float2bfloat16_rn(v);
                }
              }
            } else {
#pragma unroll
              for (int n = 0; n < 16; n += 2) {
                if (c0 + n < nvalid) {
                  __nv_bfloat162 v = gateup_act2(ag[ci * 16 + n], au[ci * 16 + n], ag[ci * 16 + n + 1], au[ci * 16 + n + 1],
                                                 p.activation, p.swiglu_limit);
                  if (!j_ok) v = __floats2bfloat162_rn(0.f, 0.f);
                  st_shared_u16(stg + (uint32_t)(c0 + n) * kStagePitch + row_local * 2, __bfloat16_as_ushort(v.x));
                  if (c0 + n + 1 < nvalid)
                    st_shared_u16(stg + (uint32_t)(c0 + n + 1) * kStagePitch + row_local * 2, __bfloat16_as_ushort(v.y));
                }
              }
            }
          } else {
#pragma unroll
            for (int n = 0; n < 16; ++n)
              if (c0 + n < nvalid)
                st_shared_u16(stg + (uint32_t)(c0 + n) * kStagePitch + row_local * 2,
                              __bfloat16_as_ushort(__float2bfloat16_rn(ag[ci * 16 + n])));
          }
        }
      }
      if (staged) {          // hand the staged tile to the store warp
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->stg_full));
        stg_phase ^= 1;
      }
      if (!GATEUP) {
        // second weight tile of the pair (features j + 128): same route once the store warp has drained the first
        const bool ok2 = mbar_wait(smem_u32(&ctl->stg_empty), stg_phase ^ 1, abort_word, 0x801);
        if (!epi_all(ok2)) break;
#pragma unroll
        for (int ci = 0; ci < kMaxChunks; ++ci) {
          const int c0 = (2 * ci + half) * 16;
          if (c0 < nvalid) {
#pragma unroll
            for (int n = 0; n < 16; ++n)
              if (c0 + n < nvalid)
                st_shared_u16(stg + (uint32_t)(c0 + n) * kStagePitch + row_local * 2,
                              __bfloat16_as_ushort(__float2bfloat16_rn(au[ci * 16 + n])));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->stg_full));
        stg_phase ^= 1;
      }
      PROF_ADD(t_fma, tt0);
    }
#ifdef B200MOE_PROFILE
    if (blockIdx.x == 0 && tid_e == 0) {     // kilo-cycles: epilogue total, waiting for an accumulator, after the k loop
      p.status[8] = (int32_t)((clock64() - t_begin_epi) >> 10);
      p.status[9] = (int32_t)(t_wait_epi >> 10);
      p.status[10] = (int32_t)(t_wait_cs >> 10);
      p.status[11] = (int32_t)(t_fma >> 10);
    }
#endif
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

}  // namespace fp8

int launch_grouped_gemm_fp8(const GemmArgs& a, cudaStream_t st) {
  using namespace fp8;
  B200_CHECK_ARG(a.N >= 16 && a.N <= 96 && a.N % 16 == 0, "fp8 grouped gemm: token tile %d is not a multiple of 16 in [16,96]",
                 a.N);
  B200_CHECK_ARG(a.Kd % 128 == 0 && a.rows % 128 == 0 && a.E > 0, "fp8 grouped gemm: K and rows must be multiples of 128");
  B200_CHECK_ARG(a.max_rows % a.N == 0, "fp8 grouped gemm: max_rows %% B != 0");
  B200_CHECK_ARG(a.w_row_scaled || a.Kd / kTileK <= kMaxKB, "fp8 grouped gemm: K=%d exceeds %d", a.Kd, kMaxKB * kTileK);
  B200_CHECK_ARG(((uintptr_t)a.w_data & 15) == 0 && ((uintptr_t)a.a_q & 15) == 0 && ((uintptr_t)a.w_scale & 3) == 0,
                 "fp8 grouped gemm: operand tensors must be 16-byte aligned");
  Params p;
  memset(&p, 0, sizeof(p));
  p.B = a.N; p.rows = a.rows; p.KB = a.Kd / kTileK;
  p.MT = a.gateup ? a.rows / kTileM : (a.rows + 2 * kTileM - 1) / (2 * kTileM);
  p.E = a.E; p.topk = a.topk; p.T = a.T; p.activation = a.activation; p.swiglu_limit = a.swiglu_limit;
  p.max_rows = a.max_rows;
  p.w_scale = (const float*)a.w_scale; p.asf = (const uint8_t*)a.asf;
  p.sorted_ids = a.sorted_ids; p.sorted_e = a.sorted_e; p.num_valid = a.num_valid; p.status = a.status;
  p.h_out = (__nv_bfloat16*)a.h_out; p.oq = (uint8_t*)a.oq; p.osf = (uint8_t*)a.osf;
  p.out_k = a.out_kp; p.out_kb = a.out_kp / 128; p.oq_term_stride = a.max_rows * (int64_t)a.out_kp;
  p.out2 = (__nv_bfloat16*)a.out2;
  p.sorted_w = a.sorted_w; p.bias = a.bias; p.y = a.gateup ? nullptr : (__nv_bfloat16*)a.y;
  p.weight_stage1 = (a.gateup && a.weight_stage1) ? 1 : 0;
  p.aq = a.act_quant ? 1 : 0;
  p.rowsc = a.w_row_scaled ? 1 : 0;
  B200_CHECK_ARG(!(p.aq && p.rowsc), "fp8 grouped gemm: 1x128 activations are not offered with row-scaled weights");
  B200_CHECK_ARG(p.weight_stage1 == 0 || a.sorted_w != nullptr, "fp8 grouped gemm: routing weights missing");
  B200_CHECK_ARG(((uintptr_t)p.y & 15) == 0, "fp8 grouped gemm: fused combine needs a 16-byte aligned output");
  if (a.gateup && a.h_out == nullptr)
    B200_CHECK_ARG(a.out_kp == a.rows && a.oq && a.osf, "fp8 gate-up: fused output buffers missing");
  {
    const cuuint64_t parts = a.gateup ? 2 : 1, pitch = (cuuint64_t)a.Kd;
    cuuint64_t dims[4] = {(cuuint64_t)a.Kd, (cuuint64_t)a.rows, parts, (cuuint64_t)a.E};
    cuuint64_t strides[3] = {pitch, pitch * (cuuint64_t)a.rows, pitch * (cuuint64_t)a.rows * parts};
    cuuint32_t box[4] = {kTileK, a.gateup ? (cuuint32_t)kTileM : 2u * kTileM, a.gateup ? 2u : 1u, 1};
    int rc = encode_map_sw(&p.tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a.w_data, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "fp8 weights");
    if (rc) return rc;
  }
  {
    const cuuint32_t terms = p.aq ? 1u : (cuuint32_t)kTerms;
    cuuint64_t dims[3] = {(cuuint64_t)a.Kd, (cuuint64_t)a.max_rows, (cuuint64_t)terms};
    cuuint64_t strides[2] = {(cuuint64_t)a.Kd, (cuuint64_t)a.Kd * (cuuint64_t)a.max_rows};
    cuuint32_t box[3] = {kTileK, (cuuint32_t)a.N, terms};
    int rc = encode_map_sw(&p.tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.a_q, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "fp8 activations");
    if (rc) return rc;
  }
  const StageGeom geo = stage_geom(a.N, p.aq);
  B200_CHECK_ARG(!p.aq || ((uintptr_t)a.asf & 15) == 0, "fp8 grouped gemm: activation scales must be 16-byte aligned");
  const int staging = (!a.gateup || a.h_out == nullptr) ? a.N * kStagePitch : 0;   // fused gate-up and down leave through it
  int stages = std::min((kSmemLimit - 1024 - kCtlBytes - staging) / geo.stage_bytes, kMaxStages);
  B200_CHECK_ARG(stages >= 2, "fp8 grouped gemm: tile does not fit shared memory");
  p.stages = stages;
  const size_t smem = 1024 + kCtlBytes + (size_t)stages * geo.stage_bytes + staging;
  const int64_t max_work = (a.max_rows / a.N) * p.MT;
  const int grid = (int)std::min<int64_t>(device_sm_count(), std::max<int64_t>(max_work, 1));
  static bool attr[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  bool& done = attr[a.gateup ? 1 : 0][dev & 63];
  if (a.gateup) {
    if (!done)
      B200_CHECK_CUDA(cudaFuncSetAttribute(moe_grouped_gemm_fp8_kernel<true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    done = true;
    B200_CHECK_CUDA(launch_chained(moe_grouped_gemm_fp8_kernel<true>, dim3(grid), dim3(kThreads), smem, st, p));
  } else {
    if (!done)
      B200_CHECK_CUDA(cudaFuncSetAttribute(moe_grouped_gemm_fp8_kernel<false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    done = true;
    B200_CHECK_CUDA(launch_chained(moe_grouped_gemm_fp8_kernel<false>, dim3(grid), dim3(kThreads), smem, st, p));
  }
  B200_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200moe
