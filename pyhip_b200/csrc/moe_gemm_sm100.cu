// Grouped GEMMs of the MoE layer on the sm_100a tensor cores: tcgen05.mma kind::mxf4 with
// per-32 E8M0 block scales on both operands.
//
// Orientation ("swap-AB"): the MMA's M side holds 128 weight rows, its N side holds the token
// tile of one sorted block (B rows, a multiple of 16), so ragged token counts cost N-padding only.
//     D[128 weight rows, tokens] += W4[128, K] * A4[tokens, K]^T
// W4: the MXFP4 weights exactly as they sit in HBM (packed E2M1, canonical layout, no repack):
//     TMA brings 128-row x 256-element tiles (128-byte rows = one swizzle span) into shared
//     memory; the K tail and the row tail are filled with zeros by the copy engine, never fetched.
// A4: an activation row is a SUM of NT packed-FP4 terms (value, residual, residual of the
//     residual ...), each with its own E8M0 scales per 32 along K.  Three terms carry a bf16
//     activation to ~2e-3 of its block maximum, which keeps the layer within cosine 0.9999 of the
//     bf16-activation oracle, while every product still runs at the FP4 tensor rate and nothing
//     is dequantised in the main loop.  The terms of a block are stacked along N when they fit
//     one instruction (N = NT*B <= 256; the epilogue adds the column groups), otherwise each term
//     is its own instruction into the same accumulator.
//
// A pipeline stage (K = 256) carries TWO 128-row weight tiles that share one activation tile: the
// gate and the up rows of the same features (gate-up GEMM), or two consecutive row tiles of the
// down projection.  It is four copy instructions: weights, all activation terms, two scale groups.
//
// Warp roles (480 threads):
//   warp 0      TMA producer
//   warps 1,14  MMA issuers, one per weight tile of the stage (whole warp walks the loop, lane 0
//               issues; descriptors are precomputed 32-bit halves -- an issuing thread manages
//               about one instruction per 100 cycles, so two of them); warp 1 owns the TMEM
//   warps 2-9   epilogue, two per TMEM lane quadrant: activation with the oracle's bf16 roundings,
//               bf16 staging tile in shared memory, block-wise re-quantisation into the down GEMM's
//               operand format, overlapped with the next tile's main loop (two TMEM accumulators)
//   warps 10-13 scale loaders: copy the stage's E8M0 scale chunks shared memory -> registers ->
//               tensor memory (tcgen05.st, one warp per lane quadrant, two TMEM scale buffers).
//               tcgen05.cp would do the same copy but runs in the MMA's own in-order pipe at
//               ~70-100 cycles per chunk, which was the limiter at small token tiles.
// In the compute-bound regime (PAIR) two CTAs of a cluster share one token tile: tcgen05.mma.cta_group::2 with
// M = 256 takes 128 weight rows from each CTA's shared memory and HALF of the token rows from each, so every CTA
// fetches its own weight tiles and only half of the token tile (the launches there sit on the L2-to-SM path, and the
// token tile is more than half of a stage's bytes with three terms).  Each CTA keeps its own accumulators, scale
// columns, scale loaders and epilogue for ITS 128-row weight tiles; the even CTA issues all MMAs, its commits arrive
// on both CTAs' barriers, and the odd CTA's scale loaders and epilogue warps arrive on the even CTA's barriers.  No
// multicast loads anywhere.
// Persistent CTAs walk the work list (sorted block, weight tile pair) in block-major order so that
// CTAs running at the same time share activation tiles and neighbouring blocks of an expert share
// weight tiles in L2.
// All barrier waits are bounded; a wait that runs out sets status[] and the CTA unwinds (frees its
// tensor memory) instead of spinning.  A build with -DB200MOE_PROFILE additionally leaves cycle counters
// of CTA 0's roles in status[4..9]; the production build carries no timing code.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <mutex>

#include "gemm_common.cuh"

namespace b200moe {

constexpr int kThreads = 480;          // TMA warp, MMA warp, 8 epilogue warps, 4 scale-loader warps, 2nd MMA warp
constexpr int kMma2Warp = 14;          // issues the MMAs of the stage's second weight tile
constexpr int kTileM = 128;          // weight rows per MMA
constexpr int kStagePitch = kTileM * 2 + 16;   // bytes per token row of the bf16 staging tile
constexpr int kTileK = kKPad;        // K per pipeline stage: 256 (4 MMA K-steps of 64, 2 scale k-blocks of 128)
constexpr int kSub = kTileK / 128;   // scale k-blocks per stage
constexpr int kRowBytes = kTileK / 2;                // one tile row: 256 packed FP4 = 128 bytes = one swizzle span
constexpr int kATileBytes = kTileM * kRowBytes;      // 16 KB
constexpr int kMaxStages = 16;
constexpr int kMaxTerms = 4;
constexpr int kTmemCols = 512;
constexpr int kSfCol0 = kAccColsLimit;   // scale columns: 2 buffers x 48 = per k-block {A: 8 columns, B: up to 16}
constexpr int kSmemLimit = 232448;       // 227 KB

struct GemmParams {
  CUtensorMap tmW;     // weights: gate-up (K, I, 2, E) box (256,128,2,1); down (K, H, 1, E) box (256,256,1,1)
  CUtensorMap tmA;     // activations (KP, max_rows, NT terms)    box (256, B, NT)
  const uint8_t* w_scale;   // [E, MT, KB, 2, 512]
  const uint8_t* asf;       // [blocks, KB, chunks, 512]
  const uint32_t* sorted_ids;
  const int32_t* sorted_e;
  const int32_t* num_valid;
  int32_t* status;
  __nv_bfloat16* h_out;
  uint8_t* oq; uint8_t* osf;
  __nv_bfloat16* out2;
  int64_t max_rows;
  int64_t oq_term_stride;
  int B, NT, rows, KB, MT, E, topk, T, stages, out_kp, out_kb, out_ts, activation;
  int k_tail_steps;    // 64-wide k-steps of the last stage that hold data (the rest of it is zero padding)
  uint8_t* gstage;     // per-CTA staging tiles in global memory (L2) instead of shared memory, or null
  float swiglu_limit;
  const float* sorted_w;   // routing weight of every sorted row (fused combine, weights applied in the gate-up stage)
  const float* bias;       // per-expert bias: gate-up [E, 2*rows] (gate then up), down [E, rows]; or null
  __nv_bfloat16* y;        // down, fused combine: zeroed [T, rows] output accumulated with bf16x2 reductions; or null
  int weight_stage1;       // gate-up: multiply h by the routing weight (the down stage then applies none)
  int MTp;                 // PAIR: work items per sorted block (two consecutive weight-tile items, one per CTA of the pair)
};

struct SmemCtl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t sf_full[2];      // scale columns of a TMEM scale buffer are in place
  uint64_t sf_empty[2];     // ... and have been consumed by the MMAs that use them
  uint32_t tmem_base;
  uint32_t abort_word;
};

// geometry shared by host and device
struct StageGeom {
  int a_bytes, b_bytes, sfa_bytes, sfb_bytes, stage_bytes;
  uint32_t tx_bytes;
};
__host__ __device__ inline StageGeom stage_geom(int parts, int B, int NT, bool pair = false) {
  StageGeom g;
  g.a_bytes = parts * kATileBytes;
  g.b_bytes = NT * (pair ? B / 2 : B) * kRowBytes;     // a CTA of a pair holds half of the token rows
  g.sfa_bytes = kSub * parts * kSfChunk;
  g.sfb_bytes = kSub * act_sf_chunks(NT, act_term_stride(B, NT, parts)) * kSfChunk;
  g.stage_bytes = (g.a_bytes + g.b_bytes + g.sfa_bytes + g.sfb_bytes + 1023) & ~1023;
  g.tx_bytes = (uint32_t)(g.a_bytes + g.b_bytes + g.sfa_bytes + g.sfb_bytes);
  return g;
}

template <bool GATEUP, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
moe_grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
  constexpr int NA = 2;   // weight tiles per stage
  const uint32_t cta_rank = PAIR ? cluster_cta_rank() : 0u;    // 0: the CTA that issues the pair's MMAs
  const int NB = PAIR ? p.B / 2 : p.B;                         // token rows of the stage's tile held by THIS CTA
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment covers every swizzle atom used here
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(smem);
  const uint32_t stage0 = smem_u32(smem) + 1024;
  const int B = p.B, NT = p.NT;
  const StageGeom geo = stage_geom(NA, B, NT, PAIR);
  const int S = p.stages;
  const bool merged = !PAIR && act_merged(B, NT, NA);   // all terms in one MMA (N = NT*B)
  const int ncol = merged ? NT * B : B;        // TMEM columns of one accumulator
  const int acc_cols = NA * ncol;
  const int n_acc = (2 * acc_cols <= kAccColsLimit) ? 2 : 1;
  const int sfb_chunks = geo.sfb_bytes / (kSub * kSfChunk);   // per 128-wide k-block

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_word = &ctl->abort_word;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 2);      // one commit per MMA warp
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tmem_full[a]), 2);
      // PAIR: the issuing CTA waits for the epilogue warps and the scale loaders of BOTH CTAs
      mbar_init(smem_u32(&ctl->tmem_empty[a]), PAIR ? 16 : 8);
      mbar_init(smem_u32(&ctl->sf_full[a]), PAIR ? 8 : 4);
      mbar_init(smem_u32(&ctl->sf_empty[a]), 2);
    }
    ctl->abort_word = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(&ctl->tmem_base), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();      // the partner's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  // This CTA holds its tensor memory now, so CTAs of the next kernel may be scheduled beside it without
  // starving it; the sort arrays and quantised activations are valid once the predecessor has completed.
  grid_dep_launch();
  grid_dep_wait();

  const int64_t rows_live = min((int64_t)p.num_valid[0], p.max_rows);
  const int n_blocks = (int)(rows_live / B);
  // work items per sorted block, and how far apart a CTA's consecutive items are: a pair of CTAs takes ONE item (two
  // consecutive weight-tile items of the unpaired numbering, one per CTA)
  const int items_per_block = PAIR ? p.MTp : p.MT;
  const int total_work = n_blocks * items_per_block;
  const int total_work_mma = (PAIR && cta_rank != 0) ? 0 : total_work;     // only the even CTA of a pair issues MMAs
  const int w_first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int w_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  // row ids of work item w's sorted block, 32 per lane group (the live rows of a block are a prefix of it)
  auto fetch_ids = [&](int w, uint32_t (&r)[4]) {
    const int r0 = (w / items_per_block) * B;
#pragma unroll
    for (int q = 0; q < 4; ++q) r[q] = (w < total_work && q * 32 + lane < B) ? p.sorted_ids[r0 + q * 32 + lane] : 0xFFFFFFFFu;
  };
  auto live_rows = [&](const uint32_t (&r)[4]) {
    int n = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      n += __popc(__ballot_sync(0xffffffffu, (int)(r[q] >> 24) < p.topk && (int)(r[q] & 0xFFFFFFu) < p.T));
    return n;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the loop (PAIR: it counts the block's live rows with ballots); lane 0 waits and issues.
    if (lane == 0) {
      prefetch_tensormap(&p.tmW);
      prefetch_tensormap(&p.tmA);
    }
    int stage = 0;
    uint32_t phase = 0;
    int64_t issued = 0;
    bool ok = true;
    PROF_DECL(t_wait);
    const int64_t sfa_step = geo.sfa_bytes;
    uint32_t pid[4];
    if (PAIR) fetch_ids(w_first, pid);
    for (int w = w_first; w < total_work && ok; w += w_step) {
      // PAIR: the MMAs span only the live rows of the block (rounded up to 16), half of them from each CTA: this
      // CTA fetches the token rows from its half's first row on (the box keeps its size; rows beyond are unused)
      int row_off = 0;
      if (PAIR) {
        const int n_mma = min(B, max(16, (live_rows(pid) + 15) & ~15));
        fetch_ids(w + w_step, pid);
        row_off = (int)cta_rank * (n_mma / 2);
      }
      if (lane == 0) {
        // (PAIR: item w covers weight-tile items 2*mp and 2*mp + 1 of the block; this CTA takes the one of its rank)
        const int b = w / items_per_block, m = PAIR ? 2 * (w - b * items_per_block) + (int)cta_rank : w - b * items_per_block;
        const bool tile_live = m < p.MT;
        const int ms = tile_live ? m : p.MT - 1;       // a tile beyond the last one borrows its neighbour's (finite) scales
        int e = p.sorted_e[b];
        if (e < 0 || e >= p.E) { p.status[2] = 1; e = 0; }
        const int r0 = b * B;
        const uint8_t* sfa = p.w_scale + ((int64_t)e * p.MT + ms) * p.KB * sfa_step;   // KB stages of kSub k-blocks
        const uint8_t* sfb = p.asf + (int64_t)b * p.KB * geo.sfb_bytes;
        for (int kb = 0; kb < p.KB; ++kb) {
          const long long tw0 = PROF_NOW();
          if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1, abort_word, 0x100 + stage)) { ok = false; break; }
          PROF_ADD(t_wait, tw0);
          const uint32_t st = stage0 + (uint32_t)stage * geo.stage_bytes;
          const uint32_t full = smem_u32(&ctl->full[stage]);
          if (PAIR) {
            // The weight tiles and this CTA's half of the token tile complete bytes on the ISSUING CTA's barrier (it
            // alone consumes them, through the MMAs); the scale chunks are consumed by this CTA's own scale loaders
            // and complete on the local barrier.
            const uint32_t ab = (uint32_t)(geo.a_bytes + geo.b_bytes), sf = (uint32_t)(geo.sfa_bytes + geo.sfb_bytes);
            mbar_expect_tx(full, cta_rank == 0 ? 2 * ab + sf : sf);
            tma_load_4d_pair(st, &p.tmW, full, kb * kTileK, m * (GATEUP ? kTileM : 2 * kTileM), 0, e);
            tma_load_3d_pair(st + geo.a_bytes, &p.tmA, full, kb * kTileK, r0 + row_off, 0);
          } else {
            mbar_expect_tx(full, geo.tx_bytes);
            tma_load_4d(st, &p.tmW, full, kb * kTileK, m * (GATEUP ? kTileM : 2 * kTileM), 0, e);
            tma_load_3d(st + geo.a_bytes, &p.tmA, full, kb * kTileK, r0, 0);
          }
          bulk_load(st + geo.a_bytes + geo.b_bytes, sfa, (uint32_t)geo.sfa_bytes, full);
          bulk_load(st + geo.a_bytes + geo.b_bytes + geo.sfa_bytes, sfb, (uint32_t)geo.sfb_bytes, full);
          sfa += sfa_step;
          sfb += geo.sfb_bytes;
          ++issued;
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    }
    if (lane == 0) {
#ifdef B200MOE_PROFILE
      if (blockIdx.x == 0) p.status[4] = (int32_t)(t_wait >> 10);   // kilo-cycles waiting for a free stage
#endif
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
  } else if (warp == 1 || warp == kMma2Warp) {
    // ------------------------------------------------------------------ MMA issuers
    // Two warps, one per weight tile of the stage (gate / up, or the two down tiles): a single
    // issuing thread tops out near 100 cycles per instruction, two double the issue rate and
    // write disjoint accumulators.  The whole warp walks the loop (uniform control flow); lane 0
    // issues.  Every barrier this role completes counts two arrivals.
    const uint32_t part = (warp == 1) ? 0u : 1u;
    uint32_t idesc[2];
#pragma unroll
    for (int s = 0; s < 2; ++s)
      idesc[s] = make_idesc_block_scaled(kFmtE2M1_mxf4, kFmtE2M1_mxf4, PAIR ? 2 * kTileM : kTileM, (uint32_t)ncol, 2 * s, 2 * s);
    const uint32_t term_lo = (uint32_t)(NB * kRowBytes) >> 4;   // descriptor step from one term to the next
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t sf_buf = 0, sf_phase = 0;   // scale columns alternate between two TMEM buffers
    bool ok = true;
    PROF_DECL(t_wait_acc);
    PROF_DECL(t_wait_full);
    PROF_DECL(t_wait_sf);
    const long long t_begin = PROF_NOW();
    (void)t_begin;
    // Per-term MMAs cover only the live rows of the block (rounded up to 16): the padding rows that end an
    // expert's last block cost neither tensor time nor operand reads.  The row ids of the NEXT item are
    // fetched while the current one is multiplied, so the count is ready without a stall.
    uint32_t nid[4];
    fetch_ids(w_first, nid);
    for (int w = w_first; w < total_work_mma && ok; w += w_step) {
      const int nlive = live_rows(nid);
      fetch_ids(w + w_step, nid);
      // (PAIR: each CTA supplies half of these rows; its producer fetched them from the half's first row on)
      const uint32_t n_mma = merged ? (uint32_t)ncol : (uint32_t)min(B, max(16, (nlive + 15) & ~15));
      uint32_t idesc_w[2];
#pragma unroll
      for (int s = 0; s < 2; ++s) idesc_w[s] = (idesc[s] & ~(0x3Fu << 17)) | ((n_mma >> 3) << 17);
      const long long ta0 = PROF_NOW();
      if (!mbar_wait(smem_u32(&ctl->tmem_empty[acc]), acc_phase ^ 1, abort_word, 0x200 + acc)) break;
      PROF_ADD(t_wait_acc, ta0);
      tc_fence_after_sync();
      const uint32_t d0 = tmem_base + acc * acc_cols + part * ncol;
      for (int kb = 0; kb < p.KB; ++kb) {
        const long long tf0 = PROF_NOW();
        if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_word, 0x300 + stage)) { ok = false; break; }
        PROF_ADD(t_wait_full, tf0);
        const long long ts0 = PROF_NOW();
        if (!mbar_wait(smem_u32(&ctl->sf_full[sf_buf]), sf_phase, abort_word, 0x500 + sf_buf)) { ok = false; break; }
        PROF_ADD(t_wait_sf, ts0);
        tc_fence_after_sync();
        __syncwarp();
        if (elect_one()) {       // one issuing lane; descriptors stay in uniform registers
          const uint32_t st = stage0 + (uint32_t)stage * geo.stage_bytes;
          const uint32_t a_lo = desc_lo_sw(st + part * kATileBytes);
          const uint32_t b_lo = desc_lo_sw(st + geo.a_bytes);
          // scale columns of this stage (written by the scale-loader warps): per 128-wide k-block
          // {A: gate/up or tile pair, 8 columns}, then {B: up to 16 columns}
          const uint32_t sfa_t = tmem_base + kSfCol0 + sf_buf * 48 + 4 * part;
          const uint32_t sfb_t = tmem_base + kSfCol0 + sf_buf * 48 + 16;
          const uint32_t first = kb != 0;
          const int nsteps = (kb == p.KB - 1) ? p.k_tail_steps : 2 * kSub;   // skip k-steps that are all padding
          if (merged) {
#pragma unroll
            for (int s = 0; s < 2 * kSub; ++s) {
              const uint32_t sa = sfa_t + 8 * (s >> 1), sb = sfb_t + 16 * (s >> 1);
              if (s < nsteps) umma_mxf4(d0, a_lo + 2 * s, b_lo + 2 * s, idesc_w[s & 1], sa, sb, s == 0 ? first : 1u);
            }
          } else {
#pragma unroll
            for (int s = 0; s < 2 * kSub; ++s) {
              const uint32_t sa = sfa_t + 8 * (s >> 1), sb = sfb_t + 16 * (s >> 1);
#pragma unroll
              for (int t = 0; t < kMaxTerms; ++t) {
                if (t < NT && s < nsteps) {
                  const uint32_t accum = (s == 0 && t == 0) ? first : 1u;
                  if (PAIR) umma_mxf4_pair(d0, a_lo + 2 * s, b_lo + t * term_lo + 2 * s, idesc_w[s & 1], sa, sb + 4 * t, accum);
                  else umma_mxf4(d0, a_lo + 2 * s, b_lo + t * term_lo + 2 * s, idesc_w[s & 1], sa, sb + 4 * t, accum);
                }
              }
            }
          }
          if (PAIR) {      // both CTAs' producers and scale loaders wait for these
            tc_commit_pair(smem_u32(&ctl->empty[stage]));
            tc_commit_pair(smem_u32(&ctl->sf_empty[sf_buf]));
          } else {
            tc_commit(smem_u32(&ctl->empty[stage]));
            tc_commit(smem_u32(&ctl->sf_empty[sf_buf]));
          }
        }
        __syncwarp();
        if (sf_buf == 1) sf_phase ^= 1;
        sf_buf ^= 1;
        if (++stage == S) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (lane == 0) {
        if (PAIR) tc_commit_pair(smem_u32(&ctl->tmem_full[acc])); else tc_commit(smem_u32(&ctl->tmem_full[acc]));
      }
      __syncwarp();
      if (n_acc == 2) { acc ^= 1; if (acc == 0) acc_phase ^= 1; } else { acc_phase ^= 1; }
    }
#ifdef B200MOE_PROFILE
    if (blockIdx.x == 0 && lane == 0 && part == 0) {   // kilo-cycles of an MMA warp: total, waiting for data, for TMEM, for scale columns (status[10])
      p.status[5] = (int32_t)((clock64() - t_begin) >> 10);
      p.status[6] = (int32_t)(t_wait_full >> 10);
      p.status[7] = (int32_t)(t_wait_acc >> 10);
      p.status[10] = (int32_t)(t_wait_sf >> 10);
    }
#endif
  } else if (warp >= 10) {
    // ------------------------------------------------------------------ scale-loader warps
    // Four warps, one per TMEM lane quadrant.  A scale chunk in shared memory is 32 rows x 16
    // bytes; lane l of every quadrant needs row l (the MMA expects the 32-row image replicated
    // in all four quadrants), so each warp reads the chunk and stores it to its own quadrant
    // with tcgen05.st -- this keeps the scale traffic out of the MMA issue stream.
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int stage = 0;
    uint32_t phase = 0, sf_buf = 0, sf_phase = 0;
    bool ok = true;
    for (int w = w_first; w < total_work && ok; w += w_step) {
      for (int kb = 0; kb < p.KB; ++kb) {
        if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_word, 0x600 + stage) ||
            !mbar_wait(smem_u32(&ctl->sf_empty[sf_buf]), sf_phase ^ 1, abort_word, 0x700 + sf_buf)) {
          ok = false;
          break;
        }
        const uint32_t sf_s = stage0 + (uint32_t)stage * geo.stage_bytes + geo.a_bytes + geo.b_bytes + lane * 16;
        const uint32_t sfa_t = tmem_base + lane_base + kSfCol0 + sf_buf * 48;
        uint4 a0 = ld_shared_v4(sf_s), a1 = ld_shared_v4(sf_s + kSfChunk), a2 = ld_shared_v4(sf_s + 2 * kSfChunk),
              a3 = ld_shared_v4(sf_s + 3 * kSfChunk);
        tmem_st_32x32b_x16(sfa_t, a0, a1, a2, a3);
#pragma unroll
        for (int kk = 0; kk < kSub; ++kk) {
#pragma unroll
          for (int c = 0; c < kMaxTerms; ++c) {
            if (c < sfb_chunks) {
              const uint4 v = ld_shared_v4(sf_s + geo.sfa_bytes + (kk * sfb_chunks + c) * kSfChunk);
              tmem_st_32x32b_x4(sfa_t + 16 + 16 * kk + 4 * c, v);
            }
          }
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_leader(smem_u32(&ctl->sf_full[sf_buf])); else mbar_arrive(smem_u32(&ctl->sf_full[sf_buf]));
        }
        if (sf_buf == 1) sf_phase ^= 1;
        sf_buf ^= 1;
        if (++stage == S) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    // Eight warps: warp w reads TMEM lanes [32*(w%4), +32) (the hardware's lane-quadrant rule);
    // the two warps of a quadrant split the token columns in alternating groups of 16.
    const int ew = warp - 2;                   // 0..7
    const int quad = warp & 3;                 // TMEM lanes [32*quad, 32*quad+32)
    const int half = ew >> 2;
    const int tid_e = ew * 32 + lane;          // 0..255
    const int row_local = quad * 32 + lane;
    const int64_t oq_pitch = p.out_kp / 2;
    const uint32_t stg = stage0 + (uint32_t)S * geo.stage_bytes;   // bf16 staging tile [B][kStagePitch]
    // the same tile in global memory (it stays in L2) when that frees the shared memory of one more pipeline stage
    uint8_t* const gstg = p.gstage ? p.gstage + (size_t)blockIdx.x * B * kStagePitch : nullptr;
    const bool fused = GATEUP && p.h_out == nullptr;
    int acc = 0;
    uint32_t acc_phase = 0;
    PROF_DECL(t_wait_epi);
    const long long t_begin_epi = PROF_NOW();
    (void)t_begin_epi;
    for (int w = w_first; w < total_work; w += w_step) {
      const int b = w / items_per_block, m = PAIR ? 2 * (w - b * items_per_block) + (int)cta_rank : w - b * items_per_block;
      const bool tile_live = m < p.MT;      // PAIR: the odd CTA's tile of the last item may lie beyond the weight rows
      const int r0 = b * B;
      // output feature of this thread: gate-up pairs gate/up of feature j; down holds j and j+128
      const int j = (GATEUP ? m * kTileM : m * 2 * kTileM) + row_local;
      // valid rows are a prefix of the block (padding sentinels follow)
      int nvalid = 0;
      for (int q = 0; q < B; q += 32) {
        const uint32_t id = (q + lane < B) ? p.sorted_ids[r0 + q + lane] : 0xFFFFFFFFu;
        nvalid += __popc(__ballot_sync(0xffffffffu, (int)(id >> 24) < p.topk && (int)(id & 0xFFFFFFu) < p.T));
      }
      if (!tile_live) nvalid = 0;       // nothing to read or store; the barrier protocol below still runs
      // all eight warps take the same decision, so nobody is left alone at a later barrier
      const long long te0 = PROF_NOW();
      const bool ok = mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_phase, abort_word, 0x400 + acc);
      if (!epi_all(ok)) break;
      PROF_ADD(t_wait_epi, te0);
      tc_fence_after_sync();
      const uint32_t t0 = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * acc_cols;
      const bool j_ok = j < p.rows;
      const bool j2_ok = !GATEUP && j + kTileM < p.rows;
      // per-expert bias of this thread's two output features (gate / up of feature j, or features j and j + 128)
      float bias0 = 0.f, bias1 = 0.f;
      if (p.bias != nullptr) {
        int e = p.sorted_e[b];
        if (e < 0 || e >= p.E) e = 0;
        const float* be = p.bias + (int64_t)e * (GATEUP ? 2 : 1) * p.rows;
        if (j_ok) bias0 = be[j];
        if (GATEUP ? j_ok : j2_ok) bias1 = be[j + (GATEUP ? p.rows : kTileM)];
      }
      const bool col_weights = GATEUP ? (p.weight_stage1 != 0) : (p.y != nullptr);
      uint32_t my_id = 0;
      for (int c0 = half * 16; c0 < nvalid; c0 += 32) {
        uint32_t g[16], u[16];
        tmem_ld_32x32b_x16(t0 + c0, g);
        tmem_ld_32x32b_x16(t0 + ncol + c0, u);
        tmem_ld_wait();
        if (merged) {
          // the terms were separate column groups of one instruction: add them up
          for (int t = 1; t < NT; ++t) {
            uint32_t g2[16], u2[16];
            tmem_ld_32x32b_x16(t0 + t * B + c0, g2);
            tmem_ld_32x32b_x16(t0 + ncol + t * B + c0, u2);
            tmem_ld_wait();
#pragma unroll
            for (int n = 0; n < 16; ++n) {
              g[n] = __float_as_uint(__uint_as_float(g[n]) + __uint_as_float(g2[n]));
              u[n] = __float_as_uint(__uint_as_float(u[n]) + __uint_as_float(u2[n]));
            }
          }
        }
        if (p.bias != nullptr) {
          // the oracle's matmul returns bf16 and the bias is added to that (one more rounding follows below)
#pragma unroll
          for (int n = 0; n < 16; ++n) {
            g[n] = __float_as_uint(bf16r(__uint_as_float(g[n])) + bias0);
            u[n] = __float_as_uint(bf16r(__uint_as_float(u[n])) + bias1);
          }
        }
        // routing weight of the chunk's token columns (lane n holds column c0 + n)
        float my_w = 1.f;
        if (col_weights && p.sorted_w != nullptr) my_w = p.sorted_w[min(r0 + c0 + (lane & 15), r0 + B - 1)];
        if (GATEUP) {
          if (!fused) {
            my_id = p.sorted_ids[min(r0 + c0 + lane, r0 + B - 1)];
#pragma unroll
            for (int n = 0; n < 16; ++n) {
              const uint32_t id = __shfl_sync(0xffffffffu, my_id, n);
              if (c0 + n < nvalid) {
                const int tok = (int)(id & 0xFFFFFFu), kk = (int)(id >> 24);
                float v = gateup_act(__uint_as_float(g[n]), __uint_as_float(u[n]), p.activation,
                                     p.swiglu_limit);
                if (p.weight_stage1) v *= __shfl_sync(0xffffffffu, my_w, n);
                if (j_ok) p.h_out[((int64_t)tok * p.topk + kk) * p.rows + j] = __float2bfloat16_rn(v);
              }
            }
          } else {
            // h (already rounded to bf16, as the oracle's h is) goes to the staging tile,
            // token-major, for the block-wise re-quantisation below
#pragma unroll
            for (int n = 0; n < 16; n += 2) {
              if (c0 + n < nvalid) {
                __nv_bfloat162 v = gateup_act2(__uint_as_float(g[n]), __uint_as_float(u[n]), __uint_as_float(g[n + 1]),
                                               __uint_as_float(u[n + 1]), p.activation, p.swiglu_limit);
                if (p.weight_stage1) {
                  const float2 f = __bfloat1622float2(v);
                  v = __floats2bfloat162_rn(f.x * __shfl_sync(0xffffffffu, my_w, n), f.y * __shfl_sync(0xffffffffu, my_w, n + 1));
                }
                if (!j_ok) v = __floats2bfloat162_rn(0.f, 0.f);
                if (gstg) {
                  *reinterpret_cast<unsigned short*>(gstg + (size_t)(c0 + n) * kStagePitch + row_local * 2) =
                      __bfloat16_as_ushort(v.x);
                  if (c0 + n + 1 < nvalid)
                    *reinterpret_cast<unsigned short*>(gstg + (size_t)(c0 + n + 1) * kStagePitch + row_local * 2) =
                        __bfloat16_as_ushort(v.y);
                } else {
                  st_shared_u16(stg + (uint32_t)(c0 + n) * kStagePitch + row_local * 2, __bfloat16_as_ushort(v.x));
                  if (c0 + n + 1 < nvalid)
                    st_shared_u16(stg + (uint32_t)(c0 + n + 1) * kStagePitch + row_local * 2, __bfloat16_as_ushort(v.y));
                }
              }
            }
          }
        } else if (p.y == nullptr) {
#pragma unroll
          for (int n = 0; n < 16; ++n) {
            if (c0 + n < nvalid) {
              __nv_bfloat16* row = p.out2 + ((int64_t)r0 + c0 + n) * p.rows + j;
              if (j_ok) row[0] = __float2bfloat16_rn(__uint_as_float(g[n]));
              if (j2_ok) row[kTileM] = __float2bfloat16_rn(__uint_as_float(u[n]));
            }
          }
        } else {
          // Fused combine: y[token, feature] += bf16(bf16(acc) * routing weight), accumulated in HBM/L2 with
          // packed bf16x2 reductions (the reference's epilogue: src/contrib/moe.py:703-787).  Neighbouring
          // lanes hold neighbouring features, so a pair of lanes swaps one value per two token columns: the
          // even lane then owns features (j, j+1) of column n, the odd lane features (j-1, j) of column n+1.
          my_id = p.sorted_ids[min(r0 + c0 + (lane & 15), r0 + B - 1)];
          const bool odd = lane & 1;
          const int jp = j & ~1;
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
                  atomicAdd(reinterpret_cast<__nv_bfloat162*>(row + kTileM),
                            odd ? __floats2bfloat162_rn(ru, u1) : __floats2bfloat162_rn(u0, ru));
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      if (fused) epi_sync(); else __syncwarp();      // staging tile complete, TMEM reads done
      if (lane == 0) {       // PAIR: the issuing CTA reuses the accumulators once both CTAs' epilogues have read theirs
        if (PAIR) mbar_arrive_leader(smem_u32(&ctl->tmem_empty[acc])); else mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
      }
      if (n_acc == 2) { acc ^= 1; if (acc == 0) acc_phase ^= 1; } else { acc_phase ^= 1; }

      if (fused) {
        // Re-quantise h into the operand format of the down GEMM: one thread per (token row,
        // 32-feature block), NT packed-FP4 terms with an E8M0 scale each -- the same arithmetic
        // as the stand-alone quantiser -- written as 16-byte vectors in sorted-row order.
        for (int unit = tid_e; unit < nvalid * 4; unit += 256) {
          const int n = unit >> 2, q = unit & 3;
          float x[32];
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            const uint4 raw = gstg ? __ldcg(reinterpret_cast<const uint4*>(gstg + (size_t)n * kStagePitch + q * 64 + v4 * 16))
                                   : ld_shared_v4(stg + (uint32_t)n * kStagePitch + q * 64 + v4 * 16);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 f = __bfloat1622float2(b2[t]);
              x[v4 * 8 + t * 2] = f.x;
              x[v4 * 8 + t * 2 + 1] = f.y;
            }
          }
          const int64_t r = (int64_t)r0 + n;
          for (int t = 0; t < NT; ++t) {
            uint4 pk;
            const int e = (t + 1 < NT) ? quant_block32_fp4<true>(x, pk) : quant_block32_fp4<false>(x, pk);
            *reinterpret_cast<uint4*>(p.oq + t * p.oq_term_stride + r * oq_pitch + (m * kTileM + q * 32) / 2) = pk;
            p.osf[act_sf_index(b, m, p.out_kb, B, NT, p.out_ts, t, n, q)] = (uint8_t)e;
          }
        }
        // the K padding of the down GEMM (features beyond the last weight tile) must hold zeros
        // and a finite scale: the CTA that owns the last tile writes it
        if (m == p.MT - 1) {
          const int pad_blocks = (p.out_kp - p.MT * kTileM) / 32;
          for (int unit = tid_e; unit < nvalid * pad_blocks; unit += 256) {
            const int n = unit / pad_blocks, qb = p.MT * 4 + unit % pad_blocks;   // 32-feature block index
            const int64_t r = (int64_t)r0 + n;
            for (int t = 0; t < NT; ++t) {
              *reinterpret_cast<uint4*>(p.oq + t * p.oq_term_stride + r * oq_pitch + qb * 16) = make_uint4(0, 0, 0, 0);
              p.osf[act_sf_index(b, qb >> 2, p.out_kb, B, NT, p.out_ts, t, n, qb & 3)] = 0;
            }
          }
        }
      }
    }
#ifdef B200MOE_PROFILE
    if (blockIdx.x == 0 && tid_e == 0) {   // kilo-cycles of an epilogue warp: total, waiting for a tile
      p.status[8] = (int32_t)((clock64() - t_begin_epi) >> 10);
      p.status[9] = (int32_t)(t_wait_epi >> 10);
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
  if (PAIR) cluster_sync_all();     // neither CTA leaves while the other's MMAs or barrier arrivals may still touch it
  if (warp == 1) {
    if (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
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

int device_sm_count() {
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

int encode_map_sw(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base,
                         const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
                         CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo, const char* what) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return set_error(-2, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, type, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(-3, "cuTensorMapEncodeTiled(%s) failed with CUresult %d (base %p dims %llu,%llu,%llu)", what,
                     (int)r, base, (unsigned long long)dims[0], (unsigned long long)dims[1],
                     (unsigned long long)(rank > 2 ? dims[2] : 0));
  return 0;
}

int launch_grouped_gemm(const GemmArgs& a, cudaStream_t st) {
  B200_CHECK_ARG(a.N >= 16 && a.N <= 128 && a.N % 16 == 0, "grouped gemm: token tile %d is not a multiple of 16 in [16,128]",
                 a.N);
  B200_CHECK_ARG(a.NT >= 1 && a.NT <= kMaxTerms, "grouped gemm: %d activation terms (1..4 supported)", a.NT);
  B200_CHECK_ARG(a.Kd % 32 == 0 && a.rows > 0 && a.E > 0, "grouped gemm: bad shape");
  B200_CHECK_ARG(a.max_rows % a.N == 0, "grouped gemm: max_rows %% B != 0");
  B200_CHECK_ARG(((uintptr_t)a.w_data & 15) == 0 && ((uintptr_t)a.a_q & 15) == 0,
                 "grouped gemm: operand tensors must be 16-byte aligned");
  const int KP = (int)round_up64(a.Kd, kTileK);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.B = a.N; p.NT = a.NT; p.rows = a.rows; p.KB = KP / kTileK;
  p.MT = a.gateup ? (a.rows + kTileM - 1) / kTileM : (a.rows + 2 * kTileM - 1) / (2 * kTileM);
  p.k_tail_steps = (a.Kd - (p.KB - 1) * kTileK + 63) / 64;
  p.E = a.E; p.topk = a.topk; p.T = a.T; p.activation = a.activation;
  p.swiglu_limit = a.swiglu_limit; p.max_rows = a.max_rows;
  p.w_scale = (const uint8_t*)a.w_scale; p.asf = (const uint8_t*)a.asf;
  p.sorted_ids = a.sorted_ids; p.sorted_e = a.sorted_e; p.num_valid = a.num_valid; p.status = a.status;
  p.h_out = (__nv_bfloat16*)a.h_out; p.oq = (uint8_t*)a.oq; p.osf = (uint8_t*)a.osf;
  p.out_kp = a.out_kp; p.out_kb = a.out_kp / 128; p.out_ts = act_term_stride(a.N, a.NT, 2);
  p.oq_term_stride = a.max_rows * (int64_t)(a.out_kp / 2);
  p.out2 = (__nv_bfloat16*)a.out2;
  p.sorted_w = a.sorted_w; p.bias = a.bias; p.y = a.gateup ? nullptr : (__nv_bfloat16*)a.y;
  p.weight_stage1 = (a.gateup && a.weight_stage1) ? 1 : 0;
  B200_CHECK_ARG(p.weight_stage1 == 0 || a.sorted_w != nullptr, "grouped gemm: routing weights missing");
  B200_CHECK_ARG(p.y == nullptr || (a.rows % 2 == 0 && ((uintptr_t)p.y & 3) == 0), "grouped gemm: fused combine needs an even row length");
  if (a.gateup && a.h_out == nullptr)
    B200_CHECK_ARG(a.out_kp == (int)round_up64(a.rows, kTileK) && a.oq && a.osf,
                   "gate-up: fused output buffers missing");

  // weights: canonical packed FP4, gate-up [E, 2, I, H/2] / down [E, H, I/2]; K and row tails are
  // zero-filled by TMA
  const cuuint64_t row_pitch = (cuuint64_t)a.Kd / 2;
  {
    const cuuint64_t parts = a.gateup ? 2 : 1;
    cuuint64_t dims[4] = {(cuuint64_t)a.Kd, (cuuint64_t)a.rows, parts, (cuuint64_t)a.E};
    cuuint64_t strides[3] = {row_pitch, row_pitch * (cuuint64_t)a.rows, row_pitch * (cuuint64_t)a.rows * parts};
    cuuint32_t box[4] = {kTileK, a.gateup ? (cuuint32_t)kTileM : 2u * kTileM, a.gateup ? 2u : 1u, 1};
    int rc = encode_map_sw(&p.tmW, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B, 4, a.w_data, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "weights");
    if (rc) return rc;
  }
  // CTA pairs (tcgen05.mma.cta_group::2) in the compute-bound regime: large token tiles whose terms are separate
  // instructions.  pair_mode 0 = this choice, 1 = never, 2 = wherever the tile allows it.
  // (a single term is the same instruction stream stacked or not, and its scale layout is the same too)
  const bool pair_ok = (!act_merged(a.N, a.NT, 2) || a.NT == 1) && a.N % 16 == 0 && device_sm_count() >= 2;
  const bool pair = pair_ok && a.pair_mode != 1 && (a.pair_mode == 2 || a.N >= 64);
  p.MTp = (p.MT + 1) / 2;
  {
    cuuint64_t dims[3] = {(cuuint64_t)KP, (cuuint64_t)a.max_rows, (cuuint64_t)a.NT};
    cuuint64_t strides[2] = {(cuuint64_t)KP / 2, (cuuint64_t)(KP / 2) * (cuuint64_t)a.max_rows};
    cuuint32_t box[3] = {kTileK, (cuuint32_t)(pair ? a.N / 2 : a.N), (cuuint32_t)a.NT};   // a CTA of a pair fetches half of the rows
    int rc = encode_map_sw(&p.tmA, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B, 3, a.a_q, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "activations");
    if (rc) return rc;
  }

  const StageGeom geo = stage_geom(2, a.N, a.NT, pair);
  int staging = (a.gateup && a.h_out == nullptr) ? a.N * kStagePitch : 0;
  int stages = (kSmemLimit - 2048 - staging) / geo.stage_bytes;
  // two stages are too few to cover the load latency: where moving the staging tile of the fused epilogue to
  // global memory (one tile per CTA, L2-resident) buys a third (a fourth for CTA pairs), do that
  const int stages_g = (kSmemLimit - 2048) / geo.stage_bytes;
  if (staging && stages < (pair ? 4 : 3) && stages_g > stages && a.gstage != nullptr &&
      a.gstage_bytes >= (int64_t)device_sm_count() * staging) {
    p.gstage = (uint8_t*)a.gstage;
    staging = 0;
    stages = stages_g;
  }
  stages = std::min(stages, kMaxStages);
  B200_CHECK_ARG(stages >= 2, "grouped gemm: tile does not fit shared memory");
  p.stages = stages;
  const size_t smem = 2048 + (size_t)stages * geo.stage_bytes + staging;

  const int64_t max_work = (a.max_rows / a.N) * (pair ? p.MTp : p.MT);
  const int sms = device_sm_count();
  const int grid = pair ? 2 * (int)std::min<int64_t>(sms / 2, std::max<int64_t>(max_work, 1))
                        : (int)std::min<int64_t>(sms, std::max<int64_t>(max_work, 1));
  void (*kernel)(GemmParams) = a.gateup ? (pair ? moe_grouped_gemm_kernel<true, true> : moe_grouped_gemm_kernel<true, false>)
                                        : (pair ? moe_grouped_gemm_kernel<false, true> : moe_grouped_gemm_kernel<false, false>);
  // the attribute belongs to the (function, device) pair and setting it is cheap: do it on every launch
  B200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
  B200_CHECK_CUDA(launch_chained_cluster(kernel, dim3(grid), dim3(kThreads), smem, st, pair ? 2 : 1, p));
  B200_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------
// known-answer probes of the hardware paths the main loop depends on
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
    mbar_expect_tx(smem_u32(&bar), kATileBytes);
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
    utccp_sf(tbase, desc_lo_sf(smem_u32(chunk)));
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

// Dense MMA rate probe: `count` block-scaled MMAs of shape 128 x N x (64 for packed FP4, 32 for e4m3) alternating
// between two accumulators, issued by one elected lane from resident pseudo-random tiles with unit scales, one
// commit, one bounded wait; reports clock cycles.  The results are never read back.  Launched on every SM at
// once and timed by the caller it gives the chip's dense tensor rate for the kind.
__global__ void __launch_bounds__(128, 1) probe_mma_rate_kernel(const int32_t* cfg, uint32_t* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot, abort_word;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < (16384 + 32768 + 1024) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem)[i] = (i < (16384 + 32768) / 4) ? ((uint32_t)(i + 1) * 2654435761u) & 0x77777777u : 0x7F7F7F7Fu;
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
  const uint32_t a = smem_u32(smem), b = a + 16384, sf = b + 32768;
  const int kind = cfg[0], N = cfg[1], count = cfg[2];
  if (warp == 0 && elect_one()) {
    utccp_sf(tbase + 448, desc_lo_sf(sf));
    utccp_sf(tbase + 456, desc_lo_sf(sf + 512));
    utccp_sf(tbase + 460, desc_lo_sf(sf + 512));
    const uint32_t fmt = kind == 0 ? kFmtE2M1_mxf4 : kFmtE4M3;
    uint32_t idesc[2];
    for (int k = 0; k < 2; ++k) idesc[k] = make_idesc_block_scaled(fmt, fmt, 128, N, kind == 0 ? 2 * k : k, kind == 0 ? 2 * k : k);
    const uint32_t a_lo = desc_lo_sw(a), b_lo = desc_lo_sw(b);
    const uint32_t d1 = tbase + N;
    const long long t0 = clock64();
    for (int i = 0; i < count; i += 4) {
      if (kind == 0) {
        umma_mxf4(tbase, a_lo, b_lo, idesc[0], tbase + 448, tbase + 456, 1);
        umma_mxf4(d1, a_lo, b_lo, idesc[0], tbase + 448, tbase + 456, 1);
        umma_mxf4(tbase, a_lo + 2, b_lo + 2, idesc[1], tbase + 448, tbase + 456, 1);
        umma_mxf4(d1, a_lo + 2, b_lo + 2, idesc[1], tbase + 448, tbase + 456, 1);
      } else {
        umma_mxf8(tbase, a_lo, b_lo, idesc[0], tbase + 448, tbase + 456, 1);
        umma_mxf8(d1, a_lo, b_lo, idesc[0], tbase + 448, tbase + 456, 1);
        umma_mxf8(tbase, a_lo + 2, b_lo + 2, idesc[1], tbase + 448, tbase + 456, 1);
        umma_mxf8(d1, a_lo + 2, b_lo + 2, idesc[1], tbase + 448, tbase + 456, 1);
      }
    }
    const long long t1 = clock64();
    tc_commit(smem_u32(&bar));
    mbar_wait(smem_u32(&bar), 0, &abort_word, 3);
    const long long t2 = clock64();
    uint32_t* o = out + 3 * blockIdx.x;
    o[0] = (uint32_t)(t1 - t0);
    o[1] = (uint32_t)(t2 - t0);
    o[2] = abort_word;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// The bounded wait itself, made to run out: a barrier that nothing ever arrives on, a limit of in[0] microseconds.
// The kernel must come back with the wait's id in the status word and the context must stay usable -- this is how
// every role of the GEMM kernels gives up on a wait instead of hanging the GPU.
__global__ void __launch_bounds__(32, 1) probe_wait_expiry_kernel(const int32_t* in, uint32_t* out) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const uint64_t t0 = global_timer_ns();
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_word, 0xBEEFu, (uint64_t)max(in[0], 1) * 1000ull);
    const uint64_t dt = global_timer_ns() - t0;
    out[0] = abort_word;
    out[1] = ok ? 1u : 0u;
    out[2] = (uint32_t)(dt / 1000ull);        // microseconds the wait lasted
  }
}

int run_debug_probe(int which, const void* in, void* out, cudaStream_t st) {
  if (which == 1) {
    CUtensorMap map;
    cuuint64_t dims[3] = {256, 128, 1};
    cuuint64_t strides[2] = {128, 128 * 128};
    cuuint32_t box[3] = {256, 128, 1};
    int rc = encode_map_sw(&map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B, 3, in, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, "probe tile");
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
  if (which == 4) {
    // the attribute belongs to the (function, device) pair and setting it is cheap: do it on every launch
    B200_CHECK_CUDA(cudaFuncSetAttribute(probe_mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));
    probe_mma_rate_kernel<<<device_sm_count(), 128, 16384 + 32768 + 1024 + 1024, st>>>((const int32_t*)in, (uint32_t*)out);
    B200_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  if (which == 5) {
    probe_wait_expiry_kernel<<<1, 32, 0, st>>>((const int32_t*)in, (uint32_t*)out);
    B200_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  return set_error(-1, "debug_probe: unknown probe %d", which);
}

}  // namespace b200moe
