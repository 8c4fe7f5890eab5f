// Device helpers shared by the grouped-GEMM kernels: activation with the oracle's roundings,
// descriptor halves, tcgen05 MMA / TMEM load-store wrappers, the epilogue warps' named barriers,
// shared-memory accessors and the block quantisers of the gate-up -> down hand-off.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "internal.h"
#include "ptx_sm100.cuh"

// Cycle counters of the GEMM roles exist only in a -DB200MOE_PROFILE build; the production kernels carry no
// timing code (the issuing threads are the ones whose instruction rate limits the main loop).
#ifdef B200MOE_PROFILE
#define PROF_DECL(name) long long name = 0
#define PROF_NOW() clock64()
#define PROF_ADD(acc, t0) acc += clock64() - (t0)
#else
#define PROF_DECL(name)
#define PROF_NOW() 0ll
#define PROF_ADD(acc, t0) ((void)(t0))
#endif

namespace b200moe {

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float gateup_act(float g, float u, int activation, float limit) {
  // the oracle's matmuls return bf16, and its activation rounds to bf16 after silu and after
  // the product (tests/contrib/moe/test_moe.py:73-83,100-106): reproduce those roundings
  g = bf16r(g);
  u = bf16r(u);
  if (activation == B200MOE_ACT_SILU) {
    float s = bf16r(g * __frcp_rn(1.f + __expf(-g)));
    return bf16r(s * u);
  }
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return bf16r(g * __frcp_rn(1.f + __expf(-1.702f * g)) * (u + 1.f));
}

// Two elements at once with packed bf16 conversions (half the conversion instructions); the same
// roundings as gateup_act, result already in bf16.
__device__ __forceinline__ float2 bf16r2(float a, float b) { return __bfloat1622float2(__floats2bfloat162_rn(a, b)); }
__device__ __forceinline__ __nv_bfloat162 gateup_act2(float g0, float u0, float g1, float u1, int activation,
                                                      float limit) {
  float2 g = bf16r2(g0, g1), u = bf16r2(u0, u1);
  if (activation == B200MOE_ACT_SILU) {
    const float2 s = bf16r2(g.x * __frcp_rn(1.f + __expf(-g.x)), g.y * __frcp_rn(1.f + __expf(-g.y)));
    return __floats2bfloat162_rn(s.x * u.x, s.y * u.y);
  }
  g.x = fminf(g.x, limit);
  g.y = fminf(g.y, limit);
  u.x = fminf(fmaxf(u.x, -limit), limit);
  u.y = fminf(fmaxf(u.y, -limit), limit);
  return __floats2bfloat162_rn(g.x * __frcp_rn(1.f + __expf(-1.702f * g.x)) * (u.x + 1.f),
                               g.y * __frcp_rn(1.f + __expf(-1.702f * g.y)) * (u.y + 1.f));
}

// (a0, a1) += s * (v0, v1) as one packed fp32x2 instruction (two FMAs per issue slot); v0/v1 are raw
// accumulator words as tcgen05.ld returns them
__device__ __forceinline__ void ffma2_scaled(float& a0, float& a1, float s, uint32_t v0, uint32_t v1) {
  asm("{\n\t.reg .b64 a, v, c;\n\t"
      "mov.b64 a, {%0, %1};\n\t"
      "mov.b64 v, {%2, %3};\n\t"
      "mov.b64 c, {%4, %4};\n\t"
      "fma.rn.f32x2 a, v, c, a;\n\t"
      "mov.b64 {%0, %1}, a;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "r"(v0), "r"(v1), "f"(s));
}

// (a0, a1) += (s0, s1) * (v0, v1): the same with one scale per element
__device__ __forceinline__ void ffma2_pair(float& a0, float& a1, float s0, float s1, uint32_t v0, uint32_t v1) {
  asm("{\n\t.reg .b64 a, v, c;\n\t"
      "mov.b64 a, {%0, %1};\n\t"
      "mov.b64 v, {%2, %3};\n\t"
      "mov.b64 c, {%4, %5};\n\t"
      "fma.rn.f32x2 a, v, c, a;\n\t"
      "mov.b64 {%0, %1}, a;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "r"(v0), "r"(v1), "f"(s0), "f"(s1));
}

// descriptor halves: the high word is constant per layout, the low word carries the address
constexpr uint32_t kDescHiSw = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, 128-byte swizzle
constexpr uint32_t kDescHiSf = (128u >> 4) | (1u << 14);                   // SBO 128, version 1, no swizzle
__device__ __forceinline__ uint32_t desc_lo_sw(uint32_t saddr) { return ((saddr >> 4) & 0x3FFFu) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_lo_sf(uint32_t saddr) { return (saddr >> 4) & 0x3FFFu; }

// D[tmem] (+)= A[smem] * B[smem]^T, packed FP4 x packed FP4, K = 64, two E8M0 scales per row
__device__ __forceinline__ void umma_mxf4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %7};\n\t"
      "mov.b64 db, {%2, %7};\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], da, db, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem),
        "r"(kDescHiSw)
      : "memory");
}
// the same across a CTA pair: M = 256 (128 rows from each CTA's shared memory), N/2 token rows from each CTA
__device__ __forceinline__ void umma_mxf4_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %7};\n\t"
      "mov.b64 db, {%2, %7};\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], da, db, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem),
        "r"(kDescHiSw)
      : "memory");
}
__device__ __forceinline__ void utccp_sf(uint32_t taddr, uint32_t lo) {
  asm volatile(
      "{\n\t.reg .b64 d;\n\t"
      "mov.b64 d, {%1, %2};\n\t"
      "tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n\t}"
      ::"r"(taddr), "r"(lo), "r"(kDescHiSf)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x4(uint32_t taddr, const uint4& v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint4& a, const uint4& b, const uint4& c,
                                                   const uint4& d) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w), "r"(c.x), "r"(c.y), "r"(c.z),
      "r"(c.w), "r"(d.x), "r"(d.y), "r"(d.z), "r"(d.w)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// named barriers among the eight epilogue warps (barrier 0 belongs to __syncthreads)
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }
__device__ __forceinline__ bool epi_all(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"((uint32_t)pred)
      : "memory");
  return out != 0;
}
__device__ __forceinline__ void st_shared_u16(uint32_t addr, unsigned short v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// quantise 32 floats to E2M1 with a shared E8M0 scale (same rule as the stand-alone quantiser):
// q gets 16 bytes (low nibble = even element); with RESIDUAL x is replaced by what the term left
// (the input of the next term; the last term of a row does not need it)
template <bool RESIDUAL = true>
__device__ __forceinline__ int quant_block32_fp4(float (&x)[32], uint4& q) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[i]));
  const int e = max((int)((__float_as_uint(amax) >> 23) & 0xFF) - 2, 0);
  const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
  const float sc = __uint_as_float(e == 0 ? 0x00400000u : ((uint32_t)e << 23));
  uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const __nv_fp4x2_storage_t pk =
        __nv_cvt_float2_to_fp4x2(make_float2(x[i] * inv, x[i + 1] * inv), __NV_E2M1, cudaRoundNearest);
    w[i >> 3] |= (uint32_t)pk << (((i >> 1) & 3) * 8);
    if (RESIDUAL) {
      __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(pk, __NV_E2M1);
      const float2 f = __half22float2(*reinterpret_cast<__half2*>(&h));
      x[i] -= f.x * sc;
      x[i + 1] -= f.y * sc;
    }
  }
  q = make_uint4(w[0], w[1], w[2], w[3]);
  return e;
}

// quantise 32 floats to e4m3 with a shared E8M0 scale: e = max(biased_exp(amax) - 7, 0) puts the
// block maximum in [128, 256) (never saturates); q gets 32 bytes, with RESIDUAL x is replaced by the residual
template <bool RESIDUAL = true>
__device__ __forceinline__ int quant_block32_e4m3(float (&x)[32], uint4& q0, uint4& q1) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[i]));
  const int e = max((int)((__float_as_uint(amax) >> 23) & 0xFF) - 7, 0);
  const float inv = __uint_as_float((uint32_t)(254 - e) << 23);
  const float sc = __uint_as_float(e == 0 ? 0x00400000u : ((uint32_t)e << 23));
  uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const __nv_fp8x2_storage_t pk =
        __nv_cvt_float2_to_fp8x2(make_float2(x[i] * inv, x[i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    w[i >> 2] |= (uint32_t)pk << ((i & 2) * 8);
    if (RESIDUAL) {
      __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(pk, __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<__half2*>(&h));
      x[i] -= f.x * sc;
      x[i + 1] -= f.y * sc;
    }
  }
  q0 = make_uint4(w[0], w[1], w[2], w[3]);
  q1 = make_uint4(w[4], w[5], w[6], w[7]);
  return e;
}

// D[tmem] (+)= A[smem] * B[smem]^T, e4m3 x e4m3 with E8M0 block scales, K = 32 per instruction
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %7};\n\t"
      "mov.b64 db, {%2, %7};\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem),
        "r"(kDescHiSw)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

}  // namespace b200moe
