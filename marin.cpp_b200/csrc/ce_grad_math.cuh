// The element arithmetic that turns stored logits into the normalised gradient n = a p - b onehot(target),
// p = exp(z_s - lse) = 2^(z_s log2e + e), e = -lse log2e (math of the reference's ce_dz, src/kernels/cross_entropy/
// ce_mma.cuh:81-91, with the common factor *grad_scale left to the dX / dW epilogues). One definition, used by the
// in-place pass and by the gradient kernels that form n in shared memory, so that every path yields the same bits:
// every product and difference is individually rounded, the exponential is ex2.approx.ftz.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ce_internal.hpp"
#include "ptx.cuh"

namespace nm::ce::gradmath {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float exponent_of(float lse) { return -lse * kLog2e; }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float lo_of(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi_of(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// a p for one stored logit
__device__ __forceinline__ float scaled_p(float zs, float e, float a) {
  return __fmul_rn(nm::ptx::ex2_approx(fmaf(zs, kLog2e, e)), a);
}

// Eight consecutive bf16 logits (one 16-byte piece) -> eight bf16 values of n.
//   hit     position 0..7 of the row's target inside this piece, anything else when it lies elsewhere
//   nvalid  how many of the eight columns exist (columns at or beyond the vocabulary size become 0)
__device__ __forceinline__ uint4 piece_bf16(uint4 raw, float e, float a, float b, int hit, int nvalid) {
  uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
  float d[8];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    d[2 * q] = scaled_p(lo_of(u[q]), e, a);
    d[2 * q + 1] = scaled_p(hi_of(u[q]), e, a);
  }
  if (static_cast<unsigned>(hit) < 8u) {       // rare: one piece per row holds the target
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (q == hit) d[q] = __fsub_rn(d[q], b);
  }
  if (nvalid < 8) {                            // rare: the ragged end of the vocabulary
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (q >= nvalid) d[q] = 0.f;
  }
  return make_uint4(pack_bf16x2(d[0], d[1]), pack_bf16x2(d[2], d[3]), pack_bf16x2(d[4], d[5]),
                    pack_bf16x2(d[6], d[7]));
}

// The same without a target and with all eight columns present: what nearly every piece of a store is.
__device__ __forceinline__ uint4 piece_bf16_plain(uint4 raw, float e, float a) {
  uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) u[q] = pack_bf16x2(scaled_p(lo_of(u[q]), e, a), scaled_p(hi_of(u[q]), e, a));
  return make_uint4(u[0], u[1], u[2], u[3]);
}

// Two logits at once on the packed f32x2 pipe (two independent, individually rounded operations per instruction: the
// same bits as the scalar form). ll, ee, aa hold (log2e, log2e), (e, e), (a, a).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint32_t scaled_p_pair(uint32_t two_bf16, uint64_t ll, uint64_t ee, uint64_t aa) {
  float x0, x1;
  asm("{\n\t"
      ".reg .b64 t;\n\t"
      "mov.b64 t, {%2, %3};\n\t"
      "fma.rn.f32x2 t, t, %4, %5;\n\t"
      "mov.b64 {%0, %1}, t;\n\t"
      "}"
      : "=f"(x0), "=f"(x1)
      : "f"(lo_of(two_bf16)), "f"(hi_of(two_bf16)), "l"(ll), "l"(ee));
  const float p0 = nm::ptx::ex2_approx(x0), p1 = nm::ptx::ex2_approx(x1);
  float d0, d1;
  asm("{\n\t"
      ".reg .b64 t;\n\t"
      "mov.b64 t, {%2, %3};\n\t"
      "mul.rn.f32x2 t, t, %4;\n\t"
      "mov.b64 {%0, %1}, t;\n\t"
      "}"
      : "=f"(d0), "=f"(d1)
      : "f"(p0), "f"(p1), "l"(aa));
  return pack_bf16x2(d0, d1);
}
__device__ __forceinline__ uint4 piece_bf16_plain2(uint4 raw, uint64_t ll, uint64_t ee, uint64_t aa) {
  return make_uint4(scaled_p_pair(raw.x, ll, ee, aa), scaled_p_pair(raw.y, ll, ee, aa), scaled_p_pair(raw.z, ll, ee, aa),
                    scaled_p_pair(raw.w, ll, ee, aa));
}

// The one element of a row that holds its target: bf16(a p - b), as a 16-bit pattern.
__device__ __forceinline__ uint16_t target_element(uint16_t raw, float e, float a, float b) {
  const float d = __fsub_rn(scaled_p(__uint_as_float(uint32_t(raw) << 16), e, a), b);
  return __bfloat16_as_ushort(__float2bfloat16_rn(d));
}

// Four consecutive f32 logits -> four bf16 values of n (the f32 store).
__device__ __forceinline__ uint2 piece_f32(float4 z, float e, float a, float b, int hit, int nvalid) {
  float d[4] = {scaled_p(z.x, e, a), scaled_p(z.y, e, a), scaled_p(z.z, e, a), scaled_p(z.w, e, a)};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    if (q == hit) d[q] = __fsub_rn(d[q], b);
    if (q >= nvalid) d[q] = 0.f;
  }
  return make_uint2(pack_bf16x2(d[0], d[1]), pack_bf16x2(d[2], d[3]));
}

}  // namespace nm::ce::gradmath
