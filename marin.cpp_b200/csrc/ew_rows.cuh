// Row helpers shared by the RMSNorm and sandwich-tail kernels (bf16 storage): one warp owns a row, a lane owns the
// 16-byte pieces lane, lane + 32, ... of it.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nm::ew {

constexpr int kRowWarps = 8;      // warps per CTA in the row kernels
constexpr int kMaxPieces = 32;    // 16-byte pieces a lane may own: D <= 32 * 32 * 8 = 8192

__device__ __forceinline__ float rb(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    f[2 * e] = __uint_as_float(u[e] << 16);
    f[2 * e + 1] = __uint_as_float(u[e] & 0xffff0000u);
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  uint32_t u[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
    u[e] = *reinterpret_cast<const uint32_t*>(&v);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(u[0], u[1], u[2], u[3]);
}

// One element of a norm backward after the row sums (levanter rounding points when LEV):
//   a = round(g dy); gc = round(dy round(x r)); dx = a r + c2 x with c2 = 2 (s (-0.5 (r / (ms + eps)))) / n
template <bool LEV>
__device__ __forceinline__ float norm_a(float g, float dy) { return LEV ? rb(__fmul_rn(g, dy)) : g * dy; }
template <bool LEV>
__device__ __forceinline__ float norm_gc(float dy, float x, float r) {
  return LEV ? rb(__fmul_rn(dy, rb(__fmul_rn(x, r)))) : dy * (x * r);
}
__device__ __forceinline__ float norm_c2(float s, float r, float ms, float eps, int n) {
  return 2.f * __fdiv_rn(__fmul_rn(s, __fmul_rn(-0.5f, __fdiv_rn(r, ms + eps))), float(n));
}
template <bool LEV>
__device__ __forceinline__ float norm_dx(float a, float r, float c2, float x) {
  return LEV ? __fadd_rn(__fmul_rn(a, r), __fmul_rn(c2, x)) : fmaf(a, r, c2 * x);
}
// forward output element: levanter bf16(g bf16(x r)) (the caller rounds the product once more when storing)
template <bool LEV>
__device__ __forceinline__ float norm_y(float g, float x, float r) {
  return LEV ? __fmul_rn(g, rb(__fmul_rn(x, r))) : g * (x * r);
}

}  // namespace nm::ew
