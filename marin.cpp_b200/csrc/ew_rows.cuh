// Row helpers shared by the RMSNorm and sandwich-tail kernels (bf16 storage): one warp owns a row, a lane owns the
// 16-byte pieces lane, lane + 32, ... of it.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nm::ew {

constexpr int kRowWarps = 8;      // warps per CTA in the row kernels


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


// ------------------------------------------------------------------------------------------------ row groups
// Geometry of the backward kernels: a CTA of 256 threads works on 256 / G rows at a time, G threads side by side on a
// row (G = 32, 64, 128 or 256), thread tg owning the 16-byte pieces tg, tg + G, ... (PP of them). A thread therefore
// keeps a whole row's share in a few registers between the reduction and the output pass (no second load), and owns
// the same columns for every row, so its gain-gradient sums never leave its registers until the part is done.
constexpr int kGroupThreads = 256;
struct RowGroup {
  int G;        // threads per row
  int group;    // which row of the CTA's current batch
  int tg;       // thread within the row
  int groups;   // rows per batch = 256 / G
};
__device__ __forceinline__ RowGroup row_group(int G) {
  return RowGroup{G, int(threadIdx.x) / G, int(threadIdx.x) % G, kGroupThreads / G};
}
inline int group_threads_for(int pieces, int pp) {   // host: smallest G with G * pp >= pieces
  for (int g = 32; g < kGroupThreads; g *= 2)
    if (g * pp >= pieces) return g;
  return kGroupThreads;
}

// Sums K values over the G threads of a row; every thread of the group gets the totals. Within a warp by shuffles, across
// the warps of a group through shared memory and a named barrier of the group's own (ids 1 ..), added in warp order.
// `buf` is [2][8 warps][K] floats; `flip` alternates between its halves so that consecutive calls need one barrier each.
template <int K>
__device__ __forceinline__ void group_sum(float (&v)[K], const RowGroup& rg, float* buf, int& flip) {
#pragma unroll
  for (int k = 0; k < K; ++k) v[k] = warp_sum(v[k]);
  if (rg.G == 32) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* b = buf + flip * (8 * K);
  flip ^= 1;
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < K; ++k) b[warp * K + k] = v[k];
  }
  asm volatile("bar.sync %0, %1;" ::"r"(1 + rg.group), "r"(rg.G) : "memory");
  const int w0 = rg.group * (rg.G / 32), nw = rg.G / 32;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    float s = 0.f;
    for (int w = 0; w < nw; ++w) s += b[(w0 + w) * K + k];
    v[k] = s;
  }
}

__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    f[2 * e] = __uint_as_float(u[e] << 16);
    f[2 * e + 1] = __uint_as_float(u[e] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint32_t u[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
    u[e] = *reinterpret_cast<const uint32_t*>(&v);
  }
  return make_uint4(u[0], u[1], u[2], u[3]);
}
__device__ __forceinline__ uint4 ldg16(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }

// End of a part: the gain-gradient sums of the CTA's row groups are added in group order and written as row `part` of
// the partial buffer. dg is this thread's [PP][8]; smem holds 256 x 8 floats.
template <int PP>
__device__ __forceinline__ void write_gain_partial(const float (&dg)[PP][8], const RowGroup& rg, int pieces, float* smem,
                                                   float* out_row) {
#pragma unroll
  for (int i = 0; i < PP; ++i) {
    const int pc = rg.tg + i * rg.G;
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; ++e) smem[threadIdx.x * 8 + e] = dg[i][e];
    __syncthreads();
    if (rg.group == 0 && pc < pieces) {
      float s[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] = 0.f;
      for (int g = 0; g < rg.groups; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) s[e] = __fadd_rn(s[e], smem[(g * rg.G + rg.tg) * 8 + e]);
      float4* o = reinterpret_cast<float4*>(out_row + pc * 8);
      o[0] = make_float4(s[0], s[1], s[2], s[3]);
      o[1] = make_float4(s[4], s[5], s[6], s[7]);
    }
  }
  __syncthreads();
}

}  // namespace nm::ew
