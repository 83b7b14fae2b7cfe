// Row helpers shared by the RMSNorm and sandwich-tail kernels (bf16 storage). Forward kernels: one warp owns a row, a lane
// owns the 16-byte pieces lane, lane + 32, ... of it. Backward kernels: row groups fed by a ring of row batches in shared
// memory, packed bf16x2 / f32x2 arithmetic for the levanter rounding points (all further down).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

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
// row (G = 32, 64, 128 or 256), thread tg owning the 16-byte pieces tg, tg + G, ... (PP of them). A thread owns the same
// columns for every row, so its gain-gradient sums never leave its registers until the part is done.
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
// Host: PP of the backward kernels for a row of `pieces` pieces. Two pieces per thread wherever a row fills a warp
// that way: the work per row that does not depend on its length (sums, statistics, waits, index arithmetic) is then
// spread over 16 elements instead of 8, and it is that work, not HBM, which bounds these kernels at one piece per thread.
inline int pieces_per_thread_for(int pieces) { return pieces <= 32 ? 1 : pieces <= 2 * kGroupThreads ? 2 : 4; }
inline int group_threads_for(int pieces, int pp) {   // host: smallest G with G * pp >= pieces
  for (int g = 32; g < kGroupThreads; g *= 2)
    if (g * pp >= pieces) return g;
  return kGroupThreads;
}

// Sums K values over the G threads of a row; every thread of the group gets the same totals. Within a warp by an xor
// butterfly; across the warps of a group through shared memory and a named barrier of the group's own (ids 1 ..): lane 0
// of a warp writes its K sums as one vector, after the barrier lane l reads the vector of the group's warp l mod 8 (zeros
// past the group's last warp) and three more butterfly steps add them up. A butterfly adds the same pairs in every lane
// (operands swapped at most), so all lanes and all warps of the group hold identical bits.
// `buf` is [2][8 warps][K rounded up to 1, 2 or 4] floats, 16-byte aligned; `flip` alternates between its halves so that
// consecutive calls need one barrier each.
template <int K>
__device__ __forceinline__ void group_sum(float (&v)[K], const RowGroup& rg, float* buf, int& flip) {
  static_assert(K >= 1 && K <= 4, "group_sum: 1 to 4 values");
  constexpr int KP = K == 1 ? 1 : K == 2 ? 2 : 4;
#pragma unroll
  for (int k = 0; k < K; ++k) v[k] = warp_sum(v[k]);
  if (rg.G == 32) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* b = buf + flip * (8 * KP);
  flip ^= 1;
  if (lane == 0) {
    if constexpr (KP == 1) b[warp] = v[0];
    else if constexpr (KP == 2) *reinterpret_cast<float2*>(b + warp * 2) = make_float2(v[0], v[1]);
    else *reinterpret_cast<float4*>(b + warp * 4) = make_float4(v[0], v[1], v[2], K == 4 ? v[K - 1] : 0.f);
  }
  asm volatile("bar.sync %0, %1;" ::"r"(1 + rg.group), "r"(rg.G) : "memory");
  const int nw = rg.G >> 5, src = lane & 7;
  const float* mine = b + (rg.group * nw + src) * KP;
  if (src < nw) {
    if constexpr (KP == 1) v[0] = mine[0];
    else if constexpr (KP == 2) {
      const float2 t = *reinterpret_cast<const float2*>(mine);
      v[0] = t.x, v[1] = t.y;
    } else {
      const float4 t = *reinterpret_cast<const float4*>(mine);
      v[0] = t.x, v[1] = t.y, v[2] = t.z;
      if constexpr (K == 4) v[K - 1] = t.w;
    }
  } else {
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = 0.f;
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1)
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] += __shfl_xor_sync(0xffffffffu, v[k], o);
}

// x / n for the row length n, bit for bit: when n is a power of two the host passes inv_n = 1 / n and the product is the
// same correctly rounded value as the quotient (a scaling by a power of two); otherwise inv_n = 0 and the division runs.
__device__ __forceinline__ float div_n(float x, int n, float inv_n) {
  return inv_n != 0.f ? __fmul_rn(x, inv_n) : __fdiv_rn(x, float(n));
}
inline float inv_if_pow2(int n) { return (n > 0 && (n & (n - 1)) == 0) ? 1.0f / float(n) : 0.f; }
__device__ __forceinline__ float norm_c2(float s, float r, float ms, float eps, int n, float inv_n) {
  return 2.f * div_n(__fmul_rn(s, __fmul_rn(-0.5f, __fdiv_rn(r, ms + eps))), n, inv_n);
}

// Two f32 values in one 64-bit register for the packed f32x2 pipe: each instruction does two independent, individually
// rounded operations, so the results are the bits of the scalar __fmul_rn / __fadd_rn / fmaf forms.
struct F2 {
  uint64_t v;
};
__device__ __forceinline__ F2 f2(float lo, float hi) {
  F2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_get(F2 a, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a.v)); }
__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) {
  F2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
  return r;
}
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) {
  F2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
  return r;
}
// bf16x2(a r + c x) with three roundings per element before the bf16 one (two products, one sum). The sum is taken with
// scalar add.rn.f32: ptxas was seen to merge a mul.rn.f32x2 feeding an add.rn.f32x2 into one fma (a single rounding, which
// shows as a different bf16 result where the sum lands next to a tie), with or without --fmad=false; a scalar add with an
// explicit rounding mode is never contracted.
__device__ __forceinline__ uint32_t axpby_bf16x2(F2 a, F2 r, F2 c, F2 x);
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) {
  F2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v));
  return r;
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

// Packed bf16 arithmetic for the levanter rounding points. The product of two bf16 values is exact in f32, so
// bf16(f32(a) * f32(b)) is one rounding of the exact product: precisely what mul.rn.bf16x2 returns, for two elements per
// instruction instead of a multiply, a conversion and a widening shift for each.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// bf16(f32(a) + f32(b)) for two elements: the f32 sum of two bf16 values rounded again to bf16 equals the exact sum
// rounded once (24 bits are more than twice 8 plus 2, so the first rounding cannot move the second), which is what
// add.rn.bf16x2 returns.
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float lo_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f32(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ F2 f2_of(uint32_t two_bf16) { return f2(lo_f32(two_bf16), hi_f32(two_bf16)); }
__device__ __forceinline__ uint32_t bf16x2_of(F2 a) {   // both halves rounded to nearest even
  float lo, hi;
  f2_get(a, lo, hi);
  return pack_bf16x2(lo, hi);
}
__device__ __forceinline__ uint32_t axpby_bf16x2(F2 a, F2 r, F2 c, F2 x) {
  float p0, p1, q0, q1;
  f2_get(f2_mul(a, r), p0, p1);
  f2_get(f2_mul(c, x), q0, q1);
  return pack_bf16x2(__fadd_rn(p0, q0), __fadd_rn(p1, q1));
}
__device__ __forceinline__ uint32_t word_of(const uint4& q, int i) { return i == 0 ? q.x : i == 1 ? q.y : i == 2 ? q.z : q.w; }

// End of a part: the gain-gradient sums of the CTA's row groups are added in group order and written as row `part` of
// the partial buffer. dg is this thread's [PP][4] pairs (elements 2 q, 2 q + 1 of piece i); smem holds 256 x 4 floats
// (half a piece per round). With one row group per CTA every thread simply writes its own sums.
template <int PP>
__device__ __forceinline__ void write_gain_partial(const F2 (&dg)[PP][4], const RowGroup& rg, int pieces, float* smem,
                                                   float* out_row) {
#pragma unroll
  for (int i = 0; i < PP; ++i) {
    const int pc = rg.tg + i * rg.G;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float4 mine;
      f2_get(dg[i][2 * h], mine.x, mine.y);
      f2_get(dg[i][2 * h + 1], mine.z, mine.w);
      if (rg.groups == 1) {
        if (pc < pieces) reinterpret_cast<float4*>(out_row + pc * 8)[h] = mine;
        continue;
      }
      __syncthreads();
      *reinterpret_cast<float4*>(smem + threadIdx.x * 4) = mine;
      __syncthreads();
      if (rg.group == 0 && pc < pieces) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int g = 0; g < rg.groups; ++g) {
          const float4 v = *reinterpret_cast<const float4*>(smem + (g * rg.G + rg.tg) * 4);
          s.x = __fadd_rn(s.x, v.x), s.y = __fadd_rn(s.y, v.y), s.z = __fadd_rn(s.z, v.z), s.w = __fadd_rn(s.w, v.w);
        }
        reinterpret_cast<float4*>(out_row + pc * 8)[h] = s;
      }
    }
  }
  if (rg.groups != 1) __syncthreads();
}

// ------------------------------------------------------------------------------------------------ batch ring
// The norm kernels (forward and backward) walk the batches (256 / G consecutive rows) of their parts in order. Thread 0
// keeps the next `stages - 1` batches of every row operand on their way into a ring in shared memory, one bulk copy per
// operand and batch (the rows of a batch are contiguous in memory), so the HBM reads in flight are set by the depth of
// the ring and not by how many loads a thread can park in registers. A thread reads its pieces of the landed batch from
// the slot in every pass that needs them (nothing is held in registers across the row sums) and its warp gives the slot
// back when it has read it for the last time (one arrive per warp). Every wait is bounded (ptx.cuh mbar_wait): one that
// runs out sets the CTA's abort flag and a bit in the status word; the CTA then runs through its remaining batches
// without waiting (its outputs are garbage, flagged by the word) and leaves after a pause for the copies in flight.
struct BatchWalk {
  int64_t row, end;   // first row of the current batch; end of the current part
  int part;
  __device__ __forceinline__ void enter(int64_t T, int64_t parts) {
    if (part < parts) row = part * T / parts, end = (part + 1) * T / parts;
  }
  __device__ __forceinline__ void begin(int64_t T, int64_t parts) {
    part = blockIdx.x;
    enter(T, parts);
  }
  __device__ __forceinline__ bool done(int64_t parts) const { return part >= parts; }
  __device__ __forceinline__ bool last_of_part(int groups) const { return row + groups >= end; }
  __device__ __forceinline__ uint32_t rows(int groups) const {
    return uint32_t(end - row < groups ? end - row : int64_t(groups));
  }
  __device__ __forceinline__ void next(int groups, int64_t T, int64_t parts) {
    row += groups;
    if (row >= end) part += gridDim.x, enter(T, parts);
  }
};

struct RowRing {
  uint32_t data, full, empty;   // shared-memory addresses: slots [stages][nops][op_bytes], then 8-byte barriers
  uint32_t op_bytes;            // bytes of one operand's slot (a multiple of 128)
  int stages, nops;
  __device__ __forceinline__ uint32_t slot(int s, int op) const { return data + uint32_t(s * nops + op) * op_bytes; }
};
constexpr int kRingWarps = kGroupThreads / 32;

// Shared memory a ring needs (host and device agree through this one function).
inline __host__ __device__ uint32_t ring_bytes(int stages, int nops, uint32_t op_bytes) {
  return uint32_t(stages) * uint32_t(nops) * op_bytes + 16u * uint32_t(stages) + 128u;
}
// Host: the slot size of an operand and the number of stages that fit when `ctas` CTAs share an SM.
inline uint32_t ring_op_bytes(int groups, int D) { return (uint32_t(groups) * uint32_t(D) * 2u + 127u) & ~127u; }
inline int ring_stages_for(int ctas, int nops, uint32_t op_bytes, uint32_t static_bytes, int most = 4) {
  const int64_t budget = int64_t(227) * 1024 / ctas - 1024 - static_bytes - 16 * most - 128;
  const int64_t fit = budget / (int64_t(nops) * op_bytes);
  return int(fit < 2 ? 2 : fit > most ? most : fit);
}

}  // namespace nm::ew
