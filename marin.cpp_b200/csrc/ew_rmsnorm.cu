// RMSNorm forward and backward (+ residual add, + gain-gradient partials) in bf16 storage, for the readout head.
// Forward: one warp per row, a lane owning the 16-byte pieces lane, lane + 32, ... of it. Backward: row groups over a ring
// of row batches in shared memory (ew_rows.cuh), rows of D <= 8192.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "ce_internal.hpp"
#include "ew_api.hpp"
#include "ew_rows.cuh"

namespace nm::ew {
namespace {

// Forward: a CTA walks parts of consecutive rows in batches, row groups and batch ring as described in ew_rows.cuh. A
// thread reads its pieces of x from the landed batch for the sum of squares and again for the output.
template <bool LEV, int PP>
__global__ void __launch_bounds__(kGroupThreads, PP <= 2 ? 2 : 1) k_rmsnorm_fwd(const __nv_bfloat16* x,
                                                                               const __nv_bfloat16* __restrict__ gain,
                                                                               __nv_bfloat16* y, float* __restrict__ rstd,
                                                                               int64_t T, int D, float eps, int64_t parts,
                                                                               int G, int stages, uint32_t op_bytes,
                                                                               float inv_n, uint32_t* status) {
  using namespace nm::ptx;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  __shared__ __align__(16) float red[2 * 8];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const RowGroup rg = row_group(G);
  const int pieces = D / 8;
  RowRing ring;
  ring.data = (smem_u32(ring_raw) + 127u) & ~127u;
  ring.op_bytes = op_bytes, ring.stages = stages, ring.nops = 1;
  ring.full = ring.data + uint32_t(stages) * op_bytes;
  ring.empty = ring.full + 8u * stages;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(ring.full + 8u * s, 1), mbar_init(ring.empty + 8u * s, kRingWarps);
    abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  auto fetch = [&](int s, const BatchWalk& b) {   // thread 0: one batch into slot s
    const uint32_t bytes = b.rows(rg.groups) * uint32_t(D) * 2u;
    const uint32_t bar = ring.full + 8u * s;
    mbar_arrive_expect_tx(bar, bytes);
    bulk_load(ring.slot(s, 0), x + b.row * D, bytes, bar);
  };
  BatchWalk w, ahead;
  w.begin(T, parts);
  ahead = w;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages - 1 && !ahead.done(parts); ++s, ahead.next(rg.groups, T, parts)) fetch(s, ahead);
  }
  int flip = 0;
  uint4 gq[PP];
#pragma unroll
  for (int i = 0; i < PP; ++i) {
    const int pc = rg.tg + i * rg.G;
    gq[i] = (y && pc < pieces) ? ldg16(gain + pc * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  int s = 0;
  uint32_t phase = 0;
  for (; !w.done(parts); w.next(rg.groups, T, parts)) {
    const int64_t row = w.row + rg.group;
    const bool on = row < w.end;
    const int64_t off = row * D;
    mbar_wait<true>(ring.full + 8u * s, phase, abort_flag, status, kErrTransformWait);
    const uint32_t at0 = ring.slot(s, 0) + uint32_t(rg.group * D + rg.tg * 8) * 2u;
    auto piece = [&](int i) {
      const int pc = rg.tg + i * rg.G;
      return (on && pc < pieces) ? ld_shared_v4(at0 + uint32_t(i * rg.G) * 16u) : make_uint4(0u, 0u, 0u, 0u);
    };
    F2 sxx = f2(0.f, 0.f);   // even and odd elements summed apart, two per instruction (the squares are exact in f32)
#pragma unroll
    for (int i = 0; i < PP; ++i) {
      const uint4 xqi = piece(i);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const F2 xx = f2_of(word_of(xqi, q));
        sxx = f2_fma(xx, xx, sxx);
      }
    }
    float sums[1];
    {
      float lo, hi;
      f2_get(sxx, lo, hi);
      sums[0] = lo + hi;
    }
    group_sum<1>(sums, rg, red, flip);
    if (threadIdx.x == 0 && !ahead.done(parts)) {   // the slot of the batch before this one takes the batch stages - 1 ahead
      const int prev = s == 0 ? stages - 1 : s - 1;
      mbar_wait(ring.empty + 8u * prev, s == 0 ? phase ^ 1u : phase, abort_flag, status, kErrProducerWait);
      fetch(prev, ahead);
      ahead.next(rg.groups, T, parts);
    }
    if (on) {
      const float r = rsqrtf(div_n(sums[0], D, inv_n) + eps);
      if (rstd && rg.tg == 0) rstd[row] = r;
      if (y) {
        const F2 rr = f2(r, r);
#pragma unroll
        for (int i = 0; i < PP; ++i) {
          const int pc = rg.tg + i * rg.G;
          if (pc < pieces) {
            const uint4 xqi = piece(i);
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const F2 xr = f2_mul(f2_of(word_of(xqi, q)), rr);
              if constexpr (LEV) o[q] = mul_bf16x2(word_of(gq[i], q), bf16x2_of(xr));   // bf16(g bf16(x r))
              else o[q] = bf16x2_of(f2_mul(f2_of(word_of(gq[i], q)), xr));
            }
            *reinterpret_cast<uint4*>(y + off + pc * 8) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    }
    __syncwarp();   // the warp has read all it needs of the slot
    if ((threadIdx.x & 31) == 0) mbar_arrive(ring.empty + 8u * s);
    if (++s == stages) s = 0, phase ^= 1u;
  }
  if (threadIdx.x == 0 && *abort_flag) __nanosleep(200000);   // an expired wait: let copies in flight land first
}

// A CTA walks parts of consecutive rows (the partition of norm_partial_rows) in batches, row groups and batch ring as
// described in ew_rows.cuh: a thread takes its pieces of dy, x (and the residual gradient) from the landed batch into
// registers, the group reduces sum x^2 and sum x a, and the same registers feed the output pass. Gain-gradient sums stay
// in the owning thread's registers for the whole part.
template <bool LEV, int PP>
__global__ void __launch_bounds__(kGroupThreads, PP == 1 ? 4 : PP == 2 ? 2 : 1) k_rmsnorm_bwd_add(const __nv_bfloat16* dy,
                                                                const __nv_bfloat16* x,
                                                                const __nv_bfloat16* __restrict__ gain,
                                                                const float* __restrict__ rstd,
                                                                const __nv_bfloat16* dres, __nv_bfloat16* dx,
                                                                float* __restrict__ partial, int64_t T, int D,
                                                                float eps, int64_t parts, int G, int stages,
                                                                uint32_t op_bytes, float inv_n, uint32_t* status) {
  using namespace nm::ptx;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  __shared__ __align__(16) float red[2 * 8 * 2];
  __shared__ __align__(16) float gsm[kGroupThreads * 4];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const RowGroup rg = row_group(G);
  const int pieces = D / 8;
  RowRing ring;
  ring.data = (smem_u32(ring_raw) + 127u) & ~127u;
  ring.op_bytes = op_bytes, ring.stages = stages, ring.nops = dres ? 3 : 2;
  ring.full = ring.data + uint32_t(stages * ring.nops) * op_bytes;
  ring.empty = ring.full + 8u * stages;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(ring.full + 8u * s, 1), mbar_init(ring.empty + 8u * s, kRingWarps);
    abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  auto fetch = [&](int s, const BatchWalk& b) {   // thread 0: one batch of every operand into slot s
    const uint32_t bytes = b.rows(rg.groups) * uint32_t(D) * 2u;
    const uint32_t bar = ring.full + 8u * s;
    mbar_arrive_expect_tx(bar, bytes * ring.nops);
    bulk_load(ring.slot(s, 0), dy + b.row * D, bytes, bar);
    bulk_load(ring.slot(s, 1), x + b.row * D, bytes, bar);
    if (dres) bulk_load(ring.slot(s, 2), dres + b.row * D, bytes, bar);
  };
  BatchWalk w, ahead;
  w.begin(T, parts);
  ahead = w;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages - 1 && !ahead.done(parts); ++s, ahead.next(rg.groups, T, parts)) fetch(s, ahead);
  }
  int flip = 0;
  uint4 gq[PP];
#pragma unroll
  for (int i = 0; i < PP; ++i) {
    const int pc = rg.tg + i * rg.G;
    gq[i] = pc < pieces ? ldg16(gain + pc * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  F2 dg[PP][4];   // gain-gradient sums of this thread's columns, two per register pair
#pragma unroll
  for (int i = 0; i < PP; ++i)
#pragma unroll
    for (int q = 0; q < 4; ++q) dg[i][q] = f2(0.f, 0.f);
  // every group runs every batch (the group reduction is a barrier of the group only, but the slot hand-back counts all
  // warps and the gain reduction at the end of a part is a barrier of the CTA)
  int s = 0;
  uint32_t phase = 0;
  for (; !w.done(parts); w.next(rg.groups, T, parts)) {
    const int64_t row = w.row + rg.group;
    const bool on = row < w.end;
    const int64_t off = row * D;
    const float r_in = (on && rstd) ? __ldg(rstd + row) : 0.f;   // asked for before the wait: lands with the batch
    mbar_wait<true>(ring.full + 8u * s, phase, abort_flag, status, kErrTransformWait);
    // a thread's pieces of the landed batch are read from the slot where a pass needs them (0 past the row's end)
    const uint32_t at0 = ring.slot(s, 0) + uint32_t(rg.group * D + rg.tg * 8) * 2u;
    auto piece = [&](int op, int i) {
      const int pc = rg.tg + i * rg.G;
      return (on && pc < pieces) ? ld_shared_v4(at0 + uint32_t(op) * op_bytes + uint32_t(i * rg.G) * 16u)
                                 : make_uint4(0u, 0u, 0u, 0u);
    };
    float sums[2] = {0.f, 0.f};   // sum x^2, sum x a
    F2 sxx = f2(0.f, 0.f), sxa = sxx;   // levanter: even and odd elements summed apart, two per instruction
#pragma unroll
    for (int i = 0; i < PP; ++i) {
      const uint4 dqi = piece(0, i), xqi = piece(1, i);
      if constexpr (LEV) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const F2 xx = f2_of(word_of(xqi, q)), aa = f2_of(mul_bf16x2(word_of(gq[i], q), word_of(dqi, q)));
          sxx = f2_fma(xx, xx, sxx);
          sxa = f2_fma(xx, aa, sxa);
        }
      } else {
        float xf[8], dyf[8], g[8];
        unpack8(xqi, xf);
        unpack8(dqi, dyf);
        unpack8(gq[i], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          sums[0] = fmaf(xf[e], xf[e], sums[0]);
          sums[1] = fmaf(xf[e], norm_a<LEV>(g[e], dyf[e]), sums[1]);
        }
      }
    }
    if constexpr (LEV) {
      float lo, hi;
      f2_get(sxx, lo, hi);
      sums[0] = lo + hi;
      f2_get(sxa, lo, hi);
      sums[1] = lo + hi;
    }
    group_sum<2>(sums, rg, red, flip);
    if (threadIdx.x == 0 && !ahead.done(parts)) {   // the slot of the batch before this one takes the batch stages - 1 ahead
      const int prev = s == 0 ? stages - 1 : s - 1;
      // (the first time round that slot is fresh: a wait for parity 1 on a new barrier returns at once)
      mbar_wait(ring.empty + 8u * prev, s == 0 ? phase ^ 1u : phase, abort_flag, status, kErrProducerWait);
      fetch(prev, ahead);
      ahead.next(rg.groups, T, parts);
    }
    if (on) {
      const float ms = div_n(sums[0], D, inv_n);
      const float r = rstd ? r_in : rsqrtf(ms + eps);
      const float c2 = norm_c2(sums[1], r, ms, eps, D, inv_n);
      const F2 rr = f2(r, r), cc = f2(c2, c2);
#pragma unroll
      for (int i = 0; i < PP; ++i) {
        const int pc = rg.tg + i * rg.G;
        if (pc < pieces) {
          const uint4 dqi = piece(0, i), xqi = piece(1, i);
          if constexpr (LEV) {
            const uint4 rqi = dres ? piece(2, i) : make_uint4(0u, 0u, 0u, 0u);
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t dw = word_of(dqi, q);
              const F2 xx = f2_of(word_of(xqi, q)), aa = f2_of(mul_bf16x2(word_of(gq[i], q), dw));
              dg[i][q] = f2_add(dg[i][q], f2_of(mul_bf16x2(dw, bf16x2_of(f2_mul(xx, rr)))));
              o[q] = axpby_bf16x2(aa, rr, cc, xx);
              if (dres) o[q] = add_bf16x2(word_of(rqi, q), o[q]);
            }
            *reinterpret_cast<uint4*>(dx + off + pc * 8) = make_uint4(o[0], o[1], o[2], o[3]);
          } else {
            float xf[8], dyf[8], g[8], d[8], gc[8];
            unpack8(xqi, xf);
            unpack8(dqi, dyf);
            unpack8(gq[i], g);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              d[e] = norm_dx<LEV>(norm_a<LEV>(g[e], dyf[e]), r, c2, xf[e]);
              gc[e] = norm_gc<LEV>(dyf[e], xf[e], r);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) dg[i][q] = f2_add(dg[i][q], f2(gc[2 * q], gc[2 * q + 1]));
            if (dres) {
              float q[8];
              unpack8(piece(2, i), q);
#pragma unroll
              for (int e = 0; e < 8; ++e) d[e] = q[e] + d[e];
            }
            *reinterpret_cast<uint4*>(dx + off + pc * 8) = pack8(d);
          }
        }
      }
    }
    __syncwarp();   // the warp has read all it needs of the slot
    if ((threadIdx.x & 31) == 0) mbar_arrive(ring.empty + 8u * s);
    if (++s == stages) s = 0, phase ^= 1u;
    if (w.last_of_part(rg.groups)) {
      if (partial) write_gain_partial<PP>(dg, rg, pieces, gsm, partial + int64_t(w.part) * D);
#pragma unroll
      for (int i = 0; i < PP; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) dg[i][q] = f2(0.f, 0.f);
    }
  }
  if (threadIdx.x == 0 && *abort_flag) __nanosleep(200000);   // an expired wait: let copies in flight land first
}

}  // namespace

int64_t norm_partial_rows(int64_t T) {
  const int64_t by_rows = std::max<int64_t>(1, (T + 15) / 16);
  return std::min<int64_t>(std::min<int64_t>(1024, by_rows), int64_t(4) * ce::sm_count());
}

void rmsnorm_fwd(const bf16_t* x, const bf16_t* gain, bf16_t* y, float* rstd, int64_t T, int D, float eps,
                 cudaStream_t st, Rounding r) {
  NM_REQUIRE(x && gain && T >= 0 && D > 0 && D % 8 == 0, "rmsnorm_fwd: x, gain, D % 8 == 0");
  NM_REQUIRE(aligned16(x, gain, y), "rmsnorm_fwd: x, gain, y must be 16-byte aligned");
  NM_REQUIRE(D <= kGroupThreads * 4 * 8, "rmsnorm_fwd: D <= 8192");
  if (T == 0) return;
  const bool lev = r == Rounding::Levanter;
  const int pieces = D / 8;
  const int pp = pieces_per_thread_for(pieces);
  const int G = group_threads_for(pieces, pp);
  const int ctas = pp <= 2 ? 2 : 1;
  const int64_t parts = norm_partial_rows(T);   // any partition of the rows would do; this one divides evenly over the grid
  const uint32_t op_bytes = ring_op_bytes(kGroupThreads / G, D);
  const int stages = ring_stages_for(ctas, 1, op_bytes, 512, 6);
  const uint32_t smem = ring_bytes(stages, 1, op_bytes);
  auto kern = pp == 1   ? (lev ? k_rmsnorm_fwd<true, 1> : k_rmsnorm_fwd<false, 1>)
              : pp == 2 ? (lev ? k_rmsnorm_fwd<true, 2> : k_rmsnorm_fwd<false, 2>)
                        : (lev ? k_rmsnorm_fwd<true, 4> : k_rmsnorm_fwd<false, 4>);
  NM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  const int grid = int(std::min<int64_t>(parts, int64_t(ce::sm_count()) * ctas));
  kern<<<grid, kGroupThreads, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                          reinterpret_cast<const __nv_bfloat16*>(gain),
                                          reinterpret_cast<__nv_bfloat16*>(y), rstd, T, D, eps, parts, G, stages, op_bytes,
                                          inv_if_pow2(D), row_status_word());
  NM_CUDA(cudaGetLastError());
}

void rmsnorm_bwd_add(const bf16_t* dy, const bf16_t* x, const bf16_t* gain, const float* rstd, const bf16_t* dres,
                     bf16_t* dx, float* dgain_partial, int64_t T, int D, float eps, cudaStream_t st, Rounding r) {
  NM_REQUIRE(dy && x && gain && dx && T >= 0 && D > 0 && D % 8 == 0, "rmsnorm_bwd_add: dy, x, gain, dx, D % 8 == 0");
  NM_REQUIRE(aligned16(dy, x, gain, dres, dx, dgain_partial), "rmsnorm_bwd_add: every pointer must be 16-byte aligned");
  NM_REQUIRE(D <= kGroupThreads * 4 * 8, "rmsnorm_bwd_add: D <= 8192");
  if (T == 0) return;
  const int64_t parts = norm_partial_rows(T);
  const bool lev = r == Rounding::Levanter;
  const int pieces = D / 8;
  const int pp = pieces_per_thread_for(pieces);
  const int G = group_threads_for(pieces, pp);
  const int ctas = pp == 1 ? 4 : pp == 2 ? 2 : 1;   // CTAs per SM the ring is sized for
  const int nops = dres ? 3 : 2;
  const uint32_t op_bytes = ring_op_bytes(kGroupThreads / G, D);
  const int stages = ring_stages_for(ctas, nops, op_bytes, 4608);
  const uint32_t smem = ring_bytes(stages, nops, op_bytes);
  auto kern = pp == 1   ? (lev ? k_rmsnorm_bwd_add<true, 1> : k_rmsnorm_bwd_add<false, 1>)
              : pp == 2 ? (lev ? k_rmsnorm_bwd_add<true, 2> : k_rmsnorm_bwd_add<false, 2>)
                        : (lev ? k_rmsnorm_bwd_add<true, 4> : k_rmsnorm_bwd_add<false, 4>);
  NM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  const int grid = int(std::min<int64_t>(parts, int64_t(ce::sm_count()) * ctas));
  kern<<<grid, kGroupThreads, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(dy),
                                          reinterpret_cast<const __nv_bfloat16*>(x),
                                          reinterpret_cast<const __nv_bfloat16*>(gain), rstd,
                                          reinterpret_cast<const __nv_bfloat16*>(dres),
                                          reinterpret_cast<__nv_bfloat16*>(dx), dgain_partial, T, D, eps, parts, G, stages,
                                          op_bytes, inv_if_pow2(D), row_status_word());
  NM_CUDA(cudaGetLastError());
}

}  // namespace nm::ew
