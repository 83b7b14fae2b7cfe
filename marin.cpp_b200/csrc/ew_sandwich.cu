// The sandwich tail around a residual add, forward and backward, in bf16 storage: optional post-norm of the branch
// output, residual add, and the next pre-norm (for the last layer: the final norm whose output feeds the LM head and
// whose input gradient is what the fused CE's dX flows into). Semantics follow the reference's
// src/kernels/elementwise/rmsnorm_kernels.cuh:100-235 (k_sandwich_fwd / k_sandwich_bwd):
//   forward   y = g_post ? norm(branch; g_post) : branch;  x_out = bf16(x_in + y);  a_next = norm(x_out; g_next)
//   backward  dx_mid = dx_out + norm_next_bwd(da_next);  dx_in = dx_mid;  dbranch = g_post ? norm_post_bwd(dx_mid) : dx_mid
// with the levanter rounding points of ew_api.hpp (or f32 chains under accurate rounding). Forward: one warp per row;
// backward: the row-group geometry of ew_rows.cuh.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "ce_internal.hpp"
#include "ew_api.hpp"
#include "ew_rows.cuh"

namespace nm::ew {
namespace {

// Forward: a CTA walks parts of consecutive rows in batches, row groups and batch ring as described in ew_rows.cuh. A
// thread reads its pieces of the branch output and of x_in from the landed batch; x_out stays in its registers (as
// stored, rounded) between the second row sum and the next norm's output.
template <bool LEV, int PP>
__global__ void __launch_bounds__(kGroupThreads, PP <= 2 ? 2 : 1) k_sandwich_fwd(const __nv_bfloat16* branch,
                                                                                const __nv_bfloat16* x_in,
                                                                                const __nv_bfloat16* __restrict__ g_post,
                                                                                const __nv_bfloat16* __restrict__ g_next,
                                                                                __nv_bfloat16* x_out, __nv_bfloat16* a_next,
                                                                                float* __restrict__ rstd_post,
                                                                                float* __restrict__ rstd_next, int64_t T,
                                                                                int D, float eps, int64_t parts, int G,
                                                                                int stages, uint32_t op_bytes, float inv_n,
                                                                                uint32_t* status) {
  using namespace nm::ptx;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  __shared__ __align__(16) float red[2 * 8];
  __shared__ __align__(16) float red1[2 * 8];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const RowGroup rg = row_group(G);
  const int pieces = D / 8;
  const bool post = g_post != nullptr;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  RowRing ring;
  ring.data = (smem_u32(ring_raw) + 127u) & ~127u;
  ring.op_bytes = op_bytes, ring.stages = stages, ring.nops = 2;
  ring.full = ring.data + uint32_t(stages * 2) * op_bytes;
  ring.empty = ring.full + 8u * stages;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(ring.full + 8u * s, 1), mbar_init(ring.empty + 8u * s, kRingWarps);
    abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  auto fetch = [&](int s, const BatchWalk& b) {   // thread 0: one batch of both operands into slot s
    const uint32_t bytes = b.rows(rg.groups) * uint32_t(D) * 2u;
    const uint32_t bar = ring.full + 8u * s;
    mbar_arrive_expect_tx(bar, bytes * 2u);
    bulk_load(ring.slot(s, 0), branch + b.row * D, bytes, bar);
    bulk_load(ring.slot(s, 1), x_in + b.row * D, bytes, bar);
  };
  BatchWalk w, ahead;
  w.begin(T, parts);
  ahead = w;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages - 1 && !ahead.done(parts); ++s, ahead.next(rg.groups, T, parts)) fetch(s, ahead);
  }
  int flip = 0, flip1 = 0;
  uint4 gnq[PP], gpq[PP];
#pragma unroll
  for (int i = 0; i < PP; ++i) {
    const int pc = rg.tg + i * rg.G;
    gnq[i] = (a_next && pc < pieces) ? ldg16(g_next + pc * 8) : zero4;
    gpq[i] = (post && pc < pieces) ? ldg16(g_post + pc * 8) : zero4;
  }
  int s = 0;
  uint32_t phase = 0;
  for (; !w.done(parts); w.next(rg.groups, T, parts)) {
    const int64_t row = w.row + rg.group;
    const bool on = row < w.end;
    const int64_t off = row * D;
    mbar_wait<true>(ring.full + 8u * s, phase, abort_flag, status, kErrTransformWait);
    const uint32_t at0 = ring.slot(s, 0) + uint32_t(rg.group * D + rg.tg * 8) * 2u;
    auto piece = [&](int op, int i) {
      const int pc = rg.tg + i * rg.G;
      return (on && pc < pieces) ? ld_shared_v4(at0 + uint32_t(op) * op_bytes + uint32_t(i * rg.G) * 16u) : zero4;
    };
    F2 rrp = f2(0.f, 0.f);
    if (post) {   // uniform over the CTA
      F2 sbb = f2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < PP; ++i) {
        const uint4 bqi = piece(0, i);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const F2 bb = f2_of(word_of(bqi, q));
          sbb = f2_fma(bb, bb, sbb);
        }
      }
      float sums[1];
      {
        float lo, hi;
        f2_get(sbb, lo, hi);
        sums[0] = lo + hi;
      }
      group_sum<1>(sums, rg, red, flip);
      const float r_p = rsqrtf(div_n(sums[0], D, inv_n) + eps);
      if (on && rstd_post && rg.tg == 0) rstd_post[row] = r_p;
      rrp = f2(r_p, r_p);
    }
    // x_out = round(x_in + y); its sum of squares is taken over the rounded values
    uint32_t xo[PP][4];
    F2 sxx = f2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < PP; ++i) {
      const int pc = rg.tg + i * rg.G;
      const uint4 bqi = piece(0, i), xqi = piece(1, i);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t bw = word_of(bqi, q), xw = word_of(xqi, q);
        if (post) {
          const F2 br = f2_mul(f2_of(bw), rrp);
          if constexpr (LEV) xo[i][q] = add_bf16x2(xw, mul_bf16x2(word_of(gpq[i], q), bf16x2_of(br)));
          else xo[i][q] = bf16x2_of(f2_add(f2_of(xw), f2_mul(f2_of(word_of(gpq[i], q)), br)));
        } else {
          xo[i][q] = add_bf16x2(xw, bw);
        }
        const F2 xx = f2_of(xo[i][q]);
        sxx = f2_fma(xx, xx, sxx);
      }
      if (on && pc < pieces)
        *reinterpret_cast<uint4*>(x_out + off + pc * 8) = make_uint4(xo[i][0], xo[i][1], xo[i][2], xo[i][3]);
    }
    float sx[1];
    {
      float lo, hi;
      f2_get(sxx, lo, hi);
      sx[0] = lo + hi;
    }
    group_sum<1>(sx, rg, red1, flip1);
    if (threadIdx.x == 0 && !ahead.done(parts)) {   // the slot of the batch before this one takes the batch stages - 1 ahead
      const int prev = s == 0 ? stages - 1 : s - 1;
      mbar_wait(ring.empty + 8u * prev, s == 0 ? phase ^ 1u : phase, abort_flag, status, kErrProducerWait);
      fetch(prev, ahead);
      ahead.next(rg.groups, T, parts);
    }
    // the slot is not read again: hand it back before the output pass
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(ring.empty + 8u * s);
    if (++s == stages) s = 0, phase ^= 1u;
    if (on) {
      const float r_n = rsqrtf(div_n(sx[0], D, inv_n) + eps);
      if (rstd_next && rg.tg == 0) rstd_next[row] = r_n;
      if (a_next) {
        const F2 rrn = f2(r_n, r_n);
#pragma unroll
        for (int i = 0; i < PP; ++i) {
          const int pc = rg.tg + i * rg.G;
          if (pc < pieces) {
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const F2 xr = f2_mul(f2_of(xo[i][q]), rrn);
              if constexpr (LEV) o[q] = mul_bf16x2(word_of(gnq[i], q), bf16x2_of(xr));
              else o[q] = bf16x2_of(f2_mul(f2_of(word_of(gnq[i], q)), xr));
            }
            *reinterpret_cast<uint4*>(a_next + off + pc * 8) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    }
  }
  if (threadIdx.x == 0 && *abort_flag) __nanosleep(200000);   // an expired wait: let copies in flight land first
}

// A CTA walks parts of consecutive rows (the partition of norm_partial_rows) in batches, row groups and batch ring as
// described in ew_rows.cuh. A thread takes its pieces of x_out, da_next, dx_out and branch from the landed batch into
// registers; the group reduces sum x_out^2, sum x_out a and sum branch^2 together, the middle gradient dx_mid is formed
// and stored, the group reduces sum branch a_post, and the branch gradient follows from the registers that are still
// there. Gain-gradient sums of both norms stay in the owning thread's registers for the whole part.
template <bool LEV, int PP>
__global__ void __launch_bounds__(kGroupThreads, PP == 1 ? 4 : PP == 2 ? 2 : 1) k_sandwich_bwd(const __nv_bfloat16* dx_out,
                                                             const __nv_bfloat16* da_next,
                                                             const __nv_bfloat16* x_out,
                                                             const __nv_bfloat16* __restrict__ g_next,
                                                             const float* __restrict__ rstd_next,
                                                             const __nv_bfloat16* branch,
                                                             const __nv_bfloat16* __restrict__ g_post,
                                                             const float* __restrict__ rstd_post,
                                                             __nv_bfloat16* dx_in, __nv_bfloat16* dbranch,
                                                             float* __restrict__ pg_next,
                                                             float* __restrict__ pg_post, int64_t T, int D,
                                                             float eps, int64_t parts, int G, int stages,
                                                             uint32_t op_bytes, float inv_n, uint32_t* status) {
  using namespace nm::ptx;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  __shared__ __align__(16) float red[2 * 8 * 4];    // the three-value reduction of every row (vectors of 4)
  __shared__ __align__(16) float red1[2 * 8 * 1];   // the one-value reduction that follows it: buffers of its own, flips of its own
  __shared__ __align__(16) float gsm[kGroupThreads * 4];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const RowGroup rg = row_group(G);
  const int pieces = D / 8;
  const bool post = g_post != nullptr;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  RowRing ring;
  ring.data = (smem_u32(ring_raw) + 127u) & ~127u;
  ring.op_bytes = op_bytes, ring.stages = stages, ring.nops = post ? 4 : 3;
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
    bulk_load(ring.slot(s, 0), x_out + b.row * D, bytes, bar);
    bulk_load(ring.slot(s, 1), da_next + b.row * D, bytes, bar);
    bulk_load(ring.slot(s, 2), dx_out + b.row * D, bytes, bar);
    if (post) bulk_load(ring.slot(s, 3), branch + b.row * D, bytes, bar);
  };
  BatchWalk w, ahead;
  w.begin(T, parts);
  ahead = w;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages - 1 && !ahead.done(parts); ++s, ahead.next(rg.groups, T, parts)) fetch(s, ahead);
  }
  int flip = 0, flip1 = 0;
  uint4 gnq[PP], gpq[PP];
#pragma unroll
  for (int i = 0; i < PP; ++i) {
    const int pc = rg.tg + i * rg.G;
    gnq[i] = pc < pieces ? ldg16(g_next + pc * 8) : zero4;
    gpq[i] = (post && pc < pieces) ? ldg16(g_post + pc * 8) : zero4;
  }
  F2 dgn[PP][4], dgp[PP][4];   // gain-gradient sums of this thread's columns, two per register pair
#pragma unroll
  for (int i = 0; i < PP; ++i)
#pragma unroll
    for (int q = 0; q < 4; ++q) dgn[i][q] = dgp[i][q] = f2(0.f, 0.f);
  int s = 0;
  uint32_t phase = 0;
  for (; !w.done(parts); w.next(rg.groups, T, parts)) {
    const int64_t row = w.row + rg.group;
    const bool on = row < w.end;
    const int64_t off = row * D;
    // the saved statistics are asked for before the wait, so that they land with the batch
    const float rn_in = (on && rstd_next) ? __ldg(rstd_next + row) : 0.f;
    const float rp_in = (on && post && rstd_post) ? __ldg(rstd_post + row) : 0.f;
    mbar_wait<true>(ring.full + 8u * s, phase, abort_flag, status, kErrTransformWait);
    // a thread's pieces of the landed batch are read from the slot where a pass needs them (0 past the row's end);
    // operands in slot order: x_out, da_next, dx_out, branch
    const uint32_t at0 = ring.slot(s, 0) + uint32_t(rg.group * D + rg.tg * 8) * 2u;
    auto piece = [&](int op, int i) {
      const int pc = rg.tg + i * rg.G;
      return (on && pc < pieces) ? ld_shared_v4(at0 + uint32_t(op) * op_bytes + uint32_t(i * rg.G) * 16u) : zero4;
    };
    float sums[3] = {0.f, 0.f, 0.f};   // sum x_out^2, sum x_out a_next, sum branch^2
    F2 sxx = f2(0.f, 0.f), sxa = sxx, sbb = sxx;   // levanter: even and odd elements summed apart, two per instruction
#pragma unroll
    for (int i = 0; i < PP; ++i) {
      const uint4 xqi = piece(0, i), aqi = piece(1, i), bqi = post ? piece(3, i) : zero4;
      if constexpr (LEV) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const F2 xx = f2_of(word_of(xqi, q)), bb = f2_of(word_of(bqi, q));
          const F2 aa = f2_of(mul_bf16x2(word_of(gnq[i], q), word_of(aqi, q)));
          sxx = f2_fma(xx, xx, sxx);
          sxa = f2_fma(xx, aa, sxa);
          sbb = f2_fma(bb, bb, sbb);
        }
      } else {
        float xo[8], da[8], g[8], b[8];
        unpack8(xqi, xo);
        unpack8(aqi, da);
        unpack8(gnq[i], g);
        unpack8(bqi, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          sums[0] = fmaf(xo[e], xo[e], sums[0]);
          sums[1] = fmaf(xo[e], norm_a<LEV>(g[e], da[e]), sums[1]);
          sums[2] = fmaf(b[e], b[e], sums[2]);
        }
      }
    }
    if constexpr (LEV) {
      float lo, hi;
      f2_get(sxx, lo, hi);
      sums[0] = lo + hi;
      f2_get(sxa, lo, hi);
      sums[1] = lo + hi;
      f2_get(sbb, lo, hi);
      sums[2] = lo + hi;
    }
    group_sum<3>(sums, rg, red, flip);
    if (threadIdx.x == 0 && !ahead.done(parts)) {   // the slot of the batch before this one takes the batch stages - 1 ahead
      const int prev = s == 0 ? stages - 1 : s - 1;
      // (the first time round that slot is fresh: a wait for parity 1 on a new barrier returns at once)
      mbar_wait(ring.empty + 8u * prev, s == 0 ? phase ^ 1u : phase, abort_flag, status, kErrProducerWait);
      fetch(prev, ahead);
      ahead.next(rg.groups, T, parts);
    }
    float r_n = 0.f, c2n = 0.f;
    if (on) {
      const float ms_n = div_n(sums[0], D, inv_n);
      r_n = rstd_next ? rn_in : rsqrtf(ms_n + eps);
      c2n = norm_c2(sums[1], r_n, ms_n, eps, D, inv_n);
    }
    const F2 rrn = f2(r_n, r_n), ccn = f2(c2n, c2n);
    // the middle gradient: stored as dx_in, kept (rounded to bf16, as stored) for the post-norm backward
    uint4 mq[PP];
    float bap[1] = {0.f};
    F2 sba = f2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < PP; ++i) {
      const int pc = rg.tg + i * rg.G;
      mq[i] = zero4;
      if (on && pc < pieces) {
        const uint4 xqi = piece(0, i), aqi = piece(1, i), oqi = piece(2, i);
        if constexpr (LEV) {
          uint32_t m[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t dw = word_of(aqi, q);
            const F2 xx = f2_of(word_of(xqi, q)), aa = f2_of(mul_bf16x2(word_of(gnq[i], q), dw));
            dgn[i][q] = f2_add(dgn[i][q], f2_of(mul_bf16x2(dw, bf16x2_of(f2_mul(xx, rrn)))));
            const uint32_t nw = axpby_bf16x2(aa, rrn, ccn, xx);
            m[q] = add_bf16x2(word_of(oqi, q), nw);
          }
          mq[i] = make_uint4(m[0], m[1], m[2], m[3]);
        } else {
          float xo[8], da[8], g[8], dxo[8], dxm[8], gc[8];
          unpack8(xqi, xo);
          unpack8(aqi, da);
          unpack8(gnq[i], g);
          unpack8(oqi, dxo);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float a = norm_a<LEV>(g[e], da[e]);
            const float dxn = norm_dx<LEV>(a, r_n, c2n, xo[e]);
            gc[e] = norm_gc<LEV>(da[e], xo[e], r_n);
            dxm[e] = dxo[e] + dxn;
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) dgn[i][q] = f2_add(dgn[i][q], f2(gc[2 * q], gc[2 * q + 1]));
          mq[i] = pack8(dxm);
        }
        *reinterpret_cast<uint4*>(dx_in + off + pc * 8) = mq[i];
        if (post) {
          const uint4 bqi = piece(3, i);
          if constexpr (LEV) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              sba = f2_fma(f2_of(word_of(bqi, q)), f2_of(mul_bf16x2(word_of(gpq[i], q), word_of(mq[i], q))), sba);
          } else {
            float b[8], gp[8], m[8];
            unpack8(bqi, b);
            unpack8(gpq[i], gp);
            unpack8(mq[i], m);
#pragma unroll
            for (int e = 0; e < 8; ++e) bap[0] = fmaf(b[e], gp[e] * m[e], bap[0]);
          }
        } else if (dbranch != dx_in) {
          *reinterpret_cast<uint4*>(dbranch + off + pc * 8) = mq[i];
        }
      }
    }
    if (post) {   // uniform over the CTA
      if constexpr (LEV) {
        float lo, hi;
        f2_get(sba, lo, hi);
        bap[0] = lo + hi;
      }
      group_sum<1>(bap, rg, red1, flip1);
      if (on) {
        const float ms_p = div_n(sums[2], D, inv_n);
        const float r_p = rstd_post ? rp_in : rsqrtf(ms_p + eps);
        const float c2p = norm_c2(bap[0], r_p, ms_p, eps, D, inv_n);
        const F2 rrp = f2(r_p, r_p), ccp = f2(c2p, c2p);
#pragma unroll
        for (int i = 0; i < PP; ++i) {
          const int pc = rg.tg + i * rg.G;
          if (pc < pieces) {
            const uint4 bqi = piece(3, i);
            if constexpr (LEV) {
              uint32_t o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint32_t mw = word_of(mq[i], q);
                const F2 bb = f2_of(word_of(bqi, q)), ap = f2_of(mul_bf16x2(word_of(gpq[i], q), mw));
                dgp[i][q] = f2_add(dgp[i][q], f2_of(mul_bf16x2(mw, bf16x2_of(f2_mul(bb, rrp)))));
                o[q] = axpby_bf16x2(ap, rrp, ccp, bb);
              }
              *reinterpret_cast<uint4*>(dbranch + off + pc * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            } else {
              float b[8], gp[8], dxm[8], db[8], gc[8];
              unpack8(bqi, b);
              unpack8(gpq[i], gp);
              unpack8(mq[i], dxm);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float ap = norm_a<LEV>(gp[e], dxm[e]);
                db[e] = norm_dx<LEV>(ap, r_p, c2p, b[e]);
                gc[e] = norm_gc<LEV>(dxm[e], b[e], r_p);
              }
#pragma unroll
              for (int q = 0; q < 4; ++q) dgp[i][q] = f2_add(dgp[i][q], f2(gc[2 * q], gc[2 * q + 1]));
              *reinterpret_cast<uint4*>(dbranch + off + pc * 8) = pack8(db);
            }
          }
        }
      }
    }
    __syncwarp();   // the warp has read all it needs of the slot
    if ((threadIdx.x & 31) == 0) mbar_arrive(ring.empty + 8u * s);
    if (++s == stages) s = 0, phase ^= 1u;
    if (w.last_of_part(rg.groups)) {
      if (pg_next) write_gain_partial<PP>(dgn, rg, pieces, gsm, pg_next + int64_t(w.part) * D);
      if (pg_post && post) write_gain_partial<PP>(dgp, rg, pieces, gsm, pg_post + int64_t(w.part) * D);
#pragma unroll
      for (int i = 0; i < PP; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) dgn[i][q] = dgp[i][q] = f2(0.f, 0.f);
    }
  }
  if (threadIdx.x == 0 && *abort_flag) __nanosleep(200000);   // an expired wait: let copies in flight land first
}

}  // namespace

void sandwich_tail_fwd(const bf16_t* branch, const bf16_t* x_in, const bf16_t* g_post, const bf16_t* g_next,
                       bf16_t* x_out, bf16_t* a_next, float* rstd_post, float* rstd_next, int64_t T, int D, float eps,
                       cudaStream_t st, Rounding r) {
  NM_REQUIRE(branch && x_in && g_next && x_out && T >= 0 && D > 0 && D % 8 == 0,
             "sandwich_tail_fwd: branch, x_in, g_next, x_out required; D % 8 == 0");
  NM_REQUIRE(aligned16(branch, x_in, g_post, g_next, x_out, a_next), "sandwich_tail_fwd: every row pointer must be "
                                                                     "16-byte aligned");
  NM_REQUIRE(D <= kGroupThreads * 4 * 8, "sandwich_tail_fwd: D <= 8192");
  if (T == 0) return;
  const bool lev = r == Rounding::Levanter;
  const int pieces = D / 8;
  const int pp = pieces_per_thread_for(pieces);
  const int G = group_threads_for(pieces, pp);
  const int ctas = pp <= 2 ? 2 : 1;
  const int64_t parts = norm_partial_rows(T);   // any partition of the rows would do; this one divides evenly over the grid
  const uint32_t op_bytes = ring_op_bytes(kGroupThreads / G, D);
  const int stages = ring_stages_for(ctas, 2, op_bytes, 512, 6);
  const uint32_t smem = ring_bytes(stages, 2, op_bytes);
  auto kern = pp == 1   ? (lev ? k_sandwich_fwd<true, 1> : k_sandwich_fwd<false, 1>)
              : pp == 2 ? (lev ? k_sandwich_fwd<true, 2> : k_sandwich_fwd<false, 2>)
                        : (lev ? k_sandwich_fwd<true, 4> : k_sandwich_fwd<false, 4>);
  auto B = [](const bf16_t* p) { return reinterpret_cast<const __nv_bfloat16*>(p); };
  auto M = [](bf16_t* p) { return reinterpret_cast<__nv_bfloat16*>(p); };
  NM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  const int grid = int(std::min<int64_t>(parts, int64_t(ce::sm_count()) * ctas));
  kern<<<grid, kGroupThreads, smem, st>>>(B(branch), B(x_in), B(g_post), B(g_next), M(x_out), M(a_next), rstd_post,
                                          rstd_next, T, D, eps, parts, G, stages, op_bytes, inv_if_pow2(D),
                                          row_status_word());
  NM_CUDA(cudaGetLastError());
}

void sandwich_tail_bwd(const bf16_t* dx_out, const bf16_t* da_next, const bf16_t* x_out, const bf16_t* g_next,
                       const float* rstd_next, const bf16_t* branch, const bf16_t* g_post, const float* rstd_post,
                       bf16_t* dx_in, bf16_t* dbranch, float* pg_next, float* pg_post, int64_t T, int D, float eps,
                       cudaStream_t st, Rounding r) {
  NM_REQUIRE(dx_out && da_next && x_out && g_next && dx_in && dbranch && T >= 0 && D > 0 && D % 8 == 0,
             "sandwich_tail_bwd: dx_out, da_next, x_out, g_next, dx_in, dbranch required; D % 8 == 0");
  NM_REQUIRE(aligned16(dx_out, da_next, x_out, g_next, branch, g_post, dx_in, dbranch, pg_next, pg_post),
             "sandwich_tail_bwd: every row pointer must be 16-byte aligned");
  NM_REQUIRE(!g_post || branch, "sandwich_tail_bwd: a post-norm needs the branch output");
  NM_REQUIRE(D <= kGroupThreads * 4 * 8, "sandwich_tail_bwd: D <= 8192");
  if (T == 0) return;
  const int64_t parts = norm_partial_rows(T);
  const bool lev = r == Rounding::Levanter;
  const int pieces = D / 8;
  const int pp = pieces_per_thread_for(pieces);
  const int G = group_threads_for(pieces, pp);
  const int ctas = pp == 1 ? 4 : pp == 2 ? 2 : 1;   // CTAs per SM the ring is sized for
  const int nops = g_post ? 4 : 3;
  const uint32_t op_bytes = ring_op_bytes(kGroupThreads / G, D);
  const int stages = ring_stages_for(ctas, nops, op_bytes, 4608);
  const uint32_t smem = ring_bytes(stages, nops, op_bytes);
  auto kern = pp == 1   ? (lev ? k_sandwich_bwd<true, 1> : k_sandwich_bwd<false, 1>)
              : pp == 2 ? (lev ? k_sandwich_bwd<true, 2> : k_sandwich_bwd<false, 2>)
                        : (lev ? k_sandwich_bwd<true, 4> : k_sandwich_bwd<false, 4>);
  auto B = [](const bf16_t* p) { return reinterpret_cast<const __nv_bfloat16*>(p); };
  auto M = [](bf16_t* p) { return reinterpret_cast<__nv_bfloat16*>(p); };
  NM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  const int grid = int(std::min<int64_t>(parts, int64_t(ce::sm_count()) * ctas));
  kern<<<grid, kGroupThreads, smem, st>>>(B(dx_out), B(da_next), B(x_out), B(g_next), rstd_next, B(branch), B(g_post),
                                          rstd_post, M(dx_in), M(dbranch), pg_next, pg_post, T, D, eps, parts, G, stages,
                                          op_bytes, inv_if_pow2(D), row_status_word());
  NM_CUDA(cudaGetLastError());
}

}  // namespace nm::ew
