// Shared pieces of the tcgen05 contraction kernels of the fused linear cross-entropy (ce_gemm.cu: the classic
// 128 x 256-tile template; ce_grad_wide.cu: the CTA-pair gradient kernels with one 512-column accumulator): launch
// parameters, the epilogue bodies (one call = 32 accumulator columns of one row, held in registers), the writers of
// the swizzled staging tiles, and the host-side tensor-map builders.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "ce_internal.hpp"
#include "ptx.cuh"

namespace nm::ce {
namespace {

using namespace nm::ptx;

constexpr int BM = 128, BN = 256, BK = 64, UK = 16;
constexpr int kBoxBytesMN = 64 * BK * 2;        // one MN-major box: 64 k-rows of 128 bytes = 8 KiB
constexpr int kTmemCols = 512;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;
enum Epi : int { kEpiLogits = 0, kEpiDx = 1, kEpiDw = 2, kEpiTest = 3 };
constexpr int kEpiBufBytes = 32 * 128;          // one 32-row x 128-byte staging tile per epilogue warp

struct GemmParams {
  int M, N, K;              // extents of this launch: accumulator rows, columns, contraction length
  int m_off;                // first A coordinate along M (dW vocabulary range start)
  int num_m, num_n;         // tiles
  int m_inner;              // 1: consecutive tile indices walk M first (logits), 0: N first
  int m_group;              // m_inner only: M tiles are walked in groups of this many (all N tiles of a group before
                            // the next group), so that the A rows of a group stay in L2 while B streams past
  int a_3d, b_3d;           // an MN-major operand whose M / N extent is a multiple of 64 is described by a 3-D tensor
                            // map (64 contiguous, K, groups of 64): one TMA instruction per stage instead of 2 or 4
  uint32_t* status;
  // logits
  void* store; int64_t ldS; int store_f32;
  float* tmax; float* tsum; int64_t ldT; float* zt; const int32_t* targets; const float* bias;
  // dX
  const float* scale; const void* dx_old; void* dx_out; int acc_mode; int out_f32; int64_t ldo;
  // dW
  float* dw; int round_bf16;
  // test
  float* c; int64_t ldc;
  // gradient kernels that form n on the fly: per-row factors, indexed by the row of the logits store
  const RowFactors* rowf;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float round_bf16f(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ---------------------------------------------------------------------------------------------- epilogues
// One call handles the 32 accumulator columns [col0, col0 + 32) of row `grow` held in v[].
struct LogitsRowState {
  float m, s, zt;
  bool hit;
};

__device__ __forceinline__ void epi_logits_chunk(const GemmParams& p, float* v, int grow, bool row_ok, int col0, int tg,
                                                 LogitsRowState& st) {
  const int V = p.N;
  const int ncols = min(32, V - col0);
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) v[j] += __ldg(p.bias + col0 + j);
  }
  if (p.store && p.store_f32 && row_ok) {   // f32 store: direct (the bf16 store leaves through the staging tile)
    float* o = static_cast<float*>(p.store) + int64_t(grow) * p.ldS + col0;
    if (ncols == 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)     // static indices only: a runtime index would move v[] to local memory
        if (j < ncols) o[j] = v[j];
    }
  }
  // online (max, sum exp): one rescale of the running sum per 32 columns
  constexpr float kLog2e = 1.4426950408889634f;
  float m_new, a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, neg;
  if (ncols == 32) {                       // every chunk but the last of a ragged vocabulary: no column predicates
    float c0 = fmaxf(v[0], v[1]), c1 = fmaxf(v[2], v[3]), c2 = fmaxf(v[4], v[5]), c3 = fmaxf(v[6], v[7]);
#pragma unroll
    for (int j = 8; j < 32; j += 8) {
      c0 = fmaxf(c0, fmaxf(v[j], v[j + 1]));
      c1 = fmaxf(c1, fmaxf(v[j + 2], v[j + 3]));
      c2 = fmaxf(c2, fmaxf(v[j + 4], v[j + 5]));
      c3 = fmaxf(c3, fmaxf(v[j + 6], v[j + 7]));
    }
    m_new = fmaxf(st.m, fmaxf(fmaxf(c0, c1), fmaxf(c2, c3)));
    neg = -m_new * kLog2e;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      a0 += ex2_approx(fmaf(v[j], kLog2e, neg));
      a1 += ex2_approx(fmaf(v[j + 1], kLog2e, neg));
      a2 += ex2_approx(fmaf(v[j + 2], kLog2e, neg));
      a3 += ex2_approx(fmaf(v[j + 3], kLog2e, neg));
    }
  } else {
    float cm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) cm = fmaxf(cm, v[j]);
    m_new = fmaxf(st.m, cm);
    neg = -m_new * kLog2e;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      a0 += (j < ncols) ? ex2_approx(fmaf(v[j], kLog2e, neg)) : 0.f;
      a1 += (j + 1 < ncols) ? ex2_approx(fmaf(v[j + 1], kLog2e, neg)) : 0.f;
      a2 += (j + 2 < ncols) ? ex2_approx(fmaf(v[j + 2], kLog2e, neg)) : 0.f;
      a3 += (j + 3 < ncols) ? ex2_approx(fmaf(v[j + 3], kLog2e, neg)) : 0.f;
    }
  }
  // st.m == -inf on the first chunk: ex2(-inf) = 0 and st.s = 0
  st.s = st.s * ex2_approx(fmaf(st.m, kLog2e, neg)) + ((a0 + a1) + (a2 + a3));
  st.m = m_new;
  if (tg >= col0 && tg < col0 + 32) {
    const int jt = tg - col0;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j == jt) st.zt = v[j];
    st.hit = true;
  }
}

__device__ __forceinline__ void epi_dx_chunk(const GemmParams& p, const float* v, int grow, int col0, float scale) {
  const int D = p.N;
  const int ncols = min(32, D - col0);   // D % 8 == 0, so ncols is a multiple of 8
  if (p.out_f32) {
    float* o = static_cast<float*>(p.dx_out) + int64_t(grow) * p.ldo + col0;
    const float* old = static_cast<const float*>(p.dx_old) + int64_t(grow) * p.ldo + col0;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      if (j < ncols) {
        float4 r = make_float4(v[j] * scale, v[j + 1] * scale, v[j + 2] * scale, v[j + 3] * scale);
        if (p.acc_mode) {
          const float4 q = *reinterpret_cast<const float4*>(old + j);
          r.x += q.x; r.y += q.y; r.z += q.z; r.w += q.w;
        }
        *reinterpret_cast<float4*>(o + j) = r;
      }
    }
    return;
  }
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.dx_out) + int64_t(grow) * p.ldo + col0;
  const __nv_bfloat16* old = static_cast<const __nv_bfloat16*>(p.dx_old) + int64_t(grow) * p.ldo + col0;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    if (j < ncols) {
      float r[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) r[e] = v[j + e] * scale;
      if (p.acc_mode) {
        const uint4 q = *reinterpret_cast<const uint4*>(old + j);
        const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float o0 = bf_lo(qq[e]), o1 = bf_hi(qq[e]);
          if (p.acc_mode == 1) {   // levanter: bf16(old + f32(bf16(acc)))
            r[2 * e] = o0 + round_bf16f(r[2 * e]);
            r[2 * e + 1] = o1 + round_bf16f(r[2 * e + 1]);
          } else {                 // accurate: bf16(old + acc)
            r[2 * e] = o0 + r[2 * e];
            r[2 * e + 1] = o1 + r[2 * e + 1];
          }
        }
      }
      *reinterpret_cast<uint4*>(o + j) =
          make_uint4(pack2(r[0], r[1]), pack2(r[2], r[3]), pack2(r[4], r[5]), pack2(r[6], r[7]));
    }
  }
}

// Staging writers: this lane's row of a 32-row staging tile, 16-byte pieces XOR-swizzled with the row the way the
// tensor map's swizzle mode expects (the tile is 1024-byte aligned). f32: a 32-row x 128-byte tile (32 columns),
// SWIZZLE_128B: piece j of row r at r * 128 + ((j ^ (r & 7)) << 4).
// bf16: a 32-row x 64-byte tile (32 columns), SWIZZLE_64B: piece j of row r at r * 64 + ((j ^ ((r >> 1) & 3)) << 4).
__device__ __forceinline__ void stage_bf16_chunk(uint32_t buf, int lane, const float* v) {
#pragma unroll
  for (int j = 0; j < 4; ++j)
    st_shared_v4(buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4), pack2(v[8 * j], v[8 * j + 1]),
                 pack2(v[8 * j + 2], v[8 * j + 3]), pack2(v[8 * j + 4], v[8 * j + 5]), pack2(v[8 * j + 6], v[8 * j + 7]));
}
__device__ __forceinline__ void stage_f32_row(uint32_t buf, int lane, const float* v, float scale, bool round_bf16) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float r0 = v[4 * j] * scale, r1 = v[4 * j + 1] * scale, r2 = v[4 * j + 2] * scale, r3 = v[4 * j + 3] * scale;
    if (round_bf16) { r0 = round_bf16f(r0); r1 = round_bf16f(r1); r2 = round_bf16f(r2); r3 = round_bf16f(r3); }
    st_shared_v4(buf + lane * 128 + ((j ^ (lane & 7)) << 4), __float_as_uint(r0), __float_as_uint(r1),
                 __float_as_uint(r2), __float_as_uint(r3));
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------- host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
  static std::once_flag once;
  static EncodeFn fn = nullptr;
  static cudaError_t err = cudaSuccess;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (err == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeFn>(p);
  });
  if (!fn) {
    cudaGetLastError();
    throw DeviceError(std::string("fused CE: cuTensorMapEncodeTiled is not available from the CUDA driver (") +
                      cudaGetErrorString(err) + "); this library needs an sm_100a device and has no other path");
  }
  return fn;
}

// bf16 matrix with `inner` contiguous elements per row, `outer` rows, row pitch ld elements; box = (box_inner, box_outer)
inline CUtensorMap make_tmap(const void* base, uint64_t inner, uint64_t outer, int64_t ld, uint32_t box_inner,
                      uint32_t box_outer, bool f32 = false, int swizzle_bytes = 128) {
  const int esz = f32 ? 4 : 2;
  NM_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0, "fused CE: a TMA operand must be 16-byte aligned");
  NM_REQUIRE((ld * esz) % 16 == 0, "fused CE: a TMA operand's row pitch must be a multiple of 16 bytes");
  NM_REQUIRE(inner > 0 && outer > 0, "fused CE: empty TMA operand");
  CUtensorMap m;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {cuuint64_t(ld) * esz};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode_fn()(&m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 swizzle_bytes == 0 ? CU_TENSOR_MAP_SWIZZLE_NONE : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw DeviceError("fused CE: cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r)) + " (inner " +
                      std::to_string(inner) + ", outer " + std::to_string(outer) + ", ld " + std::to_string(ld) + ")");
  return m;
}
// K-major operand [rows, K]: box = 64 k x `rows_per_box` rows. MN-major operand [K, MN]: box = 64 mn x 64 k.
inline CUtensorMap tmap_kmajor(const void* base, int64_t rows, int64_t K, int64_t ld, int rows_per_box) {
  return make_tmap(base, uint64_t(K), uint64_t(rows), ld, BK, uint32_t(rows_per_box));
}
inline CUtensorMap tmap_mnmajor(const void* base, int64_t K, int64_t MN, int64_t ld) {
  return make_tmap(base, uint64_t(MN), uint64_t(K), ld, 64, BK);
}
// The same operand when MN % 64 == 0, as a 3-D tensor (64 contiguous, K rows of pitch ld, MN / 64 groups 64 elements
// apart): a box of (64, 64 k, `groups`) lands in shared memory as `groups` consecutive 64-k x 128-byte blocks, which
// is the layout the 2-D boxes are placed in one by one.
inline CUtensorMap tmap_mnmajor_3d(const void* base, int64_t K, int64_t MN, int64_t ld, int groups) {
  NM_REQUIRE(MN % 64 == 0, "fused CE: the 3-D operand map needs an extent that is a multiple of 64");
  NM_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0 && (ld * 2) % 16 == 0, "fused CE: TMA operand alignment");
  CUtensorMap m;
  const cuuint64_t dims[3] = {64, cuuint64_t(K), cuuint64_t(MN / 64)};
  const cuuint64_t strides[2] = {cuuint64_t(ld) * 2, 128};
  const cuuint32_t box[3] = {64, BK, cuuint32_t(groups)};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw DeviceError("fused CE: cuTensorMapEncodeTiled (3-D) failed with CUresult " + std::to_string(int(r)));
  return m;
}
inline CUtensorMap tmap_mn_a(const void* base, int64_t K, int64_t MN, int64_t ld, int& is3d) {
  is3d = MN % 64 == 0;
  return is3d ? tmap_mnmajor_3d(base, K, MN, ld, BM / 64) : tmap_mnmajor(base, K, MN, ld);
}
inline CUtensorMap tmap_mn_b(const void* base, int64_t K, int64_t MN, int64_t ld, int& is3d, int ncta) {
  is3d = MN % 64 == 0;
  return is3d ? tmap_mnmajor_3d(base, K, MN, ld, BN / ncta / 64) : tmap_mnmajor(base, K, MN, ld);
}

// epilogue staging tile as a tensor-map box: 32 rows x 32 columns (f32: 128-byte rows, SWIZZLE_128B; bf16: 64-byte
// rows, SWIZZLE_64B)
inline CUtensorMap tmap_epilogue(void* base, int64_t rows, int64_t cols, int64_t ld, bool f32) {
  return make_tmap(base, uint64_t(cols), uint64_t(rows), ld, 32, 32, f32, f32 ? 128 : 64);
}

}  // namespace nm::ce
