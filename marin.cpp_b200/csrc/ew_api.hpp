// The RMSNorm pair the readout head calls around the fused CE (bf16 storage). Semantics follow the reference's
// src/kernels/elementwise/rmsnorm_kernels.cuh:3-9:
//   levanter  forward   ms = sum(x^2) / D; r = rsqrt(ms + eps); y = bf16(x r); out = bf16(g y)
//             backward  a = bf16(g dy); dg += f32(bf16(dy y)); s = sum(x a); c = (s (-0.5 (r / (ms + eps)))) / D;
//                       dx = bf16(a r + c (2 x)); with a residual gradient: bf16(dres + bf16(dx))
//   accurate  f32 throughout, one rounding per stored output (dg accumulates dy x r in f32)
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "marincpp/core.hpp"

namespace nm::ew {

// Number of gain-gradient partial rows the backward writes for T rows on the current device:
// min(1024, ceil(T / 16), 4 x SMs) parts of consecutive rows (reference ew_api.hpp:18-21).
int64_t norm_partial_rows(int64_t T);

void rmsnorm_fwd(const bf16_t* x, const bf16_t* gain, bf16_t* y, float* rstd, int64_t T, int D, float eps,
                 cudaStream_t st, Rounding r = Rounding::Levanter);
// dx = norm backward of dy (+ dres when given; dres may equal dx); dgain_partial [norm_partial_rows(T), D] or nullptr
void rmsnorm_bwd_add(const bf16_t* dy, const bf16_t* x, const bf16_t* gain, const float* rstd, const bf16_t* dres,
                     bf16_t* dx, float* dgain_partial, int64_t T, int D, float eps, cudaStream_t st,
                     Rounding r = Rounding::Levanter);

}  // namespace nm::ew
