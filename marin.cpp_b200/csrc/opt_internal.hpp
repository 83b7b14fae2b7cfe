// Internal interface between the AdamH host code (opt_api.cpp) and its kernels (opt_adamh.cu).
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "marincpp/core.hpp"

namespace nm::opt {

// Element ranges of the flat [V, D] tensor this rank owns: global offset (into the gradient and the bf16 replica),
// compact offset (into the rank's own master / moment arrays, which hold only owned elements) and length.
constexpr int kMaxRanges = 64;
struct Ranges {
  int n = 0;
  int64_t goff[kMaxRanges];
  int64_t coff[kMaxRanges];
  int64_t len[kMaxRanges];
};

// Scalars of one step in device memory (f64): sum over the whole tensor (all ranks) of g^2, p^2, a^2 and p a.
enum : int { kSumG = 0, kSumPP = 1, kSumAA = 2, kSumPA = 3, kNumScalars = 4 };

struct Hyper {
  float eta, b1, b2, one_minus_b1, one_minus_b2, eps, bc1, bc2, grad_scale, max_norm, clip_gn;
  int clip_mode;   // 0 none, 1 (clip_gn, clip) given by the caller, 2 gn = sqrt(f32(scal[kSumG])) on the device
  int clip;
};

// Row blocks of the one-tensor entry points (device arrays): block id per row, per-block learning-rate multiplier
// (nullable: 1), per-block frozen flag (nullable: none).
struct BlockTab {
  const int32_t* block_of_row;
  const float* lr_mult;
  const uint8_t* frozen;
  int n_blocks;
};

constexpr int kMaxBlocksTotal = 148 * 8;
int partial_blocks(const Ranges& r);   // partial slots (of 1 or 3 doubles) a launch over r writes

// out (+)= sum over the ranges of (g * grad_scale)^2
void launch_sumsq(const float* g, const Ranges& r, float grad_scale, double* partial, double* out, bool accumulate,
                  cudaStream_t st);
// pass 1: mu, nu updated in place; scal[kSumPP..kSumPA] = this rank's sums (the caller all-reduces them)
void launch_moments(const Ranges& r, const float* g, const float* p, float* mu, float* nu, const Hyper& h, double* scal,
                    double* partial, cudaStream_t st);
// pass 2: p updated in place, bf16(p) written at the global positions of w16 (nullable)
void launch_apply(const Ranges& r, float* p, const float* mu, const float* nu, void* w16, const Hyper& h,
                  const double* scal, cudaStream_t st);
// plain Adam in one pass: p += (-eta) a (h.eta is the Adam learning rate); scal is read only with clip_mode 2
void launch_adam(const Ranges& r, const float* g, float* p, float* mu, float* nu, void* w16, const Hyper& h,
                 const double* scal, cudaStream_t st);
// the same updates with a row partition; row_partial: rows * 3 doubles, blk_scal: n_blocks * 3 doubles (scratch)
void launch_blk_adamh(const float* g, float* p, float* mu, float* nu, void* w16, int64_t rows, int64_t cols,
                      const Hyper& h, const BlockTab& bt, double* row_partial, double* blk_scal, cudaStream_t st);
void launch_blk_adam(const float* g, float* p, float* mu, float* nu, void* w16, int64_t rows, int64_t cols,
                     const Hyper& h, const BlockTab& bt, cudaStream_t st);
void launch_master_from_bf16(const Ranges& r, const void* w16, float* p, cudaStream_t st);

}  // namespace nm::opt
