// Core types of the fused-CE drop-in: scalar dtypes, the rounding policy enums, the error convention.
// Mirrors the part of the reference's include/marincpp/core.hpp the CE path needs (reference:
// include/marincpp/core.hpp:25-34 DType, :41-48 bf16 helpers, :62-76 Rounding / CeDwRound, :113-132 errors), with the
// same names, enumerator values and macro spellings, so a translation unit written against the reference header
// (src/model/baseline.cpp:366-373) compiles unchanged against this one.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

typedef struct CUstream_st* cudaStream_t;

namespace nm {

enum class DType : uint8_t { f32 = 0, bf16 = 1, f16 = 2, i32 = 3, u32 = 4, i64 = 5, u8 = 6, f64 = 7 };
constexpr size_t dtype_size(DType t) {
  switch (t) {
    case DType::f32: case DType::i32: case DType::u32: return 4;
    case DType::bf16: case DType::f16: return 2;
    case DType::i64: case DType::f64: return 8;
    case DType::u8: return 1;
  }
  return 0;
}

// bfloat16 storage for host code and headers; device code uses __nv_bfloat16 (same bits).
struct bf16_t { uint16_t bits; };
static_assert(sizeof(bf16_t) == 2, "bf16_t is two bytes");

// f32 <-> bf16 on the host, round to nearest even; NaN stays a quiet NaN.
inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7f800000u) == 0x7f800000u && (u & 0x007fffffu)) return static_cast<uint16_t>((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
inline float bf16_bits_to_f32(uint16_t b) {
  const uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// Rounding policy of the dX accumulate epilogue (Levanter: bf16(old + f32(bf16(acc))); Accurate: bf16(old + acc)).
enum class Rounding : uint8_t { Levanter = 0, Accurate = 1 };
// Strict dW mode: each chunk's dW is rounded to bf16 before it is added to the per-microbatch accumulator.
enum class CeDwRound : uint8_t { None = 0, PerChunkBf16 = 1 };

// Errors. fatal() throws nm::Fatal (bad argument / unmet requirement); a failed CUDA or NCCL call throws
// nm::DeviceError. The C ABI turns them into NM_ERR_INVALID / NM_ERR_DEVICE plus nm_last_error().
struct Fatal : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct DeviceError : Fatal {
  using Fatal::Fatal;
};
[[noreturn]] void fatal(const char* where, const std::string& msg);
void cuda_check(int err, const char* expr, const char* where);
void nccl_check(int err, const char* expr, const char* where);

#define NM_STR2(x) #x
#define NM_STR(x) NM_STR2(x)
#define NM_WHERE __FILE__ ":" NM_STR(__LINE__)
#define NM_CUDA(x) ::nm::cuda_check(static_cast<int>(x), #x, NM_WHERE)
#define NM_NCCL(x) ::nm::nccl_check(static_cast<int>(x), #x, NM_WHERE)
#define NM_REQUIRE(cond, msg) \
  do { if (!(cond)) ::nm::fatal(NM_WHERE, std::string("requirement failed: " #cond ": ") + (msg)); } while (0)

inline constexpr int kMaxGpus = 8;
inline constexpr size_t kArenaAlign = 256;   // every workspace region starts on a 256-byte boundary

}  // namespace nm
