// nm_ce_forward_noalloc: the forward (statistics + loss) half of the fused linear cross-entropy for callers that cannot
// supply or allocate a workspace. Its scratch (per-tile softmax partials and lse of one chunk) lives in a file-scope
// device array of fixed size that every GPU using this library holds from load to exit.
//
// Who needs this: code that runs where device allocation is off limits. Two cases seen with this library's host: (1) a
// trainer that makes one arena allocation up front and plans every buffer in it (the design of the reference's memory
// plan) has no spare region to hand to an evaluation or probe call that was not in the plan; (2) while any thread of
// the process has a stream capture open in the global or thread-local capture mode, cudaMalloc / cudaFree are not
// permitted, so a helper thread that wants a quick loss read-out cannot size and allocate a workspace on the spot.
//
// Rules of use:
//   * The first call on a device looks up the device address of the array (cudaGetSymbolAddress, with that device
//     current) and caches it; make that first call before any stream capture begins.
//   * All calls on a device share the one array and it keeps whatever the previous call left. The only word that must
//     start at zero, the wait-status word, is cleared on the stream at the start of every call; everything else is
//     written before it is read within a call.
//   * Two calls whose kernels may overlap on the same GPU (different streams, or different host threads) race on the
//     array. Serialise them.
//   * With r = min(chunk_rows, T) rows per chunk the scratch needed is 256 + 8 ceil(V / 256) r + 4 r bytes (each
//     region rounded up to 256); a call that needs more than kScratchBytes (16 MiB) is refused with NM_ERR_INVALID.
//     At V = 128256 that allows r up to 4096.
//   * The kernels' waits are bounded; one that ran out leaves a bit in the array's status word and the losses of that
//     call are not to be trusted. nm_ce_forward_noalloc_status reads the word (it synchronises the stream).
// Neither entry point makes an allocation of any kind: no cudaMalloc / cudaFree, no allocating library call.
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>
#include <string>

#include "abi_guard.hpp"
#include "ce_internal.hpp"
#include "marincpp/capi_ce.h"

namespace nm::ce {
namespace {

constexpr size_t kScratchBytes = size_t(16) << 20;
static __device__ __align__(256) unsigned char g_ce_static_scratch[kScratchBytes];

std::mutex g_scratch_mu;
void* g_scratch_ptr[kMaxDeviceOrdinals] = {};

// The array's name is only a host-side handle; kernels need its device address, which differs per device.
void* scratch_of_current_device() {
  const int dev = current_device_info().ordinal;
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    NM_CUDA(cudaGetSymbolAddress(&p, g_ce_static_scratch));
    NM_REQUIRE(p && reinterpret_cast<uintptr_t>(p) % 256 == 0, "nm_ce_forward_noalloc: scratch address not aligned");
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}

void forward_noalloc(const void* x, const void* w, const int32_t* targets, const float* weight, float* loss_tok,
                     float* lse, float* loss_partial, int64_t T, int D, int V, int chunk_rows, float z_loss,
                     int32_t ignore_index, cudaStream_t st) {
  NM_REQUIRE(T >= 0 && D > 0 && V > 0, "nm_ce_forward_noalloc: T >= 0, D > 0, V > 0");
  NM_REQUIRE(D % 8 == 0, "nm_ce_forward_noalloc: D must be a multiple of 8");
  NM_REQUIRE(chunk_rows > 0, "nm_ce_forward_noalloc: chunk_rows must be positive");
  if (T == 0) return;
  NM_REQUIRE(x && w && targets && weight && loss_tok, "nm_ce_forward_noalloc: x, w, targets, weight and loss_tok are "
                                                      "required");
  // the same regions, in the same order, as the head of a caller-owned workspace; no chunk is longer than the call
  const int64_t rows = std::min<int64_t>(chunk_rows, T);
  Arena measure(nullptr);
  const uint64_t need = layout_forward(measure, V, rows).bytes;
  NM_REQUIRE(need <= kScratchBytes,
             "nm_ce_forward_noalloc: V = " + std::to_string(V) + " with " + std::to_string(rows) +
                 " rows per chunk needs " + std::to_string(need) + " bytes of scratch, more than the built-in " +
                 std::to_string(kScratchBytes) + "; use a smaller chunk_rows, or nm_fused_linear_ce with a workspace");
  NM_REQUIRE(device_arch() >= 100, "nm_ce_forward_noalloc: sm_100a kernels only");
  Arena arena(scratch_of_current_device());
  const Regions regions = layout_forward(arena, V, rows);
  run_forward(regions, x, w, targets, weight, loss_tok, lse, loss_partial, T, D, V, int(rows), z_loss, ignore_index, st);
}

}  // namespace
}  // namespace nm::ce

extern "C" int nm_ce_forward_noalloc(const void* x, const void* w, const int32_t* targets, const float* weight,
                                     float* loss_tok, float* lse, float* loss_partial, int64_t T, int D, int V,
                                     int chunk_rows, float z_loss_weight, int32_t ignore_index, void* stream) {
  return nm::abi::guarded([&] {
    nm::ce::forward_noalloc(x, w, targets, weight, loss_tok, lse, loss_partial, T, D, V, chunk_rows, z_loss_weight,
                            ignore_index, static_cast<cudaStream_t>(stream));
  });
}

extern "C" int nm_ce_forward_noalloc_status(void* stream, uint32_t* status_host) {
  return nm::abi::guarded([&] {
    NM_REQUIRE(status_host != nullptr, "nm_ce_forward_noalloc_status: status_host is required");
    auto st = static_cast<cudaStream_t>(stream);
    // word 0 of the built-in array is the status word of the calls made on this device
    NM_CUDA(cudaMemcpyAsync(status_host, nm::ce::scratch_of_current_device(), sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    NM_CUDA(cudaStreamSynchronize(st));
    if (*status_host != 0)
      throw nm::DeviceError("nm_ce_forward_noalloc: a bounded device-side wait ran out (status bits " +
                            std::to_string(*status_host) + "); the losses of that call are invalid");
  });
}

// Test hook: runs the short bounded-wait probe of nm_ce_test_wait_timeout against the status word of the built-in
// scratch, so that the word afterwards holds what a kernel of this entry point whose wait ran out would have left.
extern "C" int nm_ce_forward_noalloc_test_timeout(int64_t limit_cycles, void* stream) {
  return nm::abi::guarded([&] {
    uint32_t* word = static_cast<uint32_t*>(nm::ce::scratch_of_current_device());
    int* saw_abort = reinterpret_cast<int*>(word + 1);   // inside the 256-byte status region
    nm::ce::launch_wait_timeout_probe(word, static_cast<long long>(limit_cycles), saw_abort,
                                      static_cast<cudaStream_t>(stream));
  });
}
