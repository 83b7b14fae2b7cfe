// The reference trainer's call site (src/model/baseline.cpp:366-373) written against this repository's headers and
// linked against its static archive: builds CeShape / CeArgs the same way, calls nm::ce_workspace_bytes and
// nm::fused_linear_ce, then sums the per-chunk losses. Prints "loss_sum <value> dw_abs <value> dx_abs <value>". Then the
// optimizer site for the head: nm::HeadAdamH (one rank owns the whole tensor) on the dW just produced, printing
// "p_abs <value> w16_abs <value>".
// Inputs: a fixed integer-hash pattern (no RNG library), so a Python test can rebuild them and compare.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "marincpp/core.hpp"
#include "marincpp/kernels/cross_entropy.hpp"
#include "marincpp/kernels/head_optim.hpp"

namespace nm { class GemmCache {}; }   // the CE path ignores it; the trainer passes its planner

static float hash_unit(uint32_t i, uint32_t salt) {   // in [-1, 1)
  uint32_t x = i * 2654435761u + salt * 40503u + 12345u;
  x ^= x >> 16; x *= 2246822519u; x ^= x >> 13; x *= 3266489917u; x ^= x >> 16;
  return float(x >> 8) * (1.0f / 8388608.0f) - 1.0f;
}

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { std::printf("CUDA error %s at %s\n", cudaGetErrorString(e), #x); return 2; } } while (0)

int main() {
  using namespace nm;
  const int64_t T = 1500;
  const int D = 512, V = 8256, chunk = 512;
  std::vector<bf16_t> hx(T * D), hw(size_t(V) * D);
  std::vector<int32_t> ht(T);
  std::vector<float> hwt(T);
  for (int64_t i = 0; i < T * D; ++i) hx[i].bits = f32_to_bf16_bits(hash_unit(uint32_t(i), 1) * 1.7f);
  for (int64_t i = 0; i < int64_t(V) * D; ++i) hw[i].bits = f32_to_bf16_bits(hash_unit(uint32_t(i), 2) * 0.035f);
  float wsum = 0.f;
  for (int64_t t = 0; t < T; ++t) {
    ht[t] = int32_t((uint32_t(t) * 7919u + 13u) % uint32_t(V));
    hwt[t] = (t % 7 == 0) ? 0.f : 1.f;
    if (t % 11 == 0) ht[t] = -100;
    if (ht[t] >= 0) wsum += hwt[t];
  }
  const float hgs = 1.0f / wsum;

  CeShape shape{T, D, V, chunk, DType::bf16, DType::bf16};
  const uint64_t ws_bytes = ce_workspace_bytes(CeImpl::B1, shape);
  void *x, *w, *dx, *ws;
  int32_t* tg; float *wt, *gs, *loss, *lse, *part, *dw;
  const int n_chunks = int((T + chunk - 1) / chunk);
  CK(cudaMalloc(&x, T * D * 2)); CK(cudaMalloc(&w, size_t(V) * D * 2)); CK(cudaMalloc(&dx, T * D * 2));
  CK(cudaMalloc(&ws, ws_bytes)); CK(cudaMalloc(&tg, T * 4)); CK(cudaMalloc(&wt, T * 4)); CK(cudaMalloc(&gs, 4));
  CK(cudaMalloc(&loss, T * 4)); CK(cudaMalloc(&lse, T * 4)); CK(cudaMalloc(&part, n_chunks * 4));
  CK(cudaMalloc(&dw, size_t(V) * D * 4));
  CK(cudaMemcpy(x, hx.data(), T * D * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(w, hw.data(), size_t(V) * D * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(tg, ht.data(), T * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(wt, hwt.data(), T * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(gs, &hgs, 4, cudaMemcpyHostToDevice));
  CK(cudaMemset(dw, 0, size_t(V) * D * 4));
  cudaStream_t s;
  CK(cudaStreamCreate(&s));

  GemmCache gemm;
  CeArgs ca{};
  ca.x = x, ca.w = w, ca.targets = tg, ca.weight = wt, ca.grad_scale = gs;
  ca.logit_bias = nullptr, ca.loss_tok = loss, ca.lse = lse, ca.loss_partial = part;
  ca.dx = dx, ca.accumulate_dx = false, ca.dw = dw, ca.dw_microbatch = nullptr;
  ca.dw_round = CeDwRound::None, ca.forward_only = false;
  try {
    fused_linear_ce(CeImpl::B1, Rounding::Levanter, shape, ca, ws, gemm, s);
  } catch (const Fatal& e) {
    std::printf("fused_linear_ce threw: %s\n", e.what());
    return 3;
  }
  CK(cudaStreamSynchronize(s));
  std::vector<float> hp(n_chunks), hdw(size_t(V) * D);
  std::vector<bf16_t> hdx(T * D);
  CK(cudaMemcpy(hp.data(), part, n_chunks * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(hdw.data(), dw, size_t(V) * D * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(hdx.data(), dx, T * D * 2, cudaMemcpyDeviceToHost));
  double ls = 0, aw = 0, ax = 0;
  for (float v : hp) ls += v;
  for (float v : hdw) aw += std::fabs(v);
  for (const bf16_t& v : hdx) ax += std::fabs(bf16_bits_to_f32(v.bits));
  std::printf("loss_sum %.9g dw_abs %.9g dx_abs %.9g\n", ls * hgs, aw, ax);

  // the head's update from that gradient: master copy from the bf16 replica, zero moments, first update
  float *p32, *mu, *nu;
  const size_t n = size_t(V) * D;
  CK(cudaMalloc(&p32, n * 4)); CK(cudaMalloc(&mu, n * 4)); CK(cudaMalloc(&nu, n * 4));
  CK(cudaMemset(mu, 0, n * 4)); CK(cudaMemset(nu, 0, n * 4));
  try {
    HeadAdamH opt(V, D, nullptr);
    if (opt.owned_elems() != int64_t(n)) { std::printf("owned_elems mismatch\n"); return 4; }
    opt.init_master(static_cast<const bf16_t*>(w), p32, s);
    AdamHStep st;
    st.t = 1, st.eta = 0.02f, st.b1 = 0.9f, st.b2 = 0.98f, st.eps = 1e-20f, st.max_grad_norm = 1.0f, st.grad_scale = 1.0f;
    opt.step(st, dw, p32, mu, nu, static_cast<bf16_t*>(w), s);
    CK(cudaStreamSynchronize(s));
  } catch (const Fatal& e) {
    std::printf("HeadAdamH threw: %s\n", e.what());
    return 5;
  }
  std::vector<float> hpn(n);
  std::vector<bf16_t> hw2(n);
  CK(cudaMemcpy(hpn.data(), p32, n * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(hw2.data(), w, n * 2, cudaMemcpyDeviceToHost));
  double ap = 0, a16 = 0;
  for (float v : hpn) ap += std::fabs(v);
  for (const bf16_t& v : hw2) a16 += std::fabs(bf16_bits_to_f32(v.bits));
  std::printf("p_abs %.9g w16_abs %.9g\n", ap, a16);
  return 0;
}
