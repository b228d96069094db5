// C entry points around the reference project's own CPU MoE headers.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit includes the reference's
// header-only implementation from where it lies (the include path is given by
// the Makefile, REF=<reference root>); no reference source is copied here.  The
// resulting oracle/_ref/libref_moe.so is the real reference algorithm, used to
// pin moe_oracle.c, to generate tests/golden/, and as the timed CPU baseline
// ("kind": "reference").  The shipped library never links or loads it.
//
// Wrapped functions (reference paths):
//   test::refGemm            test/singleGPU/cpp/moe/reference/refGemm.h:11-29
//   test::refMoeGate         test/singleGPU/cpp/moe/reference/refMoeGate.h:16-33
//   test::refExpertFFN1      test/singleGPU/cpp/moe/reference/refExpertFFN1.h:51-65
//   test::refFullMoe         test/singleGPU/cpp/moe/reference/refFullMoe.h:9-69
#include <cstring>
#include <vector>

#include "test/singleGPU/cpp/moe/reference/refFullMoe.h"

#include <unistd.h>

#include <thread>

extern "C" {

void ref_gemm_nt(const float* A, const float* B, float* C, int M, int N, int K) {
  auto out = test::refGemm(A, B, M, N, K);
  std::memcpy(C, out.data(), out.size() * sizeof(float));
}

void ref_gate(const float* tokens, const float* gate_w, int T, int E, int H,
              int topk, float* topk_w, int* topk_idx) {
  auto g = test::refMoeGate(tokens, gate_w, T, E, H, topk);
  std::memcpy(topk_w, g.topkVals.data(), g.topkVals.size() * sizeof(float));
  std::memcpy(topk_idx, g.topkIdx.data(), g.topkIdx.size() * sizeof(int));
}

void ref_ffn1(const float* tokens, const float* w13, int rows, int H, int I,
              float* out) {
  auto o = test::refExpertFFN1(tokens, w13, rows, H, I);
  std::memcpy(out, o.data(), o.size() * sizeof(float));
}

// The reference function as shipped: one call over all tokens, one thread.
void ref_full_moe(const float* tokens, const float* gate_w, const float* w13,
                  const float* w2, int T, int E, int H, int topk, int I,
                  float* out) {
  if (T <= 0) return;
  auto o = test::refFullMoe(tokens, gate_w, w13, w2, T, E, H, topk, I);
  std::memcpy(out, o.data(), o.size() * sizeof(float));
}

// Same function called once per token from a pool of std::threads.  Tokens are
// independent in the reference, so the result equals ref_full_moe bit for bit;
// this is how "all host cores" are used for the timed baseline.
void ref_full_moe_mt(const float* tokens, const float* gate_w, const float* w13,
                     const float* w2, int T, int E, int H, int topk, int I,
                     float* out, int threads) {
  if (T <= 0) return;
  if (threads < 1) threads = 1;
  if (threads > T) threads = T;
  auto work = [=](int tid) {
    for (int t = tid; t < T; t += threads) {
      auto o = test::refFullMoe(tokens + size_t(t) * size_t(H), gate_w, w13, w2,
                                1, E, H, topk, I);
      std::memcpy(out + size_t(t) * size_t(H), o.data(), size_t(H) * sizeof(float));
    }
  };
  std::vector<std::thread> pool;
  for (int i = 1; i < threads; ++i) pool.emplace_back(work, i);
  work(0);
  for (auto& th : pool) th.join();
}

int ref_max_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n < 1 ? 1 : int(n);
}

}  // extern "C"
