// A C++ caller of the reference-shaped entry points, as the reference's own integration tests are
// (test/singleGPU/cpp/moe/moeTest.cpp:28-70, moeApiTest.cpp:5-12): GetDistributedUniqueId by value,
// CreateLauncher with a C++ reference argument, Launch through the vtable, DestroyLauncher.
//   launcher_api_test errors                 the create-time error paths (no GPU needed)   -> exit 0 if all hold
//   launcher_api_test run <tokens> <file>    the reference's layer (Qwen3-30B-A3B shape, fp32 tensors) on
//                                            generated inputs; the fp32 output goes to <file>
// Inputs: element i of tensor `salt` is ((h(i, salt) >> 24) - 128) / 128 * scale with an integer hash h,
// values that bf16 holds exactly; the Python side of the test regenerates them for the CPU oracle.
#include <cuda_runtime_api.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "../../include/iMoeKernelLauncher.h"

static float Value(uint64_t i, uint32_t salt, float scale) {
  uint32_t u = (uint32_t)i * 2654435761u + salt;
  u ^= u >> 15;
  u *= 2246822519u;
  u ^= u >> 13;
  return ((float)(u >> 24) - 128.0f) / 128.0f * scale;
}

static float* DeviceTensor(uint64_t n, uint32_t salt, float scale) {
  std::vector<float> h(n);
  for (uint64_t i = 0; i < n; ++i) h[i] = Value(i, salt, scale);
  float* d = nullptr;
  if (cudaMalloc(reinterpret_cast<void**>(&d), n * sizeof(float)) != cudaSuccess) return nullptr;
  if (cudaMemcpy(d, h.data(), n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
  return d;
}

static int Errors() {
  int bad = 0;
  const moe::DistributedUniqueId empty = GetDistributedUniqueId(true);
  for (int i = 0; i < 128; ++i) bad += empty.data[i] != 0;
  const moe::DistributedUniqueId a = GetDistributedUniqueId(false), b = GetDistributedUniqueId(false);
  bad += memcmp(a.data, empty.data, 128) == 0;
  bad += memcmp(a.data, b.data, 128) == 0;
  // the reference's API test: null weights and 1024 tokens must fail and leave the pointer alone
  moe::IMoeKernelLauncher* launcher = nullptr;
  const cudaError_t e = CreateLauncher(&launcher, nullptr, nullptr, nullptr, 1024, nullptr, empty, 0, 1);
  bad += e != cudaErrorUnknown;
  bad += launcher != nullptr;
  bad += CreateLauncher(&launcher, nullptr, nullptr, nullptr, 16, nullptr, empty, 3, 2) == cudaSuccess;  // bad rank
  bad += launcher != nullptr;
  bad += DestroyLauncher(nullptr, nullptr) == cudaSuccess;
  printf("errors: %d violations\n", bad);
  return bad ? 1 : 0;
}

static int Run(int tokens, const char* path) {
  const uint64_t E = 128, H = 2048, I = 768;
  float* gate = DeviceTensor(E * H, 1u, 0.03125f);
  float* w13 = DeviceTensor(E * 2 * I * H, 2u, 0.03125f);
  float* w2 = DeviceTensor(E * H * I, 3u, 0.03125f);
  float* x = DeviceTensor((uint64_t)tokens * H, 4u, 2.0f);
  float* out = nullptr;
  if (!gate || !w13 || !w2 || !x || cudaMalloc(reinterpret_cast<void**>(&out), (uint64_t)tokens * H * 4) != cudaSuccess) {
    printf("allocation failed\n");
    return 2;
  }
  const moe::DistributedUniqueId uid = GetDistributedUniqueId(true);
  moe::IMoeKernelLauncher* launcher = nullptr;
  cudaError_t e = CreateLauncher(&launcher, gate, w13, w2, tokens + 2, nullptr, uid, 0, 1);
  if (e != cudaSuccess || !launcher) {
    printf("CreateLauncher failed: %d\n", (int)e);
    return 3;
  }
  // too many tokens: an error code, not a crash
  if (launcher->Launch(x, out, tokens + 3, nullptr) == cudaSuccess) return 4;
  e = launcher->Launch(x, out, tokens, nullptr);  // virtual call, as the reference's callers make it
  if (e != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    printf("Launch failed: %d\n", (int)e);
    return 5;
  }
  std::vector<float> h((uint64_t)tokens * H);
  if (cudaMemcpy(h.data(), out, h.size() * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return 6;
  // in place, as the reference's vLLM wrapper calls it (output aliasing the tokens)
  e = launcher->Launch(x, x, tokens, nullptr);
  std::vector<float> h2((uint64_t)tokens * H);
  if (e != cudaSuccess || cudaMemcpy(h2.data(), x, h2.size() * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return 7;
  if (memcmp(h.data(), h2.data(), h.size() * 4) != 0) {
    printf("in-place result differs\n");
    return 8;
  }
  e = DestroyLauncher(launcher, nullptr);
  if (e != cudaSuccess) return 9;
  FILE* f = fopen(path, "wb");
  if (!f || fwrite(h.data(), 4, h.size(), f) != h.size()) return 10;
  fclose(f);
  printf("run ok: %d tokens\n", tokens);
  return 0;
}

int main(int argc, char** argv) {
  if (argc >= 2 && strcmp(argv[1], "errors") == 0) return Errors();
  if (argc >= 4 && strcmp(argv[1], "run") == 0) return Run(atoi(argv[2]), argv[3]);
  printf("usage: launcher_api_test errors | run <tokens> <file>\n");
  return 64;
}
