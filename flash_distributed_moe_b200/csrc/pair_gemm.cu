// Self-test of the CTA-pair tensor-core primitive the layer's FFN tiles are built
// from: one cluster of two CTAs computes D[256, N] = W[256, K] * X[N, K]^T with
// tcgen05.mma.cta_group::2 (bf16 in, fp32 out).  CTA c of the pair loads rows
// [128c, 128c + 128) of W and rows [c*N/2, (c+1)*N/2) of X; the even CTA issues
// the MMAs, which read both CTAs' shared memory and write rows [128c, 128c + 128)
// of D into CTA c's tensor memory.  Exposed as FlashMoeTestPairGemm.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/flashmoe_c.h"
#include "host_layout.h"
#include "ptx.cuh"

namespace fdmoe {
namespace {

constexpr int kPgStages = 6;
constexpr int kPgStageA = 128 * 64 * 2;  // 16 KB: 128 W rows x 64 k
constexpr int kPgStageB = 128 * 64 * 2;  // up to 128 X rows x 64 k
constexpr int kPgStageBytes = kPgStageA + kPgStageB;
constexpr uint64_t kPgTimeoutNs = 200000000ull;  // every wait gives up after 0.2 s

struct PgCtl {
  uint64_t full_bar[kPgStages];   // used in the even CTA only: both CTAs' loads land
  uint64_t empty_bar[kPgStages];  // per CTA: the MMAs have read this CTA's stage
  uint64_t tmem_full;             // per CTA: the accumulator is complete
  uint32_t tmem_base;
  volatile uint32_t abort;
};

__device__ __forceinline__ bool pg_wait(PgCtl& c, uint64_t* bar, uint32_t parity, uint32_t* status, uint32_t code) {
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (!ptx::mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (c.abort) return false;
      if (ptx::globaltimer_ns() - t0 > kPgTimeoutNs) {
        c.abort = 1u;
        atomicCAS(status, 0u, code | (blockIdx.x << 8));
        return false;
      }
    }
  }
  return true;
}

__global__ void __launch_bounds__(128, 1)
pair_gemm_kernel(const __grid_constant__ FdmoeTensorMap tm_w, const __grid_constant__ FdmoeTensorMap tm_x,
                 float* __restrict__ D, int N, int K, int box_rows, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* stage = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  PgCtl& c = *reinterpret_cast<PgCtl*>(stage + kPgStages * kPgStageBytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t cta = ptx::cluster_ctarank();  // 0 = the CTA that issues the MMAs
  const int nhalf = N / 2;
  const uint32_t nkb = (uint32_t)(K / 64);

  if (tid == 0) {
    for (int s = 0; s < kPgStages; ++s) {
      ptx::mbar_init(&c.full_bar[s], 1);  // the even CTA's arrival, which announces the bytes of both
      ptx::mbar_init(&c.empty_bar[s], 1);
    }
    ptx::mbar_init(&c.tmem_full, 1);
    c.abort = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc2(&c.tmem_base, 256);
    ptx::tmem_relinquish2();
  }
  ptx::tcgen05_fence_before();
  ptx::cluster_sync();  // barriers of both CTAs are initialised before anyone signals them
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = c.tmem_base;

  if (warp == 0 && lane == 0) {
    // producer: this CTA's share of both operands, completion counted on the even CTA's barrier
    const uint32_t pair_bytes = 2u * (uint32_t)(128 + nhalf) * 64u * 2u;
    for (uint32_t kb = 0; kb < nkb; ++kb) {
      const uint32_t s = kb % kPgStages, ph = (kb / kPgStages) & 1u;
      if (!pg_wait(c, &c.empty_bar[s], ph ^ 1u, status, 1u)) break;
      const uint32_t full0 = ptx::map_to_cta(ptx::smem_u32(&c.full_bar[s]), 0u);
      if (cta == 0u) ptx::mbar_expect_tx(&c.full_bar[s], pair_bytes);
      uint8_t* sa = stage + s * kPgStageBytes;
      ptx::tma_load_2d_pair(sa, &tm_w, full0, (int32_t)(kb * 64u), (int32_t)(cta * 128u));
      for (int r = 0; r < nhalf; r += box_rows)
        ptx::tma_load_2d_pair(sa + kPgStageA + r * 128, &tm_x, full0, (int32_t)(kb * 64u), (int32_t)cta * nhalf + r);
    }
  } else if (warp == 1 && lane == 0 && cta == 0) {
    const uint32_t idesc = ptx::make_idesc_bf16(256, (uint32_t)N);
    bool ok = true;
    const uint64_t t_begin = ptx::globaltimer_ns();
    for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
      const uint32_t s = kb % kPgStages, ph = (kb / kPgStages) & 1u;
      ok = pg_wait(c, &c.full_bar[s], ph, status, 2u);
      if (!ok) break;
      ptx::tcgen05_fence_after();
      const uint32_t sa = ptx::smem_u32(stage + s * kPgStageBytes);
      const uint64_t da = ptx::make_smem_desc_sw128(sa), db = ptx::make_smem_desc_sw128(sa + kPgStageA);
#pragma unroll
      for (uint32_t k4 = 0; k4 < 4; ++k4) ptx::umma_bf16_pair(tmem_base, da + k4 * 2u, db + k4 * 2u, idesc, (kb | k4) != 0u);
      // the stage is free in both CTAs once these MMAs have read it
      ptx::umma_commit_pair(ptx::smem_u32(&c.empty_bar[s]));
      ptx::umma_commit_pair(ptx::map_to_cta(ptx::smem_u32(&c.empty_bar[s]), 1u));
    }
    if (ok) {
      ptx::umma_commit_pair(ptx::smem_u32(&c.tmem_full));
      ptx::umma_commit_pair(ptx::map_to_cta(ptx::smem_u32(&c.tmem_full), 1u));
      if (blockIdx.x == 0) status[1] = (uint32_t)(ptx::globaltimer_ns() - t_begin);  // main loop, first wait to last issue
    }
  }
  __syncwarp();

  // epilogue: warp w reads lanes [32w, 32w + 32) of this CTA's accumulator
  bool ok = pg_wait(c, &c.tmem_full, 0u, status, 3u);
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    ptx::tcgen05_fence_after();
    const int row = (int)cta * 128 + warp * 32 + lane;
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t v[32];
      ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (c0 + i < N) D[(size_t)row * N + c0 + i] = __uint_as_float(v[i]);
    }
  }
  ptx::tcgen05_fence_before();
  ptx::cluster_sync();  // nobody frees tensor memory or leaves while its partner may still signal it
  if (warp == 2) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc2(tmem_base, 256);
  }
}

}  // namespace
}  // namespace fdmoe

extern "C" int FlashMoeTestPairGemm(const void* W, const void* X, float* D, int N, int K, int boxRows,
                                    unsigned* mainLoopNs, void* stream_) {
  using namespace fdmoe;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!W || !X || !D || N < 16 || N > 256 || N % 16 != 0 || K < 64 || K % 64 != 0 || boxRows < 8 || boxRows % 8 != 0 ||
      (N / 2) % boxRows != 0)
    return (int)cudaErrorInvalidValue;
  EncodeTiledFn enc = GetEncodeTiled();
  if (!enc) return (int)cudaErrorUnknown;
  FdmoeTensorMap tm_w, tm_x;
  cudaError_t e = MakeTensorMap(enc, &tm_w, W, 256, (uint64_t)K, 128);
  if (e != cudaSuccess) return (int)e;
  e = MakeTensorMap(enc, &tm_x, X, (uint64_t)N, (uint64_t)K, (uint32_t)boxRows);
  if (e != cudaSuccess) return (int)e;
  const int smem = kPgStages * kPgStageBytes + (int)sizeof(PgCtl) + 1024;
  e = cudaFuncSetAttribute(pair_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  uint32_t* status = nullptr;
  e = cudaMalloc(reinterpret_cast<void**>(&status), 8);
  if (e != cudaSuccess) return (int)e;
  cudaMemsetAsync(status, 0, 8, stream);
  cudaLaunchConfig_t cfg = {};
  // (experiments) several clusters computing the same product, to load the memory system
  const char* nc = getenv("FLASHMOE_PAIR_CLUSTERS");
  const int clusters = nc ? atoi(nc) : 1;
  cfg.gridDim = dim3(2 * (clusters > 0 ? clusters : 1), 1, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, pair_gemm_kernel, tm_w, tm_x, D, N, K, boxRows, status);
  uint32_t hs2[2] = {0, 0};
  if (e == cudaSuccess) e = cudaMemcpyAsync(hs2, status, 8, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  cudaFree(status);
  if (e != cudaSuccess) return (int)e;
  const uint32_t hs = hs2[0];
  if (mainLoopNs) *mainLoopNs = hs2[1];
  if (hs != 0) {
    MOE_ERROR_LOG("pair GEMM self-test: a bounded wait ran out (code 0x%x)", hs);
    return (int)cudaErrorUnknown;
  }
  return 0;
}
