// FlashMoeLaunchNoAlloc: the MoE layer for callers that must not allocate.
//
// Some hosts of this library run in places where device allocation is off
// limits: inside a serving engine after it has frozen its memory pool (a later
// cudaMalloc would fragment or exceed the budget it planned), inside callbacks
// that may not call allocating runtime functions, or in processes whose memory
// is fully handed to another allocator.  For them this one entry point runs the
// same persistent kernel as IMoeKernelLauncher::Launch, but takes every byte of
// scratch (work queue, counters, row sidebands, packed rows, activations,
// weighted rows) from one fixed array that lives in the library image.
//
// Limits and rules, all checked or documented here:
//   * single rank, bf16 tensors, tokensNum >= 0;
//   * the scratch of the call must fit kScratchBytes (32 MiB); larger layers or
//     batches are rejected with cudaErrorInvalidValue and a message.  Every GPU
//     on which this library is loaded holds those 32 MiB until the process ends;
//   * the first call on a device resolves the array's device address and raises
//     the kernel's shared-memory limit; with lazy module loading it may also be
//     the moment the 32 MiB become resident on that device.  Make that first call
//     early: before any stream capture and before the host freezes its memory
//     budget;
//   * every call uses the same array and begins by clearing the part of it that
//     has to start from zero (queue, counters, status).  Two calls that overlap
//     on the GPU (different streams, or threads) would corrupt each other: keep
//     calls on one device ordered;
//   * the call returns after the layer has finished (it synchronises `stream`
//     to read the device-side status word); a device-side timeout is reported as
//     cudaErrorUnknown;
//   * no cudaMalloc / cudaFree / cudaHostAlloc, no torch allocator, nothing that
//     allocates is called on any path of this function.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <mutex>

#include "../../include/flashmoe_c.h"
#include "host_layout.h"
#include "moe_types.h"

namespace {

constexpr size_t kScratchBytes = 32u << 20;

// The scratch itself.  In host code this name is only a handle for
// cudaGetSymbolAddress: it is NOT a device pointer and must never be passed to a
// kernel or to cudaMemset as if it were one.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
struct PerDevice {
  unsigned char* base = nullptr;  // device address of g_no_alloc_scratch on this device
  int grid = 0;
  fdmoe::EncodeTiledFn encode = nullptr;
};
PerDevice g_dev[kMaxDevices];
std::mutex g_mutex;

#define NA_CHECK(expr)                                                                              \
  do {                                                                                              \
    const cudaError_t _e = static_cast<cudaError_t>(expr);                                          \
    if (_e != cudaSuccess) {                                                                        \
      fprintf(stderr, "[MOE CUDA ERROR: %s:%d] %s\n", __FILE__, __LINE__, cudaGetErrorString(_e)); \
      return (int)_e;                                                                               \
    }                                                                                               \
  } while (0)

// Once per device, with that device current: device address of the array, kernel
// attributes, driver entry point for the TMA descriptors.
int SetUpDevice(int dev, PerDevice** out) {
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  PerDevice& d = g_dev[dev];
  if (!d.base) {
    void* ptr = nullptr;
    NA_CHECK(cudaGetSymbolAddress(&ptr, g_no_alloc_scratch));
    int smem = 0, grid = 0;
    NA_CHECK(fdmoe_kernel_prepare(&smem, &grid));
    d.encode = fdmoe::GetEncodeTiled();
    if (!d.encode) {
      MOE_ERROR_LOG("cuTensorMapEncodeTiled is not available from this driver");
      return (int)cudaErrorUnknown;
    }
    d.grid = grid;
    d.base = static_cast<unsigned char*>(ptr);
  }
  *out = &d;
  return 0;
}

}  // namespace

extern "C" int FlashMoeLaunchNoAlloc(const void* gateWeights, const void* ffn1ExpertWeights,
                                     const void* ffn2ExpertWeights, const void* tokens, void* output,
                                     int tokensNum, const FlashMoeConfig* config, void* stream_) {
  using namespace fdmoe;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  FlashMoeConfig cfg = {2048, 768, 128, 8, 0, {0, 0, 0}};  // Qwen3-30B-A3B layer, as CreateLauncher
  if (config) cfg = *config;
  if (cfg.dtype != 0 || cfg.hiddenSize <= 0 || cfg.hiddenSize % FDMOE_TILE_N2 != 0 ||
      cfg.hiddenSize > FDMOE_MAX_HIDDEN || cfg.expertIntermediateSize <= 0 ||
      cfg.expertIntermediateSize % FDMOE_TILE_N1 != 0 || cfg.expertsNum <= 0 ||
      cfg.expertsNum > FDMOE_MAX_EXPERTS || cfg.topk <= 0 || cfg.topk > FDMOE_MAX_TOPK ||
      cfg.topk > cfg.expertsNum) {
    MOE_ERROR_LOG("FlashMoeLaunchNoAlloc: unsupported layer (bf16 only) H=%d I=%d E=%d K=%d dtype=%d",
                  cfg.hiddenSize, cfg.expertIntermediateSize, cfg.expertsNum, cfg.topk, cfg.dtype);
    return (int)cudaErrorInvalidValue;
  }
  if (tokensNum < 0 || !gateWeights || !ffn1ExpertWeights || !ffn2ExpertWeights ||
      (tokensNum > 0 && (!tokens || !output)))
    return (int)cudaErrorInvalidValue;

  int dev = 0;
  NA_CHECK(cudaGetDevice(&dev));
  PerDevice* d = nullptr;
  {
    // the lock covers the one-time set-up only: every device has its own copy of the array, and
    // keeping calls on one device apart is the caller's duty
    std::lock_guard<std::mutex> lock(g_mutex);
    const int rc = SetUpDevice(dev, &d);
    if (rc != 0) return rc;
  }

  // ---- geometry of this call (same rules as the launcher's Init, world size 1)
  Geometry g;
  g.H = cfg.hiddenSize;
  g.I = cfg.expertIntermediateSize;
  g.E = cfg.expertsNum;
  g.K = cfg.topk;
  g.El = g.E;
  g.world = 1;
  g.max_tokens_local = g.max_tokens_max = std::max(tokensNum, 1);
  g.max_tokens_sum = g.max_tokens_max;
  g.combine_group = 8;
  if (!FinishGeometry(g, d->grid)) return (int)cudaErrorInvalidValue;
  const ArenaLayout L = MakeLayout(g);
  // regions the launcher allocates separately follow the arena inside the same array
  size_t off = AlignUp(L.total, 1024);
  const size_t off_act = off;
  off += AlignUp((size_t)g.El * g.cap_rows * g.I * 2, 1024);
  const size_t off_idx = off;
  off += AlignUp((size_t)g.max_tokens_max * g.K * 4, 256);
  const size_t off_w = off;
  off += AlignUp((size_t)g.max_tokens_max * g.K * 4, 256);
  const size_t off_dst = off;
  off += AlignUp((size_t)g.max_tokens_max, 256);
  if (off > kScratchBytes) {
    MOE_ERROR_LOG("FlashMoeLaunchNoAlloc: this call needs %zu bytes of scratch, the fixed array holds %zu "
                  "(H=%d I=%d E=%d K=%d tokens=%d); use CreateLauncher/Launch for larger problems",
                  off, kScratchBytes, g.H, g.I, g.E, g.K, tokensNum);
    return (int)cudaErrorInvalidValue;
  }

  unsigned char* base = d->base;
  // everything that must start from zero: control block, counters, queue slots
  // (their sequence words), row sidebands; the row payload regions are fully
  // written before they are read
  NA_CHECK(cudaMemsetAsync(base, 0, L.ystage, stream));

  FdmoeParams p;
  memset(&p, 0, sizeof(p));
  const uint64_t exp_rows = (uint64_t)g.El * g.cap_rows;
  NA_CHECK(MakeTensorMap(d->encode, &p.tm_packed, base + L.packed, exp_rows, g.H, 128));
  NA_CHECK(MakeTensorMap(d->encode, &p.tm_w13, ffn1ExpertWeights, (uint64_t)g.El * 2 * g.I, g.H, 128));
  NA_CHECK(MakeTensorMap(d->encode, &p.tm_act, base + off_act, exp_rows, g.I, 128));
  NA_CHECK(MakeTensorMap(d->encode, &p.tm_w2, ffn2ExpertWeights, (uint64_t)g.El * g.H, g.I, 256));
  NA_CHECK(MakeTensorMap(d->encode, &p.tm_gate, gateWeights, (uint64_t)g.E, g.H, std::min(128, g.E)));
  p.gate_rows = tokensNum <= 32 * d->grid ? 32 : (tokensNum <= 64 * d->grid ? 64 : 128);
  if (tokensNum > 0)
    NA_CHECK(MakeTensorMap(d->encode, &p.tm_x, tokens, (uint64_t)tokensNum, g.H, std::min(p.gate_rows, tokensNum)));
  FdmoePeer& me = p.peers[0];
  me.ctl = reinterpret_cast<FdmoeCtl*>(base + L.ctl);
  me.slots[0] = reinterpret_cast<FdmoeSlot*>(base + L.slots[0]);
  me.slots[1] = reinterpret_cast<FdmoeSlot*>(base + L.slots[1]);
  me.slots[2] = reinterpret_cast<FdmoeSlot*>(base + L.slots[2]);
  me.expert_cnt = reinterpret_cast<uint32_t*>(base + L.expert_cnt);
  me.landed = reinterpret_cast<uint32_t*>(base + L.landed);
  me.grp_cnt = reinterpret_cast<uint32_t*>(base + L.grp_cnt);
  me.packed = base + L.packed;
  me.meta = reinterpret_cast<FdmoeRowMeta*>(base + L.meta);
  me.ystage = base + L.ystage;
  p.H = g.H;
  p.I = g.I;
  p.E = g.E;
  p.K = g.K;
  p.El = g.El;
  p.world = 1;
  p.rank = 0;
  p.T = tokensNum;
  p.cap_rows = g.cap_rows;
  p.MT = g.MT;
  p.queue_mask = (int32_t)(g.queue_cap - 1);
  p.combine_group = g.combine_group;
  p.mode = 0;
  p.epoch = 1;
  p.disp_conc = d->grid;
  p.batch_mt = 0;
  p.timeout_ns = 2000ull * 1000000ull;
  p.peer_timeout_ns = p.timeout_ns;
  p.x = tokens;
  p.out = output;
  p.gate_w = gateWeights;
  p.act = base + off_act;
  p.topk_idx = reinterpret_cast<int32_t*>(base + off_idx);
  p.topk_w = reinterpret_cast<float*>(base + off_w);
  p.tok_flag = base + off_dst;
  p.ffn1_done = reinterpret_cast<uint32_t*>(base + L.ffn1_done);
  p.ffn2_done = reinterpret_cast<uint32_t*>(base + L.ffn2_done);
  NA_CHECK(fdmoe_kernel_launch(&p, d->grid, stream));

  // the device-side status word lives in the control block: read it back
  NA_CHECK(cudaStreamSynchronize(stream));
  uint32_t status[2] = {0, 0};
  NA_CHECK(cudaMemcpy(status, base + L.ctl + offsetof(FdmoeCtl, status), sizeof(status), cudaMemcpyDeviceToHost));
  if (status[0] != 0) {
    MOE_ERROR_LOG("FlashMoeLaunchNoAlloc: device-side error %u (info 0x%x)", status[0], status[1]);
    return (int)cudaErrorUnknown;
  }
  return 0;
}
