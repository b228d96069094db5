// Host launcher of the B200 MoE layer: owns the scratch memory, the symmetric
// arena that peers write into, the TMA descriptors and the per-launch reset,
// and starts the one persistent kernel per Launch.  Talks to CUDA device code
// only through the thin C ABI declared in moe_types.h.
//
// Reference counterparts: src/hip/launcher/moeKernelLauncher.hip:58-93 (launch),
// :96-187 (Init), :190-204 (Deinit), src/moeKernelLauncher.cpp:15-55 (C shims),
// src/hip/kernel/remote/remoteComManager.h:33-87 (multi-rank bring-up).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <vector>

#include "../../include/flashmoe_c.h"
#include "../../include/iMoeKernelLauncher.h"
#include "bootstrap.h"
#include "host_layout.h"
#include "moe_types.h"

#undef MOE_ERROR_LOG
#define MOE_ERROR_LOG(...)                                   \
  do {                                                       \
    fprintf(stderr, "[MOE ERROR: %s:%d] ", __FILE__, __LINE__); \
    fprintf(stderr, __VA_ARGS__);                            \
    fprintf(stderr, "\n");                                   \
  } while (0)

// Propagates a CUDA error code, printing where it happened (same convention as
// the reference's HIP_ERROR_CHECK, src/hip/hipHostCommon.h:11-19).
#define CUDA_ERROR_CHECK(expr)                                                      \
  do {                                                                              \
    const cudaError_t _e = static_cast<cudaError_t>(expr);                          \
    if (_e != cudaSuccess) {                                                        \
      fprintf(stderr, "[MOE CUDA ERROR: %s:%d] %s\n", __FILE__, __LINE__, cudaGetErrorString(_e)); \
      return _e;                                                                    \
    }                                                                               \
  } while (0)

namespace moe {
IMoeKernelLauncher::~IMoeKernelLauncher() {}
}  // namespace moe

namespace fdmoe {
namespace {

int EnvInt(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

}  // namespace

class MoeKernelLauncher final : public moe::IMoeKernelLauncher {
 public:
  MoeKernelLauncher() = default;
  ~MoeKernelLauncher() override {}

  cudaError_t Init(const void* gateW, const void* w13, const void* w2, int maxTokens, cudaStream_t stream,
                   const moe::DistributedUniqueId& uid, int rank, int world, const moe::MoeConfig& cfg);
  cudaError_t Deinit(cudaStream_t stream);
  cudaError_t Launch(const void* tokens, void* output, int tokensNum, cudaStream_t stream) override;
  cudaError_t LaunchHost(const void* hostTokens, void* hostOutput, int tokensNum, cudaStream_t stream);
  cudaError_t DebugRead(int which, void* dst, size_t offset, size_t bytes);
  cudaError_t TestTaskSystem(int32_t* data, int n, cudaStream_t stream);
  cudaError_t TestQueueGemm(const uint32_t* rowsPerExpert, const void* A, void* out, cudaStream_t stream);
  cudaError_t TestStall(cudaStream_t stream);
  void LastStatus(uint32_t* code, uint32_t* info) const {
    if (code) *code = status_host_ ? status_host_[0] : 0;
    if (info) *info = status_host_ ? status_host_[1] : 0;
  }

 private:
  cudaError_t LaunchBf16(const void* tokens, void* output, int tokensNum, cudaStream_t stream, int mode,
                         uint32_t expected_static);
  cudaError_t LaunchDevice(const void* tokens, void* output, int tokensNum, cudaStream_t stream);
  cudaError_t PrefillTasks(const std::vector<FdmoeSlot>& tasks, cudaStream_t stream);
  void FreeAll();

  Geometry g_;
  ArenaLayout layout_;
  int rank_ = 0, world_ = 1, dtype_ = moe::MOE_DTYPE_BF16;
  int grid_ = 0, smem_ = 0;
  uint32_t epoch_ = 0;
  FdmoeParams params_;
  uint8_t* arena_ = nullptr;
  std::vector<void*> peer_bases_;  // mapped peer arenas (peer_bases_[rank_] == arena_)
  void* act_ = nullptr;
  int32_t* topk_idx_ = nullptr;
  float* topk_w_ = nullptr;
  uint8_t* tok_flag_ = nullptr;  // per token: routed by a GATEFIX task
  uint32_t* status_host_ = nullptr;
  uint32_t* status_dev_ = nullptr;
  // fp32 I/O mode: bf16 copies of the weights and token staging
  void *gate_bf16_ = nullptr, *w13_bf16_ = nullptr, *w2_bf16_ = nullptr;
  void *tok_bf16_ = nullptr, *out_bf16_ = nullptr;
  // host-buffer entry point staging
  // Two sets of device staging buffers and three internal streams (copy in, layer, copy out), so
  // that consecutive calls overlap one call's copies with the other's kernel.
  struct HostPipe {
    void* in[2] = {nullptr, nullptr};
    void* out[2] = {nullptr, nullptr};
    cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
    cudaEvent_t copied_in[2] = {nullptr, nullptr}, ran[2] = {nullptr, nullptr}, copied_out[2] = {nullptr, nullptr};
    cudaEvent_t direct = nullptr;  // last Launch() made directly on a caller's stream
    bool direct_pending = false;
    uint64_t calls = 0;
    bool ready = false;
  } pipe_;
  cudaError_t InitHostPipe();
  void DestroyHostPipe();
  uint32_t* prof_ = nullptr;  // optional event trace (FLASHMOE_PROFILE=1)
  uint32_t* stuck_ = nullptr;  // per CTA and warp: where a role gave up waiting
  float* debug_logits_ = nullptr;  // optional gate-logit dump (FLASHMOE_DEBUG_LOGITS=1)
  EncodeTiledFn encode_ = nullptr;
  Bootstrap boot_;
  bool inited_ = false;
};

void MoeKernelLauncher::FreeAll() {
  for (int r = 0; r < (int)peer_bases_.size(); ++r)
    if (r != rank_ && peer_bases_[r]) cudaIpcCloseMemHandle(peer_bases_[r]);
  peer_bases_.clear();
  void* ptrs[] = {arena_, act_, topk_idx_, topk_w_, tok_flag_, gate_bf16_, w13_bf16_, w2_bf16_,
                  tok_bf16_, out_bf16_, pipe_.in[0], pipe_.in[1], pipe_.out[0], pipe_.out[1], prof_, debug_logits_,
                  stuck_};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  arena_ = nullptr;
  act_ = nullptr;
  topk_idx_ = nullptr;
  topk_w_ = nullptr;
  tok_flag_ = nullptr;
  gate_bf16_ = w13_bf16_ = w2_bf16_ = tok_bf16_ = out_bf16_ = nullptr;
  pipe_.in[0] = pipe_.in[1] = pipe_.out[0] = pipe_.out[1] = nullptr;
  prof_ = nullptr;
  debug_logits_ = nullptr;
  stuck_ = nullptr;
  if (status_host_) cudaFreeHost(status_host_);
  status_host_ = nullptr;
  boot_.Close();
}

cudaError_t MoeKernelLauncher::Init(const void* gateW, const void* w13, const void* w2, int maxTokens,
                                    cudaStream_t stream, const moe::DistributedUniqueId& uid, int rank,
                                    int world, const moe::MoeConfig& cfg) {
  // ---- argument and capacity checks: no CUDA call, nothing dereferenced
  if (world < 1 || world > FDMOE_MAX_WORLD || rank < 0 || rank >= world) {
    MOE_ERROR_LOG("bad rank/world %d/%d (world size 1..%d)", rank, world, FDMOE_MAX_WORLD);
    return cudaErrorInvalidValue;
  }
  if (cfg.hiddenSize <= 0 || cfg.hiddenSize % FDMOE_TILE_N2 != 0 || cfg.hiddenSize > FDMOE_MAX_HIDDEN || cfg.expertIntermediateSize <= 0 ||
      cfg.expertIntermediateSize % FDMOE_TILE_N1 != 0 || cfg.expertsNum <= 0 ||
      cfg.expertsNum > FDMOE_MAX_EXPERTS || cfg.expertsNum % world != 0 || cfg.topk <= 0 ||
      cfg.topk > FDMOE_MAX_TOPK || cfg.topk > cfg.expertsNum ||
      (cfg.dtype != moe::MOE_DTYPE_BF16 && cfg.dtype != moe::MOE_DTYPE_FP32)) {
    MOE_ERROR_LOG("unsupported layer shape H=%d I=%d E=%d K=%d dtype=%d world=%d", cfg.hiddenSize,
                  cfg.expertIntermediateSize, cfg.expertsNum, cfg.topk, cfg.dtype, world);
    return cudaErrorInvalidValue;
  }
  if (maxTokens < 0) return cudaErrorInvalidValue;
  // Capacity: the token-indexed and expert-indexed scratch must fit the budget
  // (FLASHMOE_MAX_SCRATCH_GB, default 64).  Like the reference's queue-capacity
  // check this comes before any pointer is looked at and reports cudaErrorUnknown.
  {
    const double budget = (double)EnvInt("FLASHMOE_MAX_SCRATCH_GB", 64) * 1e9;
    const double rows = (double)maxTokens * world;
    const double need = rows * (cfg.expertsNum / world) * (cfg.hiddenSize + cfg.expertIntermediateSize) * 2.0 +
                        (double)maxTokens * cfg.topk * cfg.hiddenSize * 2.0;
    if (need > budget) {
      MOE_ERROR_LOG("maxTokens=%d needs %.1f GB of scratch, budget is %.1f GB", maxTokens, need / 1e9,
                    budget / 1e9);
      return cudaErrorUnknown;
    }
  }
  if (!gateW || !w13 || !w2) {
    MOE_ERROR_LOG("null weight pointer");
    return cudaErrorUnknown;
  }

  rank_ = rank;
  world_ = world;
  dtype_ = cfg.dtype;
  g_.H = cfg.hiddenSize;
  g_.I = cfg.expertIntermediateSize;
  g_.E = cfg.expertsNum;
  g_.K = cfg.topk;
  g_.world = world;
  g_.El = g_.E / world;
  g_.max_tokens_local = maxTokens;

  CUDA_ERROR_CHECK(fdmoe_kernel_prepare(&smem_, &grid_));
  const int grid_env = EnvInt("FLASHMOE_GRID", 0);
  if (grid_env > 0 && grid_env < grid_) grid_ = grid_env;

  // ---- multi-rank bring-up: exchange sizes, then IPC handles of the arenas
  if (world > 1) {
    if (boot_.Init(uid.data, rank, world, EnvInt("FLASHMOE_BOOTSTRAP_TIMEOUT_MS", 30000)) != 0) {
      MOE_ERROR_LOG("multi-rank bootstrap failed (rank %d of %d)", rank, world);
      FreeAll();
      return cudaErrorUnknown;
    }
  }
  struct Hello {
    int32_t H, I, E, K, dtype, max_tokens;
  } mine = {g_.H, g_.I, g_.E, g_.K, dtype_, maxTokens};
  std::vector<Hello> all((size_t)world);
  if (boot_.AllGather(&mine, all.data(), sizeof(mine)) != 0) {
    FreeAll();
    return cudaErrorUnknown;
  }
  g_.max_tokens_max = 0;
  g_.max_tokens_sum = 0;
  for (const Hello& h : all) {
    if (h.H != g_.H || h.I != g_.I || h.E != g_.E || h.K != g_.K || h.dtype != dtype_) {
      MOE_ERROR_LOG("ranks disagree about the layer shape");
      FreeAll();
      return cudaErrorUnknown;
    }
    g_.max_tokens_max = std::max(g_.max_tokens_max, h.max_tokens);
    g_.max_tokens_sum += h.max_tokens;
  }
  g_.combine_group = std::max(1, EnvInt("FLASHMOE_COMBINE_GROUP", 8));
  if (!FinishGeometry(g_, grid_)) {
    MOE_ERROR_LOG("maxTokens=%d: more expert-buffer rows than a dispatch word can address", maxTokens);
    FreeAll();
    return cudaErrorUnknown;
  }
  layout_ = MakeLayout(g_);

  // ---- allocations
  CUDA_ERROR_CHECK(cudaMalloc(reinterpret_cast<void**>(&arena_), layout_.total));
  CUDA_ERROR_CHECK(cudaMemsetAsync(arena_, 0, layout_.packed, stream));  // everything but the row payload
  CUDA_ERROR_CHECK(cudaMalloc(&act_, (size_t)g_.El * g_.cap_rows * g_.I * 2));
  CUDA_ERROR_CHECK(cudaMalloc(reinterpret_cast<void**>(&topk_idx_), std::max<size_t>(4, (size_t)maxTokens * g_.K * 4)));
  CUDA_ERROR_CHECK(cudaMalloc(reinterpret_cast<void**>(&topk_w_), std::max<size_t>(4, (size_t)maxTokens * g_.K * 4)));
  CUDA_ERROR_CHECK(cudaMalloc(reinterpret_cast<void**>(&tok_flag_), std::max<size_t>(16, (size_t)maxTokens)));
  CUDA_ERROR_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), 64, cudaHostAllocMapped));
  memset(status_host_, 0, 64);
  CUDA_ERROR_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev_), status_host_, 0));

  const void* gate_dev = gateW;
  const void* w13_dev = w13;
  const void* w2_dev = w2;
  if (dtype_ == moe::MOE_DTYPE_FP32) {
    const uint64_t n_gate = (uint64_t)g_.E * g_.H, n13 = (uint64_t)g_.El * 2 * g_.I * g_.H,
                   n2 = (uint64_t)g_.El * g_.H * g_.I;
    CUDA_ERROR_CHECK(cudaMalloc(&gate_bf16_, n_gate * 2));
    CUDA_ERROR_CHECK(cudaMalloc(&w13_bf16_, n13 * 2));
    CUDA_ERROR_CHECK(cudaMalloc(&w2_bf16_, n2 * 2));
    CUDA_ERROR_CHECK(cudaMalloc(&tok_bf16_, std::max<size_t>(16, (size_t)maxTokens * g_.H * 2)));
    CUDA_ERROR_CHECK(cudaMalloc(&out_bf16_, std::max<size_t>(16, (size_t)maxTokens * g_.H * 2)));
    CUDA_ERROR_CHECK(fdmoe_cast_f32_to_bf16(static_cast<const float*>(gateW), gate_bf16_, n_gate, stream));
    CUDA_ERROR_CHECK(fdmoe_cast_f32_to_bf16(static_cast<const float*>(w13), w13_bf16_, n13, stream));
    CUDA_ERROR_CHECK(fdmoe_cast_f32_to_bf16(static_cast<const float*>(w2), w2_bf16_, n2, stream));
    gate_dev = gate_bf16_;
    w13_dev = w13_bf16_;
    w2_dev = w2_bf16_;
  }

  // ---- map the peers' arenas
  peer_bases_.assign((size_t)world, nullptr);
  peer_bases_[rank] = arena_;
  if (world > 1) {
    cudaIpcMemHandle_t mine_h;
    CUDA_ERROR_CHECK(cudaIpcGetMemHandle(&mine_h, arena_));
    std::vector<cudaIpcMemHandle_t> handles((size_t)world);
    if (boot_.AllGather(&mine_h, handles.data(), sizeof(mine_h)) != 0) {
      FreeAll();
      return cudaErrorUnknown;
    }
    for (int r = 0; r < world; ++r) {
      if (r == rank) continue;
      const cudaError_t e = cudaIpcOpenMemHandle(&peer_bases_[r], handles[r], cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        MOE_ERROR_LOG("rank %d cannot map the arena of rank %d: %s (peer access over NVLink is required)",
                      rank, r, cudaGetErrorString(e));
        FreeAll();
        return cudaErrorUnknown;
      }
    }
  }

  // ---- kernel parameters that do not change between launches
  memset(&params_, 0, sizeof(params_));
  EncodeTiledFn enc = GetEncodeTiled();
  if (!enc) {
    MOE_ERROR_LOG("cuTensorMapEncodeTiled is not available from this driver");
    FreeAll();
    return cudaErrorUnknown;
  }
  const uint64_t exp_rows = (uint64_t)g_.El * g_.cap_rows;
  CUDA_ERROR_CHECK(MakeTensorMap(enc, &params_.tm_packed, arena_ + layout_.packed, exp_rows, g_.H, 128));
  CUDA_ERROR_CHECK(MakeTensorMap(enc, &params_.tm_w13, w13_dev, (uint64_t)g_.El * 2 * g_.I, g_.H, 128));
  CUDA_ERROR_CHECK(MakeTensorMap(enc, &params_.tm_act, act_, exp_rows, g_.I, 128));
  CUDA_ERROR_CHECK(MakeTensorMap(enc, &params_.tm_w2, w2_dev, (uint64_t)g_.El * g_.H, g_.I, 256));
  CUDA_ERROR_CHECK(MakeTensorMap(enc, &params_.tm_gate, gate_dev, (uint64_t)g_.E, g_.H, std::min(128, g_.E)));
  encode_ = enc;
  for (int r = 0; r < world; ++r) {
    uint8_t* b = static_cast<uint8_t*>(peer_bases_[r]);
    FdmoePeer& pv = params_.peers[r];
    pv.ctl = reinterpret_cast<FdmoeCtl*>(b + layout_.ctl);
    pv.slots[0] = reinterpret_cast<FdmoeSlot*>(b + layout_.slots[0]);
    pv.slots[1] = reinterpret_cast<FdmoeSlot*>(b + layout_.slots[1]);
    pv.slots[2] = reinterpret_cast<FdmoeSlot*>(b + layout_.slots[2]);
    pv.expert_cnt = reinterpret_cast<uint32_t*>(b + layout_.expert_cnt);
    pv.landed = reinterpret_cast<uint32_t*>(b + layout_.landed);
    pv.grp_cnt = reinterpret_cast<uint32_t*>(b + layout_.grp_cnt);
    pv.packed = b + layout_.packed;
    pv.meta = reinterpret_cast<FdmoeRowMeta*>(b + layout_.meta);
    pv.ystage = b + layout_.ystage;
  }
  params_.H = g_.H;
  params_.I = g_.I;
  params_.E = g_.E;
  params_.K = g_.K;
  params_.El = g_.El;
  params_.world = world;
  params_.rank = rank;
  params_.cap_rows = g_.cap_rows;
  params_.MT = g_.MT;
  params_.queue_mask = (int32_t)(g_.queue_cap - 1);
  params_.combine_group = g_.combine_group;
  params_.gate_rows = 128;  // per launch: 32, 64 or 128 by token count
  // Two budgets for device-side waits.  Inside a launch every wait (queue, pipeline stage,
  // accumulator) gives up after FLASHMOE_TIMEOUT_MS.  The wait for the peers to enter a launch has a
  // budget of its own: ranks reach a collective Launch as far apart as their hosts let them (uneven
  // batches, host work between steps, a first-call warm-up), which says nothing about a fault.
  params_.timeout_ns = (uint64_t)std::max(1, EnvInt("FLASHMOE_TIMEOUT_MS", 2000)) * 1000000ull;
  params_.peer_timeout_ns = (uint64_t)std::max(1, EnvInt("FLASHMOE_PEER_TIMEOUT_MS", 60000)) * 1000000ull;
  // DISPATCH tasks worked on at a time (0 = chosen per launch, see LaunchBf16), and m-tiles per
  // publication batch (0 = chosen per launch from the token counts).
  params_.disp_conc = std::max(0, EnvInt("FLASHMOE_DISPATCH_WORKERS", 0));
  params_.batch_mt = std::max(0, EnvInt("FLASHMOE_BATCH_MT", 0));
  params_.gate_w = gate_dev;
  params_.act = act_;
  params_.topk_idx = topk_idx_;
  params_.topk_w = topk_w_;
  params_.tok_flag = tok_flag_;
  params_.ffn1_done = reinterpret_cast<uint32_t*>(arena_ + layout_.ffn1_done);
  params_.ffn2_done = reinterpret_cast<uint32_t*>(arena_ + layout_.ffn2_done);
  params_.status_host = status_dev_;
  {
    const size_t bytes = (size_t)grid_ * 16 * 16;
    CUDA_ERROR_CHECK(cudaMalloc(reinterpret_cast<void**>(&stuck_), bytes));
    CUDA_ERROR_CHECK(cudaMemsetAsync(stuck_, 0, bytes, stream));
    params_.stuck = stuck_;
  }
  if (EnvInt("FLASHMOE_DEBUG_LOGITS", 0)) {
    CUDA_ERROR_CHECK(cudaMalloc(reinterpret_cast<void**>(&debug_logits_), std::max<size_t>(4, (size_t)maxTokens * 128 * 4)));
    params_.debug_logits = debug_logits_;
  }
  if (EnvInt("FLASHMOE_PROFILE", 0)) {
    const size_t bytes = (size_t)grid_ * FDMOE_PROF_EVENTS * 16;
    CUDA_ERROR_CHECK(cudaMalloc(reinterpret_cast<void**>(&prof_), bytes));
    CUDA_ERROR_CHECK(cudaMemsetAsync(prof_, 0, bytes, stream));
    params_.prof = prof_;
  }

  CUDA_ERROR_CHECK(cudaStreamSynchronize(stream));
  // every rank's arena is zeroed and mapped before anyone may launch
  if (boot_.Barrier() != 0) {
    FreeAll();
    return cudaErrorUnknown;
  }
  inited_ = true;
  return cudaSuccess;
}

cudaError_t MoeKernelLauncher::Deinit(cudaStream_t stream) {
  cudaError_t first = cudaStreamSynchronize(stream);
  DestroyHostPipe();  // drains the internal streams of the host-buffer entry point
  // no rank unmaps or frees while a peer may still be writing into its arena
  if (world_ > 1 && inited_) boot_.Barrier();
  FreeAll();
  inited_ = false;
  return first;
}

cudaError_t MoeKernelLauncher::LaunchBf16(const void* tokens, void* output, int tokensNum, cudaStream_t stream,
                                          int mode, uint32_t expected_static) {
  if (status_host_[0] != 0) {
    MOE_ERROR_LOG("launcher is unusable after device-side error %u (info 0x%x); destroy and re-create it",
                  status_host_[0], status_host_[1]);
    return cudaErrorUnknown;
  }
  ++epoch_;
  CUDA_ERROR_CHECK(cudaMemsetAsync(arena_ + layout_.zero_begin, 0, layout_.zero_end - layout_.zero_begin, stream));
  FdmoeParams p = params_;
  if (tokensNum > 0 && mode == 0) {
    // the token matrix moves between launches: its TMA descriptor is rebuilt (host-only arithmetic)
    // GATE tile height: the smallest of 32/64/128 tokens that still gives every SM at most one tile,
    // so that the gate phase spreads over as many SMs as possible
    // (with peers: always 32, many small tiles let the tensor cores start on the first rows while
    // later tiles are still being dispatched over NVLink)
    int rows = 128;
    if (tokensNum <= 32 * grid_ || world_ > 1) rows = 32;
    else if (tokensNum <= 64 * grid_) rows = 64;
    p.gate_rows = EnvInt("FLASHMOE_GATE_ROWS", rows);
    if (p.gate_rows != 32 && p.gate_rows != 64 && p.gate_rows != 128) p.gate_rows = rows;
    CUDA_ERROR_CHECK(MakeTensorMap(encode_, &p.tm_x, tokens, (uint64_t)tokensNum, g_.H,
                                   std::min(p.gate_rows, tokensNum)));
  }
  if (p.disp_conc <= 0) {
    // One GPU: every worker may copy rows (the copies are bound by memory writes).  With peers the
    // links set the pace of the dispatch and a third of the workers keeps them busy, while the others
    // feed the tensor cores with the batches that have landed (measured on four GPUs at 4096 tokens
    // per GPU: 48 workers 0.771 ms, 96 workers 0.824 ms, all workers 0.812 ms).
    p.disp_conc = world_ == 1 ? grid_ : std::max(1, grid_ / 3);
  }
  p.T = tokensNum;
  p.x = tokens;
  p.out = output;
  p.mode = mode;
  p.expected_static = expected_static;
  p.epoch = epoch_;
  return static_cast<cudaError_t>(fdmoe_kernel_launch(&p, grid_, stream));
}

cudaError_t MoeKernelLauncher::Launch(const void* tokens, void* output, int tokensNum, cudaStream_t stream) {
  if (!inited_) return cudaErrorNotReady;
  if (tokensNum < 0 || tokensNum > g_.max_tokens_local) {
    MOE_ERROR_LOG("tokensNum=%d exceeds maxTokens=%d", tokensNum, g_.max_tokens_local);
    return cudaErrorInvalidValue;
  }
  if (tokensNum > 0 && (!tokens || !output)) return cudaErrorInvalidValue;
  if (pipe_.ready && stream != pipe_.s_run) {
    // launches share the scratch arena: this one runs after the last one made through LaunchHost,
    // and the next LaunchHost after this one
    if (pipe_.calls) CUDA_ERROR_CHECK(cudaStreamWaitEvent(stream, pipe_.ran[(pipe_.calls - 1) & 1], 0));
    const cudaError_t e = LaunchDevice(tokens, output, tokensNum, stream);
    if (e != cudaSuccess) return e;
    CUDA_ERROR_CHECK(cudaEventRecord(pipe_.direct, stream));
    pipe_.direct_pending = true;
    return cudaSuccess;
  }
  return LaunchDevice(tokens, output, tokensNum, stream);
}

cudaError_t MoeKernelLauncher::LaunchDevice(const void* tokens, void* output, int tokensNum, cudaStream_t stream) {
  if (dtype_ == moe::MOE_DTYPE_BF16) return LaunchBf16(tokens, output, tokensNum, stream, 0, 0);
  const uint64_t n = (uint64_t)tokensNum * g_.H;
  CUDA_ERROR_CHECK(fdmoe_cast_f32_to_bf16(static_cast<const float*>(tokens), tok_bf16_, n, stream));
  CUDA_ERROR_CHECK(LaunchBf16(tok_bf16_, out_bf16_, tokensNum, stream, 0, 0));
  return static_cast<cudaError_t>(fdmoe_cast_bf16_to_f32(out_bf16_, static_cast<float*>(output), n, stream));
}

cudaError_t MoeKernelLauncher::InitHostPipe() {
  const size_t esz = dtype_ == moe::MOE_DTYPE_FP32 ? 4 : 2;
  const size_t cap = std::max<size_t>(16, (size_t)g_.max_tokens_local * g_.H * esz);
  for (int i = 0; i < 2; ++i) {
    CUDA_ERROR_CHECK(cudaMalloc(&pipe_.in[i], cap));
    CUDA_ERROR_CHECK(cudaMalloc(&pipe_.out[i], cap));
    CUDA_ERROR_CHECK(cudaEventCreateWithFlags(&pipe_.copied_in[i], cudaEventDisableTiming));
    CUDA_ERROR_CHECK(cudaEventCreateWithFlags(&pipe_.ran[i], cudaEventDisableTiming));
    CUDA_ERROR_CHECK(cudaEventCreateWithFlags(&pipe_.copied_out[i], cudaEventDisableTiming));
  }
  CUDA_ERROR_CHECK(cudaEventCreateWithFlags(&pipe_.direct, cudaEventDisableTiming));
  CUDA_ERROR_CHECK(cudaStreamCreateWithFlags(&pipe_.s_in, cudaStreamNonBlocking));
  CUDA_ERROR_CHECK(cudaStreamCreateWithFlags(&pipe_.s_run, cudaStreamNonBlocking));
  CUDA_ERROR_CHECK(cudaStreamCreateWithFlags(&pipe_.s_out, cudaStreamNonBlocking));
  pipe_.ready = true;
  return cudaSuccess;
}

void MoeKernelLauncher::DestroyHostPipe() {
  cudaStream_t* streams[] = {&pipe_.s_in, &pipe_.s_run, &pipe_.s_out};
  for (cudaStream_t* st : streams)
    if (*st) {
      cudaStreamSynchronize(*st);
      cudaStreamDestroy(*st);
      *st = nullptr;
    }
  cudaEvent_t* events[] = {&pipe_.copied_in[0], &pipe_.copied_in[1], &pipe_.ran[0],   &pipe_.ran[1],
                           &pipe_.copied_out[0], &pipe_.copied_out[1], &pipe_.direct};
  for (cudaEvent_t* ev : events)
    if (*ev) {
      cudaEventDestroy(*ev);
      *ev = nullptr;
    }
  pipe_.ready = false;
  pipe_.calls = 0;
  pipe_.direct_pending = false;
}

// Host buffers in, host buffers out.  The input must be complete in host memory when the call is
// made; the result is complete once `stream` has reached this point (synchronise it, or order
// later work after it).  Copy in, layer and copy out run on internal streams with two sets of
// staging buffers: back-to-back calls overlap the copies of one with the kernel of the other, so a
// stream of calls runs at the pace of the slowest of the three.
cudaError_t MoeKernelLauncher::LaunchHost(const void* hostTokens, void* hostOutput, int tokensNum,
                                          cudaStream_t stream) {
  if (!inited_) return cudaErrorNotReady;
  if (tokensNum < 0 || tokensNum > g_.max_tokens_local) return cudaErrorInvalidValue;
  if (tokensNum > 0 && (!hostTokens || !hostOutput)) return cudaErrorInvalidValue;
  if (!pipe_.ready) CUDA_ERROR_CHECK(InitHostPipe());
  const size_t esz = dtype_ == moe::MOE_DTYPE_FP32 ? 4 : 2;
  const size_t bytes = (size_t)tokensNum * g_.H * esz;
  const int slot = (int)(pipe_.calls & 1);
  const bool reused = pipe_.calls >= 2;
  // copy in: the staging buffer is free once the kernel of two calls ago has run
  if (reused) CUDA_ERROR_CHECK(cudaStreamWaitEvent(pipe_.s_in, pipe_.ran[slot], 0));
  if (bytes) CUDA_ERROR_CHECK(cudaMemcpyAsync(pipe_.in[slot], hostTokens, bytes, cudaMemcpyHostToDevice, pipe_.s_in));
  CUDA_ERROR_CHECK(cudaEventRecord(pipe_.copied_in[slot], pipe_.s_in));
  // layer: after its input has arrived, the result buffer has been copied out, and any launch made directly
  CUDA_ERROR_CHECK(cudaStreamWaitEvent(pipe_.s_run, pipe_.copied_in[slot], 0));
  if (reused) CUDA_ERROR_CHECK(cudaStreamWaitEvent(pipe_.s_run, pipe_.copied_out[slot], 0));
  if (pipe_.direct_pending) {
    CUDA_ERROR_CHECK(cudaStreamWaitEvent(pipe_.s_run, pipe_.direct, 0));
    pipe_.direct_pending = false;
  }
  CUDA_ERROR_CHECK(LaunchDevice(pipe_.in[slot], pipe_.out[slot], tokensNum, pipe_.s_run));
  CUDA_ERROR_CHECK(cudaEventRecord(pipe_.ran[slot], pipe_.s_run));
  // copy out, then the caller's stream joins
  CUDA_ERROR_CHECK(cudaStreamWaitEvent(pipe_.s_out, pipe_.ran[slot], 0));
  if (bytes) CUDA_ERROR_CHECK(cudaMemcpyAsync(hostOutput, pipe_.out[slot], bytes, cudaMemcpyDeviceToHost, pipe_.s_out));
  CUDA_ERROR_CHECK(cudaEventRecord(pipe_.copied_out[slot], pipe_.s_out));
  CUDA_ERROR_CHECK(cudaStreamWaitEvent(stream, pipe_.copied_out[slot], 0));
  ++pipe_.calls;
  return cudaSuccess;
}

cudaError_t MoeKernelLauncher::DebugRead(int which, void* dst, size_t offset, size_t bytes) {
  if (!inited_) return cudaErrorNotReady;
  CUDA_ERROR_CHECK(cudaDeviceSynchronize());
  const void* src = nullptr;
  size_t size = 0;
  int32_t info[4] = {g_.cap_rows, g_.El, grid_, smem_};
  switch (which) {
    case 0: src = topk_idx_; size = (size_t)g_.max_tokens_local * g_.K * 4; break;
    case 1: src = topk_w_; size = (size_t)g_.max_tokens_local * g_.K * 4; break;
    case 2: src = arena_ + layout_.expert_cnt; size = (size_t)g_.El * 4; break;
    case 3: src = arena_ + layout_.packed; size = (size_t)g_.El * g_.cap_rows * g_.H * 2; break;
    case 4: src = arena_ + layout_.meta; size = (size_t)g_.El * g_.cap_rows * sizeof(FdmoeRowMeta); break;
    case 5: src = act_; size = (size_t)g_.El * g_.cap_rows * g_.I * 2; break;
    case 6: src = arena_ + layout_.ystage; size = (size_t)g_.max_tokens_max * g_.K * g_.H * 2; break;
    case 7:
      memcpy(dst, info, std::min(bytes, sizeof(info)));
      return cudaSuccess;
    case 9: src = debug_logits_; size = debug_logits_ ? (size_t)g_.max_tokens_local * 128 * 4 : 0; break;
    case 10: src = stuck_; size = (size_t)grid_ * 16 * 16; break;
    case 8: src = prof_; size = prof_ ? (size_t)grid_ * FDMOE_PROF_EVENTS * 16 : 0; break;
    default: return cudaErrorInvalidValue;
  }
  if (offset >= size) return cudaSuccess;
  const size_t n = std::min(bytes, size - offset);
  return cudaMemcpy(dst, static_cast<const uint8_t*>(src) + offset, n, cudaMemcpyDeviceToHost);
}

// Writes tasks into the queue from the host (mode 2 launches only).
cudaError_t MoeKernelLauncher::PrefillTasks(const std::vector<FdmoeSlot>& tasks, cudaStream_t stream) {
  CUDA_ERROR_CHECK(cudaStreamSynchronize(stream));
  if (pipe_.ready) CUDA_ERROR_CHECK(cudaStreamSynchronize(pipe_.s_run));
  FdmoeCtl ctl;
  CUDA_ERROR_CHECK(cudaMemcpy(&ctl, arena_ + layout_.ctl, sizeof(ctl), cudaMemcpyDeviceToHost));
  const uint32_t head = ctl.q[1].head;
  FdmoeSlot* slots = reinterpret_cast<FdmoeSlot*>(arena_ + layout_.slots[1]);
  for (size_t i = 0; i < tasks.size(); ++i) {
    FdmoeSlot s = tasks[i];
    const uint32_t ticket = head + (uint32_t)i;
    s.seq = ticket + 1u;
    CUDA_ERROR_CHECK(cudaMemcpy(&slots[ticket & (g_.queue_cap - 1)], &s, sizeof(s), cudaMemcpyHostToDevice));
  }
  FdmoeQueueCtl q1 = ctl.q[1];
  q1.head = head + (uint32_t)tasks.size();
  q1.avail += (uint32_t)tasks.size();
  return cudaMemcpy(arena_ + layout_.ctl + offsetof(FdmoeCtl, q) + sizeof(FdmoeQueueCtl), &q1, 12, cudaMemcpyHostToDevice);
}

cudaError_t MoeKernelLauncher::TestTaskSystem(int32_t* data, int n, cudaStream_t stream) {
  if (!inited_) return cudaErrorNotReady;
  if (n <= 0 || n % 256 != 0 || (uint32_t)(n / 256) * 2u + 1024u > g_.queue_cap) return cudaErrorInvalidValue;
  std::vector<FdmoeSlot> tasks((size_t)n / 256);
  for (size_t i = 0; i < tasks.size(); ++i) tasks[i] = FdmoeSlot{0, FDMOE_TASK_TESTA, (uint32_t)i, 0};
  CUDA_ERROR_CHECK(PrefillTasks(tasks, stream));
  params_.test_buf = data;
  const cudaError_t e = LaunchBf16(nullptr, nullptr, 0, stream, 2, (uint32_t)tasks.size() * 2u);
  params_.test_buf = nullptr;
  return e;
}

// A launch that expects one task nobody ever publishes: every worker's bounded wait for work runs out,
// the kernel records FDMOE_ERR_TIMEOUT_QUEUE and returns.
cudaError_t MoeKernelLauncher::TestStall(cudaStream_t stream) {
  if (!inited_) return cudaErrorNotReady;
  return LaunchBf16(nullptr, nullptr, 0, stream, 2, 1u);
}

cudaError_t MoeKernelLauncher::TestQueueGemm(const uint32_t* rowsPerExpert, const void* A, void* out,
                                             cudaStream_t stream) {
  if (!inited_ || dtype_ != moe::MOE_DTYPE_BF16) return cudaErrorNotReady;
  std::vector<FdmoeSlot> tasks;
  std::vector<FdmoeRowMeta> meta;
  const uint32_t nt2 = (uint32_t)(g_.H / FDMOE_TILE_N2);
  size_t row0 = 0;
  for (int e = 0; e < g_.El; ++e) {
    const uint32_t rows = rowsPerExpert[e];
    if (rows > (uint32_t)g_.cap_rows) return cudaErrorInvalidValue;
    if (rows == 0) continue;
    CUDA_ERROR_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(act_) + (size_t)e * g_.cap_rows * g_.I * 2,
                                     static_cast<const uint8_t*>(A) + row0 * g_.I * 2, (size_t)rows * g_.I * 2,
                                     cudaMemcpyDeviceToDevice, stream));
    meta.resize(rows);
    for (uint32_t r = 0; r < rows; ++r) meta[r] = FdmoeRowMeta{(int32_t)(row0 + r), rank_ << 8, 1.0f, 0};
    CUDA_ERROR_CHECK(cudaMemcpy(arena_ + layout_.meta + (size_t)e * g_.cap_rows * sizeof(FdmoeRowMeta), meta.data(),
                                rows * sizeof(FdmoeRowMeta), cudaMemcpyHostToDevice));
    for (uint32_t j = 0; j * 128 < rows; ++j)
      for (uint32_t n = 0; n < nt2; ++n)
        tasks.push_back(FdmoeSlot{0, (uint32_t)FDMOE_TASK_FFN2 | ((uint32_t)e << 8) | (n << 20), j,
                                  std::min<uint32_t>(128, rows - j * 128)});
    row0 += rows;
  }
  if (tasks.size() + 1024 > g_.queue_cap) return cudaErrorInvalidValue;
  CUDA_ERROR_CHECK(PrefillTasks(tasks, stream));
  // rows are their own "tokens": K = 1 and the result buffer stands in for the staging area
  const int saved_k = params_.K;
  void* saved_y = params_.peers[rank_].ystage;
  params_.K = 1;
  params_.peers[rank_].ystage = out;
  const cudaError_t e = LaunchBf16(nullptr, nullptr, 0, stream, 2, (uint32_t)tasks.size());
  params_.K = saved_k;
  params_.peers[rank_].ystage = saved_y;
  return e;
}

}  // namespace fdmoe

// =============================================================== C exports
namespace {
const moe::MoeConfig kQwen3_30B_A3B = {2048, 768, 128, 8, moe::MOE_DTYPE_BF16, {0, 0, 0}};
// What the reference's CreateLauncher means: its compile-time layer (src/hip/common/metadata.h:7-13)
// with fp32 weights, tokens and output (python/pyMoeLauncherTorch.cpp:24-31).
const moe::MoeConfig kReferenceLayer = {2048, 768, 128, 8, moe::MOE_DTYPE_FP32, {0, 0, 0}};

cudaError_t CreateImpl(moe::IMoeKernelLauncher** launcher, const void* gateW, const void* w13, const void* w2,
                       int maxTokens, cudaStream_t stream, const moe::DistributedUniqueId& uid, int rank,
                       int world, const moe::MoeConfig& cfg) {
  if (!launcher) return cudaErrorInvalidValue;
  fdmoe::MoeKernelLauncher* l = new (std::nothrow) fdmoe::MoeKernelLauncher();
  if (!l) return cudaErrorMemoryAllocation;
  const cudaError_t e = l->Init(gateW, w13, w2, maxTokens, stream, uid, rank, world, cfg);
  if (e != cudaSuccess) {
    l->Deinit(stream);
    delete l;
    return e;
  }
  *launcher = l;
  return cudaSuccess;
}
}  // namespace

extern "C" moe::DistributedUniqueId GetDistributedUniqueId(bool empty) {
  moe::DistributedUniqueId id;
  memset(id.data, 0, sizeof(id.data));
  if (!empty && fdmoe::MakeUniqueId(id.data) != 0) MOE_ERROR_LOG("could not create a unique id");
  return id;
}

extern "C" cudaError_t CreateLauncher(moe::IMoeKernelLauncher** launcher, const void* gateWeights,
                                      const void* ffn1ExpertWeights, const void* ffn2ExpertWeights,
                                      int maxTokens, cudaStream_t stream, const moe::DistributedUniqueId& uid,
                                      int rank, int worldSize) {
  return CreateImpl(launcher, gateWeights, ffn1ExpertWeights, ffn2ExpertWeights, maxTokens, stream, uid, rank,
                    worldSize, kReferenceLayer);
}

extern "C" cudaError_t CreateLauncherEx(moe::IMoeKernelLauncher** launcher, const void* gateWeights,
                                        const void* ffn1ExpertWeights, const void* ffn2ExpertWeights,
                                        int maxTokens, cudaStream_t stream, const moe::DistributedUniqueId& uid,
                                        int rank, int worldSize, const moe::MoeConfig* config) {
  return CreateImpl(launcher, gateWeights, ffn1ExpertWeights, ffn2ExpertWeights, maxTokens, stream, uid, rank,
                    worldSize, config ? *config : kQwen3_30B_A3B);
}

extern "C" cudaError_t DestroyLauncher(moe::IMoeKernelLauncher* launcher, cudaStream_t stream) {
  if (!launcher) return cudaErrorInvalidValue;
  fdmoe::MoeKernelLauncher* l = static_cast<fdmoe::MoeKernelLauncher*>(launcher);
  const cudaError_t e = l->Deinit(stream);
  delete l;
  return e;
}

// ------------------------------------------------------------- flat C ABI
static fdmoe::MoeKernelLauncher* AsLauncher(FlashMoeHandle h) {
  return reinterpret_cast<fdmoe::MoeKernelLauncher*>(h);
}

extern "C" int FlashMoeGetUniqueId(int empty, uint8_t out[128]) {
  const moe::DistributedUniqueId id = GetDistributedUniqueId(empty != 0);
  memcpy(out, id.data, 128);
  return 0;
}

extern "C" int FlashMoeCreate(FlashMoeHandle* out, const void* gateWeights, const void* ffn1ExpertWeights,
                              const void* ffn2ExpertWeights, int maxTokens, void* stream, const uint8_t uid[128],
                              int rank, int worldSize, const FlashMoeConfig* config) {
  if (!out || !uid) return (int)cudaErrorInvalidValue;
  moe::DistributedUniqueId id;
  memcpy(id.data, uid, 128);
  moe::MoeConfig cfg = kQwen3_30B_A3B;
  if (config) {
    static_assert(sizeof(FlashMoeConfig) == sizeof(moe::MoeConfig), "config layouts must match");
    memcpy(&cfg, config, sizeof(cfg));
  }
  moe::IMoeKernelLauncher* l = nullptr;
  const cudaError_t e = CreateImpl(&l, gateWeights, ffn1ExpertWeights, ffn2ExpertWeights, maxTokens,
                                   static_cast<cudaStream_t>(stream), id, rank, worldSize, cfg);
  if (e == cudaSuccess) *out = reinterpret_cast<FlashMoeHandle>(static_cast<fdmoe::MoeKernelLauncher*>(l));
  return (int)e;
}

extern "C" int FlashMoeLaunch(FlashMoeHandle h, const void* tokens, void* output, int tokensNum, void* stream) {
  if (!h) return (int)cudaErrorInvalidValue;
  return (int)AsLauncher(h)->Launch(tokens, output, tokensNum, static_cast<cudaStream_t>(stream));
}

extern "C" int FlashMoeLaunchHost(FlashMoeHandle h, const void* hostTokens, void* hostOutput, int tokensNum,
                                  void* stream) {
  if (!h) return (int)cudaErrorInvalidValue;
  return (int)AsLauncher(h)->LaunchHost(hostTokens, hostOutput, tokensNum, static_cast<cudaStream_t>(stream));
}

extern "C" int FlashMoeDestroy(FlashMoeHandle h, void* stream) {
  if (!h) return (int)cudaErrorInvalidValue;
  return (int)DestroyLauncher(AsLauncher(h), static_cast<cudaStream_t>(stream));
}

extern "C" int FlashMoeGetLastStatus(FlashMoeHandle h, uint32_t* code, uint32_t* info) {
  if (!h) return (int)cudaErrorInvalidValue;
  AsLauncher(h)->LastStatus(code, info);
  return 0;
}

extern "C" int FlashMoeDebugRead(FlashMoeHandle h, int which, void* dst, size_t offset, size_t bytes) {
  if (!h || !dst) return (int)cudaErrorInvalidValue;
  return (int)AsLauncher(h)->DebugRead(which, dst, offset, bytes);
}

extern "C" int FlashMoeTestTaskSystem(FlashMoeHandle h, int32_t* data, int n, void* stream) {
  if (!h) return (int)cudaErrorInvalidValue;
  return (int)AsLauncher(h)->TestTaskSystem(data, n, static_cast<cudaStream_t>(stream));
}

extern "C" int FlashMoeTestQueueGemm(FlashMoeHandle h, const uint32_t* rowsPerExpertHost, const void* A,
                                     void* out, void* stream) {
  if (!h || !rowsPerExpertHost) return (int)cudaErrorInvalidValue;
  return (int)AsLauncher(h)->TestQueueGemm(rowsPerExpertHost, A, out, static_cast<cudaStream_t>(stream));
}

extern "C" int FlashMoeTestStall(FlashMoeHandle h, void* stream) {
  if (!h) return (int)cudaErrorInvalidValue;
  return (int)AsLauncher(h)->TestStall(static_cast<cudaStream_t>(stream));
}

extern "C" const char* FlashMoeErrorString(int code) { return cudaGetErrorString(static_cast<cudaError_t>(code)); }
