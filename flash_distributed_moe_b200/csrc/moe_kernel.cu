// The persistent MoE-layer kernel for sm_100a and its thin C ABI.
//
// One CTA per SM.  Phase A: CTAs claim 32-token gate tiles (fp32 gate GEMM in
// the reference's accumulation order, top-k, fp32/fp64 softmax, row pack into
// the owning rank's expert buffers).  Phase B: every CTA becomes a worker that
// pulls tile tasks from a ticket-based global queue: FFN1 (SwiGLU) and FFN2
// (down projection) tiles run on tcgen05 with TMEM accumulators fed by TMA,
// COMBINE sums a token group's K result rows in slot order.  Cross-GPU traffic
// is plain stores and scoped atomics into peers' symmetric buffers.
//
// Counterparts in the reference project (HIP, MI300X):
//   persistent kernel + phases     src/hip/kernel/moeKernel.h:37-107
//   gate tile, top-k + softmax     src/hip/kernel/tasks/internal/gateBlock.h:10-42, topkBlock.h:23-98
//   FFN1 / FFN2 / reduce tasks     src/hip/kernel/tasks/ffn1Task.h:12-64, ffn2Task.h:11-70, reduceTask.h:7-26
//   ticket queue, worker loop      src/hip/taskSystem/workQueue.h:77-134, taskManager.h:153-247, workerLoop.h:14-40
//   dispatch / return pattern      test/multiGPU/cpp/rocshmem/moeLikeCommPattern.cpp:61-255
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "moe_types.h"
#include "ptx.cuh"

namespace fdmoe {

using bf16 = __nv_bfloat16;

constexpr int kThreads = 384;  // 12 warps
constexpr int kWarpSched = 0;  // pops global tickets, feeds the CTA task ring
constexpr int kWarpTma = 1;    // issues TMA loads
constexpr int kWarpMma = 2;    // issues tcgen05.mma
constexpr int kWarpTmem = 3;   // allocates / frees TMEM
constexpr int kWarpEpi0 = 4;   // warps 4..11: epilogues and SIMT tasks
constexpr int kEpiThreads = 256;

constexpr int kStages = 4;
constexpr int kStageA = FDMOE_TILE_M * FDMOE_TILE_K * 2;  // 16 KB
constexpr int kStageB = 256 * FDMOE_TILE_K * 2;           // 32 KB
constexpr int kStageBytes = kStageA + kStageB;            // 48 KB
constexpr int kRing = 3;
constexpr int kTmemCols = 512;
constexpr int kAccCols = 256;

struct __align__(16) SmemCtl {
  uint64_t full_bar[kStages];
  uint64_t empty_bar[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t ring_full[kRing];
  uint64_t ring_empty[kRing];
  FdmoeSlot ring[kRing];
  uint32_t tmem_base;
  volatile uint32_t abort;
  int32_t cur_tile;
  int32_t flag;
  uint32_t q_t0;
  uint32_t q_total;
  uint32_t prof_n;
  uint32_t cnt[128];
  uint32_t base[128];
  uint32_t pre[132];
  uint32_t full_tiles[128];
  uint32_t rem_rows[128];
  int32_t tk_idx[FDMOE_GATE_TOKENS][FDMOE_MAX_TOPK];
  float tk_w[FDMOE_GATE_TOKENS][FDMOE_MAX_TOPK];
  uint32_t lpos[FDMOE_GATE_TOKENS][FDMOE_MAX_TOPK];
};

constexpr int kSmemBytes = kStages * kStageBytes + (int)sizeof(SmemCtl) + 1024;

// ------------------------------------------------------------ scoped helpers
template <bool S>
__device__ __forceinline__ void fence_acqrel() {
  if (S)
    asm volatile("fence.acq_rel.sys;" ::: "memory");
  else
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
}
template <bool S>
__device__ __forceinline__ void fence_sc() {
  if (S)
    asm volatile("fence.sc.sys;" ::: "memory");
  else
    asm volatile("fence.sc.gpu;" ::: "memory");
}
template <bool S>
__device__ __forceinline__ uint32_t atom_add(uint32_t* p, uint32_t v) {
  uint32_t old;
  if (S)
    asm volatile("atom.relaxed.sys.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  else
    asm volatile("atom.relaxed.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
template <bool S>
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  if (S)
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  else
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
template <bool S>
__device__ __forceinline__ uint32_t ld_relaxed(const uint32_t* p) {
  uint32_t v;
  if (S)
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  else
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
template <bool S>
__device__ __forceinline__ void st_release(uint32_t* p, uint32_t v) {
  if (S)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
  else
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
template <bool S>
__device__ __forceinline__ void st_relaxed(uint32_t* p, uint32_t v) {
  if (S)
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
  else
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Barrier over the 256 epilogue threads that also ANDs a predicate, so that the
// whole group takes the same decision after a bounded wait.
__device__ __forceinline__ bool epi_vote_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 256, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(r)
      : "r"((uint32_t)ok)
      : "memory");
  return r != 0;
}

__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  return __ldcg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Optional event trace (one writer thread per phase): {kind, t0, t1, t2} in ns,
// low 32 bits of the global timer.  Slot 0 of each CTA holds the event count.
__device__ __forceinline__ uint32_t prof_now() { return (uint32_t)ptx::globaltimer_ns(); }
__device__ __forceinline__ void prof_event(const FdmoeParams& p, SmemCtl& sc, uint32_t kind,
                                           uint32_t t0, uint32_t t1, uint32_t t2) {
  if (!p.prof) return;
  const uint32_t i = ++sc.prof_n;
  if (i >= FDMOE_PROF_EVENTS) return;
  uint32_t* e = p.prof + ((size_t)blockIdx.x * FDMOE_PROF_EVENTS + i) * 4;
  e[0] = kind; e[1] = t0; e[2] = t1; e[3] = t2;
  p.prof[(size_t)blockIdx.x * FDMOE_PROF_EVENTS * 4] = i;
}

// ------------------------------------------------------- error / abort path
// Records the first error, raises the CTA-local and the rank-wide abort flags.
__device__ __noinline__ void raise_error(const FdmoeParams& p, SmemCtl& sc, uint32_t code,
                                         uint32_t info) {
  FdmoeCtl* ctl = p.peers[p.rank].ctl;
  if (atomicCAS(&ctl->status, 0u, code) == 0u) {
    ctl->status_info = info;
    if (p.status_host) {
      ptx::st_relaxed_sys(p.status_host + 1, info);
      ptx::st_release_sys(p.status_host, code);
    }
  }
  sc.abort = 1;
  __threadfence();
  atomicExch(&ctl->closed, 2u);
}

// Bounded mbarrier wait.  Returns false (after raising the error) on timeout
// or when another role of this CTA has aborted.
__device__ __forceinline__ bool wait_bar(const FdmoeParams& p, SmemCtl& sc, uint64_t* bar,
                                         uint32_t parity, uint32_t err_code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (sc.abort) return false;
      if (ptx::globaltimer_ns() - t0 > p.timeout_ns) {
        raise_error(p, sc, err_code, (blockIdx.x << 8) | (threadIdx.x >> 5));
        return false;
      }
    }
  }
  return true;
}

// ------------------------------------------------------------- global queue
// Producers take `n` consecutive tickets with one atomic add on head, fill the
// slots and publish each with a release store of ticket+1.
template <bool S, class Gen>
__device__ __forceinline__ void queue_push(const FdmoeParams& p, const FdmoePeer& q, uint32_t n,
                                           Gen gen) {
  const uint32_t t0 = atom_add<S>(&q.ctl->q_head, n);
  for (uint32_t i = 0; i < n; ++i) {
    FdmoeSlot* s = &q.slots[(t0 + i) & (uint32_t)p.queue_mask];
    uint32_t a, b, c;
    gen(i, a, b, c);
    s->a = a;
    s->b = b;
    s->c = c;
    st_release<S>(&s->seq, t0 + i + 1u);
  }
}

__device__ __forceinline__ uint32_t task_word(uint32_t kind, uint32_t e, uint32_t n) {
  return kind | (e << 8) | (n << 20);
}

// Consumer: take a ticket, wait (bounded) until its slot is published or the
// queue is closed.  Single thread.
template <bool S>
__device__ __forceinline__ FdmoeSlot queue_pop(const FdmoeParams& p, SmemCtl& sc) {
  const FdmoePeer& me = p.peers[p.rank];
  FdmoeSlot out;
  out.seq = 0;
  out.a = FDMOE_TASK_EXIT;
  out.b = 0;
  out.c = 0;
  if (sc.abort) return out;
  const uint32_t ticket = atomicAdd(&me.ctl->q_tail, 1u);
  FdmoeSlot* s = &me.slots[ticket & (uint32_t)p.queue_mask];
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (ld_acquire<S>(&s->seq) == ticket + 1u) break;
    if (ld_relaxed<S>(&me.ctl->closed) != 0u || sc.abort) return out;
    if ((++spins & 15u) == 0u) {
      if (ptx::globaltimer_ns() - t0 > p.timeout_ns) {
        raise_error(p, sc, FDMOE_ERR_TIMEOUT_QUEUE, (blockIdx.x << 8));
        return out;
      }
      __nanosleep(100);
    }
  }
  out.a = s->a;
  out.b = s->b;
  out.c = s->c;
  return out;
}

// Closes this rank's queue once the flush has run, every m-tile of its experts
// has finished FFN2 and every token of this rank has been combined.  Called
// after each of those three kinds of event; the sequentially-consistent fence
// guarantees that the last caller sees the other two conditions.
__device__ __forceinline__ void maybe_close(const FdmoeParams& p) {
  FdmoeCtl* ctl = p.peers[p.rank].ctl;
  fence_sc<false>();
  if (ld_relaxed<false>(&ctl->flush_done) == 0u) return;
  if (ld_relaxed<false>(&ctl->mtiles_done) != ld_relaxed<false>(&ctl->mtiles_total)) return;
  if (ld_relaxed<false>(&ctl->tokens_combined) != ld_relaxed<false>(&ctl->tokens_launch)) return;
  st_release<false>(&ctl->closed, 1u);
}

// This rank's gate phase is complete (all its rows are written and fenced):
// tell every rank; whoever completes a rank's count asks it to flush.
template <bool S>
__device__ void gate_phase_finished(const FdmoeParams& p) {
  FdmoeCtl* ctl = p.peers[p.rank].ctl;
  if (p.mode == 1) {
    fence_acqrel<false>();
    st_release<false>(&ctl->closed, 1u);
    return;
  }
  for (int q = 0; q < p.world; ++q) {
    fence_acqrel<S>();
    const uint32_t prev = atom_add<S>(&p.peers[q].ctl->ranks_done, 1u);
    if (prev == (uint32_t)p.world - 1u) {
      fence_acqrel<S>();
      queue_push<S>(p, p.peers[q], 1u, [](uint32_t, uint32_t& a, uint32_t& b, uint32_t& c) {
        a = FDMOE_TASK_FLUSH;
        b = 0;
        c = 0;
      });
    }
  }
}

// ================================================================== phase A
// One gate tile: logits for 32 tokens x E experts with fp32 FMAs, k strictly
// ascending per output (bf16 x bf16 products are exact in fp32, so this equals
// the reference's `acc += a*b` bit for bit), top-k with the lower index winning
// ties, softmax over the kept logits in double, then the rows are packed into
// the owners' expert buffers.
template <bool S>
__device__ void gate_tile(const FdmoeParams& p, uint8_t* stage, SmemCtl& sc, int tile,
                          int n_tiles) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.H, E = p.E, K = p.K;
  const int t0 = tile * FDMOE_GATE_TOKENS;
  const int nt = min(FDMOE_GATE_TOKENS, p.T - t0);
  float* As = reinterpret_cast<float*>(stage);  // [2][32 k][32 tok]
  float* Bs = As + 2 * 32 * 32;                 // [2][32 k][128 exp]
  float* logits = Bs + 2 * 32 * 128;            // [32 tok][128 exp]
  const bf16* x = reinterpret_cast<const bf16*>(p.x);
  const bf16* wg = reinterpret_cast<const bf16*>(p.gate_w);
  const FdmoePeer& me = p.peers[p.rank];

  if (tid < 128) sc.cnt[tid] = 0;
  const uint32_t pt0 = p.prof ? prof_now() : 0u;

  // ---- gate GEMM: warps 0-3 compute (8 tokens x 4 experts per thread), warps
  // 4-11 stage the next 32-wide k chunk (bf16 -> fp32, transposed to [k][row]).
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int nchunks = H / 32;
  auto stage_chunk = [&](int c, int b) {
    uint4 v[3];
    int pidx[3];
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      const int pi = (tid - 128) + u * 256;
      pidx[u] = pi;
      v[u] = make_uint4(0, 0, 0, 0);
      if (pi < 128) {
        const int r = pi & 31, q = pi >> 5;
        if (r < nt) v[u] = *reinterpret_cast<const uint4*>(x + (size_t)(t0 + r) * H + c * 32 + q * 8);
      } else if (pi < 640) {
        const int pp = pi - 128;
        const int r = pp & 127, q = pp >> 7;
        if (r < E) v[u] = __ldg(reinterpret_cast<const uint4*>(wg + (size_t)r * H + c * 32 + q * 8));
      }
    }
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      const int pi = pidx[u];
      float* dst;
      int stride;
      if (pi < 128) {
        const int r = pi & 31, q = pi >> 5;
        dst = As + b * 1024 + (q * 8) * 32 + r;
        stride = 32;
      } else if (pi < 640) {
        const int pp = pi - 128;
        const int r = pp & 127, q = pp >> 7;
        dst = Bs + b * 4096 + (q * 8) * 128 + r;
        stride = 128;
      } else {
        continue;
      }
      const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dst[(2 * i) * stride] = bf16_lo(w[i]);
        dst[(2 * i + 1) * stride] = bf16_hi(w[i]);
      }
    }
  };

  if (tid >= 128) stage_chunk(0, 0);
  __syncthreads();
  for (int c = 0; c < nchunks; ++c) {
    const int b = c & 1;
    if (tid >= 128) {
      if (c + 1 < nchunks) stage_chunk(c + 1, b ^ 1);
    } else {
      const float* a = As + b * 1024 + warp * 8;
      const float* bb = Bs + b * 4096 + lane * 4;
#pragma unroll 8
      for (int k = 0; k < 32; ++k) {
        const float4 a0 = *reinterpret_cast<const float4*>(a + k * 32);
        const float4 a1 = *reinterpret_cast<const float4*>(a + k * 32 + 4);
        const float4 bv = *reinterpret_cast<const float4*>(bb + k * 128);
        const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const float bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bw[j], acc[i][j]);
      }
    }
    __syncthreads();
  }
  if (tid < 128) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *reinterpret_cast<float4*>(logits + (warp * 8 + i) * 128 + lane * 4) =
          make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
  }
  __syncthreads();
  const uint32_t pt1 = p.prof ? prof_now() : 0u;

  // ---- top-k + softmax: one warp per token, 4 logits per lane.
  for (int tok = warp; tok < nt; tok += kThreads / 32) {
    float v[4];
    uint32_t taken = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = lane + 32 * i;
      v[i] = (e < E) ? logits[tok * 128 + e] : -INFINITY;
      if (e >= E) taken |= 1u << i;
    }
    float myv = 0.f;
    int myi = 0;
    for (int k = 0; k < K; ++k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = lane + 32 * i;
        if (!((taken >> i) & 1u) && (v[i] > bv || (v[i] == bv && e < bi))) {
          bv = v[i];
          bi = e;
        }
      }
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (ov > bv || (ov == bv && oi < bi)) {
          bv = ov;
          bi = oi;
        }
      }
      if ((bi & 31) == lane && bi < 128) taken |= 1u << (bi >> 5);
      if (lane == k) {
        myv = bv;
        myi = bi;
      }
    }
    // softmax over the K kept logits: running-max form of the reference with the
    // values already in descending order, so the max is the first one and the
    // sum is accumulated as 1 + e_1 + e_2 + ... in that order, all in double.
    const double m = (double)__shfl_sync(0xffffffffu, myv, 0);
    const double ex = (lane < K) ? exp((double)myv - m) : 0.0;
    double sum = 1.0;
    for (int j = 1; j < K; ++j) sum += __shfl_sync(0xffffffffu, ex, j);
    const float w = (float)(ex / sum);
    if (lane < K) {
      p.topk_idx[(size_t)(t0 + tok) * K + lane] = myi;
      p.topk_w[(size_t)(t0 + tok) * K + lane] = w;
      sc.tk_idx[tok][lane] = myi;
      sc.tk_w[tok][lane] = w;
      sc.lpos[tok][lane] = atomicAdd(&sc.cnt[myi & 127], 1u);
    }
  }
  __syncthreads();

  // ---- reserve rows in the owners' expert buffers: one atomic per expert.
  if (tid < E) {
    const uint32_t cnt = sc.cnt[tid];
    if (cnt) {
      const int owner = tid / p.El, le = tid - owner * p.El;
      const uint32_t base = atom_add<S>(&p.peers[owner].expert_cnt[le], cnt);
      if (base + cnt > (uint32_t)p.cap_rows) raise_error(p, sc, FDMOE_ERR_ROW_OVERFLOW, tid);
      sc.base[tid] = base;
    }
  }
  __syncthreads();

  // ---- pack: copy each token row to its K destinations, one warp per token.
  if (!sc.abort) {
    for (int tok = warp; tok < nt; tok += kThreads / 32) {
      const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(t0 + tok) * H);
      for (int seg = 0; seg < H / 2048 + ((H % 2048) ? 1 : 0); ++seg) {
        uint4 r[8];
        const int vbase = seg * 256;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int vi = vbase + lane + 32 * i;
          r[i] = (vi < H / 8) ? src[vi] : make_uint4(0, 0, 0, 0);
        }
        for (int k = 0; k < K; ++k) {
          const int e = sc.tk_idx[tok][k];
          const int owner = e / p.El, le = e - owner * p.El;
          const size_t row = (size_t)le * p.cap_rows + sc.base[e] + sc.lpos[tok][k];
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.peers[owner].packed) + row * H);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int vi = vbase + lane + 32 * i;
            if (vi < H / 8) dst[vi] = r[i];
          }
          if (seg == 0 && lane == 0) {
            // FdmoeRowMeta {token, home << 8 | slot, weight, pad} as one 16-byte store
            *reinterpret_cast<uint4*>(&p.peers[owner].meta[row]) =
                make_uint4((uint32_t)(t0 + tok), (uint32_t)((p.rank << 8) | k),
                           __float_as_uint(sc.tk_w[tok][k]), 0u);
          }
        }
      }
    }
  }
  ptx::fence_proxy_async();  // packed rows are read by TMA later
  __syncthreads();

  // ---- landed accounting (eager mode): the writer that completes a 128-row
  // tile publishes its FFN1 tasks on the owner's queue.
  if (p.eager && p.mode == 0 && tid < E && sc.cnt[tid]) {
    const uint32_t cnt = sc.cnt[tid], base = sc.base[tid];
    const int owner = tid / p.El, le = tid - owner * p.El;
    const uint32_t nt1 = (uint32_t)(p.I / FDMOE_TILE_N1);
    fence_acqrel<S>();
    const uint32_t j0 = base / 128u, j1 = (base + cnt - 1u) / 128u;
    for (uint32_t j = j0; j <= j1; ++j) {
      const uint32_t lo = max(base, j * 128u), hi = min(base + cnt, (j + 1u) * 128u);
      const uint32_t add = hi - lo;
      const uint32_t prev = atom_add<S>(&p.peers[owner].tile_landed[(size_t)le * p.MT + j], add);
      if (prev + add == 128u) {
        fence_acqrel<S>();
        queue_push<S>(p, p.peers[owner], nt1, [&](uint32_t i, uint32_t& a, uint32_t& b, uint32_t& c) {
          a = task_word(FDMOE_TASK_FFN1, (uint32_t)le, i);
          b = j;
          c = 128u;
        });
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    prof_event(p, sc, 100u, pt0, pt1, prof_now());
    fence_acqrel<S>();
    const uint32_t done = atomicAdd(&me.ctl->gate_done, 1u) + 1u;
    if (done == (uint32_t)n_tiles) gate_phase_finished<S>(p);
  }
}

// ================================================================== phase B
// FLUSH: every rank's gate phase is complete, so the per-expert row counts are
// final.  Publishes FFN1 tasks for all tiles (or, in eager mode, only for the
// partial last tile of each expert), ordered by expert so that tiles sharing
// weights run close together.  Executed by the 256 epilogue threads.
template <bool S>
__device__ void flush_task(const FdmoeParams& p, SmemCtl& sc, int etid) {
  const FdmoePeer& me = p.peers[p.rank];
  const uint32_t nt1 = (uint32_t)(p.I / FDMOE_TILE_N1);
  fence_acqrel<S>();
  if (etid < p.El) {
    const uint32_t cnt = ld_relaxed<S>(&me.expert_cnt[etid]);
    const uint32_t full = cnt / 128u, rem = cnt % 128u;
    sc.full_tiles[etid] = full;
    sc.rem_rows[etid] = rem;
    sc.pre[etid + 1] = p.eager ? (rem ? nt1 : 0u) : (full + (rem ? 1u : 0u)) * nt1;
  }
  epi_bar();
  if (etid == 0) {
    sc.pre[0] = 0;
    uint32_t mt = 0;
    for (int e = 0; e < p.El; ++e) {
      sc.pre[e + 1] += sc.pre[e];
      mt += sc.full_tiles[e] + (sc.rem_rows[e] ? 1u : 0u);
    }
    const uint32_t total = sc.pre[p.El];
    sc.q_total = total;
    sc.q_t0 = total ? atom_add<false>(&me.ctl->q_head, total) : 0u;
    st_relaxed<false>(&me.ctl->mtiles_total, mt);
  }
  epi_bar();
  const uint32_t total = sc.q_total, t0 = sc.q_t0;
  for (uint32_t idx = etid; idx < total; idx += kEpiThreads) {
    int lo = 0, hi = p.El;  // largest e with pre[e] <= idx
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (sc.pre[mid] <= idx) lo = mid; else hi = mid;
    }
    const uint32_t e = (uint32_t)lo, r = idx - sc.pre[lo];
    const uint32_t full = sc.full_tiles[e], rem = sc.rem_rows[e];
    uint32_t j, n, rows;
    if (p.eager) {
      j = full; n = r; rows = rem;
    } else {
      j = r / nt1; n = r - j * nt1; rows = (j < full) ? 128u : rem;
    }
    FdmoeSlot* s = &me.slots[(t0 + idx) & (uint32_t)p.queue_mask];
    s->a = task_word(FDMOE_TASK_FFN1, e, n);
    s->b = j;
    s->c = rows;
    st_release<false>(&s->seq, t0 + idx + 1u);
  }
  epi_bar();
  if (etid == 0) {
    fence_acqrel<false>();
    st_release<false>(&me.ctl->flush_done, 1u);
    maybe_close(p);
  }
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  return g / (1.0f + __expf(-g)) * u;
}

// FFN1 epilogue: act[row, n*128 + c] = silu(D[row, c]) * D[row, 128 + c].
__device__ __forceinline__ void ffn1_epilogue(const FdmoeParams& p, uint32_t taddr, int q, int h,
                                              int lane, uint32_t e, uint32_t j, uint32_t n,
                                              uint32_t rows) {
  const uint32_t row = q * 32 + lane;
  bf16* dst = reinterpret_cast<bf16*>(p.act) +
              ((size_t)e * p.cap_rows + (size_t)j * 128 + row) * p.I + n * FDMOE_TILE_N1 + h * 64;
  const uint32_t tbase = taddr + ((uint32_t)(q * 32) << 16) + h * 64;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t g[32], u[32];
    ptx::tmem_ld_32x32(tbase + c * 32, g);
    ptx::tmem_ld_32x32(tbase + 128 + c * 32, u);
    ptx::tmem_ld_wait();
    if (row < rows) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const int i = v * 8 + w * 2;
          ow[w] = pack_bf16(silu_mul(__uint_as_float(g[i]), __uint_as_float(u[i])),
                            silu_mul(__uint_as_float(g[i + 1]), __uint_as_float(u[i + 1])));
        }
        *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = o;
      }
    }
  }
}

// FFN2 epilogue: y[token, slot, n*256 + c] = D[row, c] * routing weight, stored
// on the token's home rank.
__device__ __forceinline__ void ffn2_epilogue(const FdmoeParams& p, uint32_t taddr, int q, int h,
                                              int lane, uint32_t e, uint32_t j, uint32_t n,
                                              uint32_t rows) {
  const uint32_t row = q * 32 + lane;
  const bool valid = row < rows;
  float wgt = 0.f;
  bf16* dst = nullptr;
  if (valid) {
    const uint4 mraw = ld_cg_u4(&p.peers[p.rank].meta[(size_t)e * p.cap_rows + (size_t)j * 128 + row]);
    const int token = (int)mraw.x, home = (int)mraw.y >> 8, slot = (int)mraw.y & 0xff;
    wgt = __uint_as_float(mraw.z);
    dst = reinterpret_cast<bf16*>(p.peers[home].ystage) + ((size_t)token * p.K + slot) * p.H +
          n * FDMOE_TILE_N2 + h * 128;
  }
  const uint32_t tbase = taddr + ((uint32_t)(q * 32) << 16) + h * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t d[32];
    ptx::tmem_ld_32x32(tbase + c * 32, d);
    ptx::tmem_ld_wait();
    if (valid) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const int i = v * 8 + w * 2;
          ow[w] = pack_bf16(__uint_as_float(d[i]) * wgt, __uint_as_float(d[i + 1]) * wgt);
        }
        *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = o;
      }
    }
  }
}

// COMBINE: out[t, :] = sum over slots k = 0..K-1 (in that order, fp32) of
// y[t, k, :], for the tokens of one group.  One warp per token.
__device__ __forceinline__ void combine_task(const FdmoeParams& p, int ewarp, int lane, uint32_t g) {
  const int t_begin = (int)g * p.combine_group;
  const int t_end = min(t_begin + p.combine_group, p.T);
  const bf16* ys = reinterpret_cast<const bf16*>(p.peers[p.rank].ystage);
  bf16* out = reinterpret_cast<bf16*>(p.out);
  const int nvec = p.H / 8;
  for (int t = t_begin + ewarp; t < t_end; t += kEpiThreads / 32) {
    for (int v = lane; v < nvec; v += 32) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int k = 0; k < p.K; ++k) {
        const uint4 r = ld_cg_u4(ys + ((size_t)t * p.K + k) * p.H + v * 8);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] += bf16_lo(w[i]);
          acc[2 * i + 1] += bf16_hi(w[i]);
        }
      }
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]);
      o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]);
      o.w = pack_bf16(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + (size_t)t * p.H + v * 8) = o;
    }
  }
}

template <bool S>
__global__ void __launch_bounds__(kThreads, 1)
moe_persistent_kernel(const __grid_constant__ FdmoeParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128-byte-swizzled stages.
  uint8_t* stage = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  SmemCtl& sc = *reinterpret_cast<SmemCtl*>(stage + kStages * kStageBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const FdmoePeer& me = p.peers[p.rank];
  FdmoeCtl* ctl = me.ctl;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&sc.full_bar[s], 1);
      ptx::mbar_init(&sc.empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&sc.tmem_full[a], 1);
      ptx::mbar_init(&sc.tmem_empty[a], kEpiThreads / 32);
    }
    for (int r = 0; r < kRing; ++r) {
      ptx::mbar_init(&sc.ring_full[r], 1);
      ptx::mbar_init(&sc.ring_empty[r], 2 + kEpiThreads / 32);
    }
    sc.abort = 0;
    sc.flag = 0;
    sc.prof_n = 0;
    ptx::fence_mbar_init();
    st_relaxed<S>(&ctl->tokens_launch, (uint32_t)p.T);
  }
  if (warp == kWarpTmem) {
    ptx::tmem_alloc(&sc.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kWarpTma && lane == 0) {
    ptx::prefetch_tmap(&p.tm_packed);
    ptx::prefetch_tmap(&p.tm_w13);
    ptx::prefetch_tmap(&p.tm_act);
    ptx::prefetch_tmap(&p.tm_w2);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = sc.tmem_base;

  // ---- multi-GPU: announce this launch to the peers and wait (bounded) until
  // every peer has entered the same launch, i.e. has reset its counters.
  if (S && p.world > 1) {
    if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
      fence_acqrel<true>();
      ptx::st_release_sys(&p.peers[tid].ctl->ready[p.rank], p.epoch);
    }
    if (tid < p.world && tid != p.rank) {
      const uint64_t t0 = ptx::globaltimer_ns();
      while (ptx::ld_acquire_sys(&ctl->ready[tid]) != p.epoch) {
        if (sc.abort || ld_relaxed<true>(&ctl->closed) == 2u) break;
        if (ptx::globaltimer_ns() - t0 > p.timeout_ns) {
          raise_error(p, sc, FDMOE_ERR_TIMEOUT_PEER, (uint32_t)tid);
          break;
        }
        __nanosleep(200);
      }
    }
    __syncthreads();
  }

  // =============================== phase A: gate tiles, claimed dynamically
  if (p.mode != 2 && !sc.abort) {
    const int n_tiles = (p.T + FDMOE_GATE_TOKENS - 1) / FDMOE_GATE_TOKENS;
    if (n_tiles == 0 && blockIdx.x == 0 && tid == 0) gate_phase_finished<S>(p);
    for (;;) {
      if (tid == 0) sc.cur_tile = (int)atomicAdd(&ctl->gate_next, 1u);
      __syncthreads();
      const int tile = sc.cur_tile;
      if (tile >= n_tiles || sc.abort) break;
      gate_tile<S>(p, stage, sc, tile, n_tiles);
      __syncthreads();
    }
  }
  __syncthreads();

  // =============================== phase B: worker loop
  const uint32_t nt1 = (uint32_t)(p.I / FDMOE_TILE_N1), nt2 = (uint32_t)(p.H / FDMOE_TILE_N2);
  const uint32_t nkb1 = (uint32_t)(p.H / FDMOE_TILE_K), nkb2 = (uint32_t)(p.I / FDMOE_TILE_K);

  if (warp == kWarpSched) {
    if (lane == 0) {
      for (uint32_t it = 0;; ++it) {
        const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
        if (!wait_bar(p, sc, &sc.ring_empty[r], ph ^ 1u, FDMOE_ERR_TIMEOUT_RING)) {
          // The ring may be wedged: hand out EXIT through every slot that is free.
          break;
        }
        const FdmoeSlot t = queue_pop<S>(p, sc);
        sc.ring[r] = t;
        ptx::mbar_arrive(&sc.ring_full[r]);
        if ((t.a & 0xffu) == FDMOE_TASK_EXIT) break;
      }
    }
    __syncwarp();
  } else if (warp == kWarpTma) {
    if (lane == 0) {
      uint32_t stage_it = 0;
      for (uint32_t it = 0;; ++it) {
        const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
        if (!wait_bar(p, sc, &sc.ring_full[r], ph, FDMOE_ERR_TIMEOUT_RING)) break;
        const FdmoeSlot t = sc.ring[r];
        const uint32_t kind = t.a & 0xffu;
        if (kind == FDMOE_TASK_EXIT) break;
        if (kind == FDMOE_TASK_FFN1 || kind == FDMOE_TASK_FFN2) {
          const uint32_t e = (t.a >> 8) & 0xfffu, n = t.a >> 20, j = t.b;
          const bool f1 = kind == FDMOE_TASK_FFN1;
          const uint32_t nkb = f1 ? nkb1 : nkb2;
          const int32_t arow = (int32_t)(e * (uint32_t)p.cap_rows + j * 128u);
          ptx::fence_proxy_async();  // rows / activations were written with generic stores
          bool ok = true;
          for (uint32_t kb = 0; kb < nkb && ok; ++kb, ++stage_it) {
            const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
            ok = wait_bar(p, sc, &sc.empty_bar[s], sph ^ 1u, FDMOE_ERR_TIMEOUT_STAGE);
            if (!ok) break;
            uint8_t* sa = stage + s * kStageBytes;
            uint8_t* sb = sa + kStageA;
            ptx::mbar_expect_tx(&sc.full_bar[s], kStageBytes);
            const int32_t kx = (int32_t)(kb * FDMOE_TILE_K);
            if (f1) {
              ptx::tma_load_2d(sa, &p.tm_packed, &sc.full_bar[s], kx, arow);
              const int32_t brow = (int32_t)(e * 2u * (uint32_t)p.I + n * FDMOE_TILE_N1);
              ptx::tma_load_2d(sb, &p.tm_w13, &sc.full_bar[s], kx, brow);
              ptx::tma_load_2d(sb + kStageA, &p.tm_w13, &sc.full_bar[s], kx, brow + p.I);
            } else {
              ptx::tma_load_2d(sa, &p.tm_act, &sc.full_bar[s], kx, arow);
              const int32_t brow = (int32_t)(e * (uint32_t)p.H + n * FDMOE_TILE_N2);
              ptx::tma_load_2d(sb, &p.tm_w2, &sc.full_bar[s], kx, brow);
            }
          }
          if (!ok) break;
        }
        ptx::mbar_arrive(&sc.ring_empty[r]);
      }
    }
    __syncwarp();
  } else if (warp == kWarpMma) {
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_bf16(128, 256);
      uint32_t stage_it = 0, tile_it = 0;
      for (uint32_t it = 0;; ++it) {
        const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
        if (!wait_bar(p, sc, &sc.ring_full[r], ph, FDMOE_ERR_TIMEOUT_RING)) break;
        const FdmoeSlot t = sc.ring[r];
        const uint32_t kind = t.a & 0xffu;
        if (kind == FDMOE_TASK_EXIT) break;
        if (kind == FDMOE_TASK_FFN1 || kind == FDMOE_TASK_FFN2) {
          const uint32_t nkb = (kind == FDMOE_TASK_FFN1) ? nkb1 : nkb2;
          const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
          ++tile_it;
          if (!wait_bar(p, sc, &sc.tmem_empty[acc], aph ^ 1u, FDMOE_ERR_TIMEOUT_TMEM)) break;
          ptx::tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + acc * kAccCols;
          bool ok = true;
          for (uint32_t kb = 0; kb < nkb; ++kb, ++stage_it) {
            const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
            ok = wait_bar(p, sc, &sc.full_bar[s], sph, FDMOE_ERR_TIMEOUT_STAGE);
            if (!ok) break;
            ptx::tcgen05_fence_after();
            const uint32_t sa = ptx::smem_u32(stage + s * kStageBytes);
            const uint64_t da = ptx::make_smem_desc_sw128(sa);
            const uint64_t db = ptx::make_smem_desc_sw128(sa + kStageA);
#pragma unroll
            for (uint32_t k4 = 0; k4 < FDMOE_TILE_K / 16; ++k4) {
              // +32 bytes per 16-element k step inside the 128-byte swizzle row
              ptx::umma_bf16(d_tmem, da + k4 * 2u, db + k4 * 2u, idesc, (kb | k4) != 0u);
            }
            ptx::umma_commit(&sc.empty_bar[s]);  // frees the stage when the MMAs have read it
          }
          if (!ok) break;
          ptx::umma_commit(&sc.tmem_full[acc]);
        }
        ptx::mbar_arrive(&sc.ring_empty[r]);
      }
    }
    __syncwarp();
  } else if (warp >= kWarpEpi0) {
    const int etid = tid - kWarpEpi0 * 32, ewarp = warp - kWarpEpi0;
    const int q = warp & 3, h = ewarp >> 2;
    uint32_t tile_it = 0;
    for (uint32_t it = 0;; ++it) {
      const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
      // the group leaves together: a lone warp breaking out would strand the
      // others at the next group barrier
      if (!epi_vote_all(wait_bar(p, sc, &sc.ring_full[r], ph, FDMOE_ERR_TIMEOUT_RING))) break;
      const FdmoeSlot t = sc.ring[r];
      const uint32_t kind = t.a & 0xffu;
      if (kind == FDMOE_TASK_EXIT) break;
      const uint32_t e = (t.a >> 8) & 0xfffu, n = t.a >> 20, j = t.b, rows = t.c;
      const uint32_t pt0 = (p.prof && etid == 0) ? prof_now() : 0u;
      uint32_t pt1 = pt0;
      if (kind == FDMOE_TASK_FFN1 || kind == FDMOE_TASK_FFN2) {
        const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
        ++tile_it;
        if (!epi_vote_all(wait_bar(p, sc, &sc.tmem_full[acc], aph, FDMOE_ERR_TIMEOUT_TMEM))) break;
        if (p.prof && etid == 0) pt1 = prof_now();
        ptx::tcgen05_fence_after();
        const uint32_t taddr = tmem_base + acc * kAccCols;
        if (kind == FDMOE_TASK_FFN1)
          ffn1_epilogue(p, taddr, q, h, lane, e, j, n, rows);
        else
          ffn2_epilogue(p, taddr, q, h, lane, e, j, n, rows);
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sc.tmem_empty[acc]);

        if (kind == FDMOE_TASK_FFN1) {
          ptx::fence_proxy_async();  // the activation tile is read by TMA in FFN2
          epi_bar();
          if (etid == 0 && p.mode != 2) {
            fence_acqrel<false>();
            const uint32_t prev = atomicAdd(&p.ffn1_done[(size_t)e * p.MT + j], 1u);
            if (prev == nt1 - 1u) {
              fence_acqrel<false>();
              queue_push<false>(p, me, nt2, [&](uint32_t i, uint32_t& a, uint32_t& b, uint32_t& c) {
                a = task_word(FDMOE_TASK_FFN2, e, i);
                b = j;
                c = rows;
              });
            }
          }
        } else {
          epi_bar();
          if (etid == 0) {
            int last = 0;
            if (p.mode != 2) {
              fence_acqrel<S>();
              const uint32_t prev = atomicAdd(&p.ffn2_done[(size_t)e * p.MT + j], 1u);
              fence_acqrel<S>();
              last = prev == nt2 - 1u;
            }
            sc.flag = last;
          }
          epi_bar();
          if (sc.flag) {
            // every hidden-column tile of this m-tile is stored: tell the home ranks
            if ((uint32_t)etid < rows) {
              const uint4 mraw = ld_cg_u4(&me.meta[(size_t)e * p.cap_rows + (size_t)j * 128 + etid]);
              const int token = (int)mraw.x, home = (int)mraw.y >> 8;
              const uint32_t g = (uint32_t)(token / p.combine_group);
              const FdmoePeer& hp = p.peers[home];
              fence_acqrel<S>();
              const uint32_t prev = atom_add<S>(&hp.tok_arrivals[g], 1u);
              const int th = (home == p.rank) ? p.T : (int)ld_relaxed<S>(&hp.ctl->tokens_launch);
              const int gt = min(p.combine_group, th - (int)g * p.combine_group);
              if (prev + 1u == (uint32_t)(gt * p.K)) {
                fence_acqrel<S>();
                queue_push<S>(p, hp, 1u, [&](uint32_t, uint32_t& a, uint32_t& b, uint32_t& c) {
                  a = FDMOE_TASK_COMBINE;
                  b = g;
                  c = 0;
                });
              }
            }
            epi_bar();
            if (etid == 0) {
              atomicAdd(&ctl->mtiles_done, 1u);
              maybe_close(p);
            }
          }
        }
      } else if (kind == FDMOE_TASK_COMBINE) {
        combine_task(p, ewarp, lane, j);
        epi_bar();
        if (etid == 0 && p.mode != 2) {
          const int t_begin = (int)j * p.combine_group;
          const int cnt = min(p.combine_group, p.T - t_begin);
          fence_acqrel<false>();
          atomicAdd(&ctl->tokens_combined, (uint32_t)cnt);
          maybe_close(p);
        }
      } else if (kind == FDMOE_TASK_FLUSH) {
        flush_task<S>(p, sc, etid);
      } else if (kind == FDMOE_TASK_TESTA || kind == FDMOE_TASK_TESTB) {
        // task-system self test: two dependent stages over a 256-element chunk
        int* ptr = p.test_buf + (size_t)j * kEpiThreads + etid;
        if (kind == FDMOE_TASK_TESTA) {
          *ptr = __ldcg(ptr) * 2;
          epi_bar();
          if (etid == 0) {
            fence_acqrel<false>();
            queue_push<false>(p, me, 1u, [&](uint32_t, uint32_t& a, uint32_t& b, uint32_t& c) {
              a = FDMOE_TASK_TESTB;
              b = j;
              c = 0;
            });
          }
        } else {
          *ptr = __ldcg(ptr) + 1;
        }
      } else {
        if (etid == 0) raise_error(p, sc, FDMOE_ERR_BAD_TASK, t.a);
      }
      if (p.mode == 2) {
        epi_bar();
        if (etid == 0) {
          fence_acqrel<false>();
          const uint32_t done = atomicAdd(&ctl->executed, 1u) + 1u;
          if (done == p.expected_static) st_release<false>(&ctl->closed, 1u);
        }
      }
      if (etid == 0) prof_event(p, sc, kind, pt0, pt1, prof_now());
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&sc.ring_empty[r]);
    }
  }

  // ---- teardown
  __syncthreads();
  if (sc.abort) {
    // give loads and MMAs that may still be in flight time to land before the
    // shared memory and TMEM of this CTA are released
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == kWarpTmem) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0) {
    fence_acqrel<false>();
    const uint32_t prev = atomicAdd(&ctl->exit_cnt, 1u);
    if (prev == gridDim.x - 1u) {
      // last CTA out: every pushed task was consumed, tickets taken by workers
      // that left on `closed` are skipped, and the rank is reopened for the next
      // launch (an aborted launch stays closed until the host re-creates it).
      fence_acqrel<false>();
      const uint32_t tail = ld_relaxed<false>(&ctl->q_tail);
      st_relaxed<false>(&ctl->q_head, tail);
      st_relaxed<false>(&ctl->exit_cnt, 0u);
      if (ld_relaxed<false>(&ctl->closed) == 1u) st_relaxed<false>(&ctl->closed, 0u);
    }
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst,
                                        uint64_t n) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n;
       i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}
__global__ void cast_bf16_to_f32_kernel(const bf16* __restrict__ src, float* __restrict__ dst,
                                        uint64_t n) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n;
       i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = __bfloat162float(src[i]);
}

}  // namespace fdmoe

// ======================================================== thin C ABI (host)
extern "C" int fdmoe_kernel_prepare(int* smem_bytes_out, int* grid_out) {
  using namespace fdmoe;
  cudaError_t err;
  err = cudaFuncSetAttribute(moe_persistent_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemBytes);
  if (err != cudaSuccess) return (int)err;
  err = cudaFuncSetAttribute(moe_persistent_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemBytes);
  if (err != cudaSuccess) return (int)err;
  int dev = 0, sms = 0, occ = 0;
  if ((err = cudaGetDevice(&dev)) != cudaSuccess) return (int)err;
  if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
    return (int)err;
  err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, moe_persistent_kernel<false>, kThreads,
                                                      kSmemBytes);
  if (err != cudaSuccess) return (int)err;
  if (occ < 1) return (int)cudaErrorLaunchOutOfResources;
  if (smem_bytes_out) *smem_bytes_out = kSmemBytes;
  if (grid_out) *grid_out = sms;  // one worker per SM
  return 0;
}

extern "C" int fdmoe_kernel_launch(const FdmoeParams* params, int grid, void* stream) {
  using namespace fdmoe;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (params->world > 1)
    moe_persistent_kernel<true><<<grid, kThreads, kSmemBytes, st>>>(*params);
  else
    moe_persistent_kernel<false><<<grid, kThreads, kSmemBytes, st>>>(*params);
  return (int)cudaGetLastError();
}

extern "C" int fdmoe_cast_f32_to_bf16(const float* src, void* dst, uint64_t n, void* stream) {
  if (n == 0) return 0;
  const int blocks = (int)((n + 1023) / 1024 < 148 * 8 ? (n + 1023) / 1024 : 148 * 8);
  fdmoe::cast_f32_to_bf16_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<fdmoe::bf16*>(dst), n);
  return (int)cudaGetLastError();
}

extern "C" int fdmoe_cast_bf16_to_f32(const void* src, float* dst, uint64_t n, void* stream) {
  if (n == 0) return 0;
  const int blocks = (int)((n + 1023) / 1024 < 148 * 8 ? (n + 1023) / 1024 : 148 * 8);
  fdmoe::cast_bf16_to_f32_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const fdmoe::bf16*>(src), dst, n);
  return (int)cudaGetLastError();
}
