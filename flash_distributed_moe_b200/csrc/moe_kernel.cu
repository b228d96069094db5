// The persistent MoE-layer kernel for sm_100a and its thin C ABI.
//
// One CTA per SM, every CTA a worker that pulls tasks from a ticket-based global
// queue and overlaps four kinds of work:
//   GATE    128-token tile: gate GEMM on tcgen05, top-k, fp64 softmax, row
//           reservation in the owners' expert buffers (tokens whose leading
//           logits are nearly tied are recomputed with fp32 FMAs in the
//           reference's accumulation order, so the selection is the reference's);
//   PACK    16-token group: copies the token rows to their K destinations;
//   FFN1/2  128-row expert tiles on tcgen05 with TMEM accumulators fed by TMA
//           (SwiGLU epilogue; routing-weight epilogue stored on the home rank);
//   COMBINE token group: ordered sum of the K weighted rows.
// Cross-GPU traffic is plain stores and scoped atomics into peers' symmetric
// buffers.
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
#include <stddef.h>
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
  int32_t flag;
  uint32_t q_t0;
  uint32_t q_total;
  uint32_t prof_n;
  uint32_t n_flagged;
  // flush scratch (per local expert)
  uint32_t pre[132];
  uint32_t full_tiles[128];
  uint32_t rem_rows[128];
  // The epilogue group runs one task at a time, so the scratch of a GATE task
  // and the store staging of an FFN task share storage.  16-byte aligned: the
  // staging buffer is accessed with 16-byte vector loads and stores.
  union alignas(16) {
    struct {
      // gate-tile scratch (per expert / per token of the tile)
      uint32_t cnt[128];
      uint32_t base[128];
      uint32_t flagged[FDMOE_GATE_TOKENS];
      float exact[8][128];                      // exact logits of the tokens being recomputed
      float half_v[2][FDMOE_GATE_TOKENS][9];    // top-9 of each 64-column half
      uint8_t half_i[2][FDMOE_GATE_TOKENS][12];
      float top_v[FDMOE_GATE_TOKENS][9];        // merged top-9 logits, descending
      uint8_t top_i[FDMOE_GATE_TOKENS][12];
      float tk_w[FDMOE_GATE_TOKENS][FDMOE_MAX_TOPK];
      uint8_t lpos[FDMOE_GATE_TOKENS][FDMOE_MAX_TOPK];
    };
    // FFN epilogues: per-warp staging of a 32-row x 64-byte chunk (80-byte pitch
    // keeps the 16-byte accesses of a quarter warp on distinct banks)
    uint8_t store_stage[kEpiThreads / 32][32 * 80];
  };
};

constexpr int kSmemBytes = kStages * kStageBytes + (int)sizeof(SmemCtl) + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA exceeds the sm_100 limit");
static_assert(offsetof(SmemCtl, store_stage) % 16 == 0 && (32 * 80) % 16 == 0 && 80 % 16 == 0,
              "store staging must keep 16-byte alignment for every warp and row");
static_assert(offsetof(SmemCtl, full_bar) % 8 == 0 && offsetof(SmemCtl, ring) % 16 == 0, "barrier / ring alignment");

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

// Single timestamp mark (trace builds of the analysis only; one writer thread).
__device__ __forceinline__ void prof_mark(const FdmoeParams& p, SmemCtl& sc, int etid, uint32_t id) {
  if (p.prof && etid == 0) prof_event(p, sc, 200u + id, prof_now(), 0u, 0u);
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

// Every token of this rank is packed (all its rows are written and fenced):
// tell every rank; whoever completes a rank's count asks it to flush.
template <bool S>
__device__ void gate_phase_finished(const FdmoeParams& p) {
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

// ===================================================================== GATE
// Top-9 of the 64 logits one thread holds (columns c0..c0+63 of its token row,
// as two raw 32-word TMEM loads), descending, the lower column winning ties.
// Branch-free selection rounds; a selected entry is replaced by -inf.
__device__ __forceinline__ void top9_of_64(uint32_t (&lo)[32], uint32_t (&hi)[32], int c0, int E, float (&tv)[9],
                                           int (&ti)[9]) {
  const uint32_t ninf = 0xff800000u;
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    if (c0 + c >= E) lo[c] = ninf;
    if (c0 + 32 + c >= E) hi[c] = ninf;
  }
#pragma unroll
  for (int r = 0; r < 9; ++r) {
    float b0 = -INFINITY, b1 = -INFINITY;
    int i0 = 255, i1 = 255;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const float f0 = __uint_as_float(lo[c]), f1 = __uint_as_float(hi[c]);
      const bool g0 = f0 > b0;
      b0 = g0 ? f0 : b0;
      i0 = g0 ? c : i0;
      const bool g1 = f1 > b1;
      b1 = g1 ? f1 : b1;
      i1 = g1 ? 32 + c : i1;
    }
    const bool up = b1 > b0;  // the upper chain wins only when strictly greater
    const float bv = up ? b1 : b0;
    const int bi = up ? i1 : i0;
    tv[r] = bv;
    ti[r] = bi == 255 ? 255 : c0 + bi;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      if (c == bi) lo[c] = ninf;
      if (32 + c == bi) hi[c] = ninf;
    }
  }
}

// Exact gate logits of up to four tokens for one expert: fp32 FMAs with k
// strictly ascending per output (bf16 x bf16 products are exact in fp32, so this
// equals the reference's `acc += a*b` bit for bit; reference refGemm.h:16-27).
// The four accumulation chains are independent, which hides the FMA latency;
// the weight row is prefetched 64 elements ahead.
__device__ __forceinline__ void exact_logits4(const FdmoeParams& p, const int (&tok)[4], int e, float (&acc)[4]) {
  const int H = p.H;
  const uint4* w = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.gate_w) + (size_t)e * H);
  const uint4* x[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[i] = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.x) + (size_t)tok[i] * H);
    acc[i] = 0.f;
  }
  uint4 wc[8], wn[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) wc[u] = __ldg(w + u);
  const int nblk = H / 64;
  for (int blk = 0; blk < nblk; ++blk) {
    if (blk + 1 < nblk) {
#pragma unroll
      for (int u = 0; u < 8; ++u) wn[u] = __ldg(w + (blk + 1) * 8 + u);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t ww[4] = {wc[u].x, wc[u].y, wc[u].z, wc[u].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 xv = x[i][blk * 8 + u];
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i] = fmaf(bf16_lo(xw[j]), bf16_lo(ww[j]), acc[i]);
          acc[i] = fmaf(bf16_hi(xw[j]), bf16_hi(ww[j]), acc[i]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) wc[u] = wn[u];
  }
}

// Warp-wide top-k over 128 logits in shared memory (lane l owns experts l,
// l+32, l+64, l+96), descending, the lower index winning ties (reference
// refTopk.h:36-58).  Result: lane k < K holds slot k.
__device__ __forceinline__ void topk_warp(const float* logits, int E, int K, int lane, float& myv, int& myi) {
  float v[4];
  uint32_t taken = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = lane + 32 * i;
    v[i] = (e < E) ? logits[e] : -INFINITY;
    if (e >= E) taken |= 1u << i;
  }
  myv = 0.f;
  myi = 0;
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
}

// Epilogue of a GATE task (256 threads).  The accumulator holds the logits of
// 128 tokens (TMEM lanes) x 128 experts (columns) as computed by the tensor
// cores, whose accumulation order is not the reference's.  A token whose
// leading nine logits contain an adjacent pair closer than `tau` (2.5e-4 of the
// logit scale, an order of magnitude above the rounding noise of either
// accumulation order over a few thousand terms) is recomputed exactly; for all
// other tokens both orders select the same experts in the same order.
template <bool S>
__device__ __noinline__ void gate_epilogue(const FdmoeParams& p, SmemCtl& sc, uint32_t taddr, uint64_t* tmem_empty_bar,
                              int q, int h, int lane, int etid, int ewarp, uint32_t tile) {
  const int E = p.E, K = p.K;
  const int t0 = (int)tile * FDMOE_GATE_TOKENS;
  const int nt = min(FDMOE_GATE_TOKENS, p.T - t0);
  const int row = q * 32 + lane;

  if (etid < 128) sc.cnt[etid] = 0;
  if (etid == 0) sc.n_flagged = 0;
  {
    uint32_t vlo[32], vhi[32];
    const uint32_t tb = taddr + ((uint32_t)(q * 32) << 16) + h * 64;
    ptx::tmem_ld_32x32(tb, vlo);
    ptx::tmem_ld_32x32(tb + 32, vhi);
    ptx::tmem_ld_wait();
    ptx::tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(tmem_empty_bar);  // accumulator is free again
    if (p.debug_logits && row < nt) {
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        p.debug_logits[(size_t)(t0 + row) * 128 + h * 64 + c] = __uint_as_float(vlo[c]);
        p.debug_logits[(size_t)(t0 + row) * 128 + h * 64 + 32 + c] = __uint_as_float(vhi[c]);
      }
    }
    prof_mark(p, sc, etid, 1);
    float tv[9];
    int ti[9];
    top9_of_64(vlo, vhi, h * 64, E, tv, ti);
    prof_mark(p, sc, etid, 2);
#pragma unroll
    for (int j = 0; j < 9; ++j) {
      sc.half_v[h][row][j] = tv[j];
      sc.half_i[h][row][j] = (uint8_t)ti[j];
    }
  }
  epi_bar();
  {
    // merge by rank: position = own rank + number of partner entries ahead of it;
    // the lower half (lower expert indices) wins ties
    const int o = h ^ 1;
#pragma unroll
    for (int j = 0; j < 9; ++j) {
      const float mv = sc.half_v[h][row][j];
      int pos = j;
#pragma unroll
      for (int m = 0; m < 9; ++m) {
        const float ov = sc.half_v[o][row][m];
        pos += (h == 0) ? (ov > mv) : (ov >= mv);
      }
      if (pos < 9 && mv > -INFINITY) {
        sc.top_v[row][pos] = mv;
        sc.top_i[row][pos] = sc.half_i[h][row][j];
      }
    }
  }
  epi_bar();
  if (etid < nt) {
    // etid == row for the first four epilogue warps
    const int cand = min(E, 9);
    const float tau = 2.5e-4f * fmaxf(1.0f, fabsf(sc.top_v[etid][0]));
    bool tie = false;
    for (int j = 0; j + 1 < cand; ++j) tie |= (sc.top_v[etid][j] - sc.top_v[etid][j + 1]) < tau;
    if (tie) sc.flagged[atomicAdd(&sc.n_flagged, 1u)] = (uint32_t)etid;
  }
  epi_bar();
  prof_mark(p, sc, etid, 3);
  // exact recompute of the flagged tokens, eight per pass: each half of the
  // group takes four tokens, one expert per thread; then one warp per token selects
  {
    const uint32_t nf = sc.n_flagged;
    const int half = etid >> 7, e = etid & 127;
    for (uint32_t f0 = 0; f0 < nf; f0 += 8) {
      int tok[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t f = f0 + (uint32_t)(half * 4 + i);
        tok[i] = t0 + (int)sc.flagged[f < nf ? f : f0];  // out-of-range entries repeat a valid token
      }
      if (f0 + (uint32_t)(half * 4) < nf && e < E) {
        float acc[4];
        exact_logits4(p, tok, e, acc);
#pragma unroll
        for (int i = 0; i < 4; ++i) sc.exact[half * 4 + i][e] = acc[i];
      }
      epi_bar();
      if (f0 + (uint32_t)ewarp < nf) {
        const int tk = (int)sc.flagged[f0 + ewarp];
        float myv;
        int myi;
        topk_warp(sc.exact[ewarp], E, K, lane, myv, myi);
        if (lane < K) {
          sc.top_v[tk][lane] = myv;
          sc.top_i[tk][lane] = (uint8_t)myi;
        }
      }
      epi_bar();
    }
  }
  prof_mark(p, sc, etid, 4);
  if (etid < nt) {
    // softmax over the K kept logits, in double, in the reference's order: the
    // values are descending, so the running max is the first one and the sum is
    // 1 + e_1 + e_2 + ... (reference refSoftmax.h:23-50)
    const double m = (double)sc.top_v[etid][0];
    double ex[FDMOE_MAX_TOPK];
    double sum = 1.0;
#pragma unroll
    for (int k = 0; k < FDMOE_MAX_TOPK; ++k) {
      if (k < K) {
        ex[k] = exp((double)sc.top_v[etid][k] - m);
        if (k > 0) sum += ex[k];
      }
    }
#pragma unroll
    for (int k = 0; k < FDMOE_MAX_TOPK; ++k) {
      if (k < K) {
        const int e = sc.top_i[etid][k];
        const float w = (float)(ex[k] / sum);
        sc.tk_w[etid][k] = w;
        sc.lpos[etid][k] = (uint8_t)atomicAdd(&sc.cnt[e], 1u);
        p.topk_idx[(size_t)(t0 + etid) * K + k] = e;
        p.topk_w[(size_t)(t0 + etid) * K + k] = w;
      }
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 5);
  // reserve rows in the owners' expert buffers: one atomic per expert and tile
  if (etid < E) {
    const uint32_t cnt = sc.cnt[etid];
    if (cnt) {
      const int owner = etid / p.El, le = etid - owner * p.El;
      const uint32_t base = atom_add<S>(&p.peers[owner].expert_cnt[le], cnt);
      if (base + cnt > (uint32_t)p.cap_rows) raise_error(p, sc, FDMOE_ERR_ROW_OVERFLOW, etid);
      sc.base[etid] = base;
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 6);
  if (etid < nt && !sc.abort) {
    for (int k = 0; k < K; ++k) {
      const int e = sc.top_i[etid][k];
      const int owner = e / p.El, le = e - owner * p.El;
      const size_t rowg = (size_t)le * p.cap_rows + sc.base[e] + sc.lpos[etid][k];
      p.dest_row[(size_t)(t0 + etid) * K + k] = (int32_t)rowg;
      // FdmoeRowMeta {token, home << 8 | slot, weight, pad} as one 16-byte store
      *reinterpret_cast<uint4*>(&p.peers[owner].meta[rowg]) =
          make_uint4((uint32_t)(t0 + etid), (uint32_t)((p.rank << 8) | k), __float_as_uint(sc.tk_w[etid][k]), 0u);
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 7);
  if (etid == 0 && !sc.abort) {
    fence_acqrel<S>();
    const uint32_t ngroups = (uint32_t)((nt + FDMOE_PACK_TOKENS - 1) / FDMOE_PACK_TOKENS);
    queue_push<false>(p, p.peers[p.rank], ngroups, [&](uint32_t i, uint32_t& a, uint32_t& b, uint32_t& c) {
      a = FDMOE_TASK_PACK;
      b = (uint32_t)t0 + i * FDMOE_PACK_TOKENS;
      c = (uint32_t)min(FDMOE_PACK_TOKENS, nt - (int)i * FDMOE_PACK_TOKENS);
    });
  }
}

// ===================================================================== PACK
// Copies `count` token rows to their K destinations each (local stores or
// stores into a peer's expert buffer), one warp per token, then accounts for
// them.  In eager mode the writer that completes a 128-row tile publishes its
// FFN1 tasks on the owner's queue.
template <bool S>
__device__ __noinline__ void pack_task(const FdmoeParams& p, SmemCtl& sc, int etid, int ewarp, int lane, uint32_t t_first,
                          uint32_t count) {
  const int H = p.H, K = p.K;
  const bf16* x = reinterpret_cast<const bf16*>(p.x);
  // a warp takes tokens ewarp and ewarp + 8 of the group and keeps the loads of both in flight
  const bool has[2] = {(uint32_t)ewarp < count, (uint32_t)ewarp + 8u < count};
  // lane k < K keeps the destination of slot k of both tokens; broadcast by shuffle when needed
  int my_row[2] = {0, 0}, my_owner[2] = {0, 0};
  const uint4* src[2];
#pragma unroll
  for (int s2 = 0; s2 < 2; ++s2) {
    const uint32_t t = t_first + (uint32_t)ewarp + 8u * s2;
    src[s2] = reinterpret_cast<const uint4*>(x + (size_t)(has[s2] ? t : t_first) * H);
    if (has[s2] && lane < K) {
      my_row[s2] = __ldcg(&p.dest_row[(size_t)t * K + lane]);
      my_owner[s2] = __ldcg(&p.topk_idx[(size_t)t * K + lane]) / p.El;
    }
  }
  for (int vbase = 0; vbase < H / 8; vbase += 256) {
    uint4 r[2][8];
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int vi = vbase + lane + 32 * i;
        r[s2][i] = (has[s2] && vi < H / 8) ? src[s2][vi] : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
      for (int k = 0; k < K; ++k) {
        const int row = __shfl_sync(0xffffffffu, my_row[s2], k);
        const int owner = __shfl_sync(0xffffffffu, my_owner[s2], k);
        if (!has[s2]) continue;
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.peers[owner].packed) + (size_t)row * H);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int vi = vbase + lane + 32 * i;
          if (vi < H / 8) dst[vi] = r[s2][i];
        }
      }
    }
  }
  ptx::fence_proxy_async();  // packed rows are read by TMA
  epi_bar();
  if (p.eager && (uint32_t)etid < count * (uint32_t)K) {
    const uint32_t t = t_first + (uint32_t)etid / (uint32_t)K, k = (uint32_t)etid % (uint32_t)K;
    const int rowg = __ldcg(&p.dest_row[(size_t)t * K + k]);
    const int owner = __ldcg(&p.topk_idx[(size_t)t * K + k]) / p.El;
    const uint32_t le = (uint32_t)rowg / (uint32_t)p.cap_rows, pos = (uint32_t)rowg % (uint32_t)p.cap_rows;
    const uint32_t j = pos / 128u, nt1 = (uint32_t)(p.I / FDMOE_TILE_N1);
    fence_acqrel<S>();
    const uint32_t prev = atom_add<S>(&p.peers[owner].tile_landed[(size_t)le * p.MT + j], 1u);
    if (prev + 1u == 128u) {
      fence_acqrel<S>();
      queue_push<S>(p, p.peers[owner], nt1, [&](uint32_t i, uint32_t& a, uint32_t& b, uint32_t& c) {
        a = task_word(FDMOE_TASK_FFN1, le, i);
        b = j;
        c = 128u;
      });
    }
  }
  if (p.eager) epi_bar();
  if (etid == 0) {
    fence_acqrel<S>();
    const uint32_t done = atomicAdd(&p.peers[p.rank].ctl->pack_done, count) + count;
    if (done == (uint32_t)p.T) gate_phase_finished<S>(p);
  }
}

// ============================================================ FLUSH and FFN
// FLUSH: every rank's gate phase is complete, so the per-expert row counts are
// final.  Publishes FFN1 tasks for all tiles (or, in eager mode, only for the
// partial last tile of each expert), ordered by expert so that tiles sharing
// weights run close together.  Executed by the 256 epilogue threads.
template <bool S>
__device__ __noinline__ void flush_task(const FdmoeParams& p, SmemCtl& sc, int etid) {
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
  }
  // one fence orders every payload above before every sequence word below
  fence_acqrel<false>();
  for (uint32_t idx = etid; idx < total; idx += kEpiThreads)
    st_relaxed<false>(&me.slots[(t0 + idx) & (uint32_t)p.queue_mask].seq, t0 + idx + 1u);
  epi_bar();
  if (etid == 0) {
    fence_acqrel<false>();
    st_release<false>(&me.ctl->flush_done, 1u);
    maybe_close(p);
  }
}

// silu(g) * u with the fast exponential and reciprocal (relative error ~1e-6, far
// below the bf16 rounding of the stored activation); g -> -inf gives -0.
__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

// Writes one 32-row x 64-byte chunk held as 16 packed words per thread (thread
// = row) through the warp's staging buffer so that every global store
// instruction covers 8 rows x 64 contiguous bytes instead of 32 rows x 16.
// dst[i] / ok[i] describe row (lane >> 2) + 8 i: pointer to the chunk's first
// byte in global memory and whether the row exists.
__device__ __forceinline__ void store_chunk_coalesced(uint8_t* st, int lane, const uint32_t (&o)[16],
                                                      uint8_t* const (&dst)[4], const bool (&ok)[4]) {
  uint4* mine = reinterpret_cast<uint4*>(st + lane * 80);
#pragma unroll
  for (int v = 0; v < 4; ++v) mine[v] = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
  __syncwarp();
  const int piece = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = (lane >> 2) + 8 * i;
    const uint4 val = *reinterpret_cast<const uint4*>(st + r * 80 + piece * 16);
    if (ok[i]) *reinterpret_cast<uint4*>(dst[i] + piece * 16) = val;
  }
  __syncwarp();
}

// FFN1 epilogue: act[row, n*128 + c] = silu(D[row, c]) * D[row, 128 + c].
__device__ __forceinline__ void ffn1_epilogue(const FdmoeParams& p, SmemCtl& sc, uint32_t taddr, int q, int h,
                                              int lane, int ewarp, uint32_t e, uint32_t j, uint32_t n,
                                              uint32_t rows) {
  uint8_t* st = sc.store_stage[ewarp];
  uint8_t* dst[4];
  bool ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t r = q * 32 + (lane >> 2) + 8 * i;
    ok[i] = r < rows && !(p.debug_flags & 1);
    dst[i] = reinterpret_cast<uint8_t*>(reinterpret_cast<bf16*>(p.act) +
                                        ((size_t)e * p.cap_rows + (size_t)j * 128 + r) * p.I +
                                        n * FDMOE_TILE_N1 + h * 64);
  }
  const uint32_t tbase = taddr + ((uint32_t)(q * 32) << 16) + h * 64;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t g[32], u[32], o[16];
    ptx::tmem_ld_32x32(tbase + c * 32, g);
    ptx::tmem_ld_32x32(tbase + 128 + c * 32, u);
    ptx::tmem_ld_wait();
    prof_mark(p, sc, ewarp * 32 + lane, 10 + c * 3);
#pragma unroll
    for (int w = 0; w < 16; ++w)
      o[w] = pack_bf16(silu_mul(__uint_as_float(g[2 * w]), __uint_as_float(u[2 * w])),
                       silu_mul(__uint_as_float(g[2 * w + 1]), __uint_as_float(u[2 * w + 1])));
    uint8_t* d2[4] = {dst[0] + c * 64, dst[1] + c * 64, dst[2] + c * 64, dst[3] + c * 64};
    prof_mark(p, sc, ewarp * 32 + lane, 11 + c * 3);
    store_chunk_coalesced(st, lane, o, d2, ok);
    prof_mark(p, sc, ewarp * 32 + lane, 12 + c * 3);
  }
}

// FFN2 epilogue: y[token, slot, n*256 + c] = D[row, c] * routing weight, stored
// on the token's home rank.
__device__ __forceinline__ void ffn2_epilogue(const FdmoeParams& p, SmemCtl& sc, uint32_t taddr, int q, int h,
                                              int lane, int ewarp, uint32_t e, uint32_t j, uint32_t n,
                                              uint32_t rows) {
  uint8_t* st = sc.store_stage[ewarp];
  const uint32_t row = q * 32 + lane;
  float wgt = 0.f;
  unsigned long long myptr = 0ull;
  if (row < rows) {
    const uint4 mraw = ld_cg_u4(&p.peers[p.rank].meta[(size_t)e * p.cap_rows + (size_t)j * 128 + row]);
    const int token = (int)mraw.x, home = (int)mraw.y >> 8, slot = (int)mraw.y & 0xff;
    wgt = __uint_as_float(mraw.z);
    myptr = reinterpret_cast<unsigned long long>(reinterpret_cast<bf16*>(p.peers[home].ystage) +
                                                 ((size_t)token * p.K + slot) * p.H + n * FDMOE_TILE_N2 + h * 128);
  }
  uint8_t* dst[4];
  bool ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const unsigned long long pp = __shfl_sync(0xffffffffu, myptr, (lane >> 2) + 8 * i);
    dst[i] = reinterpret_cast<uint8_t*>(pp);
    ok[i] = pp != 0ull && !(p.debug_flags & 1);
  }
  const uint32_t tbase = taddr + ((uint32_t)(q * 32) << 16) + h * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t d[32], o[16];
    ptx::tmem_ld_32x32(tbase + c * 32, d);
    ptx::tmem_ld_wait();
#pragma unroll
    for (int w = 0; w < 16; ++w)
      o[w] = pack_bf16(__uint_as_float(d[2 * w]) * wgt, __uint_as_float(d[2 * w + 1]) * wgt);
    uint8_t* d2[4] = {dst[0] + c * 64, dst[1] + c * 64, dst[2] + c * 64, dst[3] + c * 64};
    store_chunk_coalesced(st, lane, o, d2, ok);
  }
}

// COMBINE: out[t, :] = sum over slots k = 0..K-1 (in that order, fp32) of
// y[t, k, :], for the tokens of one group.  One warp per token; the K loads of
// a 16-byte column vector are issued together, then summed in slot order.
__device__ __noinline__ void combine_task(const FdmoeParams& p, int ewarp, int lane, uint32_t g) {
  const int t_begin = (int)g * p.combine_group;
  const int t_end = min(t_begin + p.combine_group, p.T);
  const bf16* ys = reinterpret_cast<const bf16*>(p.peers[p.rank].ystage);
  bf16* out = reinterpret_cast<bf16*>(p.out);
  const int nvec = p.H / 8, K = p.K;
  for (int t = t_begin + ewarp; t < t_end; t += kEpiThreads / 32) {
    const bf16* yt = ys + (size_t)t * K * p.H;
    for (int v = lane; v < nvec; v += 64) {
      const bool two = v + 32 < nvec;
      uint4 r0[FDMOE_MAX_TOPK], r1[FDMOE_MAX_TOPK];
#pragma unroll
      for (int k = 0; k < FDMOE_MAX_TOPK; ++k) {
        if (k < K) {
          r0[k] = ld_cg_u4(yt + (size_t)k * p.H + v * 8);
          if (two) r1[k] = ld_cg_u4(yt + (size_t)k * p.H + (v + 32) * 8);
        }
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (half == 1 && !two) break;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
        for (int k = 0; k < FDMOE_MAX_TOPK; ++k) {
          if (k < K) {
            const uint4 r = half ? r1[k] : r0[k];
            const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              acc[2 * i] += bf16_lo(w[i]);
              acc[2 * i + 1] += bf16_hi(w[i]);
            }
          }
        }
        uint4 o;
        o.x = pack_bf16(acc[0], acc[1]);
        o.y = pack_bf16(acc[2], acc[3]);
        o.z = pack_bf16(acc[4], acc[5]);
        o.w = pack_bf16(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(out + (size_t)t * p.H + (v + half * 32) * 8) = o;
      }
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
    ptx::prefetch_tmap(&p.tm_x);
    ptx::prefetch_tmap(&p.tm_gate);
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

  // ---- seed the queue: one GATE task per 128-token tile (nothing to gate: the
  // rank's "gate phase" is finished at once, it may still serve its peers)
  if (p.mode != 2 && !sc.abort && blockIdx.x == 0 && tid == 0) {
    const uint32_t n_tiles = (uint32_t)((p.T + FDMOE_GATE_TOKENS - 1) / FDMOE_GATE_TOKENS);
    if (n_tiles == 0) {
      gate_phase_finished<S>(p);
    } else {
      queue_push<false>(p, me, n_tiles, [](uint32_t i, uint32_t& a, uint32_t& b, uint32_t& c) {
        a = FDMOE_TASK_GATE;
        b = i;
        c = 0;
      });
    }
  }

  // =============================== worker loop
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
        if (kind == FDMOE_TASK_FFN1 || kind == FDMOE_TASK_FFN2 || kind == FDMOE_TASK_GATE) {
          const uint32_t e = (t.a >> 8) & 0xfffu, n = t.a >> 20, j = t.b;
          const bool f1 = kind == FDMOE_TASK_FFN1, gt = kind == FDMOE_TASK_GATE;
          const uint32_t nkb = (f1 || gt) ? nkb1 : nkb2;
          const int32_t arow = gt ? (int32_t)(j * FDMOE_GATE_TOKENS) : (int32_t)(e * (uint32_t)p.cap_rows + j * 128u);
          // bytes one GATE stage receives: both boxes are clamped to the tensor extents
          const uint32_t gate_bytes = (uint32_t)(min(128, p.T) + min(128, p.E)) * FDMOE_TILE_K * 2u;
          ptx::fence_proxy_async();  // rows / activations were written with generic stores
          bool ok = true;
          for (uint32_t kb = 0; kb < nkb && ok; ++kb, ++stage_it) {
            const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
            ok = wait_bar(p, sc, &sc.empty_bar[s], sph ^ 1u, FDMOE_ERR_TIMEOUT_STAGE);
            if (!ok) break;
            uint8_t* sa = stage + s * kStageBytes;
            uint8_t* sb = sa + kStageA;
            ptx::mbar_expect_tx(&sc.full_bar[s], gt ? gate_bytes : (uint32_t)kStageBytes);
            const int32_t kx = (int32_t)(kb * FDMOE_TILE_K);
            if (gt) {
              ptx::tma_load_2d(sa, &p.tm_x, &sc.full_bar[s], kx, arow);
              ptx::tma_load_2d(sb, &p.tm_gate, &sc.full_bar[s], kx, 0);
            } else if (f1) {
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
      constexpr uint32_t idesc256 = ptx::make_idesc_bf16(128, 256);
      constexpr uint32_t idesc128 = ptx::make_idesc_bf16(128, 128);
      uint32_t stage_it = 0, tile_it = 0;
      for (uint32_t it = 0;; ++it) {
        const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
        if (!wait_bar(p, sc, &sc.ring_full[r], ph, FDMOE_ERR_TIMEOUT_RING)) break;
        const FdmoeSlot t = sc.ring[r];
        const uint32_t kind = t.a & 0xffu;
        if (kind == FDMOE_TASK_EXIT) break;
        if (kind == FDMOE_TASK_FFN1 || kind == FDMOE_TASK_FFN2 || kind == FDMOE_TASK_GATE) {
          const uint32_t nkb = (kind == FDMOE_TASK_FFN2) ? nkb2 : nkb1;
          const uint32_t idesc = (kind == FDMOE_TASK_GATE) ? idesc128 : idesc256;
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
      if (kind == FDMOE_TASK_GATE) {
        const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
        ++tile_it;
        if (!epi_vote_all(wait_bar(p, sc, &sc.tmem_full[acc], aph, FDMOE_ERR_TIMEOUT_TMEM))) break;
        if (p.prof && etid == 0) pt1 = prof_now();
        ptx::tcgen05_fence_after();
        gate_epilogue<S>(p, sc, tmem_base + acc * kAccCols, &sc.tmem_empty[acc], q, h, lane, etid, ewarp, j);
      } else if (kind == FDMOE_TASK_PACK) {
        pack_task<S>(p, sc, etid, ewarp, lane, j, rows);
      } else if (kind == FDMOE_TASK_FFN1 || kind == FDMOE_TASK_FFN2) {
        const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
        ++tile_it;
        if (!epi_vote_all(wait_bar(p, sc, &sc.tmem_full[acc], aph, FDMOE_ERR_TIMEOUT_TMEM))) break;
        if (p.prof && etid == 0) pt1 = prof_now();
        ptx::tcgen05_fence_after();
        const uint32_t taddr = tmem_base + acc * kAccCols;
        if (kind == FDMOE_TASK_FFN1)
          ffn1_epilogue(p, sc, taddr, q, h, lane, ewarp, e, j, n, rows);
        else
          ffn2_epilogue(p, sc, taddr, q, h, lane, ewarp, e, j, n, rows);
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sc.tmem_empty[acc]);
        const uint32_t pta = (p.prof && etid == 0) ? prof_now() : 0u;

        if (kind == FDMOE_TASK_FFN1) {
          if (!(p.debug_flags & 4)) ptx::fence_proxy_async();  // the activation tile is read by TMA in FFN2
          prof_mark(p, sc, etid, 20);
          epi_bar();
          prof_mark(p, sc, etid, 21);
          if (etid == 0 && p.mode != 2) {
            if (!(p.debug_flags & 2)) fence_acqrel<false>();
            prof_mark(p, sc, etid, 22);
            const uint32_t prev = atomicAdd(&p.ffn1_done[(size_t)e * p.MT + j], 1u);
            prof_mark(p, sc, etid, 23);
            if (prev == nt1 - 1u) {
              if (!(p.debug_flags & 2)) fence_acqrel<false>();
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
              if (!(p.debug_flags & 2)) fence_acqrel<S>();
              const uint32_t prev = atomicAdd(&p.ffn2_done[(size_t)e * p.MT + j], 1u);
              if (!(p.debug_flags & 2)) fence_acqrel<S>();
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
        if (etid == 0) prof_event(p, sc, kind + 16u, pt1, pta, prof_now());
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
