// The persistent MoE-layer kernel for sm_100a and its thin C ABI.
//
// One CTA per SM, every CTA a worker that takes tasks from the rank's three task queues (queue 0:
// FFN2, COMBINE, GATEFIX, GATED; queue 1: FFN1; queue 2: DISPATCH) or claims the next GATE tile, and
// overlaps these kinds of work:
//   GATE     token tile: gate GEMM on tcgen05, top-k, softmax; indices and weights go to global
//            memory.  Tokens whose leading logits are nearly tied are recomputed by a GATEFIX task
//            with fp32 FMAs in the reference's accumulation order, so the selection is the
//            reference's;
//   DISPATCH the rows of one GATE tile: rows are reserved in the owners' expert buffers, every
//            token row is brought into shared memory once and goes out as K bulk copies, one per
//            selected expert, into the owner's buffer (local, or a peer's over NVLink);
//   FFN1/2   128-row expert tiles on tcgen05 with TMEM accumulators fed by TMA (SwiGLU epilogue;
//            routing-weight epilogue stored on the token's home rank).  The sender whose rows
//            complete a batch of m-tiles of an expert publishes the batch's FFN1 tiles on the
//            owner's queue; what is left when every rank has gated is published by the owner's
//            GATED task, expert by expert;
//   COMBINE  token group: ordered sum of the K weighted rows, published by whoever delivers the
//            group's last row.
// Cross-GPU traffic is plain stores, bulk stores and relaxed system-scope atomics into peers'
// symmetric buffers.  System-scope fences cost microseconds on this hardware (several times more
// while host copies are in flight), so they are issued once per task that talked to a peer, never
// per row or per tile of local work.
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
constexpr int kWarpTmem = 3;   // allocates / frees TMEM; completion warp in between
constexpr int kWarpEpi0 = 4;   // warps 4..11: epilogues and SIMT tasks
constexpr int kEpiThreads = 256;

constexpr int kStages = 4;
constexpr int kStageA = FDMOE_TILE_M * FDMOE_TILE_K * 2;  // 16 KB
constexpr int kStageB = 256 * FDMOE_TILE_K * 2;           // 32 KB
constexpr int kStageBytes = kStageA + kStageB;            // 48 KB
constexpr int kRing = 3;
constexpr int kFixBlocks = 3;  // k-blocks of gate weights per stage in a GATEFIX task (3 x 16 KB)
constexpr int kDone = 8;  // depth of the hand-off ring to the completion warp
constexpr int kTmemCols = 512;
constexpr int kAccCols = 256;

struct __align__(64) SmemCtl {
  uint64_t full_bar[kStages];
  uint64_t empty_bar[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t ring_full[kRing];
  uint64_t ring_empty[kRing];
  FdmoeSlot ring[kRing];
  uint64_t done_full[kDone];   // epilogue -> completion warp: a tile's stores are issued
  uint64_t done_empty[kDone];
  FdmoeSlot done_ring[kDone];
  uint32_t tmem_base;
  volatile uint32_t abort;
  volatile uint32_t skip_done;  // COMBINE / GATEFIX tasks finished by the epilogue warps
  int32_t flag;
  uint32_t q_t0;
  uint32_t q_total;
  uint32_t prof_n;
  uint32_t n_flagged;
  uint32_t pre[16];  // GATED scratch: per-warp totals
  uint32_t run_round2;  // set by a task body that found this rank's GATED round due: the group runs it next
  uint32_t batch_mt;    // m-tiles per publication batch of this launch (identical on all ranks)
  uint32_t tokens_all;  // tokens of all ranks this launch
  // The epilogue group runs one task at a time, so the scratch of a GATE task
  // and the store staging of an FFN task share storage.  16-byte aligned: the
  // staging buffer is accessed with 16-byte vector loads and stores.
  union alignas(16) {
    struct {
      // GATE task scratch (per expert / per token of the tile)
      uint32_t cnt[128];
      uint32_t base[128];
      uint32_t flagged[FDMOE_GATE_TOKENS];
      uint8_t isflag[FDMOE_GATE_TOKENS];
      float logit_tile[32][132];                // one 32-token quarter of the logits (padded rows)
      float top_v[FDMOE_GATE_TOKENS][9];        // top-9 logits per token, descending
      uint8_t top_i[FDMOE_GATE_TOKENS][12];
      float tk_w[FDMOE_GATE_TOKENS][FDMOE_MAX_TOPK];
      uint8_t lpos[FDMOE_GATE_TOKENS][FDMOE_MAX_TOPK];
    };
    struct {
      // GATEFIX task scratch: two token rows and their exact logits
      uint4 xrow[2][FDMOE_MAX_HIDDEN / 8];
      float exact[2][128];
      uint2 fix_dst[2][FDMOE_MAX_TOPK];         // {expert, row in the owner's buffers} of each slot, or {~0, 0}
    };
    // FFN epilogues: per-warp staging of 32 rows x 128 bytes (chunks swizzled within a row)
    uint8_t store_stage[kEpiThreads / 32][32 * 128];
  };
  // Copy of the kernel parameters for the task bodies that are compiled as separate functions:
  // there the parameter block is only reachable through a generic pointer, and every access to
  // the constant bank through one costs on the order of a hundred cycles; shared memory does not.
  // TMA descriptors are always taken from the original, so the copy leaves them out: it starts at
  // the member after them (see task_params()).
  alignas(64) uint8_t params_tail[sizeof(FdmoeParams) - offsetof(FdmoeParams, peers)];
};

// The parameter block as the out-of-line task bodies see it: every member from `peers` on is read
// from the shared-memory copy; the TMA descriptors in front of it are not part of the copy and must
// not be touched through this reference.
__device__ __forceinline__ const FdmoeParams& task_params(const SmemCtl& sc) {
  static_assert(offsetof(SmemCtl, params_tail) >= offsetof(FdmoeParams, peers), "the view must start inside SmemCtl");
  return *reinterpret_cast<const FdmoeParams*>(reinterpret_cast<const uint8_t*>(&sc) +
                                               (offsetof(SmemCtl, params_tail) - offsetof(FdmoeParams, peers)));
}

constexpr int kSmemBytes = kStages * kStageBytes + (int)sizeof(SmemCtl) + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA exceeds the sm_100 limit");
static_assert(offsetof(SmemCtl, xrow) % 16 == 0 && offsetof(SmemCtl, logit_tile) % 16 == 0 && (132 * 4) % 16 == 0,
              "vector accesses to the gate scratch need 16-byte alignment");
static_assert(offsetof(SmemCtl, store_stage) % 16 == 0, "store staging must keep 16-byte alignment");
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
__device__ __forceinline__ uint32_t atom_exch(uint32_t* p, uint32_t v) {
  uint32_t old;
  if (S)
    asm volatile("atom.acq_rel.sys.global.exch.b32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  else
    asm volatile("atom.acq_rel.gpu.global.exch.b32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
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

// Where a role gave up waiting (diagnostics, one record per CTA and warp):
// {error code, byte offset of the barrier inside SmemCtl, parity, microseconds waited}.
__device__ __noinline__ void record_stuck(const FdmoeParams& p, SmemCtl& sc, uint64_t* bar, uint32_t parity,
                                          uint32_t err_code, uint64_t waited_ns) {
  if (!p.stuck) return;
  uint32_t* r = p.stuck + ((size_t)blockIdx.x * 16 + (threadIdx.x >> 5)) * 4;
  r[0] = err_code;
  r[1] = (uint32_t)(reinterpret_cast<uint8_t*>(bar) - reinterpret_cast<uint8_t*>(&sc));
  r[2] = parity;
  r[3] = (uint32_t)(waited_ns / 1000ull);
}

// Bounded mbarrier wait.  Returns false (after raising the error) on timeout
// or when another role of this CTA has aborted.  `budgets`: how many wait budgets to allow (the
// roles that wait for the scheduler's next task allow two, so that a worker without work reports
// the scheduler's own time-out).
__device__ __forceinline__ bool wait_bar(const FdmoeParams& p, SmemCtl& sc, uint64_t* bar,
                                         uint32_t parity, uint32_t err_code, uint32_t budgets = 1u) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      const uint64_t waited = ptx::globaltimer_ns() - t0;
      if (sc.abort) {
        record_stuck(p, sc, bar, parity, err_code | 0x100u, waited);
        return false;
      }
      if (waited > budgets * p.timeout_ns) {
        record_stuck(p, sc, bar, parity, err_code, waited);
        raise_error(p, sc, err_code, (blockIdx.x << 8) | (threadIdx.x >> 5));
        return false;
      }
    }
  }
  return true;
}

// Same wait without raising an error: one budget's worth of polling.
__device__ __forceinline__ bool wait_idle(const FdmoeParams& p, SmemCtl& sc, uint64_t* bar, uint32_t parity) {
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (sc.abort || ptx::globaltimer_ns() - t0 > p.timeout_ns) return false;
      __nanosleep(200);
    }
  }
  return true;
}

// ------------------------------------------------------------- task queues
// A rank has three queues.  Producers (this rank's workers and, for queue slots in the symmetric
// arena, its peers) take `n` consecutive tickets with one atomic add on head, fill the slots,
// publish each with a store of ticket + 1 after one fence, and then add `n` to the queue's count of
// available tasks.  Consumers (this rank's workers only) first take one unit of that count (giving
// it back if there was none), and only then a ticket from tail: a consumer never holds a ticket
// for a task that does not exist yet, so it can always turn to another queue, and no
// compare-and-swap loop serialises the workers.
// `S`: the queue belongs to a peer (system-scope atomics and fence), else to this GPU.
template <bool S, class Gen>
__device__ __forceinline__ void queue_push(const FdmoeParams& p, const FdmoePeer& q, int qi, uint32_t n, Gen gen) {
  const uint32_t t0 = atom_add<S>(&q.ctl->q[qi].head, n);
  FdmoeSlot* slots = q.slots[qi];
  for (uint32_t i = 0; i < n; ++i) {
    FdmoeSlot* s = &slots[(t0 + i) & (uint32_t)p.queue_mask];
    uint32_t a, b, c;
    gen(i, a, b, c);
    s->a = a;
    s->b = b;
    s->c = c;
  }
  // one fence orders every payload (and whatever the caller wrote or observed before) ahead of
  // the sequence words; a release store per slot would pay for a fence each time
  fence_acqrel<S>();
  for (uint32_t i = 0; i < n; ++i) st_relaxed<S>(&slots[(t0 + i) & (uint32_t)p.queue_mask].seq, t0 + i + 1u);
  atom_add<S>(&q.ctl->q[qi].avail, n);
}

// Push onto the queue of rank `r`: system scope only when that is another GPU.
template <bool S, class Gen>
__device__ __forceinline__ void queue_push_rank(const FdmoeParams& p, int r, int qi, uint32_t n, Gen gen) {
  if (S && r != p.rank)
    queue_push<true>(p, p.peers[r], qi, n, gen);
  else
    queue_push<false>(p, p.peers[r], qi, n, gen);
}

__device__ __forceinline__ uint32_t task_word(uint32_t kind, uint32_t e, uint32_t n) {
  return kind | (e << 8) | (n << 20);
}

__device__ __forceinline__ FdmoeSlot exit_task() {
  FdmoeSlot out;
  out.seq = 0;
  out.a = FDMOE_TASK_EXIT;
  out.b = 0;
  out.c = 0;
  return out;
}

// Takes the oldest task of queue `qi` of this rank if there is one (single thread).  Returns
// false when the queue is empty (or on an error, with sc.abort raised).
template <bool S>
__device__ __forceinline__ bool try_pop(const FdmoeParams& p, SmemCtl& sc, int qi, FdmoeSlot& out) {
  const FdmoePeer& me = p.peers[p.rank];
  FdmoeQueueCtl* q = &me.ctl->q[qi];
  if ((int32_t)ld_relaxed<S>(&q->avail) <= 0) return false;
  if ((int32_t)atomicSub(&q->avail, 1u) <= 0) {
    atomicAdd(&q->avail, 1u);  // others were faster: give the unit back
    return false;
  }
  // one published task is ours: its ticket (tickets are published in order of completion of the
  // pushes, so the slot of this ticket may still be a moment away)
  const uint32_t t = atomicAdd(&q->tail, 1u);
  FdmoeSlot* s = &me.slots[qi][t & (uint32_t)p.queue_mask];
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (ld_acquire<S>(&s->seq) != t + 1u) {
    if ((++spins & 15u) == 0u) {
      if (sc.abort) return false;
      if (ptx::globaltimer_ns() - t0 > p.timeout_ns) {
        raise_error(p, sc, FDMOE_ERR_TIMEOUT_QUEUE, (blockIdx.x << 8) | 1u);
        return false;
      }
    }
  }
  out.seq = 0;
  out.a = s->a;
  out.b = s->b;
  out.c = s->c;
  return true;
}

// The next task of this worker (single thread).  On one GPU: a DISPATCH task first (everything else
// waits for rows), then queue 0, a GATE tile, queue 1.  With peers: queue 0 first, then a DISPATCH task
// unless enough workers are dispatching already (the links set the pace of the dispatch, a part of the
// workers saturates them while the others feed the tensor cores), then a GATE tile, then queue 1; both
// orders were measured on both set-ups and each is the faster one where it is used.
// Waits (bounded) while there is nothing to do and the rank's work is not finished.
template <bool S>
__device__ __forceinline__ FdmoeSlot next_task(const FdmoeParams& p, SmemCtl& sc, uint32_t gate_tiles) {
  FdmoeCtl* ctl = p.peers[p.rank].ctl;
  FdmoeSlot out;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (sc.abort) return exit_task();
    if (S && try_pop<S>(p, sc, 0, out)) return out;
    if ((int32_t)ld_relaxed<false>(&ctl->q[2].avail) > 0 && ld_relaxed<false>(&ctl->disp_active) < (uint32_t)p.disp_conc) {
      if (atomicAdd(&ctl->disp_active, 1u) < (uint32_t)p.disp_conc && try_pop<false>(p, sc, 2, out)) return out;
      atomicSub(&ctl->disp_active, 1u);
    }
    if (!S && try_pop<S>(p, sc, 0, out)) return out;
    if (gate_tiles != 0u && ld_relaxed<false>(&ctl->gate_next) < gate_tiles) {
      const uint32_t g = atomicAdd(&ctl->gate_next, 1u);
      if (g < gate_tiles) {
        out.seq = 0;
        out.a = FDMOE_TASK_GATE;
        out.b = g;
        out.c = 0;
        return out;
      }
    }
    if (try_pop<S>(p, sc, 1, out)) return out;
    if (ld_relaxed<false>(&ctl->closed) != 0u) return exit_task();
    if ((++spins & 15u) == 0u) {
      if (ptx::globaltimer_ns() - t0 > p.timeout_ns) {
        raise_error(p, sc, FDMOE_ERR_TIMEOUT_QUEUE, (blockIdx.x << 8));
        return exit_task();
      }
    }
    __nanosleep(spins < 64u ? 40 : 200);
  }
}

// Closes this rank's queues once GATED has run, every m-tile of its experts
// has finished FFN2 and every token of this rank has been combined.  Called
// after each of those three kinds of event; the sequentially-consistent fence
// guarantees that the last caller sees the other two conditions.
__device__ __forceinline__ void maybe_close(const FdmoeParams& p) {
  FdmoeCtl* ctl = p.peers[p.rank].ctl;
  fence_sc<false>();
  if (ld_relaxed<false>(&ctl->gated_done) == 0u) return;
  if (ld_relaxed<false>(&ctl->mtiles_done) != ld_relaxed<false>(&ctl->mtiles_total)) return;
  if (ld_relaxed<false>(&ctl->tokens_combined) != ld_relaxed<false>(&ctl->tokens_launch)) return;
  st_release<false>(&ctl->closed, 1u);
}

// m-tiles per publication batch of a launch with `tokens_all` tokens over all ranks.  A sender
// that completes a batch of an expert publishes its FFN1 tiles at once, so the tensor cores
// start while rows are still travelling; every batch of an expert re-reads the expert's weights,
// which is cheap when a rank holds few experts (their weights stay in L2) and expensive when it
// holds all of them.  One GPU: no batches, every expert is published whole once gating has
// finished.  More GPUs: about `world` batches per expert, at least two m-tiles each.
// A pure function of values every rank knows, so that all ranks agree.
__device__ __forceinline__ uint32_t batch_mt_of(const FdmoeParams& p, uint32_t tokens_all) {
  if (p.batch_mt > 0) return (uint32_t)min(p.batch_mt, p.MT);
  if (p.world == 1) return (uint32_t)p.MT;
  const uint32_t mt_expert = (uint32_t)(((uint64_t)tokens_all * p.K / p.E) / FDMOE_TILE_M);
  const uint32_t b = mt_expert / (uint32_t)p.world;
  if (b < 2u) return (uint32_t)p.MT;
  return min(min(b, 8u), (uint32_t)p.MT);
}

// Tokens of rank `r` in this launch.
__device__ __forceinline__ uint32_t tokens_of_rank(const FdmoeParams& p, int r) {
  if (r == p.rank) return (uint32_t)p.T;
  return ld_relaxed<false>(&p.peers[p.rank].ctl->tokens_of[p.epoch & 1u][r]);
}

// All rows [b * B * 128, (b + 1) * B * 128) of local expert `le` of rank `owner` have landed: the FFN1
// tiles of those B m-tiles go onto the owner's queue 1, m-tile major (single thread; the caller
// observed the landing counter, the fence inside the push orders the rows before the tasks).
template <bool S>
__device__ __forceinline__ void publish_batch(const FdmoeParams& p, int owner, uint32_t le, uint32_t b, uint32_t B) {
  const uint32_t nt1 = (uint32_t)(p.I / FDMOE_TILE_N1);
  queue_push_rank<S>(p, owner, 1, B * nt1, [&](uint32_t i, uint32_t& a, uint32_t& bb, uint32_t& c) {
    const uint32_t j = i / nt1;
    a = task_word(FDMOE_TASK_FFN1, le, i - j * nt1);
    bb = b * B + j;
    c = 128u;
  });
}

// `n` more rows [row0, row0 + n) of local expert `le` of rank `owner` have landed (n <= 128, the rows
// lie in one or two batches).  The caller has made the rows visible (fence) before.  Publishes
// every batch this completes.
template <bool S>
__device__ __forceinline__ void rows_landed(const FdmoeParams& p, uint32_t B, int owner, uint32_t le, uint32_t row0,
                                            uint32_t n) {
  const uint32_t RB = B * FDMOE_TILE_M;
  const FdmoePeer& op = p.peers[owner];
  const uint32_t b0 = row0 / RB;
  const uint32_t n0 = min(n, (b0 + 1u) * RB - row0);
  if (atom_add<S>(&op.landed[(size_t)le * p.MT + b0], n0) + n0 == RB) publish_batch<S>(p, owner, le, b0, B);
  if (n > n0) {
    if (atom_add<S>(&op.landed[(size_t)le * p.MT + b0 + 1u], n - n0) + (n - n0) == RB)
      publish_batch<S>(p, owner, le, b0 + 1u, B);
  }
}

// The routing of every token of this rank is decided and its rows have landed on their owners:
// tell every rank.  Whoever brings a rank's count to the world size hands it the GATED task (its
// row counts are final); if that is the caller's own rank and `sc` is given, the caller's
// epilogue group runs it next (flag run_round2).  Called by one full warp.
template <bool S>
__device__ __forceinline__ void gating_finished(const FdmoeParams& p, SmemCtl* sc, int lane) {
  fence_acqrel<S>();
  uint32_t prev = 0u;
  if (lane < p.world) prev = atom_add<S>(&p.peers[lane].ctl->ranks_gated, 1u);
  const bool last = lane < p.world && prev == (uint32_t)p.world - 1u;
  if (last) {
    if (sc && lane == p.rank)
      sc->run_round2 = 1u;
    else
      queue_push_rank<S>(p, lane, 0, 1u, [](uint32_t, uint32_t& a, uint32_t& b, uint32_t& c) {
        a = FDMOE_TASK_GATED;
        b = 0;
        c = 0;
      });
  }
  __syncwarp();
}

// Counts `n` tokens of this rank as gated; the caller has landed their rows.  Called by one full warp.
template <bool S>
__device__ __forceinline__ void count_gated(const FdmoeParams& p, SmemCtl& sc, int lane, uint32_t n) {
  uint32_t done = 0u;
  if (lane == 0) {
    fence_acqrel<false>();
    done = atomicAdd(&p.peers[p.rank].ctl->gated_tokens, n) + n;
  }
  done = __shfl_sync(0xffffffffu, done, 0);
  if (n && done == (uint32_t)p.T) gating_finished<S>(p, &sc, lane);
}

// Monotonic unsigned key of a float (larger float <=> larger key; -0 counts as +0).
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f + 0.0f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Warp-wide top-k of four rows of 128 logits at once (lane l owns experts l,
// l+32, l+64, l+96 of each row), descending, the lower index winning ties
// (reference refTopk.h:36-58).  Each round is one warp-wide max over the value
// keys and one warp-wide min over the indices that hold that value
// (redux.sync), for four independent rows.  Lane k < K ends up holding slot k.
__device__ __forceinline__ void topk_warp4(const float* r0, int pitch, int E, int K, int lane, float (&myv)[4],
                                           int (&myi)[4]) {
  uint32_t key[4][4];  // key 0 marks "taken / not an expert" (no finite float maps to it)
#pragma unroll
  for (int r = 0; r < 4; ++r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = lane + 32 * i;
      key[r][i] = (e < E) ? max(order_key(r0[r * pitch + e]), 1u) : 0u;
    }
    myv[r] = 0.f;
    myi[r] = 0;
  }
  for (int k = 0; k < K; ++k) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      // local best: ascending i is ascending expert index, strict '>' keeps the lower one
      uint32_t bk = key[r][0];
      int bi = 0;
#pragma unroll
      for (int i = 1; i < 4; ++i) {
        if (key[r][i] > bk) {
          bk = key[r][i];
          bi = i;
        }
      }
      const uint32_t m = __reduce_max_sync(0xffffffffu, bk);
      const uint32_t cand = (bk == m) ? (uint32_t)(lane + 32 * bi) : 0xffffffffu;
      const uint32_t win = __reduce_min_sync(0xffffffffu, cand);
      if ((win & 31u) == (uint32_t)lane) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if ((win >> 5) == (uint32_t)i) key[r][i] = 0u;
      }
      if (lane == k) {
        myv[r] = key_to_float(m);
        myi[r] = (int)win;
      }
    }
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
// cores, whose accumulation order is not the reference's.  Measured on B200 the
// two orders differ by at most 2.7e-9 * H of the logit scale.  A token whose
// leading nine logits contain an adjacent pair closer than tau = 3e-8 * H of the
// scale (more than five times that difference on each side) is handed to a
// GATEFIX task, which recomputes its logits in the reference's order; for every
// other token both orders select the same experts in the same order.
//
// The selection and the routing weights go to global memory, and a DISPATCH task for the tile's
// tokens onto queue 2.
template <bool S>
__device__ __noinline__ void gate_epilogue(const FdmoeParams& p, SmemCtl& sc, uint32_t taddr,
                                           uint64_t* tmem_empty_bar, int q, int h, int lane, int etid, int ewarp,
                                           uint32_t tile) {
  const int E = p.E, K = p.K;
  const int t0 = (int)tile * p.gate_rows;
  const int nt = min(p.gate_rows, p.T - t0);
  const int kk = min(E, 9);
  const int npass = p.gate_rows / 32;

  if (etid < 128) sc.cnt[etid] = 0;
  if (etid == 0) sc.n_flagged = 0;
  // ---- one pass per TMEM lane quadrant: the two warps that may read the
  // quadrant spill its 32 rows to shared memory, then every warp extracts the
  // top-9 of four rows with warp-wide arg-max rounds
  prof_mark(p, sc, etid, 40);
  if (q >= npass) {
    // this warp's TMEM lanes hold no token of the tile: it only has to release the accumulator
    ptx::tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(tmem_empty_bar);
  }
  for (int pass = 0; pass < npass; ++pass) {
    if (q == pass) {
      uint32_t v[32];
      const uint32_t tb = taddr + ((uint32_t)(q * 32) << 16) + h * 64;
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        ptx::tmem_ld_32x32(tb + c2 * 32, v);
        ptx::tmem_ld_wait();
        float* dst = &sc.logit_tile[lane][h * 64 + c2 * 32];
#pragma unroll
        for (int c = 0; c < 32; c += 4)
          *reinterpret_cast<uint4*>(dst + c) = make_uint4(v[c], v[c + 1], v[c + 2], v[c + 3]);
        if (p.debug_logits && q * 32 + lane < nt) {
#pragma unroll
          for (int c = 0; c < 32; ++c)
            p.debug_logits[(size_t)(t0 + q * 32 + lane) * 128 + h * 64 + c2 * 32 + c] = __uint_as_float(v[c]);
        }
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tmem_empty_bar);  // this warp is done with the accumulator
    }
    epi_bar();
    prof_mark(p, sc, etid, 41);
    {
      float myv[4];
      int myi[4];
      topk_warp4(sc.logit_tile[ewarp * 4], 132, E, kk, lane, myv, myi);
      if (lane < kk) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          sc.top_v[pass * 32 + ewarp * 4 + r][lane] = myv[r];
          sc.top_i[pass * 32 + ewarp * 4 + r][lane] = (uint8_t)myi[r];
        }
      }
    }
    epi_bar();
    prof_mark(p, sc, etid, 42);
  }
  prof_mark(p, sc, etid, 2);
  if (etid < FDMOE_GATE_TOKENS) {
    bool tie = false;
    if (etid < nt) {
      const float tau = 3e-8f * (float)p.H * fmaxf(1.0f, fabsf(sc.top_v[etid][0]));
      for (int j = 0; j + 1 < kk; ++j) tie |= (sc.top_v[etid][j] - sc.top_v[etid][j + 1]) < tau;
      if (tie) sc.flagged[atomicAdd(&sc.n_flagged, 1u)] = (uint32_t)etid;
    }
    sc.isflag[etid] = tie ? 1 : 0;
  }
  epi_bar();
  prof_mark(p, sc, etid, 3);
  // nearly tied tokens go to GATEFIX tasks right away (queue 0: idle workers take them at once),
  // so that they are re-gated while this tile dispatches its rows
  if (etid == 0 && !sc.abort) {
    const uint32_t nf = sc.n_flagged, nfix = (nf + 1u) / 2u;
    if (nfix) {
      queue_push<false>(p, p.peers[p.rank], 0, nfix, [&](uint32_t i, uint32_t& a, uint32_t& b, uint32_t& c) {
        a = FDMOE_TASK_GATEFIX;
        b = (uint32_t)t0 + sc.flagged[2 * i];
        c = (2 * i + 1 < nf) ? (uint32_t)t0 + sc.flagged[2 * i + 1] : 0xffffffffu;
      });
    }
  }
  if (etid < nt) {
    if (!sc.isflag[etid]) {
      // softmax over the K kept logits in the reference's order: the values are descending, so
      // the running max is the first one and the sum is 1 + e_1 + e_2 + ... (reference
      // refSoftmax.h:23-50, which works in double; fp32 with the accurate expf stays within 3e-7 of
      // it, far inside the 1e-5 the routing weights are held to, and costs a tenth of the time)
      const float m = sc.top_v[etid][0];
      float ex[FDMOE_MAX_TOPK];
      float sum = 1.0f;
#pragma unroll
      for (int k = 0; k < FDMOE_MAX_TOPK; ++k) {
        if (k < K) {
          ex[k] = expf(sc.top_v[etid][k] - m);
          if (k > 0) sum += ex[k];
        }
      }
#pragma unroll
      for (int k = 0; k < FDMOE_MAX_TOPK; ++k) {
        if (k < K) {
          p.topk_idx[(size_t)(t0 + etid) * K + k] = sc.top_i[etid][k];
          p.topk_w[(size_t)(t0 + etid) * K + k] = ex[k] / sum;
        }
      }
    }
    p.tok_flag[t0 + etid] = sc.isflag[etid];  // 1: the token's GATEFIX task routes and sends it
  }
  epi_bar();
  prof_mark(p, sc, etid, 5);
  if (etid == 0 && !sc.abort) {
    // (the fence inside the push orders the routing written by the other threads before the barrier
    // ahead of the task)
    queue_push<false>(p, p.peers[p.rank], 2, 1u, [&](uint32_t, uint32_t& a, uint32_t& b, uint32_t& c) {
      a = FDMOE_TASK_DISPATCH;
      b = (uint32_t)t0;
      c = (uint32_t)nt;
    });
  }
}

// ================================================================= DISPATCH
// Rows of a token tile that fit one pipeline stage (the stage holds whole token rows).
__device__ __forceinline__ uint32_t dispatch_rows_per_stage(int H) {
  return min(16u, (uint32_t)kStageBytes / ((uint32_t)H * 2u));
}

// Copies the rows of tokens [t0, t0 + nt) (nt <= 128) into the expert buffers of their owners.
// First the task reserves rows: one atomic per expert on the owner's row counter.  Rows are reserved
// when they are about to be sent, not when the tokens are gated, so that an expert's buffer fills in
// the order of the dispatch and its first batch of m-tiles is complete long before its last.
// Then the TMA warp brings the token rows (contiguous in the token matrix) into the pipeline stages;
// one thread per (row of the stage, slot) writes the row's sideband and sends the row to the expert's
// owner as one bulk copy (local, or a peer's memory over NVLink), so a token row is read once and
// written K times.  A stage goes back to the TMA warp as soon as the copies out of it have read
// their rows.  When all copies of the task are written, one thread per expert counts the task's rows
// as landed on their owner (one fence first) and publishes the FFN1 tiles of every batch this
// completes.  Returns false when the group has to give up.
template <bool S>
__device__ __noinline__ bool dispatch_task(const FdmoeParams& p, SmemCtl& sc, uint8_t* stage, uint32_t& stage_it,
                                           int etid, int ewarp, int lane, uint32_t t0, uint32_t nt) {
  const uint32_t K = (uint32_t)p.K;
  const uint32_t rowb = (uint32_t)p.H * 2u, rps = dispatch_rows_per_stage(p.H);
  const uint32_t nstage = (nt + rps - 1u) / rps;
  const uint32_t kNoRow = 0xffffffffu;
  if (etid < 128) sc.cnt[etid] = 0;
  if (etid == 0) sc.n_flagged = 0;
  epi_bar();
  if ((uint32_t)etid < nt) {
    const bool fl = __ldcg(&p.tok_flag[t0 + etid]) != 0;
    sc.isflag[etid] = fl ? 1 : 0;
    if (fl) {
      atomicAdd(&sc.n_flagged, 1u);
    } else {
      for (uint32_t k = 0; k < K; ++k) {
        const int e = __ldcg(&p.topk_idx[(size_t)(t0 + etid) * K + k]);
        sc.top_i[etid][k] = (uint8_t)e;
        sc.lpos[etid][k] = (uint8_t)atomicAdd(&sc.cnt[e], 1u);
      }
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 50);
  if (etid < p.E) {
    const uint32_t cnt = sc.cnt[etid];
    if (cnt) {
      const int owner = etid / p.El, le = etid - owner * p.El;
      uint32_t base;
      if (S && owner != p.rank)
        base = atom_add<true>(&p.peers[owner].expert_cnt[le], cnt);
      else
        base = atom_add<false>(&p.peers[owner].expert_cnt[le], cnt);
      if (base + cnt > (uint32_t)p.cap_rows) raise_error(p, sc, FDMOE_ERR_ROW_OVERFLOW, etid);
      sc.base[etid] = base;
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 51);
  uint32_t prev_s = 0u;
  for (uint32_t i = 0; i < nstage; ++i, ++stage_it) {
    const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
    const uint32_t nrows = min(rps, nt - i * rps);
    uint32_t my_d = kNoRow, my_w = 0u;
    const uint32_t r = (uint32_t)etid / K, k = (uint32_t)etid - r * K;
    const uint32_t tok = i * rps + r;  // within the task
    if ((uint32_t)etid < nrows * K && !sc.isflag[tok] && !sc.abort) {
      const uint32_t e = sc.top_i[tok][k];
      const uint32_t owner = e / (uint32_t)p.El, le = e - owner * (uint32_t)p.El;
      my_d = (owner << 28) | (le * (uint32_t)p.cap_rows + sc.base[e] + sc.lpos[tok][k]);
      my_w = __float_as_uint(__ldcg(&p.topk_w[(size_t)(t0 + tok) * K + k]));
    }
    if (!epi_vote_all(wait_bar(p, sc, &sc.full_bar[s], sph, FDMOE_ERR_TIMEOUT_STAGE))) return false;
    prof_mark(p, sc, etid, 52);
    if (my_d != kNoRow) {
      const FdmoePeer& op = p.peers[my_d >> 28];
      const uint32_t rowg = my_d & 0x0fffffffu;
      // FdmoeRowMeta {token, home << 8 | slot, weight, pad} as one 16-byte store
      *reinterpret_cast<uint4*>(&op.meta[rowg]) = make_uint4(t0 + tok, (uint32_t)((p.rank << 8) | k), my_w, 0u);
      ptx::bulk_store_1d(reinterpret_cast<uint8_t*>(op.packed) + (size_t)rowg * rowb,
                         stage + s * kStageBytes + r * rowb, rowb);
    }
    ptx::bulk_commit_group();
    if (i > 0u) {
      ptx::bulk_wait_group_read1();  // this thread's copy of the stage before this one has read its row
      epi_bar();
      if (etid == 0) ptx::mbar_arrive(&sc.empty_bar[prev_s]);
    }
    prev_s = s;
  }
  if (nstage) {
    ptx::bulk_wait_group_read0();
    epi_bar();
    if (etid == 0) ptx::mbar_arrive(&sc.empty_bar[prev_s]);
  }
  prof_mark(p, sc, etid, 53);
  ptx::bulk_wait_group0();  // this thread's copies are written
  epi_bar();
  prof_mark(p, sc, etid, 54);
  // The rows of this task have landed: count them per expert (and batch) on the owner and publish
  // the FFN1 tiles of every batch this completes.  One fence per signalling thread orders the rows
  // and sidebands (written by other threads of the group, before the barrier) first; it is the only
  // system-scope fence of the task, issued when nothing else of this worker is in flight.
  if (etid < p.E && !sc.abort) {
    const uint32_t cnt = sc.cnt[etid];
    if (cnt) {
      const int owner = etid / p.El, le = etid - owner * p.El;
      if (S && owner != p.rank) {
        fence_acqrel<true>();
        rows_landed<true>(p, sc.batch_mt, owner, (uint32_t)le, sc.base[etid], cnt);
      } else {
        fence_acqrel<false>();
        rows_landed<false>(p, sc.batch_mt, owner, (uint32_t)le, sc.base[etid], cnt);
      }
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 55);
  if (ewarp == 0) {
    if (lane == 0) atomicSub(&p.peers[p.rank].ctl->disp_active, 1u);
    count_gated<S>(p, sc, lane, nt - sc.n_flagged);
  }
  return true;
}

// ================================================================== GATEFIX
// Up to two tokens whose leading tensor-core logits were nearly tied: all E
// logits are recomputed with fp32 FMAs in the reference's order (128 threads per
// token, one expert each), then top-k, softmax, row reservation and the dispatch
// of the token's K rows, i.e. everything GATE does for the other tokens.
template <bool S>
__device__ __noinline__ bool gatefix_task(const FdmoeParams& p, SmemCtl& sc, uint8_t* stage, uint32_t& stage_it,
                                          int etid, int ewarp, int lane, uint32_t tok_a, uint32_t tok_b) {
  const int H = p.H, E = p.E, K = p.K;
  const int half = etid >> 7, e = etid & 127;
  const uint32_t tok = half ? tok_b : tok_a;
  const bool live = tok != 0xffffffffu;
  const bf16* x = reinterpret_cast<const bf16*>(p.x);
  if (live) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)tok * H);
    for (int v = e; v < H / 8; v += 128) sc.xrow[half][v] = src[v];
  }
  epi_bar();
  prof_mark(p, sc, etid, 30);
  // Exact logits: fp32 FMAs with k strictly ascending per output (bf16 x bf16
  // products are exact in fp32, so this equals the reference's `acc += a*b` bit
  // for bit; reference refGemm.h:16-27).  The gate weights arrive up to 192 columns
  // (three 64-column boxes) per stage through the stage ring (TMA, 128-byte swizzle: 16-byte chunk c of row r
  // sits at chunk c ^ (r & 7)); the token row is broadcast from shared memory.
  {
    float acc = 0.f;
    const uint32_t nkb = (uint32_t)(H / FDMOE_TILE_K);
    for (uint32_t kb = 0; kb < nkb; kb += kFixBlocks, ++stage_it) {
      const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
      if (!epi_vote_all(wait_bar(p, sc, &sc.full_bar[s], sph, FDMOE_ERR_TIMEOUT_STAGE))) return false;
      if (live && e < E) {
        const uint32_t nb = min((uint32_t)kFixBlocks, nkb - kb);
        for (uint32_t i = 0; i < nb; ++i) {
          const uint4* tile = reinterpret_cast<const uint4*>(stage + s * kStageBytes + i * kStageA);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 wv = tile[e * 8 + (c ^ (e & 7))];
            const uint4 xv = sc.xrow[half][(kb + i) * 8 + c];
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              acc = fmaf(bf16_lo(xw[j]), bf16_lo(ww[j]), acc);
              acc = fmaf(bf16_hi(xw[j]), bf16_hi(ww[j]), acc);
            }
          }
        }
      }
      epi_bar();  // every thread has read the stage
      if (etid == 0) ptx::mbar_arrive(&sc.empty_bar[s]);
    }
    if (live && e < E) sc.exact[half][e] = acc;
  }
  epi_bar();
  prof_mark(p, sc, etid, 31);
  if (live && (ewarp & 3) == 0) {
    float myv;
    int myi;
    topk_warp(sc.exact[half], E, K, lane, myv, myi);
    // softmax in the reference's order (refSoftmax.h:23-50), in fp32 as in the GATE task
    const float m = __shfl_sync(0xffffffffu, myv, 0);
    const float ex = (lane < K) ? expf(myv - m) : 0.0f;
    float sum = 1.0f;
    for (int j = 1; j < K; ++j) sum += __shfl_sync(0xffffffffu, ex, j);
    if (lane < K) {
      const float w = ex / sum;
      const int owner = myi / p.El, le = myi - owner * p.El;
      uint32_t pos;
      if (S && owner != p.rank)
        pos = atom_add<true>(&p.peers[owner].expert_cnt[le], 1u);
      else
        pos = atom_add<false>(&p.peers[owner].expert_cnt[le], 1u);
      sc.fix_dst[half][lane] = make_uint2(0xffffffffu, 0u);
      if (pos >= (uint32_t)p.cap_rows) {
        raise_error(p, sc, FDMOE_ERR_ROW_OVERFLOW, (uint32_t)myi);
      } else {
        const size_t rowg = (size_t)le * p.cap_rows + pos;
        sc.fix_dst[half][lane] = make_uint2((uint32_t)myi, pos);
        p.topk_idx[(size_t)tok * K + lane] = myi;
        p.topk_w[(size_t)tok * K + lane] = w;
        *reinterpret_cast<uint4*>(&p.peers[owner].meta[rowg]) =
            make_uint4(tok, (uint32_t)((p.rank << 8) | lane), __float_as_uint(w), 0u);
      }
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 32);
  // The token row (still in shared memory) goes to its K rows in the owners' expert buffers.
  if (live) {
    for (int k = 0; k < K; ++k) {
      const uint2 d = sc.fix_dst[half][k];
      if (d.x == 0xffffffffu) continue;
      const int owner = (int)d.x / p.El, le = (int)d.x - owner * p.El;
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.peers[owner].packed) +
                                            ((size_t)le * p.cap_rows + d.y) * H);
      for (int v = e; v < H / 8; v += 128) dst[v] = sc.xrow[half][v];
    }
    ptx::fence_proxy_async();  // packed rows are read by TMA
  }
  epi_bar();
  // the rows have been stored (by all threads, before the barrier): count them on their owners
  if (live && e < K) {
    const uint2 d = sc.fix_dst[half][e];
    if (d.x != 0xffffffffu) {
      const int owner = (int)d.x / p.El, le = (int)d.x - owner * p.El;
      if (S && owner != p.rank) {
        fence_acqrel<true>();
        rows_landed<true>(p, sc.batch_mt, owner, (uint32_t)le, d.y, 1u);
      } else {
        fence_acqrel<false>();
        rows_landed<false>(p, sc.batch_mt, owner, (uint32_t)le, d.y, 1u);
      }
    }
  }
  epi_bar();
  if (ewarp == 0) count_gated<S>(p, sc, lane, (tok_b != 0xffffffffu) ? 2u : 1u);
  return true;
}

// ==================================================================== GATED
// Every rank has gated and all rows have landed: the row counts of this rank's experts are final.
// Sets the number of m-tiles this rank will process (termination) and publishes, expert by expert,
// the FFN1 tiles of every m-tile that no sender has published as part of a complete batch: with
// batches of B m-tiles, an expert with F full m-tiles has had its first (F / B) * B published.
template <bool S>
__device__ __noinline__ void gated_task(const FdmoeParams& p, SmemCtl& sc, int etid) {
  const FdmoePeer& me = p.peers[p.rank];
  const int lane = etid & 31, w = etid >> 5;
  const uint32_t B = sc.batch_mt;
  const uint32_t nt1 = (uint32_t)(p.I / FDMOE_TILE_N1);
  // (the caller observed every rank's gating count with an atomic or took this task from the queue
  // with an acquire load; order this thread's reads after that)
  fence_acqrel<S>();
  uint32_t lcnt = 0, ntile = 0, first = 0;
  if (etid < p.El) {
    lcnt = ld_relaxed<S>(&me.expert_cnt[etid]);
    ntile = (lcnt + 127u) / 128u;
    first = ((lcnt / 128u) / B) * B;
  }
  const uint32_t mytasks = (ntile - first) * nt1;
  uint32_t inc = mytasks, inc_tile = ntile;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t a = __shfl_up_sync(0xffffffffu, inc, off);
    const uint32_t b = __shfl_up_sync(0xffffffffu, inc_tile, off);
    if (lane >= off) {
      inc += a;
      inc_tile += b;
    }
  }
  if (lane == 31 && w < 4) {
    sc.pre[w] = inc;
    sc.pre[8 + w] = inc_tile;
  }
  epi_bar();
  uint32_t before = 0, all = 0, mt = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i < w) before += sc.pre[i];
    all += sc.pre[i];
    mt += sc.pre[8 + i];
  }
  if (etid == 0) {
    st_relaxed<false>(&me.ctl->mtiles_total, mt);
    sc.q_t0 = all ? atom_add<false>(&me.ctl->q[1].head, all) : 0u;
  }
  epi_bar();
  if (mytasks) {
    const uint32_t t1 = sc.q_t0 + before + inc - mytasks;
    const uint32_t full = lcnt / 128u, rem = lcnt % 128u;
    FdmoeSlot* slots = me.slots[1];
    for (uint32_t idx = 0; idx < mytasks; ++idx) {
      const uint32_t jt = first + idx / nt1, n = idx % nt1;
      FdmoeSlot* sl = &slots[(t1 + idx) & (uint32_t)p.queue_mask];
      sl->a = task_word(FDMOE_TASK_FFN1, (uint32_t)etid, n);
      sl->b = jt;
      sl->c = (jt < full) ? 128u : rem;
    }
    fence_acqrel<false>();
    for (uint32_t idx = 0; idx < mytasks; ++idx)
      st_relaxed<false>(&slots[(t1 + idx) & (uint32_t)p.queue_mask].seq, t1 + idx + 1u);
    atom_add<false>(&me.ctl->q[1].avail, mytasks);
  }
  epi_bar();
  if (etid == 0) {
    st_release<false>(&me.ctl->gated_done, 1u);
    maybe_close(p);
  }
}

// silu(g) * u with the fast exponential and reciprocal (relative error ~1e-6, far
// below the bf16 rounding of the stored activation); g -> -inf gives -0.
__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

// Epilogue stores go through a per-warp staging buffer of 32 rows x 128 bytes so that every global
// store instruction covers 4 rows x 128 contiguous bytes (whole cache lines; over NVLink, packets of
// 128 bytes) instead of 32 rows x 16.  The thread that owns row r of the accumulator quadrant puts
// its packed words into row r of the buffer; the 16-byte chunk c of a row sits at chunk c ^ (r & 7),
// which keeps both the row-wise writes and the line-wise reads free of bank conflicts.
__device__ __forceinline__ void stage_half_row(uint8_t* st, int lane, int half, const uint32_t (&o)[16]) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const int c = half * 4 + v;
    *reinterpret_cast<uint4*>(st + lane * 128 + ((c ^ (lane & 7)) << 4)) =
        make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
  }
}

// Stores the staged 32 x 128-byte block: lane l writes chunk (l & 7) of rows (l >> 3) + 4 i.
// `myptr`: this lane's row pointer (first byte of its 128-byte segment in global memory), 0 = no row.
__device__ __forceinline__ void store_staged_rows(uint8_t* st, int lane, unsigned long long myptr) {
  __syncwarp();
  const int c = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = (lane >> 3) + 4 * i;
    const unsigned long long pp = __shfl_sync(0xffffffffu, myptr, r);
    const uint4 val = *reinterpret_cast<const uint4*>(st + r * 128 + ((c ^ (r & 7)) << 4));
    if (pp != 0ull) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pp) + (c << 4)) = val;
  }
  __syncwarp();
}

// FFN1 epilogue: act[row, n*128 + c] = silu(D[row, c]) * D[row, 128 + c].
__device__ __forceinline__ void ffn1_epilogue(const FdmoeParams& p, SmemCtl& sc, uint32_t taddr, int q, int h,
                                              int lane, int ewarp, uint32_t e, uint32_t j, uint32_t n,
                                              uint32_t rows) {
  uint8_t* st = sc.store_stage[ewarp];
  const uint32_t row = q * 32 + lane;
  unsigned long long myptr = 0ull;
  if (row < rows)
    myptr = reinterpret_cast<unsigned long long>(reinterpret_cast<bf16*>(p.act) +
                                                 ((size_t)e * p.cap_rows + (size_t)j * 128 + row) * p.I +
                                                 n * FDMOE_TILE_N1 + h * 64);
  const uint32_t tbase = taddr + ((uint32_t)(q * 32) << 16) + h * 64;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t g[32], u[32], o[16];
    ptx::tmem_ld_32x32(tbase + c * 32, g);
    ptx::tmem_ld_32x32(tbase + 128 + c * 32, u);
    ptx::tmem_ld_wait();
#pragma unroll
    for (int w = 0; w < 16; ++w)
      o[w] = pack_bf16(silu_mul(__uint_as_float(g[2 * w]), __uint_as_float(u[2 * w])),
                       silu_mul(__uint_as_float(g[2 * w + 1]), __uint_as_float(u[2 * w + 1])));
    stage_half_row(st, lane, c, o);
  }
  store_staged_rows(st, lane, myptr);
}

// FFN2 epilogue: y[token, slot, n*256 + c] = D[row, c] * routing weight, stored
// on the token's home rank.  Returns whether this thread's row went to another GPU.
__device__ __forceinline__ bool ffn2_epilogue(const FdmoeParams& p, SmemCtl& sc, uint32_t taddr, int q, int h,
                                              int lane, int ewarp, uint32_t e, uint32_t j, uint32_t n,
                                              uint32_t rows) {
  uint8_t* st = sc.store_stage[ewarp];
  const uint32_t row = q * 32 + lane;
  float wgt = 0.f;
  unsigned long long myptr = 0ull;
  bool remote = false;
  if (row < rows) {
    const uint4 mraw = ld_cg_u4(&p.peers[p.rank].meta[(size_t)e * p.cap_rows + (size_t)j * 128 + row]);
    const int token = (int)mraw.x, home = (int)mraw.y >> 8, slot = (int)mraw.y & 0xff;
    wgt = __uint_as_float(mraw.z);
    remote = home != p.rank;
    myptr = reinterpret_cast<unsigned long long>(reinterpret_cast<bf16*>(p.peers[home].ystage) +
                                                 ((size_t)token * p.K + slot) * p.H + n * FDMOE_TILE_N2 + h * 128);
  }
  const uint32_t tbase = taddr + ((uint32_t)(q * 32) << 16) + h * 128;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t d[32], o[16];
      ptx::tmem_ld_32x32(tbase + (pass * 2 + c) * 32, d);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int w = 0; w < 16; ++w)
        o[w] = pack_bf16(__uint_as_float(d[2 * w]) * wgt, __uint_as_float(d[2 * w + 1]) * wgt);
      stage_half_row(st, lane, c, o);
    }
    store_staged_rows(st, lane, myptr ? myptr + (unsigned long long)(pass * 128) : 0ull);
  }
  return remote;
}

// COMBINE streams the K weighted rows of each token of a group through the
// shared-memory stage ring with 1-D bulk copies (issued by the TMA warp) in
// pieces of up to 2048 columns: stage layout [K][piece], the piece's bytes per slot row.
constexpr int kCombineCols = 2048;

// k-blocks a tile task puts into one pipeline stage: two for GATE tiles of up to 64 tokens
// (H is a multiple of 256, so the number of k-blocks is even), one otherwise.
__device__ __forceinline__ uint32_t gate_kblocks_per_stage(bool is_gate, int gate_rows) {
  return (is_gate && gate_rows <= 64) ? 2u : 1u;
}

// Pipeline stages a DISPATCH task of `nt` tokens takes (whole token rows per stage).
__device__ __forceinline__ uint32_t dispatch_stages(const FdmoeParams& p, uint32_t nt) {
  const uint32_t rps = dispatch_rows_per_stage(p.H);
  return (nt + rps - 1u) / rps;
}

// Barrier over the 256 epilogue threads that also ORs a predicate.
__device__ __forceinline__ bool epi_vote_any(bool v) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 1, 256, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(r)
      : "r"((uint32_t)v)
      : "memory");
  return r != 0;
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
    for (int d = 0; d < kDone; ++d) {
      ptx::mbar_init(&sc.done_full[d], 1);
      ptx::mbar_init(&sc.done_empty[d], 1);
    }
    sc.abort = 0;
    sc.run_round2 = 0;
    sc.skip_done = 0;
    sc.flag = 0;
    sc.prof_n = 0;
    ptx::fence_mbar_init();
    st_relaxed<false>(&ctl->tokens_launch, (uint32_t)p.T);
  }
  {
    static_assert(sizeof(FdmoeParams) % 16 == 0 && offsetof(FdmoeParams, peers) % 16 == 0,
                  "parameter block is copied in 16-byte pieces");
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(&p) + offsetof(FdmoeParams, peers));
    uint4* dst = reinterpret_cast<uint4*>(sc.params_tail);
    for (int i = tid; i < (int)(sizeof(sc.params_tail) / 16); i += kThreads) dst[i] = src[i];
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

  // ---- multi-GPU: announce this launch (and this rank's token count) to the peers and wait,
  // with a budget of its own, until every peer has entered the same launch, i.e. has reset its
  // counters.  A peer that is already one launch further has passed this one.
  if (S && p.world > 1) {
    if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
      FdmoeCtl* pc = p.peers[tid].ctl;
      st_relaxed<true>(&pc->tokens_of[p.epoch & 1u][p.rank], (uint32_t)p.T);
      ptx::st_release_sys(&pc->ready[p.rank], p.epoch);
    }
    if (tid < p.world && tid != p.rank) {
      const uint64_t t0 = ptx::globaltimer_ns();
      uint32_t spins = 0;
      while ((int32_t)(ptx::ld_acquire_sys(&ctl->ready[tid]) - p.epoch) < 0) {
        if (sc.abort || ld_relaxed<true>(&ctl->closed) == 2u) break;
        if (ptx::globaltimer_ns() - t0 > p.peer_timeout_ns) {
          raise_error(p, sc, FDMOE_ERR_TIMEOUT_PEER, (uint32_t)tid);
          break;
        }
        __nanosleep(++spins < 1000u ? 200 : 2000);
      }
    }
    __syncthreads();
  }
  if (tid == 0) {
    uint32_t all = 0u;
    for (int r = 0; r < p.world; ++r) all += tokens_of_rank(p, r);
    sc.tokens_all = all;
    sc.batch_mt = batch_mt_of(p, all);
  }
  __syncthreads();

  // ---- GATE tiles are claimed from a counter by whichever worker is free.  Nothing to gate:
  // the rank's "gate phase" is finished at once (it may still serve its peers).
  const uint32_t gate_tiles =
      (p.mode != 2 && p.T > 0 && p.gate_rows > 0) ? (uint32_t)((p.T + p.gate_rows - 1) / p.gate_rows) : 0u;
  if (p.mode != 2 && gate_tiles == 0u && blockIdx.x == 0 && warp == 0 && !sc.abort) gating_finished<S>(p, nullptr, lane);

  // =============================== worker loop
  const uint32_t nt1 = (uint32_t)(p.I / FDMOE_TILE_N1), nt2 = (uint32_t)(p.H / FDMOE_TILE_N2);
  const uint32_t nkb1 = (uint32_t)(p.H / FDMOE_TILE_K), nkb2 = (uint32_t)(p.I / FDMOE_TILE_K);

  if (warp == kWarpSched) {
    if (lane == 0) {
      for (uint32_t it = 0;; ++it) {
        const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
        if (!wait_bar(p, sc, &sc.ring_empty[r], ph ^ 1u, FDMOE_ERR_TIMEOUT_RING)) break;
        const FdmoeSlot t = next_task<S>(p, sc, gate_tiles);
        sc.ring[r] = t;
        ptx::mbar_arrive(&sc.ring_full[r]);
        const uint32_t kind = t.a & 0xffu;
        if (kind == FDMOE_TASK_EXIT) break;
        if (kind != FDMOE_TASK_FFN1 && kind != FDMOE_TASK_FFN2 && kind != FDMOE_TASK_COMBINE) {
          // Only tile tasks (and COMBINE, whose rows travel as bulk copies) profit from being queued
          // behind one another (their loads and MMAs run ahead of the epilogue).  Behind a long task
          // of another kind a claimed task would just sit here while other workers idle: wait until
          // it is done.
          if (!wait_bar(p, sc, &sc.ring_empty[r], ph, FDMOE_ERR_TIMEOUT_RING)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == kWarpTma) {
    if (lane == 0) {
      uint32_t stage_it = 0;
      for (uint32_t it = 0;; ++it) {
        const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
        if (!wait_bar(p, sc, &sc.ring_full[r], ph, FDMOE_ERR_TIMEOUT_RING, 2u)) break;
        const FdmoeSlot t = sc.ring[r];
        const uint32_t kind = t.a & 0xffu;
        if (kind == FDMOE_TASK_EXIT) break;
        if (kind == FDMOE_TASK_FFN1 || kind == FDMOE_TASK_FFN2 || kind == FDMOE_TASK_GATE) {
          const uint32_t e = (t.a >> 8) & 0xfffu, n = t.a >> 20, j = t.b;
          const bool f1 = kind == FDMOE_TASK_FFN1, gt = kind == FDMOE_TASK_GATE;
          const uint32_t nkb = (f1 || gt) ? nkb1 : nkb2;
          const int32_t arow = gt ? (int32_t)(j * (uint32_t)p.gate_rows) : (int32_t)(e * (uint32_t)p.cap_rows + j * 128u);
          // bytes one GATE stage receives: both boxes are clamped to the tensor extents
          const uint32_t gate_bytes = (uint32_t)(min(p.gate_rows, p.T) + min(128, p.E)) * FDMOE_TILE_K * 2u;
          // GATE tiles of up to 64 tokens are bound by the round trip of a stage, not by its size:
          // they put two k-blocks into one stage (A 2 x 8 KB, B 2 x 16 KB)
          const uint32_t gk = gate_kblocks_per_stage(gt, p.gate_rows);
          ptx::fence_proxy_async();  // rows / activations were written with generic stores
          bool ok = true;
          for (uint32_t kb = 0; kb < nkb && ok; kb += gk, ++stage_it) {
            const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
            ok = wait_bar(p, sc, &sc.empty_bar[s], sph ^ 1u, FDMOE_ERR_TIMEOUT_STAGE);
            if (!ok) break;
            uint8_t* sa = stage + s * kStageBytes;
            uint8_t* sb = sa + kStageA;
            ptx::mbar_expect_tx(&sc.full_bar[s], gt ? gk * gate_bytes : (uint32_t)kStageBytes);
            const int32_t kx = (int32_t)(kb * FDMOE_TILE_K);
            if (gt) {
              for (uint32_t i = 0; i < gk; ++i) {
                ptx::tma_load_2d(sa + i * (kStageA / 2), &p.tm_x, &sc.full_bar[s], kx + (int32_t)(i * FDMOE_TILE_K), arow);
                ptx::tma_load_2d(sb + i * kStageA, &p.tm_gate, &sc.full_bar[s], kx + (int32_t)(i * FDMOE_TILE_K), 0);
              }
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
        } else if (kind == FDMOE_TASK_DISPATCH) {
          // the tokens' rows: contiguous in the token matrix, one bulk copy per stage
          const uint32_t rowb = (uint32_t)p.H * 2u, rps = dispatch_rows_per_stage(p.H);
          const uint32_t nt = t.c;
          const uint8_t* xb = reinterpret_cast<const uint8_t*>(p.x) + (size_t)t.b * rowb;
          bool ok = true;
          for (uint32_t r0 = 0; r0 < nt && ok; r0 += rps, ++stage_it) {
            const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
            ok = wait_bar(p, sc, &sc.empty_bar[s], sph ^ 1u, FDMOE_ERR_TIMEOUT_STAGE);
            if (!ok) break;
            const uint32_t bytes = min(rps, nt - r0) * rowb;
            ptx::mbar_expect_tx(&sc.full_bar[s], bytes);
            ptx::bulk_load_1d(stage + s * kStageBytes, xb + (size_t)r0 * rowb, bytes, &sc.full_bar[s]);
          }
          if (!ok) break;
        } else if (kind == FDMOE_TASK_GATEFIX) {
          bool ok = true;
          for (uint32_t kb = 0; kb < nkb1; kb += kFixBlocks, ++stage_it) {
            const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
            ok = wait_bar(p, sc, &sc.empty_bar[s], sph ^ 1u, FDMOE_ERR_TIMEOUT_STAGE);
            if (!ok) break;
            const uint32_t nb = min((uint32_t)kFixBlocks, nkb1 - kb);
            const uint32_t blk_bytes = (uint32_t)min(128, p.E) * FDMOE_TILE_K * 2u;
            ptx::mbar_expect_tx(&sc.full_bar[s], nb * blk_bytes);
            for (uint32_t i = 0; i < nb; ++i)
              ptx::tma_load_2d(stage + s * kStageBytes + i * kStageA, &p.tm_gate, &sc.full_bar[s],
                               (int32_t)((kb + i) * FDMOE_TILE_K), 0);
          }
          if (!ok) break;
        } else if (kind == FDMOE_TASK_COMBINE) {
          const int t_begin = (int)t.b, t_end = t_begin + (int)t.c;
          const bf16* ys = reinterpret_cast<const bf16*>(me.ystage);
          ptx::fence_proxy_async();  // the rows were written with generic stores
          bool ok = true;
          for (int tk = t_begin; tk < t_end && ok; ++tk) {
            for (int c0 = 0; c0 < p.H; c0 += kCombineCols, ++stage_it) {
              const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
              ok = wait_bar(p, sc, &sc.empty_bar[s], sph ^ 1u, FDMOE_ERR_TIMEOUT_STAGE);
              if (!ok) break;
              const uint32_t wbytes = (uint32_t)min(kCombineCols, p.H - c0) * 2u;
              uint8_t* sa = stage + s * kStageBytes;
              ptx::mbar_expect_tx(&sc.full_bar[s], wbytes * (uint32_t)p.K);
              if (p.H <= kCombineCols) {
                // the K rows of a token are contiguous: one copy
                ptx::bulk_load_1d(sa, ys + (size_t)tk * p.K * p.H, wbytes * (uint32_t)p.K, &sc.full_bar[s]);
              } else {
                for (int k = 0; k < p.K; ++k)
                  ptx::bulk_load_1d(sa + k * wbytes, ys + ((size_t)tk * p.K + k) * p.H + c0, wbytes, &sc.full_bar[s]);
              }
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
      uint32_t stage_it = 0, tile_it = 0, skips = 0;
      for (uint32_t it = 0;; ++it) {
        const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
        if (!wait_bar(p, sc, &sc.ring_full[r], ph, FDMOE_ERR_TIMEOUT_RING, 2u)) break;
        const FdmoeSlot t = sc.ring[r];
        const uint32_t kind = t.a & 0xffu;
        if (kind == FDMOE_TASK_EXIT) break;
        bool ok = true;
        if (kind == FDMOE_TASK_FFN1 || kind == FDMOE_TASK_FFN2 || kind == FDMOE_TASK_GATE) {
          const uint32_t nkb = (kind == FDMOE_TASK_FFN2) ? nkb2 : nkb1;
          const uint32_t idesc = (kind == FDMOE_TASK_GATE) ? idesc128 : idesc256;
          const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
          ++tile_it;
          if (!wait_bar(p, sc, &sc.tmem_empty[acc], aph ^ 1u, FDMOE_ERR_TIMEOUT_TMEM)) break;
          ptx::tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + acc * kAccCols;
          const uint32_t gk = gate_kblocks_per_stage(kind == FDMOE_TASK_GATE, p.gate_rows);
          for (uint32_t kb = 0; kb < nkb; kb += gk, ++stage_it) {
            const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
            ok = wait_bar(p, sc, &sc.full_bar[s], sph, FDMOE_ERR_TIMEOUT_STAGE);
            if (!ok) break;
            ptx::tcgen05_fence_after();
            const uint32_t sa = ptx::smem_u32(stage + s * kStageBytes);
            for (uint32_t i = 0; i < gk; ++i) {
              // (a GATE stage with two k-blocks: A at 8 KB, B at 16 KB steps)
              const uint64_t da = ptx::make_smem_desc_sw128(sa + i * (kStageA / 2));
              const uint64_t db = ptx::make_smem_desc_sw128(sa + kStageA + i * kStageA);
#pragma unroll
              for (uint32_t k4 = 0; k4 < FDMOE_TILE_K / 16; ++k4) {
                // +32 bytes per 16-element k step inside the 128-byte swizzle row
                ptx::umma_bf16(d_tmem, da + k4 * 2u, db + k4 * 2u, idesc, (kb | i | k4) != 0u);
              }
            }
            ptx::umma_commit(&sc.empty_bar[s]);  // frees the stage when the MMAs have read it
          }
          if (!ok) break;
          ptx::umma_commit(&sc.tmem_full[acc]);
        }
        if (kind == FDMOE_TASK_DISPATCH || kind == FDMOE_TASK_GATEFIX || kind == FDMOE_TASK_COMBINE) {
          // Stages of these tasks are consumed
          // by the epilogue warps.  This warp must not run ahead of them: a stage barrier only tells
          // phases apart by parity, so a waiter more than one phase ahead would take an old completion
          // for its own.  Wait until the epilogue has finished the task, then step over its stages.
          ++skips;
          const uint64_t t0w = ptx::globaltimer_ns();
          uint32_t spins = 0;
          while (sc.skip_done < skips) {
            if ((++spins & 63u) == 0u) {
              if (sc.abort) { ok = false; break; }
              if (ptx::globaltimer_ns() - t0w > 4ull * p.timeout_ns) {
                raise_error(p, sc, FDMOE_ERR_TIMEOUT_STAGE, (blockIdx.x << 8) | 2u);
                ok = false;
                break;
              }
              __nanosleep(100);
            }
          }
          if (!ok) break;
          if (kind == FDMOE_TASK_DISPATCH) {
            stage_it += dispatch_stages(p, t.c);
          } else if (kind == FDMOE_TASK_GATEFIX) {
            stage_it += (nkb1 + kFixBlocks - 1) / kFixBlocks;
          } else {
            stage_it += t.c * (uint32_t)((p.H + kCombineCols - 1) / kCombineCols);
          }
        }
        ptx::mbar_arrive(&sc.ring_empty[r]);
      }
    }
    __syncwarp();
  } else if (warp >= kWarpEpi0) {
    const int etid = tid - kWarpEpi0 * 32, ewarp = warp - kWarpEpi0;
    const int q = warp & 3, h = ewarp >> 2;
    uint32_t tile_it = 0, done_it = 0, stage_it = 0;
    for (uint32_t it = 0;; ++it) {
      const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
      // the group leaves together: a lone warp breaking out would strand the
      // others at the next group barrier
      if (!epi_vote_all(wait_bar(p, sc, &sc.ring_full[r], ph, FDMOE_ERR_TIMEOUT_RING, 2u))) break;
      const FdmoeSlot t = sc.ring[r];
      const uint32_t kind = t.a & 0xffu;
      if (kind == FDMOE_TASK_EXIT) break;
      const uint32_t e = (t.a >> 8) & 0xfffu, n = t.a >> 20, j = t.b, rows = t.c;
      const uint32_t pt0 = (p.prof && etid == 0) ? prof_now() : 0u;
      uint32_t pt1 = pt0;
      if (kind == FDMOE_TASK_GATE) {
        const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
        ++tile_it;
        stage_it += nkb1 / gate_kblocks_per_stage(true, p.gate_rows);
        if (!epi_vote_all(wait_bar(p, sc, &sc.tmem_full[acc], aph, FDMOE_ERR_TIMEOUT_TMEM))) break;
        if (p.prof && etid == 0) pt1 = prof_now();
        ptx::tcgen05_fence_after();
        gate_epilogue<S>(task_params(sc), sc, tmem_base + acc * kAccCols, &sc.tmem_empty[acc], q, h, lane, etid, ewarp, j);
      } else if (kind == FDMOE_TASK_DISPATCH) {
        if (!dispatch_task<S>(task_params(sc), sc, stage, stage_it, etid, ewarp, lane, j, rows)) break;
        if (etid == 0) {
          __threadfence_block();
          sc.skip_done = sc.skip_done + 1u;
        }
      } else if (kind == FDMOE_TASK_GATEFIX) {
        if (!gatefix_task<S>(task_params(sc), sc, stage, stage_it, etid, ewarp, lane, j, rows)) break;
        if (etid == 0) {
          __threadfence_block();
          sc.skip_done = sc.skip_done + 1u;
        }
      } else if (kind == FDMOE_TASK_FFN1 || kind == FDMOE_TASK_FFN2) {
        const uint32_t acc = tile_it & 1u, aph = (tile_it >> 1) & 1u;
        ++tile_it;
        stage_it += (kind == FDMOE_TASK_FFN1) ? nkb1 : nkb2;
        if (!epi_vote_all(wait_bar(p, sc, &sc.tmem_full[acc], aph, FDMOE_ERR_TIMEOUT_TMEM))) break;
        if (p.prof && etid == 0) pt1 = prof_now();
        ptx::tcgen05_fence_after();
        const uint32_t taddr = tmem_base + acc * kAccCols;
        bool remote = false;
        if (kind == FDMOE_TASK_FFN1)
          ffn1_epilogue(p, sc, taddr, q, h, lane, ewarp, e, j, n, rows);
        else
          remote = ffn2_epilogue(p, sc, taddr, q, h, lane, ewarp, e, j, n, rows);
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sc.tmem_empty[acc]);
        const uint32_t pta = (p.prof && etid == 0) ? prof_now() : 0u;

        // The tile's stores are issued.  Dependency counting, successor pushes and
        // the notifications of the home ranks are done by the completion warp, off
        // the epilogue's critical path.
        // activations are read by TMA in FFN2, weighted rows by bulk copies in COMBINE
        ptx::fence_proxy_async();
        const bool any_remote = S ? epi_vote_any(remote) : (epi_bar(), false);
        if (etid == 0 && p.mode != 2) {
          const uint32_t d = done_it % kDone, dph = (done_it / kDone) & 1u;
          if (wait_bar(p, sc, &sc.done_empty[d], dph ^ 1u, FDMOE_ERR_TIMEOUT_RING)) {
            FdmoeSlot dt = t;
            dt.seq = any_remote ? 1u : 0u;  // rows of this tile went to another GPU
            sc.done_ring[d] = dt;
            ptx::mbar_arrive(&sc.done_full[d]);
          }
        }
        ++done_it;
        if (etid == 0) prof_event(p, sc, kind + 16u, pt1, pta, prof_now());
      } else if (kind == FDMOE_TASK_COMBINE) {
        // out[t, :] = sum over slots k = 0..K-1 (in that order, fp32) of y[t, k, :]
        const int t_begin = (int)j, t_end = t_begin + (int)rows;
        bf16* outp = reinterpret_cast<bf16*>(p.out);
        bool ok = true;
        for (int tk = t_begin; tk < t_end && ok; ++tk) {
          for (int c0 = 0; c0 < p.H; c0 += kCombineCols, ++stage_it) {
            const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
            const bool landed = wait_bar(p, sc, &sc.full_bar[s], sph, FDMOE_ERR_TIMEOUT_STAGE);
            const int nvec = min(kCombineCols, p.H - c0) / 8;
            if (landed && etid < nvec) {
              const uint4* sm = reinterpret_cast<const uint4*>(stage + s * kStageBytes) + etid;
              float acc[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[i] = 0.f;
              for (int k = 0; k < p.K; ++k) {
                const uint4 rr = sm[k * nvec];
                const uint32_t w[4] = {rr.x, rr.y, rr.z, rr.w};
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
              *reinterpret_cast<uint4*>(outp + (size_t)tk * p.H + c0 + etid * 8) = o;
            }
            ok = epi_vote_all(landed);  // every thread has read the stage (or the group gives up together)
            if (!ok) break;
            if (etid == 0) ptx::mbar_arrive(&sc.empty_bar[s]);
          }
        }
        if (!ok) break;
        if (etid == 0) {
          __threadfence_block();
          sc.skip_done = sc.skip_done + 1u;
        }
        if (etid == 0 && p.mode != 2) {
          fence_acqrel<false>();
          atomicAdd(&ctl->tokens_combined, (uint32_t)(t_end - t_begin));
          maybe_close(p);
        }
      } else if (kind == FDMOE_TASK_GATED) {
        gated_task<S>(task_params(sc), sc, etid);
      } else if (kind == FDMOE_TASK_TESTA || kind == FDMOE_TASK_TESTB) {
        // task-system self test: two dependent stages over a 256-element chunk
        int* ptr = p.test_buf + (size_t)j * kEpiThreads + etid;
        if (kind == FDMOE_TASK_TESTA) {
          *ptr = __ldcg(ptr) * 2;
          epi_bar();
          if (etid == 0) {
            fence_acqrel<false>();
            // (alternating queues, so that the test exercises both)
            queue_push<false>(p, me, (int)(j & 1u), 1u, [&](uint32_t, uint32_t& a, uint32_t& b, uint32_t& c) {
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
      if (kind == FDMOE_TASK_DISPATCH || kind == FDMOE_TASK_GATEFIX) {
        // the task may have found this rank's GATED round due: run it here and now
        epi_bar();
        const bool r2 = sc.run_round2 != 0u;
        epi_bar();
        if (r2) {
          if (etid == 0) sc.run_round2 = 0u;
          gated_task<S>(task_params(sc), sc, etid);
        }
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
    if (etid == 0 && p.mode != 2) {
      // tell the completion warp that nothing more will come
      const uint32_t d = done_it % kDone, dph = (done_it / kDone) & 1u;
      if (wait_bar(p, sc, &sc.done_empty[d], dph ^ 1u, FDMOE_ERR_TIMEOUT_RING)) {
        sc.done_ring[d].a = FDMOE_TASK_EXIT;
        ptx::mbar_arrive(&sc.done_full[d]);
      }
    }
  } else if (warp == kWarpTmem && p.mode != 2) {
    // ---- completion warp: per finished tile, count it and publish what it unblocks.  It takes
    // every entry that is ready at once and pays one fence for all of them.
    const uint32_t G = (uint32_t)p.combine_group;
    uint32_t it = 0;
    for (bool running = true; running;) {
      const uint32_t d0 = it % kDone, dph0 = (it / kDone) & 1u;
      int ok = 1;
      uint32_t nready = 1u;
      if (lane == 0) {
        // This warp may legitimately idle for a whole launch, so its own budget is four
        // times the others': whoever actually stalls reports first.
        ok = 0;
        for (int tries = 0; tries < 4 && !ok && !sc.abort; ++tries)
          ok = wait_idle(p, sc, &sc.done_full[d0], dph0) ? 1 : 0;
        if (!ok && !sc.abort) raise_error(p, sc, FDMOE_ERR_TIMEOUT_RING, (blockIdx.x << 8) | 3u);
        if (ok) {
          while (nready < (uint32_t)kDone) {
            const uint32_t i2 = it + nready;
            if (!ptx::mbar_try_wait(&sc.done_full[i2 % kDone], (i2 / kDone) & 1u)) break;
            ++nready;
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      nready = __shfl_sync(0xffffffffu, nready, 0);
      // The stores of these tiles were made by the epilogue warps (handed over through the ring's
      // barriers), the weighted rows of FFN2 tiles possibly on other GPUs: one fence of the widest
      // scope needed makes them visible before anything counts them.
      {
        bool rem = false;
        if ((uint32_t)lane < nready) {
          const FdmoeSlot& tt = sc.done_ring[(it + (uint32_t)lane) % kDone];
          rem = S && (tt.a & 0xffu) == FDMOE_TASK_FFN2 && tt.seq != 0u;
        }
        if (__any_sync(0xffffffffu, rem))
          fence_acqrel<true>();
        else
          fence_acqrel<false>();
      }
      for (uint32_t i = 0; i < nready; ++i, ++it) {
        const uint32_t d = it % kDone;
        const FdmoeSlot t = sc.done_ring[d];
        const uint32_t kind = t.a & 0xffu;
        if (kind == FDMOE_TASK_EXIT) {
          running = false;
          break;
        }
        const uint32_t e = (t.a >> 8) & 0xfffu, j = t.b, rows = t.c;
        if (kind == FDMOE_TASK_FFN1) {
          if (lane == 0) {
            const uint32_t prev = atomicAdd(&p.ffn1_done[(size_t)e * p.MT + j], 1u);
            if (prev == nt1 - 1u) {
              // (the fence inside the push orders the other tiles' activations, observed through the
              // counter, before the tasks)
              queue_push<false>(p, me, 0, nt2, [&](uint32_t i3, uint32_t& a, uint32_t& b, uint32_t& c) {
                a = task_word(FDMOE_TASK_FFN2, e, i3);
                b = j;
                c = rows;
              });
            }
          }
        } else {
          int last = 0;
          if (lane == 0) last = atomicAdd(&p.ffn2_done[(size_t)e * p.MT + j], 1u) == nt2 - 1u;
          last = __shfl_sync(0xffffffffu, last, 0);
          if (last) {
            // Every hidden-column tile of this m-tile is stored (the other tiles' workers fenced before
            // they counted): its rows are counted per COMBINE group on their home ranks, and whoever
            // delivers the last row of a group publishes the group's COMBINE task there.  A lane owns up
            // to four rows; it first counts them all, then publishes the groups it completed with one
            // fence for the whole warp (the last m-tiles of a launch complete dozens of groups each).
            fence_acqrel<false>();
            uint32_t c_home[4], c_first[4], c_ntok[4], nc = 0u;
            // (the four counter updates of a lane are issued back to back, their results are looked
            // at afterwards: over NVLink each takes microseconds to answer)
            uint32_t r_home[4], r_first[4], r_ntok[4], r_got[4];
#pragma unroll
            for (uint32_t rr = 0; rr < 4u; ++rr) {
              const uint32_t r = rr * 32u + (uint32_t)lane;
              r_home[rr] = 0xffffffffu;
              r_first[rr] = 0u;
              r_ntok[rr] = 0u;
              r_got[rr] = 0u;
              c_home[rr] = 0u;
              c_first[rr] = 0u;
              c_ntok[rr] = 0u;
              if (r < rows) {
                const uint4 mraw = ld_cg_u4(&me.meta[(size_t)e * p.cap_rows + (size_t)j * 128 + r]);
                const int hm = (int)mraw.y >> 8;
                const uint32_t g = mraw.x / G;
                const uint32_t th = tokens_of_rank(p, hm);
                r_home[rr] = (uint32_t)hm;
                r_first[rr] = g * G;
                r_ntok[rr] = min(G, th - g * G);
                if (S && hm != p.rank)
                  r_got[rr] = atom_add<true>(&p.peers[hm].grp_cnt[g], 1u) + 1u;
                else
                  r_got[rr] = atom_add<false>(&p.peers[hm].grp_cnt[g], 1u) + 1u;
              }
            }
#pragma unroll
            for (uint32_t rr = 0; rr < 4u; ++rr) {
              if (r_home[rr] != 0xffffffffu && r_got[rr] == r_ntok[rr] * (uint32_t)p.K) {
#pragma unroll
                for (uint32_t c = 0; c < 4u; ++c) {
                  if (c == nc) {
                    c_home[c] = r_home[rr];
                    c_first[c] = r_first[rr];
                    c_ntok[c] = r_ntok[rr];
                  }
                }
                ++nc;
              }
            }
            uint32_t ticket[4];
            bool any_remote = false;
#pragma unroll
            for (uint32_t c = 0; c < 4u; ++c) {
              ticket[c] = 0u;
              if (c < nc) {
                const FdmoePeer& hp = p.peers[c_home[c]];
                const bool rem = S && (int)c_home[c] != p.rank;
                any_remote |= rem;
                ticket[c] = rem ? atom_add<true>(&hp.ctl->q[0].head, 1u) : atom_add<false>(&hp.ctl->q[0].head, 1u);
                FdmoeSlot* sl = &hp.slots[0][ticket[c] & (uint32_t)p.queue_mask];
                sl->a = FDMOE_TASK_COMBINE;
                sl->b = c_first[c];
                sl->c = c_ntok[c];
              }
            }
            if (__any_sync(0xffffffffu, nc != 0u)) {
              if (__any_sync(0xffffffffu, any_remote))
                fence_acqrel<true>();
              else
                fence_acqrel<false>();
#pragma unroll
              for (uint32_t c = 0; c < 4u; ++c) {
                if (c < nc) {
                  const FdmoePeer& hp = p.peers[c_home[c]];
                  if (S && (int)c_home[c] != p.rank) {
                    st_relaxed<true>(&hp.slots[0][ticket[c] & (uint32_t)p.queue_mask].seq, ticket[c] + 1u);
                    atom_add<true>(&hp.ctl->q[0].avail, 1u);
                  } else {
                    st_relaxed<false>(&hp.slots[0][ticket[c] & (uint32_t)p.queue_mask].seq, ticket[c] + 1u);
                    atom_add<false>(&hp.ctl->q[0].avail, 1u);
                  }
                }
              }
            }
            __syncwarp();
            if (lane == 0) {
              atomicAdd(&ctl->mtiles_done, 1u);
              maybe_close(p);
            }
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sc.done_empty[d]);
      }
    }
    __syncwarp();
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
      // last CTA out: whatever is left in the queues (nothing after a clean launch) is dropped and
      // the rank is reopened for the next launch (an aborted launch stays closed until the host
      // re-creates it).
      fence_acqrel<false>();
      for (int qi = 0; qi < 3; ++qi) {
        st_relaxed<false>(&ctl->q[qi].tail, ld_relaxed<false>(&ctl->q[qi].head));
        st_relaxed<false>(&ctl->q[qi].avail, 0u);
      }
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
