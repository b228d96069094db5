// The persistent MoE-layer kernel for sm_100a and its thin C ABI.
//
// One CTA per SM, every CTA a worker that pulls tasks from a ticket-based global
// queue and overlaps these kinds of work:
//   GATE    token tile: gate GEMM on tcgen05, top-k, softmax, row reservation in
//           the owners' expert buffers and entries in this rank's per-expert send
//           lists (tokens whose leading logits are nearly tied are recomputed by a
//           GATEFIX task with fp32 FMAs in the reference's accumulation order, so
//           the selection is the reference's);
//   GATED   all ranks have gated: lays out this rank's PACK tasks, expert by expert;
//   PACK    up to 72 rows of one expert: bulk copies into the owner's expert buffer;
//           the sender that completes an expert publishes its FFN1 tiles;
//   FFN1/2  128-row expert tiles on tcgen05 with TMEM accumulators fed by TMA
//           (SwiGLU epilogue; routing-weight epilogue stored on the home rank);
//   COMBINE token group: ordered sum of the K weighted rows.
// Cross-GPU traffic is plain stores, bulk stores and scoped atomics into peers'
// symmetric buffers.
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
constexpr int kDone = 4;  // depth of the hand-off ring to the completion warp
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
  uint32_t run_round2;  // set by a task body that found this rank's second GATED round due: the group runs it next
  // Copy of the kernel parameters for the task bodies that are compiled as separate functions:
  // there the parameter block is only reachable through a generic pointer, and every access to
  // the constant bank through one costs on the order of a hundred cycles; shared memory does not.
  // (TMA descriptors are always taken from the original.)
  FdmoeParams params;
  // The epilogue group runs one task at a time, so the scratch of a GATE task
  // and the store staging of an FFN task share storage.  16-byte aligned: the
  // staging buffer is accessed with 16-byte vector loads and stores.
  union alignas(16) {
    struct {
      // GATE task scratch (per expert / per token of the tile)
      uint32_t cnt[128];
      uint32_t base[128];
      uint32_t sbase[128];                      // first send-list entry of the tile per expert
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
    // FFN epilogues: per-warp staging of a 32-row x 64-byte chunk (80-byte pitch
    // keeps the 16-byte accesses of a quarter warp on distinct banks)
    uint8_t store_stage[kEpiThreads / 32][32 * 80];
  };
};

constexpr int kSmemBytes = kStages * kStageBytes + (int)sizeof(SmemCtl) + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA exceeds the sm_100 limit");
static_assert(offsetof(SmemCtl, xrow) % 16 == 0 && offsetof(SmemCtl, logit_tile) % 16 == 0 && (132 * 4) % 16 == 0,
              "vector accesses to the gate scratch need 16-byte alignment");
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

// Bounded mbarrier wait.  Returns false (after raising the error) on timeout
// or when another role of this CTA has aborted.
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
// or when another role of this CTA has aborted.
__device__ __forceinline__ bool wait_bar(const FdmoeParams& p, SmemCtl& sc, uint64_t* bar,
                                         uint32_t parity, uint32_t err_code) {
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
      if (waited > p.timeout_ns) {
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
  }
  // one fence orders every payload (and whatever the caller wrote before) ahead of the
  // sequence words; a release store per slot would pay for a fence each time
  fence_acqrel<S>();
  for (uint32_t i = 0; i < n; ++i) st_relaxed<S>(&q.slots[(t0 + i) & (uint32_t)p.queue_mask].seq, t0 + i + 1u);
}

// Tokens per COMBINE task of a rank with T tokens: at most `cap`, and such that the tasks fill
// whole waves of `grid` workers (e.g. 4096 tokens on 148 workers: 14 tokens, 293 tasks, two
// waves).  A pure function of T, so that a peer can publish another rank's COMBINE tasks.
__device__ __forceinline__ uint32_t combine_group_of(int T, int grid, int cap) {
  if (T <= 0) return 1u;
  const int waves = (T + cap * grid - 1) / (cap * grid);
  const int g = (T + waves * grid - 1) / (waves * grid);
  return (uint32_t)max(1, min(g, cap));
}

__device__ __forceinline__ uint32_t task_word(uint32_t kind, uint32_t e, uint32_t n) {
  return kind | (e << 8) | (n << 20);
}

// Consumer (single thread).  A task in the rank's urgent word goes first; otherwise take a
// ticket and wait (bounded) until its slot is published or the queue is closed.  While it waits
// the consumer also serves the urgent word; the ticket it holds then stays with it
// (`has_ticket`) and is waited for on the next call.
// Urgent word: 0 = none, else 0x80000000 | kind | b << 8.  It carries the GATED tasks, which must
// not queue up behind the hundreds of PACK tasks they publish.
__device__ __forceinline__ FdmoeSlot urgent_task(uint32_t word) {
  FdmoeSlot out;
  out.seq = 0;
  out.a = word & 0xffu;
  out.b = (word >> 8) & 0xffu;
  out.c = 0;
  return out;
}
template <bool S>
__device__ __forceinline__ void push_urgent(const FdmoeParams& p, const FdmoePeer& q, uint32_t kind, uint32_t b) {
  fence_acqrel<S>();
  const uint32_t old = atom_exch<S>(&q.ctl->urgent, 0x80000000u | kind | (b << 8));
  if (old != 0u) {  // (never two at a time by construction; do not lose it if it happens)
    queue_push<S>(p, q, 1u, [old](uint32_t, uint32_t& a, uint32_t& bb, uint32_t& c) {
      a = old & 0xffu;
      bb = (old >> 8) & 0xffu;
      c = 0;
    });
  }
}
template <bool S>
__device__ __forceinline__ FdmoeSlot queue_pop(const FdmoeParams& p, SmemCtl& sc, uint32_t& ticket, bool& has_ticket) {
  const FdmoePeer& me = p.peers[p.rank];
  FdmoeSlot out;
  out.seq = 0;
  out.a = FDMOE_TASK_EXIT;
  out.b = 0;
  out.c = 0;
  if (sc.abort) return out;
  if (!has_ticket) {
    if (ld_relaxed<S>(&me.ctl->urgent) != 0u) {
      const uint32_t u = atom_exch<S>(&me.ctl->urgent, 0u);
      if (u != 0u) return urgent_task(u);
    }
    ticket = atomicAdd(&me.ctl->q_tail, 1u);
    has_ticket = true;
  }
  FdmoeSlot* s = &me.slots[ticket & (uint32_t)p.queue_mask];
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (ld_acquire<S>(&s->seq) == ticket + 1u) break;
    if (ld_relaxed<S>(&me.ctl->closed) != 0u || sc.abort) return out;
    if (ld_relaxed<S>(&me.ctl->urgent) != 0u) {
      const uint32_t u = atom_exch<S>(&me.ctl->urgent, 0u);
      if (u != 0u) return urgent_task(u);
    }
    if ((++spins & 15u) == 0u) {
      if (ptx::globaltimer_ns() - t0 > p.timeout_ns) {
        raise_error(p, sc, FDMOE_ERR_TIMEOUT_QUEUE, (blockIdx.x << 8));
        return out;
      }
      __nanosleep(100);
    }
  }
  has_ticket = false;
  out.a = s->a;
  out.b = s->b;
  out.c = s->c;
  return out;
}

// Closes this rank's queue once GATED has run, every m-tile of its experts
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

// The routing of every token of this rank is decided (rows reserved on their
// owners, send lists complete): tell every rank; whoever completes a rank's
// count hands it the GATED task, from which its row counts are final.
// Two things must have happened before rank q's second GATED round may run: every rank has gated,
// and rank q has laid out its first round (a rank without tokens has none and counts both at once).
// Whoever brings the count to two hands rank q the task.
// `sc` non-null: the caller is thread 0 of an epilogue group at the end of a task; if the round
// falls to its own rank the group runs it right away (flag run_round2) instead of queueing it.
template <bool S>
__device__ __forceinline__ void second_round_ready(const FdmoeParams& p, SmemCtl* sc, int q, uint32_t n) {
  fence_acqrel<S>();
  const uint32_t prev = atom_add<S>(&p.peers[q].ctl->round2_rdv, n);
  if (prev + n == 2u) {
    if (sc && q == p.rank)
      sc->run_round2 = 1u;
    else
      push_urgent<S>(p, p.peers[q], FDMOE_TASK_GATED, 0u);  // second round
  }
}

template <bool S>
__device__ void gating_finished(const FdmoeParams& p, SmemCtl* sc) {
  for (int q = 0; q < p.world; ++q) {
    fence_acqrel<S>();
    const uint32_t prev = atom_add<S>(&p.peers[q].ctl->ranks_gated, 1u);
    // rank q's second round starts when every rank has gated and its own first round is laid out
    if (prev == (uint32_t)p.world - 1u) second_round_ready<S>(p, sc, q, 1u);
  }
}

// Counts `n` tokens of this rank as gated; the caller has written their send-list entries.
template <bool S>
__device__ __forceinline__ void count_gated(const FdmoeParams& p, SmemCtl& sc, uint32_t n) {
  fence_acqrel<S>();
  const uint32_t done = atomicAdd(&p.peers[p.rank].ctl->gated_tokens, n) + n;
  if (n && done == (uint32_t)p.T) gating_finished<S>(p, &sc);
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
// leading nine logits contain an adjacent pair closer than tau = 6e-8 * H of the
// scale (more than ten times that difference on each side) is handed to a
// GATEFIX task, which recomputes its logits in the reference's order; for every
// other token both orders select the same experts in the same order.
template <bool S>
__device__ __noinline__ void gate_epilogue(const FdmoeParams& p, SmemCtl& sc, uint32_t taddr, uint64_t* tmem_empty_bar,
                                           int q, int h, int lane, int etid, int ewarp, uint32_t tile) {
  const int E = p.E, K = p.K;
  const int t0 = (int)tile * p.gate_rows;
  const int nt = min(p.gate_rows, p.T - t0);
  const int kk = min(E, 9);
  const int npass = p.gate_rows / 32;

  if (etid < 128) sc.cnt[etid] = 0;
  if (etid == 0) sc.n_flagged = 0;
  // ---- four passes, one per TMEM lane quadrant: the two warps that may read the
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
      const float tau = 6e-8f * (float)p.H * fmaxf(1.0f, fabsf(sc.top_v[etid][0]));
      for (int j = 0; j + 1 < kk; ++j) tie |= (sc.top_v[etid][j] - sc.top_v[etid][j + 1]) < tau;
      if (tie) sc.flagged[atomicAdd(&sc.n_flagged, 1u)] = (uint32_t)etid;
    }
    sc.isflag[etid] = tie ? 1 : 0;
  }
  epi_bar();
  prof_mark(p, sc, etid, 3);
  if (etid < nt && !sc.isflag[etid]) {
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
        const int e = sc.top_i[etid][k];
        const float w = ex[k] / sum;
        sc.tk_w[etid][k] = w;
        sc.lpos[etid][k] = (uint8_t)atomicAdd(&sc.cnt[e], 1u);
        p.topk_idx[(size_t)(t0 + etid) * K + k] = e;
        p.topk_w[(size_t)(t0 + etid) * K + k] = w;
      }
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 5);
  // reserve rows in the owners' expert buffers and entries in this rank's send
  // lists: one atomic each per expert and tile
  if (etid < E) {
    const uint32_t cnt = sc.cnt[etid];
    if (cnt) {
      const int owner = etid / p.El, le = etid - owner * p.El;
      const uint32_t base = atom_add<S>(&p.peers[owner].expert_cnt[le], cnt);
      if (base + cnt > (uint32_t)p.cap_rows) raise_error(p, sc, FDMOE_ERR_ROW_OVERFLOW, etid);
      sc.base[etid] = base;
      sc.sbase[etid] = atomicAdd(&p.send_cnt[etid], cnt);
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 6);
  if (etid < nt && !sc.isflag[etid] && !sc.abort) {
    for (int k = 0; k < K; ++k) {
      const int e = sc.top_i[etid][k];
      const int owner = e / p.El, le = e - owner * p.El;
      const size_t rowg = (size_t)le * p.cap_rows + sc.base[e] + sc.lpos[etid][k];
      const size_t ent = (size_t)e * p.send_stride + sc.sbase[e] + sc.lpos[etid][k];
      p.send_src[ent] = ((t0 + etid) << 4) | k;
      p.send_dst[ent] = (int32_t)rowg;
      // FdmoeRowMeta {token, home << 8 | slot, weight, pad} as one 16-byte store
      *reinterpret_cast<uint4*>(&p.peers[owner].meta[rowg]) =
          make_uint4((uint32_t)(t0 + etid), (uint32_t)((p.rank << 8) | k), __float_as_uint(sc.tk_w[etid][k]), 0u);
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 7);
  if (etid == 0 && !sc.abort) {
    const uint32_t nf = sc.n_flagged, nfix = (nf + 1u) / 2u;
    if (nfix) {
      fence_acqrel<false>();
      queue_push<false>(p, p.peers[p.rank], nfix, [&](uint32_t i, uint32_t& a, uint32_t& b, uint32_t& c) {
        a = FDMOE_TASK_GATEFIX;
        b = (uint32_t)t0 + sc.flagged[2 * i];
        c = (2 * i + 1 < nf) ? (uint32_t)t0 + sc.flagged[2 * i + 1] : 0xffffffffu;
      });
    }
    count_gated<S>(p, sc, (uint32_t)nt - nf);
    // the last GATE tile of this rank: its rows so far (all but those of nearly tied tokens) can be packed
    const uint32_t tiles = (uint32_t)((p.T + p.gate_rows - 1) / p.gate_rows);
    fence_acqrel<false>();
    if (atomicAdd(&p.peers[p.rank].ctl->gate_tiles_done, 1u) + 1u == tiles) {
      if (p.pack_early)
        push_urgent<false>(p, p.peers[p.rank], FDMOE_TASK_GATED, 1u);  // first round now
      else
        second_round_ready<S>(p, &sc, p.rank, 1u);  // both rounds once every rank has gated
    }
  }
}

// ===================================================================== PACK
// Sends `count` rows of one expert (entries [first, first + count) of this rank's
// send list for it) to the expert's owner.  The rows travel as bulk copies:
// the TMA warp brings up to pack_rows_per_stage() token rows into a pipeline
// stage, the lanes of the first epilogue warp send one row each from there into
// the owner's expert buffer (local, or a peer's over NVLink).  The sender whose
// rows complete the expert while its row count is known to be final (every rank
// has gated) publishes the expert's FFN1 tile tasks on the owner's queue; an
// expert that completes earlier is left to the owner's second GATED round.
__device__ __forceinline__ uint32_t pack_rows_per_stage(int H) {
  return min(16u, (uint32_t)kStageBytes / ((uint32_t)H * 2u));
}

// TMA-warp side of a PACK task (one thread): brings the token rows of the piece into the
// pipeline stages, up to pack_rows_per_stage() rows per stage.  The source indices of the
// next stage are fetched while the current one is waited for and issued.
__device__ __noinline__ bool pack_loads(const FdmoeParams& p, SmemCtl& sc, uint8_t* stage, uint32_t& stage_it,
                                        uint32_t e, uint32_t first, uint32_t count) {
  const uint32_t rowb = (uint32_t)p.H * 2u, rps = pack_rows_per_stage(p.H);
  const int32_t* src_list = p.send_src + (size_t)e * p.send_stride + first;
  const uint8_t* xb = reinterpret_cast<const uint8_t*>(p.x);
  int32_t cur[16], nxt[16];
#pragma unroll
  for (uint32_t i = 0; i < 16; ++i) cur[i] = (i < rps && i < count) ? __ldcg(src_list + i) : 0;
  for (uint32_t b0 = 0; b0 < count; b0 += rps, ++stage_it) {
    const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
    const uint32_t nrows = min(rps, count - b0);
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i) nxt[i] = (i < rps && b0 + rps + i < count) ? __ldcg(src_list + b0 + rps + i) : 0;
    if (!wait_bar(p, sc, &sc.empty_bar[s], sph ^ 1u, FDMOE_ERR_TIMEOUT_STAGE)) return false;
    ptx::mbar_expect_tx(&sc.full_bar[s], nrows * rowb);
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i)
      if (i < nrows)
        ptx::bulk_load_1d(stage + s * kStageBytes + i * rowb, xb + (size_t)(cur[i] >> 4) * rowb, rowb, &sc.full_bar[s]);
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i) cur[i] = nxt[i];
  }
  return true;
}

// All rows of local expert `le` of rank `op` have landed and their number `total` is final: its FFN1
// tile tasks go onto that rank's queue, m-tile major, so that the tiles of one expert run together and
// share its weights through L2.  Called by the whole epilogue group; exactly one caller per expert and
// launch gets to publish (flag `published`).
template <bool S>
__device__ __forceinline__ void publish_expert_tiles(const FdmoeParams& p, SmemCtl& sc, int etid, const FdmoePeer& op,
                                                     uint32_t le, uint32_t total) {
  const uint32_t nt1 = (uint32_t)(p.I / FDMOE_TILE_N1);
  const uint32_t full = total / 128u, rem = total % 128u, ntask = ((total + 127u) / 128u) * nt1;
  if (etid == 0) {
    sc.q_total = 0u;
    if (atom_exch<S>(&op.published[le], 1u) == 0u) {
      fence_acqrel<S>();  // the senders' rows (observed through the counter) before the tasks
      sc.q_t0 = atom_add<S>(&op.ctl->q_head, ntask);
      sc.q_total = ntask;
    }
  }
  epi_bar();
  if (sc.q_total) {
    const uint32_t t0 = sc.q_t0;
    bool any = false;
    for (uint32_t idx = etid; idx < ntask; idx += kEpiThreads) {
      const uint32_t j = idx / nt1, n = idx - j * nt1;
      FdmoeSlot* sl = &op.slots[(t0 + idx) & (uint32_t)p.queue_mask];
      sl->a = task_word(FDMOE_TASK_FFN1, le, n);
      sl->b = j;
      sl->c = (j < full) ? 128u : rem;
      any = true;
    }
    if (any) {
      fence_acqrel<S>();
      for (uint32_t idx = etid; idx < ntask; idx += kEpiThreads)
        st_relaxed<S>(&op.slots[(t0 + idx) & (uint32_t)p.queue_mask].seq, t0 + idx + 1u);
    }
  }
  epi_bar();  // sc.q_t0 / sc.q_total may be rewritten only after everyone has read them
}

template <bool S>
__device__ __noinline__ bool pack_task(const FdmoeParams& p, SmemCtl& sc, uint8_t* stage, uint32_t& stage_it, int etid,
                                       int ewarp, int lane, uint32_t e, uint32_t first, uint32_t count) {
  const int H = p.H;
  const uint32_t rowb = (uint32_t)H * 2u, rps = pack_rows_per_stage(H);
  const int owner = (int)e / p.El, le = (int)e - owner * p.El;
  const FdmoePeer& op = p.peers[owner];
  uint8_t* packed = reinterpret_cast<uint8_t*>(op.packed);
  const int32_t* dst_list = p.send_dst + (size_t)e * p.send_stride + first;
  for (uint32_t b0 = 0; b0 < count; b0 += rps, ++stage_it) {
    const uint32_t s = stage_it % kStages, sph = (stage_it / kStages) & 1u;
    const uint32_t nrows = min(rps, count - b0);
    int32_t d = 0;
    if (ewarp == 0 && (uint32_t)lane < nrows) d = __ldcg(dst_list + b0 + lane);
    if (!epi_vote_all(wait_bar(p, sc, &sc.full_bar[s], sph, FDMOE_ERR_TIMEOUT_STAGE))) return false;
    if (ewarp == 0) {
      if ((uint32_t)lane < nrows) {
        ptx::bulk_store_1d(packed + (size_t)d * rowb, stage + s * kStageBytes + (uint32_t)lane * rowb, rowb);
        ptx::bulk_commit_group();
        ptx::bulk_wait_group_read0();
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&sc.empty_bar[s]);
    }
  }
  if (ewarp == 0) {
    ptx::bulk_wait_group0();  // this lane's rows are written
    __syncwarp();
  }
  ptx::fence_proxy_async();  // packed rows are read by TMA
  epi_bar();
  if (etid == 0) {
    fence_acqrel<S>();
    const uint32_t prev = atom_add<S>(&op.landed[le], count);
    // Complete?  The row count of the expert is only final once every rank has gated; before that
    // the second GATED round of the owner will look at the expert again.  (Sequentially consistent
    // fences here and there: of this check and that look, at least one sees the other's update.)
    fence_sc<S>();
    const uint32_t total = ld_relaxed<S>(&op.expert_cnt[le]);
    const bool final_cnt = ld_acquire<S>(&op.ctl->ranks_gated) == (uint32_t)p.world;
    sc.flag = (final_cnt && prev + count == total) ? (int)total : 0;
  }
  epi_bar();
  if (sc.flag) publish_expert_tiles<S>(p, sc, etid, op, (uint32_t)le, (uint32_t)sc.flag);
  if (etid == 32) {
    // this piece is done: the next entry of this rank's pack list may go out
    FdmoeCtl* myctl = p.peers[p.rank].ctl;
    const uint32_t nxt = atomicAdd(&myctl->pack_cursor, 1u);
    if (nxt < ld_relaxed<false>(&myctl->pack_total)) {
      const uint4 t = ld_cg_u4(reinterpret_cast<const uint4*>(p.pack_list) + nxt);
      queue_push<false>(p, p.peers[p.rank], 1u, [&](uint32_t, uint32_t& a, uint32_t& b, uint32_t& c) {
        a = t.x;
        b = t.y;
        c = t.z;
      });
    }
  }
  epi_bar();  // sc.flag / sc.q_t0 may be rewritten by the next task only after everyone has read them
  return true;
}

// ================================================================== GATEFIX
// Up to two tokens whose leading tensor-core logits were nearly tied: all E
// logits are recomputed with fp32 FMAs in the reference's order (128 threads per
// token, one expert each), then top-k, softmax, row reservation and send-list
// entries, i.e. everything GATE does for the other tokens.
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
      const uint32_t pos = atom_add<S>(&p.peers[owner].expert_cnt[le], 1u);
      sc.fix_dst[half][lane] = make_uint2(0xffffffffu, 0u);
      if (pos >= (uint32_t)p.cap_rows) {
        raise_error(p, sc, FDMOE_ERR_ROW_OVERFLOW, (uint32_t)myi);
      } else {
        const size_t rowg = (size_t)le * p.cap_rows + pos;
        sc.fix_dst[half][lane] = make_uint2((uint32_t)myi, (uint32_t)rowg);  // this task sends the row itself (below)
        p.topk_idx[(size_t)tok * K + lane] = myi;
        p.topk_w[(size_t)tok * K + lane] = w;
        *reinterpret_cast<uint4*>(&p.peers[owner].meta[rowg]) =
            make_uint4(tok, (uint32_t)((p.rank << 8) | lane), __float_as_uint(w), 0u);
      }
    }
  }
  epi_bar();
  prof_mark(p, sc, etid, 32);
  // The token row (still in shared memory) goes to its K rows in the owners' expert buffers: these few
  // rows do not pass through PACK tasks.  Their landing counts as gated only below, so no expert can be
  // found complete with its count believed final before these rows are there; the second GATED round
  // looks at the experts they completed.
  if (live) {
    for (int k = 0; k < K; ++k) {
      const uint2 d = sc.fix_dst[half][k];
      if (d.x == 0xffffffffu) continue;
      const int owner = (int)d.x / p.El;
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.peers[owner].packed) + (size_t)d.y * H);
      for (int v = e; v < H / 8; v += 128) dst[v] = sc.xrow[half][v];
    }
    fence_acqrel<S>();
    ptx::fence_proxy_async();  // packed rows are read by TMA
  }
  epi_bar();
  if (live && e < K) {
    const uint2 d = sc.fix_dst[half][e];
    if (d.x != 0xffffffffu) {
      const int owner = (int)d.x / p.El, le = (int)d.x - owner * p.El;
      fence_acqrel<S>();
      atom_add<S>(&p.peers[owner].landed[le], 1u);
    }
  }
  epi_bar();
  if (etid == 0) count_gated<S>(p, sc, (tok_b != 0xffffffffu) ? 2u : 1u);
  return true;
}

// ============================================================ GATED and FFN
// GATED, first round, as soon as this rank's GATE tiles are done: lays out this rank's PACK tasks
// (pieces of FDMOE_PACK_ROWS rows of its send lists: the rows of all tokens but the nearly tied
// ones, which their GATEFIX tasks send themselves) in sending order and publishes the first
// pack_window of them; every PACK task that finishes publishes the next one, so that packing,
// whose pace is set by memory writes or by NVLink, shares the workers with the GATEFIX tasks and
// with the FFN1 tiles of experts that have already landed.  Sending order: step i goes to local
// expert i / world of rank (rank + 1 + i) % world, so that at every step the ranks send to
// different owners and the experts of all ranks complete one after the other.
// Second round, once every rank has gated (row counts are final): the number of m-tiles this
// rank will process (termination), and a look at this rank's experts for any that landed
// completely before their count was known to be final.
template <bool S>
__device__ __noinline__ void gated_task(const FdmoeParams& p, SmemCtl& sc, int etid, bool first_round) {
  const FdmoePeer& me = p.peers[p.rank];
  const int lane = etid & 31, w = etid >> 5;
  // (the task was taken from the queue with an acquire load ordered after the events it stands for)
  uint32_t ntile = 0, npack = 0, ecnt = 0, lcnt = 0;
  const int e_send = (etid < p.E) ? ((p.rank + 1 + etid) % p.world) * p.El + etid / p.world : 0;
  if (!first_round && etid < p.El) {
    lcnt = ld_relaxed<S>(&me.expert_cnt[etid]);
    ntile = (lcnt + 127u) / 128u;
  }
  if (first_round && etid < p.E) {
    ecnt = __ldcg(&p.send_cnt[e_send]);
    npack = (ecnt + FDMOE_PACK_ROWS - 1) / FDMOE_PACK_ROWS;
  }
  uint32_t inc_pack = npack, inc_tile = ntile;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t a = __shfl_up_sync(0xffffffffu, inc_pack, off);
    const uint32_t b = __shfl_up_sync(0xffffffffu, inc_tile, off);
    if (lane >= off) {
      inc_pack += a;
      inc_tile += b;
    }
  }
  if (lane == 31 && w < 4) {
    sc.pre[w] = inc_pack;
    sc.pre[8 + w] = inc_tile;
  }
  epi_bar();
  uint32_t off_pack = 0, total = 0, mt = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i < w) off_pack += sc.pre[i];
    total += sc.pre[i];
    mt += sc.pre[8 + i];
  }
  if (first_round) {
    const uint32_t window = min(total, (uint32_t)p.pack_window);
    if (etid == 0) {
      sc.q_t0 = window ? atom_add<false>(&me.ctl->q_head, window) : 0u;
      st_relaxed<false>(&me.ctl->pack_total, total);
      st_relaxed<false>(&me.ctl->pack_cursor, window);
    }
    // the tasks in sending order: entries [first, first + count) of the expert's send list
    uint4* plist = reinterpret_cast<uint4*>(p.pack_list);
    const uint32_t firstslot = off_pack + inc_pack - npack;  // exclusive prefix in sending order
    for (uint32_t r = 0; r < npack; ++r)
      plist[firstslot + r] = make_uint4(task_word(FDMOE_TASK_PACK, (uint32_t)e_send, 0u), r * FDMOE_PACK_ROWS,
                                        min((uint32_t)FDMOE_PACK_ROWS, ecnt - r * FDMOE_PACK_ROWS), 0u);
    epi_bar();
    const uint32_t t0 = sc.q_t0;
    bool any = false;
    for (uint32_t idx = (uint32_t)etid; idx < window; idx += kEpiThreads) {
      const uint4 t = ld_cg_u4(&plist[idx]);
      FdmoeSlot* sl = &me.slots[(t0 + idx) & (uint32_t)p.queue_mask];
      sl->a = t.x;
      sl->b = t.y;
      sl->c = t.z;
      any = true;
    }
    // one fence orders every payload (and the list, the cursor and the total) before every sequence word below
    if (any || etid == 0) fence_acqrel<false>();
    for (uint32_t idx = (uint32_t)etid; idx < window; idx += kEpiThreads)
      st_relaxed<false>(&me.slots[(t0 + idx) & (uint32_t)p.queue_mask].seq, t0 + idx + 1u);
    epi_bar();
    if (etid == 0 && p.pack_early) second_round_ready<S>(p, &sc, p.rank, 1u);
    return;
  }
  if (etid == 0) st_relaxed<false>(&me.ctl->mtiles_total, mt);
  // Experts of this rank whose rows had all landed while their count was not yet known to be final:
  // nobody has published their tiles.  (Fence: see pack_task.)  Every thread looks at one expert and
  // claims it; the tasks of all claimed experts are published in one batch.
  fence_sc<S>();
  const uint32_t nt1 = (uint32_t)(p.I / FDMOE_TILE_N1);
  const bool cand = etid < p.El && lcnt != 0u && ld_relaxed<S>(&me.landed[etid]) == lcnt &&
                    atom_exch<S>(&me.published[etid], 1u) == 0u;
  const uint32_t mytasks = cand ? ((lcnt + 127u) / 128u) * nt1 : 0u;
  uint32_t inc = mytasks;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t a = __shfl_up_sync(0xffffffffu, inc, off);
    if (lane >= off) inc += a;
  }
  if (lane == 31 && w < 4) sc.pre[w] = inc;
  epi_bar();
  uint32_t before = 0, all = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i < w) before += sc.pre[i];
    all += sc.pre[i];
  }
  if (etid == 0 && all) {
    fence_acqrel<S>();
    sc.q_t0 = atom_add<false>(&me.ctl->q_head, all);
  }
  epi_bar();
  if (mytasks) {
    const uint32_t t1 = sc.q_t0 + before + inc - mytasks;
    const uint32_t full = lcnt / 128u, rem = lcnt % 128u;
    for (uint32_t idx = 0; idx < mytasks; ++idx) {
      const uint32_t jt = idx / nt1, n = idx - jt * nt1;
      FdmoeSlot* sl = &me.slots[(t1 + idx) & (uint32_t)p.queue_mask];
      sl->a = task_word(FDMOE_TASK_FFN1, (uint32_t)etid, n);
      sl->b = jt;
      sl->c = (jt < full) ? 128u : rem;
    }
    fence_acqrel<false>();
    for (uint32_t idx = 0; idx < mytasks; ++idx)
      st_relaxed<false>(&me.slots[(t1 + idx) & (uint32_t)p.queue_mask].seq, t1 + idx + 1u);
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

// COMBINE streams the K weighted rows of each token of a group through the
// shared-memory stage ring with 1-D bulk copies (issued by the TMA warp) in
// pieces of up to 2048 columns: stage layout [K][piece], 4 KB per slot row.
constexpr int kCombineCols = 2048;

// k-blocks a tile task puts into one pipeline stage: two for GATE tiles of up to 64 tokens
// (H is a multiple of 256, so the number of k-blocks is even), one otherwise.
__device__ __forceinline__ uint32_t gate_kblocks_per_stage(bool is_gate, int gate_rows) {
  return (is_gate && gate_rows <= 64) ? 2u : 1u;
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
    st_relaxed<S>(&ctl->tokens_launch, (uint32_t)p.T);
  }
  {
    static_assert(sizeof(FdmoeParams) % 16 == 0, "parameter block is copied in 16-byte pieces");
    const uint4* src = reinterpret_cast<const uint4*>(&p);
    uint4* dst = reinterpret_cast<uint4*>(&sc.params);
    for (int i = tid; i < (int)(sizeof(FdmoeParams) / 16); i += kThreads) dst[i] = src[i];
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

  // ---- seed the queue: every CTA publishes its share of the GATE tasks (tile b, b + grid, ...),
  // so that all tiles are available at once.  Nothing to gate: the rank's "gate phase" is
  // finished at once (it may still serve its peers).
  if (p.mode != 2 && !sc.abort && tid == 0) {
    const uint32_t n_tiles = (p.T > 0 && p.gate_rows > 0) ? (uint32_t)((p.T + p.gate_rows - 1) / p.gate_rows) : 0u;
    if (n_tiles == 0) {
      if (blockIdx.x == 0) {
        second_round_ready<S>(p, nullptr, p.rank, 1u);  // no first round to wait for
        gating_finished<S>(p, nullptr);
      }
    } else if (blockIdx.x < n_tiles) {
      const uint32_t mine = (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
      queue_push<false>(p, me, mine, [](uint32_t i, uint32_t& a, uint32_t& b, uint32_t& c) {
        a = FDMOE_TASK_GATE;
        b = blockIdx.x + i * gridDim.x;
        c = 0;
      });
    }
  }

  // =============================== worker loop
  const uint32_t nt1 = (uint32_t)(p.I / FDMOE_TILE_N1), nt2 = (uint32_t)(p.H / FDMOE_TILE_N2);
  const uint32_t nkb1 = (uint32_t)(p.H / FDMOE_TILE_K), nkb2 = (uint32_t)(p.I / FDMOE_TILE_K);

  if (warp == kWarpSched) {
    if (lane == 0) {
      uint32_t ticket = 0;
      bool has_ticket = false;
      for (uint32_t it = 0;; ++it) {
        const uint32_t r = it % kRing, ph = (it / kRing) & 1u;
        if (!wait_bar(p, sc, &sc.ring_empty[r], ph ^ 1u, FDMOE_ERR_TIMEOUT_RING)) {
          // The ring may be wedged: hand out EXIT through every slot that is free.
          break;
        }
        const FdmoeSlot t = queue_pop<S>(p, sc, ticket, has_ticket);
        sc.ring[r] = t;
        ptx::mbar_arrive(&sc.ring_full[r]);
        const uint32_t kind = t.a & 0xffu;
        if (kind == FDMOE_TASK_EXIT) break;
        if (kind != FDMOE_TASK_FFN1 && kind != FDMOE_TASK_FFN2 && kind != FDMOE_TASK_COMBINE && kind != FDMOE_TASK_PACK) {
          // Only tile tasks (and COMBINE / PACK, whose rows travel as bulk copies) profit from being queued behind one another (their loads and
          // MMAs run ahead of the epilogue).  Behind a long task of another kind a claimed
          // ticket would just sit here while other workers idle: wait until it is done.
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
        if (!wait_bar(p, sc, &sc.ring_full[r], ph, FDMOE_ERR_TIMEOUT_RING)) break;
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
            if ((p.debug_flags & 8) && !gt) {  // timing experiment: tiles computed from stale operands
              ptx::mbar_arrive(&sc.full_bar[s]);
              continue;
            }
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
        } else if (kind == FDMOE_TASK_PACK) {
          const bool ok = pack_loads(sc.params, sc, stage, stage_it, (t.a >> 8) & 0xfffu, t.b, t.c);
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
              for (int k = 0; k < p.K; ++k)
                ptx::bulk_load_1d(sa + k * (kCombineCols * 2), ys + ((size_t)tk * p.K + k) * p.H + c0, wbytes,
                                  &sc.full_bar[s]);
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
          const uint32_t gk = gate_kblocks_per_stage(kind == FDMOE_TASK_GATE, p.gate_rows);
          bool ok = true;
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
        } else if (kind == FDMOE_TASK_GATEFIX || kind == FDMOE_TASK_COMBINE || kind == FDMOE_TASK_PACK) {
          // The stages of these tasks are consumed by the epilogue warps.  This warp must not
          // run ahead of them: a stage barrier only tells phases apart by parity, so a waiter
          // more than one phase ahead would take an old completion for its own.  Wait until
          // the epilogue has finished the task, then step over its stages.
          ++skips;
          const uint64_t t0w = ptx::globaltimer_ns();
          uint32_t spins = 0;
          bool ok = true;
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
          if (kind == FDMOE_TASK_GATEFIX) {
            stage_it += (nkb1 + kFixBlocks - 1) / kFixBlocks;
          } else if (kind == FDMOE_TASK_PACK) {
            const uint32_t rps = pack_rows_per_stage(p.H);
            stage_it += (t.c + rps - 1u) / rps;
          } else {
            const int t_begin = (int)t.b, t_end = t_begin + (int)t.c;
            stage_it += (uint32_t)((t_end - t_begin) * ((p.H + kCombineCols - 1) / kCombineCols));
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
        stage_it += nkb1 / gate_kblocks_per_stage(true, p.gate_rows);
        if (!epi_vote_all(wait_bar(p, sc, &sc.tmem_full[acc], aph, FDMOE_ERR_TIMEOUT_TMEM))) break;
        if (p.prof && etid == 0) pt1 = prof_now();
        ptx::tcgen05_fence_after();
        gate_epilogue<S>(sc.params, sc, tmem_base + acc * kAccCols, &sc.tmem_empty[acc], q, h, lane, etid, ewarp, j);
      } else if (kind == FDMOE_TASK_PACK) {
        if (!pack_task<S>(sc.params, sc, stage, stage_it, etid, ewarp, lane, e, j, rows)) break;
        if (etid == 0) {
          __threadfence_block();
          sc.skip_done = sc.skip_done + 1u;
        }
      } else if (kind == FDMOE_TASK_GATEFIX) {
        if (!gatefix_task<S>(sc.params, sc, stage, stage_it, etid, ewarp, lane, j, rows)) break;
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
        if (kind == FDMOE_TASK_FFN1)
          ffn1_epilogue(p, sc, taddr, q, h, lane, ewarp, e, j, n, rows);
        else
          ffn2_epilogue(p, sc, taddr, q, h, lane, ewarp, e, j, n, rows);
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sc.tmem_empty[acc]);
        const uint32_t pta = (p.prof && etid == 0) ? prof_now() : 0u;

        // The tile's stores are issued.  Dependency counting, successor pushes and
        // the notifications of the home ranks are done by the completion warp, off
        // the epilogue's critical path.
        // activations are read by TMA in FFN2, weighted rows by bulk copies in COMBINE
        if (!(p.debug_flags & 4)) ptx::fence_proxy_async();
        epi_bar();
        if (etid == 0 && p.mode != 2) {
          const uint32_t d = done_it % kDone, dph = (done_it / kDone) & 1u;
          if (wait_bar(p, sc, &sc.done_empty[d], dph ^ 1u, FDMOE_ERR_TIMEOUT_RING)) {
            sc.done_ring[d] = t;
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
                const uint4 rr = sm[k * (kCombineCols / 8)];
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
        if (j == 0u && !p.pack_early) gated_task<S>(sc.params, sc, etid, true);  // packing was held back until now
        gated_task<S>(sc.params, sc, etid, j == 1u);
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
      if (kind == FDMOE_TASK_GATE || kind == FDMOE_TASK_GATEFIX || kind == FDMOE_TASK_GATED) {
        // the task may have found this rank's second GATED round due: run it here and now
        epi_bar();
        const bool r2 = sc.run_round2 != 0u;
        epi_bar();
        if (r2) {
          if (etid == 0) sc.run_round2 = 0u;
          if (!p.pack_early) gated_task<S>(sc.params, sc, etid, true);
          gated_task<S>(sc.params, sc, etid, false);
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
    // ---- completion warp: per finished tile, count it and publish what it unblocks
    for (uint32_t it = 0;; ++it) {
      const uint32_t d = it % kDone, dph = (it / kDone) & 1u;
      int ok = 1;
      if (lane == 0) {
        // This warp may legitimately idle for a whole launch, so its own budget is four
        // times the others': whoever actually stalls reports first.
        ok = 0;
        for (int tries = 0; tries < 4 && !ok && !sc.abort; ++tries)
          ok = wait_idle(p, sc, &sc.done_full[d], dph) ? 1 : 0;
        if (!ok && !sc.abort) raise_error(p, sc, FDMOE_ERR_TIMEOUT_RING, (blockIdx.x << 8) | 3u);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const FdmoeSlot t = sc.done_ring[d];
      const uint32_t kind = t.a & 0xffu;
      if (kind == FDMOE_TASK_EXIT) break;
      const uint32_t e = (t.a >> 8) & 0xfffu, j = t.b, rows = t.c;
      if (kind == FDMOE_TASK_FFN1) {
        if (lane == 0) {
          if (!(p.debug_flags & 2)) fence_acqrel<false>();
          const uint32_t prev = atomicAdd(&p.ffn1_done[(size_t)e * p.MT + j], 1u);
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
        int last = 0;
        if (lane == 0) {
          if (!(p.debug_flags & 2)) fence_acqrel<S>();
          const uint32_t prev = atomicAdd(&p.ffn2_done[(size_t)e * p.MT + j], 1u);
          if (!(p.debug_flags & 2)) fence_acqrel<S>();
          last = prev == nt2 - 1u;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          // every hidden-column tile of this m-tile is stored: tell each home rank how many
          // of its rows that makes (one counter update per home rank and m-tile)
          uint32_t cnt[FDMOE_MAX_WORLD];
#pragma unroll
          for (int w = 0; w < FDMOE_MAX_WORLD; ++w) cnt[w] = 0u;
          if (p.world == 1) {
            if (lane == 0) cnt[0] = rows;  // every row is this rank's own
          } else {
            for (uint32_t r = lane; r < rows; r += 32) {
              const uint4 mraw = ld_cg_u4(&me.meta[(size_t)e * p.cap_rows + (size_t)j * 128 + r]);
              const int home = (int)mraw.y >> 8;
#pragma unroll
              for (int w = 0; w < FDMOE_MAX_WORLD; ++w) cnt[w] += (home == w) ? 1u : 0u;
            }
          }
          uint32_t mine = 0u;
#pragma unroll
          for (int w = 0; w < FDMOE_MAX_WORLD; ++w) {
            const uint32_t c = __reduce_add_sync(0xffffffffu, cnt[w]);
            if (lane == w) mine = c;
          }
          uint32_t th = 0u;
          if (lane < p.world && mine) {
            const FdmoePeer& hp = p.peers[lane];
            fence_acqrel<S>();
            const uint32_t prev = atom_add<S>(&hp.ctl->rows_arrived, mine);
            const uint32_t tl = (lane == p.rank) ? (uint32_t)p.T : ld_relaxed<S>(&hp.ctl->tokens_launch);
            if (prev + mine == tl * (uint32_t)p.K) th = tl;  // that home rank has all its rows
          }
          // ranks completed by this m-tile get their COMBINE tasks, published by the whole warp
          uint32_t complete = __ballot_sync(0xffffffffu, th != 0u);
          while (complete) {
            const int home = __ffs(complete) - 1;
            complete &= complete - 1u;
            const uint32_t tl = __shfl_sync(0xffffffffu, th, home);
            const FdmoePeer& hp = p.peers[home];
            const uint32_t grp = combine_group_of((int)tl, (int)gridDim.x, p.combine_group);
            const uint32_t ntask = (tl + grp - 1u) / grp;
            uint32_t t0 = 0u;
            if (lane == 0) {
              fence_acqrel<S>();
              t0 = atom_add<S>(&hp.ctl->q_head, ntask);
            }
            t0 = __shfl_sync(0xffffffffu, t0, 0);
            for (uint32_t i = lane; i < ntask; i += 32) {
              FdmoeSlot* sl = &hp.slots[(t0 + i) & (uint32_t)p.queue_mask];
              sl->a = FDMOE_TASK_COMBINE;
              sl->b = i * grp;
              sl->c = min(grp, tl - i * grp);
            }
            fence_acqrel<S>();  // each lane: its payloads (and the arrival counts seen above) before its sequence words
            for (uint32_t i = lane; i < ntask; i += 32)
              st_relaxed<S>(&hp.slots[(t0 + i) & (uint32_t)p.queue_mask].seq, t0 + i + 1u);
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
