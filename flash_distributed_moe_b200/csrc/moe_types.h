// Plain structs shared by the host launcher (C++) and the device code (CUDA).
// Everything here is POD so that it can cross the thin C ABI between them.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FDMOE_MAX_WORLD = 8,
  FDMOE_MAX_TOPK = 8,
  FDMOE_MAX_EXPERTS = 128,
  FDMOE_MAX_HIDDEN = 4096,  // a token row is staged in shared memory by the exact gate path
  FDMOE_TILE_M = 128,    // rows of one expert's packed buffer per GEMM tile
  FDMOE_TILE_N1 = 128,   // FFN1: activation columns per tile (MMA N = 2 * 128: gate + up)
  FDMOE_TILE_N2 = 256,   // FFN2: hidden columns per tile
  FDMOE_TILE_K = 64,     // one 128-byte swizzle atom of bf16 per stage
  FDMOE_GATE_TOKENS = 128,  // tokens per gate tile (one tcgen05 M tile)
};

// Task kinds.  A rank has three queues: queue 0 (taken first) holds what unblocks other work or
// frees memory early (FFN2 tiles, COMBINE groups, exact re-gating, the GATED round), queue 1 the
// FFN1 tiles, queue 2 the DISPATCH tasks, of which only a few run at a time when rows cross
// NVLink (the links, not the SMs, set their pace).  GATE tiles are not queued: workers claim them
// from a counter.
enum {
  FDMOE_TASK_NONE = 0,
  FDMOE_TASK_FFN1 = 1,     // (expert, m_tile, n_tile, rows): SwiGLU tile
  FDMOE_TASK_FFN2 = 2,     // (expert, m_tile, n_tile, rows): down-projection tile
  FDMOE_TASK_COMBINE = 3,  // (first token, count): ordered sum over the K slots
  FDMOE_TASK_GATED = 4,    // every rank has finished gating: row counts are final, publish what is left
  FDMOE_TASK_TESTA = 5,    // task-system self test: x[i] *= 2 over a chunk, then push TESTB
  FDMOE_TASK_TESTB = 6,    // task-system self test: x[i] += 1 over a chunk
  FDMOE_TASK_EXIT = 7,
  FDMOE_TASK_GATE = 8,     // (token tile): gate GEMM, top-k, softmax, row reservation
  FDMOE_TASK_DISPATCH = 9, // (first token, count): copies the tokens' rows into the owners' expert buffers
  FDMOE_TASK_GATEFIX = 10, // (token, token): exact fp32 gate of nearly tied tokens and their dispatch
};

// Status codes written by the kernel (first error wins).
enum {
  FDMOE_OK = 0,
  FDMOE_ERR_TIMEOUT_QUEUE = 1,   // a worker found no work for too long, or a claimed slot was never published
  FDMOE_ERR_TIMEOUT_RING = 2,    // CTA-internal task ring
  FDMOE_ERR_TIMEOUT_STAGE = 3,   // TMA/MMA shared-memory stage barrier
  FDMOE_ERR_TIMEOUT_TMEM = 4,    // accumulator hand-off barrier
  FDMOE_ERR_TIMEOUT_PEER = 5,    // a peer rank never entered the launch
  FDMOE_ERR_QUEUE_OVERFLOW = 6,
  FDMOE_ERR_BAD_TASK = 7,
  FDMOE_ERR_ROW_OVERFLOW = 8,    // more rows for an expert than its buffer holds
};

// One slot of a task queue (16 bytes).  `seq` == ticket + 1 once the slot
// holds the task of that ticket.
typedef struct {
  uint32_t seq;
  uint32_t a;  // kind | expert << 8 | n_tile << 20
  uint32_t b;  // m_tile, or first token, or chunk index
  uint32_t c;  // valid rows in the tile, or token count
} FdmoeSlot;

// Sideband of one packed row (16 bytes): where its result goes.
typedef struct {
  int32_t token;      // index of the token on its home rank
  int32_t home_slot;  // home rank << 8 | slot k
  float weight;       // routing weight of (token, slot)
  int32_t pad;
} FdmoeRowMeta;

// State of one task queue, on a 128-byte line of its own.  Producers (this rank and its peers)
// take tickets from `head` and add what they have published to `avail`; this rank's workers take
// a unit of `avail` (a signed count) and then a ticket from `tail`.
typedef struct {
  uint32_t head;
  uint32_t tail;
  uint32_t avail;
  uint32_t pad[29];
} FdmoeQueueCtl;

// Per-rank control block.  Lives in the rank's symmetric arena so that peers
// can reach it.  Fields on separate 128-byte lines are written by different
// agents.
typedef struct {
  // --- persistent state (never zeroed between launches)
  FdmoeQueueCtl q[3];
  uint32_t closed;  // 0 running, 1 finished, 2 aborted
  uint32_t status;  // first error code
  uint32_t status_info;
  uint32_t exit_cnt;
  uint32_t pad2[28];
  uint32_t ready[32];  // ready[r] = launch epoch of peer r (written by peer r)
  uint32_t tokens_of[2][16];  // [epoch & 1][r] = tokens of rank r in that launch (written by rank r)
  // --- per-launch counters: [launch_begin, launch_end) is zeroed before each launch
  uint32_t launch_begin;
  uint32_t gated_tokens;     // tokens of this rank whose routing is decided and whose rows have landed
  uint32_t ranks_gated;      // ranks whose gating is finished (incl. this one)
  uint32_t gated_done;       // the second gating round of this launch has run (tile total is set)
  uint32_t mtiles_total;     // m-tiles of this rank's experts this launch
  uint32_t mtiles_done;      // m-tiles whose FFN2 is complete
  uint32_t tokens_combined;
  uint32_t tokens_launch;    // tokens of this rank this launch (written at kernel start)
  uint32_t executed;         // tasks finished (used only with expected_static)
  uint32_t gate_next;        // next GATE tile to claim
  uint32_t disp_active;      // DISPATCH tasks being worked on
  uint32_t pad3[21];
} FdmoeCtl;

// What one rank can reach of a peer (or of itself): all device pointers valid
// in this process.
typedef struct {
  FdmoeCtl* ctl;
  FdmoeSlot* slots[3];     // the task queues
  uint32_t* expert_cnt;    // [El]       rows reserved per local expert
  uint32_t* landed;        // [El * MT]  rows landed per local expert and batch of m-tiles (batch b at [le * MT + b])
  uint32_t* grp_cnt;       // [groups]   weighted rows that have come back, per COMBINE group of this rank's tokens
  void* packed;            // bf16 [El * cap_rows, H]
  FdmoeRowMeta* meta;      // [El * cap_rows]
  void* ystage;            // bf16 [max_tokens, K, H]
} FdmoePeer;

// 128-byte opaque TMA descriptor (CUtensorMap), kept as raw words so that this
// header does not need cuda.h.
typedef struct __attribute__((aligned(64))) {
  uint64_t opaque[16];
} FdmoeTensorMap;

typedef struct {
  FdmoeTensorMap tm_packed;  // [El*cap_rows, H]   box 64 x 128
  FdmoeTensorMap tm_w13;     // [El*2I, H]         box 64 x 128
  FdmoeTensorMap tm_act;     // [El*cap_rows, I]   box 64 x 128
  FdmoeTensorMap tm_w2;      // [El*H, I]          box 64 x 256
  FdmoeTensorMap tm_x;       // [T, H]             box 64 x min(128, T)   (rebuilt per launch)
  FdmoeTensorMap tm_gate;    // [E, H]             box 64 x min(128, E)

  FdmoePeer peers[FDMOE_MAX_WORLD];  // peers[rank] is this rank itself

  // shape
  int32_t H, I, E, K, El;
  int32_t world, rank;
  int32_t T;            // tokens this launch
  int32_t cap_rows;     // rows per expert buffer (multiple of 128)
  int32_t MT;           // cap_rows / 128
  int32_t queue_mask;   // capacity - 1 of either queue (capacity is a power of two)
  int32_t combine_group;  // tokens per COMBINE task
  int32_t gate_rows;    // tokens per GATE task: 32, 64 or 128 (rows of the 128-row MMA tile that are used)
  int32_t disp_conc;    // DISPATCH tasks worked on at a time
  int32_t batch_mt;     // m-tiles per publication batch; 0 = chosen from the token counts of the launch
  int32_t mode;         // 0 full layer; 2 static tasks only (no gate)
  uint32_t expected_static;  // mode 2: tasks pre-filled by the host
  uint32_t epoch;       // launch counter (identical on all ranks)
  uint64_t timeout_ns;       // budget of every device-side wait inside a launch
  uint64_t peer_timeout_ns;  // budget of the wait for the peers to enter the launch

  const void* x;        // bf16 [T, H]
  void* out;            // bf16 [T, H] (may alias x)
  const void* gate_w;   // bf16 [E, H]
  void* act;            // bf16 [El * cap_rows, I]
  int32_t* topk_idx;    // [max_tokens, K]
  float* topk_w;        // [max_tokens, K]
  uint8_t* tok_flag;    // [max_tokens] 1: nearly tied token, routed and sent by its GATEFIX task
  uint32_t* ffn1_done;  // [El * MT]
  uint32_t* ffn2_done;  // [El * MT]
  uint32_t* status_host;  // mapped pinned word: first error code, readable without a sync
  int32_t* test_buf;    // task-system self test payload
  float* debug_logits;  // optional dump of the tensor-core gate logits [T, 128] (NULL = off)
  uint32_t* stuck;      // [grid][16 warps][4] where each role gave up waiting (diagnostics)
  uint32_t* prof;       // optional event trace, FDMOE_PROF_EVENTS x 4 words per CTA (NULL = off)
} FdmoeParams;

enum { FDMOE_PROF_EVENTS = 512 };

// Thin C ABI between the C++ host launcher and the CUDA translation unit.
// All functions return a cudaError_t value as int.
int fdmoe_kernel_prepare(int* smem_bytes_out, int* grid_out);
int fdmoe_kernel_launch(const FdmoeParams* params, int grid, void* stream);
int fdmoe_cast_f32_to_bf16(const float* src, void* dst, uint64_t n, void* stream);
int fdmoe_cast_bf16_to_f32(const void* src, float* dst, uint64_t n, void* stream);

#ifdef __cplusplus
}
#endif
