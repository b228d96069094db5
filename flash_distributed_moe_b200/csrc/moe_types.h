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
  FDMOE_PACK_ROWS = 72,     // rows per PACK task (rows of one expert, sent by one rank)
};

// Task kinds held by the global work queue.
enum {
  FDMOE_TASK_NONE = 0,
  FDMOE_TASK_FFN1 = 1,     // (expert, m_tile, n_tile, rows): SwiGLU tile
  FDMOE_TASK_FFN2 = 2,     // (expert, m_tile, n_tile, rows): down-projection tile
  FDMOE_TASK_COMBINE = 3,  // (token group): ordered sum over the K slots
  FDMOE_TASK_GATED = 4,    // every rank has finished gating: row counts are final, start the dispatch
  FDMOE_TASK_TESTA = 5,    // task-system self test: x[i] *= 2 over a chunk, then push TESTB
  FDMOE_TASK_TESTB = 6,    // task-system self test: x[i] += 1 over a chunk
  FDMOE_TASK_EXIT = 7,
  FDMOE_TASK_GATE = 8,     // (token tile): gate GEMM, top-k, softmax, row reservation
  FDMOE_TASK_PACK = 9,     // (expert, first entry, count): copy this rank's rows for one expert to its owner
  FDMOE_TASK_GATEFIX = 10, // (token, token): exact fp32 gate of nearly tied tokens
};

// Status codes written by the kernel (first error wins).
enum {
  FDMOE_OK = 0,
  FDMOE_ERR_TIMEOUT_QUEUE = 1,   // a worker waited too long for its ticket
  FDMOE_ERR_TIMEOUT_RING = 2,    // CTA-internal task ring
  FDMOE_ERR_TIMEOUT_STAGE = 3,   // TMA/MMA shared-memory stage barrier
  FDMOE_ERR_TIMEOUT_TMEM = 4,    // accumulator hand-off barrier
  FDMOE_ERR_TIMEOUT_PEER = 5,    // a peer rank never signalled readiness
  FDMOE_ERR_QUEUE_OVERFLOW = 6,
  FDMOE_ERR_BAD_TASK = 7,
  FDMOE_ERR_ROW_OVERFLOW = 8,    // more rows for an expert than its buffer holds
};

// One slot of the ticket queue (16 bytes).  `seq` == ticket + 1 once the slot
// holds the task of that ticket.
typedef struct {
  uint32_t seq;
  uint32_t a;  // kind | expert << 8 | n_tile << 20
  uint32_t b;  // m_tile, or token group, or chunk index
  uint32_t c;  // valid rows in the tile
} FdmoeSlot;

// Sideband of one packed row (16 bytes): where its result goes.
typedef struct {
  int32_t token;      // index of the token on its home rank
  int32_t home_slot;  // home rank << 8 | slot k
  float weight;       // routing weight of (token, slot)
  int32_t pad;
} FdmoeRowMeta;

// Per-rank control block.  Lives in the rank's symmetric arena so that peers
// can reach it.  Fields on separate 128-byte lines are written by different
// agents.
typedef struct {
  // --- persistent queue state (never zeroed between launches)
  uint32_t q_head;
  uint32_t pad0[31];
  uint32_t q_tail;
  uint32_t pad1[31];
  uint32_t closed;  // 0 running, 1 finished, 2 aborted
  uint32_t status;  // first error code
  uint32_t status_info;
  uint32_t exit_cnt;
  uint32_t urgent;  // a task that goes before the queue: 0, or 0x80000000 | kind | b << 8 (cleared by whoever takes it)
  uint32_t pad2[27];
  uint32_t ready[32];  // ready[r] = launch epoch of peer r (written by peer r)
  // --- per-launch counters: [launch_begin, launch_end) is zeroed before each launch
  uint32_t launch_begin;
  uint32_t gated_tokens;     // tokens of this rank whose routing is decided
  uint32_t rows_arrived;     // weighted rows of this rank's tokens that have come back (T*K when complete)
  uint32_t ranks_gated;      // ranks whose gating is finished (incl. this one)
  uint32_t gated_done;        // the GATED task of this launch has run (tile total and pack list are set)
  uint32_t mtiles_total;     // m-tiles of this rank's experts this launch
  uint32_t mtiles_done;      // m-tiles whose FFN2 is complete
  uint32_t tokens_combined;
  uint32_t tokens_launch;    // tokens of this rank this launch (written at kernel start)
  uint32_t executed;         // tasks finished (used only with expected_static)
  uint32_t pack_total;       // PACK tasks of this rank this launch (entries of its pack list)
  uint32_t pack_cursor;      // next entry of the pack list to publish
  uint32_t gate_tiles_done;  // GATE tiles of this rank that have finished
  uint32_t round2_rdv;       // 2 when both this rank's first round is laid out and every rank has gated
  uint32_t pad3[18];
} FdmoeCtl;

// What one rank can reach of a peer (or of itself): all device pointers valid
// in this process.
typedef struct {
  FdmoeCtl* ctl;
  FdmoeSlot* slots;
  uint32_t* expert_cnt;    // [El]       rows allocated per local expert
  uint32_t* landed;        // [El]       rows landed per local expert
  uint32_t* published;     // [El]       1 once the expert's FFN1 tiles have been published
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
  int32_t queue_mask;   // capacity - 1 (capacity is a power of two)
  int32_t combine_group;  // most tokens per COMBINE task
  int32_t gate_rows;    // tokens per GATE task: 32, 64 or 128 (rows of the 128-row MMA tile that are used)
  int32_t mode;         // 0 full layer; 2 static tasks only (no gate)
  int32_t debug_flags;  // timing experiments only (results become invalid): 1 skip FFN stores,
                        // 2 skip completion fences, 4 skip proxy fences, 8 skip the operand loads of FFN tiles
  uint32_t expected_static;  // mode 2: tasks pre-filled by the host
  uint32_t epoch;       // launch counter (identical on all ranks)
  uint64_t timeout_ns;  // budget of every device-side wait

  const void* x;        // bf16 [T, H]
  void* out;            // bf16 [T, H] (may alias x)
  const void* gate_w;   // bf16 [E, H]
  void* act;            // bf16 [El * cap_rows, I]
  int32_t* topk_idx;    // [max_tokens, K]
  float* topk_w;        // [max_tokens, K]
  // this rank's send lists, one per (global) expert: entry i of expert e is at [e * send_stride + i]
  uint32_t* send_cnt;   // [E] entries per expert (zeroed per launch)
  int32_t* send_src;    // token << 4 | slot
  int32_t* send_dst;    // row in the owner's expert buffers
  int32_t send_stride;  // = max tokens of this rank (an expert gets at most one row per token)
  // this rank's PACK tasks of the launch in sending order, {a, b, c, 0} each; `pack_window` of them
  // are outstanding at a time (every finished PACK task publishes the next entry)
  uint32_t* pack_list;
  int32_t pack_window;
  int32_t pack_early;   // 1: packing starts when this rank's GATE tiles are done; 0: when every rank has gated
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
