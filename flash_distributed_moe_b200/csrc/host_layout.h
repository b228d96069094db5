// Host-side helpers shared by the launcher and the allocation-free entry point:
// the layout of a rank's scratch arena and the construction of TMA descriptors.
// Pure host arithmetic plus one driver entry point lookup; no allocation.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>

#include <algorithm>

#include "moe_types.h"

#ifndef MOE_ERROR_LOG
#define MOE_ERROR_LOG(...)                                      \
  do {                                                          \
    fprintf(stderr, "[MOE ERROR: %s:%d] ", __FILE__, __LINE__); \
    fprintf(stderr, __VA_ARGS__);                               \
    fprintf(stderr, "\n");                                      \
  } while (0)
#endif

namespace fdmoe {

inline size_t AlignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline uint32_t NextPow2(uint64_t v) {
  uint32_t p = 1;
  while (p < v) p <<= 1;
  return p;
}

// Offsets of every region inside a rank's symmetric arena.  Identical on all
// ranks, so a peer's regions are found from its base pointer alone.
struct ArenaLayout {
  size_t ctl = 0;
  size_t expert_cnt = 0, landed = 0, grp_cnt = 0, ffn1_done = 0, ffn2_done = 0;
  size_t zero_begin = 0, zero_end = 0;  // per-launch reset range
  size_t slots[3] = {0, 0, 0};
  size_t meta = 0, ystage = 0, packed = 0;
  size_t total = 0;
};

struct Geometry {
  int H = 0, I = 0, E = 0, K = 0, El = 0, world = 1;
  int max_tokens_local = 0;  // this rank
  int max_tokens_max = 0;    // largest over ranks (sizes token-indexed regions)
  int64_t max_tokens_sum = 0;  // all ranks (sizes expert buffers)
  int cap_rows = 0, MT = 0, combine_group = 8;  // combine_group: tokens per COMBINE task
  uint32_t queue_cap = 0;
};

// Slots of any task queue of a rank: at least every task one launch can publish there, so
// that a slot is never reused within a launch.  Tile tasks of the rank's experts (FFN1 in one
// queue, FFN2 in the other), COMBINE tasks (one per group of combine_group tokens), GATEFIX
// tasks (two tokens each, every token in the worst case, rounded up per GATE tile), the GATED round,
// and DISPATCH tasks (one per GATE tile of at least 32 tokens).
inline uint64_t WorstCaseQueueTasks(const Geometry& g) {
  const uint64_t rows_max = std::min<uint64_t>((uint64_t)g.max_tokens_sum * g.K, (uint64_t)g.El * g.cap_rows);
  const uint64_t mtiles = rows_max / FDMOE_TILE_M + g.El;
  const uint64_t tiles = mtiles * (uint64_t)std::max(g.I / FDMOE_TILE_N1, g.H / FDMOE_TILE_N2);
  const uint64_t gate_tiles = (uint64_t)g.max_tokens_max / 32 + 1;
  return tiles + (uint64_t)g.max_tokens_max / std::max(1, g.combine_group) + 1 +
         (uint64_t)g.max_tokens_max / 2 + gate_tiles + 1;
}

inline uint32_t QueueCapacity(const Geometry& g, int grid) {
  return NextPow2(WorstCaseQueueTasks(g) + (uint64_t)grid + 2048);
}

// Derived sizes once the token bounds, the shape and combine_group are known: rows of a local expert's
// buffer (an expert receives at most one row per token of any rank), m-tiles per expert, queue
// capacity.  Returns false when the expert buffers would hold more rows than a dispatch word can
// address (28 bits).
inline bool FinishGeometry(Geometry& g, int grid) {
  const uint64_t cap = AlignUp((size_t)std::max<int64_t>(g.max_tokens_sum, 1), FDMOE_TILE_M);
  if ((uint64_t)g.El * cap >= (1ull << 28)) return false;
  g.cap_rows = (int)cap;
  g.MT = g.cap_rows / FDMOE_TILE_M;
  g.queue_cap = QueueCapacity(g, grid);
  return true;
}

inline size_t CombineGroups(const Geometry& g) {
  return (size_t)g.max_tokens_max / std::max(1, g.combine_group) + 2;
}

inline ArenaLayout MakeLayout(const Geometry& g) {
  ArenaLayout L;
  size_t off = 0;
  L.ctl = off;
  off += AlignUp(sizeof(FdmoeCtl), 128);
  L.zero_begin = L.ctl + offsetof(FdmoeCtl, launch_begin);
  L.expert_cnt = off;
  off += AlignUp((size_t)g.El * 4, 128);
  L.landed = off;
  off += AlignUp((size_t)g.El * g.MT * 4, 128);
  L.grp_cnt = off;
  off += AlignUp(CombineGroups(g) * 4, 128);
  L.ffn1_done = off;
  off += AlignUp((size_t)g.El * g.MT * 4, 128);
  L.ffn2_done = off;
  off += AlignUp((size_t)g.El * g.MT * 4, 128);
  L.zero_end = off;
  off = AlignUp(off, 1024);  // the regions from here on start on 1024-byte boundaries
  for (int q = 0; q < 3; ++q) {
    L.slots[q] = off;
    off += AlignUp((size_t)g.queue_cap * sizeof(FdmoeSlot), 1024);
  }
  L.meta = off;
  off += AlignUp((size_t)g.El * g.cap_rows * sizeof(FdmoeRowMeta), 1024);
  L.ystage = off;
  off += AlignUp((size_t)g.max_tokens_max * g.K * g.H * 2, 1024);
  L.packed = off;
  off += AlignUp((size_t)g.El * g.cap_rows * g.H * 2, 1024);
  L.total = off;
  return L;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn GetEncodeTiled() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<EncodeTiledFn>(fn);
}

// Row-major bf16 matrix [rows, cols]; one TMA box is 64 columns (128 bytes, the
// swizzle span) by box_rows rows.
inline cudaError_t MakeTensorMap(EncodeTiledFn enc, FdmoeTensorMap* out, const void* base, uint64_t rows,
                          uint64_t cols, uint32_t box_rows) {
  static_assert(sizeof(CUtensorMap) == sizeof(FdmoeTensorMap), "tensor map size");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {FDMOE_TILE_K, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    MOE_ERROR_LOG("cuTensorMapEncodeTiled failed with %d (rows %llu cols %llu)", (int)r,
                  (unsigned long long)rows, (unsigned long long)cols);
    return cudaErrorInvalidValue;
  }
  return cudaSuccess;
}

}  // namespace fdmoe
