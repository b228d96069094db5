// Public C++ interface of libflashMoe.so (B200 build).
//
// Same names, arity, argument meaning and error convention as the reference
// project's include/iMoeKernelLauncher.h:9-39, with cudaError_t / cudaStream_t
// in place of hipError_t / hipStream_t (an int-sized enum and an opaque pointer
// in both runtimes, so the calling shape is unchanged).
//
// Contract (reference include/iMoeKernelLauncher.h, src/moeKernelLauncher.cpp:15-55,
// src/hip/launcher/moeKernelLauncher.hip:96-212):
//   * weights, tokens and output are borrowed device pointers, never copied or freed;
//   * gate weights [E,H], FFN1 weights [E/world, 2I, H] (rows 0..I-1 gate
//     projection, I..2I-1 up projection), FFN2 weights [E/world, H, I], tokens and
//     output [T,H], all contiguous; `output` may alias `tokens`;
//   * Launch is asynchronous on `stream`; one Launch in flight per launcher; with worldSize == 1 it
//     only enqueues work on `stream` and can be captured into a CUDA graph, with peers it cannot;
//   * with worldSize > 1, CreateLauncher, every Launch and DestroyLauncher are
//     collective over the ranks; tokensNum may differ per rank and may be 0;
//   * errors are return codes (cudaSuccess == 0); a configuration that does not
//     fit returns cudaErrorUnknown, as the reference does for its capacity check.
//
// The reference fixes shape and dtype at compile time (Qwen3-30B-A3B, fp32).
// This build takes them at run time through CreateLauncherEx; CreateLauncher
// keeps the reference's implicit layer exactly: hidden 2048, 128 experts, top-8,
// intermediate 768, and fp32 weights, tokens and output (converted to bf16 at the
// boundary), so a caller written against the reference header gets what it
// expects.  bf16 tensors, the native path, go through CreateLauncherEx.
#pragma once

#include <cuda_runtime_api.h>
#include <stdint.h>

namespace moe {

// Main interface of the MoE kernel launcher
// (reference: include/iMoeKernelLauncher.h:9-17; vtable order Launch, dtor).
class IMoeKernelLauncher {
 public:
  // Runs the MoE layer on `tokensNum` tokens.
  virtual cudaError_t Launch(const void* tokens, void* output, int tokensNum,
                             cudaStream_t stream) = 0;

  virtual ~IMoeKernelLauncher();
};

// 128 opaque bytes that identify one multi-rank job
// (reference: include/iMoeKernelLauncher.h:19-21).
struct DistributedUniqueId {
  uint8_t data[128];
};

// Element type of tokens, output and weights.
enum MoeDType : int32_t {
  MOE_DTYPE_BF16 = 0,  // native path
  MOE_DTYPE_FP32 = 1,  // reference-compatible I/O: weights are converted to bf16 once at
                       // create, tokens/output are cast on the way in and out
};

// Run-time layer description for CreateLauncherEx.
struct MoeConfig {
  int32_t hiddenSize;              // H, multiple of 256
  int32_t expertIntermediateSize;  // I, multiple of 128
  int32_t expertsNum;              // E, <= 128, divisible by worldSize
  int32_t topk;                    // K, <= 8
  int32_t dtype;                   // MoeDType
  int32_t reserved[3];             // must be zero
};

}  // namespace moe

// Returns the id a multi-rank job is created with; empty=true gives all zeros
// (single rank).  Creates no CUDA context and no threads, so it may be called
// in a parent process that forks the ranks afterwards
// (reference: include/iMoeKernelLauncher.h:26, src/moeKernelLauncher.cpp:15-30).
extern "C" moe::DistributedUniqueId GetDistributedUniqueId(bool empty);

// Creates a launcher for the reference's layer: Qwen3-30B-A3B shape, fp32 tensors
// (reference: include/iMoeKernelLauncher.h:29-35, src/moeKernelLauncher.cpp:33-46).
// *launcher is written only on success.
extern "C" cudaError_t CreateLauncher(moe::IMoeKernelLauncher** launcher,
                                      const void* gateWeights,
                                      const void* ffn1ExpertWeights,
                                      const void* ffn2ExpertWeights,
                                      int maxTokens, cudaStream_t stream,
                                      const moe::DistributedUniqueId& uid,
                                      int rank, int worldSize);

// Same, with the layer shape and dtype given at run time (config == NULL: the
// Qwen3-30B-A3B shape with bf16 tensors).  The reference has no such call: its
// shape is the compile-time struct src/hip/common/metadata.h:7-13.
extern "C" cudaError_t CreateLauncherEx(moe::IMoeKernelLauncher** launcher,
                                        const void* gateWeights,
                                        const void* ffn1ExpertWeights,
                                        const void* ffn2ExpertWeights,
                                        int maxTokens, cudaStream_t stream,
                                        const moe::DistributedUniqueId& uid,
                                        int rank, int worldSize,
                                        const moe::MoeConfig* config);

// Destroys a launcher; synchronises `stream`
// (reference: include/iMoeKernelLauncher.h:38-39, src/moeKernelLauncher.cpp:49-55).
extern "C" cudaError_t DestroyLauncher(moe::IMoeKernelLauncher* launcher,
                                       cudaStream_t stream);
