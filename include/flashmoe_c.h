/* Flat C ABI of libflashMoe.so: the same operations as iMoeKernelLauncher.h for
 * callers that cannot bind a C++ vtable (ctypes, cgo, JNI, ...).  Plain
 * pointers and sizes only.  Every function returns a cudaError_t value as int
 * (0 == success) unless stated otherwise.
 *
 * Each entry names the reference interface it stands for (paths relative to the
 * reference project).
 */
#ifndef FLASHMOE_C_H_
#define FLASHMOE_C_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct FlashMoeHandle_t* FlashMoeHandle;

typedef struct {
  int32_t hiddenSize;
  int32_t expertIntermediateSize;
  int32_t expertsNum;
  int32_t topk;
  int32_t dtype; /* 0 bf16, 1 fp32 I/O */
  int32_t reserved[3];
} FlashMoeConfig;

/* GetDistributedUniqueId (include/iMoeKernelLauncher.h:26): fills 128 bytes. */
int FlashMoeGetUniqueId(int empty, uint8_t out[128]);

/* CreateLauncher / CreateLauncherEx (include/iMoeKernelLauncher.h:29-35,
 * python/pyMoeLauncherTorch.cpp:71-107).  config == NULL selects the
 * Qwen3-30B-A3B shape in bf16.  `stream` is a cudaStream_t. */
int FlashMoeCreate(FlashMoeHandle* out, const void* gateWeights, const void* ffn1ExpertWeights,
                   const void* ffn2ExpertWeights, int maxTokens, void* stream,
                   const uint8_t uid[128], int rank, int worldSize, const FlashMoeConfig* config);

/* IMoeKernelLauncher::Launch (include/iMoeKernelLauncher.h:12-13,
 * python/pyMoeLauncherTorch.cpp:44-61): device pointers, asynchronous. */
int FlashMoeLaunch(FlashMoeHandle h, const void* tokens, void* output, int tokensNum, void* stream);

/* Launch with HOST buffers: copies `tokens` to the device, runs the layer and
 * copies the result back.  The input must be complete in host memory when the
 * call is made; the result is complete once `stream` has reached this point.
 * Returns after enqueueing (pinned host memory).  The three steps run on
 * internal streams with two sets of staging buffers, so back-to-back calls
 * overlap the copies of one call with the kernel of the other.  The reference's
 * tests do the same three steps by hand (test/singleGPU/cpp/moe/moeTest.cpp:38-56). */
int FlashMoeLaunchHost(FlashMoeHandle h, const void* hostTokens, void* hostOutput, int tokensNum,
                       void* stream);

/* DestroyLauncher (include/iMoeKernelLauncher.h:38-39). */
int FlashMoeDestroy(FlashMoeHandle h, void* stream);

/* First device-side error of the launcher since creation (0 == none) and its
 * detail word; does not synchronise.  The reference has no counterpart: its
 * device waits are unbounded (src/hip/taskSystem/taskManager.h:208-215). */
int FlashMoeGetLastStatus(FlashMoeHandle h, uint32_t* code, uint32_t* info);

/* Stage buffers of the last launch, for parity tests (the reference checks the
 * same stages with purpose-built kernels, test/singleGPU/cpp/moe/internal/).
 * `which`: 0 top-k indices int32 [T,K]; 1 routing weights fp32 [T,K];
 * 2 rows per local expert uint32 [E_local]; 3 packed rows bf16 [E_local*cap,H];
 * 4 row sideband 16 B [E_local*cap]; 5 activations bf16 [E_local*cap,I];
 * 6 weighted expert outputs bf16 [maxTokens,K,H]; 7 {cap_rows, E_local, grid, smem} int32[4];
 * 8 event trace of the last launch (only with FLASHMOE_PROFILE=1 at create): per CTA 512 records of
 * {kind, t0, t1, t2} uint32 ns, record 0 = {count,...}.
 * Copies min(bytes, size) bytes starting at `offset` to host memory `dst`
 * after synchronising the device. */
int FlashMoeDebugRead(FlashMoeHandle h, int which, void* dst, size_t offset, size_t bytes);

/* Task-system self test (reference: test/singleGPU/cpp/taskSystem/
 * saxpyCoherenceTest.hip:43-143): every element of `data` (device, int32,
 * n a multiple of 256) goes through two dependent tasks, x*2 then +1, the
 * second pushed by the first through the global queue. */
int FlashMoeTestTaskSystem(FlashMoeHandle h, int32_t* data, int n, void* stream);

/* Runs pre-built FFN2-style tile tasks through the queue as a plain grouped
 * GEMM: out[r, :] = A[r, :] * W2[expert]^T for rows written into the expert
 * buffers by the caller (reference: test/singleGPU/cpp/taskSystem/gemmTest/
 * gemmTest.cpp:69-73).  `rowsPerExpert[E_local]`, `A` bf16 [sum rows, I] host
 * order by expert, `out` bf16 [sum rows, H]; device pointers. */
int FlashMoeTestQueueGemm(FlashMoeHandle h, const uint32_t* rowsPerExpertHost, const void* A,
                          void* out, void* stream);

/* Test hook for the device-side time-outs (the reference has no counterpart: its device waits are
 * unbounded, src/hip/taskSystem/taskManager.h:208-215): a launch that expects one task nobody ever
 * publishes.  Every worker's wait for work runs out after FLASHMOE_TIMEOUT_MS, the kernel records
 * status 1 (a worker found no work for too long) and returns; the context stays usable, the launcher
 * refuses further launches until it is destroyed and created again.  Nothing faults or hangs. */
int FlashMoeTestStall(FlashMoeHandle h, void* stream);

/* The whole layer in one call that allocates nothing (no counterpart in the reference, whose
 * launcher always allocates its scratch in Init, src/hip/launcher/moeKernelLauncher.hip:139-165).
 * For callers that may not touch the device allocator: an engine that has frozen its memory pool,
 * a callback that must not call allocating runtime functions, a process whose memory belongs to
 * another allocator.  All scratch comes from a fixed 32 MiB array inside the library image (held
 * on every GPU that loads the library); a call whose scratch does not fit is rejected with
 * cudaErrorInvalidValue.  Single rank, bf16, device pointers.  config == NULL means the
 * Qwen3-30B-A3B shape, whose 128 expert buffers alone exceed the array, so that call is always
 * rejected: pass the (smaller) layer you run.  The first call on a device does one-time set-up (it
 * may be the moment the 32 MiB become resident there): make it before any stream capture and before
 * the host freezes its memory budget.  Calls share the array: do not let two of them overlap on a
 * GPU.  Every call synchronises `stream` and returns after the layer has finished; a device-side
 * error is reported as cudaErrorUnknown. */
int FlashMoeLaunchNoAlloc(const void* gateWeights, const void* ffn1ExpertWeights,
                          const void* ffn2ExpertWeights, const void* tokens, void* output, int tokensNum,
                          const FlashMoeConfig* config, void* stream);

const char* FlashMoeErrorString(int code);

#ifdef __cplusplus
}
#endif
#endif /* FLASHMOE_C_H_ */
