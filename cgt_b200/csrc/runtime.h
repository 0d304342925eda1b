// Internal header of libcgt_b200.so: process-wide runtime state, error helpers, launch accounting.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdint>
#include <string>
#include "../../include/cgt_common.h"
#include "../../include/cgt_b200.h"

#define CGTB_API extern "C" __attribute__((visibility("default")))

namespace cgtb {

struct Runtime {
  int device = -1;
  cudaStream_t stream = nullptr;
  int sm_count = 148;
  bool ready = false;
};
Runtime& rt();

// Fails loudly (status + message) when cgtb_init was never called or no GPU is present.
bool require_runtime(const char* who);

extern std::atomic<long> g_kernel_launches;

// Scratch memory for kernels that need global memory beyond their inputs and outputs. Inside an
// interpreter the block belongs to the running instruction and keeps its address across runs (so a
// captured CUDA graph stays valid); outside it comes from one process-wide block on the runtime stream.
void* scratch(size_t nbytes);
// a second, independent block of the same owner, for a caller that itself invokes code using scratch()
void* scratch_outer(size_t nbytes);

struct ScratchOwner {  // one per interpreter instruction
  void* ptr = nullptr;
  size_t cap = 0;
  void* outer_ptr = nullptr;
  size_t outer_cap = 0;
};
void set_scratch_owner(ScratchOwner* o);  // nullptr -> process-wide block
void free_scratch_owner(ScratchOwner* o);

// set while a stream capture is in progress: pool misses then fail instead of calling cudaMalloc
void set_capturing(bool on);
bool capturing();
long device_malloc_count();

int fail(const char* fmt, ...);  // records the message, returns 1

// non-zero (with a recorded message) when the tensor-core GEMM raised its time-out flag; call on an idle stream
int sgemm_tc_check();

}  // namespace cgtb

#define CGTB_CUDA_TRY(expr)                                                                      \
  do {                                                                                           \
    cudaError_t e_ = (expr);                                                                     \
    if (e_ != cudaSuccess) return cgtb::fail("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
  } while (0)

// every kernel launch of the library goes through this, so launches can be counted
#define CGTB_LAUNCH(kernel, grid, block, smem, ...)                                  \
  do {                                                                               \
    kernel<<<(grid), (block), (smem), cgtb::rt().stream>>>(__VA_ARGS__);             \
    cgtb::g_kernel_launches.fetch_add(1, std::memory_order_relaxed);                 \
  } while (0)

#define CGTB_CHECK_LAUNCH(name)                                                                  \
  do {                                                                                           \
    cudaError_t e_ = cudaGetLastError(); /* reads AND clears: a refused launch must not poison later calls */ \
    if (e_ != cudaSuccess) return cgtb::fail("%s launch failed: %s", name, cudaGetErrorString(e_)); \
  } while (0)

static inline long cgtb_ceil_div(long a, long b) { return (a + b - 1) / b; }
