// Sum / Max over the outer and inner axes of a float32 array viewed as [R0, K, R1], for callers that
// must not allocate: the partial results of the split reduction live in one fixed array in device
// memory that is part of the loaded module, not in memory obtained at call time.
//
// Who needs this: code that runs where an allocation is forbidden or can fail late, e.g. a callback
// on a latency-critical path, a process whose device memory is handed out completely to another
// allocator, or a caller that must keep the address space of the device unchanged between calls.
// cgtb_reduce() takes its partials from the runtime's scratch pool, which may call cudaMalloc the
// first time a size is seen; this entry point never does.
//
// Properties a caller has to know:
//  * The first call on a device looks the array's address up (cudaGetSymbolAddress), which makes the
//    CUDA runtime load the module. That is set-up work: make one call before any stream capture or
//    any region in which the CUDA runtime must stay quiet.
//  * Every call in the process shares the one array. Nothing in it has to start at zero: each call
//    writes every partial it later reads, so no clearing is needed and no state survives a call.
//  * Because the array is shared, two calls that overlap in time (from two threads, or if the
//    runtime stream were ever replaced by several streams) race on it. Calls issued one after the
//    other on the runtime stream are ordered by the stream and are safe.
//  * Limits: K <= CGTB_REDUCE_STATIC_MAX_K kept elements, R0 and R1 below 2^30, float32 only. Larger
//    requests are refused with an error; nothing is launched for them.
#include <cfloat>

#include "cgt_b200.h"
#include "runtime.h"

using namespace cgtb;

namespace {

// capacity of the shared array in floats: 32768 floats = 128 KiB
constexpr long kStaticPartials = 32768;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_reduce_static_partials[kStaticPartials];

float* g_partials_addr[kMaxDevices];  // per device, looked up once

__device__ __forceinline__ float rs_init(int kind) { return kind == CGTB_R_SUM ? 0.f : -FLT_MAX; }
__device__ __forceinline__ float rs_op(int kind, float a, float b) { return kind == CGTB_R_SUM ? a + b : fmaxf(a, b); }

// Block (k, split) folds its share of rows R0 and columns R1 of output k; threads run along R1.
// The order of the additions (strided per-thread sums, shuffle tree, one partial per warp, tree over
// the warps) is the one cgtb_reduce uses for this layout, so both give the same bits.
__global__ void reduce_static_partial_kernel(int kind, int R0, int K, int R1, int r0chunk, int r1chunk, int n1,
                                             const float* __restrict__ in, float* __restrict__ out, int nsplit) {
  const int k = blockIdx.x, split = blockIdx.y;
  const int s0 = split / n1, s1 = split - s0 * n1;
  const int a0 = s0 * r0chunk, a1 = min(a0 + r0chunk, R0);
  const int b0 = s1 * r1chunk, b1 = min(b0 + r1chunk, R1);
  float acc = rs_init(kind);
  for (int r0 = a0; r0 < a1; ++r0) {
    const float* row = in + ((size_t)r0 * K + k) * R1;
    for (int r1 = b0 + threadIdx.x; r1 < b1; r1 += blockDim.x) acc = rs_op(kind, acc, row[r1]);
  }
  __shared__ float warp_part[32];
  for (int d = 16; d > 0; d >>= 1) acc = rs_op(kind, acc, __shfl_down_sync(0xffffffffu, acc, d));
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) warp_part[wid] = acc;
  __syncthreads();
  if (wid == 0) {
    const int nw = blockDim.x >> 5;
    acc = lane < nw ? warp_part[lane] : rs_init(kind);
    for (int d = 16; d > 0; d >>= 1) acc = rs_op(kind, acc, __shfl_down_sync(0xffffffffu, acc, d));
    if (lane == 0) out[(size_t)k * nsplit + split] = acc;
  }
}

__global__ void reduce_static_finish_kernel(int kind, int K, int nsplit, const float* __restrict__ part,
                                            float* __restrict__ out) {
  for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < K; k += gridDim.x * blockDim.x) {
    float acc = rs_init(kind);
    for (int s = 0; s < nsplit; ++s) acc = rs_op(kind, acc, part[(size_t)k * nsplit + s]);
    out[k] = acc;
  }
}

}  // namespace

CGTB_API long cgtb_reduce_static_max_k(void) { return CGTB_REDUCE_STATIC_MAX_K; }

CGTB_API int cgtb_reduce_rkr_f32_static(int kind, long R0, long K, long R1, const float* in, float* out) {
  if (!require_runtime("cgtb_reduce_rkr_f32_static")) return 1;
  if (kind != CGTB_R_SUM && kind != CGTB_R_MAX) return fail("cgtb_reduce_rkr_f32_static: unknown kind %d", kind);
  if (R0 < 0 || K < 0 || R1 < 0) return fail("cgtb_reduce_rkr_f32_static: negative extent");
  if (K > CGTB_REDUCE_STATIC_MAX_K)
    return fail("cgtb_reduce_rkr_f32_static: K=%ld is beyond the maximum of %d kept elements of the fixed scratch array; "
                "use cgtb_reduce", K, (int)CGTB_REDUCE_STATIC_MAX_K);
  if (R0 >= (1L << 30) || R1 >= (1L << 30))
    return fail("cgtb_reduce_rkr_f32_static: R0=%ld / R1=%ld beyond the maximum of 2^30-1; use cgtb_reduce", R0, R1);
  if (K == 0) return 0;
  const int dev = rt().device;
  if (dev < 0 || dev >= kMaxDevices) return fail("cgtb_reduce_rkr_f32_static: device index %d not supported", dev);
  if (!g_partials_addr[dev]) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_reduce_static_partials);
    if (e != cudaSuccess || !p)
      return fail("cgtb_reduce_rkr_f32_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_partials_addr[dev] = p;
  }
  float* part = g_partials_addr[dev];
  if (R0 == 0 || R1 == 0) R0 = R1 = 0;  // empty reduction: every output is the identity
  // the split of cgtb_reduce for this layout: fill the machine, first along R0, then along R1
  const int threads = R1 >= 256 ? 256 : (R1 >= 64 ? 64 : 32);
  const long want = (long)rt().sm_count * 4;
  const long per_k = cgtb_ceil_div(want, K);
  int n0 = (K < want && R0 > 1) ? (int)std::min<long>(per_k, R0) : 1;
  const int r0chunk = R0 ? (int)cgtb_ceil_div(R0, n0) : 1;
  n0 = R0 ? (int)cgtb_ceil_div(R0, r0chunk) : 1;
  int n1 = 1;
  if ((long)K * n0 < want && R1 > 8192) n1 = (int)std::min<long>(cgtb_ceil_div(want, (long)K * n0), cgtb_ceil_div(R1, 4096));
  const int r1chunk = R1 ? (int)cgtb_ceil_div(R1, n1) : 1;
  n1 = R1 ? (int)cgtb_ceil_div(R1, r1chunk) : 1;
  const int nsplit = n0 * n1;
  if (nsplit > 65535 || (long)K * nsplit > kStaticPartials)
    return fail("cgtb_reduce_rkr_f32_static: %ld partial results exceed the fixed scratch array of %ld floats; use cgtb_reduce",
                (long)K * nsplit, kStaticPartials);
  dim3 grid((unsigned)K, (unsigned)nsplit);
  if (nsplit == 1) {
    CGTB_LAUNCH(reduce_static_partial_kernel, grid, threads, 0, kind, (int)R0, (int)K, (int)R1, r0chunk, r1chunk, n1, in, out, 1);
  } else {
    CGTB_LAUNCH(reduce_static_partial_kernel, grid, threads, 0, kind, (int)R0, (int)K, (int)R1, r0chunk, r1chunk, n1, in, part, nsplit);
    CGTB_LAUNCH(reduce_static_finish_kernel, (unsigned)cgtb_ceil_div(K, 128), 128, 0, kind, (int)K, nsplit, part, out);
  }
  CGTB_CHECK_LAUNCH("reduce_rkr_f32_static");
  return 0;
}
