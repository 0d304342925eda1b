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
#include "reduce_rkr.h"

using namespace cgtb;

namespace {

// capacity of the shared array in floats: 32768 floats = 128 KiB
constexpr long kStaticPartials = 32768;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_reduce_static_partials[kStaticPartials];

float* g_partials_addr[kMaxDevices];  // per device, looked up once

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
  if (R1 == 1 && R0 > 1)
    return fail("cgtb_reduce_rkr_f32_static: R1 == 1 (a column reduction [R0, K]) is not split and needs no scratch; use cgtb_reduce");
  const int dev = rt().device;
  if (dev < 0 || dev >= kMaxDevices) return fail("cgtb_reduce_rkr_f32_static: device index %d not supported", dev);
  if (!g_partials_addr[dev]) {
    // the symbol resolves for the calling thread's CURRENT device: it must be the one the runtime is bound to
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != dev) {
      cudaError_t es = cudaSetDevice(dev);
      if (es != cudaSuccess) return fail("cgtb_reduce_rkr_f32_static: cudaSetDevice(%d) failed: %s", dev, cudaGetErrorString(es));
    }
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_reduce_static_partials);
    if (e != cudaSuccess || !p)
      return fail("cgtb_reduce_rkr_f32_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_partials_addr[dev] = p;
  }
  float* part = g_partials_addr[dev];
  if (R0 == 0 || R1 == 0) R0 = R1 = 0;  // empty reduction: every output is the identity
  // the work split and the kernels of cgtb_reduce for this layout (reduce_rkr.h): same bits
  const rkr::Plan pl = rkr::plan<float>(R0, K, R1, rt().sm_count, in);
  if ((long)K * pl.nsplit > kStaticPartials)
    return fail("cgtb_reduce_rkr_f32_static: %ld partial results exceed the fixed scratch array of %ld floats; use cgtb_reduce",
                (long)K * pl.nsplit, kStaticPartials);
  dim3 grid((unsigned)K, (unsigned)pl.nsplit);
  if (pl.nsplit == 1) {
    CGTB_LAUNCH(rkr::partial_kernel<float>, grid, pl.threads, 0, kind, (int)R0, (int)K, (int)R1, pl.r0chunk, pl.r1chunk, pl.n1, pl.vec, pl.cols, in, out, 1);
  } else {
    CGTB_LAUNCH(rkr::partial_kernel<float>, grid, pl.threads, 0, kind, (int)R0, (int)K, (int)R1, pl.r0chunk, pl.r1chunk, pl.n1, pl.vec, pl.cols, in, part, pl.nsplit);
    CGTB_LAUNCH(rkr::finish_kernel<float>, (unsigned)cgtb_ceil_div(K, 128), 128, 0, kind, (long)K, pl.nsplit, part, out);
  }
  CGTB_CHECK_LAUNCH("reduce_rkr_f32_static");
  return 0;
}
