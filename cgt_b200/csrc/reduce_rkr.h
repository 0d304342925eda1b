// Sum / Max of an array viewed as [R0, K, R1] over R0 and R1 (bias gradients Sum{0,2,3} of NCHW, row sums,
// full sums): the kernels and the work split shared by cgtb_reduce and cgtb_reduce_rkr_f32_static, so that
// both produce the same bits.
//
// Block (k, split) folds rows [a0, a1) of R0 and columns [b0, b1) of R1 of output k; its 256 threads
// form (rows x columns) with the columns along R1. When R1 and the chunk are multiples of 4 and the input is 16-byte aligned the row is read as
// float4 with four independent accumulators per thread (four loads' worth of bytes in flight per
// instruction, no add-latency chain); the partial is ((a0 + a1) + (a2 + a3)), then a shuffle tree, one
// value per warp, and a tree over the warps. A second kernel folds the per-split partials in split order.
#pragma once
#include <cfloat>
#include <limits>
#include <type_traits>

#include "runtime.h"

namespace cgtb {
namespace rkr {

template <typename T>
__device__ __forceinline__ T init(int kind) {
  return kind == CGTB_R_SUM ? T(0) : -std::numeric_limits<T>::max();
}
template <> __device__ __forceinline__ float init<float>(int kind) { return kind == CGTB_R_SUM ? 0.f : -FLT_MAX; }
template <> __device__ __forceinline__ double init<double>(int kind) { return kind == CGTB_R_SUM ? 0.0 : -DBL_MAX; }

template <typename T>
__device__ __forceinline__ T op(int kind, T a, T b) {
  if (kind == CGTB_R_SUM) return a + b;
  return (T)fmax((double)a, (double)b);
}
template <> __device__ __forceinline__ float op<float>(int kind, float a, float b) { return kind == CGTB_R_SUM ? a + b : fmaxf(a, b); }

template <typename T>
__device__ __forceinline__ T shfl_down(T v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }
template <> __device__ __forceinline__ int8_t shfl_down<int8_t>(int8_t v, int d) { return (int8_t)__shfl_down_sync(0xffffffffu, (int)v, d); }

template <typename T>
__device__ __forceinline__ T block_fold(int kind, T acc) {
  __shared__ T warp_part[32];
  for (int d = 16; d > 0; d >>= 1) acc = op<T>(kind, acc, shfl_down<T>(acc, d));
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) warp_part[wid] = acc;
  __syncthreads();
  if (wid == 0) {
    const int nw = blockDim.x >> 5;
    acc = lane < nw ? warp_part[lane] : init<T>(kind);
    for (int d = 16; d > 0; d >>= 1) acc = op<T>(kind, acc, shfl_down<T>(acc, d));
  }
  return acc;  // valid in thread 0
}

template <typename T>
__global__ void partial_kernel(int kind, int R0, int K, int R1, int r0chunk, int r1chunk, int n1, int vec, int cols,
                               const T* __restrict__ in, T* __restrict__ out, int nsplit) {
  const int k = blockIdx.x, split = blockIdx.y;
  const int s0 = split / n1, s1 = split - s0 * n1;  // the split index covers (R0 chunk, R1 chunk)
  const int a0 = s0 * r0chunk, a1 = min(a0 + r0chunk, R0);
  const int b0 = s1 * r1chunk, b1 = min(b0 + r1chunk, R1);
  T acc = init<T>(kind);
  if (std::is_same<T, float>::value && vec) {
    T p0 = init<T>(kind), p1 = p0, p2 = p0, p3 = p0;
    const int q0 = b0 >> 2, q1 = b1 >> 2;
    const int tx4 = threadIdx.x % cols, ty4 = threadIdx.x / cols, rows4 = blockDim.x / cols;
    for (int r0 = a0 + ty4; r0 < a1; r0 += rows4) {
      const float4* row = reinterpret_cast<const float4*>(in + ((size_t)r0 * K + k) * R1);
      for (int q = q0 + tx4; q < q1; q += cols) {
        const float4 v = __ldg(row + q);
        p0 = op<T>(kind, p0, (T)v.x);
        p1 = op<T>(kind, p1, (T)v.y);
        p2 = op<T>(kind, p2, (T)v.z);
        p3 = op<T>(kind, p3, (T)v.w);
      }
    }
    acc = op<T>(kind, op<T>(kind, p0, p1), op<T>(kind, p2, p3));
  } else {
    // short rows: the block's threads form (rows x columns) so that several rows are read at once
    const int tx = threadIdx.x % cols, ty = threadIdx.x / cols, rows = blockDim.x / cols;
    for (int r0 = a0 + ty; r0 < a1; r0 += rows) {
      const T* row = in + ((size_t)r0 * K + k) * R1;
      for (int r1 = b0 + tx; r1 < b1; r1 += cols) acc = op<T>(kind, acc, row[r1]);
    }
  }
  acc = block_fold<T>(kind, acc);
  if (threadIdx.x == 0) out[(size_t)k * nsplit + split] = acc;
}

template <typename T>
__global__ void finish_kernel(int kind, long osize, int nsplit, const T* __restrict__ part, T* __restrict__ out) {
  for (long o = (long)blockIdx.x * blockDim.x + threadIdx.x; o < osize; o += (long)gridDim.x * blockDim.x) {
    T acc = init<T>(kind);
    for (int s = 0; s < nsplit; ++s) acc = op<T>(kind, acc, part[o * nsplit + s]);
    out[o] = acc;
  }
}

struct Plan {
  int threads, cols, r0chunk, r1chunk, n0, n1, nsplit, vec;
};

// spread the work of one output over several blocks so that the grid fills the machine: first along R0,
// then along R1 (in chunks that keep float4 alignment)
template <typename T>
inline Plan plan(long R0, long K, long R1, int sm_count, const void* in) {
  Plan p;
  p.vec = (std::is_same<T, float>::value && (R1 & 3) == 0 && ((uintptr_t)in & 15) == 0 && R1 >= 4) ? 1 : 0;
  const long per_thread = p.vec ? 4 : 1;
  // threads along a row: a power of two covering the row's units (float4 or element), at most 256;
  // the other threads of the 256-thread block take further rows of the R0 chunk
  const long units = cgtb_ceil_div(R1, per_thread);
  p.cols = 1;
  while (p.cols < 256 && p.cols < units) p.cols *= 2;
  p.threads = 256;
  const long want = (long)sm_count * 4;
  const long per_k = cgtb_ceil_div(want, K);
  int n0 = (K < want && R0 > 1) ? (int)std::min<long>(per_k, R0) : 1;
  p.r0chunk = R0 ? (int)cgtb_ceil_div(R0, n0) : 1;
  n0 = R0 ? (int)cgtb_ceil_div(R0, p.r0chunk) : 1;
  int n1 = 1;
  if ((long)K * n0 < want && R1 > 8192) n1 = (int)std::min<long>(cgtb_ceil_div(want, (long)K * n0), cgtb_ceil_div(R1, 4096));
  long r1chunk = R1 ? cgtb_ceil_div(R1, n1) : 1;
  r1chunk = cgtb_ceil_div(r1chunk, 4) * 4;
  n1 = R1 ? (int)cgtb_ceil_div(R1, r1chunk) : 1;
  if ((long)n0 * n1 > 65535) {
    n1 = std::max(1, 65535 / n0);
    r1chunk = cgtb_ceil_div(cgtb_ceil_div(R1, n1), 4) * 4;
    n1 = (int)cgtb_ceil_div(R1, r1chunk);
  }
  p.r1chunk = (int)r1chunk;
  p.n0 = n0;
  p.n1 = n1;
  p.nsplit = n0 * n1;
  return p;
}

}  // namespace rkr
}  // namespace cgtb
