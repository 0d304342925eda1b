// fp32 / fp64 FMA GEMM for Mul22 and BatchedMul22 (cgt/core.py:2195-2206, 2272-2286).
//
// This is the general-shape path: any M, N, K, any leading dimensions, all four transpose
// combinations, fp64 as well. The tensor-core path (gemm_tcgen05.cu) takes the fp32 shapes it
// supports; cgtb_sgemm chooses between the two.
//
// 64x64 output tile per CTA, K step 16, 256 threads with a 4x4 register tile each. Skinny products
// with a long K (weight gradients: M x N of a few thousand elements, K up to 131072) are split along
// K across CTAs; partial tiles go to scratch memory and are folded in split order by a second kernel,
// so the result does not depend on scheduling.
#include "runtime.h"

using namespace cgtb;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// element (m,k) of op(A) is A[m*sam + k*sak]; element (k,n) of op(B) is B[k*sbk + n*sbn]
template <typename T, bool A_KFAST, bool B_NFAST>
__global__ void __launch_bounds__(256) gemm_simt_kernel(long M, long N, long K, const T* __restrict__ A, long sam, long sak,
                                                        long strideA, const T* __restrict__ B, long sbk, long sbn,
                                                        long strideB, T* __restrict__ C, long ldc, long strideC, int nsplit,
                                                        long kchunk) {
  __shared__ T As[BK][BM + 4];
  __shared__ T Bs[BK][BN + 4];
  const int batch = blockIdx.z / nsplit, split = blockIdx.z % nsplit;
  A += batch * strideA;
  B += batch * strideB;
  // with split-K the output is the scratch slab [batch][split][M][N] (ldc == N there)
  C += (nsplit > 1) ? ((long)batch * nsplit + split) * M * N : batch * strideC;
  const long m0 = (long)blockIdx.y * BM, n0 = (long)blockIdx.x * BN;
  const long k_begin = split * kchunk, k_end = min(K, k_begin + kchunk);
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, each 4 x 4 outputs
  T acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = T(0);

  for (long k0 = k_begin; k0 < k_end; k0 += BK) {
    // A tile: BM x BK = 1024 elements, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int idx = tid + e * 256;
      int mm, kk;
      if (A_KFAST) { kk = idx % BK; mm = idx / BK; } else { mm = idx % BM; kk = idx / BM; }
      long m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < M && k < k_end) ? A[m * sam + k * sak] : T(0);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int idx = tid + e * 256;
      int nn, kk;
      if (B_NFAST) { nn = idx % BN; kk = idx / BN; } else { kk = idx % BK; nn = idx / BK; }
      long n = n0 + nn, k = k0 + kk;
      Bs[kk][nn] = (n < N && k < k_end) ? B[k * sbk + n * sbn] : T(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      T a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  const long ld = (nsplit > 1) ? N : ldc;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    long m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      long n = n0 + tx * TN + j;
      if (n < N) C[m * ld + n] = acc[i][j];
    }
  }
}

template <typename T>
__global__ void splitk_fold_kernel(long P, long M, long N, int nsplit, const T* __restrict__ part, T* __restrict__ C,
                                   long ldc, long strideC) {
  long total = P * M * N;
  for (long f = (long)blockIdx.x * blockDim.x + threadIdx.x; f < total; f += (long)gridDim.x * blockDim.x) {
    long n = f % N, t = f / N;
    long m = t % M, p = t / M;
    const T* src = part + (p * nsplit) * M * N + m * N + n;
    T acc = src[0];
    for (int s = 1; s < nsplit; ++s) acc += src[(long)s * M * N];
    C[p * strideC + m * ldc + n] = acc;
  }
}

template <typename T>
int gemm_simt(int tA, int tB, long P, long M, long N, long K, const T* A, long lda, long strideA, const T* B, long ldb,
              long strideB, T* C, long ldc, long strideC) {
  if (P <= 0 || M <= 0 || N <= 0) return 0;
  long sam = tA ? 1 : lda, sak = tA ? lda : 1;
  long sbk = tB ? 1 : ldb, sbn = tB ? ldb : 1;
  long tiles = cgtb_ceil_div(M, BM) * cgtb_ceil_div(N, BN) * P;
  int nsplit = 1;
  long want = (long)rt().sm_count * 2;
  if (tiles < want && K >= 1024) {
    nsplit = (int)std::min<long>(cgtb_ceil_div(want, tiles), K / 256);
    if (nsplit < 1) nsplit = 1;
    if (nsplit > 512) nsplit = 512;
  }
  long kchunk = cgtb_ceil_div(cgtb_ceil_div(K, nsplit), BK) * BK;
  nsplit = (int)cgtb_ceil_div(K > 0 ? K : 1, kchunk > 0 ? kchunk : 1);
  if (K == 0) { nsplit = 1; kchunk = BK; }
  if (P * nsplit > 65535) return fail("gemm: batch x split-K = %ld exceeds the grid limit", P * nsplit);
  T* part = nullptr;
  if (nsplit > 1) {
    part = (T*)scratch((size_t)P * nsplit * M * N * sizeof(T));
    if (!part) return 1;
  }
  dim3 grid((unsigned)cgtb_ceil_div(N, BN), (unsigned)cgtb_ceil_div(M, BM), (unsigned)(P * nsplit));
  T* dst = nsplit > 1 ? part : C;
#define GEMM_GO(AK, BNF)                                                                                              \
  CGTB_LAUNCH((gemm_simt_kernel<T, AK, BNF>), grid, 256, 0, M, N, K, A, sam, sak, strideA, B, sbk, sbn, strideB, dst, ldc, \
              strideC, nsplit, kchunk)
  if (!tA && !tB) GEMM_GO(true, true);
  else if (!tA && tB) GEMM_GO(true, false);
  else if (tA && !tB) GEMM_GO(false, true);
  else GEMM_GO(false, false);
#undef GEMM_GO
  if (nsplit > 1) {
    long total = P * M * N;
    long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 8);
    CGTB_LAUNCH(splitk_fold_kernel<T>, (unsigned)blocks, 256, 0, P, M, N, nsplit, part, C, ldc, strideC);
  }
  CGTB_CHECK_LAUNCH("gemm_simt");
  return 0;
}

}  // namespace

namespace {
// Products with few outputs and a short K (the classifier layer: 128 x 10 x 256 and its gradients):
// LANES consecutive threads share one output element, lane l taking k = l, l + LANES, ...; eight
// products' operands are loaded before the first multiply-add so that a thread has sixteen loads in
// flight (the kernel is bound by memory latency, not by bytes or flops). The lanes' sums are combined
// by a shuffle tree: a fixed order, so results are reproducible. A tiled kernel spends its time on
// pipeline fill and barriers for these shapes.
template <int LANES>
__global__ void sgemm_small_kernel(int tA, int tB, long M, long N, long K, const float* __restrict__ A, long lda, long strideA,
                                   const float* __restrict__ B, long ldb, long strideB, float* __restrict__ C, long ldc,
                                   long strideC) {
  const long p = blockIdx.y;
  const long gthread = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long e = gthread / LANES;
  const int l = (int)(gthread % LANES);
  const bool live = e < M * N;
  const long ee = live ? e : 0;
  const long m = ee / N, n = ee - m * N;
  const float* a = A + p * strideA + (tA ? m : m * lda);
  const float* b = B + p * strideB + (tB ? n * ldb : n);
  const long sa = tA ? lda : 1, sb = tB ? 1 : ldb;
  float acc = 0.f;
  for (long k0 = l; k0 < K; k0 += 8L * LANES) {
    float av[8], bv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const long k = k0 + (long)u * LANES;
      const bool ok = live && k < K;
      av[u] = ok ? __ldg(a + k * sa) : 0.f;
      bv[u] = ok ? __ldg(b + k * sb) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) acc = fmaf(av[u], bv[u], acc);
  }
#pragma unroll
  for (int d = LANES / 2; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (live && l == 0) C[p * strideC + m * ldc + n] = acc;
}
// The same product when both operands run along K in memory (C = A . B^T, row-major A [M, K] and B [N, K]) and M, N are
// multiples of four: a warp owns a 4 x 4 block of outputs, so a row of A or B that it reads (one coalesced 128-byte
// load per 32 values of k) feeds four outputs instead of one: an eighth of the L2 traffic of one warp per output
// (64 x 128 x 512, the LSTM's hidden-state gradient: 33 MB of loads become 4 MB). Every output is still accumulated
// by lane l over k = l, l + 32, ... in ascending order and the lanes are folded by the same shuffle tree: the bits of
// sgemm_small_kernel<32>.
__global__ void __launch_bounds__(256) sgemm_small_nt4_kernel(long M, long N, long K, const float* __restrict__ A, long lda, long strideA,
                                                             const float* __restrict__ B, long ldb, long strideB, float* __restrict__ C,
                                                             long ldc, long strideC) {
  const long p = blockIdx.y;
  const long w = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int l = threadIdx.x & 31;
  const long nb = N / 4;
  if (w >= (M / 4) * nb) return;
  const long m0 = 4 * (w / nb), n0 = 4 * (w % nb);
  const float* a = A + p * strideA + m0 * lda;
  const float* b = B + p * strideB + n0 * ldb;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  constexpr int U = 8;   // 64 loads per lane in flight: the kernel is bound by the latency of its load rounds
  for (long k0 = l; k0 < K; k0 += 32 * U) {
    float av[U][4], bv[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long k = k0 + 32 * u;
      const bool ok = k < K;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[u][i] = ok ? __ldg(a + i * lda + k) : 0.f;
        bv[u][i] = ok ? __ldg(b + i * ldb + k) : 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[u][i], bv[u][j], acc[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) acc[i][j] += __shfl_xor_sync(0xffffffffu, acc[i][j], d);
    }
  if (l < 4) {   // lane i stores row i of the block
    float* c = C + p * strideC + (m0 + l) * ldc + n0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (l == i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) c[j] = acc[i][j];
      }
  }
}
}  // namespace

// Products too large for one warp per output and too small to repay the tensor-core kernel's fixed cost (tensor-map
// fetch, tensor-memory allocation, a multi-stage ring that such a product never fills: 10-25 us for the 64 x 512 x 128
// products of the unrolled LSTM): plain FMA tiles. A block owns a 16 x 16 tile of C; its KS groups of 256 threads
// walk interleaved 16-wide slices of K, each thread one output, operands staged through shared memory with loads
// that are contiguous for either storage order, the next slice's words already in flight while the current one is
// used; the groups' partial sums are added in group order. One fixed order of operations: reproducible.
namespace {
// Output stage: C = (addend + addend_bias) + (A.B + bias) with row vectors bias, addend_bias [N] and a matrix addend
// [M, N]; every pointer may be null. Plain float32 additions in exactly this association: the sum of two affine
// pre-activations (x.W + b) + (h.U + c) as the separate kernels form it.
struct TileEpilogue {
  const float* bias;
  const float* addend;
  long ldd;
  const float* addend_bias;
};
template <int KS>
__global__ void __launch_bounds__(256 * KS) sgemm_tile16_kernel(int tA, int tB, long M, long N, long K, const float* __restrict__ A, long lda,
                                                               long strideA, const float* __restrict__ B, long ldb, long strideB,
                                                               float* __restrict__ C, long ldc, long strideC, const TileEpilogue ep) {
  __shared__ float As[KS][16][17];  // [m][k]
  __shared__ float Bs[KS][16][17];  // [k][n]
  const int tx = threadIdx.x & 15, ty = (threadIdx.x >> 4) & 15, kz = threadIdx.x >> 8;
  const long m0 = (long)blockIdx.y * 16, n0 = (long)blockIdx.x * 16;
  A += (long)blockIdx.z * strideA;
  B += (long)blockIdx.z * strideB;
  C += (long)blockIdx.z * strideC;
  const long niter = (K + 16L * KS - 1) / (16L * KS);
  auto load_a = [&](long k0) -> float {
    if (!tA) { const long m = m0 + ty, k = k0 + tx; return (m < M && k < K) ? A[m * lda + k] : 0.f; }
    const long m = m0 + tx, k = k0 + ty;
    return (m < M && k < K) ? A[k * lda + m] : 0.f;
  };
  auto load_b = [&](long k0) -> float {
    if (!tB) { const long k = k0 + ty, n = n0 + tx; return (k < K && n < N) ? B[k * ldb + n] : 0.f; }
    const long n = n0 + ty, k = k0 + tx;
    return (k < K && n < N) ? B[n * ldb + k] : 0.f;
  };
  float acc = 0.f;
  float a = load_a((long)kz * 16), b = load_b((long)kz * 16);
  for (long it = 0; it < niter; ++it) {
    if (!tA) As[kz][ty][tx] = a; else As[kz][tx][ty] = a;
    if (!tB) Bs[kz][ty][tx] = b; else Bs[kz][tx][ty] = b;
    __syncthreads();
    if (it + 1 < niter) {
      const long k0 = ((it + 1) * KS + kz) * 16;
      a = load_a(k0);
      b = load_b(k0);
    }
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) acc = fmaf(As[kz][ty][kk], Bs[kz][kk][tx], acc);
    __syncthreads();
  }
  if (KS > 1) {
    As[kz][ty][tx] = acc;
    __syncthreads();
    if (kz == 0) {
#pragma unroll
      for (int z = 1; z < KS; ++z) acc += As[z][ty][tx];
    }
  }
  if (kz == 0 && m0 + ty < M && n0 + tx < N) {
    const long m = m0 + ty, n = n0 + tx;
    if (ep.bias) acc = __fadd_rn(acc, ep.bias[n]);
    if (ep.addend) {
      float t = ep.addend[m * ep.ldd + n];
      if (ep.addend_bias) t = __fadd_rn(t, ep.addend_bias[n]);
      acc = __fadd_rn(t, acc);
    }
    C[m * ldc + n] = acc;
  }
}
}  // namespace

namespace cgtb {
// returns 0 done, -1 not eligible
static int sgemm_tile16_ep(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B, long ldb,
                           long strideB, float* C, long ldc, long strideC, const TileEpilogue& ep) {
  if (P <= 0 || M <= 0 || N <= 0) return 0;
  if (K <= 0 || M * N * K > (1L << 25) || P > 65535 || cgtb_ceil_div(M, 16) > 65535) return -1;
  dim3 grid((unsigned)cgtb_ceil_div(N, 16), (unsigned)cgtb_ceil_div(M, 16), (unsigned)P);
  const long blocks = (long)grid.x * grid.y * grid.z;
  if (blocks < 4L * rt().sm_count && K >= 64)
    CGTB_LAUNCH(sgemm_tile16_kernel<4>, grid, 1024, 0, tA, tB, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC, ep);
  else
    CGTB_LAUNCH(sgemm_tile16_kernel<1>, grid, 256, 0, tA, tB, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC, ep);
  CGTB_CHECK_LAUNCH("sgemm_tile16");
  return 0;
}
int sgemm_tile16(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B, long ldb,
                 long strideB, float* C, long ldc, long strideC) {
  return sgemm_tile16_ep(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC, TileEpilogue{nullptr, nullptr, 0, nullptr});
}
// the FMA-tile product with its output stage; -1 when the product is not one the dispatcher gives to that kernel
int sgemm_tile16_bias_add(int tA, int tB, long M, long N, long K, const float* A, long lda, const float* B, long ldb, const float* bias,
                          const float* addend, long ldd, const float* addend_bias, float* C, long ldc) {
  if (M * N <= 2048 || (!tA && tB)) return -1;   // the dispatcher sends these to the warp-per-output kernel
  return sgemm_tile16_ep(tA, tB, 1, M, N, K, A, lda, 0, B, ldb, 0, C, ldc, 0, TileEpilogue{bias, addend, ldd, addend_bias});
}

// returns 0 done, -1 not a small product
int sgemm_small(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B, long ldb,
                long strideB, float* C, long ldc, long strideC) {
  if (P <= 0 || M <= 0 || N <= 0) return 0;
  if (M * N > 65536 || K > 2048 || M * N * K > (1L << 24) || P > 65535) return -1;
  const int lanes = K >= 128 ? 32 : (K >= 32 ? 8 : 1);
  if (lanes == 32 && !tA && tB && M % 4 == 0 && N % 4 == 0 && M * N >= 1024) {
    dim3 grid4((unsigned)cgtb_ceil_div((M / 4) * (N / 4) * 32, 256), (unsigned)P);
    CGTB_LAUNCH(sgemm_small_nt4_kernel, grid4, 256, 0, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
    CGTB_CHECK_LAUNCH("sgemm_small");
    return 0;
  }
  dim3 grid((unsigned)cgtb_ceil_div(M * N * lanes, 256), (unsigned)P);
  if (lanes == 32) CGTB_LAUNCH(sgemm_small_kernel<32>, grid, 256, 0, tA, tB, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
  else if (lanes == 8) CGTB_LAUNCH(sgemm_small_kernel<8>, grid, 256, 0, tA, tB, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
  else CGTB_LAUNCH(sgemm_small_kernel<1>, grid, 256, 0, tA, tB, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
  CGTB_CHECK_LAUNCH("sgemm_small");
  return 0;
}

int sgemm_simt(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
               long ldb, long strideB, float* C, long ldc, long strideC) {
  return gemm_simt<float>(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
}
}  // namespace cgtb

CGTB_API int cgtb_dgemm(int tA, int tB, long M, long N, long K, const double* A, long lda, const double* B, long ldb,
                        double* C, long ldc) {
  if (!require_runtime("cgtb_dgemm")) return 1;
  return gemm_simt<double>(tA, tB, 1, M, N, K, A, lda, 0, B, ldb, 0, C, ldc, 0);
}
