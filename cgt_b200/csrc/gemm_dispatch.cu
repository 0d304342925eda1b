// Mul22 / BatchedMul22 entry points: choose between the tcgen05 tensor-core kernels (3xTF32 split
// precision; TMA-fed for 16-byte-aligned operands, gemm_tma.cu, register-fed otherwise,
// gemm_tcgen05.cu) and the fp32 FMA kernel (gemm_simt.cu).
// Products with few outputs and a short K go to a one-thread-per-output kernel (gemm_simt.cu).
// impl: 0 automatic, 1 FMA (tiled), 2 tensor cores (either feed), 3 register-fed only, 4 TMA-fed only,
// 5 the small-product kernel only.
#include "runtime.h"
#include "tc_util.h"

namespace cgtb {
int sgemm_simt(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
               long ldb, long strideB, float* C, long ldc, long strideC);
// returns 0 done, 1 error, -1 shape not supported by the tensor-core kernel
int sgemm_tc(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
             long ldb, long strideB, float* C, long ldc, long strideC, const ConvEpilogue* ep = nullptr);

int sgemm_tma(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
              long ldb, long strideB, float* C, long ldc, long strideC, const ConvEpilogue* ep = nullptr);

int sgemm_small(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
                long ldb, long strideB, float* C, long ldc, long strideC);
int sgemm_tile16(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
                 long ldb, long strideB, float* C, long ldc, long strideC);

int sgemm_dispatch(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
                   long ldb, long strideB, float* C, long ldc, long strideC, int impl) {
  if (!require_runtime("sgemm")) return 1;
  // one warp per output suits few outputs, or operands that both run along K in memory (its lanes read along K);
  // the FMA tiles take the other products below the size at which the tensor-core kernels' fixed cost is repaid
  const bool warp_per_output = impl == 5 || (impl == 0 && (M * N <= 2048 || (!tA && tB)));
  if (warp_per_output) {
    int rc = sgemm_small(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
    if (rc >= 0) return rc;
    if (impl == 5) return fail("sgemm: M=%ld N=%ld K=%ld is not a small product", M, N, K);
  }
  if (impl == 0 || impl == 6) {
    int rc = sgemm_tile16(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
    if (rc >= 0) return rc;
    if (impl == 6) return fail("sgemm: M=%ld N=%ld K=%ld is too large for the FMA-tile kernel", M, N, K);
  }
  if (impl != 1) {
    int rc = -1;
    if (impl != 3) rc = sgemm_tma(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
    if (rc >= 0) return rc;
    if (impl == 4) return fail("sgemm: M=%ld N=%ld K=%ld with these strides is not eligible for the TMA-fed kernel", M, N, K);
    rc = sgemm_tc(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
    if (rc >= 0) return rc;
    if (impl >= 2) return fail("sgemm: shape M=%ld N=%ld K=%ld is not supported by the tensor-core kernel", M, N, K);
  }
  return sgemm_simt(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
}
}  // namespace cgtb

CGTB_API int cgtb_sgemm(int tA, int tB, long M, long N, long K, const float* A, long lda, const float* B, long ldb, float* C,
                        long ldc, int impl) {
  return cgtb::sgemm_dispatch(tA, tB, 1, M, N, K, A, lda, 0, B, ldb, 0, C, ldc, 0, impl);
}
namespace cgtb {
int sgemm_tile16_bias_add(int tA, int tB, long M, long N, long K, const float* A, long lda, const float* B, long ldb, const float* bias,
                          const float* addend, long ldd, const float* addend_bias, float* C, long ldc);
}
CGTB_API int cgtb_sgemm_bias_add(int tA, int tB, long M, long N, long K, const float* A, long lda, const float* B, long ldb,
                                 const float* bias, const float* addend, long ldd, const float* addend_bias, float* C, long ldc) {
  if (!cgtb::require_runtime("cgtb_sgemm_bias_add")) return 1;
  if (addend_bias && !addend) return cgtb::fail("cgtb_sgemm_bias_add: addend_bias without addend");
  const int rc = cgtb::sgemm_tile16_bias_add(tA, tB, M, N, K, A, lda, B, ldb, bias, addend, ldd, addend_bias, C, ldc);
  if (rc < 0)
    return cgtb::fail("cgtb_sgemm_bias_add: M=%ld N=%ld K=%ld (tA=%d tB=%d) is not a product of the FMA-tile kernel (M*N > 2048, M*N*K <= 2^25, "
                      "not A.B^T); use cgtb_sgemm and add afterwards", M, N, K, tA, tB);
  return rc;
}
CGTB_API int cgtb_sgemm_batched(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA,
                                const float* B, long ldb, long strideB, float* C, long ldc, long strideC, int impl) {
  return cgtb::sgemm_dispatch(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC, impl);
}

// ------------------------------------------------------------------------------------------------
// Output stage of a convolution layer as the reference's graph spells it (cgt/nn.py:87-100, 44-45,
// 228-233): Mul22(col, W^T) gives [B*H*W, C] (channels last); Transpose{0,3,1,2} makes it NCHW; the
// bias [1,C,1,1] is Repeat-ed and added; relu is t * (t >= 0) with an int8 mask that the backward
// pass re-uses. Here the GEMM result is turned into both outputs in one pass: t = g + bias[c],
// mask = (t >= 0), y = t * mask, written as NCHW planes. The arithmetic is the separate kernels'
// (float add, compare with 0.f, float multiply), so the values are bit-identical to the Op-by-Op graph.
// A block stages 128 pixels x C channels through shared memory: coalesced reads along channels,
// coalesced writes along pixels.
// ------------------------------------------------------------------------------------------------
namespace {
constexpr int kTilePix = 128;
__global__ void __launch_bounds__(256) bias_relu_nchw_kernel(const float* __restrict__ g, const float* __restrict__ bias, long M, int C,
                                                           long HW, float* __restrict__ y, int8_t* __restrict__ mask, int tilepix) {
  extern __shared__ float tile[];  // [tilepix][C + 1], tilepix = 32 or 128
  const int stride = C + 1;
  const long m0 = (long)blockIdx.x * tilepix;
  const int npix = (int)((M - m0) < tilepix ? (M - m0) : tilepix);
  const int n = npix * C;
  const float* src = g + m0 * C;
  // rows of C contiguous floats: consecutive threads read consecutive addresses; four loads in flight
  if ((int)blockDim.x % C == 0) {
    // a thread keeps its channel and walks down the rows: no index division per element
    const int c = threadIdx.x % C, r0 = threadIdx.x / C, dr = blockDim.x / C;
    for (int r = r0; r < npix; r += 16 * dr) {  // sixteen loads in flight: one round trip for a 128 x 32 tile
      float v[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) v[k] = (r + k * dr < npix) ? src[(r + k * dr) * C + c] : 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k)
        if (r + k * dr < npix) tile[(r + k * dr) * stride + c] = v[k];
    }
  } else {
    for (int e0 = threadIdx.x; e0 < n; e0 += 4 * blockDim.x) {
      float v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int e = e0 + k * blockDim.x;
        v[k] = e < n ? src[e] : 0.f;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int e = e0 + k * blockDim.x;
        if (e < n) {
          const int r = e / C, c = e - r * C;
          tile[r * stride + c] = v[k];
        }
      }
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  size_t obase[kTilePix / 32];
  bool ok[kTilePix / 32];
#pragma unroll
  for (int q = 0; q < kTilePix / 32; ++q) {
    const int r = lane + 32 * q;
    ok[q] = r < npix;  // false for every q beyond a 32-pixel tile
    const long m = m0 + (ok[q] ? r : 0);
    const long b = m / HW, pix = m - b * HW;
    obase[q] = (size_t)b * C * HW + pix;
  }
  for (int c = warp; c < C; c += nwarps) {
    const float bc = bias[c];
    const size_t coff = (size_t)c * HW;
    const float* trow = tile + lane * stride + c;
#pragma unroll
    for (int q = 0; q < kTilePix / 32; ++q) {
      if (ok[q]) {
        const float t = trow[32 * q * stride] + bc;
        const int8_t mk = (int8_t)(t >= 0.f);
        const size_t o = obase[q] + coff;
        mask[o] = mk;
        y[o] = t * (float)mk;
      }
    }
  }
}
}  // namespace

namespace {
// dst [R, ld] = src [R, K] with zeros in the columns beyond K
__global__ void pad_rows_kernel(const float* __restrict__ src, int R, int K, float* __restrict__ dst, int ld) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= R * ld) return;
  const int r = i / ld, k = i - r * ld;
  dst[i] = k < K ? src[(size_t)r * K + k] : 0.f;
}
}  // namespace

CGTB_API int cgtb_conv_bias_relu_ld(const float* col, long M, long K, long ldcol, const float* w, int C, const float* bias, long HW,
                                    float* y_nchw, int8_t* mask_nchw) {
  if (!cgtb::require_runtime("cgtb_conv_bias_relu")) return 1;
  if (M <= 0 || C <= 0) return 0;
  if (HW <= 0 || M % HW != 0) return cgtb::fail("cgtb_conv_bias_relu: %ld rows are not whole images of %ld pixels", M, HW);
  if (C > 384) return cgtb::fail("cgtb_conv_bias_relu: at most 384 channels");
  if (ldcol < K) return cgtb::fail("cgtb_conv_bias_relu: row pitch %ld below the row length %ld", ldcol, K);
  // Filter rows of K entries start on 16-byte boundaries only when K is a multiple of 4. When the column
  // matrix has such a pitch but K does not, the (small) filter matrix is copied to the same pitch so that
  // both operands qualify for the TMA-fed product; the product still runs over K entries.
  long ldw = K;
  size_t wpad_bytes = 0;
  if ((K & 3) != 0 && (ldcol & 3) == 0 && (long)C * ldcol < (1L << 24)) {
    ldw = ldcol;
    wpad_bytes = (((size_t)C * ldw * sizeof(float)) + 255) & ~(size_t)255;
  }
  auto padded_w = [&](float* dst) {
    CGTB_LAUNCH(pad_rows_kernel, (unsigned)cgtb_ceil_div((long)C * ldw, 256), 256, 0, w, C, (int)K, dst, (int)ldw);
  };
  const float* wuse = w;
  if (wpad_bytes) {
    float* wp = (float*)cgtb::scratch_outer(wpad_bytes);
    if (!wp) return 1;
    padded_w(wp);
    wuse = wp;
  }
  // products that the dispatcher gives to the FMA kernels (below the tensor-core kernels' break-even size) take the
  // staged path below: the same product kernel, hence the same bits, as Mul22 followed by the separate output stage
  if (M * (long)C * K > (1L << 25)) {
    // the tensor-core kernels apply the output stage to the accumulator tile when the product is not split
    // along K: no intermediate matrix at all
    cgtb::ConvEpilogue ep = {bias, y_nchw, mask_nchw, HW};
    int rc = cgtb::sgemm_tma(0, 1, 1, M, C, K, col, ldcol, 0, wuse, ldw, 0, nullptr, C, 0, &ep);
    if (rc < 0) rc = cgtb::sgemm_tc(0, 1, 1, M, C, K, col, ldcol, 0, wuse, ldw, 0, nullptr, C, 0, &ep);
    if (rc >= 0) return rc;
  }
  // the product may use scratch() for split-K; a larger request may move the outer block, so the padded
  // filters are written again at its start
  char* blk = (char*)cgtb::scratch_outer(wpad_bytes + (size_t)M * C * sizeof(float));
  if (!blk) return 1;
  if (wpad_bytes) {
    padded_w((float*)blk);
    wuse = (const float*)blk;
  }
  float* g = (float*)(blk + wpad_bytes);
  int rc = cgtb::sgemm_dispatch(0, 1, 1, M, C, K, col, ldcol, 0, wuse, ldw, 0, g, C, 0, 0);
  if (rc) return rc;
  // small products: 32-pixel tiles so that the grid still covers the machine
  const int tilepix = (M >= (long)kTilePix * 2 * cgtb::rt().sm_count) ? kTilePix : 32;
  const size_t smem = (size_t)tilepix * (C + 1) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(bias_relu_nchw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cgtb::fail("cgtb_conv_bias_relu: %s", cudaGetErrorString(e));
  }
  CGTB_LAUNCH(bias_relu_nchw_kernel, (unsigned)cgtb_ceil_div(M, tilepix), 256, smem, g, bias, M, C, HW, y_nchw, mask_nchw, tilepix);
  CGTB_CHECK_LAUNCH("conv_bias_relu");
  return 0;
}

CGTB_API int cgtb_conv_bias_relu(const float* col, long M, long K, const float* w, int C, const float* bias, long HW, float* y_nchw,
                                 int8_t* mask_nchw) {
  return cgtb_conv_bias_relu_ld(col, M, K, K, w, C, bias, HW, y_nchw, mask_nchw);
}

// ------------------------------------------------------------------------------------------------
// Input stage of a convolution layer's backward pass as the reference's graph spells it: the relu
// pullback g * mask (ElwiseBinary), its Transpose{0,2,3,1} to channels-last for the weight- and
// data-gradient products, and Sum{0,2,3} of the same tensor for the bias gradient (cgt/nn.py:44-45,
// 87-100, 228-233 differentiated). One pass: a block takes up to 128 pixels of one image for all
// channels, multiplies, writes the pixels as channels-last rows (one contiguous run) and leaves one
// partial channel sum per block; the partial sums are then added in block order by the column-sum
// kernel, so the bias gradient is reproducible (its summation order differs from Sum's).
// ------------------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(256) relu_grad_nhwc_kernel(const int8_t* __restrict__ mask, const float* __restrict__ g, int C,
                                                           long HW, float* __restrict__ gt, float* __restrict__ partial) {
  extern __shared__ float tile[];  // [128][C + 1]
  const int stride = C + 1;
  const long b = blockIdx.y;
  const long p0 = (long)blockIdx.x * 128;
  const int npix = (int)((HW - p0) < 128 ? (HW - p0) : 128);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const size_t plane0 = (size_t)b * C * HW + p0;
  // a warp takes four channels at a time and issues all their loads (16 mask bytes, 16 gradient words per
  // lane) before the first use: the pass is bound by latency, not by bytes
  for (int c0 = warp; c0 < C; c0 += 4 * nwarps) {
    float v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * nwarps;
      const size_t base = plane0 + (size_t)(c < C ? c : 0) * HW;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int px = lane + 32 * q;
        v[u][q] = (c < C && px < npix) ? (float)mask[base + px] * g[base + px] : 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * nwarps;
      if (c >= C) break;
      float sum = (v[u][0] + v[u][1]) + (v[u][2] + v[u][3]);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (lane + 32 * q < npix) tile[(lane + 32 * q) * stride + c] = v[u][q];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
      if (lane == 0) partial[((size_t)b * gridDim.x + blockIdx.x) * C + c] = sum;
    }
  }
  __syncthreads();
  float* dst = gt + ((size_t)b * HW + p0) * C;  // npix rows of C floats: one contiguous run
  const int n = npix * C;
  if ((int)blockDim.x % C == 0) {
    const int c = threadIdx.x % C, r0 = threadIdx.x / C, dr = blockDim.x / C;
    for (int r = r0; r < npix; r += dr) dst[r * C + c] = tile[r * stride + c];
  } else {
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      const int r = e / C, c = e - r * C;
      dst[e] = tile[r * stride + c];
    }
  }
}
}  // namespace

CGTB_API int cgtb_relu_grad_nhwc(const int8_t* mask_nchw, const float* g_nchw, long B, int C, long HW, float* gt_nhwc, float* bias_grad) {
  if (!cgtb::require_runtime("cgtb_relu_grad_nhwc")) return 1;
  if (B <= 0 || C <= 0 || HW <= 0) return 0;
  if (C > 384 || B > 65535) return cgtb::fail("cgtb_relu_grad_nhwc: at most 384 channels and 65535 images");
  const long ntiles = cgtb_ceil_div(HW, 128);
  float* partial = (float*)cgtb::scratch_outer((size_t)B * ntiles * C * sizeof(float));
  if (!partial) return 1;
  const size_t smem = (size_t)128 * (C + 1) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(relu_grad_nhwc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cgtb::fail("cgtb_relu_grad_nhwc: %s", cudaGetErrorString(e));
  }
  dim3 grid((unsigned)ntiles, (unsigned)B);
  CGTB_LAUNCH(relu_grad_nhwc_kernel, grid, 256, smem, mask_nchw, g_nchw, C, HW, gt_nhwc, partial);
  CGTB_CHECK_LAUNCH("relu_grad_nhwc");
  const long shape[2] = {B * ntiles, C};
  const int reduced[2] = {1, 0};
  return cgtb_reduce(CGTB_R_SUM, cgtb_f4, 2, shape, reduced, partial, bias_grad);
}
