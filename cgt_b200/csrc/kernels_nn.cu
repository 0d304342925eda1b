// im2col / col2im, max-pool forward / pullback, cross-channel LRN forward / backward for sm_100a.
//
// All of these are HBM-bound stencil or copy kernels: threads are laid out along the contiguous axis
// of the larger side of the transfer, shared memory stages the re-used input, and the arithmetic order
// follows the reference's CPU loops wherever the result depends on it (pool argmax tie-breaking,
// pool-pullback and col2im accumulation order), so integer outputs are bit-exact and float sums are
// added in the same sequence.
#include "runtime.h"
#include <cfloat>

using namespace cgtb;

// ================================================================================================
// im2col : col[b, h, w, c] = x[b, c_im, h*sh - ph + i, w*sw - pw + j],  c = (c_im*kh + i)*kw + j
// (include/im2col.h:6-28). One block per (b, h) output row: the C x kh x W input slab that row needs
// is staged in shared memory with out-of-image rows zero-filled, then written out as Wo*Z contiguous
// floats with consecutive threads on consecutive column channels.
// ================================================================================================
template <typename T>
__global__ void im2col_rows_kernel(const T* __restrict__ x, T* __restrict__ col, int C, int H, int W, int kh, int kw,
                                   int ph, int pw, int sh, int sw, int Ho, int Wo, int rows_per_block, long total_rows) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* slab = reinterpret_cast<T*>(smem_raw);             // [C][kh][W]
  const int Z = C * kh * kw;
  int* rowoff = reinterpret_cast<int*>(slab + (size_t)C * kh * W);  // [Z] : (c_im*kh + i)*W
  int* joff = rowoff + Z;                               // [Z] : j - pw

  for (int c = threadIdx.x; c < Z; c += blockDim.x) {
    int j = c % kw;
    int i = (c / kw) % kh;
    int c_im = c / (kw * kh);
    rowoff[c] = (c_im * kh + i) * W;
    joff[c] = j - pw;
  }
  for (int r = 0; r < rows_per_block; ++r) {
    long row = (long)blockIdx.x * rows_per_block + r;  // row = b*Ho + h
    if (row >= total_rows) break;
    long b = row / Ho;
    int h = (int)(row - b * Ho);
    const T* xb = x + b * (long)C * H * W;
    __syncthreads();
    const int slab_n = C * kh * W;
    for (int s = threadIdx.x; s < slab_n; s += blockDim.x) {
      int wq = s % W;
      int i = (s / W) % kh;
      int c_im = s / (W * kh);
      int hin = h * sh - ph + i;
      slab[s] = (hin >= 0 && hin < H) ? xb[((long)c_im * H + hin) * W + wq] : T(0);
    }
    __syncthreads();
    T* out = col + row * (long)Wo * Z;
    const int n_out = Wo * Z;
    // idx -> (w, c) without a division in the loop
    int w = threadIdx.x / Z;
    int c = threadIdx.x - w * Z;
    const int dw = blockDim.x / Z, dc = blockDim.x - dw * Z;
    for (int idx = threadIdx.x; idx < n_out; idx += blockDim.x) {
      int win = w * sw + joff[c];
      out[idx] = (win >= 0 && win < W) ? slab[rowoff[c] + win] : T(0);
      w += dw;
      c += dc;
      if (c >= Z) { c -= Z; w += 1; }
    }
  }
}

// fallback when the slab does not fit in shared memory: one thread per output element
template <typename T>
__global__ void im2col_direct_kernel(const T* __restrict__ x, T* __restrict__ col, long total, int C, int H, int W,
                                     int kh, int kw, int ph, int pw, int sh, int sw, int Ho, int Wo) {
  const int Z = C * kh * kw;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    int c = (int)(idx % Z);
    long row = idx / Z;
    int w = (int)(row % Wo);
    long t = row / Wo;
    int h = (int)(t % Ho);
    long b = t / Ho;
    int j = c % kw, i = (c / kw) % kh, c_im = c / (kw * kh);
    int hin = h * sh - ph + i, win = w * sw - pw + j;
    col[idx] = (hin >= 0 && hin < H && win >= 0 && win < W) ? x[((b * C + c_im) * H + hin) * W + win] : T(0);
  }
}

template <typename T>
static int im2col_launch(const T* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh, int sw, T* col) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  if (B <= 0 || Ho <= 0 || Wo <= 0) return 0;
  const int Z = C * kh * kw;
  size_t smem = (size_t)C * kh * W * sizeof(T) + 2 * (size_t)Z * sizeof(int);
  long total_rows = B * Ho;
  if (smem <= 200 * 1024) {
    if (smem > 48 * 1024)
      CGTB_CUDA_TRY(cudaFuncSetAttribute(im2col_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // several rows per block when a row is short, so each block moves at least ~16K elements
    int rpb = 1;
    while ((long)rpb * Wo * Z < 16384 && rpb < 8) rpb *= 2;
    long blocks = cgtb_ceil_div(total_rows, rpb);
    CGTB_LAUNCH(im2col_rows_kernel<T>, (unsigned)blocks, 256, smem, x, col, C, H, W, kh, kw, ph, pw, sh, sw, Ho, Wo, rpb,
                total_rows);
  } else {
    long total = total_rows * Wo * Z;
    long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 16);
    CGTB_LAUNCH(im2col_direct_kernel<T>, (unsigned)blocks, 256, 0, x, col, total, C, H, W, kh, kw, ph, pw, sh, sw, Ho, Wo);
  }
  CGTB_CHECK_LAUNCH("im2col");
  return 0;
}

CGTB_API int cgtb_im2col(int dtype, const void* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                         int sw, void* col) {
  if (!require_runtime("cgtb_im2col")) return 1;
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0) return fail("cgtb_im2col: kernel and stride must be positive");
  if (dtype == cgtb_f4) return im2col_launch<float>((const float*)x, B, C, H, W, kh, kw, ph, pw, sh, sw, (float*)col);
  if (dtype == cgtb_f8) return im2col_launch<double>((const double*)x, B, C, H, W, kh, kw, ph, pw, sh, sw, (double*)col);
  return fail("cgtb_im2col: unsupported dtype %d", dtype);
}

// ================================================================================================
// col2im (include/im2col.h:30-50) written as a gather: one thread per image pixel adds the column
// entries that map onto it in ascending column-channel order (i, then j), which is the order in
// which the reference's scatter loop reaches that pixel, so the float sum is bit-identical and no
// atomics are needed.
// ================================================================================================
template <typename T>
__global__ void col2im_gather_kernel(const T* __restrict__ col, T* __restrict__ im, long total, int C, int H, int W,
                                     int kh, int kw, int ph, int pw, int sh, int sw, int Ho, int Wo) {
  const int Z = C * kh * kw;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    int xw = (int)(idx % W);
    long t = idx / W;
    int y = (int)(t % H);
    t /= H;
    int c_im = (int)(t % C);
    long b = t / C;
    const T* colb = col + b * (long)Ho * Wo * Z;
    T acc = T(0);
    for (int i = 0; i < kh; ++i) {
      int hn = y + ph - i;
      if (hn < 0) break;
      int h = hn / sh;
      if (h * sh != hn || h >= Ho) continue;
      for (int j = 0; j < kw; ++j) {
        int wn = xw + pw - j;
        if (wn < 0) break;
        int w = wn / sw;
        if (w * sw != wn || w >= Wo) continue;
        acc += colb[((long)h * Wo + w) * Z + (c_im * kh + i) * kw + j];
      }
    }
    im[idx] = acc;
  }
}

template <typename T>
static int col2im_launch(const T* col, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh, int sw, T* im) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  long total = B * C * H * W;
  if (total <= 0) return 0;
  long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 32);
  CGTB_LAUNCH(col2im_gather_kernel<T>, (unsigned)blocks, 256, 0, col, im, total, C, H, W, kh, kw, ph, pw, sh, sw, Ho, Wo);
  CGTB_CHECK_LAUNCH("col2im");
  return 0;
}

CGTB_API int cgtb_col2im(int dtype, const void* col, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                         int sw, void* im) {
  if (!require_runtime("cgtb_col2im")) return 1;
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0) return fail("cgtb_col2im: kernel and stride must be positive");
  if (dtype == cgtb_f4) return col2im_launch<float>((const float*)col, B, C, H, W, kh, kw, ph, pw, sh, sw, (float*)im);
  if (dtype == cgtb_f8) return col2im_launch<double>((const double*)col, B, C, H, W, kh, kw, ph, pw, sh, sw, (double*)im);
  return fail("cgtb_col2im: unsupported dtype %d", dtype);
}

// ================================================================================================
// max pool forward (include/pooling.h:24-71). One thread per pooled element; the window is scanned
// h-major with a strict '>' from (-FLT_MAX, -1), so ties and NaNs resolve exactly as in the CPU loop.
// ================================================================================================
template <typename T>
__global__ void max_pool_kernel(const T* __restrict__ x, T* __restrict__ top, int32_t* __restrict__ mask, long total,
                                int H, int W, int kh, int kw, int ph, int pw, int sh, int sw, int PH, int PW) {
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    int px = (int)(idx % PW);
    long t = idx / PW;
    int py = (int)(t % PH);
    long plane = t / PH;
    const T* xp = x + plane * (long)H * W;
    int hstart = py * sh - ph, wstart = px * sw - pw;
    int hend = min(hstart + kh, H), wend = min(wstart + kw, W);
    hstart = max(hstart, 0);
    wstart = max(wstart, 0);
    T best = T(-FLT_MAX);
    int besti = -1;
    for (int h = hstart; h < hend; ++h)
      for (int w = wstart; w < wend; ++w) {
        T v = xp[h * W + w];
        if (v > best) { best = v; besti = h * W + w; }
      }
    top[idx] = best;
    mask[idx] = besti;
  }
}

// max pool pullback (include/pooling.h:73-104) as a gather: one thread per input pixel visits the
// pooled windows that can contain it in ascending (ph, pw) order and adds the gradients whose argmax
// is this pixel; the reference scatter reaches each pixel in the same order.
template <typename T>
__global__ void max_pool_pullback_kernel(const int32_t* __restrict__ mask, const T* __restrict__ gtop, T* __restrict__ gx,
                                         long total, int H, int W, int kh, int kw, int ph, int pw, int sh, int sw,
                                         int PH, int PW) {
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    int w = (int)(idx % W);
    long t = idx / W;
    int h = (int)(t % H);
    long plane = t / H;
    const int32_t* mp = mask + plane * (long)PH * PW;
    const T* gp = gtop + plane * (long)PH * PW;
    // windows with py*sh - ph <= h < py*sh - ph + kh
    int py0 = (h + ph - kh + 1 <= 0) ? 0 : (h + ph - kh + 1 + sh - 1) / sh;
    int py1 = min((h + ph) / sh, PH - 1);
    int px0 = (w + pw - kw + 1 <= 0) ? 0 : (w + pw - kw + 1 + sw - 1) / sw;
    int px1 = min((w + pw) / sw, PW - 1);
    const int me = h * W + w;
    T acc = T(0);
    for (int py = py0; py <= py1; ++py)
      for (int px = px0; px <= px1; ++px)
        if (mp[py * PW + px] == me) acc += gp[py * PW + px];
    gx[idx] = acc;
  }
}

CGTB_API int cgtb_max_pool(int dtype, const void* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                           int sw, int PH, int PW, void* top, int32_t* mask) {
  if (!require_runtime("cgtb_max_pool")) return 1;
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0) return fail("cgtb_max_pool: kernel and stride must be positive");
  long total = B * C * PH * PW;
  if (total <= 0) return 0;
  long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 32);
  if (dtype == cgtb_f4)
    CGTB_LAUNCH(max_pool_kernel<float>, (unsigned)blocks, 256, 0, (const float*)x, (float*)top, mask, total, H, W, kh, kw,
                ph, pw, sh, sw, PH, PW);
  else if (dtype == cgtb_f8)
    CGTB_LAUNCH(max_pool_kernel<double>, (unsigned)blocks, 256, 0, (const double*)x, (double*)top, mask, total, H, W, kh,
                kw, ph, pw, sh, sw, PH, PW);
  else
    return fail("cgtb_max_pool: unsupported dtype %d", dtype);
  CGTB_CHECK_LAUNCH("max_pool");
  return 0;
}

CGTB_API int cgtb_max_pool_pullback(int dtype, const int32_t* mask, const void* gtop, long B, int C, int PH, int PW,
                                    int H, int W, int kh, int kw, int ph, int pw, int sh, int sw, void* gx) {
  if (!require_runtime("cgtb_max_pool_pullback")) return 1;
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0) return fail("cgtb_max_pool_pullback: kernel and stride must be positive");
  long total = B * C * H * W;
  if (total <= 0) return 0;
  long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 32);
  if (dtype == cgtb_f4)
    CGTB_LAUNCH(max_pool_pullback_kernel<float>, (unsigned)blocks, 256, 0, mask, (const float*)gtop, (float*)gx, total, H,
                W, kh, kw, ph, pw, sh, sw, PH, PW);
  else if (dtype == cgtb_f8)
    CGTB_LAUNCH(max_pool_pullback_kernel<double>, (unsigned)blocks, 256, 0, mask, (const double*)gtop, (double*)gx, total,
                H, W, kh, kw, ph, pw, sh, sw, PH, PW);
  else
    return fail("cgtb_max_pool_pullback: unsupported dtype %d", dtype);
  CGTB_CHECK_LAUNCH("max_pool_pullback");
  return 0;
}

// ================================================================================================
// Cross-channel LRN (include/lrn.cuh). One thread per element; the window sum is formed directly
// (ascending channel) instead of the reference's running add/subtract, which removes the serial
// dependency along channels and is at least as accurate. scale = 1. + accum*(alpha/n) is evaluated
// with the product in T and the sum in double, as the reference expression does.
//   forward window of channel c : [c - (n-1)/2, c + n - (n-1)/2 - 1]
//   backward window of channel c: [c - (n - (n+1)/2), c + (n+1)/2 - 1]
// ================================================================================================
template <typename T>
__global__ void lrn_forward_kernel(const T* __restrict__ x, T* __restrict__ top, T* __restrict__ scale, long total,
                                   int C, int HW, int size, T alpha_over_size, T negative_beta) {
  const int pre = (size - 1) / 2, post = size - pre - 1;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    int hw = (int)(idx % HW);
    long t = idx / HW;
    int c = (int)(t % C);
    long n = t / C;
    const T* col = x + n * (long)C * HW + hw;
    int lo = max(c - pre, 0), hi = min(c + post, C - 1);
    T acc = T(0);
    for (int k = lo; k <= hi; ++k) {
      T v = col[(long)k * HW];
      acc += v * v;
    }
    T s = (T)(1. + (double)(acc * alpha_over_size));
    scale[idx] = s;
    top[idx] = col[(long)c * HW] * pow(s, negative_beta);
  }
}

template <typename T>
__global__ void lrn_backward_kernel(const T* __restrict__ x, const T* __restrict__ top, const T* __restrict__ scale,
                                    const T* __restrict__ gtop, T* __restrict__ gx, long total, int C, int HW, int size,
                                    T negative_beta, T cache_ratio) {
  const int pre = size - (size + 1) / 2, post = size - pre - 1;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    int hw = (int)(idx % HW);
    long t = idx / HW;
    int c = (int)(t % C);
    long n = t / C;
    long base = n * (long)C * HW + hw;
    int lo = max(c - pre, 0), hi = min(c + post, C - 1);
    T acc = T(0);
    for (int k = lo; k <= hi; ++k) {
      long o = base + (long)k * HW;
      acc += gtop[o] * top[o] / scale[o];
    }
    gx[idx] = gtop[idx] * pow(scale[idx], negative_beta) - cache_ratio * x[idx] * acc;
  }
}

CGTB_API int cgtb_lrn_forward(int dtype, const void* x, long N, int C, int H, int W, int size, double alpha, double beta,
                              void* top, void* scale) {
  if (!require_runtime("cgtb_lrn_forward")) return 1;
  if (size <= 0) return fail("cgtb_lrn_forward: localsize must be positive");
  long total = N * C * H * W;
  if (total <= 0) return 0;
  long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 32);
  if (dtype == cgtb_f4)
    CGTB_LAUNCH(lrn_forward_kernel<float>, (unsigned)blocks, 256, 0, (const float*)x, (float*)top, (float*)scale, total, C,
                H * W, size, (float)(alpha / size), (float)(-beta));
  else if (dtype == cgtb_f8)
    CGTB_LAUNCH(lrn_forward_kernel<double>, (unsigned)blocks, 256, 0, (const double*)x, (double*)top, (double*)scale, total,
                C, H * W, size, alpha / size, -beta);
  else
    return fail("cgtb_lrn_forward: unsupported dtype %d", dtype);
  CGTB_CHECK_LAUNCH("lrn_forward");
  return 0;
}

CGTB_API int cgtb_lrn_backward(int dtype, const void* x, const void* top, const void* scale, const void* gtop, long N,
                               int C, int H, int W, int size, double alpha, double beta, void* gx) {
  if (!require_runtime("cgtb_lrn_backward")) return 1;
  if (size <= 0) return fail("cgtb_lrn_backward: localsize must be positive");
  long total = N * C * H * W;
  if (total <= 0) return 0;
  long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 32);
  if (dtype == cgtb_f4)
    CGTB_LAUNCH(lrn_backward_kernel<float>, (unsigned)blocks, 256, 0, (const float*)x, (const float*)top,
                (const float*)scale, (const float*)gtop, (float*)gx, total, C, H * W, size, (float)(-beta),
                (float)(2. * alpha * beta / size));
  else if (dtype == cgtb_f8)
    CGTB_LAUNCH(lrn_backward_kernel<double>, (unsigned)blocks, 256, 0, (const double*)x, (const double*)top,
                (const double*)scale, (const double*)gtop, (double*)gx, total, C, H * W, size, -beta,
                2. * alpha * beta / size);
  else
    return fail("cgtb_lrn_backward: unsupported dtype %d", dtype);
  CGTB_CHECK_LAUNCH("lrn_backward");
  return 0;
}
