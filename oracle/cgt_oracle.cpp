// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// CPU restatement of the reference's native CPU kernels for the compiled-graph execution path.
// Only the test-suite, the smoke check and the benchmark's cpu_baseline / reference arm may load
// this library; the CUDA library never calls into it.
//
// Each function names the reference file:line whose arithmetic and loop order it follows.
// Parity pin: every function here is compared bit-for-bit against the reference's own headers
// (im2col.h, pooling.h, lrn.cuh compiled as C++) by tests/test_oracle.py when oracle/_ref is
// built, and against the golden vectors in tests/golden/ that were generated from them.
// The sgemm of Mul22 is not restated here: the harness calls OpenBLAS through numpy
// (reference pin: OpenBLAS v0.2.14, 4build/download_and_build_openblas.py:14; this image
// carries 0.3.30, so GEMM parity is pinned to tolerance only).
//
// Build: g++ -O2 -ffp-contract=off -std=c++17 -shared -fPIC (see oracle/build_oracle.py).
#include <math.h>
#include <cmath>
#include <cfloat>
#include <cstdint>
#include <cstring>
#include <limits>
#include <algorithm>
#include "../include/cgt_b200_ops.h"

#define ORC_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------------------------
// im2col / col2im : include/im2col.h:6-50, driven per image by cgt/nn_ops/im2col.py:47-60, 78-92
// Column layout is channels-last: col[b, h, w, c] with c = c_im*kh*kw + h_off*kw + w_off.
// ---------------------------------------------------------------------------------------------
template <typename T>
static void im2col_image(const T* im, int channels, int height, int width, int kh, int kw, int ph,
                         int pw, int sh, int sw, T* col) {
  int height_col = (height + 2 * ph - kh) / sh + 1;
  int width_col = (width + 2 * pw - kw) / sw + 1;
  int channels_col = channels * kh * kw;
  for (int c = 0; c < channels_col; ++c) {
    int w_offset = c % kw;
    int h_offset = (c / kw) % kh;
    int c_im = c / kh / kw;
    for (int h = 0; h < height_col; ++h) {
      for (int w = 0; w < width_col; ++w) {
        int h_pad = h * sh - ph + h_offset;
        int w_pad = w * sw - pw + w_offset;
        T v = 0;
        if (h_pad >= 0 && h_pad < height && w_pad >= 0 && w_pad < width)
          v = im[(c_im * height + h_pad) * width + w_pad];
        col[(long)channels_col * width_col * h + (long)channels_col * w + c] = v;
      }
    }
  }
}

template <typename T>
static void col2im_image(const T* col, int channels, int height, int width, int kh, int kw, int ph,
                         int pw, int sh, int sw, T* im) {
  for (long i = 0; i < (long)height * width * channels; ++i) im[i] = T(0);
  int height_col = (height + 2 * ph - kh) / sh + 1;
  int width_col = (width + 2 * pw - kw) / sw + 1;
  int channels_col = channels * kh * kw;
  // accumulation order: column channel (c_im, i, j) outermost, then h, then w
  for (int c = 0; c < channels_col; ++c) {
    int w_offset = c % kw;
    int h_offset = (c / kw) % kh;
    int c_im = c / kh / kw;
    for (int h = 0; h < height_col; ++h) {
      for (int w = 0; w < width_col; ++w) {
        int h_pad = h * sh - ph + h_offset;
        int w_pad = w * sw - pw + w_offset;
        if (h_pad >= 0 && h_pad < height && w_pad >= 0 && w_pad < width)
          im[(c_im * height + h_pad) * width + w_pad] +=
              col[(long)channels_col * width_col * h + (long)channels_col * w + c];
      }
    }
  }
}

ORC_API void orc_im2col_f32(const float* x, long B, int C, int H, int W, int kh, int kw, int ph,
                            int pw, int sh, int sw, float* col) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  long imstride = (long)C * H * W, colstride = (long)Ho * Wo * C * kh * kw;
  for (long b = 0; b < B; ++b)
    im2col_image<float>(x + b * imstride, C, H, W, kh, kw, ph, pw, sh, sw, col + b * colstride);
}
ORC_API void orc_im2col_f64(const double* x, long B, int C, int H, int W, int kh, int kw, int ph,
                            int pw, int sh, int sw, double* col) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  long imstride = (long)C * H * W, colstride = (long)Ho * Wo * C * kh * kw;
  for (long b = 0; b < B; ++b)
    im2col_image<double>(x + b * imstride, C, H, W, kh, kw, ph, pw, sh, sw, col + b * colstride);
}
ORC_API void orc_col2im_f32(const float* col, long B, int C, int H, int W, int kh, int kw, int ph,
                            int pw, int sh, int sw, float* im) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  long imstride = (long)C * H * W, colstride = (long)Ho * Wo * C * kh * kw;
  for (long b = 0; b < B; ++b)
    col2im_image<float>(col + b * colstride, C, H, W, kh, kw, ph, pw, sh, sw, im + b * imstride);
}
ORC_API void orc_col2im_f64(const double* col, long B, int C, int H, int W, int kh, int kw, int ph,
                            int pw, int sh, int sw, double* im) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  long imstride = (long)C * H * W, colstride = (long)Ho * Wo * C * kh * kw;
  for (long b = 0; b < B; ++b)
    col2im_image<double>(col + b * colstride, C, H, W, kh, kw, ph, pw, sh, sw, im + b * imstride);
}

// ---------------------------------------------------------------------------------------------
// max pool forward / pullback : include/pooling.h:24-104.
// Window clipped to the image; strict '>' so the first maximum in (h, w) scan order wins;
// value initialised to -FLT_MAX (for every dtype) and mask to -1; mask = h*W + w inside the plane.
// The pooled size PH x PW is an input here because the reference takes it from the output array
// that Alloc sized with MaxPool.shp_apply (cgt/nn_ops/max_pool_2d.py:36-43).
// ---------------------------------------------------------------------------------------------
template <typename T>
static void max_pool_t(const T* bottom, long B, int C, int H, int W, int kh, int kw, int ph, int pw,
                       int sh, int sw, int PH, int PW, T* top, int32_t* mask) {
  long top_count = B * C * PH * PW;
  for (long i = 0; i < top_count; ++i) top[i] = T(-FLT_MAX);
  for (long i = 0; i < top_count; ++i) mask[i] = -1;
  for (long n = 0; n < B; ++n) {
    for (int c = 0; c < C; ++c) {
      for (int py = 0; py < PH; ++py) {
        for (int px = 0; px < PW; ++px) {
          int hstart = py * sh - ph;
          int wstart = px * sw - pw;
          int hend = std::min(hstart + kh, H);
          int wend = std::min(wstart + kw, W);
          hstart = std::max(hstart, 0);
          wstart = std::max(wstart, 0);
          const int pool_index = py * PW + px;
          for (int h = hstart; h < hend; ++h) {
            for (int w = wstart; w < wend; ++w) {
              const int index = h * W + w;
              if (bottom[index] > top[pool_index]) {
                top[pool_index] = bottom[index];
                mask[pool_index] = index;
              }
            }
          }
        }
      }
      bottom += (long)H * W;
      top += (long)PH * PW;
      mask += (long)PH * PW;
    }
  }
}

template <typename T>
static void max_pool_pullback_t(const int32_t* mask, const T* top_diff, long B, int C, int PH,
                                int PW, int H, int W, T* bottom_diff) {
  for (long i = 0; i < B * C * H * W; ++i) bottom_diff[i] = T(0);
  for (long n = 0; n < B; ++n) {
    for (int c = 0; c < C; ++c) {
      for (int py = 0; py < PH; ++py) {
        for (int px = 0; px < PW; ++px) {
          const int index = py * PW + px;
          const int bottom_index = mask[index];
          // the reference writes out of bounds for a mask of -1 (an all-NaN window); skipped here
          if (bottom_index >= 0) bottom_diff[bottom_index] += top_diff[index];
        }
      }
      bottom_diff += (long)H * W;
      top_diff += (long)PH * PW;
      mask += (long)PH * PW;
    }
  }
}

ORC_API void orc_max_pool_f32(const float* x, long B, int C, int H, int W, int kh, int kw, int ph,
                              int pw, int sh, int sw, int PH, int PW, float* top, int32_t* mask) {
  max_pool_t<float>(x, B, C, H, W, kh, kw, ph, pw, sh, sw, PH, PW, top, mask);
}
ORC_API void orc_max_pool_f64(const double* x, long B, int C, int H, int W, int kh, int kw, int ph,
                              int pw, int sh, int sw, int PH, int PW, double* top, int32_t* mask) {
  max_pool_t<double>(x, B, C, H, W, kh, kw, ph, pw, sh, sw, PH, PW, top, mask);
}
ORC_API void orc_max_pool_pullback_f32(const int32_t* mask, const float* gtop, long B, int C, int PH,
                                       int PW, int H, int W, float* gx) {
  max_pool_pullback_t<float>(mask, gtop, B, C, PH, PW, H, W, gx);
}
ORC_API void orc_max_pool_pullback_f64(const int32_t* mask, const double* gtop, long B, int C,
                                       int PH, int PW, int H, int W, double* gx) {
  max_pool_pullback_t<double>(mask, gtop, B, C, PH, PW, H, W, gx);
}

// ---------------------------------------------------------------------------------------------
// cross-channel LRN : include/lrn.cuh:3-114, launch arithmetic cgt/nn_ops/cross_channel_lrn.py:
// 27-37 (forward: alpha/localsize and -beta narrowed to T) and 78-82 (backward: -beta and
// 2*alpha*beta/localsize narrowed to T). One sliding window per (n, h, w) column; the running
// sums are updated by add-then-subtract exactly as the reference kernels do, so the rounding is
// the same. The literal `1.` in the scale formula is a double: the product is computed in T, the
// sum in double, and the result narrowed to T.
// ---------------------------------------------------------------------------------------------
template <typename T>
static void lrn_forward_t(const T* in, long num, int channels, int height, int width, int size,
                          double alpha, double beta, T* top, T* scale) {
  const T alpha_over_size = (T)(alpha / size);
  const T negative_beta = (T)(-beta);
  long nthreads = num * height * width;
  int step = height * width;
  for (long index = 0; index < nthreads; ++index) {
    int w = index % width;
    int h = (index / width) % height;
    long n = index / width / height;
    long offset = (n * channels * height + h) * width + w;
    const T* sin = in + offset;
    T* sscale = scale + offset;
    int head = 0;
    int pre_pad = (size - 1) / 2;
    int post_pad = size - pre_pad - 1;
    T accum = 0;
    while (head < post_pad) {
      accum += sin[(long)head * step] * sin[(long)head * step];
      ++head;
    }
    while (head < size) {
      accum += sin[(long)head * step] * sin[(long)head * step];
      sscale[(long)(head - post_pad) * step] = (T)(1. + accum * alpha_over_size);
      ++head;
    }
    while (head < channels) {
      accum += sin[(long)head * step] * sin[(long)head * step];
      accum -= sin[(long)(head - size) * step] * sin[(long)(head - size) * step];
      sscale[(long)(head - post_pad) * step] = (T)(1. + accum * alpha_over_size);
      ++head;
    }
    while (head < channels + post_pad) {
      accum -= sin[(long)(head - size) * step] * sin[(long)(head - size) * step];
      sscale[(long)(head - post_pad) * step] = (T)(1. + accum * alpha_over_size);
      ++head;
    }
  }
  long total = num * channels * height * width;
  for (long i = 0; i < total; ++i) top[i] = in[i] * std::pow(scale[i], negative_beta);
}

template <typename T>
static void lrn_backward_t(const T* bottom, const T* top, const T* scale, const T* top_diff, long num,
                           int channels, int height, int width, int size, double alpha, double beta,
                           T* bottom_diff) {
  const T negative_beta = (T)(-beta);
  const T cache_ratio = (T)(2. * alpha * beta / size);
  long nthreads = num * height * width;
  int step = height * width;
  for (long index = 0; index < nthreads; ++index) {
    int w = index % width;
    int h = (index / width) % height;
    long n = index / width / height;
    long offset = (n * channels * height + h) * width + w;
    const T* b = bottom + offset;
    const T* t = top + offset;
    const T* s = scale + offset;
    const T* td = top_diff + offset;
    T* bd = bottom_diff + offset;
    int head = 0;
    int pre_pad = size - (size + 1) / 2;
    int post_pad = size - pre_pad - 1;
    T accum = 0;
#define ORC_IDX(k) ((long)(k) * step)
    while (head < post_pad) {
      accum += td[ORC_IDX(head)] * t[ORC_IDX(head)] / s[ORC_IDX(head)];
      ++head;
    }
    while (head < size) {
      accum += td[ORC_IDX(head)] * t[ORC_IDX(head)] / s[ORC_IDX(head)];
      bd[ORC_IDX(head - post_pad)] =
          td[ORC_IDX(head - post_pad)] * std::pow(s[ORC_IDX(head - post_pad)], negative_beta) -
          cache_ratio * b[ORC_IDX(head - post_pad)] * accum;
      ++head;
    }
    while (head < channels) {
      accum += td[ORC_IDX(head)] * t[ORC_IDX(head)] / s[ORC_IDX(head)];
      accum -= td[ORC_IDX(head - size)] * t[ORC_IDX(head - size)] / s[ORC_IDX(head - size)];
      bd[ORC_IDX(head - post_pad)] =
          td[ORC_IDX(head - post_pad)] * std::pow(s[ORC_IDX(head - post_pad)], negative_beta) -
          cache_ratio * b[ORC_IDX(head - post_pad)] * accum;
      ++head;
    }
    while (head < channels + post_pad) {
      accum -= td[ORC_IDX(head - size)] * t[ORC_IDX(head - size)] / s[ORC_IDX(head - size)];
      bd[ORC_IDX(head - post_pad)] =
          td[ORC_IDX(head - post_pad)] * std::pow(s[ORC_IDX(head - post_pad)], negative_beta) -
          cache_ratio * b[ORC_IDX(head - post_pad)] * accum;
      ++head;
    }
#undef ORC_IDX
  }
}

ORC_API void orc_lrn_forward_f32(const float* x, long N, int C, int H, int W, int size, double alpha,
                                 double beta, float* top, float* scale) {
  lrn_forward_t<float>(x, N, C, H, W, size, alpha, beta, top, scale);
}
ORC_API void orc_lrn_forward_f64(const double* x, long N, int C, int H, int W, int size,
                                 double alpha, double beta, double* top, double* scale) {
  lrn_forward_t<double>(x, N, C, H, W, size, alpha, beta, top, scale);
}
ORC_API void orc_lrn_backward_f32(const float* x, const float* top, const float* scale,
                                  const float* gtop, long N, int C, int H, int W, int size,
                                  double alpha, double beta, float* gx) {
  lrn_backward_t<float>(x, top, scale, gtop, N, C, H, W, size, alpha, beta, gx);
}
ORC_API void orc_lrn_backward_f64(const double* x, const double* top, const double* scale,
                                  const double* gtop, long N, int C, int H, int W, int size,
                                  double alpha, double beta, double* gx) {
  lrn_backward_t<double>(x, top, scale, gtop, N, C, H, W, size, alpha, beta, gx);
}

// ---------------------------------------------------------------------------------------------
// Elementwise unary / binary : loops cgt/core.py:1204-1214 and 1342-1353; C expressions
// cgt/core.py:1119-1133 and 1141-1151; dtype map np2c cgt/core.py:1155-1157.
// The generated code is `static inline OUT scalar_f(IN x) { return <cexpr>; }` compiled as C++
// with <math.h>, so exp/log/tanh/... pick the overload of the INPUT type, double literals force
// double arithmetic for the rest of that sub-expression, and the result narrows to OUT on return.
// ---------------------------------------------------------------------------------------------
template <typename TI, typename TO>
static inline TO unary_apply(int op, TI x) {
  switch (op) {
    case CGTB_U_ABS: return (TO)(fabs(x));
    case CGTB_U_CEIL: return (TO)(ceil(x));
    case CGTB_U_COS: return (TO)(cos(x));
    case CGTB_U_EXP: return (TO)(exp(x));
    case CGTB_U_ICEIL: return (TO)((int)ceil(x));
    case CGTB_U_IFLOOR: return (TO)((int)floor(x));
    case CGTB_U_LOG: return (TO)(log(x));
    case CGTB_U_NEG: return (TO)(-x);
    case CGTB_U_SIGN: return (TO)(2 * (x > 0) - 1);
    case CGTB_U_SIN: return (TO)(sin(x));
    case CGTB_U_SQUARE: return (TO)(x * x);
    case CGTB_U_SQRT: return (TO)(sqrt(x));
    case CGTB_U_TANH: return (TO)(tanh(x));
    case CGTB_U_SIGMOID: return (TO)(1.0 / (1.0 + exp(-x)));
    case CGTB_U_SOFTPLUS: return (TO)((x > 0) ? (x + log(exp(-x) + 1)) : log(1 + exp(x)));
    case CGTB_U_CAST: return (TO)(x);
  }
  return TO(0);
}

template <typename TX, typename TY, typename TO>
static inline TO binary_apply(int op, TX x, TY y) {
  switch (op) {
    case CGTB_B_MUL: return (TO)(x * y);
    case CGTB_B_ADD: return (TO)(x + y);
    case CGTB_B_SUB: return (TO)(x - y);
    case CGTB_B_DIV: return (TO)((x + 0.0) / y);
    case CGTB_B_LT: return (TO)(x < y);
    case CGTB_B_GT: return (TO)(x > y);
    case CGTB_B_LE: return (TO)(x <= y);
    case CGTB_B_GE: return (TO)(x >= y);
    case CGTB_B_POW: return (TO)(pow(x, y));
    case CGTB_B_EQ: return (TO)(x == y);
    case CGTB_B_NE: return (TO)(x != y);
  }
  return TO(0);
}

template <typename TI, typename TO>
static void unary_loop(int op, long n, const void* in, void* out) {
  const TI* a = (const TI*)in;
  TO* o = (TO*)out;
  for (long i = 0; i < n; ++i) o[i] = unary_apply<TI, TO>(op, a[i]);
}

// dispatch helpers over the dtype codes (numpy type numbers)
#define ORC_FOR_DTYPE(code, T, ...)                           \
  switch (code) {                                             \
    case cgtb_i1: { typedef int8_t T; __VA_ARGS__; } break;   \
    case cgtb_i2: { typedef int16_t T; __VA_ARGS__; } break;  \
    case cgtb_i4: { typedef int32_t T; __VA_ARGS__; } break;  \
    case cgtb_i8: { typedef int64_t T; __VA_ARGS__; } break;  \
    case cgtb_f4: { typedef float T; __VA_ARGS__; } break;    \
    case cgtb_f8: { typedef double T; __VA_ARGS__; } break;   \
    default: return -1;                                       \
  }

ORC_API int orc_unary(int op, int dt_in, int dt_out, long n, const void* in, void* out) {
  ORC_FOR_DTYPE(dt_in, TI, ORC_FOR_DTYPE(dt_out, TO, unary_loop<TI, TO>(op, n, in, out)));
  return 0;
}

template <typename TX, typename TY, typename TO>
static void binary_loop(int op, long n, const void* x, const void* y, void* out, int sx, int sy) {
  const TX* a = (const TX*)x;
  const TY* b = (const TY*)y;
  TO* o = (TO*)out;
  for (long i = 0; i < n; ++i) o[i] = binary_apply<TX, TY, TO>(op, a[sx ? 0 : i], b[sy ? 0 : i]);
}

// scalar_x / scalar_y: the operand is 0-d and is read at index 0 (cgt/core.py:1337-1338)
ORC_API int orc_binary(int op, int dt_x, int dt_y, int dt_out, long n, const void* x, const void* y,
                       void* out, int scalar_x, int scalar_y) {
  ORC_FOR_DTYPE(dt_x, TX,
                ORC_FOR_DTYPE(dt_y, TY,
                              ORC_FOR_DTYPE(dt_out, TO,
                                            binary_loop<TX, TY, TO>(op, n, x, y, out, scalar_x,
                                                                    scalar_y))));
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Reductions : gen_reduction_code cgt/core.py:1663-1685; Sum "x+y" init 0 (:1708);
// Max "fmax(x,y)" init -numeric_limits<T>::max() (:1737). keepdims always. The output is the
// accumulator and the input is walked in row-major order, so the fp32 order is sequential.
// ---------------------------------------------------------------------------------------------
template <typename T>
static void reduce_t(int kind, int ndim, const long* shape, const int* reduced, const T* in, T* out) {
  long oshape[CGTB_MAX_NDIM], ostride[CGTB_MAX_NDIM];
  long osize = 1, isize = 1;
  for (int i = 0; i < ndim; ++i) {
    oshape[i] = reduced[i] ? 1 : shape[i];
    isize *= shape[i];
  }
  for (int i = ndim - 1; i >= 0; --i) {
    ostride[i] = osize;
    osize *= oshape[i];
  }
  T init = (kind == CGTB_R_SUM) ? T(0) : -std::numeric_limits<T>::max();
  for (long i = 0; i < osize; ++i) out[i] = init;
  long idx[CGTB_MAX_NDIM] = {0};
  for (long f = 0; f < isize; ++f) {
    long o = 0;
    for (int i = 0; i < ndim; ++i)
      if (!reduced[i]) o += idx[i] * ostride[i];
    T x = out[o], y = in[f];
    out[o] = (kind == CGTB_R_SUM) ? (T)(x + y) : (T)fmax(x, y);
    for (int i = ndim - 1; i >= 0; --i) {
      if (++idx[i] < shape[i]) break;
      idx[i] = 0;
    }
  }
}

ORC_API int orc_reduce(int kind, int dtype, int ndim, const long* shape, const int* reduced,
                       const void* in, void* out) {
  ORC_FOR_DTYPE(dtype, T, reduce_t<T>(kind, ndim, shape, reduced, (const T*)in, (T*)out));
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Data movement. All arrays are C-contiguous.
//   Repeat      cgt/core.py:1527-1542  out[i...] = in[i... with 0 on the repeated axes]
//   Transpose   cgt/core.py:1578-1594  out[i0..] = in[i_{invperm}]  i.e. out axis k is in axis axes[k]
//   GetSli      cgt/core.py:1793-1812  out[.., i, ..] = in[.., start + step*i, ..]
//   IncSli      cgt/core.py:1839-1861  out = in (copy unless aliased); out[.., start+step*i, ..] += inc
//   GetFlat     cgt/core.py:1977-1987  out[i] = x.flat[k[i]]
//   IncFlat     cgt/core.py:2012-2023  out = x; out.flat[k[i]] += p[i], serially (duplicates add up)
//   Concatenate cgt/core.py:1490-1509
//   Fill        cgt/core.py:998-1007 ; Arange cgt/core.py:1037-1048
// ---------------------------------------------------------------------------------------------
template <typename T>
static void repeat_t(int ndim, const long* oshape, const int* rep, const T* in, T* out) {
  long ishape[CGTB_MAX_NDIM], istride[CGTB_MAX_NDIM];
  long osize = 1, acc = 1;
  for (int i = 0; i < ndim; ++i) {
    ishape[i] = rep[i] ? 1 : oshape[i];
    osize *= oshape[i];
  }
  for (int i = ndim - 1; i >= 0; --i) {
    istride[i] = acc;
    acc *= ishape[i];
  }
  long idx[CGTB_MAX_NDIM] = {0};
  for (long f = 0; f < osize; ++f) {
    long s = 0;
    for (int i = 0; i < ndim; ++i)
      if (!rep[i]) s += idx[i] * istride[i];
    out[f] = in[s];
    for (int i = ndim - 1; i >= 0; --i) {
      if (++idx[i] < oshape[i]) break;
      idx[i] = 0;
    }
  }
}
ORC_API int orc_repeat(int dtype, int ndim, const long* out_shape, const int* repeated, const void* in,
                       void* out) {
  ORC_FOR_DTYPE(dtype, T, repeat_t<T>(ndim, out_shape, repeated, (const T*)in, (T*)out));
  return 0;
}

template <typename T>
static void transpose_t(int ndim, const long* ishape, const int* axes, const T* in, T* out) {
  long oshape[CGTB_MAX_NDIM], istride[CGTB_MAX_NDIM];
  long acc = 1, osize = 1;
  for (int i = ndim - 1; i >= 0; --i) {
    istride[i] = acc;
    acc *= ishape[i];
  }
  for (int i = 0; i < ndim; ++i) {
    oshape[i] = ishape[axes[i]];
    osize *= oshape[i];
  }
  long idx[CGTB_MAX_NDIM] = {0};
  for (long f = 0; f < osize; ++f) {
    long s = 0;
    for (int i = 0; i < ndim; ++i) s += idx[i] * istride[axes[i]];
    out[f] = in[s];
    for (int i = ndim - 1; i >= 0; --i) {
      if (++idx[i] < oshape[i]) break;
      idx[i] = 0;
    }
  }
}
ORC_API int orc_transpose(int dtype, int ndim, const long* in_shape, const int* axes, const void* in,
                          void* out) {
  ORC_FOR_DTYPE(dtype, T, transpose_t<T>(ndim, in_shape, axes, (const T*)in, (T*)out));
  return 0;
}

// strided slice helper: view the array as [outer, n_axis, inner]
template <typename T>
static void getsli_t(long outer, long n_in, long inner, long start, long step, long n_out, const T* in,
                     T* out) {
  for (long o = 0; o < outer; ++o)
    for (long i = 0; i < n_out; ++i)
      for (long k = 0; k < inner; ++k)
        out[(o * n_out + i) * inner + k] = in[(o * n_in + start + step * i) * inner + k];
}
ORC_API int orc_getsli(int dtype, long outer, long n_in, long inner, long start, long step, long n_out,
                       const void* in, void* out) {
  ORC_FOR_DTYPE(dtype, T, getsli_t<T>(outer, n_in, inner, start, step, n_out, (const T*)in, (T*)out));
  return 0;
}
template <typename T>
static void incsli_t(long outer, long n_x, long inner, long start, long step, long n_inc, const T* x,
                     const T* inc, T* out) {
  if (out != x) memcpy(out, x, sizeof(T) * outer * n_x * inner);
  for (long o = 0; o < outer; ++o)
    for (long i = 0; i < n_inc; ++i)
      for (long k = 0; k < inner; ++k)
        out[(o * n_x + start + step * i) * inner + k] += inc[(o * n_inc + i) * inner + k];
}
ORC_API int orc_incsli(int dtype, long outer, long n_x, long inner, long start, long step, long n_inc,
                       const void* x, const void* inc, void* out) {
  ORC_FOR_DTYPE(dtype, T,
                incsli_t<T>(outer, n_x, inner, start, step, n_inc, (const T*)x, (const T*)inc, (T*)out));
  return 0;
}

template <typename T>
static void getflat_t(long n, const T* x, const int64_t* k, T* out) {
  for (long i = 0; i < n; ++i) out[i] = x[k[i]];
}
ORC_API int orc_getflat(int dtype, long n, const void* x, const int64_t* k, void* out) {
  ORC_FOR_DTYPE(dtype, T, getflat_t<T>(n, (const T*)x, k, (T*)out));
  return 0;
}
template <typename T>
static void incflat_t(long xsize, long n, const T* x, const int64_t* k, const T* p, T* out) {
  if (out != x) memcpy(out, x, sizeof(T) * xsize);
  for (long i = 0; i < n; ++i) out[k[i]] += p[i];
}
ORC_API int orc_incflat(int dtype, long xsize, long n, const void* x, const int64_t* k, const void* p,
                        void* out) {
  ORC_FOR_DTYPE(dtype, T, incflat_t<T>(xsize, n, (const T*)x, k, (const T*)p, (T*)out));
  return 0;
}

// one input of a concatenation, written at offset `pos` along the axis; view [outer, n_axis, inner]
template <typename T>
static void concat_part_t(long outer, long n_in, long n_out, long inner, long pos, const T* in, T* out) {
  for (long o = 0; o < outer; ++o)
    for (long i = 0; i < n_in; ++i)
      for (long k = 0; k < inner; ++k)
        out[(o * n_out + pos + i) * inner + k] = in[(o * n_in + i) * inner + k];
}
ORC_API int orc_concat_part(int dtype, long outer, long n_in, long n_out, long inner, long pos,
                            const void* in, void* out) {
  ORC_FOR_DTYPE(dtype, T, concat_part_t<T>(outer, n_in, n_out, inner, pos, (const T*)in, (T*)out));
  return 0;
}

// Fill: the closure value is a long for integer dtypes and a double otherwise (cgt/core.py:995-997)
ORC_API int orc_fill(int dtype, long n, double fvalue, long ivalue, void* out) {
  switch (dtype) {
    case cgtb_i1: for (long i = 0; i < n; ++i) ((int8_t*)out)[i] = (int8_t)ivalue; break;
    case cgtb_i2: for (long i = 0; i < n; ++i) ((int16_t*)out)[i] = (int16_t)ivalue; break;
    case cgtb_i4: for (long i = 0; i < n; ++i) ((int32_t*)out)[i] = (int32_t)ivalue; break;
    case cgtb_i8: for (long i = 0; i < n; ++i) ((int64_t*)out)[i] = (int64_t)ivalue; break;
    case cgtb_f4: for (long i = 0; i < n; ++i) ((float*)out)[i] = (float)fvalue; break;
    case cgtb_f8: for (long i = 0; i < n; ++i) ((double*)out)[i] = fvalue; break;
    default: return -1;
  }
  return 0;
}
