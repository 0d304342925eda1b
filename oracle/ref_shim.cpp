// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// Thin extern "C" wrappers around the reference's OWN native CPU code, compiled from the reference
// tree where it lies (nothing is copied): include/im2col.h, include/pooling.h,
// include/cgt_common.h + src/cgt_common.cpp, and include/lrn.cuh compiled as plain C++ (the
// reference has no CPU LRN; its CUDA kernels are grid-stride loops that become sequential loops
// when blockIdx/blockDim/gridDim/threadIdx are the trivial values below).
//
// Built by oracle/build_oracle.py into oracle/_ref/libcgt_ref.so when the reference tree is
// present. Used to pin oracle/cgt_oracle.cpp and to generate tests/golden/.
#include "cgt_common.h"
#include <cmath>
#include <math.h>
#include <cstdint>
using std::pow;

#include "im2col.h"
#include "pooling.h"

// ---- CUDA keyword shim for lrn.cuh ----
#define __global__
struct ref_dim3_ { int x; };
static const ref_dim3_ blockIdx = {0}, blockDim = {1}, gridDim = {1}, threadIdx = {0};
#include "lrn.cuh"

#define REF_API extern "C" __attribute__((visibility("default")))

// im2col_cpu / col2im_cpu take the geometry as template parameters (include/im2col.h:5,30), so
// only the geometries listed here can be run through the reference code.
#define REF_GEOMETRIES(X) \
  X(5, 5, 2, 2, 1, 1)     \
  X(11, 11, 2, 2, 4, 4)   \
  X(4, 4, 0, 0, 1, 1)     \
  X(3, 3, 1, 1, 2, 2)     \
  X(3, 3, 1, 1, 3, 3)     \
  X(4, 7, 3, 6, 1, 1)     \
  X(3, 3, 0, 0, 1, 1)     \
  X(2, 3, 1, 0, 2, 1)     \
  X(1, 1, 0, 0, 1, 1)

template <typename T>
static int im2col_dispatch(const T* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw,
                           int sh, int sw, T* col) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  long ims = (long)C * H * W, cols = (long)Ho * Wo * C * kh * kw;
#define X(KH, KW, PH, PW, SH, SW)                                                        \
  if (kh == KH && kw == KW && ph == PH && pw == PW && sh == SH && sw == SW) {            \
    for (long b = 0; b < B; ++b)                                                         \
      im2col_cpu<T, KH, KW, PH, PW, SH, SW>(x + b * ims, C, H, W, col + b * cols);       \
    return 0;                                                                            \
  }
  REF_GEOMETRIES(X)
#undef X
  return -1;
}

template <typename T>
static int col2im_dispatch(const T* col, long B, int C, int H, int W, int kh, int kw, int ph, int pw,
                           int sh, int sw, T* im) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  long ims = (long)C * H * W, cols = (long)Ho * Wo * C * kh * kw;
#define X(KH, KW, PH, PW, SH, SW)                                                        \
  if (kh == KH && kw == KW && ph == PH && pw == PW && sh == SH && sw == SW) {            \
    for (long b = 0; b < B; ++b)                                                         \
      col2im_cpu<T, KH, KW, PH, PW, SH, SW>(col + b * cols, C, H, W, im + b * ims);      \
    return 0;                                                                            \
  }
  REF_GEOMETRIES(X)
#undef X
  return -1;
}

REF_API int ref_im2col_f32(const float* x, long B, int C, int H, int W, int kh, int kw, int ph,
                           int pw, int sh, int sw, float* col) {
  return im2col_dispatch<float>(x, B, C, H, W, kh, kw, ph, pw, sh, sw, col);
}
REF_API int ref_im2col_f64(const double* x, long B, int C, int H, int W, int kh, int kw, int ph,
                           int pw, int sh, int sw, double* col) {
  return im2col_dispatch<double>(x, B, C, H, W, kh, kw, ph, pw, sh, sw, col);
}
REF_API int ref_col2im_f32(const float* col, long B, int C, int H, int W, int kh, int kw, int ph,
                           int pw, int sh, int sw, float* im) {
  return col2im_dispatch<float>(col, B, C, H, W, kh, kw, ph, pw, sh, sw, im);
}
REF_API int ref_col2im_f64(const double* col, long B, int C, int H, int W, int kh, int kw, int ph,
                           int pw, int sh, int sw, double* im) {
  return col2im_dispatch<double>(col, B, C, H, W, kh, kw, ph, pw, sh, sw, im);
}

template <typename T>
static cgtArray* view4(const T* p, long a, long b, long c, long d, cgtDtype dt) {
  long shape[4] = {a, b, c, d};
  cgtArray* out = new cgtArray(4, shape, dt, cgtCPU, (void*)p, false);
  out->Retain();
  return out;
}

template <typename T>
static void max_pool_ref(const T* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                         int sw, int PH, int PW, T* top, int32_t* mask, cgtDtype dt) {
  conv_closure cl = {kh, kw, ph, pw, sh, sw};
  cgtArray* ab = view4(x, B, C, H, W, dt);
  cgtArray* at = view4(top, B, C, PH, PW, dt);
  cgtArray* am = view4(mask, B, C, PH, PW, cgt_i4);
  max_pool<T>(&cl, ab, at, am);
  ab->Release();
  at->Release();
  am->Release();
}
REF_API void ref_max_pool_f32(const float* x, long B, int C, int H, int W, int kh, int kw, int ph,
                              int pw, int sh, int sw, int PH, int PW, float* top, int32_t* mask) {
  max_pool_ref<float>(x, B, C, H, W, kh, kw, ph, pw, sh, sw, PH, PW, top, mask, cgt_f4);
}
REF_API void ref_max_pool_f64(const double* x, long B, int C, int H, int W, int kh, int kw, int ph,
                              int pw, int sh, int sw, int PH, int PW, double* top, int32_t* mask) {
  max_pool_ref<double>(x, B, C, H, W, kh, kw, ph, pw, sh, sw, PH, PW, top, mask, cgt_f8);
}

template <typename T>
static void max_pool_pullback_ref(const int32_t* mask, const T* gtop, long B, int C, int PH, int PW,
                                  int H, int W, T* gx, cgtDtype dt) {
  // bottom and top are only used for their shapes (include/pooling.h:83-89)
  cgtArray* ab = view4(gx, B, C, H, W, dt);
  cgtArray* at = view4(gtop, B, C, PH, PW, dt);
  cgtArray* am = view4(mask, B, C, PH, PW, cgt_i4);
  cgtArray* agt = view4(gtop, B, C, PH, PW, dt);
  cgtArray* agx = view4(gx, B, C, H, W, dt);
  max_pool_pullback<T>(ab, at, am, agt, agx);
  ab->Release();
  at->Release();
  am->Release();
  agt->Release();
  agx->Release();
}
REF_API void ref_max_pool_pullback_f32(const int32_t* mask, const float* gtop, long B, int C, int PH,
                                       int PW, int H, int W, float* gx) {
  max_pool_pullback_ref<float>(mask, gtop, B, C, PH, PW, H, W, gx, cgt_f4);
}
REF_API void ref_max_pool_pullback_f64(const int32_t* mask, const double* gtop, long B, int C, int PH,
                                       int PW, int H, int W, double* gx) {
  max_pool_pullback_ref<double>(mask, gtop, B, C, PH, PW, H, W, gx, cgt_f8);
}

// launch arithmetic of cgt/nn_ops/cross_channel_lrn.py:27-37 and 78-82
template <typename T>
static void lrn_forward_ref(const T* x, long N, int C, int H, int W, int size, double alpha, double beta,
                            T* top, T* scale) {
  int n = (int)(N * H * W);
  LRNFillScale<T>(n, x, (int)N, C, H, W, size, alpha / size, scale);
  n = (int)(N * C * W * H);
  LRNComputeOutput<T>(n, x, scale, -beta, top);
}
template <typename T>
static void lrn_backward_ref(const T* x, const T* top, const T* scale, const T* gtop, long N, int C,
                             int H, int W, int size, double alpha, double beta, T* gx) {
  int n = (int)(N * W * H);
  LRNComputeDiff<T>(n, x, top, scale, gtop, (int)N, C, H, W, size, -beta, 2. * alpha * beta / size, gx);
}
REF_API void ref_lrn_forward_f32(const float* x, long N, int C, int H, int W, int size, double alpha,
                                 double beta, float* top, float* scale) {
  lrn_forward_ref<float>(x, N, C, H, W, size, alpha, beta, top, scale);
}
REF_API void ref_lrn_forward_f64(const double* x, long N, int C, int H, int W, int size,
                                 double alpha, double beta, double* top, double* scale) {
  lrn_forward_ref<double>(x, N, C, H, W, size, alpha, beta, top, scale);
}
REF_API void ref_lrn_backward_f32(const float* x, const float* top, const float* scale,
                                  const float* gtop, long N, int C, int H, int W, int size,
                                  double alpha, double beta, float* gx) {
  lrn_backward_ref<float>(x, top, scale, gtop, N, C, H, W, size, alpha, beta, gx);
}
REF_API void ref_lrn_backward_f64(const double* x, const double* top, const double* scale,
                                  const double* gtop, long N, int C, int H, int W, int size,
                                  double alpha, double beta, double* gx) {
  lrn_backward_ref<double>(x, top, scale, gtop, N, C, H, W, size, alpha, beta, gx);
}
