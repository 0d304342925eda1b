// Built-in Op callables: the functions the interpreter reaches through ReturnByRef / ReturnByVal.
//
// Each has one of the reference's two callable signatures (include/cgt_common.h:176-177 of the
// reference) and a closure struct whose fields are the Op's closure triples, in order, exactly as the
// Python side lays them out with ctypes. Where the reference generates a C++ loop per Op instance
// (cgt/core.py, cgt/nn_ops/*.py), these read the geometry from the arrays and the closure and launch
// the CUDA kernels of this library. An array on the host is accepted only where the reference's
// placement rule puts one: 0-d scalars and shape arithmetic (cgt/compilation.py:63-64); tensor
// work on host arrays is refused rather than emulated.
#include "runtime.h"
#include <cmath>
#include <cstring>
#include <limits>
#include <type_traits>

using namespace cgtb;

namespace cgtb {
int sgemm_dispatch(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
                   long ldb, long strideB, float* C, long ldc, long strideC, int impl);
}

#define OP_BYREF(name) CGTB_API void name(void* cl0, cgtObject** reads, cgtObject* write0)
#define OP_BYVAL(name) CGTB_API cgtObject* name(void* cl0, cgtObject** reads)
#define ARR(o) ((cgtArray*)(o))

static const long kHostTensorLimit = 64;  // host arrays larger than this are tensor work, not scalar bookkeeping

static bool on_gpu(cgtArray* a) { return a->devtype() == cgtGPU; }
static bool all_gpu(std::initializer_list<cgtArray*> as) {
  for (auto a : as) if (!on_gpu(a)) return false;
  return true;
}
static bool host_scalar_ok(const char* op, std::initializer_list<cgtArray*> as) {
  for (auto a : as) {
    if (on_gpu(a)) { fail("%s: operands live on different devices (a Transport is missing)", op); return false; }
    if (a->size() > kHostTensorLimit) {
      fail("%s: a %ld-element tensor was placed on the host; this backend has no CPU implementation of tensor ops", op, a->size());
      return false;
    }
  }
  return true;
}
static long host_i8(cgtObject* o) { return ARR(o)->at<long>(0); }

// ------------------------------------------------------------------------------------------------
// host-side scalar expressions (same promotions as the device versions in kernels_elem.cu)
// ------------------------------------------------------------------------------------------------
template <typename TI, typename TO>
static TO h_unary(int op, TI x) {
  typedef typename std::conditional<std::is_floating_point<TI>::value, TI, double>::type TM;
  switch (op) {
    case CGTB_U_ABS: return (TO)(std::fabs((TM)x));
    case CGTB_U_CEIL: return (TO)(std::ceil((TM)x));
    case CGTB_U_COS: return (TO)(std::cos((TM)x));
    case CGTB_U_EXP: return (TO)(std::exp((TM)x));
    case CGTB_U_ICEIL: return (TO)((int)std::ceil((TM)x));
    case CGTB_U_IFLOOR: return (TO)((int)std::floor((TM)x));
    case CGTB_U_LOG: return (TO)(std::log((TM)x));
    case CGTB_U_NEG: return (TO)(-x);
    case CGTB_U_SIGN: return (TO)(2 * (x > 0) - 1);
    case CGTB_U_SIN: return (TO)(std::sin((TM)x));
    case CGTB_U_SQUARE: return (TO)(x * x);
    case CGTB_U_SQRT: return (TO)(std::sqrt((TM)x));
    case CGTB_U_TANH: return (TO)(std::tanh((TM)x));
    case CGTB_U_SIGMOID: return (TO)(1.0 / (1.0 + std::exp((TM)(-x))));
    case CGTB_U_SOFTPLUS: return (TO)((x > 0) ? (x + std::log(std::exp((TM)(-x)) + 1)) : std::log(1 + std::exp((TM)x)));
    case CGTB_U_CAST: return (TO)(x);
  }
  return TO(0);
}
template <typename TX, typename TY, typename TO>
static TO h_binary(int op, TX x, TY y) {
  switch (op) {
    case CGTB_B_MUL: return (TO)(x * y);
    case CGTB_B_ADD: return (TO)(x + y);
    case CGTB_B_SUB: return (TO)(x - y);
    case CGTB_B_DIV: return (TO)((x + 0.0) / y);
    case CGTB_B_LT: return (TO)(x < y);
    case CGTB_B_GT: return (TO)(x > y);
    case CGTB_B_LE: return (TO)(x <= y);
    case CGTB_B_GE: return (TO)(x >= y);
    case CGTB_B_POW: {
      if (std::is_same<TX, float>::value && std::is_same<TY, float>::value) return (TO)(std::pow((float)x, (float)y));
      return (TO)(std::pow((double)x, (double)y));
    }
    case CGTB_B_EQ: return (TO)(x == y);
    case CGTB_B_NE: return (TO)(x != y);
  }
  return TO(0);
}
#define HOST_FOR_DTYPE(code, T, ...)                          \
  switch (code) {                                             \
    case cgt_i1: { typedef int8_t T; __VA_ARGS__; } break;    \
    case cgt_i2: { typedef int16_t T; __VA_ARGS__; } break;   \
    case cgt_i4: { typedef int32_t T; __VA_ARGS__; } break;   \
    case cgt_i8: { typedef int64_t T; __VA_ARGS__; } break;   \
    case cgt_f4: { typedef float T; __VA_ARGS__; } break;     \
    case cgt_f8: { typedef double T; __VA_ARGS__; } break;    \
    default: fail("unsupported dtype %d", (int)(code));       \
  }

// ------------------------------------------------------------------------------------------------
// ElwiseUnary / ElwiseBinary (cgt/core.py:1160-1378)
// ------------------------------------------------------------------------------------------------
struct UnaryClosure { int op; };
OP_BYREF(cgtb_op_elwise_unary) {
  UnaryClosure* cl = (UnaryClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *w = ARR(write0);
  if (w->size() != x->size()) { fail("ElwiseUnary: output has %ld elements, input %ld", w->size(), x->size()); return; }
  if (all_gpu({x, w})) { cgtb_unary(cl->op, x->dtype(), w->dtype(), x->size(), x->data(), w->data()); return; }
  if (!host_scalar_ok("ElwiseUnary", {x, w})) return;
  long n = x->size();
  HOST_FOR_DTYPE(x->dtype(), TI, HOST_FOR_DTYPE(w->dtype(), TO, {
    for (long i = 0; i < n; ++i) w->at<TO>(i) = h_unary<TI, TO>(cl->op, x->at<TI>(i));
  }));
}

struct BinaryClosure { int op; int scalar_x; int scalar_y; };
OP_BYREF(cgtb_op_elwise_binary) {
  BinaryClosure* cl = (BinaryClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *y = ARR(reads[1]), *w = ARR(write0);
  long n = cl->scalar_x ? y->size() : x->size();
  if (w->size() != n || (!cl->scalar_x && !cl->scalar_y && x->size() != y->size())) {
    fail("Shape error in elementwise binary operation. You might be missing a call to cgt.broadcast(...)");
    return;
  }
  if (all_gpu({x, y, w})) {
    cgtb_binary(cl->op, x->dtype(), y->dtype(), w->dtype(), n, x->data(), y->data(), w->data(), cl->scalar_x, cl->scalar_y);
    return;
  }
  if (!host_scalar_ok("ElwiseBinary", {x, y, w})) return;
  HOST_FOR_DTYPE(x->dtype(), TX, HOST_FOR_DTYPE(y->dtype(), TY, HOST_FOR_DTYPE(w->dtype(), TO, {
    for (long i = 0; i < n; ++i)
      w->at<TO>(i) = h_binary<TX, TY, TO>(cl->op, x->at<TX>(cl->scalar_x ? 0 : i), y->at<TY>(cl->scalar_y ? 0 : i));
  })));
}

// FusedElwise: closure = the program (include/cgt_b200.h). reads = the program's inputs; write = the
// output array, or a tuple of arrays when the program has several outputs. Broadcast extents come
// from the shapes: the input's non-unit axes form one run [d0, d1] of the output's axes.
// FusedRows: elementwise operations and row sums over the rows of an [R, C] matrix. The closure is the program
// followed by C; R comes from the first result (which has R or R*C elements).
struct FusedRowsClosure { cgtbRowProgram prog; int C; };
OP_BYREF(cgtb_op_fused_rows) {
  const FusedRowsClosure* cl = (const FusedRowsClosure*)cl0;
  const cgtbRowProgram& P = cl->prog;
  cgtArray* outs[CGTB_FUSED_MAX_OUT];
  if (P.n_out == 1) outs[0] = ARR(write0);
  else {
    cgtTuple* tup = (cgtTuple*)write0;
    for (int j = 0; j < P.n_out; ++j) outs[j] = (cgtArray*)tup->getitem(j);
  }
  const long C = cl->C;
  const long R = P.out_col[0] ? outs[0]->size() : outs[0]->size() / C;
  const void* in[CGTB_FUSED_MAX_IN];
  void* out[CGTB_FUSED_MAX_OUT];
  for (int j = 0; j < P.n_out; ++j) {
    if (outs[j]->devtype() != cgtGPU || outs[j]->dtype() != cgt_f4 || outs[j]->size() != (P.out_col[j] ? R : R * C)) {
      fail("FusedRows: result %d is not a float32 GPU array of the expected size", j);
      return;
    }
    out[j] = outs[j]->data();
  }
  for (int k = 0; k < P.n_in; ++k) {
    cgtArray* x = ARR(reads[k]);
    const int kind = P.in_kind[k];
    const long want = kind == CGTB_FIN_F4 ? R * C : ((kind == CGTB_FIN_COL || kind == CGTB_FIN_ROWHOT) ? R : (kind == CGTB_FIN_ROW ? C : 1));
    const bool scalar_i8 = kind == CGTB_FIN_SCALAR_I8 || kind == CGTB_FIN_ROWHOT;
    if (x->devtype() != cgtGPU || x->size() != want || x->dtype() != (scalar_i8 ? cgt_i8 : cgt_f4)) {
      fail("FusedRows: operand %d has the wrong size, dtype or device", k);
      return;
    }
    in[k] = x->data();
  }
  cgtb_fused_rows(&P, R, C, in, out);
}

// OneHotRows: (idx int64 [R]) -> float32 [R, C] with a one in column idx[r] of row r. Closure: C.
struct OneHotRowsClosure { long C; };
OP_BYREF(cgtb_op_onehot_rows) {
  const OneHotRowsClosure* cl = (const OneHotRowsClosure*)cl0;
  cgtArray *idx = ARR(reads[0]), *w = ARR(write0);
  if (!on_gpu(idx) || !on_gpu(w) || idx->dtype() != cgt_i8 || w->dtype() != cgt_f4 || w->size() != idx->size() * cl->C) {
    fail("OneHotRows: an int64 GPU vector of R column numbers and a float32 GPU result of R x %ld", cl->C);
    return;
  }
  cgtb_onehot_rows((const long*)idx->data(), idx->size(), cl->C, (float*)w->data());
}

// MaskedRowSum: (x f4 [R, C], m f4 [R, C]) -> [R, 1]: the sum of each row's elements where m is not zero
OP_BYREF(cgtb_op_masked_row_sum) {
  cgtArray *x = ARR(reads[0]), *m = ARR(reads[1]), *w = ARR(write0);
  if (!all_gpu({x, m, w}) || x->ndim() != 2 || x->dtype() != cgt_f4 || m->dtype() != cgt_f4 || w->dtype() != cgt_f4 || m->size() != x->size() ||
      w->size() != x->shape()[0]) {
    fail("MaskedRowSum: two float32 GPU matrices of one shape [R, C] and a float32 GPU result of R elements");
    return;
  }
  cgtb_masked_row_sum((const float*)x->data(), (const float*)m->data(), x->shape()[0], x->shape()[1], (float*)w->data());
}

// ScatterCols: k column pieces placed into a zero matrix. Closure: k, C, offsets, widths; reads = the pieces.
struct ScatterColsClosure { int k; long C; long off[8]; long width[8]; };
OP_BYREF(cgtb_op_scatter_cols) {
  const ScatterColsClosure* cl = (const ScatterColsClosure*)cl0;
  cgtArray* w = ARR(write0);
  if (cl->k < 1 || cl->k > 8) { fail("ScatterCols: between 1 and 8 pieces"); return; }
  if (!on_gpu(w) || w->dtype() != cgt_f4 || w->ndim() != 2 || w->shape()[1] != cl->C) { fail("ScatterCols: the result must be a float32 GPU matrix with %ld columns", cl->C); return; }
  const long R = w->shape()[0];
  const void* pieces[8];
  for (int j = 0; j < cl->k; ++j) {
    cgtArray* y = ARR(reads[j]);
    if (!on_gpu(y) || y->dtype() != cgt_f4 || y->size() != R * cl->width[j]) { fail("ScatterCols: piece %d is not a float32 GPU array of %ld x %ld", j, R, cl->width[j]); return; }
    pieces[j] = y->data();
  }
  cgtb_scatter_cols(R, cl->C, cl->k, cl->off, cl->width, pieces, w->data());
}

// MultiFusedElwise: one FusedElwise program over k independent tensors in one launch. The closure is the program
// followed by k; reads = the k operand lists back to back (n_in each), then the result arrays of tensors 1..k-1
// (the instruction's own write location is tensor 0's result). The compiler forms it from k parameter updates.
struct MultiFusedClosure { cgtbFusedProgram prog; int k; };
// FusedElwise: the program, then for every CGTB_FIN_VIEW_F4 input the row length of its matrix and its first column
struct FusedClosure { cgtbFusedProgram prog; long view_pitch[CGTB_FUSED_MAX_IN]; long view_off[CGTB_FUSED_MAX_IN]; };
OP_BYREF(cgtb_op_multi_fused_elwise) {
  const MultiFusedClosure* cl = (const MultiFusedClosure*)cl0;
  const int k = cl->k, n_in = cl->prog.n_in;
  if (k < 1 || k > 24 || n_in < 1 || n_in > 4) { fail("MultiFusedElwise: unsupported group of %d tensors with %d inputs", k, n_in); return; }
  const void* in[24 * 4];
  void* out[24];
  long n[24];
  for (int t = 0; t < k; ++t) {
    cgtArray* w = ARR(t == 0 ? write0 : reads[k * n_in + t - 1]);
    if (w->devtype() != cgtGPU || w->dtype() != cgt_f4) { fail("MultiFusedElwise: results must be float32 GPU arrays"); return; }
    out[t] = w->data();
    n[t] = w->size();
    for (int q = 0; q < n_in; ++q) {
      cgtArray* x = ARR(reads[t * n_in + q]);
      if (x->devtype() != cgtGPU) { fail("MultiFusedElwise: operands must be on the GPU"); return; }
      if (cl->prog.in_kind[q] == CGTB_FIN_F4 && x->size() != n[t]) { fail("MultiFusedElwise: operand and result sizes differ"); return; }
      in[t * n_in + q] = x->data();
    }
  }
  cgtb_fused_elwise_multi(&cl->prog, k, n, in, out);
}
OP_BYREF(cgtb_op_fused_elwise) {
  const cgtbFusedProgram* prog = (const cgtbFusedProgram*)cl0;
  cgtArray* outs[CGTB_FUSED_MAX_OUT];
  if (prog->n_out == 1 && write0->kind() == cgtObject::ArrayKind) {
    outs[0] = ARR(write0);
  } else {
    cgtTuple* tup = (cgtTuple*)write0;
    for (int q = 0; q < prog->n_out; ++q) outs[q] = ARR(tup->getitem(q));
  }
  cgtArray* w = outs[0];
  const long n = w->size();
  const void* in[CGTB_FUSED_MAX_IN];
  void* out[CGTB_FUSED_MAX_OUT];
  long bk[CGTB_FUSED_MAX_IN], binner[CGTB_FUSED_MAX_IN];
  for (int q = 0; q < prog->n_out; ++q) {
    if (outs[q]->size() != n || outs[q]->devtype() != cgtGPU) { fail("FusedElwise: outputs must be GPU arrays of one size"); return; }
    out[q] = outs[q]->data();
  }
  for (int k = 0; k < prog->n_in; ++k) {
    cgtArray* x = ARR(reads[k]);
    if (x->devtype() != cgtGPU) { fail("FusedElwise: operands must be on the GPU"); return; }
    in[k] = x->data();
    bk[k] = binner[k] = 1;
    const int kind = prog->in_kind[k];
    if ((kind == CGTB_FIN_F4 || kind == CGTB_FIN_I1) && x->size() != n) {
      fail("Shape error in a fused elementwise chain. You might be missing a call to cgt.broadcast(...)");
      return;
    }
    if (kind == CGTB_FIN_VIEW_F4) {
      const FusedClosure* fc = (const FusedClosure*)cl0;
      const long W = prog->view_width;
      if (W <= 0 || n % W != 0 || x->dtype() != cgt_f4 || x->size() != (n / W) * fc->view_pitch[k]) {
        fail("FusedElwise: operand %d is not the [%ld, %ld] matrix whose columns the chain reads", k, W > 0 ? n / W : 0, fc->view_pitch[k]);
        return;
      }
      bk[k] = fc->view_pitch[k];
      binner[k] = fc->view_off[k];
    }
    if (kind == CGTB_FIN_BCAST_F4) {
      if (x->ndim() != w->ndim()) { fail("FusedElwise: a broadcast operand must have the rank of the result"); return; }
      int d0 = -1, d1 = -1;
      for (int d = 0; d < x->ndim(); ++d) {
        if (x->shape()[d] != 1) {
          if (x->shape()[d] != w->shape()[d]) { fail("FusedElwise: broadcast operand does not match the result's shape"); return; }
          if (d0 < 0) d0 = d;
          d1 = d;
        }
      }
      long kk = 1, inner = 1;
      if (d0 >= 0) {
        for (int d = d0; d <= d1; ++d) {
          if (x->shape()[d] != w->shape()[d]) { fail("FusedElwise: the kept axes of a broadcast operand must be adjacent"); return; }
          kk *= w->shape()[d];
        }
        for (int d = d1 + 1; d < w->ndim(); ++d) inner *= w->shape()[d];
      }
      bk[k] = kk;
      binner[k] = inner;
    }
  }
  cgtb_fused_elwise(prog, n, in, bk, binner, out);
}

// ------------------------------------------------------------------------------------------------
// Mul22 / BatchedMul22 (cgt/core.py:2129-2288). Closure layout of the reference: tA, tB, handle.
// ------------------------------------------------------------------------------------------------
struct Mul22Closure { bool tA; bool tB; void* handle; };
OP_BYREF(cgtb_op_mul22) {
  Mul22Closure* cl = (Mul22Closure*)cl0;
  cgtArray *A = ARR(reads[0]), *B = ARR(reads[1]), *C = ARR(write0);
  if (!all_gpu({A, B, C})) { fail("Mul22: operands must be on the GPU; there is no CPU GEMM in this backend"); return; }
  long lda = A->shape()[1], ldb = B->shape()[1], ldc = C->shape()[1];
  long M = C->shape()[0], N = C->shape()[1], K = A->shape()[cl->tA ? 0 : 1];
  long Kb = B->shape()[cl->tB ? 1 : 0], Ma = A->shape()[cl->tA ? 1 : 0], Nb = B->shape()[cl->tB ? 0 : 1];
  if (K != Kb || M != Ma || N != Nb) { fail("shape mismatch at matrix-matrix multiplication: (%ld x %ld) * (%ld x %ld) -> (%ld x %ld)", Ma, K, Kb, Nb, M, N); return; }
  if (A->dtype() == cgt_f4)
    sgemm_dispatch(cl->tA, cl->tB, 1, M, N, K, (const float*)A->data(), lda, 0, (const float*)B->data(), ldb, 0, (float*)C->data(), ldc, 0, 0);
  else if (A->dtype() == cgt_f8)
    cgtb_dgemm(cl->tA, cl->tB, M, N, K, (const double*)A->data(), lda, (const double*)B->data(), ldb, (double*)C->data(), ldc);
  else
    fail("Mul22: unsupported dtype %d", (int)A->dtype());
}
// Mul22BiasAdd: (A, B, bias [1,N], addend [M,N], addend_bias [1,N]) -> (addend + addend_bias) + (A.B + bias)
OP_BYREF(cgtb_op_mul22_bias_add) {
  Mul22Closure* cl = (Mul22Closure*)cl0;
  cgtArray *A = ARR(reads[0]), *B = ARR(reads[1]), *bias = ARR(reads[2]), *add = ARR(reads[3]), *abias = ARR(reads[4]), *C = ARR(write0);
  if (!all_gpu({A, B, bias, add, abias, C})) { fail("Mul22BiasAdd: operands must be on the GPU"); return; }
  long lda = A->shape()[1], ldb = B->shape()[1], ldc = C->shape()[1];
  long M = C->shape()[0], N = C->shape()[1], K = A->shape()[cl->tA ? 0 : 1];
  long Kb = B->shape()[cl->tB ? 1 : 0], Ma = A->shape()[cl->tA ? 1 : 0], Nb = B->shape()[cl->tB ? 0 : 1];
  if (K != Kb || M != Ma || N != Nb || A->dtype() != cgt_f4 || B->dtype() != cgt_f4 || bias->dtype() != cgt_f4 || add->dtype() != cgt_f4 ||
      abias->dtype() != cgt_f4 || bias->size() != N || abias->size() != N || add->size() != M * N) {
    fail("Mul22BiasAdd: operand shapes do not fit together");
    return;
  }
  cgtb_sgemm_bias_add(cl->tA, cl->tB, M, N, K, (const float*)A->data(), lda, (const float*)B->data(), ldb, (const float*)bias->data(),
                      (const float*)add->data(), N, (const float*)abias->data(), (float*)C->data(), ldc);
}
struct BMul22Closure { bool tA; bool tB; };
OP_BYREF(cgtb_op_batched_mul22) {
  BMul22Closure* cl = (BMul22Closure*)cl0;
  cgtArray *A = ARR(reads[0]), *B = ARR(reads[1]), *C = ARR(write0);
  if (!all_gpu({A, B, C})) { fail("BatchedMul22: operands must be on the GPU"); return; }
  if (A->dtype() != cgt_f4) { fail("BatchedMul22: only float32 is implemented on the GPU"); return; }
  long P = A->shape()[0];
  long lda = A->shape()[2], ldb = B->shape()[2], ldc = C->shape()[2];
  long M = C->shape()[1], N = C->shape()[2], K = A->shape()[1 + (cl->tA ? 0 : 1)];
  if (B->shape()[0] != P || C->shape()[0] != P || B->shape()[1 + (cl->tB ? 1 : 0)] != K) { fail("shape mismatch at batched matrix multiplication"); return; }
  sgemm_dispatch(cl->tA, cl->tB, P, M, N, K, (const float*)A->data(), lda, A->stride(0), (const float*)B->data(), ldb,
                 B->stride(0), (float*)C->data(), ldc, C->stride(0), 0);
}

// ------------------------------------------------------------------------------------------------
// Im2Col / Col2Im / MaxPool / MaxPoolPullback share the reference's conv_closure (include/pooling.h:7-14)
// ------------------------------------------------------------------------------------------------
struct ConvClosure { int kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w; };
// the same followed by a flag: the filter operand is the layer's bank in its own layout, not a rearranged copy
struct ConvClosureW { int kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, w_bank, pre; };   // pre: the last read is the bank's [w_hi | w_lo] copy
OP_BYREF(cgtb_op_im2col) {
  ConvClosure* cl = (ConvClosure*)cl0;
  cgtArray *im = ARR(reads[0]), *col = ARR(write0);
  if (!all_gpu({im, col})) { fail("Im2Col: operands must be on the GPU"); return; }
  const long* s = im->shape();
  // the output's last extent is the row pitch: C*kh*kw, or more when the compiler asked for padded rows
  cgtb_im2col_ld(im->dtype(), im->data(), s[0], (int)s[1], (int)s[2], (int)s[3], cl->kernel_h, cl->kernel_w, cl->pad_h, cl->pad_w,
                 cl->stride_h, cl->stride_w, col->shape()[3], col->data());
}
OP_BYREF(cgtb_op_col2im) {
  ConvClosure* cl = (ConvClosure*)cl0;
  cgtArray *col = ARR(reads[0]), *im = ARR(write0);
  if (!all_gpu({col, im})) { fail("Col2Im: operands must be on the GPU"); return; }
  long B = host_i8(reads[1]), C = host_i8(reads[2]), H = host_i8(reads[3]), W = host_i8(reads[4]);
  cgtb_col2im(col->dtype(), col->data(), B, (int)C, (int)H, (int)W, cl->kernel_h, cl->kernel_w, cl->pad_h, cl->pad_w,
              cl->stride_h, cl->stride_w, im->data());
}
// ConvBiasRelu: (col [M,K], w [C,K], bias [1,C,1,1], B, C, H, W) -> tuple(mask i1 NCHW, y f4 NCHW)
OP_BYREF(cgtb_op_conv_bias_relu) {
  cgtArray *col = ARR(reads[0]), *w = ARR(reads[1]), *bias = ARR(reads[2]);
  cgtTuple* out = (cgtTuple*)write0;
  cgtArray *mask = ARR(out->getitem(0)), *y = ARR(out->getitem(1));
  if (!all_gpu({col, w, bias, mask, y})) { fail("ConvBiasRelu: operands must be on the GPU"); return; }
  const long* d = y->shape();
  // col rows may be padded beyond the K entries of a filter row (cgtb_im2col_ld)
  const long M = col->shape()[0], ldcol = col->shape()[1], K = w->shape()[1], C = d[1], HW = d[2] * d[3];
  if (col->ndim() != 2 || w->ndim() != 2 || y->ndim() != 4 || col->dtype() != cgt_f4 || w->shape()[0] != C || ldcol < K ||
      bias->size() != C || M != d[0] * HW || mask->size() != y->size()) {
    fail("ConvBiasRelu: operand shapes do not fit together");
    return;
  }
  cgtb_conv_bias_relu_ld((const float*)col->data(), M, K, ldcol, (const float*)w->data(), (int)C, (const float*)bias->data(), HW,
                         (float*)y->data(), (int8_t*)mask->data());
}
// ConvDirectFwd / ConvDirectWgrad: the first layer of an image network directly from the NCHW image (closure: the six
// ints of the reference's conv_closure; the filter gradient adds the number of filters)
struct ConvDirectClosure { int kh, kw, ph, pw, sv, sh, cout; };
OP_BYREF(cgtb_op_conv_direct_fwd) {
  const ConvDirectClosure* cl = (const ConvDirectClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *w = ARR(reads[1]), *bias = ARR(reads[2]);
  cgtTuple* out = (cgtTuple*)write0;
  cgtArray *mask = ARR(out->getitem(0)), *y = ARR(out->getitem(1));
  if (!all_gpu({x, w, bias, mask, y})) { fail("ConvDirectFwd: operands must be on the GPU"); return; }
  if (x->ndim() != 4 || y->ndim() != 4 || x->dtype() != cgt_f4 || cl->sv != 1 || cl->sh != 1) { fail("ConvDirectFwd: a stride-1 convolution of a float32 NCHW image"); return; }
  const long* xs = x->shape();
  const long* d = y->shape();
  if (d[0] != xs[0] || d[2] != xs[2] || d[3] != xs[3] || w->size() != d[1] * xs[1] * cl->kh * cl->kw || bias->size() != d[1] || mask->size() != y->size()) {
    fail("ConvDirectFwd: operand shapes do not fit together");
    return;
  }
  cgtb_conv_direct_fwd_bias_relu((const float*)x->data(), xs[0], (int)xs[1], (int)xs[2], (int)xs[3], (const float*)w->data(), (int)d[1], cl->kh,
                                 cl->kw, cl->ph, cl->pw, (const float*)bias->data(), (float*)y->data(), (signed char*)mask->data());
}
OP_BYREF(cgtb_op_conv_direct_wgrad) {
  const ConvDirectClosure* cl = (const ConvDirectClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *dy = ARR(reads[1]), *out = ARR(write0);
  if (!all_gpu({x, dy, out})) { fail("ConvDirectWgrad: operands must be on the GPU"); return; }
  if (x->ndim() != 4 || x->dtype() != cgt_f4 || dy->dtype() != cgt_f4 || cl->sv != 1 || cl->sh != 1) { fail("ConvDirectWgrad: a stride-1 convolution of a float32 NCHW image"); return; }
  const long* xs = x->shape();
  if (dy->size() != xs[0] * xs[2] * xs[3] * cl->cout || out->size() != (long)cl->cout * xs[1] * cl->kh * cl->kw) {
    fail("ConvDirectWgrad: operand shapes do not fit together");
    return;
  }
  cgtb_conv_direct_wgrad((const float*)x->data(), xs[0], (int)xs[1], (int)xs[2], (int)xs[3], (const float*)dy->data(), cl->cout, cl->kh, cl->kw,
                         cl->ph, cl->pw, (float*)out->data());
}
// ConvDirectWgradRelu: (x NCHW, relu mask i1 NCHW, g f4 NCHW) -> tuple(filter gradient [Cout, Cin*kh*kw], bias gradient [1,Cout,1,1])
OP_BYREF(cgtb_op_conv_direct_wgrad_relu) {
  const ConvDirectClosure* cl = (const ConvDirectClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *mask = ARR(reads[1]), *g = ARR(reads[2]);
  cgtTuple* out = (cgtTuple*)write0;
  cgtArray *dw = ARR(out->getitem(0)), *db = ARR(out->getitem(1));
  if (!all_gpu({x, mask, g, dw, db})) { fail("ConvDirectWgradRelu: operands must be on the GPU"); return; }
  if (x->ndim() != 4 || x->dtype() != cgt_f4 || g->dtype() != cgt_f4 || mask->dtype() != cgt_i1 || cl->sv != 1 || cl->sh != 1) {
    fail("ConvDirectWgradRelu: a stride-1 convolution of a float32 NCHW image, an int8 mask and a float32 gradient");
    return;
  }
  const long* xs = x->shape();
  if (g->size() != xs[0] * xs[2] * xs[3] * cl->cout || mask->size() != g->size() || dw->size() != (long)cl->cout * xs[1] * cl->kh * cl->kw ||
      db->size() != cl->cout) {
    fail("ConvDirectWgradRelu: operand shapes do not fit together");
    return;
  }
  cgtb_conv_direct_wgrad_relu((const float*)x->data(), xs[0], (int)xs[1], (int)xs[2], (int)xs[3], (const signed char*)mask->data(),
                              (const float*)g->data(), cl->cout, cl->kh, cl->kw, cl->ph, cl->pw, (float*)dw->data(), (float*)db->data());
}
// ConvWgrad: (dy [M,C], col [M,ldcol]) -> dy^T * col[:, :K] as [C,K]: the filter gradient from a column matrix
// with padded rows; K is the output's second extent
OP_BYREF(cgtb_op_conv_wgrad) {
  cgtArray *dy = ARR(reads[0]), *col = ARR(reads[1]), *out = ARR(write0);
  if (!all_gpu({dy, col, out})) { fail("ConvWgrad: operands must be on the GPU"); return; }
  if (dy->ndim() != 2 || col->ndim() != 2 || out->ndim() != 2 || dy->dtype() != cgt_f4 || col->dtype() != cgt_f4 ||
      dy->shape()[0] != col->shape()[0] || out->shape()[0] != dy->shape()[1] || out->shape()[1] > col->shape()[1]) {
    fail("ConvWgrad: operand shapes do not fit together");
    return;
  }
  const long M = dy->shape()[0], C = dy->shape()[1], K = out->shape()[1];
  sgemm_dispatch(1, 0, 1, C, K, M, (const float*)dy->data(), C, 0, (const float*)col->data(), col->shape()[1], 0,
                 (float*)out->data(), K, 0, 0);
}
// ReluGradNHWC: (mask i1 NCHW, g f4 NCHW) -> tuple(mask*g transposed to NHWC, Sum{0,2,3}(mask*g) as [1,C,1,1])
OP_BYREF(cgtb_op_relu_grad_nhwc) {
  cgtArray *mask = ARR(reads[0]), *g = ARR(reads[1]);
  cgtTuple* out = (cgtTuple*)write0;
  cgtArray *gt = ARR(out->getitem(0)), *bsum = ARR(out->getitem(1));
  if (!all_gpu({mask, g, gt, bsum})) { fail("ReluGradNHWC: operands must be on the GPU"); return; }
  const long* d = g->shape();
  if (g->ndim() != 4 || g->dtype() != cgt_f4 || mask->size() != g->size() || gt->size() != g->size() || bsum->size() != d[1]) {
    fail("ReluGradNHWC: operand shapes do not fit together");
    return;
  }
  cgtb_relu_grad_nhwc((const int8_t*)mask->data(), (const float*)g->data(), d[0], (int)d[1], d[2] * d[3], (float*)gt->data(),
                      (float*)bsum->data());
}
// ConvDgrad: (dy NHWC, filters rearranged to [C, kh, kw, Cin], B, C, H, W) -> dx NCHW
OP_BYREF(cgtb_op_conv_dgrad) {
  ConvClosureW* cl = (ConvClosureW*)cl0;
  cgtArray *dy = ARR(reads[0]), *wr = ARR(reads[1]), *dx = ARR(write0);
  if (!all_gpu({dy, wr, dx})) { fail("ConvDgrad: operands must be on the GPU"); return; }
  const long* s = dy->shape();
  const long* d = dx->shape();
  const long* ws = wr->shape();
  const bool wok = cl->w_bank ? (ws[0] == s[3] && ws[1] == d[1] && ws[2] == cl->kernel_h && ws[3] == cl->kernel_w)
                              : (ws[0] == d[1] && ws[1] == cl->kernel_h && ws[2] == cl->kernel_w && ws[3] == s[3]);
  if (dy->ndim() != 4 || wr->ndim() != 4 || dx->ndim() != 4 || dy->dtype() != cgt_f4 || !wok || s[0] != d[0]) {
    fail("ConvDgrad: operand shapes do not fit together");
    return;
  }
  if (cl->pre) {
    cgtArray* sp = ARR(reads[6]);
    if (!cl->w_bank || !on_gpu(sp) || sp->dtype() != cgt_f4 || sp->size() != 2 * wr->size()) { fail("ConvDgrad: the split filter copy does not fit the bank"); return; }
    cgtb_conv_dgrad_pre((const float*)dy->data(), s[0], (int)s[1], (int)s[2], (int)s[3], (const float*)wr->data(), (const float*)sp->data(), (int)d[1],
                        (int)d[2], (int)d[3], cl->kernel_h, cl->kernel_w, cl->pad_h, cl->pad_w, (float*)dx->data());
    return;
  }
  (cl->w_bank ? cgtb_conv_dgrad_bank : cgtb_conv_dgrad)((const float*)dy->data(), s[0], (int)s[1], (int)s[2], (int)s[3], (const float*)wr->data(), (int)d[1], (int)d[2],
                  (int)d[3], cl->kernel_h, cl->kernel_w, cl->pad_h, cl->pad_w, (float*)dx->data());
}
// ConvFwdBiasRelu: (x NHWC [B,H,W,Cin], filters rearranged to [Cout,kh,kw,Cin], bias [1,Cout,1,1], B, Cout, Ho, Wo)
// -> tuple(mask i1 NCHW, y f4 NCHW): a stride-1 convolution layer's forward pass without a column matrix
OP_BYREF(cgtb_op_conv_fwd_bias_relu) {
  ConvClosureW* cl = (ConvClosureW*)cl0;
  cgtArray *x = ARR(reads[0]), *wr = ARR(reads[1]), *bias = ARR(reads[2]);
  cgtTuple* out = (cgtTuple*)write0;
  cgtArray *mask = ARR(out->getitem(0)), *y = ARR(out->getitem(1));
  if (!all_gpu({x, wr, bias, mask, y})) { fail("ConvFwdBiasRelu: operands must be on the GPU"); return; }
  const long* s = x->shape();
  const long* d = y->shape();
  const long* ws = wr->shape();
  const bool wok = cl->w_bank ? (ws[0] == d[1] && ws[1] == s[3] && ws[2] == cl->kernel_h && ws[3] == cl->kernel_w)
                              : (ws[0] == d[1] && ws[1] == cl->kernel_h && ws[2] == cl->kernel_w && ws[3] == s[3]);
  if (x->ndim() != 4 || wr->ndim() != 4 || y->ndim() != 4 || x->dtype() != cgt_f4 || !wok || s[0] != d[0] ||
      bias->size() != d[1] || mask->size() != y->size()) {
    fail("ConvFwdBiasRelu: operand shapes do not fit together");
    return;
  }
  if (cl->pre) {
    cgtArray* sp = ARR(reads[7]);
    if (!cl->w_bank || !on_gpu(sp) || sp->dtype() != cgt_f4 || sp->size() != 2 * wr->size()) { fail("ConvFwdBiasRelu: the split filter copy does not fit the bank"); return; }
    cgtb_conv_fwd_bias_relu_pre((const float*)x->data(), s[0], (int)s[1], (int)s[2], (int)s[3], (const float*)wr->data(), (const float*)sp->data(),
                                (int)d[1], (int)d[2], (int)d[3], cl->kernel_h, cl->kernel_w, cl->pad_h, cl->pad_w, (const float*)bias->data(),
                                (float*)y->data(), (int8_t*)mask->data());
    return;
  }
  (cl->w_bank ? cgtb_conv_fwd_bias_relu_bank : cgtb_conv_fwd_bias_relu)((const float*)x->data(), s[0], (int)s[1], (int)s[2], (int)s[3], (const float*)wr->data(), (int)d[1],
                          (int)d[2], (int)d[3], cl->kernel_h, cl->kernel_w, cl->pad_h, cl->pad_w, (const float*)bias->data(),
                          (float*)y->data(), (int8_t*)mask->data());
}
// SplitFilterBanks: (banks...) -> tuple of [2, n_out, taps * n_src] copies, job j from read src[j]; one launch for all
struct SplitBanksClosure { int njobs; int src[8]; int n_out[8]; int n_src[8]; int taps[8]; int layout[8]; };
OP_BYREF(cgtb_op_split_filter_banks) {
  const SplitBanksClosure* cl = (const SplitBanksClosure*)cl0;
  if (cl->njobs < 1 || cl->njobs > 8) { fail("SplitFilterBanks: between 1 and 8 jobs"); return; }
  cgtTuple* out = (cgtTuple*)write0;
  const float* banks[8];
  float* outs[8];
  for (int j = 0; j < cl->njobs; ++j) {
    cgtArray *w = ARR(reads[cl->src[j]]), *o = ARR(out->getitem(j));
    const long n = (long)cl->n_out[j] * cl->n_src[j] * cl->taps[j];
    if (!on_gpu(w) || !on_gpu(o) || w->dtype() != cgt_f4 || o->dtype() != cgt_f4 || w->size() != n || o->size() != 2 * n) {
      fail("SplitFilterBanks: job %d: a float32 GPU bank of %ld elements and a float32 GPU result of twice as many", j, n);
      return;
    }
    banks[j] = (const float*)w->data();
    outs[j] = (float*)o->data();
  }
  cgtb_split_filter_banks(cl->njobs, banks, cl->n_out, cl->n_src, cl->taps, cl->layout, outs);
}
// ConvWgradImplicit: (x NHWC [B,H,W,Cin], dy NHWC [B,Ho,Wo,Cout]) -> filter gradient [Cout, Cin*kh*kw]
OP_BYREF(cgtb_op_conv_wgrad_implicit) {
  ConvClosure* cl = (ConvClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *dy = ARR(reads[1]), *dw = ARR(write0);
  if (!all_gpu({x, dy, dw})) { fail("ConvWgradImplicit: operands must be on the GPU"); return; }
  const long* s = x->shape();
  const long* g = dy->shape();
  if (x->ndim() != 4 || dy->ndim() != 4 || dw->ndim() != 2 || x->dtype() != cgt_f4 || dy->dtype() != cgt_f4 || s[0] != g[0] ||
      dw->shape()[0] != g[3] || dw->shape()[1] != s[3] * cl->kernel_h * cl->kernel_w) {
    fail("ConvWgradImplicit: operand shapes do not fit together");
    return;
  }
  cgtb_conv_wgrad((const float*)x->data(), s[0], (int)s[1], (int)s[2], (int)s[3], (const float*)dy->data(), (int)g[1], (int)g[2],
                  (int)g[3], cl->kernel_h, cl->kernel_w, cl->pad_h, cl->pad_w, (float*)dw->data());
}
OP_BYREF(cgtb_op_max_pool) {
  ConvClosure* cl = (ConvClosure*)cl0;
  cgtArray* x = ARR(reads[0]);
  cgtTuple* out = (cgtTuple*)write0;
  cgtArray *top = ARR(out->getitem(0)), *mask = ARR(out->getitem(1));
  if (!all_gpu({x, top, mask})) { fail("MaxPool: operands must be on the GPU"); return; }
  const long* s = x->shape();
  cgtb_max_pool(x->dtype(), x->data(), s[0], (int)s[1], (int)s[2], (int)s[3], cl->kernel_h, cl->kernel_w, cl->pad_h, cl->pad_w,
                cl->stride_h, cl->stride_w, (int)top->shape()[2], (int)top->shape()[3], top->data(), (int32_t*)mask->data());
}
OP_BYREF(cgtb_op_max_pool_pullback) {
  ConvClosure* cl = (ConvClosure*)cl0;
  // reads: x, pooled, mask, gpooled ; x and pooled only give shapes (include/pooling.h:83-89)
  cgtArray *x = ARR(reads[0]), *mask = ARR(reads[2]), *gtop = ARR(reads[3]), *gx = ARR(write0);
  if (!all_gpu({x, mask, gtop, gx})) { fail("MaxPoolPullback: operands must be on the GPU"); return; }
  const long* s = x->shape();
  cgtb_max_pool_pullback(gtop->dtype(), (const int32_t*)mask->data(), gtop->data(), s[0], (int)s[1], (int)mask->shape()[2],
                         (int)mask->shape()[3], (int)s[2], (int)s[3], cl->kernel_h, cl->kernel_w, cl->pad_h, cl->pad_w,
                         cl->stride_h, cl->stride_w, gx->data());
}

// ------------------------------------------------------------------------------------------------
// CrossChannelLRN (cgt/nn_ops/cross_channel_lrn.py:8-13 closure: localsize, alpha, beta)
// ------------------------------------------------------------------------------------------------
struct LrnClosure { int localsize; double alpha; double beta; };
OP_BYREF(cgtb_op_lrn_forward) {
  LrnClosure* cl = (LrnClosure*)cl0;
  cgtArray* x = ARR(reads[0]);
  cgtTuple* out = (cgtTuple*)write0;
  cgtArray *top = ARR(out->getitem(0)), *scale = ARR(out->getitem(1));
  if (!all_gpu({x, top, scale})) { fail("CrossChannelLRNForward: operands must be on the GPU"); return; }
  const long* s = x->shape();
  cgtb_lrn_forward(x->dtype(), x->data(), s[0], (int)s[1], (int)s[2], (int)s[3], cl->localsize, cl->alpha, cl->beta, top->data(),
                   scale->data());
}
OP_BYREF(cgtb_op_lrn_backward) {
  LrnClosure* cl = (LrnClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *top = ARR(reads[1]), *scale = ARR(reads[2]), *gtop = ARR(reads[3]), *gx = ARR(write0);
  if (!all_gpu({x, top, scale, gtop, gx})) { fail("CrossChannelLRNBackward: operands must be on the GPU"); return; }
  const long* s = x->shape();
  cgtb_lrn_backward(x->dtype(), x->data(), top->data(), scale->data(), gtop->data(), s[0], (int)s[1], (int)s[2], (int)s[3],
                    cl->localsize, cl->alpha, cl->beta, gx->data());
}

// ------------------------------------------------------------------------------------------------
// Sum / Max (cgt/core.py:1687-1738). axes are a bit mask.
// ------------------------------------------------------------------------------------------------
struct ReduceClosure { int kind; int axes_mask; };
OP_BYREF(cgtb_op_reduce) {
  ReduceClosure* cl = (ReduceClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *w = ARR(write0);
  int red[CGTB_MAX_NDIM];
  for (int i = 0; i < x->ndim(); ++i) red[i] = (cl->axes_mask >> i) & 1;
  if (all_gpu({x, w})) { cgtb_reduce(cl->kind, x->dtype(), x->ndim(), x->shape(), red, x->data(), w->data()); return; }
  fail("Sum/Max: operands must be on the GPU");
}

// ------------------------------------------------------------------------------------------------
// Repeat / Transpose / slices / flat indices / Concatenate / Fill / constants
// ------------------------------------------------------------------------------------------------
struct RepeatClosure { int axes_mask; };
OP_BYREF(cgtb_op_repeat) {
  RepeatClosure* cl = (RepeatClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *w = ARR(write0);
  int rep[CGTB_MAX_NDIM];
  for (int i = 0; i < w->ndim(); ++i) {
    rep[i] = (cl->axes_mask >> i) & 1;
    if (rep[i] && x->shape()[i] != 1) { fail("Repeat: axis %d of the input has extent %ld, expected 1", i, x->shape()[i]); return; }
  }
  if (!all_gpu({x, w})) { fail("Repeat: operands must be on the GPU"); return; }
  cgtb_repeat(x->dtype(), w->ndim(), w->shape(), rep, x->data(), w->data());
}
struct TransposeClosure { long perm; };  // 4 bits per output axis
OP_BYREF(cgtb_op_transpose) {
  TransposeClosure* cl = (TransposeClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *w = ARR(write0);
  int axes[CGTB_MAX_NDIM];
  for (int i = 0; i < x->ndim(); ++i) axes[i] = (int)((cl->perm >> (4 * i)) & 15);
  if (!all_gpu({x, w})) { fail("Transpose: operands must be on the GPU"); return; }
  cgtb_transpose(x->dtype(), x->ndim(), x->shape(), axes, x->data(), w->data());
}
struct AxisClosure { int axis; };
static void split3(cgtArray* a, int axis, long* outer, long* n, long* inner) {
  *outer = 1; *inner = 1;
  for (int i = 0; i < axis; ++i) *outer *= a->shape()[i];
  for (int i = axis + 1; i < a->ndim(); ++i) *inner *= a->shape()[i];
  *n = a->shape()[axis];
}
OP_BYREF(cgtb_op_getsli) {
  AxisClosure* cl = (AxisClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *w = ARR(write0);
  long start = host_i8(reads[1]), step = host_i8(reads[3]);
  long outer, n_in, inner;
  split3(x, cl->axis, &outer, &n_in, &inner);
  if (!all_gpu({x, w})) { fail("GetSli: operands must be on the GPU"); return; }
  cgtb_getsli(x->dtype(), outer, n_in, inner, start, step, w->shape()[cl->axis], x->data(), w->data());
}
OP_BYREF(cgtb_op_incsli) {
  AxisClosure* cl = (AxisClosure*)cl0;
  cgtArray *x = ARR(reads[0]), *inc = ARR(reads[4]), *w = ARR(write0);
  long start = host_i8(reads[1]), step = host_i8(reads[3]);
  long outer, n_x, inner;
  split3(x, cl->axis, &outer, &n_x, &inner);
  if (!all_gpu({x, inc, w})) { fail("IncSli: operands must be on the GPU"); return; }
  if (x->size() != w->size()) { fail("IncSli: output size differs from input size"); return; }
  cgtb_incsli(x->dtype(), outer, n_x, inner, start, step, inc->shape()[cl->axis], x->data(), inc->data(), w->data());
}
OP_BYREF(cgtb_op_getflat) {
  cgtArray *x = ARR(reads[0]), *k = ARR(reads[1]), *w = ARR(write0);
  if (!all_gpu({x, k, w})) { fail("GetFlatIndices: operands must be on the GPU"); return; }
  if (k->dtype() != cgt_i8) { fail("GetFlatIndices: indices must be int64"); return; }
  cgtb_getflat(x->dtype(), w->size(), x->data(), (const int64_t*)k->data(), w->data());
}
OP_BYREF(cgtb_op_incflat) {
  cgtArray *x = ARR(reads[0]), *k = ARR(reads[1]), *p = ARR(reads[2]), *w = ARR(write0);
  if (!all_gpu({x, k, p, w})) { fail("IncFlatIndices: operands must be on the GPU"); return; }
  if (k->dtype() != cgt_i8) { fail("IncFlatIndices: indices must be int64"); return; }
  cgtb_incflat(x->dtype(), x->size(), p->size(), x->data(), (const int64_t*)k->data(), p->data(), w->data());
}
OP_BYVAL(cgtb_op_leading_slice) {  // rows [start, stop) of a C-contiguous array as a view that retains its source
  cgtArray* in = ARR(reads[0]);
  const long start = host_i8(reads[1]), stop = host_i8(reads[2]);
  if (in->ndim() < 1 || in->ndim() > CGTB_MAX_NDIM) { fail("LeadingSlice: needs an array of 1 to %d axes", CGTB_MAX_NDIM); return nullptr; }
  if (start < 0 || stop < start || stop > in->shape()[0]) { fail("LeadingSlice: rows [%ld, %ld) outside the %ld rows of the array", start, stop, in->shape()[0]); return nullptr; }
  long shape[CGTB_MAX_NDIM], row = 1;
  for (int i = 0; i < in->ndim(); ++i) shape[i] = in->shape()[i];
  for (int i = 1; i < in->ndim(); ++i) row *= shape[i];
  shape[0] = stop - start;
  char* base = (char*)in->data() + (size_t)start * (size_t)row * (size_t)cgt_itemsize(in->dtype());
  return new cgtArray(in->ndim(), shape, in->dtype(), in->devtype(), base, (cgtObject*)in);
}
struct ConcatClosure { int axis; int n_in; };
OP_BYREF(cgtb_op_concatenate) {
  ConcatClosure* cl = (ConcatClosure*)cl0;
  cgtArray* w = ARR(write0);
  if (cl->axis == 0 && cl->n_in >= 2 && cl->n_in <= 64) {
    // pieces are contiguous runs: one launch for all of them
    const void* pieces[64];
    long bytes[64], total = 0;
    for (int i = 0; i < cl->n_in; ++i) {
      cgtArray* x = ARR(reads[i]);
      if (!all_gpu({x, w})) { fail("Concatenate: operands must be on the GPU"); return; }
      if (x->dtype() != w->dtype()) { fail("Concatenate: operands of different dtypes"); return; }
      pieces[i] = x->data();
      bytes[i] = x->nbytes();
      total += bytes[i];
    }
    if (total != w->nbytes()) { fail("Concatenate: the parts have %ld bytes, the result %ld", total, (long)w->nbytes()); return; }
    cgtb_concat_rows(cl->n_in, pieces, bytes, w->data());
    return;
  }
  long pos = 0;
  for (int i = 0; i < cl->n_in; ++i) {
    cgtArray* x = ARR(reads[i]);
    if (!all_gpu({x, w})) { fail("Concatenate: operands must be on the GPU"); return; }
    long outer, n_in, inner;
    split3(x, cl->axis, &outer, &n_in, &inner);
    if (cgtb_concat_part(x->dtype(), outer, n_in, w->shape()[cl->axis], inner, pos, x->data(), w->data())) return;
    pos += n_in;
  }
}
struct FillClosure { double fvalue; long ivalue; };
OP_BYREF(cgtb_op_fill) {
  FillClosure* cl = (FillClosure*)cl0;
  cgtArray* w = ARR(write0);
  if (on_gpu(w)) { cgtb_fill(w->dtype(), w->size(), cl->fvalue, cl->ivalue, w->data()); return; }
  if (!host_scalar_ok("Fill", {w})) return;
  long n = w->size();
  HOST_FOR_DTYPE(w->dtype(), T, {
    for (long i = 0; i < n; ++i) w->at<T>(i) = std::is_floating_point<T>::value ? (T)cl->fvalue : (T)cl->ivalue;
  });
}
// ConstantTensor, byref (cgt/core.py:914-935): copy the closure's host buffer into the output,
// which may live on either device.
struct ConstClosure { int ndim; void* shape; unsigned char dtype; void* data; };
OP_BYREF(cgtb_op_constant) {
  ConstClosure* cl = (ConstClosure*)cl0;
  cgtArray* w = ARR(write0);
  cgtb_memcpy((int)w->devtype(), cgtbCPU, w->data(), cl->data, w->nbytes(), 0);
}
// Transport (cgt/core.py:1596-1612)
OP_BYREF(cgtb_op_transport) { cgt_copy_object(write0, reads[0]); }

// ------------------------------------------------------------------------------------------------
// by-value ops: host bookkeeping that never touches array data
// ------------------------------------------------------------------------------------------------
struct ReshapeClosure { int ndim; };
OP_BYVAL(cgtb_op_reshape) {  // cgt/core.py:1451-1465; the view retains its source
  ReshapeClosure* cl = (ReshapeClosure*)cl0;
  cgtArray* in = ARR(reads[0]);
  long shape[CGTB_MAX_NDIM], total = 1;
  if (cl->ndim > CGTB_MAX_NDIM) { fail("Reshape: ndim %d too large", cl->ndim); return nullptr; }
  for (int i = 0; i < cl->ndim; ++i) {
    shape[i] = host_i8(reads[i + 1]);
    if (shape[i] < 0) { fail("negative size in reshape not supported"); return nullptr; }
    total *= shape[i];
  }
  if (total != in->size()) { fail("Reshape: cannot view %ld elements as %ld", in->size(), total); return nullptr; }
  return new cgtArray(cl->ndim, shape, in->dtype(), in->devtype(), in->data(), (cgtObject*)in);
}
struct SizeClosure { int ax; };
OP_BYVAL(cgtb_op_size) {  // cgt/core.py:1421-1430
  SizeClosure* cl = (SizeClosure*)cl0;
  cgtArray* out = new cgtArray(0, nullptr, cgt_i8, cgtCPU);
  out->at<long>(0) = ARR(reads[0])->shape()[cl->ax];
  return out;
}
OP_BYVAL(cgtb_op_arange) {  // cgt/core.py:1037-1048 : host int64 vector
  long start = host_i8(reads[0]), stop = host_i8(reads[1]), step = host_i8(reads[2]);
  if (step == 0) { fail("Arange: zero step"); return nullptr; }
  long size = (stop - start) / step;
  if (size < 0) size = 0;
  cgtArray* out = new cgtArray(1, &size, cgt_i8, cgtCPU);
  for (long i = 0; i < size; ++i) out->at<long>(i) = start + i * step;
  return out;
}
struct TupleIndexClosure { int idx; };
OP_BYVAL(cgtb_op_tuple_index) {  // cgt/core.py:2437-2442
  TupleIndexClosure* cl = (TupleIndexClosure*)cl0;
  cgtTuple* t = (cgtTuple*)reads[0];
  if (cl->idx < 0 || cl->idx >= t->len) { fail("TupleIndex: index %d out of range", cl->idx); return nullptr; }
  return t->getitem(cl->idx);
}
struct DataClosure { void* pptr; };
OP_BYVAL(cgtb_op_in_memory_data) {  // cgt/core.py:557-564
  DataClosure* cl = (DataClosure*)cl0;
  return *(cgtObject**)cl->pptr;
}
