/* C ABI of libcgt_b200.so: the B200 (sm_100a) execution backend for CGT compiled graphs.
 *
 * Plain C, plain pointers and sizes. Every entry point returns 0 on success and non-zero on failure
 * unless stated otherwise; the message of the last failure on the calling thread is read with
 * cgtb_last_error(). Nothing aborts, and no entry point falls back to a CPU implementation:
 * tensor work always runs as CUDA kernels on the runtime's current stream.
 *
 * Each group names the reference interface it replaces (paths inside the reference project).
 */
#ifndef CGT_B200_H
#define CGT_B200_H
#include <stdint.h>
#include "cgt_b200_ops.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cgtbObject cgtbObject; /* a cgtObject* (array or tuple), reference-counted */
typedef struct cgtbGraph cgtbGraph;   /* execution graph under construction */
typedef struct cgtbInterp cgtbInterp; /* interpreter bound to one execution graph */

/* ------------------------------------------------------------------------------------------------
 * Runtime. Replaces the implicit "device 0, default stream, cudaMalloc per array" behaviour of
 * src/cgt_common.cpp:110-153 and include/cgt_cuda.h.
 * ---------------------------------------------------------------------------------------------- */
int cgtb_init(int device);                 /* bind this process to one GPU; creates stream + pools */
int cgtb_initialized(void);                /* 1 after a successful cgtb_init */
int cgtb_device(void);                     /* device index bound by cgtb_init, -1 before */
const char* cgtb_last_error(void);         /* message of the last failure ("" if none) */
void cgtb_clear_error(void);
int cgtb_synchronize(void);                /* cudaStreamSynchronize on the runtime stream */
void* cgtb_stream(void);                   /* the runtime's cudaStream_t */
int cgtb_pool_stats(long* reserved_bytes, long* in_use_bytes, long* high_water_bytes, long* n_device_mallocs);
int cgtb_pool_trim(void);                  /* return cached blocks to the driver */
long cgtb_kernel_launches(void);           /* kernels launched by this library since load */
int cgtb_sm_count(void);

/* Timing on the runtime stream (CUDA events) and an L2 flush for benchmarks. */
void* cgtb_event_new(void);
int cgtb_event_record(void* event);
int cgtb_event_elapsed_ms(void* start, void* stop, float* ms); /* waits for `stop` */
void cgtb_event_free(void* event);
int cgtb_l2_flush(void);                   /* memset of a 256 MiB device buffer */
/* Asks the CUDA runtime for a launch it refuses on the host (too many threads per block; nothing reaches the GPU)
 * and returns that failure. For tests of the error model: the refusal is reported by this call only and later
 * calls are unaffected. No counterpart in the reference (include/cgt_cuda.h:11-16 prints CUDA errors and goes on). */
int cgtb_selftest_refused_launch(void);

/* Raw memory. devtype: 0 host (pinned), 1 device. (src/cgt_common.cpp:110-153) */
void* cgtb_alloc(int devtype, long nbytes);
void cgtb_free(int devtype, void* p);
int cgtb_memcpy(int dst_devtype, int src_devtype, void* dst, const void* src, long nbytes, int sync);
/* Input prefetch (no counterpart in the reference, whose Transport copies inside the step: cgt/core.py:1419-1430).
 * Host->device copies of a later step's inputs on a second stream, into caller-owned staging buffers grouped in
 * slots 0..3. begin(slot): the copy stream waits until the step that last read the slot has finished (see release);
 * h2d: one copy, queued and returned at once; mark(slot): closes the slot's group; join(slot): the runtime stream
 * waits for that group only; release(slot): call after queueing the step that reads the slot. src_host should be
 * page-locked (cgtb_alloc with devtype 0). None of the calls synchronises the host. */
int cgtb_prefetch_begin(int slot);
int cgtb_prefetch_h2d(void* dst_device, const void* src_host, long nbytes);
int cgtb_prefetch_mark(int slot);
int cgtb_prefetch_join(int slot);
int cgtb_prefetch_release(int slot);
int cgtb_memset(void* dev_ptr, int value, long nbytes);

/* ------------------------------------------------------------------------------------------------
 * Objects. Replaces numpy<->cgtArray marshalling in src/cycgt.pyx:92-140 and CppArrayWrapper
 * (src/cycgt.pyx:371-401).
 * ---------------------------------------------------------------------------------------------- */
cgtbObject* cgtb_array_new(int ndim, const long* shape, int dtype, int devtype);
/* copy=1: new owning array on devtype filled from host memory; copy=0: view of host memory */
cgtbObject* cgtb_array_from_host(int ndim, const long* shape, int dtype, int devtype, void* host, int copy);
/* non-owning view of device memory the caller keeps alive */
cgtbObject* cgtb_array_view_device(int ndim, const long* shape, int dtype, void* dev_ptr);
int cgtb_array_to_host(cgtbObject* a, void* host_dst);          /* synchronous */
int cgtb_array_set_from_host(cgtbObject* a, const void* host);  /* synchronous */
int cgtb_array_ndim(cgtbObject* a);
const long* cgtb_array_shape(cgtbObject* a);
int cgtb_array_dtype(cgtbObject* a);
int cgtb_array_devtype(cgtbObject* a);
void* cgtb_array_data(cgtbObject* a);
long cgtb_array_nbytes(cgtbObject* a);
cgtbObject* cgtb_tuple_new(int len);
int cgtb_tuple_len(cgtbObject* t);
cgtbObject* cgtb_tuple_get(cgtbObject* t, int i);               /* borrowed */
int cgtb_tuple_set(cgtbObject* t, int i, cgtbObject* o);        /* retains o */
int cgtb_object_kind(cgtbObject* o);                            /* 1 array, 2 tuple */
void cgtb_retain(cgtbObject* o);
void cgtb_release(cgtbObject* o);

/* ------------------------------------------------------------------------------------------------
 * Execution graph + interpreter. Replaces the instruction constructors and create_interpreter of
 * include/execution.h:47-162 and the marshalling in src/cycgt.pyx:338-369, 404-434.
 * A memory location is (index, devtype). Callables have the reference signatures
 *   byref: void f(void* closure, cgtObject** reads, cgtObject* write)   (cgt_common.h:176)
 *   byval: cgtObject* f(void* closure, cgtObject** reads)               (cgt_common.h:177)
 * ---------------------------------------------------------------------------------------------- */
#define CGTB_INSTR_QUICK 1        /* host bookkeeping only: never touches array data */
#define CGTB_INSTR_TRANSPORT 2    /* cross-device copy: runs outside captured CUDA graphs */
#define CGTB_INSTR_NOCAPTURE 4    /* must not be stream-captured (e.g. a Python callback) */
#define CGTB_INSTR_ONCE 8         /* inputs are compile-time constants: fire on the first run only */

cgtbGraph* cgtb_graph_new(long n_args, long n_locs);
void cgtb_graph_free(cgtbGraph* g);
int cgtb_graph_add_load_argument(cgtbGraph* g, const char* repr, int arg_index, long wloc, int wdev);
int cgtb_graph_add_alloc(cgtbGraph* g, const char* repr, int dtype, int n_shape, const long* shape_locs, long wloc, int wdev);
int cgtb_graph_add_build_tup(cgtbGraph* g, const char* repr, int n, const long* read_locs, long wloc, int wdev);
int cgtb_graph_add_return_byref(cgtbGraph* g, const char* repr, int n, const long* read_locs, const int* read_devs,
                                long wloc, int wdev, void* fptr, void* closure, int flags);
int cgtb_graph_add_return_byval(cgtbGraph* g, const char* repr, int n, const long* read_locs, const int* read_devs,
                                long wloc, int wdev, void* fptr, void* closure, int flags);

#define CGTB_INTERP_CUDA_GRAPHS 1 /* capture steady-state device segments into CUDA graphs and replay them */
#define CGTB_INTERP_PROFILE 2     /* time every instruction with CUDA events (per-Op table) */
cgtbInterp* cgtb_interp_new(cgtbGraph* g, int n_out, const long* out_locs, int flags);
void cgtb_interp_free(cgtbInterp* it);
/* args: tuple of arrays (host or device). *out: new reference to a tuple of the output objects.
 * Returns after the runtime stream has been synchronised, so host outputs are readable. */
int cgtb_interp_run(cgtbInterp* it, cgtbObject* args, cgtbObject** out);
/* counters: [0] runs, [1] kernels launched by instructions in the last run, [2] graph launches in the
 * last run, [3] segments captured so far, [4] kernels inside captured graphs, [5] device instructions in the graph,
 * [6] host nanoseconds of the last run up to its final wait for the stream, [7] steady runs so far (runs that
 * repeated the arguments' buffers and shapes of the run before and skipped the host bookkeeping) */
int cgtb_interp_stats(cgtbInterp* it, long* counters, int n);
/* Tell every interpreter that a shared variable's array was replaced (not merely overwritten): the next run of each
 * does its host bookkeeping in full. */
void cgtb_state_version_bump(void);
/* fn(ctx) is called in every cgtb_interp_run after the run's device work has been queued and before the run waits
 * for it: the place for host work that should overlap the step (queueing the next batch's upload). NULL removes it. */
int cgtb_interp_set_before_sync(cgtbInterp* it, void (*fn)(void*), void* ctx);
/* per-instruction accumulated milliseconds when CGTB_INTERP_PROFILE is set; returns n_instrs */
int cgtb_interp_profile(cgtbInterp* it, double* ms, long* counts, int cap);
const char* cgtb_interp_instr_repr(cgtbInterp* it, int i);
/* call one callable directly (reference: cycgt.apply_byref, src/cycgt.pyx:439-449) */
int cgtb_apply_byref(void* fptr, void* closure, int n, cgtbObject** reads, cgtbObject* write);

/* ------------------------------------------------------------------------------------------------
 * Kernels with plain device pointers. All arrays are C-contiguous; all launches go to the runtime
 * stream. dtype arguments are numpy type numbers (cgtbDtype).
 * ---------------------------------------------------------------------------------------------- */
/* Mul22: C[M,N] = op(A) op(B), alpha 1, beta 0, row-major; lda/ldb/ldc are stored row lengths.
 * Replaces cblas_sgemm / cublasSgemm_v2 in cgt/core.py:2195-2222. 3xTF32 split on tcgen05 tensor
 * cores where the shape allows, fp32 FMA kernels otherwise and for products too small to repay the tensor-core
 * kernels' fixed cost. impl: 0 auto, 1 generic FMA kernel, 2 any tensor-core kernel, 3 register-fed tensor-core kernel,
 * 4 TMA-fed tensor-core kernel, 5 one warp per output (few outputs), 6 16 x 16 FMA tiles (M*N*K <= 2^25); a forced
 * choice that does not accept the shape fails. */
int cgtb_sgemm(int tA, int tB, long M, long N, long K, const float* A, long lda, const float* B, long ldb,
               float* C, long ldc, int impl);
/* BatchedMul22 (cgt/core.py:2272-2286): P independent products, operands strideX apart */
int cgtb_sgemm_batched(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA,
                       const float* B, long ldb, long strideB, float* C, long ldc, long strideC, int impl);

/* C = (addend + addend_bias) + (op(A).op(B) + bias): a product with the additions that follow it in an affine layer fed by
 * two inputs, z = (x.W + b) + (h.U + c) (cgt/nn.py Affine applied twice and added, as the reference's recurrent demos
 * do), in the product's output stage. bias, addend_bias: [N] rows; addend: [M, N] with row pitch ldd; each may be null
 * (addend_bias only with addend). The additions are plain float32 additions in exactly this association, so the result
 * has the bits of cgtb_sgemm followed by the three additions. Only products that cgtb_sgemm gives to its FMA-tile
 * kernel (M*N > 2048, M*N*K <= 2^25, not A.B^T); others are refused. */
int cgtb_sgemm_bias_add(int tA, int tB, long M, long N, long K, const float* A, long lda, const float* B, long ldb,
                        const float* bias, const float* addend, long ldd, const float* addend_bias, float* C, long ldc);
int cgtb_dgemm(int tA, int tB, long M, long N, long K, const double* A, long lda, const double* B, long ldb,
               double* C, long ldc);

/* Im2Col / Col2Im (include/im2col.h:6-50, cgt/nn_ops/im2col.py:47-92); col is [B,Ho,Wo,C*kh*kw] */
int cgtb_im2col(int dtype, const void* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                int sw, void* col);
/* The same with column rows ldcol >= C*kh*kw entries apart; entries beyond C*kh*kw are written as zeros. A pitch
 * that is a multiple of 4 puts every row of a float32 column matrix on a 16-byte boundary, which the TMA-fed GEMM
 * needs (a 3-channel 5x5 convolution has rows of 75 entries). */
int cgtb_im2col_ld(int dtype, const void* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                   int sw, long ldcol, void* col);
int cgtb_col2im(int dtype, const void* col, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                int sw, void* im);

/* MaxPool / MaxPoolPullback (include/pooling.h:24-104); mask is int32 h*W+w within the plane */
int cgtb_max_pool(int dtype, const void* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                  int sw, int PH, int PW, void* top, int32_t* mask);
int cgtb_max_pool_pullback(int dtype, const int32_t* mask, const void* gtop, long B, int C, int PH, int PW, int H,
                           int W, int kh, int kw, int ph, int pw, int sh, int sw, void* gx);

/* CrossChannelLRN forward/backward (include/lrn.cuh:3-114, cgt/nn_ops/cross_channel_lrn.py:27-37,78-82) */
int cgtb_lrn_forward(int dtype, const void* x, long N, int C, int H, int W, int size, double alpha, double beta,
                     void* top, void* scale);
int cgtb_lrn_backward(int dtype, const void* x, const void* top, const void* scale, const void* gtop, long N, int C,
                      int H, int W, int size, double alpha, double beta, void* gx);

/* Data gradient of a stride-1 convolution in one kernel. Replaces the pair Mul22(dy, W) + Col2Im that the
 * reference's graph holds for it (cgt/nn_ops/im2col.py:Im2Col.pullback, include/im2col.h:30-50): no column
 * matrix is written or read.
 *   dx[b, c, y, x] = sum_{i, j, co} dy[b, y + ph - i, x + pw - j, co] * w_rearranged[c][(i*kw + j)*Cin + co]
 * dy_nhwc [B, Ho, Wo, Cin]; w_rearranged [C][kh*kw*Cin] (the filter bank [Cin, C, kh, kw] transposed to
 * [C, kh, kw, Cin]); dx_nchw [B, C, H, W]. float32, 3xTF32 tensor-core arithmetic like cgtb_sgemm.
 * Supported: Cin a multiple of 32, C a multiple of 16 and at most 128, W at most 128, 16-byte-aligned operands. */
int cgtb_conv_dgrad(const float* dy_nhwc, long B, int Ho, int Wo, int Cin, const float* w_rearranged, int C, int H, int W,
                    int kh, int kw, int ph, int pw, float* dx_nchw);

/* Forward pass of a stride-1 convolution layer in one kernel, without a column matrix: replaces Im2Col, Mul22,
 * Reshape, Transpose{0,3,1,2}, Repeat, ElwiseBinary +, >=, * of cgt/nn.py:87-100, 44-45, 228-233 (include/im2col.h:6-28).
 *   t[b, n, y, x] = bias[n] + sum_{i, j, c} x[b, y + i - ph, x + j - pw, c] * w_rearranged[n][(i*kw + j)*Cin + c]
 *   mask = (t >= 0), y = t * mask
 * x_nhwc [B, H, W, Cin]; w_rearranged [Cout][kh*kw*Cin] (the filter bank [Cout, Cin, kh, kw] transposed to
 * [Cout, kh, kw, Cin]); y_nchw, mask_nchw [B, Cout, Ho, Wo] with Ho = H + 2 ph - kh + 1. float32, 3xTF32 like cgtb_sgemm;
 * the sum runs over (tap, channel) instead of (channel, tap), so values agree with cgtb_conv_bias_relu to float32
 * rounding, not bit for bit. Supported: Cin a multiple of 32, Cout a multiple of 16 (of 128 above 128), Wo <= 128. */
int cgtb_conv_fwd_bias_relu(const float* x_nhwc, long B, int H, int W, int Cin, const float* w_rearranged, int Cout, int Ho,
                            int Wo, int kh, int kw, int ph, int pw, const float* bias, float* y_nchw, int8_t* mask_nchw);
/* The same with the filter bank as the layer stores it, w_bank [Cout, Cin, kh, kw]: the rearrangement is part of the
 * call's filter-splitting kernel, no transposed copy is needed. */
int cgtb_conv_fwd_bias_relu_bank(const float* x_nhwc, long B, int H, int W, int Cin, const float* w_bank, int Cout, int Ho,
                                 int Wo, int kh, int kw, int ph, int pw, const float* bias, float* y_nchw, int8_t* mask_nchw);
/* Filter gradient of a stride-1 convolution in one kernel (plus an ordered fold of its K splits), without a column
 * matrix: replaces Mul22{T,N}(dy, Im2Col(x)) of the differentiated cgt/nn.py:93-100 (cgt/core.py:2162-2175).
 *   dw[n][c][i][j] = sum_{b, y, x} dy[b, y, x, n] * x[b, y + i - ph, x + j - pw, c]
 * x_nhwc [B, H, W, Cin]; dy_nhwc [B, Ho, Wo, Cout]; dw [Cout][Cin*kh*kw]. float32, 3xTF32.
 * Supported: Cin a multiple of 32, Cout a multiple of 16 (of 128 above 128), Wo <= 32. */
int cgtb_conv_wgrad(const float* x_nhwc, long B, int H, int W, int Cin, const float* dy_nhwc, int Ho, int Wo, int Cout, int kh,
                    int kw, int ph, int pw, float* dw);

/* cgtb_conv_dgrad with the filter bank as the layer stores it, w_bank [Cin, C, kh, kw] (Cin = channels of dy). */
int cgtb_conv_dgrad_bank(const float* dy_nhwc, long B, int Ho, int Wo, int Cin, const float* w_bank, int C, int H, int W,
                         int kh, int kw, int ph, int pw, float* dx_nchw);

/* The filter splitting of the two calls above as a step of its own, for all layers at once. The convolution kernels
 * take their filters as K-major [w_hi | w_lo] (3xTF32 operands; K runs over (tap, source channel)); cgtb_conv_fwd_bias_relu_bank and
 * cgtb_conv_dgrad_bank make that copy in a small kernel of their own on every call. The filters change only when the
 * parameters are updated, so a training step can make all copies in ONE launch before its first convolution:
 * job j reads banks[j] ([n_out, n_src, taps] for layout 1, the forward product; [n_src, n_out, taps] for layout 2, the
 * data gradient) and writes out[j], float32 [2][n_out][taps * n_src], 16-byte aligned. At most 8 jobs.
 * cgtb_conv_fwd_bias_relu_pre / cgtb_conv_dgrad_pre are the two calls with such a copy passed in (w_split; the bank is
 * still passed and is used when the extents send the call to the kernel that converts in its loop). Same bits. */
int cgtb_split_filter_banks(int njobs, const float* const* banks, const int* n_out, const int* n_src, const int* taps,
                            const int* layout, float* const* out);
int cgtb_conv_fwd_bias_relu_pre(const float* x_nhwc, long B, int H, int W, int Cin, const float* w_bank, const float* w_split, int Cout,
                                int Ho, int Wo, int kh, int kw, int ph, int pw, const float* bias, float* y_nchw, int8_t* mask_nchw);
int cgtb_conv_dgrad_pre(const float* dy_nhwc, long B, int Ho, int Wo, int Cin, const float* w_bank, const float* w_split, int C, int H,
                        int W, int kh, int kw, int ph, int pw, float* dx_nchw);

/* Output stage of a convolution layer in one call: Mul22(col, w^T) -> NCHW -> + bias -> relu with its mask.
 * Replaces the Op sequence Mul22, Reshape, Transpose{0,3,1,2}, Repeat, ElwiseBinary +, >=, * of cgt/nn.py:87-100,
 * 44-45, 228-233; values are bit-identical to that sequence run through cgtb_sgemm and the elementwise kernels.
 * col [M, K] (M = B*HW rows, channels-last pixels), w [C, K], bias [C]; y_nchw, mask_nchw [B, C, HW]. float32. */
int cgtb_conv_bias_relu(const float* col, long M, long K, const float* w, int C, const float* bias, long HW, float* y_nchw,
                        int8_t* mask_nchw);
/* The same for a column matrix whose rows are ldcol >= K entries apart (cgtb_im2col_ld); w stays [C, K]. */
int cgtb_conv_bias_relu_ld(const float* col, long M, long K, long ldcol, const float* w, int C, const float* bias, long HW,
                           float* y_nchw, int8_t* mask_nchw);

/* Input stage of a convolution layer's backward pass in one call: gt = transpose(mask * g) to channels-last and
 * bias_grad[c] = sum over images and pixels of mask * g. Replaces ElwiseBinary *, Transpose{0,2,3,1} and Sum{0,2,3}
 * of the differentiated cgt/nn.py:44-45, 87-100, 228-233. mask_nchw (int8), g_nchw [B, C, HW]; gt_nhwc [B, HW, C];
 * bias_grad [C]. gt has the bits of the Op sequence; bias_grad is summed in a different (fixed) order. */
int cgtb_relu_grad_nhwc(const int8_t* mask_nchw, const float* g_nchw, long B, int C, long HW, float* gt_nhwc, float* bias_grad);

/* ElwiseUnary / ElwiseBinary (cgt/core.py:1160-1378). scalar_x / scalar_y: operand is a 0-d array
 * in device memory, read at index 0. */
int cgtb_unary(int op, int dt_in, int dt_out, long n, const void* in, void* out);
int cgtb_binary(int op, int dt_x, int dt_y, int dt_out, long n, const void* x, const void* y, void* out,
                int scalar_x, int scalar_y);

/* A chain of ElwiseUnary / ElwiseBinary Ops over one index space evaluated by ONE kernel (no counterpart
 * in the reference, which launches one generated loop per Op; cgt/core.py:1160-1378 define the Ops).
 * Values are float32 or 0/1 truth values; every operation is carried out exactly as the separate
 * kernels of cgtb_unary / cgtb_binary do it, so the results have the same bits.
 * Registers 0 .. n_in-1 hold the inputs, register n_in+j the result of operation j. */
#define CGTB_FUSED_MAX_IN 16
#define CGTB_FUSED_MAX_OPS 32
#define CGTB_FUSED_MAX_OUT 12
enum { CGTB_FIN_F4 = 0, CGTB_FIN_I1 = 1, CGTB_FIN_SCALAR_F4 = 2, CGTB_FIN_SCALAR_I8 = 3, CGTB_FIN_BCAST_F4 = 4,
       CGTB_FIN_VIEW_F4 = 7 /* columns of a wider float32 matrix, see cgtb_fused_elwise; 5 and 6 belong to cgtbRowProgram */ };
typedef struct {
  int n_in, n_ops, n_out;
  int in_kind[CGTB_FUSED_MAX_IN];    /* CGTB_FIN_*; a scalar is a 0-d array in device memory */
  int op_arity[CGTB_FUSED_MAX_OPS];  /* 1: CGTB_U_* opcode, 2: CGTB_B_* opcode */
  int op_code[CGTB_FUSED_MAX_OPS];
  int op_a[CGTB_FUSED_MAX_OPS], op_b[CGTB_FUSED_MAX_OPS];
  int out_reg[CGTB_FUSED_MAX_OUT];
  int out_dtype[CGTB_FUSED_MAX_OUT]; /* cgtb_f4 or cgtb_i1 */
  /* NULL: the library's register-machine kernel runs the program. Otherwise the launcher of a kernel
   * generated for this program: int f(long n, const void* const* in, const long* bcast_k,
   * const long* bcast_inner, void* const* out, int vectorised, void* stream, int sm_count), 0 on success. */
  void* launcher;
  long view_width;                   /* row length of the index space; read only when an input is a CGTB_FIN_VIEW_F4 */
} cgtbFusedProgram;
/* in[k]: device pointer of input k. A CGTB_FIN_BCAST_F4 input holds bcast_k[k] values; element i of the
 * index space reads value (i / bcast_inner[k]) % bcast_k[k] (a bias [1,C,1,1] over [B,C,H,W]: k = C,
 * inner = H*W). A CGTB_FIN_VIEW_F4 input is a row-major matrix with rows of bcast_k[k] elements, of which columns
 * [bcast_inner[k], bcast_inner[k] + view_width) are read: element i of the [n / view_width, view_width] index space
 * reads in[k][(i / view_width) * bcast_k[k] + bcast_inner[k] + i % view_width] (a column slice of a matrix, GetSli
 * along axis 1 in cgt/core.py:1767-1812, consumed without a copy). out[q]: device pointer of output q, n elements each. */
int cgtb_fused_elwise(const cgtbFusedProgram* prog, long n, const void* const* in, const long* bcast_k,
                      const long* bcast_inner, void* const* out);

/* The same program over several independent tensors in one launch (the parameter updates of a training step): one
 * float32 output per tensor, at most 4 inputs, each a float32 tensor of the output's size or a scalar; `in` holds
 * ntensors * prog->n_in device pointers, tensor-major. Same bits as cgtb_fused_elwise per tensor. No counterpart in
 * the reference. */
int cgtb_fused_elwise_multi(const cgtbFusedProgram* prog, int ntensors, const long* n, const void* const* in, void* const* out);

/* A chain of elementwise operations and row sums over the rows of an [R, C] matrix, C <= 128, in one launch (a softmax,
 * its logarithm and its pullback are such chains): one warp per row, values in registers, a row sum by warp shuffles.
 * Registers hold either one value per element of the row or one value per row; in_kind: CGTB_FIN_F4 an [R, C] array,
 * CGTB_FIN_COL an [R] array (one value per row), CGTB_FIN_ROW a [C] array (the same for every row), a scalar, or
 * CGTB_FIN_ROWHOT an int64 [R] array of column numbers: the register holds 1 in column in[row] of the row and 0 elsewhere
 * (the matrix that cgtb_onehot_rows writes, never formed).
 * op_arity 1 / 2 as in cgtbFusedProgram; op_arity 3: the sum of register op_a over the row (kept in every lane).
 * out_col[j] != 0: output j has one value per row ([R]), else [R, C]. The sum order differs from cgtb_reduce: results
 * agree with the separate launches to rounding, not bit for bit. No counterpart in the reference. */
enum { CGTB_FIN_COL = 5, CGTB_FIN_ROW = 6, CGTB_FIN_ROWHOT = 8 };
typedef struct {
  int n_in, n_ops, n_out;
  int in_kind[CGTB_FUSED_MAX_IN];
  int op_arity[CGTB_FUSED_MAX_OPS];
  int op_code[CGTB_FUSED_MAX_OPS];
  int op_a[CGTB_FUSED_MAX_OPS], op_b[CGTB_FUSED_MAX_OPS];
  int out_reg[CGTB_FUSED_MAX_OUT];
  int out_col[CGTB_FUSED_MAX_OUT];
  /* NULL: the library's register-machine kernel runs the program. Otherwise the launcher of a kernel generated for
   * this program: int f(long R, long C, const void* const* in, void* const* out, void* stream), 0 on success. */
  void* launcher;
} cgtbRowProgram;
int cgtb_fused_rows(const cgtbRowProgram* prog, long R, long C, const void* const* in, void* const* out);

/* out[r][c] = (c == idx[r]) ? 1 : 0, float32 [R, C]; idx int64 [R]. The selection matrix behind x[arange(R), idx]
 * (GetFlatIndices, cgt/core.py:1781-1812) and its gradient (IncFlatIndices on zeros, cgt/core.py:1814-1860) on the rows of
 * an [R, C] matrix: x[r, idx[r]] = sum_c x[r][c] * out[r][c]. A row whose index is outside [0, C) is all zeros. */
int cgtb_onehot_rows(const long* idx, long R, long C, float* out);
/* out[r] = sum over c of x[r][c] where m[r][c] != 0 (float32 [R, C] -> [R]); lane c % 32 adds its elements in order, the
 * lanes are folded by xor shuffles. With m = cgtb_onehot_rows(idx) this is x[r][idx[r]] exactly: selected, not
 * multiplied, so an infinite element outside the selection does not reach the result. */
int cgtb_masked_row_sum(const float* x, const float* m, long R, long C, float* out);

/* out[R, C] = zeros with k float32 pieces placed side by side: piece j ([R, width[j]]) occupies columns
 * [offset[j], offset[j] + width[j]); the pieces do not overlap. What a sum of IncSli(zeros, ...) over disjoint column
 * ranges computes (the gradient of several GetSli of one matrix, cgt/core.py:1767-1861), in one launch and without
 * the zero fills. k <= 8. */
int cgtb_scatter_cols(long R, long C, int k, const long* offset, const long* width, const void* const* pieces, void* out);

/* A stride-1 "same" convolution layer on very few input channels (the first layer of an image network: 3 channels,
 * 5 x 5 filters, 32 filters, images 32 pixels wide), forward with bias + relu + mask and filter gradient, computed
 * directly from the NCHW image with FMA tiles: no column matrix (the reference forms Im2Col then Mul22,
 * cgt/nn.py:93-100, include/im2col.h:6-28; with 3 input channels the column matrix is 25 times the image and the
 * product has only 75 terms per output). x [B, Cin, H, W]; w [Cout][Cin*kh*kw] (the bank as stored); y / mask NCHW
 * [B, Cout, H, W]; dy channels-last [B, H, W, Cout]; dw [Cout][Cin*kh*kw]. Supported: Cin 3, kh = kw = 5, ph = pw = 2,
 * Cout 32, W 32, H a multiple of 8; anything else is refused (use cgtb_im2col + cgtb_conv_bias_relu / cgtb_sgemm).
 * Sums run in float32 FMA order (tap by tap), not in the GEMM's: float32 tolerance against the column-matrix path. */
int cgtb_conv_direct_fwd_bias_relu(const float* x_nchw, long B, int Cin, int H, int W, const float* w, int Cout, int kh, int kw, int ph,
                                   int pw, const float* bias, float* y_nchw, signed char* mask_nchw);
int cgtb_conv_direct_wgrad(const float* x_nchw, long B, int Cin, int H, int W, const float* dy_nhwc, int Cout, int kh, int kw, int ph,
                           int pw, float* dw);
/* The same filter gradient taken straight from the layer's backward inputs: dy = mask * g with the relu's NCHW mask
 * (int8 0/1) and the NCHW gradient g of the relu output (the reference's ElwiseBinary multiply, cgt/nn.py:44-45
 * differentiated), formed while the kernel stages its tile; dbias[Cout] = sum of dy over batch and pixels (the
 * reference's Sum{0,2,3}). Neither dy nor its channels-last copy is written. */
int cgtb_conv_direct_wgrad_relu(const float* x_nchw, long B, int Cin, int H, int W, const signed char* mask_nchw, const float* g_nchw,
                                int Cout, int kh, int kw, int ph, int pw, float* dw, float* dbias);

/* Sum / Max over a set of axes, keepdims (cgt/core.py:1663-1738) */
int cgtb_reduce(int kind, int dtype, int ndim, const long* shape, const int* reduced, const void* in, void* out);

/* No counterpart in the reference. Sum (kind 0) or Max (kind 1) of a float32 array viewed as
 * [R0, K, R1] over R0 and R1, out[K], for callers that must not allocate device or host memory at call
 * time (latency-critical callbacks, processes whose device memory belongs to another allocator).
 * Same bits as cgtb_reduce on that layout (R1 > 1; a pure column reduction, R1 == 1 with R0 > 1, is refused: it
 * is not split and needs no scratch, use cgtb_reduce). The partial results live in one fixed 128 KiB array in
 * device memory that every call shares: the first call per device looks its address up (set-up work,
 * do it before any stream capture); calls that overlap in time race on the array, calls issued in
 * sequence on the runtime stream do not; nothing in the array has to be cleared between calls.
 * Refused with an error: K > CGTB_REDUCE_STATIC_MAX_K, R0 or R1 >= 2^30, R1 == 1 with R0 > 1. */
#define CGTB_REDUCE_STATIC_MAX_K 8192
int cgtb_reduce_rkr_f32_static(int kind, long R0, long K, long R1, const float* in, float* out);
long cgtb_reduce_static_max_k(void);

/* Repeat, Transpose, GetSli, IncSli, GetFlatIndices, IncFlatIndices, Concatenate, Fill
 * (cgt/core.py:1511-1594, 1767-1861, 1960-2023, 1467-1509, 966-1007) */
int cgtb_repeat(int dtype, int ndim, const long* out_shape, const int* repeated, const void* in, void* out);
int cgtb_transpose(int dtype, int ndim, const long* in_shape, const int* axes, const void* in, void* out);
int cgtb_getsli(int dtype, long outer, long n_in, long inner, long start, long step, long n_out, const void* in,
                void* out);
int cgtb_incsli(int dtype, long outer, long n_x, long inner, long start, long step, long n_inc, const void* x,
                const void* inc, void* out);
int cgtb_getflat(int dtype, long n, const void* x, const int64_t* k, void* out);
int cgtb_incflat(int dtype, long xsize, long n, const void* x, const int64_t* k, const void* p, void* out);
int cgtb_concat_part(int dtype, long outer, long n_in, long n_out, long inner, long pos, const void* in, void* out);
/* Concatenate along axis 0 in ONE launch: n <= 64 contiguous pieces of bytes[i] bytes are copied back to back into out
 * (np.concatenate of C-contiguous arrays along their first axis, cgt/core.py:1467-1509). */
int cgtb_concat_rows(int n, const void* const* pieces, const long* bytes, void* out);
int cgtb_fill(int dtype, long n, double fvalue, long ivalue, void* out);

/* ------------------------------------------------------------------------------------------------
 * Data-parallel gradient exchange (no counterpart in the reference, which has no collectives).
 * One process per GPU. NCCL is opened at run time from `nccl_path`; rank 0 creates the 128-byte id and
 * the host side distributes it before every rank calls cgtb_comm_init.
 * ---------------------------------------------------------------------------------------------- */
int cgtb_comm_load(const char* nccl_path);
int cgtb_comm_unique_id(char* out128);
int cgtb_comm_init(const char* id128, int rank, int world);
int cgtb_comm_world(void);
int cgtb_comm_rank(void);
int cgtb_comm_check(void);   /* non-zero when NCCL reported an asynchronous error */
int cgtb_comm_abort(void);
int cgtb_comm_destroy(void);
/* out[i] = sum over ranks of in[i] for n float buffers, one NCCL group on the runtime stream */
int cgtb_allreduce_sum(int dtype, int n, const void* const* in, void* const* out, const long* counts);

/* The same exchange for small float32 payloads as ONE kernel over peer memory (no library collective, so the call is
 * an ordinary launch that a CUDA graph can hold). Every rank: cgtb_peer_alloc (its symmetric buffer: two data and two result slots of
 * slot_bytes; returns the 64-byte cudaIpc handle), the host side gathers the handles of all ranks, cgtb_peer_open maps
 * them (ranks on one node, at most 8). cgtb_peer_allreduce_sum: out[i] = sum over ranks of in[i], summed in rank order on
 * every rank (replicas stay bit-identical). The kernel's waits for the other ranks are bounded by a cycle budget
 * (cgtb_peer_set_wait_cycles, default about a second): on expiry the call's result is invalid, the failure is
 * reported by the next cgtb_synchronize / cgtb_interp_run, and the library stays usable.
 * In a slot the tensors lie back to back, each starting at a multiple of four elements (the payload that fits is the
 * sum of the tensors' sizes, each rounded up to 16 bytes).
 * cgtb_peer_selftest_*: a two-rank group inside one process whose second rank never arrives (post() plays it for the
 * next call, with a payload in the slot's layout), for testing the bounded wait on one GPU without faulting or
 * hanging anything. */
int cgtb_peer_alloc(long slot_bytes, char* handle64);
int cgtb_peer_open(const char* handles, int rank, int world);
int cgtb_peer_close(void);
int cgtb_peer_world(void);
long cgtb_peer_slot_bytes(void);
int cgtb_peer_set_wait_cycles(long cycles);
/* payloads of more than `bytes` (default one megabyte; 0: every payload) take the two-phase kernel: every rank sums one
 * slice of the elements over all ranks into its result slot, then all ranks collect the slices; each element crosses
 * the links twice whatever the number of ranks instead of once per peer */
int cgtb_peer_set_two_phase_bytes(long bytes);
/* out3: calls so far, nanoseconds spent until every rank's flag was seen, nanoseconds start to end (block 0's clock,
 * summed over the calls): tells waiting for slower ranks from the exchange itself */
int cgtb_peer_timing(long* out3);
int cgtb_peer_allreduce_sum(int n, const void* const* in, void* const* out, const long* counts);
int cgtb_peer_selftest_open(long slot_bytes);
int cgtb_peer_selftest_post(const float* host_payload, long count);

#ifdef __cplusplus
}
#endif
#endif
