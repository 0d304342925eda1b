// Elementwise unary/binary, reductions and data-movement kernels for sm_100a.
//
// Elementwise kernels process 16 bytes of the widest operand per thread per step (128-bit loads and
// stores where the type allows); the operator is a kernel argument that every thread of the launch
// agrees on, so the switch costs one uniform branch. The scalar expressions are the reference's C
// expressions (cgt/core.py:1119-1133, 1141-1151) evaluated with the same promotions: math functions
// in the input type, sub-expressions with a double literal in double, result narrowed to the output type.
#include "runtime.h"
#include "reduce_rkr.h"
#include "cgt_elwise.h"
#include <cfloat>
#include <limits>

using namespace cgtb;

constexpr int kVec = 4;

template <typename TI, typename TO>
__global__ void unary_kernel(int op, long n, const TI* __restrict__ in, TO* __restrict__ out, bool aligned) {
  const long nvec = aligned ? n / kVec : 0;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    Pack<TI, kVec> a = load_pack<TI, kVec>(in + i * kVec);
    Pack<TO, kVec> r;
#pragma unroll
    for (int k = 0; k < kVec; ++k) r.v[k] = unary_apply<TI, TO>(op, a.v[k]);
    store_pack<TO, kVec>(out + i * kVec, r);
  }
  for (long i = nvec * kVec + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    out[i] = unary_apply<TI, TO>(op, in[i]);
}

// SX / SY: operand is a 0-d array read at index 0
template <typename TX, typename TY, typename TO, bool SX, bool SY>
__global__ void binary_kernel(int op, long n, const TX* __restrict__ x, const TY* __restrict__ y, TO* __restrict__ out,
                              bool aligned) {
  const long nvec = aligned ? n / kVec : 0;
  TX xs = SX ? x[0] : TX(0);
  TY ys = SY ? y[0] : TY(0);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    Pack<TX, kVec> a;
    Pack<TY, kVec> b;
    if (!SX) a = load_pack<TX, kVec>(x + i * kVec);
    if (!SY) b = load_pack<TY, kVec>(y + i * kVec);
    Pack<TO, kVec> r;
#pragma unroll
    for (int k = 0; k < kVec; ++k) r.v[k] = binary_apply<TX, TY, TO>(op, SX ? xs : a.v[k], SY ? ys : b.v[k]);
    store_pack<TO, kVec>(out + i * kVec, r);
  }
  for (long i = nvec * kVec + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    out[i] = binary_apply<TX, TY, TO>(op, SX ? xs : x[i], SY ? ys : y[i]);
}

static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

static inline unsigned elem_grid(long n) {
  long blocks = cgtb_ceil_div(cgtb_ceil_div(n, kVec), 256);
  long cap = (long)rt().sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

#define CGTB_FOR_DTYPE(code, T, ...)                           \
  switch (code) {                                              \
    case cgtb_i1: { typedef int8_t T; __VA_ARGS__; } break;    \
    case cgtb_i4: { typedef int32_t T; __VA_ARGS__; } break;   \
    case cgtb_i8: { typedef int64_t T; __VA_ARGS__; } break;   \
    case cgtb_f4: { typedef float T; __VA_ARGS__; } break;     \
    case cgtb_f8: { typedef double T; __VA_ARGS__; } break;    \
    default: return fail("unsupported dtype code %d", (int)(code)); \
  }

template <typename TI, typename TO>
static int unary_launch(int op, long n, const void* in, void* out) {
  bool al = aligned16(in) && aligned16(out);
  CGTB_LAUNCH((unary_kernel<TI, TO>), elem_grid(n), 256, 0, op, n, (const TI*)in, (TO*)out, al);
  return 0;
}

CGTB_API int cgtb_unary(int op, int dt_in, int dt_out, long n, const void* in, void* out) {
  if (!require_runtime("cgtb_unary")) return 1;
  if (op < 0 || op >= CGTB_U_COUNT) return fail("cgtb_unary: bad opcode %d", op);
  if (n <= 0) return 0;
  CGTB_FOR_DTYPE(dt_in, TI, CGTB_FOR_DTYPE(dt_out, TO, { int rc = unary_launch<TI, TO>(op, n, in, out); if (rc) return rc; }));
  CGTB_CHECK_LAUNCH("unary");
  return 0;
}

template <typename TX, typename TY, typename TO>
static int binary_launch(int op, long n, const void* x, const void* y, void* out, int sx, int sy) {
  bool al = aligned16(out) && (sx || aligned16(x)) && (sy || aligned16(y));
  unsigned g = elem_grid(n);
  if (sx && sy) return fail("cgtb_binary: both operands scalar; scalar-scalar arithmetic stays on the host");
  if (sx) CGTB_LAUNCH((binary_kernel<TX, TY, TO, true, false>), g, 256, 0, op, n, (const TX*)x, (const TY*)y, (TO*)out, al);
  else if (sy) CGTB_LAUNCH((binary_kernel<TX, TY, TO, false, true>), g, 256, 0, op, n, (const TX*)x, (const TY*)y, (TO*)out, al);
  else CGTB_LAUNCH((binary_kernel<TX, TY, TO, false, false>), g, 256, 0, op, n, (const TX*)x, (const TY*)y, (TO*)out, al);
  return 0;
}

// Output dtypes the typing rules can produce for a pair of inputs (cgt/core.py:1309-1322): the
// promoted type, the float type, or i1. Instantiating only these keeps the binary count small.
template <typename TX, typename TY>
static int binary_dispatch_out(int op, int dt_out, long n, const void* x, const void* y, void* out, int sx, int sy) {
  switch (dt_out) {
    case cgtb_i1: return binary_launch<TX, TY, int8_t>(op, n, x, y, out, sx, sy);
    case cgtb_i4: return binary_launch<TX, TY, int32_t>(op, n, x, y, out, sx, sy);
    case cgtb_i8: return binary_launch<TX, TY, int64_t>(op, n, x, y, out, sx, sy);
    case cgtb_f4: return binary_launch<TX, TY, float>(op, n, x, y, out, sx, sy);
    case cgtb_f8: return binary_launch<TX, TY, double>(op, n, x, y, out, sx, sy);
  }
  return fail("cgtb_binary: unsupported output dtype %d", dt_out);
}

CGTB_API int cgtb_binary(int op, int dt_x, int dt_y, int dt_out, long n, const void* x, const void* y, void* out,
                         int scalar_x, int scalar_y) {
  if (!require_runtime("cgtb_binary")) return 1;
  if (op < 0 || op >= CGTB_B_COUNT) return fail("cgtb_binary: bad opcode %d", op);
  if (n <= 0) return 0;
  CGTB_FOR_DTYPE(dt_x, TX, CGTB_FOR_DTYPE(dt_y, TY, {
    int rc = binary_dispatch_out<TX, TY>(op, dt_out, n, x, y, out, scalar_x, scalar_y);
    if (rc) return rc;
  }));
  CGTB_CHECK_LAUNCH("binary");
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Fused chains of elementwise Ops: a small register machine over float values. Each operation calls
// the same unary_apply / binary_apply instantiation that the separate kernels use for float operands
// (truth values are held as 0.f / 1.f, which is what the separate kernels' int8 -> float conversion
// yields), so a fused chain and the Op-by-Op sequence agree bit for bit. The register file is indexed
// with run-time operand numbers and therefore lives in local memory (L1); the chains are HBM-bound.
// ------------------------------------------------------------------------------------------------
struct FusedArgs {
  cgtbFusedProgram prog;
  const void* in[CGTB_FUSED_MAX_IN];
  long bk[CGTB_FUSED_MAX_IN], binner[CGTB_FUSED_MAX_IN];
  void* out[CGTB_FUSED_MAX_OUT];
  long n;
};

template <int V>
__global__ void fused_elwise_kernel(const FusedArgs a) {
  const cgtbFusedProgram& P = a.prog;
  const long nv = a.n / V;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    float r[CGTB_FUSED_MAX_IN + CGTB_FUSED_MAX_OPS][V];
    for (int k = 0; k < P.n_in; ++k) {
      switch (P.in_kind[k]) {
        case CGTB_FIN_F4: {
          Pack<float, V> p = load_pack<float, V>((const float*)a.in[k] + i * V);
#pragma unroll
          for (int v = 0; v < V; ++v) r[k][v] = p.v[v];
        } break;
        case CGTB_FIN_I1: {
          Pack<int8_t, V> p = load_pack<int8_t, V>((const int8_t*)a.in[k] + i * V);
#pragma unroll
          for (int v = 0; v < V; ++v) r[k][v] = (float)p.v[v];
        } break;
        case CGTB_FIN_SCALAR_F4: {
          const float s = *(const float*)a.in[k];
#pragma unroll
          for (int v = 0; v < V; ++v) r[k][v] = s;
        } break;
        case CGTB_FIN_SCALAR_I8: {
          const float s = (float)*(const long*)a.in[k];
#pragma unroll
          for (int v = 0; v < V; ++v) r[k][v] = s;
        } break;
        case CGTB_FIN_VIEW_F4: {  // columns [binner, binner + W) of a matrix with rows of bk elements
          const long W = P.view_width, row = (i * V) / W, col = i * V - row * W;
          Pack<float, V> p = load_pack<float, V>((const float*)a.in[k] + row * a.bk[k] + a.binner[k] + col);
#pragma unroll
          for (int v = 0; v < V; ++v) r[k][v] = p.v[v];
        } break;
        default: {  // broadcast: one value per pack when the run length is a multiple of V, else one index per element
          const float* src = (const float*)a.in[k];
          if (a.binner[k] % V == 0) {
            const float s = src[((i * V) / a.binner[k]) % a.bk[k]];
#pragma unroll
            for (int v = 0; v < V; ++v) r[k][v] = s;
          } else {
#pragma unroll
            for (int v = 0; v < V; ++v) r[k][v] = src[((i * V + v) / a.binner[k]) % a.bk[k]];
          }
        } break;
      }
    }
    for (int o = 0; o < P.n_ops; ++o) {
      const int dst = P.n_in + o, ra = P.op_a[o], code = P.op_code[o];
      if (P.op_arity[o] == 1) {
#pragma unroll
        for (int v = 0; v < V; ++v) r[dst][v] = unary_apply<float, float>(code, r[ra][v]);
      } else {
        const int rb = P.op_b[o];
#pragma unroll
        for (int v = 0; v < V; ++v) r[dst][v] = binary_apply<float, float, float>(code, r[ra][v], r[rb][v]);
      }
    }
    for (int q = 0; q < P.n_out; ++q) {
      const int src = P.out_reg[q];
      if (P.out_dtype[q] == cgtb_f4) {
        Pack<float, V> p;
#pragma unroll
        for (int v = 0; v < V; ++v) p.v[v] = r[src][v];
        store_pack<float, V>((float*)a.out[q] + i * V, p);
      } else {
        Pack<int8_t, V> p;
#pragma unroll
        for (int v = 0; v < V; ++v) p.v[v] = (int8_t)r[src][v];
        store_pack<int8_t, V>((int8_t*)a.out[q] + i * V, p);
      }
    }
  }
}

CGTB_API int cgtb_fused_elwise(const cgtbFusedProgram* prog, long n, const void* const* in, const long* bcast_k,
                               const long* bcast_inner, void* const* out) {
  if (!require_runtime("cgtb_fused_elwise")) return 1;
  if (!prog) return fail("cgtb_fused_elwise: null program");
  if (prog->n_in < 1 || prog->n_in > CGTB_FUSED_MAX_IN || prog->n_ops < 1 || prog->n_ops > CGTB_FUSED_MAX_OPS || prog->n_out < 1 ||
      prog->n_out > CGTB_FUSED_MAX_OUT)
    return fail("cgtb_fused_elwise: program of %d inputs, %d operations, %d outputs exceeds the limits", prog->n_in, prog->n_ops,
                prog->n_out);
  if (n <= 0) return 0;
  FusedArgs a;
  a.prog = *prog;
  a.n = n;
  bool vec = (n % kVec) == 0;
  for (int k = 0; k < prog->n_in; ++k) {
    a.in[k] = in[k];
    a.bk[k] = a.binner[k] = 1;
    const int kind = prog->in_kind[k];
    if ((kind < CGTB_FIN_F4 || kind > CGTB_FIN_BCAST_F4) && kind != CGTB_FIN_VIEW_F4) return fail("cgtb_fused_elwise: bad input kind %d", kind);
    if (kind == CGTB_FIN_F4) vec = vec && aligned16(in[k]);
    if (kind == CGTB_FIN_VIEW_F4) {
      const long W = prog->view_width;
      if (W <= 0 || n % W != 0 || !bcast_k || !bcast_inner || bcast_inner[k] < 0 || bcast_inner[k] + W > bcast_k[k])
        return fail("cgtb_fused_elwise: input %d is not a column range of width %ld inside its matrix", k, W);
      a.bk[k] = bcast_k[k];
      a.binner[k] = bcast_inner[k];
      vec = vec && aligned16(in[k]) && W % kVec == 0 && bcast_k[k] % kVec == 0 && bcast_inner[k] % kVec == 0;
    }
    if (kind == CGTB_FIN_I1) vec = vec && (((uintptr_t)in[k] & 3) == 0);
    if (kind == CGTB_FIN_BCAST_F4) {
      if (!bcast_k || !bcast_inner || bcast_k[k] <= 0 || bcast_inner[k] <= 0) return fail("cgtb_fused_elwise: bad broadcast extents");
      a.bk[k] = bcast_k[k];
      a.binner[k] = bcast_inner[k];
    }
  }
  for (int o = 0; o < prog->n_ops; ++o) {
    const int lim = prog->n_in + o;
    const bool un = prog->op_arity[o] == 1;
    if ((!un && prog->op_arity[o] != 2) || prog->op_a[o] < 0 || prog->op_a[o] >= lim || (!un && (prog->op_b[o] < 0 || prog->op_b[o] >= lim)))
      return fail("cgtb_fused_elwise: operation %d reads a register that is not defined yet", o);
    if (prog->op_code[o] < 0 || prog->op_code[o] >= (un ? (int)CGTB_U_COUNT : (int)CGTB_B_COUNT)) return fail("cgtb_fused_elwise: bad opcode");
  }
  for (int q = 0; q < prog->n_out; ++q) {
    a.out[q] = out[q];
    if (prog->out_reg[q] < 0 || prog->out_reg[q] >= prog->n_in + prog->n_ops) return fail("cgtb_fused_elwise: bad output register");
    if (prog->out_dtype[q] == cgtb_f4) vec = vec && aligned16(out[q]);
    else if (prog->out_dtype[q] == cgtb_i1) vec = vec && (((uintptr_t)out[q] & 3) == 0);
    else return fail("cgtb_fused_elwise: outputs are float32 or int8");
  }
  if (prog->launcher) {
    // a kernel generated for exactly this program (same scalar templates, operands in registers)
    typedef int (*Launcher)(long, const void* const*, const long*, const long*, void* const*, int, void*, int);
    if (((Launcher)prog->launcher)(n, a.in, a.bk, a.binner, a.out, vec ? 1 : 0, (void*)rt().stream, rt().sm_count))
      return fail("cgtb_fused_elwise: the generated kernel failed to launch");
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    return 0;
  }
  if (vec) CGTB_LAUNCH(fused_elwise_kernel<kVec>, elem_grid(n), 256, 0, a);
  else CGTB_LAUNCH(fused_elwise_kernel<1>, elem_grid(n * kVec), 256, 0, a);
  CGTB_CHECK_LAUNCH("fused_elwise");
  return 0;
}

// The same program applied to several independent tensors in ONE launch (blockIdx.y = tensor): the parameter
// updates of a training step are eight tiny tensors with one and the same chain (p - lr * g), and as separate
// launches each costs a few microseconds of launch and dependency latency, far more than its bytes. One output of
// float32, inputs that are float32 tensors of the output's size or scalars. Same scalar templates as the single-tensor
// kernel: same bits.
constexpr int kMultiMaxTensors = 24;
constexpr int kMultiMaxIn = 4;
struct FusedMultiArgs {
  cgtbFusedProgram prog;
  int ntensors;
  long n[kMultiMaxTensors];
  const void* in[kMultiMaxTensors][kMultiMaxIn];
  float* out[kMultiMaxTensors];
  unsigned char vec[kMultiMaxTensors];   // the tensor's arrays are 16-byte aligned: groups of four
};
// One element (V = 1) or one aligned group of four (V = 4) of tensor t
template <int V>
__device__ __forceinline__ void fused_multi_apply(const FusedMultiArgs& a, int t, long i) {
  const cgtbFusedProgram& P = a.prog;
  float r[kMultiMaxIn + CGTB_FUSED_MAX_OPS][V];
  for (int k = 0; k < P.n_in; ++k) {
    if (P.in_kind[k] == CGTB_FIN_F4) {
      if (V == 4) {
        const float4 v = ((const float4*)a.in[t][k])[i];
        r[k][0] = v.x; r[k][1 % V] = v.y; r[k][2 % V] = v.z; r[k][3 % V] = v.w;
      } else {
        r[k][0] = ((const float*)a.in[t][k])[i];
      }
    } else {
      const float v = P.in_kind[k] == CGTB_FIN_SCALAR_F4 ? *(const float*)a.in[t][k] : (float)*(const long*)a.in[t][k];
#pragma unroll
      for (int q = 0; q < V; ++q) r[k][q] = v;
    }
  }
  for (int o = 0; o < P.n_ops; ++o) {
    const int dst = P.n_in + o, ra = P.op_a[o], code = P.op_code[o];
    if (P.op_arity[o] == 1) {
#pragma unroll
      for (int q = 0; q < V; ++q) r[dst][q] = unary_apply<float, float>(code, r[ra][q]);
    } else {
      const int rb = P.op_b[o];
#pragma unroll
      for (int q = 0; q < V; ++q) r[dst][q] = binary_apply<float, float, float>(code, r[ra][q], r[rb][q]);
    }
  }
  const int ro = P.out_reg[0];
  if (V == 4) ((float4*)a.out[t])[i] = make_float4(r[ro][0], r[ro][1 % V], r[ro][2 % V], r[ro][3 % V]);
  else a.out[t][i] = r[ro][0];
}
// blockIdx.y = tensor. A tensor whose arrays are 16-byte aligned is walked in groups of four, its last n % 4 elements
// one by one; the others element by element.
__global__ void fused_elwise_multi_kernel(const FusedMultiArgs a) {
  const int t = blockIdx.y;
  const long n = a.n[t], stride = (long)gridDim.x * blockDim.x, i0 = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (a.vec[t]) {
    const long nv = n >> 2;
    for (long i = i0; i < nv; i += stride) fused_multi_apply<4>(a, t, i);
    for (long i = (nv << 2) + i0; i < n; i += stride) fused_multi_apply<1>(a, t, i);
  } else {
    for (long i = i0; i < n; i += stride) fused_multi_apply<1>(a, t, i);
  }
}

// in: ntensors * prog->n_in device pointers, tensor-major; n[t] elements and out[t] per tensor
CGTB_API int cgtb_fused_elwise_multi(const cgtbFusedProgram* prog, int ntensors, const long* n, const void* const* in, void* const* out) {
  if (!require_runtime("cgtb_fused_elwise_multi")) return 1;
  if (!prog || prog->n_in < 1 || prog->n_in > kMultiMaxIn || prog->n_ops < 1 || prog->n_ops > CGTB_FUSED_MAX_OPS || prog->n_out != 1 ||
      prog->out_dtype[0] != cgtb_f4)
    return fail("cgtb_fused_elwise_multi: one float32 output, at most %d inputs", kMultiMaxIn);
  if (ntensors < 1 || ntensors > kMultiMaxTensors) return fail("cgtb_fused_elwise_multi: between 1 and %d tensors", kMultiMaxTensors);
  for (int k = 0; k < prog->n_in; ++k)
    if (prog->in_kind[k] != CGTB_FIN_F4 && prog->in_kind[k] != CGTB_FIN_SCALAR_F4 && prog->in_kind[k] != CGTB_FIN_SCALAR_I8)
      return fail("cgtb_fused_elwise_multi: inputs must be float32 tensors or scalars");
  for (int o = 0; o < prog->n_ops; ++o) {
    const int lim = prog->n_in + o;
    const bool un = prog->op_arity[o] == 1;
    if ((!un && prog->op_arity[o] != 2) || prog->op_a[o] < 0 || prog->op_a[o] >= lim || (!un && (prog->op_b[o] < 0 || prog->op_b[o] >= lim)) ||
        prog->op_code[o] < 0 || prog->op_code[o] >= (un ? (int)CGTB_U_COUNT : (int)CGTB_B_COUNT))
      return fail("cgtb_fused_elwise_multi: malformed program");
  }
  if (prog->out_reg[0] < 0 || prog->out_reg[0] >= prog->n_in + prog->n_ops) return fail("cgtb_fused_elwise_multi: bad output register");
  FusedMultiArgs a;
  a.prog = *prog;
  a.ntensors = ntensors;
  long nmax = 0;
  for (int t = 0; t < ntensors; ++t) {
    a.n[t] = n[t] > 0 ? n[t] : 0;
    nmax = std::max(nmax, a.n[t]);
    a.out[t] = (float*)out[t];
    for (int k = 0; k < prog->n_in; ++k) a.in[t][k] = in[(size_t)t * prog->n_in + k];
  }
  if (nmax == 0) return 0;
  for (int t = 0; t < ntensors; ++t) {
    // groups of four only for large tensors: a small one is bound by the latency of one thread's chain of operations
    // (run from the register machine's local memory), which a group of four makes four times as long
    bool vec = ((uintptr_t)a.out[t] & 15) == 0 && a.n[t] >= (1L << 18);
    for (int k = 0; k < prog->n_in && vec; ++k)
      if (prog->in_kind[k] == CGTB_FIN_F4 && ((uintptr_t)a.in[t][k] & 15) != 0) vec = false;
    a.vec[t] = vec ? 1 : 0;
  }
  // the largest tensor sets the row of blocks; smaller tensors leave the tail of their row idle
  const long per_block = nmax >= (1L << 18) ? 1024 : 256;
  dim3 grid((unsigned)std::min<long>(cgtb_ceil_div(nmax, per_block), 2L * rt().sm_count), (unsigned)ntensors);
  CGTB_LAUNCH(fused_elwise_multi_kernel, grid, 256, 0, a);
  CGTB_CHECK_LAUNCH("fused_elwise_multi");
  return 0;
}

// Elementwise operations and row sums over the rows of an [R, C] matrix in one launch: one warp per row, element
// c of the row lives in lane c % 32, slot c / 32 (E slots per lane, C <= 32 E). A register holds a value per element or,
// after a row sum, the same value in every lane and slot; elementwise operations do not need to know which. Lanes
// beyond C compute on zeros and take part neither in sums nor in stores.
struct RowArgs {
  cgtbRowProgram prog;
  long R, C;
  const void* in[CGTB_FUSED_MAX_IN];
  void* out[CGTB_FUSED_MAX_OUT];
};
template <int E>
__global__ void fused_rows_kernel(const RowArgs a) {
  const cgtbRowProgram& P = a.prog;
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.R) return;
  const long C = a.C;
  float r[CGTB_FUSED_MAX_IN + CGTB_FUSED_MAX_OPS][E];
  for (int k = 0; k < P.n_in; ++k) {
    const int kind = P.in_kind[k];
    if (kind == CGTB_FIN_F4 || kind == CGTB_FIN_ROW) {
      const float* src = (const float*)a.in[k] + (kind == CGTB_FIN_F4 ? row * C : 0);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const long c = lane + 32 * e;
        r[k][e] = c < C ? src[c] : 0.0f;
      }
    } else if (kind == CGTB_FIN_ROWHOT) {
      const long hot = ((const long*)a.in[k])[row];
#pragma unroll
      for (int e = 0; e < E; ++e) r[k][e] = (lane + 32 * e == hot) ? 1.0f : 0.0f;
    } else {
      const float v = kind == CGTB_FIN_COL ? ((const float*)a.in[k])[row]
                                           : (kind == CGTB_FIN_SCALAR_F4 ? *(const float*)a.in[k] : (float)*(const long*)a.in[k]);
#pragma unroll
      for (int e = 0; e < E; ++e) r[k][e] = v;
    }
  }
  for (int o = 0; o < P.n_ops; ++o) {
    const int dst = P.n_in + o, ra = P.op_a[o], code = P.op_code[o], arity = P.op_arity[o];
    if (arity == 1) {
#pragma unroll
      for (int e = 0; e < E; ++e) r[dst][e] = unary_apply<float, float>(code, r[ra][e]);
    } else if (arity == 2) {
      const int rb = P.op_b[o];
#pragma unroll
      for (int e = 0; e < E; ++e) r[dst][e] = binary_apply<float, float, float>(code, r[ra][e], r[rb][e]);
    } else {
      float s = 0.0f;
      if (arity == 3) {
#pragma unroll
        for (int e = 0; e < E; ++e)
          if (lane + 32 * e < C) s += r[ra][e];
      } else {   // 4: the elements of a where b is not zero (no product: an infinite unselected element stays out)
        const int rb = P.op_b[o];
#pragma unroll
        for (int e = 0; e < E; ++e)
          if (lane + 32 * e < C && r[rb][e] != 0.0f) s += r[ra][e];
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
#pragma unroll
      for (int e = 0; e < E; ++e) r[dst][e] = s;
    }
  }
  for (int j = 0; j < P.n_out; ++j) {
    const int ro = P.out_reg[j];
    if (P.out_col[j]) {
      if (lane == 0) ((float*)a.out[j])[row] = r[ro][0];
    } else {
      float* dst = (float*)a.out[j] + row * C;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const long c = lane + 32 * e;
        if (c < C) dst[c] = r[ro][e];
      }
    }
  }
}

namespace {
__global__ void onehot_rows_kernel(const long* __restrict__ idx, long R, long C, float* __restrict__ out) {
  const long n = R * C;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = i / C;
    out[i] = (i - r * C == idx[r]) ? 1.0f : 0.0f;
  }
}
}  // namespace
namespace {
__global__ void masked_row_sum_kernel(const float* __restrict__ x, const float* __restrict__ m, long R, long C, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= R) return;
  float s = 0.0f;
  for (long c = lane; c < C; c += 32)
    if (m[row * C + c] != 0.0f) s += x[row * C + c];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
  if (lane == 0) out[row] = s;
}
}  // namespace
CGTB_API int cgtb_masked_row_sum(const float* x, const float* m, long R, long C, float* out) {
  if (!require_runtime("cgtb_masked_row_sum")) return 1;
  if (R < 0 || C < 1) return fail("cgtb_masked_row_sum: R >= 0 and C >= 1");
  if (R == 0) return 0;
  CGTB_LAUNCH(masked_row_sum_kernel, (unsigned)cgtb_ceil_div(R, 4), 128, 0, x, m, R, C, out);
  CGTB_CHECK_LAUNCH("masked_row_sum");
  return 0;
}
CGTB_API int cgtb_onehot_rows(const long* idx, long R, long C, float* out) {
  if (!require_runtime("cgtb_onehot_rows")) return 1;
  if (R < 0 || C < 1) return fail("cgtb_onehot_rows: R >= 0 and C >= 1");
  if (R == 0) return 0;
  const long blocks = std::min<long>(cgtb_ceil_div(R * C, 256), (long)rt().sm_count * 8);
  CGTB_LAUNCH(onehot_rows_kernel, (unsigned)blocks, 256, 0, idx, R, C, out);
  CGTB_CHECK_LAUNCH("onehot_rows");
  return 0;
}

CGTB_API int cgtb_fused_rows(const cgtbRowProgram* prog, long R, long C, const void* const* in, void* const* out) {
  if (!require_runtime("cgtb_fused_rows")) return 1;
  if (!prog || prog->n_in < 1 || prog->n_in > CGTB_FUSED_MAX_IN || prog->n_ops < 1 || prog->n_ops > CGTB_FUSED_MAX_OPS || prog->n_out < 1 ||
      prog->n_out > CGTB_FUSED_MAX_OUT)
    return fail("cgtb_fused_rows: program outside the limits");
  if (C < 1 || C > 128) return fail("cgtb_fused_rows: rows of 1 to 128 elements, got %ld", C);
  for (int k = 0; k < prog->n_in; ++k) {
    const int kind = prog->in_kind[k];
    if (kind != CGTB_FIN_F4 && kind != CGTB_FIN_SCALAR_F4 && kind != CGTB_FIN_SCALAR_I8 && kind != CGTB_FIN_COL && kind != CGTB_FIN_ROW &&
        kind != CGTB_FIN_ROWHOT)
      return fail("cgtb_fused_rows: unsupported input kind %d", kind);
  }
  for (int o = 0; o < prog->n_ops; ++o) {
    const int lim = prog->n_in + o, ar = prog->op_arity[o];
    if (ar < 1 || ar > 4 || prog->op_a[o] < 0 || prog->op_a[o] >= lim || ((ar == 2 || ar == 4) && (prog->op_b[o] < 0 || prog->op_b[o] >= lim)) ||
        (ar == 1 && (prog->op_code[o] < 0 || prog->op_code[o] >= (int)CGTB_U_COUNT)) ||
        (ar == 2 && (prog->op_code[o] < 0 || prog->op_code[o] >= (int)CGTB_B_COUNT)))
      return fail("cgtb_fused_rows: malformed program");
  }
  for (int j = 0; j < prog->n_out; ++j)
    if (prog->out_reg[j] < 0 || prog->out_reg[j] >= prog->n_in + prog->n_ops) return fail("cgtb_fused_rows: bad output register");
  if (R <= 0) return 0;
  RowArgs a;
  a.prog = *prog;
  a.R = R;
  a.C = C;
  for (int k = 0; k < prog->n_in; ++k) a.in[k] = in[k];
  for (int j = 0; j < prog->n_out; ++j) a.out[j] = out[j];
  if (prog->launcher) {
    // a kernel generated for exactly this program (same scalar templates, values in registers)
    typedef int (*Launcher)(long, long, const void* const*, void* const*, void*);
    if (((Launcher)prog->launcher)(R, C, a.in, a.out, (void*)rt().stream)) return fail("cgtb_fused_rows: the generated kernel failed to launch");
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    return 0;
  }
  const int warps = 4;
  const unsigned blocks = (unsigned)cgtb_ceil_div(R, warps);
  if (C <= 32) CGTB_LAUNCH(fused_rows_kernel<1>, blocks, warps * 32, 0, a);
  else if (C <= 64) CGTB_LAUNCH(fused_rows_kernel<2>, blocks, warps * 32, 0, a);
  else CGTB_LAUNCH(fused_rows_kernel<4>, blocks, warps * 32, 0, a);
  CGTB_CHECK_LAUNCH("fused_rows");
  return 0;
}

// Column pieces placed into a zero matrix (the sum of padded slices that the gradient of column slices is).
constexpr int kScatterMax = 8;
struct ScatterArgs {
  long R, C;
  int k;
  long off[kScatterMax], width[kScatterMax];
  const float* piece[kScatterMax];
  float* out;
};
__global__ void scatter_cols_kernel(const ScatterArgs a) {
  const long n = a.R * a.C;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = i / a.C, c = i - r * a.C;
    float v = 0.f;
    for (int j = 0; j < a.k; ++j) {
      const long d = c - a.off[j];
      if (d >= 0 && d < a.width[j]) { v = a.piece[j][r * a.width[j] + d]; break; }
    }
    a.out[i] = v;
  }
}
CGTB_API int cgtb_scatter_cols(long R, long C, int k, const long* offset, const long* width, const void* const* pieces, void* out) {
  if (!require_runtime("cgtb_scatter_cols")) return 1;
  if (k < 1 || k > kScatterMax) return fail("cgtb_scatter_cols: between 1 and %d pieces", kScatterMax);
  if (R <= 0 || C <= 0) return 0;
  ScatterArgs a;
  a.R = R;
  a.C = C;
  a.k = k;
  a.out = (float*)out;
  for (int j = 0; j < k; ++j) {
    if (offset[j] < 0 || width[j] < 0 || offset[j] + width[j] > C) return fail("cgtb_scatter_cols: piece %d lies outside the %ld columns", j, C);
    for (int q = 0; q < j; ++q)
      if (offset[j] < a.off[q] + a.width[q] && a.off[q] < offset[j] + width[j]) return fail("cgtb_scatter_cols: pieces %d and %d overlap", q, j);
    a.off[j] = offset[j];
    a.width[j] = width[j];
    a.piece[j] = (const float*)pieces[j];
  }
  const unsigned blocks = (unsigned)std::min<long>(cgtb_ceil_div(R * C, 256), 8L * rt().sm_count);
  CGTB_LAUNCH(scatter_cols_kernel, blocks, 256, 0, a);
  CGTB_CHECK_LAUNCH("scatter_cols");
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Reductions (cgt/core.py:1663-1738), keepdims. The reduced index space is split across
// `nsplit` blocks per output element; each block folds its slice with a warp-shuffle tree and writes
// one partial, and a second kernel folds the partials in a fixed order, so results are deterministic.
// Adjacent axes with the same kept/reduced flag are merged on the host before launch.
// ------------------------------------------------------------------------------------------------
struct ReduceGeom {
  int nk, nr;                 // number of kept / reduced merged axes
  long kshape[CGTB_MAX_NDIM], kstride[CGTB_MAX_NDIM];
  long rshape[CGTB_MAX_NDIM], rstride[CGTB_MAX_NDIM];
};

template <typename T>
__device__ __forceinline__ T red_init(int kind) {
  return kind == CGTB_R_SUM ? T(0) : -std::numeric_limits<T>::max();
}
template <> __device__ __forceinline__ float red_init<float>(int kind) { return kind == CGTB_R_SUM ? 0.f : -FLT_MAX; }
template <> __device__ __forceinline__ double red_init<double>(int kind) { return kind == CGTB_R_SUM ? 0.0 : -DBL_MAX; }

template <typename T>
__device__ __forceinline__ T red_op(int kind, T a, T b) {
  if (kind == CGTB_R_SUM) return a + b;
  return (T)fmax((double)a, (double)b);
}
template <> __device__ __forceinline__ float red_op<float>(int kind, float a, float b) { return kind == CGTB_R_SUM ? a + b : fmaxf(a, b); }

template <typename T>
__device__ __forceinline__ T shfl_down_t(T v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }
template <> __device__ __forceinline__ int8_t shfl_down_t<int8_t>(int8_t v, int d) { return (int8_t)__shfl_down_sync(0xffffffffu, (int)v, d); }

template <typename T>
__global__ void reduce_kernel(int kind, ReduceGeom g, long rsize, long chunk, const T* __restrict__ in, T* __restrict__ out,
                              int nsplit) {
  long o = blockIdx.x;
  int split = blockIdx.y;
  long base = 0, rem = o;
  for (int i = g.nk - 1; i >= 0; --i) {
    long q = rem / g.kshape[i];
    base += (rem - q * g.kshape[i]) * g.kstride[i];
    rem = q;
  }
  long r0 = split * chunk, r1 = min(r0 + chunk, rsize);
  T acc = red_init<T>(kind);
  for (long r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
    long off = base, rr = r;
    for (int i = g.nr - 1; i >= 0; --i) {
      long q = rr / g.rshape[i];
      off += (rr - q * g.rshape[i]) * g.rstride[i];
      rr = q;
    }
    acc = red_op<T>(kind, acc, in[off]);
  }
  __shared__ T warp_part[32];
  for (int d = 16; d > 0; d >>= 1) acc = red_op<T>(kind, acc, shfl_down_t<T>(acc, d));
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) warp_part[wid] = acc;
  __syncthreads();
  if (wid == 0) {
    int nw = blockDim.x >> 5;
    acc = lane < nw ? warp_part[lane] : red_init<T>(kind);
    for (int d = 16; d > 0; d >>= 1) acc = red_op<T>(kind, acc, shfl_down_t<T>(acc, d));
    if (lane == 0) out[o * nsplit + split] = acc;
  }
}

template <typename T>
__global__ void reduce_finish_kernel(int kind, long osize, int nsplit, const T* __restrict__ part, T* __restrict__ out) {
  for (long o = (long)blockIdx.x * blockDim.x + threadIdx.x; o < osize; o += (long)gridDim.x * blockDim.x) {
    T acc = red_init<T>(kind);
    for (int s = 0; s < nsplit; ++s) acc = red_op<T>(kind, acc, part[o * nsplit + s]);
    out[o] = acc;
  }
}

// The fast path for an input viewed as [R0, K, R1] with R0 and R1 reduced lives in reduce_rkr.h.
// [R0, K] with R0 reduced and K contiguous (column sums: the bias gradient of a dense layer). Block =
// 32 columns x G row groups (G = 8, or 32 for many rows): lane along K (coalesced rows), row group g adds rows
// g, g+G, ... with four loads in flight, and the G partial sums of a column are folded in a fixed order through
// shared memory. One thread walking all R0 rows of its column would pay the memory latency R0 times.
template <typename T, int G>
__global__ void __launch_bounds__(32 * G) reduce_rk_kernel(int kind, int R0, int K, const T* __restrict__ in, T* __restrict__ out) {
  __shared__ T part[G][33];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  for (int k0 = blockIdx.x * 32; k0 < K; k0 += gridDim.x * 32) {
    const int k = k0 + lane;
    T acc = red_init<T>(kind);
    if (k < K) {
      int r0 = g;
      for (; r0 + 3 * G < R0; r0 += 4 * G) {
        const T v0 = in[(size_t)r0 * K + k], v1 = in[(size_t)(r0 + G) * K + k], v2 = in[(size_t)(r0 + 2 * G) * K + k],
                v3 = in[(size_t)(r0 + 3 * G) * K + k];
        acc = red_op<T>(kind, red_op<T>(kind, red_op<T>(kind, red_op<T>(kind, acc, v0), v1), v2), v3);
      }
      for (; r0 < R0; r0 += G) acc = red_op<T>(kind, acc, in[(size_t)r0 * K + k]);
    }
    part[g][lane] = acc;
    __syncthreads();
    if (g == 0 && k < K) {
      T r = part[0][lane];
#pragma unroll
      for (int q = 1; q < G; ++q) r = red_op<T>(kind, r, part[q][lane]);
      out[k] = r;
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void reduce_identity_kernel(int kind, long n, T* __restrict__ out) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) out[i] = red_init<T>(kind);
}

template <typename T>
static int reduce_launch(int kind, int ndim, const long* shape, const int* reduced, const T* in, T* out) {
  ReduceGeom g;
  g.nk = g.nr = 0;
  long stride[CGTB_MAX_NDIM], acc = 1;
  for (int i = ndim - 1; i >= 0; --i) { stride[i] = acc; acc *= shape[i]; }
  if (acc == 0) {
    // nothing to reduce: every kept element is the identity of the operation (the reference's loop leaves the
    // initial value in place, cgt/core.py:1663-1685)
    long kept = 1;
    for (int i = 0; i < ndim; ++i) if (!reduced[i]) kept *= shape[i];
    if (kept > 0) CGTB_LAUNCH(reduce_identity_kernel<T>, (unsigned)std::min<long>(cgtb_ceil_div(kept, 256), 4096), 256, 0, kind, kept, out);
    return 0;
  }
  long osize = 1, rsize = 1;
  // merge adjacent axes of the same class: axis i (outer) and i+1 (inner) merge when both are in the
  // same class, since then stride[i] == shape[i+1]*stride[i+1]
  for (int i = 0; i < ndim; ++i) {
    if (shape[i] == 1) continue;
    bool r = reduced[i] != 0;
    int& n = r ? g.nr : g.nk;
    long* sh = r ? g.rshape : g.kshape;
    long* st = r ? g.rstride : g.kstride;
    bool merged = false;
    if (n > 0) {
      // previous axis of this class is adjacent iff no axis of the other class with extent > 1 lies between
      bool adjacent = true;
      for (int j = i - 1; j >= 0; --j) {
        if (shape[j] == 1) continue;
        adjacent = ((reduced[j] != 0) == r);
        break;
      }
      if (adjacent) { sh[n - 1] *= shape[i]; st[n - 1] = stride[i]; merged = true; }
    }
    if (!merged) { sh[n] = shape[i]; st[n] = stride[i]; n++; }
    if (r) rsize *= shape[i]; else osize *= shape[i];
  }
  // ---- fast paths on the merged geometry
  {
    long R0 = 1, K = 1, R1 = 1;
    bool match = false;
    if (g.nk <= 1 && g.nr == 2 && g.nk == 1 && g.rstride[1] == 1 && g.kstride[0] == g.rshape[1] &&
        g.rstride[0] == g.kshape[0] * g.rshape[1]) {
      R0 = g.rshape[0]; K = g.kshape[0]; R1 = g.rshape[1]; match = true;            // [R0, K, R1]
    } else if (g.nr == 1 && g.rstride[0] == 1 && (g.nk == 0 || (g.nk == 1 && g.kstride[0] == g.rshape[0]))) {
      K = g.nk ? g.kshape[0] : 1; R1 = g.rshape[0]; match = true;                    // [K, R1]
    } else if (g.nr == 1 && g.nk == 1 && g.kstride[0] == 1 && g.rstride[0] == g.kshape[0]) {
      R0 = g.rshape[0]; K = g.kshape[0]; R1 = 1; match = true;                       // [R0, K]
    }
    if (match && R0 < (1L << 30) && K < 65536L * 16 && R1 < (1L << 30)) {
      if (R1 == 1 && K >= 1) {
        if (R0 <= 4096 || K >= 1024) {
          const unsigned blocks = (unsigned)std::min<long>(cgtb_ceil_div(K, 32), 4096);
          if (R0 >= 256 && blocks <= 2u * (unsigned)rt().sm_count) {  // few columns, many rows: more row groups
            CGTB_LAUNCH((reduce_rk_kernel<T, 32>), blocks, 1024, 0, kind, (int)R0, (int)K, in, out);
          } else {
            CGTB_LAUNCH((reduce_rk_kernel<T, 8>), blocks, 256, 0, kind, (int)R0, (int)K, in, out);
          }
          return 0;
        }
      } else if (K <= 65535) {
        const rkr::Plan pl = rkr::plan<T>(R0, K, R1, rt().sm_count, in);
        dim3 grid((unsigned)K, (unsigned)pl.nsplit);
        if (pl.nsplit == 1) {
          CGTB_LAUNCH(rkr::partial_kernel<T>, grid, pl.threads, 0, kind, (int)R0, (int)K, (int)R1, pl.r0chunk, pl.r1chunk, pl.n1, pl.vec, pl.cols, in, out, 1);
        } else {
          T* part = (T*)scratch((size_t)K * pl.nsplit * sizeof(T));
          if (!part) return 1;
          CGTB_LAUNCH(rkr::partial_kernel<T>, grid, pl.threads, 0, kind, (int)R0, (int)K, (int)R1, pl.r0chunk, pl.r1chunk, pl.n1, pl.vec, pl.cols, in, part, pl.nsplit);
          CGTB_LAUNCH(rkr::finish_kernel<T>, (unsigned)cgtb_ceil_div(K, 128), 128, 0, kind, K, pl.nsplit, part, out);
        }
        return 0;
      }
    }
  }
  int threads = rsize >= 256 ? 256 : (rsize >= 64 ? 64 : 32);
  // split long reductions so that the grid fills the machine
  long want = (long)rt().sm_count * 4;
  int nsplit = 1;
  if (osize < want && rsize > 4096) {
    nsplit = (int)std::min<long>(cgtb_ceil_div(want, osize), cgtb_ceil_div(rsize, 2048));
    if (nsplit > 1024) nsplit = 1024;
    if (nsplit < 1) nsplit = 1;
  }
  long chunk = cgtb_ceil_div(rsize, nsplit);
  if (osize > 2147483647L) return fail("cgtb_reduce: too many output elements");
  dim3 grid((unsigned)osize, (unsigned)nsplit);
  if (nsplit == 1) {
    CGTB_LAUNCH(reduce_kernel<T>, grid, threads, 0, kind, g, rsize, chunk, in, out, 1);
  } else {
    T* part = (T*)scratch((size_t)osize * nsplit * sizeof(T));
    if (!part) return 1;
    CGTB_LAUNCH(reduce_kernel<T>, grid, threads, 0, kind, g, rsize, chunk, in, part, nsplit);
    CGTB_LAUNCH(reduce_finish_kernel<T>, (unsigned)cgtb_ceil_div(osize, 128), 128, 0, kind, osize, nsplit, part, out);
  }
  return 0;
}

CGTB_API int cgtb_reduce(int kind, int dtype, int ndim, const long* shape, const int* reduced, const void* in, void* out) {
  if (!require_runtime("cgtb_reduce")) return 1;
  if (ndim > CGTB_MAX_NDIM) return fail("cgtb_reduce: ndim %d too large", ndim);
  CGTB_FOR_DTYPE(dtype, T, { int rc = reduce_launch<T>(kind, ndim, shape, reduced, (const T*)in, (T*)out); if (rc) return rc; });
  CGTB_CHECK_LAUNCH("reduce");
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Data movement. Templated on the element size only (1, 2, 4, 8 bytes).
// ------------------------------------------------------------------------------------------------
template <int BYTES> struct bytes_type;
template <> struct bytes_type<1> { typedef uint8_t type; };
template <> struct bytes_type<2> { typedef uint16_t type; };
template <> struct bytes_type<4> { typedef uint32_t type; };
template <> struct bytes_type<8> { typedef uint64_t type; };

static inline int dtype_bytes(int dtype) {
  switch (dtype) {
    case cgtb_i1: return 1;
    case cgtb_i2: return 2;
    case cgtb_i4: case cgtb_f4: return 4;
    case cgtb_i8: case cgtb_f8: return 8;
  }
  return 0;
}

#define CGTB_FOR_BYTES(nbytes, U, ...)                                           \
  switch (nbytes) {                                                              \
    case 1: { typedef uint8_t U; __VA_ARGS__; } break;                           \
    case 2: { typedef uint16_t U; __VA_ARGS__; } break;                          \
    case 4: { typedef uint32_t U; __VA_ARGS__; } break;                          \
    case 8: { typedef uint64_t U; __VA_ARGS__; } break;                          \
    default: return fail("unsupported element size %d", (int)(nbytes));          \
  }

struct GatherGeom {
  int nd;
  long oshape[CGTB_MAX_NDIM];
  long istride[CGTB_MAX_NDIM];  // input stride for each output axis (0 on repeated axes)
};

// out[flat] = in[sum_k idx_k * istride_k] : serves Repeat and the general Transpose
template <typename U>
__global__ void gather_kernel(GatherGeom g, long total, const U* __restrict__ in, U* __restrict__ out) {
  for (long f = (long)blockIdx.x * blockDim.x + threadIdx.x; f < total; f += (long)gridDim.x * blockDim.x) {
    long rem = f, off = 0;
    for (int i = g.nd - 1; i >= 0; --i) {
      long q = rem / g.oshape[i];
      off += (rem - q * g.oshape[i]) * g.istride[i];
      rem = q;
    }
    out[f] = in[off];
  }
}

static inline unsigned flat_grid(long n, int per_thread = 1) {
  long blocks = cgtb_ceil_div(cgtb_ceil_div(n, per_thread), 256);
  long cap = (long)rt().sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

// Repeat fast path: output viewed as [R0, K, R1] with out[r0, k, r1] = in[k] (a bias broadcast).
// One block row per (r0, k) pair; no per-element division.
template <typename U>
__global__ void repeat_rkr_kernel(long rows, int K, int R1, const U* __restrict__ in, U* __restrict__ out) {
  for (long row = blockIdx.x; row < rows; row += gridDim.x) {
    const U v = in[row % K];
    U* dst = out + row * R1;
    for (int r1 = threadIdx.x; r1 < R1; r1 += blockDim.x) dst[r1] = v;
  }
}
template <typename U>
__global__ void repeat_rk_kernel(long total, int K, const U* __restrict__ in, U* __restrict__ out) {
  for (long f = (long)blockIdx.x * blockDim.x + threadIdx.x; f < total; f += (long)gridDim.x * blockDim.x)
    out[f] = in[(unsigned)(f % K)];
}

CGTB_API int cgtb_repeat(int dtype, int ndim, const long* out_shape, const int* repeated, const void* in, void* out) {
  if (!require_runtime("cgtb_repeat")) return 1;
  if (ndim > CGTB_MAX_NDIM) return fail("cgtb_repeat: ndim %d too large", ndim);
  GatherGeom g;
  g.nd = 0;
  long total = 1, acc = 1;
  long istride[CGTB_MAX_NDIM];
  for (int i = ndim - 1; i >= 0; --i) {
    istride[i] = repeated[i] ? 0 : acc;
    if (!repeated[i]) acc *= out_shape[i];
    total *= out_shape[i];
  }
  if (total <= 0) return 0;
  // merge adjacent axes: both repeated, or both kept (kept axes are contiguous in the input)
  for (int i = 0; i < ndim; ++i) {
    if (out_shape[i] == 1) continue;
    if (g.nd > 0) {
      bool prev_rep = g.istride[g.nd - 1] == 0, cur_rep = repeated[i] != 0;
      if (prev_rep == cur_rep) {
        g.oshape[g.nd - 1] *= out_shape[i];
        g.istride[g.nd - 1] = istride[i];
        continue;
      }
    }
    g.oshape[g.nd] = out_shape[i];
    g.istride[g.nd] = istride[i];
    g.nd++;
  }
  // [R0 repeated, K kept, R1 repeated] and [R0 repeated, K kept]
  if (g.nd == 3 && g.istride[0] == 0 && g.istride[1] == 1 && g.istride[2] == 0 && g.oshape[1] < (1L << 31) && g.oshape[2] < (1L << 31)) {
    long rows = g.oshape[0] * g.oshape[1];
    int R1 = (int)g.oshape[2];
    int threads = R1 >= 256 ? 256 : (R1 >= 128 ? 128 : (R1 >= 64 ? 64 : 32));
    unsigned blocks = (unsigned)std::min<long>(rows, (long)rt().sm_count * 32);
    CGTB_FOR_BYTES(dtype_bytes(dtype), U, CGTB_LAUNCH(repeat_rkr_kernel<U>, blocks, threads, 0, rows, (int)g.oshape[1], R1, (const U*)in, (U*)out));
  } else if (g.nd == 2 && g.istride[0] == 0 && g.istride[1] == 1 && g.oshape[1] < (1L << 31)) {
    CGTB_FOR_BYTES(dtype_bytes(dtype), U, CGTB_LAUNCH(repeat_rk_kernel<U>, flat_grid(total), 256, 0, total, (int)g.oshape[1], (const U*)in, (U*)out));
  } else {
    CGTB_FOR_BYTES(dtype_bytes(dtype), U, CGTB_LAUNCH(gather_kernel<U>, flat_grid(total), 256, 0, g, total, (const U*)in, (U*)out));
  }
  CGTB_CHECK_LAUNCH("repeat");
  return 0;
}

// batched 2-D transpose through a padded shared-memory tile: in [P, R, Cc] -> out [P, Cc, R].
// 32-bit offsets inside a matrix (the host checks R*Cc < 2^31), one pointer per thread advanced by a
// constant, and no bounds tests on full tiles: about ten instructions per element instead of seventy.
template <typename U>
__global__ void transpose_tile_kernel(const U* __restrict__ in, U* __restrict__ out, int R, int Cc) {
  __shared__ U tile[32][33];
  const size_t pbase = (size_t)blockIdx.z * R * Cc;
  const U* ip = in + pbase;
  U* op = out + pbase;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;  // block (32, 8)
  if (r0 + 32 <= R && c0 + 32 <= Cc) {
    const U* src = ip + (r0 + ty) * Cc + c0 + tx;
#pragma unroll
    for (int k = 0; k < 4; ++k) tile[ty + 8 * k][tx] = src[8 * k * Cc];
    __syncthreads();
    U* dst = op + (c0 + ty) * R + r0 + tx;
#pragma unroll
    for (int k = 0; k < 4; ++k) dst[8 * k * R] = tile[tx][ty + 8 * k];
  } else {
    for (int dy = ty; dy < 32; dy += 8) {
      const int r = r0 + dy, c = c0 + tx;
      if (r < R && c < Cc) tile[dy][tx] = ip[r * Cc + c];
    }
    __syncthreads();
    for (int dy = ty; dy < 32; dy += 8) {
      const int c = c0 + dy, r = r0 + tx;
      if (r < R && c < Cc) op[c * R + r] = tile[tx][dy];
    }
  }
}

CGTB_API int cgtb_transpose(int dtype, int ndim, const long* in_shape, const int* axes, const void* in, void* out) {
  if (!require_runtime("cgtb_transpose")) return 1;
  if (ndim > CGTB_MAX_NDIM) return fail("cgtb_transpose: ndim %d too large", ndim);
  long istride[CGTB_MAX_NDIM], acc = 1;
  for (int i = ndim - 1; i >= 0; --i) { istride[i] = acc; acc *= in_shape[i]; }
  long total = acc;
  if (total <= 0) return 0;
  // group output axes: consecutive output axes that are also consecutive input axes travel together
  int gstart[CGTB_MAX_NDIM], glen[CGTB_MAX_NDIM], ng = 0;
  for (int k = 0; k < ndim; ++k) {
    if (in_shape[axes[k]] == 1) continue;
    if (ng > 0) {
      // last non-unit input axis of the previous group
      int last = gstart[ng - 1] + glen[ng - 1] - 1;
      bool contiguous = axes[k] > last;
      for (int a = last + 1; a < axes[k] && contiguous; ++a) contiguous = in_shape[a] == 1;
      if (contiguous) { glen[ng - 1] = axes[k] - gstart[ng - 1] + 1; continue; }
    }
    gstart[ng] = axes[k];
    glen[ng] = 1;
    ng++;
  }
  long gsize[CGTB_MAX_NDIM], gstride[CGTB_MAX_NDIM];
  for (int q = 0; q < ng; ++q) {
    gsize[q] = 1;
    for (int a = gstart[q]; a < gstart[q] + glen[q]; ++a) gsize[q] *= in_shape[a];
    gstride[q] = istride[gstart[q] + glen[q] - 1];
  }
  int nbytes = dtype_bytes(dtype);
  if (ng <= 1) {  // no data reordering
    CGTB_CUDA_TRY(cudaMemcpyAsync(out, in, (size_t)total * nbytes, cudaMemcpyDeviceToDevice, rt().stream));
    return 0;
  }
  // fast path: [P, R, Cc] -> [P, Cc, R]
  bool batched2d = false;
  long P = 1, R = 0, Cc = 0;
  if (ng == 2 && gstart[0] > gstart[1]) { R = gsize[1]; Cc = gsize[0]; batched2d = true; }
  if (ng == 3 && gstart[0] < gstart[2] && gstart[2] < gstart[1] && gstride[0] == gsize[1] * gsize[2]) {
    P = gsize[0]; R = gsize[2]; Cc = gsize[1]; batched2d = true;
  }
  if (batched2d && P <= 65535 && cgtb_ceil_div(R, 32) <= 65535 && R * Cc < (1L << 31)) {
    // output is [P, Cc, R] with input [P, R, Cc]
    dim3 grid((unsigned)cgtb_ceil_div(Cc, 32), (unsigned)cgtb_ceil_div(R, 32), (unsigned)P), block(32, 8);
    CGTB_FOR_BYTES(nbytes, U, CGTB_LAUNCH(transpose_tile_kernel<U>, grid, block, 0, (const U*)in, (U*)out, (int)R, (int)Cc));
    CGTB_CHECK_LAUNCH("transpose");
    return 0;
  }
  GatherGeom g;
  g.nd = ng;
  for (int q = 0; q < ng; ++q) { g.oshape[q] = gsize[q]; g.istride[q] = gstride[q]; }
  CGTB_FOR_BYTES(nbytes, U, CGTB_LAUNCH(gather_kernel<U>, flat_grid(total), 256, 0, g, total, (const U*)in, (U*)out));
  CGTB_CHECK_LAUNCH("transpose");
  return 0;
}

// strided slice along one axis of a [outer, n, inner] view
template <typename U>
__global__ void getsli_kernel(long total, long n_in, long inner, long start, long step, long n_out, const U* __restrict__ in,
                              U* __restrict__ out) {
  for (long f = (long)blockIdx.x * blockDim.x + threadIdx.x; f < total; f += (long)gridDim.x * blockDim.x) {
    long k = f % inner, t = f / inner;
    long i = t % n_out, o = t / n_out;
    out[f] = in[(o * n_in + start + step * i) * inner + k];
  }
}
CGTB_API int cgtb_getsli(int dtype, long outer, long n_in, long inner, long start, long step, long n_out, const void* in,
                         void* out) {
  if (!require_runtime("cgtb_getsli")) return 1;
  long total = outer * n_out * inner;
  if (total <= 0) return 0;
  long last = start + step * (n_out - 1);
  if (start < 0 || start >= n_in || last < 0 || last >= n_in) return fail("cgtb_getsli: slice out of range");
  CGTB_FOR_BYTES(dtype_bytes(dtype), U,
                 CGTB_LAUNCH(getsli_kernel<U>, flat_grid(total), 256, 0, total, n_in, inner, start, step, n_out, (const U*)in, (U*)out));
  CGTB_CHECK_LAUNCH("getsli");
  return 0;
}

template <typename T>
__global__ void incsli_kernel(long total, long n_x, long inner, long start, long step, long n_inc, const T* __restrict__ inc,
                              T* __restrict__ out) {
  for (long f = (long)blockIdx.x * blockDim.x + threadIdx.x; f < total; f += (long)gridDim.x * blockDim.x) {
    long k = f % inner, t = f / inner;
    long i = t % n_inc, o = t / n_inc;
    out[(o * n_x + start + step * i) * inner + k] += inc[f];
  }
}
CGTB_API int cgtb_incsli(int dtype, long outer, long n_x, long inner, long start, long step, long n_inc, const void* x,
                         const void* inc, void* out) {
  if (!require_runtime("cgtb_incsli")) return 1;
  long xsize = outer * n_x * inner, total = outer * n_inc * inner;
  if (xsize <= 0) return 0;
  if (step == 0) return fail("cgtb_incsli: zero step");
  long last = start + step * (n_inc - 1);
  if (n_inc > 0 && (start < 0 || start >= n_x || last < 0 || last >= n_x)) return fail("cgtb_incsli: slice out of range");
  if (out != x) CGTB_CUDA_TRY(cudaMemcpyAsync(out, x, (size_t)xsize * dtype_bytes(dtype), cudaMemcpyDeviceToDevice, rt().stream));
  if (total <= 0) return 0;
  CGTB_FOR_DTYPE(dtype, T, CGTB_LAUNCH(incsli_kernel<T>, flat_grid(total), 256, 0, total, n_x, inner, start, step, n_inc, (const T*)inc, (T*)out));
  CGTB_CHECK_LAUNCH("incsli");
  return 0;
}

template <typename U>
__global__ void getflat_kernel(long n, long xsize_guard, const U* __restrict__ x, const int64_t* __restrict__ k, U* __restrict__ out) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) out[i] = x[k[i]];
}
CGTB_API int cgtb_getflat(int dtype, long n, const void* x, const int64_t* k, void* out) {
  if (!require_runtime("cgtb_getflat")) return 1;
  if (n <= 0) return 0;
  CGTB_FOR_BYTES(dtype_bytes(dtype), U, CGTB_LAUNCH(getflat_kernel<U>, flat_grid(n), 256, 0, n, 0, (const U*)x, k, (U*)out));
  CGTB_CHECK_LAUNCH("getflat");
  return 0;
}

// IncFlatIndices (cgt/core.py:2012-2023): out.flat[k[i]] += p[i] in index order, so duplicate indices
// accumulate in the reference's order: the FIRST occurrence of an index owns the whole ordered sum
// for that index, every later occurrence does nothing.
template <typename T>
__global__ void incflat_kernel(int n, const int64_t* __restrict__ k, const T* __restrict__ p, T* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char incflat_smem[];
  int64_t* ks = reinterpret_cast<int64_t*>(incflat_smem);  // the whole index list, staged once per block
  for (int j = threadIdx.x; j < n; j += blockDim.x) ks[j] = k[j];
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t me = ks[i];
  // one branch-free pass counts the duplicates of this index before and after position i
  int before = 0, after = 0;
  for (int j = 0; j < n; ++j) {
    const bool m = ks[j] == me;
    before += (m && j < i);
    after += (m && j > i);
  }
  if (before) return;  // an earlier occurrence owns the ordered sum for this index
  T acc = out[me] + p[i];
  if (after)
    for (int j = i + 1; j < n; ++j)
      if (ks[j] == me) acc += p[j];
  out[me] = acc;
}
// large index lists: atomics (integer results stay exact; float sums of duplicates may reorder)
template <typename T>
__global__ void incflat_atomic_kernel(long n, const int64_t* __restrict__ k, const T* __restrict__ p, T* __restrict__ out) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) atomicAdd(&out[k[i]], p[i]);
}
template <typename T> struct has_atomic { static const bool value = false; };
template <> struct has_atomic<float> { static const bool value = true; };
template <> struct has_atomic<double> { static const bool value = true; };
template <> struct has_atomic<int32_t> { static const bool value = true; };

template <typename T>
static int incflat_launch(long n, const int64_t* k, const T* p, T* out) {
  if (n <= 4096 || !has_atomic<T>::value) {
    if (n > 4096) return fail("cgtb_incflat: %ld indices of a dtype without atomicAdd", n);
    CGTB_LAUNCH(incflat_kernel<T>, (unsigned)cgtb_ceil_div(n, 256), 256, (size_t)n * sizeof(int64_t), (int)n, k, p, out);
  } else {
    if constexpr (has_atomic<T>::value) CGTB_LAUNCH(incflat_atomic_kernel<T>, flat_grid(n), 256, 0, n, k, p, out);
  }
  return 0;
}
CGTB_API int cgtb_incflat(int dtype, long xsize, long n, const void* x, const int64_t* k, const void* p, void* out) {
  if (!require_runtime("cgtb_incflat")) return 1;
  if (xsize <= 0) return 0;
  if (out != x) CGTB_CUDA_TRY(cudaMemcpyAsync(out, x, (size_t)xsize * dtype_bytes(dtype), cudaMemcpyDeviceToDevice, rt().stream));
  if (n <= 0) return 0;
  CGTB_FOR_DTYPE(dtype, T, { int rc = incflat_launch<T>(n, k, (const T*)p, (T*)out); if (rc) return rc; });
  CGTB_CHECK_LAUNCH("incflat");
  return 0;
}

template <typename U>
__global__ void concat_part_kernel(long total, long n_in, long n_out, long inner, long pos, const U* __restrict__ in,
                                   U* __restrict__ out) {
  for (long f = (long)blockIdx.x * blockDim.x + threadIdx.x; f < total; f += (long)gridDim.x * blockDim.x) {
    long k = f % inner, t = f / inner;
    long i = t % n_in, o = t / n_in;
    out[(o * n_out + pos + i) * inner + k] = in[f];
  }
}
// Concatenation along axis 0: every piece is one contiguous run. One launch for all pieces (blockIdx.y = piece).
constexpr int kConcatMax = 64;
struct ConcatRowsArgs {
  const unsigned char* src[kConcatMax];
  long bytes[kConcatMax], off[kConcatMax];
  unsigned char* out;
};
__global__ void concat_rows_kernel(const ConcatRowsArgs a) {
  const int t = blockIdx.y;
  const unsigned char* src = a.src[t];
  unsigned char* dst = a.out + a.off[t];
  const long n = a.bytes[t], stride = (long)gridDim.x * blockDim.x, i0 = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if ((((uintptr_t)src | (uintptr_t)dst | (uintptr_t)n) & 15) == 0) {
    for (long i = i0; i < (n >> 4); i += stride) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else if ((((uintptr_t)src | (uintptr_t)dst | (uintptr_t)n) & 3) == 0) {
    for (long i = i0; i < (n >> 2); i += stride) reinterpret_cast<uint32_t*>(dst)[i] = reinterpret_cast<const uint32_t*>(src)[i];
  } else {
    for (long i = i0; i < n; i += stride) dst[i] = src[i];
  }
}
CGTB_API int cgtb_concat_rows(int n, const void* const* pieces, const long* bytes, void* out) {
  if (!require_runtime("cgtb_concat_rows")) return 1;
  if (n < 1 || n > kConcatMax) return fail("cgtb_concat_rows: between 1 and %d pieces", kConcatMax);
  ConcatRowsArgs a;
  a.out = (unsigned char*)out;
  long off = 0, nmax = 0;
  for (int i = 0; i < n; ++i) {
    if (bytes[i] < 0) return fail("cgtb_concat_rows: negative size");
    a.src[i] = (const unsigned char*)pieces[i];
    a.bytes[i] = bytes[i];
    a.off[i] = off;
    off += bytes[i];
    nmax = std::max(nmax, bytes[i]);
  }
  if (nmax == 0) return 0;
  dim3 grid((unsigned)std::max<long>(1, std::min<long>(cgtb_ceil_div(nmax, 16 * 256), 32)), (unsigned)n);
  CGTB_LAUNCH(concat_rows_kernel, grid, 256, 0, a);
  CGTB_CHECK_LAUNCH("concat_rows");
  return 0;
}

CGTB_API int cgtb_concat_part(int dtype, long outer, long n_in, long n_out, long inner, long pos, const void* in, void* out) {
  if (!require_runtime("cgtb_concat_part")) return 1;
  long total = outer * n_in * inner;
  if (total <= 0) return 0;
  if (pos < 0 || pos + n_in > n_out) return fail("cgtb_concat_part: part does not fit");
  CGTB_FOR_BYTES(dtype_bytes(dtype), U,
                 CGTB_LAUNCH(concat_part_kernel<U>, flat_grid(total), 256, 0, total, n_in, n_out, inner, pos, (const U*)in, (U*)out));
  CGTB_CHECK_LAUNCH("concat");
  return 0;
}

template <typename T>
__global__ void fill_kernel(long n, T v, T* __restrict__ out) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) out[i] = v;
}
CGTB_API int cgtb_fill(int dtype, long n, double fvalue, long ivalue, void* out) {
  if (!require_runtime("cgtb_fill")) return 1;
  if (n <= 0) return 0;
  switch (dtype) {
    case cgtb_i1: CGTB_LAUNCH(fill_kernel<int8_t>, flat_grid(n), 256, 0, n, (int8_t)ivalue, (int8_t*)out); break;
    case cgtb_i4: CGTB_LAUNCH(fill_kernel<int32_t>, flat_grid(n), 256, 0, n, (int32_t)ivalue, (int32_t*)out); break;
    case cgtb_i8: CGTB_LAUNCH(fill_kernel<int64_t>, flat_grid(n), 256, 0, n, (int64_t)ivalue, (int64_t*)out); break;
    case cgtb_f4: CGTB_LAUNCH(fill_kernel<float>, flat_grid(n), 256, 0, n, (float)fvalue, (float*)out); break;
    case cgtb_f8: CGTB_LAUNCH(fill_kernel<double>, flat_grid(n), 256, 0, n, fvalue, (double*)out); break;
    default: return fail("cgtb_fill: unsupported dtype %d", dtype);
  }
  CGTB_CHECK_LAUNCH("fill");
  return 0;
}
