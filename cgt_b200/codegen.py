"""Run-time code generation for elementwise Ops whose C expression is not one of the prebuilt ones.

Counterpart of the generated-kernel branch of ElwiseUnary.get_native_compile_info in the reference
(cgt/core.py:1216-1239): the expression string becomes a `__device__` function inside a vectorised
grid-stride kernel, compiled by nvcc for sm_100a into the hash-keyed library cache.
"""
import os

from . import core

_CUDA_TEMPLATE = r"""
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>
__forceinline__ __device__ %(cdtype1)s scalar_$function(%(cdtype0)s x) { return %(cexpr)s; }
__global__ void ${function}_kernel(const long n, const %(cdtype0)s* __restrict__ in, %(cdtype1)s* __restrict__ out) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    out[i] = scalar_$function(in[i]);
}
void launchker_$function(long n, const %(cdtype0)s* x, %(cdtype1)s* y, void* stream) {
  if (n <= 0) return;
  long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ${function}_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(n, x, y);
}
"""

_CPP_TEMPLATE = r"""
extern void launchker_${function}(long, const %(cdtype0)s*, %(cdtype1)s*, void*);
static inline %(cdtype1)s host_scalar_$function(%(cdtype0)s x) { return %(cexpr)s; }
CGT_EXPORT_C void $function(void* cldata, cgtArray** reads, cgtArray* write) {
    cgtArray* read = reads[0];
    long n = read->size();
    if (read->devtype() == cgtGPU) {
        launchker_$function(n, (const %(cdtype0)s*)read->data(), (%(cdtype1)s*)write->data(), cgt_current_stream());
    } else {
        cgt_check(n <= 64, "a tensor was placed on the host; this backend has no CPU implementation of tensor ops");
        for (long i = 0; i < n && n <= 64; ++i) write->at<%(cdtype1)s>(i) = host_scalar_$function(read->at<%(cdtype0)s>(i));
    }
}
"""


def unary_from_cexpr(op, input_types, devtype):
    out_dtype = op.typ_apply(input_types).dtype
    d = dict(cdtype0=core.np2c[input_types[0].dtype], cdtype1=core.np2c[out_dtype], cexpr=op.info.cexpr)
    return core.NativeCompileInfo(_CPP_TEMPLATE % d, includes=["math.h", "stdint.h"], link_flags="-lm",
                                  gpu_deref_mask=(True,), extra_srcs=[core.SrcFile("cuda", _CUDA_TEMPLATE % d)])


# ================================================================
# Fused elementwise chains
# ================================================================

_FUSED_HEAD = r"""
#include <cuda_runtime.h>
#include "cgt_elwise.h"
"""


def fused_source(op):
    """CUDA source of the kernel for one FusedElwise program. Every operation calls the scalar template
    the separate kernels use (float operands, literal opcode), values stay in registers, scalars are
    read once per thread. Compiled without multiply-add contraction: the separate kernels round every
    product before the next Op adds to it."""
    n_in = len(op.in_kinds)
    params, hoist, loads = [], [], []
    for (k, kind) in enumerate(op.in_kinds):
        if kind == 0:
            params.append("const float* __restrict__ in%d" % k)
            loads.append(("pack", "const Pack<float, V> p%d = load_pack<float, V>(in%d + i * V);" % (k, k), "p%d.v[v]" % k))
        elif kind == 1:
            params.append("const int8_t* __restrict__ in%d" % k)
            loads.append(("pack", "const Pack<int8_t, V> p%d = load_pack<int8_t, V>(in%d + i * V);" % (k, k), "(float)p%d.v[v]" % k))
        elif kind == 2:
            params.append("const float* __restrict__ in%d" % k)
            hoist.append("const float s%d = in%d[0];" % (k, k))
            loads.append(("none", "", "s%d" % k))
        elif kind == 3:
            params.append("const long* __restrict__ in%d" % k)
            hoist.append("const float s%d = (float)in%d[0];" % (k, k))
            loads.append(("none", "", "s%d" % k))
        elif kind == 7:
            # columns [bi, bi + W) of a matrix with rows of bk elements; W is a literal of this chain
            params.append("const float* __restrict__ in%d, const long bk%d, const long bi%d" % (k, k, k))
            W = op.static_shape[1]
            loads.append(("pack", "const I row%d = (i * V) / (I)%d;\n    const Pack<float, V> p%d = load_pack<float, V>(in%d + (size_t)row%d * bk%d + bi%d "
                          "+ ((i * V) - row%d * (I)%d));" % (k, W, k, k, k, k, k, k, W), "p%d.v[v]" % k))
        else:
            params.append("const float* __restrict__ in%d, const long bk%d, const long bi%d" % (k, k, k))
            # one value per pack when the run length is a multiple of V, else one index per element
            loads.append(("pack", "float b%d[V];\n    if ((I)bi%d %% V == 0) {\n      const float t = in%d[((i * V) / (I)bi%d) %% (I)bk%d];\n"
                          "#pragma unroll\n      for (int v = 0; v < V; ++v) b%d[v] = t;\n    } else {\n"
                          "#pragma unroll\n      for (int v = 0; v < V; ++v) b%d[v] = in%d[((i * V + v) / (I)bi%d) %% (I)bk%d];\n    }"
                          % (k, k, k, k, k, k, k, k, k, k), "b%d[v]" % k))
    outs = []
    for (q, dt) in enumerate(op.out_dtypes):
        ctype = "float" if dt == "f4" else "int8_t"
        params.append("%s* __restrict__ out%d" % (ctype, q))
        outs.append(ctype)
    lines = ["// I: index type (32-bit when the element count allows: the broadcast index needs a division)",
             "template <int V, typename I>", "__global__ void fused_kernel(const I n, %s) {" % ", ".join(params)]
    lines += ["  " + h for h in hoist]
    lines.append("  const I nv = n / V;")
    lines.append("  for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (I)gridDim.x * blockDim.x) {")
    for (_kind, stmt, _expr) in loads:
        if stmt:
            lines.append("    " + stmt)
    for (q, ctype) in enumerate(outs):
        lines.append("    Pack<%s, V> o%d;" % (ctype, q))
    lines.append("#pragma unroll")
    lines.append("    for (int v = 0; v < V; ++v) {")
    for (k, (_kind, _stmt, expr)) in enumerate(loads):
        lines.append("      const float r%d = %s;" % (k, expr))
    for (j, (arity, code, a, b)) in enumerate(op.program):
        if arity == 1:
            lines.append("      const float r%d = unary_apply<float, float>(%d, r%d);" % (n_in + j, code, a))
        else:
            lines.append("      const float r%d = binary_apply<float, float, float>(%d, r%d, r%d);" % (n_in + j, code, a, b))
    for (q, (reg, ctype)) in enumerate(zip(op.out_regs, outs)):
        lines.append("      o%d.v[v] = (%s)r%d;" % (q, ctype, reg))
    lines.append("    }")
    for (q, ctype) in enumerate(outs):
        lines.append("    store_pack<%s, V>(out%d + i * V, o%d);" % (ctype, q, q))
    lines += ["  }", "}"]
    args = []
    for (k, kind) in enumerate(op.in_kinds):
        ctype = {0: "float", 1: "int8_t", 2: "float", 3: "long", 4: "float", 7: "float"}[kind]
        args.append("(const %s*)in[%d]" % (ctype, k))
        if kind in (4, 7):
            args += ["bk[%d]" % k, "bi[%d]" % k]
    for (q, ctype) in enumerate(outs):
        args.append("(%s*)out[%d]" % (ctype, q))
    lines += [
        'extern "C" __attribute__((visibility("default"))) int cgtb_fused_launch(long n, const void* const* in, const long* bk,',
        "    const long* bi, void* const* out, int vectorised, void* stream, int sm_count) {",
        "  const long work = vectorised ? n / 4 : n;",
        "  long blocks = (work + 255) / 256;",
        "  if (blocks > (long)sm_count * 16) blocks = (long)sm_count * 16;",
        "  if (blocks < 1) blocks = 1;",
        "  const bool small = n < (1L << 31);",
        "  if (vectorised && small) fused_kernel<4, unsigned><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((unsigned)n, %s);" % ", ".join(args),
        "  else if (vectorised) fused_kernel<4, long><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(n, %s);" % ", ".join(args),
        "  else if (small) fused_kernel<1, unsigned><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((unsigned)n, %s);" % ", ".join(args),
        "  else fused_kernel<1, long><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(n, %s);" % ", ".join(args),
        "  return cudaPeekAtLastError() != cudaSuccess;",
        "}",
    ]
    return _FUSED_HEAD + "\n".join(lines) + "\n"


def rows_source(op):
    """CUDA source of the kernel for one FusedRows program: one warp per row, element c of the row in lane c % 32,
    slot c / 32; every operation calls the scalar template the separate kernels use; a row sum adds the lane's valid
    slots in order and then folds the lanes with xor shuffles (16, 8, 4, 2, 1), as the library's kernel does."""
    n_in = len(op.in_kinds)
    lines = ["template <int E>", "__global__ void __launch_bounds__(128) rows_kernel(const long R, const long C, const void* const* in_, void* const* out_) {"]
    params, args = [], []
    for (k, kind) in enumerate(op.in_kinds):
        ctype = "long" if kind in (3, 8) else "float"
        params.append("const %s* __restrict__ in%d" % (ctype, k))
        args.append("(const %s*)in[%d]" % (ctype, k))
    for q in range(len(op.out_regs)):
        params.append("float* __restrict__ out%d" % q)
        args.append("(float*)out[%d]" % q)
    lines = ["template <int E>",
             "__global__ void __launch_bounds__(128) rows_kernel(const long R, const long C, %s) {" % ", ".join(params),
             "  const int lane = threadIdx.x & 31;",
             "  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);",
             "  if (row >= R) return;"]
    for (k, kind) in enumerate(op.in_kinds):
        lines.append("  float r%d[E];" % k)
        if kind in (0, 6):
            base = "in%d + row * C" % k if kind == 0 else "in%d" % k
            lines += ["#pragma unroll", "  for (int e = 0; e < E; ++e) { const long c = lane + 32 * e; r%d[e] = c < C ? (%s)[c] : 0.0f; }" % (k, base)]
        elif kind == 8:
            lines += ["  { const long hot = in%d[row];" % k, "#pragma unroll",
                      "    for (int e = 0; e < E; ++e) r%d[e] = (lane + 32 * e == hot) ? 1.0f : 0.0f; }" % k]
        else:
            src = {5: "in%d[row]" % k, 2: "in%d[0]" % k, 3: "(float)in%d[0]" % k}[kind]
            lines += ["  { const float v = %s;" % src, "#pragma unroll", "    for (int e = 0; e < E; ++e) r%d[e] = v; }" % k]
    for (j, (arity, code, a, b)) in enumerate(op.program):
        d = n_in + j
        lines.append("  float r%d[E];" % d)
        if arity == 1:
            lines += ["#pragma unroll", "  for (int e = 0; e < E; ++e) r%d[e] = unary_apply<float, float>(%d, r%d[e]);" % (d, code, a)]
        elif arity == 2:
            lines += ["#pragma unroll", "  for (int e = 0; e < E; ++e) r%d[e] = binary_apply<float, float, float>(%d, r%d[e], r%d[e]);" % (d, code, a, b)]
        else:
            cond = "lane + 32 * e < C" if arity == 3 else "lane + 32 * e < C && r%d[e] != 0.0f" % b
            lines += ["  { float s = 0.0f;", "#pragma unroll", "    for (int e = 0; e < E; ++e) if (%s) s += r%d[e];" % (cond, a),
                      "#pragma unroll", "    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);",
                      "#pragma unroll", "    for (int e = 0; e < E; ++e) r%d[e] = s; }" % d]
    for (q, (reg, col)) in enumerate(zip(op.out_regs, op.out_cols)):
        if col:
            lines.append("  if (lane == 0) out%d[row] = r%d[0];" % (q, reg))
        else:
            lines += ["#pragma unroll", "  for (int e = 0; e < E; ++e) { const long c = lane + 32 * e; if (c < C) out%d[row * C + c] = r%d[e]; }" % (q, reg)]
    lines.append("}")
    call = "(R, C, %s)" % ", ".join(args)
    lines += [
        'extern "C" __attribute__((visibility("default"))) int cgtb_rows_launch(long R, long C, const void* const* in, void* const* out, void* stream) {',
        "  const unsigned blocks = (unsigned)((R + 3) / 4);",
        "  if (C <= 32) rows_kernel<1><<<blocks, 128, 0, (cudaStream_t)stream>>>%s;" % call,
        "  else if (C <= 64) rows_kernel<2><<<blocks, 128, 0, (cudaStream_t)stream>>>%s;" % call,
        "  else rows_kernel<4><<<blocks, 128, 0, (cudaStream_t)stream>>>%s;" % call,
        "  return cudaPeekAtLastError() != cudaSuccess;",
        "}",
    ]
    return _FUSED_HEAD + "\n".join(lines) + "\n"


_fused_libs = {}


def rows_launcher(op):
    """Address of the generated launcher for a FusedRows program, or None (the library's kernel runs it then)."""
    return _generated_launcher(rows_source(op), "rows_", "cgtb_rows_launch", "a fused row chain")



def fused_launcher(op):
    """Address of the generated launcher for this program (compiled into the hash-keyed cache on first
    use), or None when generation is switched off or the compiler is not available: the library's
    register-machine kernel then runs the program."""
    return _generated_launcher(fused_source(op), "fused_", "cgtb_fused_launch", "a fused elementwise chain")


def _generated_launcher(src, tag, symbol, what):
    import ctypes
    import os.path as osp
    from . import compilation, utils
    if not core.get_config().get("jit_fused_elementwise", True):
        return None
    info = compilation.get_compile_info()
    prefix = tag + utils.hash_seq1(src, "fmad=false", str(compilation.CPP_ABI_VERSION))
    if prefix in _fused_libs:
        return _fused_libs[prefix][1]
    libpath = osp.join(info["CACHE_ROOT"], prefix + ".so")
    try:
        if not osp.exists(libpath):
            srcpath = osp.join(info["CACHE_ROOT"], prefix + ".cu")
            with open(srcpath, "w") as fh:
                fh.write(src)
            compilation._call("nvcc %s -o %s.tmp -shared -gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 "
                              "-fmad=false -Xcompiler -fPIC %s -L/usr/local/cuda/lib64 -lcudart"
                              % (srcpath, libpath, info["INCLUDES"]))
            os.replace(libpath + ".tmp", libpath)
        lib = ctypes.CDLL(libpath)
        addr = ctypes.cast(getattr(lib, symbol), ctypes.c_void_p).value
    except (RuntimeError, OSError) as err:
        import sys
        sys.stderr.write("cgt_b200: no generated kernel for %s (%s); using the built-in one\n" % (what, str(err).splitlines()[0]))
        _fused_libs[prefix] = (None, None)
        return None
    _fused_libs[prefix] = (lib, addr)
    return addr
