"""Run-time code generation for elementwise Ops whose C expression is not one of the prebuilt ones.

Counterpart of the generated-kernel branch of ElwiseUnary.get_native_compile_info in the reference
(cgt/core.py:1216-1239): the expression string becomes a `__device__` function inside a vectorised
grid-stride kernel, compiled by nvcc for sm_100a into the hash-keyed library cache.
"""
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
