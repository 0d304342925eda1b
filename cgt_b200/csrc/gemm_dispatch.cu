// Mul22 / BatchedMul22 entry points: choose between the tcgen05 tensor-core kernels (3xTF32 split
// precision; TMA-fed for 16-byte-aligned operands, gemm_tma.cu, register-fed otherwise,
// gemm_tcgen05.cu) and the fp32 FMA kernel (gemm_simt.cu).
// Products with few outputs and a short K go to a one-thread-per-output kernel (gemm_simt.cu).
// impl: 0 automatic, 1 FMA (tiled), 2 tensor cores (either feed), 3 register-fed only, 4 TMA-fed only,
// 5 the small-product kernel only.
#include "runtime.h"

namespace cgtb {
int sgemm_simt(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
               long ldb, long strideB, float* C, long ldc, long strideC);
// returns 0 done, 1 error, -1 shape not supported by the tensor-core kernel
int sgemm_tc(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
             long ldb, long strideB, float* C, long ldc, long strideC);

int sgemm_tma(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
              long ldb, long strideB, float* C, long ldc, long strideC);

int sgemm_small(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
                long ldb, long strideB, float* C, long ldc, long strideC);

int sgemm_dispatch(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B,
                   long ldb, long strideB, float* C, long ldc, long strideC, int impl) {
  if (!require_runtime("sgemm")) return 1;
  if (impl == 0 || impl == 5) {
    int rc = sgemm_small(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC);
    if (rc >= 0) return rc;
    if (impl == 5) return fail("sgemm: M=%ld N=%ld K=%ld is not a small product", M, N, K);
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
CGTB_API int cgtb_sgemm_batched(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA,
                                const float* B, long ldb, long strideB, float* C, long ldc, long strideC, int impl) {
  return cgtb::sgemm_dispatch(tA, tB, P, M, N, K, A, lda, strideA, B, ldb, strideB, C, ldc, strideC, impl);
}
