// Device helpers shared by the tcgen05 GEMM kernels: mbarriers with bounded waits, the 3xTF32 split,
// the K-major 128-byte-swizzled tile layout, UMMA descriptors and the MMA / commit instructions.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace cgtb {
namespace tc {

constexpr int kBK = 32;      // K depth of one stage: 32 floats = one 128-byte swizzle row
constexpr int kXRows = 128;  // UMMA M
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr long long kWaitCycles = 2000000000LL;  // about one second of SM clock: far beyond any legitimate wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive and announce `bytes` of asynchronous copies that will complete on this barrier
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// bounded wait: false when the phase did not complete within the cycle budget
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if ((spin & 1023u) == 1023u && clock64() - t0 > kWaitCycles) return false;
    if (mbar_try(bar, parity)) return true;
  }
  return false;
}
// bounded wait that also gives up as soon as another role of the CTA has raised `*abort_flag`
__device__ __forceinline__ bool mbar_wait_or_abort(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;   // the common case in a pipeline that runs ahead: no clock read
  const long long t0 = clock64();
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 255u) == 255u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) return false;
    }
  }
  return false;
}
// bounded, abortable wait for a role that has nothing else to do for a long time (epilogue warps waiting for a whole
// tile): sleeps between polls so that it does not take issue slots and shared-memory bandwidth from the working warps
__device__ __forceinline__ bool mbar_wait_sleepy(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
  const long long t0 = clock64();
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try(bar, parity)) return true;
    __nanosleep(400);
    if ((spin & 15u) == 15u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) return false;
    }
  }
  return false;
}
// the same for a converged warp: lane 0 waits, the other lanes sleep at the shuffle; afterwards every
// lane observes the completed phase itself, so the data the barrier guards is visible to each of them
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const volatile int* abort_flag, int lane) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait_or_abort(bar, parity, abort_flag) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (ok) (void)mbar_try(bar, parity);
  return ok != 0;
}

// 3xTF32 split: hi = x rounded to TF32's 11 significant bits, lo = x - hi (exact in fp32) cut to TF32.
//
// Which pipe does the work decides the speed of these kernels: cvt.rna.tf32.f32 issues at 16 lanes per
// clock per SM and integer adds / masks / selects at 64, while fp32 multiplies and adds issue at 128.
// So hi is rounded with Dekker's splitting (c = 8193*x; hi = c - (c - x): three fp32 operations,
// round to nearest), lo needs one mask, and the guard for non-finite values is evaluated once per four
// elements on the sum of the residuals. Non-finite inputs, and finite ones so large that 8193*x
// overflows, take the slow path: hi = x with its low mantissa bits cleared (NaN stays NaN, inf stays
// inf), lo = the rest or 0.
__device__ __forceinline__ void split_tf32_slow(float x, uint32_t& hi, uint32_t& lo) {
  const uint32_t b = __float_as_uint(x);
  const uint32_t h = b & 0xFFFFE000u;
  const float r = __fadd_rn(x, -__uint_as_float(h));
  const bool finite = fabsf(r) <= 3.0e38f;         // false for inf - inf and for NaN
  hi = finite ? h : (b | ((b & 0x1FFFu) ? 0x2000u : 0u)) & 0xFFFFE000u;  // keep a NaN's mantissa non-zero
  lo = finite ? (__float_as_uint(r) & 0xFFFFE000u) : 0u;
}
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  const float c = __fmul_rn(x, 8193.0f);
  const float h = __fadd_rn(c, -__fadd_rn(c, -x));
  const float r = __fadd_rn(x, -h);
  if (fabsf(r) <= 3.0e38f) {
    hi = __float_as_uint(h);
    lo = __float_as_uint(r) & 0xFFFFE000u;
  } else {
    split_tf32_slow(x, hi, lo);
  }
}
// four elements at once (one 16-byte chunk of a tile row)
__device__ __forceinline__ void split_tf32x4(float x0, float x1, float x2, float x3, uint4& hi, uint4& lo) {
  const float c0 = __fmul_rn(x0, 8193.0f), c1 = __fmul_rn(x1, 8193.0f), c2 = __fmul_rn(x2, 8193.0f), c3 = __fmul_rn(x3, 8193.0f);
  const float h0 = __fadd_rn(c0, -__fadd_rn(c0, -x0)), h1 = __fadd_rn(c1, -__fadd_rn(c1, -x1));
  const float h2 = __fadd_rn(c2, -__fadd_rn(c2, -x2)), h3 = __fadd_rn(c3, -__fadd_rn(c3, -x3));
  const float r0 = __fadd_rn(x0, -h0), r1 = __fadd_rn(x1, -h1), r2 = __fadd_rn(x2, -h2), r3 = __fadd_rn(x3, -h3);
  // each residual is below 2^-11 of its element, so the sum overflows or is NaN only if one of them is
  const float s = __fadd_rn(__fadd_rn(fabsf(r0), fabsf(r1)), __fadd_rn(fabsf(r2), fabsf(r3)));
  if (s <= 3.0e38f) {
    hi = make_uint4(__float_as_uint(h0), __float_as_uint(h1), __float_as_uint(h2), __float_as_uint(h3));
    lo = make_uint4(__float_as_uint(r0) & 0xFFFFE000u, __float_as_uint(r1) & 0xFFFFE000u, __float_as_uint(r2) & 0xFFFFE000u,
                    __float_as_uint(r3) & 0xFFFFE000u);
  } else {
    split_tf32_slow(x0, hi.x, lo.x);
    split_tf32_slow(x1, hi.y, lo.y);
    split_tf32_slow(x2, hi.z, lo.z);
    split_tf32_slow(x3, hi.w, lo.w);
  }
}

// byte offset of element (row, k) inside a K-major tile with 128-byte rows and the 128B swizzle:
// 16-byte chunk index XOR (row mod 8); 8-row groups are 1024 bytes apart
__device__ __forceinline__ uint32_t tile_off(int row, int k) {
  return (uint32_t)row * 128u + ((((uint32_t)k >> 2) ^ ((uint32_t)row & 7u)) << 4) + (((uint32_t)k & 3u) << 2);
}

// shared-memory matrix descriptor: K-major, SWIZZLE_128B, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);      // start address, 16-byte units
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                       // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
  return d;
}

// shared-memory matrix descriptor of an MN-major 32-bit operand (the M or N index runs along the 128-byte rows, one row
// per K index). For 32-bit elements the only MN-major layout of the tensor core is the 128-byte swizzle with 32-byte
// atoms (layout type 1; what CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B writes): 32 consecutive M/N elements x 4 K rows
// form one 512-byte atom in which the 32-byte chunks of row r are permuted by r % 4. `lbo` = bytes from one group of 32
// M/N elements to the next; groups of 4 K rows are 512 bytes apart (dense rows).
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t saddr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;
  return d;
}
// instruction descriptor as below with both operands MN-major
__device__ __forceinline__ uint32_t make_idesc_tf32_mn(int un) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(un >> 3) << 17) | ((uint32_t)(kXRows >> 4) << 24);
}

// instruction descriptor: D fp32, A/B tf32, both K-major, N = un, M = 128
__device__ __forceinline__ uint32_t make_idesc_tf32(int un) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(un >> 3) << 17) | ((uint32_t)(kXRows >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
// same, executed by a converged warp: one elected lane issues, operands stay warp-uniform
__device__ __forceinline__ void mma_tf32_elect(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
// issued by a thread that is already alone in its branch (e.g. inside `if (elect_one())`): no lane mask operand,
// no election per instruction. Measured on B200 for 128 x N x 8 TF32: 49-67 cycles per instruction for N = 32-64
// against 85-110 with the masked, per-instruction-elected form above.
__device__ __forceinline__ void mma_tf32_one(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the same with the A operand in tensor memory (128 lanes x 8 columns at tmem_a)
__device__ __forceinline__ void mma_tf32_ts_one(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 16 consecutive accumulator columns of this warp's 32 TMEM lanes
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 8 consecutive accumulator columns of this warp's 32 TMEM lanes
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace tc

// Optional output stage of a product whose rows are channels-last pixels (a convolution layer): instead of
// C[m, n] the kernel writes t = C[m, n] + bias[n], mask = (t >= 0), y = t * mask as NCHW planes
// y[((m / HW) * N + n) * HW + m % HW]. Only for products that are neither swapped nor split along K.
struct ConvEpilogue {
  const float* bias;
  float* y;
  int8_t* mask;
  long HW;
};

// host-mapped flag that the tensor-core kernels raise on a wait time-out (device address); nullptr on failure
int* tc_error_flag();
// ordered fold of a split-K slab [P][nsplit][M*N] into C
void tc_splitk_fold(long P, long M, long N, int nsplit, const float* part, float* C, long ldc, long strideC);

}  // namespace cgtb
