// Mul22 / BatchedMul22 for 16-byte-aligned operands: the TMA-fed variant of the tcgen05 3xTF32 GEMM.
//
// The products of the configurations are skinny (a 28800 x 800 column matrix against 32 filters), so the
// kernel is a streaming problem: what matters is how many bytes of the big operand are in flight per
// SM. Here the tensor-memory accelerator moves raw fp32 tiles global -> shared memory
// (cp.async.bulk.tensor, completion counted on an mbarrier), so the bytes in flight are set by the
// depth of a ring of raw stages and not by registers or by what the compiler does with the loads.
//
//   warp 9   one thread issues the TMA loads of K block kb into raw stage kb % RS (X tile 128 x 32,
//            Y tile UN x 32) as soon as that stage has been released;
//   warps 0-7 convert raw fp32 into the TF32 operands of the 3xTF32 product, in the K-major
//            128-byte-swizzled layout of the UMMA descriptor, into conversion stage kb % CS:
//            * a K-contiguous X tile arrives already in that layout (TMA SWIZZLE_128B) and the MMA reads
//              it in place as x_hi -- the tensor core uses the upper 19 bits of each word, i.e. x with
//              its low mantissa bits cut -- so only x_lo = x - cut(x) is computed (two fp32-pipe
//              operations and a mask per element, one 16-byte store per four);
//            * a row-contiguous X tile (a transposed source) arrives as [k][row] and is transposed by
//              the conversion's addressing into x_hi and x_lo;
//            * the small Y tile is always converted into y_hi | y_lo, stored back to back;
//   warp 8   issues the MMAs through one elected lane of the converged warp (descriptors stay in
//            uniform registers): per K step x_hi * [y_hi | y_lo] as ONE instruction with 2*UN accumulator
//            columns, and x_lo * y_hi. Two instructions instead of three matter because a 128 x N x 8
//            TF32 instruction costs about 45 cycles for every N <= 64. Its commits release the
//            conversion stage and, for an X tile read in place, the raw stage; it owns the TMEM allocation;
//   after the last block warps 0-7 are the epilogue: TMEM -> registers, add the two column halves,
//            store to C or to the split-K slab (float4 rows, or coalesced columns for a swapped tile).
//
// What was measured on the way (B200): cvt.rna.tf32.f32 runs on the 16-lane conversion pipe and integer
// rounding on the 64-lane integer pipe, either of which made the split, not HBM, the limit; one
// thread issuing tcgen05.mma from divergent code pays ~60 cycles per instruction for moving the
// descriptors into uniform registers; polling an mbarrier from one lane of a diverged warp starves the
// working warps, all lanes polling does not.
//
// Out-of-range rows and the K tail are zero-filled by the TMA unit. Every wait is bounded and
// abortable; on expiry the kernel raises the host-mapped flag, the producer waits for its copies in
// flight, TMEM is freed and the kernel returns.
//
// Eligibility (otherwise the register-fed kernel of gemm_tcgen05.cu runs): base addresses 16-byte
// aligned, leading dimensions and batch strides multiples of 4 floats.
#include <cuda.h>  // CUtensorMap and its enums; the encoder is looked up at run time, libcuda is not linked

#include <algorithm>
#include <cstring>

#include "runtime.h"
#include "tc_util.h"

using namespace cgtb;
using namespace cgtb::tc;

namespace {

constexpr int kConvWarps = 8;
constexpr int kConvThreads = kConvWarps * 32;
constexpr int kThreadsTma = kConvThreads + 64;  // + MMA warp + TMA warp
constexpr int kMaxRaw = 8;
constexpr int kMaxConv = 2;

struct TmaParams {
  float* C;          // output or split-K slab
  long ldc;
  long c_batch_stride;
  int swapped;       // X is op(B): tile row i is product column n
  long K;
  long kchunk;       // K elements per split (multiple of kBK)
  int nsplit;
  long M, N;
  long xrows, yrows; // valid rows of X and Y
  int UN;
  int raw_stages, conv_stages;
  int tmem_cols;
  int* err;
  // tile grid: the CTAs of the (persistent) launch walk it with stride gridDim.x
  int xtiles, ytiles;
  long total_tiles;  // xtiles * ytiles * batches * nsplit
  // Implicit convolution (CONV 1: forward product / data gradient): the X tile of K block kb is not a block of a
  // stored matrix but the window of the NHWC tensor behind mapX that kernel tap (i, j) of that block addresses;
  // see conv_implicit_tma. CONV 2 (filter gradient): see conv_wgrad_tma.
  int csign;            // +1: tap (i, j) reads the source at (y + i - ph, x + j - pw); -1: at (y + ph - i, x + pw - j)
  int cW, cHW;          // width and pixels of an output image
  int cC;               // output channels (= N of the product)
  int ckw, ckpt;        // kernel width; K blocks per tap (source channels / 32)
  int cph, cpw;         // padding
  int crows, cnimg;     // image rows and images per tile
  int cnbands;          // tiles per image when an image spans several tiles
  int cB;               // images
  int cx_tx;            // bytes one X load delivers (the box may be smaller than 128 rows)
  ConvEpilogue ep;      // ep.y != nullptr: bias + relu + NCHW output stage instead of storing C
  // filter gradient (CONV 2)
  int wunits;           // (tap, 32-channel chunk) units = kh*kw*Cs/32; an X tile holds four of them
  int wkk;              // kh*kw
  int wbh, wnrg;        // image rows per K block; K blocks per image
  int wnpx;             // pixels per K block (wbh * width <= 32); the remaining K slots are zero
};

#ifdef CGTB_TMA_TRACE
__device__ long long g_tma_trace[128 * 8];
#define TRACE(kbi, slot) do { if (blockIdx.x == 0 && (kbi) < 128) g_tma_trace[(kbi) * 8 + (slot)] = clock64(); } while (0)
#else
#define TRACE(kbi, slot) do { } while (0)
#endif

struct Tile {
  int xt, yt, batch, split, nkb;
  long k_begin;
};
__device__ __forceinline__ Tile tile_of(const TmaParams& p, long t) {
  Tile c;
  c.xt = (int)(t % p.xtiles);
  const long r = t / p.xtiles;
  c.yt = (int)(r % p.ytiles);
  const int z = (int)(r / p.ytiles);
  c.batch = z / p.nsplit;
  c.split = z - c.batch * p.nsplit;
  c.k_begin = (long)c.split * p.kchunk;
  const long k_end = (c.k_begin + p.kchunk < p.K) ? c.k_begin + p.kchunk : p.K;
  c.nkb = (int)((k_end - c.k_begin + kBK - 1) / kBK);
  return c;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// raw K-major tile (already swizzled by the TMA load): linear pass over 16-byte chunks
__device__ __forceinline__ void convert_kmajor(const unsigned char* raw, unsigned char* hi, unsigned char* lo, int nchunks, int tid) {
  for (int c0 = tid; c0 < nchunks; c0 += 4 * kConvThreads) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * kConvThreads;
      if (c < nchunks) v[u] = *reinterpret_cast<const uint4*>(raw + (size_t)c * 16);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * kConvThreads;
      if (c < nchunks) {
        uint4 h, l;
        split_tf32x4(__uint_as_float(v[u].x), __uint_as_float(v[u].y), __uint_as_float(v[u].z), __uint_as_float(v[u].w), h, l);
        *reinterpret_cast<uint4*>(hi + (size_t)c * 16) = h;
        *reinterpret_cast<uint4*>(lo + (size_t)c * 16) = l;
      }
    }
  }
}

// K-major X tile that the MMA reads in place as the hi operand (the tensor core uses the upper 19 bits
// of each fp32 word): only lo = x - (x with its 13 low mantissa bits cleared) is computed and stored.
// The difference is exact (at most 13 significant bits) and is stored unmasked: the tensor core cuts its low
// bits itself, exactly as it cuts those of x. Non-finite inputs: a NaN stays NaN through x itself; for an
// infinite x the split gives non-finite products whose kind is not defined (the cross term inf * y_lo is NaN
// when y_lo is zero or of the other sign, in every variant of the 3xTF32 scheme), so no guard is spent here.
// The residual has up to 13 significant bits and the tensor core keeps 11 of them by cutting: half a unit of the
// last kept place is added to the bit pattern first, so that the cut rounds to nearest (the error of the product
// falls from 2^-21 to 2^-22 of |x y|, that of a split with a rounded hi part).
__device__ __forceinline__ uint32_t lo_of(uint32_t b) {
  const uint32_t r = __float_as_uint(__fadd_rn(__uint_as_float(b), -__uint_as_float(b & 0xFFFFE000u)));
  return (r & 0x7F800000u) != 0x7F800000u ? r + 0x1000u : r;   // a NaN residual (x was NaN or infinite) stays NaN
}
__device__ __forceinline__ void convert_kmajor_lo(const unsigned char* raw, unsigned char* lo, int nchunks, int tid) {
  for (int c0 = tid; c0 < nchunks; c0 += 4 * kConvThreads) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * kConvThreads;
      if (c < nchunks) v[u] = *reinterpret_cast<const uint4*>(raw + (size_t)c * 16);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * kConvThreads;
      if (c < nchunks) *reinterpret_cast<uint4*>(lo + (size_t)c * 16) = make_uint4(lo_of(v[u].x), lo_of(v[u].y), lo_of(v[u].z), lo_of(v[u].w));
    }
  }
}


// Epilogue of one tile, run by the eight epilogue warps: accumulator (TMEM) -> registers -> global memory.
template <int CONV, int NCOLGROUPS = kConvWarps / 4>
__device__ __forceinline__ void store_tile(const TmaParams& p, const Tile& c, uint32_t tmem_d, int quarter, int colgroup, int lane) {
  const int UN = p.UN;
  const long x0 = (long)c.xt * kXRows, y0 = (long)c.yt * UN;
  // Accumulator -> registers -> global memory. A thread owns tile row (quarter*32 + lane) and 8
  // consecutive columns per chunk (8); columns [0, UN) hold hi*hi + lo*hi and [UN, 2UN) hold hi*lo.
  const int nchunks = UN / 8;
  const int row = quarter * 32 + lane;
  const long i_g = x0 + row;
  const int batch = c.batch, split = c.split;
  float* cbase = (p.nsplit > 1) ? p.C + ((long)batch * p.nsplit + split) * p.M * p.N : p.C + batch * p.c_batch_stride;
  const long ld = (p.nsplit > 1) ? p.N : p.ldc;
  const bool vec_ok = ((ld & 3) == 0) && (((uintptr_t)cbase & 15) == 0);
  // where tile row `row` goes when the result is stored as NCHW planes (implicit convolution, or the output
  // stage of a convolution layer on a stored column matrix)
  bool pvalid = false;
  long pb = 0, ppix = 0, pHW = 1, pC = 1;
  if (CONV == 1) {
    const int tile = c.xt;
    pHW = p.cHW;
    pC = p.cC;
    if (p.cnimg > 1) {
      const int li = row / p.cHW;
      pb = (long)tile * p.cnimg + li;
      ppix = row - li * p.cHW;
      pvalid = li < p.cnimg && pb < p.cB;
    } else {
      pb = tile / p.cnbands;
      ppix = (long)(tile - pb * p.cnbands) * p.crows * p.cW + row;
      pvalid = row < p.crows * p.cW && ppix < p.cHW;
    }
  } else if (CONV == 0 && p.ep.y) {
    pHW = p.ep.HW;
    pC = p.yrows;
    pvalid = i_g < p.xrows;
    pb = i_g / pHW;
    ppix = i_g - pb * pHW;
  }
  // filter gradient: tile row = (unit, channel) -> column (32*chunk + channel)*kh*kw + tap of the result
  long wcol = -1;
  if (CONV == 2) {
    const int unit = c.xt * 4 + (row >> 5);
    if (unit < p.wunits) {
      const int tap = unit / p.ckpt, q = unit - tap * p.ckpt;
      wcol = (long)(32 * q + (row & 31)) * p.wkk + tap;
    }
  }
  for (int ch = colgroup; ch < nchunks; ch += NCOLGROUPS) {
    const int c0 = ch * 8;
    uint32_t r1[8], r2[8];
    const uint32_t taddr = tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
    tmem_ld8(taddr, r1);
    tmem_ld8(taddr + (uint32_t)UN, r2);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r1[j]) + __uint_as_float(r2[j]);
    const long j0 = y0 + c0;
    if (CONV == 2) {
      if (wcol >= 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j0 + j < p.yrows) cbase[(j0 + j) * ld + wcol] = v[j];
      }
    } else if (CONV == 1 || p.ep.y) {
      // NCHW planes: the lanes of a warp write consecutive pixels of one channel plane
      if (pvalid) {
        if (p.ep.y) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (j0 + j < pC) {
              const float tt = v[j] + p.ep.bias[j0 + j];
              const int8_t mk = (int8_t)(tt >= 0.f);
              const size_t o = ((size_t)pb * pC + (j0 + j)) * pHW + ppix;
              p.ep.mask[o] = mk;
              p.ep.y[o] = tt * (float)mk;
            }
          }
        } else {
          // with K splits every split writes its own copy of the whole result; a fold adds them in order
          float* dst = p.C + (size_t)split * p.cB * pC * pHW + ((size_t)pb * pC + j0) * pHW + ppix;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j0 + j < pC) dst[(size_t)j * pHW] = v[j];
        }
      }
    } else if (i_g < p.xrows) {
      if (!p.swapped) {  // tile row = product row: 32 contiguous bytes per thread
        float* dst = cbase + i_g * ld + j0;
        if (vec_ok && j0 + 8 <= p.yrows) {
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j0 + j < p.yrows) dst[j] = v[j];
        }
      } else {           // tile row = product column: the lanes of a warp write consecutive addresses
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j0 + j < p.yrows) cbase[(j0 + j) * ld + i_g] = v[j];
      }
    }
  }
}

// One CTA walks tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... of the tile grid (persistent launch): the
// barriers, the TMEM allocation and the tensor-map fetch are paid once per CTA, and the TMA producer runs ahead
// across tile boundaries, so that the K blocks of the next tile are in flight while this tile's accumulator is
// being stored. Ring positions and barrier phases run on over the tiles.
template <bool XMN, bool YMN, int CONV>
__global__ void __launch_bounds__(kThreadsTma, 2)
sgemm_tma_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY, const TmaParams p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t raw_full[kMaxRaw];
  __shared__ __align__(8) uint64_t raw_empty[kMaxRaw];
  __shared__ __align__(8) uint64_t conv_full[kMaxConv];
  __shared__ __align__(8) uint64_t conv_empty[kMaxConv];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int UN = p.UN, RS = p.raw_stages, CS = p.conv_stages;
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t x_bytes = kXRows * 128u, y_bytes = (uint32_t)UN * 128u;
  // The X tile is the MMA's hi operand as it lies in the raw stage, whatever its storage order: a K-major tile is a
  // box of 128 rows x 128 bytes (128-byte swizzle), an MN-major tile four boxes of 32 K rows x 128 bytes (32 rows of
  // the operand each; 128-byte swizzle with 32-byte atoms, the tensor core's only MN-major layout for 32-bit
  // elements), and the MMA's descriptors name the order. No transposition anywhere: only x_lo, y_hi (a copy) and
  // y_lo are produced, by linear passes over 16-byte chunks that do not need to know the layout.
  constexpr bool XDIRECT = true;
  const uint32_t cx_bytes = XDIRECT ? x_bytes : 2 * x_bytes;  // conversion stage: [X hi] X lo, Y hi, Y lo
  const uint32_t conv_bytes = cx_bytes + 2 * y_bytes, raw_bytes = x_bytes + y_bytes;
  unsigned char* conv0 = smem;
  unsigned char* raw0 = smem + (size_t)CS * conv_bytes;
  volatile int* abortp = &abort_flag;

  if (tid == 0) {
    for (int s = 0; s < RS; ++s) {
      mbar_init(smem_u32(&raw_full[s]), 1);
      mbar_init(smem_u32(&raw_empty[s]), XDIRECT ? 1 : kConvWarps);  // released by the MMAs' commit / by the converters
    }
    for (int s = 0; s < CS; ++s) {
      mbar_init(smem_u32(&conv_full[s]), kConvWarps);
      mbar_init(smem_u32(&conv_empty[s]), 1);
    }
    mbar_init(smem_u32(&accum_bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (CONV == 2 && p.wnpx < kBK) {
    // a K block holds wnpx < 32 pixel rows; the TMA boxes never write rows wnpx..31 of the 32-row sub-tiles, and the
    // MMAs read all 32: those rows are zeroed once, in every raw stage, and stay zero
    const int subtiles = (int)(raw_bytes / 4096u), tail16 = (kBK - p.wnpx) * 8;   // 16-byte chunks per sub-tile tail
    for (int i = tid; i < RS * subtiles * tail16; i += kThreadsTma) {
      const int st = i / (subtiles * tail16), r = i - st * subtiles * tail16, sub = r / tail16, c = r - sub * tail16;
      *reinterpret_cast<uint4*>(raw0 + (size_t)st * raw_bytes + (size_t)sub * 4096 + (size_t)p.wnpx * 128 + (size_t)c * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kConvWarps) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;

  if (warp < kConvWarps) {
    // ------------------------------------------------ converters, then the tile's epilogue
    int rs = 0, cs = 0;
    int tkb = 0;
    (void)tkb;
    uint32_t rphase = 0, cphase = 0, it = 0;
    for (long t = blockIdx.x; t < p.total_tiles; t += gridDim.x, ++it) {
      const Tile c = tile_of(p, t);
      bool ok = true;
      for (int kb = 0; kb < c.nkb; ++kb) {
        ok = mbar_wait_or_abort(smem_u32(&raw_full[rs]), rphase, abortp);
        if (tid == 0) TRACE(tkb, 1);
        ok = ok && mbar_wait_or_abort(smem_u32(&conv_empty[cs]), cphase ^ 1u, abortp);
        if (tid == 0) TRACE(tkb, 2);
        if (!ok) break;
        const unsigned char* rx = raw0 + (size_t)rs * raw_bytes;
        const unsigned char* ry = rx + x_bytes;
        unsigned char* cx = conv0 + (size_t)cs * conv_bytes;
        unsigned char* cy = cx + cx_bytes;
        convert_kmajor_lo(rx, cx, kXRows * 8, tid);          // x_lo in the raw tile's own layout
        if (tid == 0) TRACE(tkb, 6);
        convert_kmajor(ry, cy, cy + y_bytes, UN * 8, tid);   // [y_hi | y_lo], likewise
        if (tid == 0) TRACE(tkb, 7);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&conv_full[cs]));
          if (!XDIRECT) mbar_arrive(smem_u32(&raw_empty[rs]));
        }
        if (tid == 0) TRACE(tkb, 3);
        ++tkb;
        if (++rs == RS) { rs = 0; rphase ^= 1u; }
        if (++cs == CS) { cs = 0; cphase ^= 1u; }
      }
      // ---------------------------------------------- epilogue of this tile
      if (ok && c.nkb > 0) ok = mbar_wait_or_abort(smem_u32(&accum_bar), it & 1u, abortp);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (!ok) *abortp = 1;
      asm volatile("bar.sync 1, %0;" ::"n"(kConvThreads) : "memory");  // the epilogue warps agree on success
      if (*abortp) {
        if (tid == 0) { *(volatile int*)p.err = 3; __threadfence_system(); }
        break;
      }
      store_tile<CONV>(p, c, tmem_d, warp & 3, warp >> 2, lane);
      // this warp's reads of the accumulator are complete before it signals anything for the next tile (the
      // first MMA of the next tile waits for a conversion that every epilogue warp takes part in)
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
  } else if (warp == kConvWarps) {
    // ------------------------------------------------ MMA issuer
    // ONE thread runs the loop: it waits for the stage, issues all MMAs of the K block and commits (no election, no
    // lane-mask operand per instruction, no warp-wide poll of the barrier and no warp synchronisation per K block:
    // the issue loop is what bounds these kernels, 45-50 cycles per tcgen05.mma). Two instructions per K step:
    // x_hi * [y_hi | y_lo] into columns [0, 2UN) and x_lo * y_hi into columns [0, UN).
    const uint32_t major_bits = (XMN ? (1u << 15) : 0u) | (YMN ? (1u << 16) : 0u);   // operand A / B is MN-major
    const uint32_t idesc1 = make_idesc_tf32(UN) | major_bits, idesc2 = make_idesc_tf32(2 * UN) | major_bits;
    bool ok = true;
    int rs = 0, cs = 0;
    int tkb = 0;
    (void)tkb;
    uint32_t cphase = 0;
    if (elect_one())
    for (long t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      const Tile c = tile_of(p, t);
      for (int kb = 0; kb < c.nkb; ++kb) {
        ok = mbar_wait_or_abort(smem_u32(&conv_full[cs]), cphase, abortp);
        if (!ok) break;
        TRACE(tkb, 4);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sbase = smem_u32(conv0 + (size_t)cs * conv_bytes);
        const uint32_t xh_addr = XDIRECT ? smem_u32(raw0 + (size_t)rs * raw_bytes) : sbase;
        const uint32_t xl_addr = XDIRECT ? sbase : sbase + x_bytes;
        // MN-major operands: groups of 32 rows of the operand (the four boxes of X, the groups of [y_hi | y_lo]) lie
        // 4096 bytes apart
        const uint64_t dxh = XMN ? make_desc_mn(xh_addr, 4096u) : make_desc(xh_addr);
        const uint64_t dxl = XMN ? make_desc_mn(xl_addr, 4096u) : make_desc(xl_addr);
        const uint64_t dyh = YMN ? make_desc_mn(sbase + cx_bytes, 4096u) : make_desc(sbase + cx_bytes);  // y_lo follows y_hi: one descriptor covers both
#pragma unroll
        for (int kk = 0; kk < kBK / 8; ++kk) {
          // K-major: 8 tf32 = 32 bytes along K inside the swizzle row; MN-major: 8 K rows = 1024 bytes
          const uint64_t advx = (uint64_t)((kk * (XMN ? 1024 : 32)) >> 4), advy = (uint64_t)((kk * (YMN ? 1024 : 32)) >> 4);
          const uint32_t first = (kb == 0 && kk == 0) ? 0u : 1u;
          mma_tf32_one(tmem_d, dxh + advx, dyh + advy, idesc2, first);
          mma_tf32_one(tmem_d, dxl + advx, dyh + advy, idesc1, 1u);
        }
        mma_commit(smem_u32(&conv_empty[cs]));
        if (XDIRECT) mma_commit(smem_u32(&raw_empty[rs]));
        TRACE(tkb, 5);
        ++tkb;
        if (++rs == RS) rs = 0;
        if (++cs == CS) { cs = 0; cphase ^= 1u; }
      }
      if (ok && c.nkb > 0) mma_commit(smem_u32(&accum_bar));
    }
    if (!ok) { *abortp = 1; *(volatile int*)p.err = 4; __threadfence_system(); }
    __syncwarp();
  } else if (CONV == 2) {
    // ------------------------------------------------ TMA producer of the filter-gradient product (one warp)
    // A K block of this product is five boxes (four shifted windows of the source, one of the gradient), and one
    // thread needs some 400 cycles to issue a 4-D box: issued by one thread, the loads, not the tensor core, set the
    // pace of the loop. Here lane u issues box u; lane 0 alone waits for the stage and arms its barrier.
    long issued = 0;
    bool ok = true;
    int rs = 0;
    uint32_t rphase = 0;
    for (long t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      const Tile c = tile_of(p, t);
      const long y0 = (long)c.yt * UN;
      for (int kb = 0; kb < c.nkb; ++kb) {
        if (lane == 0) ok = mbar_wait_or_abort(smem_u32(&raw_empty[rs]), rphase ^ 1u, abortp);
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
        if (lane == 0) TRACE((int)issued, 0);
        const uint32_t bar = smem_u32(&raw_full[rs]);
        const int k0 = (int)(c.k_begin + (long)kb * kBK);
        const uint32_t dx = smem_u32(raw0 + (size_t)rs * raw_bytes);
        const int gkb = k0 / kBK;
        const int b = gkb / p.wnrg, yrow0 = (gkb - b * p.wnrg) * p.wbh;
        int nunits = p.wunits - c.xt * 4;
        nunits = nunits > 4 ? 4 : nunits;
        const uint32_t px_bytes = (uint32_t)p.wnpx * 128u;
        if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)nunits * px_bytes + (uint32_t)p.wnpx * (uint32_t)UN * 4u);
        __syncwarp();
        if (lane < nunits) {
          const int unit = c.xt * 4 + lane;
          const int tap = unit / p.ckpt, q = unit - tap * p.ckpt;
          const int ti = tap / p.ckw, tj = tap - ti * p.ckw;
          tma_load_4d(dx + (uint32_t)lane * 4096u, &mapX, 32 * q, tj - p.cpw, yrow0 + ti - p.cph, b, bar);
        } else if (lane >= 4 && lane < 4 + UN / 32) {
          // the gradient's tile as groups of 32 channels, each a sub-tile of 32 pixel rows x 128 bytes
          const int g = lane - 4;
          tma_load_4d(dx + x_bytes + (uint32_t)g * 4096u, &mapY, (int)y0 + 32 * g, 0, yrow0, b, bar);
        }
        __syncwarp();
        ++issued;
        if (++rs == RS) { rs = 0; rphase ^= 1u; }
      }
    }
    if (lane == 0 && (!ok || *abortp)) {
      *abortp = 1;
      *(volatile int*)p.err = 5;
      __threadfence_system();
      // copies already issued still write this CTA's shared memory: wait (bounded) until they have landed
      for (long j = (issued > RS ? issued - RS : 0); j < issued; ++j) mbar_wait(smem_u32(&raw_full[j % RS]), (uint32_t)(j / RS) & 1u);
    }
  } else if (CONV == 0) {
    // ------------------------------------------------ TMA producer of the plain product (one warp)
    // lanes 0..3 issue the boxes of X (one when K-major, four groups of 32 rows when MN-major), lanes 4.. those of Y
    // (one, or UN / 32 groups); lane 0 alone waits for the stage and arms its barrier. Rows and K indices beyond the
    // operand are zero-filled by the TMA unit.
    long issued = 0;
    bool ok = true;
    int rs = 0;
    uint32_t rphase = 0;
    const int nx = XMN ? 4 : 1, ny = YMN ? UN / 32 : 1;
    for (long t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      const Tile c = tile_of(p, t);
      const long x0 = (long)c.xt * kXRows, y0 = (long)c.yt * UN;
      for (int kb = 0; kb < c.nkb; ++kb) {
        if (lane == 0) ok = mbar_wait_or_abort(smem_u32(&raw_empty[rs]), rphase ^ 1u, abortp);
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
        if (lane == 0) TRACE((int)issued, 0);
        const uint32_t bar = smem_u32(&raw_full[rs]);
        const int k0 = (int)(c.k_begin + (long)kb * kBK);
        const uint32_t dx = smem_u32(raw0 + (size_t)rs * raw_bytes);
        if (lane == 0) mbar_arrive_expect_tx(bar, raw_bytes);
        __syncwarp();
        if (lane < nx) {
          if (XMN) tma_load_3d(dx + (uint32_t)lane * 4096u, &mapX, (int)x0 + 32 * lane, k0, c.batch, bar);
          else tma_load_3d(dx, &mapX, k0, (int)x0, c.batch, bar);
        } else if (lane >= 4 && lane < 4 + ny) {
          const int g = lane - 4;
          if (YMN) tma_load_3d(dx + x_bytes + (uint32_t)g * 4096u, &mapY, (int)y0 + 32 * g, k0, c.batch, bar);
          else tma_load_3d(dx + x_bytes, &mapY, k0, (int)y0, c.batch, bar);
        }
        __syncwarp();
        ++issued;
        if (++rs == RS) { rs = 0; rphase ^= 1u; }
      }
    }
    if (lane == 0 && (!ok || *abortp)) {
      *abortp = 1;
      *(volatile int*)p.err = 5;
      __threadfence_system();
      // copies already issued still write this CTA's shared memory: wait (bounded) until they have landed
      for (long j = (issued > RS ? issued - RS : 0); j < issued; ++j) mbar_wait(smem_u32(&raw_full[j % RS]), (uint32_t)(j / RS) & 1u);
    }
  } else if (lane == 0) {
    // ------------------------------------------------ TMA producer of the per-tap implicit convolution (one thread)
    long issued = 0;
    bool ok = true;
    int rs = 0;
    uint32_t rphase = 0;
    for (long t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      const Tile c = tile_of(p, t);
      const long x0 = (long)c.xt * kXRows, y0 = (long)c.yt * UN;
      for (int kb = 0; kb < c.nkb; ++kb) {
        ok = mbar_wait_or_abort(smem_u32(&raw_empty[rs]), rphase ^ 1u, abortp);
        if (!ok) break;
        TRACE((int)issued, 0);
        const uint32_t bar = smem_u32(&raw_full[rs]);
        const int k0 = (int)(c.k_begin + (long)kb * kBK);
        const uint32_t dx = smem_u32(raw0 + (size_t)rs * raw_bytes);
        if (CONV == 1) {
          // tap (i, j) of this K block reads the tensor shifted by csign * (i - ph, j - pw); rows and columns that
          // fall outside the tensor are zero-filled by the TMA unit: that is the convolution's padding
          mbar_arrive_expect_tx(bar, (uint32_t)p.cx_tx + y_bytes);
          const int gkb = k0 / kBK;  // K block within the whole product (this tile may hold one K split)
          const int tap = gkb / p.ckpt, q = gkb - tap * p.ckpt;
          const int ti = tap / p.ckw, tj = tap - ti * p.ckw;
          const int tile = c.xt;
          const int b0 = p.cnimg > 1 ? tile * p.cnimg : tile / p.cnbands;
          const int yrow0 = p.cnimg > 1 ? 0 : (tile - b0 * p.cnbands) * p.crows;
          tma_load_4d(dx, &mapX, 32 * q, p.csign * (tj - p.cpw), yrow0 + p.csign * (ti - p.cph), b0, bar);
          tma_load_3d(dx + x_bytes, &mapY, k0, (int)y0, c.batch, bar);
        }
        ++issued;
        if (++rs == RS) { rs = 0; rphase ^= 1u; }
      }
    }
    if (!ok || *abortp) {
      *abortp = 1;
      *(volatile int*)p.err = 5;
      __threadfence_system();
      // copies already issued still write this CTA's shared memory: wait (bounded) until they have landed
      for (long j = (issued > RS ? issued - RS : 0); j < issued; ++j) mbar_wait(smem_u32(&raw_full[j % RS]), (uint32_t)(j / RS) & 1u);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kConvWarps) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)p.tmem_cols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// Implicit convolution (forward product / data gradient) with the input tile resident in shared memory and the
// X operand in tensor memory.
//
// What bounds sgemm_tma_kernel<.., 1> above (measured on B200 with per-role cycle stamps): every kernel tap re-loads
// its shifted window of the input through the TMA unit (25 boxes of 15 KB per tile of a 5x5 convolution: the L2
// -> SM path saturates), every tcgen05.mma re-reads its 4 KB X operand from shared memory, and one thread needs a
// thousand cycles to issue the loads of one K block. Here
//   * the input rows a tile needs, with their halo, are loaded ONCE per tile (one box per 32 channels) into a
//     double-buffered shared-memory tile; tap (i, j) of the convolution is then only a different row offset when
//     the conversion warps read their pixel's 32 channels;
//   * the conversion warps write x and x_lo = x - cut(x) straight into tensor memory (tcgen05.st), from where the
//     MMAs take their A operand: shared memory carries the input tile once plus the small filter tiles;
//   * the filter bank is split once per call into K-major [2][N][K] (hi, lo) by split_rows_kernel, so the TMA
//     unit delivers [w_hi | w_lo] in its final layout: one box per K block, no conversion in the loop;
//   * per K block ONE elected thread issues the eight MMAs and the commits.
// One CTA per SM (it owns all 512 TMEM columns: accumulator + ring of A stages), persistent over the tile grid.
//   warp 17   halo producer: the tile's input rows into halo buffer it % HB
//   warp 18   filter producer: [w_hi | w_lo] of K block g into ring stage g % WS
//   warps 0-15 pixel rows -> registers -> (x, x_lo) -> TMEM A stage g % AS (four groups of four warps, group g % 4);
//             after the tile's last block: epilogue
//   warp 16   MMAs: D[0,2UN) += A_hi * [w_hi|w_lo], D[0,UN) += A_lo * w_hi; commits release the A stage and the filter stage
// ------------------------------------------------------------------------------------------------
constexpr int kMaxA = 8;
constexpr int kGroups = 4;                                  // conversion groups of four warps (one per TMEM lane quarter)
constexpr int kCvtWarps = 4 * kGroups;
constexpr int kCvtThreads = 32 * kCvtWarps;
constexpr int kEpiWarps = 4;                                // epilogue warps (one per TMEM lane quarter)
constexpr int kThreadsConv = kCvtThreads + 3 * 32 + 32 * kEpiWarps;

struct ConvTsaParams {
  TmaParams t;           // tile grid, convolution geometry, epilogue (raw_stages = filter stages, conv_stages = A stages)
  int hw, hh;            // halo tile: (Wd + kw - 1) columns, (crows + kh - 1) rows per image
  int kh;
  int halo_bufs;         // 1 or 2
  uint32_t chunk_bytes;  // one 32-channel plane of the halo tile, rounded up to 1024 bytes
  int hx0, hy0;          // source coordinates of halo element (0, 0) relative to the tile's first output pixel
  int nacc;              // accumulators in TMEM (2: the epilogue of a tile overlaps the MMAs of the next)
  int acc_cols;          // TMEM columns of one accumulator
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}

__global__ void __launch_bounds__(kThreadsConv, 1)
conv_tsa_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY, const ConvTsaParams cp) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t halo_full[2];
  __shared__ __align__(8) uint64_t halo_empty[2];
  __shared__ __align__(8) uint64_t a_full[kMaxA];    // stage s: TMEM A stage s and filter stage s are both ready
  __shared__ __align__(8) uint64_t a_empty[kMaxA];   // the MMAs that read stage s have completed
  __shared__ __align__(8) uint64_t accum_full[2];
  __shared__ __align__(8) uint64_t accum_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const TmaParams& p = cp.t;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int UN = p.UN, AS = p.conv_stages, HB = cp.halo_bufs;  // AS stages: TMEM A stage + filter stage each
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t w_bytes = 2u * (uint32_t)UN * 128u;                  // [w_hi | w_lo] of one K block
  const uint32_t halo_bytes = (uint32_t)p.ckpt * cp.chunk_bytes;
  unsigned char* halo0 = smem;
  unsigned char* w0 = smem + (size_t)HB * halo_bytes;
  const int NACC = cp.nacc;
  const uint32_t acol0 = (uint32_t)(cp.nacc * cp.acc_cols);  // first column of the A stages, behind the accumulator(s)
  volatile int* abortp = &abort_flag;

  if (tid == 0) {
    for (int s = 0; s < HB; ++s) {
      mbar_init(smem_u32(&halo_full[s]), 1);
      mbar_init(smem_u32(&halo_empty[s]), kCvtWarps);
    }
    for (int s = 0; s < AS; ++s) {
      mbar_init(smem_u32(&a_full[s]), 5);   // the four warps of one conversion group + the filter producer (with its bytes)
      mbar_init(smem_u32(&a_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&accum_full[s]), 1);
      mbar_init(smem_u32(&accum_empty[s]), kEpiWarps);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kCvtWarps) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;

  if (warp < kCvtWarps) {
    // ------------------------------------------------ pixel rows -> tensor memory, then the tile's epilogue
    // Sixteen warps in four groups; group g converts K blocks g, g + 4, ... of the CTA's block sequence (a block's
    // conversion is a short chain of dependent steps -- shared-memory loads, the split, tcgen05.st, its wait, the
    // arrival -- so four blocks in flight hide that latency). Within a group warp w serves TMEM lanes 32*(w%4)..+31:
    // a thread owns one pixel of the tile and all 32 channels of the K block.
    const int quarter = warp & 3, group = warp >> 2;
    const int row = quarter * 32 + lane;   // tile row = TMEM lane = pixel of the tile
    // halo row of this pixel for tap (0, 0); rows of the tile that hold no pixel read row 0 (never stored)
    int base_row = 0;
    {
      int li = 0, pix = row;
      if (p.cnimg > 1) { li = row / p.cHW; pix = row - li * p.cHW; }
      const int ly = pix / p.cW, lx = pix - ly * p.cW;
      if (li < p.cnimg && ly < p.crows) base_row = (li * cp.hh + ly) * cp.hw + lx;
    }
    int as = 0;
    int tkb = 0;
    (void)tkb;
    uint32_t aphase = 0, it = 0, g4 = 0;   // g4: the CTA's K block count modulo 4
    for (long t = blockIdx.x; t < p.total_tiles; t += gridDim.x, ++it) {
      const Tile c = tile_of(p, t);
      const int hb = HB > 1 ? (int)(it & 1u) : 0;
      const uint32_t hphase = HB > 1 ? (it >> 1) & 1u : it & 1u;
      bool ok = mbar_wait_or_abort(smem_u32(&halo_full[hb]), hphase, abortp);
      if (tid == 0) TRACE(tkb, 1);
      const unsigned char* halo = halo0 + (size_t)hb * halo_bytes;
      // K block of the whole product = (tap, channel chunk); (ti, tj) = the tap's kernel row and column
      const int gkb = (int)(c.k_begin / kBK);
      int tap = gkb / p.ckpt, q = gkb - tap * p.ckpt;
      int ti = tap / p.ckw, tj = tap - ti * p.ckw;
      for (int kb = 0; kb < c.nkb && ok; ++kb) {
        if ((int)g4 == group) {
          ok = mbar_wait_or_abort(smem_u32(&a_empty[as]), aphase ^ 1u, abortp);
          if (!ok) break;
          if (tid == 0) TRACE(tkb, 2);
          const int oi = p.csign > 0 ? ti : cp.kh - 1 - ti, oj = p.csign > 0 ? tj : p.ckw - 1 - tj;
          const int hr = base_row + oi * cp.hw + oj;
          const uint4* rowp = reinterpret_cast<const uint4*>(halo + (size_t)q * cp.chunk_bytes + (size_t)hr * 128);
          uint32_t hi[32], lo[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 u = rowp[j ^ (hr & 7)];  // 16-byte chunks swizzled by the TMA unit
            hi[4 * j] = u.x; hi[4 * j + 1] = u.y; hi[4 * j + 2] = u.z; hi[4 * j + 3] = u.w;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) lo[j] = lo_of(hi[j]);
          if (tid == 0) TRACE(tkb, 6);
          const uint32_t taddr = tmem_d + ((uint32_t)(quarter * 32) << 16) + acol0 + (uint32_t)as * 64u;
          tmem_st32(taddr, hi);
          tmem_st32(taddr + 32u, lo);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          if (tid == 0) TRACE(tkb, 7);
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&a_full[as]));
          if (tid == 0) TRACE(tkb, 3);
        }
        ++tkb;
        g4 = (g4 + 1u) & 3u;
        if (++as == AS) { as = 0; aphase ^= 1u; }
        if (++q == p.ckpt) {
          q = 0;
          ++tap;
          if (++tj == p.ckw) { tj = 0; ++ti; }
        }
      }
      // this warp has read all it needs of the halo tile
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&halo_empty[hb]));
      if (!ok) {
        if (lane == 0) { *abortp = 1; *(volatile int*)p.err = 3; __threadfence_system(); }
        break;
      }
    }
  } else if (warp == kCvtWarps) {
    // ------------------------------------------------ MMA issuer (one thread: waits, issues the K block's MMAs, commits)
    const uint32_t idesc1 = make_idesc_tf32(UN), idesc2 = make_idesc_tf32(2 * UN);
    bool ok = true;
    int as = 0;
    int tkb = 0;
    (void)tkb;
    uint32_t aphase = 0;
    uint32_t it = 0;
    if (elect_one())
    for (long t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
      const Tile c = tile_of(p, t);
      // accumulator it % NACC: the epilogue warps must have drained its previous tile
      const int ab = NACC > 1 ? (int)(it & 1u) : 0;
      const uint32_t use = NACC > 1 ? it >> 1 : it;
      ok = mbar_wait_or_abort(smem_u32(&accum_empty[ab]), (use & 1u) ^ 1u, abortp);
      if (!ok) break;
      const uint32_t tmem_acc = tmem_d + (uint32_t)(ab * cp.acc_cols);
      for (int kb = 0; kb < c.nkb; ++kb) {
        ok = mbar_wait_or_abort(smem_u32(&a_full[as]), aphase, abortp);
        if (!ok) break;
        TRACE(tkb, 4);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_hi = tmem_d + acol0 + (uint32_t)as * 64u, a_lo = a_hi + 32u;
        const uint64_t dyh = make_desc(smem_u32(w0 + (size_t)as * w_bytes));  // w_lo follows w_hi
#pragma unroll
        for (int kk = 0; kk < kBK / 8; ++kk) {
          const uint64_t adv = (uint64_t)((kk * 32) >> 4);
          const uint32_t first = (kb == 0 && kk == 0) ? 0u : 1u;
          mma_tf32_ts_one(tmem_acc, a_hi + (uint32_t)(kk * 8), dyh + adv, idesc2, first);
          mma_tf32_ts_one(tmem_acc, a_lo + (uint32_t)(kk * 8), dyh + adv, idesc1, 1u);
        }
        mma_commit(smem_u32(&a_empty[as]));
        TRACE(tkb, 5);
        ++tkb;
        if (++as == AS) { as = 0; aphase ^= 1u; }
      }
      if (ok) mma_commit(smem_u32(&accum_full[ab]));
    }
    if (!ok) { *abortp = 1; *(volatile int*)p.err = 4; __threadfence_system(); }
    __syncwarp();
  } else if (warp == kCvtWarps + 1) {
    if (lane == 0) {
      // ---------------------------------------------- halo producer: the input rows of tile `it` into buffer it % HB
      bool ok = true;
      uint32_t it = 0;
      long issued = 0;
      for (long t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
        const Tile c = tile_of(p, t);
        const int hb = HB > 1 ? (int)(it & 1u) : 0;
        const uint32_t hphase = HB > 1 ? (it >> 1) & 1u : it & 1u;
        ok = mbar_wait_or_abort(smem_u32(&halo_empty[hb]), hphase ^ 1u, abortp);
        if (!ok) break;
        const int tile = c.xt;
        const int b0 = p.cnimg > 1 ? tile * p.cnimg : tile / p.cnbands;
        const int yrow0 = p.cnimg > 1 ? 0 : (tile - b0 * p.cnbands) * p.crows;
        const uint32_t bar = smem_u32(&halo_full[hb]);
        mbar_arrive_expect_tx(bar, (uint32_t)p.ckpt * (uint32_t)p.cx_tx);
        const uint32_t dst = smem_u32(halo0 + (size_t)hb * halo_bytes);
        for (int q = 0; q < p.ckpt; ++q) tma_load_4d(dst + (uint32_t)q * cp.chunk_bytes, &mapX, 32 * q, cp.hx0, yrow0 + cp.hy0, b0, bar);
        ++issued;
      }
      if (!ok || *abortp) {
        *abortp = 1;
        *(volatile int*)p.err = 5;
        __threadfence_system();
        for (long j = (issued > HB ? issued - HB : 0); j < issued; ++j)
          mbar_wait(smem_u32(&halo_full[HB > 1 ? (j & 1) : 0]), HB > 1 ? (uint32_t)(j >> 1) & 1u : (uint32_t)j & 1u);
      }
    }
  } else if (warp == kCvtWarps + 2) {
   if (lane == 0) {
    // ------------------------------------------------ filter producer: [w_hi | w_lo] of every K block
    bool ok = true;
    int as = 0;
    uint32_t aphase = 0;
    long issued = 0;
    for (long t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      const Tile c = tile_of(p, t);
      const int y0 = c.yt * UN;
      for (int kb = 0; kb < c.nkb; ++kb) {
        ok = mbar_wait_or_abort(smem_u32(&a_empty[as]), aphase ^ 1u, abortp);
        if (!ok) break;
        TRACE((int)issued, 0);
        const uint32_t bar = smem_u32(&a_full[as]);
        mbar_arrive_expect_tx(bar, w_bytes);
        tma_load_3d(smem_u32(w0 + (size_t)as * w_bytes), &mapY, (int)(c.k_begin + (long)kb * kBK), y0, 0, bar);
        ++issued;
        if (++as == AS) { as = 0; aphase ^= 1u; }
      }
    }
    if (!ok || *abortp) {
      *abortp = 1;
      *(volatile int*)p.err = 6;
      __threadfence_system();
      // Copies already issued still write this CTA's shared memory. Their barrier also counts the conversion
      // warps, which may never arrive now: wait for the bytes by polling a bounded time instead.
      const long long t0 = clock64();
      while (clock64() - t0 < 4000000LL) { }
    }
   }
  } else {
    // ------------------------------------------------ epilogue warps: accumulator it % NACC -> global memory
    const int quarter = warp & 3;
    bool ok = true;
    uint32_t it = 0;
    for (long t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
      const Tile c = tile_of(p, t);
      const int ab = NACC > 1 ? (int)(it & 1u) : 0;
      const uint32_t use = NACC > 1 ? it >> 1 : it;
      ok = mbar_wait_sleepy(smem_u32(&accum_full[ab]), use & 1u, abortp);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      store_tile<1, 1>(p, c, tmem_d + (uint32_t)(ab * cp.acc_cols), quarter, 0, lane);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&accum_empty[ab]));
    }
    if (!ok && lane == 0) { *abortp = 1; *(volatile int*)p.err = 7; __threadfence_system(); }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kCvtWarps) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)p.tmem_cols) : "memory");
  }
}

// Y [rows] x [K] (element (r, k) at Y[r*ld + k], or Y[k*ld + r] when `mn`) -> out[0][r][k] = y rounded to TF32,
// out[1][r][k] = the rest cut to TF32, rows of Kp >= K entries, zeros beyond K.
__global__ void split_rows_kernel(const float* __restrict__ Y, long rows, long K, long ld, int mn, float* __restrict__ out, long Kp) {
  const long n = rows * Kp;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = mn ? i % rows : i / Kp, k = mn ? i / rows : i - (i / Kp) * Kp;  // consecutive threads read consecutive addresses
    uint32_t h = 0, l = 0;
    if (k < K) split_tf32(mn ? Y[k * ld + r] : Y[r * ld + k], h, l);
    out[r * Kp + k] = __uint_as_float(h);
    out[n + r * Kp + k] = __uint_as_float(l);
  }
}

// Filter bank -> the K-major operand of the implicit convolution: row r (an output channel of the product), entry
// k = tap*Cs + c. layout 0: already so, W[r*K + k]; 1: bank [N][Cs][kk] (a layer's filters as stored, forward
// product): W[(r*Cs + c)*kk + tap]; 2: bank [Cs][N][kk] (the same filters, data gradient): W[(c*N + r)*kk + tap].
// split != 0: out[0][r][k] = w rounded to TF32, out[1][r][k] = the rest cut to TF32; split == 0: out[r][k] = w.
__global__ void split_filter_kernel(const float* __restrict__ W, int N, int Cs, int kk, int layout, int split, float* __restrict__ out) {
  const long K = (long)kk * Cs, n = (long)N * K;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / K);
    const int k = (int)(i - (long)r * K);
    const int tap = k / Cs, c = k - tap * Cs;
    float w;
    if (layout == 1) w = W[((long)r * Cs + c) * kk + tap];
    else if (layout == 2) w = W[((long)c * N + r) * kk + tap];
    else w = W[i];
    if (split) {
      uint32_t h, l;
      split_tf32(w, h, l);
      out[i] = __uint_as_float(h);
      out[n + i] = __uint_as_float(l);
    } else {
      out[i] = w;
    }
  }
}

// The same split for several (bank, layout) jobs in one launch: job = blockIdx.y.
constexpr int kMaxSplitJobs = 8;
struct SplitJobs {
  const float* W[kMaxSplitJobs];
  float* out[kMaxSplitJobs];
  int N[kMaxSplitJobs], Cs[kMaxSplitJobs], kk[kMaxSplitJobs], layout[kMaxSplitJobs];
};
__global__ void split_filter_banks_kernel(const SplitJobs jobs) {
  const int j = blockIdx.y;
  const float* __restrict__ W = jobs.W[j];
  float* __restrict__ out = jobs.out[j];
  const int N = jobs.N[j], Cs = jobs.Cs[j], kk = jobs.kk[j], layout = jobs.layout[j];
  const long K = (long)kk * Cs, n = (long)N * K;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / K);
    const int k = (int)(i - (long)r * K);
    const int tap = k / Cs, c = k - tap * Cs;
    const float w = layout == 1 ? W[((long)r * Cs + c) * kk + tap] : W[((long)c * N + r) * kk + tap];
    uint32_t h, l;
    split_tf32(w, h, l);
    out[i] = __uint_as_float(h);
    out[n + i] = __uint_as_float(l);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encoder() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
    else
      cudaGetLastError();
  }
  return fn;
}

struct Side {
  const float* base;
  long ld;
  bool mn;        // rows contiguous: element(row, k) = base[k*ld + row]
  long rows;
  long bstride;
};

bool aligned_for_tma(const Side& s, long P) {
  if (((uintptr_t)s.base & 15) != 0 || (s.ld & 3) != 0 || s.ld <= 0) return false;
  if (P > 1 && ((s.bstride & 3) != 0 || s.bstride <= 0)) return false;
  return true;
}

// 3-d tensor map over (inner, outer, batch); box = one tile of `box_rows` rows by 32 k
bool encode(CUtensorMap* map, const Side& s, long K, long P, int box_rows) {
  EncodeTiledFn fn = encoder();
  if (!fn) return false;
  cuuint64_t dims[3], strides[2];
  cuuint32_t box[3], estr[3] = {1, 1, 1};
  if (s.mn) {   // groups of 32 rows of the operand: one 128-byte row per K index
    dims[0] = (cuuint64_t)s.rows; dims[1] = (cuuint64_t)K;
    box[0] = 32; box[1] = kBK;
  } else {
    dims[0] = (cuuint64_t)K; dims[1] = (cuuint64_t)s.rows;
    box[0] = kBK; box[1] = (cuuint32_t)box_rows;
  }
  dims[2] = (cuuint64_t)P;
  box[2] = 1;
  strides[0] = (cuuint64_t)s.ld * 4;
  strides[1] = (cuuint64_t)(P > 1 ? s.bstride : (long)dims[1] * s.ld) * 4;
  if (dims[0] >= (1ull << 32) || dims[1] >= (1ull << 32) || strides[0] >= (1ull << 40) || strides[1] >= (1ull << 40)) return false;
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)s.base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  s.mn ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// stage counts for a kernel with conversion stages of conv_bytes and raw stages of raw_bytes: two CTAs per SM when
// one conversion stage and at least two raw stages fit in half of the SM's shared memory, otherwise one CTA per
// SM with two conversion stages and as many raw stages as fit. Returns false when nothing fits.
bool choose_stages(long conv_bytes, long raw_bytes, long nkb, int* conv_stages, int* raw_stages) {
  const long half = 110L * 1024 - 1024, whole = 224L * 1024 - 1024;
  int cs, rs;
  if ((half - 2 * conv_bytes) / raw_bytes >= 3) {
    cs = 2;
    rs = (int)std::min<long>(kMaxRaw, (half - 2 * conv_bytes) / raw_bytes);
  } else if ((half - conv_bytes) / raw_bytes >= 2) {
    cs = 1;
    rs = (int)std::min<long>(kMaxRaw, (half - conv_bytes) / raw_bytes);
  } else {
    cs = 2;
    rs = (int)std::min<long>(kMaxRaw, (whole - 2 * conv_bytes) / raw_bytes);
    if (rs < 2) return false;
  }
  (void)nkb;
  *conv_stages = cs;
  *raw_stages = rs;
  return true;
}

// CTAs of the persistent launch: every tile at once when they all fit on the machine (two CTAs per SM when the
// shared memory allows), otherwise one full wave that walks the tile grid
unsigned persistent_grid(long total_tiles, size_t smem_bytes) {
  const long per_sm = (smem_bytes <= 110u * 1024u) ? 2 : 1;
  const long slots = (long)rt().sm_count * per_sm;
  return (unsigned)std::min<long>(total_tiles, slots);
}

template <bool XMN, bool YMN, int CONV>
int launch_tma(const CUtensorMap& mapX, const CUtensorMap& mapY, const TmaParams& p, size_t smem) {
  static bool cfg = false;
  if (!cfg) {
    const int cap = 227 * 1024 - 2048;
    CGTB_CUDA_TRY(cudaFuncSetAttribute(sgemm_tma_kernel<XMN, YMN, CONV>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
    cfg = true;
  }
  const unsigned grid = persistent_grid(p.total_tiles, smem);
  CGTB_LAUNCH((sgemm_tma_kernel<XMN, YMN, CONV>), grid, kThreadsTma, smem, mapX, mapY, p);
  return 0;
}

// The convolution kernel with the input tile in shared memory and X in tensor memory is the default;
// CGTB_CONV_TSA=0 selects the kernel that loads a box per tap (for comparisons).
bool use_tsa() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("CGTB_CONV_TSA");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

// Pre-split Y (rows x K) into [2][rows][Kp] at `dst` and build its tensor map (box 32 x UN x 1, third coordinate
// 0 = hi, 1 = lo).
bool split_y(const Side& Y, long K, int UN, float* dst, long Kp, CUtensorMap* mapY, int filter_layout = 0, int Cs = 0, int kk = 0) {
  const long n = Y.rows * Kp;
  const unsigned blocks = (unsigned)std::min<long>(cgtb_ceil_div(n, 256), 8L * rt().sm_count);
  if (filter_layout < 0) { /* dst already holds [2][rows][Kp] (cgtb_split_filter_banks) */ }
  else if (filter_layout) CGTB_LAUNCH(split_filter_kernel, blocks, 256, 0, Y.base, (int)Y.rows, Cs, kk, filter_layout, 1, dst);
  else CGTB_LAUNCH(split_rows_kernel, blocks, 256, 0, Y.base, Y.rows, K, Y.ld, Y.mn ? 1 : 0, dst, Kp);
  EncodeTiledFn fn = encoder();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)Kp, (cuuint64_t)Y.rows, 2};
  cuuint64_t strides[2] = {(cuuint64_t)Kp * 4, (cuuint64_t)Y.rows * Kp * 4};
  cuuint32_t box[3] = {kBK, (cuuint32_t)UN, 2}, estr[3] = {1, 1, 1};
  if (strides[0] >= (1ull << 40) || strides[1] >= (1ull << 40)) return false;
  return fn(mapY, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)dst, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

namespace cgtb {

// returns 0 done, 1 error, -1 not eligible (the caller falls back to the register-fed kernel)
int sgemm_tma(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B, long ldb,
              long strideB, float* C, long ldc, long strideC, const ConvEpilogue* ep) {
  if (P <= 0 || M <= 0 || N <= 0) return 0;
  if (K < kBK) return -1;
  if (M * N < 1024 && K < 256) return -1;
  if (M >= (1L << 31) || N >= (1L << 31) || K >= (1L << 31)) return -1;
  Side sA = {A, lda, tA != 0, M, strideA};   // rows of op(A) are m; stored [K, M] when transposed
  Side sB = {B, ldb, tB == 0, N, strideB};   // rows of op(B)^T are n; stored [K, N] when not transposed
  if (!aligned_for_tma(sA, P) || !aligned_for_tma(sB, P)) return -1;
  TmaParams p;
  memset(&p, 0, sizeof(p));
  p.ep = ConvEpilogue{nullptr, nullptr, nullptr, 1};
  if (ep) p.ep = *ep;
  p.swapped = (N > M) ? 1 : 0;
  if (ep && (p.swapped || P != 1)) return -1;
  const Side& X = p.swapped ? sB : sA;
  const Side& Y = p.swapped ? sA : sB;
  long ydim = Y.rows;
  int ytiles = (int)cgtb_ceil_div(ydim, 128);
  const int ugran = Y.mn ? 32 : 16;   // an MN-major Y arrives in groups of 32 rows
  int UN = (int)(cgtb_ceil_div(cgtb_ceil_div(ydim, ytiles), ugran) * ugran);
  if (UN < ugran) UN = ugran;
  ytiles = (int)cgtb_ceil_div(ydim, UN);
  long xtiles = cgtb_ceil_div(X.rows, kXRows);
  p.UN = UN;
  p.tmem_cols = 32;
  while (p.tmem_cols < 2 * UN) p.tmem_cols *= 2;  // hi*hi + lo*hi in [0, UN), hi*lo in [UN, 2UN)
  p.xrows = X.rows;
  p.yrows = Y.rows;
  const long cx_bytes = 1L * kXRows * 128;  // X is read in place as the hi operand: the conversion stage holds x_lo only
  const long conv_bytes = cx_bytes + 2L * UN * 128, raw_bytes = (long)kXRows * 128 + (long)UN * 128;
  int conv_stages, raw_stages;
  long nkb_total = cgtb_ceil_div(K, kBK);
  if (!choose_stages(conv_bytes, raw_bytes, nkb_total, &conv_stages, &raw_stages)) return -1;
  long tiles = xtiles * ytiles * P;
  int nsplit = 1;
  long want = (long)rt().sm_count;
  if (tiles < want && nkb_total >= 8) {
    nsplit = (int)std::min<long>(std::max<long>(1, (2 * want) / tiles), nkb_total / 4);  // at most two CTAs per SM: one wave
    if (nsplit < 1) nsplit = 1;
  }
  long kchunk = cgtb_ceil_div(nkb_total, nsplit) * kBK;
  nsplit = (int)cgtb_ceil_div(K, kchunk);
  if (xtiles > 2147483647L / ((long)ytiles * P * nsplit)) return -1;
  if (ep && nsplit > 1) return -1;  // the output stage needs whole sums
  p.conv_stages = conv_stages;
  p.raw_stages = raw_stages;
  p.nsplit = nsplit;
  p.kchunk = kchunk;
  p.K = K;
  p.M = M;
  p.N = N;
  p.ldc = ldc;
  p.c_batch_stride = strideC;
  p.xtiles = (int)xtiles;
  p.ytiles = ytiles;
  p.total_tiles = xtiles * ytiles * P * nsplit;
  p.err = tc_error_flag();
  if (!p.err) return 1;
  CUtensorMap mapX, mapY;
  if (!encode(&mapX, X, K, P, kXRows) || !encode(&mapY, Y, K, P, UN)) return -1;
  float* part = nullptr;
  if (nsplit > 1) {
    part = (float*)scratch((size_t)P * nsplit * M * N * sizeof(float));
    if (!part) return 1;
    p.C = part;
  } else {
    p.C = C;
  }
  size_t smem = (size_t)conv_stages * conv_bytes + (size_t)raw_stages * raw_bytes;
  smem += 1024;
  int rc;
  if (X.mn && Y.mn) rc = launch_tma<true, true, 0>(mapX, mapY, p, smem);
  else if (X.mn) rc = launch_tma<true, false, 0>(mapX, mapY, p, smem);
  else if (Y.mn) rc = launch_tma<false, true, 0>(mapX, mapY, p, smem);
  else rc = launch_tma<false, false, 0>(mapX, mapY, p, smem);
  if (rc) return rc;
  if (nsplit > 1) tc_splitk_fold(P, M, N, nsplit, part, C, ldc, strideC);
  CGTB_CHECK_LAUNCH("sgemm_tma");
  return 0;
}

// Stride-1 convolution as an implicit GEMM, without a column matrix: serves the forward product of a layer
// (sign +1; the reference forms Im2Col then Mul22(col, W^T): cgt/nn.py:93-100, include/im2col.h:6-28) and its data
// gradient (sign -1; the reference forms Mul22(dy, W) and then Col2Im: cgt/nn_ops/im2col.py, include/im2col.h:30-50):
//   out[b, n, y, x] = sum_{i, j, c} src[b, y + sign*(i - ph), x + sign*(j - pw), c] * wr[n][(i*kw + j)*Cs + c]
// src is NHWC [B, Hs, Ws, Cs], wr holds one row of kh*kw*Cs entries per output channel, out is NCHW [B, N, Hd, Wd].
// It is the GEMM above with M = pixels, N = output channels, K = kh*kw*Cs whose X operand is never stored: for K
// block (tap, 32 source channels) the TMA unit loads the window of src that the tap addresses, a box of whole image
// rows whose out-of-range rows and columns it zero-fills (the padding). A tile is `rows` image rows of one image
// (rows*Wd <= 128 pixels) or, for small images, several whole images. With `ep` the bias / relu / mask output stage
// is applied to the accumulator (forward product of a layer).
// returns 0 done, 1 error, -1 not eligible
int conv_implicit_tma(const float* src, long B, int Hs, int Ws, int Cs, const float* wr, int w_layout, int N, int Hd, int Wd, int kh,
                      int kw, int ph, int pw, int sign, float* out, const ConvEpilogue* ep, const float* presplit) {
  if (B <= 0 || N <= 0 || Hd <= 0 || Wd <= 0) return 0;
  if (Cs % 32 != 0 || N % 16 != 0 || Wd > 128 || B >= (1L << 30) || kh <= 0 || kw <= 0) return -1;
  if (((uintptr_t)src & 15) != 0 || ((uintptr_t)wr & 15) != 0) return -1;
  const long K = (long)kh * kw * Cs;
  const int HW = Hd * Wd;
  ConvTsaParams cp;
  memset(&cp, 0, sizeof(cp));
  TmaParams& p = cp.t;
  p.ep = ConvEpilogue{nullptr, nullptr, nullptr, 1};
  if (ep) p.ep = *ep;
  p.csign = sign;
  p.cW = Wd;
  p.cHW = HW;
  p.cC = N;
  p.ckw = kw;
  p.ckpt = Cs / 32;
  p.cph = ph;
  p.cpw = pw;
  p.cB = (int)B;
  const long want = (long)rt().sm_count;
  const int ytiles = (int)cgtb_ceil_div(N, 128);
  const int UN = (int)(cgtb_ceil_div(cgtb_ceil_div(N, ytiles), 16) * 16);
  if (UN * ytiles != N) return -1;  // equal column tiles only
  p.UN = UN;
  p.xrows = 0;
  p.yrows = N;
  const long nkb = K / kBK;
  EncodeTiledFn fn = encoder();
  if (!fn) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)Cs, (cuuint64_t)Ws, (cuuint64_t)Hs, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)Cs * 4, (cuuint64_t)Ws * Cs * 4, (cuuint64_t)Hs * Ws * Cs * 4};
  cuuint32_t estr[4] = {1, 1, 1, 1};

  // tile = `crows` image rows of one image (crows*Wd <= 128 pixels) or, for small images, several whole images
  auto tile_geometry = [&](long max_imgs) {
    if (HW <= 128) {
      // several small images per tile, but not so many that the tile count falls below the number of SMs
      long nimg = std::min<long>(std::min<long>(128 / HW, B), max_imgs);
      while (nimg > 1 && cgtb_ceil_div(B, nimg) * ytiles < want) --nimg;
      p.cnimg = (int)nimg;
      p.crows = Hd;
      p.cnbands = 1;
      return cgtb_ceil_div(B, p.cnimg);
    }
    p.cnimg = 1;
    const int max_rows = 128 / Wd;
    p.cnbands = (int)cgtb_ceil_div(Hd, max_rows);
    p.crows = (int)cgtb_ceil_div(Hd, p.cnbands);  // equal bands
    return B * p.cnbands;
  };

  bool tsa = use_tsa();
  size_t smem = 0;
  long tiles = 0;
  int conv_stages = 0, raw_stages = 0;
  if (tsa) {
    // shared memory: HB halo tiles + a ring of filter stages; TMEM: accumulator + A stages of 64 columns
    // TMEM: one or two accumulators of 2*UN columns (rounded to 64), then A stages of 64 columns
    cp.acc_cols = (2 * UN + 63) & ~63;
    cp.nacc = (512 - 2 * cp.acc_cols) / 64 >= 3 ? 2 : 1;
    const int as = std::min<int>(kMaxA, (512 - cp.nacc * cp.acc_cols) / 64);
    const long w_bytes = 2L * UN * 128;
    const long budget = 222L * 1024;
    long max_imgs = 128;
    bool fits = false;
    for (int attempt = 0; attempt < 8 && !fits; ++attempt) {
      tiles = tile_geometry(max_imgs);
      cp.hw = Wd + kw - 1;
      cp.hh = p.crows + kh - 1;
      const long rows = (long)cp.hw * cp.hh * p.cnimg;
      cp.chunk_bytes = (uint32_t)((rows * 128 + 1023) & ~1023L);
      const long halo_bytes = (long)p.ckpt * cp.chunk_bytes;
      if (2 * halo_bytes + 3 * w_bytes <= budget) cp.halo_bufs = 2;
      else if (halo_bytes + 2 * w_bytes <= budget) cp.halo_bufs = 1;
      else cp.halo_bufs = 0;
      if (cp.halo_bufs && cp.hw <= 256 && cp.hh <= 256) {
        fits = true;
        // a stage = 64 TMEM columns (x, x_lo of one K block) + one filter tile pair in shared memory
        conv_stages = (int)std::min<long>(as, (budget - cp.halo_bufs * halo_bytes) / w_bytes);
        raw_stages = conv_stages;
        smem = std::max<size_t>((size_t)(cp.halo_bufs * halo_bytes + conv_stages * w_bytes + 1024), (size_t)120 * 1024);
      } else if (p.cnimg > 1) {
        max_imgs = p.cnimg - 1;   // fewer images per tile: a smaller halo tile
      } else {
        break;
      }
    }
    if (!fits || conv_stages < 2) {
      tsa = false;
    } else {
      p.tmem_cols = 512;
      p.cx_tx = (int)((long)cp.hw * cp.hh * p.cnimg * 128);
      cp.kh = kh;
      cp.hx0 = sign > 0 ? -pw : pw - (kw - 1);
      cp.hy0 = sign > 0 ? -ph : ph - (kh - 1);
    }
  }
  if (!tsa) {
    tiles = tile_geometry(128);
    p.cx_tx = 32 * Wd * p.crows * p.cnimg * (int)sizeof(float);
    p.tmem_cols = 32;
    while (p.tmem_cols < 2 * UN) p.tmem_cols *= 2;
    const long conv_bytes = 1L * kXRows * 128 + 2L * UN * 128, raw_bytes = (long)kXRows * 128 + (long)UN * 128;
    if (!choose_stages(conv_bytes, raw_bytes, nkb, &conv_stages, &raw_stages)) return -1;
    smem = (size_t)conv_stages * conv_bytes + (size_t)raw_stages * raw_bytes + 1024;
  }
  if (tiles > 2147483647L / 8) return -1;
  p.conv_stages = conv_stages;
  p.raw_stages = raw_stages;
  // few tiles with a long K loop (small images, many taps): split K over CTAs, each split writing its own
  // copy of the result. Not with the output stage, which needs whole sums.
  int nsplit = 1;
  const long slots = tsa ? want : 2 * want;  // CTAs resident at once
  if (!ep && tiles * ytiles < want && nkb >= 8)
    nsplit = (int)std::max<long>(1, std::min<long>(std::max<long>(1, slots / (tiles * ytiles)), nkb / 4));
  const long kchunk = cgtb_ceil_div(nkb, nsplit) * kBK;
  nsplit = (int)cgtb_ceil_div(K, kchunk);
  p.nsplit = nsplit;
  p.kchunk = kchunk;
  p.K = K;
  p.M = B * HW;
  p.N = N;
  p.ldc = N;
  p.c_batch_stride = 0;
  p.xtiles = (int)tiles;
  p.ytiles = ytiles;
  p.total_tiles = tiles * ytiles * nsplit;
  const long total = B * (long)N * HW;
  // the pre-split filters (or, for the kernel that converts in its loop, the rearranged copy of a filter bank)
  if (presplit && (((uintptr_t)presplit & 15) != 0)) presplit = nullptr;
  // `presplit`: [w_hi | w_lo] of these filters in the kernel's layout, made earlier in the step (cgtb_split_filter_banks)
  const size_t split_bytes = tsa ? (presplit ? 0 : ((((size_t)2 * N * K * sizeof(float)) + 255) & ~(size_t)255))
                                 : (w_layout ? ((((size_t)N * K * sizeof(float)) + 255) & ~(size_t)255) : 0);
  const size_t slab_bytes = nsplit > 1 ? (size_t)nsplit * total * sizeof(float) : 0;
  char* blk = nullptr;
  if (split_bytes + slab_bytes) {
    blk = (char*)scratch(split_bytes + slab_bytes);
    if (!blk) return 1;
  }
  float* part = (float*)(blk + split_bytes);
  p.C = nsplit > 1 ? part : out;
  p.err = tc_error_flag();
  if (!p.err) return 1;
  CUtensorMap mapX, mapY;
  {
    cuuint32_t box[4] = {32, (cuuint32_t)(tsa ? cp.hw : Wd), (cuuint32_t)(tsa ? cp.hh : p.crows), (cuuint32_t)p.cnimg};
    if (box[1] > 256 || box[2] > 256 || box[3] > 256) return -1;
    CUresult r = fn(&mapX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)src, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -1;
  }
  Side Y = {wr, K, false, N, 0};
  if (tsa) {
    if (presplit ? !split_y(Y, K, UN, const_cast<float*>(presplit), K, &mapY, -1)
                 : !split_y(Y, K, UN, (float*)blk, K, &mapY, w_layout, Cs, kh * kw))
      return -1;
    static bool cfg = false;
    if (!cfg) {
      CGTB_CUDA_TRY(cudaFuncSetAttribute(conv_tsa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048));
      cfg = true;
    }
    const unsigned grid = (unsigned)std::min<long>(p.total_tiles, want);  // one CTA per SM
    CGTB_LAUNCH(conv_tsa_kernel, grid, kThreadsConv, smem, mapX, mapY, cp);
  } else {
    if (w_layout) {
      const unsigned blocks = (unsigned)std::min<long>(cgtb_ceil_div((long)N * K, 256), 8L * rt().sm_count);
      CGTB_LAUNCH(split_filter_kernel, blocks, 256, 0, wr, N, Cs, kh * kw, w_layout, 0, (float*)blk);
      Y.base = (const float*)blk;
    }
    if (!encode(&mapY, Y, K, 1, UN)) return -1;
    int rc = launch_tma<false, false, 1>(mapX, mapY, p, smem);
    if (rc) return rc;
  }
  if (nsplit > 1) tc_splitk_fold(1, 1, total, nsplit, part, out, total, 0);
  CGTB_CHECK_LAUNCH("conv_implicit");
  return 0;
}

// Filter gradient of a stride-1 convolution without a column matrix (the reference forms Mul22{T,N}(dy, col) on the
// Im2Col output: cgt/nn.py:93-100 differentiated, cgt/core.py:2162-2175):
//   dw[n][c][i][j] = sum_{b, y, x} dy[b, y, x, n] * src[b, y + i - ph, x + j - pw, c]
// src NHWC [B, Hs, Ws, Cs], dy NHWC [B, Hd, Wd, N], dw [N][Cs*kh*kw] (the filter bank's own layout). It is the product
// dy^T . col with the sum over pixels as the K dimension: a K block is `wbh` rows of one image (at most 32 pixels, the
// rest of the block's K slots are zeros); an X tile holds four (tap, 32-channel) units, each the same pixels of src
// shifted by its tap (one TMA box per unit, out-of-range rows and columns zero-filled); the conversion warps
// transpose both operands into the K-major layout while splitting them. K is split over CTAs, every split writes
// its own slab in dw's layout and an ordered fold adds the slabs.
// returns 0 done, 1 error, -1 not eligible
int conv_wgrad_tma(const float* src, long B, int Hs, int Ws, int Cs, const float* dy, int Hd, int Wd, int N, int kh, int kw, int ph,
                   int pw, float* dw) {
  if (N <= 0 || Cs <= 0 || kh <= 0 || kw <= 0) return 0;
  if (Cs % 32 != 0 || N % 4 != 0 || Wd > 32 || Wd <= 0 || Hd <= 0 || B <= 0 || B >= (1L << 24)) return -1;
  if (((uintptr_t)src & 15) != 0 || ((uintptr_t)dy & 15) != 0) return -1;
  const long Kc = (long)kh * kw * Cs;  // columns of the result
  TmaParams p;
  memset(&p, 0, sizeof(p));
  p.ep = ConvEpilogue{nullptr, nullptr, nullptr, 1};
  p.ckw = kw;
  p.ckpt = Cs / 32;
  p.cph = ph;
  p.cpw = pw;
  p.wkk = kh * kw;
  p.wunits = kh * kw * (Cs / 32);
  p.wbh = std::min<int>(32 / Wd, Hd);
  p.wnrg = (int)cgtb_ceil_div(Hd, p.wbh);
  p.wnpx = p.wbh * Wd;
  const int ytiles = (int)cgtb_ceil_div(N, 128);
  // whole groups of 32 channels (one 128-byte row each); channels beyond N are zero-filled by the TMA unit and never stored
  int UN = (int)(cgtb_ceil_div(cgtb_ceil_div(N, ytiles), 32) * 32);
  p.UN = UN;
  p.tmem_cols = 32;
  while (p.tmem_cols < 2 * UN) p.tmem_cols *= 2;
  p.yrows = N;
  p.xrows = Kc;
  const long xtiles = cgtb_ceil_div(p.wunits, 4);
  const long nkb_total = B * p.wnrg;
  // conversion stage: x_lo, [y_hi | y_lo]; raw stage: x (read in place as x_hi), y
  const long conv_bytes = 1L * kXRows * 128 + 2L * UN * 128, raw_bytes = (long)kXRows * 128 + (long)UN * 128;
  int conv_stages, raw_stages;
  if (!choose_stages(conv_bytes, raw_bytes, nkb_total, &conv_stages, &raw_stages)) return -1;
  const long tiles = xtiles * ytiles;
  const long want = (long)rt().sm_count;
  int nsplit = 1;
  if (tiles < 2 * want && nkb_total >= 8) nsplit = (int)std::max<long>(1, std::min<long>((2 * want) / tiles, nkb_total / 4));
  const long kchunk = cgtb_ceil_div(nkb_total, nsplit) * kBK;
  nsplit = (int)cgtb_ceil_div(nkb_total * kBK, kchunk);
  p.conv_stages = conv_stages;
  p.raw_stages = raw_stages;
  p.nsplit = nsplit;
  p.kchunk = kchunk;
  p.K = nkb_total * kBK;
  p.M = N;
  p.N = Kc;
  p.ldc = Kc;
  p.c_batch_stride = 0;
  p.xtiles = (int)xtiles;
  p.ytiles = ytiles;
  p.total_tiles = tiles * nsplit;
  p.swapped = 1;
  float* part = nullptr;
  if (nsplit > 1) {
    part = (float*)scratch((size_t)nsplit * N * Kc * sizeof(float));
    if (!part) return 1;
    p.C = part;
  } else {
    p.C = dw;
  }
  p.err = tc_error_flag();
  if (!p.err) return 1;
  EncodeTiledFn fn = encoder();
  if (!fn) return -1;
  CUtensorMap mapX, mapY;
  cuuint32_t estr[4] = {1, 1, 1, 1};
  {
    cuuint64_t dims[4] = {(cuuint64_t)Cs, (cuuint64_t)Ws, (cuuint64_t)Hs, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)Cs * 4, (cuuint64_t)Ws * Cs * 4, (cuuint64_t)Hs * Ws * Cs * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)Wd, (cuuint32_t)p.wbh, 1};
    CUresult r = fn(&mapX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)src, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -1;
  }
  {
    cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)Wd, (cuuint64_t)Hd, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)N * 4, (cuuint64_t)Wd * N * 4, (cuuint64_t)Hd * Wd * N * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)Wd, (cuuint32_t)p.wbh, 1};   // one box per group of 32 channels
    CUresult r = fn(&mapY, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)dy, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -1;
  }
  size_t smem = (size_t)conv_stages * conv_bytes + (size_t)raw_stages * raw_bytes + 1024;
  int rc = launch_tma<true, true, 2>(mapX, mapY, p, smem);
  if (rc) return rc;
  if (nsplit > 1) tc_splitk_fold(1, N, Kc, nsplit, part, dw, Kc, 0);
  CGTB_CHECK_LAUNCH("conv_wgrad");
  return 0;
}

}  // namespace cgtb

static int conv_dgrad_any(const float* dy_nhwc, long B, int Ho, int Wo, int Cin, const float* w, int layout, int C, int H, int W, int kh,
                          int kw, int ph, int pw, float* dx_nchw, const float* presplit = nullptr) {
  if (!require_runtime("cgtb_conv_dgrad")) return 1;
  if (C > 128) return fail("cgtb_conv_dgrad: at most 128 image channels");
  int rc = cgtb::conv_implicit_tma(dy_nhwc, B, Ho, Wo, Cin, w, layout, C, H, W, kh, kw, ph, pw, -1, dx_nchw, nullptr, presplit);
  if (rc < 0)
    return fail("cgtb_conv_dgrad: not supported for Cin=%d (multiple of 32), C=%d (multiple of 16, at most 128), W=%d (at most 128) "
                "or an unaligned operand; use cgtb_sgemm + cgtb_col2im", Cin, C, W);
  return rc;
}
CGTB_API int cgtb_conv_dgrad(const float* dy_nhwc, long B, int Ho, int Wo, int Cin, const float* w_rearranged, int C, int H, int W,
                             int kh, int kw, int ph, int pw, float* dx_nchw) {
  return conv_dgrad_any(dy_nhwc, B, Ho, Wo, Cin, w_rearranged, 0, C, H, W, kh, kw, ph, pw, dx_nchw);
}
CGTB_API int cgtb_conv_dgrad_bank(const float* dy_nhwc, long B, int Ho, int Wo, int Cin, const float* w_bank, int C, int H, int W,
                                  int kh, int kw, int ph, int pw, float* dx_nchw) {
  return conv_dgrad_any(dy_nhwc, B, Ho, Wo, Cin, w_bank, 2, C, H, W, kh, kw, ph, pw, dx_nchw);
}

static int conv_fwd_any(const float* x_nhwc, long B, int H, int W, int Cin, const float* w, int layout, int Cout, int Ho, int Wo, int kh,
                        int kw, int ph, int pw, const float* bias, float* y_nchw, int8_t* mask_nchw, const float* presplit = nullptr) {
  if (!require_runtime("cgtb_conv_fwd_bias_relu")) return 1;
  if (Ho != H + 2 * ph - kh + 1 || Wo != W + 2 * pw - kw + 1)
    return fail("cgtb_conv_fwd_bias_relu: output %dx%d is not that of a stride-1 %dx%d convolution of %dx%d with padding %d,%d", Ho, Wo,
                kh, kw, H, W, ph, pw);
  cgtb::ConvEpilogue ep = {bias, y_nchw, mask_nchw, (long)Ho * Wo};
  int rc = cgtb::conv_implicit_tma(x_nhwc, B, H, W, Cin, w, layout, Cout, Ho, Wo, kh, kw, ph, pw, +1, nullptr, &ep, presplit);
  if (rc < 0)
    return fail("cgtb_conv_fwd_bias_relu: not supported for Cin=%d (multiple of 32), Cout=%d (multiple of 16; of 128 when above 128), "
                "Wo=%d (at most 128) or an unaligned operand; use cgtb_im2col + cgtb_conv_bias_relu", Cin, Cout, Wo);
  return rc;
}
CGTB_API int cgtb_conv_fwd_bias_relu(const float* x_nhwc, long B, int H, int W, int Cin, const float* w_rearranged, int Cout, int Ho,
                                     int Wo, int kh, int kw, int ph, int pw, const float* bias, float* y_nchw, int8_t* mask_nchw) {
  return conv_fwd_any(x_nhwc, B, H, W, Cin, w_rearranged, 0, Cout, Ho, Wo, kh, kw, ph, pw, bias, y_nchw, mask_nchw);
}
CGTB_API int cgtb_conv_fwd_bias_relu_bank(const float* x_nhwc, long B, int H, int W, int Cin, const float* w_bank, int Cout, int Ho,
                                          int Wo, int kh, int kw, int ph, int pw, const float* bias, float* y_nchw, int8_t* mask_nchw) {
  return conv_fwd_any(x_nhwc, B, H, W, Cin, w_bank, 1, Cout, Ho, Wo, kh, kw, ph, pw, bias, y_nchw, mask_nchw);
}

CGTB_API int cgtb_conv_fwd_bias_relu_pre(const float* x_nhwc, long B, int H, int W, int Cin, const float* w_bank, const float* w_split,
                                         int Cout, int Ho, int Wo, int kh, int kw, int ph, int pw, const float* bias, float* y_nchw,
                                         int8_t* mask_nchw) {
  return conv_fwd_any(x_nhwc, B, H, W, Cin, w_bank, 1, Cout, Ho, Wo, kh, kw, ph, pw, bias, y_nchw, mask_nchw, w_split);
}
CGTB_API int cgtb_conv_dgrad_pre(const float* dy_nhwc, long B, int Ho, int Wo, int Cin, const float* w_bank, const float* w_split, int C,
                                 int H, int W, int kh, int kw, int ph, int pw, float* dx_nchw) {
  return conv_dgrad_any(dy_nhwc, B, Ho, Wo, Cin, w_bank, 2, C, H, W, kh, kw, ph, pw, dx_nchw, w_split);
}
CGTB_API int cgtb_split_filter_banks(int njobs, const float* const* banks, const int* n_out, const int* n_src, const int* taps,
                                     const int* layout, float* const* out) {
  if (!require_runtime("cgtb_split_filter_banks")) return 1;
  if (njobs < 1 || njobs > kMaxSplitJobs) return fail("cgtb_split_filter_banks: between 1 and %d jobs", kMaxSplitJobs);
  SplitJobs jobs;
  memset(&jobs, 0, sizeof(jobs));
  long most = 0;
  for (int j = 0; j < njobs; ++j) {
    if (!banks[j] || !out[j] || n_out[j] < 1 || n_src[j] < 1 || taps[j] < 1 || (layout[j] != 1 && layout[j] != 2))
      return fail("cgtb_split_filter_banks: job %d: null pointer, empty extent or a layout other than 1 (forward) / 2 (data gradient)", j);
    jobs.W[j] = banks[j];
    jobs.out[j] = out[j];
    jobs.N[j] = n_out[j];
    jobs.Cs[j] = n_src[j];
    jobs.kk[j] = taps[j];
    jobs.layout[j] = layout[j];
    most = std::max<long>(most, (long)n_out[j] * n_src[j] * taps[j]);
  }
  const unsigned bx = (unsigned)std::min<long>(cgtb_ceil_div(most, 256), 2L * rt().sm_count);
  CGTB_LAUNCH(split_filter_banks_kernel, dim3(bx, (unsigned)njobs), 256, 0, jobs);
  CGTB_CHECK_LAUNCH("split_filter_banks");
  return 0;
}

CGTB_API int cgtb_conv_wgrad(const float* x_nhwc, long B, int H, int W, int Cin, const float* dy_nhwc, int Ho, int Wo, int Cout, int kh,
                             int kw, int ph, int pw, float* dw) {
  if (!require_runtime("cgtb_conv_wgrad")) return 1;
  if (Ho != H + 2 * ph - kh + 1 || Wo != W + 2 * pw - kw + 1)
    return fail("cgtb_conv_wgrad: gradient %dx%d is not that of a stride-1 %dx%d convolution of %dx%d with padding %d,%d", Ho, Wo, kh,
                kw, H, W, ph, pw);
  int rc = cgtb::conv_wgrad_tma(x_nhwc, B, H, W, Cin, dy_nhwc, Ho, Wo, Cout, kh, kw, ph, pw, dw);
  if (rc < 0)
    return fail("cgtb_conv_wgrad: not supported for Cin=%d (multiple of 32), Cout=%d (multiple of 4), Wo=%d "
                "(at most 32) or an unaligned operand; use cgtb_im2col + cgtb_sgemm", Cin, Cout, Wo);
  return rc;
}

#ifdef CGTB_TMA_TRACE
CGTB_API int cgtb_debug_tma_trace(long long* host) {
  cudaStreamSynchronize(rt().stream);
  return cudaMemcpyFromSymbol(host, g_tma_trace, sizeof(long long) * 128 * 8) == cudaSuccess ? 0 : 1;
}
#endif
