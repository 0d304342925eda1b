// Mul22 / BatchedMul22 on the 5th-generation tensor cores of sm_100a: tcgen05.mma kind::tf32 with the
// accumulator in tensor memory (TMEM), fp32 semantics kept by the 3xTF32 split
//     a*b ~= a_hi*b_hi + a_lo*b_hi + a_hi*b_lo,   x_hi = tf32(x), x_lo = tf32(x - x_hi)
// (the dropped a_lo*b_lo term is below 2^-22 relative). Replaces cblas_sgemm / cublasSgemm_v2 in the
// reference (cgt/core.py:2195-2222).
//
// Shape of the kernel
//   * One CTA computes one 128 x UN output tile (UN a multiple of 16, at most 256) for one K slice.
//     The operand with the larger output extent is put on the 128-row side ("X"), the other on the UN
//     side ("Y"); when that is op(B), the tile is written back transposed, so skinny weight-gradient
//     products (M = 32, K = 131072) still fill the 128 TMEM lanes.
//   * Warps 0-7 load: global -> registers -> (hi, lo) split -> shared memory, written directly in the
//     K-major, 128-byte-swizzled layout that the UMMA shared-memory descriptor describes. Going through
//     registers is what makes the split free, lets any leading dimension and any of the four transpose
//     combinations feed the same MMA configuration (a transposed source is transposed on the way in),
//     and zero-fills ragged edges. Each thread keeps the loads of the next two or three K blocks in
//     flight in registers while the current one is split and stored.
//   * Warp 8 issues the MMAs through one elected lane (8 per 32-deep K block: per K step
//     x_hi * [y_hi | y_lo] as one instruction with 2*UN accumulator columns, and x_lo * y_hi) and
//     commits them to the stage's "empty" mbarrier; the warp owns the TMEM allocation.
//   * After the last K block the eight loader warps become the epilogue: tcgen05.ld the accumulator
//     (lane = tile row; the two warps of a lane quarter take alternate 16-column chunks), stage it in
//     the idle pipeline memory and write C with coalesced stores, or a split-K slab that a second kernel
//     folds in split order.
//   * Every mbarrier wait is bounded; on expiry the kernel raises a flag in host-mapped memory, skips
//     the remaining work, still frees its TMEM and returns. The host reports the flag after the stream
//     has been synchronised.
//
// Roofline: the configuration's products are skinny (N of 32..64 outputs per 75..800-long row), so
// they are bound by streaming A from HBM, not by the tensor pipe: 4*(M*K + K*N + M*N) bytes per call.
#include "runtime.h"
#include "tc_util.h"

using namespace cgtb;
using namespace cgtb::tc;

namespace {

constexpr int kLoaderWarps = 8;
constexpr int kLoaderThreads = kLoaderWarps * 32;
constexpr int kThreads = kLoaderThreads + 32;  // 8 loader/epilogue warps + 1 MMA warp
constexpr int kMaxStages = 4;

struct Operand {
  const float* base;
  long ld;        // stored row length
  int kcontig;    // 1: element(row, k) = base[row*ld + k]; 0: element(row, k) = base[k*ld + row]
  int mode;       // loader access pattern (see TileLoader): 0 rows contiguous, 1 K contiguous, 2 K contiguous + 16-byte aligned
  long rows;      // valid rows of this operand (M or N of the product)
  long batch_stride;
};

struct Params {
  Operand X, Y;
  float* C;          // output or split-K slab
  long ldc;          // row length of C in the product's own (m, n) orientation
  long c_batch_stride;
  int swapped;       // X is op(B): tile row i is product column n
  long K;
  long kchunk;       // K elements per split (multiple of kBK)
  int nsplit;
  long M, N;         // product extents, for the slab layout
  int UN;            // tile columns
  int stages;
  int tmem_cols;
  int* err;          // host-mapped error flag
  ConvEpilogue ep;   // ep.y != nullptr: bias + relu + NCHW output stage instead of storing C
};

// Operand tiles travel global -> registers -> shared memory in two steps so that the loads of the
// next K block are in flight while the current one is split and stored. Three access patterns, fixed
// at compile time per operand:
//   MODE 0  rows contiguous in memory (a transposed source): threads along rows, 4 k per unit;
//   MODE 1  K contiguous: lanes along k, one 128-byte row segment per warp instruction;
//   MODE 2  K contiguous and 16-byte aligned: 128-bit loads, 8 lanes per row.
// NV is the number of register slots a thread owns for the tile (16 for the 128-row X tile, R/8 with a
// minimum of 4 for an R-row Y tile). Everything that does not change from one K block to the next -- the thread's row
// pointer, its shared-memory offset, which of its slots fall inside the matrix -- is computed once.
template <int MODE, int NV>
struct TileLoader {
  const float* p0;   // first element this thread loads in K block 0 (clamped to a valid address)
  long step;         // element distance between consecutive slots (MODE 0: between consecutive k)
  uint32_t off0;     // shared-memory byte offset of slot 0
  uint32_t valid;    // bit u set: slot u (MODE 0: pair u) lies inside the matrix
  long ld;
  int kofs;          // this thread's k offset inside the block (MODE 1: lane, MODE 2: 4*(lane&7))

  __device__ __forceinline__ void init(const Operand& op, const float* base, long row0, int R, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    ld = op.ld;
    valid = 0u;
    if (MODE == 1) {
      kofs = lane;
      const int r0 = warp;
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        int r = r0 + kLoaderWarps * u;
        if (r < R && row0 + r < op.rows) valid |= 1u << u;
      }
      p0 = base + (row0 + r0) * ld + lane;
      step = (long)kLoaderWarps * ld;
      off0 = tile_off(r0, lane);           // slot u: + u * 8 rows = + u * 1024 bytes (row mod 8 unchanged)
    } else if (MODE == 2) {
      const int sub = lane >> 3, c = lane & 7;
      kofs = 4 * c;
      const int r0 = warp * 4 + sub;
#pragma unroll
      for (int u = 0; u < NV / 4; ++u) {
        int r = r0 + kLoaderWarps * 4 * u;
        if (r < R && row0 + r < op.rows) valid |= 1u << u;
      }
      p0 = base + (row0 + r0) * ld + 4 * c;
      step = (long)kLoaderWarps * 4 * ld;
      off0 = tile_off(r0, 4 * c);          // slot u: + u * 32 rows = + u * 4096 bytes
    } else {
      kofs = 0;
      p0 = base;
      step = ld;
      off0 = 0;
      // unit q -> (row = q % R, k quad = q / R in 0..7); a thread owns units tid, tid + 256, ...
#pragma unroll
      for (int un = 0; un < NV / 4; ++un) {
        int q = tid + kLoaderThreads * un;
        int kq = q / R, r = q - kq * R;
        if (kq < 8 && row0 + r < op.rows) valid |= 1u << un;
      }
    }
  }

  // full == true: the whole 32-deep block lies inside K (no per-element k checks)
  __device__ __forceinline__ void fetch(const Operand& op, const float* base, long row0, int R, long k0, long k_end, bool full,
                                        float (&v)[NV], int tid) const {
    if (MODE == 1) {
      const bool kin = full || (k0 + kofs < k_end);
      const float* p = p0 + k0;
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        v[u] = (((valid >> u) & 1u) && kin) ? __ldg(p) : 0.f;
        p += step;
      }
    } else if (MODE == 2) {
      const float* p = p0 + k0;
      const long kk = k0 + kofs;
#pragma unroll
      for (int u = 0; u < NV / 4; ++u) {
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if ((valid >> u) & 1u) {
          if (full || kk + 3 < k_end) {
            q = __ldg(reinterpret_cast<const float4*>(p));
          } else {
            if (kk + 0 < k_end) q.x = __ldg(p + 0);
            if (kk + 1 < k_end) q.y = __ldg(p + 1);
            if (kk + 2 < k_end) q.z = __ldg(p + 2);
          }
        }
        v[4 * u + 0] = q.x; v[4 * u + 1] = q.y; v[4 * u + 2] = q.z; v[4 * u + 3] = q.w;
        p += step;
      }
    } else {
#pragma unroll
      for (int un = 0; un < NV / 4; ++un) {
        int q = tid + kLoaderThreads * un;
        int kq = q / R, r = q - kq * R;
        const bool rin = (valid >> un) & 1u;
        const float* p = base + (k0 + kq * 4) * ld + row0 + r;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          v[4 * un + u] = (rin && (full || k0 + kq * 4 + u < k_end)) ? __ldg(p) : 0.f;
          p += ld;
        }
      }
    }
  }

  __device__ __forceinline__ void stash(int R, const float (&v)[NV], unsigned char* s_hi, unsigned char* s_lo, int tid) const {
    const int warp = tid >> 5;
    if (MODE == 1) {
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        if (warp + kLoaderWarps * u < R) {
          uint32_t hi, lo;
          split_tf32(v[u], hi, lo);
          const uint32_t off = off0 + (uint32_t)u * 1024u;  // 32 lanes -> 32 distinct banks
          *reinterpret_cast<uint32_t*>(s_hi + off) = hi;
          *reinterpret_cast<uint32_t*>(s_lo + off) = lo;
        }
      }
    } else if (MODE == 2) {
      const int r0 = warp * 4 + ((tid & 31) >> 3);
#pragma unroll
      for (int u = 0; u < NV / 4; ++u) {
        if (r0 + kLoaderWarps * 4 * u < R) {
          uint4 h, l;
          split_tf32x4(v[4 * u + 0], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3], h, l);
          const uint32_t off = off0 + (uint32_t)u * 4096u;
          *reinterpret_cast<uint4*>(s_hi + off) = h;
          *reinterpret_cast<uint4*>(s_lo + off) = l;
        }
      }
    } else {
#pragma unroll
      for (int un = 0; un < NV / 4; ++un) {
        int q = tid + kLoaderThreads * un;
        int kq = q / R, r = q - kq * R;
        if (kq < 8) {
          uint4 h, l;
          split_tf32x4(v[4 * un + 0], v[4 * un + 1], v[4 * un + 2], v[4 * un + 3], h, l);
          const uint32_t off = tile_off(r, kq * 4);
          *reinterpret_cast<uint4*>(s_hi + off) = h;
          *reinterpret_cast<uint4*>(s_lo + off) = l;
        }
      }
    }
  }
};

template <int XMODE, int YMODE, int YNV, int DEPTH>
__global__ void __launch_bounds__(kThreads, (YNV <= 16 ? 2 : 1)) sgemm_tc_kernel(const Params p) {
  static_assert(YNV % 4 == 0 && YNV >= 4, "Y slots come in quads");
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int epi_fail;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int UN = p.UN, S = p.stages;
  // tiles start on a 1024-byte boundary so that the swizzle pattern is anchored at offset 0
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t x_bytes = kXRows * 128u, y_bytes = (uint32_t)UN * 128u;
  const uint32_t stage_bytes = 2 * x_bytes + 2 * y_bytes;

  const int batch = blockIdx.z / p.nsplit, split = blockIdx.z % p.nsplit;
  const long x0 = (long)blockIdx.x * kXRows, y0 = (long)blockIdx.y * UN;
  const long k_begin = (long)split * p.kchunk;
  const long k_end = (k_begin + p.kchunk < p.K) ? k_begin + p.kchunk : p.K;
  const int nkb = (int)((k_end - k_begin + kBK - 1) / kBK);
  const float* xbase = p.X.base + batch * p.X.batch_stride;
  const float* ybase = p.Y.base + batch * p.Y.batch_stride;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full_bar[s]), kLoaderThreads);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&accum_bar), 1);
    epi_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kLoaderWarps) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;
  bool ok = true;

  if (warp < kLoaderWarps) {
    // ------------------------------------------------ producers
    // DEPTH register buffers per thread: the loads of blocks kb+1 .. kb+DEPTH-1 are in flight while block
    // kb is split and stored, which is what keeps enough bytes outstanding to cover HBM latency.
    float xb[DEPTH][16], yb[DEPTH][YNV];
    TileLoader<XMODE, 16> lx;
    TileLoader<YMODE, YNV> ly;
    lx.init(p.X, xbase, x0, kXRows, tid);
    ly.init(p.Y, ybase, y0, UN, tid);
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      if (d < nkb) {
        const long k1 = k_begin + (long)d * kBK;
        const bool full = k1 + kBK <= k_end;
        lx.fetch(p.X, xbase, x0, kXRows, k1, k_end, full, xb[d], tid);
        ly.fetch(p.Y, ybase, y0, UN, k1, k_end, full, yb[d], tid);
      }
    }
    for (int kb0 = 0; kb0 < nkb && ok; kb0 += DEPTH) {
#pragma unroll
      for (int d = 0; d < DEPTH; ++d) {
        const int kb = kb0 + d;
        if (kb < nkb && ok) {
          const int s = kb % S;
          const uint32_t phase = (uint32_t)(kb / S) & 1u;
          ok = mbar_wait(smem_u32(&empty_bar[s]), phase ^ 1u);
          if (ok) {
            unsigned char* st = smem + (size_t)s * stage_bytes;
            lx.stash(kXRows, xb[d], st, st + x_bytes, tid);
            ly.stash(UN, yb[d], st + 2 * x_bytes, st + 2 * x_bytes + y_bytes, tid);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core
            mbar_arrive(smem_u32(&full_bar[s]));
            if (kb + DEPTH < nkb) {
              const long k1 = k_begin + (long)(kb + DEPTH) * kBK;
              const bool full = k1 + kBK <= k_end;
              lx.fetch(p.X, xbase, x0, kXRows, k1, k_end, full, xb[d], tid);
              ly.fetch(p.Y, ybase, y0, UN, k1, k_end, full, yb[d], tid);
            }
          }
        }
      }
    }
    // ------------------------------------------------ epilogue
    if (ok && nkb > 0) ok = mbar_wait(smem_u32(&accum_bar), 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!ok) epi_fail = 1;
    asm volatile("bar.sync 1, %0;" ::"n"(kLoaderThreads) : "memory");  // the 8 epilogue warps agree on success
    if (*(volatile int*)&epi_fail) {
      if (tid == 0) { *(volatile int*)p.err = 1; __threadfence_system(); }
    } else {
      // Accumulator -> shared-memory staging (the pipeline stages are idle now) -> coalesced stores.
      // TMEM lane quarter of a warp is (warp % 4); the two warps of a quarter take alternate chunks.
      float* stg = reinterpret_cast<float*>(smem);
      const int stride = UN + 1;  // odd: conflict-free both for row-wise writes and column-wise reads
      const int quarter = warp & 3, colhalf = warp >> 2;
      const int nchunks = UN / 16;
      for (int ch = colhalf; ch < nchunks; ch += 2) {
        const int c0 = ch * 16;
        uint32_t r[16];
        uint32_t taddr = tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        uint32_t r2[16];
        tmem_ld16(taddr + (uint32_t)UN, r2);  // columns [UN, 2UN) hold the x_hi * y_lo term
        float* dst = stg + (quarter * 32 + lane) * stride + c0;
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[j] = __uint_as_float(r[j]) + __uint_as_float(r2[j]);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kLoaderThreads) : "memory");
      float* cbase = (p.nsplit > 1) ? p.C + ((long)batch * p.nsplit + split) * p.M * p.N : p.C + batch * p.c_batch_stride;
      const long ld = (p.nsplit > 1) ? p.N : p.ldc;
      if (p.ep.y) {      // convolution output stage: lanes along pixels (tile rows), NCHW planes
        size_t obase[kXRows / 32];
        bool rok[kXRows / 32];
#pragma unroll
        for (int q = 0; q < kXRows / 32; ++q) {
          const long i_g = x0 + lane + 32 * q;
          rok[q] = i_g < p.X.rows;
          const long mm = rok[q] ? i_g : 0;
          const long b = mm / p.ep.HW, pix = mm - b * p.ep.HW;
          obase[q] = (size_t)b * p.Y.rows * p.ep.HW + pix;
        }
        for (int col = warp; col < UN; col += kLoaderWarps) {
          const long j_g = y0 + col;
          if (j_g >= p.Y.rows) break;
          const float bc = p.ep.bias[j_g];
          const size_t coff = (size_t)j_g * p.ep.HW;
#pragma unroll
          for (int q = 0; q < kXRows / 32; ++q) {
            if (rok[q]) {
              const float t = stg[(lane + 32 * q) * stride + col] + bc;
              const int8_t mk = (int8_t)(t >= 0.f);
              p.ep.mask[obase[q] + coff] = mk;
              p.ep.y[obase[q] + coff] = t * (float)mk;
            }
          }
        }
      } else if (!p.swapped) {  // tile row = product row: lanes along the product's columns
        for (int row = warp; row < kXRows; row += kLoaderWarps) {
          const long i_g = x0 + row;
          if (i_g >= p.X.rows) break;
          for (int col = lane; col < UN; col += 32) {
            const long j_g = y0 + col;
            if (j_g < p.Y.rows) cbase[i_g * ld + j_g] = stg[row * stride + col];
          }
        }
      } else {           // tile row = product column: lanes along tile rows
        for (int col = warp; col < UN; col += kLoaderWarps) {
          const long j_g = y0 + col;
          if (j_g >= p.Y.rows) break;
          for (int row = lane; row < kXRows; row += 32) {
            const long i_g = x0 + row;
            if (i_g < p.X.rows) cbase[j_g * ld + i_g] = stg[row * stride + col];
          }
        }
      }
    }
  } else {
    // ------------------------------------------------ MMA issuer
    // The whole warp runs the loop so that descriptors and addresses stay warp-uniform (uniform
    // registers feed tcgen05.mma directly); one elected lane issues. Two instructions per K step:
    // x_hi * [y_hi | y_lo] into accumulator columns [0, 2UN) and x_lo * y_hi into columns [0, UN).
    const uint32_t idesc1 = make_idesc_tf32(UN), idesc2 = make_idesc_tf32(2 * UN);
    for (int kb = 0; kb < nkb && ok; ++kb) {
      const int s = kb % S;
      const uint32_t phase = (uint32_t)(kb / S) & 1u;
      ok = mbar_wait(smem_u32(&full_bar[s]), phase);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t sbase = smem_u32(smem + (size_t)s * stage_bytes);
      const uint64_t dxh = make_desc(sbase), dxl = make_desc(sbase + x_bytes);
      const uint64_t dyh = make_desc(sbase + 2 * x_bytes);  // y_lo follows y_hi: one descriptor covers both
#pragma unroll
      for (int kk = 0; kk < kBK / 8; ++kk) {
        const uint64_t adv = (uint64_t)((kk * 32) >> 4);  // 8 tf32 = 32 bytes along K inside the swizzle row
        const uint32_t first = (kb == 0 && kk == 0) ? 0u : 1u;
        mma_tf32_elect(tmem_d, dxh + adv, dyh + adv, idesc2, first);
        mma_tf32_elect(tmem_d, dxl + adv, dyh + adv, idesc1, 1u);
      }
      if (elect_one()) mma_commit(smem_u32(&empty_bar[s]));  // frees the stage once these MMAs have read it
      __syncwarp();
    }
    if (ok && nkb > 0 && elect_one()) mma_commit(smem_u32(&accum_bar));
    __syncwarp();
    if (!ok && lane == 0) { *(volatile int*)p.err = 2; __threadfence_system(); }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kLoaderWarps) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)p.tmem_cols) : "memory");
  }
}

// Ordered fold of a split-K slab [P][nsplit][M*N] into C. With few splits a thread owns one output and
// adds the partials in split order. With many splits (a weight gradient whose K is the whole batch)
// eight threads share an output: thread g adds splits g, g+8, ... in order and the eight sums are
// combined as a fixed tree, so the result does not depend on scheduling.
__global__ void splitk_fold_tc_kernel(long P, long MN, int nsplit, const float* __restrict__ part, float* __restrict__ C, long M,
                                      long N, long ldc, long strideC) {
  long total = P * MN;
  for (long f = (long)blockIdx.x * blockDim.x + threadIdx.x; f < total; f += (long)gridDim.x * blockDim.x) {
    long p = f / MN, e = f - p * MN;
    long m = e / N, n = e - m * N;
    const float* src = part + (p * nsplit) * MN + e;
    float acc = src[0];
    for (int s = 1; s < nsplit; ++s) acc += src[(long)s * MN];
    C[p * strideC + m * ldc + n] = acc;
  }
}
constexpr int kFoldGroups = 8;
__global__ void __launch_bounds__(32 * kFoldGroups) splitk_fold_wide_kernel(long P, long MN, int nsplit, const float* __restrict__ part,
                                                                           float* __restrict__ C, long M, long N, long ldc,
                                                                           long strideC) {
  __shared__ float sums[kFoldGroups][33];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const long total = P * MN;
  for (long f0 = (long)blockIdx.x * 32; f0 < total; f0 += (long)gridDim.x * 32) {
    const long f = f0 + lane;
    float acc = 0.f;
    long p = 0, e = 0;
    if (f < total) {
      p = f / MN;
      e = f - p * MN;
      const float* src = part + (p * nsplit) * MN + e;
      for (int s = g; s < nsplit; s += kFoldGroups) acc += src[(long)s * MN];
    }
    sums[g][lane] = acc;
    __syncthreads();
    if (g == 0 && f < total) {
      const float r = ((sums[0][lane] + sums[1][lane]) + (sums[2][lane] + sums[3][lane])) +
                      ((sums[4][lane] + sums[5][lane]) + (sums[6][lane] + sums[7][lane]));
      const long m = e / N, n = e - m * N;
      C[p * strideC + m * ldc + n] = r;
    }
    __syncthreads();
  }
}

int* g_err_host = nullptr;  // host-mapped flag written by the kernel on a wait time-out
int* g_err_dev = nullptr;

}  // namespace

namespace cgtb {

// Reports (and clears) a time-out raised by the tensor-core kernel. Call after the stream is idle.
int* tc_error_flag() {
  if (!g_err_host) {
    if (cudaHostAlloc((void**)&g_err_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) { fail("cudaHostAlloc failed"); return nullptr; }
    *g_err_host = 0;
    if (cudaHostGetDevicePointer((void**)&g_err_dev, g_err_host, 0) != cudaSuccess) { fail("cudaHostGetDevicePointer failed"); return nullptr; }
  }
  return g_err_dev;
}

void tc_splitk_fold(long P, long M, long N, int nsplit, const float* part, float* C, long ldc, long strideC) {
  long total = P * M * N;
  if (nsplit >= 2 * kFoldGroups) {
    long blocks = std::min<long>(cgtb_ceil_div(total, 32), (long)rt().sm_count * 16);
    CGTB_LAUNCH(splitk_fold_wide_kernel, (unsigned)blocks, 32 * kFoldGroups, 0, P, M * N, nsplit, part, C, M, N, ldc, strideC);
  } else {
    long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 8);
    CGTB_LAUNCH(splitk_fold_tc_kernel, (unsigned)blocks, 256, 0, P, M * N, nsplit, part, C, M, N, ldc, strideC);
  }
}

int sgemm_tc_check() {
  if (g_err_host && *g_err_host) {
    int code = *g_err_host;
    *g_err_host = 0;
    return fail("a bounded device-side wait expired (code %d: 3-7 a barrier of the tensor-core GEMM / convolution kernels, 8 a rank "
                "of the peer-memory all-reduce did not arrive); the result of that call is invalid", code);
  }
  return 0;
}

int sgemm_tc(int tA, int tB, long P, long M, long N, long K, const float* A, long lda, long strideA, const float* B, long ldb,
             long strideB, float* C, long ldc, long strideC, const ConvEpilogue* ep) {
  if (P <= 0 || M <= 0 || N <= 0) return 0;
  if (K <= 0) return -1;                      // all-zero product: the FMA kernel handles it
  if (M * N < 1024 && K < 256) return -1;     // tiny: not worth a tensor-core launch
  if (!tc_error_flag()) return 1;
  Params p;
  auto mode_of = [](const float* base, long ld, long bstride, int kcontig) {
    if (!kcontig) return 0;
    bool al = ((uintptr_t)base & 15) == 0 && (ld & 3) == 0 && (bstride & 3) == 0;
    return al ? 2 : 1;
  };
  Operand opA = {A, lda, tA ? 0 : 1, mode_of(A, lda, strideA, tA ? 0 : 1), M, strideA};   // rows of op(A) are m
  Operand opB = {B, ldb, tB ? 1 : 0, mode_of(B, ldb, strideB, tB ? 1 : 0), N, strideB};   // rows of op(B)^T are n
  p.swapped = (N > M) ? 1 : 0;
  p.ep = ConvEpilogue{nullptr, nullptr, nullptr, 1};
  if (ep) {
    if (p.swapped || P != 1) return -1;
    p.ep = *ep;
  }
  p.X = p.swapped ? opB : opA;
  p.Y = p.swapped ? opA : opB;
  long ydim = p.Y.rows;
  int ytiles = (int)cgtb_ceil_div(ydim, 128);  // tiles of at most 128 columns keep two CTAs resident per SM
  int UN = (int)(cgtb_ceil_div(cgtb_ceil_div(ydim, ytiles), 16) * 16);
  if (UN < 16) UN = 16;
  ytiles = (int)cgtb_ceil_div(ydim, UN);
  long xtiles = cgtb_ceil_div(p.X.rows, kXRows);
  p.UN = UN;
  p.tmem_cols = 32;
  while (p.tmem_cols < 2 * UN) p.tmem_cols *= 2;  // hi*hi + lo*hi in [0, UN), hi*lo in [UN, 2UN)
  const long stage_bytes = 2L * kXRows * 128 + 2L * UN * 128;
  long nkb_total = cgtb_ceil_div(K, kBK);
  // split K when the output tiles alone cannot fill the machine
  long tiles = xtiles * ytiles * P;
  int nsplit = 1;
  long want = (long)rt().sm_count;
  if (tiles < want && nkb_total >= 8) {
    nsplit = (int)std::min<long>(std::max<long>(1, (2 * want) / tiles), nkb_total / 4);  // at most two CTAs per SM: one wave
    if (nsplit < 1) nsplit = 1;
  }
  long kchunk = cgtb_ceil_div(nkb_total, nsplit) * kBK;
  nsplit = (int)cgtb_ceil_div(K, kchunk);
  if ((long)P * nsplit > 65535 || ytiles > 65535) return -1;
  if (ep && nsplit > 1) return -1;  // the output stage needs whole sums
  p.nsplit = nsplit;
  p.kchunk = kchunk;
  p.K = K;
  p.M = M;
  p.N = N;
  long nkb = kchunk / kBK;
  // two resident CTAs per SM double the warps that hide instruction latency: prefer a stage count
  // that leaves room for a second CTA when two stages fit in half of the SM's shared memory
  const int fit_half = (int)((110L * 1024 - 1024) / stage_bytes);
  int stages = fit_half >= 2 ? std::min(fit_half, 3) : std::min<int>(3, (int)((200L * 1024) / stage_bytes));
  if (stages > nkb) stages = (int)std::max<long>(nkb, 1);
  if (stages < 1) stages = 1;
  p.stages = stages;
  p.ldc = ldc;
  p.c_batch_stride = strideC;
  p.err = g_err_dev;
  float* part = nullptr;
  if (nsplit > 1) {
    part = (float*)scratch((size_t)P * nsplit * M * N * sizeof(float));
    if (!part) return 1;
    p.C = part;
  } else {
    p.C = C;
  }
  size_t smem = (size_t)stages * stage_bytes;
  size_t staging = (size_t)kXRows * (UN + 1) * sizeof(float);  // epilogue staging re-uses the stage memory
  if (smem < staging) smem = staging;
  smem += 1024;
  dim3 grid((unsigned)xtiles, (unsigned)ytiles, (unsigned)(P * nsplit));
  const int cap = 227 * 1024 - 2048;
  // one instantiation per (X access pattern, Y access pattern, Y register slots)
#define TC_LAUNCH(XM, YM, NVY, DEP)                                                                                \
  {                                                                                                                \
    static bool cfg = false;                                                                                       \
    if (!cfg) { CGTB_CUDA_TRY(cudaFuncSetAttribute(sgemm_tc_kernel<XM, YM, NVY, DEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap)); cfg = true; } \
    CGTB_LAUNCH((sgemm_tc_kernel<XM, YM, NVY, DEP>), grid, kThreads, smem, p);                                      \
  }
  // Y register slots = UN/8 (minimum 4); small Y tiles leave room for a third register buffer
#define TC_CASE(XM, YM)                                                                                            \
  if (p.X.mode == XM && p.Y.mode == YM) {                                                                          \
    if (UN <= 32) TC_LAUNCH(XM, YM, 4, 3)                                                                          \
    else if (UN <= 64) TC_LAUNCH(XM, YM, 8, 3)                                                                     \
    else if (UN <= 128) TC_LAUNCH(XM, YM, 16, 2)                                                                   \
    else TC_LAUNCH(XM, YM, 32, 2)                                                                                  \
  }
  TC_CASE(0, 0) TC_CASE(0, 1) TC_CASE(0, 2) TC_CASE(1, 0) TC_CASE(1, 1) TC_CASE(1, 2) TC_CASE(2, 0) TC_CASE(2, 1) TC_CASE(2, 2)
#undef TC_CASE
#undef TC_LAUNCH
  if (nsplit > 1) tc_splitk_fold(P, M, N, nsplit, part, C, ldc, strideC);
  CGTB_CHECK_LAUNCH("sgemm_tc");
  return 0;
}

}  // namespace cgtb
