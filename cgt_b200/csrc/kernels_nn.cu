// im2col / col2im, max-pool forward / pullback, cross-channel LRN forward / backward for sm_100a.
//
// All of these are HBM-bound stencil or copy kernels: threads are laid out along the contiguous axis
// of the larger side of the transfer, shared memory stages the re-used input, and the arithmetic order
// follows the reference's CPU loops wherever the result depends on it (pool argmax tie-breaking,
// pool-pullback and col2im accumulation order), so integer outputs are bit-exact and float sums are
// added in the same sequence.
#include "runtime.h"
#include <cfloat>
#include <initializer_list>
#include <type_traits>

using namespace cgtb;

// ================================================================================================
// im2col : col[b, h, w, c] = x[b, c_im, h*sh - ph + i, w*sw - pw + j],  c = (c_im*kh + i)*kw + j
// (include/im2col.h:6-28). One block per (b, h) output row (several when rows are short): the
// C x kh input rows that the output row needs are staged in shared memory, each padded with zeros to
// Wp = (Wo-1)*sw + kw entries and zero for rows outside the image, so the copy-out needs no range
// test: col[.., w, c] = slab[offp[c] + w*sw] with offp[c] = (c_im*kh + i)*Wp + j. A thread owns four
// consecutive column channels (one 16-byte store per w) when the row pitch is a multiple of 4, else
// single channels, and walks along w; consecutive threads write consecutive addresses.
// A column row may be wider than Z (pitch Zp > Z, chosen by the caller so that rows start on 16-byte
// boundaries and the tensor-memory accelerator can address them): the extra entries are written as
// zeros, read from one all-zero slab row appended for that purpose.
// ================================================================================================
template <typename T>
__global__ void __launch_bounds__(256, 5) im2col_rows_kernel(const T* __restrict__ x, T* __restrict__ col, int C, int H, int W, int kh, int kw,
                                   int ph, int pw, int sh, int sw, int Ho, int Wo, int rows_per_block, long total_rows,
                                   int vec4, int Zp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int Zreal = C * kh * kw, Wp = (Wo - 1) * sw + kw, nrows = C * kh;
  const int Z = Zp;                                                  // entries per column row as stored
  int* offp = reinterpret_cast<int*>(smem_raw);                      // [Zp], padded to a multiple of 4
  T* slab = reinterpret_cast<T*>(offp + ((Z + 3) & ~3));             // [C*kh (+ 1 zero row)][Wp]
  for (int c = threadIdx.x; c < Z; c += blockDim.x) {
    const int j = c % kw, ri = c / kw;
    offp[c] = c < Zreal ? ri * Wp + j : nrows * Wp;
  }
  if (Zp > Zreal)
    for (int q = threadIdx.x; q < Wp; q += blockDim.x) slab[nrows * Wp + q] = T(0);
  for (int r = 0; r < rows_per_block; ++r) {
    const long row = (long)blockIdx.x * rows_per_block + r;  // row = b*Ho + h
    if (row >= total_rows) break;
    const long b = row / Ho;
    const int h = (int)(row - b * Ho);
    const T* xb = x + b * (long)C * H * W;
    __syncthreads();  // the previous row's copy-out has finished reading the slab (and offp is written)
    // staging: a warp takes four slab rows at a time (lanes along the row, no index division per
    // element) and issues their loads before the first store: bound by latency, not by bytes
    {
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
      for (int ri0 = warp; ri0 < nrows; ri0 += 4 * nwarps) {
        const T* src[4];
        bool rok[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int ri = ri0 + u * nwarps;
          const int c_im = ri / kh, i = ri - c_im * kh;
          const int hin = h * sh - ph + i;
          rok[u] = ri < nrows && hin >= 0 && hin < H;
          src[u] = xb + ((long)c_im * H + (rok[u] ? hin : 0)) * W - pw;
        }
        for (int wq = lane; wq < Wp; wq += 32) {
          const bool wok = wq >= pw && wq < W + pw;
          T v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = (rok[u] && wok) ? __ldg(src[u] + wq) : T(0);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (ri0 + u * nwarps < nrows) slab[(ri0 + u * nwarps) * Wp + wq] = v[u];
        }
      }
    }
    __syncthreads();
    T* out = col + row * (long)Wo * Z;
    if (vec4) {
      typedef typename std::conditional<sizeof(T) == 4, float4, double4>::type V4;
      // G groups of Z/4 threads when a row has few quads: group g takes w = g, g + G, ...
      const int zq = Z / 4;
      const int G = zq < (int)blockDim.x ? (int)blockDim.x / zq : 1;
      const int g = G > 1 ? (int)threadIdx.x / zq : 0;
      for (int q = G > 1 ? (int)threadIdx.x - g * zq : (int)threadIdx.x; q < zq && g < G; q += blockDim.x) {
        const int4 o = *reinterpret_cast<const int4*>(offp + 4 * q);
        const T *s0 = slab + o.x, *s1 = slab + o.y, *s2 = slab + o.z, *s3 = slab + o.w;
        V4* dst = reinterpret_cast<V4*>(out + 4 * q);
        for (int w = g; w < Wo; w += G) {
          const int k = w * sw;
          V4 v;
          v.x = s0[k]; v.y = s1[k]; v.z = s2[k]; v.w = s3[k];
          dst[(long)w * zq] = v;
        }
      }
    } else if (Z <= (int)blockDim.x / 2) {
      // few column channels: G groups of Z threads, group g takes w = g, g + G, ...
      const int G = blockDim.x / Z, g = threadIdx.x / Z, c = threadIdx.x - g * Z;
      if (g < G) {
        const T* s0 = slab + offp[c];
        for (int w = g; w < Wo; w += G) out[(long)w * Z + c] = s0[w * sw];
      }
    } else {
      for (int c = threadIdx.x; c < Z; c += blockDim.x) {
        const T* s0 = slab + offp[c];
        for (int w = 0; w < Wo; ++w) out[(long)w * Z + c] = s0[w * sw];
      }
    }
  }
}

// fallback when the slab does not fit in shared memory: one thread per output element
template <typename T>
__global__ void im2col_direct_kernel(const T* __restrict__ x, T* __restrict__ col, long total, int C, int H, int W,
                                     int kh, int kw, int ph, int pw, int sh, int sw, int Ho, int Wo, int Zp) {
  const int Z = C * kh * kw;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    int c = (int)(idx % Zp);
    long row = idx / Zp;
    if (c >= Z) { col[idx] = T(0); continue; }
    int w = (int)(row % Wo);
    long t = row / Wo;
    int h = (int)(t % Ho);
    long b = t / Ho;
    int j = c % kw, i = (c / kw) % kh, c_im = c / (kw * kh);
    int hin = h * sh - ph + i, win = w * sw - pw + j;
    col[idx] = (hin >= 0 && hin < H && win >= 0 && win < W) ? x[((b * C + c_im) * H + hin) * W + win] : T(0);
  }
}

template <typename T>
static int im2col_launch(const T* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh, int sw, long ldcol, T* col) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  if (B <= 0 || Ho <= 0 || Wo <= 0) return 0;
  const int Z = C * kh * kw;
  if (ldcol < Z || ldcol > Z + 1024) return fail("cgtb_im2col: row pitch %ld does not fit rows of %d entries", ldcol, Z);
  const int Zp = (int)ldcol;
  const int Wp = (Wo - 1) * sw + kw;
  size_t smem = (size_t)((Zp + 3) & ~3) * sizeof(int) + (size_t)(C * kh + (Zp > Z ? 1 : 0)) * Wp * sizeof(T);
  long total_rows = B * Ho;
  if (smem <= 200 * 1024) {
    if (smem > 48 * 1024)
      CGTB_CUDA_TRY(cudaFuncSetAttribute(im2col_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // several rows per block when a row is short, so each block moves at least ~16K elements
    int rpb = 1;
    while ((long)rpb * Wo * Zp < 16384 && rpb < 8) rpb *= 2;
    // ... but not at the price of a grid that leaves SMs short of resident blocks (measured: the CIFAR step gains
    // 2 % when the 6x6 and 32x32 layers get 10 blocks per SM instead of 1.3 and 3.5)
    while (rpb > 1 && cgtb_ceil_div(total_rows, rpb) < 10L * rt().sm_count) rpb /= 2;
    long blocks = cgtb_ceil_div(total_rows, rpb);
    const int vec4 = ((Zp & 3) == 0 && ((uintptr_t)col & (4 * sizeof(T) - 1)) == 0) ? 1 : 0;
    CGTB_LAUNCH(im2col_rows_kernel<T>, (unsigned)blocks, 256, smem, x, col, C, H, W, kh, kw, ph, pw, sh, sw, Ho, Wo, rpb,
                total_rows, vec4, Zp);
  } else {
    long total = total_rows * Wo * Zp;
    long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 16);
    CGTB_LAUNCH(im2col_direct_kernel<T>, (unsigned)blocks, 256, 0, x, col, total, C, H, W, kh, kw, ph, pw, sh, sw, Ho, Wo, Zp);
  }
  CGTB_CHECK_LAUNCH("im2col");
  return 0;
}

CGTB_API int cgtb_im2col_ld(int dtype, const void* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                            int sw, long ldcol, void* col) {
  if (!require_runtime("cgtb_im2col")) return 1;
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0) return fail("cgtb_im2col: kernel and stride must be positive");
  if (dtype == cgtb_f4) return im2col_launch<float>((const float*)x, B, C, H, W, kh, kw, ph, pw, sh, sw, ldcol, (float*)col);
  if (dtype == cgtb_f8) return im2col_launch<double>((const double*)x, B, C, H, W, kh, kw, ph, pw, sh, sw, ldcol, (double*)col);
  return fail("cgtb_im2col: unsupported dtype %d", dtype);
}

CGTB_API int cgtb_im2col(int dtype, const void* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                         int sw, void* col) {
  return cgtb_im2col_ld(dtype, x, B, C, H, W, kh, kw, ph, pw, sh, sw, (long)C * kh * kw, col);
}

// ================================================================================================
// col2im (include/im2col.h:30-50) written as a gather: one thread per image pixel adds the column
// entries that map onto it in ascending column-channel order (i, then j), which is the order in
// which the reference's scatter loop reaches that pixel, so the float sum is bit-identical and no
// atomics are needed.
// ================================================================================================
template <typename T, typename I>
__global__ void col2im_gather_kernel(const T* __restrict__ col, T* __restrict__ im, I total, int C, int H, int W,
                                     int kh, int kw, int ph, int pw, int sh, int sw, int Ho, int Wo) {
  const int Z = C * kh * kw;
  for (I idx = (I)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (I)gridDim.x * blockDim.x) {
    I t = idx / (I)W;
    int xw = (int)(idx - t * (I)W);
    I t2 = t / (I)H;
    int y = (int)(t - t2 * (I)H);
    I b = t2 / (I)C;
    int c_im = (int)(t2 - b * (I)C);
    const T* colb = col + b * (long)Ho * Wo * Z;
    T acc = T(0);
    for (int i = 0; i < kh; ++i) {
      int hn = y + ph - i;
      if (hn < 0) break;
      int h = hn / sh;
      if (h * sh != hn || h >= Ho) continue;
      for (int j = 0; j < kw; ++j) {
        int wn = xw + pw - j;
        if (wn < 0) break;
        int w = wn / sw;
        if (w * sw != wn || w >= Wo) continue;
        acc += colb[((long)h * Wo + w) * Z + (c_im * kh + i) * kw + j];
      }
    }
    im[idx] = acc;
  }
}

// Staged variant for images of at most 1024/CG pixels: one block per (image, group of CG channels), one
// thread per pixel of the group. The block streams its slice of the column matrix exactly once, one
// output-grid row h at a time (Wo segments of CG*kh*kw contiguous values) through a ring of shared-memory
// slabs filled by cp.async, from h = Ho-1 down to 0, so that for every pixel the kernel offset
// i = y + ph - h*sh rises from slab to slab and j rises inside a slab: the (i, j) order of the gather
// above, bit-identical sums. Lanes run along c, then x: the slab addresses of a warp fall into distinct
// banks for the usual odd kernels. The result leaves through shared memory as contiguous planes.
template <typename T, int STAGES>
__global__ void __launch_bounds__(1024, 2) col2im_image_kernel(const T* __restrict__ col, T* __restrict__ im, int C, int H, int W,
                                                          int kh, int kw, int ph, int pw, int sh, int sw, int Ho, int Wo,
                                                          int CG, int ngroups) {
  extern __shared__ __align__(16) unsigned char smem_img[];
  T* ring = reinterpret_cast<T*>(smem_img);
  const int Z = C * kh * kw, CGZ = CG * kh * kw, slab_n = Wo * CGZ;
  const int b = blockIdx.x / ngroups, g = blockIdx.x - b * ngroups;
  const int t = threadIdx.x;
  const int npix = CG * H * W;
  const int c = t % CG, x = (t / CG) % W, y = t / (CG * W);
  const bool active = t < npix;
  const T* colb = col + (size_t)b * Ho * Wo * Z + (size_t)g * CGZ;
  const int seg16 = CGZ * (int)sizeof(T) / 16;  // 16-byte units per segment
  // Slabs travel in groups of G: one commit group, one wait and one pair of block barriers per G
  // slabs (the barriers, not the bytes, were the cost with 29 warps per block). NG groups form the ring.
  constexpr int G = 3, NG = STAGES / G;
  static_assert(STAGES % G == 0 && NG >= 2, "the ring holds whole groups");
  const int ngroups_total = (Ho + G - 1) / G;
  // a thread copies the same 16-byte units of every slab: their offsets are computed once
  constexpr int NQ = 2;
  const int nunits = Wo * seg16;
  uint32_t soff[NQ], doff[NQ];
#pragma unroll
  for (int u = 0; u < NQ; ++u) {
    const int q = t + u * blockDim.x;
    const int w = q / seg16, r = q - w * seg16;
    soff[u] = (uint32_t)((size_t)w * Z * sizeof(T) + (size_t)r * 16);
    doff[u] = (uint32_t)((size_t)w * CGZ * sizeof(T) + (size_t)r * 16);
  }
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
  auto prefetch_group = [&](int gi) {
    if (gi < ngroups_total) {
      const int slot0 = (gi % NG) * G;
#pragma unroll
      for (int s2 = 0; s2 < G; ++s2) {
        const int h = Ho - 1 - (gi * G + s2);
        if (h >= 0) {
          const uint32_t dst = ring_s + (uint32_t)((size_t)(slot0 + s2) * slab_n * sizeof(T));
          const unsigned char* src = reinterpret_cast<const unsigned char*>(colb + (size_t)h * Wo * Z);
#pragma unroll
          for (int u = 0; u < NQ; ++u)
            if (t + u * (int)blockDim.x < nunits)
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + doff[u]), "l"(src + soff[u]) : "memory");
          for (int q = t + NQ * blockDim.x; q < nunits; q += blockDim.x) {  // blocks with few threads
            const int w = q / seg16, r = q - w * seg16;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)((size_t)w * CGZ * sizeof(T) + (size_t)r * 16)),
                         "l"(src + ((size_t)w * Z * sizeof(T) + (size_t)r * 16))
                         : "memory");
          }
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // an empty group keeps the group count uniform
  };
#pragma unroll
  for (int gi = 0; gi < NG - 1; ++gi) prefetch_group(gi);
  T acc = T(0);
  for (int gi = 0; gi < ngroups_total; ++gi) {
    prefetch_group(gi + NG - 1);
    asm volatile("cp.async.wait_group %0;" ::"n"(NG - 1) : "memory");
    __syncthreads();
#pragma unroll
    for (int s2 = 0; s2 < G; ++s2) {
      const int h = Ho - 1 - (gi * G + s2);
      const int i = y + ph - h * sh;
      if (h >= 0 && active && i >= 0 && i < kh) {
        const T* base = ring + (size_t)((gi % NG) * G + s2) * slab_n + (c * kh + i) * kw;
        if (sw == 1) {  // unit stride: no division, j limited so that 0 <= x + pw - j < Wo
          const int j0 = max(0, x + pw - (Wo - 1)), j1 = min(kw - 1, x + pw);
          for (int j = j0; j <= j1; ++j) acc += base[(x + pw - j) * CGZ + j];
        } else {
          for (int j = 0; j < kw; ++j) {
            const int wn = x + pw - j;
            if (wn < 0) break;
            const int w = wn / sw;
            if (w * sw != wn || w >= Wo) continue;
            acc += base[w * CGZ + j];
          }
        }
      }
    }
    __syncthreads();  // this group's slots are the target of the prefetch issued in the next iteration
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  T* outb = ring;
  if (active) outb[(c * H + y) * W + x] = acc;
  __syncthreads();
  T* imb = im + ((size_t)b * C + (size_t)g * CG) * H * W;
  for (int q = t; q < npix; q += blockDim.x) imb[q] = outb[q];
}

template <typename T>
static int col2im_launch(const T* col, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh, int sw, T* im) {
  int Ho = (H + 2 * ph - kh) / sh + 1, Wo = (W + 2 * pw - kw) / sw + 1;
  long total = B * C * H * W;
  if (total <= 0) return 0;
  if (Ho > 0 && Wo > 0 && (long)H * W <= 1024 && B * C < (1L << 30)) {
    // staged kernel: the largest channel group CG dividing C whose pixels fit one block and whose
    // segments are whole 16-byte units
    int CG = 0;
    for (int cand = C; cand >= 1; --cand)
      if (C % cand == 0 && (long)cand * H * W <= 1024 && ((long)cand * kh * kw * sizeof(T)) % 16 == 0) { CG = cand; break; }
    constexpr int kStages = 9;  // three groups of three slabs: six slabs in flight per block while three are summed
    if (CG > 0 && ((uintptr_t)col & 15) == 0 && ((long)C * kh * kw * sizeof(T)) % 16 == 0) {
      const long slab_bytes = (long)Wo * CG * kh * kw * sizeof(T);
      const size_t smem = (size_t)std::max<long>(kStages * slab_bytes, (long)CG * H * W * sizeof(T));
      if (smem <= 96 * 1024) {
        const int threads = (int)(cgtb_ceil_div((long)CG * H * W, 32) * 32);
        if (smem > 48 * 1024)
          CGTB_CUDA_TRY(cudaFuncSetAttribute((col2im_image_kernel<T, kStages>), cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        CGTB_LAUNCH((col2im_image_kernel<T, kStages>), (unsigned)(B * (C / CG)), threads, smem, col, im, C, H, W, kh, kw, ph, pw,
                    sh, sw, Ho, Wo, CG, C / CG);
        CGTB_CHECK_LAUNCH("col2im");
        return 0;
      }
    }
  }
  long blocks = std::min<long>(cgtb_ceil_div(total, 256), (long)rt().sm_count * 32);
  if (total < (1L << 31))  // 32-bit index arithmetic: a 64-bit division costs several times a 32-bit one
    CGTB_LAUNCH((col2im_gather_kernel<T, unsigned>), (unsigned)blocks, 256, 0, col, im, (unsigned)total, C, H, W, kh, kw, ph, pw, sh, sw, Ho, Wo);
  else
    CGTB_LAUNCH((col2im_gather_kernel<T, long>), (unsigned)blocks, 256, 0, col, im, total, C, H, W, kh, kw, ph, pw, sh, sw, Ho, Wo);
  CGTB_CHECK_LAUNCH("col2im");
  return 0;
}

CGTB_API int cgtb_col2im(int dtype, const void* col, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                         int sw, void* im) {
  if (!require_runtime("cgtb_col2im")) return 1;
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0) return fail("cgtb_col2im: kernel and stride must be positive");
  if (dtype == cgtb_f4) return col2im_launch<float>((const float*)col, B, C, H, W, kh, kw, ph, pw, sh, sw, (float*)im);
  if (dtype == cgtb_f8) return col2im_launch<double>((const double*)col, B, C, H, W, kh, kw, ph, pw, sh, sw, (double*)im);
  return fail("cgtb_col2im: unsupported dtype %d", dtype);
}

// ================================================================================================
// max pool forward (include/pooling.h:24-71). One thread per pooled element; the window is scanned
// h-major with a strict '>' from (-FLT_MAX, -1), so ties and NaNs resolve exactly as in the CPU loop.
//
// Thread layout for both pooling kernels: threadIdx.x runs along the row, threadIdx.y along rows,
// threadIdx.z over image planes (several small planes share a block), blockIdx.x over plane groups:
// no thread divides an index. Window extents and strides are template parameters for the common
// 3x3/2 and 2x2/2 windows (0 = taken from the arguments), which turns the window arithmetic into shifts.
// ================================================================================================
struct PoolGeom {
  int H, W, kh, kw, ph, pw, sh, sw, PH, PW;
};

template <typename T, int KH, int KW, int SH, int SW>
__global__ void max_pool_kernel(const T* __restrict__ x, T* __restrict__ top, int32_t* __restrict__ mask, long planes,
                                const PoolGeom g) {
  const int kh = KH ? KH : g.kh, kw = KW ? KW : g.kw, sh = SH ? SH : g.sh, sw = SW ? SW : g.sw;
  const int px = blockIdx.z * blockDim.x + threadIdx.x, py = blockIdx.y * blockDim.y + threadIdx.y;
  const long plane = (long)blockIdx.x * blockDim.z + threadIdx.z;
  if (px >= g.PW || py >= g.PH || plane >= planes) return;
  const T* xp = x + plane * (long)g.H * g.W;
  T best = T(-FLT_MAX);
  int besti = -1;
  if constexpr (KH > 0) {
    // compile-time window: every load is issued up front (clamped address), the scan order stays h-major
    const int h0 = py * SH - g.ph, w0 = px * SW - g.pw;
    T v[KH][KW];
#pragma unroll
    for (int dh = 0; dh < KH; ++dh)
#pragma unroll
      for (int dw = 0; dw < KW; ++dw) {
        const int h = h0 + dh, w = w0 + dw;
        const bool ok = h >= 0 && h < g.H && w >= 0 && w < g.W;
        v[dh][dw] = ok ? xp[h * g.W + w] : T(-FLT_MAX);  // never greater than `best`: skipped like an outside cell
      }
#pragma unroll
    for (int dh = 0; dh < KH; ++dh)
#pragma unroll
      for (int dw = 0; dw < KW; ++dw)
        if (v[dh][dw] > best) { best = v[dh][dw]; besti = (h0 + dh) * g.W + (w0 + dw); }
  } else {
    int hstart = py * sh - g.ph, wstart = px * sw - g.pw;
    const int hend = min(hstart + kh, g.H), wend = min(wstart + kw, g.W);
    hstart = max(hstart, 0);
    wstart = max(wstart, 0);
    for (int h = hstart; h < hend; ++h)
      for (int w = wstart; w < wend; ++w) {
        const T v = xp[h * g.W + w];
        if (v > best) { best = v; besti = h * g.W + w; }
      }
  }
  const long o = (plane * g.PH + py) * g.PW + px;
  top[o] = best;
  mask[o] = besti;
}

// max pool pullback (include/pooling.h:73-104) as a gather: one thread per input pixel visits the
// pooled windows that can contain it in ascending (ph, pw) order and adds the gradients whose argmax
// is this pixel; the reference scatter reaches each pixel in the same order.
template <typename T, int KH, int KW, int SH, int SW>
__global__ void max_pool_pullback_kernel(const int32_t* __restrict__ mask, const T* __restrict__ gtop, T* __restrict__ gx,
                                         long planes, const PoolGeom g) {
  const int kh = KH ? KH : g.kh, kw = KW ? KW : g.kw, sh = SH ? SH : g.sh, sw = SW ? SW : g.sw;
  const int w = blockIdx.z * blockDim.x + threadIdx.x, h = blockIdx.y * blockDim.y + threadIdx.y;
  const long plane = (long)blockIdx.x * blockDim.z + threadIdx.z;
  if (w >= g.W || h >= g.H || plane >= planes) return;
  const int32_t* mp = mask + plane * (long)g.PH * g.PW;
  const T* gp = gtop + plane * (long)g.PH * g.PW;
  // windows with py*sh - ph <= h < py*sh - ph + kh
  const int hy = h + g.ph - kh + 1, wx = w + g.pw - kw + 1;
  const int py0 = hy <= 0 ? 0 : (hy + sh - 1) / sh;
  const int py1 = min((h + g.ph) / sh, g.PH - 1);
  const int px0 = wx <= 0 ? 0 : (wx + sw - 1) / sw;
  const int px1 = min((w + g.pw) / sw, g.PW - 1);
  const int me = h * g.W + w;
  T acc = T(0);
  if constexpr (KH > 0) {
    // at most NY x NX windows cover a pixel: load every mask / gradient pair first (clamped address),
    // then add the matching ones in (py, px) order
    constexpr int NY = (KH + SH - 1) / SH, NX = (KW + SW - 1) / SW;
    int mv[NY][NX];
    T gv[NY][NX];
#pragma unroll
    for (int a = 0; a < NY; ++a)
#pragma unroll
      for (int b = 0; b < NX; ++b) {
        const int py = py0 + a, px = px0 + b;
        const bool ok = py <= py1 && px <= px1;
        const int o = ok ? py * g.PW + px : 0;
        mv[a][b] = ok ? mp[o] : -2;
        gv[a][b] = gp[o];
      }
#pragma unroll
    for (int a = 0; a < NY; ++a)
#pragma unroll
      for (int b = 0; b < NX; ++b)
        if (mv[a][b] == me) acc += gv[a][b];
  } else {
    for (int py = py0; py <= py1; ++py)
      for (int px = px0; px <= px1; ++px)
        if (mp[py * g.PW + px] == me) acc += gp[py * g.PW + px];
  }
  gx[(plane * g.H + h) * g.W + w] = acc;
}

// Pullback for rows whose length is a multiple of four (compile-time window): a thread owns four
// consecutive pixels. The windows that can cover them span NY rows x NXG columns of the pooled plane;
// their masks and gradients are loaded once (instead of once per pixel), every pixel then adds its
// matches in (py, px) order, and the four sums leave as one 16-byte store.
template <typename T, int KH, int KW, int SH, int SW>
__global__ void max_pool_pullback_vec4_kernel(const int32_t* __restrict__ mask, const T* __restrict__ gtop, T* __restrict__ gx,
                                              long planes, const PoolGeom g) {
  constexpr int NY = (KH + SH - 1) / SH, NXG = (KW + 2) / SW + 1;
  const int w0 = 4 * (blockIdx.z * blockDim.x + threadIdx.x), h = blockIdx.y * blockDim.y + threadIdx.y;
  const long plane = (long)blockIdx.x * blockDim.z + threadIdx.z;
  if (w0 >= g.W || h >= g.H || plane >= planes) return;
  const int32_t* mp = mask + plane * (long)g.PH * g.PW;
  const T* gp = gtop + plane * (long)g.PH * g.PW;
  const int hy = h + g.ph - KH + 1, wx = w0 + g.pw - KW + 1;
  const int py0 = hy <= 0 ? 0 : (hy + SH - 1) / SH;
  const int py1 = min((h + g.ph) / SH, g.PH - 1);
  const int px0 = wx <= 0 ? 0 : (wx + SW - 1) / SW;
  const int px1 = min((w0 + 3 + g.pw) / SW, g.PW - 1);
  int mv[NY][NXG];
  T gv[NY][NXG];
#pragma unroll
  for (int a = 0; a < NY; ++a)
#pragma unroll
    for (int b = 0; b < NXG; ++b) {
      const int py = py0 + a, px = px0 + b;
      const bool ok = py <= py1 && px <= px1;
      const int o = ok ? py * g.PW + px : 0;
      mv[a][b] = ok ? mp[o] : -2;
      gv[a][b] = gp[o];
    }
  T acc[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int me = h * g.W + w0 + p;
    T s = T(0);
#pragma unroll
    for (int a = 0; a < NY; ++a)
#pragma unroll
      for (int b = 0; b < NXG; ++b)
        if (mv[a][b] == me) s += gv[a][b];  // the mask names this pixel only if the window covers it
    acc[p] = s;
  }
  typedef typename std::conditional<sizeof(T) == 4, float4, double4>::type V4;
  V4 v;
  v.x = acc[0]; v.y = acc[1]; v.z = acc[2]; v.w = acc[3];
  *reinterpret_cast<V4*>(gx + (plane * g.H + h) * g.W + w0) = v;
}

// block (x, y, planes) and grid for a plane of `rows` x `cols` elements
static void pool_launch_dims(long planes, int rows, int cols, dim3& grid, dim3& block) {
  int bx = 1;
  while (bx < 32 && bx < cols) bx *= 2;
  int by = 1;
  while (by < 256 / bx && by < rows) by *= 2;
  int bz = 256 / (bx * by);
  if (bz > planes) bz = (int)std::max<long>(planes, 1);
  block = dim3(bx, by, bz);
  grid = dim3((unsigned)cgtb_ceil_div(planes, bz), (unsigned)cgtb_ceil_div(rows, by), (unsigned)cgtb_ceil_div(cols, bx));
}

#define CGTB_POOL_DISPATCH(KERNEL, T, ...)                                                             \
  do {                                                                                                 \
    if (kh == 3 && kw == 3 && sh == 2 && sw == 2) CGTB_LAUNCH((KERNEL<T, 3, 3, 2, 2>), grid, block, 0, __VA_ARGS__); \
    else if (kh == 2 && kw == 2 && sh == 2 && sw == 2) CGTB_LAUNCH((KERNEL<T, 2, 2, 2, 2>), grid, block, 0, __VA_ARGS__); \
    else CGTB_LAUNCH((KERNEL<T, 0, 0, 0, 0>), grid, block, 0, __VA_ARGS__);                                  \
  } while (0)

CGTB_API int cgtb_max_pool(int dtype, const void* x, long B, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
                           int sw, int PH, int PW, void* top, int32_t* mask) {
  if (!require_runtime("cgtb_max_pool")) return 1;
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0) return fail("cgtb_max_pool: kernel and stride must be positive");
  const long planes = B * C;
  if (planes * PH * PW <= 0) return 0;
  if (planes >= (1L << 31)) return fail("cgtb_max_pool: too many image planes");
  const PoolGeom g = {H, W, kh, kw, ph, pw, sh, sw, PH, PW};
  dim3 grid, block;
  pool_launch_dims(planes, PH, PW, grid, block);
  if (grid.y > 65535 || grid.z > 65535) return fail("cgtb_max_pool: plane too large");
  if (dtype == cgtb_f4)
    CGTB_POOL_DISPATCH(max_pool_kernel, float, (const float*)x, (float*)top, mask, planes, g);
  else if (dtype == cgtb_f8)
    CGTB_POOL_DISPATCH(max_pool_kernel, double, (const double*)x, (double*)top, mask, planes, g);
  else
    return fail("cgtb_max_pool: unsupported dtype %d", dtype);
  CGTB_CHECK_LAUNCH("max_pool");
  return 0;
}

CGTB_API int cgtb_max_pool_pullback(int dtype, const int32_t* mask, const void* gtop, long B, int C, int PH, int PW,
                                    int H, int W, int kh, int kw, int ph, int pw, int sh, int sw, void* gx) {
  if (!require_runtime("cgtb_max_pool_pullback")) return 1;
  if (kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0) return fail("cgtb_max_pool_pullback: kernel and stride must be positive");
  const long planes = B * C;
  if (planes * H * W <= 0) return 0;
  if (planes >= (1L << 31)) return fail("cgtb_max_pool_pullback: too many image planes");
  const PoolGeom g = {H, W, kh, kw, ph, pw, sh, sw, PH, PW};
  dim3 grid, block;
  pool_launch_dims(planes, H, W, grid, block);
  if (grid.y > 65535 || grid.z > 65535) return fail("cgtb_max_pool_pullback: plane too large");
  const bool known = (kh == 3 && kw == 3 && sh == 2 && sw == 2) || (kh == 2 && kw == 2 && sh == 2 && sw == 2);
  if (dtype == cgtb_f4 && known && (W % 4) == 0 && ((uintptr_t)gx & 15) == 0) {
    pool_launch_dims(planes, H, W / 4, grid, block);
    if (kh == 3) CGTB_LAUNCH((max_pool_pullback_vec4_kernel<float, 3, 3, 2, 2>), grid, block, 0, mask, (const float*)gtop, (float*)gx, planes, g);
    else CGTB_LAUNCH((max_pool_pullback_vec4_kernel<float, 2, 2, 2, 2>), grid, block, 0, mask, (const float*)gtop, (float*)gx, planes, g);
  } else if (dtype == cgtb_f4)
    CGTB_POOL_DISPATCH(max_pool_pullback_kernel, float, mask, (const float*)gtop, (float*)gx, planes, g);
  else if (dtype == cgtb_f8)
    CGTB_POOL_DISPATCH(max_pool_pullback_kernel, double, mask, (const double*)gtop, (double*)gx, planes, g);
  else
    return fail("cgtb_max_pool_pullback: unsupported dtype %d", dtype);
  CGTB_CHECK_LAUNCH("max_pool_pullback");
  return 0;
}

// ================================================================================================
// Cross-channel LRN (include/lrn.cuh). One thread per element; the window sum is formed directly
// (ascending channel) instead of the reference's running add/subtract, which removes the serial
// dependency along channels and is at least as accurate. scale = 1. + accum*(alpha/n) is evaluated
// with the product in T and the sum in double, as the reference expression does.
//   forward window of channel c : [c - (n-1)/2, c + n - (n-1)/2 - 1]
//   backward window of channel c: [c - (n - (n+1)/2), c + (n+1)/2 - 1]
// ================================================================================================
// grid = (ceil(HW / blockDim), C, N): the channel and image come from the block index, no thread divides
template <typename T>
__global__ void lrn_forward_kernel(const T* __restrict__ x, T* __restrict__ top, T* __restrict__ scale, int C, int HW,
                                   int size, T alpha_over_size, T negative_beta) {
  const int pre = (size - 1) / 2, post = size - pre - 1;
  const int hw = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (hw >= HW) return;
  const size_t nbase = (size_t)blockIdx.z * C * HW + hw;
  const T* col = x + nbase;
  const int lo = max(c - pre, 0), hi = min(c + post, C - 1);
  T acc = T(0);
  for (int k = lo; k <= hi; ++k) {
    const T v = col[k * HW];
    acc += v * v;
  }
  const T s = (T)(1. + (double)(acc * alpha_over_size));
  const size_t o = nbase + (size_t)c * HW;
  scale[o] = s;
  top[o] = col[c * HW] * pow(s, negative_beta);
}

template <typename T>
__global__ void lrn_backward_kernel(const T* __restrict__ x, const T* __restrict__ top, const T* __restrict__ scale,
                                    const T* __restrict__ gtop, T* __restrict__ gx, int C, int HW, int size,
                                    T negative_beta, T cache_ratio) {
  const int pre = size - (size + 1) / 2, post = size - pre - 1;
  const int hw = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (hw >= HW) return;
  const size_t nbase = (size_t)blockIdx.z * C * HW + hw;
  const int lo = max(c - pre, 0), hi = min(c + post, C - 1);
  T acc = T(0);
  for (int k = lo; k <= hi; ++k) {
    const size_t o = nbase + (size_t)k * HW;
    acc += gtop[o] * top[o] / scale[o];
  }
  const size_t idx = nbase + (size_t)c * HW;
  gx[idx] = gtop[idx] * pow(scale[idx], negative_beta) - cache_ratio * x[idx] * acc;
}

// float32 with the channel window staged in shared memory: a block takes kLrnTP consecutive pixels of one image for
// ALL channels, reads every input element from global memory once (runs of consecutive pixels per channel, several
// loads per thread in flight; 128-bit when the plane size allows), forms the window sums from the staged tile and
// writes its results as the same runs. Same operations in the same order as the kernels above: same bits.
// V = elements per access (4: HW a multiple of four and 16-byte aligned arrays).
constexpr int kLrnTP = 32;
// scale^(-beta) for the two exponents the networks of the reference use (cgt/nn_ops/cross_channel_lrn.py: beta 0.75;
// its test: 0.5) from square roots, which are correctly rounded: s^-0.5 = 1 / sqrt(s), s^-0.75 = 1 / (sqrt(s) * sqrt(sqrt(s))).
// A handful of instructions instead of the hundred of powf, to within 2 units in the last place of it. mode 0: powf.
__device__ __forceinline__ float lrn_pow(float s, float negative_beta, int mode) {
  if (mode == 1) return __fdiv_rn(1.0f, __fsqrt_rn(s));
  if (mode == 2) { const float r = __fsqrt_rn(s); return __fdiv_rn(1.0f, __fmul_rn(r, __fsqrt_rn(r))); }
  return pow(s, negative_beta);
}
static int lrn_pow_mode(double beta) { return beta == 0.5 ? 1 : (beta == 0.75 ? 2 : 0); }
template <int V>
__global__ void __launch_bounds__(256) lrn_forward_tile_kernel(const float* __restrict__ x, float* __restrict__ top, float* __restrict__ scale,
                                                             int C, int HW, int size, float alpha_over_size, float negative_beta, int pmode) {
  extern __shared__ float sx[];  // [C][kLrnTP]
  constexpr int PT = kLrnTP / V;           // threads along the pixels of a tile
  constexpr int CSTEP = 256 / PT;          // channels covered by one pass of the block
  const int pre = (size - 1) / 2, post = size - pre - 1;
  const int p = (threadIdx.x % PT) * V, c0 = threadIdx.x / PT;
  const int p0 = blockIdx.x * kLrnTP;
  const size_t base = (size_t)blockIdx.y * C * HW + p0 + p;
  const bool live = p0 + p < HW;   // with V = 4 a group of four is inside the plane or outside it as a whole
  for (int cb = c0; cb < C; cb += 8 * CSTEP) {
    float v[8][V];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = cb + u * CSTEP;
#pragma unroll
      for (int q = 0; q < V; ++q) v[u][q] = 0.f;
      if (c < C && live) {
        if (V == 4) {
          const float4 t = *reinterpret_cast<const float4*>(x + base + (size_t)c * HW);
          v[u][0] = t.x; v[u][1 % V] = t.y; v[u][2 % V] = t.z; v[u][3 % V] = t.w;
        } else {
          v[u][0] = x[base + (size_t)c * HW];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = cb + u * CSTEP;
      if (c < C) {
#pragma unroll
        for (int q = 0; q < V; ++q) sx[c * kLrnTP + p + q] = v[u][q];
      }
    }
  }
  __syncthreads();
  if (!live) return;
  for (int c = c0; c < C; c += CSTEP) {
    const int lo = max(c - pre, 0), hi = min(c + post, C - 1);
    float acc[V], s[V], y[V];
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = 0.f;
    for (int k = lo; k <= hi; ++k) {
#pragma unroll
      for (int q = 0; q < V; ++q) {
        const float t = sx[k * kLrnTP + p + q];
        acc[q] += t * t;
      }
    }
#pragma unroll
    for (int q = 0; q < V; ++q) {
      s[q] = (float)(1. + (double)(acc[q] * alpha_over_size));
      y[q] = sx[c * kLrnTP + p + q] * lrn_pow(s[q], negative_beta, pmode);
    }
    const size_t o = base + (size_t)c * HW;
    if (V == 4) {
      *reinterpret_cast<float4*>(scale + o) = make_float4(s[0], s[1 % V], s[2 % V], s[3 % V]);
      *reinterpret_cast<float4*>(top + o) = make_float4(y[0], y[1 % V], y[2 % V], y[3 % V]);
    } else {
      scale[o] = s[0];
      top[o] = y[0];
    }
  }
}

template <int V>
__global__ void __launch_bounds__(256) lrn_backward_tile_kernel(const float* __restrict__ x, const float* __restrict__ top,
                                                              const float* __restrict__ scale, const float* __restrict__ gtop,
                                                              float* __restrict__ gx, int C, int HW, int size, float negative_beta,
                                                              float cache_ratio, int pmode) {
  extern __shared__ float sr[];  // [C][kLrnTP]: gtop * top / scale
  constexpr int PT = kLrnTP / V;
  constexpr int CSTEP = 256 / PT;
  const int pre = size - (size + 1) / 2, post = size - pre - 1;
  const int p = (threadIdx.x % PT) * V, c0 = threadIdx.x / PT;
  const int p0 = blockIdx.x * kLrnTP;
  const size_t base = (size_t)blockIdx.y * C * HW + p0 + p;
  const bool live = p0 + p < HW;
  for (int cb = c0; cb < C; cb += 4 * CSTEP) {
    float g[4][V], t[4][V], sc[4][V];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = cb + u * CSTEP;
#pragma unroll
      for (int q = 0; q < V; ++q) { g[u][q] = 0.f; t[u][q] = 0.f; sc[u][q] = 1.f; }
      if (c < C && live) {
        const size_t o = base + (size_t)c * HW;
        if (V == 4) {
          const float4 a = *reinterpret_cast<const float4*>(gtop + o), b = *reinterpret_cast<const float4*>(top + o),
                       d = *reinterpret_cast<const float4*>(scale + o);
          g[u][0] = a.x; g[u][1 % V] = a.y; g[u][2 % V] = a.z; g[u][3 % V] = a.w;
          t[u][0] = b.x; t[u][1 % V] = b.y; t[u][2 % V] = b.z; t[u][3 % V] = b.w;
          sc[u][0] = d.x; sc[u][1 % V] = d.y; sc[u][2 % V] = d.z; sc[u][3 % V] = d.w;
        } else {
          g[u][0] = gtop[o]; t[u][0] = top[o]; sc[u][0] = scale[o];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = cb + u * CSTEP;
      if (c < C) {
#pragma unroll
        for (int q = 0; q < V; ++q) sr[c * kLrnTP + p + q] = g[u][q] * t[u][q] / sc[u][q];
      }
    }
  }
  __syncthreads();
  if (!live) return;
  for (int c = c0; c < C; c += CSTEP) {
    const int lo = max(c - pre, 0), hi = min(c + post, C - 1);
    const size_t o = base + (size_t)c * HW;
    // this thread's own elements again: they were read a moment ago and come from the cache
    float g[V], sc[V], xv[V], acc[V], r[V];
    if (V == 4) {
      const float4 a = *reinterpret_cast<const float4*>(gtop + o), d = *reinterpret_cast<const float4*>(scale + o),
                   e = *reinterpret_cast<const float4*>(x + o);
      g[0] = a.x; g[1 % V] = a.y; g[2 % V] = a.z; g[3 % V] = a.w;
      sc[0] = d.x; sc[1 % V] = d.y; sc[2 % V] = d.z; sc[3 % V] = d.w;
      xv[0] = e.x; xv[1 % V] = e.y; xv[2 % V] = e.z; xv[3 % V] = e.w;
    } else {
      g[0] = gtop[o]; sc[0] = scale[o]; xv[0] = x[o];
    }
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = 0.f;
    for (int k = lo; k <= hi; ++k) {
#pragma unroll
      for (int q = 0; q < V; ++q) acc[q] += sr[k * kLrnTP + p + q];
    }
#pragma unroll
    for (int q = 0; q < V; ++q) r[q] = g[q] * lrn_pow(sc[q], negative_beta, pmode) - cache_ratio * xv[q] * acc[q];
    if (V == 4) *reinterpret_cast<float4*>(gx + o) = make_float4(r[0], r[1 % V], r[2 % V], r[3 % V]);
    else gx[o] = r[0];
  }
}

static bool lrn_tile_ok(long N, int C) { return N <= 65535 && (size_t)C * kLrnTP * sizeof(float) <= 200 * 1024; }
static bool lrn_vec4(int HW, std::initializer_list<const void*> ptrs) {
  if (HW % 4 != 0) return false;
  for (const void* q : ptrs) if (((uintptr_t)q & 15) != 0) return false;
  return true;
}
template <typename K>
static int lrn_smem_attr(K kernel, size_t smem) {
  if (smem > 48 * 1024) CGTB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  return 0;
}

CGTB_API int cgtb_lrn_forward(int dtype, const void* x, long N, int C, int H, int W, int size, double alpha, double beta,
                              void* top, void* scale) {
  if (!require_runtime("cgtb_lrn_forward")) return 1;
  if (size <= 0) return fail("cgtb_lrn_forward: localsize must be positive");
  long total = N * C * H * W;
  if (total <= 0) return 0;
  if (N > 65535 || C > 65535 || (long)C * H * W >= (1L << 31)) return fail("cgtb_lrn_forward: extents too large");
  const int HW = H * W;
  if (dtype == cgtb_f4 && lrn_tile_ok(N, C)) {
    const size_t smem = (size_t)C * kLrnTP * sizeof(float);
    dim3 tgrid((unsigned)cgtb_ceil_div(HW, kLrnTP), (unsigned)N);
    if (lrn_vec4(HW, {x, top, scale})) {
      if (lrn_smem_attr(lrn_forward_tile_kernel<4>, smem)) return 1;
      CGTB_LAUNCH(lrn_forward_tile_kernel<4>, tgrid, 256, smem, (const float*)x, (float*)top, (float*)scale, C, HW, size,
                  (float)(alpha / size), (float)(-beta), lrn_pow_mode(beta));
    } else {
      if (lrn_smem_attr(lrn_forward_tile_kernel<1>, smem)) return 1;
      CGTB_LAUNCH(lrn_forward_tile_kernel<1>, tgrid, 256, smem, (const float*)x, (float*)top, (float*)scale, C, HW, size,
                  (float)(alpha / size), (float)(-beta), lrn_pow_mode(beta));
    }
    CGTB_CHECK_LAUNCH("lrn_forward");
    return 0;
  }
  const int threads = HW >= 256 ? 256 : (HW >= 128 ? 128 : 64);
  dim3 grid((unsigned)cgtb_ceil_div(HW, threads), (unsigned)C, (unsigned)N);
  if (dtype == cgtb_f4)
    CGTB_LAUNCH(lrn_forward_kernel<float>, grid, threads, 0, (const float*)x, (float*)top, (float*)scale, C, HW, size,
                (float)(alpha / size), (float)(-beta));
  else if (dtype == cgtb_f8)
    CGTB_LAUNCH(lrn_forward_kernel<double>, grid, threads, 0, (const double*)x, (double*)top, (double*)scale, C, HW, size,
                alpha / size, -beta);
  else
    return fail("cgtb_lrn_forward: unsupported dtype %d", dtype);
  CGTB_CHECK_LAUNCH("lrn_forward");
  return 0;
}

CGTB_API int cgtb_lrn_backward(int dtype, const void* x, const void* top, const void* scale, const void* gtop, long N,
                               int C, int H, int W, int size, double alpha, double beta, void* gx) {
  if (!require_runtime("cgtb_lrn_backward")) return 1;
  if (size <= 0) return fail("cgtb_lrn_backward: localsize must be positive");
  long total = N * C * H * W;
  if (total <= 0) return 0;
  if (N > 65535 || C > 65535 || (long)C * H * W >= (1L << 31)) return fail("cgtb_lrn_backward: extents too large");
  const int HW = H * W;
  if (dtype == cgtb_f4 && lrn_tile_ok(N, C)) {
    const size_t smem = (size_t)C * kLrnTP * sizeof(float);
    dim3 tgrid((unsigned)cgtb_ceil_div(HW, kLrnTP), (unsigned)N);
    if (lrn_vec4(HW, {x, top, scale, gtop, gx})) {
      if (lrn_smem_attr(lrn_backward_tile_kernel<4>, smem)) return 1;
      CGTB_LAUNCH(lrn_backward_tile_kernel<4>, tgrid, 256, smem, (const float*)x, (const float*)top, (const float*)scale,
                  (const float*)gtop, (float*)gx, C, HW, size, (float)(-beta), (float)(2. * alpha * beta / size), lrn_pow_mode(beta));
    } else {
      if (lrn_smem_attr(lrn_backward_tile_kernel<1>, smem)) return 1;
      CGTB_LAUNCH(lrn_backward_tile_kernel<1>, tgrid, 256, smem, (const float*)x, (const float*)top, (const float*)scale,
                  (const float*)gtop, (float*)gx, C, HW, size, (float)(-beta), (float)(2. * alpha * beta / size), lrn_pow_mode(beta));
    }
    CGTB_CHECK_LAUNCH("lrn_backward");
    return 0;
  }
  const int threads = HW >= 256 ? 256 : (HW >= 128 ? 128 : 64);
  dim3 grid((unsigned)cgtb_ceil_div(HW, threads), (unsigned)C, (unsigned)N);
  if (dtype == cgtb_f4)
    CGTB_LAUNCH(lrn_backward_kernel<float>, grid, threads, 0, (const float*)x, (const float*)top, (const float*)scale,
                (const float*)gtop, (float*)gx, C, HW, size, (float)(-beta), (float)(2. * alpha * beta / size));
  else if (dtype == cgtb_f8)
    CGTB_LAUNCH(lrn_backward_kernel<double>, grid, threads, 0, (const double*)x, (const double*)top, (const double*)scale,
                (const double*)gtop, (double*)gx, C, HW, size, -beta, 2. * alpha * beta / size);
  else
    return fail("cgtb_lrn_backward: unsupported dtype %d", dtype);
  CGTB_CHECK_LAUNCH("lrn_backward");
  return 0;
}


// ================================================================================================
// Direct convolution of a layer with very few input channels (CIFAR conv1: 3 -> 32 channels, 5 x 5, pad 2, 32 x 32
// images). Through a column matrix this layer costs an im2col that writes 25 times the image, a forward product and
// a filter-gradient product that both stream that matrix again: three HBM-bound passes over 40 MB for 0.63 GFLOP.
// Here a block takes 8 image rows of one image: the input rows with their halo (3 x 12 x 36 floats) live in shared
// memory, the sums in registers. Shared memory hands 128 bytes per clock to the registers of an SM while its FMA
// pipes retire 128 FMAs, so every float read from shared memory has to feed at least 4 FMAs of its thread; both
// kernels are tiled for that.
//   forward: a thread owns one image column x 8 rows x 8 output channels (64 sums); a warp is the 32 columns of one
//     channel group. Per (input channel, filter column) it reads its 12 input values once (conflict-free), then per
//     filter row two 128-bit broadcast reads of 8 weights feed 64 FMAs. The filters sit in shared memory as
//     [tap][channel] with the 4-channel groups XOR-swizzled by the tap, which spreads the transposing fill over
//     8 banks. The epilogue adds the bias and writes relu and mask as NCHW planes (a warp writes 32 consecutive
//     pixels of one plane).
//   filter gradient: a thread owns 2 output channels x the 25 taps of one input channel (50 sums) for one image row
//     of the band; walking along the row it keeps a 5 x 5 window of input values in registers (5 new values per
//     pixel) and reads the pixel's 2 gradients: 7 floats feed 50 FMAs. The 8 rows of the band are added in row order
//     through shared memory, each block leaves its 32 x 75 partial result, and the partial results are added in block
//     order by the split-K fold kernel (reproducible).
// ================================================================================================
namespace {
constexpr int kDcRows = 8;   // image rows per block
constexpr int kDcFwdThreads = 128, kDcWgradThreads = 384;

// Input rows y0-PAD .. y0+kDcRows+PAD of one image with a zero halo, as xs[ci][row][PAD + column]. Every thread issues
// all of its 128-bit loads before it stores any of them, so a block pays one memory latency for the band.
template <int CIN, int KS, int WIDTH, int NT>
__device__ __forceinline__ void conv_direct_load_band(float (*xs)[kDcRows + KS - 1][WIDTH + KS], const float* __restrict__ xb, int H, int y0,
                                                      int tid) {
  constexpr int PAD = KS / 2, HR = kDcRows + KS - 1, Q = WIDTH / 4, NV = CIN * HR * Q, ROUNDS = (NV + NT - 1) / NT;
  float4 v[ROUNDS];
#pragma unroll
  for (int t = 0; t < ROUNDS; ++t) {
    const int e = tid + t * NT, row = e / Q, ci = row / HR, hy = row - ci * HR, gy = y0 + hy - PAD;
    v[t] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e < NV && gy >= 0 && gy < H) v[t] = *reinterpret_cast<const float4*>(xb + ((size_t)ci * H + gy) * WIDTH + 4 * (e % Q));
  }
#pragma unroll
  for (int t = 0; t < ROUNDS; ++t) {
    const int e = tid + t * NT, row = e / Q, ci = row / HR, hy = row - ci * HR;
    if (e < NV) {
      float* d = &xs[ci][hy][PAD + 4 * (e % Q)];
      d[0] = v[t].x; d[1] = v[t].y; d[2] = v[t].z; d[3] = v[t].w;
    }
  }
  for (int e = tid; e < CIN * HR * 2 * PAD; e += NT) {   // halo columns
    const int row = e / (2 * PAD), c = e - row * 2 * PAD;
    xs[row / HR][row % HR][c < PAD ? c : WIDTH + c] = 0.f;
  }
}

template <int CIN, int KS, int COUT, int WIDTH>
__global__ void __launch_bounds__(kDcFwdThreads) conv_direct_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                        const float* __restrict__ bias, int H, float* __restrict__ y,
                                                                        int8_t* __restrict__ mask) {
  constexpr int HR = kDcRows + KS - 1, K = CIN * KS * KS, CG = 8, WP = COUT + 4, WROUNDS = (K * COUT + kDcFwdThreads - 1) / kDcFwdThreads;
  static_assert(WIDTH == 32 && COUT == CG * (kDcFwdThreads / 32), "a warp is the 32 columns of one group of 8 channels");
  __shared__ float xs[CIN][HR][WIDTH + KS];   // row pitch 37 floats: a warp's column reads are conflict-free
  __shared__ __align__(16) float ws[K][WP];   // [tap][channel]; pitch 36 floats spreads the transposing stores over 8 banks
  __shared__ float bs[COUT];
  const int tid = threadIdx.x, cg = tid >> 5, lane = tid & 31;
  const int bands = H / kDcRows, b = blockIdx.x / bands, y0 = (blockIdx.x % bands) * kDcRows;
  {
    float wv[WROUNDS];
#pragma unroll
    for (int t = 0; t < WROUNDS; ++t) {
      const int e = tid + t * kDcFwdThreads;
      wv[t] = e < K * COUT ? w[e] : 0.f;
    }
    conv_direct_load_band<CIN, KS, WIDTH, kDcFwdThreads>(xs, x + (size_t)b * CIN * H * WIDTH, H, y0, tid);
#pragma unroll
    for (int t = 0; t < WROUNDS; ++t) {   // w[oc][k] -> ws[k][oc]
      const int e = tid + t * kDcFwdThreads, oc = e / K, k = e - oc * K;
      if (e < K * COUT) ws[k][oc] = wv[t];
    }
    if (tid < COUT) bs[tid] = bias[tid];
  }
  __syncthreads();
  float acc[kDcRows][CG];
#pragma unroll
  for (int r = 0; r < kDcRows; ++r)
#pragma unroll
    for (int q = 0; q < CG; ++q) acc[r][q] = 0.f;
#pragma unroll 1
  for (int ci = 0; ci < CIN; ++ci) {
    const float* xcol = &xs[ci][0][lane];
    const float* wrow = &ws[ci * KS * KS][cg * CG];
#pragma unroll
    for (int j = 0; j < KS; ++j) {
      float xc[HR];
#pragma unroll
      for (int r = 0; r < HR; ++r) xc[r] = xcol[r * (WIDTH + KS) + j];
#pragma unroll
      for (int i = 0; i < KS; ++i) {
        const float4 wa = *reinterpret_cast<const float4*>(wrow + (i * KS + j) * WP);
        const float4 wb = *reinterpret_cast<const float4*>(wrow + (i * KS + j) * WP + 4);
#pragma unroll
        for (int r = 0; r < kDcRows; ++r) {
          const float xv = xc[r + i];
          acc[r][0] = fmaf(xv, wa.x, acc[r][0]);
          acc[r][1] = fmaf(xv, wa.y, acc[r][1]);
          acc[r][2] = fmaf(xv, wa.z, acc[r][2]);
          acc[r][3] = fmaf(xv, wa.w, acc[r][3]);
          acc[r][4] = fmaf(xv, wb.x, acc[r][4]);
          acc[r][5] = fmaf(xv, wb.y, acc[r][5]);
          acc[r][6] = fmaf(xv, wb.z, acc[r][6]);
          acc[r][7] = fmaf(xv, wb.w, acc[r][7]);
        }
      }
    }
  }
  const size_t plane = (size_t)H * WIDTH;
  float* yo = y + ((size_t)b * COUT + cg * CG) * plane + (size_t)y0 * WIDTH + lane;
  int8_t* mo = mask + ((size_t)b * COUT + cg * CG) * plane + (size_t)y0 * WIDTH + lane;
#pragma unroll
  for (int q = 0; q < CG; ++q) {
    const float bv = bs[cg * CG + q];
#pragma unroll
    for (int r = 0; r < kDcRows; ++r) {
      const float t = acc[r][q] + bv;
      const int8_t m = (int8_t)(t >= 0.f);
      mo[q * plane + r * WIDTH] = m;
      yo[q * plane + r * WIDTH] = t * (float)m;
    }
  }
}

// RELU: the gradient arrives as the NCHW gradient g of the layer's relu output with the relu's NCHW mask; the kernel
// forms dy = mask * g while it stages the band and also leaves the band's bias gradient (the sum of dy over its
// pixels) behind the 32 x 75 partial result.
template <int CIN, int KS, int COUT, int WIDTH, bool RELU>
__global__ void __launch_bounds__(kDcWgradThreads, 2) conv_direct_wgrad_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                                              const int8_t* __restrict__ mask, int H,
                                                                              float* __restrict__ part) {
  constexpr int HR = kDcRows + KS - 1, K = CIN * KS * KS, NPIX = kDcRows * WIDTH, NPAIR = COUT / 2, NQ = NPIX * COUT / 4;
  constexpr int DROUNDS = (NQ + kDcWgradThreads - 1) / kDcWgradThreads, SROUNDS = (NPIX * COUT + kDcWgradThreads - 1) / kDcWgradThreads;
  constexpr int DP = RELU ? COUT + 1 : COUT;   // floats per pixel in dys; the odd pitch keeps the transposing stores conflict-free
  constexpr int PSTRIDE = COUT * K + (RELU ? COUT : 0);
  static_assert(NPAIR * CIN * kDcRows == kDcWgradThreads && kDcRows == 8, "one thread per (channel pair, input channel, band row)");
  static_assert(!RELU || (COUT == 32 && NPIX == 256), "the bias gradient is summed by 8 x 32 threads over 32 pixels each");
  __shared__ float xs[CIN][HR][WIDTH + KS];
  __shared__ float bsum[8][COUT];
  // [NPIX][DP] gradients during the sweep, then up to 4 x [COUT*K] sums of the row tree
  extern __shared__ __align__(16) float dys[];
  const int tid = threadIdx.x;
  const int bands = H / kDcRows, b = blockIdx.x / bands, y0 = (blockIdx.x % bands) * kDcRows;
  if constexpr (RELU) {
    // channel c's 256 values of the band are contiguous in its NCHW plane
    const size_t base = (size_t)b * COUT * H * WIDTH + (size_t)y0 * WIDTH;
    const float* gsrc = dy + base;
    const int8_t* msrc = mask + base;
    float gv[SROUNDS];
    int8_t mv[SROUNDS];
#pragma unroll
    for (int t = 0; t < SROUNDS; ++t) {
      const int e = tid + t * kDcWgradThreads, c = e / NPIX, px = e - c * NPIX;
      const bool ok = e < NPIX * COUT;
      gv[t] = ok ? gsrc[(size_t)c * H * WIDTH + px] : 0.f;
      mv[t] = ok ? msrc[(size_t)c * H * WIDTH + px] : (int8_t)0;
    }
    conv_direct_load_band<CIN, KS, WIDTH, kDcWgradThreads>(xs, x + (size_t)b * CIN * H * WIDTH, H, y0, tid);
#pragma unroll
    for (int t = 0; t < SROUNDS; ++t) {
      const int e = tid + t * kDcWgradThreads, c = e / NPIX, px = e - c * NPIX;
      if (e < NPIX * COUT) dys[px * DP + c] = gv[t] * (float)mv[t];
    }
    __syncthreads();
    if (tid < 8 * COUT) {   // bias gradient: 8 segments of 32 pixels per channel, added in segment order below
      const int c = tid % COUT, seg = tid / COUT;
      float sum = 0.f;
#pragma unroll 8
      for (int q = 0; q < NPIX / 8; ++q) sum += dys[(seg * (NPIX / 8) + q) * DP + c];
      bsum[seg][c] = sum;
    }
  } else {
    const float4* dsrc = reinterpret_cast<const float4*>(dy + ((size_t)b * H + y0) * WIDTH * COUT);   // NPIX * COUT contiguous floats
    float4 dv[DROUNDS];
#pragma unroll
    for (int t = 0; t < DROUNDS; ++t) {
      const int e = tid + t * kDcWgradThreads;
      dv[t] = e < NQ ? dsrc[e] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    conv_direct_load_band<CIN, KS, WIDTH, kDcWgradThreads>(xs, x + (size_t)b * CIN * H * WIDTH, H, y0, tid);
#pragma unroll
    for (int t = 0; t < DROUNDS; ++t) {
      const int e = tid + t * kDcWgradThreads;
      if (e < NQ) reinterpret_cast<float4*>(dys)[e] = dv[t];
    }
  }
  __syncthreads();
  const int pair = tid % NPAIR, rest = tid / NPAIR, ci = rest % CIN, row = rest / CIN;
  float acc[2][KS][KS];
#pragma unroll
  for (int i = 0; i < KS; ++i)
#pragma unroll
    for (int j = 0; j < KS; ++j) acc[0][i][j] = acc[1][i][j] = 0.f;
  float xw[KS][KS];   // xw[i][c % KS] = xs[ci][row + i][c] for the KS columns under the current pixel
  const float* xrow = &xs[ci][row][0];
#pragma unroll
  for (int i = 0; i < KS; ++i)
#pragma unroll
    for (int c = 0; c < KS - 1; ++c) xw[i][c] = xrow[i * (WIDTH + KS) + c];
  const float* drow = dys + (size_t)row * WIDTH * DP + 2 * pair;
#pragma unroll
  for (int pc = 0; pc < WIDTH; ++pc) {
#pragma unroll
    for (int i = 0; i < KS; ++i) xw[i][(pc + KS - 1) % KS] = xrow[i * (WIDTH + KS) + pc + KS - 1];
    float2 d;
    if constexpr (RELU) d = make_float2(drow[pc * DP], drow[pc * DP + 1]);
    else d = *reinterpret_cast<const float2*>(drow + pc * DP);
#pragma unroll
    for (int i = 0; i < KS; ++i)
#pragma unroll
      for (int j = 0; j < KS; ++j) {
        const float xv = xw[i][(pc + j) % KS];
        acc[0][i][j] = fmaf(d.x, xv, acc[0][i][j]);
        acc[1][i][j] = fmaf(d.y, xv, acc[1][i][j]);
      }
  }
  __syncthreads();   // every thread is done with the gradients: their space now holds the tree's sums
  // rows are added as ((r0+r4) + (r2+r6)) + ((r1+r5) + (r3+r7)): the upper half of the live rows hands its sums over
  const int col0 = (2 * pair) * K + ci * KS * KS;
#pragma unroll
  for (int half = kDcRows / 2; half >= 1; half /= 2) {
    if (row >= half && row < 2 * half) {
      float* dst = dys + (size_t)(row - half) * COUT * K + col0;
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int t = 0; t < KS * KS; ++t) dst[a * K + t] = acc[a][t / KS][t % KS];
    }
    __syncthreads();
    if (row < half) {
      const float* src = dys + (size_t)row * COUT * K + col0;
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int t = 0; t < KS * KS; ++t) acc[a][t / KS][t % KS] += src[a * K + t];
    }
    __syncthreads();
  }
  if (row == 0) {
    float* dst = dys + col0;
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int t = 0; t < KS * KS; ++t) dst[a * K + t] = acc[a][t / KS][t % KS];
  }
  __syncthreads();
  float* dst = part + (size_t)blockIdx.x * PSTRIDE;
  for (int e = tid; e < COUT * K; e += kDcWgradThreads) dst[e] = dys[e];
  if constexpr (RELU) {
    if (tid < COUT)
      dst[COUT * K + tid] = ((bsum[0][tid] + bsum[1][tid]) + (bsum[2][tid] + bsum[3][tid])) +
                            ((bsum[4][tid] + bsum[5][tid]) + (bsum[6][tid] + bsum[7][tid]));
  }
}

// Ordered sum of the blocks' partial results [nsplit][n0 + n1] into out0[n0] and out1[n1]: thread group g adds splits
// g, g+8, ... in order and the eight sums are combined as a fixed tree (the arithmetic of the split-K fold).
__global__ void __launch_bounds__(256) conv_direct_fold_kernel(const float* __restrict__ part, int nsplit, int n0, int n1,
                                                               float* __restrict__ out0, float* __restrict__ out1) {
  __shared__ float sums[8][33];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5, total = n0 + n1;
  const int e = blockIdx.x * 32 + lane;
  float acc = 0.f;
  if (e < total)
    for (int s2 = g; s2 < nsplit; s2 += 8) acc += part[(size_t)s2 * total + e];
  sums[g][lane] = acc;
  __syncthreads();
  if (g == 0 && e < total) {
    const float r = ((sums[0][lane] + sums[1][lane]) + (sums[2][lane] + sums[3][lane])) +
                    ((sums[4][lane] + sums[5][lane]) + (sums[6][lane] + sums[7][lane]));
    if (e < n0) out0[e] = r;
    else out1[e - n0] = r;
  }
}
bool conv_direct_ok(long B, int Cin, int H, int W, int Cout, int kh, int kw, int ph, int pw) {
  return Cin == 3 && kh == 5 && kw == 5 && ph == 2 && pw == 2 && Cout == 32 && W == 32 && H % kDcRows == 0 && H > 0 && B > 0 &&
         B * (H / kDcRows) < (1L << 30);
}
}  // namespace

namespace cgtb {
void tc_splitk_fold(long P, long M, long N, int nsplit, const float* part, float* C, long ldc, long strideC);
}

CGTB_API int cgtb_conv_direct_fwd_bias_relu(const float* x, long B, int Cin, int H, int W, const float* w, int Cout, int kh, int kw, int ph,
                                            int pw, const float* bias, float* y, signed char* mask) {
  if (!require_runtime("cgtb_conv_direct_fwd_bias_relu")) return 1;
  if (B <= 0) return 0;
  if (!conv_direct_ok(B, Cin, H, W, Cout, kh, kw, ph, pw) || ((uintptr_t)x & 15) != 0)   // the image rows are read as 128-bit words
    return fail("cgtb_conv_direct_fwd_bias_relu: not supported for Cin=%d kh=%d kw=%d pad=%d,%d Cout=%d H=%d W=%d (3, 5, 5, 2, 2, 32, multiple of 8, 32) "
                "or an image that does not start on a 16-byte boundary", Cin, kh, kw, ph, pw, Cout, H, W);
  const unsigned blocks = (unsigned)(B * (H / kDcRows));
  CGTB_LAUNCH((conv_direct_fwd_kernel<3, 5, 32, 32>), blocks, kDcFwdThreads, 0, x, w, bias, H, y, (int8_t*)mask);
  CGTB_CHECK_LAUNCH("conv_direct_fwd");
  return 0;
}
static int conv_direct_wgrad_any(const char* who, const float* x, long B, int Cin, int H, int W, const float* dy, const signed char* mask,
                                 int Cout, int kh, int kw, int ph, int pw, float* dw, float* dbias) {
  if (!require_runtime(who)) return 1;
  if (B <= 0) return 0;
  const bool relu = mask != nullptr;
  if (!conv_direct_ok(B, Cin, H, W, Cout, kh, kw, ph, pw) || ((uintptr_t)dy & 15) != 0 || ((uintptr_t)x & 15) != 0)
    return fail("%s: not supported for Cin=%d kh=%d kw=%d pad=%d,%d Cout=%d H=%d W=%d (3, 5, 5, 2, 2, 32, multiple of 8, 32) or an unaligned operand",
                who, Cin, kh, kw, ph, pw, Cout, H, W);
  const long blocks = B * (H / kDcRows);
  const int K = Cin * kh * kw, pstride = Cout * K + (relu ? Cout : 0);
  float* part = (float*)scratch((size_t)blocks * pstride * sizeof(float));
  if (!part) return 1;
  const size_t smem = std::max<size_t>((size_t)kDcRows * 32 * 33, (size_t)(kDcRows / 2) * Cout * K) * sizeof(float);
  static bool attr = false;
  if (!attr) {
    CGTB_CUDA_TRY(cudaFuncSetAttribute(conv_direct_wgrad_kernel<3, 5, 32, 32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CGTB_CUDA_TRY(cudaFuncSetAttribute(conv_direct_wgrad_kernel<3, 5, 32, 32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr = true;
  }
  if (relu) {
    CGTB_LAUNCH((conv_direct_wgrad_kernel<3, 5, 32, 32, true>), (unsigned)blocks, kDcWgradThreads, smem, x, dy, (const int8_t*)mask, H, part);
    CGTB_LAUNCH(conv_direct_fold_kernel, (unsigned)cgtb_ceil_div(pstride, 32), 256, 0, part, (int)blocks, Cout * K, Cout, dw, dbias);
  } else {
    CGTB_LAUNCH((conv_direct_wgrad_kernel<3, 5, 32, 32, false>), (unsigned)blocks, kDcWgradThreads, smem, x, dy, (const int8_t*)nullptr, H, part);
    if (blocks > 1) cgtb::tc_splitk_fold(1, Cout, K, (int)blocks, part, dw, K, 0);
    else CGTB_CUDA_TRY(cudaMemcpyAsync(dw, part, (size_t)Cout * K * sizeof(float), cudaMemcpyDeviceToDevice, rt().stream));
  }
  CGTB_CHECK_LAUNCH(who);
  return 0;
}
CGTB_API int cgtb_conv_direct_wgrad(const float* x, long B, int Cin, int H, int W, const float* dy, int Cout, int kh, int kw, int ph, int pw,
                                    float* dw) {
  return conv_direct_wgrad_any("cgtb_conv_direct_wgrad", x, B, Cin, H, W, dy, nullptr, Cout, kh, kw, ph, pw, dw, nullptr);
}
CGTB_API int cgtb_conv_direct_wgrad_relu(const float* x, long B, int Cin, int H, int W, const signed char* mask, const float* g, int Cout,
                                         int kh, int kw, int ph, int pw, float* dw, float* dbias) {
  if (!mask || !dbias) return fail("cgtb_conv_direct_wgrad_relu: mask and dbias are required");
  return conv_direct_wgrad_any("cgtb_conv_direct_wgrad_relu", x, B, Cin, H, W, g, mask, Cout, kh, kw, ph, pw, dw, dbias);
}
