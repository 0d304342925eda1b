// Gradient all-reduce over peer memory for small payloads: one kernel per call, no library collective.
//
// Why: the CIFAR-shape convnet's gradients are 0.33 MB. Through NCCL that exchange is latency-bound and, being a
// library call that may not be stream-captured here, it cuts the step's CUDA graph in two. This kernel is an
// ordinary launch on the runtime stream: it can be captured with the rest of the step (one graph launch per
// step at every number of GPUs) and it does pack, exchange, sum and unpack in one go.
//
// Every rank owns one "symmetric" device buffer (cudaMalloc'd on its own GPU, exported with cudaIpcGetMemHandle
// and mapped by the other ranks' processes with cudaIpcOpenMemHandle; the host side carries the 64-byte handles):
//   [ header: epoch, block counters | flags of the data slots | flags of the result slots | data slot 0 | data slot 1 |
//     result slot 0 | result slot 1 ]
// One call = one epoch e, using data slot e % 2:
//   1. the blocks copy this rank's tensors into its own slot (packed); the last block to finish publishes
//      flag[slot] = e with a system-scope release;
//   2. every block waits, with a cycle budget, until the flag of every rank's slot reads e (system-scope acquire
//      loads from peer memory over NVLink);
//   3. every block sums its share of the elements over the ranks' slots IN RANK ORDER (plain peer loads) and
//      writes the sums to the result tensors: all ranks add in the same order, so replicas stay bit-identical;
//   4. the last block to finish advances the epoch.
// Two slots are enough: a rank can begin epoch e + 2 (which overwrites slot e % 2) only after it has seen every
// rank's flag of epoch e + 1, i.e. after every rank has finished its kernel of epoch e.
// Payloads beyond a megabyte take the two-phase kernel instead (every rank would otherwise read every other rank's whole
// payload: world times the bytes over NVLink): after the flags of step 2 rank r sums only slice r of the elements over
// all ranks' data slots, in rank order, into its own RESULT slot and publishes a second flag; after every rank's second
// flag has been seen, every rank copies all slices from their owners' result slots into its result tensors. Each
// element crosses NVLink twice whatever the number of ranks, is summed once, in one order, by one rank: replicas stay
// bit-identical. The result slots alternate like the data slots and are safe for the same reason.
// A wait that runs out of budget raises the host-mapped error flag (code 8), the kernel skips the sum, still
// advances its epoch and returns: the context stays usable and the host reports the failure at the next
// synchronisation. Nothing here uses multicast or TMA on peer memory: plain loads and stores only.
#include "runtime.h"
#include "tc_util.h"

#include <algorithm>
#include <cstring>

using namespace cgtb;

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxTensors = 32;
constexpr size_t kHeaderBytes = 1024;   // header + the two flags, each on its own 128-byte line

struct Header {
  unsigned long long epoch;     // last completed epoch of this rank
  unsigned int packed_blocks;   // blocks that have finished packing in the running call
  unsigned int done_blocks;     // blocks that have finished the running call
  unsigned int reduced_blocks;  // two-phase kernel: blocks that have written their part of this rank's slice
  unsigned int pad_;
  // block 0's nanosecond stamps of the last call (%globaltimer): start, after the wait for the peers, end; and sums
  unsigned long long t_start, t_waited, t_end, sum_wait_ns, sum_total_ns, calls;
};

struct PeerTable {
  char* base[kMaxRanks];   // every rank's symmetric buffer as mapped in this process (base[rank] = the local one)
};
struct TensorTable {
  const float* src[kMaxTensors];
  float* dst[kMaxTensors];
  long off[kMaxTensors + 1];   // tensor t starts at element off[t] of the packed payload (a multiple of four)
  long cnt[kMaxTensors];       // and has cnt[t] elements; off[t+1] - off[t] is cnt[t] rounded up to four
  int n;
};

struct State {
  int rank = 0, world = 1;
  char* local = nullptr;
  bool local_owned = false;
  char* mapped[kMaxRanks] = {nullptr};
  bool opened[kMaxRanks] = {false};
  size_t slot_bytes = 0;
  long long wait_cycles = 2000000000LL;
  size_t two_phase_bytes = 1u << 20;   // payloads beyond this take the two-phase kernel
  char* fake_peer = nullptr;   // self-test: a second buffer in this process that stands for a rank that never arrives
  unsigned long long fake_epoch = 0;
} g;

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned long long* flag_of(char* base, int slot) {
  return reinterpret_cast<unsigned long long*>(base + 256 + 128 * slot);
}
__device__ __forceinline__ float* slot_of(char* base, int slot, size_t slot_bytes) {
  return reinterpret_cast<float*>(base + kHeaderBytes + (size_t)slot * slot_bytes);
}
__device__ __forceinline__ unsigned long long* flag2_of(char* base, int slot) {
  return reinterpret_cast<unsigned long long*>(base + 512 + 128 * slot);
}
__device__ __forceinline__ float* result_of(char* base, int slot, size_t slot_bytes) {
  return reinterpret_cast<float*>(base + kHeaderBytes + (size_t)(2 + slot) * slot_bytes);
}
// bounded wait of threads 0..world-1 for every rank's flag (at `which`: 0 data, 1 result) to reach `epoch`
__device__ __forceinline__ bool wait_flags(const PeerTable& pt, int world, int slot, int which, unsigned long long epoch, long long wait_cycles) {
  bool ok = true;
  if ((int)threadIdx.x < world) {
    const unsigned long long* f = which ? flag2_of(pt.base[threadIdx.x], slot) : flag_of(pt.base[threadIdx.x], slot);
    const long long t0 = clock64();
    ok = false;
    for (unsigned int spin = 0; spin < (1u << 30); ++spin) {
      if (ld_acquire_sys(f) == epoch) { ok = true; break; }
      if ((spin & 63u) == 63u && clock64() - t0 > wait_cycles) break;
    }
  }
  return ok;
}

__global__ void __launch_bounds__(256) peer_allreduce_kernel(const TensorTable tt, const PeerTable pt, int rank, int world, size_t slot_bytes,
                                                           long long wait_cycles, int* err) {
  __shared__ int failed;
  Header* hdr = reinterpret_cast<Header*>(pt.base[rank]);
  const unsigned long long epoch = hdr->epoch + 1;   // stable during the call: only the call's last block writes it, at the end
  const int slot = (int)(epoch & 1ull);
  const long total = tt.off[tt.n];
  if (threadIdx.x == 0) failed = 0;
  const bool stamps = blockIdx.x == 0 && threadIdx.x == 0;
  unsigned long long t_start = 0, t_waited = 0;
  if (stamps) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
  // 1. pack this rank's tensors into its own slot. Every tensor starts on a 16-byte boundary of the slot (off[] are
  // multiples of four elements), so a group of four elements never straddles two tensors.
  float* mine = slot_of(pt.base[rank], slot, slot_bytes);
  const long ngroups = total >> 2;   // total is a multiple of four as well
  for (long q = (long)blockIdx.x * blockDim.x + threadIdx.x; q < ngroups; q += (long)gridDim.x * blockDim.x) {
    const long i = q << 2;
    int t = 0;
    while (t + 1 < tt.n && i >= tt.off[t + 1]) ++t;
    const long j = i - tt.off[t], cnt = tt.cnt[t];
    const float* src = tt.src[t] + j;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j + 4 <= cnt && (((uintptr_t)src) & 15) == 0) {
      v = *reinterpret_cast<const float4*>(src);
    } else {
      if (j < cnt) v.x = src[0];
      if (j + 1 < cnt) v.y = src[1];
      if (j + 2 < cnt) v.z = src[2];
      if (j + 3 < cnt) v.w = src[3];
    }
    *reinterpret_cast<float4*>(mine + i) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&hdr->packed_blocks, 1u);
    if (prev == gridDim.x - 1) {
      hdr->packed_blocks = 0;
      st_release_sys(flag_of(pt.base[rank], slot), epoch);   // every block's slot writes happen-before this store
    }
  }
  // 2. wait (bounded) for every rank's flag of this epoch
  if ((int)threadIdx.x < world) {
    const unsigned long long* f = flag_of(pt.base[threadIdx.x], slot);
    const long long t0 = clock64();
    bool ok = false;
    for (unsigned int spin = 0; spin < (1u << 30); ++spin) {
      if (ld_acquire_sys(f) == epoch) { ok = true; break; }
      if ((spin & 63u) == 63u && clock64() - t0 > wait_cycles) break;
    }
    if (!ok) failed = 1;
  }
  __syncthreads();
  if (stamps) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_waited));
  if (failed) {
    if (threadIdx.x == 0 && blockIdx.x == 0) { *(volatile int*)err = 8; __threadfence_system(); }
  } else {
    // 3. sum over the ranks' slots in rank order, straight into the result tensors: four elements per thread, the
    // loads of all ranks in flight before the first addition
    for (long q = (long)blockIdx.x * blockDim.x + threadIdx.x; q < ngroups; q += (long)gridDim.x * blockDim.x) {
      const long i = q << 2;
      float4 v[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < world)   // cache-global loads: a line of a peer's slot must not be served from this SM's L1
          v[r] = __ldcg(reinterpret_cast<const float4*>(slot_of(pt.base[r], slot, slot_bytes) + i));
      float4 acc = v[0];
#pragma unroll
      for (int r = 1; r < kMaxRanks; ++r)
        if (r < world) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
      int t = 0;
      while (t + 1 < tt.n && i >= tt.off[t + 1]) ++t;
      const long j = i - tt.off[t], cnt = tt.cnt[t];
      float* dst = tt.dst[t] + j;
      if (j + 4 <= cnt && (((uintptr_t)dst) & 15) == 0) {
        *reinterpret_cast<float4*>(dst) = acc;
      } else {
        if (j < cnt) dst[0] = acc.x;
        if (j + 1 < cnt) dst[1] = acc.y;
        if (j + 2 < cnt) dst[2] = acc.z;
        if (j + 3 < cnt) dst[3] = acc.w;
      }
    }
  }
  // 4. the last block advances the epoch
  __syncthreads();
  if (stamps) {
    unsigned long long t_end;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_end));
    hdr->t_start = t_start;
    hdr->t_waited = t_waited;
    hdr->t_end = t_end;
    hdr->sum_wait_ns += t_waited - t_start;   // packing included: it is a few hundred nanoseconds
    hdr->sum_total_ns += t_end - t_start;
    hdr->calls += 1;
  }
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(&hdr->done_blocks, 1u);
    if (prev == gridDim.x - 1) {
      hdr->done_blocks = 0;
      hdr->epoch = epoch;
    }
  }
}

// Two-phase variant for large payloads (see the head of this file).
__global__ void __launch_bounds__(256) peer_allreduce2_kernel(const TensorTable tt, const PeerTable pt, int rank, int world, size_t slot_bytes,
                                                            long long wait_cycles, int* err) {
  __shared__ int failed;
  Header* hdr = reinterpret_cast<Header*>(pt.base[rank]);
  const unsigned long long epoch = hdr->epoch + 1;
  const int slot = (int)(epoch & 1ull);
  const long total = tt.off[tt.n], ngroups = total >> 2;
  const long stride = (long)gridDim.x * blockDim.x, q0 = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (threadIdx.x == 0) failed = 0;
  const bool stamps = blockIdx.x == 0 && threadIdx.x == 0;
  unsigned long long t_start = 0, t_waited = 0;
  if (stamps) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
  // 1. pack (as in the one-phase kernel)
  float* mine = slot_of(pt.base[rank], slot, slot_bytes);
  for (long q = q0; q < ngroups; q += stride) {
    const long i = q << 2;
    int t = 0;
    while (t + 1 < tt.n && i >= tt.off[t + 1]) ++t;
    const long j = i - tt.off[t], cnt = tt.cnt[t];
    const float* src = tt.src[t] + j;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j + 4 <= cnt && (((uintptr_t)src) & 15) == 0) {
      v = *reinterpret_cast<const float4*>(src);
    } else {
      if (j < cnt) v.x = src[0];
      if (j + 1 < cnt) v.y = src[1];
      if (j + 2 < cnt) v.z = src[2];
      if (j + 3 < cnt) v.w = src[3];
    }
    *reinterpret_cast<float4*>(mine + i) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&hdr->packed_blocks, 1u);
    if (prev == gridDim.x - 1) {
      hdr->packed_blocks = 0;
      st_release_sys(flag_of(pt.base[rank], slot), epoch);
    }
  }
  // 2. every rank's data
  if (!wait_flags(pt, world, slot, 0, epoch, wait_cycles)) failed = 1;
  __syncthreads();
  if (stamps) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_waited));
  const bool bad1 = failed != 0;
  // 3. this rank's slice of the groups, summed over the ranks in rank order, into this rank's result slot
  const long per = (ngroups + world - 1) / world, g0 = (long)rank * per, g1 = g0 + per < ngroups ? g0 + per : ngroups;
  float* res = result_of(pt.base[rank], slot, slot_bytes);
  if (!bad1) {
    // two groups per iteration, the loads of all ranks for both in flight before the first addition
    for (long q = g0 + q0; q < g1; q += 2 * stride) {
      const long i0 = q << 2, i1 = (q + stride) << 2;
      const bool two = q + stride < g1;
      float4 v[kMaxRanks], w[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < world) {
          const float* base = slot_of(pt.base[r], slot, slot_bytes);
          v[r] = __ldcg(reinterpret_cast<const float4*>(base + i0));
          if (two) w[r] = __ldcg(reinterpret_cast<const float4*>(base + i1));
        }
      float4 acc = v[0], bcc = w[0];
#pragma unroll
      for (int r = 1; r < kMaxRanks; ++r)
        if (r < world) {
          acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
          if (two) { bcc.x += w[r].x; bcc.y += w[r].y; bcc.z += w[r].z; bcc.w += w[r].w; }
        }
      *reinterpret_cast<float4*>(res + i0) = acc;
      if (two) *reinterpret_cast<float4*>(res + i1) = bcc;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&hdr->reduced_blocks, 1u);
    if (prev == gridDim.x - 1) {
      hdr->reduced_blocks = 0;
      // a rank whose first wait failed publishes nothing: the others' second wait runs out as well
      if (!bad1) st_release_sys(flag2_of(pt.base[rank], slot), epoch);
    }
  }
  // 4. every rank's slice
  if (!bad1 && !wait_flags(pt, world, slot, 1, epoch, wait_cycles)) failed = 1;
  __syncthreads();
  if (failed) {
    if (threadIdx.x == 0 && blockIdx.x == 0) { *(volatile int*)err = 8; __threadfence_system(); }
  } else {
    // 5. all slices from their owners' result slots into the result tensors
    for (long qq = q0; qq < ngroups; qq += 4 * stride) {
     float4 got[4];
#pragma unroll
     for (int u = 0; u < 4; ++u) {   // four loads in flight
       const long q = qq + u * stride;
       if (q < ngroups) got[u] = __ldcg(reinterpret_cast<const float4*>(result_of(pt.base[(int)(q / per)], slot, slot_bytes) + (q << 2)));
     }
#pragma unroll
     for (int u = 0; u < 4; ++u) {
      const long q = qq + u * stride;
      if (q >= ngroups) break;
      const long i = q << 2;
      const float4 acc = got[u];
      int t = 0;
      while (t + 1 < tt.n && i >= tt.off[t + 1]) ++t;
      const long j = i - tt.off[t], cnt = tt.cnt[t];
      float* dst = tt.dst[t] + j;
      if (j + 4 <= cnt && (((uintptr_t)dst) & 15) == 0) {
        *reinterpret_cast<float4*>(dst) = acc;
      } else {
        if (j < cnt) dst[0] = acc.x;
        if (j + 1 < cnt) dst[1] = acc.y;
        if (j + 2 < cnt) dst[2] = acc.z;
        if (j + 3 < cnt) dst[3] = acc.w;
      }
     }
    }
  }
  // 6. the last block advances the epoch
  __syncthreads();
  if (stamps) {
    unsigned long long t_end;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_end));
    hdr->t_start = t_start;
    hdr->t_waited = t_waited;
    hdr->t_end = t_end;
    hdr->sum_wait_ns += t_waited - t_start;
    hdr->sum_total_ns += t_end - t_start;
    hdr->calls += 1;
  }
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(&hdr->done_blocks, 1u);
    if (prev == gridDim.x - 1) {
      hdr->done_blocks = 0;
      hdr->epoch = epoch;
    }
  }
}

int alloc_buffer(size_t slot_bytes, char** out) {
  char* p = nullptr;
  const size_t bytes = kHeaderBytes + 4 * slot_bytes;   // two data slots, two result slots
  CGTB_CUDA_TRY(cudaMalloc((void**)&p, bytes));
  CGTB_CUDA_TRY(cudaMemset(p, 0, bytes));
  *out = p;
  return 0;
}

}  // namespace

namespace cgtb {
// true when the peer-memory all-reduce can take a payload of `bytes`
bool peer_ready(size_t bytes) { return g.local && g.world > 1 && bytes + 16 * kMaxTensors <= g.slot_bytes; }  // padding to 16 bytes per tensor

int peer_allreduce(int n, const void* const* in, void* const* out, const long* counts) {
  TensorTable tt;
  tt.n = n;
  tt.off[0] = 0;
  for (int i = 0; i < n; ++i) {
    tt.src[i] = (const float*)in[i];
    tt.dst[i] = (float*)out[i];
    tt.cnt[i] = counts[i] > 0 ? counts[i] : 0;
    tt.off[i + 1] = tt.off[i] + ((tt.cnt[i] + 3) & ~3L);
  }
  if ((size_t)tt.off[n] * sizeof(float) > g.slot_bytes) return fail("peer all-reduce: %ld bytes (tensors padded to 16 bytes) exceed the slot", tt.off[n] * 4);
  const long total = tt.off[n];
  if (total == 0) return 0;
  PeerTable pt;
  for (int r = 0; r < kMaxRanks; ++r) pt.base[r] = r < g.world ? g.mapped[r] : nullptr;
  int* err = tc_error_flag();
  if (!err) return 1;
  if ((size_t)total * sizeof(float) > g.two_phase_bytes) {
    // every block polls the flags and must be resident together with the others: no more blocks than fit at once
    static int per_sm = 0;
    if (per_sm == 0) {
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, peer_allreduce2_kernel, 256, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    }
    const unsigned blocks = (unsigned)std::max<long>(1, std::min<long>(cgtb_ceil_div(total, 2048), (long)per_sm * rt().sm_count));
    CGTB_LAUNCH(peer_allreduce2_kernel, blocks, 256, 0, tt, pt, g.rank, g.world, g.slot_bytes, g.wait_cycles, err);
    CGTB_CHECK_LAUNCH("peer_allreduce");
    return 0;
  }
  // few blocks: the payload is small and every block polls every rank's flag
  const unsigned blocks = (unsigned)std::max<long>(1, std::min<long>(cgtb_ceil_div(total, 1024), 128));  // one group of four per thread
  CGTB_LAUNCH(peer_allreduce_kernel, blocks, 256, 0, tt, pt, g.rank, g.world, g.slot_bytes, g.wait_cycles, err);
  CGTB_CHECK_LAUNCH("peer_allreduce");
  return 0;
}
}  // namespace cgtb

// Block 0's timing of the calls so far: out[0] calls, out[1] nanoseconds from kernel start until every rank's flag was
// seen (packing and the wait for slower ranks), out[2] nanoseconds from start to end, both summed over the calls.
CGTB_API int cgtb_peer_timing(long* out3) {
  if (!g.local) return fail("cgtb_peer_timing: no symmetric buffer");
  Header h;
  CGTB_CUDA_TRY(cudaStreamSynchronize(rt().stream));
  CGTB_CUDA_TRY(cudaMemcpy(&h, g.local, sizeof(h), cudaMemcpyDeviceToHost));
  out3[0] = (long)h.calls;
  out3[1] = (long)h.sum_wait_ns;
  out3[2] = (long)h.sum_total_ns;
  return 0;
}

// Payloads of more than `bytes` take the two-phase kernel (default one megabyte; 0: always).
CGTB_API int cgtb_peer_set_two_phase_bytes(long bytes) {
  if (bytes < 0) return fail("cgtb_peer_set_two_phase_bytes: negative size");
  g.two_phase_bytes = (size_t)bytes;
  return 0;
}

// Allocate this rank's symmetric buffer (two data and two result slots of slot_bytes) and return its 64-byte IPC handle.
CGTB_API int cgtb_peer_alloc(long slot_bytes, char* handle64) {
  if (!require_runtime("cgtb_peer_alloc")) return 1;
  if (g.local) return fail("cgtb_peer_alloc: the symmetric buffer already exists");
  if (slot_bytes <= 0 || slot_bytes > (64L << 20)) return fail("cgtb_peer_alloc: slot size %ld out of range", slot_bytes);
  const size_t sb = ((size_t)slot_bytes + 255) & ~(size_t)255;
  if (alloc_buffer(sb, &g.local)) return 1;
  g.local_owned = true;
  g.slot_bytes = sb;
  cudaIpcMemHandle_t h;
  CGTB_CUDA_TRY(cudaIpcGetMemHandle(&h, g.local));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
// Map the other ranks' buffers: handles = world * 64 bytes in rank order (this rank's own entry is ignored).
CGTB_API int cgtb_peer_open(const char* handles, int rank, int world) {
  if (!require_runtime("cgtb_peer_open")) return 1;
  if (!g.local) return fail("cgtb_peer_open: call cgtb_peer_alloc first");
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return fail("cgtb_peer_open: rank %d of %d not supported (at most %d)", rank, world, kMaxRanks);
  for (int r = 0; r < world; ++r) {
    if (r == rank) { g.mapped[r] = g.local; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + 64 * r, 64);
    void* p = nullptr;
    CGTB_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    g.mapped[r] = (char*)p;
    g.opened[r] = true;
  }
  g.rank = rank;
  g.world = world;
  return 0;
}
CGTB_API int cgtb_peer_close(void) {
  if (rt().ready) cudaStreamSynchronize(rt().stream);
  for (int r = 0; r < kMaxRanks; ++r) {
    if (g.opened[r]) cudaIpcCloseMemHandle(g.mapped[r]);
    g.opened[r] = false;
    g.mapped[r] = nullptr;
  }
  if (g.fake_peer) { cudaFree(g.fake_peer); g.fake_peer = nullptr; }
  if (g.local && g.local_owned) cudaFree(g.local);
  g.local = nullptr;
  g.world = 1;
  g.rank = 0;
  g.slot_bytes = 0;
  return 0;
}
CGTB_API int cgtb_peer_world(void) { return g.local ? g.world : 1; }
CGTB_API long cgtb_peer_slot_bytes(void) { return (long)g.slot_bytes; }
// cycle budget of the kernel's flag waits (default about one second of SM clock)
CGTB_API int cgtb_peer_set_wait_cycles(long cycles) {
  if (cycles <= 0) return fail("cgtb_peer_set_wait_cycles: must be positive");
  g.wait_cycles = cycles;
  return 0;
}
// out[i] = sum over ranks of in[i] for n float32 buffers through the peer-memory kernel
CGTB_API int cgtb_peer_allreduce_sum(int n, const void* const* in, void* const* out, const long* counts) {
  if (!require_runtime("cgtb_peer_allreduce_sum")) return 1;
  if (!g.local || g.world < 2) return fail("cgtb_peer_allreduce_sum: no peer group (cgtb_peer_alloc / cgtb_peer_open)");
  if (n < 1 || n > kMaxTensors) return fail("cgtb_peer_allreduce_sum: between 1 and %d tensors", kMaxTensors);
  long total = 0;   // in the slot every tensor starts on a 16-byte boundary
  for (int i = 0; i < n; ++i) total += ((counts[i] > 0 ? counts[i] : 0) + 3) & ~3L;
  if ((size_t)total * 4 > g.slot_bytes) return fail("cgtb_peer_allreduce_sum: %ld bytes exceed the slot of %ld bytes", total * 4, (long)g.slot_bytes);
  return cgtb::peer_allreduce(n, in, out, counts);
}

// Self-test on ONE GPU: a group of two "ranks" in this process, rank 0 real, rank 1 a second buffer that nobody
// drives. A call then waits for a flag that is never set: the bounded wait must expire, the error must be reported and
// the library must stay usable. cgtb_peer_selftest_post() plays the missing rank for the NEXT call: it writes that rank's
// payload and flag from the host, so that call completes with the sum.
CGTB_API int cgtb_peer_selftest_open(long slot_bytes) {
  if (!require_runtime("cgtb_peer_selftest_open")) return 1;
  if (g.local) return fail("cgtb_peer_selftest_open: a peer group already exists");
  const size_t sb = ((size_t)slot_bytes + 255) & ~(size_t)255;
  if (alloc_buffer(sb, &g.local)) return 1;
  if (alloc_buffer(sb, &g.fake_peer)) return 1;
  g.local_owned = true;
  g.slot_bytes = sb;
  g.rank = 0;
  g.world = 2;
  g.mapped[0] = g.local;
  g.mapped[1] = g.fake_peer;
  return 0;
}
CGTB_API int cgtb_peer_selftest_post(const float* host_payload, long count) {
  if (!g.fake_peer) return fail("cgtb_peer_selftest_post: no self-test group");
  if ((size_t)count * 4 > g.slot_bytes) return fail("cgtb_peer_selftest_post: payload too large");
  CGTB_CUDA_TRY(cudaStreamSynchronize(rt().stream));
  Header h;
  CGTB_CUDA_TRY(cudaMemcpy(&h, g.local, sizeof(h), cudaMemcpyDeviceToHost));
  const unsigned long long epoch = h.epoch + 1;
  const int slot = (int)(epoch & 1ull);
  CGTB_CUDA_TRY(cudaMemcpy(g.fake_peer + kHeaderBytes + (size_t)slot * g.slot_bytes, host_payload, (size_t)count * 4, cudaMemcpyHostToDevice));
  CGTB_CUDA_TRY(cudaMemcpy(g.fake_peer + 256 + 128 * slot, &epoch, sizeof(epoch), cudaMemcpyHostToDevice));
  return 0;
}
