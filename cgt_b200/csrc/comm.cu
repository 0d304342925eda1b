// Gradient exchange for minibatch-sharded data parallelism: one process per GPU, NCCL over
// NVLink / NVSwitch. The reference has no collective of any kind (its MemLocation carries only a
// devtype, include/execution.h:42), so this is an addition behind a new Op ("AllReduce").
//
// NCCL is not linked: the library that PyTorch ships is opened at run time (path given by the
// caller), so the process holds a single NCCL instance. The unique id is created on rank 0 and
// distributed by the host side (a torch.distributed / gloo broadcast).
#include "runtime.h"
#include <dlfcn.h>
#include <nccl.h>
#include <algorithm>
#include <cstring>

using namespace cgtb;

namespace {
struct Nccl {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
} g;

template <typename F>
bool sym(F& f, const char* name) {
  f = (F)dlsym(g.handle, name);
  if (!f) fail("NCCL library lacks symbol %s", name);
  return f != nullptr;
}
}  // namespace

// Many small gradients: one collective on a packed copy instead of one per tensor. A group of k small
// all-reduces runs as k latency-bound rounds (8 tensors, 0.33 MB in all: the eight-GPU step lost 115 us
// to them); packed, it is one round plus two copy kernels. Words are 4 bytes (a float64 tensor is two
// words per element), tensor t occupies words [off[t], off[t+1]) of the packed buffer.
namespace {
constexpr int kPackMax = 32;
constexpr long kPackLimitBytes = 4L << 20;
struct PackArgs {
  const uint32_t* src[kPackMax];
  uint32_t* dst[kPackMax];
  long off[kPackMax + 1];
  int n;
};
// dir 0: tensors -> packed; dir 1: packed -> result tensors
__global__ void pack_kernel(const PackArgs a, uint32_t* __restrict__ flat, int dir) {
  const long total = a.off[a.n];
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int t = 0;
    while (t + 1 < a.n && i >= a.off[t + 1]) ++t;
    const long j = i - a.off[t];
    if (dir == 0) flat[i] = a.src[t][j];
    else a.dst[t][j] = flat[i];
  }
}
}  // namespace

#define NCCL_TRY(expr)                                                                                  \
  do {                                                                                                  \
    ncclResult_t r_ = (expr);                                                                           \
    if (r_ != ncclSuccess) return fail("%s failed: %s", #expr, g.GetErrorString ? g.GetErrorString(r_) : "?"); \
  } while (0)

CGTB_API int cgtb_comm_load(const char* nccl_path) {
  if (g.handle) return 0;
  g.handle = dlopen(nccl_path, RTLD_NOW | RTLD_GLOBAL);
  if (!g.handle) return fail("cannot open NCCL library %s: %s", nccl_path, dlerror());
  bool ok = sym(g.GetUniqueId, "ncclGetUniqueId") && sym(g.CommInitRank, "ncclCommInitRank") &&
            sym(g.AllReduce, "ncclAllReduce") && sym(g.GroupStart, "ncclGroupStart") && sym(g.GroupEnd, "ncclGroupEnd") &&
            sym(g.CommDestroy, "ncclCommDestroy") && sym(g.CommAbort, "ncclCommAbort") &&
            sym(g.CommGetAsyncError, "ncclCommGetAsyncError") && sym(g.GetErrorString, "ncclGetErrorString");
  if (!ok) { dlclose(g.handle); g.handle = nullptr; return 1; }
  return 0;
}
// 128-byte id for the other ranks
CGTB_API int cgtb_comm_unique_id(char* out128) {
  if (!g.handle) return fail("cgtb_comm_unique_id: NCCL not loaded");
  ncclUniqueId id;
  NCCL_TRY(g.GetUniqueId(&id));
  memcpy(out128, &id, sizeof(id));
  return 0;
}
CGTB_API int cgtb_comm_init(const char* id128, int rank, int world) {
  if (!require_runtime("cgtb_comm_init")) return 1;
  if (!g.handle) return fail("cgtb_comm_init: NCCL not loaded");
  if (g.comm) return fail("cgtb_comm_init: communicator already exists");
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  NCCL_TRY(g.CommInitRank(&g.comm, world, id, rank));
  g.rank = rank;
  g.world = world;
  return 0;
}
CGTB_API int cgtb_comm_world(void) { return g.comm ? g.world : 1; }
CGTB_API int cgtb_comm_rank(void) { return g.comm ? g.rank : 0; }
CGTB_API int cgtb_comm_destroy(void) {
  if (g.comm) {
    if (rt().ready) cudaStreamSynchronize(rt().stream);
    g.CommDestroy(g.comm);
    g.comm = nullptr;
  }
  return 0;
}
// 0 when the communicator is healthy; records the asynchronous error otherwise (rank-failure detection
// is host-side: the caller polls this between steps)
CGTB_API int cgtb_comm_check(void) {
  if (!g.comm) return 0;
  ncclResult_t st = ncclSuccess;
  NCCL_TRY(g.CommGetAsyncError(g.comm, &st));
  if (st != ncclSuccess && st != ncclInProgress) return fail("NCCL asynchronous error: %s", g.GetErrorString(st));
  return 0;
}
CGTB_API int cgtb_comm_abort(void) {
  if (g.comm) { g.CommAbort(g.comm); g.comm = nullptr; }
  return 0;
}

// sum over ranks of `n` buffers (float32 / float64), all queued as one NCCL group on the runtime stream
CGTB_API int cgtb_allreduce_sum(int dtype, int n, const void* const* in, void* const* out, const long* counts) {
  if (!require_runtime("cgtb_allreduce_sum")) return 1;
  ncclDataType_t dt;
  size_t esize;
  if (dtype == cgtb_f4) { dt = ncclFloat32; esize = 4; }
  else if (dtype == cgtb_f8) { dt = ncclFloat64; esize = 8; }
  else return fail("cgtb_allreduce_sum: unsupported dtype %d", dtype);
  if (!g.comm) {  // single process: the sum over one rank is a copy
    for (int i = 0; i < n; ++i)
      if (in[i] != out[i])
        CGTB_CUDA_TRY(cudaMemcpyAsync(out[i], in[i], (size_t)counts[i] * esize, cudaMemcpyDeviceToDevice, rt().stream));
    return 0;
  }
  long total_elems = 0;
  for (int i = 0; i < n; ++i) total_elems += counts[i] > 0 ? counts[i] : 0;
  if (n >= 2 && n <= kPackMax && total_elems > 0 && total_elems * (long)esize <= kPackLimitBytes) {
    const long wpe = (long)esize / 4;  // words per element
    PackArgs a;
    a.n = n;
    a.off[0] = 0;
    for (int i = 0; i < n; ++i) {
      a.src[i] = (const uint32_t*)in[i];
      a.dst[i] = (uint32_t*)out[i];
      a.off[i + 1] = a.off[i] + (counts[i] > 0 ? counts[i] : 0) * wpe;
    }
    uint32_t* flat = (uint32_t*)scratch((size_t)a.off[n] * 4);
    if (!flat) return 1;
    const unsigned blocks = (unsigned)std::min<long>(cgtb_ceil_div(a.off[n], 256), 2L * rt().sm_count);
    CGTB_LAUNCH(pack_kernel, blocks, 256, 0, a, flat, 0);
    NCCL_TRY(g.AllReduce(flat, flat, (size_t)total_elems, dt, ncclSum, g.comm, rt().stream));
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    CGTB_LAUNCH(pack_kernel, blocks, 256, 0, a, flat, 1);
    CGTB_CHECK_LAUNCH("allreduce pack");
    return 0;
  }
  NCCL_TRY(g.GroupStart());
  for (int i = 0; i < n; ++i) {
    ncclResult_t r = g.AllReduce(in[i], out[i], (size_t)counts[i], dt, ncclSum, g.comm, rt().stream);
    if (r != ncclSuccess) { g.GroupEnd(); return fail("ncclAllReduce failed: %s", g.GetErrorString(r)); }
  }
  NCCL_TRY(g.GroupEnd());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

namespace cgtb {
bool peer_ready(size_t bytes);
int peer_allreduce(int n, const void* const* in, void* const* out, const long* counts);
}  // namespace cgtb

// Op callable of the peer-memory variant (small float32 payloads; capturable: an ordinary kernel launch). Fails
// loudly when the payload does not fit the symmetric buffer: it never falls back to the library collective, which
// must stay outside captured graphs.
CGTB_API void cgtb_op_allreduce_peer(void* cl0, cgtObject** reads, cgtObject* write0) {
  struct Closure { int n; };
  Closure* cl = (Closure*)cl0;
  cgtTuple* out = (cgtTuple*)write0;
  const void* in[32];
  void* dst[32];
  long counts[32];
  if (cl->n > 32) { fail("AllReduce (peer memory): more than 32 tensors in one group"); return; }
  long total = 0;
  for (int i = 0; i < cl->n; ++i) {
    cgtArray *a = (cgtArray*)reads[i], *o = (cgtArray*)out->getitem(i);
    if (a->devtype() != cgtGPU || o->devtype() != cgtGPU || a->dtype() != cgt_f4 || a->size() != o->size()) {
      fail("AllReduce (peer memory): operands must be float32 device arrays of equal sizes");
      return;
    }
    in[i] = a->data();
    dst[i] = o->data();
    counts[i] = a->size();
    total += a->size();
  }
  if (!cgtb::peer_ready((size_t)total * 4)) {
    fail("AllReduce (peer memory): no peer group, or %ld bytes exceed its slot", total * 4);
    return;
  }
  cgtb::peer_allreduce(cl->n, in, dst, counts);
}

// Op callable: reads g_1..g_k (device arrays), writes a tuple of k arrays with the rank-sums.
struct AllReduceClosure { int n; };
CGTB_API void cgtb_op_allreduce(void* cl0, cgtObject** reads, cgtObject* write0) {
  AllReduceClosure* cl = (AllReduceClosure*)cl0;
  cgtTuple* out = (cgtTuple*)write0;
  const void* in[64];
  void* dst[64];
  long counts[64];
  if (cl->n > 64) { fail("AllReduce: more than 64 tensors in one group"); return; }
  int dtype = -1;
  for (int i = 0; i < cl->n; ++i) {
    cgtArray *a = (cgtArray*)reads[i], *o = (cgtArray*)out->getitem(i);
    if (a->devtype() != cgtGPU || o->devtype() != cgtGPU) { fail("AllReduce: operands must be on the GPU"); return; }
    if (dtype < 0) dtype = a->dtype();
    if ((int)a->dtype() != dtype || a->size() != o->size()) { fail("AllReduce: mixed dtypes or sizes"); return; }
    in[i] = a->data();
    dst[i] = o->data();
    counts[i] = a->size();
  }
  cgtb_allreduce_sum(dtype, cl->n, in, dst, counts);
}
