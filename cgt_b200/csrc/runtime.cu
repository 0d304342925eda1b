// Runtime of libcgt_b200.so: device binding, stream, caching device pool, pinned host pool, error
// channel, and the cgtArray / cgtTuple object model behind the C ABI.
//
// Replaces src/cgt_common.cpp of the reference (cudaMalloc / cudaFree / synchronous cudaMemcpy per
// array) with pooled, stream-ordered equivalents.
#include "runtime.h"
#include <cstdarg>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace cgtb {

static Runtime g_rt;
Runtime& rt() { return g_rt; }
std::atomic<long> g_kernel_launches{0};

// ---------------------------------------------------------------- errors
static thread_local std::string t_err;
static thread_local cgtStatus t_status = cgtStatusOK;

int fail(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_err = buf;
  t_status = cgtStatusErr;
  return 1;
}

bool require_runtime(const char* who) {
  if (g_rt.ready) return true;
  fail("%s: the CUDA runtime of libcgt_b200 is not initialised (call cgtb_init(device) on a machine with a GPU); "
       "there is no CPU fallback",
       who);
  return false;
}

// ---------------------------------------------------------------- pools
// Size classes: four per power of two, 512-byte floor. A freed block goes on the free list of its
// class and is handed out again LIFO, so a steady-state step allocates nothing from the driver.
static size_t size_class(size_t n) {
  if (n < 512) return 512;
  size_t p = 512;
  while (p * 2 <= n) p *= 2;  // p <= n < 2p
  size_t q = p / 4;
  size_t r = ((n - p + q - 1) / q) * q + p;
  return r;
}

struct Pool {
  std::mutex mu;
  std::map<size_t, std::vector<void*>> free_lists;
  std::unordered_map<void*, size_t> live;  // ptr -> class size
  long reserved = 0, in_use = 0, high_water = 0, n_mallocs = 0;
  bool pinned_host = false;

  void* get(size_t nbytes) {
    size_t cls = size_class(nbytes ? nbytes : 1);
    std::lock_guard<std::mutex> lk(mu);
    auto& fl = free_lists[cls];
    void* p = nullptr;
    if (!fl.empty()) {
      p = fl.back();
      fl.pop_back();
    } else {
      if (capturing()) {
        fail("memory pool miss for %zu bytes during CUDA graph capture", nbytes);
        return nullptr;
      }
      cudaError_t e = pinned_host ? cudaHostAlloc(&p, cls, cudaHostAllocDefault) : cudaMalloc(&p, cls);
      if (e != cudaSuccess) {
        fail("%s of %zu bytes failed: %s", pinned_host ? "cudaHostAlloc" : "cudaMalloc", cls, cudaGetErrorString(e));
        return nullptr;
      }
      reserved += (long)cls;
      n_mallocs += 1;
    }
    live[p] = cls;
    in_use += (long)cls;
    if (in_use > high_water) high_water = in_use;
    return p;
  }
  void put(void* p) {
    if (!p) return;
    std::lock_guard<std::mutex> lk(mu);
    auto it = live.find(p);
    if (it == live.end()) return;  // not ours
    size_t cls = it->second;
    live.erase(it);
    in_use -= (long)cls;
    free_lists[cls].push_back(p);
  }
  void trim() {
    std::lock_guard<std::mutex> lk(mu);
    for (auto& kv : free_lists) {
      for (void* p : kv.second) {
        if (pinned_host) cudaFreeHost(p); else cudaFree(p);
        reserved -= (long)kv.first;
      }
      kv.second.clear();
    }
  }
};

static Pool g_dev_pool;
static Pool g_host_pool;

// Small pinned-host allocations (scalars, shape values) are carved from 1 MiB slabs: one
// cudaHostAlloc per slab instead of one per scalar.
struct HostSlabs {
  std::mutex mu;
  static constexpr size_t kSlab = 1 << 20, kMaxSmall = 4096;
  char* cur = nullptr;
  size_t used = kSlab;
  std::map<size_t, std::vector<void*>> free_lists;
  std::unordered_map<void*, size_t> live;
  static size_t cls(size_t n) { size_t c = 64; while (c < n) c *= 2; return c; }
  void* get(size_t n) {
    size_t c = cls(n ? n : 1);
    std::lock_guard<std::mutex> lk(mu);
    auto& fl = free_lists[c];
    void* p;
    if (!fl.empty()) { p = fl.back(); fl.pop_back(); }
    else {
      if (used + c > kSlab) {
        void* s = nullptr;
        cudaError_t e = g_rt.ready ? cudaHostAlloc(&s, kSlab, cudaHostAllocDefault) : cudaErrorInitializationError;
        if (e != cudaSuccess) { s = aligned_alloc(64, kSlab); }  // no GPU: plain host memory
        cur = (char*)s;
        used = 0;
      }
      p = cur + used;
      used += c;
    }
    live[p] = c;
    return p;
  }
  bool put(void* p) {
    std::lock_guard<std::mutex> lk(mu);
    auto it = live.find(p);
    if (it == live.end()) return false;
    free_lists[it->second].push_back(p);
    live.erase(it);
    return true;
  }
};
static HostSlabs g_slabs;

static thread_local bool t_capturing = false;
void set_capturing(bool on) { t_capturing = on; }
bool capturing() { return t_capturing; }
long device_malloc_count() { return g_dev_pool.n_mallocs; }

// ---------------------------------------------------------------- scratch
static thread_local ScratchOwner* t_scratch_owner = nullptr;
static ScratchOwner g_global_scratch;
void set_scratch_owner(ScratchOwner* o) { t_scratch_owner = o; }
void free_scratch_owner(ScratchOwner* o) {
  if (o && o->ptr) { g_dev_pool.put(o->ptr); o->ptr = nullptr; o->cap = 0; }
  if (o && o->outer_ptr) { g_dev_pool.put(o->outer_ptr); o->outer_ptr = nullptr; o->outer_cap = 0; }
}
void* scratch(size_t nbytes) {
  ScratchOwner* o = t_scratch_owner ? t_scratch_owner : &g_global_scratch;
  if (o->cap >= nbytes && o->ptr) return o->ptr;
  if (o->ptr) {
    // the old block may still be in use by kernels already queued on the stream; the pool hands a
    // freed block only to later work on the same stream, so returning it here is safe
    g_dev_pool.put(o->ptr);
    o->ptr = nullptr;
    o->cap = 0;
  }
  o->ptr = g_dev_pool.get(nbytes);
  o->cap = o->ptr ? size_class(nbytes) : 0;
  return o->ptr;
}

void* scratch_outer(size_t nbytes) {
  ScratchOwner* o = t_scratch_owner ? t_scratch_owner : &g_global_scratch;
  if (o->outer_cap >= nbytes && o->outer_ptr) return o->outer_ptr;
  if (o->outer_ptr) {
    g_dev_pool.put(o->outer_ptr);
    o->outer_ptr = nullptr;
    o->outer_cap = 0;
  }
  o->outer_ptr = g_dev_pool.get(nbytes);
  o->outer_cap = o->outer_ptr ? size_class(nbytes) : 0;
  return o->outer_ptr;
}

}  // namespace cgtb

using namespace cgtb;

// ================================================================== C ABI: runtime
CGTB_API int cgtb_init(int device) {
  if (g_rt.ready) {
    if (g_rt.device == device) return 0;
    return fail("cgtb_init: already bound to device %d (one GPU per process)", g_rt.device);
  }
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail("cgtb_init: no CUDA device available (%s); this backend has no CPU fallback",
                e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  if (device < 0 || device >= n) return fail("cgtb_init: device %d out of range (have %d)", device, n);
  CGTB_CUDA_TRY(cudaSetDevice(device));
  cudaDeviceProp prop;
  CGTB_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail("cgtb_init: device %d is sm_%d%d; this library carries sm_100a code only", device, prop.major, prop.minor);
  CGTB_CUDA_TRY(cudaStreamCreateWithFlags(&g_rt.stream, cudaStreamNonBlocking));
  g_rt.device = device;
  g_rt.sm_count = prop.multiProcessorCount;
  g_host_pool.pinned_host = true;
  g_rt.ready = true;
  return 0;
}
CGTB_API int cgtb_initialized(void) { return g_rt.ready ? 1 : 0; }
CGTB_API int cgtb_device(void) { return g_rt.ready ? g_rt.device : -1; }
CGTB_API const char* cgtb_last_error(void) { return t_err.c_str(); }
CGTB_API void cgtb_clear_error(void) { t_err.clear(); t_status = cgtStatusOK; }
CGTB_API int cgtb_synchronize(void) {
  if (!require_runtime("cgtb_synchronize")) return 1;
  CGTB_CUDA_TRY(cudaStreamSynchronize(g_rt.stream));
  return sgemm_tc_check();
}
CGTB_API void* cgtb_stream(void) { return (void*)g_rt.stream; }
CGTB_API int cgtb_pool_stats(long* reserved, long* in_use, long* high, long* n_mallocs) {
  std::lock_guard<std::mutex> lk(g_dev_pool.mu);
  if (reserved) *reserved = g_dev_pool.reserved;
  if (in_use) *in_use = g_dev_pool.in_use;
  if (high) *high = g_dev_pool.high_water;
  if (n_mallocs) *n_mallocs = g_dev_pool.n_mallocs;
  return 0;
}
CGTB_API int cgtb_pool_trim(void) {
  if (!require_runtime("cgtb_pool_trim")) return 1;
  cudaStreamSynchronize(g_rt.stream);
  g_dev_pool.trim();
  return 0;
}
CGTB_API long cgtb_kernel_launches(void) { return g_kernel_launches.load(); }
CGTB_API int cgtb_sm_count(void) { return g_rt.sm_count; }

// ================================================================== C ABI: memory
CGTB_API void* cgtb_alloc(int devtype, long nbytes) {
  if (devtype == cgtbGPU) {
    if (!require_runtime("cgtb_alloc(device)")) return nullptr;
    return g_dev_pool.get((size_t)nbytes);
  }
  if ((size_t)nbytes <= HostSlabs::kMaxSmall || !g_rt.ready) {
    if ((size_t)nbytes <= HostSlabs::kMaxSmall) return g_slabs.get((size_t)nbytes);
    return malloc((size_t)nbytes);  // no GPU bound: host-only use (CPU tests of the host logic)
  }
  return g_host_pool.get((size_t)nbytes);
}
CGTB_API void cgtb_free(int devtype, void* p) {
  if (!p) return;
  if (devtype == cgtbGPU) { g_dev_pool.put(p); return; }
  if (g_slabs.put(p)) return;
  {
    std::lock_guard<std::mutex> lk(g_host_pool.mu);
    if (!g_host_pool.live.count(p)) { free(p); return; }
  }
  g_host_pool.put(p);
}
CGTB_API int cgtb_memcpy(int dst_dev, int src_dev, void* dst, const void* src, long nbytes, int sync) {
  if (nbytes == 0) return 0;
  if (dst_dev == cgtbCPU && src_dev == cgtbCPU) { memcpy(dst, src, (size_t)nbytes); return 0; }
  if (!require_runtime("cgtb_memcpy")) return 1;
  cudaMemcpyKind kind = (src_dev == cgtbCPU) ? cudaMemcpyHostToDevice
                        : (dst_dev == cgtbCPU) ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
  CGTB_CUDA_TRY(cudaMemcpyAsync(dst, src, (size_t)nbytes, kind, g_rt.stream));
  if (sync) CGTB_CUDA_TRY(cudaStreamSynchronize(g_rt.stream));
  return 0;
}
CGTB_API int cgtb_memset(void* p, int value, long nbytes) {
  if (!require_runtime("cgtb_memset")) return 1;
  CGTB_CUDA_TRY(cudaMemsetAsync(p, value, (size_t)nbytes, g_rt.stream));
  return 0;
}

// reference-named wrappers used by Op code (include/cgt_common.h)
CGTB_API void cgt_set_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  fail("%s", buf);
}
CGTB_API cgtStatus cgt_get_status(void) { return t_status; }
CGTB_API void cgt_clear_error(void) { cgtb_clear_error(); }
CGTB_API void* cgt_alloc(cgtDevtype d, long size) { return cgtb_alloc((int)d, size); }
CGTB_API void cgt_free(cgtDevtype d, void* p) { cgtb_free((int)d, p); }
CGTB_API void cgt_memcpy(cgtDevtype dd, cgtDevtype sd, void* dst, void* src, long n) { cgtb_memcpy((int)dd, (int)sd, dst, src, n, 0); }
CGTB_API void cgt_stream_synchronize(void) { if (g_rt.ready) cudaStreamSynchronize(g_rt.stream); }
CGTB_API void* cgt_current_stream(void) { return (void*)g_rt.stream; }

// ================================================================== objects
void cgtArray::set_shape(int ndim, const long* shape) {
  ndim_ = ndim;
  for (int i = 0; i < ndim && i < CGTB_MAX_NDIM; ++i) shape_[i] = shape[i];
}
cgtArray::cgtArray(int ndim, const long* shape, cgtDtype dtype, cgtDevtype devtype)
    : cgtObject(ArrayKind), dtype_(dtype), devtype_(devtype), ownsdata_(true), base_(nullptr) {
  set_shape(ndim, shape);
  data_ = cgt_alloc(devtype_, nbytes() > 0 ? nbytes() : 1);
}
cgtArray::cgtArray(int ndim, const long* shape, cgtDtype dtype, cgtDevtype devtype, void* fromdata, bool copy)
    : cgtObject(ArrayKind), dtype_(dtype), devtype_(devtype), ownsdata_(copy), base_(nullptr) {
  set_shape(ndim, shape);
  if (copy) {
    data_ = cgt_alloc(devtype_, nbytes() > 0 ? nbytes() : 1);
    if (data_ && fromdata) cgtb_memcpy((int)devtype_, cgtbCPU, data_, fromdata, nbytes(), 1);
  } else {
    data_ = fromdata;
  }
}
cgtArray::cgtArray(int ndim, const long* shape, cgtDtype dtype, cgtDevtype devtype, void* data, cgtObject* base)
    : cgtObject(ArrayKind), dtype_(dtype), devtype_(devtype), ownsdata_(false), data_(data), base_(base) {
  set_shape(ndim, shape);
  if (base_) base_->Retain();
}
cgtArray::~cgtArray() {
  if (ownsdata_) cgt_free(devtype_, data_);
  if (base_) base_->Release();
}
void cgtArray::print() {
  printf("Array{shape=(");
  for (int i = 0; i < ndim_; ++i) printf(i ? ", %ld" : "%ld", shape_[i]);
  printf("), dtype=%i, dev=%i}", (int)dtype_, (int)devtype_);
}
cgtTuple::cgtTuple(int n) : cgtObject(TupleKind), len(n) { members = new IRC<cgtObject>[n > 0 ? n : 1]; }
cgtTuple::~cgtTuple() { delete[] members; }

CGTB_API void cgt_copy_array(cgtArray* to, cgtArray* from) {
  if (!(from->size() == to->size() && from->dtype() == to->dtype())) {
    fail("cgt_copy_array: size or dtype mismatch");
    return;
  }
  cgtb_memcpy((int)to->devtype(), (int)from->devtype(), to->data(), from->data(), from->nbytes(), 0);
}
CGTB_API void cgt_copy_tuple(cgtTuple* to, cgtTuple* from) {
  for (int i = 0; i < to->size(); ++i) cgt_copy_object(to->getitem(i), from->getitem(i));
}
CGTB_API void cgt_copy_object(cgtObject* to, cgtObject* from) {
  if (to->kind() != from->kind()) { fail("cgt_copy_object: kind mismatch"); return; }
  if (to->kind() == cgtObject::ArrayKind) cgt_copy_array((cgtArray*)to, (cgtArray*)from);
  else cgt_copy_tuple((cgtTuple*)to, (cgtTuple*)from);
}

// ================================================================== C ABI: objects
static inline cgtArray* A(cgtbObject* o) { return (cgtArray*)o; }
static inline cgtTuple* T(cgtbObject* o) { return (cgtTuple*)o; }

CGTB_API cgtbObject* cgtb_array_new(int ndim, const long* shape, int dtype, int devtype) {
  if (ndim > CGTB_MAX_NDIM) { fail("cgtb_array_new: ndim %d > %d", ndim, CGTB_MAX_NDIM); return nullptr; }
  if (devtype == cgtbGPU && !require_runtime("cgtb_array_new(device)")) return nullptr;
  cgtArray* a = new cgtArray(ndim, shape, (cgtDtype)dtype, (cgtDevtype)devtype);
  if (!a->data()) { delete a; return nullptr; }
  a->Retain();
  return (cgtbObject*)a;
}
CGTB_API cgtbObject* cgtb_array_from_host(int ndim, const long* shape, int dtype, int devtype, void* host, int copy) {
  if (ndim > CGTB_MAX_NDIM) { fail("cgtb_array_from_host: ndim %d > %d", ndim, CGTB_MAX_NDIM); return nullptr; }
  if (devtype == cgtbGPU && !require_runtime("cgtb_array_from_host(device)")) return nullptr;
  if (!copy && devtype != cgtbCPU) { fail("cgtb_array_from_host: a view must stay on the host"); return nullptr; }
  cgtArray* a = new cgtArray(ndim, shape, (cgtDtype)dtype, (cgtDevtype)devtype, host, copy != 0);
  if (!a->data() && a->nbytes() > 0) { delete a; return nullptr; }
  a->Retain();
  return (cgtbObject*)a;
}
CGTB_API cgtbObject* cgtb_array_view_device(int ndim, const long* shape, int dtype, void* dev_ptr) {
  cgtArray* a = new cgtArray(ndim, shape, (cgtDtype)dtype, cgtGPU, dev_ptr, false);
  a->Retain();
  return (cgtbObject*)a;
}
CGTB_API int cgtb_array_to_host(cgtbObject* o, void* dst) {
  cgtArray* a = A(o);
  return cgtb_memcpy(cgtbCPU, (int)a->devtype(), dst, a->data(), a->nbytes(), 1);
}
CGTB_API int cgtb_array_set_from_host(cgtbObject* o, const void* src) {
  cgtArray* a = A(o);
  return cgtb_memcpy((int)a->devtype(), cgtbCPU, a->data(), src, a->nbytes(), 1);
}
CGTB_API int cgtb_array_ndim(cgtbObject* o) { return A(o)->ndim(); }
CGTB_API const long* cgtb_array_shape(cgtbObject* o) { return A(o)->shape(); }
CGTB_API int cgtb_array_dtype(cgtbObject* o) { return (int)A(o)->dtype(); }
CGTB_API int cgtb_array_devtype(cgtbObject* o) { return (int)A(o)->devtype(); }
CGTB_API void* cgtb_array_data(cgtbObject* o) { return A(o)->data(); }
CGTB_API long cgtb_array_nbytes(cgtbObject* o) { return A(o)->nbytes(); }
CGTB_API cgtbObject* cgtb_tuple_new(int len) {
  cgtTuple* t = new cgtTuple(len);
  t->Retain();
  return (cgtbObject*)t;
}
CGTB_API int cgtb_tuple_len(cgtbObject* o) { return T(o)->len; }
CGTB_API cgtbObject* cgtb_tuple_get(cgtbObject* o, int i) { return (cgtbObject*)T(o)->getitem(i); }
CGTB_API int cgtb_tuple_set(cgtbObject* o, int i, cgtbObject* v) {
  if (i < 0 || i >= T(o)->len) return fail("cgtb_tuple_set: index %d out of range", i);
  T(o)->setitem(i, (cgtObject*)v);
  return 0;
}
CGTB_API int cgtb_object_kind(cgtbObject* o) { return (int)((cgtObject*)o)->kind(); }
CGTB_API void cgtb_retain(cgtbObject* o) { if (o) ((cgtObject*)o)->Retain(); }
CGTB_API void cgtb_release(cgtbObject* o) { if (o) ((cgtObject*)o)->Release(); }

// ================================================================== C ABI: timing helpers
CGTB_API void* cgtb_event_new(void) {
  if (!require_runtime("cgtb_event_new")) return nullptr;
  cudaEvent_t e = nullptr;
  if (cudaEventCreate(&e) != cudaSuccess) { fail("cudaEventCreate failed"); return nullptr; }
  return (void*)e;
}
CGTB_API int cgtb_event_record(void* e) {
  if (!require_runtime("cgtb_event_record")) return 1;
  CGTB_CUDA_TRY(cudaEventRecord((cudaEvent_t)e, g_rt.stream));
  return 0;
}
CGTB_API int cgtb_event_elapsed_ms(void* e0, void* e1, float* ms) {
  CGTB_CUDA_TRY(cudaEventSynchronize((cudaEvent_t)e1));
  CGTB_CUDA_TRY(cudaEventElapsedTime(ms, (cudaEvent_t)e0, (cudaEvent_t)e1));
  return 0;
}
CGTB_API void cgtb_event_free(void* e) { if (e) cudaEventDestroy((cudaEvent_t)e); }
// ================================================================== C ABI: input prefetch on a copy stream
// Uploading the next batch while the current step computes. A staging slot goes through
//   begin(slot)   copy stream waits until the step that last read the slot's buffers has finished
//   h2d(...)      copies on the copy stream
//   mark(slot)    closes the slot's group of copies
//   join(slot)    runtime stream waits for that group (not for groups queued behind it)
//   release(slot) recorded on the runtime stream after the consuming step has been queued
// No call here synchronises the host. `src` should be page-locked, otherwise the driver stages the copy
// and it does not overlap.
namespace {
constexpr int kPrefetchSlots = 4;
cudaStream_t g_copy_stream = nullptr;
cudaEvent_t g_copy_done[kPrefetchSlots] = {}, g_slot_free[kPrefetchSlots] = {};
bool g_slot_used[kPrefetchSlots] = {};
bool copy_stream_ready() {
  if (g_copy_stream) return true;
  bool ok = cudaStreamCreateWithFlags(&g_copy_stream, cudaStreamNonBlocking) == cudaSuccess;
  for (int i = 0; ok && i < kPrefetchSlots; ++i)
    ok = cudaEventCreateWithFlags(&g_copy_done[i], cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&g_slot_free[i], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    g_copy_stream = nullptr;
    fail("cannot create the copy stream");
  }
  return ok;
}
bool slot_ok(const char* who, int slot) {
  if (slot >= 0 && slot < kPrefetchSlots) return true;
  fail("%s: slot %d out of range", who, slot);
  return false;
}
}  // namespace
CGTB_API int cgtb_prefetch_begin(int slot) {
  if (!require_runtime("cgtb_prefetch_begin") || !slot_ok("cgtb_prefetch_begin", slot) || !copy_stream_ready()) return 1;
  if (g_slot_used[slot]) CGTB_CUDA_TRY(cudaStreamWaitEvent(g_copy_stream, g_slot_free[slot], 0));
  return 0;
}
CGTB_API int cgtb_prefetch_h2d(void* dst_device, const void* src_host, long nbytes) {
  if (!require_runtime("cgtb_prefetch_h2d")) return 1;
  if (nbytes < 0 || (nbytes > 0 && (!dst_device || !src_host))) return fail("cgtb_prefetch_h2d: bad arguments");
  if (!copy_stream_ready()) return 1;
  if (nbytes > 0) CGTB_CUDA_TRY(cudaMemcpyAsync(dst_device, src_host, (size_t)nbytes, cudaMemcpyHostToDevice, g_copy_stream));
  return 0;
}
CGTB_API int cgtb_prefetch_mark(int slot) {
  if (!require_runtime("cgtb_prefetch_mark") || !slot_ok("cgtb_prefetch_mark", slot) || !copy_stream_ready()) return 1;
  CGTB_CUDA_TRY(cudaEventRecord(g_copy_done[slot], g_copy_stream));
  return 0;
}
CGTB_API int cgtb_prefetch_join(int slot) {
  if (!require_runtime("cgtb_prefetch_join") || !slot_ok("cgtb_prefetch_join", slot) || !copy_stream_ready()) return 1;
  CGTB_CUDA_TRY(cudaStreamWaitEvent(g_rt.stream, g_copy_done[slot], 0));
  return 0;
}
CGTB_API int cgtb_prefetch_release(int slot) {
  if (!require_runtime("cgtb_prefetch_release") || !slot_ok("cgtb_prefetch_release", slot) || !copy_stream_ready()) return 1;
  CGTB_CUDA_TRY(cudaEventRecord(g_slot_free[slot], g_rt.stream));
  g_slot_used[slot] = true;
  return 0;
}
// overwrite a buffer larger than L2 (126 MB on B200) so that the next kernels start from a cold L2
CGTB_API int cgtb_l2_flush(void) {
  if (!require_runtime("cgtb_l2_flush")) return 1;
  static void* buf = nullptr;
  static const size_t kBytes = (size_t)256 << 20;
  if (!buf) CGTB_CUDA_TRY(cudaMalloc(&buf, kBytes));
  CGTB_CUDA_TRY(cudaMemsetAsync(buf, 0, kBytes, g_rt.stream));
  return 0;
}

// A launch that the CUDA runtime refuses on the host (2048 threads per block exceed the limit of 1024): nothing
// reaches the GPU. Exists so that a test can check that such a refusal is reported once, with its own name, and
// does not stay behind as the process's "last error" for later, healthy calls to trip over.
static __global__ void selftest_noop_kernel(int* p) { if (p) *p = 0; }
CGTB_API int cgtb_selftest_refused_launch(void) {
  if (!require_runtime("cgtb_selftest_refused_launch")) return 1;
  CGTB_LAUNCH(selftest_noop_kernel, 1, 2048, 0, (int*)nullptr);
  CGTB_CHECK_LAUNCH("selftest_refused_launch");
  return 0;
}
