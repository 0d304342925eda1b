/* Object model of the B200 execution backend, source-compatible with the names that reference-style
 * Op code strings use (reference: include/cgt_common.h:73-227, include/IRC.h).
 *
 * Differences from the reference, all deliberate:
 *   - arrays carry a device index and, for views, a retained base object, so a Reshape view keeps
 *     its source alive (the reference view does not: cgt/core.py:1461);
 *   - device memory comes from a caching pool and host memory owned by the runtime is pinned;
 *   - cgt_memcpy is asynchronous on the runtime's current CUDA stream (the reference uses a
 *     synchronous cudaMemcpy, src/cgt_common.cpp:138-153); callers that read the bytes on the host
 *     call cgt_stream_synchronize() first;
 *   - errors are recorded and returned as status codes, nothing aborts the process.
 *
 * User-defined Ops compiled at run time include this header and link against libcgt_b200.so.
 */
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include "cgt_b200_ops.h"

#define CGT_EXPORT __attribute__((visibility("default")))
#define CGT_EXPORT_C extern "C" __attribute__((visibility("default")))

/* dtype / devtype enums keep the reference's spelling; values are numpy type numbers */
typedef enum cgtDtype {
  cgt_i1 = cgtb_i1, cgt_i2 = cgtb_i2, cgt_i4 = cgtb_i4, cgt_i8 = cgtb_i8,
  cgt_f4 = cgtb_f4, cgt_f8 = cgtb_f8
} cgtDtype;
typedef enum cgtDevtype { cgtCPU = cgtbCPU, cgtGPU = cgtbGPU } cgtDevtype;

static inline int cgt_itemsize(cgtDtype d) {
  switch (d) {
    case cgt_i1: return 1;
    case cgt_i2: return 2;
    case cgt_i4: case cgt_f4: return 4;
    case cgt_i8: case cgt_f8: return 8;
  }
  return -1;
}

/* ---- error channel: status + message, read back through cgtb_last_error() ---- */
typedef enum { cgtStatusOK = 0, cgtStatusErr = 1 } cgtStatus;
CGT_EXPORT_C void cgt_set_error(const char* fmt, ...);
CGT_EXPORT_C cgtStatus cgt_get_status(void);
CGT_EXPORT_C void cgt_clear_error(void);
static inline void clear_error() { cgt_clear_error(); }
#define cgt_check(x, msg, ...) do { if (!(x)) cgt_set_error(msg, ##__VA_ARGS__); } while (0)
/* the reference aborts here (cgt_common.h:183-191); this build records the failure instead */
#define cgt_assert(x) do { if (!(x)) cgt_set_error("Assertion failed: %s (%s:%d)", #x, __FILE__, __LINE__); } while (0)

/* ---- memory (reference: cgt_alloc/cgt_free/cgt_memcpy, src/cgt_common.cpp:110-153) ---- */
CGT_EXPORT_C void* cgt_alloc(cgtDevtype devtype, long size);
CGT_EXPORT_C void cgt_free(cgtDevtype devtype, void* ptr);
CGT_EXPORT_C void cgt_memcpy(cgtDevtype dest_type, cgtDevtype src_type, void* dest_ptr, void* src_ptr, long nbytes);
CGT_EXPORT_C void cgt_stream_synchronize(void);
CGT_EXPORT_C void* cgt_current_stream(void); /* cudaStream_t of the calling thread's runtime context */

/* ---- objects ---- */
class cgtObject {
 public:
  enum ObjectKind { UndefKind = 0, ArrayKind = 1, TupleKind = 2 };
  explicit cgtObject(ObjectKind k) : refs_(0), kind_(k) {}
  ObjectKind kind() const { return kind_; }
  void Retain() const { refs_.fetch_add(1, std::memory_order_relaxed); }
  inline void Release() const;
  unsigned refcount() const { return refs_.load(std::memory_order_relaxed); }
 protected:
  ~cgtObject() {}
 private:
  mutable std::atomic<unsigned> refs_;
  ObjectKind kind_;
};

/* intrusive smart pointer (reference: IRC<T>, include/IRC.h:79-147) */
template <class T>
class IRC {
 public:
  IRC() : p_(nullptr) {}
  IRC(T* p) : p_(p) { if (p_) p_->Retain(); }
  IRC(const IRC& o) : p_(o.p_) { if (p_) p_->Retain(); }
  ~IRC() { if (p_) p_->Release(); }
  IRC& operator=(const IRC& o) { reset(o.p_); return *this; }
  IRC& operator=(T* p) { reset(p); return *this; }
  void reset(T* p) { if (p) p->Retain(); T* old = p_; p_ = p; if (old) old->Release(); }
  T* get() const { return p_; }
  T* operator->() const { return p_; }
  T& operator*() const { return *p_; }
  explicit operator bool() const { return p_ != nullptr; }
 private:
  T* p_;
};

class cgtArray : public cgtObject {
 public:
  /* owning array: storage from cgt_alloc(devtype) */
  CGT_EXPORT cgtArray(int ndim, const long* shape, cgtDtype dtype, cgtDevtype devtype);
  /* copy == true : owning array initialised from host memory `fromdata`
   * copy == false: non-owning view of `fromdata`, which already lives on `devtype` */
  CGT_EXPORT cgtArray(int ndim, const long* shape, cgtDtype dtype, cgtDevtype devtype, void* fromdata, bool copy);
  /* view that keeps `base` alive */
  CGT_EXPORT cgtArray(int ndim, const long* shape, cgtDtype dtype, cgtDevtype devtype, void* data, cgtObject* base);
  CGT_EXPORT ~cgtArray();

  int ndim() const { return ndim_; }
  const long* shape() const { return shape_; }
  long size() const { long s = 1; for (int i = 0; i < ndim_; ++i) s *= shape_[i]; return s; }
  long nbytes() const { return size() * cgt_itemsize(dtype_); }
  long stride(int i) const {
    if (ndim_ == 0) return 0;
    long s = 1;
    for (int j = i + 1; j < ndim_; ++j) s *= shape_[j];
    return s;
  }
  cgtDtype dtype() const { return dtype_; }
  cgtDevtype devtype() const { return devtype_; }
  bool ownsdata() const { return ownsdata_; }
  void* data() { return data_; }
  const void* data() const { return data_; }

  template <typename T> T& at() { return static_cast<T*>(data_)[0]; }
  template <typename T> T& at(long i) { return static_cast<T*>(data_)[i]; }
  template <typename T> T& at(long i, long j) { return static_cast<T*>(data_)[i * shape_[1] + j]; }
  template <typename T> T& at(long i, long j, long k) { return static_cast<T*>(data_)[(i * shape_[1] + j) * shape_[2] + k]; }
  template <typename T> T& at(long i, long j, long k, long l) {
    return static_cast<T*>(data_)[((i * shape_[1] + j) * shape_[2] + k) * shape_[3] + l];
  }
  CGT_EXPORT void print();

 private:
  void set_shape(int ndim, const long* shape);
  int ndim_;
  long shape_[CGTB_MAX_NDIM];
  cgtDtype dtype_;
  cgtDevtype devtype_;
  bool ownsdata_;
  void* data_;
  cgtObject* base_; /* retained while this view lives; may be NULL */
};

class cgtTuple : public cgtObject {
 public:
  CGT_EXPORT explicit cgtTuple(int len);
  CGT_EXPORT ~cgtTuple();
  void setitem(int i, cgtObject* o) { members[i] = o; }
  cgtObject* getitem(int i) { return members[i].get(); }
  int size() { return len; }
  int len;
  IRC<cgtObject>* members;
};

inline void cgtObject::Release() const {
  if (refs_.fetch_sub(1, std::memory_order_acq_rel) == 1) {
    if (kind_ == ArrayKind) delete static_cast<const cgtArray*>(this);
    else if (kind_ == TupleKind) delete static_cast<const cgtTuple*>(this);
  }
}

static inline bool cgt_is_array(cgtObject* o) { return o->kind() == cgtObject::ArrayKind; }
static inline bool cgt_is_tuple(cgtObject* o) { return o->kind() == cgtObject::TupleKind; }

/* copy `from` into `to`, crossing devices when they differ (reference: src/cgt_common.cpp:72-90) */
CGT_EXPORT_C void cgt_copy_object(cgtObject* to, cgtObject* from);
CGT_EXPORT_C void cgt_copy_array(cgtArray* to, cgtArray* from);
CGT_EXPORT_C void cgt_copy_tuple(cgtTuple* to, cgtTuple* from);

/* kernel-side boundary: the two callable signatures of the reference (cgt_common.h:176-177) */
typedef void (*cgtByRefFun)(void* closure, cgtObject** reads, cgtObject* write);
typedef cgtObject* (*cgtByValFun)(void* closure, cgtObject** reads);
