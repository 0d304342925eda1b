// Execution-graph interpreter for devtype "gpu".
//
// Same instruction set and callable ABI as the reference's SequentialInterpreter
// (src/execution.cpp:19-58, 247-292): LoadArgument, Alloc (re-allocates only when the shape changes),
// BuildTup, ReturnByRef, ReturnByVal. What differs is how device work is issued:
//
//   * every device instruction enqueues kernels on the runtime's CUDA stream and returns at once;
//   * cross-device copies (Transport) are asynchronous; a host instruction that reads array data
//     waits for the stream only when a device->host copy is outstanding;
//   * the instruction list is cut into spans at every Transport / non-capturable instruction. Once a
//     span has run twice with identical buffer addresses (steady state: no allocation happens any
//     more), its device instructions are captured into a CUDA graph and later runs replay the graph
//     with one launch. The replay is used only while a key over all buffer addresses and small host
//     operands that the span's device instructions see is unchanged, so a shape change, a set_value()
//     on a shared variable or a changed host scalar falls back to eager issue and re-capture;
//   * a run whose arguments have the buffers, shapes and small host values of the run before it, with no
//     shared variable replaced in between and no allocation in the run before, is a steady run: its host
//     bookkeeping instructions (Alloc, BuildTup, views, shape arithmetic) would reproduce what the storage
//     already holds, so they are skipped, and a span's graph is launched without recomputing its key. Host
//     instructions that compute on array data still run; from the first one whose result differs from the run
//     before, the rest of the run takes the full path again. Without this the host walks the whole instruction
//     list before each launch: thousands of instructions for an unrolled recurrent network, more time than
//     the device needs for them.
#include "runtime.h"
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

using namespace cgtb;

namespace {

enum Kind { kLoadArgument, kAlloc, kBuildTup, kReturnByRef, kReturnByVal };
enum Klass { kMeta, kHostData, kDevice, kBarrier };

struct Loc {
  long idx;
  int dev;
};

struct Instr {
  Kind kind;
  std::string repr;
  int flags = 0;
  std::vector<Loc> reads;
  Loc write{0, 0};
  int arg_index = 0;
  cgtDtype dtype = cgt_f4;
  void* fptr = nullptr;
  void* closure = nullptr;
  Klass klass = kMeta;
  bool fired = false;
  bool arg_view = false;  // host bookkeeping on (a view of) an argument: fired in steady runs too
  ScratchOwner scratch;
  double prof_ms = 0;
  long prof_count = 0;
};

struct Span {
  int begin = 0, end = 0;  // [begin, end)
  bool barrier = false;    // single Transport / non-capturable instruction
  int n_device = 0;
  bool has_hostdata = false;
  cudaGraphExec_t exec = nullptr;
  uint64_t exec_key = 0, last_key = 0;
  bool have_last = false, capture_failed = false;
  long graph_kernels = 0;
};

}  // namespace

struct cgtbGraph {
  long n_args, n_locs;
  std::vector<Instr> instrs;
};

struct cgtbInterp {
  cgtbGraph* g;
  std::vector<Loc> outs;
  std::vector<IRC<cgtObject>> storage;
  cgtTuple* args = nullptr;
  int flags = 0;
  std::vector<Span> spans;
  bool host_pending = false;  // a device->host copy has been queued and not yet waited for
  long runs = 0, last_launches = 0, last_graph_launches = 0, captured = 0;
  long mallocs_at_run_start = 0;
  bool prev_run_allocated = true;
  void (*before_sync)(void*) = nullptr;  // called once per run after all device work has been queued
  void* before_sync_ctx = nullptr;
  // steady-run detection
  std::vector<uint64_t> arg_sig;        // signature of the previous run's arguments
  long state_version_seen = -1;
  bool steady = false;                  // this run repeats the previous one as far as host bookkeeping goes
  bool host_dirty = false;              // a host data instruction of this run produced a new value
  bool prev_run_ok = false;
  uint64_t args_read_in_place = ~0ull;  // arguments whose device buffer a captured instruction reads directly
  long last_host_ns = 0;                // host time of the last run up to the final wait for the stream
  long steady_runs = 0;
};

static std::atomic<long> g_state_version{0};
// Called by the host side whenever a shared variable's array is replaced (a set_value with a new shape).
CGTB_API void cgtb_state_version_bump(void) { g_state_version.fetch_add(1, std::memory_order_relaxed); }

// ------------------------------------------------------------------------------------------------
// graph construction
// ------------------------------------------------------------------------------------------------
CGTB_API cgtbGraph* cgtb_graph_new(long n_args, long n_locs) {
  cgtbGraph* g = new cgtbGraph();
  g->n_args = n_args;
  g->n_locs = n_locs;
  return g;
}
CGTB_API void cgtb_graph_free(cgtbGraph* g) {
  if (!g) return;
  for (auto& in : g->instrs) free_scratch_owner(&in.scratch);
  delete g;
}

static int check_loc(cgtbGraph* g, long idx) {
  if (idx < 0 || idx >= g->n_locs) return fail("memory location %ld out of range (n_locs %ld)", idx, g->n_locs);
  return 0;
}

CGTB_API int cgtb_graph_add_load_argument(cgtbGraph* g, const char* repr, int arg_index, long wloc, int wdev) {
  if (check_loc(g, wloc)) return 1;
  if (arg_index < 0 || arg_index >= g->n_args) return fail("LoadArgument: argument index %d out of range", arg_index);
  Instr in;
  in.kind = kLoadArgument;
  in.repr = repr ? repr : "";
  in.arg_index = arg_index;
  in.write = {wloc, wdev};
  g->instrs.push_back(in);
  return 0;
}
CGTB_API int cgtb_graph_add_alloc(cgtbGraph* g, const char* repr, int dtype, int n_shape, const long* shape_locs, long wloc,
                                  int wdev) {
  if (check_loc(g, wloc)) return 1;
  if (n_shape > CGTB_MAX_NDIM) return fail("Alloc: ndim %d too large", n_shape);
  Instr in;
  in.kind = kAlloc;
  in.repr = repr ? repr : "";
  in.dtype = (cgtDtype)dtype;
  for (int i = 0; i < n_shape; ++i) {
    if (check_loc(g, shape_locs[i])) return 1;
    in.reads.push_back({shape_locs[i], cgtbCPU});
  }
  in.write = {wloc, wdev};
  g->instrs.push_back(in);
  return 0;
}
CGTB_API int cgtb_graph_add_build_tup(cgtbGraph* g, const char* repr, int n, const long* read_locs, long wloc, int wdev) {
  if (check_loc(g, wloc)) return 1;
  Instr in;
  in.kind = kBuildTup;
  in.repr = repr ? repr : "";
  for (int i = 0; i < n; ++i) {
    if (check_loc(g, read_locs[i])) return 1;
    in.reads.push_back({read_locs[i], wdev});
  }
  in.write = {wloc, wdev};
  g->instrs.push_back(in);
  return 0;
}
static int add_return(cgtbGraph* g, Kind kind, const char* repr, int n, const long* read_locs, const int* read_devs, long wloc,
                      int wdev, void* fptr, void* closure, int flags) {
  if (check_loc(g, wloc)) return 1;
  if (!fptr) return fail("%s: null function pointer", repr ? repr : "Return");
  Instr in;
  in.kind = kind;
  in.repr = repr ? repr : "";
  in.flags = flags;
  for (int i = 0; i < n; ++i) {
    if (check_loc(g, read_locs[i])) return 1;
    in.reads.push_back({read_locs[i], read_devs ? read_devs[i] : wdev});
  }
  in.write = {wloc, wdev};
  in.fptr = fptr;
  in.closure = closure;
  g->instrs.push_back(in);
  return 0;
}
CGTB_API int cgtb_graph_add_return_byref(cgtbGraph* g, const char* repr, int n, const long* read_locs, const int* read_devs,
                                         long wloc, int wdev, void* fptr, void* closure, int flags) {
  return add_return(g, kReturnByRef, repr, n, read_locs, read_devs, wloc, wdev, fptr, closure, flags);
}
CGTB_API int cgtb_graph_add_return_byval(cgtbGraph* g, const char* repr, int n, const long* read_locs, const int* read_devs,
                                         long wloc, int wdev, void* fptr, void* closure, int flags) {
  return add_return(g, kReturnByVal, repr, n, read_locs, read_devs, wloc, wdev, fptr, closure, flags);
}

// ------------------------------------------------------------------------------------------------
// interpreter
// ------------------------------------------------------------------------------------------------
// Cut the instruction list into spans at every barrier instruction. A fire-once barrier (a constant's
// transport) that has already fired no longer separates its neighbours, so after the first run the
// whole step usually collapses into one span per real transfer.
static void build_spans(cgtbInterp* it) {
  for (auto& s : it->spans)
    if (s.exec) cudaGraphExecDestroy(s.exec);
  it->spans.clear();
  auto& instrs = it->g->instrs;
  int n = (int)instrs.size();
  auto is_barrier = [&](int k) {
    Instr& in = instrs[(size_t)k];
    return in.klass == kBarrier && !((in.flags & CGTB_INSTR_ONCE) && in.fired);
  };
  int i = 0;
  while (i < n) {
    Span s;
    s.begin = i;
    if (is_barrier(i)) {
      s.barrier = true;
      s.end = i + 1;
    } else {
      int j = i;
      while (j < n && !is_barrier(j)) {
        if (instrs[(size_t)j].klass == kDevice) s.n_device++;
        if (instrs[(size_t)j].klass == kHostData) s.has_hostdata = true;
        ++j;
      }
      s.end = j;
    }
    it->spans.push_back(s);
    i = s.end;
  }
}

CGTB_API cgtbInterp* cgtb_interp_new(cgtbGraph* g, int n_out, const long* out_locs, int flags) {
  if (!g) { fail("cgtb_interp_new: null graph"); return nullptr; }
  cgtbInterp* it = new cgtbInterp();
  it->g = g;
  it->flags = flags;
  it->storage.resize((size_t)g->n_locs);
  for (int i = 0; i < n_out; ++i) {
    if (check_loc(g, out_locs[i])) { delete it; return nullptr; }
    it->outs.push_back({out_locs[i], 0});
  }
  bool any_device = false;
  for (auto& in : g->instrs) {
    if (in.kind == kLoadArgument || in.kind == kAlloc || in.kind == kBuildTup) in.klass = kMeta;
    else if (in.flags & (CGTB_INSTR_TRANSPORT | CGTB_INSTR_NOCAPTURE)) in.klass = kBarrier;
    else if (in.flags & CGTB_INSTR_QUICK) in.klass = kMeta;
    else if (in.write.dev == cgtbGPU) in.klass = (in.kind == kReturnByRef) ? kDevice : kBarrier;
    else in.klass = kHostData;
    if (in.write.dev == cgtbGPU) any_device = true;
    for (auto& r : in.reads) if (r.dev == cgtbGPU) any_device = true;
  }
  if (any_device && !require_runtime("cgtb_interp_new")) { delete it; return nullptr; }
  {
    // Bookkeeping instructions that see an argument object directly or through other bookkeeping (views, tuples,
    // sizes, allocations shaped by them) cannot be skipped in steady runs: the caller passes new objects every time.
    // from_arg[loc]: the arguments (bit i = argument i, the last bit stands for all beyond 62) that location loc holds
    // or views. An argument that a device instruction reads in place must keep its buffer for a run to be steady (the
    // captured graphs hold that address); one that only copies (Transport, a barrier) and bookkeeping look at may
    // move: a batch handed over in alternating staging buffers is still a steady run.
    std::vector<uint64_t> from_arg((size_t)g->n_locs, 0);
    uint64_t in_place = 0;
    for (auto& in : g->instrs) {
      if (in.klass == kDevice) {
        for (auto& r : in.reads) in_place |= from_arg[(size_t)r.idx];
        in_place |= from_arg[(size_t)in.write.idx];
        continue;
      }
      if (in.klass != kMeta) continue;
      uint64_t dep = in.kind == kLoadArgument ? (1ull << (in.arg_index < 63 ? in.arg_index : 63)) : 0;
      for (auto& r : in.reads) dep |= from_arg[(size_t)r.idx];
      in.arg_view = dep != 0;
      if (dep) from_arg[(size_t)in.write.idx] |= dep;
    }
    it->args_read_in_place = in_place;
  }
  build_spans(it);
  return it;
}

CGTB_API void cgtb_interp_free(cgtbInterp* it) {
  if (!it) return;
  if (rt().ready) cudaStreamSynchronize(rt().stream);
  for (auto& s : it->spans)
    if (s.exec) cudaGraphExecDestroy(s.exec);
  delete it;
}

static inline cgtObject* get(cgtbInterp* it, const Loc& l) { return it->storage[(size_t)l.idx].get(); }

static int fire(cgtbInterp* it, Instr& in) {
  switch (in.kind) {
    case kLoadArgument: {
      if (in.arg_index >= it->args->len) return fail("LoadArgument: missing argument %d", in.arg_index);
      it->storage[(size_t)in.write.idx] = it->args->members[in.arg_index].get();
      return 0;
    }
    case kAlloc: {
      int nd = (int)in.reads.size();
      long shape[CGTB_MAX_NDIM];
      for (int i = 0; i < nd; ++i) {
        cgtArray* sv = (cgtArray*)get(it, in.reads[(size_t)i]);
        if (!sv || sv->kind() != cgtObject::ArrayKind || sv->dtype() != cgt_i8 || sv->devtype() != cgtCPU)
          return fail("Alloc (%s): shape component %d is not a host int64 scalar", in.repr.c_str(), i);
        shape[i] = sv->at<long>(0);
        if (shape[i] < 0) return fail("Alloc (%s): negative extent", in.repr.c_str());
      }
      cgtObject* cur0 = get(it, in.write);
      cgtArray* cur = (cur0 && cur0->kind() == cgtObject::ArrayKind) ? (cgtArray*)cur0 : nullptr;
      bool same = cur && cur->ownsdata() && cur->ndim() == nd && cur->dtype() == in.dtype &&
                  (int)cur->devtype() == in.write.dev;
      for (int i = 0; same && i < nd; ++i) same = cur->shape()[i] == shape[i];
      if (!same) {
        cgtArray* a = new cgtArray(nd, shape, in.dtype, (cgtDevtype)in.write.dev);
        if (!a->data()) { a->Retain(); a->Release(); return 1; }
        it->storage[(size_t)in.write.idx] = a;
      }
      return 0;
    }
    case kBuildTup: {
      // rebuilt only when a member object changed, so a steady-state run allocates nothing
      cgtObject* cur0 = get(it, in.write);
      int n = (int)in.reads.size();
      if (cur0 && cur0->kind() == cgtObject::TupleKind && ((cgtTuple*)cur0)->len == n) {
        cgtTuple* t = (cgtTuple*)cur0;
        bool same = true;
        for (int i = 0; same && i < n; ++i) same = t->getitem(i) == get(it, in.reads[(size_t)i]);
        if (same) return 0;
      }
      cgtTuple* t = new cgtTuple(n);
      for (int i = 0; i < n; ++i) t->setitem(i, get(it, in.reads[(size_t)i]));
      it->storage[(size_t)in.write.idx] = t;
      return 0;
    }
    case kReturnByRef:
    case kReturnByVal: {
      int n = (int)in.reads.size();
      cgtObject* reads_small[16];
      std::vector<cgtObject*> reads_big;
      cgtObject** reads = reads_small;
      if (n > 16) { reads_big.resize((size_t)n); reads = reads_big.data(); }
      for (int i = 0; i < n; ++i) {
        reads[i] = get(it, in.reads[(size_t)i]);
        if (!reads[i]) return fail("%s: input %d was never produced", in.repr.c_str(), i);
      }
      set_scratch_owner(&in.scratch);
      if (in.kind == kReturnByRef) {
        cgtObject* w = get(it, in.write);
        if (!w) { set_scratch_owner(nullptr); return fail("%s: output was never allocated", in.repr.c_str()); }
        ((cgtByRefFun)in.fptr)(in.closure, reads, w);
      } else {
        cgtObject* r = ((cgtByValFun)in.fptr)(in.closure, reads);
        if (r) it->storage[(size_t)in.write.idx] = r;
        else if (cgt_get_status() == cgtStatusOK) fail("%s: callable returned NULL", in.repr.c_str());
      }
      set_scratch_owner(nullptr);
      if (cgt_get_status() != cgtStatusOK) {
        std::string msg = cgtb_last_error();
        return fail("%s: %s", in.repr.c_str(), msg.c_str());
      }
      return 0;
    }
  }
  return 0;
}

static inline uint64_t mix(uint64_t h, uint64_t v) {
  h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
  return h;
}
static uint64_t key_of_object(uint64_t h, cgtObject* o, int dev) {
  if (!o) return mix(h, 0);
  if (o->kind() == cgtObject::ArrayKind) {
    cgtArray* a = (cgtArray*)o;
    h = mix(h, (uint64_t)(uintptr_t)a->data());
    // a captured graph bakes shape-derived launch parameters into its nodes, and the pool can hand the same block
    // to a differently shaped array of equal size: the extents and the dtype are part of the key
    h = mix(h, ((uint64_t)a->ndim() << 8) | (uint64_t)a->dtype());
    for (int d = 0; d < a->ndim(); ++d) h = mix(h, (uint64_t)a->shape()[d]);
    if (a->devtype() == cgtCPU && a->nbytes() <= 64 && a->data()) {  // small host operand read at launch time
      uint64_t buf[8] = {0};
      memcpy(buf, a->data(), (size_t)a->nbytes());
      for (int i = 0; i < 8; ++i) h = mix(h, buf[i]);
    }
  } else {
    cgtTuple* t = (cgtTuple*)o;
    for (int i = 0; i < t->len; ++i) h = key_of_object(h, t->getitem(i), dev);
  }
  return h;
}
static uint64_t span_key(cgtbInterp* it, const Span& s) {
  uint64_t h = 1469598103934665603ull;
  for (int i = s.begin; i < s.end; ++i) {
    Instr& in = it->g->instrs[(size_t)i];
    if (in.klass != kDevice) continue;
    for (auto& r : in.reads) h = key_of_object(h, get(it, r), r.dev);
    h = key_of_object(h, get(it, in.write), in.write.dev);
  }
  return h;
}

static int fire_profiled(cgtbInterp* it, Instr& in) {
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0, rt().stream);
  int rc = fire(it, in);
  cudaEventRecord(e1, rt().stream);
  cudaEventSynchronize(e1);
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  in.prof_ms += ms;
  in.prof_count += 1;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return rc;
}

// ------------------------------------------------------------------------------------------------
// Capture with several streams. Stream capture of a single stream yields a linear chain of kernel nodes; the
// step's data flow is wider than that (filter gradients next to the data-gradient chain, eight parameter updates,
// the operand preparations of a layer). During capture every device instruction is given the address ranges it
// reads and writes (its operands' device buffers, views and in-place results included, since ranges are
// compared, not locations); an instruction depends on the earlier ones whose writes overlap what it touches or
// whose reads overlap what it writes. It is issued on one of a few side streams that join the capture through
// events: the stream of a dependency if that dependency is the stream's last instruction, otherwise the stream
// idle for longest, after waiting for the events of its dependencies. The graph then holds the true edges and
// independent kernels run side by side. Arithmetic is untouched: the same kernels on the same buffers.
// ------------------------------------------------------------------------------------------------
struct AddrRange { uintptr_t lo, hi; };

static void collect_ranges(cgtObject* o, std::vector<AddrRange>& out) {
  if (!o) return;
  if (o->kind() == cgtObject::ArrayKind) {
    cgtArray* a = (cgtArray*)o;
    if (a->devtype() == cgtGPU && a->data() && a->nbytes() > 0) out.push_back({(uintptr_t)a->data(), (uintptr_t)a->data() + (uintptr_t)a->nbytes()});
  } else {
    cgtTuple* t = (cgtTuple*)o;
    for (int i = 0; i < t->len; ++i) collect_ranges(t->getitem(i), out);
  }
}
static bool overlap(const std::vector<AddrRange>& a, const std::vector<AddrRange>& b) {
  for (const AddrRange& x : a)
    for (const AddrRange& y : b)
      if (x.lo < y.hi && y.lo < x.hi) return true;
  return false;
}

constexpr int kMaxGraphStreams = 8;
static cudaStream_t g_side_streams[kMaxGraphStreams];
static int g_n_side_streams = 0;
static std::vector<cudaEvent_t> g_capture_events;

static int graph_streams() {
  static int n = -1;
  if (n < 0) {
    // default 1 (a linear chain): measured on the five benchmark configurations, two to six streams changed the step
    // time by less than the run-to-run spread, because the large kernels fill every SM and the small ones form
    // dependent chains; the option stays for graphs with wide, independent branches
    const char* e = getenv("CGTB_GRAPH_STREAMS");
    n = e ? atoi(e) : 1;
    if (n < 1) n = 1;
    if (n > kMaxGraphStreams) n = kMaxGraphStreams;
  }
  return n;
}
static cudaEvent_t capture_event(size_t i) {
  while (g_capture_events.size() <= i) {
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    g_capture_events.push_back(e);
  }
  return g_capture_events[i];
}

// Fires the device instructions of span s inside the running capture of `origin`, spread over side streams.
static int fire_span_multistream(cgtbInterp* it, Span& s, cudaStream_t origin) {
  auto& instrs = it->g->instrs;
  const int NS = graph_streams();
  while (g_n_side_streams < NS) {
    if (cudaStreamCreateWithFlags(&g_side_streams[g_n_side_streams], cudaStreamNonBlocking) != cudaSuccess) return fail("cudaStreamCreate failed");
    ++g_n_side_streams;
  }
  struct Node { int instr; int stream; std::vector<AddrRange> rd, wr; bool opaque; };
  std::vector<Node> nodes;
  std::vector<int> last_on_stream((size_t)NS, -1);   // node index of the last instruction issued on each stream
  std::vector<long> last_use((size_t)NS, -1);
  std::vector<bool> joined((size_t)NS, false);
  // event 0: the fork point on the origin stream
  cudaEvent_t fork = capture_event(0);
  if (!fork) return fail("cudaEventCreate failed");
  CGTB_CUDA_TRY(cudaEventRecord(fork, origin));
  int rc = 0;
  long tick = 0;
  for (int i = s.begin; i < s.end && !rc; ++i) {
    Instr& in = instrs[(size_t)i];
    if (in.klass != kDevice) continue;
    if ((in.flags & CGTB_INSTR_ONCE) && in.fired) continue;
    Node nd;
    nd.instr = i;
    nd.opaque = (in.kind != kReturnByRef);   // a device instruction that creates its own result: ordered against everything
    for (auto& r : in.reads) collect_ranges(get(it, r), nd.rd);
    if (!nd.opaque) collect_ranges(get(it, in.write), nd.wr);
    // dependencies: the latest conflicting instruction per stream is enough (a stream is ordered)
    std::vector<int> dep_of_stream((size_t)NS, -1);
    for (int j = (int)nodes.size() - 1; j >= 0; --j) {
      const Node& e = nodes[(size_t)j];
      if (dep_of_stream[(size_t)e.stream] >= 0) continue;
      if (nd.opaque || e.opaque || overlap(e.wr, nd.rd) || overlap(e.wr, nd.wr) || overlap(e.rd, nd.wr)) dep_of_stream[(size_t)e.stream] = j;
    }
    // stream choice
    int chosen = -1;
    for (int st = 0; st < NS; ++st)
      if (dep_of_stream[(size_t)st] >= 0 && dep_of_stream[(size_t)st] == last_on_stream[(size_t)st] && (chosen < 0 || dep_of_stream[(size_t)st] > dep_of_stream[(size_t)chosen])) chosen = st;
    if (chosen < 0) {
      for (int st = 0; st < NS; ++st)
        if (chosen < 0 || last_use[(size_t)st] < last_use[(size_t)chosen]) chosen = st;
    }
    cudaStream_t cs = g_side_streams[chosen];
    if (!joined[(size_t)chosen]) {
      CGTB_CUDA_TRY(cudaStreamWaitEvent(cs, fork, 0));
      joined[(size_t)chosen] = true;
    }
    for (int st = 0; st < NS; ++st) {
      const int d = dep_of_stream[(size_t)st];
      if (d < 0 || st == chosen) continue;
      cudaEvent_t ev = capture_event((size_t)d + 1);
      if (!ev) return fail("cudaEventCreate failed");
      CGTB_CUDA_TRY(cudaStreamWaitEvent(cs, ev, 0));
    }
    nd.stream = chosen;
    cudaStream_t saved = rt().stream;
    rt().stream = cs;
    rc = fire(it, in);
    rt().stream = saved;
    if (rc) break;
    cudaEvent_t mine = capture_event(nodes.size() + 1);
    if (!mine) return fail("cudaEventCreate failed");
    CGTB_CUDA_TRY(cudaEventRecord(mine, cs));
    last_on_stream[(size_t)chosen] = (int)nodes.size();
    last_use[(size_t)chosen] = tick++;
    nodes.push_back(std::move(nd));
  }
  // join every side stream back into the origin
  for (int st = 0; st < NS; ++st) {
    if (!joined[(size_t)st]) continue;
    const int l = last_on_stream[(size_t)st];
    if (l >= 0) CGTB_CUDA_TRY(cudaStreamWaitEvent(origin, capture_event((size_t)l + 1), 0));
    else {
      cudaEvent_t ev = capture_event(nodes.size() + 2 + (size_t)st);
      CGTB_CUDA_TRY(cudaEventRecord(ev, g_side_streams[st]));
      CGTB_CUDA_TRY(cudaStreamWaitEvent(origin, ev, 0));
    }
  }
  return rc;
}

static int run_span(cgtbInterp* it, Span& s) {
  auto& instrs = it->g->instrs;
  const bool profile = (it->flags & CGTB_INTERP_PROFILE) && rt().ready;
  if (s.barrier) {
    Instr& in = instrs[(size_t)s.begin];
    if ((in.flags & CGTB_INSTR_ONCE) && in.fired) return 0;
    bool is_transport = in.flags & CGTB_INSTR_TRANSPORT;
    if (!is_transport && rt().ready) {  // arbitrary callable: give it a quiet stream
      cudaStreamSynchronize(rt().stream);
      it->host_pending = false;
    }
    int rc = profile ? fire_profiled(it, in) : fire(it, in);
    if (rc) return rc;
    in.fired = true;
    if (is_transport && in.write.dev == cgtbCPU) it->host_pending = true;
    return 0;
  }
  if (s.has_hostdata && it->host_pending) {
    CGTB_CUDA_TRY(cudaStreamSynchronize(rt().stream));
    it->host_pending = false;
  }
  // pass 1: host bookkeeping and host scalar arithmetic, in program order
  for (int i = s.begin; i < s.end; ++i) {
    Instr& in = instrs[(size_t)i];
    if (in.klass == kDevice) continue;
    if ((in.flags & CGTB_INSTR_ONCE) && in.fired) continue;
    const bool fast = it->steady && !it->host_dirty;
    if (fast && in.klass == kMeta && !in.arg_view) continue;  // the storage already holds its result
    if (fast && in.klass == kHostData) {
      // did this instruction produce the value it produced in the run before? (small results only: a large one
      // counts as new)
      unsigned char before[64];
      size_t nb = 0;
      bool small = false;
      cgtObject* w = get(it, in.write);
      if (w && w->kind() == cgtObject::ArrayKind && ((cgtArray*)w)->devtype() == cgtCPU && ((cgtArray*)w)->nbytes() <= 64 &&
          ((cgtArray*)w)->data()) {
        nb = (size_t)((cgtArray*)w)->nbytes();
        memcpy(before, ((cgtArray*)w)->data(), nb);
        small = true;
      }
      if (fire(it, in)) return 1;
      cgtObject* w2 = get(it, in.write);
      if (!small || w2 != w || memcmp(before, ((cgtArray*)w2)->data(), nb) != 0) it->host_dirty = true;
      in.fired = true;
      continue;
    }
    if (fire(it, in)) return 1;
    in.fired = true;
  }
  if (s.n_device == 0) return 0;
  // pass 2: device instructions, replayed from a CUDA graph when the span is in steady state
  bool use_graphs = (it->flags & CGTB_INTERP_CUDA_GRAPHS) && !profile && !s.capture_failed && s.n_device >= 2;
  if (use_graphs && it->steady && !it->host_dirty && s.exec && s.have_last && s.exec_key == s.last_key) {
    // nothing that the key covers can have changed since the run before, which launched this graph
    CGTB_CUDA_TRY(cudaGraphLaunch(s.exec, rt().stream));
    it->last_graph_launches += 1;
    it->last_launches += s.graph_kernels;
    return 0;
  }
  uint64_t key = use_graphs ? span_key(it, s) : 0;
  if (use_graphs && s.exec && s.exec_key == key) {
    s.last_key = key;
    s.have_last = true;
    CGTB_CUDA_TRY(cudaGraphLaunch(s.exec, rt().stream));
    it->last_graph_launches += 1;
    it->last_launches += s.graph_kernels;
    return 0;
  }
  bool capture = use_graphs && s.have_last && s.last_key == key && !it->prev_run_allocated;
  s.last_key = key;
  s.have_last = true;
  if (capture) {
    if (s.exec) { cudaGraphExecDestroy(s.exec); s.exec = nullptr; }
    long launches0 = g_kernel_launches.load();
    cudaError_t e = cudaStreamBeginCapture(rt().stream, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
      set_capturing(true);
      int rc = 0;
      if (graph_streams() > 1) {
        rc = fire_span_multistream(it, s, rt().stream);
      } else {
        for (int i = s.begin; i < s.end && !rc; ++i) {
          Instr& in = instrs[(size_t)i];
          if (in.klass != kDevice) continue;
          if ((in.flags & CGTB_INSTR_ONCE) && in.fired) continue;
          rc = fire(it, in);
        }
      }
      set_capturing(false);
      cudaGraph_t graph = nullptr;
      e = cudaStreamEndCapture(rt().stream, &graph);
      if (rc == 0 && e == cudaSuccess && graph) {
        e = cudaGraphInstantiate(&s.exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e == cudaSuccess) {
          s.exec_key = key;   // == s.last_key
          s.graph_kernels = g_kernel_launches.load() - launches0;
          it->captured += 1;
          for (int i = s.begin; i < s.end; ++i)
            if (instrs[(size_t)i].klass == kDevice) instrs[(size_t)i].fired = true;
          CGTB_CUDA_TRY(cudaGraphLaunch(s.exec, rt().stream));
          it->last_graph_launches += 1;
          it->last_launches += s.graph_kernels;
          return 0;
        }
        s.exec = nullptr;
      } else if (graph) {
        cudaGraphDestroy(graph);
      }
    }
    // capture did not work for this span: clear the sticky capture error and issue eagerly from now on
    cudaGetLastError();
    cgtb_clear_error();
    s.capture_failed = true;
  }
  for (int i = s.begin; i < s.end; ++i) {
    Instr& in = instrs[(size_t)i];
    if (in.klass != kDevice) continue;
    if ((in.flags & CGTB_INSTR_ONCE) && in.fired) continue;
    long l0 = g_kernel_launches.load();
    int rc = profile ? fire_profiled(it, in) : fire(it, in);
    if (rc) return rc;
    in.fired = true;
    it->last_launches += g_kernel_launches.load() - l0;
  }
  return 0;
}

CGTB_API int cgtb_interp_run(cgtbInterp* it, cgtbObject* args_obj, cgtbObject** out) {
  if (!it || !args_obj || !out) return fail("cgtb_interp_run: null argument");
  cgtTuple* args = (cgtTuple*)args_obj;
  if (((cgtObject*)args_obj)->kind() != cgtObject::TupleKind || args->len != it->g->n_args)
    return fail("cgtb_interp_run: expected a tuple of %ld arguments", it->g->n_args);
  cgtb_clear_error();
  const auto host_t0 = std::chrono::steady_clock::now();
  it->args = args;
  it->last_launches = 0;
  it->last_graph_launches = 0;
  long mallocs0 = device_malloc_count();
  int rc = 0;
  {
    // signature of the arguments: buffers, dtypes and extents; the bytes of small host arrays (they may be read
    // as operands at launch time); for large host arrays only the shape (they are copied by a Transport)
    std::vector<uint64_t> sig;
    sig.reserve(16);
    std::vector<std::pair<cgtObject*, bool>> stack;   // (object, its device address matters)
    for (int i = 0; i < args->len; ++i)
      stack.push_back({args->getitem(i), ((it->args_read_in_place >> (i < 63 ? i : 63)) & 1ull) != 0});
    while (!stack.empty()) {
      cgtObject* o = stack.back().first;
      const bool pinned = stack.back().second;
      stack.pop_back();
      if (!o) { sig.push_back(0); continue; }
      if (o->kind() == cgtObject::TupleKind) {
        cgtTuple* t = (cgtTuple*)o;
        sig.push_back(0x7475706cull + (uint64_t)t->len);
        for (int i = 0; i < t->len; ++i) stack.push_back({t->getitem(i), pinned});
        continue;
      }
      cgtArray* a = (cgtArray*)o;
      sig.push_back(((uint64_t)a->ndim() << 16) | ((uint64_t)a->dtype() << 8) | (uint64_t)a->devtype());
      for (int d = 0; d < a->ndim(); ++d) sig.push_back((uint64_t)a->shape()[d]);
      if (a->devtype() == cgtGPU) { if (pinned) sig.push_back((uint64_t)(uintptr_t)a->data()); }
      else if (a->nbytes() <= 64 && a->data()) {
        uint64_t buf[8] = {0};
        memcpy(buf, a->data(), (size_t)a->nbytes());
        for (int i = 0; i < 8; ++i) sig.push_back(buf[i]);
      }
    }
    const long ver = g_state_version.load(std::memory_order_relaxed);
    static const bool allow = []() { const char* e = getenv("CGTB_STEADY_RUNS"); return !(e && e[0] == '0'); }();
    it->steady = allow && it->prev_run_ok && !it->prev_run_allocated && it->runs >= 2 && ver == it->state_version_seen &&
                 sig == it->arg_sig && !(it->flags & CGTB_INTERP_PROFILE);
    it->arg_sig.swap(sig);
    it->state_version_seen = ver;
    it->host_dirty = false;
    if (it->steady) it->steady_runs += 1;
  }
  // The before-sync hook (host work that should overlap this run's device work, e.g. queueing the next batch's
  // upload) runs as soon as the last span that queues device work or a copy has been issued: the host-only
  // spans after it (arithmetic on a scalar that was copied back) wait for the stream.
  long last_queueing = -1;
  for (size_t i = 0; i < it->spans.size(); ++i)
    if (it->spans[i].barrier || it->spans[i].n_device > 0) last_queueing = (long)i;
  bool hooked = false;
  for (size_t i = 0; i < it->spans.size(); ++i) {
    rc = run_span(it, it->spans[i]);
    if (rc) break;
    if ((long)i == last_queueing && it->before_sync) {
      it->before_sync(it->before_sync_ctx);
      hooked = true;
    }
  }
  it->args = nullptr;
  if (!rc && !hooked && it->before_sync) it->before_sync(it->before_sync_ctx);
  it->last_host_ns = (long)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - host_t0).count();
  if (rt().ready) {
    cudaError_t e = cudaStreamSynchronize(rt().stream);
    it->host_pending = false;
    if (e != cudaSuccess && !rc) rc = fail("device work of this run failed: %s", cudaGetErrorString(e));
    if (!rc) rc = sgemm_tc_check();
  }
  it->prev_run_allocated = device_malloc_count() != mallocs0;
  it->prev_run_ok = rc == 0;
  it->runs += 1;
  if (it->runs == 1 && !rc) build_spans(it);  // fire-once barriers are out of the way now
  if (rc) return rc;
  cgtTuple* o = new cgtTuple((int)it->outs.size());
  o->Retain();
  for (size_t i = 0; i < it->outs.size(); ++i) o->setitem((int)i, get(it, it->outs[i]));
  *out = (cgtbObject*)o;
  return 0;
}

CGTB_API int cgtb_interp_set_before_sync(cgtbInterp* it, void (*fn)(void*), void* ctx) {
  if (!it) return fail("cgtb_interp_set_before_sync: null interpreter");
  it->before_sync = fn;
  it->before_sync_ctx = ctx;
  return 0;
}

CGTB_API int cgtb_interp_stats(cgtbInterp* it, long* c, int n) {
  long graph_kernels = 0, dev = 0;
  for (auto& s : it->spans) { if (s.exec) graph_kernels += s.graph_kernels; dev += s.n_device; }
  long v[8] = {it->runs, it->last_launches, it->last_graph_launches, it->captured, graph_kernels, dev, it->last_host_ns, it->steady_runs};
  for (int i = 0; i < n && i < 8; ++i) c[i] = v[i];
  return 0;
}
CGTB_API int cgtb_interp_profile(cgtbInterp* it, double* ms, long* counts, int cap) {
  int n = (int)it->g->instrs.size();
  for (int i = 0; i < n && i < cap; ++i) { ms[i] = it->g->instrs[(size_t)i].prof_ms; counts[i] = it->g->instrs[(size_t)i].prof_count; }
  return n;
}
CGTB_API const char* cgtb_interp_instr_repr(cgtbInterp* it, int i) {
  if (i < 0 || i >= (int)it->g->instrs.size()) return "";
  return it->g->instrs[(size_t)i].repr.c_str();
}
CGTB_API int cgtb_apply_byref(void* fptr, void* closure, int n, cgtbObject** reads, cgtbObject* write) {
  if (!fptr) return fail("cgtb_apply_byref: null function pointer");
  cgtb_clear_error();
  ((cgtByRefFun)fptr)(closure, (cgtObject**)reads, (cgtObject*)write);
  if (cgt_get_status() != cgtStatusOK) return 1;
  if (rt().ready) CGTB_CUDA_TRY(cudaStreamSynchronize(rt().stream));
  return 0;
}
