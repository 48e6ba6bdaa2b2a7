// Native replay of a recorded training step.
//
// The reference walks its topological order in Python every step and calls one ctypes entry per node
// (python/athena/gpu_ops/executor.py:140-152; vdnnExecutor.py:261-325 adds the swap bookkeeping).  Here a planned
// step is a fixed list of actions at fixed addresses: kernel entries of the native libraries, event records and
// stream waits, copies between the region and pinned host buffers.  Every one of them is an `extern "C"` function
// that returns an int status, so the executor records (function, argument values) once while it runs a step the
// ordinary way, and this file replays the list from one C call: no interpreter between two launches.
//
//   tsb_tape_create   copies the action list (function addresses, per-argument type code and 8-byte value cell,
//                     by-pointer host data such as shape vectors and peer pointer tables) and prepares one call
//                     interface per action
//   tsb_tape_replay   fills the dynamic cells (arguments that change from step to step, e.g. the epoch of the flag
//                     words of the gradient exchange) and calls the actions in order; stops at the first non-zero
//                     status and reports which action returned it
//
// Calls with run-time signatures go through libffi, the same library the interpreter's own foreign-function layer
// uses; it is opened with dlopen at first use (no header of it is needed: the handful of declarations below is its
// stable public C interface).  Without it tsb_tape_available() returns 0 and the executor keeps its Python loop.
#include <dlfcn.h>
#include <stdint.h>
#include <string.h>

#include <chrono>
#include <vector>

#define TSB_OK 0
#define TSB_ERR_ARG 1
#define TSB_ERR_UNSUPPORTED 7

namespace {

struct FfiType {                 // libffi's ffi_type
  size_t size;
  unsigned short alignment;
  unsigned short type;
  FfiType** elements;
};
typedef int (*PrepCif)(void* cif, int abi, unsigned nargs, FfiType* rtype, FfiType** atypes);
typedef void (*FfiCall)(void* cif, void (*fn)(void), void* rvalue, void** avalue);

#if defined(__x86_64__)
constexpr int kDefaultAbi = 2;   // FFI_UNIX64
#elif defined(__aarch64__)
constexpr int kDefaultAbi = 1;   // FFI_SYSV
#else
constexpr int kDefaultAbi = -1;
#endif

struct Ffi {
  bool tried = false, ok = false;
  PrepCif prep = nullptr;
  FfiCall call = nullptr;
  FfiType *t_ptr = nullptr, *t_i32 = nullptr, *t_u32 = nullptr, *t_i64 = nullptr, *t_f32 = nullptr, *t_f64 = nullptr;
};

Ffi& ffi() {
  static Ffi f;
  if (f.tried) return f;
  f.tried = true;
  if (kDefaultAbi < 0) return f;
  void* h = nullptr;
  for (const char* name : {"libffi.so.8", "libffi.so.7", "libffi.so"}) {
    h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) return f;
  f.prep = reinterpret_cast<PrepCif>(dlsym(h, "ffi_prep_cif"));
  f.call = reinterpret_cast<FfiCall>(dlsym(h, "ffi_call"));
  f.t_ptr = static_cast<FfiType*>(dlsym(h, "ffi_type_pointer"));
  f.t_i32 = static_cast<FfiType*>(dlsym(h, "ffi_type_sint32"));
  f.t_u32 = static_cast<FfiType*>(dlsym(h, "ffi_type_uint32"));
  f.t_i64 = static_cast<FfiType*>(dlsym(h, "ffi_type_sint64"));
  f.t_f32 = static_cast<FfiType*>(dlsym(h, "ffi_type_float"));
  f.t_f64 = static_cast<FfiType*>(dlsym(h, "ffi_type_double"));
  f.ok = f.prep && f.call && f.t_ptr && f.t_i32 && f.t_u32 && f.t_i64 && f.t_f32 && f.t_f64 &&
         f.t_ptr->size == sizeof(void*) && f.t_i32->size == 4 && f.t_f64->size == 8;
  return f;
}

FfiType* type_of(char code) {
  Ffi& f = ffi();
  switch (code) {
    case 'p': case 'b': return f.t_ptr;
    case 'i': return f.t_i32;
    case 'u': return f.t_u32;
    case 'q': return f.t_i64;
    case 'f': return f.t_f32;
    case 'd': return f.t_f64;
    default: return nullptr;
  }
}

struct alignas(16) Cif { unsigned char bytes[96]; };   // room for libffi's ffi_cif on every supported ABI

struct Tape {
  std::vector<void (*)(void)> fn;
  std::vector<int> arg_begin;                 // action -> first argument
  std::vector<uint64_t> cell;                 // one 8-byte cell per argument (little-endian value)
  std::vector<uint64_t> dyn_cell;             // one per dynamic slot
  std::vector<void*> avalue;                  // per argument: address of its cell
  std::vector<FfiType*> atype;
  std::vector<Cif> cif;
  std::vector<unsigned char> blob;            // host data passed by pointer
};

}  // namespace

extern "C" {

int tsb_tape_available() { return ffi().ok ? 1 : 0; }

// n actions; action a has arguments [arg_begin[a], arg_begin[a + 1]).  Per argument: `types` (p pointer, i / u
// 32-bit int, q 64-bit int, f float, d double, b pointer into `blob` at byte offset `values`), `values` (raw bits),
// `dyn_slot` (-1, or the slot whose value is supplied at every replay).  Returns an opaque handle or null.
void* tsb_tape_create(int n, void* const* fns, const int* arg_begin, const char* types, const uint64_t* values,
                      const int* dyn_slot, int n_dyn, const unsigned char* blob, long long blob_bytes) {
  Ffi& f = ffi();
  if (!f.ok || n < 0 || !arg_begin || n_dyn < 0 || blob_bytes < 0) return nullptr;
  const int total = arg_begin[n];
  Tape* t = new Tape();
  t->fn.resize(n);
  t->arg_begin.assign(arg_begin, arg_begin + n + 1);
  t->cell.assign(values, values + total);
  t->dyn_cell.assign(n_dyn, 0);
  t->avalue.resize(total);
  t->atype.resize(total);
  t->cif.resize(n);
  t->blob.assign(blob, blob + blob_bytes);
  for (int i = 0; i < total; ++i) {
    t->atype[i] = type_of(types[i]);
    if (!t->atype[i] || dyn_slot[i] >= n_dyn) { delete t; return nullptr; }
    if (types[i] == 'b') {
      if (values[i] > (uint64_t)blob_bytes) { delete t; return nullptr; }
      t->cell[i] = reinterpret_cast<uint64_t>(t->blob.data() + values[i]);
    }
    t->avalue[i] = dyn_slot[i] >= 0 ? static_cast<void*>(&t->dyn_cell[dyn_slot[i]]) : static_cast<void*>(&t->cell[i]);
  }
  for (int a = 0; a < n; ++a) {
    t->fn[a] = reinterpret_cast<void (*)(void)>(fns[a]);
    const int b = arg_begin[a], e = arg_begin[a + 1];
    if (!fns[a] || e < b ||
        f.prep(t->cif[a].bytes, kDefaultAbi, (unsigned)(e - b), f.t_i32, t->atype.data() + b) != 0) {
      delete t;
      return nullptr;
    }
  }
  return t;
}

// Calls the actions [first, last) in order.  dyn: n_dyn 8-byte values for the dynamic slots.  Returns the first
// non-zero status (0 if none); *failed_at receives that action's index (-1 if none), *host_ns the time spent here.
int tsb_tape_replay(void* tape, int first, int last, const uint64_t* dyn, int n_dyn, int* failed_at,
                    long long* host_ns) {
  Tape* t = static_cast<Tape*>(tape);
  if (failed_at) *failed_at = -1;
  if (!t || n_dyn != (int)t->dyn_cell.size() || first < 0 || last > (int)t->fn.size()) return TSB_ERR_ARG;
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < n_dyn; ++i) t->dyn_cell[i] = dyn[i];
  FfiCall call = ffi().call;
  int status = TSB_OK;
  for (int a = first; a < last; ++a) {
    uint64_t ret = 0;                          // integral results are widened to a full register
    call(t->cif[a].bytes, t->fn[a], &ret, t->avalue.data() + t->arg_begin[a]);
    if ((int)ret != 0) {
      status = (int)ret;
      if (failed_at) *failed_at = a;
      break;
    }
  }
  if (host_ns)
    *host_ns = std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
  return status;
}

int tsb_tape_length(void* tape) { return tape ? (int)static_cast<Tape*>(tape)->fn.size() : 0; }

void tsb_tape_destroy(void* tape) { delete static_cast<Tape*>(tape); }

}  // extern "C"
