// The C API of gemmars_b200 (include/gemmars_b200.h): a thin layer over the library's engine.
//
// The reference's C API is a thin layer over its engine module (src/capi.rs:1-12: opaque
// handle, thread-local last error, caller-freed strings, no panic across the boundary,
// 0 stop | 1 length | 2 cancelled | -1 error).  This one has the same conventions over this
// library's engine, which is Python: the functions here take the interpreter's lock, hand their
// arguments (pointers as integers) to gemmars_b200/capi/host.py, and turn an exception into an
// error return.  In a process that has no interpreter yet (a C program), the first call starts
// one, for the Python installation that holds torch.  There is no second engine, loader or
// cache behind this API: what it loads and steps is gemmars_b200.Engine.
#include <Python.h>
#include <dlfcn.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "gemmars_b200.h"

#ifndef GB_PYTHON_EXECUTABLE
#define GB_PYTHON_EXECUTABLE "python3"
#endif
#ifndef GB_DEFAULT_HOME
#define GB_DEFAULT_HOME ""
#endif
#define GB_VERSION "0.2.0"

struct GbEngine {
  PyObject* engine;          // a gemmars_b200.Engine
  std::atomic<int> cancel;   // set by gb_engine_cancel, read by the running generation
};

namespace {

thread_local std::string g_error;

void set_error(const std::string& msg) { g_error = msg; }

// The folder that contains the package: the environment's, else the nearest folder above this
// library that has gemmars_b200/capi/host.py in it (the library is built inside the package),
// else the folder the library was built from.
std::string package_home() {
  if (const char* env = std::getenv("GEMMARS_B200_HOME")) return env;
  Dl_info info;
  if (dladdr((const void*)&set_error, &info) && info.dli_fname) {
    std::string p = info.dli_fname;
    for (int i = 0; i < 8; ++i) {
      const size_t cut = p.find_last_of('/');
      if (cut == std::string::npos || cut == 0) break;
      p.erase(cut);
      const std::string probe = p + "/gemmars_b200/capi/host.py";
      if (FILE* f = std::fopen(probe.c_str(), "r")) {
        std::fclose(f);
        return p;
      }
    }
  }
  return GB_DEFAULT_HOME;
}

std::once_flag g_start_once;
std::string g_start_error;

// Starts an interpreter if the process has none.  The thread that starts it gives the lock up
// again at once, so that every call, from any thread, takes it the same way.
void start_python() {
  if (Py_IsInitialized()) return;
  PyConfig config;
  PyConfig_InitPythonConfig(&config);
  config.install_signal_handlers = 0;
  config.parse_argv = 0;
  const char* exe = std::getenv("GEMMARS_B200_PYTHON");
  if (!exe || !*exe) exe = GB_PYTHON_EXECUTABLE;
  PyStatus st = PyConfig_SetBytesString(&config, &config.program_name, exe);
  if (!PyStatus_Exception(st)) st = PyConfig_SetBytesString(&config, &config.executable, exe);
  if (!PyStatus_Exception(st)) st = Py_InitializeFromConfig(&config);
  PyConfig_Clear(&config);
  if (PyStatus_Exception(st)) {
    g_start_error = std::string("cannot start the Python interpreter (") + exe + "): " + (st.err_msg ? st.err_msg : "unknown");
    return;
  }
  PyEval_SaveThread();
}

struct Gil {
  PyGILState_STATE state;
  Gil() : state(PyGILState_Ensure()) {}
  ~Gil() { PyGILState_Release(state); }
};

// The pending Python exception as "Type: message"; clears it.
std::string take_exception() {
  PyObject *type = nullptr, *value = nullptr, *trace = nullptr;
  PyErr_Fetch(&type, &value, &trace);
  PyErr_NormalizeException(&type, &value, &trace);
  std::string msg = "unknown error";
  if (value) {
    PyObject* s = PyObject_Str(value);
    const char* text = s ? PyUnicode_AsUTF8(s) : nullptr;
    const char* name = type ? ((PyTypeObject*)type)->tp_name : "Exception";
    msg = std::string(name) + ": " + (text ? text : "");
    Py_XDECREF(s);
    PyErr_Clear();
  }
  Py_XDECREF(type);
  Py_XDECREF(value);
  Py_XDECREF(trace);
  return msg;
}

PyObject* g_host = nullptr;   // the module gemmars_b200.capi.host (kept for the life of the process)

// With the lock held: the host module, imported on first use.
PyObject* host_module() {
  if (g_host) return g_host;
  const std::string home = package_home();
  if (!home.empty()) {
    PyObject* path = PySys_GetObject("path");   // borrowed
    PyObject* entry = PyUnicode_FromString(home.c_str());
    if (path && entry && PySequence_Contains(path, entry) == 0) PyList_Insert(path, 0, entry);
    Py_XDECREF(entry);
  }
  g_host = PyImport_ImportModule("gemmars_b200.capi.host");
  return g_host;
}

bool ready() {
  std::call_once(g_start_once, start_python);
  if (!g_start_error.empty()) {
    set_error(g_start_error);
    return false;
  }
  return true;
}

// Calls host.<name>(args...) under the lock; nullptr (with the error set) when it raised.
template <typename... Args>
PyObject* call_host(const char* name, const char* format, Args... args) {
  PyObject* host = host_module();
  if (!host) {
    set_error("cannot import gemmars_b200.capi.host: " + take_exception());
    return nullptr;
  }
  PyObject* out = PyObject_CallMethod(host, name, format, args...);
  if (!out) set_error(take_exception());
  return out;
}

char* out_string(PyObject* text) {
  const char* s = text ? PyUnicode_AsUTF8(text) : nullptr;
  if (!s) {
    set_error(text ? take_exception() : "no text");
    return nullptr;
  }
  char* copy = (char*)std::malloc(std::strlen(s) + 1);
  if (copy) std::strcpy(copy, s);
  else set_error("out of memory");
  return copy;
}

// An int result of a host call, or `error` when it raised.
int int_result(PyObject* out, int error) {
  if (!out) return error;
  const long v = PyLong_AsLong(out);
  Py_DECREF(out);
  if (v == -1 && PyErr_Occurred()) {
    set_error(take_exception());
    return error;
  }
  return (int)v;
}

typedef unsigned long long ull;

}  // namespace

extern "C" {

const char* gb_version(void) { return GB_VERSION; }

const char* gb_last_error(void) { return g_error.c_str(); }

void gb_string_free(char* s) { std::free(s); }

char* gb_devices(void) {
  if (!ready()) return nullptr;
  Gil gil;
  PyObject* out = call_host("devices", nullptr);
  char* text = out ? out_string(out) : nullptr;
  Py_XDECREF(out);
  return text;
}

GbEngine* gb_engine_load(const char* model, const char* options) {
  if (!model) {
    set_error("model is NULL");
    return nullptr;
  }
  if (!ready()) return nullptr;
  Gil gil;
  PyObject* engine = call_host("load", "ss", model, options ? options : "");
  if (!engine) return nullptr;
  GbEngine* e = new (std::nothrow) GbEngine{engine, {0}};
  if (!e) {
    Py_DECREF(engine);
    set_error("out of memory");
  }
  return e;
}

void gb_engine_free(GbEngine* e) {
  if (!e) return;
  if (Py_IsInitialized()) {
    Gil gil;
    PyObject* out = call_host("free", "O", e->engine);
    Py_XDECREF(out);
    Py_DECREF(e->engine);
  }
  delete e;
}

#define GB_ENGINE_OR(ret)            \
  if (!e) {                          \
    set_error("engine is NULL");     \
    return ret;                      \
  }                                  \
  if (!ready()) return ret;          \
  Gil gil;

int gb_engine_set(GbEngine* e, const char* key, const char* value) {
  GB_ENGINE_OR(-1)
  if (!key) {
    set_error("key is NULL");
    return -1;
  }
  return int_result(call_host("set", "Oss", e->engine, key, value ? value : ""), -1);
}

int gb_engine_open_slot(GbEngine* e) {
  GB_ENGINE_OR(-1)
  return int_result(call_host("open_slot", "O", e->engine), -1);
}

int gb_engine_close_slot(GbEngine* e, int slot) {
  GB_ENGINE_OR(-1)
  return int_result(call_host("close_slot", "Oi", e->engine, slot), -1);
}

int gb_engine_step(GbEngine* e, const GbStepItem* items, int n_items, float* logits, size_t capacity) {
  GB_ENGINE_OR(-1)
  if (n_items < 0 || (n_items > 0 && !items)) {
    set_error("items is NULL");
    return -1;
  }
  return int_result(call_host("step", "OKiKK", e->engine, (ull)(uintptr_t)items, n_items, (ull)(uintptr_t)logits, (ull)capacity), -1);
}

int gb_engine_generate(GbEngine* e, const int32_t* const* prompts, const int32_t* prompt_lens, int n, int32_t* out_tokens,
                       int out_stride, int32_t* out_lens, int32_t* out_reasons, gb_token_fn cb, void* user) {
  GB_ENGINE_OR(-1)
  if (n < 0 || (n > 0 && (!prompts || !prompt_lens || !out_lens || !out_reasons || (!out_tokens && out_stride > 0)))) {
    set_error("a prompt or result array is NULL");
    return -1;
  }
  e->cancel.store(0);
  return int_result(call_host("generate", "OKKiKiKKKKK", e->engine, (ull)(uintptr_t)prompts, (ull)(uintptr_t)prompt_lens, n,
                              (ull)(uintptr_t)out_tokens, out_stride, (ull)(uintptr_t)out_lens, (ull)(uintptr_t)out_reasons,
                              (ull)(uintptr_t)cb, (ull)(uintptr_t)user, (ull)(uintptr_t)&e->cancel), -1);
}

static int run_turn(GbEngine* e, const char* what, const int32_t* tokens, int n_tokens, int32_t* out, int capacity,
                    int32_t* out_len, gb_token_fn cb, void* user) {
  GB_ENGINE_OR(-1)
  if (n_tokens < 0 || (n_tokens > 0 && !tokens) || (capacity > 0 && !out)) {
    set_error("tokens or out is NULL");
    return -1;
  }
  e->cancel.store(0);
  return int_result(call_host(what, "OKiKiKKKK", e->engine, (ull)(uintptr_t)tokens, n_tokens, (ull)(uintptr_t)out, capacity,
                              (ull)(uintptr_t)out_len, (ull)(uintptr_t)cb, (ull)(uintptr_t)user, (ull)(uintptr_t)&e->cancel), -1);
}

int gb_engine_send(GbEngine* e, const int32_t* tokens, int n_tokens, int32_t* out, int capacity, int32_t* out_len,
                   gb_token_fn cb, void* user) {
  return run_turn(e, "send", tokens, n_tokens, out, capacity, out_len, cb, user);
}

int gb_engine_complete(GbEngine* e, const int32_t* tokens, int n_tokens, int32_t* out, int capacity, int32_t* out_len,
                       gb_token_fn cb, void* user) {
  return run_turn(e, "complete", tokens, n_tokens, out, capacity, out_len, cb, user);
}

int gb_engine_reset(GbEngine* e) {
  GB_ENGINE_OR(-1)
  return int_result(call_host("reset", "O", e->engine), -1);
}

void gb_engine_cancel(const GbEngine* e) {
  if (e) const_cast<GbEngine*>(e)->cancel.store(1);
}

char* gb_engine_info_json(GbEngine* e) {
  GB_ENGINE_OR(nullptr)
  PyObject* out = call_host("info_json", "O", e->engine);
  char* text = out ? out_string(out) : nullptr;
  Py_XDECREF(out);
  return text;
}

char* gb_engine_stats_json(GbEngine* e) {
  GB_ENGINE_OR(nullptr)
  PyObject* out = call_host("stats_json", "O", e->engine);
  char* text = out ? out_string(out) : nullptr;
  Py_XDECREF(out);
  return text;
}

}  // extern "C"
