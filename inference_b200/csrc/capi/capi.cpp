// libswb200_capi.so: the C ABI of swb200_contracts.h over the Python framework layer.
//
// The library never links libpython. If the process already hosts an interpreter (it was loaded from Python) the
// interpreter's own symbols are used; otherwise libpython is opened at run time and an interpreter is started. Every
// entry point funnels into one Python function, inference_b200.capi.dispatch(op, payload_json) -> result_json, so the
// interpreter surface used here is a dozen functions resolved by name.
#include "swb200_contracts.h"

#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

namespace {

struct PyApi {
  int (*Py_IsInitialized)();
  void (*Py_InitializeEx)(int);
  int (*PyGILState_Ensure)();
  void (*PyGILState_Release)(int);
  void* (*PyEval_SaveThread)();
  void* (*PyImport_ImportModule)(const char*);
  void* (*PyObject_GetAttrString)(void*, const char*);
  void* (*PyObject_CallFunction)(void*, const char*, ...);
  const char* (*PyUnicode_AsUTF8)(void*);
  void* (*PyErr_Occurred)();
  void (*PyErr_Print)();
  void (*PyErr_Clear)();
  void (*Py_DecRef)(void*);
  int (*PyRun_SimpleString)(const char*);
  bool ok = false;
};

PyApi g_py;
std::mutex g_mu;
thread_local std::string t_error;

template <class F>
bool bind(void* lib, const char* name, F& fn) {
  void* p = dlsym(lib ? lib : RTLD_DEFAULT, name);
  if (!p) return false;
  fn = reinterpret_cast<F>(p);
  return true;
}

bool load_python() {
  if (g_py.ok) return true;
  void* lib = nullptr;
  if (!dlsym(RTLD_DEFAULT, "Py_IsInitialized")) {
    const char* names[] = {getenv("SWB_LIBPYTHON"), "libpython3.12.so.1.0", "libpython3.12.so", "libpython3.so"};
    for (const char* n : names) {
      if (n && *n && (lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break;
    }
    if (!lib) {
      t_error = "no Python interpreter in the process and libpython could not be opened (set SWB_LIBPYTHON)";
      return false;
    }
  }
  bool ok = bind(lib, "Py_IsInitialized", g_py.Py_IsInitialized) && bind(lib, "Py_InitializeEx", g_py.Py_InitializeEx) &&
            bind(lib, "PyGILState_Ensure", g_py.PyGILState_Ensure) &&
            bind(lib, "PyGILState_Release", g_py.PyGILState_Release) &&
            bind(lib, "PyEval_SaveThread", g_py.PyEval_SaveThread) &&
            bind(lib, "PyImport_ImportModule", g_py.PyImport_ImportModule) &&
            bind(lib, "PyObject_GetAttrString", g_py.PyObject_GetAttrString) &&
            bind(lib, "PyObject_CallFunction", g_py.PyObject_CallFunction) &&
            bind(lib, "PyUnicode_AsUTF8", g_py.PyUnicode_AsUTF8) && bind(lib, "PyErr_Occurred", g_py.PyErr_Occurred) &&
            bind(lib, "PyErr_Print", g_py.PyErr_Print) && bind(lib, "PyErr_Clear", g_py.PyErr_Clear) &&
            bind(lib, "Py_DecRef", g_py.Py_DecRef) && bind(lib, "PyRun_SimpleString", g_py.PyRun_SimpleString);
  if (!ok) {
    t_error = "the Python library lacks a required symbol";
    return false;
  }
  if (!g_py.Py_IsInitialized()) {
    g_py.Py_InitializeEx(0);
    g_py.PyEval_SaveThread();   // release the GIL taken by initialisation; calls re-acquire it per entry
  }
  g_py.ok = true;
  return true;
}

// Escapes a C string into a JSON string literal.
std::string jstr(const char* s) {
  if (!s) return "null";
  std::string o = "\"";
  for (const unsigned char* p = reinterpret_cast<const unsigned char*>(s); *p; ++p) {
    switch (*p) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\r': o += "\\r"; break;
      case '\t': o += "\\t"; break;
      default:
        if (*p < 0x20) {
          char b[8];
          std::snprintf(b, sizeof b, "\\u%04x", *p);
          o += b;
        } else {
          o += static_cast<char>(*p);
        }
    }
  }
  return o + "\"";
}

char* dup_string(const std::string& s) {
  char* p = static_cast<char*>(std::malloc(s.size() + 1));
  if (p) std::memcpy(p, s.c_str(), s.size() + 1);
  return p;
}

}  // namespace

struct swb_runtime {
  void* dispatch = nullptr;   // inference_b200.capi.dispatch
  unsigned long long id = 0;
};

namespace {

// Calls dispatch(op, payload). The reply is "<status>\n<body>": body is the result JSON, or the error message.
int call(swb_runtime* rt, const char* op, const std::string& payload, std::string* body) {
  if (!rt || !rt->dispatch) {
    t_error = "runtime is not open";
    return SWB_E_INVALID;
  }
  const int gil = g_py.PyGILState_Ensure();
  int status = SWB_E_PYTHON;
  void* r = g_py.PyObject_CallFunction(rt->dispatch, "Kss", rt->id, op, payload.c_str());
  if (!r) {
    if (g_py.PyErr_Occurred()) g_py.PyErr_Print();
    g_py.PyErr_Clear();
    t_error = std::string("dispatch('") + op + "') raised";
  } else {
    const char* s = g_py.PyUnicode_AsUTF8(r);
    if (!s) {
      g_py.PyErr_Clear();
      t_error = "dispatch returned a non-string";
    } else {
      status = std::atoi(s);
      const char* nl = std::strchr(s, '\n');
      std::string rest = nl ? nl + 1 : "";
      if (status == 0) {
        if (body) *body = rest;
      } else {
        t_error = rest;
      }
    }
    g_py.Py_DecRef(r);
  }
  g_py.PyGILState_Release(gil);
  return status;
}

int call_out(swb_runtime* rt, const char* op, const std::string& payload, char** out) {
  std::string body;
  const int rc = call(rt, op, payload, &body);
  if (rc == 0 && out) *out = dup_string(body);
  return rc;
}

std::string ptr_json(const void* p) { return std::to_string(reinterpret_cast<unsigned long long>(p)); }

}  // namespace

extern "C" {

const char* swb_rt_last_error(void) { return t_error.c_str(); }
void swb_rt_free_string(char* s) { std::free(s); }

int swb_rt_open(const char* bundle, const char* package_root, swb_runtime** out) {
  if (!bundle || !out) {
    t_error = "bundle and out must not be null";
    return SWB_E_INVALID;
  }
  std::lock_guard<std::mutex> g(g_mu);
  if (!load_python()) return SWB_E_PYTHON;
  const int gil = g_py.PyGILState_Ensure();
  int rc = SWB_E_PYTHON;
  if (package_root && *package_root) {
    std::string code = "import sys\np = " + jstr(package_root) + "\nif p not in sys.path:\n    sys.path.insert(0, p)\n";
    g_py.PyRun_SimpleString(code.c_str());
  }
  void* mod = g_py.PyImport_ImportModule("inference_b200.capi");
  if (!mod) {
    if (g_py.PyErr_Occurred()) g_py.PyErr_Print();
    g_py.PyErr_Clear();
    t_error = "could not import inference_b200.capi (is package_root right?)";
  } else {
    void* fn = g_py.PyObject_GetAttrString(mod, "dispatch");
    g_py.Py_DecRef(mod);
    if (!fn) {
      g_py.PyErr_Clear();
      t_error = "inference_b200.capi has no dispatch()";
    } else {
      auto* rt = new swb_runtime();
      rt->dispatch = fn;
      g_py.PyGILState_Release(gil);
      std::string body;
      rc = call(rt, "open", "{\"bundle\": " + jstr(bundle) + "}", &body);
      if (rc == 0) {
        rt->id = std::strtoull(body.c_str(), nullptr, 10);
        *out = rt;
      } else {
        const int g2 = g_py.PyGILState_Ensure();
        g_py.Py_DecRef(fn);
        g_py.PyGILState_Release(g2);
        delete rt;
      }
      return rc;
    }
  }
  g_py.PyGILState_Release(gil);
  return rc;
}

void swb_rt_close(swb_runtime* rt) {
  if (!rt) return;
  call(rt, "close", "{}", nullptr);
  const int gil = g_py.PyGILState_Ensure();
  g_py.Py_DecRef(rt->dispatch);
  g_py.PyGILState_Release(gil);
  delete rt;
}

int swb_rt_catalog_json(swb_runtime* rt, char** out_json) { return call_out(rt, "catalog", "{}", out_json); }

int swb_text_load(swb_runtime* rt, const char* provider_id, const char* load_spec_json, uint64_t* out_handle) {
  if (!load_spec_json || !out_handle) return SWB_E_INVALID;
  std::string body;
  const int rc = call(rt, "text_load", "{\"provider_id\": " + jstr(provider_id) + ", \"spec\": " + load_spec_json + "}",
                      &body);
  if (rc == 0) *out_handle = std::strtoull(body.c_str(), nullptr, 10);
  return rc;
}

int swb_text_descriptor_json(swb_runtime* rt, uint64_t handle, char** out_json) {
  return call_out(rt, "descriptor", "{\"handle\": " + std::to_string(handle) + "}", out_json);
}

int swb_text_generate(swb_runtime* rt, uint64_t handle, const char* request_json, swb_event_cb on_event, void* user,
                      char** out_json) {
  if (!request_json) return SWB_E_INVALID;
  return call_out(rt, "text_generate",
                  "{\"handle\": " + std::to_string(handle) + ", \"request\": " + request_json + ", \"callback\": " +
                      ptr_json(reinterpret_cast<const void*>(on_event)) + ", \"user\": " + ptr_json(user) + "}",
                  out_json);
}

int swb_prepare_snapshot(swb_runtime* rt, const char* spec_json, char** out_report_json) {
  if (!spec_json) return SWB_E_INVALID;
  return call_out(rt, "prepare", std::string("{\"spec\": ") + spec_json + "}", out_report_json);
}

int swb_gen_load(swb_runtime* rt, const char* generator_id, const char* load_spec_json, uint64_t* out_handle) {
  if (!generator_id || !load_spec_json || !out_handle) return SWB_E_INVALID;
  std::string body;
  const int rc = call(rt, "gen_load", "{\"id\": " + jstr(generator_id) + ", \"spec\": " + load_spec_json + "}", &body);
  if (rc == 0) *out_handle = std::strtoull(body.c_str(), nullptr, 10);
  return rc;
}

int swb_gen_descriptor_json(swb_runtime* rt, uint64_t handle, char** out_json) {
  return call_out(rt, "descriptor", "{\"handle\": " + std::to_string(handle) + "}", out_json);
}

int swb_gen_generate(swb_runtime* rt, uint64_t handle, const char* request_json, swb_event_cb on_progress, void* user,
                     char** out_json) {
  if (!request_json) return SWB_E_INVALID;
  return call_out(rt, "gen_generate",
                  "{\"handle\": " + std::to_string(handle) + ", \"request\": " + request_json + ", \"callback\": " +
                      ptr_json(reinterpret_cast<const void*>(on_progress)) + ", \"user\": " + ptr_json(user) + "}",
                  out_json);
}

long long swb_gen_image_copy(swb_runtime* rt, uint64_t handle, int index, uint8_t* dst, size_t capacity) {
  std::string body;
  const int rc = call(rt, "gen_image_copy",
                      "{\"handle\": " + std::to_string(handle) + ", \"index\": " + std::to_string(index) +
                          ", \"dst\": " + ptr_json(dst) + ", \"capacity\": " + std::to_string(capacity) + "}",
                      &body);
  return rc == 0 ? std::strtoll(body.c_str(), nullptr, 10) : rc;
}

int swb_handle_free(swb_runtime* rt, uint64_t handle) {
  return call(rt, "free", "{\"handle\": " + std::to_string(handle) + "}", nullptr);
}

}  // extern "C"
