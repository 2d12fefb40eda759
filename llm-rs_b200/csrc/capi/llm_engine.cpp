// The engine's C entry points (see llm_engine.h). They call the Python module llm_rs_b200.capi, which
// holds the engines; the interpreter is the process's own when there is one, else the one this library was
// built against, started at the first llm_create. The interpreter's functions are looked up at run time
// (a Python process already has them; linking a second copy in would give it two interpreters).
#include "llm_engine.h"

#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <string>

#ifndef LLMRS_PY_LIB
#define LLMRS_PY_LIB "libpython3.so"
#endif
#ifndef LLMRS_PY_PATHS
#define LLMRS_PY_PATHS ""
#endif

namespace {

typedef struct _object PyObject;
typedef int PyGILState_STATE;

struct Py {
    int (*IsInitialized)();
    void (*InitializeEx)(int);
    void* (*SaveThread)();
    PyGILState_STATE (*GILEnsure)();
    void (*GILRelease)(PyGILState_STATE);
    PyObject* (*ImportModule)(const char*);
    PyObject* (*GetAttrString)(PyObject*, const char*);
    PyObject* (*CallFunction)(PyObject*, const char*, ...);
    long long (*AsLongLong)(PyObject*);
    PyObject* (*ErrOccurred)();
    void (*ErrFetch)(PyObject**, PyObject**, PyObject**);
    PyObject* (*Str)(PyObject*);
    const char* (*AsUTF8)(PyObject*);
    void (*DecRef)(PyObject*);
    int (*RunSimpleString)(const char*);
    PyObject* module = nullptr;     // llm_rs_b200.capi
    bool ready = false;
};

Py g_py;
std::mutex g_mutex;
thread_local char g_error[1024] = "";

int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return -1;
}

template <typename F>
bool sym(void* lib, const char* name, F* out) {
    *out = reinterpret_cast<F>(dlsym(lib, name));
    return *out != nullptr;
}

// Finds the interpreter's functions: in the process if it has an interpreter, else in the library it was built against.
bool load_python() {
    if (g_py.ready) return true;
    void* lib = RTLD_DEFAULT;
    if (dlsym(RTLD_DEFAULT, "Py_IsInitialized") == nullptr) {
        lib = dlopen(LLMRS_PY_LIB, RTLD_NOW | RTLD_GLOBAL);
        if (lib == nullptr) {
            fail("no Python interpreter in this process and %s cannot be loaded: %s", LLMRS_PY_LIB, dlerror());
            return false;
        }
    }
    Py& p = g_py;
    bool ok = sym(lib, "Py_IsInitialized", &p.IsInitialized) && sym(lib, "Py_InitializeEx", &p.InitializeEx) &&
              sym(lib, "PyEval_SaveThread", &p.SaveThread) && sym(lib, "PyGILState_Ensure", &p.GILEnsure) &&
              sym(lib, "PyGILState_Release", &p.GILRelease) && sym(lib, "PyImport_ImportModule", &p.ImportModule) &&
              sym(lib, "PyObject_GetAttrString", &p.GetAttrString) &&
              sym(lib, "PyObject_CallFunction", &p.CallFunction) && sym(lib, "PyLong_AsLongLong", &p.AsLongLong) &&
              sym(lib, "PyErr_Occurred", &p.ErrOccurred) && sym(lib, "PyErr_Fetch", &p.ErrFetch) &&
              sym(lib, "PyObject_Str", &p.Str) && sym(lib, "PyUnicode_AsUTF8", &p.AsUTF8) &&
              sym(lib, "Py_DecRef", &p.DecRef) && sym(lib, "PyRun_SimpleString", &p.RunSimpleString);
    if (!ok) {
        fail("the Python library lacks a function this library needs");
        return false;
    }
    if (!p.IsInitialized()) {
        p.InitializeEx(0);      // no signal handlers: the host program keeps its own
        p.SaveThread();         // release the lock that initialisation left held; every call takes it again
    }
    p.ready = true;
    return true;
}

// The Python exception that is set, as text, into the error record; clears it.
void take_python_error(const char* what) {
    PyObject *type = nullptr, *value = nullptr, *trace = nullptr;
    g_py.ErrFetch(&type, &value, &trace);
    std::string text = "unknown error";
    if (value != nullptr) {
        PyObject* s = g_py.Str(value);
        if (s != nullptr) {
            const char* c = g_py.AsUTF8(s);
            if (c != nullptr) text = c;
            g_py.DecRef(s);
        }
    }
    if (type) g_py.DecRef(type);
    if (value) g_py.DecRef(value);
    if (trace) g_py.DecRef(trace);
    fail("%s: %s", what, text.c_str());
}

struct Gil {
    PyGILState_STATE state;
    Gil() : state(g_py.GILEnsure()) {}
    ~Gil() { g_py.GILRelease(state); }
};

// Imports llm_rs_b200.capi once (with the lock held). The package lies three folders above this library.
bool load_module() {
    if (g_py.module != nullptr) return true;
    Dl_info info;
    std::string here = ".";
    if (dladdr(reinterpret_cast<void*>(&load_python), &info) && info.dli_fname) {
        here = info.dli_fname;
        for (int up = 0; up < 4; ++up) {    // <root>/llm-rs_b200/csrc/_build/lib.so -> <root>
            size_t at = here.find_last_of('/');
            here = at == std::string::npos ? "." : here.substr(0, at);
        }
    }
    std::string code = "import sys\nfor _p in reversed(r'''" LLMRS_PY_PATHS "'''.split(':')):\n"
                       "    if _p and _p not in sys.path: sys.path.insert(0, _p)\n"
                       "_r = r'''" + here + "'''\n"
                       "if _r not in sys.path: sys.path.insert(0, _r)\n";
    if (g_py.RunSimpleString(code.c_str()) != 0) {
        fail("setting up sys.path failed");
        return false;
    }
    PyObject* top = g_py.ImportModule("llm_rs_b200");
    if (top == nullptr) {
        take_python_error("importing llm_rs_b200");
        return false;
    }
    g_py.DecRef(top);
    g_py.module = g_py.ImportModule("llm_rs_b200.capi");
    if (g_py.module == nullptr) {
        take_python_error("importing llm_rs_b200.capi");
        return false;
    }
    return true;
}

}  // namespace

// Calls llm_rs_b200.capi.NAME(...) (arguments as PyObject_CallFunction takes them) and stores its integer result.
#define CALL(NAME, OUT, FMT, ...)                                                        \
    [&]() -> bool {                                                                      \
        PyObject* py_fn_ = g_py.GetAttrString(g_py.module, NAME);                        \
        if (py_fn_ == nullptr) { take_python_error(NAME); return false; }                \
        PyObject* py_res_ = g_py.CallFunction(py_fn_, FMT, __VA_ARGS__);                 \
        g_py.DecRef(py_fn_);                                                             \
        if (py_res_ == nullptr) { take_python_error(NAME); return false; }               \
        *(OUT) = g_py.AsLongLong(py_res_);                                               \
        g_py.DecRef(py_res_);                                                            \
        if (g_py.ErrOccurred()) { take_python_error(NAME); return false; }               \
        return true;                                                                     \
    }()

extern "C" {

__attribute__((visibility("default"))) const char* llm_last_error(void) { return g_error; }

__attribute__((visibility("default"))) void* llm_create(const LlmEngineConfig* c) {
    g_error[0] = 0;
    if (c == nullptr || c->model_path == nullptr) {
        fail("llm_create: a configuration with a model_path is needed");
        return nullptr;
    }
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!load_python()) return nullptr;
    }
    Gil gil;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!load_module()) return nullptr;
    }
    long long handle = 0;
    if (!CALL("create", &handle, "siisii", c->model_path, c->block_pool_size, c->page_size,
              c->dtype ? c->dtype : "", c->max_requests, c->cuda_graphs))
        return nullptr;
    return reinterpret_cast<void*>(static_cast<intptr_t>(handle));
}

__attribute__((visibility("default"))) uint64_t llm_submit(void* engine, const LlmRequest* r) {
    g_error[0] = 0;
    if (engine == nullptr || r == nullptr || r->prompt == nullptr || r->n_prompt < 1) {
        fail("llm_submit: an engine and a request with at least one prompt token are needed");
        return 0;
    }
    Gil gil;
    long long id = 0;
    if (!CALL("submit", &id, "LLifffiiKi", (long long)(intptr_t)engine, (long long)(intptr_t)r->prompt, r->n_prompt,
              (double)r->temperature, (double)r->top_p, (double)r->repetition_penalty, r->top_k, r->max_tokens,
              (unsigned long long)r->seed, r->ignore_eos))
        return 0;
    return static_cast<uint64_t>(id);
}

__attribute__((visibility("default"))) int llm_poll(void* engine, uint64_t request_id, LlmResult* out) {
    g_error[0] = 0;
    if (engine == nullptr || out == nullptr) return fail("llm_poll: an engine and a result to fill are needed");
    Gil gil;
    long long packed = 0;
    if (!CALL("poll", &packed, "LK", (long long)(intptr_t)engine, (unsigned long long)request_id)) return -1;
    out->token = static_cast<int32_t>(static_cast<uint32_t>(packed & 0xffffffffLL));
    out->finished = static_cast<int>((packed >> 32) & 1);
    out->reason = static_cast<int>((packed >> 40) & 0xff);
    return 0;
}

__attribute__((visibility("default"))) int llm_step(void* engine) {
    g_error[0] = 0;
    if (engine == nullptr) return fail("llm_step: no engine");
    Gil gil;
    long long n = 0;
    if (!CALL("step", &n, "L", (long long)(intptr_t)engine)) return -1;
    return static_cast<int>(n);
}

__attribute__((visibility("default"))) int llm_has_work(void* engine) {
    g_error[0] = 0;
    if (engine == nullptr) return fail("llm_has_work: no engine");
    Gil gil;
    long long n = 0;
    if (!CALL("has_work", &n, "L", (long long)(intptr_t)engine)) return -1;
    return static_cast<int>(n);
}

__attribute__((visibility("default"))) int llm_destroy(void* engine) {
    g_error[0] = 0;
    if (engine == nullptr) return 0;
    Gil gil;
    long long n = 0;
    if (!CALL("destroy", &n, "L", (long long)(intptr_t)engine)) return -1;
    return 0;
}

}  // extern "C"
