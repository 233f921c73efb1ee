// The C interface of vlrf_b200.h.  The engine's host side is Python; this library hosts an interpreter for it (or
// joins the one of the process that loaded it) and forwards every call to vlrf_b200/capi/bridge.py, which hands
// over to the package's own entry point.  Nothing is computed here: no forward pass, no cache, no loader.
//
// Built with the paths of the checkout and of the interpreter that built it; VLRF_B200_HOME and VLRF_B200_PYTHON
// override them at run time.
#include "vlrf_b200.h"

#include <Python.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#ifndef VLRF_B200_DEFAULT_HOME
#define VLRF_B200_DEFAULT_HOME ""
#endif
#ifndef VLRF_B200_DEFAULT_PYTHON
#define VLRF_B200_DEFAULT_PYTHON ""
#endif

struct VlrfB200Model_t { long handle; uint32_t seed; };

namespace {

thread_local char g_error[1024] = "";
std::once_flag g_started;
bool g_ok = false;
PyObject* g_bridge = nullptr;

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

std::string python_error() {
    PyObject *type = nullptr, *value = nullptr, *trace = nullptr;
    PyErr_Fetch(&type, &value, &trace);
    PyErr_NormalizeException(&type, &value, &trace);
    std::string text = "unknown Python error";
    if (value != nullptr) {
        PyObject* s = PyObject_Str(value);
        if (s != nullptr) {
            const char* c = PyUnicode_AsUTF8(s);
            if (c != nullptr) text = c;
            Py_DECREF(s);
        }
    }
    Py_XDECREF(type); Py_XDECREF(value); Py_XDECREF(trace);
    return text;
}

void start_python() {
    const char* home = getenv("VLRF_B200_HOME");
    if (home == nullptr || !*home) home = VLRF_B200_DEFAULT_HOME;
    bool own = false;
    if (!Py_IsInitialized()) {
        const char* exe = getenv("VLRF_B200_PYTHON");
        if (exe == nullptr || !*exe) exe = VLRF_B200_DEFAULT_PYTHON;
        PyConfig config;
        PyConfig_InitPythonConfig(&config);
        config.install_signal_handlers = 0;
        config.parse_argv = 0;
        if (*exe) PyConfig_SetBytesString(&config, &config.program_name, exe);   // its pyvenv.cfg, if any, gives the packages
        PyStatus st = Py_InitializeFromConfig(&config);
        PyConfig_Clear(&config);
        if (PyStatus_Exception(st)) {
            set_error("the Python interpreter did not start: %s", st.err_msg ? st.err_msg : "no message");
            return;
        }
        own = true;
    }
    PyGILState_STATE gil = own ? PyGILState_UNLOCKED : PyGILState_Ensure();
    if (*home) {
        PyObject* path = PySys_GetObject("path");        // borrowed
        PyObject* entry = PyUnicode_FromString(home);
        if (path != nullptr && entry != nullptr && !PySequence_Contains(path, entry)) PyList_Insert(path, 0, entry);
        Py_XDECREF(entry);
    }
    g_bridge = PyImport_ImportModule("vlrf_b200.capi.bridge");
    if (g_bridge == nullptr) {
        set_error("cannot import vlrf_b200.capi.bridge (VLRF_B200_HOME=%s): %s", home, python_error().c_str());
    } else {
        g_ok = true;
    }
    if (own) PyEval_SaveThread();        // the interpreter stays; calls take the lock when they need it
    else PyGILState_Release(gil);
}

bool ready() {
    std::call_once(g_started, start_python);
    if (!g_ok && !g_error[0]) set_error("the library could not start its Python side (see the first call's error)");
    return g_ok;
}

// Calls bridge.<name>(args…) → (status, value); returns the status, keeps the message of a failure, and hands the
// value (a new reference, or null) to `value_out` when that is wanted.
VlrfB200Status call_bridge(const char* name, PyObject** value_out, const char* fmt, ...) {
    if (!ready()) return VLRF_B200_ERR_DEVICE;
    PyGILState_STATE gil = PyGILState_Ensure();
    VlrfB200Status status = VLRF_B200_ERR_UNKNOWN;
    PyObject* fn = PyObject_GetAttrString(g_bridge, name);
    PyObject* args = nullptr;
    if (fn != nullptr) {
        va_list ap;
        va_start(ap, fmt);
        args = Py_VaBuildValue(fmt, ap);
        va_end(ap);
    }
    PyObject* result = (fn != nullptr && args != nullptr) ? PyObject_CallObject(fn, args) : nullptr;
    if (result == nullptr || !PyTuple_Check(result) || PyTuple_Size(result) != 2) {
        set_error("%s: %s", name, PyErr_Occurred() ? python_error().c_str() : "the bridge returned no (status, value)");
    } else {
        status = (VlrfB200Status)PyLong_AsLong(PyTuple_GetItem(result, 0));
        PyObject* value = PyTuple_GetItem(result, 1);       // borrowed
        if (status != VLRF_B200_OK) {
            const char* msg = PyUnicode_Check(value) ? PyUnicode_AsUTF8(value) : nullptr;
            set_error("%s", msg ? msg : "no message");
        } else if (value_out != nullptr) {
            Py_INCREF(value);
            *value_out = value;
        }
    }
    Py_XDECREF(result); Py_XDECREF(args); Py_XDECREF(fn);
    PyGILState_Release(gil);
    return status;
}

VlrfB200Status call_for_long(const char* name, long long* out, const char* fmt, long a, long b = 0) {
    PyObject* value = nullptr;
    VlrfB200Status st = call_bridge(name, &value, fmt, a, b);
    if (st == VLRF_B200_OK && value != nullptr) {
        PyGILState_STATE gil = PyGILState_Ensure();
        *out = PyLong_AsLongLong(value);
        Py_DECREF(value);
        PyGILState_Release(gil);
    }
    return st;
}

#define NEED(cond) do { if (!(cond)) { set_error("%s: invalid argument (%s)", __func__, #cond); return VLRF_B200_ERR_INVALID_ARG; } } while (0)
#define ADDR(p) ((unsigned long long)(uintptr_t)(p))

}  // namespace

extern "C" {

const char* vlrf_b200_status_str(VlrfB200Status s) {
    switch (s) {
        case VLRF_B200_OK: return "ok";
        case VLRF_B200_ERR_INVALID_ARG: return "invalid argument";
        case VLRF_B200_ERR_OUT_OF_MEMORY: return "out of memory";
        case VLRF_B200_ERR_IO: return "file cannot be read";
        case VLRF_B200_ERR_BAD_MODEL: return "not a model this library can load";
        case VLRF_B200_ERR_NOT_INIT: return "the handle holds no model";
        case VLRF_B200_ERR_CTX_FULL: return "the cache or the model's positions are used up";
        case VLRF_B200_ERR_DEVICE: return "no usable CUDA device or kernel library";
        default: return "unknown error";
    }
}

const char* vlrf_b200_last_error(void) { return g_error; }
const char* vlrf_b200_version(void) { return "vlrf_b200 0.2 (C interface over the Python engine)"; }

VlrfB200Model vlrf_b200_create_model(void) {
    long long handle = 0;
    PyObject* value = nullptr;
    if (call_bridge("create", &value, "()") != VLRF_B200_OK || value == nullptr) return nullptr;
    PyGILState_STATE gil = PyGILState_Ensure();
    handle = PyLong_AsLongLong(value);
    Py_DECREF(value);
    PyGILState_Release(gil);
    VlrfB200Model m = new VlrfB200Model_t;
    m->handle = (long)handle;
    m->seed = 42;
    return m;
}

void vlrf_b200_free_model(VlrfB200Model m) {
    if (m == nullptr) return;
    call_bridge("free", nullptr, "(l)", m->handle);
    delete m;
}

static VlrfB200Status not_init_if_lookup(VlrfB200Status st) {
    return (st == VLRF_B200_ERR_UNKNOWN && strstr(g_error, "LookupError") != nullptr) ? VLRF_B200_ERR_NOT_INIT : st;
}

VlrfB200Status vlrf_b200_load_dir(VlrfB200Model m, const char* dir, const char* dtype, int32_t max_tokens, int32_t n_slots) {
    NEED(m != nullptr && dir != nullptr && max_tokens >= 0 && n_slots >= 0);
    return call_bridge("load_dir", nullptr, "(lssii)", m->handle, dir, dtype ? dtype : "bfloat16", (int)max_tokens, (int)n_slots);
}

VlrfB200Status vlrf_b200_init_random(VlrfB200Model m, const char* config, uint32_t seed, const char* dtype, int32_t max_tokens,
                                     int32_t n_slots) {
    NEED(m != nullptr && config != nullptr && max_tokens >= 0 && n_slots >= 0);
    return call_bridge("init_random", nullptr, "(lsIsii)", m->handle, config, (unsigned)seed, dtype ? dtype : "bfloat16",
                       (int)max_tokens, (int)n_slots);
}

VlrfB200Status vlrf_b200_get_info(VlrfB200Model m, VlrfB200ModelInfo* out) {
    NEED(m != nullptr && out != nullptr);
    return not_init_if_lookup(call_bridge("get_info", nullptr, "(lK)", m->handle, ADDR(out)));
}

VlrfB200Status vlrf_b200_get_config(VlrfB200Model m, char* out, int32_t cap) {
    NEED(m != nullptr && out != nullptr && cap > 0);
    return not_init_if_lookup(call_bridge("get_config", nullptr, "(lKi)", m->handle, ADDR(out), (int)cap));
}

VlrfB200Status vlrf_b200_model_summary(VlrfB200Model m, char* out, int32_t cap) {
    NEED(m != nullptr && out != nullptr && cap > 0);
    return not_init_if_lookup(call_bridge("model_summary", nullptr, "(lKi)", m->handle, ADDR(out), (int)cap));
}

int64_t vlrf_b200_kv_cache_bytes(VlrfB200Model m) {
    if (m == nullptr) return -1;
    long long v = -1;
    return call_for_long("kv_cache_bytes", &v, "(l)", m->handle) == VLRF_B200_OK ? v : -1;
}

void vlrf_b200_default_sampling(VlrfB200Sampling* p) {
    if (p == nullptr) return;
    memset(p, 0, sizeof(*p));
    p->max_new_tokens = 128; p->temperature = 0.8f; p->top_p = 0.9f; p->top_k = 50; p->use_sampling = 1;
    p->repetition_penalty = 1.0f; p->seed = 42; p->n_stop_ids = -1;
}

VlrfB200Status vlrf_b200_set_seed(VlrfB200Model m, uint32_t seed) {
    NEED(m != nullptr);
    m->seed = seed;
    return VLRF_B200_OK;
}

VlrfB200Status vlrf_b200_generate_ids(VlrfB200Model m, const int32_t* ids, const int32_t* lens, int32_t n_prompts,
                                      const VlrfB200Sampling* params, int32_t n_params, int32_t* out_ids, int32_t out_cap,
                                      int32_t* out_lens, int32_t* out_reasons) {
    NEED(m != nullptr && lens != nullptr && n_prompts > 0 && out_lens != nullptr && out_cap >= 0 && (out_ids != nullptr || out_cap == 0));
    VlrfB200Sampling fallback;
    if (params == nullptr) {
        vlrf_b200_default_sampling(&fallback);
        fallback.seed = m->seed;
        params = &fallback;
        n_params = 1;
    }
    return not_init_if_lookup(call_bridge("generate_ids", nullptr, "(lKKiKiKiKK)", m->handle, ADDR(ids), ADDR(lens), (int)n_prompts,
                                          ADDR(params), (int)n_params, ADDR(out_ids), (int)out_cap, ADDR(out_lens), ADDR(out_reasons)));
}

VlrfB200Status vlrf_b200_get_logits(VlrfB200Model m, const int32_t* ids, int32_t n, float* out) {
    NEED(m != nullptr && ids != nullptr && n > 0 && out != nullptr);
    return not_init_if_lookup(call_bridge("get_logits", nullptr, "(lKiK)", m->handle, ADDR(ids), (int)n, ADDR(out)));
}

VlrfB200Status vlrf_b200_start_sequence(VlrfB200Model m, int32_t* out_slot) {
    NEED(m != nullptr && out_slot != nullptr);
    long long v = -1;
    VlrfB200Status st = not_init_if_lookup(call_for_long("start_sequence", &v, "(l)", m->handle));
    if (st == VLRF_B200_OK) *out_slot = (int32_t)v;
    return st;
}

VlrfB200Status vlrf_b200_reset_slot(VlrfB200Model m, int32_t slot) {
    NEED(m != nullptr);
    return not_init_if_lookup(call_bridge("reset_slot", nullptr, "(li)", m->handle, (int)slot));
}

int32_t vlrf_b200_context_length(VlrfB200Model m, int32_t slot) {
    if (m == nullptr) return -1;
    long long v = -1;
    return call_for_long("context_length", &v, "(ll)", m->handle, (long)slot) == VLRF_B200_OK ? (int32_t)v : -1;
}

VlrfB200Status vlrf_b200_step(VlrfB200Model m, int32_t n_entries, const int32_t* slots, const int32_t* counts, const int32_t* tokens,
                              const int32_t* want_counts, const int32_t* want, float* out, int32_t out_rows_cap) {
    NEED(m != nullptr && n_entries > 0 && slots != nullptr && counts != nullptr && tokens != nullptr && want_counts != nullptr && out_rows_cap >= 0);
    return not_init_if_lookup(call_bridge("step", nullptr, "(liKKKKKKi)", m->handle, (int)n_entries, ADDR(slots), ADDR(counts),
                                          ADDR(tokens), ADDR(want_counts), ADDR(want), ADDR(out), (int)out_rows_cap));
}

VlrfB200Status vlrf_b200_presets(char* out, int32_t cap) {
    NEED(out != nullptr && cap > 0);
    return call_bridge("presets", nullptr, "(Ki)", ADDR(out), (int)cap);
}

VlrfB200Status vlrf_b200_describe_dir(const char* dir, char* out, int32_t cap) {
    NEED(dir != nullptr && out != nullptr && cap > 0);
    return call_bridge("describe_dir", nullptr, "(sKi)", dir, ADDR(out), (int)cap);
}

VlrfB200Status vlrf_b200_write_random_model(const char* config, uint32_t seed, const char* out_dir) {
    NEED(config != nullptr && out_dir != nullptr);
    return call_bridge("write_random_model", nullptr, "(sIs)", config, (unsigned)seed, out_dir);
}

}  // extern "C"
