// The C API of oracle_engine_b200 (oe.h): a thin layer over the library's Python engine.
//
// It owns no model, cache or kernel.  Each call takes the interpreter's lock, calls one function of
// oracle_engine_b200.capi.bridge with integers and strings (arrays go by address and are read and
// written there), and turns a Python exception into the calling thread's oe_last_error().  Loaded
// into a Python process it uses that process's interpreter; in a C or C++ program it starts one.
#include <Python.h>

#include <dlfcn.h>

#include <cstdarg>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <string>

#include "oe.h"

struct oe_engine {
    PyObject* engine;      // the Python Engine (owned reference)
};

namespace {

thread_local std::string g_error;
std::once_flag g_once;
bool g_python_ok = false;
std::string g_python_error;
PyObject* g_bridge = nullptr;      // the module oracle_engine_b200.capi.bridge (owned, kept for the process)

// The folder that holds the package: this library lies in <root>/oracle_engine_b200/capi/_build/.
std::string package_root() {
    Dl_info info;
    if (!dladdr(reinterpret_cast<void*>(&package_root), &info) || !info.dli_fname) return "";
    std::string path = info.dli_fname;
    char* real = realpath(path.c_str(), nullptr);
    if (real) { path = real; free(real); }
    for (int up = 0; up < 4; up++) {
        const size_t cut = path.find_last_of('/');
        if (cut == std::string::npos) return "";
        path.erase(cut);
    }
    return path;
}

void start_python() {
    if (!Py_IsInitialized()) {
        PyConfig config;
        PyConfig_InitPythonConfig(&config);
        const char* exe = getenv("OE_PYTHON");
        PyStatus st = PyConfig_SetBytesString(&config, &config.program_name, (exe && *exe) ? exe : "python3");
        if (!PyStatus_Exception(st)) st = Py_InitializeFromConfig(&config);
        PyConfig_Clear(&config);
        if (PyStatus_Exception(st)) {
            g_python_error = std::string("the Python interpreter did not start: ") + (st.err_msg ? st.err_msg : "?");
            return;
        }
        PyEval_SaveThread();          // calls take the lock themselves, from any thread
    }
    PyGILState_STATE gil = PyGILState_Ensure();
    const std::string root = package_root();
    PyObject* sys_path = PySys_GetObject("path");          // borrowed
    if (sys_path && !root.empty()) {
        PyObject* entry = PyUnicode_FromString(root.c_str());
        if (entry && !PySequence_Contains(sys_path, entry)) PyList_Insert(sys_path, 0, entry);
        Py_XDECREF(entry);
    }
    g_bridge = PyImport_ImportModule("oracle_engine_b200.capi.bridge");
    if (!g_bridge) {
        PyObject *type, *value, *trace;
        PyErr_Fetch(&type, &value, &trace);
        PyObject* text = value ? PyObject_Str(value) : nullptr;
        g_python_error = std::string("oracle_engine_b200 could not be imported: ") +
                         (text && PyUnicode_Check(text) ? PyUnicode_AsUTF8(text) : "?");
        Py_XDECREF(text); Py_XDECREF(type); Py_XDECREF(value); Py_XDECREF(trace);
    } else {
        g_python_ok = true;
    }
    PyGILState_Release(gil);
}

bool ready() {
    std::call_once(g_once, start_python);
    if (!g_python_ok) g_error = g_python_error;
    return g_python_ok;
}

// The pending Python exception as "Type: message" in g_error; clears it.
void keep_exception() {
    PyObject *type, *value, *trace;
    PyErr_Fetch(&type, &value, &trace);
    PyErr_NormalizeException(&type, &value, &trace);
    std::string msg;
    if (type) {
        PyObject* name = PyObject_GetAttrString(type, "__name__");
        if (name && PyUnicode_Check(name)) msg = PyUnicode_AsUTF8(name);
        Py_XDECREF(name);
        PyErr_Clear();
    }
    PyObject* text = value ? PyObject_Str(value) : nullptr;
    if (text && PyUnicode_Check(text)) msg += std::string(msg.empty() ? "" : ": ") + PyUnicode_AsUTF8(text);
    PyErr_Clear();
    Py_XDECREF(text); Py_XDECREF(type); Py_XDECREF(value); Py_XDECREF(trace);
    g_error = msg.empty() ? "unknown error" : msg;
}

// bridge.<name>(*args built from `format`); a new reference, or nullptr with g_error set.  Lock held.
PyObject* call(const char* name, const char* format, ...) {
    va_list va;
    va_start(va, format);
    PyObject* args = Py_VaBuildValue(format, va);
    va_end(va);
    PyObject* fn = args ? PyObject_GetAttrString(g_bridge, name) : nullptr;
    PyObject* out = fn ? PyObject_CallObject(fn, args) : nullptr;
    Py_XDECREF(fn);
    Py_XDECREF(args);
    if (!out) keep_exception();
    return out;
}

// An integer result; `fail` when the call failed.
long long as_int(PyObject* out, long long fail) {
    if (!out) return fail;
    const long long v = PyLong_AsLongLong(out);
    Py_DECREF(out);
    if (v == -1 && PyErr_Occurred()) { keep_exception(); return fail; }
    return v;
}

struct Lock {
    PyGILState_STATE state;
    Lock() : state(PyGILState_Ensure()) {}
    ~Lock() { PyGILState_Release(state); }
};

bool usable(oe_engine* e) {
    if (e && e->engine) return true;
    g_error = "the engine handle is null";
    return false;
}

}  // namespace

extern "C" {

void oe_default_params(oe_gen_params* p) {
    if (!p) return;
    p->n_predict = 256; p->temperature = 0.7f; p->top_p = 0.9f; p->top_k = 40;
    p->repeat_penalty = 1.15f; p->repeat_last_n = 64; p->seed = 0; p->ignore_eos = 0;
    p->batch_size = 0; p->max_step_tokens = 0;
}

const char* oe_last_error(void) { return g_error.c_str(); }

oe_engine* oe_load(const char* model_dir, const char* dtype, long long max_tokens) {
    if (!model_dir || !dtype) { g_error = "model_dir and dtype must be given"; return nullptr; }
    if (!ready()) return nullptr;
    Lock lock;
    PyObject* engine = call("load", "(ssL)", model_dir, dtype, max_tokens);
    if (!engine) return nullptr;
    oe_engine* e = new oe_engine{engine};
    return e;
}

void oe_free(oe_engine* e) {
    if (!e) return;
    if (e->engine && g_python_ok) {
        Lock lock;
        Py_DECREF(e->engine);
    }
    delete e;
}

int oe_vocab_size(oe_engine* e) {
    if (!usable(e) || !ready()) return -1;
    Lock lock;
    return (int)as_int(call("vocab_size", "(O)", e->engine), -1);
}

int oe_max_seq_len(oe_engine* e) {
    if (!usable(e) || !ready()) return -1;
    Lock lock;
    return (int)as_int(call("max_seq_len", "(O)", e->engine), -1);
}

int oe_alloc_slot(oe_engine* e) {
    if (!usable(e) || !ready()) return -1;
    Lock lock;
    return (int)as_int(call("alloc_slot", "(O)", e->engine), -1);
}

int oe_free_slot(oe_engine* e, int slot) {
    if (!usable(e) || !ready()) return -1;
    Lock lock;
    return (int)as_int(call("free_slot", "(Oi)", e->engine, slot), -1);
}

int oe_step(oe_engine* e, int n_seqs, const int* slots, const int* tokens, const int* q_lens, const int* want,
            const int* n_want, float* logits_out) {
    if (!usable(e) || !ready()) return -1;
    Lock lock;
    return (int)as_int(call("step", "(OiKKKKKK)", e->engine, n_seqs, (unsigned long long)(uintptr_t)slots,
                            (unsigned long long)(uintptr_t)tokens, (unsigned long long)(uintptr_t)q_lens,
                            (unsigned long long)(uintptr_t)want, (unsigned long long)(uintptr_t)n_want,
                            (unsigned long long)(uintptr_t)logits_out), -1);
}

int oe_generate(oe_engine* e, int n_prompts, const int* tokens, const int* lens, const oe_gen_params* p,
                int* out_tokens, int* out_lens, oe_token_callback on_token, void* user) {
    if (!usable(e) || !ready()) return -1;
    oe_gen_params defaults;
    oe_default_params(&defaults);
    if (!p) p = &defaults;
    if (p->n_predict < 0) { g_error = "n_predict must be >= 0"; return -1; }
    Lock lock;
    return (int)as_int(call("generate", "(OiKKidfidiLiiiKKKK)", e->engine, n_prompts,
                            (unsigned long long)(uintptr_t)tokens, (unsigned long long)(uintptr_t)lens,
                            p->n_predict, (double)p->temperature, p->top_p, p->top_k, (double)p->repeat_penalty,
                            p->repeat_last_n, p->seed, p->ignore_eos, p->batch_size, p->max_step_tokens,
                            (unsigned long long)(uintptr_t)out_tokens, (unsigned long long)(uintptr_t)out_lens,
                            (unsigned long long)(uintptr_t)on_token, (unsigned long long)(uintptr_t)user), -1);
}

}  // extern "C"
