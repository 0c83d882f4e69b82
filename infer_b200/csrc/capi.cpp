// A C handle API over the engine (the shape the reference has no counterpart for; its tools link the C++ classes
// directly, kernels/batch_gpu.h:38-72): create an engine from a model folder or a random-weights spec, admit requests,
// run steps of (request, next tokens, wanted places), read logits, generate, destroy. For embedders that are not
// Python: a C or C++ program links this library and libpython, and never sees a Python object.
//
// The engine itself (layers from parts, cache manager, step function, scheduler) is the package's Python code driving
// the CUDA libraries; this file is the boundary. Every call takes the interpreter lock, calls one method of
// infer_b200.capi.Handle with plain integers and memory views of the caller's arrays, and turns exceptions into an
// error code plus a message (ib_api_last_error). If no interpreter runs in the process yet, the first ib_engine_create
// starts one. Calls on one handle must not overlap; different handles may be used from different threads.
//
// All functions return 0 on success and a negative code on failure unless stated otherwise.
#include <Python.h>

#include <cstdint>
#include <cstring>
#include <mutex>
#include <string>

#define IB_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_error;

struct Gil {
    PyGILState_STATE st;
    Gil() : st(PyGILState_Ensure()) {}
    ~Gil() { PyGILState_Release(st); }
};

// Records the pending Python exception as the thread's last error; returns -1.
int fail_from_python(const char* where) {
    PyObject *type = nullptr, *value = nullptr, *trace = nullptr;
    PyErr_Fetch(&type, &value, &trace);
    PyErr_NormalizeException(&type, &value, &trace);
    std::string msg = where;
    msg += ": ";
    if (type) {
        PyObject* name = PyObject_GetAttrString(type, "__name__");
        if (name) { const char* s = PyUnicode_AsUTF8(name); if (s) { msg += s; msg += ": "; } Py_DECREF(name); }
    }
    if (value) {
        PyObject* text = PyObject_Str(value);
        if (text) { const char* s = PyUnicode_AsUTF8(text); if (s) msg += s; Py_DECREF(text); }
    }
    PyErr_Clear();
    Py_XDECREF(type); Py_XDECREF(value); Py_XDECREF(trace);
    g_error = msg;
    return -1;
}

int fail(const char* msg) { g_error = msg; return -2; }

// Starts an interpreter if the process has none (a C host); releases the lock it then holds, so that Gil works alike
// in both kinds of process.
void ensure_interpreter() {
    static std::once_flag once;
    std::call_once(once, [] {
        if (!Py_IsInitialized()) {
            Py_InitializeEx(0);
            PyEval_SaveThread();
        }
    });
}

PyObject* view(const void* p, int64_t bytes, bool writable) {
    if (bytes <= 0 || !p) return PyBytes_FromStringAndSize("", 0);
    return PyMemoryView_FromMemory(reinterpret_cast<char*>(const_cast<void*>(p)), Py_ssize_t(bytes), writable ? PyBUF_WRITE : PyBUF_READ);
}

// Calls handle.<method>(*args) (args: a new reference to a tuple, consumed); returns a new reference or null.
PyObject* call(PyObject* handle, const char* method, PyObject* args) {
    if (!args) return nullptr;
    PyObject* fn = PyObject_GetAttrString(handle, method);
    if (!fn) { Py_DECREF(args); return nullptr; }
    PyObject* res = PyObject_CallObject(fn, args);
    Py_DECREF(fn);
    Py_DECREF(args);
    return res;
}

int64_t sum32(const int32_t* a, int n) {
    int64_t s = 0;
    for (int i = 0; i < n; i++) s += a[i] > 0 ? a[i] : 0;
    return s;
}

}  // namespace

struct ib_engine {
    PyObject* handle;
};

IB_API const char* ib_api_last_error(void) { return g_error.c_str(); }

// model_dir: a folder with config.json and model.safetensors, or null with random_spec: a preset name, a path to a
// config.json, or a JSON object of config.json keys (weights drawn from weights_seed). dtype: "bfloat16" or "float32".
// slots: live requests; max_seq: longest request; kv_blocks: pages of 16 positions in the cache pool (0: slots x
// max_seq positions); chunk: most tokens of one scheduler step in ib_engine_generate. Returns null on failure.
IB_API ib_engine* ib_engine_create(const char* model_dir, const char* random_spec, uint64_t weights_seed, const char* dtype,
                                   int slots, int max_seq, int kv_blocks, int chunk) {
    ensure_interpreter();
    Gil gil;
    PyObject* mod = PyImport_ImportModule("infer_b200.capi");
    if (!mod) { fail_from_python("ib_engine_create (import infer_b200.capi; is the package on sys.path / PYTHONPATH?)"); return nullptr; }
    PyObject* cls = PyObject_GetAttrString(mod, "Handle");
    Py_DECREF(mod);
    if (!cls) { fail_from_python("ib_engine_create"); return nullptr; }
    PyObject* args = Py_BuildValue("(zzKsiiii)", model_dir, random_spec, (unsigned long long)weights_seed,
                                   dtype ? dtype : "bfloat16", slots, max_seq, kv_blocks, chunk);
    PyObject* obj = args ? PyObject_CallObject(cls, args) : nullptr;
    Py_XDECREF(args);
    Py_DECREF(cls);
    if (!obj) { fail_from_python("ib_engine_create"); return nullptr; }
    ib_engine* e = new ib_engine{obj};
    return e;
}

IB_API void ib_engine_destroy(ib_engine* e) {
    if (!e) return;
    {
        Gil gil;
        PyObject* r = call(e->handle, "close", PyTuple_New(0));
        if (!r) PyErr_Clear();
        Py_XDECREF(r);
        Py_DECREF(e->handle);
    }
    delete e;
}

// Vocabulary size (the length of a row of logits), or a negative code.
IB_API int64_t ib_engine_vocab_size(ib_engine* e) {
    if (!e) return fail("ib_engine_vocab_size: null handle");
    Gil gil;
    PyObject* r = call(e->handle, "vocab_size", PyTuple_New(0));
    if (!r) return fail_from_python("ib_engine_vocab_size");
    const int64_t v = PyLong_AsLongLong(r);
    Py_DECREF(r);
    return v;
}

IB_API int ib_engine_add_request(ib_engine* e, int64_t request_id) {
    if (!e) return fail("ib_engine_add_request: null handle");
    Gil gil;
    PyObject* r = call(e->handle, "add_request", Py_BuildValue("(L)", (long long)request_id));
    if (!r) return fail_from_python("ib_engine_add_request");
    Py_DECREF(r);
    return 0;
}

// The request's pages and state slot go back to the pools.
IB_API int ib_engine_end_request(ib_engine* e, int64_t request_id) {
    if (!e) return fail("ib_engine_end_request: null handle");
    Gil gil;
    PyObject* r = call(e->handle, "end_request", Py_BuildValue("(L)", (long long)request_id));
    if (!r) return fail_from_python("ib_engine_end_request");
    Py_DECREF(r);
    return 0;
}

// One step: entry i is request ids[i] with its next n_tokens[i] tokens (all entries' tokens back to back in `tokens`)
// and n_want[i] wanted places among them (back to back in `want`, indices into the entry's own tokens). All entries
// run as one batch from the cache. With ran == null the step is all or nothing (a negative code if the pages for all
// entries together are not free; nothing changed). With ran != null, entries that cannot get their pages or would
// pass the sequence limit are left out (ran[i] = 0, their requests untouched) and the others run (ran[i] = 1).
// The logits of the wanted places of the entries that ran stay on the device until the next step; read them with
// ib_engine_get_logits. Returns the number of logit rows, or a negative code.
IB_API int64_t ib_engine_step(ib_engine* e, int n_entries, const int64_t* ids, const int32_t* n_tokens, const int32_t* tokens,
                              const int32_t* n_want, const int32_t* want, int32_t* ran) {
    if (!e) return fail("ib_engine_step: null handle");
    if (n_entries < 0 || (n_entries > 0 && (!ids || !n_tokens || !tokens || !n_want))) return fail("ib_engine_step: null array");
    const int64_t total_tokens = sum32(n_tokens, n_entries), total_want = sum32(n_want, n_entries);
    if (total_want > 0 && !want) return fail("ib_engine_step: places are wanted but `want` is null");
    Gil gil;
    PyObject* args = Py_BuildValue("(iNNNNNN)", n_entries, view(ids, int64_t(n_entries) * 8, false), view(n_tokens, int64_t(n_entries) * 4, false),
                                   view(tokens, total_tokens * 4, false), view(n_want, int64_t(n_entries) * 4, false),
                                   view(want, total_want * 4, false), ran ? view(ran, int64_t(n_entries) * 4, true) : (Py_INCREF(Py_None), Py_None));
    PyObject* r = call(e->handle, "step", args);
    if (!r) return fail_from_python("ib_engine_step");
    const int64_t rows = PyLong_AsLongLong(r);
    Py_DECREF(r);
    return rows;
}

// Copies the last step's logits, float [rows, vocab] in the order of the entries and of their wanted places, to host
// memory. capacity_floats must be at least rows * vocab. Returns the number of rows, or a negative code.
IB_API int64_t ib_engine_get_logits(ib_engine* e, float* out, int64_t capacity_floats) {
    if (!e) return fail("ib_engine_get_logits: null handle");
    if (!out && capacity_floats > 0) return fail("ib_engine_get_logits: null buffer");
    Gil gil;
    PyObject* r = call(e->handle, "copy_logits", Py_BuildValue("(N)", view(out, capacity_floats * 4, true)));
    if (!r) return fail_from_python("ib_engine_get_logits");
    const int64_t rows = PyLong_AsLongLong(r);
    Py_DECREF(r);
    return rows;
}

// Generates up to max_new tokens for each of n_prompts prompts (lengths in prompt_lens, token ids back to back in
// prompt_tokens) under continuous batching. temperature 0 = greedy; otherwise seeded sampling (sample_seed). eos_id < 0:
// never stop on a token. out_tokens is [n_prompts, max_new]; out_lens[i] receives how many were generated for prompt i
// (the eos token, if hit, included).
IB_API int ib_engine_generate(ib_engine* e, int n_prompts, const int32_t* prompt_lens, const int32_t* prompt_tokens, int max_new,
                              float temperature, uint64_t sample_seed, int64_t eos_id, int32_t* out_tokens, int32_t* out_lens) {
    if (!e) return fail("ib_engine_generate: null handle");
    if (n_prompts < 0 || max_new < 0 || (n_prompts > 0 && (!prompt_lens || !prompt_tokens || !out_tokens || !out_lens)))
        return fail("ib_engine_generate: bad arguments");
    const int64_t total = sum32(prompt_lens, n_prompts);
    Gil gil;
    PyObject* args = Py_BuildValue("(iNNidKLNN)", n_prompts, view(prompt_lens, int64_t(n_prompts) * 4, false), view(prompt_tokens, total * 4, false),
                                   max_new, double(temperature), (unsigned long long)sample_seed, (long long)eos_id,
                                   view(out_tokens, int64_t(n_prompts) * max_new * 4, true), view(out_lens, int64_t(n_prompts) * 4, true));
    PyObject* r = call(e->handle, "generate", args);
    if (!r) return fail_from_python("ib_engine_generate");
    Py_DECREF(r);
    return 0;
}
