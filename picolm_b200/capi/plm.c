/* The C face of picolm_b200 (plm.h): every function forwards to picolm_b200/capi/host.py inside an
 * interpreter that this library starts in the calling process on first use, or joins if the process is a
 * Python process already.  No model code lives here: the engine behind the calls is the library's own.
 *
 * The interpreter is started for the Python executable named by $PLM_PYTHON (default: the one the library
 * was built with), so that the executable's environment (its site-packages, where torch lives) is the
 * interpreter's; the package is found under $PLM_PACKAGE_ROOT (default: where it was built).
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <pthread.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "plm.h"

#ifndef PLM_DEFAULT_PYTHON
#define PLM_DEFAULT_PYTHON "python3"
#endif
#ifndef PLM_DEFAULT_ROOT
#define PLM_DEFAULT_ROOT "."
#endif

struct plm_model { long handle; };
struct plm_ctx { long handle; long model; };

static __thread char t_error[2048];
static pthread_mutex_t g_init_lock = PTHREAD_MUTEX_INITIALIZER;
static int g_ready = 0;
static PyObject* g_host = NULL; /* the module picolm_b200.capi.host */

static void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

const char* plm_last_error(void) { return t_error; }

plm_sampling plm_sampling_default(void) {
    plm_sampling s = {0.8f, 40, 0.9f, 0.05f, 42};
    return s;
}

/* The pending Python exception as this thread's error text; returns the API's code for it. */
static int take_exception(void) {
    PyObject *type = NULL, *value = NULL, *tb = NULL;
    int code = PLM_API_ERROR;
    PyErr_Fetch(&type, &value, &tb);
    PyErr_NormalizeException(&type, &value, &tb);
    if (value != NULL) {
        PyObject* text = PyObject_Str(value);
        const char* name = type ? ((PyTypeObject*)type)->tp_name : "error";
        set_error("%s: %s", name, text ? PyUnicode_AsUTF8(text) : "(no message)");
        Py_XDECREF(text);
        if (g_host != NULL) {
            PyObject* c = PyObject_CallMethod(g_host, "classify", "O", value);
            if (c != NULL) {
                code = (int)PyLong_AsLong(c);
                Py_DECREF(c);
            }
            PyErr_Clear();
        }
    } else {
        set_error("unknown failure inside the interpreter");
    }
    Py_XDECREF(type);
    Py_XDECREF(value);
    Py_XDECREF(tb);
    return code;
}

/* Start or join the interpreter and import the host module.  Returns 0, or a code with the error set.
 * On success the caller holds the GIL through *gil. */
static int enter(PyGILState_STATE* gil) {
    pthread_mutex_lock(&g_init_lock);
    if (!g_ready && !Py_IsInitialized()) {
        PyConfig config;
        PyConfig_InitPythonConfig(&config);
        const char* exe = getenv("PLM_PYTHON");
        if (exe == NULL || !*exe) exe = PLM_DEFAULT_PYTHON;
        PyStatus st = PyConfig_SetBytesString(&config, &config.program_name, exe);
        if (!PyStatus_Exception(st)) {
            config.install_signal_handlers = 0;
            config.parse_argv = 0;
            st = Py_InitializeFromConfig(&config);
        }
        PyConfig_Clear(&config);
        if (PyStatus_Exception(st)) {
            set_error("the Python interpreter could not be started for %s: %s", exe, st.err_msg ? st.err_msg : "?");
            pthread_mutex_unlock(&g_init_lock);
            return PLM_API_ERROR;
        }
        PyEval_SaveThread(); /* the GIL is taken again per call */
    }
    pthread_mutex_unlock(&g_init_lock); /* not held while waiting for the GIL: its holder may be in here too */
    *gil = PyGILState_Ensure();
    if (!g_ready) { /* read and written under the GIL */
        const char* root = getenv("PLM_PACKAGE_ROOT");
        if (root == NULL || !*root) root = PLM_DEFAULT_ROOT;
        PyObject* path = PySys_GetObject("path"); /* borrowed */
        PyObject* entry = PyUnicode_FromString(root);
        if (path != NULL && entry != NULL && PySequence_Contains(path, entry) == 0) PyList_Insert(path, 0, entry);
        Py_XDECREF(entry);
        g_host = PyImport_ImportModule("picolm_b200.capi.host");
        if (g_host == NULL) {
            int code = take_exception();
            PyGILState_Release(*gil);
            return code;
        }
        g_ready = 1;
    }
    t_error[0] = '\0';
    return PLM_API_OK;
}

/* A memoryview over the caller's array (None for NULL). */
static PyObject* view(const void* p, size_t bytes, int writable) {
    if (p == NULL) Py_RETURN_NONE;
    return PyMemoryView_FromMemory((char*)p, (Py_ssize_t)bytes, writable ? PyBUF_WRITE : PyBUF_READ);
}

/* Finish a call: `result` is what the host function returned (NULL: it raised). */
static int leave(PyObject* result, PyGILState_STATE gil, long* value_out) {
    int code = PLM_API_OK;
    if (result == NULL) {
        code = take_exception();
    } else {
        if (value_out != NULL && PyLong_Check(result)) *value_out = PyLong_AsLong(result);
        Py_DECREF(result);
    }
    PyGILState_Release(gil);
    return code;
}

#define NEED(cond, what)                       \
    do {                                       \
        if (!(cond)) {                         \
            set_error("%s", what);             \
            return PLM_API_BAD_ARGUMENT;       \
        }                                      \
    } while (0)

int plm_config_from_json(const char* path, char* out, size_t out_capacity) {
    NEED(path && out && out_capacity > 0, "plm_config_from_json: path and out must be given");
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    PyObject* r = PyObject_CallMethod(g_host, "config_json", "s", path);
    if (r != NULL) {
        Py_ssize_t n = 0;
        const char* text = PyUnicode_AsUTF8AndSize(r, &n);
        if (text == NULL || (size_t)n + 1 > out_capacity) {
            Py_DECREF(r);
            PyErr_Clear();
            PyGILState_Release(gil);
            set_error("plm_config_from_json: the text needs %zd bytes, out has %zu", n + 1, out_capacity);
            return PLM_API_BAD_ARGUMENT;
        }
        memcpy(out, text, (size_t)n + 1);
    }
    return leave(r, gil, NULL);
}

static int new_model(PyObject* r, PyGILState_STATE gil, plm_model** out) {
    long h = 0;
    int code = leave(r, gil, &h);
    if (code) return code;
    *out = (plm_model*)malloc(sizeof(plm_model));
    if (*out == NULL) {
        set_error("out of memory");
        return PLM_API_ERROR;
    }
    (*out)->handle = h;
    return PLM_API_OK;
}

int plm_model_load(const char* model_dir, const char* dtype, plm_model** out) {
    NEED(model_dir && dtype && out, "plm_model_load: model_dir, dtype and out must be given");
    *out = NULL;
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    return new_model(PyObject_CallMethod(g_host, "model_load", "ss", model_dir, dtype), gil, out);
}

int plm_model_random(const char* config_json, uint64_t seed, const char* dtype, const char* out_dir, plm_model** out) {
    NEED(config_json && dtype && out_dir && out, "plm_model_random: config_json, dtype, out_dir and out must be given");
    *out = NULL;
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    return new_model(PyObject_CallMethod(g_host, "model_random", "sKss", config_json, (unsigned long long)seed, dtype,
                                         out_dir), gil, out);
}

int plm_model_free(plm_model* model) {
    if (model == NULL) return PLM_API_OK;
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    code = leave(PyObject_CallMethod(g_host, "model_free", "l", model->handle), gil, NULL);
    free(model);
    return code;
}

int plm_model_vocab_size(const plm_model* model, int* out) {
    NEED(model && out, "plm_model_vocab_size: model and out must be given");
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    long v = 0;
    code = leave(PyObject_CallMethod(g_host, "model_vocab_size", "l", model->handle), gil, &v);
    *out = (int)v;
    return code;
}

int plm_ctx_create(plm_model* model, int n_slots, int max_context, plm_ctx** out) {
    NEED(model && out, "plm_ctx_create: model and out must be given");
    *out = NULL;
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    long h = 0;
    code = leave(PyObject_CallMethod(g_host, "ctx_create", "lii", model->handle, n_slots, max_context), gil, &h);
    if (code) return code;
    *out = (plm_ctx*)malloc(sizeof(plm_ctx));
    if (*out == NULL) {
        set_error("out of memory");
        return PLM_API_ERROR;
    }
    (*out)->handle = h;
    (*out)->model = model->handle;
    return PLM_API_OK;
}

int plm_ctx_free(plm_ctx* ctx) {
    if (ctx == NULL) return PLM_API_OK;
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    code = leave(PyObject_CallMethod(g_host, "ctx_free", "l", ctx->handle), gil, NULL);
    free(ctx);
    return code;
}

int plm_slot_reset(plm_ctx* ctx, int slot) {
    NEED(ctx, "plm_slot_reset: ctx must be given");
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    return leave(PyObject_CallMethod(g_host, "slot_reset", "li", ctx->handle, slot), gil, NULL);
}

int plm_slot_length(plm_ctx* ctx, int slot, int* out) {
    NEED(ctx && out, "plm_slot_length: ctx and out must be given");
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    long v = 0;
    code = leave(PyObject_CallMethod(g_host, "slot_length", "li", ctx->handle, slot), gil, &v);
    *out = (int)v;
    return code;
}

int plm_step(plm_ctx* ctx, int n_seqs, const int* slots, const int* n_new, const int* tokens, int n_logit_rows,
             const int* logit_rows, float* logits_out) {
    NEED(ctx && slots && n_new && tokens, "plm_step: ctx, slots, n_new and tokens must be given");
    NEED(n_seqs > 0, "plm_step: n_seqs must be positive");
    NEED(n_logit_rows >= 0, "plm_step: n_logit_rows must not be negative");
    size_t total = 0;
    for (int i = 0; i < n_seqs; ++i) {
        NEED(n_new[i] > 0, "plm_step: every sequence must bring at least one token");
        total += (size_t)n_new[i];
    }
    int vocab = 0;
    {
        plm_model m = {ctx->model};
        int code = plm_model_vocab_size(&m, &vocab);
        if (code) return code;
    }
    const size_t rows = logit_rows ? (size_t)n_logit_rows : (size_t)n_seqs;
    NEED(rows == 0 || logits_out, "plm_step: logits_out must be given when logits are wanted");
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    PyObject* a = view(slots, sizeof(int) * (size_t)n_seqs, 0);
    PyObject* b = view(n_new, sizeof(int) * (size_t)n_seqs, 0);
    PyObject* c = view(tokens, sizeof(int) * total, 0);
    PyObject* d = view(logit_rows, sizeof(int) * (size_t)n_logit_rows, 0);
    PyObject* e = view(rows ? logits_out : NULL, sizeof(float) * rows * (size_t)vocab, 1);
    PyObject* r = (a && b && c && d && e)
                      ? PyObject_CallMethod(g_host, "step", "liOOOOiO", ctx->handle, n_seqs, a, b, c, d, n_logit_rows, e)
                      : NULL;
    Py_XDECREF(a); Py_XDECREF(b); Py_XDECREF(c); Py_XDECREF(d); Py_XDECREF(e);
    return leave(r, gil, NULL);
}

int plm_sample(plm_ctx* ctx, const float* logits, int rows, const plm_sampling* sampling, uint64_t* rng_states,
               int* tokens_out) {
    NEED(ctx && logits && tokens_out && rows > 0, "plm_sample: ctx, logits, tokens_out and rows > 0 must be given");
    plm_sampling s = sampling ? *sampling : plm_sampling_default();
    NEED(s.temperature <= 0.0f || rng_states, "plm_sample: rng_states must be given unless the sampling is greedy");
    int vocab = 0;
    {
        plm_model m = {ctx->model};
        int code = plm_model_vocab_size(&m, &vocab);
        if (code) return code;
    }
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    PyObject* a = view(logits, sizeof(float) * (size_t)rows * (size_t)vocab, 0);
    PyObject* b = view(rng_states, sizeof(uint64_t) * (size_t)rows, 1);
    PyObject* c = view(tokens_out, sizeof(int) * (size_t)rows, 1);
    PyObject* r = (a && b && c) ? PyObject_CallMethod(g_host, "sample", "lOififfOO", ctx->handle, a, rows,
                                                      (double)s.temperature, s.top_k, (double)s.top_p, (double)s.min_p, b, c)
                                : NULL;
    Py_XDECREF(a); Py_XDECREF(b); Py_XDECREF(c);
    return leave(r, gil, NULL);
}

int plm_generate(plm_ctx* ctx, int n_prompts, const int* const* prompts, const int* prompt_lens, int max_new,
                 const plm_sampling* sampling, const int* stop_ids, int n_stop, int* const* out_tokens, int* out_lens) {
    NEED(ctx && prompts && prompt_lens && out_tokens && out_lens, "plm_generate: ctx, prompts, prompt_lens, out_tokens "
                                                                   "and out_lens must be given");
    NEED(n_prompts > 0 && max_new >= 0, "plm_generate: n_prompts must be positive and max_new not negative");
    plm_sampling s = sampling ? *sampling : plm_sampling_default();
    PyGILState_STATE gil;
    int code = enter(&gil);
    if (code) return code;
    PyObject* ps = PyList_New(n_prompts);
    PyObject* outs = PyList_New(n_prompts);
    int ok = ps != NULL && outs != NULL;
    for (int i = 0; ok && i < n_prompts; ++i) {
        if (prompts[i] == NULL || prompt_lens[i] <= 0 || (max_new > 0 && out_tokens[i] == NULL)) {
            ok = 0;
            PyErr_Format(PyExc_ValueError, "plm_generate: prompt %d is empty or has no output buffer", i);
            break;
        }
        PyObject* p = view(prompts[i], sizeof(int) * (size_t)prompt_lens[i], 0);
        PyObject* o = view(out_tokens[i], sizeof(int) * (size_t)(max_new > 0 ? max_new : 1), 1);
        if (p == NULL || o == NULL) {
            Py_XDECREF(p); Py_XDECREF(o);
            ok = 0;
            break;
        }
        PyList_SET_ITEM(ps, i, p);
        PyList_SET_ITEM(outs, i, o);
    }
    PyObject* stop = ok ? view(stop_ids, sizeof(int) * (size_t)(n_stop > 0 ? n_stop : 0), 0) : NULL;
    PyObject* lens = ok ? view(out_lens, sizeof(int) * (size_t)n_prompts, 1) : NULL;
    PyObject* r = NULL;
    if (ok && stop && lens)
        r = PyObject_CallMethod(g_host, "generate", "lOififfKOiOO", ctx->handle, ps, max_new, (double)s.temperature, s.top_k,
                                (double)s.top_p, (double)s.min_p, (unsigned long long)s.seed, stop, n_stop, outs, lens);
    Py_XDECREF(ps); Py_XDECREF(outs); Py_XDECREF(stop); Py_XDECREF(lens);
    return leave(r, gil, NULL);
}
