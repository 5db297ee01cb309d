/* CPython front of the retrieval object, the counterpart of the reference's pybind11 module
 * (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp:200-225): submit / wait / get_result with numpy arrays in and
 * out, calling the C ABI (ucmx_retrieval_*) directly.  ESA makes three of these calls per request and layer
 * (ucm/sparse/esa/esa.py:286-339), so what a call costs on the host is what the plug-in's retrieval costs once the
 * GPU work is one launch per layer; through ctypes a call is 3-5 us, here well under one.
 *
 * The module does not link against the library: ucmx/retrieval.py hands it the addresses of the three entry points
 * once (bind), so the C ABI stays the only boundary.  ucmx.retrieval.RetrievalWorkerBackend derives from the type
 * defined here, so the three methods are called without a Python frame in between.  Arrays that are not plain
 * C-contiguous float32 / int32 go to the subclass's _submit_converted, which converts and calls submit again; a status
 * other than success goes to the callable given to bind, which raises what the ctypes route raises. */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#define NPY_NO_DEPRECATED_API NPY_1_7_API_VERSION
#include <numpy/arrayobject.h>
#include <stdint.h>

typedef int32_t (*submit_fn)(void*, const float*, int32_t, int32_t, int32_t, const int32_t*, int32_t, int32_t*);
typedef int32_t (*wait_fn)(void*, int32_t);
typedef int32_t (*get_fn)(void*, int32_t, int32_t*, float*);
typedef int32_t (*shape_fn)(void*, int32_t, int32_t*, int32_t*);

static submit_fn g_submit;
static wait_fn g_wait;
static get_fn g_get;
static shape_fn g_shape;
static PyObject* g_on_error;   /* callable(function name, status): raises */
static PyObject *g_key_indices, *g_key_scores;   /* the result dictionary's keys, made once */

#define UCMX_ENOOBJ (-50005)

static PyObject* raise_status(const char* fn, int32_t st)
{
    if (g_on_error) {
        PyObject* r = PyObject_CallFunction(g_on_error, "si", fn, (int)st);
        Py_XDECREF(r);
        if (PyErr_Occurred()) return NULL;
    }
    PyErr_Format(PyExc_RuntimeError, "%s failed with status %d", fn, (int)st);
    return NULL;
}

#define SHAPE_SLOTS 8192   /* result shapes kept here, by id % SHAPE_SLOTS; a request whose slot has been taken over by a
                              newer one asks the library for its shape instead */

typedef struct {
    PyObject_HEAD
    void* handle;
    int32_t dim;
    int32_t last_rid;   /* the largest request id a submit of this object has returned (-1: none yet) */
    struct {
        int32_t rid, rows, k;
    } shape[SHAPE_SLOTS];
} FastBackend;

static int fb_init(FastBackend* self, PyObject* args, PyObject* kw)
{
    unsigned long long h = 0;
    int dim = 0;
    (void)kw;
    if (!PyArg_ParseTuple(args, "Ki", &h, &dim)) return -1;   /* (a subclass calls this once it has its handle) */
    self->handle = (void*)(uintptr_t)h;
    self->dim = dim;
    self->last_rid = -1;
    for (int i = 0; i < SHAPE_SLOTS; ++i) self->shape[i].rid = -1;
    return 0;
}

static int plain(PyObject* o, int typenum)
{
    if (!PyArray_CheckExact(o)) return 0;
    PyArrayObject* a = (PyArrayObject*)o;
    return PyArray_TYPE(a) == typenum && PyArray_NDIM(a) == 2 && PyArray_IS_C_CONTIGUOUS(a);
}

/* submit(query float32 [b, dim], topk, indexes int32 [b, n]) -> request id */
static PyObject* fb_submit(FastBackend* self, PyObject* const* args, Py_ssize_t nargs)
{
    if (nargs != 3) {
        PyErr_SetString(PyExc_TypeError, "submit(query, topk, indexes)");
        return NULL;
    }
    if (!g_submit) {
        PyErr_SetString(PyExc_RuntimeError, "not bound to the library");
        return NULL;
    }
    if (!self->handle) {
        PyErr_SetString(PyExc_RuntimeError, "the retrieval object is closed");
        return NULL;
    }
    PyObject *q = args[0], *idx = args[2];
    if (!plain(q, NPY_FLOAT32) || !plain(idx, NPY_INT32)) {
        /* one- or three-dimensional plain arrays are shape errors, anything else is for the Python side to convert */
        if (PyArray_CheckExact(q) && PyArray_CheckExact(idx) && PyArray_TYPE((PyArrayObject*)q) == NPY_FLOAT32 &&
            PyArray_TYPE((PyArrayObject*)idx) == NPY_INT32 && PyArray_IS_C_CONTIGUOUS((PyArrayObject*)q) &&
            PyArray_IS_C_CONTIGUOUS((PyArrayObject*)idx)) {
            if (PyArray_NDIM((PyArrayObject*)q) != 2) {
                PyErr_SetString(PyExc_RuntimeError, "Query dim mismatch");
                return NULL;
            }
            PyErr_SetString(PyExc_RuntimeError, "Query and indexes batch mismatch");
            return NULL;
        }
        return PyObject_CallMethod((PyObject*)self, "_submit_converted", "OOO", q, args[1], idx);
    }
    const long topk = PyLong_AsLong(args[1]);
    if (topk == -1 && PyErr_Occurred()) return NULL;
    PyArrayObject *qa = (PyArrayObject*)q, *ia = (PyArrayObject*)idx;
    const npy_intp rows = PyArray_DIM(qa, 0), dim = PyArray_DIM(qa, 1), n = PyArray_DIM(ia, 1);
    if (dim != self->dim) {
        PyErr_SetString(PyExc_RuntimeError, "Query dim mismatch");
        return NULL;
    }
    if (PyArray_DIM(ia, 0) != rows) {
        PyErr_SetString(PyExc_RuntimeError, "Query and indexes batch mismatch");
        return NULL;
    }
    int32_t rid = -1;
    const int32_t st = g_submit(self->handle, (const float*)PyArray_DATA(qa), (int32_t)rows, (int32_t)dim, (int32_t)topk,
                                (const int32_t*)PyArray_DATA(ia), (int32_t)n, &rid);
    if (st != 0) return raise_status("ucmx_retrieval_submit", st);
    const int slot = (int)((uint32_t)rid % SHAPE_SLOTS);
    if (rid > self->last_rid) self->last_rid = rid;
    self->shape[slot].rid = rid;
    self->shape[slot].rows = (int32_t)rows;
    self->shape[slot].k = (int32_t)(topk < n ? topk : n);
    return PyLong_FromLong(rid);
}

/* wait(req_id): returns when the request's result is on the host (the GIL is released while the stream is waited for) */
static PyObject* fb_wait(FastBackend* self, PyObject* arg)
{
    const long rid = PyLong_AsLong(arg);
    if (rid == -1 && PyErr_Occurred()) return NULL;
    if (!self->handle || !g_wait) {
        PyErr_SetString(PyExc_RuntimeError, "the retrieval object is closed");
        return NULL;
    }
    int32_t st;
    Py_BEGIN_ALLOW_THREADS
    st = g_wait(self->handle, (int32_t)rid);
    Py_END_ALLOW_THREADS
    if (st == 0) Py_RETURN_NONE;
    if (st == UCMX_ENOOBJ) {
        PyErr_SetString(PyExc_RuntimeError, "Bad req_id");
        return NULL;
    }
    return raise_status("ucmx_retrieval_wait", st);
}

/* get_result(req_id) -> {"indices": int32 [b, k], "scores": float32 [b, k]}; the request is forgotten afterwards */
static PyObject* fb_get_result(FastBackend* self, PyObject* arg)
{
    const long rid = PyLong_AsLong(arg);
    if (rid == -1 && PyErr_Occurred()) return NULL;
    if (!self->handle || !g_wait) {
        PyErr_SetString(PyExc_RuntimeError, "the retrieval object is closed");
        return NULL;
    }
    const int slot = (int)((uint32_t)rid % SHAPE_SLOTS);
    int32_t rows = 0, k = 0;
    if (rid >= 0 && self->shape[slot].rid == (int32_t)rid) {
        rows = self->shape[slot].rows;
        k = self->shape[slot].k;
    } else if (rid < 0 || rid > self->last_rid || !g_shape || g_shape(self->handle, (int32_t)rid, &rows, &k) != 0) {
        PyErr_SetString(PyExc_RuntimeError, "Result not ready");
        return NULL;
    }
    npy_intp dims[2] = {rows, k};
    PyObject* indices = PyArray_SimpleNew(2, dims, NPY_INT32);
    PyObject* scores = PyArray_SimpleNew(2, dims, NPY_FLOAT32);
    if (!indices || !scores) {
        Py_XDECREF(indices);
        Py_XDECREF(scores);
        return NULL;
    }
    const int32_t st = g_get(self->handle, (int32_t)rid, (int32_t*)PyArray_DATA((PyArrayObject*)indices),
                             (float*)PyArray_DATA((PyArrayObject*)scores));
    if (st != 0) {
        Py_DECREF(indices);
        Py_DECREF(scores);
        if (st == UCMX_ENOOBJ) {
            PyErr_SetString(PyExc_RuntimeError, "Result not ready");
            return NULL;
        }
        return raise_status("ucmx_retrieval_get_result", st);
    }
    if (self->shape[slot].rid == (int32_t)rid) self->shape[slot].rid = -1;
    PyObject* d = PyDict_New();
    if (!d || PyDict_SetItem(d, g_key_indices, indices) < 0 || PyDict_SetItem(d, g_key_scores, scores) < 0) {
        Py_XDECREF(d);
        d = NULL;
    }
    Py_DECREF(indices);
    Py_DECREF(scores);
    return d;
}

static PyMethodDef fb_methods[] = {
    {"submit", (PyCFunction)(void (*)(void))fb_submit, METH_FASTCALL, "submit(query, topk, indexes)"},
    {"wait", (PyCFunction)fb_wait, METH_O, "wait(req_id)"},
    {"get_result", (PyCFunction)fb_get_result, METH_O, "get_result(req_id)"},
    {NULL, NULL, 0, NULL}};

static PyTypeObject FastBackendType = {
    PyVarObject_HEAD_INIT(NULL, 0).tp_name = "_ucmx_fast.Backend",
    .tp_basicsize = sizeof(FastBackend),
    .tp_flags = Py_TPFLAGS_DEFAULT | Py_TPFLAGS_BASETYPE,
    .tp_new = PyType_GenericNew,
    .tp_init = (initproc)fb_init,
    .tp_methods = fb_methods,
};

/* bind(submit_address, wait_address, get_result_address, result_shape_address, on_error): the entry points of the
 * loaded library and the callable that turns a failed status into the package's exception */
static PyObject* mod_bind(PyObject* self, PyObject* args)
{
    unsigned long long a = 0, b = 0, c = 0, d = 0;
    PyObject* on_error = NULL;
    (void)self;
    if (!PyArg_ParseTuple(args, "KKKKO", &a, &b, &c, &d, &on_error)) return NULL;
    g_submit = (submit_fn)(uintptr_t)a;
    g_wait = (wait_fn)(uintptr_t)b;
    g_get = (get_fn)(uintptr_t)c;
    g_shape = (shape_fn)(uintptr_t)d;
    Py_XINCREF(on_error);
    Py_XDECREF(g_on_error);
    g_on_error = on_error;
    Py_RETURN_NONE;
}

static PyMethodDef mod_methods[] = {{"bind", mod_bind, METH_VARARGS, "bind(submit, wait, get_result, result_shape addresses, on_error)"},
                                    {NULL, NULL, 0, NULL}};

static struct PyModuleDef moddef = {PyModuleDef_HEAD_INIT, "_ucmx_fast", "CPython front of ucmx_retrieval_*", -1, mod_methods,
                                    NULL, NULL, NULL, NULL};

PyMODINIT_FUNC PyInit__ucmx_fast(void)
{
    import_array();
    if (PyType_Ready(&FastBackendType) < 0) return NULL;
    g_key_indices = PyUnicode_InternFromString("indices");
    g_key_scores = PyUnicode_InternFromString("scores");
    if (!g_key_indices || !g_key_scores) return NULL;
    PyObject* m = PyModule_Create(&moddef);
    if (!m) return NULL;
    Py_INCREF(&FastBackendType);
    if (PyModule_AddObject(m, "Backend", (PyObject*)&FastBackendType) < 0) {
        Py_DECREF(&FastBackendType);
        Py_DECREF(m);
        return NULL;
    }
    return m;
}
