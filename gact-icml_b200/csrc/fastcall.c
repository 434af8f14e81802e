/*
 * gact._fastcall: the two calls the saved-tensor hooks make for every tensor, as CPython built-ins.
 *
 * ctypes spends about 1.8 us converting the twelve arguments of gact_quantize on every call; a training step
 * makes several hundred such calls, each in front of a kernel of a few microseconds.  These wrappers take the
 * same arguments as plain Python integers (None for a null pointer) and forward them to the C ABI of
 * libgact_b200.so unchanged; they return the library's status code.  The GIL is kept: the calls only enqueue a
 * kernel.  gact/_native.py falls back to ctypes when this module was not built.
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <stdint.h>

#include "gact_b200.h"

static int as_ptr(PyObject* o, void** out) {
    if (o == Py_None) { *out = NULL; return 0; }
    unsigned long long v = PyLong_AsUnsignedLongLong(o);
    if (v == (unsigned long long)-1 && PyErr_Occurred()) return -1;
    *out = (void*)(uintptr_t)v;
    return 0;
}

static int as_i64(PyObject* o, int64_t* out) {
    long long v = PyLong_AsLongLong(o);
    if (v == -1 && PyErr_Occurred()) return -1;
    *out = (int64_t)v;
    return 0;
}

static int as_int(PyObject* o, int* out) {
    long v = PyLong_AsLong(o);
    if (v == -1 && PyErr_Occurred()) return -1;
    *out = (int)v;
    return 0;
}

/* quantize(x, dtype, n, bits, seed, rng_mode, noise, fma_mode, packed, qmin, qscale, stream) -> status */
static PyObject* fc_quantize(PyObject* self, PyObject* const* a, Py_ssize_t nargs) {
    (void)self;
    if (nargs != 12) { PyErr_SetString(PyExc_TypeError, "quantize takes 12 arguments"); return NULL; }
    void *x, *noise, *packed, *qmin, *qscale, *stream;
    int dtype, bits, rng, fma;
    int64_t n;
    if (as_ptr(a[0], &x) || as_int(a[1], &dtype) || as_i64(a[2], &n) || as_int(a[3], &bits)) return NULL;
    unsigned long long seed = PyLong_AsUnsignedLongLongMask(a[4]);
    if (seed == (unsigned long long)-1 && PyErr_Occurred()) return NULL;
    if (as_int(a[5], &rng) || as_ptr(a[6], &noise) || as_int(a[7], &fma) || as_ptr(a[8], &packed) || as_ptr(a[9], &qmin) ||
        as_ptr(a[10], &qscale) || as_ptr(a[11], &stream))
        return NULL;
    return PyLong_FromLong(gact_quantize(x, dtype, n, bits, (uint64_t)seed, rng, (const float*)noise, fma, packed, qmin, qscale, stream));
}

/* dequantize(packed, qmin, qscale, dtype, n, bits, out, stream) -> status */
static PyObject* fc_dequantize(PyObject* self, PyObject* const* a, Py_ssize_t nargs) {
    (void)self;
    if (nargs != 8) { PyErr_SetString(PyExc_TypeError, "dequantize takes 8 arguments"); return NULL; }
    void *packed, *qmin, *qscale, *out, *stream;
    int dtype, bits;
    int64_t n;
    if (as_ptr(a[0], &packed) || as_ptr(a[1], &qmin) || as_ptr(a[2], &qscale) || as_int(a[3], &dtype) || as_i64(a[4], &n) ||
        as_int(a[5], &bits) || as_ptr(a[6], &out) || as_ptr(a[7], &stream))
        return NULL;
    return PyLong_FromLong(gact_dequantize(packed, qmin, qscale, dtype, n, bits, out, stream));
}

static PyMethodDef methods[] = {
    {"quantize", (PyCFunction)(void (*)(void))fc_quantize, METH_FASTCALL, "gact_quantize with integer arguments; returns the status"},
    {"dequantize", (PyCFunction)(void (*)(void))fc_dequantize, METH_FASTCALL, "gact_dequantize with integer arguments; returns the status"},
    {NULL, NULL, 0, NULL}};

static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, "_fastcall", "direct CPython entry points for the hot calls of libgact_b200", -1, methods,
                                    NULL, NULL, NULL, NULL};

PyMODINIT_FUNC PyInit__fastcall(void) { return PyModule_Create(&module); }
