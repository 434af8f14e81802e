/*
 * gact._hooks: the per-tensor fast path of the saved-tensor hooks (Quantizer.quantize / Quantizer.dequantize for
 * floating-point activations) as native code.
 *
 * A training step runs these hooks about a thousand times, each in front of a kernel of a few microseconds, and in
 * Python one call costs 9-10 us (attribute look-ups on the tensor, torch.empty, the stream query, building the
 * payload object).  Here the same decisions are taken on the at::Tensor directly: filter, tid / width / seed look-up in
 * the Quantizer's own dictionaries (which stay the single source of truth: auto precision and user code read and
 * write them from Python), one allocation from PyTorch's caching allocator, the library call through the C ABI, and
 * the tuple autograd keeps.  Everything that is not the plain case - dropout masks, 32-bit passthrough, swapping,
 * value-fingerprint deduplication - is handed back to the Python implementation untouched (the functions return
 * NotImplemented *before* changing any state).
 *
 * Behaviour mirrors gact/quantizer.py line by line; reference: gact/gact/quantizer.py:47-69,95-195.
 * This module belongs to the Python layer (it links against libtorch); the kernels stay behind the C ABI of
 * libgact_b200.so, which it calls like any other client.
 */
#include <Python.h>

#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/Dtype.h>
#include <torch/csrc/Exceptions.h>
#include <torch/csrc/autograd/python_variable.h>

#include <algorithm>
#include <vector>

#include "gact_b200.h"

namespace {

long long g_launches = 0;          // library kernels enqueued from here (benchmarks report it)

// interned attribute names
#define GACT_NAMES(X)                                                                                                         \
    X(unrelated_tensors) X(tid) X(iter) X(tids_registered) X(bits) X(seeds) X(dims) X(default_bit) X(seed_iter) X(seed_offset)    \
    X(swap) X(ptr_qtensor_map) X(layer_key_map) X(_live) X(check_dup) X(dedup_saved) X(keep_layout) X(rng_mode) X(fma)           \
    X(quantize_bf16) X(shape) X(dtype) X(buf) X(n) X(strides) X(pack_bool_masks)
#define X(name) PyObject* s_##name = nullptr;
GACT_NAMES(X)
#undef X
PyObject* g_packed_type = nullptr;      // gact.ops.Packed

struct Ref {                            // owned reference
    PyObject* p;
    explicit Ref(PyObject* o = nullptr) : p(o) {}
    ~Ref() { Py_XDECREF(p); }
    Ref(const Ref&) = delete;
    Ref& operator=(const Ref&) = delete;
    PyObject* release() { PyObject* o = p; p = nullptr; return o; }
    explicit operator bool() const { return p != nullptr; }
};

inline PyObject* attr(PyObject* o, PyObject* name) { return PyObject_GetAttr(o, name); }

bool truthy_attr(PyObject* o, PyObject* name, bool& out) {
    Ref v(attr(o, name));
    if (!v) return false;
    const int t = PyObject_IsTrue(v.p);
    if (t < 0) return false;
    out = t != 0;
    return true;
}

bool ll_attr(PyObject* o, PyObject* name, long long& out) {
    Ref v(attr(o, name));
    if (!v) return false;
    out = PyLong_AsLongLong(v.p);
    return !(out == -1 && PyErr_Occurred());
}

inline PyObject* not_mine() { Py_RETURN_NOTIMPLEMENTED; }

// layout of the single-buffer payload (the same arithmetic as gact/ops.py:_layout)
struct Layout {
    int64_t G, nbytes, off_min, off_scale, total;
    int code;
};
bool layout_of(int64_t n, int bits, at::ScalarType st, Layout& L) {
    L.G = (n + GACT_GROUP_SIZE - 1) / GACT_GROUP_SIZE;
    L.nbytes = gact_packed_bytes(n, bits);
    if (L.nbytes < 0) return false;
    const int es = st == at::kFloat ? 4 : 2;
    const int ss = st == at::kBFloat16 ? 4 : es;
    L.code = st == at::kFloat ? GACT_F32 : st == at::kHalf ? GACT_F16 : GACT_BF16;
    L.off_min = (L.nbytes + 15) / 16 * 16;
    L.off_scale = (L.off_min + L.G * es + 15) / 16 * 16;
    L.total = L.off_scale + L.G * ss;
    return true;
}

// True when the strides describe a permutation of a contiguous block (no gaps, no overlap)
bool dense_permutation(const at::Tensor& t) {
    const int d = (int)t.dim();
    std::pair<int64_t, int64_t> dims[8];
    int m = 0;
    for (int i = 0; i < d; i++)
        if (t.size(i) != 1) dims[m++] = {t.stride(i), t.size(i)};
    std::sort(dims, dims + m);
    int64_t expect = 1;
    for (int i = 0; i < m; i++) {
        if (dims[i].first != expect) return false;
        expect *= dims[i].second;
    }
    return true;
}

int rng_code(PyObject* mode) {
    if (!PyUnicode_Check(mode)) return -1;
    if (PyUnicode_CompareWithASCIIString(mode, "fast") == 0) return GACT_RNG_FAST;
    if (PyUnicode_CompareWithASCIIString(mode, "curand") == 0) return GACT_RNG_CURAND;
    if (PyUnicode_CompareWithASCIIString(mode, "rtn") == 0) return GACT_RNG_RTN;
    return -1;                                   // external noise goes through the Python path
}

PyObject* status_error(int st, const char* what) {
    PyErr_Format((st == GACT_ERR_BITS || st == GACT_ERR_DTYPE || st == GACT_ERR_SIZE || st == GACT_ERR_MODE) ? PyExc_ValueError : PyExc_RuntimeError,
                 "%s: %s (status %d)", what, gact_error_string(st), st);
    return nullptr;
}

// 1 = the tensor's address is listed in quantizer.unrelated_tensors (parameters), 0 = not, -1 = error
int is_unrelated(PyObject* self, const at::Tensor& t) {
    Ref unrelated(attr(self, s_unrelated_tensors));
    Ref ptr(PyLong_FromUnsignedLongLong((unsigned long long)(uintptr_t)t.data_ptr()));
    if (!unrelated || !ptr) return -1;
    return PySequence_Contains(unrelated.p, ptr.p);
}

// torch.bool dropout masks: the decisions of Quantizer.check_quantize and the payload of Quantizer._quantize_mask,
// (True, True, [words, shape, torch.bool]).  No quantizer state is involved.
PyObject* quantize_bool_mask(PyObject* self, PyObject* config, PyObject* input, const at::Tensor& t) {
    bool on = false;
    if (!truthy_attr(config, s_pack_bool_masks, on)) return nullptr;
    if (!on || t.layout() != at::kStrided || t.numel() == 0 || !t.is_cuda()) return PyTuple_Pack(2, Py_False, input);
    const int hit = is_unrelated(self, t);
    if (hit < 0) return nullptr;
    if (hit) return PyTuple_Pack(2, Py_False, input);
    const at::Tensor x = t.contiguous();
    const int64_t n = x.numel();
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor words = at::empty({gact_mask_words(n)}, at::TensorOptions().dtype(at::kInt).device(x.device()));
    void* stream = (void*)c10::cuda::getCurrentCUDAStream(x.device().index()).stream();
    const int rc = gact_mask_pack((const uint8_t*)x.data_ptr(), n, (uint32_t*)words.data_ptr(), nullptr, stream);
    g_launches++;
    if (rc) return status_error(rc, "gact_mask_pack");
    Ref words_o(THPVariable_Wrap(words)), shape(attr(input, s_shape)), dtype_o(attr(input, s_dtype));
    if (!words_o || !shape || !dtype_o) return nullptr;
    Ref payload(PyList_New(3));
    if (!payload) return nullptr;
    PyList_SET_ITEM(payload.p, 0, words_o.release());
    PyList_SET_ITEM(payload.p, 1, shape.release());
    PyList_SET_ITEM(payload.p, 2, dtype_o.release());
    return PyTuple_Pack(3, Py_True, Py_True, payload.p);
}

// the inverse, for payloads of the form [int32 words, shape, torch.bool]; NotImplemented for anything else
PyObject* dequantize_bool_mask(PyObject* payload) {
    if (!PyList_Check(payload) || PyList_GET_SIZE(payload) != 3) return not_mine();
    PyObject *words_o = PyList_GET_ITEM(payload, 0), *shape = PyList_GET_ITEM(payload, 1), *dtype_o = PyList_GET_ITEM(payload, 2);
    if (!THPVariable_Check(words_o) || !PyTuple_Check(shape) || !THPDtype_Check(dtype_o) || ((THPDtype*)dtype_o)->scalar_type != at::kBool)
        return not_mine();
    const at::Tensor& words = THPVariable_Unpack(words_o);
    if (!words.is_cuda() || words.scalar_type() != at::kInt || !words.is_contiguous()) return not_mine();
    std::vector<int64_t> dims((size_t)PyTuple_GET_SIZE(shape));
    int64_t n = 1;
    for (size_t i = 0; i < dims.size(); i++) {
        dims[i] = PyLong_AsLongLong(PyTuple_GET_ITEM(shape, (Py_ssize_t)i));
        if (dims[i] == -1 && PyErr_Occurred()) return nullptr;
        n *= dims[i];
    }
    if (words.numel() < gact_mask_words(n)) return not_mine();            // the Python path words the error
    c10::cuda::CUDAGuard guard(words.device());
    at::Tensor out = at::empty(dims, at::TensorOptions().dtype(at::kBool).device(words.device()));
    void* stream = (void*)c10::cuda::getCurrentCUDAStream(words.device().index()).stream();
    const int rc = gact_mask_unpack((const uint32_t*)words.data_ptr(), n, (uint8_t*)out.data_ptr(), stream);
    g_launches++;
    if (rc) return status_error(rc, "gact_mask_unpack");
    return THPVariable_Wrap(out);
}

// quantize(quantizer, config, tensor) -> the tuple autograd keeps, or NotImplemented
PyObject* hooks_quantize(PyObject*, PyObject* const* args, Py_ssize_t nargs) {
    HANDLE_TH_ERRORS
    if (nargs != 3) { PyErr_SetString(PyExc_TypeError, "quantize(quantizer, config, tensor)"); return nullptr; }
    PyObject *self = args[0], *config = args[1], *input = args[2];
    if (!THPVariable_Check(input)) return not_mine();
    const at::Tensor& t = THPVariable_Unpack(input);
    const at::ScalarType st = t.scalar_type();
    if (st == at::kBFloat16) {
        bool bf16_on = false;
        if (!truthy_attr(config, s_quantize_bf16, bf16_on)) return nullptr;
        if (!bf16_on) return not_mine();
    } else if (st == at::kBool) {
        return quantize_bool_mask(self, config, input, t);
    } else if (st != at::kFloat && st != at::kHalf) {
        return not_mine();                       // uint8 masks and everything else: the Python filter decides
    }
    bool swap = false, check_dup = false, dedup = false;
    if (!truthy_attr(self, s_swap, swap) || !truthy_attr(config, s_check_dup, check_dup) || !truthy_attr(config, s_dedup_saved, dedup)) return nullptr;
    if (swap || check_dup) return not_mine();

    // the filter of check_quantize, cheapest tests first
    bool pass = t.requires_grad() && t.layout() == at::kStrided && t.dim() >= 2 && t.dim() <= 4 && t.is_cuda();
    if (pass) {
        Ref unrelated(attr(self, s_unrelated_tensors));
        Ref ptr(PyLong_FromUnsignedLongLong((unsigned long long)(uintptr_t)t.data_ptr()));
        if (!unrelated || !ptr) return nullptr;
        const int hit = PySequence_Contains(unrelated.p, ptr.p);
        if (hit < 0) return nullptr;
        pass = hit == 0;
    }
    if (!pass) return PyTuple_Pack(2, Py_False, input);

    long long tid, iter;
    if (!ll_attr(self, s_tid, tid) || !ll_attr(self, s_iter, iter)) return nullptr;
    Ref map(attr(self, s_ptr_qtensor_map)), live(attr(self, s__live)), bits_d(attr(self, s_bits));
    if (!map || !live || !bits_d) return nullptr;
    Ref tid_o(PyLong_FromLongLong(tid));
    if (!tid_o) return nullptr;

    // The same tensor object saved again, unmodified: share the payload of its first save (identity + version).
    Ref key;                                     // owned
    Ref id_o(PyLong_FromVoidPtr(input));
    if (!id_o) return nullptr;
    const long long version = (long long)t._version();
    if (dedup) {
        PyObject* seen = PyDict_GetItemWithError(live.p, id_o.p);          // borrowed
        if (!seen && PyErr_Occurred()) return nullptr;
        if (seen && PyTuple_Check(seen) && PyTuple_GET_SIZE(seen) == 3) {
            PyObject* target = PyWeakref_GetObject(PyTuple_GET_ITEM(seen, 0));   // borrowed
            if (target == input && PyLong_AsLongLong(PyTuple_GET_ITEM(seen, 1)) == version) {
                const int has = PyDict_Contains(map.p, PyTuple_GET_ITEM(seen, 2));
                if (has < 0) return nullptr;
                if (has) { key.p = PyTuple_GET_ITEM(seen, 2); Py_INCREF(key.p); }
            }
        }
    }
    const bool shared = (bool)key;
    if (!shared) { key.p = tid_o.p; Py_INCREF(key.p); }
    PyObject* entry = PyDict_GetItemWithError(map.p, key.p);               // borrowed
    if (!entry && PyErr_Occurred()) return nullptr;

    // width of a new payload; 32 bit (debug passthrough) is the Python path's business - nothing has been changed yet
    long long bit = 0, default_bit = 0, tids_registered = 0;
    if (!entry) {
        if (!ll_attr(self, s_default_bit, default_bit)) return nullptr;
        if (iter == 0) {
            bit = default_bit;
        } else {
            PyObject* b = PyDict_GetItemWithError(bits_d.p, tid_o.p);      // borrowed
            if (!b && PyErr_Occurred()) return nullptr;
            if (b) {
                bit = PyLong_AsLongLong(b);
                if (bit == -1 && PyErr_Occurred()) return nullptr;
            } else {
                if (!ll_attr(self, s_tids_registered, tids_registered)) return nullptr;
                if (tid >= tids_registered) { PyErr_SetObject(PyExc_KeyError, tid_o.p); return nullptr; }
                bit = default_bit;
            }
        }
        if (bit == 32) return not_mine();
    }
    Ref rng_o(attr(config, s_rng_mode));
    if (!rng_o) return nullptr;
    const int rng = rng_code(rng_o.p);
    if (rng < 0) return not_mine();

    // ---- from here on state changes ----
    Ref next_tid(PyLong_FromLongLong(tid + 1));
    if (!next_tid || PyObject_SetAttr(self, s_tid, next_tid.p) < 0) return nullptr;
    if (iter == 0 && PyObject_SetAttr(self, s_tids_registered, next_tid.p) < 0) return nullptr;
    if (dedup && !shared) {
        Ref wr(PyWeakref_NewRef(input, nullptr)), ver(PyLong_FromLongLong(version));
        if (!wr || !ver) return nullptr;
        Ref rec(PyTuple_Pack(3, wr.p, ver.p, key.p));
        if (!rec || PyDict_SetItem(live.p, id_o.p, rec.p) < 0) return nullptr;
    }
    {
        Ref lkm(attr(self, s_layer_key_map));
        if (!lkm || PyDict_SetItem(lkm.p, tid_o.p, key.p) < 0) return nullptr;
    }
    Ref shape(attr(input, s_shape));
    if (!shape) return nullptr;

    if (entry) {                                 // same tensor saved again: share the payload
        if (!PyList_Check(entry) || PyList_GET_SIZE(entry) != 3) { PyErr_SetString(PyExc_RuntimeError, "malformed payload entry"); return nullptr; }
        const long long cnt = PyLong_AsLongLong(PyList_GET_ITEM(entry, 1));
        Ref inc(PyLong_FromLongLong(cnt + 1));
        if (!inc || PyList_SetItem(entry, 1, inc.release()) < 0) return nullptr;
        return PyTuple_Pack(5, Py_True, Py_False, key.p, shape.p, tid_o.p);
    }

    Ref seeds_d(attr(self, s_seeds));
    if (!seeds_d) return nullptr;
    if (iter == 0) {
        Ref dims_d(attr(self, s_dims)), bit_o(PyLong_FromLongLong(bit)), numel_o(PyLong_FromLongLong(t.numel()));
        if (!dims_d || !bit_o || !numel_o) return nullptr;
        if (PyDict_SetItem(bits_d.p, tid_o.p, bit_o.p) < 0 || PyDict_SetItem(dims_d.p, tid_o.p, numel_o.p) < 0 ||
            PyDict_SetItem(seeds_d.p, tid_o.p, tid_o.p) < 0)
            return nullptr;
    }
    // seed = seeds[tid] + seed_iter + seed_offset, reduced to 64 bits
    unsigned long long seed = 0;
    {
        PyObject* s0 = PyDict_GetItemWithError(seeds_d.p, tid_o.p);        // borrowed
        if (!s0 && PyErr_Occurred()) return nullptr;
        Ref si(attr(self, s_seed_iter)), so(attr(self, s_seed_offset));
        if (!si || !so) return nullptr;
        Ref a(PyNumber_Add(s0 ? s0 : tid_o.p, si.p));
        if (!a) return nullptr;
        Ref b(PyNumber_Add(a.p, so.p));
        if (!b) return nullptr;
        seed = PyLong_AsUnsignedLongLongMask(b.p);
        if (seed == (unsigned long long)-1 && PyErr_Occurred()) return nullptr;
    }
    bool keep_layout = false, fma = true;
    if (!truthy_attr(config, s_keep_layout, keep_layout) || !truthy_attr(config, s_fma, fma)) return nullptr;

    // quantize_compact: memory order of a dense permuted view is compressed as it is (no contiguous copy)
    at::Tensor x = t;
    Ref strides;                                 // None, or the source's strides
    if (!t.is_contiguous()) {
        if (keep_layout && dense_permutation(t)) {
            strides.p = PyTuple_New(t.dim());
            if (!strides) return nullptr;
            for (int64_t i = 0; i < t.dim(); i++) PyTuple_SET_ITEM(strides.p, i, PyLong_FromLongLong(t.stride(i)));
        } else {
            x = t.contiguous();
        }
    }
    if (!strides) { strides.p = Py_None; Py_INCREF(Py_None); }
    const int64_t n = x.numel();
    Layout L;
    if (!layout_of(n, (int)bit, st, L)) { PyErr_Format(PyExc_ValueError, "bits must be 1, 2, 4, 8 or 32, got %lld", bit); return nullptr; }
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor buf = at::empty({L.total}, at::TensorOptions().dtype(at::kByte).device(x.device()));
    unsigned char* base = (unsigned char*)buf.data_ptr();
    void* stream = (void*)c10::cuda::getCurrentCUDAStream(x.device().index()).stream();
    const int rc = gact_quantize(x.data_ptr(), L.code, n, (int)bit, (uint64_t)seed, rng, nullptr, fma ? 1 : 0, base, base + L.off_min,
                                 base + L.off_scale, stream);
    g_launches++;
    if (rc) return status_error(rc, "gact_quantize");

    Ref buf_o(THPVariable_Wrap(buf)), dtype_o(attr(input, s_dtype)), bit_o(PyLong_FromLongLong(bit)), n_o(PyLong_FromLongLong(n));
    if (!buf_o || !dtype_o || !bit_o || !n_o) return nullptr;
    PyObject* pargs[5] = {buf_o.p, bit_o.p, dtype_o.p, n_o.p, strides.p};
    Ref packed(PyObject_Vectorcall(g_packed_type, pargs, 5, nullptr));
    if (!packed) return nullptr;
    Ref one(PyLong_FromLong(1));
    Ref rec(PyList_New(3));
    if (!one || !rec) return nullptr;
    PyList_SET_ITEM(rec.p, 0, packed.release());
    PyList_SET_ITEM(rec.p, 1, one.release());
    Py_INCREF(tid_o.p);
    PyList_SET_ITEM(rec.p, 2, tid_o.p);
    if (PyDict_SetItem(map.p, key.p, rec.p) < 0) return nullptr;
    return PyTuple_Pack(5, Py_True, Py_False, key.p, shape.p, tid_o.p);
    END_HANDLE_TH_ERRORS
}

// dequantize(quantizer, saved) -> tensor, or NotImplemented
PyObject* hooks_dequantize(PyObject*, PyObject* const* args, Py_ssize_t nargs) {
    HANDLE_TH_ERRORS
    if (nargs != 2) { PyErr_SetString(PyExc_TypeError, "dequantize(quantizer, saved)"); return nullptr; }
    PyObject *self = args[0], *saved = args[1];
    if (!PyTuple_Check(saved) || PyTuple_GET_SIZE(saved) < 2) return not_mine();
    if (PyTuple_GET_ITEM(saved, 0) != Py_True) {          // not quantized: the tensor itself
        if (PyTuple_GET_ITEM(saved, 0) != Py_False) return not_mine();
        PyObject* r = PyTuple_GET_ITEM(saved, 1);
        Py_INCREF(r);
        return r;
    }
    if (PyTuple_GET_SIZE(saved) == 3 && PyTuple_GET_ITEM(saved, 1) == Py_True) return dequantize_bool_mask(PyTuple_GET_ITEM(saved, 2));
    if (PyTuple_GET_SIZE(saved) != 5 || PyTuple_GET_ITEM(saved, 1) != Py_False) return not_mine();
    bool swap = false;
    if (!truthy_attr(self, s_swap, swap)) return nullptr;
    if (swap) return not_mine();
    PyObject *key = PyTuple_GET_ITEM(saved, 2), *shape = PyTuple_GET_ITEM(saved, 3);
    Ref map(attr(self, s_ptr_qtensor_map));
    if (!map) return nullptr;
    PyObject* entry = PyDict_GetItemWithError(map.p, key);                 // borrowed
    if (!entry) {
        if (PyErr_Occurred()) return nullptr;
        return not_mine();                                                 // let the Python path raise its KeyError
    }
    if (!PyList_Check(entry) || PyList_GET_SIZE(entry) != 3) return not_mine();
    PyObject* q = PyList_GET_ITEM(entry, 0);
    if ((PyObject*)Py_TYPE(q) != g_packed_type || !PyTuple_Check(shape)) return not_mine();

    Ref buf_o(attr(q, s_buf)), dtype_o(attr(q, s_dtype)), strides_o(attr(q, s_strides));
    long long bits = 0, n = 0;
    if (!buf_o || !dtype_o || !strides_o || !ll_attr(q, s_bits, bits) || !ll_attr(q, s_n, n)) return nullptr;
    if (!THPVariable_Check(buf_o.p) || !THPDtype_Check(dtype_o.p)) return not_mine();
    const at::Tensor& buf = THPVariable_Unpack(buf_o.p);
    if (!buf.is_cuda()) return not_mine();
    const at::ScalarType st = ((THPDtype*)dtype_o.p)->scalar_type;
    Layout L;
    if (!layout_of(n, (int)bits, st, L)) return not_mine();
    std::vector<int64_t> dims((size_t)PyTuple_GET_SIZE(shape));
    for (size_t i = 0; i < dims.size(); i++) {
        dims[i] = PyLong_AsLongLong(PyTuple_GET_ITEM(shape, (Py_ssize_t)i));
        if (dims[i] == -1 && PyErr_Occurred()) return nullptr;
    }
    c10::cuda::CUDAGuard guard(buf.device());
    const auto opts = at::TensorOptions().dtype(st).device(buf.device());
    at::Tensor out;
    if (strides_o.p == Py_None) {
        out = at::empty(dims, opts);
    } else {
        if (!PyTuple_Check(strides_o.p) || (size_t)PyTuple_GET_SIZE(strides_o.p) != dims.size()) return not_mine();
        std::vector<int64_t> str(dims.size());
        for (size_t i = 0; i < dims.size(); i++) {
            str[i] = PyLong_AsLongLong(PyTuple_GET_ITEM(strides_o.p, (Py_ssize_t)i));
            if (str[i] == -1 && PyErr_Occurred()) return nullptr;
        }
        out = at::empty_strided(dims, str, opts);
    }
    unsigned char* base = (unsigned char*)buf.data_ptr();
    void* stream = (void*)c10::cuda::getCurrentCUDAStream(buf.device().index()).stream();
    const int rc = gact_dequantize(base, base + L.off_min, base + L.off_scale, L.code, n, (int)bits, out.data_ptr(), stream);
    g_launches++;
    if (rc) return status_error(rc, "gact_dequantize");

    // ref-count of the shared payload
    const long long cnt = PyLong_AsLongLong(PyList_GET_ITEM(entry, 1)) - 1;
    if (cnt < 0) {
        PyErr_Format(PyExc_RuntimeError, "[Error] Ref count < 0 %S %lld", key, cnt);
        return nullptr;
    }
    if (cnt == 0) {
        if (PyDict_DelItem(map.p, key) < 0) return nullptr;
    } else {
        Ref dec(PyLong_FromLongLong(cnt));
        if (!dec || PyList_SetItem(entry, 1, dec.release()) < 0) return nullptr;
    }
    return THPVariable_Wrap(out);
    END_HANDLE_TH_ERRORS
}

PyObject* hooks_launches(PyObject*, PyObject*) { return PyLong_FromLongLong(g_launches); }

PyObject* hooks_bind(PyObject*, PyObject* packed_type) {
    Py_INCREF(packed_type);
    Py_XDECREF(g_packed_type);
    g_packed_type = packed_type;
    Py_RETURN_NONE;
}

PyMethodDef methods[] = {
    {"quantize", (PyCFunction)(void (*)(void))hooks_quantize, METH_FASTCALL,
     "quantize(quantizer, config, tensor): Quantizer.quantize for floating-point tensors; NotImplemented for anything else"},
    {"dequantize", (PyCFunction)(void (*)(void))hooks_dequantize, METH_FASTCALL,
     "dequantize(quantizer, saved): Quantizer.dequantize for payloads made by quantize; NotImplemented for anything else"},
    {"launches", hooks_launches, METH_NOARGS, "number of library kernels enqueued by this module"},
    {"bind", hooks_bind, METH_O, "bind(Packed): the payload class of gact.ops"},
    {nullptr, nullptr, 0, nullptr}};

PyModuleDef module = {PyModuleDef_HEAD_INIT, "_hooks", "native fast path of the saved-tensor hooks", -1, methods, nullptr, nullptr, nullptr, nullptr};

}  // namespace

PyMODINIT_FUNC PyInit__hooks(void) {
#define X(name) s_##name = PyUnicode_InternFromString(#name);
    GACT_NAMES(X)
#undef X
    return PyModule_Create(&module);
}
