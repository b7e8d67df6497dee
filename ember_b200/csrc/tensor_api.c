/* tensor_api.c -- CPython binding of the attention path (module ember_b200._core._tensor).
 *
 * Written in the style of the reference's binding (src/tensor/tensor_api.c): a `_Tensor` type that
 * owns one device buffer (d_ptr + element count first in the struct, as in
 * src/core/tensor_types.h:6-9), METH_VARARGS module functions that parse with "O!" against the
 * type, validate sizes (ValueError with a formatted message, as tensor_api.c:196-199,338-347),
 * allocate the results (MemoryError on failure, as :28-31), call ONE extern "C" function of the
 * CUDA library and wrap the result. Shapes are passed from Python as ints because the native
 * object only knows its element count (tensor_api.c:386-394). Additions over the reference: a
 * dtype field (0 = float32, 1 = bfloat16) and a 64-bit element count after the reference's two
 * fields; native status codes become Python exceptions instead of exit().
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <structmember.h>

#include "../../include/ember_b200.h"

typedef struct {
    PyObject_HEAD void *d_ptr;
    int size;            /* element count, saturated at INT_MAX (reference field) */
    int dtype;           /* EMBER_F32 / EMBER_BF16 */
    long long size64;    /* exact element count */
    PyObject *base;      /* owner of the memory when this tensor is a view (else NULL) */
} _Tensor;

static PyTypeObject _TensorType;

static size_t elem_size(int dtype) { return dtype == EMBER_BF16 ? 2 : 4; }

static PyObject *raise_status(int rc)
{
    PyObject *exc = rc == EMBER_ERR_INVALID ? PyExc_ValueError
                    : rc == EMBER_ERR_NOMEM ? PyExc_MemoryError
                                            : PyExc_RuntimeError;
    PyErr_Format(exc, "%s: %s", ember_status_string(rc), ember_last_error());
    return NULL;
}

/* ---- allocation helper: a result _Tensor with `n` device elements of `dtype` ---- */
static _Tensor *alloc_result(long long n, int dtype)
{
    _Tensor *t = (_Tensor *)_TensorType.tp_alloc(&_TensorType, 0);
    if (!t) return NULL;
    t->size64 = n;
    t->size = n > 2147483647LL ? 2147483647 : (int)n;
    t->dtype = dtype;
    t->base = NULL;
    t->d_ptr = alloc_memory((size_t)(n > 0 ? n : 1) * elem_size(dtype));
    if (!t->d_ptr) {
        Py_DECREF(t);
        PyErr_Format(PyExc_MemoryError, "Failed to allocate device memory: %s", ember_last_error());
        return NULL;
    }
    return t;
}

static void _Tensor_dealloc(_Tensor *self)
{
    if (self->base)
        Py_DECREF(self->base); /* a view: the owner frees the memory */
    else if (self->d_ptr)
        free_memory(self->d_ptr);
    Py_TYPE(self)->tp_free((PyObject *)self);
}

static int _Tensor_init(_Tensor *self, PyObject *args, PyObject *kwds)
{
    long long n = 0;
    int dtype = EMBER_F32;
    if (!PyArg_ParseTuple(args, "L|i", &n, &dtype)) return -1;
    if (n < 0 || (dtype != EMBER_F32 && dtype != EMBER_BF16)) {
        PyErr_SetString(PyExc_ValueError, "_Tensor(size, dtype): size must be >= 0 and dtype 0 or 1");
        return -1;
    }
    self->size64 = n;
    self->size = n > 2147483647LL ? 2147483647 : (int)n;
    self->dtype = dtype;
    self->base = NULL;
    self->d_ptr = alloc_memory((size_t)(n > 0 ? n : 1) * elem_size(dtype));
    if (!self->d_ptr) {
        PyErr_Format(PyExc_MemoryError, "Failed to allocate device memory: %s", ember_last_error());
        return -1;
    }
    return 0;
}

/* host float32 buffer -> this tensor (converted on the device when the tensor is bf16) */
static int upload_f32(_Tensor *t, const float *host, long long n)
{
    if (t->dtype == EMBER_F32) {
        copy_to_device(t->d_ptr, host, (size_t)n * 4);
        return 0;
    }
    void *stage = alloc_memory((size_t)n * 4);
    if (!stage) {
        PyErr_Format(PyExc_MemoryError, "Failed to allocate device memory: %s", ember_last_error());
        return -1;
    }
    copy_to_device(stage, host, (size_t)n * 4);
    int rc = ember_f32_to_bf16((const float *)stage, t->d_ptr, (size_t)n, NULL);
    free_memory(stage); /* stream-ordered: released after the conversion has run */
    if (rc) {
        raise_status(rc);
        return -1;
    }
    return 0;
}

/* _from_numpy(buffer, dtype=0): C-contiguous float32 buffer -> device tensor
 * (reference: tensor_api.c:151-186, which also insists on format "f"). */
static PyObject *_from_numpy(PyObject *module, PyObject *args)
{
    PyObject *obj;
    int dtype = EMBER_F32;
    if (!PyArg_ParseTuple(args, "O|i", &obj, &dtype)) return NULL;
    if (dtype != EMBER_F32 && dtype != EMBER_BF16) {
        PyErr_SetString(PyExc_ValueError, "dtype must be 0 (float32) or 1 (bfloat16)");
        return NULL;
    }
    Py_buffer view;
    if (PyObject_GetBuffer(obj, &view, PyBUF_C_CONTIGUOUS | PyBUF_FORMAT) < 0) return NULL;
    if (!view.format || view.format[0] != 'f' || view.format[1] != '\0' || view.itemsize != 4) {
        PyBuffer_Release(&view);
        PyErr_SetString(PyExc_TypeError, "Expected a C-contiguous float32 array");
        return NULL;
    }
    long long n = (long long)(view.len / 4);
    _Tensor *t = alloc_result(n, dtype);
    if (t && n > 0 && upload_f32(t, (const float *)view.buf, n) < 0) {
        Py_DECREF(t);
        t = NULL;
    }
    PyBuffer_Release(&view);
    return (PyObject *)t;
}

/* tensor._copy_to_buffer(writable float32 buffer): device -> host, widening bf16; waits for the
 * device like the reference's _to_np (tensor_api.c:132-149). */
static PyObject *_Tensor_copy_to_buffer(_Tensor *self, PyObject *args)
{
    PyObject *obj;
    if (!PyArg_ParseTuple(args, "O", &obj)) return NULL;
    Py_buffer view;
    if (PyObject_GetBuffer(obj, &view, PyBUF_C_CONTIGUOUS | PyBUF_WRITABLE | PyBUF_FORMAT) < 0) return NULL;
    if (!view.format || view.format[0] != 'f' || view.itemsize != 4 || (long long)(view.len / 4) != self->size64) {
        PyBuffer_Release(&view);
        PyErr_Format(PyExc_ValueError, "Expected a writable float32 buffer of %lld elements", self->size64);
        return NULL;
    }
    if (self->size64 > 0) {
        if (self->dtype == EMBER_F32) {
            copy_from_device(view.buf, self->d_ptr, (size_t)self->size64 * 4);
        } else {
            void *stage = alloc_memory((size_t)self->size64 * 4);
            if (!stage) {
                PyBuffer_Release(&view);
                PyErr_Format(PyExc_MemoryError, "Failed to allocate device memory: %s", ember_last_error());
                return NULL;
            }
            int rc = ember_bf16_to_f32(self->d_ptr, (float *)stage, (size_t)self->size64, NULL);
            if (!rc) copy_from_device(view.buf, stage, (size_t)self->size64 * 4);
            free_memory(stage);
            if (rc) {
                PyBuffer_Release(&view);
                return raise_status(rc);
            }
        }
    }
    PyBuffer_Release(&view);
    Py_RETURN_NONE;
}

static PyObject *_Tensor_ptr(_Tensor *self, PyObject *noargs)
{
    return PyLong_FromVoidPtr(self->d_ptr);
}

/* _convert(t, dtype) -> new tensor of the other storage type (or t itself) */
static PyObject *_convert(PyObject *module, PyObject *args)
{
    _Tensor *t;
    int dtype;
    if (!PyArg_ParseTuple(args, "O!i", &_TensorType, &t, &dtype)) return NULL;
    if (dtype == t->dtype) {
        Py_INCREF(t);
        return (PyObject *)t;
    }
    if (dtype != EMBER_F32 && dtype != EMBER_BF16) {
        PyErr_SetString(PyExc_ValueError, "dtype must be 0 (float32) or 1 (bfloat16)");
        return NULL;
    }
    _Tensor *out = alloc_result(t->size64, dtype);
    if (!out) return NULL;
    int rc = dtype == EMBER_BF16 ? ember_f32_to_bf16((const float *)t->d_ptr, out->d_ptr, (size_t)t->size64, NULL)
                                 : ember_bf16_to_f32(t->d_ptr, (float *)out->d_ptr, (size_t)t->size64, NULL);
    if (rc) {
        Py_DECREF(out);
        return raise_status(rc);
    }
    return (PyObject *)out;
}

static int check_sizes(const char *fn, _Tensor *q, _Tensor *k, _Tensor *v, long long bh, int lq, int lk, int d)
{
    if (bh <= 0 || lq <= 0 || lk <= 0 || d <= 0 || bh > 2147483647LL) {
        PyErr_Format(PyExc_ValueError, "%s: extents must be positive (B*H=%lld Lq=%d Lk=%d D=%d)", fn, bh, lq, lk, d);
        return -1;
    }
    if (q->size64 != bh * lq * d || k->size64 != bh * lk * d || v->size64 != k->size64) {
        PyErr_Format(PyExc_ValueError, "%s: size mismatch: q %lld (expected %lld), k %lld, v %lld (expected %lld)", fn,
                     q->size64, bh * lq * d, k->size64, v->size64, bh * lk * d);
        return -1;
    }
    if (q->dtype != k->dtype || k->dtype != v->dtype) {
        PyErr_Format(PyExc_TypeError, "%s: q, k and v must share a dtype", fn);
        return -1;
    }
    return 0;
}

/* _attention_fwd(q, k, v, B, H, Lq, Lk, D, scale, causal) -> (out, lse) */
static PyObject *_attention_fwd(PyObject *module, PyObject *args)
{
    _Tensor *q, *k, *v;
    int B, H, lq, lk, d, causal;
    float scale;
    if (!PyArg_ParseTuple(args, "O!O!O!iiiiifi", &_TensorType, &q, &_TensorType, &k, &_TensorType, &v, &B, &H, &lq,
                          &lk, &d, &scale, &causal))
        return NULL;
    const long long bh = (long long)B * H;
    if (check_sizes("attention", q, k, v, bh, lq, lk, d) < 0) return NULL;
    _Tensor *out = alloc_result(bh * lq * d, q->dtype);
    if (!out) return NULL;
    _Tensor *lse = alloc_result(bh * lq, EMBER_F32);
    if (!lse) {
        Py_DECREF(out);
        return NULL;
    }
    int rc = ember_attention_fwd(q->d_ptr, k->d_ptr, v->d_ptr, out->d_ptr, (float *)lse->d_ptr, (int)bh, lq, lk, d,
                                 scale, causal, q->dtype, NULL);
    if (rc) {
        Py_DECREF(out);
        Py_DECREF(lse);
        return raise_status(rc);
    }
    return Py_BuildValue("(NN)", out, lse);
}

/* _attention_bwd(q, k, v, out, lse, dout, B, H, Lq, Lk, D, scale, causal[, (dq, dk, dv)]) -> (dq, dk, dv)
 * The optional last argument supplies the three result tensors (for instance views of one buffer,
 * so that the gradients lie back to back); without it they are allocated. */
static PyObject *_attention_bwd(PyObject *module, PyObject *args)
{
    _Tensor *q, *k, *v, *o, *lse, *g;
    int B, H, lq, lk, d, causal;
    float scale;
    PyObject *outs = NULL;
    if (!PyArg_ParseTuple(args, "O!O!O!O!O!O!iiiiifi|O", &_TensorType, &q, &_TensorType, &k, &_TensorType, &v,
                          &_TensorType, &o, &_TensorType, &lse, &_TensorType, &g, &B, &H, &lq, &lk, &d, &scale, &causal,
                          &outs))
        return NULL;
    const long long bh = (long long)B * H;
    if (check_sizes("attention_backward", q, k, v, bh, lq, lk, d) < 0) return NULL;
    if (o->size64 != q->size64 || g->size64 != q->size64 || lse->size64 != bh * lq) {
        PyErr_Format(PyExc_ValueError, "attention_backward: size mismatch: out %lld, dout %lld (expected %lld), lse %lld (expected %lld)",
                     o->size64, g->size64, q->size64, lse->size64, bh * lq);
        return NULL;
    }
    if (o->dtype != q->dtype || g->dtype != q->dtype || lse->dtype != EMBER_F32) {
        PyErr_SetString(PyExc_TypeError, "attention_backward: out/dout must have q's dtype and lse must be float32");
        return NULL;
    }
    _Tensor *dq = NULL, *dk = NULL, *dv = NULL;
    void *ws = NULL;
    if (outs && outs != Py_None) {
        if (!PyArg_ParseTuple(outs, "O!O!O!", &_TensorType, &dq, &_TensorType, &dk, &_TensorType, &dv)) return NULL;
        if (dq->size64 != q->size64 || dk->size64 != k->size64 || dv->size64 != v->size64 || dq->dtype != q->dtype ||
            dk->dtype != q->dtype || dv->dtype != q->dtype) {
            PyErr_SetString(PyExc_ValueError, "attention_backward: the supplied result tensors do not match q, k and v");
            return NULL;
        }
        Py_INCREF(dq);
        Py_INCREF(dk);
        Py_INCREF(dv);
    } else {
        dq = alloc_result(q->size64, q->dtype);
        if (dq) dk = alloc_result(k->size64, q->dtype);
        if (dk) dv = alloc_result(v->size64, q->dtype);
    }
    const size_t wsn = ember_attention_workspace_bytes(EMBER_OP_BWD, (int)bh, lq, lk, d, q->dtype, 0);
    if (dv) {
        ws = alloc_memory(wsn);
        if (!ws) PyErr_Format(PyExc_MemoryError, "Failed to allocate device memory: %s", ember_last_error());
    }
    if (!ws) {
        Py_XDECREF(dq);
        Py_XDECREF(dk);
        Py_XDECREF(dv);
        return NULL;
    }
    int rc = ember_attention_bwd(q->d_ptr, k->d_ptr, v->d_ptr, o->d_ptr, (const float *)lse->d_ptr, g->d_ptr, dq->d_ptr,
                                 dk->d_ptr, dv->d_ptr, (int)bh, lq, lk, d, scale, causal, q->dtype, ws, wsn, NULL);
    free_memory(ws); /* stream-ordered: released after the kernels that use it */
    if (rc) {
        Py_DECREF(dq);
        Py_DECREF(dk);
        Py_DECREF(dv);
        return raise_status(rc);
    }
    return Py_BuildValue("(NNN)", dq, dk, dv);
}

/* _attention_decode(q, k, v, B, H, Lk, D, scale, num_splits) -> (out, lse) */
static PyObject *_attention_decode(PyObject *module, PyObject *args)
{
    _Tensor *q, *k, *v;
    int B, H, lk, d, splits;
    float scale;
    if (!PyArg_ParseTuple(args, "O!O!O!iiiifi", &_TensorType, &q, &_TensorType, &k, &_TensorType, &v, &B, &H, &lk, &d,
                          &scale, &splits))
        return NULL;
    const long long bh = (long long)B * H;
    if (check_sizes("attention_decode", q, k, v, bh, 1, lk, d) < 0) return NULL;
    _Tensor *out = alloc_result(bh * d, q->dtype);
    if (!out) return NULL;
    _Tensor *lse = alloc_result(bh, EMBER_F32);
    if (!lse) {
        Py_DECREF(out);
        return NULL;
    }
    const size_t wsn = ember_attention_workspace_bytes(EMBER_OP_DECODE, (int)bh, 1, lk, d, q->dtype, splits);
    void *ws = NULL;
    if (wsn) {
        ws = alloc_memory(wsn);
        if (!ws) {
            Py_DECREF(out);
            Py_DECREF(lse);
            PyErr_Format(PyExc_MemoryError, "Failed to allocate device memory: %s", ember_last_error());
            return NULL;
        }
    }
    int rc = ember_attention_decode(q->d_ptr, k->d_ptr, v->d_ptr, out->d_ptr, (float *)lse->d_ptr, (int)bh, lk, d, scale,
                                    q->dtype, splits, ws, wsn, NULL);
    if (ws) free_memory(ws);
    if (rc) {
        Py_DECREF(out);
        Py_DECREF(lse);
        return raise_status(rc);
    }
    return Py_BuildValue("(NN)", out, lse);
}

/* t._view(offset, size) -> a tensor over elements [offset, offset + size) of t's memory. The view
 * keeps t alive and never frees; it lets the three (B, H, L, D) tensors a fused q/k/v projection
 * writes back to back be handed to attention without a copy. */
static PyObject *_Tensor_view(_Tensor *self, PyObject *args)
{
    long long off, n;
    if (!PyArg_ParseTuple(args, "LL", &off, &n)) return NULL;
    if (off < 0 || n < 0 || off + n > self->size64) {
        PyErr_Format(PyExc_ValueError, "_view: [%lld, %lld) is outside a tensor of %lld elements", off, off + n,
                     self->size64);
        return NULL;
    }
    _Tensor *t = (_Tensor *)_TensorType.tp_alloc(&_TensorType, 0);
    if (!t) return NULL;
    t->size64 = n;
    t->size = n > 2147483647LL ? 2147483647 : (int)n;
    t->dtype = self->dtype;
    t->d_ptr = (char *)self->d_ptr + (size_t)off * elem_size(self->dtype);
    t->base = self->base ? self->base : (PyObject *)self;
    Py_INCREF(t->base);
    return (PyObject *)t;
}

/* _linear_fwd(x, w, bias | None, m, n, k, x_heads, y_heads, seq, head_dim) -> y
 * The reference's Linear.forward (ember/nn/layers.py:45-48) as one call. */
static PyObject *_linear_fwd(PyObject *module, PyObject *args)
{
    _Tensor *x, *w;
    PyObject *bias_o;
    long long m;
    int n, k, xh, yh, seq, hd;
    if (!PyArg_ParseTuple(args, "O!O!OLiiiiii", &_TensorType, &x, &_TensorType, &w, &bias_o, &m, &n, &k, &xh, &yh, &seq, &hd))
        return NULL;
    _Tensor *bias = NULL;
    if (bias_o != Py_None) {
        if (!PyObject_TypeCheck(bias_o, &_TensorType)) {
            PyErr_SetString(PyExc_TypeError, "linear: bias must be a _Tensor or None");
            return NULL;
        }
        bias = (_Tensor *)bias_o;
    }
    if (m <= 0 || n <= 0 || k <= 0 || x->size64 != m * k || w->size64 != (long long)k * n || (bias && bias->size64 != n)) {
        PyErr_Format(PyExc_ValueError, "linear: size mismatch: x %lld (expected %lld), w %lld (expected %lld), bias %lld (expected %d)",
                     x->size64, m * k, w->size64, (long long)k * n, bias ? bias->size64 : (long long)n, n);
        return NULL;
    }
    if (w->dtype != x->dtype || (bias && bias->dtype != x->dtype)) {
        PyErr_SetString(PyExc_TypeError, "linear: x, w and bias must share a dtype");
        return NULL;
    }
    _Tensor *y = alloc_result(m * n, x->dtype);
    if (!y) return NULL;
    int rc = ember_linear_fwd(x->d_ptr, w->d_ptr, bias ? bias->d_ptr : NULL, y->d_ptr, m, n, k, x->dtype, xh, yh, seq, hd, NULL);
    if (rc) {
        Py_DECREF(y);
        return raise_status(rc);
    }
    return (PyObject *)y;
}

/* _linear_bwd(x, w, grad_y, m, n, k, x_heads, y_heads, seq, head_dim, need_grad_x, need_grad_b)
 *   -> (grad_x | None, grad_w, grad_b | None): the reference's Linear.backward (layers.py:50-56). */
static PyObject *_linear_bwd(PyObject *module, PyObject *args)
{
    _Tensor *x, *w, *g;
    long long m;
    int n, k, xh, yh, seq, hd, need_dx, need_db;
    if (!PyArg_ParseTuple(args, "O!O!O!Liiiiiiii", &_TensorType, &x, &_TensorType, &w, &_TensorType, &g, &m, &n, &k, &xh,
                          &yh, &seq, &hd, &need_dx, &need_db))
        return NULL;
    if (m <= 0 || n <= 0 || k <= 0 || x->size64 != m * k || w->size64 != (long long)k * n || g->size64 != m * n) {
        PyErr_Format(PyExc_ValueError, "linear_backward: size mismatch: x %lld (expected %lld), w %lld (expected %lld), grad_y %lld (expected %lld)",
                     x->size64, m * k, w->size64, (long long)k * n, g->size64, m * n);
        return NULL;
    }
    if (w->dtype != x->dtype || g->dtype != x->dtype) {
        PyErr_SetString(PyExc_TypeError, "linear_backward: x, w and grad_y must share a dtype");
        return NULL;
    }
    _Tensor *dx = NULL, *dw = NULL, *db = NULL;
    dw = alloc_result((long long)k * n, x->dtype);
    if (dw && need_dx) dx = alloc_result(m * k, x->dtype);
    if (dw && (!need_dx || dx) && need_db) db = alloc_result(n, x->dtype);
    if (!dw || (need_dx && !dx) || (need_db && !db)) {
        Py_XDECREF(dx);
        Py_XDECREF(dw);
        Py_XDECREF(db);
        return NULL;
    }
    int rc = ember_linear_bwd(x->d_ptr, w->d_ptr, g->d_ptr, dx ? dx->d_ptr : NULL, dw->d_ptr, db ? db->d_ptr : NULL, m, n, k,
                              x->dtype, xh, yh, seq, hd, NULL);
    if (rc) {
        Py_XDECREF(dx);
        Py_DECREF(dw);
        Py_XDECREF(db);
        return raise_status(rc);
    }
    PyObject *odx = dx ? (PyObject *)dx : Py_NewRef(Py_None), *odb = db ? (PyObject *)db : Py_NewRef(Py_None);
    return Py_BuildValue("(NNN)", odx, dw, odb);
}

/* _softmax(x, rows, cols, log) -> y: softmax (log = 0) or log-softmax (log = 1) over the last axis. */
static PyObject *_softmax(PyObject *module, PyObject *args)
{
    _Tensor *x;
    long long rows;
    int cols, lg;
    if (!PyArg_ParseTuple(args, "O!Lii", &_TensorType, &x, &rows, &cols, &lg)) return NULL;
    if (rows <= 0 || cols <= 0 || x->size64 != rows * cols) {
        PyErr_Format(PyExc_ValueError, "softmax: size mismatch: tensor has %lld elements, rows*cols = %lld", x->size64,
                     rows * cols);
        return NULL;
    }
    _Tensor *y = alloc_result(x->size64, x->dtype);
    if (!y) return NULL;
    int rc = ember_softmax_fwd(x->d_ptr, y->d_ptr, rows, cols, x->dtype, lg, NULL);
    if (rc) {
        Py_DECREF(y);
        return raise_status(rc);
    }
    return (PyObject *)y;
}

/* _cross_entropy_fwd(pred, target, rows, cols) -> (loss, probs); loss is a 1-element float32 tensor.
 * CrossEntropyLoss.forward of the reference (ember/loss/losses.py:42-51). */
static PyObject *_cross_entropy_fwd(PyObject *module, PyObject *args)
{
    _Tensor *pred, *target;
    long long rows;
    int cols;
    if (!PyArg_ParseTuple(args, "O!O!Li", &_TensorType, &pred, &_TensorType, &target, &rows, &cols)) return NULL;
    if (rows <= 0 || cols <= 0 || pred->size64 != rows * cols || target->size64 != pred->size64) {
        PyErr_Format(PyExc_ValueError, "cross_entropy: size mismatch: pred %lld, target %lld, rows*cols = %lld",
                     pred->size64, target->size64, rows * cols);
        return NULL;
    }
    if (pred->dtype != target->dtype) {
        PyErr_SetString(PyExc_TypeError, "cross_entropy: pred and target must share a dtype");
        return NULL;
    }
    _Tensor *probs = alloc_result(pred->size64, pred->dtype), *loss = NULL;
    void *ws = NULL;
    const size_t wsn = ember_cross_entropy_workspace_bytes(rows);
    if (probs) loss = alloc_result(1, EMBER_F32);
    if (loss) {
        ws = alloc_memory(wsn);
        if (!ws) PyErr_Format(PyExc_MemoryError, "Failed to allocate device memory: %s", ember_last_error());
    }
    if (!ws) {
        Py_XDECREF(probs);
        Py_XDECREF(loss);
        return NULL;
    }
    int rc = ember_cross_entropy_fwd(pred->d_ptr, target->d_ptr, probs->d_ptr, (float *)loss->d_ptr, rows, cols, pred->dtype,
                                     ws, wsn, NULL);
    free_memory(ws); /* stream-ordered: released after the kernels that use it */
    if (rc) {
        Py_DECREF(probs);
        Py_DECREF(loss);
        return raise_status(rc);
    }
    return Py_BuildValue("(NN)", loss, probs);
}

/* _cross_entropy_bwd(probs, target, rows, cols) -> grad = (probs - target) / rows */
static PyObject *_cross_entropy_bwd(PyObject *module, PyObject *args)
{
    _Tensor *probs, *target;
    long long rows;
    int cols;
    if (!PyArg_ParseTuple(args, "O!O!Li", &_TensorType, &probs, &_TensorType, &target, &rows, &cols)) return NULL;
    if (rows <= 0 || cols <= 0 || probs->size64 != rows * cols || target->size64 != probs->size64 ||
        probs->dtype != target->dtype) {
        PyErr_SetString(PyExc_ValueError, "cross_entropy_backward: probs and target must both be (rows, cols) of one dtype");
        return NULL;
    }
    _Tensor *g = alloc_result(probs->size64, probs->dtype);
    if (!g) return NULL;
    int rc = ember_cross_entropy_bwd(probs->d_ptr, target->d_ptr, g->d_ptr, rows, cols, probs->dtype, NULL);
    if (rc) {
        Py_DECREF(g);
        return raise_status(rc);
    }
    return (PyObject *)g;
}

/* _kv_append(k_cache, v_cache, k_new, v_new, B, Hkv, capacity, D, n_new, pos) -> None
 * Writes (B, Hkv, n_new, D) rows into the (B, Hkv, capacity, D) caches at rows [pos, pos + n_new). */
static PyObject *_kv_append(PyObject *module, PyObject *args)
{
    _Tensor *kc, *vc, *kn, *vn;
    int B, H, cap, d, n_new, pos;
    if (!PyArg_ParseTuple(args, "O!O!O!O!iiiiii", &_TensorType, &kc, &_TensorType, &vc, &_TensorType, &kn, &_TensorType, &vn,
                          &B, &H, &cap, &d, &n_new, &pos))
        return NULL;
    const long long cache_n = (long long)B * H * cap * d, new_n = (long long)B * H * n_new * d;
    if (B <= 0 || H <= 0 || cap <= 0 || d <= 0 || n_new <= 0 || kc->size64 != cache_n || vc->size64 != cache_n ||
        kn->size64 != new_n || vn->size64 != new_n) {
        PyErr_Format(PyExc_ValueError, "kv_append: size mismatch: caches %lld/%lld (expected %lld), new rows %lld/%lld (expected %lld)",
                     kc->size64, vc->size64, cache_n, kn->size64, vn->size64, new_n);
        return NULL;
    }
    if (kc->dtype != vc->dtype || kn->dtype != kc->dtype || vn->dtype != kc->dtype) {
        PyErr_SetString(PyExc_TypeError, "kv_append: caches and new rows must share a dtype");
        return NULL;
    }
    int rc = ember_kv_cache_append(kc->d_ptr, vc->d_ptr, kn->d_ptr, vn->d_ptr, B, H, cap, d, n_new, pos, NULL, NULL, 0, 0,
                                   kc->dtype, NULL);
    if (rc) return raise_status(rc);
    Py_RETURN_NONE;
}

/* _decode_cache(q, k_cache, v_cache, B, Hq, Hkv, lk, capacity, D, scale, num_splits) -> (out, lse)
 * One query row per (batch, query head) against the first lk rows of the caches. */
static PyObject *_decode_cache(PyObject *module, PyObject *args)
{
    _Tensor *q, *kc, *vc;
    int B, Hq, Hkv, lk, cap, d, splits;
    float scale;
    if (!PyArg_ParseTuple(args, "O!O!O!iiiiiifi", &_TensorType, &q, &_TensorType, &kc, &_TensorType, &vc, &B, &Hq, &Hkv, &lk,
                          &cap, &d, &scale, &splits))
        return NULL;
    const long long cache_n = (long long)B * Hkv * cap * d;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || cap <= 0 || d <= 0 || q->size64 != (long long)B * Hq * d || kc->size64 != cache_n ||
        vc->size64 != cache_n) {
        PyErr_Format(PyExc_ValueError, "decode_cache: size mismatch: q %lld (expected %lld), caches %lld/%lld (expected %lld)",
                     q->size64, (long long)B * Hq * d, kc->size64, vc->size64, cache_n);
        return NULL;
    }
    if (kc->dtype != q->dtype || vc->dtype != q->dtype) {
        PyErr_SetString(PyExc_TypeError, "decode_cache: q and the caches must share a dtype");
        return NULL;
    }
    _Tensor *out = alloc_result(q->size64, q->dtype), *lse = NULL;
    void *ws = NULL;
    const size_t wsn = ember_attention_decode_cache_workspace_bytes(B, Hq, Hkv, lk, d, splits);
    if (out) lse = alloc_result((long long)B * Hq, EMBER_F32);
    if (lse) {
        ws = alloc_memory(wsn ? wsn : 256);
        if (!ws) PyErr_Format(PyExc_MemoryError, "Failed to allocate device memory: %s", ember_last_error());
    }
    if (!ws) {
        Py_XDECREF(out);
        Py_XDECREF(lse);
        return NULL;
    }
    int rc = ember_attention_decode_cache(q->d_ptr, kc->d_ptr, vc->d_ptr, out->d_ptr, (float *)lse->d_ptr, B, Hq, Hkv, lk, cap, d,
                                          scale, q->dtype, NULL, NULL, 0, 0, splits, ws, wsn, NULL);
    free_memory(ws); /* stream-ordered: released after the kernels that use it */
    if (rc) {
        Py_DECREF(out);
        Py_DECREF(lse);
        return raise_status(rc);
    }
    return Py_BuildValue("(NN)", out, lse);
}

static PyObject *_sync(PyObject *module, PyObject *noargs)
{
    sync_device();
    Py_RETURN_NONE;
}

static PyMethodDef _Tensor_methods[] = {
    {"_copy_to_buffer", (PyCFunction)_Tensor_copy_to_buffer, METH_VARARGS, "Copy to a writable float32 host buffer"},
    {"_ptr", (PyCFunction)_Tensor_ptr, METH_NOARGS, "Device address as an int"},
    {"_view", (PyCFunction)_Tensor_view, METH_VARARGS, "A tensor over a range of this tensor's elements"},
    {NULL}};

static PyMemberDef _Tensor_members[] = {{"size", T_LONGLONG, offsetof(_Tensor, size64), READONLY, "element count"},
                                        {"dtype", T_INT, offsetof(_Tensor, dtype), READONLY, "0 float32, 1 bfloat16"},
                                        {NULL}};

#define OP_METHOD(NAME) {#NAME, (PyCFunction)NAME, METH_VARARGS, "Attention path: " #NAME}

static PyMethodDef module_methods[] = {OP_METHOD(_from_numpy),
                                       OP_METHOD(_convert),
                                       OP_METHOD(_attention_fwd),
                                       OP_METHOD(_attention_bwd),
                                       OP_METHOD(_attention_decode),
                                       OP_METHOD(_linear_fwd),
                                       OP_METHOD(_linear_bwd),
                                       OP_METHOD(_softmax),
                                       OP_METHOD(_cross_entropy_fwd),
                                       OP_METHOD(_cross_entropy_bwd),
                                       OP_METHOD(_kv_append),
                                       OP_METHOD(_decode_cache),
                                       {"_sync", (PyCFunction)_sync, METH_NOARGS, "Wait for the library stream"},
                                       {NULL, NULL, 0, NULL}};

static struct PyModuleDef tensor_module = {PyModuleDef_HEAD_INIT, "_tensor",
                                           "B200 attention path behind the reference's binding surface", -1, module_methods};

static PyTypeObject _TensorType = {
    PyVarObject_HEAD_INIT(NULL, 0).tp_name = "ember_b200._core._tensor._Tensor",
    .tp_basicsize = sizeof(_Tensor),
    .tp_flags = Py_TPFLAGS_DEFAULT,
    .tp_new = PyType_GenericNew,
    .tp_init = (initproc)_Tensor_init,
    .tp_dealloc = (destructor)_Tensor_dealloc,
    .tp_methods = _Tensor_methods,
    .tp_members = _Tensor_members,
};

PyMODINIT_FUNC PyInit__tensor(void)
{
    if (PyType_Ready(&_TensorType) < 0) return NULL;
    PyObject *m = PyModule_Create(&tensor_module);
    if (!m) return NULL;
    Py_INCREF(&_TensorType);
    if (PyModule_AddObject(m, "_Tensor", (PyObject *)&_TensorType) < 0) {
        Py_DECREF(&_TensorType);
        Py_DECREF(m);
        return NULL;
    }
    PyModule_AddIntConstant(m, "F32", EMBER_F32);
    PyModule_AddIntConstant(m, "BF16", EMBER_BF16);
    return m;
}
