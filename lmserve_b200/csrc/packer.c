/* Host-side packing of one step's request list into the int32 upload buffer of
 * lms_build_step_indices, as a CPython extension module (lmserve_b200._packer).
 *
 * LMServe's model worker walks the request list in Python and builds one list per index array
 * (runtime/worker/llm_worker/model_worker.py:330-407); converting those lists element by element
 * is what its per-step preparation costs.  This module walks the same request objects in C and
 * writes
 *     [input_len | filled_token_len | context_len | len(block_ids)]   (batch entries each)
 *     block_ids of every request, concatenated
 *     input_ids of every request, concatenated
 * straight into a caller-provided buffer (the pinned staging memory).  The requests are any
 * objects with the InferInput attributes of proto/worker.proto:40-47; block_ids and input_ids are
 * any sequences of integers.  Sorting stays with the caller (list.sort, as the reference does).
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <stdint.h>

/* Attribute names, interned once at module start-up (a lookup by C string builds a new str
 * object per call). */
static PyObject *s_input_len, *s_filled_token_len, *s_context_len, *s_block_ids, *s_input_ids;

/* Value of a Python int: the one-digit ("compact") form that every id, length and position here
 * has is read in place; anything else takes the general conversion. */
static inline int as_i32(PyObject* v, int32_t* out, const char* what) {
  long long x;
#if PY_VERSION_HEX >= 0x030C0000
  if (PyLong_CheckExact(v) && PyUnstable_Long_IsCompact((const PyLongObject*)v)) {
    x = (long long)PyUnstable_Long_CompactValue((const PyLongObject*)v);
  } else
#endif
  {
    x = PyLong_AsLongLong(v);
    if (x == -1 && PyErr_Occurred()) return -1;
  }
  if (x < INT32_MIN || x > INT32_MAX) {
    PyErr_Format(PyExc_OverflowError, "%s does not fit 32 bits", what);
    return -1;
  }
  *out = (int32_t)x;
  return 0;
}

static int get_i32(PyObject* obj, PyObject* name, const char* what, int32_t* out) {
  PyObject* v = PyObject_GetAttr(obj, name);
  if (!v) return -1;
  const int rc = as_i32(v, out, what);
  Py_DECREF(v);
  return rc;
}

/* Copies the integers of `seq` (already a list or tuple) to dst[0..n). */
static int copy_ints(PyObject* fast, Py_ssize_t n, int32_t* dst, const char* what) {
  PyObject** items = PySequence_Fast_ITEMS(fast);
  for (Py_ssize_t i = 0; i < n; ++i)
    if (as_i32(items[i], dst + i, what)) return -1;
  return 0;
}

/* pack(inputs, out) -> (batch, total_tokens, total_blocks, prefill_input_len, num_prefill, num_decode,
 *                       prefill_blocks, decode_blocks)
 * `out` is a writable, C-contiguous buffer of int32 (a numpy array); ValueError when it is too
 * small or when a request is inconsistent, with the messages of the pure-Python packer. */
static PyObject* pack(PyObject* self, PyObject* args) {
  PyObject* inputs;
  Py_buffer out;
  if (!PyArg_ParseTuple(args, "Ow*", &inputs, &out)) return NULL;
  PyObject* result = NULL;
  PyObject* reqs = PySequence_Fast(inputs, "inputs must be a sequence of requests");
  PyObject** blocks = NULL;
  PyObject** ids = NULL;
  Py_ssize_t batch = 0;
  if (!reqs) goto done;
  if (out.itemsize != 4 && out.itemsize != 1) {
    PyErr_SetString(PyExc_TypeError, "out must be an int32 (or byte) buffer");
    goto done;
  }
  batch = PySequence_Fast_GET_SIZE(reqs);
  {
    const Py_ssize_t cap = out.len / 4;
    int32_t* buf = (int32_t*)out.buf;
    if (4 * batch > cap) {
      PyErr_Format(PyExc_ValueError, "step needs at least %zd int32 words of staging, the buffer has %zd",
                   4 * batch, cap);
      goto done;
    }
    blocks = (PyObject**)PyMem_Calloc(batch ? batch : 1, sizeof(PyObject*));
    ids = (PyObject**)PyMem_Calloc(batch ? batch : 1, sizeof(PyObject*));
    if (!blocks || !ids) {
      PyErr_NoMemory();
      goto done;
    }
    long long total_tokens = 0, total_blocks = 0, prefill_len = 0, n_pre = 0, n_dec = 0;
    long long prefill_blocks = 0, decode_blocks = 0;
    for (Py_ssize_t b = 0; b < batch; ++b) {
      PyObject* r = PySequence_Fast_GET_ITEM(reqs, b);
      int32_t q, filled, ctx;
      if (get_i32(r, s_input_len, "input_len", &q) ||
          get_i32(r, s_filled_token_len, "filled_token_len", &filled) ||
          get_i32(r, s_context_len, "context_len", &ctx))
        goto done;
      PyObject* a = PyObject_GetAttr(r, s_block_ids);
      if (!a) goto done;
      blocks[b] = PySequence_Fast(a, "block_ids must be a sequence");
      Py_DECREF(a);
      if (!blocks[b]) goto done;
      a = PyObject_GetAttr(r, s_input_ids);
      if (!a) goto done;
      ids[b] = PySequence_Fast(a, "input_ids must be a sequence");
      Py_DECREF(a);
      if (!ids[b]) goto done;
      const Py_ssize_t n_ids = PySequence_Fast_GET_SIZE(ids[b]);
      if (n_ids != q) {
        PyErr_Format(PyExc_ValueError, "request %zd: input_len %d but %zd input ids", b, (int)q, n_ids);
        goto done;
      }
      if ((long long)ctx - filled != q) {
        PyErr_Format(PyExc_ValueError,
                     "request %zd: context_len - filled_token_len = %lld but input_len = %d", b,
                     (long long)ctx - filled, (int)q);
        goto done;
      }
      const Py_ssize_t nb = PySequence_Fast_GET_SIZE(blocks[b]);
      if (q > 1) {
        prefill_len += q;
        ++n_pre;
        prefill_blocks += nb;
      } else if (q == 1) {
        ++n_dec;
        decode_blocks += nb;
      }
      buf[b] = q;
      buf[batch + b] = filled;
      buf[2 * batch + b] = ctx;
      buf[3 * batch + b] = (int32_t)nb;
      total_tokens += q > 0 ? q : 0;
      total_blocks += nb;
    }
    const long long need = 4 * (long long)batch + total_blocks + total_tokens;
    if (need > cap || total_blocks > INT32_MAX || total_tokens > INT32_MAX) {
      PyErr_Format(PyExc_ValueError, "step needs %lld int32 words of staging, the buffer has %zd", need, cap);
      goto done;
    }
    int32_t* dst = buf + 4 * batch;
    for (Py_ssize_t b = 0; b < batch; ++b) {
      const Py_ssize_t nb = PySequence_Fast_GET_SIZE(blocks[b]);
      if (copy_ints(blocks[b], nb, dst, "block_ids")) goto done;
      dst += nb;
    }
    for (Py_ssize_t b = 0; b < batch; ++b) {
      const Py_ssize_t n = PySequence_Fast_GET_SIZE(ids[b]);
      if (copy_ints(ids[b], n, dst, "input_ids")) goto done;
      dst += n;
    }
    result = Py_BuildValue("(nLLLLLLL)", batch, total_tokens, total_blocks, prefill_len, n_pre, n_dec,
                           prefill_blocks, decode_blocks);
  }
done:
  if (blocks)
    for (Py_ssize_t b = 0; b < batch; ++b) Py_XDECREF(blocks[b]);
  if (ids)
    for (Py_ssize_t b = 0; b < batch; ++b) Py_XDECREF(ids[b]);
  PyMem_Free(blocks);
  PyMem_Free(ids);
  Py_XDECREF(reqs);
  PyBuffer_Release(&out);
  return result;
}

/* flatten_dict(src_to_dst, out) -> n: writes the (src, dst) pairs of {src: [dst, ...]} - the
 * argument of LMServe's copy_blocks (ops/cache_ops.py:8-15) - into the int64 buffer `out`
 * ([n, 2], row-major) in the dict's iteration order.  ValueError if `out` is too small. */
static PyObject* flatten_dict(PyObject* self, PyObject* args) {
  PyObject* d;
  Py_buffer out;
  if (!PyArg_ParseTuple(args, "O!w*", &PyDict_Type, &d, &out)) return NULL;
  int64_t* dst = (int64_t*)out.buf;
  const Py_ssize_t cap = out.len / 16;
  Py_ssize_t n = 0, pos = 0;
  PyObject *key, *value;
  PyObject* result = NULL;
  while (PyDict_Next(d, &pos, &key, &value)) {
    const long long src = PyLong_AsLongLong(key);
    if (src == -1 && PyErr_Occurred()) goto done;
    PyObject* fast = PySequence_Fast(value, "destinations must be a sequence of block ids");
    if (!fast) goto done;
    const Py_ssize_t m = PySequence_Fast_GET_SIZE(fast);
    if (n + m > cap) {
      Py_DECREF(fast);
      PyErr_SetString(PyExc_ValueError, "pair buffer too small for the block map");
      goto done;
    }
    PyObject** items = PySequence_Fast_ITEMS(fast);
    for (Py_ssize_t i = 0; i < m; ++i) {
      const long long dd = PyLong_AsLongLong(items[i]);
      if (dd == -1 && PyErr_Occurred()) {
        Py_DECREF(fast);
        goto done;
      }
      dst[2 * (n + i)] = src;
      dst[2 * (n + i) + 1] = dd;
    }
    n += m;
    Py_DECREF(fast);
  }
  result = PyLong_FromSsize_t(n);
done:
  PyBuffer_Release(&out);
  return result;
}

static int get_i64(PyObject* obj, PyObject* name, int64_t* out) {
  PyObject* v = PyObject_GetAttr(obj, name);
  if (!v) return -1;
  const long long x = PyLong_AsLongLong(v);
  Py_DECREF(v);
  if (x == -1 && PyErr_Occurred()) return -1;
  *out = x;
  return 0;
}

/* flatten_entries(entries, out) -> n: (e.src_block_id, e.dst_block_id) of every entry of a
 * BlockMapping (proto/worker.proto:78-86) into the int64 buffer `out` ([n, 2]). */
static PyObject* flatten_entries(PyObject* self, PyObject* args) {
  PyObject* entries;
  Py_buffer out;
  if (!PyArg_ParseTuple(args, "Ow*", &entries, &out)) return NULL;
  PyObject* result = NULL;
  PyObject* src_name = PyUnicode_InternFromString("src_block_id");
  PyObject* dst_name = PyUnicode_InternFromString("dst_block_id");
  PyObject* fast = PySequence_Fast(entries, "entries must be a sequence");
  if (!fast || !src_name || !dst_name) goto done;
  {
    const Py_ssize_t n = PySequence_Fast_GET_SIZE(fast);
    if (n > out.len / 16) {
      PyErr_SetString(PyExc_ValueError, "pair buffer too small for the entries");
      goto done;
    }
    int64_t* dst = (int64_t*)out.buf;
    for (Py_ssize_t i = 0; i < n; ++i) {
      PyObject* e = PySequence_Fast_GET_ITEM(fast, i);
      if (get_i64(e, src_name, dst + 2 * i) || get_i64(e, dst_name, dst + 2 * i + 1)) goto done;
    }
    result = PyLong_FromSsize_t(n);
  }
done:
  Py_XDECREF(fast);
  Py_XDECREF(src_name);
  Py_XDECREF(dst_name);
  PyBuffer_Release(&out);
  return result;
}

/* call_plan(fn_address, plan_handle, stream) -> status
 *
 * Calls an `int fn(const void* plan, void* stream)` entry point of the C ABI (lms_write_plan_run)
 * through its address.  The decode loop issues one such call per layer per step; going through
 * ctypes costs about a microsecond per call in argument conversion, a third of what the launch
 * itself takes.  The three arguments are plain integers (addresses), nothing is dereferenced
 * here. */
typedef int (*plan_run_fn)(const void*, void*);

static PyObject* call_plan(PyObject* self, PyObject* const* args, Py_ssize_t nargs) {
  (void)self;
  if (nargs != 3) {
    PyErr_SetString(PyExc_TypeError, "call_plan(fn_address, plan_handle, stream)");
    return NULL;
  }
  void* fn = PyLong_AsVoidPtr(args[0]);
  void* plan = PyLong_AsVoidPtr(args[1]);
  void* stream = PyLong_AsVoidPtr(args[2]);
  if (PyErr_Occurred()) return NULL;
  if (fn == NULL) {
    PyErr_SetString(PyExc_ValueError, "call_plan: NULL function address");
    return NULL;
  }
  plan_run_fn run;
  memcpy(&run, &fn, sizeof(run)); /* object pointer -> function pointer without a cast warning */
  return PyLong_FromLong((long)run(plan, stream));
}

static PyMethodDef methods[] = {
    {"flatten_dict", flatten_dict, METH_VARARGS, "flatten_dict(src_to_dst, out) -> number of pairs"},
    {"flatten_entries", flatten_entries, METH_VARARGS, "flatten_entries(entries, out) -> number of pairs"},
    {"pack", pack, METH_VARARGS,
     "pack(inputs, out) -> (batch, total_tokens, total_blocks, prefill_input_len, num_prefill, num_decode, "
     "prefill_blocks, decode_blocks)"},
    {"call_plan", (PyCFunction)(void (*)(void))call_plan, METH_FASTCALL,
     "call_plan(fn_address, plan_handle, stream) -> status of int fn(plan, stream)"},
    {NULL, NULL, 0, NULL}};

static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, "_packer",
                                    "Packs a step's request list into the index-preparation upload buffer.",
                                    -1, methods};

PyMODINIT_FUNC PyInit__packer(void) {
  s_input_len = PyUnicode_InternFromString("input_len");
  s_filled_token_len = PyUnicode_InternFromString("filled_token_len");
  s_context_len = PyUnicode_InternFromString("context_len");
  s_block_ids = PyUnicode_InternFromString("block_ids");
  s_input_ids = PyUnicode_InternFromString("input_ids");
  if (!s_input_len || !s_filled_token_len || !s_context_len || !s_block_ids || !s_input_ids) return NULL;
  return PyModule_Create(&module);
}
