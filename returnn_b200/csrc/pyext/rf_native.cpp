// CPython extension with the dimension bookkeeping of the frontend in native code. Every RF op on named-dim tensors starts with
// the same small computations on tuples of Dim objects (which axis of a goes where in b, the merged dims of a binary op); in
// Python these loops cost more than launching the kernel that follows. The functions compare dims by identity first and fall
// back to ``==`` (Dim.__eq__), like the Python versions in returnn_b200/tensor/tensor.py and returnn_b200/frontend/_utils.py,
// which remain the specification and the fallback.
//
// Reference counterpart: returnn/frontend/_native/*.cpp (tensor_ops.cpp, module.cpp: native versions of
// Tensor.copy_compatible_to_dims_raw, get_out_permutation_to_dims and the binary-op fast path).
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <vector>

namespace {

// 1 equal, 0 different, -1 error
int dim_equal(PyObject* a, PyObject* b) {
  if (a == b) return 1;
  return PyObject_RichCompareBool(a, b, Py_EQ);
}

bool as_fast_seq(PyObject* obj, const char* what, PyObject** out) {
  *out = PySequence_Fast(obj, what);
  return *out != nullptr;
}

// match_dims(own, dims) -> list: for every entry of dims the index in own of the first unused equal dim, or -1
PyObject* match_dims(PyObject*, PyObject* args) {
  PyObject *own_o, *dims_o;
  if (!PyArg_ParseTuple(args, "OO", &own_o, &dims_o)) return nullptr;
  PyObject *own, *dims;
  if (!as_fast_seq(own_o, "own must be a sequence", &own)) return nullptr;
  if (!as_fast_seq(dims_o, "dims must be a sequence", &dims)) {
    Py_DECREF(own);
    return nullptr;
  }
  const Py_ssize_t n_own = PySequence_Fast_GET_SIZE(own), n = PySequence_Fast_GET_SIZE(dims);
  std::vector<char> used((size_t)n_own, 0);
  PyObject* res = PyList_New(n);
  if (!res) {
    Py_DECREF(own);
    Py_DECREF(dims);
    return nullptr;
  }
  for (Py_ssize_t j = 0; j < n; ++j) {
    PyObject* d = PySequence_Fast_GET_ITEM(dims, j);
    long found = -1;
    for (Py_ssize_t i = 0; i < n_own; ++i) {
      if (used[(size_t)i]) continue;
      const int eq = dim_equal(PySequence_Fast_GET_ITEM(own, i), d);
      if (eq < 0) {
        Py_DECREF(res);
        Py_DECREF(own);
        Py_DECREF(dims);
        return nullptr;
      }
      if (eq) {
        found = (long)i;
        used[(size_t)i] = 1;
        break;
      }
    }
    PyList_SET_ITEM(res, j, PyLong_FromLong(found));
  }
  Py_DECREF(own);
  Py_DECREF(dims);
  return res;
}

// same_dims(a, b) -> bool: equal length and pairwise equal
PyObject* same_dims(PyObject*, PyObject* args) {
  PyObject *a_o, *b_o;
  if (!PyArg_ParseTuple(args, "OO", &a_o, &b_o)) return nullptr;
  PyObject *a, *b;
  if (!as_fast_seq(a_o, "a must be a sequence", &a)) return nullptr;
  if (!as_fast_seq(b_o, "b must be a sequence", &b)) {
    Py_DECREF(a);
    return nullptr;
  }
  bool same = PySequence_Fast_GET_SIZE(a) == PySequence_Fast_GET_SIZE(b);
  for (Py_ssize_t i = 0; same && i < PySequence_Fast_GET_SIZE(a); ++i) {
    const int eq = dim_equal(PySequence_Fast_GET_ITEM(a, i), PySequence_Fast_GET_ITEM(b, i));
    if (eq < 0) {
      Py_DECREF(a);
      Py_DECREF(b);
      return nullptr;
    }
    same = eq != 0;
  }
  Py_DECREF(a);
  Py_DECREF(b);
  if (same) Py_RETURN_TRUE;
  Py_RETURN_FALSE;
}

int contains(PyObject* seq, PyObject* d) {
  for (Py_ssize_t i = 0; i < PySequence_Fast_GET_SIZE(seq); ++i) {
    const int eq = dim_equal(PySequence_Fast_GET_ITEM(seq, i), d);
    if (eq) return eq;
  }
  return 0;
}

// 1 if every dim of a occurs in b, 0 if not, -1 on error
int subset(PyObject* a, PyObject* b) {
  for (Py_ssize_t i = 0; i < PySequence_Fast_GET_SIZE(a); ++i) {
    const int c = contains(b, PySequence_Fast_GET_ITEM(a, i));
    if (c <= 0) return c;
  }
  return 1;
}

// merge_dims(ad, bd) -> tuple: the dims of a binary op's result. The operand whose dims contain the other's keeps its order
// (the longer one first); otherwise a's dims followed by the dims only b has.
PyObject* merge_dims(PyObject*, PyObject* args) {
  PyObject *a_o, *b_o;
  if (!PyArg_ParseTuple(args, "OO", &a_o, &b_o)) return nullptr;
  PyObject *a, *b;
  if (!as_fast_seq(a_o, "a must be a sequence", &a)) return nullptr;
  if (!as_fast_seq(b_o, "b must be a sequence", &b)) {
    Py_DECREF(a);
    return nullptr;
  }
  const Py_ssize_t na = PySequence_Fast_GET_SIZE(a), nb = PySequence_Fast_GET_SIZE(b);
  PyObject* res = nullptr;
  auto as_tuple = [](PyObject* s) { return PySequence_Tuple(s); };
  int a_in_b = 0, b_in_a = 0;
  if (nb == 0) res = as_tuple(a);
  else if (na == 0) res = as_tuple(b);
  else {
    a_in_b = subset(a, b);
    if (a_in_b >= 0) b_in_a = subset(b, a);
    if (a_in_b < 0 || b_in_a < 0) {
      Py_DECREF(a);
      Py_DECREF(b);
      return nullptr;
    }
    if (nb > na && a_in_b) res = as_tuple(b);
    else if (b_in_a) res = as_tuple(a);
    else if (a_in_b) res = as_tuple(b);
    else {
      std::vector<PyObject*> extra;
      for (Py_ssize_t i = 0; i < nb; ++i) {
        PyObject* d = PySequence_Fast_GET_ITEM(b, i);
        const int c = contains(a, d);
        if (c < 0) {
          Py_DECREF(a);
          Py_DECREF(b);
          return nullptr;
        }
        if (!c) extra.push_back(d);
      }
      res = PyTuple_New(na + (Py_ssize_t)extra.size());
      if (res) {
        for (Py_ssize_t i = 0; i < na; ++i) {
          PyObject* d = PySequence_Fast_GET_ITEM(a, i);
          Py_INCREF(d);
          PyTuple_SET_ITEM(res, i, d);
        }
        for (size_t i = 0; i < extra.size(); ++i) {
          Py_INCREF(extra[i]);
          PyTuple_SET_ITEM(res, na + (Py_ssize_t)i, extra[i]);
        }
      }
    }
  }
  Py_DECREF(a);
  Py_DECREF(b);
  return res;
}

// ---------------------------------------------------------------------------------------------------------------------------
// raw-tensor side: the view of a raw tensor whose axes follow another dim order (axes the tensor lacks get size 1), and the
// preparation of a binary op. The raw tensor is only touched through its own methods (permute, __getitem__), so any array type
// with these works.

// view of `raw` (axes `own`) with axes in the order of `dims`; new reference, or nullptr with an exception set.
// `own` and `dims` are fast sequences.
PyObject* compatible_raw(PyObject* raw, PyObject* own, PyObject* dims) {
  const Py_ssize_t n_own = PySequence_Fast_GET_SIZE(own), n = PySequence_Fast_GET_SIZE(dims);
  std::vector<char> used((size_t)n_own, 0);
  std::vector<long> found((size_t)n, -1);
  bool identity = n == n_own;
  Py_ssize_t n_found = 0;
  for (Py_ssize_t j = 0; j < n; ++j) {
    PyObject* d = PySequence_Fast_GET_ITEM(dims, j);
    for (Py_ssize_t i = 0; i < n_own; ++i) {
      if (used[(size_t)i]) continue;
      const int eq = dim_equal(PySequence_Fast_GET_ITEM(own, i), d);
      if (eq < 0) return nullptr;
      if (eq) {
        found[(size_t)j] = (long)i;
        used[(size_t)i] = 1;
        ++n_found;
        break;
      }
    }
    if (found[(size_t)j] != (long)j) identity = false;
  }
  if (n_found != n_own) {
    PyErr_Format(PyExc_ValueError, "tensor dims %R are not all in the target dims %R", own, dims);
    return nullptr;
  }
  if (identity) {
    Py_INCREF(raw);
    return raw;
  }
  PyObject* cur = raw;
  Py_INCREF(cur);
  // permute when the existing axes change their relative order
  bool sorted = true;
  long last = -1;
  for (Py_ssize_t j = 0; j < n; ++j) {
    if (found[(size_t)j] < 0) continue;
    if (found[(size_t)j] < last) sorted = false;
    last = found[(size_t)j];
  }
  if (!sorted) {
    PyObject* perm = PyTuple_New(n_own);
    if (!perm) {
      Py_DECREF(cur);
      return nullptr;
    }
    Py_ssize_t k = 0;
    for (Py_ssize_t j = 0; j < n; ++j)
      if (found[(size_t)j] >= 0) PyTuple_SET_ITEM(perm, k++, PyLong_FromLong(found[(size_t)j]));
    PyObject* meth = PyObject_GetAttrString(cur, "permute");
    PyObject* res = meth ? PyObject_CallObject(meth, perm) : nullptr;
    Py_XDECREF(meth);
    Py_DECREF(perm);
    Py_DECREF(cur);
    if (!res) return nullptr;
    cur = res;
  }
  if (n != n_own) {  // raw[None / slice(None), ...]: size-1 axes where the tensor has no such dim
    PyObject* key = PyTuple_New(n);
    PyObject* full = key ? PySlice_New(nullptr, nullptr, nullptr) : nullptr;
    if (!key || !full) {
      Py_XDECREF(key);
      Py_XDECREF(full);
      Py_DECREF(cur);
      return nullptr;
    }
    for (Py_ssize_t j = 0; j < n; ++j) {
      PyObject* item = found[(size_t)j] < 0 ? Py_None : full;
      Py_INCREF(item);
      PyTuple_SET_ITEM(key, j, item);
    }
    Py_DECREF(full);
    PyObject* res = PyObject_GetItem(cur, key);
    Py_DECREF(key);
    Py_DECREF(cur);
    if (!res) return nullptr;
    cur = res;
  }
  return cur;
}

// copy_compatible_raw(raw, own_dims, target_dims) -> raw view
PyObject* copy_compatible_raw(PyObject*, PyObject* args) {
  PyObject *raw, *own_o, *dims_o;
  if (!PyArg_ParseTuple(args, "OOO", &raw, &own_o, &dims_o)) return nullptr;
  PyObject *own, *dims;
  if (!as_fast_seq(own_o, "own must be a sequence", &own)) return nullptr;
  if (!as_fast_seq(dims_o, "dims must be a sequence", &dims)) {
    Py_DECREF(own);
    return nullptr;
  }
  PyObject* res = compatible_raw(raw, own, dims);
  Py_DECREF(own);
  Py_DECREF(dims);
  return res;
}

// bin_op_prepare(a_raw, a_dims, b_raw, b_dims) -> (a_view, b_view, out_dims): both operands as views over the merged dims of a
// binary op. Fast paths without any matching work: the very same dims tuple, or one operand without dims (a scalar).
PyObject* bin_op_prepare(PyObject* self, PyObject* args) {
  PyObject *a_raw, *a_dims_o, *b_raw, *b_dims_o;
  if (!PyArg_ParseTuple(args, "OOOO", &a_raw, &a_dims_o, &b_raw, &b_dims_o)) return nullptr;
  if (a_dims_o == b_dims_o && PyTuple_Check(a_dims_o)) return PyTuple_Pack(3, a_raw, b_raw, a_dims_o);
  PyObject *ad, *bd;
  if (!as_fast_seq(a_dims_o, "a dims must be a sequence", &ad)) return nullptr;
  if (!as_fast_seq(b_dims_o, "b dims must be a sequence", &bd)) {
    Py_DECREF(ad);
    return nullptr;
  }
  PyObject* res = nullptr;
  const Py_ssize_t na = PySequence_Fast_GET_SIZE(ad), nb = PySequence_Fast_GET_SIZE(bd);
  if (nb == 0 || na == 0) {
    PyObject* out = PySequence_Tuple(nb == 0 ? ad : bd);
    if (out) {
      res = PyTuple_Pack(3, a_raw, b_raw, out);
      Py_DECREF(out);
    }
  } else {
    PyObject* margs = PyTuple_Pack(2, ad, bd);
    PyObject* out = margs ? merge_dims(self, margs) : nullptr;
    Py_XDECREF(margs);
    if (out) {
      PyObject* av = compatible_raw(a_raw, ad, out);
      PyObject* bv = av ? compatible_raw(b_raw, bd, out) : nullptr;
      if (av && bv) res = PyTuple_Pack(3, av, bv, out);
      Py_XDECREF(av);
      Py_XDECREF(bv);
      Py_DECREF(out);
    }
  }
  Py_DECREF(ad);
  Py_DECREF(bd);
  return res;
}

PyMethodDef methods[] = {
    {"match_dims", match_dims, METH_VARARGS, "for every dim of `dims` the index in `own` of the first unused equal dim, or -1"},
    {"same_dims", same_dims, METH_VARARGS, "whether two dim sequences are pairwise equal"},
    {"merge_dims", merge_dims, METH_VARARGS, "dims of the result of a binary op on tensors with these dims"},
    {"copy_compatible_raw", copy_compatible_raw, METH_VARARGS, "view of a raw tensor with axes in the order of other dims (size 1 where missing)"},
    {"bin_op_prepare", bin_op_prepare, METH_VARARGS, "(a view, b view, out dims) of a binary op"},
    {nullptr, nullptr, 0, nullptr}};

PyModuleDef module_def = {PyModuleDef_HEAD_INIT, "_rf_native", "native dimension bookkeeping of the frontend", -1, methods};

}  // namespace

PyMODINIT_FUNC PyInit__rf_native(void) { return PyModule_Create(&module_def); }
