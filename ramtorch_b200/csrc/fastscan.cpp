// Host-side helper of the optimizer class: one pass, in C++, over an optimizer's parameter list
// and state dicts.
//
// The reference walks its parameters in a Python loop every step (adamw.py:111-232).  The fused
// step needs, per step, only to confirm that nothing but the gradients changed since the tensor
// table was built, and to collect the gradients' addresses.  Done in Python that is half a dozen
// passes over the list (about 0.5 us per tensor: ~10 ms for 20,000 tensors, comparable to the GPU
// time of the update itself); here it is one pass of ~0.1 us per tensor.  Nothing in this file
// touches tensor DATA or launches anything: it reads pointers and properties.
#include <torch/csrc/autograd/python_variable.h>
#include <torch/extension.h>

namespace {

// out[k] = {parameter data pointer, gradient data pointer (0: no gradient, -1: sparse), properties}
// properties = scalar type | contiguous << 8 | sparse << 9 | (cuda device index + 1) << 16
// Returns the index of the first list entry whose identity differs from ids[k], or -1.
int64_t scan_params(py::list params, at::Tensor ids, at::Tensor out) {
  const int64_t n = (int64_t)PyList_GET_SIZE(params.ptr());
  TORCH_CHECK(ids.dtype() == at::kLong && ids.is_contiguous() && ids.numel() == n, "ids: int64[n] expected");
  TORCH_CHECK(out.dtype() == at::kLong && out.is_contiguous() && out.numel() == n * 3, "out: int64[n, 3] expected");
  const int64_t* want = ids.data_ptr<int64_t>();
  int64_t* o = out.data_ptr<int64_t>();
  int64_t first_bad = -1;
  for (int64_t k = 0; k < n; ++k) {
    PyObject* obj = PyList_GET_ITEM(params.ptr(), k);
    if (reinterpret_cast<int64_t>(obj) != want[k] && first_bad < 0) first_bad = k;
    TORCH_CHECK(THPVariable_Check(obj), "parameter ", k, " is not a tensor");
    const at::Tensor& p = THPVariable_Unpack(obj);
    const at::Tensor& g = p.grad();
    o[3 * k] = reinterpret_cast<int64_t>(p.unsafeGetTensorImpl()->data());
    if (!g.defined()) {
      o[3 * k + 1] = 0;
      o[3 * k + 2] = 0;
      continue;
    }
    const bool sparse = g.layout() != at::kStrided;
    o[3 * k + 1] = sparse ? -1 : reinterpret_cast<int64_t>(g.unsafeGetTensorImpl()->data());
    o[3 * k + 2] = (int64_t)g.scalar_type() | ((!sparse && g.is_contiguous()) ? 256 : 0) | (sparse ? 512 : 0) |
                   ((int64_t)(g.device().is_cuda() ? g.device().index() + 1 : 0) << 16);
  }
  return first_bad;
}

// Identity of every parameter in the list, as scan_params compares it.
void param_ids(py::list params, at::Tensor ids) {
  const int64_t n = (int64_t)PyList_GET_SIZE(params.ptr());
  TORCH_CHECK(ids.dtype() == at::kLong && ids.is_contiguous() && ids.numel() == n, "ids: int64[n] expected");
  int64_t* o = ids.data_ptr<int64_t>();
  for (int64_t k = 0; k < n; ++k) o[k] = reinterpret_cast<int64_t>(PyList_GET_ITEM(params.ptr(), k));
}

// Every state dict must still hold the cached moment tensors (by identity) and the cached step
// counter.  Returns -1, or the index of the first state that differs (nothing is changed then).
// With check == false nothing is verified.  Afterwards the counters are all changed by `delta`
// (+1 for a step, -1 to take one back, 0 to leave them), in the dicts and in `steps`.
int64_t check_states(py::list states, at::Tensor ema_ids, at::Tensor ema_sq_ids, at::Tensor steps, bool check, int64_t delta) {
  const int64_t n = (int64_t)PyList_GET_SIZE(states.ptr());
  for (const at::Tensor* t : {&ema_ids, &ema_sq_ids, &steps})
    TORCH_CHECK(t->dtype() == at::kLong && t->is_contiguous() && t->numel() == n, "int64[n] expected");
  static PyObject* k_ema = PyUnicode_InternFromString("ema");
  static PyObject* k_ema_sq = PyUnicode_InternFromString("ema_squared");
  static PyObject* k_step = PyUnicode_InternFromString("step");
  const int64_t *a = ema_ids.data_ptr<int64_t>(), *b = ema_sq_ids.data_ptr<int64_t>();
  int64_t* s = steps.data_ptr<int64_t>();
  for (int64_t k = 0; check && k < n; ++k) {
    PyObject* st = PyList_GET_ITEM(states.ptr(), k);
    if (!PyDict_Check(st)) return k;
    PyObject* step = PyDict_GetItem(st, k_step);          // borrowed
    if (reinterpret_cast<int64_t>(PyDict_GetItem(st, k_ema)) != a[k] ||
        reinterpret_cast<int64_t>(PyDict_GetItem(st, k_ema_sq)) != b[k] || step == nullptr || !PyLong_CheckExact(step) ||
        PyLong_AsLongLong(step) != s[k])
      return k;
  }
  if (delta != 0) {
    for (int64_t k = 0; k < n; ++k) {
      s[k] += delta;
      PyObject* next = PyLong_FromLongLong(s[k]);
      PyDict_SetItem(PyList_GET_ITEM(states.ptr(), k), k_step, next);
      Py_DECREF(next);
    }
  }
  return -1;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("scan_params", &scan_params);
  m.def("param_ids", &param_ids);
  m.def("check_states", &check_states);
}
