/* CPython module `_q4call`: the per-token foreign call without ctypes.
 *
 * ctypes converts every argument of a call through its generic machinery, about 0.15 us per
 * argument on the hosts this was measured on; q4_layer_gemv has seven.  This module makes the same
 * call from C with the arguments taken straight out of Python ints.  It does not link against the
 * CUDA library: `bind` receives the address of q4_layer_gemv (as ctypes resolved it) once. */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <stddef.h>

typedef int (*layer_gemv_fn)(const void* layer, const void* x, void* y, int M,
                             void* workspace, size_t workspace_bytes, void* stream);
static layer_gemv_fn g_layer_gemv = NULL;

static PyObject* q4call_bind(PyObject* self, PyObject* arg) {
  void* p = PyLong_AsVoidPtr(arg);
  if (p == NULL && PyErr_Occurred()) return NULL;
  g_layer_gemv = (layer_gemv_fn)p;
  Py_RETURN_NONE;
}

/* layer_gemv(handle, x_ptr, y_ptr, M, workspace_ptr, workspace_bytes, stream) -> int (the C return code) */
static PyObject* q4call_layer_gemv(PyObject* self, PyObject* const* args, Py_ssize_t nargs) {
  if (nargs != 7) {
    PyErr_SetString(PyExc_TypeError, "layer_gemv takes 7 arguments");
    return NULL;
  }
  if (g_layer_gemv == NULL) {
    PyErr_SetString(PyExc_RuntimeError, "_q4call: not bound to the library");
    return NULL;
  }
  void* layer = PyLong_AsVoidPtr(args[0]);
  void* x = PyLong_AsVoidPtr(args[1]);
  void* y = PyLong_AsVoidPtr(args[2]);
  long M = PyLong_AsLong(args[3]);
  void* ws = PyLong_AsVoidPtr(args[4]);
  size_t ws_bytes = PyLong_AsSize_t(args[5]);
  void* stream = PyLong_AsVoidPtr(args[6]);
  if (PyErr_Occurred()) return NULL;
  if (M < 0 || M > 1 << 20) {
    PyErr_SetString(PyExc_ValueError, "layer_gemv: M out of range");
    return NULL;
  }
  int rc = g_layer_gemv(layer, x, y, (int)M, ws, ws_bytes, stream);
  return PyLong_FromLong(rc);
}

static PyMethodDef q4call_methods[] = {
    {"bind", q4call_bind, METH_O, "bind(address of q4_layer_gemv)"},
    {"layer_gemv", (PyCFunction)(void (*)(void))q4call_layer_gemv, METH_FASTCALL,
     "layer_gemv(handle, x_ptr, y_ptr, M, workspace_ptr, workspace_bytes, stream) -> return code"},
    {NULL, NULL, 0, NULL}};

static struct PyModuleDef q4call_module = {PyModuleDef_HEAD_INIT, "_q4call", NULL, -1, q4call_methods};

PyMODINIT_FUNC PyInit__q4call(void) { return PyModule_Create(&q4call_module); }
