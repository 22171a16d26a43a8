/* CPython extension-module stub for the drop-in tree.
 *
 * The reference finds its kernels as extension modules by directory and file name
 * (low_bits_training/quantization/tk_gemm.py:298-318,3426-3447; fused_te_linear.py:3782-3805;
 * mxfp4_backend.py:110-199; gate tools/check_fp4_runtime_abi.py:16-47).  This file is compiled
 * once per module name (-DSTUB_NAME=..., -DSTUB_MIRROR="...", -DSTUB_UP=n) into
 * <package>/fp4_runtime/<same sub-path>/<name><EXT_SUFFIX>.  On import it loads the Python mirror
 * module of this package, which binds the C ABI of libfp4b200.so, and re-exports its public
 * names, so that pointing FP4_MATMUL_ROOT at <package>/fp4_runtime swaps the kernels in.
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <dlfcn.h>
#include <stdio.h>

#define STR2(x) #x
#define STR(x) STR2(x)
#define CAT2(a, b) a##b
#define CAT(a, b) CAT2(a, b)

static struct PyModuleDef stub_def = {PyModuleDef_HEAD_INIT, STR(STUB_NAME),
                                      "drop-in stub re-exporting the libfp4b200 mirror module", -1, NULL};

PyMODINIT_FUNC CAT(PyInit_, STUB_NAME)(void) {
  Dl_info info;
  if (!dladdr((void*)&stub_def, &info) || !info.dli_fname) {
    PyErr_SetString(PyExc_ImportError, "stub: cannot locate its own shared object");
    return NULL;
  }
  PyObject* m = PyModule_Create(&stub_def);
  if (!m) return NULL;
  PyObject* ns = PyModule_GetDict(m); /* borrowed */
  PyObject* so = PyUnicode_FromString(info.dli_fname);
  PyDict_SetItemString(ns, "_so_path", so);
  Py_DECREF(so);
  if (!PyDict_GetItemString(ns, "__builtins__")) PyDict_SetItemString(ns, "__builtins__", PyEval_GetBuiltins());
  char code[1024];
  snprintf(code, sizeof code,
           "import importlib as _il, os as _os, sys as _sys\n"
           "_root = _os.path.abspath(_os.path.join(_os.path.dirname(_so_path), *(['..'] * %d)))\n"
           "if _root not in _sys.path: _sys.path.insert(0, _root)\n"
           "_mirror = _il.import_module('mfu-fp4-training_b200.%s')\n"
           "globals().update({k: v for k, v in vars(_mirror).items() if not k.startswith('_')})\n",
           STUB_UP, STUB_MIRROR);
  PyObject* r = PyRun_String(code, Py_file_input, ns, ns);
  if (!r) {
    Py_DECREF(m);
    return NULL;
  }
  Py_DECREF(r);
  return m;
}
