/*
 * Import shim: makes an operator module of this library loadable by the reference's own,
 * unmodified loader.
 *
 * The reference imports build/lib<name>.so (after copying it to a scratch directory) with
 * importlib as the module "mkernel_release_<name>", so the file must be a CPython extension that
 * exports PyInit_mkernel_release_<name> (python/load_module.py:19-74; the reference builds it
 * with -DTORCH_EXTENSION_NAME=mkernel_release_<name>, Makefile:150-170).  This file, compiled once
 * per operator name with -DMK_KERNEL=<name>, is that extension: on import it fills its own
 * namespace from mkernel_b200.load_module.populate(module, "<name>"), i.e. with DistBuffer and
 * the operator functions that call the C ABI of libmkernel_b200.so.  It holds no kernels itself
 * and does not depend on its own location; the mkernel_b200 package must be importable.
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>

#ifndef MK_KERNEL
#error "compile with -DMK_KERNEL=<operator module name>"
#endif
#define MK_STR2(x) #x
#define MK_STR(x) MK_STR2(x)
#define MK_CAT2(a, b) a##b
#define MK_CAT(a, b) MK_CAT2(a, b)

static int shim_exec(PyObject* module) {
  PyObject* loader = PyImport_ImportModule("mkernel_b200.load_module");
  if (loader == NULL) return -1;
  PyObject* r = PyObject_CallMethod(loader, "populate", "Os", module, MK_STR(MK_KERNEL));
  Py_DECREF(loader);
  if (r == NULL) return -1;
  Py_DECREF(r);
  return 0;
}

static PyModuleDef_Slot shim_slots[] = {
    {Py_mod_exec, (void*)shim_exec},
    {0, NULL},
};

static struct PyModuleDef shim_def = {
    PyModuleDef_HEAD_INIT,
    "mkernel_release_" MK_STR(MK_KERNEL),
    "B200-native stand-in for the reference's lib" MK_STR(MK_KERNEL) ".so",
    0,
    NULL,
    shim_slots,
    NULL,
    NULL,
    NULL,
};

PyMODINIT_FUNC MK_CAT(PyInit_mkernel_release_, MK_KERNEL)(void) {
  return PyModuleDef_Init(&shim_def);
}
