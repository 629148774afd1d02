// Registration shim with the macro names the reference's bindings use
// (kernel-builder's registration.h is not part of that repository):
//   TORCH_LIBRARY_EXPAND(NAME, m) { ... }   operator library in namespace NAME
//   REGISTER_EXTENSION(NAME)                empty CPython module so the shared
//                                           object can also be imported
#pragma once

#include <Python.h>
#include <torch/library.h>

#define FRT_CONCAT_(a, b) a##b
#define FRT_CONCAT(a, b) FRT_CONCAT_(a, b)
#define FRT_STRINGIFY_(x) #x
#define FRT_STRINGIFY(x) FRT_STRINGIFY_(x)

#define TORCH_LIBRARY_EXPAND(NAME, MODULE) TORCH_LIBRARY(NAME, MODULE)
#define TORCH_LIBRARY_IMPL_EXPAND(NAME, KEY, MODULE) TORCH_LIBRARY_IMPL(NAME, KEY, MODULE)

#define REGISTER_EXTENSION(NAME)                                                          \
  PyMODINIT_FUNC FRT_CONCAT(PyInit_, NAME)() {                                            \
    static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, FRT_STRINGIFY(NAME), nullptr, 0, nullptr}; \
    return PyModule_Create(&module);                                                      \
  }
