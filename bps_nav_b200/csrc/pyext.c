/* CPython binding of the two calls a trainer makes every simulator step.
 *
 * The reference exposes RolloutGenerator::stepStart / stepEnd through pybind11
 * (simulator/simulator.cpp:1785-1809), which reads the numpy action array
 * through the buffer protocol at a cost of well under a microsecond.  ctypes
 * needs several microseconds to find an array's address and convert eight
 * arguments; with a simulator step of ~50 us that shows in the end-to-end rate.
 * This module does what the pybind11 layer does, on top of the C ABI of
 * include/bpsn.h (linked from libbpsn.so).  It holds no state and computes
 * nothing; bps_sim.py falls back to ctypes for the same calls when the module
 * has not been built.
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <stdint.h>

#include "../../include/bpsn.h"

/* step_start(handle, group, actions, num_envs, stream, reward_out, mask_out, polar_out) -> status
 * actions: C-contiguous int64 buffer of num_envs items (numpy array) -> host actions. */
static PyObject* py_step_start(PyObject* self, PyObject* const* args, Py_ssize_t nargs) {
  (void)self;
  if (nargs != 8) {
    PyErr_SetString(PyExc_TypeError, "step_start takes 8 arguments");
    return NULL;
  }
  void* handle = PyLong_AsVoidPtr(args[0]);
  unsigned long group = PyLong_AsUnsignedLong(args[1]);
  Py_ssize_t num_envs = PyLong_AsSsize_t(args[3]);
  void* stream = PyLong_AsVoidPtr(args[4]);
  void* reward = args[5] == Py_None ? NULL : PyLong_AsVoidPtr(args[5]);
  void* mask = args[6] == Py_None ? NULL : PyLong_AsVoidPtr(args[6]);
  void* polar = args[7] == Py_None ? NULL : PyLong_AsVoidPtr(args[7]);
  if (PyErr_Occurred())
    return NULL;
  Py_buffer view;
  if (PyObject_GetBuffer(args[2], &view, PyBUF_C_CONTIGUOUS | PyBUF_FORMAT) != 0)
    return NULL;
  int ok = view.itemsize == 8 && view.len == num_envs * 8 && view.format &&
           (view.format[0] == 'l' || view.format[0] == 'q');
  int32_t rc = 0;
  if (ok)
    rc = bpsn_step_start_ex((bpsn_sim*)handle, (uint32_t)group, (const int64_t*)view.buf,
                            BPSN_MEM_HOST, stream, (float*)reward, (uint8_t*)mask, (float*)polar);
  PyBuffer_Release(&view);
  if (!ok) {
    PyErr_SetString(PyExc_RuntimeError,
                    "actions must be a C-contiguous int64 array with one item per environment of the group");
    return NULL;
  }
  return PyLong_FromLong(rc);
}

/* step_start_device(handle, group, actions_ptr, stream, reward_out, mask_out, polar_out) -> status */
static PyObject* py_step_start_device(PyObject* self, PyObject* const* args, Py_ssize_t nargs) {
  (void)self;
  if (nargs != 7) {
    PyErr_SetString(PyExc_TypeError, "step_start_device takes 7 arguments");
    return NULL;
  }
  void* handle = PyLong_AsVoidPtr(args[0]);
  unsigned long group = PyLong_AsUnsignedLong(args[1]);
  void* actions = PyLong_AsVoidPtr(args[2]);
  void* stream = PyLong_AsVoidPtr(args[3]);
  void* reward = args[4] == Py_None ? NULL : PyLong_AsVoidPtr(args[4]);
  void* mask = args[5] == Py_None ? NULL : PyLong_AsVoidPtr(args[5]);
  void* polar = args[6] == Py_None ? NULL : PyLong_AsVoidPtr(args[6]);
  if (PyErr_Occurred())
    return NULL;
  return PyLong_FromLong(bpsn_step_start_ex((bpsn_sim*)handle, (uint32_t)group,
                                            (const int64_t*)actions, BPSN_MEM_DEVICE, stream,
                                            (float*)reward, (uint8_t*)mask, (float*)polar));
}

/* step_end(handle, group) -> status */
static PyObject* py_step_end(PyObject* self, PyObject* const* args, Py_ssize_t nargs) {
  (void)self;
  if (nargs != 2) {
    PyErr_SetString(PyExc_TypeError, "step_end takes 2 arguments");
    return NULL;
  }
  void* handle = PyLong_AsVoidPtr(args[0]);
  unsigned long group = PyLong_AsUnsignedLong(args[1]);
  if (PyErr_Occurred())
    return NULL;
  int32_t rc;
  /* the wait for the device happens here: let other Python threads run meanwhile
     (the reference holds the GIL; releasing it changes nothing for a single-threaded caller) */
  Py_BEGIN_ALLOW_THREADS
  rc = bpsn_step_end((bpsn_sim*)handle, (uint32_t)group);
  Py_END_ALLOW_THREADS
  return PyLong_FromLong(rc);
}

static PyMethodDef methods[] = {
    {"step_start", (PyCFunction)(void (*)(void))py_step_start, METH_FASTCALL,
     "bpsn_step_start_ex with host actions read through the buffer protocol"},
    {"step_start_device", (PyCFunction)(void (*)(void))py_step_start_device, METH_FASTCALL,
     "bpsn_step_start_ex with a device pointer to int64 actions"},
    {"step_end", (PyCFunction)(void (*)(void))py_step_end, METH_FASTCALL, "bpsn_step_end"},
    {NULL, NULL, 0, NULL}};

static struct PyModuleDef moddef = {PyModuleDef_HEAD_INIT, "_bpsn_fast",
                                    "per-step calls of the bpsn C ABI", -1, methods,
                                    NULL, NULL, NULL, NULL};

PyMODINIT_FUNC PyInit__bpsn_fast(void) {
  return PyModule_Create(&moddef);
}
