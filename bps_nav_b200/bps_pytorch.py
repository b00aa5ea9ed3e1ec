"""Drop-in for the reference's ``bps_pytorch`` extension (``simulator/pytorch.cpp:13-75``):
wrap a raw CUDA device pointer carried in an unnamed PyCapsule as a torch tensor, and the
reverse.  No copies, no ownership transfer, no kernels."""
import ctypes as C

import numpy as np
import torch


class _DeviceArray:
    def __init__(self, ptr, shape, dtype):
        self.__cuda_array_interface__ = {
            "shape": tuple(int(s) for s in shape), "typestr": np.dtype(dtype).str,
            "data": (int(ptr), False), "version": 3, "strides": None,
        }


def _capsule_pointer(capsule):
    f = C.pythonapi.PyCapsule_GetPointer
    f.restype = C.c_void_p
    f.argtypes = [C.py_object, C.c_char_p]
    return f(capsule, None)


def _wrap(capsule, dev_id, shape, dtype):
    ptr = _capsule_pointer(capsule)
    if not ptr:
        raise RuntimeError("capsule holds a null device pointer")
    return torch.as_tensor(_DeviceArray(ptr, shape, dtype), device=f"cuda:{int(dev_id)}")


def make_color_tensor(ptr_capsule, dev_id, batch_size, resolution):
    """uint8 CUDA tensor ``[batch, resolution[0], resolution[1], 4]`` -- the dimensions in the
    order ``pytorch.cpp:13-27`` gives them.  ``resolution`` is what the generator was built
    with, ``[width, height]`` (``simulator/simulator.cpp:381-383``), while the memory holds
    ``height`` rows of ``width`` pixels per image: for square images the two readings agree, for
    any other shape the reference's tensor has its two image dimensions labelled the wrong way
    round and ``t.view(batch, resolution[1], resolution[0], 4)`` is the image."""
    return _wrap(ptr_capsule, dev_id, (batch_size, resolution[0], resolution[1], 4), np.uint8)


def make_depth_tensor(ptr_capsule, dev_id, batch_size, resolution):
    """float32 CUDA tensor ``[batch, resolution[0], resolution[1]]`` (``pytorch.cpp:31-45``); see
    ``make_color_tensor`` for what that means for images that are not square."""
    return _wrap(ptr_capsule, dev_id, (batch_size, resolution[0], resolution[1]), np.float32)


def make_fcout_tensor(ptr_capsule, dev_id, batch_size, num_features):
    """float16 CUDA tensor ``[batch, features]`` (``pytorch.cpp:48-62``)."""
    return _wrap(ptr_capsule, dev_id, (batch_size, num_features), np.float16)


def tensor_to_capsule(tensor):
    """Unnamed capsule holding ``tensor.data_ptr()`` (``pytorch.cpp:64-67``)."""
    f = C.pythonapi.PyCapsule_New
    f.restype = C.py_object
    f.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p]
    return f(tensor.data_ptr(), None, None)
