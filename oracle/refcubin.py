"""TEST INFRASTRUCTURE — launch entries of the reference's own cubins (oracle/_ref) on a GPU.

Thin ctypes layer over the CUDA driver API: load a cubin built by oracle/build_ref.py, look
up an `extern "C"` entry and launch it with the manifest's grid/block.  Arguments are torch
CUDA tensors (device pointer), Python ints (C int), `I64(v)` (long long) or Python floats.
Used only by GPU tests and by tests/golden/make_golden.py; the shipped library never runs
reference code.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")

_cuda = None
_modules = {}


class I64(int):
    """Marks an integer argument as a 64-bit kernel parameter (long / long long)."""


def _drv():
    global _cuda
    if _cuda is None:
        import torch
        torch.cuda.init()
        torch.zeros(1, device="cuda")          # make the primary context current
        _cuda = ctypes.CDLL("libcuda.so.1")
        _check(_cuda.cuInit(0))
    return _cuda


def _check(rc):
    if rc != 0:
        raise RuntimeError("CUDA driver error %d" % rc)


def available(module):
    return os.path.exists(os.path.join(REF_DIR, module + ".cubin"))


def function(module, entry):
    d = _drv()
    if module not in _modules:
        mod = ctypes.c_void_p()
        _check(d.cuModuleLoad(ctypes.byref(mod), os.path.join(REF_DIR, module + ".cubin").encode()))
        _modules[module] = mod
    fn = ctypes.c_void_p()
    _check(d.cuModuleGetFunction(ctypes.byref(fn), _modules[module], entry.encode()))
    return fn


def load_external(path, entry):
    """Same, for an arbitrary cubin path (used to launch this library's drop-in cubins)."""
    d = _drv()
    key = "path:" + path
    if key not in _modules:
        mod = ctypes.c_void_p()
        _check(d.cuModuleLoad(ctypes.byref(mod), path.encode()))
        _modules[key] = mod
    fn = ctypes.c_void_p()
    _check(d.cuModuleGetFunction(ctypes.byref(fn), _modules[key], entry.encode()))
    return fn


def launch(fn, grid, block, args, stream=None):
    import torch
    d = _drv()
    vals = []
    for a in args:
        if a is None:
            vals.append(ctypes.c_void_p(0))
        elif hasattr(a, "data_ptr"):
            vals.append(ctypes.c_void_p(a.data_ptr()))
        elif isinstance(a, I64):
            vals.append(ctypes.c_longlong(int(a)))
        elif isinstance(a, bool):
            vals.append(ctypes.c_int(int(a)))
        elif isinstance(a, int):
            vals.append(ctypes.c_int(a))
        elif isinstance(a, float):
            vals.append(ctypes.c_float(a))
        else:
            raise TypeError(type(a))
    ptrs = (ctypes.c_void_p * len(vals))(*[ctypes.cast(ctypes.byref(v), ctypes.c_void_p) for v in vals])
    g = tuple(grid) + (1,) * (3 - len(grid)) if not isinstance(grid, int) else (grid, 1, 1)
    b = tuple(block) + (1,) * (3 - len(block)) if not isinstance(block, int) else (block, 1, 1)
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream if stream is None else stream)
    _check(d.cuLaunchKernel(fn, g[0], g[1], g[2], b[0], b[1], b[2], 0, s, ptrs, None))


def run(module, entry, grid, block, args):
    launch(function(module, entry), grid, block, args)
