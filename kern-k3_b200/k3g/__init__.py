"""ctypes binding of libk3g.so (the C ABI declared in include/k3g.h).

The binding is generated from the header at import time: every prototype
`int k3g_*(...)` becomes `k3g.lib.<name>` with argtypes set, and `k3g.call(name, *args)`
accepts torch tensors (their device pointers are passed), Python ints and floats, and raises
`K3gError` on a non-zero return.  There is no fallback: if the shared library is missing the
import fails, and nothing here computes on the CPU.
"""
import ctypes
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
HEADER = os.path.join(os.path.dirname(_ROOT), "include", "k3g.h")
LIB_PATH = os.path.join(_ROOT, "lib", "libk3g.so")
CUBIN_DIR = os.path.join(_ROOT, "lib", "cubin")

ERRORS = {-1: "K3G_ENULL: a required pointer is null", -2: "K3G_ESHAPE: unsupported size",
          -3: "K3G_EALIGN: pointer not 16-byte aligned", -4: "K3G_ERANGE: index argument out of range",
          -5: "K3G_ELIMIT: size beyond a built-in maximum"}


class K3gError(RuntimeError):
    def __init__(self, name, code):
        self.code = code
        msg = ERRORS.get(code, "cudaError %d" % code if code > 0 else "error %d" % code)
        super().__init__("%s failed: %s" % (name, msg))


_CTYPES = {"int": ctypes.c_int, "float": ctypes.c_float, "long long": ctypes.c_longlong,
           "unsigned long long": ctypes.c_ulonglong, "unsigned": ctypes.c_uint}


def parse_header(path=HEADER):
    """Return {name: [(ctype_string, arg_name), ...]} for every `int k3g_*(...)` prototype."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for m in re.finditer(r"\bint\s+(k3g_\w+)\s*\(([^)]*)\)\s*;", text):
        args = []
        body = m.group(2).strip()
        if body and body != "void":
            for a in body.split(","):
                a = " ".join(a.split())
                mm = re.match(r"(.*?)(\w+)$", a)
                ty = mm.group(1).strip()
                args.append((ty, mm.group(2)))
        protos[m.group(1)] = args
    return protos


def _ctype(ty):
    if "*" in ty:
        return ctypes.c_void_p
    return _CTYPES[ty.replace("const ", "").strip()]


PROTOTYPES = parse_header()

if not os.path.exists(LIB_PATH):
    raise ImportError("libk3g.so is not built (%s); run `python kern-k3_b200/build.py`" % LIB_PATH)
lib = ctypes.CDLL(LIB_PATH)
for _name, _args in PROTOTYPES.items():
    _fn = getattr(lib, _name)      # AttributeError here = header declares a symbol the library lacks
    _fn.restype = ctypes.c_int
    _fn.argtypes = [_ctype(t) for t, _ in _args]


def _ptr(x):
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return ctypes.c_void_p(x.data_ptr())
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    if hasattr(x, "ctypes"):          # numpy array (host_ arguments)
        return ctypes.c_void_p(x.ctypes.data)
    if isinstance(x, (ctypes._SimpleCData, ctypes.Array)):   # host out-parameters
        return ctypes.cast(ctypes.pointer(x) if isinstance(x, ctypes._SimpleCData) else x, ctypes.c_void_p)
    if isinstance(x, (bytes, bytearray)):
        return ctypes.cast(ctypes.c_char_p(bytes(x)), ctypes.c_void_p)
    raise TypeError("cannot pass %r as a pointer" % type(x))


def raw(name, *args):
    """Call an entry point, return its integer status."""
    spec = PROTOTYPES[name]
    if len(args) != len(spec):
        raise TypeError("%s takes %d arguments (%s), got %d" % (name, len(spec), ", ".join(n for _, n in spec), len(args)))
    conv = []
    for (ty, _), a in zip(spec, args):
        conv.append(_ptr(a) if "*" in ty else a)
    return getattr(lib, name)(*conv)


def call(name, *args):
    rc = raw(name, *args)
    if rc != 0:
        raise K3gError(name, rc)


def current_stream():
    import torch
    return torch.cuda.current_stream().cuda_stream
