"""Loader for libb200k.so.  There is no fallback: if the CUDA library has not been built or cannot be
loaded, importing callers get an exception that says so."""
import ctypes
import os

from . import _abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200k.so")
_lib = None


class B200KError(RuntimeError):
    """A libb200k entry point returned a negative status."""

    def __init__(self, code, message):
        super().__init__("b200k error %d: %s" % (code, message))
        self.code = code


def load_library():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s is missing: build it with `python -m armnn_b200.build` (nvcc, sm_100a). "
                "There is no CPU or PyTorch fallback for the B200Acc kernels." % LIB_PATH)
        _lib = _abi.declare_product(ctypes.CDLL(LIB_PATH))
    return _lib


def check(rc):
    if rc != 0:
        raise B200KError(rc, load_library().b200k_last_error().decode())


def call(name, params, stream=0):
    """Invoke b200k_<name>(&params, stream) and raise B200KError on failure."""
    lib = load_library()
    check(getattr(lib, "b200k_" + name)(ctypes.byref(params), ctypes.c_void_p(stream)))
