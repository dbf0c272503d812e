"""B200-native int8 quantized-linear path for Self-evolve-diffusion-cpp.

The product is the C-ABI library `libsdq.so` (include/sdq.h) built from `csrc/`
and the C++ drop-in `libsd_b200.so`; this Python package is a thin ctypes
binding used by the tests and the benchmark.  The directory name is not a
valid Python identifier: load it with `__graft_entry__.load_package()`.
"""
from .sdq import Sdq, SdqError, DeviceBuffer, lib_path, build  # noqa: F401
from . import sharding  # noqa: F401


def __getattr__(name):
    # `parallel` needs torch; import it only when asked for
    if name == "parallel":
        import importlib
        return importlib.import_module(__name__ + ".parallel")
    raise AttributeError(name)
