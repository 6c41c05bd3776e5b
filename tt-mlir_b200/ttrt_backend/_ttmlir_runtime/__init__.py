"""Stand-in for `ttrt.runtime._ttmlir_runtime`, the nanobind extension module of tt-mlir's Python runtime
(runtime/python/runtime/runtime.cpp, runtime/python/binary/binary.cpp), backed by the B200 target.

tt-mlir's `ttrt` tool is plain Python on top of that one extension module: `ttrt/runtime/__init__.py`
and `ttrt/binary/__init__.py` import their names from `ttrt.runtime._ttmlir_runtime.{runtime,binary}`.
Putting THIS package where the extension module would be (inside `ttrt/runtime/`, or anywhere on the
path together with an import alias) lets the unmodified `ttrt` sources drive the CUDA backend:

    ttrt/runtime/_ttmlir_runtime/__init__.py   <- this package (or a symlink to it)
    ttrt/runtime/_ttmlir_runtime/runtime.py
    ttrt/runtime/_ttmlir_runtime/binary.py

The submodules bind the C ABI of libttb200.so through ctypes (tt-mlir_b200/runtime_api.py); nanobind is
not needed.  Names, argument order and return shapes follow the nanobind definitions cited in each
submodule.
"""

import importlib.util
import os
import sys


def _load_runtime_api():
    """The ctypes binding lives in the package one level above ttrt_backend/ (directory `tt-mlir_b200`,
    imported as `ttmlir_b200`)."""
    if "ttmlir_b200" not in sys.modules:
        here = os.path.dirname(os.path.realpath(__file__))
        pkg_dir = os.path.dirname(os.path.dirname(here))
        spec = importlib.util.spec_from_file_location("ttmlir_b200", os.path.join(pkg_dir, "__init__.py"),
                                                      submodule_search_locations=[pkg_dir])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["ttmlir_b200"] = mod
        spec.loader.exec_module(mod)
    import ttmlir_b200.runtime_api as api
    return api


api = _load_runtime_api()

from . import binary, runtime  # noqa: E402,F401
