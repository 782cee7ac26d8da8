r"""
Loader of the native extension (C++ host runtime + sm_100a kernels).

The reference imports its single pybind module ``fmoe_cuda`` unconditionally
(``fmoe/functions.py:9``, ``fmoe/linear.py:9``) and therefore cannot even be imported
on a machine without the built extension.  Here the extension is built in-tree
(``fastmoe_b200/_build/fmoe_b200_native.so``) and loaded lazily:

* tensors on a CUDA device always go through the extension; if it is missing the call
  fails loudly, never silently falling back to eager PyTorch;
* tensors on the CPU use the extension's C++ CPU ops when it is loaded and the pure
  PyTorch restatement in :mod:`fastmoe_b200.ops.torch_impl` otherwise, which is what
  lets the CPU test tier run on a box where nothing was compiled.
"""
import importlib.util
import os
import sys
import threading

_LOCK = threading.Lock()
_MOD = None
_TRIED = False
_ERR = None

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD_DIR = os.path.join(PKG_DIR, "_build")
MODULE_NAME = "fmoe_b200_native"


def so_path():
    return os.path.join(BUILD_DIR, MODULE_NAME + ".so")


def _load():
    global _MOD, _TRIED, _ERR
    with _LOCK:
        if _TRIED:
            return _MOD
        _TRIED = True
        path = so_path()
        if not os.path.exists(path):
            _ERR = "native extension not built: %s (run `python -m fastmoe_b200.build`)" % path
            return None
        try:
            import torch  # noqa: F401  (libtorch must be loaded before the extension)
            spec = importlib.util.spec_from_file_location(MODULE_NAME, path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            sys.modules[MODULE_NAME] = mod
            _MOD = mod
        except Exception as exc:  # pylint: disable=broad-except
            _ERR = "native extension failed to load: %r" % (exc,)
            _MOD = None
        return _MOD


def available():
    r"""True when the compiled extension could be imported."""
    return _load() is not None


def load_error():
    _load()
    return _ERR


def get():
    r"""The extension module; raises when it is absent."""
    mod = _load()
    if mod is None:
        raise RuntimeError(
            "fastmoe_b200: %s. CUDA tensors require the compiled sm_100a extension; "
            "there is no eager fallback on the GPU." % _ERR)
    return mod


def for_tensor(t):
    r"""Extension for a CUDA tensor (mandatory) or for a CPU tensor (optional, may be ``None``)."""
    if t.is_cuda:
        return get()
    return _load()
