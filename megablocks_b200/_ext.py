"""Loader for the in-tree sm_100a extension ``megablocks_b200._C``.

The extension is built in place by ``setup.py build_ext --inplace`` (see
``__graft_entry__.build``).  Ops call :func:`ext` whenever they are handed a
CUDA tensor; if the shared object is missing that call raises instead of
quietly falling back to eager PyTorch, so a GPU run can never pass on a
fallback path by accident.  CPU tensors never touch the extension.
"""

import importlib
import threading

_lock = threading.Lock()
_module = None
_error = None


def try_ext():
    """Return the extension module or ``None`` when it cannot be imported."""
    global _module, _error
    if _module is not None or _error is not None:
        return _module
    with _lock:
        if _module is None and _error is None:
            try:
                import torch  # noqa: F401  (libtorch must be loaded before the extension)
                _module = importlib.import_module('megablocks_b200._C')
            except Exception as exc:  # pragma: no cover - depends on the build
                _error = exc
    return _module


def ext():
    """Return the extension module; raise a clear error when it is not built."""
    module = try_ext()
    if module is None:
        raise RuntimeError(
            'megablocks_b200._C (the sm_100a CUDA extension) is not available: '
            f'{_error!r}. Build it with `python setup.py build_ext --inplace` '
            'at the repository root.')
    return module


def available() -> bool:
    return try_ext() is not None
