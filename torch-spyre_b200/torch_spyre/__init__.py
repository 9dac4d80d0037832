"""B200-native implementation of torch-spyre's data-parallel hot path.

The package keeps the reference's import name and public surface
(torch_spyre/__init__.py:24-163 of the reference): importing it renames the
PrivateUse1 backend to ``spyre``, registers the ``torch.spyre`` device module, patches
``Tensor.__repr__`` and registers the aten kernels and the Inductor backend.  Underneath,
``spyre:N`` is CUDA device N and every kernel is hand-written sm_100a CUDA reached through
the C ABI of ``lib/libspyre_b200.so``.
"""
from __future__ import annotations

import importlib
import os
import threading
import types

from .constants import DEVICE_NAME
from .layout import storage_nbytes  # noqa: F401

_runtime_init_lock = threading.Lock()


class _SpyreImpl:
    """State behind the ``torch.spyre`` module; the C++ module is loaded on first use."""

    def __init__(self):
        self._initialized = False
        self._in_bad_fork = False
        try:
            os.register_at_fork(after_in_child=self._mark_after_fork)
        except Exception:
            pass

    def _lazy_init(self):
        if self._initialized:
            return
        with _runtime_init_lock:
            if self._initialized:
                return
            self._C = importlib.import_module("torch_spyre._C")
            self._C.start_runtime()
            self._initialized = True

    def __getattr__(self, name):
        if name == "_C":
            self._lazy_init()
            return self.__dict__["_C"]
        raise AttributeError(name)

    def _is_in_bad_fork(self) -> bool:
        return self._in_bad_fork

    def _mark_after_fork(self):
        # a CUDA context does not survive fork(): the child must not touch the device
        self._in_bad_fork = True

    def manual_seed(self, seed: int, device=None) -> None:
        import torch

        if device is None:
            torch.cuda.manual_seed(int(seed))
            return
        index = device.index if isinstance(device, torch.device) else int(device)
        if not 0 <= index < torch.cuda.device_count():
            raise RuntimeError(f"manual_seed: no spyre device {index}")
        with torch.cuda.device(index):
            torch.cuda.manual_seed(int(seed))

    def manual_seed_all(self, seed: int) -> None:
        import torch

        torch.cuda.manual_seed_all(int(seed))

    def is_available(self) -> bool:
        return bool(self._C.is_available())

    def device_count(self) -> int:
        return int(self._C.device_count())

    def current_device(self) -> int:
        # on a machine without a device (compile-only use with fake tensors) index 0 is reported
        return int(self._C.current_device()) if self.is_available() else 0

    def is_initialized(self) -> bool:
        return self._initialized

    def init(self) -> None:
        self._lazy_init()

    def set_device(self, idx: int) -> None:
        self._C.set_device(int(idx))

    def synchronize(self, idx: int | None = None) -> None:
        self._C.synchronize(-1 if idx is None else int(idx))


def make_spyre_module() -> types.ModuleType:
    impl = _SpyreImpl()
    mod = types.ModuleType(DEVICE_NAME)
    mod.__doc__ = "Spyre backend module (CUDA-backed)."
    for name in ("_is_in_bad_fork", "manual_seed", "manual_seed_all", "is_available",
                 "device_count", "current_device", "set_device", "synchronize", "is_initialized", "init"):
        setattr(mod, name, getattr(impl, name))
    mod._is_compiled = lambda: True

    def __getattr__(name):
        c = impl._C
        if hasattr(c, name):
            return getattr(c, name)
        raise AttributeError(name)

    mod.__getattr__ = __getattr__
    mod._impl = impl
    return mod


def _autoload():
    """Entry point for torch's backend autoload; safe to call more than once."""
    if getattr(_autoload, "_ran", False):
        return
    _autoload._ran = True

    import torch

    from ._monkey_patch import _patch_tensor_for_spyre

    _patch_tensor_for_spyre()
    torch.utils.rename_privateuse1_backend(DEVICE_NAME)
    torch._register_device_module(DEVICE_NAME, make_spyre_module())
    torch.utils.generate_methods_for_privateuse1_backend(for_tensor=True, for_module=True,
                                                         for_storage=False)
    # the C++ half registers allocator, guard and the core aten kernels at load time
    torch.spyre._impl._lazy_init()
    from . import ops  # noqa: F401  (aten kernels implemented over the C ABI)

    try:
        from ._inductor import _autoload as inductor_autoload
    except ImportError:
        inductor_autoload = None
    if inductor_autoload is not None:
        inductor_autoload()


def __getattr__(name):
    if name == "SpyreTensorLayout":
        from ._C import SpyreTensorLayout

        return SpyreTensorLayout
    raise AttributeError(name)


if os.environ.get("TORCH_DEVICE_BACKEND_AUTOLOAD", "1") != "0":
    _autoload()
