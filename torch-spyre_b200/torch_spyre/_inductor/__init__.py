"""Spyre backend for torch.compile (reference: torch_spyre/_inductor/__init__.py:18-98)."""
from .constants import DEVICE_NAME


class Unsupported(RuntimeError):
    def __init__(self, thing) -> None:
        super().__init__(f"Spyre backend does not support: {thing}")


def _autoload():
    if getattr(_autoload, "_ran", False):
        return
    _autoload._ran = True

    from torch._dynamo.device_interface import register_interface_for_device

    from torch_spyre.utils.device_interface import SpyreInterface

    register_interface_for_device(DEVICE_NAME, SpyreInterface)

    from torch._inductor.codegen.common import register_backend_for_device, register_device_op_overrides

    from torch_spyre.utils.device_op_overrides import SpyreDeviceOpOverrides

    register_device_op_overrides(device=DEVICE_NAME, device_op_overrides=SpyreDeviceOpOverrides())

    from .dsc import SuperDSCScheduling
    from .wrapper import SpyrePythonWrapperCodegen

    register_backend_for_device(DEVICE_NAME, SuperDSCScheduling, SpyrePythonWrapperCodegen)

    import torch_spyre._inductor.customops  # noqa: F401

    from .compiler import install_aot_hook

    install_aot_hook()

    # the runtime half of launch_kernel lives in Python
    from torch_spyre import _C

    from .runtime.kernel_runner import launch_kernel

    _C.set_kernel_launcher(launch_kernel)
