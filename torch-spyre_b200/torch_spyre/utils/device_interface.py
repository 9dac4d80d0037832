"""Dynamo device interface for ``spyre`` (reference: torch_spyre/utils/device_interface.py:
32-53), backed by the CUDA device the spyre index maps to."""
import torch
from torch._dynamo.device_interface import DeviceInterface, caching_worker_current_devices


class _B200Properties:
    """What Inductor's heuristics ask a device for, for compile-only use on a machine without the
    device (a B200's figures)."""
    name = "NVIDIA B200"
    multi_processor_count = 148
    total_memory = 180 * 1024 ** 3
    major, minor = 10, 0
    max_threads_per_multi_processor = 2048
    warp_size = 32
    regs_per_multiprocessor = 65536
    shared_memory_per_block_optin = 232448


def _device_properties(device=None):
    if torch.cuda.is_available():
        index = device.index if isinstance(device, torch.device) else device
        return torch.cuda.get_device_properties(index or 0)
    return _B200Properties()


class SpyreInterface(DeviceInterface):
    class Worker:
        @staticmethod
        def set_device(device: int):
            caching_worker_current_devices["spyre"] = device

        @staticmethod
        def current_device() -> int:
            return caching_worker_current_devices.get("spyre", 0)

        @staticmethod
        def get_device_properties(device=None):
            return _device_properties(device)

    @staticmethod
    def get_device_properties(device=None):
        return _device_properties(device)

    @staticmethod
    def current_device() -> int:
        return torch.spyre.current_device()

    @staticmethod
    def set_device(device) -> None:
        idx = device.index if isinstance(device, torch.device) else int(device)
        torch.spyre.set_device(idx or 0)

    @staticmethod
    def device_count() -> int:
        return torch.spyre.device_count()

    @staticmethod
    def is_available() -> bool:
        return torch.spyre.is_available()

    @staticmethod
    def synchronize(device=None) -> None:
        torch.spyre.synchronize()

    @staticmethod
    def get_compute_capability(device=None):
        return "sm_100a"

    @staticmethod
    def is_bf16_supported(including_emulation: bool = False) -> bool:
        return False

    @staticmethod
    def maybe_exchange_device(device: int) -> int:
        old = torch.spyre.current_device()
        if device >= 0 and device != old:
            torch.spyre.set_device(device)
        return old

    @staticmethod
    def exchange_device(device: int) -> int:
        return SpyreInterface.maybe_exchange_device(device)

    @staticmethod
    def get_raw_stream(device_idx: int) -> int:
        return torch.cuda.current_stream(device_idx).cuda_stream
