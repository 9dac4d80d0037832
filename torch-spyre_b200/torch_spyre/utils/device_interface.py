"""Dynamo device interface for ``spyre`` (reference: torch_spyre/utils/device_interface.py:
32-53), backed by the CUDA device the spyre index maps to."""
import torch
from torch._dynamo.device_interface import DeviceInterface, caching_worker_current_devices


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
            return torch.cuda.get_device_properties(device or 0)

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
