"""Device-specific lines of Inductor's generated wrapper (reference: SpyreDeviceOpOverrides,
torch_spyre/utils/device_op_overrides.py:20-36).  The reference stubs all of them out; here
``spyre:N`` is CUDA device N with real streams, so they do real work."""
from textwrap import dedent

from torch._inductor.codegen.common import DeviceOpOverrides


class SpyreDeviceOpOverrides(DeviceOpOverrides):
    def import_get_raw_stream_as(self, name: str) -> str:
        return dedent(
            f"""
            def {name}(device_idx):
                import torch
                return torch.cuda.current_stream(device_idx).cuda_stream
            """
        )

    def set_device(self, device_idx: int) -> str:
        return f"torch.spyre.set_device({device_idx})"

    def synchronize(self) -> str:
        return "torch.spyre.synchronize()"

    def device_guard(self, device_idx: int) -> str:
        return f"torch.cuda.device({device_idx})"
