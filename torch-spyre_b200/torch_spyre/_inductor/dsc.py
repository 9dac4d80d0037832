"""Scheduling class registered for the spyre device with Inductor.

The reference registers ``SuperDSCScheduling`` (a SIMDScheduling that emits one SuperDSC
kernel per node, torch_spyre/_inductor/dsc.py:28-63).  Graphs with spyre inputs are taken
over earlier here, at the AOT-autograd boundary (see compiler.py), so Inductor's own
lowering never schedules a spyre node; the class exists to keep the registration, and says so
loudly if Inductor ever reaches it."""
from torch._inductor.scheduler import BaseScheduling


class SuperDSCScheduling(BaseScheduling):
    def _refuse(self, *args, **kwargs):
        from . import Unsupported

        raise Unsupported("Inductor loop-level scheduling of a spyre graph; spyre graphs are "
                          "compiled by torch_spyre._inductor.compiler")

    can_fuse_vertical = can_fuse_horizontal = codegen_node = codegen_template = _refuse

    def group_fn(self, sizes):
        return tuple(tuple(s) for s in sizes)

    def flush(self):
        pass

    def ready_to_flush(self):
        return False

    def codegen_sync(self):
        pass

    def get_backend_features(self, device):
        return {}
