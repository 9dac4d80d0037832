"""Kernel descriptions handed from the compiler to the runtime.

Same dataclasses as the reference (torch_spyre/_inductor/runtime/__init__.py:20-45).  Where the
reference's ``KernelSpec.op`` names one Spyre op and ``op_info`` carries op-specific constants,
here ``op`` names a kernel family of the CUDA library and ``op_info`` carries the fused
program."""
import dataclasses
from typing import Any, Dict, List, Union

import torch


@dataclasses.dataclass
class TensorArg:
    is_input: bool
    arg_index: int
    dtype: torch.dtype


@dataclasses.dataclass
class ConstantArg:
    value: Union[bool, float, int]
    dtype: torch.dtype


@dataclasses.dataclass
class KernelSpec:
    op: str
    is_reduction: bool
    dimensions: List[int]
    args: List[Union[TensorArg, ConstantArg]]
    scales: List[List[int]]
    op_info: Dict[str, Any]


@dataclasses.dataclass
class UnimplementedOp:
    op: str
