"""Analysis of the scheduler nodes Inductor hands to the spyre backend: loop bodies -> one fused
program for ``ts_pointwise_chain``, described by a ``KernelSpec``.

Counterpart of the reference's SpyreKernel (torch_spyre/_inductor/spyre_kernel.py:85-369), which
records the single op of a node, its tensor accesses and constants, and derives
``KernelSpec.dimensions`` / ``scales`` / ``args`` from the index expressions.  The same derivation is
done here, with two differences: a kernel may hold a whole fused group of pointwise ops ended by a
reduction over the innermost dim (the reference refuses "multi-op kernel"), and what comes out is a
program for the accumulator machine of the CUDA library instead of the name of one Spyre op.

A loop body is read from its FX graph (``LoopBody.root_block.graph``): ``load`` / ``store`` /
``reduction`` / ``store_reduction`` / ``constant`` / ``to_dtype`` and the pointwise ops.  Every
tensor access must walk its buffer in row-major order over the iteration dims it depends on
(``scale`` 1) and not at all over the others (``scale`` -1, a broadcast); anything else (transposed
reads, gathers, masked sub-blocks) raises ``Unsupported`` and the graph is compiled by the
FX-level planner instead.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Sequence, Tuple

import sympy
import torch
from torch.fx import Graph, Node

from . import Unsupported, fusion
from .runtime import KernelSpec, TensorArg

aten = torch.ops.aten

# Inductor op name -> aten overload the fusion lineariser understands
_UNARY = {
    "exp": aten.exp.default, "log": aten.log.default, "sqrt": aten.sqrt.default, "rsqrt": aten.rsqrt.default,
    "reciprocal": aten.reciprocal.default, "sigmoid": aten.sigmoid.default, "tanh": aten.tanh.default,
    "relu": aten.relu.default, "neg": aten.neg.default, "abs": aten.abs.default, "sin": aten.sin.default,
    "cos": aten.cos.default, "erf": aten.erf.default, "floor": aten.floor.default, "ceil": aten.ceil.default,
    "sign": aten.sign.default, "log1p": aten.log1p.default, "expm1": aten.expm1.default,
    "logical_not": aten.logical_not.default,
}
_BINARY = {
    "add": aten.add.Tensor, "sub": aten.sub.Tensor, "mul": aten.mul.Tensor, "truediv": aten.div.Tensor,
    "maximum": aten.maximum.default, "minimum": aten.minimum.default, "pow": aten.pow.Tensor_Tensor,
    "eq": aten.eq.Tensor, "ne": aten.ne.Tensor, "lt": aten.lt.Tensor, "le": aten.le.Tensor,
    "gt": aten.gt.Tensor, "ge": aten.ge.Tensor,
}
_SCALAR_FORM = {aten.add.Tensor: aten.add.Scalar, aten.sub.Tensor: aten.sub.Scalar, aten.mul.Tensor: aten.mul.Scalar,
                aten.div.Tensor: aten.div.Scalar, aten.pow.Tensor_Tensor: aten.pow.Tensor_Scalar,
                aten.eq.Tensor: aten.eq.Scalar, aten.ne.Tensor: aten.ne.Scalar, aten.lt.Tensor: aten.lt.Scalar,
                aten.le.Tensor: aten.le.Scalar, aten.gt.Tensor: aten.gt.Scalar, aten.ge.Tensor: aten.ge.Scalar}
_REDUCTIONS = {"sum": aten.sum.dim_IntList, "max": aten.amax.default, "min": aten.amin.default}
_FLOATS = (torch.float16, torch.float32, torch.bfloat16)


@dataclasses.dataclass
class TensorAccess:
    name: str                      # buffer name
    index: sympy.Expr
    dtype: torch.dtype
    shape: Tuple[int, ...]         # extent per iteration dim (1 where the access does not depend on it)


@dataclasses.dataclass
class KernelSummary:
    dimensions: List[int]                  # iteration space, reduction dim last
    inputs: List[TensorAccess]             # in the program's operand order
    outputs: List[TensorAccess]            # full-shape stores, in STORE slot order
    reduction_out: Optional[TensorAccess]
    spec: KernelSpec


def access_shape(index: sympy.Expr, variables: Sequence[sympy.Symbol], ranges: Sequence[int], what: str):
    """(shape, scale) of a buffer access: the access must be a row-major walk over the iteration
    dims it depends on.  scale is 1 for a dim walked, -1 for a dim ignored (the reference's
    analyze_tensor_access, spyre_kernel.py:162-171)."""
    index = sympy.expand(index)
    free = index.free_symbols
    for s in free:
        if s not in variables:
            raise Unsupported(f"{what}: index {index} uses {s}, which is not an iteration variable")
    shape, scale = [], []
    expect = 1
    for v, n in reversed(list(zip(variables, ranges))):
        if v in free and n != 1:
            coeff = index.coeff(v)
            if coeff != expect:
                raise Unsupported(f"{what}: index {index} is not a row-major walk (stride {coeff} for {v}, "
                                  f"a contiguous access has {expect})")
            expect *= n
            shape.append(n)
            scale.append(1)
        else:
            shape.append(1)
            scale.append(-1)
    rest = index - sum(index.coeff(v) * v for v in free)
    if sympy.simplify(rest) != 0:
        raise Unsupported(f"{what}: index {index} has an offset or a non-linear term")
    return tuple(reversed(shape)), list(reversed(scale))


class SpyreKernel:
    """Collects the loop bodies of one (possibly fused) scheduler node and turns them into a
    KernelSpec.  ``nodes`` are Inductor SchedulerNodes in execution order."""

    def __init__(self, nodes, removable=lambda name: False):
        self.nodes = list(nodes)
        self.removable = removable
        self.graph = Graph()
        self.values: Dict[str, Node] = {}          # buffer name -> value stored into it inside this kernel
        self.input_nodes: Dict[Tuple[str, Tuple[int, ...]], Node] = {}
        self.input_access: Dict[Node, TensorAccess] = {}
        self.stored: List[Tuple[Node, TensorAccess]] = []
        self.reduction: Optional[Tuple[Node, TensorAccess, str]] = None
        self.dimensions: Optional[List[int]] = None
        self.order: List[Node] = []
        self.reduce_scale = 1.0
        self.scaled_from: Optional[str] = None   # buffer of the unscaled reduction, when an epilogue rescaled it

    # -- building the value graph -----------------------------------------------------------
    def _meta(self, shape, dtype=torch.float16):
        return torch.empty(tuple(shape), dtype=dtype, device="meta")

    def _placeholder(self, acc: TensorAccess) -> Node:
        key = (acc.name, acc.shape)
        if key not in self.input_nodes:
            n = self.graph.placeholder(f"{acc.name}_{len(self.input_nodes)}")
            n.meta["val"] = self._meta(acc.shape)
            self.input_nodes[key] = n
            self.input_access[n] = acc
        return self.input_nodes[key]

    def _call(self, target, args, mask=False) -> Node:
        n = self.graph.call_function(target, tuple(args))
        n.meta["val"] = self._meta(self.dimensions, torch.bool if mask else torch.float16)
        self.order.append(n)
        return n

    def _read_body(self, snode) -> None:
        if self.reduction is not None:
            # the only thing that may follow a reduction inside its kernel is a scaling of the reduced
            # value by constants (what mean lowers to): it becomes the program's reduce_scale
            return self._read_scale_epilogue(snode)
        body = snode._body
        iter_sizes, red_sizes = snode._sizes
        variables = list(body.iter_vars) + list(body.reduce_vars)
        ranges = [int(body.var_ranges[v]) for v in variables]
        if any(isinstance(s, sympy.Expr) and not s.is_number for s in list(iter_sizes) + list(red_sizes)):
            raise Unsupported("dynamic shapes")
        dims = ranges or [1]
        if len(body.reduce_vars) > 1:
            raise Unsupported(f"reduction over {len(body.reduce_vars)} dims in one kernel")
        if self.dimensions is None:
            self.dimensions = dims
        elif list(self.dimensions) != dims:
            raise Unsupported(f"fused nodes with different iteration spaces: {self.dimensions} vs {dims}")
        env: Dict[Node, Any] = {}
        g = body.root_block.graph
        if len(body.subblocks):
            raise Unsupported("masked sub-blocks")
        for n in g.nodes:
            if n.op == "placeholder":
                continue
            if n.op == "output":
                continue
            if n.op == "call_module":
                if n.target == "get_index":
                    env[n] = body.indexing_exprs[n.args[0]]
                    continue
                raise Unsupported(f"loop body calls {n.target}")
            if n.op != "call_method":
                raise Unsupported(f"loop body node {n.op}")
            args = [env.get(a, a) if isinstance(a, Node) else a for a in n.args[1:]]
            env[n] = self._op(n.target, args, variables, ranges)

    def _read_scale_epilogue(self, snode) -> None:
        body = snode._body
        variables = list(body.iter_vars) + list(body.reduce_vars)
        ranges = [int(body.var_ranges[v]) for v in variables]
        if body.reduce_vars or len(body.subblocks) or (ranges or [1]) != (list(self.dimensions[:-1]) or [1]):
            raise Unsupported("ops after the reduction of a fused kernel")
        src_node, red_acc, kind = self.reduction
        env: Dict[Node, Any] = {}
        for n in body.root_block.graph.nodes:
            if n.op in ("placeholder", "output"):
                continue
            if n.op == "call_module" and n.target == "get_index":
                env[n] = body.indexing_exprs[n.args[0]]
                continue
            if n.op != "call_method":
                raise Unsupported("ops after the reduction of a fused kernel")
            a = [env.get(x, x) if isinstance(x, Node) else x for x in n.args[1:]]
            t = n.target
            if t == "load" and a[0] == red_acc.name:
                env[n] = ("reduced", 1.0)
            elif t == "constant":
                env[n] = float(a[0])
            elif t == "to_dtype" and (isinstance(a[0], float) or (isinstance(a[0], tuple) and a[1] in _FLOATS)):
                env[n] = a[0]
            elif t in ("mul", "truediv") and kind == "sum":
                x, y = a
                if isinstance(x, tuple) and isinstance(y, float):
                    env[n] = ("reduced", x[1] * y if t == "mul" else x[1] / y)
                elif isinstance(y, tuple) and isinstance(x, float) and t == "mul":
                    env[n] = ("reduced", y[1] * x)
                else:
                    raise Unsupported("ops after the reduction of a fused kernel")
            elif t == "store" and isinstance(a[2], tuple):
                import torch._inductor.virtualized as virtualized
                if virtualized.V.graph.get_dtype(a[0]) != torch.float16:
                    raise Unsupported("reduced result stored in another dtype")
                shape, _ = access_shape(a[1], variables, ranges, f"store {a[0]}")
                if list(shape) != list(self.dimensions[:-1] or [1]):
                    raise Unsupported("reduced result not laid out over the outer dims")
                self.values[a[0]] = src_node
                self.reduction = (src_node, TensorAccess(a[0], a[1], torch.float16, tuple(shape)), kind)
                self.reduce_scale *= a[2][1]
                self.scaled_from = red_acc.name
            else:
                raise Unsupported("ops after the reduction of a fused kernel")

    def _op(self, name: str, args: list, variables, ranges):
        if name == "load":
            buf, index = args[0], args[1]
            if buf in self.values:      # produced earlier in this kernel: use the value, not the memory
                return self.values[buf]
            import torch._inductor.virtualized as virtualized
            dtype = virtualized.V.graph.get_dtype(buf)
            if dtype != torch.float16:
                raise Unsupported(f"load of a {dtype} buffer")
            shape, _ = access_shape(index, variables, ranges, f"load {buf}")
            return self._placeholder(TensorAccess(buf, index, dtype, shape))
        if name == "constant":
            value, dtype = args[0], args[1]
            if dtype not in _FLOATS and dtype not in (torch.int64, torch.int32, torch.bool):
                raise Unsupported(f"constant of dtype {dtype}")
            return float(value)
        if name == "to_dtype":
            x, dtype = args[0], args[1]
            if dtype in _FLOATS or isinstance(x, float):
                return x                # every value of a program is an fp16 value: nothing to convert
            raise Unsupported(f"conversion to {dtype}")
        if name in _UNARY:
            (x,) = args
            if isinstance(x, float):
                raise Unsupported(f"{name} of a constant")
            return self._call(_UNARY[name], [x])
        if name == "square":
            (x,) = args
            return self._call(aten.mul.Tensor, [x, x])
        if name in _BINARY:
            a, b = args[0], args[1]
            target = _BINARY[name]
            if isinstance(a, float) and isinstance(b, float):
                raise Unsupported(f"{name} of two constants")
            if isinstance(a, float) or isinstance(b, float):
                target = _SCALAR_FORM.get(target, target)
                if target is aten.pow.Tensor_Scalar and isinstance(a, float):
                    raise Unsupported("constant base of pow")
            return self._call(target, [a, b], mask=name in ("eq", "ne", "lt", "le", "gt", "ge"))
        if name == "where":
            c, a, b = args
            return self._call(aten.where.self, [c, a, b])
        if name == "store":
            buf, index, value = args[0], args[1], args[2]
            if len(args) > 3 and args[3] is not None:
                raise Unsupported(f"store mode {args[3]}")
            import torch._inductor.virtualized as virtualized
            if virtualized.V.graph.get_dtype(buf) != torch.float16:
                raise Unsupported(f"store into a {virtualized.V.graph.get_dtype(buf)} buffer")
            if not isinstance(value, Node):
                raise Unsupported("store of a constant")
            shape, _ = access_shape(index, variables, ranges, f"store {buf}")
            if list(shape) != list(self.dimensions):
                raise Unsupported(f"store {buf} does not cover the iteration space {self.dimensions}")
            self.values[buf] = value
            if not self.removable(buf):
                self.stored.append((value, TensorAccess(buf, index, torch.float16, shape)))
            return None
        if name == "reduction":
            dtype, src_dtype, kind, value = args
            if kind not in _REDUCTIONS or not isinstance(value, Node) or dtype not in _FLOATS:
                raise Unsupported(f"reduction {kind}")
            return ("reduction", kind, value, dtype)
        if name == "store_reduction":
            buf, index, value = args
            if not (isinstance(value, tuple) and value and value[0] == "reduction"):
                raise Unsupported("store_reduction of something that is not a reduction")
            shape, _ = access_shape(index, variables, ranges, f"store_reduction {buf}")
            if list(shape[:-1]) != list(self.dimensions[:-1]) or shape[-1] != 1:
                raise Unsupported(f"reduced output {buf} is not laid out over the outer dims")
            import torch._inductor.virtualized as virtualized
            self.reduction = (value[2], TensorAccess(buf, index, virtualized.V.graph.get_dtype(buf), tuple(shape[:-1])),
                              value[1])
            return None
        raise Unsupported(f"loop body op {name}")

    # -- program --------------------------------------------------------------------------
    def summarize(self) -> KernelSummary:
        for snode in self.nodes:
            self._read_body(snode)
        if not self.order and self.reduction is None and not self.stored:
            raise Unsupported("kernel with no output")
        # a bare copy or a bare reduction has no op node: give the lineariser one to hang things on
        members = list(self.order)
        stored_nodes = {id(v) for v, _ in self.stored}
        red_src = self.reduction[0] if self.reduction else None
        for v, _ in self.stored:
            if v.op == "placeholder":
                raise Unsupported("plain copy kernel")
        if red_src is not None and red_src.op == "placeholder":
            # reduce a tensor as it is: x * 1 keeps the value and gives the group a member
            red_src = self._call(aten.mul.Scalar, [red_src, 1.0])
            members = list(self.order)
        if not members:
            raise Unsupported("kernel without pointwise work")
        if red_src is not None and red_src is not members[-1]:
            raise Unsupported("reduction of a value that is not the last one computed")
        group = fusion.Group(members, tuple(self.dimensions))
        red_node = None
        if self.reduction is not None:
            kind = self.reduction[2]
            red_node = self.graph.call_function(_REDUCTIONS[kind], (red_src, [-1]))
            red_node.meta["val"] = self._meta(self.dimensions[:-1] or [1])
            group.reduction = red_node

        def users_outside(n: Node) -> bool:
            return id(n) in stored_nodes

        if self.reduction is not None and self.reduction[1].dtype != torch.float16:
            raise Unsupported(f"reduction result kept in {self.reduction[1].dtype}")
        try:
            prog = fusion.linearise(group, users_outside)
        except fusion.CannotFuse as e:
            raise Unsupported(f"fused group does not fit one program: {e}")
        prog.reduce_scale *= self.reduce_scale
        inputs = [self.input_access[n] for n in prog.inputs]
        out_by_node = {id(v): acc for v, acc in self.stored}
        outputs = [out_by_node[id(n)] for n in prog.outputs]
        if len(outputs) != len(self.stored):
            raise Unsupported("a value is stored to two buffers")
        args: List[Any] = [TensorArg(True, i, acc.dtype) for i, acc in enumerate(inputs)]
        k = len(inputs)
        for acc in outputs:
            args.append(TensorArg(False, k, acc.dtype))
            k += 1
        red_acc = self.reduction[1] if self.reduction else None
        if red_acc is not None:
            args.append(TensorArg(False, k, red_acc.dtype))
        dims = list(self.dimensions)
        variables_scale = lambda acc: [1 if s != 1 or d == 1 else -1 for s, d in zip(acc.shape, dims)]  # noqa: E731
        scales = [variables_scale(a) for a in inputs] + [variables_scale(a) for a in outputs]
        if red_acc is not None:
            scales.append([1] * (len(dims) - 1) + [-1])
        op_info = {
            "insns": prog.insns, "n_inputs": len(inputs), "n_outputs": len(outputs),
            "input_shapes": [tuple(a.shape) for a in inputs],
            "reduce": prog.reduce, "reduce_scale": prog.reduce_scale, "keepdim": False,
        }
        spec = KernelSpec(op="fused_pointwise" + ("_rowreduce" if prog.reduce else ""),
                          is_reduction=prog.reduce is not None, dimensions=dims, args=args, scales=scales,
                          op_info=op_info)
        return KernelSummary(dims, inputs, outputs, red_acc, spec)
