"""Fusion of pointwise (+ trailing row reduction) groups of an aten FX graph into programs
for the accumulator machine of ``ts_pointwise_chain``.

This is the counterpart of the reference's kernel analysis (SpyreKernel,
torch_spyre/_inductor/spyre_kernel.py:85-369), with one difference that matters for
bandwidth: the reference emits one device program per op (fusion is switched off in
torch_spyre/_inductor/choices.py:58-83); here a whole group of pointwise ops, optionally ended
by a reduction over the innermost dim, becomes one program and therefore one pass over HBM.

Nothing in this module touches a device: it maps FX nodes to instruction lists.
"""
from __future__ import annotations

import dataclasses
import operator
from typing import Dict, List, Optional, Sequence, Set, Tuple

import torch
from torch.fx import Node

aten = torch.ops.aten

MAX_INSNS, MAX_INPUTS, MAX_OUTPUTS, MAX_SLOTS = 32, 8, 4, 4

# aten overload -> opcode name (see include/spyre_b200.h)
UNARY = {
    aten.abs.default: "ABS", aten.neg.default: "NEG", aten.exp.default: "EXP",
    aten.log.default: "LOG", aten.sqrt.default: "SQRT", aten.rsqrt.default: "RSQRT",
    aten.reciprocal.default: "RECIP", aten.sigmoid.default: "SIGMOID", aten.tanh.default: "TANH",
    aten.relu.default: "RELU", aten.silu.default: "SILU", aten.sin.default: "SIN",
    aten.cos.default: "COS", aten.erf.default: "ERF", aten.floor.default: "FLOOR",
    aten.ceil.default: "CEIL", aten.sign.default: "SIGN", aten.log1p.default: "LOG1P",
    aten.expm1.default: "EXPM1", aten.mish.default: "MISH", aten.logical_not.default: "LOGICAL_NOT",
}
# (opcode when acc holds the first operand, opcode when acc holds the second operand or None)
BINARY = {
    aten.add.Tensor: ("ADD", "ADD"), aten.add.Scalar: ("ADD", "ADD"),
    aten.sub.Tensor: ("SUB", "RSUB"), aten.sub.Scalar: ("SUB", "RSUB"),
    aten.mul.Tensor: ("MUL", "MUL"), aten.mul.Scalar: ("MUL", "MUL"),
    aten.div.Tensor: ("DIV", "RDIV"), aten.div.Scalar: ("DIV", "RDIV"),
    aten.maximum.default: ("MAX", "MAX"), aten.minimum.default: ("MIN", "MIN"),
    aten.rsub.Scalar: ("RSUB", None),
    aten.pow.Tensor_Scalar: ("POW", None), aten.pow.Tensor_Tensor: ("POW", None),
    aten.eq.Tensor: ("EQ", "EQ"), aten.eq.Scalar: ("EQ", "EQ"),
    aten.ne.Tensor: ("NE", "NE"), aten.ne.Scalar: ("NE", "NE"),
    aten.lt.Tensor: ("LT", "GT"), aten.lt.Scalar: ("LT", "GT"),
    aten.le.Tensor: ("LE", "GE"), aten.le.Scalar: ("LE", "GE"),
    aten.gt.Tensor: ("GT", "LT"), aten.gt.Scalar: ("GT", "LT"),
    aten.ge.Tensor: ("GE", "LE"), aten.ge.Scalar: ("GE", "LE"),
}
REDUCTIONS = {aten.sum.dim_IntList: "sum", aten.amax.default: "max", aten.amin.default: "min",
              aten.mean.dim: "mean"}


def _meta(n: Node):
    return n.meta.get("val") if isinstance(n, Node) else None


def node_shape(n: Node) -> Optional[Tuple[int, ...]]:
    v = _meta(n)
    if isinstance(v, torch.Tensor):
        try:
            return tuple(int(s) for s in v.shape)
        except Exception:
            return None
    return None


def _is_fp16_tensor(n) -> bool:
    v = _meta(n)
    return isinstance(v, torch.Tensor) and v.dtype == torch.float16


COMPARES = {aten.eq.Tensor, aten.eq.Scalar, aten.ne.Tensor, aten.ne.Scalar, aten.lt.Tensor,
            aten.lt.Scalar, aten.le.Tensor, aten.le.Scalar, aten.gt.Tensor, aten.gt.Scalar,
            aten.ge.Tensor, aten.ge.Scalar}


def _is_mask(n) -> bool:
    """A comparison of fp16 tensors: bool in the graph, fp16 0/1 inside a fused program."""
    return (isinstance(n, Node) and n.op == "call_function" and n.target in COMPARES
            and all(_is_fp16_tensor(a) or isinstance(a, (int, float, bool)) for a in n.args[:2])
            and any(_is_fp16_tensor(a) for a in n.args[:2]))


def is_pointwise(n: Node) -> bool:
    if n.op != "call_function":
        return False
    if _is_mask(n):
        return True
    if not _is_fp16_tensor(n):
        return False
    t = n.target
    if t in UNARY:
        return True
    if t is aten.gelu.default:
        return True
    if t in BINARY:
        if t in (aten.add.Tensor, aten.sub.Tensor, aten.add.Scalar, aten.sub.Scalar, aten.rsub.Scalar):
            if n.kwargs.get("alpha", 1) != 1 or len(n.args) > 2:
                return False
        return all(_is_fp16_tensor(a) or isinstance(a, (int, float, bool)) for a in n.args[:2])
    if t is aten.where.self:
        return (_is_fp16_tensor(n.args[0]) or _is_mask(n.args[0])) and \
            all(_is_fp16_tensor(a) or isinstance(a, (int, float)) for a in n.args[1:3])
    return False


def reduction_kind(n: Node) -> Optional[Tuple[str, bool]]:
    """(kind, keepdim) if n reduces exactly the innermost dim of an fp16 tensor."""
    if n.op != "call_function" or n.target not in REDUCTIONS or not _is_fp16_tensor(n):
        return None
    src = n.args[0]
    shape = node_shape(src) if isinstance(src, Node) else None
    if not shape or not _is_fp16_tensor(src):
        return None
    dims = n.args[1] if len(n.args) > 1 else n.kwargs.get("dim")
    if dims is None or isinstance(dims, int):
        dims = [dims] if dims is not None else []
    dims = [d % len(shape) for d in dims]
    if dims != [len(shape) - 1]:
        return None
    keepdim = bool(n.args[2]) if len(n.args) > 2 else bool(n.kwargs.get("keepdim", False))
    if n.kwargs.get("dtype") not in (None, torch.float16):
        return None
    return REDUCTIONS[n.target], keepdim


# ---- grouping ------------------------------------------------------------------------

@dataclasses.dataclass
class Group:
    nodes: List[Node]                 # pointwise nodes, in graph order
    shape: Tuple[int, ...]            # iteration space
    reduction: Optional[Node] = None  # trailing reduction over the innermost dim


def build_groups(graph: torch.fx.Graph) -> Tuple[List[Group], Dict[Node, Group]]:
    order = {n: i for i, n in enumerate(graph.nodes)}
    deps: Dict[Node, Set[Node]] = {}
    for n in graph.nodes:
        d: Set[Node] = set()
        for a in n.all_input_nodes:
            d.add(a)
            d |= deps[a]
        deps[n] = d
    groups: List[Group] = []
    owner: Dict[Node, Group] = {}

    def can_join(n: Node, g: Group) -> bool:
        if g.reduction is not None:
            return False
        gset = set(g.nodes)
        for a in n.all_input_nodes:
            if a in gset:
                continue
            if deps[a] & gset:   # an outside input that itself needs the group's result
                return False
        return True

    def try_merge(a: Group, b: Group) -> bool:
        """Merge b into a if no outside node sits between them in the dependency order."""
        merged = sorted(a.nodes + b.nodes, key=lambda m: order[m])
        mset = set(merged)
        for m in merged:
            for inp in m.all_input_nodes:
                if inp not in mset and deps[inp] & mset:
                    return False
        a.nodes = merged
        for m in b.nodes:
            owner[m] = a
        groups.remove(b)
        return True

    for n in graph.nodes:
        if is_pointwise(n):
            shape = node_shape(n)
            cands: List[Group] = []
            for a in n.all_input_nodes:
                g = owner.get(a)
                if g is not None and g not in cands and g.shape == shape and can_join(n, g):
                    cands.append(g)
            cands.sort(key=lambda g: order[g.nodes[-1]], reverse=True)
            target = cands[0] if cands else None
            if target is None:
                target = Group([], shape)
                groups.append(target)
            else:
                for other in cands[1:]:
                    try_merge(target, other)
            target.nodes.append(n)
            owner[n] = target
            continue
        rk = reduction_kind(n)
        if rk is not None:
            src = n.args[0]
            g = owner.get(src)
            if g is not None and g.reduction is None and g.nodes[-1] is src and g.shape == node_shape(src):
                g.reduction = n
                owner[n] = g
    return groups, owner


# ---- linearisation ---------------------------------------------------------------------

@dataclasses.dataclass
class Program:
    insns: List[Tuple[str, tuple, tuple]]   # (opcode, operand A, operand B); operand = (kind, idx, imm)
    inputs: List[Node]                      # external tensor operands, in first-use order
    outputs: List[Node]                     # full-shape results, index = STORE slot
    shape: Tuple[int, ...]
    reduce: Optional[str] = None            # "sum" / "max" / "min"
    reduce_scale: float = 1.0
    keepdim: bool = False
    reduce_node: Optional[Node] = None


class CannotFuse(Exception):
    pass


NONE, TENSOR, IMM, SAVED = 0, 1, 2, 3
_NOP = (NONE, 0, 0.0)


def linearise(g: Group, users_outside) -> Program:
    """Turns a group into accumulator-machine code.  `users_outside(node)` tells whether a
    node's value is needed outside the group (another kernel or a graph output)."""
    nodes = g.nodes
    pos = {n: i for i, n in enumerate(nodes)}
    inside = set(nodes)
    insns: List[Tuple[str, tuple, tuple]] = []
    inputs: List[Node] = []
    outputs: List[Node] = []
    slot_of: Dict[Node, int] = {}
    free_slots = list(range(MAX_SLOTS))

    def last_use(n: Node) -> int:
        return max([pos[u] for u in n.users if u in inside] + [-1])

    def tensor_operand(n: Node):
        if n not in inputs:
            if len(inputs) == MAX_INPUTS:
                raise CannotFuse("too many inputs")
            inputs.append(n)
        return (TENSOR, inputs.index(n), 0.0)

    def operand(a, acc: Optional[Node]):
        if isinstance(a, Node):
            if a in inside:
                if a in slot_of:
                    return (SAVED, slot_of[a], 0.0)
                raise CannotFuse("operand neither in the accumulator nor saved")
            return tensor_operand(a)
        return (IMM, 0, float(a))

    def must_save(n: Node, i: int) -> bool:
        uses = [u for u in n.users if u in inside]
        for u in uses:
            if pos[u] != i + 1:
                return True
            tensor_args = [a for a in u.args if isinstance(a, Node)]
            if tensor_args.count(n) > 1:
                return True
            if u.target is aten.where.self and u.args[0] is not n:
                return True
            if u.target in BINARY and len(u.args) > 1 and u.args[1] is n and BINARY[u.target][1] is None:
                return True
        return False

    acc: Optional[Node] = None
    for i, n in enumerate(nodes):
        t = n.target
        args = list(n.args)
        if t in UNARY or t is aten.gelu.default:
            src = args[0]
            if acc is not src:
                insns.append(("LOAD", operand(src, acc), _NOP))
            if t is aten.gelu.default:
                op = "GELU_TANH" if n.kwargs.get("approximate", "none") == "tanh" else "GELU"
            else:
                op = UNARY[t]
            insns.append((op, _NOP, _NOP))
        elif t in BINARY:
            a, b = args[0], args[1]
            fwd, rev = BINARY[t]
            if acc is not None and acc is a and not (acc is b):
                insns.append((fwd, operand(b, acc), _NOP))
            elif acc is not None and acc is b and rev is not None and not (acc is a):
                insns.append((rev, operand(a, acc), _NOP))
            else:
                if not isinstance(a, Node):
                    # scalar first operand: start from the tensor with the reversed opcode
                    if rev is None:
                        raise CannotFuse("scalar base of pow")
                    if acc is not b:
                        insns.append(("LOAD", operand(b, acc), _NOP))
                    insns.append((rev, operand(a, acc), _NOP))
                else:
                    if acc is not a:
                        insns.append(("LOAD", operand(a, acc), _NOP))
                    insns.append((fwd, operand(b, acc), _NOP))
        elif t is aten.where.self:
            cond, a, b = args[0], args[1], args[2]
            if acc is not cond:
                insns.append(("LOAD", operand(cond, acc), _NOP))
            insns.append(("WHERE", operand(a, acc), operand(b, acc)))
        else:
            raise CannotFuse(f"unexpected node {n}")
        acc = n
        # free slots whose last use was this node
        for m in list(slot_of):
            if last_use(m) <= i:
                free_slots.append(slot_of.pop(m))
        if must_save(n, i):
            if not free_slots:
                raise CannotFuse("more than 4 live intermediate values")
            free_slots.sort()
            slot_of[n] = free_slots.pop(0)
            insns.append(("SAVE", (NONE, slot_of[n], 0.0), _NOP))
        if users_outside(n) and not (g.reduction is not None and n is nodes[-1]
                                     and all(u is g.reduction for u in n.users)):
            if not _is_fp16_tensor(n):
                raise CannotFuse("a boolean mask is needed outside the fused group")
            if len(outputs) == MAX_OUTPUTS:
                raise CannotFuse("too many outputs")
            outputs.append(n)
            insns.append(("STORE", (NONE, len(outputs) - 1, 0.0), _NOP))
    if len(insns) > MAX_INSNS:
        raise CannotFuse("program too long")
    prog = Program(insns, inputs, outputs, g.shape)
    if g.reduction is not None:
        kind, keepdim = reduction_kind(g.reduction)
        prog.reduce = "sum" if kind == "mean" else kind
        prog.reduce_scale = 1.0 / g.shape[-1] if kind == "mean" else 1.0
        prog.keepdim = keepdim
        prog.reduce_node = g.reduction
    elif not outputs:
        raise CannotFuse("group with no visible result")
    return prog


def emulate(prog: Program, values: Dict[Node, torch.Tensor]) -> Dict[Node, torch.Tensor]:
    """Reference executor of a program on host tensors, op by op in fp16: used by the tests to
    check that linearisation preserves the graph's meaning."""
    import torch.nn.functional as F

    un = {"ABS": torch.abs, "NEG": torch.neg, "EXP": torch.exp, "LOG": torch.log, "SQRT": torch.sqrt,
          "RSQRT": torch.rsqrt, "RECIP": torch.reciprocal, "SIGMOID": torch.sigmoid,
          "TANH": torch.tanh, "RELU": torch.relu, "SILU": F.silu, "GELU": F.gelu,
          "GELU_TANH": lambda x: F.gelu(x, approximate="tanh"), "SIN": torch.sin, "COS": torch.cos,
          "ERF": torch.erf, "FLOOR": torch.floor, "CEIL": torch.ceil, "SIGN": torch.sign,
          "LOG1P": torch.log1p, "EXPM1": torch.expm1, "MISH": F.mish,
          "LOGICAL_NOT": lambda x: (x == 0).to(x.dtype)}
    bi = {"ADD": lambda x, y: x + y, "SUB": lambda x, y: x - y, "RSUB": lambda x, y: y - x,
          "MUL": lambda x, y: x * y, "DIV": lambda x, y: x / y, "RDIV": lambda x, y: y / x,
          "MAX": torch.maximum, "MIN": torch.minimum, "POW": torch.pow,
          "EQ": lambda x, y: (x == y).to(x.dtype), "NE": lambda x, y: (x != y).to(x.dtype),
          "LT": lambda x, y: (x < y).to(x.dtype), "LE": lambda x, y: (x <= y).to(x.dtype),
          "GT": lambda x, y: (x > y).to(x.dtype), "GE": lambda x, y: (x >= y).to(x.dtype)}
    shape = prog.shape
    slots: Dict[int, torch.Tensor] = {}
    out: Dict[Node, torch.Tensor] = {}
    acc = torch.zeros(shape, dtype=torch.float16)

    def val(opnd):
        kind, idx, imm = opnd
        if kind == TENSOR:
            return values[prog.inputs[idx]].expand(shape)
        if kind == IMM:
            return torch.full(shape, imm, dtype=torch.float16)
        if kind == SAVED:
            return slots[idx]
        raise AssertionError("operand missing")

    for op, a, b in prog.insns:
        if op == "LOAD":
            acc = val(a).clone()
        elif op == "SAVE":
            slots[a[1]] = acc.clone()
        elif op == "STORE":
            out[prog.outputs[a[1]]] = acc.clone()
        elif op == "WHERE":
            acc = torch.where(acc != 0, val(a), val(b))
        elif op in un:
            acc = un[op](acc)
        else:
            acc = bi[op](acc, val(a))
    if prog.reduce:
        fn = {"sum": lambda t: t.sum(-1, keepdim=prog.keepdim),
              "max": lambda t: t.amax(-1, keepdim=prog.keepdim),
              "min": lambda t: t.amin(-1, keepdim=prog.keepdim)}[prog.reduce]
        r = fn(acc.float())
        out[prog.reduce_node] = (r * prog.reduce_scale).half()
    return out
