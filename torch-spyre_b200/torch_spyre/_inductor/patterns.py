"""Graph rewrites that turn what stock model code traces to into the fused spyre ops.

The reference removes Inductor's own fusion patterns and decomposes layer norm into its custom
ops before lowering (torch_spyre/_inductor/__init__.py:81-84, decompositions.py:26-58).  Here the
direction is the opposite: sub-graphs that have a dedicated kernel are recognised and replaced
by one node, so that an unmodified module (the decoder layer of the reference's own
tests/test_modules.py:178-211) runs on the fused kernels.

* ``rewrite_dynamo_graph`` runs on the graph dynamo hands to the backend (torch-level calls):
  ``F.scaled_dot_product_attention(..., is_causal=True)`` -> ``spyre.sdpa_causal``.
* ``rewrite_aten_graph`` runs on the aten graph AOT autograd produces:
  the fp32 RMS-norm idiom -> ``spyre.rms_norm``; rotary position embedding on
  ``[batch, heads, seq, 128]`` views of a projection -> ``spyre.rotary``; a residual added to a
  matmul -> ``addmm`` with a matrix-shaped bias, which the GEMM adds in its epilogue;
  ``silu(x @ Wg^T) * (x @ Wu^T)`` -> ``spyre.swiglu_linear`` (one GEMM over interleaved weights).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch.fx import GraphModule, Node

aten = torch.ops.aten


def _is(n, target) -> bool:
    return isinstance(n, Node) and n.op == "call_function" and n.target is target


def _only_users(n: Node, *users: Node) -> bool:
    return set(n.users) == set(users)


def _shape(n: Node):
    v = n.meta.get("val", n.meta.get("example_value"))
    return tuple(v.shape) if isinstance(v, torch.Tensor) else None


def _dtype(n: Node):
    v = n.meta.get("val", n.meta.get("example_value"))
    return v.dtype if isinstance(v, torch.Tensor) else None


# ---- dynamo level -----------------------------------------------------------------------

def rewrite_dynamo_graph(gm: GraphModule) -> int:
    """Causal SDPA calls without a mask or dropout become one ``spyre.sdpa_causal`` node."""
    sdpa = torch._C._nn.scaled_dot_product_attention
    count = 0
    for n in list(gm.graph.nodes):
        if n.op != "call_function" or n.target is not sdpa:
            continue
        names = ("query", "key", "value", "attn_mask", "dropout_p", "is_causal", "scale", "enable_gqa")
        bound = dict(zip(names, n.args))
        bound.update(n.kwargs)
        if not bound.get("is_causal") or bound.get("attn_mask") is not None or bound.get("dropout_p", 0.0):
            continue
        q, k, v = bound["query"], bound["key"], bound["value"]
        qs, ks, vs = _shape(q), _shape(k), _shape(v)
        if qs is None or len(qs) != 4 or ks != qs or vs != qs:
            continue   # grouped-query attention or a cached key length: not the fused kernel's case
        if qs[-1] != 128 or any(_dtype(t) != torch.float16 for t in (q, k, v)):
            continue   # the fused kernel is built for head_dim 128 in fp16; leave stock SDPA alone
        scale = bound.get("scale")
        if scale is None:
            scale = 1.0 / math.sqrt(qs[-1])
        with gm.graph.inserting_before(n):
            new = gm.graph.call_function(torch.ops.spyre.sdpa_causal.default, (q, k, v, float(scale)))
        new.meta = dict(n.meta)
        n.replace_all_uses_with(new)
        gm.graph.erase_node(n)
        count += 1
    if count:
        gm.graph.lint()
        gm.recompile()
    return count


# ---- aten level -------------------------------------------------------------------------

def _match_rms_norm(mulw: Node):
    """weight * (x.float() * rsqrt(mean(x.float()^2, -1, keepdim) + eps)).half()"""
    if not _is(mulw, aten.mul.Tensor):
        return None
    for wi in (0, 1):
        w, c16 = mulw.args[wi], mulw.args[1 - wi]
        if not (_is(c16, aten._to_copy.default) and c16.kwargs.get("dtype") == torch.float16):
            continue
        m = c16.args[0]
        if not _is(m, aten.mul.Tensor):
            continue
        for xi in (0, 1):
            x32, r = m.args[xi], m.args[1 - xi]
            if not (_is(r, aten.rsqrt.default) and _is(x32, aten._to_copy.default)):
                continue
            a = r.args[0]
            if not (_is(a, aten.add.Tensor) and isinstance(a.args[1], (int, float))):
                continue
            mean = a.args[0]
            if not _is(mean, aten.mean.dim):
                continue
            p = mean.args[0]
            if not (_is(p, aten.pow.Tensor_Scalar) and p.args[1] == 2 and p.args[0] is x32):
                continue
            x = x32.args[0]
            xs, ws = _shape(x), _shape(w) if isinstance(w, Node) else None
            dims = list(mean.args[1])
            keep = mean.args[2] if len(mean.args) > 2 else mean.kwargs.get("keepdim", False)
            if xs is None or ws is None or len(ws) != 1 or ws[0] != xs[-1] or not keep:
                continue
            if dims not in ([-1], [len(xs) - 1]) or x32.kwargs.get("dtype") != torch.float32:
                continue
            if not (_only_users(c16, mulw) and _only_users(m, c16) and _only_users(r, m) and
                    _only_users(a, r) and _only_users(mean, a) and _only_users(p, mean) and
                    _only_users(x32, p, m)):
                continue
            return x, w, float(a.args[1]), [mulw, c16, m, r, a, mean, p, x32]
    return None


def _swaps_seq_and_heads(n) -> bool:
    """transpose(1, 2) of a 4-D tensor, in either of the forms tracing leaves it in."""
    if _is(n, aten.transpose.int):
        return tuple(n.args[1:]) in ((1, 2), (2, 1))
    return _is(n, aten.permute.default) and list(n.args[1]) == [0, 2, 1, 3]


def _match_rotary(add: Node):
    """q*cos + cat(-q[..., 64:], q[..., :64]) * sin with q = proj.view(b, s, h, 128).transpose(1, 2)
    and cos / sin = table.unsqueeze(1), table [b, s, 128].  Returns (proj, cos, sin, heads, nodes)."""
    if not _is(add, aten.add.Tensor) or len(add.args) != 2:
        return None
    for i in (0, 1):
        m1, m2 = add.args[i], add.args[1 - i]
        if not (_is(m1, aten.mul.Tensor) and _is(m2, aten.mul.Tensor)):
            continue
        q, cos_u = m1.args
        cat, sin_u = m2.args
        if not (_is(cat, aten.cat.default) and _swaps_seq_and_heads(q)):
            continue
        parts = cat.args[0]
        dim = cat.args[1] if len(cat.args) > 1 else 0
        qs = _shape(q)
        if qs is None or len(qs) != 4 or qs[-1] != 128 or dim not in (-1, 3) or len(parts) != 2:
            continue
        neg, lo = parts
        if not (_is(neg, aten.neg.default) and _is(lo, aten.slice.Tensor)):
            continue
        hi = neg.args[0]
        if not _is(hi, aten.slice.Tensor):
            continue

        def sl(n):
            a = list(n.args) + [None] * (5 - len(n.args))
            return a[0], a[1], a[2] or 0, a[3]
        if sl(lo)[0] is not q or sl(hi)[0] is not q or sl(lo)[1] not in (3, -1) or sl(hi)[1] not in (3, -1):
            continue
        if sl(lo)[2] != 0 or sl(lo)[3] != 64 or sl(hi)[2] != 64 or (sl(hi)[3] or 1 << 62) < 128:
            continue
        if not (_is(cos_u, aten.unsqueeze.default) and _is(sin_u, aten.unsqueeze.default)):
            continue
        if cos_u.args[1] != 1 or sin_u.args[1] != 1:
            continue
        cos, sin = cos_u.args[0], sin_u.args[0]
        view = q.args[0]
        if not (_is(view, aten.view.default) or _is(view, aten._unsafe_view.default)):
            continue
        proj = view.args[0]
        ps, cs = _shape(proj), _shape(cos)
        b, h, s, d = qs
        if ps != (b, s, h * d) or cs != (b, s, d) or _shape(sin) != cs:
            continue
        if not (_only_users(m1, add) and _only_users(m2, add) and _only_users(cat, m2) and
                _only_users(neg, cat) and _only_users(hi, neg) and _only_users(lo, cat) and
                _only_users(q, m1, lo, hi) and _only_users(view, q)):
            continue
        return proj, cos, sin, h, [add, m1, m2, cat, neg, hi, lo, q, view]
    return None


def _match_residual_mm(add: Node):
    """res + mm(a, b).view(shape)  (either operand order; the view is optional)."""
    if not _is(add, aten.add.Tensor) or len(add.args) != 2 or add.kwargs.get("alpha", 1) != 1:
        return None
    for i in (0, 1):
        res, prod = add.args[i], add.args[1 - i]
        if not isinstance(res, Node) or not isinstance(prod, Node):
            continue
        view = prod if (_is(prod, aten.view.default) or _is(prod, aten._unsafe_view.default)) else None
        mm = view.args[0] if view is not None else prod
        if not _is(mm, aten.mm.default):
            continue
        ms, rs, outs = _shape(mm), _shape(res), _shape(add)
        if ms is None or rs is None or rs != outs or len(ms) != 2:
            continue
        if ms[0] * ms[1] != math.prod(rs) or rs[-1] != ms[1]:
            continue
        if view is not None and not (_only_users(view, add) and _only_users(mm, view)):
            continue
        if view is None and not _only_users(mm, add):
            continue
        if res is mm or res is view:
            continue
        return res, mm, view
    return None


def _linear_parts(v):
    """(view, mm, x2d, weight) of ``mm(x2d, weight^T)`` seen through an optional view."""
    view = v if (_is(v, aten.view.default) or _is(v, aten._unsafe_view.default)) else None
    mm = view.args[0] if view is not None else v
    if not _is(mm, aten.mm.default):
        return None
    wt = mm.args[1]
    if _is(wt, aten.permute.default) and list(wt.args[1]) == [1, 0]:
        w = wt.args[0]
    elif _is(wt, aten.t.default):
        w = wt.args[0]
    else:
        return None
    if view is not None and not _only_users(mm, view):
        return None
    return view, mm, mm.args[0], w


def _same_matrix(a, b) -> bool:
    """The same node, or two views of one source with the same shape."""
    if a is b:
        return True
    views = (aten.view.default, aten._unsafe_view.default, aten.reshape.default)
    return (isinstance(a, Node) and isinstance(b, Node) and a.target in views and b.target in views and
            a.args[0] is b.args[0] and _shape(a) == _shape(b) and _shape(a) is not None)


def _match_swiglu(mul: Node):
    """silu(x @ Wg^T) * (x @ Wu^T)"""
    if not _is(mul, aten.mul.Tensor) or len(mul.args) != 2:
        return None
    for i in (0, 1):
        act, up = mul.args[i], mul.args[1 - i]
        if not (_is(act, aten.silu.default) and _only_users(act, mul) and isinstance(up, Node)):
            continue
        gp, upp = _linear_parts(act.args[0]), _linear_parts(up)
        if gp is None or upp is None:
            continue
        (gv, gmm, gx, wg), (uv, umm, ux, wu) = gp, upp
        ws = _shape(wg)
        if ws is None or ws != _shape(wu) or len(ws) != 2 or ws[0] % 64 or not _same_matrix(gx, ux):
            continue
        g_out = gv if gv is not None else gmm
        u_out = uv if uv is not None else umm
        if not (_only_users(g_out, act) and _only_users(u_out, mul)):
            continue
        return gx, wg, wu, [mul, act] + [n for n in (gv, gmm, uv, umm) if n is not None]
    return None


def _match_fp32_softmax(back: Node):
    """softmax(x, dim, dtype=float32).to(float16) on an fp16 x, as model code writes it to keep the
    reduction in fp32: _to_copy(fp16 -> fp32) -> _softmax -> _to_copy(-> fp16).  The device's fp16
    softmax already computes in fp32 and rounds once at the end, which is exactly this."""
    if not _is(back, aten._to_copy.default) or _dtype(back) != torch.float16 or not back.args:
        return None
    sm = back.args[0]
    if not _is(sm, aten._softmax.default) or _dtype(sm) != torch.float32 or not _only_users(sm, back):
        return None
    if len(sm.args) < 3 or sm.args[2]:
        return None
    up = sm.args[0]
    if not _is(up, aten._to_copy.default) or _dtype(up) != torch.float32 or not _only_users(up, sm):
        return None
    x = up.args[0]
    if not isinstance(x, Node) or _dtype(x) != torch.float16:
        return None
    # only a dtype change on either side: no move to another device, no other layout, no copy semantics
    here = x.meta["val"].device if isinstance(x.meta.get("val"), torch.Tensor) else None
    for conv in (up, back):
        for key, value in conv.kwargs.items():
            if key == "dtype" or value is None or (key == "layout" and value == torch.strided) or \
                    (key == "device" and here is not None and torch.device(value) == here) or \
                    (key in ("non_blocking", "pin_memory") and not value):
                continue
            return None
    return x, sm.args[1], [back, sm, up]


def rewrite_aten_graph(gm: GraphModule) -> int:
    g = gm.graph
    count = 0
    for n in list(g.nodes):
        if n.op != "call_function" or not n.users and n.op != "output":
            continue
        hit = _match_fp32_softmax(n)
        if hit is not None:
            x, dim, dead = hit
            with g.inserting_before(n):
                new = g.call_function(aten._softmax.default, (x, dim, False))
            new.meta = dict(n.meta)
            n.replace_all_uses_with(new)
            for d in dead:
                g.erase_node(d)
            count += 1
            continue
        hit = _match_swiglu(n)
        if hit is not None:
            x2d, wg, wu, dead = hit
            rows, n_out = _shape(x2d)[0], _shape(wg)[0]
            with g.inserting_before(n):
                fused = g.call_function(torch.ops.spyre.swiglu_linear.default, (x2d, wg, wu))
                new = g.call_function(aten.reshape.default, (fused, list(_shape(n))))
            fused.meta = {"val": torch.empty((rows, n_out), dtype=torch.float16, device="meta")}
            new.meta = dict(n.meta)
            n.replace_all_uses_with(new)
            for d in dead:
                g.erase_node(d)
            count += 1
            continue
        hit = _match_residual_mm(n)
        if hit is not None:
            res, mm, view = hit
            m_rows, n_cols = _shape(mm)
            out_shape = list(_shape(n))
            with g.inserting_before(n):
                res2 = g.call_function(aten.reshape.default, (res, [m_rows, n_cols]))
                am = g.call_function(aten.addmm.default, (res2, mm.args[0], mm.args[1]))
                new = g.call_function(aten.reshape.default, (am, out_shape))
            for node, shp in ((res2, (m_rows, n_cols)), (am, (m_rows, n_cols))):
                node.meta = {"val": torch.empty(shp, dtype=torch.float16, device="meta")}
            new.meta = dict(n.meta)
            n.replace_all_uses_with(new)
            g.erase_node(n)
            if view is not None:
                g.erase_node(view)
            g.erase_node(mm)
            count += 1
            continue
        hit = _match_rms_norm(n)
        if hit is not None:
            x, w, eps, dead = hit
            with g.inserting_before(n):
                new = g.call_function(torch.ops.spyre.rms_norm.default, (x, w, eps))
            new.meta = dict(n.meta)
            n.replace_all_uses_with(new)
            for d in dead:
                g.erase_node(d)
            count += 1
            continue
        hit = _match_rotary(n)
        if hit is not None:
            proj, cos, sin, heads, dead = hit
            b, h, s, d = _shape(n)
            with g.inserting_before(n):
                # per-batch tables [b, s, 128] are one table over b*s positions
                x2 = g.call_function(aten.view.default, (proj, [1, b * s, h * d]))
                c2 = g.call_function(aten.view.default, (cos, [b * s, d]))
                s2 = g.call_function(aten.view.default, (sin, [b * s, d]))
                rot = g.call_function(torch.ops.spyre.rotary.default, (x2, c2, s2, heads))
                v4 = g.call_function(aten.view.default, (rot, [b, s, h, d]))
                new = g.call_function(aten.transpose.int, (v4, 1, 2))
            for node, shp in ((x2, (1, b * s, h * d)), (c2, (b * s, d)), (s2, (b * s, d)),
                              (rot, (1, b * s, h * d)), (v4, (b, s, h, d))):
                node.meta = {"val": torch.empty(shp, dtype=torch.float16, device="meta")}
            new.meta = dict(n.meta)
            n.replace_all_uses_with(new)
            for dnode in dead:
                g.erase_node(dnode)
            count += 1
    if count:
        # unsqueeze nodes of the tables and the like may have lost their last user
        g.eliminate_dead_code()
        g.lint()
        gm.recompile()
    return count
