"""Capture: ``torch.export`` (strict) -> core-ATen graph, optionally the joint forward+backward.

Follows the reference's capture stage (compiler/mesh_compiler/export.py:112-212): export, decompose, and
read the signature into state (parameters, buffers, lifted constants), user inputs, and outputs with
their roles (user output, loss, parameter gradient, input gradient, buffer / input mutation).
Shapes are static: a symbolic dimension raises (export.py:155-160).  ``loss=<index>`` switches to the
joint graph via ``torch.export.experimental._export_forward_backward`` (export.py:119-122); unpatched
torch gives gradients for parameters, and gradients of user inputs are taken through explicit
outputs where the exporter provides them.
"""
from __future__ import annotations

import math
import warnings

import torch
from torch.utils import _pytree as pytree
from torch.export.graph_signature import InputKind, OutputKind

from .ir import Exported

_IN_KINDS = {InputKind.PARAMETER: "parameter", InputKind.BUFFER: "buffer", InputKind.CONSTANT_TENSOR: "constant"}
_OUT_KINDS = {OutputKind.USER_OUTPUT: "user", OutputKind.LOSS_OUTPUT: "loss",
              OutputKind.GRADIENT_TO_PARAMETER: "grad_param", OutputKind.GRADIENT_TO_USER_INPUT: "grad_input",
              OutputKind.BUFFER_MUTATION: "mutation", OutputKind.USER_INPUT_MUTATION: "mutation"}


_TABLE = None


def _default_table() -> dict:
    """The default decomposition table, built once per process (building it walks every registered operator)."""
    global _TABLE
    if _TABLE is None:
        _TABLE = dict(torch.export.default_decompositions())
    return dict(_TABLE)


def _views_may_copy(gm: torch.fx.GraphModule) -> int:
    """Every ``view`` of the traced module becomes a ``reshape`` before the graph is traced again with composite
    operators expanded.  The first trace runs fused operators (attention above all) whose results have the memory
    layout of their kernels; module code after them (``transpose(1, 2)`` then ``view``) relies on that layout.  Expanded
    into products and a softmax, the same value comes out dense in another order, and a ``view`` that was legal on the
    first layout is not on the second: a ``reshape`` copies there and stays a view everywhere else."""
    n = 0
    for node in gm.graph.nodes:
        if node.op == "call_function" and node.target in (torch.ops.aten.view.default, torch.ops.aten._unsafe_view.default):
            node.target = torch.ops.aten.reshape.default
            n += 1
    if n:
        gm.recompile()
    return n


def _training_table() -> dict:
    """The default table with attention kept one differentiable operator (``compiler/attention_op.py``) where it has
    neither a mask tensor nor dropout; ``MESH_ATTENTION_OP=0`` leaves it to the plain expansion."""
    import os
    table = _default_table()
    if os.environ.get("MESH_ATTENTION_OP", "1") != "0":
        from .attention_op import substitute as attention
        table[torch.ops.aten.scaled_dot_product_attention.default] = attention
    return table


def _inference_table() -> dict:
    """The default table without attention, which inference graphs keep whole."""
    table = _default_table()
    table.pop(torch.ops.aten.scaled_dot_product_attention.default, None)
    return table


def export(module: torch.nn.Module, args: tuple, kwargs: dict | None = None, *, loss: int | None = None,
           strict: bool = True, decompositions=None, inner_cuts: bool = False) -> Exported:
    """Export ``module(*args, **kwargs)``; with ``loss`` (index of the loss among flat outputs) the joint graph.
    ``inner_cuts``: an input is cut along an inner leading dimension (see :func:`unflatten_linears`): linear layers keep
    their operands' leading dimensions apart (inference graphs)."""
    tied = _untie(module) if loss is not None else {}
    frozen = []
    try:
        try:
            exported = _export(module, args, kwargs, loss, strict, decompositions, inner_cuts)
        except AssertionError as e:
            if loss is None or "did not receive a gradient" not in str(e):
                raise
            # parameters the loss does not depend on (a shared table reached only through its other names, a head that
            # this call does not use): the joint capture refuses them.  Find them with one eager backward pass and
            # capture again with those left out of the gradients
            frozen = _without_gradient(module, args, kwargs, loss)
            if not frozen:
                raise
            for p in frozen:
                p.requires_grad_(False)
            exported = _export(module, args, kwargs, loss, strict, decompositions, inner_cuts)
    finally:
        for p in frozen:
            p.requires_grad_(True)
        _retie(module, tied)
    for name, (qual, _tensor) in list(exported.state.items()):
        if qual in tied:                                    # the placeholder reads the shared tensor, not the stand-in
            exported.state[name] = (qual, tied[qual][1])
    exported.tied = {alias: first for alias, (first, _p) in tied.items()}
    return exported


def _untie(module: torch.nn.Module) -> dict:
    """Parameters that are one tensor under several names (an output projection tied to the embedding): the joint
    forward+backward capture wants a gradient per parameter name and refuses a name that gets none, so every later
    name gets a stand-in of its own for the capture.  Returns ``{later name: (first name, the shared parameter)}``;
    the program then returns, under both names, the sum of the two gradients (:func:`tied_gradients`)."""
    seen, tied = {}, {}
    for name, p in module.named_parameters(remove_duplicate=False):
        if id(p) in seen:
            tied[name] = (seen[id(p)], p)
        else:
            seen[id(p)] = name
    for name, (_first, p) in tied.items():
        owner, _, leaf = name.rpartition(".")
        holder = module.get_submodule(owner) if owner else module
        holder._parameters[leaf] = torch.nn.Parameter(p.detach().clone(), requires_grad=p.requires_grad)
    return tied


def _without_gradient(module: torch.nn.Module, args, kwargs, loss: int) -> list:
    """The parameters (requiring gradients) that get none when output ``loss`` of ``module(*args)`` is differentiated."""
    params = [p for p in module.parameters() if p.requires_grad]
    saved = [p.grad for p in params]
    for p in params:
        p.grad = None
    try:
        out = module(*args, **(kwargs or {}))
        flat = pytree.tree_leaves(out)
        flat[loss].backward()
        return [p for p in params if p.grad is None]
    finally:
        for p, g in zip(params, saved):
            p.grad = g


def _retie(module: torch.nn.Module, tied: dict) -> None:
    for name, (_first, p) in tied.items():
        owner, _, leaf = name.rpartition(".")
        holder = module.get_submodule(owner) if owner else module
        holder._parameters[leaf] = p


def tied_gradients(grads: dict, tied: dict) -> dict:
    """Gradients by parameter name, with the names that share a tensor carrying the sum of their gradients."""
    if not tied:
        return grads
    total: dict = {}
    for name, g in grads.items():
        first = tied.get(name, name)
        if g is not None:
            total[first] = g if total.get(first) is None else total[first] + g
        else:
            total.setdefault(first, None)
    out = {name: total.get(tied.get(name, name)) for name in grads}
    for first in set(tied.values()):                       # a first name that is only ever reached through the others
        if first not in out and first in total:
            out[first] = total[first]
    return out


def _export(module, args, kwargs, loss, strict, decompositions, inner_cuts) -> Exported:
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ep = torch.export.export(module, tuple(args), kwargs or {}, strict=strict)
        if decompositions is None and loss is None:
            # inference keeps attention as one operation (the placement has a rule for heads cut over processors and
            # the executor can hand it to a fused kernel); the joint forward+backward export needs it decomposed
            decompositions = _inference_table()
        if loss is not None:
            _views_may_copy(ep.graph_module)
        ep = ep.run_decompositions(decompositions if decompositions is not None else
                                   (_training_table() if loss is not None else _default_table()))
        if expand_loops(ep.graph_module) + merge_repeats(ep.graph_module) + \
                ((unflatten_products(ep.graph_module) + (unflatten_linears(ep.graph_module) if inner_cuts else 0))
                 if loss is None else 0):
            # results that were items of a loop operator, or repeats of another node, are other nodes now: the
            # signature names them
            out_node = next(n for n in ep.graph_module.graph.nodes if n.op == "output")
            for spec, node in zip(ep.graph_signature.output_specs, out_node.args[0]):
                if isinstance(node, torch.fx.Node) and hasattr(spec.arg, "name"):
                    spec.arg.name = node.name
        if loss is not None and inner_cuts:
            outermost_rows(ep.graph_module, int(inner_cuts) if not isinstance(inner_cuts, bool) else 1)
        if loss is not None:
            from torch.export.experimental import _export_forward_backward
            # ``loss`` counts the module's own outputs; new values of mutated buffers come before them in the graph
            users = [i for i, spec in enumerate(ep.graph_signature.output_specs) if spec.kind == OutputKind.USER_OUTPUT]
            _detach_mutations(ep, keep=users[loss])
            paths = [(n.target, n.meta.get("nn_module_stack")) for n in ep.graph_module.graph.nodes if n.op == "call_function"]
            ep = _export_forward_backward(ep, joint_loss_index=users[loss])
            restore_module_paths(ep, paths)
            merge_repeats(ep.graph_module)                    # the backward half repeats views and transposes of the forward
            unflatten_products(ep.graph_module)
    return read(ep, training=loss is not None)


def restore_module_paths(ep, forward: list, window: int = 16) -> int:
    """Give the nodes of a joint forward+backward graph the submodule paths (``nn_module_stack``) that the joint trace
    drops, so that placements and share solvers can go by model part in training graphs too (the reference's ``segment``,
    examples/parallel.py:92-95).  ``forward``: ``(target, stack)`` of the forward graph's operator nodes, in order.  The
    joint graph starts with the same operators in the same order (with a few inserted or dropped): they are matched
    in order within a small window.  A backward node gets the path of the latest forward value or parameter it reads
    (the activations and weights its layer saved), else that of the gradient it continues."""
    gm = ep.graph_module
    owners = {}
    for spec in ep.graph_signature.input_specs:
        target = getattr(spec, "target", None)
        if isinstance(target, str) and "." in target:
            parts = target.split(".")[:-1]
            owners[spec.arg.name] = {".".join(parts[: i + 1]): (".".join(parts[: i + 1]), "torch.nn.modules.module.Module") for i in range(len(parts))}
    nodes = [n for n in gm.graph.nodes if n.op == "call_function"]
    j, at, given = 0, {}, 0                                # at: node name -> position of its forward anchor
    for i, n in enumerate(nodes):
        if j >= len(forward):
            break
        hit = next((k for k in range(j, min(j + window, len(forward))) if forward[k][0] is n.target), None)
        if hit is None:
            continue
        if forward[hit][1]:
            n.meta["nn_module_stack"] = forward[hit][1]
            given += 1
        at[n.name] = i
        j = hit + 1
    matched = set(at)
    stack_at = {i: nodes[i].meta.get("nn_module_stack") for i in at.values()}
    for n in nodes:
        if n.name in matched:
            continue
        saved, grads, owner, kept = -1, [], None, []
        for a in n.all_input_nodes:
            if a.name in owners:
                owner = owners[a.name]                       # a parameter: its layer, whatever the order
            elif a.name in matched:
                kept.append(a)                               # an activation the forward pass saved
            elif a.name in at:
                grads.append(at[a.name])                     # a gradient on its way back
        limit = min(grads) if grads else len(nodes)
        for a in kept:
            # the operator being differentiated read this activation (or made it): of the forward readers that come no
            # later than the gradient's own anchor, the latest - an activation saved as a layer's input was made by
            # the layer before, and the node belongs to the layer that read it
            readers = [at[u.name] for u in a.users if u.name in matched and at[u.name] <= limit]
            saved = max(saved, max(readers) if readers else at[a.name])
        if saved >= 0:
            here = saved
        elif grads:
            here = min(grads)                                # gradients flow towards earlier layers
        else:
            here = None
        stack = owner or (stack_at.get(here) if here is not None else None)
        if here is not None:
            at[n.name] = here
        elif owner is not None and grads == []:
            pass
        if stack:
            n.meta["nn_module_stack"] = stack
            stack_at.setdefault(here, stack) if here is not None else None
            given += 1
    return given


def _detach_mutations(ep, keep: int | None = None) -> int:
    """New values of mutated buffers and inputs (running statistics of a batch norm, step counters) and outputs other
    than the loss (output ``keep``) are results of the forward pass that nothing differentiates: cut them off the
    autograd graph, as eager mode does when it updates buffers under ``no_grad``.  Without this the joint export
    refuses any forward output that requires a gradient."""
    gm = ep.graph_module
    out_node = next(n for n in gm.graph.nodes if n.op == "output")
    outs = list(out_node.args[0])
    changed = 0
    for i, spec in enumerate(ep.graph_signature.output_specs):
        if i == keep or spec.kind not in (OutputKind.BUFFER_MUTATION, OutputKind.USER_INPUT_MUTATION, OutputKind.USER_OUTPUT):
            continue
        node = outs[i]
        val = node.meta.get("val") if isinstance(node, torch.fx.Node) else None
        if not isinstance(val, torch.Tensor) or not val.dtype.is_floating_point:
            continue
        with gm.graph.inserting_before(out_node):
            cut = gm.graph.call_function(torch.ops.aten.detach.default, (node,))
        cut.meta["val"] = val.detach()
        outs[i] = cut
        if hasattr(spec.arg, "name"):
            spec.arg.name = cut.name
        changed += 1
    if changed:
        out_node.args = (tuple(outs),)
        gm.recompile()
    return changed


def _inline(graph, body: torch.fx.GraphModule, operands: list, before: torch.fx.Node) -> list:
    """Copy ``body``'s nodes in front of ``before`` with its placeholders bound to ``operands``; returns its outputs."""
    holders = [n for n in body.graph.nodes if n.op == "placeholder"]
    if len(holders) != len(operands):
        raise ValueError(f"loop body takes {len(holders)} values, {len(operands)} given")
    env = dict(zip(holders, operands))
    with graph.inserting_before(before):
        out = graph.graph_copy(body.graph, env)
    return list(out) if isinstance(out, (tuple, list)) else [out]


def _made(graph, before, target, args, val):
    with graph.inserting_before(before):
        node = graph.call_function(target, args)
    node.meta["val"] = val
    return node


def unflatten_products(gm: torch.fx.GraphModule) -> int:
    """``view([B, H, m, k] -> [B*H, m, k])``, the same for the other operand, ``bmm``, ``view`` back to ``[B, H, m, n]``
    is how attention's two products reach the graph.  Merging batch and heads hides the heads from the placement (a cut
    along an inner merged dimension has no description), so the values would be gathered; the pattern is rewritten to
    one product over the four-dimensional operands, whose leading dimensions are both batch dimensions to the rules."""
    aten = torch.ops.aten
    views = (aten.view.default, aten._unsafe_view.default, aten.reshape.default)

    def opened(node):
        """``(the 4-D value a flattened operand came from, whether its last two dimensions are swapped)`` or None."""
        if not (isinstance(node, torch.fx.Node) and node.op == "call_function"):
            return None
        if node.target is aten.permute.default and list(node.args[1]) == [0, 2, 1]:      # the backward's transposed operands
            inner = opened(node.args[0])
            return None if inner is None else (inner[0], not inner[1])
        if node.target not in views:
            return None
        src = node.args[0]
        a, v = src.meta.get("val"), node.meta.get("val")
        if not (isinstance(a, torch.Tensor) and isinstance(v, torch.Tensor)) or a.ndim != 4 or v.ndim != 3:
            return None
        return (src, False) if (a.shape[0] * a.shape[1] == v.shape[0] and tuple(a.shape[2:]) == tuple(v.shape[1:])) else None

    def four(found, before):
        src, swapped = found
        if not swapped:
            return src
        with gm.graph.inserting_before(before):
            t = gm.graph.call_function(aten.permute.default, (src, [0, 1, 3, 2]))
        t.meta["val"] = src.meta["val"].permute(0, 1, 3, 2)
        return t

    done = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target is not aten.bmm.default:
            continue
        fa, fb = opened(node.args[0]), opened(node.args[1])
        if fa is None or fb is None or tuple(fa[0].meta["val"].shape[:2]) != tuple(fb[0].meta["val"].shape[:2]):
            continue
        lead = tuple(fa[0].meta["val"].shape[:2])
        out = node.meta["val"]
        want = lead + tuple(out.shape[1:])
        users = list(node.users)
        if not users or not all(u.op == "call_function" and u.target in views and tuple(u.meta["val"].shape) == want for u in users):
            continue
        a4, b4 = four(fa, node), four(fb, node)
        with gm.graph.inserting_before(node):
            prod = gm.graph.call_function(aten.matmul.default, (a4, b4))
        prod.meta.update({k: v for k, v in node.meta.items() if k != "val"})
        prod.meta["val"] = users[0].meta["val"]
        for u in users:
            u.replace_all_uses_with(prod)
            gm.graph.erase_node(u)
        gm.graph.erase_node(node)
        done += 1
    if done:
        gm.graph.eliminate_dead_code()                        # the flattened views and their transposes
        gm.graph.lint()
        gm.recompile()
    return done


def unflatten_linears(gm: torch.fx.GraphModule) -> int:
    """A linear layer on an input with several leading dimensions reaches the graph as ``view([..., K] -> [M, K])``,
    ``mm`` / ``addmm`` with the weight, ``view`` back to ``[..., N]``.  Merging the leading dimensions hides all but the
    outermost of them from the placement: a cut along an inner one (the batch of a sequence-first ``[T, B, E]`` layout,
    as inside ``nn.MultiheadAttention``) has no description on the merged dimension, so the value would be gathered.
    The pattern is rewritten to one product of the un-merged operand with the weight (``matmul`` of ``[..., K]`` and
    ``[K, N]``, plus the bias), whose leading dimensions are all row dimensions to the rules.  When the flattened view
    also merges trailing dimensions into ``K`` (``[T, B, H, hd] -> [T*B, H*hd]``), a view that merges only those is
    put in front."""
    aten = torch.ops.aten
    views = (aten.view.default, aten._unsafe_view.default, aten.reshape.default)

    def leading(shape, K):
        """Leading dimensions of ``shape`` once its trailing dimensions are merged to ``K`` (or None)."""
        acc, i = 1, len(shape)
        while i > 0 and acc < K:
            i -= 1
            acc *= shape[i]
        if acc != K or i < 2:                               # nothing to keep apart unless two leading dimensions remain
            return None
        return tuple(shape[:i])

    done = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target not in (aten.mm.default, aten.addmm.default):
            continue
        off = 1 if node.target is aten.addmm.default else 0
        if len(node.kwargs) or len(node.args) != 2 + off:
            continue
        flat, w = node.args[off], node.args[off + 1]
        if not (isinstance(flat, torch.fx.Node) and flat.op == "call_function" and flat.target in views and isinstance(w, torch.fx.Node)):
            continue
        src = flat.args[0]
        a, f, wv, out = (n.meta.get("val") for n in (src, flat, w, node))
        if not all(isinstance(t, torch.Tensor) for t in (a, f, wv, out)) or f.ndim != 2 or wv.ndim != 2 or a.ndim < 3:
            continue
        M, K = f.shape
        lead = leading(tuple(a.shape), K)
        if lead is None or math.prod(lead) != M:
            continue
        want = lead + (out.shape[1],)
        users = list(node.users)
        if not users or not all(u.op == "call_function" and u.target in views and tuple(u.meta["val"].shape) == want for u in users):
            continue
        with gm.graph.inserting_before(node):
            x = src
            if tuple(a.shape) != lead + (K,):
                x = gm.graph.call_function(aten.view.default, (src, list(lead + (K,))))
                x.meta["val"] = a.reshape(lead + (K,))
            prod = gm.graph.call_function(aten.matmul.default, (x, w))
            prod.meta.update({k: v for k, v in node.meta.items() if k != "val"})
            prod.meta["val"] = users[0].meta["val"]
            res = prod
            if off:
                res = gm.graph.call_function(aten.add.Tensor, (prod, node.args[0]))
                res.meta.update({k: v for k, v in node.meta.items() if k != "val"})
                res.meta["val"] = users[0].meta["val"]
        for u in users:
            u.replace_all_uses_with(res)
            gm.graph.erase_node(u)
        gm.graph.erase_node(node)
        done += 1
    if done:
        gm.graph.eliminate_dead_code()
        gm.graph.lint()
        gm.recompile()
    return done


def outermost_rows(gm: torch.fx.GraphModule, dim: int) -> int:
    """The training-graph counterpart of :func:`unflatten_linears`.  There the weight gradient contracts over the merged
    rows, so the rows have to stay merged; instead the merge is made in another order: the leading dimension ``dim``
    (the one that is cut: the tokens of a ``[B, T, E]`` layout) is moved to the front first,

        view([B, T, K] -> [B*T, K]); mm; view([B*T, N] -> [B, T, N])
            ->  permute -> [T, B, K]; clone; view([T*B, K]); mm; view([T, B, N]); permute -> [B, T, N]

    which makes the cut the outermost factor of the rows - something the view rule describes - in the forward product
    and, through differentiation of the rewritten graph, in both backward products: activations cut along the tokens
    stay cut through the linear layers of a training step with several samples (the price is the transposing copy)."""
    aten = torch.ops.aten
    views = (aten.view.default, aten._unsafe_view.default, aten.reshape.default)
    done = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target not in (aten.mm.default, aten.addmm.default):
            continue
        off = 1 if node.target is aten.addmm.default else 0
        if len(node.kwargs) or len(node.args) != 2 + off:
            continue
        flat, w = node.args[off], node.args[off + 1]
        if not (isinstance(flat, torch.fx.Node) and flat.op == "call_function" and flat.target in views and isinstance(w, torch.fx.Node)):
            continue
        src = flat.args[0]
        a, f, out = (n.meta.get("val") for n in (src, flat, node))
        if not all(isinstance(t, torch.Tensor) for t in (a, f, out)) or f.ndim != 2 or a.ndim < 3 or not 0 < dim < a.ndim - 1:
            continue
        lead = tuple(a.shape[:-1])
        if math.prod(lead) != f.shape[0] or a.shape[-1] != f.shape[1] or math.prod(lead[:dim]) == 1:
            continue
        want = lead + (out.shape[1],)
        users = list(node.users)
        if not users or not all(u.op == "call_function" and u.target in views and tuple(u.meta["val"].shape) == want for u in users):
            continue
        nd = a.ndim
        perm = [dim] + [d for d in range(nd - 1) if d != dim] + [nd - 1]
        back = [perm.index(d) for d in range(nd)]
        with gm.graph.inserting_before(node):
            moved = gm.graph.call_function(aten.permute.default, (src, perm))
            moved.meta["val"] = a.permute(perm)
            dense = gm.graph.call_function(aten.clone.default, (moved,), {"memory_format": torch.contiguous_format})
            dense.meta["val"] = a.permute(perm).contiguous()
            rows = gm.graph.call_function(aten.view.default, (dense, [f.shape[0], f.shape[1]]))
            rows.meta["val"] = dense.meta["val"].reshape(f.shape[0], f.shape[1])
            for n in (moved, dense, rows):
                n.meta.update({k: v for k, v in flat.meta.items() if k != "val"})
        node.replace_input_with(flat, rows)
        with gm.graph.inserting_after(node):
            shaped = gm.graph.call_function(aten.view.default, (node, [a.shape[d] for d in perm[:-1]] + [out.shape[1]]))
        with gm.graph.inserting_after(shaped):
            restored = gm.graph.call_function(aten.permute.default, (shaped, back))
        shaped.meta.update({k: v for k, v in users[0].meta.items() if k != "val"})
        restored.meta.update({k: v for k, v in users[0].meta.items() if k != "val"})
        shaped.meta["val"] = out.reshape([a.shape[d] for d in perm[:-1]] + [out.shape[1]])
        restored.meta["val"] = shaped.meta["val"].permute(back)
        for u in users:
            u.replace_all_uses_with(restored)
            gm.graph.erase_node(u)
        done += 1
    if done:
        gm.graph.eliminate_dead_code()
        gm.graph.lint()
        gm.recompile()
        _views_may_copy(gm)        # what comes back from a product is a permuted value now: later views of it may have to copy
    return done


def merge_repeats(gm: torch.fx.GraphModule) -> int:
    """Nodes that apply the same operator to the same operands are one node (the three views of one normalised
    activation that feed the query, key and value projections, for instance): what is cut, gathered or reduced once for
    one of them then serves all.  The captured graph is functional, so equal operator and operands mean equal values;
    random draws are left alone.  Returns how many nodes were merged."""
    import operator

    def key_of(a):
        if isinstance(a, torch.fx.Node):
            return ("node", a.name)
        if isinstance(a, (list, tuple)):
            return (type(a).__name__, tuple(key_of(x) for x in a))
        if isinstance(a, dict):
            return ("dict", tuple(sorted((k, key_of(v)) for k, v in a.items())))
        if isinstance(a, (torch.dtype, torch.device, torch.layout, torch.memory_format)):
            return ("torch", str(a))
        return (type(a).__name__, a)
    seen: dict = {}
    outputs = {a for n in gm.graph.nodes if n.op == "output" for a in n.all_input_nodes}
    merged = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function":
            continue
        name = str(node.target)
        if any(w in name for w in ("rand", "dropout", "bernoulli", "normal", "multinomial", "higher_order")):
            continue                                          # two draws are two values
        if node.target is not operator.getitem and not isinstance(node.meta.get("val"), torch.Tensor):
            continue                                          # operators with several results keep their own node
        try:
            key = (name, key_of(node.args), key_of(node.kwargs))
            hash(key)
        except TypeError:
            continue
        first = seen.get(key)
        if first is None:
            seen[key] = node
        elif node not in outputs:                            # a result the caller reads keeps its node
            node.replace_all_uses_with(first)
            gm.graph.erase_node(node)
            merged += 1
    if merged:
        gm.graph.lint()
        gm.recompile()
    return merged


def expand_loops(gm: torch.fx.GraphModule) -> int:
    """Unroll the ``map`` and ``scan`` higher-order operators of a captured graph (the reference expands them the same
    way at capture, compiler/mesh_compiler/export.py:112-130): iteration ``i`` of the body is copied into the graph
    with ``x[i]`` as its element, the per-iteration results are stacked, and a scan's carry flows from copy to copy.
    After this every node is a plain operator, which is what the placement stage has rules for.  Returns how many
    operators were expanded (nested ones count)."""
    import operator
    hop = torch.ops.higher_order
    done = 0
    while True:
        node = next((n for n in gm.graph.nodes if n.op == "call_function" and n.target in (hop.map_impl, hop.scan)), None)
        if node is None:
            break
        graph = gm.graph
        body = getattr(gm, node.args[0].target)
        if node.target is hop.map_impl:
            carried, xs, extra = [], list(node.args[1]), list(node.args[2])
        else:
            carried, xs, extra = list(node.args[1]), list(node.args[2]), list(node.args[3]) if len(node.args) > 3 else []
        steps = xs[0].meta["val"].shape[0]
        order = range(steps - 1, -1, -1) if node.kwargs.get("reverse", False) else range(steps)
        rows: list[list] = []
        for i in order:
            elems = [_made(graph, node, torch.ops.aten.select.int, (x, 0, i), torch.ops.aten.select.int(x.meta["val"], 0, i)) for x in xs]
            out = _inline(graph, body, carried + elems + extra, node)
            carried, ys = out[: len(carried)], out[len(carried):]
            rows.append(ys)
        if node.kwargs.get("reverse", False):
            rows.reverse()
        stacked = []
        for j in range(len(rows[0]) if rows else 0):
            parts = [r[j] for r in rows]
            stacked.append(_made(graph, node, torch.ops.aten.stack.default, (parts, 0),
                                 torch.ops.aten.stack.default([p.meta["val"] for p in parts], 0)))
        results = carried + stacked
        for user in list(node.users):
            if user.op == "call_function" and user.target is operator.getitem:
                user.replace_all_uses_with(results[user.args[1]])
                graph.erase_node(user)
            else:
                raise NotImplementedError(f"{node.name} is used whole by {user.name}")
        holder = node.args[0]
        graph.erase_node(node)
        if not holder.users:
            graph.erase_node(holder)
        done += 1
    if done:
        gm.graph.lint()
        gm.recompile()
    return done


def read(ep, training: bool = False) -> Exported:
    gm = ep.graph_module
    sig = ep.graph_signature
    state, kinds, users = {}, {}, []
    for spec in sig.input_specs:
        name = spec.arg.name
        if spec.kind in _IN_KINDS:
            if spec.kind == InputKind.CONSTANT_TENSOR:
                tensor = ep.constants[spec.target]
            else:
                tensor = ep.state_dict.get(spec.target)
                if tensor is None:
                    tensor = ep.constants[spec.target]
            state[name] = (spec.target, tensor)
            kinds[name] = _IN_KINDS[spec.kind]
        elif spec.kind == InputKind.USER_INPUT:
            users.append(name)
        elif spec.kind == InputKind.TOKEN:
            state[name] = (name, torch.empty(0))
            kinds[name] = "token"
        else:
            raise NotImplementedError(f"input kind {spec.kind} of {name}")
    outputs, mutations = [], {}
    for i, spec in enumerate(sig.output_specs):
        kind = _OUT_KINDS.get(spec.kind)
        if kind is None:
            raise NotImplementedError(f"output kind {spec.kind}")
        outputs.append((kind, spec.target))
        if kind == "mutation":
            # the placeholder that holds the mutated buffer / input
            for s in sig.input_specs:
                if s.target == spec.target or s.arg.name == spec.target:
                    mutations[i] = s.arg.name
    for node in gm.graph.nodes:
        val = node.meta.get("val")
        for v in (val if isinstance(val, (tuple, list)) else [val]):
            if isinstance(v, torch.Tensor) and any(not isinstance(s, int) for s in v.shape):
                raise ValueError(f"symbolic dimension in {node.name}: shapes must be static")
    return Exported(gm, state, kinds, users, outputs, ep.call_spec.in_spec, ep.call_spec.out_spec, mutations, training, ep)


def calls(program: torch.nn.Module, args: tuple, functions, **options) -> tuple[Exported, dict]:
    """Whole-program capture for ``compile_program``: the outer ``forward`` may only call the named
    functions (submodule qualified names); the calls are inlined in one graph and each node keeps the
    submodule it came from, from which the per-function call counts are read
    (compiler/mesh_compiler/export.py:237-256, :342-349)."""
    exp = export(program, args, **options)
    names = {f if isinstance(f, str) else getattr(f, "__name__", str(f)) for f in functions}
    counts: dict[str, set] = {n: set() for n in names}
    for node in exp.graph_module.graph.nodes:
        stack = node.meta.get("nn_module_stack") or {}
        for key, (qual, _cls) in stack.items():
            if qual in counts:
                counts[qual].add(key)
    return exp, {k: max(1, len(v)) for k, v in counts.items()}


# ----------------------------------------------------------------------------- substitution of a function by parts
class Parts(torch.nn.Module):
    """What a substituted function becomes: its parts called in order.  ``wiring[p]`` lists where part ``p`` takes each
    input from - ``("call", i)``: input ``i`` of the original call; ``("part", q, o)``: output ``o`` of the earlier part
    ``q`` - and ``results[k] = (p, o)`` names the part output that is output ``k`` of the original call."""

    def __init__(self, parts, wiring, results):
        super().__init__()
        self.names = [name for name, _ in parts]
        for name, m in parts:
            self.add_module(name, m)
        self.wiring = [list(w) for w in wiring]
        self.results = list(results)

    def forward(self, *args):
        made: list[tuple] = []
        for name, inputs in zip(self.names, self.wiring):
            argv = [args[s[1]] if s[0] == "call" else made[s[1]][s[2]] for s in inputs]
            out = getattr(self, name)(*argv)
            made.append(tuple(out) if isinstance(out, (tuple, list)) else (out,))
        outs = tuple(made[p][o] for p, o in self.results)
        return outs[0] if len(outs) == 1 else outs


def substitute(program: torch.nn.Module, key, parts, results=None) -> int:
    """Replace every call of the function ``key`` in ``program`` by calls of ``parts``, in order, and return how many
    were replaced.  ``key``: a submodule's qualified name, a module class, or a predicate over ``(name, module)``.
    ``parts``: ``[(name, module, inputs)]`` with ``inputs`` as in :class:`Parts`; a module given as a callable
    ``make(original)`` is built per replaced call (so that parts can take over the original's parameters).
    ``results``: which part outputs are the original call's outputs (default: all outputs of the last part).

    The reference rewrites its call graph in place (compiler/mesh_compiler/export.py:525-640: every call of ``key``
    becomes the calls of ``parts``, an input a call input or an earlier part's output, ``results`` mapping part outputs
    to the call's outputs) and uses it to outline iterative linear algebra into repeated calls of one step
    (compiler/mesh_compiler/decompose.py).  Here calls are inlined at capture and every node remembers the submodule it
    came from, so the rewrite happens one level up, on the module tree, before the capture: the captured graph then
    carries the parts as call instances of their own (``calls.analyse`` sees them, placements can name them)."""
    def matches(name, m):
        if isinstance(key, str):
            return name == key
        if isinstance(key, type):
            return isinstance(m, key)
        return bool(key(name, m))

    found = [(name, m) for name, m in program.named_modules() if name and matches(name, m)]
    # a match inside another match would be replaced with its parent: keep outermost ones only
    found = [(n, m) for n, m in found if not any(n.startswith(o + ".") for o, _ in found)]
    for name, original in found:
        built = [(pname, (make(original) if not isinstance(make, torch.nn.Module) else make)) for pname, make, _ in parts]
        wiring = [inputs for _, _, inputs in parts]
        res = results
        if res is None:
            res = [(len(parts) - 1, 0)]
        parent_name, _, leaf = name.rpartition(".")
        parent = program.get_submodule(parent_name) if parent_name else program
        setattr(parent, leaf, Parts(built, wiring, res))
    return len(found)
