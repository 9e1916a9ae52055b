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

import warnings

import torch
from torch.export.graph_signature import InputKind, OutputKind

from .ir import Exported

_IN_KINDS = {InputKind.PARAMETER: "parameter", InputKind.BUFFER: "buffer", InputKind.CONSTANT_TENSOR: "constant"}
_OUT_KINDS = {OutputKind.USER_OUTPUT: "user", OutputKind.LOSS_OUTPUT: "loss",
              OutputKind.GRADIENT_TO_PARAMETER: "grad_param", OutputKind.GRADIENT_TO_USER_INPUT: "grad_input",
              OutputKind.BUFFER_MUTATION: "mutation", OutputKind.USER_INPUT_MUTATION: "mutation"}


def export(module: torch.nn.Module, args: tuple, kwargs: dict | None = None, *, loss: int | None = None,
           strict: bool = True, decompositions=None) -> Exported:
    """Export ``module(*args, **kwargs)``; with ``loss`` (index of the loss among flat outputs) the joint graph."""
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ep = torch.export.export(module, tuple(args), kwargs or {}, strict=strict)
        if decompositions is None and loss is None:
            # inference keeps attention as one operation (the placement has a rule for heads cut over processors and
            # the executor can hand it to a fused kernel); the joint forward+backward export needs it decomposed
            decompositions = torch.export.default_decompositions()
            for op in (torch.ops.aten.scaled_dot_product_attention.default,):
                decompositions.pop(op, None)
        ep = ep.run_decompositions(decompositions) if decompositions is not None else ep.run_decompositions()
        if loss is not None:
            from torch.export.experimental import _export_forward_backward
            ep = _export_forward_backward(ep, joint_loss_index=loss)
    return read(ep, training=loss is not None)


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
