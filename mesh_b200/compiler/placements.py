"""A library of placement callables for models whose source the user does not want to touch.

A placement is any callable ``node -> None | processor | (dimension, processors, units)`` (see
:mod:`mesh_b200.compiler.placement`); the reference's examples each write their own from the parameter names of the
model at hand (examples/parallel.py:77-95: Megatron by ``wq/wk/wv/w1/w3`` and ``wo/w2``; examples/pl.py: layers by
their ``nn_module_stack`` path).  These builders state the same things by name patterns, so that a model from another
library is placed without editing it:

* :func:`tensor_parallel`: column-parallel and row-parallel linear layers (and convolutions) by parameter name,
  vocabulary-parallel embeddings;
* :func:`data_parallel`, :func:`sequence_parallel`: cut the user inputs;
* :func:`pipeline`: whole submodules on one processor each;
* :func:`grid`: pipeline stages, tensor-parallel layers and cut inputs on a grid of processors whose axes have roles;
* :func:`combine`: the first builder that states something for a node wins.

Placeholder names are the qualified parameter names with dots replaced by underscores and a ``p_`` (parameter),
``b_`` (buffer) or ``c_`` (constant) prefix; user inputs keep the names of ``forward``'s arguments.
"""
from __future__ import annotations

import re
from typing import Callable, Iterable, Sequence


def _matcher(patterns: Iterable[str]) -> Callable[[str], bool]:
    """Does a placeholder name contain one of ``patterns`` as a whole path component (``q_proj`` matches
    ``p_model_layers_0_self_attn_q_proj_weight``, not ``..._xq_proj_weight``)?  A pattern may be a regular expression."""
    compiled = [re.compile(rf"(?:^|_)(?:{p})(?:_|$)") for p in patterns]
    return lambda name: any(c.search(name) for c in compiled)


def _is_state(node) -> bool:
    return node.op == "placeholder" and node.name.startswith(("p_", "b_", "c_"))


def tensor_parallel(processors: Sequence[str], column: Iterable[str] = (), row: Iterable[str] = (),
                    vocabulary: Iterable[str] = (), units=None, transposed: Iterable[str] = ()) -> Callable:
    """Megatron-style placement by parameter name.

    ``column``: layers whose weight is cut along its output features (dimension 0 of a linear or convolution weight),
    with their bias; ``row``: layers whose weight is cut along its input features (dimension 1), bias whole (it is added
    after the sum); ``vocabulary``: embeddings cut along the vocabulary (dimension 0: a masked lookup and one
    all-reduce).  ``transposed`` names layers whose weight is stored ``[in, out]`` (transposed convolutions, GPT-2's
    ``Conv1D``): their column / row dimensions swap.  ``units``: optional share ratios or ``"striped"``."""
    names = tuple(processors)
    is_col, is_row, is_vocab, is_t = _matcher(column), _matcher(row), _matcher(vocabulary), _matcher(transposed)

    def placement(node):
        if not _is_state(node):
            return None
        n = node.name
        val = node.meta.get("val")
        nd = getattr(val, "ndim", 0)
        flip = bool(list(transposed)) and is_t(n)
        if n.endswith("_weight") and nd >= 2:
            if is_col(n):
                return (1 if flip else 0, names, units)
            if is_row(n):
                return (0 if flip else 1, names, units)
            if is_vocab(n):
                return (0, names, units)
        if n.endswith("_bias") and nd == 1 and is_col(n):
            return (0, names, units)
        return None
    return placement


def data_parallel(processors: Sequence[str], inputs: Iterable[str] | None = None, dim: int = 0, units=None) -> Callable:
    """Cut the named user inputs (default: every tensor input) along ``dim``: parameters stay whole everywhere and
    their gradients are all-reduced."""
    names = tuple(processors)
    wanted = None if inputs is None else set(inputs)

    def placement(node):
        if node.op != "placeholder" or _is_state(node):
            return None
        val = node.meta.get("val")
        if getattr(val, "ndim", 0) <= dim:
            return None
        if wanted is not None and node.name not in wanted:
            return None
        return (dim, names, units)
    return placement


def sequence_parallel(processors: Sequence[str], inputs: Iterable[str] | None = None, dim: int = 1, units=None) -> Callable:
    """Cut the user inputs along the sequence dimension (``units="striped"`` balances causal attention)."""
    return data_parallel(processors, inputs, dim, units)


def pipeline(stages: dict) -> Callable:
    """``{module path pattern: processor}``: every operator traced from a submodule whose qualified path matches a
    pattern (a regular expression, matched at the start: ``"model.layers.[0-3]\\."``) runs on that processor, with
    its parameters; the compiler inserts the sends and receives between stages."""
    compiled = [(re.compile(p), proc) for p, proc in stages.items()]

    def of_path(path: str):
        for pat, proc in compiled:
            if pat.match(path):
                return proc
        return None

    def placement(node):
        if _is_state(node):
            path = node.name.split("_", 1)[1]
            for pat, proc in compiled:                     # parameter names carry underscores where the path has dots
                if re.match(pat.pattern.replace(r"\.", "_").replace(".", "_"), path):
                    return proc
            return None
        stack = node.meta.get("nn_module_stack")
        if not stack:
            return None
        for _key, (qual, _cls) in reversed(list(stack.items())):
            proc = of_path(qual + ".")
            if proc is not None:
                return proc
        return None
    return placement


def grid(axes: Sequence[str], *, stages: dict | None = None, stage_axis: str | None = None, column: Iterable[str] = (),
         row: Iterable[str] = (), vocabulary: Iterable[str] = (), tensor_axis: str | None = None,
         inputs: dict | None = None) -> Callable:
    """One placement for a grid of processors whose axes have roles - the compiled form of a hybrid job such as
    ``("pp", "cp", "tp")`` with ``compile_module(..., mesh=(2, 2, 2))``.

    * ``stages`` / ``stage_axis``: ``{module path pattern: coordinate}`` - the submodules that run on each coordinate of
      the pipeline axis.  Their parameters live there (``"@k"`` along that axis) and their operators run there, forward
      and backward; the other axes of an operator are left to propagation (``...``).
    * ``column`` / ``row`` / ``vocabulary`` / ``tensor_axis``: Megatron cuts of the named layers along the tensor axis.
    * ``inputs``: ``{input name: {axis name: dimension}}`` - cuts of the user inputs (tokens over a context axis, samples
      over a data axis); inputs enter at coordinate 0 of the pipeline axis.
    """
    axes = tuple(axes)
    na = len(axes)
    s_ax = axes.index(stage_axis) if stage_axis is not None else None
    t_ax = axes.index(tensor_axis) if tensor_axis is not None else None
    compiled = [(re.compile(p), k) for p, k in (stages or {}).items()]
    is_col, is_row, is_vocab = _matcher(column), _matcher(row), _matcher(vocabulary)
    inputs = inputs or {}

    def stage_of_path(path: str):
        for pat, k in compiled:
            if pat.match(path):
                return k
        return None

    def stage_of_parameter(name: str):
        path = name.split("_", 1)[1]
        for pat, k in compiled:
            if re.match(pat.pattern.replace(r"\.", "_").replace(".", "_"), path):
                return k
        return None

    def placement(node):
        if _is_state(node):
            dims = [None] * na
            k = stage_of_parameter(node.name) if s_ax is not None else None
            if k is not None:
                dims[s_ax] = f"@{k}"
            nd = getattr(node.meta.get("val"), "ndim", 0)
            if t_ax is not None:
                if node.name.endswith("_weight") and nd >= 2:
                    dims[t_ax] = 0 if (is_col(node.name) or is_vocab(node.name)) else 1 if is_row(node.name) else None
                elif node.name.endswith("_bias") and nd == 1 and is_col(node.name):
                    dims[t_ax] = 0
            return (tuple(dims), None, None) if any(d is not None for d in dims) else None
        if node.op == "placeholder":
            dims = [None] * na
            for axis, dim in inputs.get(node.name, {}).items():
                dims[axes.index(axis)] = dim
            if s_ax is not None:
                dims[s_ax] = "@0"
            return (tuple(dims), None, None) if any(d is not None for d in dims) else None
        if s_ax is None:
            return None
        stack = node.meta.get("nn_module_stack")
        if not stack:
            return None
        for _key, (qual, _cls) in reversed(list(stack.items())):
            k = stage_of_path(qual + ".")
            if k is not None:
                dims = [...] * na
                dims[s_ax] = f"@{k}"
                return (tuple(dims), None, None)
        return None
    return placement


def combine(*placements: Callable) -> Callable:
    """One placement from several: the first that states something for a node wins."""
    def placement(node):
        for p in placements:
            stated = p(node)
            if stated is not None:
                return stated
        return None
    return placement


# name patterns of a common family of decoder models (Llama, Mistral, Qwen2, Gemma: the same parameter names)
LLAMA = {"column": ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"), "row": ("o_proj", "down_proj")}
