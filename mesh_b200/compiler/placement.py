"""GSPMD-style sharding propagation and collective insertion.

The caller states placements with a callable ``placement(node) -> None | str | (dimension, processors, units)``
called for every node (compiler/mesh_compiler/placement.py:837-864):

* ``str``: the value lives whole on that processor;
* ``(dimension, processors, units)``: sharded along ``dimension`` over ``processors``; ``units`` is ``None``
  (``torch.chunk`` sizes), a tuple of ratios (unequal shards, nearest integers with least-error +-1 repair and
  optional bounds), a tuple of P+1 edges, or ``"striped"`` (processor j holds elements j, j+P, ...);
* tuples for ``dimension`` / nested tuples for ``processors``: one entry per axis of an N-D mesh.

Unstated nodes inherit through per-op rules; a contraction over a sharded dimension leaves a *partial*
value that is reduced where a replicated or sharded value is needed (all-reduce / reduce-scatter);
mismatches are resharded: sharded->replicated = all-gather (kind ``broadcast``), dim a -> dim b =
all-to-all (``alltoall``), partial -> * = ``reduce``, owner -> owner = ``permute``
(placement.py:250-340, :812-834).  A rule miss is never an error: the inputs are gathered and the op
runs replicated (placement.py:656-657).  Replicated constants (masks, aranges) are *sliced locally*
when they meet a sharded value, so a causal mask follows a striped or unequal sequence split with no
special case.
"""
from __future__ import annotations

import math
import operator
from typing import Any, Callable

import torch

from .ir import JOIN, PAGES, Mesh, O, P, Plan, R, Ref, S, Spec, Step, Transfer, pack

aten = torch.ops.aten


# ----------------------------------------------------------------------------- shard sizes
def counts(n: int, units=None, parts: int = 1, lower=None, upper=None) -> list[int]:
    """Sizes of ``parts`` shards of ``n`` elements (reference: placement.py:65-87).

    ``units is None``: ``torch.chunk`` sizes (``ceil(n / parts)``, trailing shards may be empty);
    ``"striped"``: shard j gets ``ceil((n - j) / parts)``; ``parts`` ratios: nearest integers, then +-1 on the
    shard whose size moves closest to its exact share until the sizes sum to ``n`` (within bounds);
    ``parts + 1`` values: explicit edges.
    """
    if units is None:
        step = -(-n // parts)
        return [max(0, min(step, n - j * step)) for j in range(parts)]
    if isinstance(units, str):
        if units != "striped":
            raise ValueError(f"unknown units {units!r}")
        return [max(0, -(-(n - j) // parts)) for j in range(parts)]
    units = list(units)
    if len(units) == parts + 1:
        return [int(units[j + 1] - units[j]) for j in range(parts)]
    if len(units) != parts:
        raise ValueError(f"{len(units)} units for {parts} processors")
    total = float(sum(units))
    exact = [n * u / total for u in units]
    lo = [0] * parts if lower is None else list(lower)
    hi = [n] * parts if upper is None else list(upper)
    sizes = [int(min(max(round(e), l), h)) for e, l, h in zip(exact, lo, hi)]
    while sum(sizes) != n:
        step = 1 if sum(sizes) < n else -1
        best, best_err = None, None
        for j in range(parts):
            new = sizes[j] + step
            if new < lo[j] or new > hi[j]:
                continue
            err = abs(new - exact[j])
            if best is None or err < best_err:
                best, best_err = j, err
        if best is None:
            raise ValueError("bounds make the shard sizes infeasible")
        sizes[best] += step
    return sizes


def striped_place(j: int, r: int, c: list[int]) -> int:
    """Global index of the j-th element held by rank r under striping with per-rank counts ``c``
    (compiler/mesh_compiler/operations.py:59-62); equal counts reduce to ``P*j + r``."""
    cr = c[r]
    return j + sum(((2 * j + 1) * co + cr - (1 if o > r else 0)) // (2 * cr) for o, co in enumerate(c) if o != r)


def local_indices(spec: Spec, coord: int, n: int) -> slice | list[int]:
    """Which elements of a dimension of size ``n`` the processor at ``coord`` holds."""
    if spec.striped:
        if len(set(spec.counts)) == 1 or all(cnt in (spec.counts[0], spec.counts[0] - 1) for cnt in spec.counts):
            return slice(coord, n, len(spec.counts))
        return [striped_place(j, coord, list(spec.counts)) for j in range(spec.counts[coord])]
    start = sum(spec.counts[:coord])
    return slice(start, start + spec.counts[coord])


# ----------------------------------------------------------------------------- op classes
POINTWISE = {
    aten.add.Tensor, aten.sub.Tensor, aten.mul.Tensor, aten.div.Tensor, aten.pow.Tensor_Scalar, aten.pow.Tensor_Tensor,
    aten.rsqrt.default, aten.sqrt.default, aten.sigmoid.default, aten.silu.default, aten.gelu.default, aten.tanh.default,
    aten.exp.default, aten.log.default, aten.neg.default, aten.abs.default, aten.reciprocal.default, aten.relu.default,
    aten.where.self, aten.eq.Scalar, aten.eq.Tensor, aten.ne.Scalar, aten.le.Scalar, aten.lt.Scalar, aten.ge.Scalar,
    aten.gt.Scalar, aten.le.Tensor, aten.lt.Tensor, aten.ge.Tensor, aten.gt.Tensor, aten.logical_and.default,
    aten.logical_or.default, aten.logical_not.default, aten.maximum.default, aten.minimum.default, aten._to_copy.default,
    aten.clone.default, aten.alias.default, aten.mul.Scalar, aten.div.Scalar, aten.add.Scalar, aten.sub.Scalar,
    aten.erf.default, aten.masked_fill.Scalar, aten.masked_fill.Tensor, aten.sigmoid_backward.default,
    aten.tanh_backward.default, aten.silu_backward.default, aten.gelu_backward.default, aten.threshold_backward.default,
    aten.clamp.default, aten.clamp_min.default, aten.clamp_max.default, aten.rsub.Scalar, aten.cos.default,
    aten.sin.default, aten.bitwise_and.Tensor, aten.bitwise_or.Tensor, aten.bitwise_not.default, aten.fill.Scalar,
    aten.zeros_like.default, aten.ones_like.default, aten.full_like.default, aten.detach.default, aten.square.default,
    aten.exp2.default, aten.log2.default, aten.softplus.default, aten.hardtanh.default, aten.leaky_relu.default,
    aten.native_dropout_backward.default, aten.sign.default, aten.floor.default, aten.ceil.default, aten.round.default,
    aten.remainder.Scalar, aten.fmod.Scalar, aten.isnan.default, aten.isinf.default, aten.nan_to_num.default,
    aten.lift_fresh_copy.default, aten.contiguous.default if hasattr(aten, "contiguous") else aten.clone.default,
}


def _overloads(*names) -> set:
    """The operator overloads named ``packet.overload`` that this build of PyTorch has (older and newer builds differ in
    which activations are primitive and which are decomposed before the compiler sees them)."""
    found = set()
    for name in names:
        packet, _, overload = name.partition(".")
        op = getattr(getattr(aten, packet, None), overload or "default", None)
        if op is not None:
            found.add(op)
    return found


# the rest of the element-by-element family: activations and their derivatives, transcendental functions, comparisons,
# integer arithmetic, three-operand blends
POINTWISE |= _overloads(
    "elu", "elu_backward", "celu", "selu", "log1p", "expm1", "log10", "log_sigmoid_forward", "log_sigmoid_backward",
    "hardswish", "hardswish_backward", "hardsigmoid", "hardsigmoid_backward", "hardtanh_backward", "leaky_relu_backward",
    "softplus_backward", "mish", "mish_backward", "relu6", "threshold", "logit", "logit_backward", "tan", "atan", "asin",
    "acos", "sinh", "cosh", "asinh", "acosh", "atanh", "atan2", "trunc", "frac", "erfc", "erfinv", "lgamma", "digamma",
    "sgn", "signbit", "positive", "hypot", "copysign.Tensor", "copysign.Scalar", "xlogy.Tensor", "logaddexp", "logaddexp2",
    "logical_xor", "bitwise_xor.Tensor", "bitwise_and.Scalar", "bitwise_or.Scalar", "bitwise_xor.Scalar",
    "bitwise_left_shift.Tensor", "bitwise_right_shift.Tensor", "ne.Tensor", "fmod.Tensor", "remainder.Tensor",
    "floor_divide", "div.Tensor_mode", "div.Scalar_mode", "pow.Scalar", "lerp.Scalar", "lerp.Tensor", "addcmul", "addcdiv",
    "clamp.Tensor", "clamp_min.Tensor", "clamp_max.Tensor", "where.ScalarOther", "where.ScalarSelf", "heaviside",
    "isfinite", "isposinf", "isneginf", "rad2deg", "deg2rad", "sinc", "i0", "special_erfcx", "special_ndtri",
    "empty_like",
)
# ops that stay "partial" when exactly the listed argument positions are partial and the rest replicated/scalars
LINEAR_IN = {
    aten.add.Tensor: "all", aten.sub.Tensor: "all", aten.neg.default: "all", aten.clone.default: "all",
    aten.alias.default: "all", aten._to_copy.default: "all", aten.detach.default: "all",
    aten.mul.Tensor: "one", aten.div.Tensor: "first", aten.mul.Scalar: "all", aten.div.Scalar: "all",
}
CREATION = {aten.full.default, aten.zeros.default, aten.ones.default, aten.arange.start_step, aten.arange.default,
            aten.arange.start, aten.scalar_tensor.default, aten.empty.memory_format, aten.new_zeros.default,
            aten.new_ones.default, aten.new_full.default, aten.new_empty.default, aten.tril_indices.default,
            aten.eye.default, aten.linspace.default}
REDUCTIONS = {aten.sum.dim_IntList: "sum", aten.sum.default: "sum", aten.mean.dim: "mean", aten.mean.default: "mean",
              aten.amax.default: "max", aten.amin.default: "min", aten.any.dim: "max", aten.any.default: "max",
              aten.all.dim: "min", aten.all.default: "min", aten.max.default: "max", aten.min.default: "min"}
SOFTMAX_LIKE = {aten._softmax.default: 1, aten._log_softmax.default: 1, aten._softmax_backward_data.default: 2,
                aten._log_softmax_backward_data.default: 2, aten.cumsum.default: 1, aten.argmax.default: 1,
                aten.topk.default: 2, aten.sort.default: 1, aten.logsumexp.default: 1}


def _trailing(core: int, outs: int, operands=None):
    """Operators over the last ``core`` dimensions of every (listed) tensor operand; the leading ones are a batch."""
    def describe(node, shapes):
        nd = len(shapes[0])
        flags = [True] * len(shapes) if operands is None else [i in operands for i in range(len(shapes))]
        if any(f and len(sh) != nd for f, sh in zip(flags, shapes)):
            return None                                     # a broadcast batch or a vector right-hand side
        return {"batched": flags, "protect": set(range(nd - core, nd)), "outs": ["S"] * outs}
    return describe


def _along(position: int, outs: int, default=-1):
    """Operators that work along one dimension (argument ``position``) of their first operand."""
    def describe(node, shapes):
        nd = len(shapes[0])
        dim = node.args[position] if len(node.args) > position else node.kwargs.get("dim", default)
        if dim is None:
            return None                                     # the operator works on the flattened tensor
        return {"batched": [True] + [False] * (len(shapes) - 1), "protect": {dim % max(nd, 1)}, "outs": ["S"] * outs}
    return describe


def _split(position: int, removes: bool = False):
    """Operators that cut their operand into a list of pieces along one dimension (``removes``: and drop it)."""
    def describe(node, shapes):
        nd = len(shapes[0])
        dim = (node.args[position] if len(node.args) > position else node.kwargs.get("dim", 0)) % max(nd, 1)
        info = {"batched": [True], "protect": {dim}, "outs": ["S"] * len(node.meta["val"])}
        if removes:
            info["out_dim"] = lambda d: d - (1 if d > dim else 0)
        return info
    return describe


def _along_reduce(position: int, outs: int, keep_position: int):
    """Reductions along one dimension that return values and indices (``max.dim``, ``kthvalue``, ...): the other
    dimensions are independent; without ``keepdim`` the dimensions behind the reduced one move up."""
    def describe(node, shapes):
        nd = max(len(shapes[0]), 1)
        dim = (node.args[position] if len(node.args) > position else node.kwargs.get("dim", -1)) % nd
        keep = node.args[keep_position] if len(node.args) > keep_position else node.kwargs.get("keepdim", False)
        info = {"batched": [True] + [False] * (len(shapes) - 1), "protect": {dim}, "outs": ["S"] * outs}
        if not keep:
            info["out_dim"] = lambda d: d - (1 if d > dim else 0)
        return info
    return describe


def _over_dims(outs: int):
    """Statistics over a list of dimensions given as the second argument (``var``, ``std``, ``var_mean``, norms): a cut
    along a dimension that stays is local (the sums of squares have no partial form here)."""
    def describe(node, shapes):
        nd = max(len(shapes[0]), 1)
        dims = node.args[1] if len(node.args) > 1 else node.kwargs.get("dim")
        if isinstance(dims, (int, float)) and node.target in _NORMS:          # (self, ord, dims, keepdim)
            dims = node.args[2] if len(node.args) > 2 else node.kwargs.get("dim")
            keep = node.args[3] if len(node.args) > 3 else node.kwargs.get("keepdim", False)
        else:
            keep = node.kwargs.get("keepdim", node.args[3] if len(node.args) > 3 else False)
        if dims is None or dims == []:
            return None
        dims = {d % nd for d in (dims if isinstance(dims, (list, tuple)) else [dims])}
        info = {"batched": [True] + [False] * (len(shapes) - 1), "protect": dims, "outs": ["S"] * outs}
        if not keep:
            info["out_dim"] = lambda d: d - sum(1 for r in dims if r < d)
        return info
    return describe


def _padded(node, shapes):
    # (input, pad, value): ``pad`` lists (before, after) pairs from the last dimension backwards; a dimension that gets no
    # padding is a batch dimension
    nd = len(shapes[0])
    pad = list(node.args[1])
    touched = {nd - 1 - i // 2 for i, p in enumerate(pad) if p != 0}
    return {"batched": [True], "protect": touched, "outs": ["S"]}


def _rolled(node, shapes):
    # (input, shifts, dims): without dims the whole tensor is rolled as one line
    nd = len(shapes[0])
    dims = node.args[2] if len(node.args) > 2 else node.kwargs.get("dims", [])
    if not dims:
        return None
    return {"batched": [True], "protect": {d % nd for d in dims}, "outs": ["S"]}


def _transformed(node, shapes):
    # (input, dims, normalization, ...): a Fourier transform along ``dims``; the other dimensions are a batch
    nd = max(len(shapes[0]), 1)
    dims = node.args[1]
    return {"batched": [True], "protect": {d % nd for d in dims}, "outs": ["S"]}


def _as_complex(node, shapes):
    # [..., 2] -> complex [...]: the last dimension is consumed
    return {"batched": [True], "protect": {len(shapes[0]) - 1}, "outs": ["S"]}


def _as_real(node, shapes):
    # complex [...] -> [..., 2]: every dimension stays where it is
    return {"batched": [True], "protect": set(), "outs": ["S"]}


def _repeated(node, shapes):
    # (input, repeats): ``repeats`` lines up with the trailing dimensions; a dimension repeated once is a batch dimension
    nd = len(shapes[0])
    reps = list(node.args[1])
    off = len(reps) - nd
    if off < 0:
        return None
    info = {"batched": [True], "protect": {d for d in range(nd) if reps[d + off] != 1}, "outs": ["S"]}
    if off:
        info["out_dim"] = lambda d: d + off
    return info


def _matrices_with_vectors(outs: int):
    """Operands that are stacks of matrices together with stacks of vectors over the same leading dimensions (an LU
    factorisation with its pivots, a matrix with a new diagonal): the leading dimensions are a batch for all of them."""
    def describe(node, shapes):
        nd = len(shapes[0])
        if nd < 3:
            return None
        return {"batched": [True] * len(shapes), "protect": {nd - 2, nd - 1}, "outs": ["S"] * outs}
    return describe


def _layer_norm(node, shapes):
    core = len(node.args[1])
    nd = len(shapes[0])
    return {"batched": [True] + [False] * (len(shapes) - 1), "protect": set(range(nd - core, nd)), "outs": ["S", "S", "S"]}


def _layer_norm_backward(node, shapes):
    # (grad_out, input, normalized_shape, mean, rstd, weight, bias, mask) -> (dx, dweight, dbias): rows are
    # independent for dx; the weight and bias gradients are sums over the rows
    core = len(node.args[2])
    nd = len(shapes[0])
    return {"batched": [True, True, True, True] + [False] * (len(shapes) - 4), "protect": set(range(nd - core, nd)),
            "outs": ["S", "P", "P"]}


# pooling: (position of the kernel / stride / padding / dilation arguments, tensor operands that have the input's
# extent, tensor operands that have the output's extent, number of outputs)
POOLS = {
    aten.avg_pool2d.default: {"kernel": 1, "stride": 2, "padding": 3, "dilation": None, "inputs": (0,), "outputs": (), "outs": 1, "backward": False},
    aten.max_pool2d_with_indices.default: {"kernel": 1, "stride": 2, "padding": 3, "dilation": 4, "inputs": (0,), "outputs": (), "outs": 2, "backward": False},
    aten.avg_pool2d_backward.default: {"kernel": 2, "stride": 3, "padding": 4, "dilation": None, "inputs": (1,), "outputs": (0,), "outs": 1, "backward": True},
    aten.max_pool2d_with_indices_backward.default: {"kernel": 2, "stride": 3, "padding": 4, "dilation": 5, "inputs": (1,), "outputs": (0, 2), "outs": 1, "backward": True},
    aten.avg_pool3d.default: {"kernel": 1, "stride": 2, "padding": 3, "dilation": None, "inputs": (0,), "outputs": (), "outs": 1, "backward": False, "spatial": 3},
    aten.max_pool3d_with_indices.default: {"kernel": 1, "stride": 2, "padding": 3, "dilation": 4, "inputs": (0,), "outputs": (), "outs": 2, "backward": False, "spatial": 3},
    aten.avg_pool3d_backward.default: {"kernel": 2, "stride": 3, "padding": 4, "dilation": None, "inputs": (1,), "outputs": (0,), "outs": 1, "backward": True, "spatial": 3},
    aten.max_pool3d_with_indices_backward.default: {"kernel": 2, "stride": 3, "padding": 4, "dilation": 5, "inputs": (1,), "outputs": (0, 2), "outs": 1, "backward": True, "spatial": 3},
}


# random draws: the executor makes them with a counter-based generator keyed by (seed, execution, draw site, logical
# element), so that a value is the same however it is cut and identical on every processor that holds a copy
DRAWS = {aten.native_dropout.default: "dropout", aten.rand_like.default: "uniform", aten.randn_like.default: "normal",
         aten.rand.default: "uniform", aten.randn.default: "normal"}


def _batch_norm_inference(node, shapes):
    # (input, weight, bias, running_mean, running_var, momentum, eps) -> (output, empty, empty): per-channel arithmetic
    return {"batched": [True] + [False] * (len(shapes) - 1), "protect": {1}, "outs": ["S", "R", "R"]}


def _group_norm(node, shapes):
    # (input, weight, bias, N, C, HxW, groups, eps) -> (output, mean, rstd): every sample is normalised on its own;
    # the batch size is an argument, which the executor replaces by the number of samples it holds
    return {"batched": [True] + [False] * (len(shapes) - 1), "protect": set(range(1, len(shapes[0]))), "outs": ["S", "S", "S"],
            "batch_arg": 3}


def _group_norm_backward(node, shapes):
    # (grad_output, input, mean, rstd, weight, N, C, HxW, groups, mask) -> (grad_input, grad_weight, grad_bias)
    return {"batched": [True, True, True, True] + [False] * (len(shapes) - 4), "protect": set(range(1, len(shapes[0]))),
            "outs": ["S", "P", "P"], "batch_arg": 5}


def _convolution(node, shapes):
    # (input, weight, bias?): samples are independent; a cut anywhere else is the halo rule's business
    return {"batched": [True] + [False] * (len(shapes) - 1), "protect": set(range(1, len(shapes[0]))), "outs": ["S"]}


def _convolution_backward(node, shapes):
    # (grad_output, input, weight, ...) -> (grad_input, grad_weight, grad_bias): the last two sum over the samples
    return {"batched": [True, True] + [False] * (len(shapes) - 2), "protect": set(range(1, len(shapes[0]))),
            "outs": ["S", "P", "P"]}


def _embedding_bag(node, shapes):
    # (weight [V, E], indices, offsets, scale_grad_by_freq, mode, ...) -> (output [bags, E], offset2bag, bag_size,
    # max_indices): the embedding columns are independent, so a table cut along E gives bags cut along E; the rows
    # (vocabulary) are protected.  Mode 2 (max) also returns per-column indices and is left to the generic path.
    mode = node.args[4] if len(node.args) > 4 else node.kwargs.get("mode", 0)
    if mode == 2 or len(shapes[0]) != 2:
        return None
    return {"batched": [True] + [False] * (len(shapes) - 1), "protect": {0}, "outs": ["S", "R", "R", "R"]}


# operators whose leading (or all but one) dimensions are independent problems: a cut there stays where it is
BATCHED = {
    aten._embedding_bag.default: _embedding_bag, aten._embedding_bag_forward_only.default: _embedding_bag,
    aten.linalg_cholesky_ex.default: _trailing(2, 2), aten.linalg_qr.default: _trailing(2, 2),
    aten._linalg_solve_ex.default: _trailing(2, 4), aten.linalg_solve_triangular.default: _trailing(2, 1),
    aten.cholesky_solve.default: _trailing(2, 1), aten.triu.default: _trailing(2, 1), aten.tril.default: _trailing(2, 1),
    aten._linalg_det.default: _trailing(2, 3), aten._linalg_slogdet.default: _trailing(2, 4),
    aten.linalg_inv_ex.default: _trailing(2, 2), aten.linalg_lu_factor_ex.default: _trailing(2, 3),
    aten.sort.default: _along(1, 2), aten.sort.stable: _along(2, 2), aten.topk.default: _along(2, 2),
    aten.cummax.default: _along(1, 2), aten.cummin.default: _along(1, 2),
    aten.split_with_sizes.default: _split(2), aten.split.Tensor: _split(2), aten.unbind.int: _split(1, removes=True),
    aten._native_batch_norm_legit_no_training.default: _batch_norm_inference,
    aten.native_group_norm.default: _group_norm, aten.native_group_norm_backward.default: _group_norm_backward,
    aten.convolution.default: _convolution, aten.convolution_backward.default: _convolution_backward,
    aten.native_layer_norm.default: _layer_norm, aten.native_layer_norm_backward.default: _layer_norm_backward,
    aten.max.dim: _along_reduce(1, 2, 2), aten.min.dim: _along_reduce(1, 2, 2), aten.kthvalue.default: _along_reduce(2, 2, 3),
    aten.median.dim: _along_reduce(1, 2, 2), aten.mode.default: _along_reduce(1, 2, 2),
    aten.prod.dim_int: _along_reduce(1, 1, 2), aten.cumprod.default: _along(1, 1), aten.logcumsumexp.default: _along(1, 1),
    aten.var.correction: _over_dims(1), aten.std.correction: _over_dims(1), aten.var_mean.correction: _over_dims(2),
    aten.std_mean.correction: _over_dims(2), aten.linalg_vector_norm.default: _over_dims(1),
    aten.constant_pad_nd.default: _padded, aten.roll.default: _rolled, aten.index_select.default: _along(1, 1),
    aten.glu.default: _along(1, 1),
    # windows over the trailing dimensions: samples and channels are independent (a cut along a window dimension is the
    # halo rule's business where there is one)
    aten.avg_pool2d.default: _trailing(2, 1, (0,)), aten.max_pool2d_with_indices.default: _trailing(2, 2, (0,)),
    aten.avg_pool2d_backward.default: _trailing(2, 1, (0, 1)),
    aten.max_pool2d_with_indices_backward.default: _trailing(2, 1, (0, 1, 2)),
    aten.avg_pool3d.default: _trailing(3, 1, (0,)), aten.max_pool3d_with_indices.default: _trailing(3, 2, (0,)),
    aten.avg_pool3d_backward.default: _trailing(3, 1, (0, 1)),
    aten.max_pool3d_with_indices_backward.default: _trailing(3, 1, (0, 1, 2)),
    aten._adaptive_avg_pool2d.default: _trailing(2, 1, (0,)), aten._adaptive_avg_pool2d_backward.default: _trailing(2, 1, (0, 1)),
    aten._adaptive_avg_pool3d.default: _trailing(3, 1, (0,)), aten._adaptive_avg_pool3d_backward.default: _trailing(3, 1, (0, 1)),
    aten.adaptive_max_pool2d.default: _trailing(2, 2, (0,)), aten.adaptive_max_pool2d_backward.default: _trailing(2, 1, (0, 1, 2)),
    aten.upsample_nearest1d.default: _trailing(1, 1, (0,)), aten.upsample_nearest2d.default: _trailing(2, 1, (0,)),
    aten.upsample_nearest3d.default: _trailing(3, 1, (0,)), aten.upsample_linear1d.default: _trailing(1, 1, (0,)),
    aten.upsample_bilinear2d.default: _trailing(2, 1, (0,)), aten.upsample_bicubic2d.default: _trailing(2, 1, (0,)),
    aten.upsample_trilinear3d.default: _trailing(3, 1, (0,)),
    aten.upsample_nearest1d.vec: _trailing(1, 1, (0,)), aten.upsample_nearest2d.vec: _trailing(2, 1, (0,)),
    aten.upsample_nearest3d.vec: _trailing(3, 1, (0,)), aten.upsample_linear1d.vec: _trailing(1, 1, (0,)),
    aten.upsample_bilinear2d.vec: _trailing(2, 1, (0,)), aten.upsample_bicubic2d.vec: _trailing(2, 1, (0,)),
    aten.upsample_trilinear3d.vec: _trailing(3, 1, (0,)),
    aten.pixel_shuffle.default: _trailing(3, 1, (0,)), aten.pixel_unshuffle.default: _trailing(3, 1, (0,)),
    aten._fft_c2c.default: _transformed, aten._fft_r2c.default: _transformed, aten._fft_c2r.default: _transformed,
    aten.view_as_complex.default: _as_complex, aten.view_as_real.default: _as_real,
    aten._cdist_forward.default: _trailing(2, 1), aten.grid_sampler_2d.default: _trailing(3, 1),
    aten._linalg_eigh.default: _trailing(2, 2), aten._linalg_svd.default: _trailing(2, 3),
    aten.linalg_matrix_exp.default: _trailing(2, 1), aten.linalg_eig.default: _trailing(2, 2),
    aten.linalg_ldl_factor_ex.default: _trailing(2, 3), aten.linalg_lu.default: _trailing(2, 3),
    aten.linalg_householder_product.default: _trailing(2, 1), aten.geqrf.default: _trailing(2, 2),
    aten.triangular_solve.default: _trailing(2, 2),
    aten.repeat.default: _repeated, aten.repeat_interleave.self_int: _along(2, 1, default=None),
    aten._cdist_backward.default: _trailing(2, 1), aten.grid_sampler_2d_backward.default: _trailing(3, 2),
    aten.linalg_lu_solve.default: _matrices_with_vectors(1), aten.lu_unpack.default: _matrices_with_vectors(3),
    aten.diagonal_scatter.default: _matrices_with_vectors(1),
}
_NORMS = {aten.linalg_vector_norm.default}
# batch norm variants: how many leading arguments are tensors (some optional), which of them have the input's shape,
# and what each output is (the input's shape, a per-channel vector, or something no cut applies to)
_CHANNEL_NORMS = {
    aten._native_batch_norm_legit_no_training.default: {"tensors": 5, "full": (0,), "outs": ("full", "vector", "vector")},
    aten._native_batch_norm_legit_functional.default: {"tensors": 5, "full": (0,), "outs": ("full", "vector", "vector", "vector", "vector")},
    aten._native_batch_norm_legit.no_stats: {"tensors": 3, "full": (0,), "outs": ("full", "vector", "vector")},
    aten.native_batch_norm.default: {"tensors": 5, "full": (0,), "outs": ("full", "vector", "vector")},
    aten.native_batch_norm_backward.default: {"tensors": 7, "full": (0, 1), "outs": ("full", "vector", "vector")},
}
_INDEX_GETS = _overloads("index.Tensor", "_unsafe_index.Tensor")
_INDEX_PUTS = _overloads("index_put.default", "_unsafe_index_put.default")


def _shape(node) -> tuple:
    v = node.meta.get("val")
    return tuple(v.shape) if isinstance(v, torch.Tensor) else ()


def _is_tensor_node(a) -> bool:
    return isinstance(a, torch.fx.Node) and isinstance(a.meta.get("val"), torch.Tensor)


class Propagator:
    """Walks the exported graph once; emits the SPMD plan."""

    def __init__(self, gm: torch.fx.GraphModule, mesh: Mesh, stated: dict, outputs_stated: dict | None = None):
        self.gm, self.mesh = gm, mesh
        self.na = len(mesh.shape)
        self.stated = stated                       # node name -> tuple[Spec] per axis
        self.spec: dict[str, tuple] = {}           # value name -> tuple[Spec]
        self.shape: dict[str, tuple] = {}
        self.dtype: dict[str, torch.dtype] = {}
        self.steps: list[Step] = []
        self.transfers: list[Transfer] = []
        self.tmp = 0
        self.channel = 0
        self.moved: dict = {}                     # (value, placement) -> the value that carries it there
        self.extended: dict = {}                  # (value, left, right) -> its halo-extended copy (forward -> backward)
        self.sites = 0                             # random draws so far: each gets its own stream of the generator
        self.renamed: dict[str, str] = {}         # node name -> value that carries it after a stated reshard

    # ---- helpers
    def fresh(self, base: str) -> str:
        self.tmp += 1
        return f"{base}__r{self.tmp}"

    def all_r(self) -> tuple:
        return tuple(R for _ in range(self.na))

    def wanted(self, name: str):
        """The placement stated for the value ``name``, with the axes it leaves open (``...`` in the N-D form) filled
        in by what propagation found; ``None`` when nothing is stated (or nothing is known of the value yet)."""
        want = self.stated.get(name)
        if want is None or all(w is not None for w in want):
            return want
        have = self.spec.get(name)
        if have is None or len(have) != len(want):
            return None
        return tuple(h if w is None else w for w, h in zip(want, have))

    def emit_collective(self, verb: str, kind: str, axis: int, src: str, spec_from: Spec, spec_to: Spec, consumer=JOIN) -> str:
        out = self.fresh(src)
        if self.mesh.shape[axis] == 1:
            # an axis of one processor: the value is already what the transfer would make of it
            self.steps.append(Step("alias", out, None, (Ref(src),)))
            self.shape[out] = self.shape[src]
            if src in self.dtype:
                self.dtype[out] = self.dtype[src]
            return out
        self.channel += 1
        shp = self.shape[src]
        nbytes = int(math.prod(shp)) * (torch.empty((), dtype=self.dtype[src]).element_size() if src in self.dtype else 4)
        dim = spec_from.dim if spec_from.kind == "S" else spec_to.dim
        cnt = spec_from.counts if spec_from.kind == "S" else spec_to.counts
        self.transfers.append(Transfer(self.channel, kind, verb, axis, src, dim, tuple(cnt), consumer, nbytes))
        self.steps.append(Step("collective", out, verb, (Ref(src),), {},
                               {"axis": axis, "from": spec_from, "to": spec_to, "channel": self.channel, "kind": kind,
                                "full_shape": shp}))
        self.shape[out] = shp
        if src in self.dtype:
            self.dtype[out] = self.dtype[src]
        return out

    def reshard(self, name: str, want: tuple) -> str:
        """Bring value ``name`` to placement ``want`` (per axis); returns the (possibly new) value name.  A value that
        was already brought to this placement is reused: values never change, so one transfer serves every reader."""
        key = (name, tuple(want))
        if key in self.moved:
            return self.moved[key]
        self.moved[key] = out = self._reshard(name, want)
        return out

    # ---- replicated cheap compute
    DUPLICATE_LIMIT = 1 << 22       # elements: beyond this a transfer is cheaper than every reader recomputing

    def _producers(self) -> dict:
        return {st.out: st for st in self.steps}

    def invariant(self, name: str, producers: dict | None = None, seen: set | None = None) -> bool:
        """Does ``name`` depend on no input of the program at all (an index table, a mask, a constant folded from
        literals)?  Such a value can be computed wherever it is read."""
        producers = self._producers() if producers is None else producers
        seen = set() if seen is None else seen
        if name in seen:
            return True
        seen.add(name)
        st = producers.get(name)
        if st is None or st.op not in ("call", "const", "alias"):
            return False                                    # a placeholder, or the result of a transfer
        if st.op == "const":
            return True                                     # every processor builds the whole module: its constants are everywhere
        if "draw" in st.meta:
            return False
        refs: list = []
        _walk_refs(st.args, refs)
        _walk_refs(st.kwargs, refs)
        return all(self.invariant(r, producers, seen) for r in refs)

    def duplicate(self, name: str) -> str:
        """Re-emit the steps that compute the invariant value ``name`` with replicated placement: every processor
        computes its own copy and no transfer is needed (the reference duplicates invariant nodes onto every reader,
        compiler/mesh_compiler/placement.py:884-903: duplicated cheap compute is free, a crossing is not)."""
        producers = self._producers()
        done: dict[str, str] = {}

        def emit(n: str) -> str:
            if n in done:
                return done[n]
            st = producers[n]
            if all(s.kind == "R" for s in self.spec.get(n, ())) and st.op != "alias":
                done[n] = n                                 # already everywhere
                return n
            args = _map_refs(st.args, emit)
            kwargs = _map_refs(st.kwargs, emit)
            out = self.fresh(n)
            self.steps.append(Step(st.op, out, st.target, args, kwargs, {k: v for k, v in st.meta.items() if k != "out_specs"}))
            self.shape[out] = self.shape[n]
            if n in self.dtype:
                self.dtype[out] = self.dtype[n]
            self.spec[out] = self.all_r()
            done[n] = out
            return out
        out = emit(name)
        self.duplicated = getattr(self, "duplicated", 0) + 1
        return out

    def _reshard(self, name: str, want: tuple) -> str:
        have = self.spec[name]
        if any(h.kind == "O" and w != h for h, w in zip(have, want)) and math.prod(self.shape.get(name, (1,)) or (1,)) <= self.DUPLICATE_LIMIT \
                and self.invariant(name):
            # a value that depends on no input, held by one processor and wanted elsewhere: recompute, do not transfer
            return self.reshard(self.duplicate(name), want)
        cur = name
        for ax in range(self.na):
            h, w = have[ax], want[ax]
            if h == w:
                continue
            new_specs = list(self.spec[cur])
            if h.kind == "P":
                if w.kind == "S":
                    cur2 = self.emit_collective("reduce_scatter", "reduce", ax, cur, h, w)
                elif w.kind == "O":
                    cur2 = self.emit_collective("reduce", "reduce", ax, cur, h, w)
                else:
                    cur2 = self.emit_collective("all_reduce", "reduce", ax, cur, h, R)
                    if w.kind == "P":
                        raise AssertionError("replicated -> partial is never requested")
            elif h.kind == "S":
                if w.kind == "R":
                    cur2 = self.emit_collective("all_gather", "broadcast", ax, cur, h, w, consumer=PAGES)
                elif w.kind == "S":
                    if h.dim == w.dim:      # same dim, other cuts: gather + slice (rare)
                        mid = self.emit_collective("all_gather", "broadcast", ax, cur, h, R)
                        self.spec[mid] = tuple(R if i == ax else s for i, s in enumerate(self.spec[cur]))
                        cur2 = self.emit_slice(mid, ax, w)
                    else:
                        cur2 = self.emit_collective("all_to_all", "alltoall", ax, cur, h, w)
                elif w.kind == "O":
                    cur2 = self.emit_collective("gather", "broadcast", ax, cur, h, w)
                else:
                    raise AssertionError(f"sharded -> {w}")
            elif h.kind == "R":
                if w.kind == "S":
                    cur2 = self.emit_slice(cur, ax, w)
                elif w.kind == "O":
                    cur2 = cur                      # every processor has it; the owner simply uses its copy
                    new_specs[ax] = w
                    cur2 = self.alias(cur, tuple(new_specs))
                    have = self.spec[cur2]
                    cur = cur2
                    continue
                else:
                    raise AssertionError(f"replicated -> {w}")
            else:  # owner
                if w.kind == "R":
                    cur2 = self.emit_collective("broadcast", "broadcast", ax, cur, h, w)
                elif w.kind == "O":
                    cur2 = self.emit_collective("send_recv", "permute", ax, cur, h, w)
                elif w.kind == "S":
                    cur2 = self.emit_collective("scatter", "broadcast", ax, cur, h, w)
                else:
                    raise AssertionError(f"owner -> {w}")
            new_specs[ax] = w
            self.spec[cur2] = tuple(new_specs)
            cur = cur2
        return cur

    def alias(self, src: str, specs: tuple) -> str:
        out = self.fresh(src)
        self.steps.append(Step("alias", out, None, (Ref(src),)))
        self.shape[out] = self.shape[src]
        if src in self.dtype:
            self.dtype[out] = self.dtype[src]
        self.spec[out] = specs
        return out

    def emit_slice(self, src: str, axis: int, w: Spec) -> str:
        out = self.fresh(src)
        self.steps.append(Step("slice", out, None, (Ref(src),), {}, {"axis": axis, "to": w}))
        self.shape[out] = self.shape[src]
        if src in self.dtype:
            self.dtype[out] = self.dtype[src]
        specs = list(self.spec[src])
        specs[axis] = w
        self.spec[out] = tuple(specs)
        return out

    # ---- per-axis rules.  Each returns (wanted specs of tensor args, out spec) for ONE axis.
    @staticmethod
    def _owned(specs):
        """The owner spec when, along one axis, some operand is whole on one coordinate and the others are whole on the
        same coordinate or replicated; else ``None``."""
        owner = next((s for s in specs if s.kind == "O"), None)
        if owner is None or any(s.kind not in ("R", "O") for s in specs):
            return None
        return owner

    def rule_pointwise(self, node, targs, specs, ax):
        out_shape = _shape(node)
        nd = len(out_shape)
        shard = None
        owner = None
        for a, s in zip(targs, specs):
            if s.kind == "S":
                ash = self.shape[a]
                d_out = s.dim + (nd - len(ash))
                if shard is None and 0 <= d_out < nd and ash[s.dim] == out_shape[d_out]:
                    shard = (d_out, s)
            elif s.kind == "O" and owner is None:
                owner = s
        partial = [s.kind == "P" for s in specs]
        if shard is None and any(partial):
            lin = LINEAR_IN.get(node.target)
            others_ok = all(s.kind in ("R", "P") for s in specs)
            if node.target in (aten.add.Tensor, aten.sub.Tensor) and any(isinstance(a, (int, float, bool)) for a in node.args[:2]):
                lin = None                                    # partial + constant: every processor would add the constant
            if node.target is aten.div.Tensor and not isinstance(node.args[0], torch.fx.Node):
                lin = None                                    # constant / partial is not linear in the partial
            if node.target not in (aten.clone.default, aten.alias.default, aten._to_copy.default, aten.detach.default) and any(
                    s.kind == "P" and s.op != "sum" for s in specs):
                lin = None                                    # only sums pass through arithmetic; a pending max or min does not
            keep = False
            if lin == "all" and all(partial) and others_ok:
                keep = True
            elif lin == "all" and len(specs) == 1:
                keep = True
            elif lin == "one" and sum(partial) == 1 and others_ok:
                keep = True
            elif lin == "first" and partial[0] and sum(partial) == 1 and others_ok:
                keep = True
            if keep and lin in ("one", "first"):
                # scaling a partial sum can wait for the sum - unless the partial value has other readers too: then each
                # of them would reduce its own product of it.  Sum it once, here, and let them share the result (the
                # single all-reduce in the backward of a column-parallel layer, whose input gradient feeds both the
                # norm's input gradient and its weight gradient).
                tensor_args = [a for a in node.args if _is_tensor_node(a)]
                if len(tensor_args) == len(specs):
                    src = tensor_args[partial.index(True)]
                    if len(src.users) > 1 and any(u.target not in LINEAR_IN for u in src.users):
                        keep = False
                    elif len(src.users) > 1 and sum(1 for u in src.users if LINEAR_IN.get(u.target) in ("one", "first")) > 1:
                        keep = False
            if keep:
                return list(specs), specs[partial.index(True)]
            return [R if s.kind == "P" else s for s in specs], (owner or R) if not any(s.kind == "S" for s in specs) else R
        if shard is not None:
            d_out, s0 = shard
            want = []
            for a in targs:
                ash = self.shape[a]
                d_in = d_out - (nd - len(ash))
                if d_in < 0 or ash[d_in] == 1 and out_shape[d_out] != 1:
                    want.append(R)                             # broadcast along the sharded dim
                else:
                    want.append(Spec("S", d_in, s0.counts, s0.striped))
            return want, Spec("S", d_out, s0.counts, s0.striped)
        if owner is not None:
            return [owner if s.kind != "R" else R for s in specs], owner
        return [R for _ in specs], R

    def rule_mm(self, node, targs, specs, ax, batch: int):
        """mm (batch=0) / bmm (batch=1): A[.., m, k] x B[.., k, n]."""
        a, b = specs
        m_dim, k_a = batch, batch + 1
        k_b, n_dim = batch, batch + 1
        sa = a.dim if a.kind == "S" else None
        sb = b.dim if b.kind == "S" else None
        if batch and sa is not None and sa < batch and (sb == sa or b.kind == "R"):      # a batch dimension: independent products
            return [a, Spec("S", sa, a.counts, a.striped)], Spec("S", sa, a.counts, a.striped)
        if batch and sb is not None and sb < batch and a.kind == "R":
            return [Spec("S", sb, b.counts, b.striped), b], Spec("S", sb, b.counts, b.striped)
        if sa == k_a and (sb == k_b or b.kind == "R"):           # contraction sharded -> partial sums
            return [a, Spec("S", k_b, a.counts, a.striped)], P()
        if sb == k_b and a.kind == "R":
            return [Spec("S", k_a, b.counts, b.striped), b], P()
        if sa == m_dim and b.kind in ("R",):
            return [a, R], Spec("S", m_dim, a.counts, a.striped)
        if sb == n_dim and a.kind == "R":
            return [R, b], Spec("S", n_dim, b.counts, b.striped)
        if sa == m_dim and sb == n_dim:
            # rows of A and columns of B cut over the same axis: one operand has to be whole.  Gather the smaller one
            # (activations of a few tokens against a large weight: gather the activations and keep the weight's cut,
            # which is Megatron's sequence-parallel layer; a small weight against many rows: gather the weight)
            if math.prod(self.shape[targs[0]]) <= math.prod(self.shape[targs[1]]):
                return [R, b], Spec("S", n_dim, b.counts, b.striped)
            return [a, R], Spec("S", m_dim, a.counts, a.striped)
        if sa == m_dim and b.kind == "P":
            return [a, R], Spec("S", m_dim, a.counts, a.striped)
        if a.kind == "P" and b.kind == "R":
            return [a, b], a
        if a.kind == "R" and b.kind == "P":
            return [a, b], b
        if a.kind == "O" or b.kind == "O":
            o = a if a.kind == "O" else b
            return [o if a.kind != "R" else R, o if b.kind != "R" else R], o
        return [R, R], R

    def rule_rows_mm(self, node, targs, specs, ax):
        """``A[..., K] x B[K, N]``: rows of A are independent; the contraction and the columns behave as in ``mm``."""
        a, b = specs
        nd = len(self.shape[targs[0]])
        k_a, n_out = nd - 1, nd - 1
        if a.kind == "S" and a.dim < k_a and b.kind == "R":                     # any leading dimension cut: local
            return [a, R], Spec("S", a.dim, a.counts, a.striped)
        if a.kind == "S" and a.dim == k_a and (b.kind == "R" or (b.kind == "S" and b.dim == 0)):
            return [a, Spec("S", 0, a.counts, a.striped)], P()                  # contraction cut: partial sums
        if b.kind == "S" and b.dim == 0 and a.kind == "R":
            return [Spec("S", k_a, b.counts, b.striped), b], P()
        if b.kind == "S" and b.dim == 1 and a.kind == "R":                      # columns cut (column-parallel weight)
            return [R, b], Spec("S", n_out, b.counts, b.striped)
        if a.kind == "S" and a.dim < k_a and b.kind == "S" and b.dim == 1:
            # rows and columns cut over the same axis: one operand has to be whole; gather the smaller one
            if math.prod(self.shape[targs[0]]) <= math.prod(self.shape[targs[1]]):
                return [R, b], Spec("S", n_out, b.counts, b.striped)
            return [a, R], Spec("S", a.dim, a.counts, a.striped)
        if a.kind == "P" and b.kind == "R":
            return [a, b], a
        if a.kind == "O" or b.kind == "O":
            o = a if a.kind == "O" else b
            return [o if a.kind != "R" else R, o if b.kind != "R" else R], o
        return [R, R], R

    def rule_view(self, node, targs, specs, ax):
        s = specs[0]
        if s.kind != "S":
            return [s], s
        ish, osh = self.shape[targs[0]], _shape(node)
        pre = int(math.prod(ish[:s.dim]))
        acc = 1
        for d_out, sz in enumerate(osh):
            if acc == pre and sz != 1 or (acc == pre and d_out == len(osh) - 1):
                n_in = ish[s.dim]
                if s.striped:
                    # round-robin rows survive a view only where their dimension is left alone (same extent, neither
                    # merged with a neighbour nor split): [B, T, E] -> [B, T, H, D] keeps tokens cut round-robin
                    if sz == n_in and int(math.prod(osh[d_out + 1:])) == int(math.prod(ish[s.dim + 1:])):
                        return [s], Spec("S", d_out, s.counts, True)
                    break
                if sz % n_in == 0:                     # the sharded dim becomes the outer factor of a merged dim
                    f = sz // n_in
                    return [s], Spec("S", d_out, tuple(c * f for c in s.counts))
                if n_in % sz == 0:                     # the sharded dim is split; shards must hold whole inner blocks
                    inner = n_in // sz
                    if all(c % inner == 0 for c in s.counts):
                        return [s], Spec("S", d_out, tuple(c // inner for c in s.counts))
                break
            acc *= sz
            if acc > pre:
                break
        return [R], R

    # ---- the walk
    def run(self, inputs_order: list[str]) -> Plan:
        input_specs, outputs, output_specs = {}, [], {}
        for node in self.gm.graph.nodes:
            if node.op == "placeholder":
                self.shape[node.name] = _shape(node)
                v = node.meta.get("val")
                if isinstance(v, torch.Tensor):
                    self.dtype[node.name] = v.dtype
                sp = self.stated.get(node.name) or self.all_r()
                sp = tuple(R if x is None else x for x in sp)          # an axis left open on an input: whole there
                self.spec[node.name] = sp
                input_specs[node.name] = sp
            elif node.op == "get_attr":
                self.shape[node.name] = _shape(node)
                self.spec[node.name] = self.all_r()
                self.steps.append(Step("const", node.name, node.target))
            elif node.op == "call_function":
                self.call(node)
            elif node.op == "output":
                flat = node.args[0] if isinstance(node.args[0], (tuple, list)) else (node.args[0],)
                for i, o in enumerate(flat):
                    if isinstance(o, torch.fx.Node):
                        want = self.stated.get(("output", i)) or self.all_r()
                        # partial and owner values are completed; sharded values stay sharded only if stated
                        name = self.reshard(self.renamed.get(o.name, o.name), want)
                        outputs.append(name)
                        output_specs[name] = want
                    else:
                        outputs.append(("const", o))
        self._describe_items()
        return Plan(self.mesh, self.steps, inputs_order, input_specs, outputs, output_specs, self.transfers,
                    dict(self.shape), dict(self.dtype))

    def _describe_items(self) -> None:
        """Operators with several results: note on the step what each item is (placement, whole shape, dtype), read off
        the ``getitem`` steps that take them apart.  The executor needs it when a processor's share of a cut operand is
        empty and it states the results itself instead of calling an operator that refuses empty operands."""
        makers = {st.out: st for st in self.steps if st.op == "call" and not st.meta.get("fallback")}
        for st in self.steps:
            if st.op != "call" or st.target is not operator.getitem or not isinstance(st.args[0], Ref):
                continue
            maker = makers.get(st.args[0].name)
            j = st.args[1]
            if maker is None or maker.target is operator.getitem or not isinstance(j, int):
                continue
            if st.out in self.spec and st.out in self.dtype and st.out in self.shape:
                maker.meta.setdefault("items", {})[j] = (self.spec[st.out], tuple(self.shape[st.out]), self.dtype[st.out])

    def call(self, node):
        before = dict(self.renamed)
        try:
            self._call(node)
        finally:
            # operands moved to this node's stated processor were renamed for this node only
            for name in getattr(self, "_moved_for_node", ()):
                if name in before:
                    self.renamed[name] = before[name]
                else:
                    self.renamed.pop(name, None)
            self._moved_for_node = []

    def _call(self, node):
        tgt = node.target
        flat_args = list(node.args)
        tnames = [self.renamed.get(a.name, a.name) for a in flat_args if _is_tensor_node(a)]
        stated = self.stated.get(node.name)
        self._moved_for_node = []
        if stated is not None and tgt is not operator.getitem and any(s is not None and s.kind == "O" for s in stated):
            # "this node runs on that processor": operands that live whole on another processor go there first, so
            # that the operator runs where it was placed (otherwise it would run where its operands are and only its
            # result would move - and every later reader on the stated processor would pull its own copy)
            for a in flat_args:
                if not _is_tensor_node(a):
                    continue
                src = self.renamed.get(a.name, a.name)
                have = self.spec.get(src)
                if have is None or len(have) != len(stated):
                    continue
                if any(w is not None and h.kind == "O" and w.kind == "O" and h.owner != w.owner for h, w in zip(have, stated)):
                    want = tuple(w if (w is not None and h.kind == "O" and w.kind == "O") else h for h, w in zip(have, stated))
                    self.renamed[a.name] = self.reshard(src, want)
                    self._moved_for_node.append(a.name)
            tnames = [self.renamed.get(a.name, a.name) for a in flat_args if _is_tensor_node(a)]
        if tgt is operator.getitem:
            src = self.renamed.get(node.args[0].name, node.args[0].name)
            self.steps.append(Step("call", node.name, tgt, (Ref(src), node.args[1])))
            self.shape[node.name] = _shape(node)
            sp = self.spec.get((src, node.args[1])) or self.spec.get(src) or self.all_r()
            self.spec[node.name] = sp
            v = node.meta.get("val")
            if isinstance(v, torch.Tensor):
                self.dtype[node.name] = v.dtype
            return
        val = node.meta.get("val")
        self.shape[node.name] = _shape(node)
        if isinstance(val, torch.Tensor):
            self.dtype[node.name] = val.dtype
        # list-of-tensor args (cat, stack, index_put): handled by the fallback below unless all equal
        list_args = [a for a in flat_args if isinstance(a, (list, tuple)) and any(_is_tensor_node(x) for x in a)]
        out_specs = []
        wants: dict[str, list] = {n: [] for n in tnames}
        meta: dict[str, Any] = {}
        handled = not list_args and isinstance(val, torch.Tensor)
        if tgt is aten.convolution.default and self.halo_convolution(node, tnames):
            return
        if tgt is aten.convolution_backward.default and self.halo_convolution_backward(node, tnames):
            return
        if tgt is aten.convolution.default and self.patch_transposed_convolution(node, tnames):
            return
        if tgt is aten.convolution_backward.default and self.patch_transposed_convolution(node, tnames, backward=True):
            return
        if tgt is aten.convolution.default and (self.channel_convolution(node, tnames) or self.depthwise_convolution(node, tnames)):
            return
        if tgt is aten.convolution_backward.default and self.depthwise_convolution(node, tnames, backward=True):
            return
        if tgt in _CHANNEL_NORMS and self.channel_norm(node, tnames):
            return
        if getattr(tgt, "namespace", None) == "mesh" and str(tgt) in ("mesh.attention.default", "mesh.attention_backward.default"):
            from . import attention_op  # noqa: F401  (registers the operators)
            if self.attention_operator(node, tnames, backward=str(tgt) == "mesh.attention_backward.default"):
                return
        if tgt is aten.convolution_backward.default and self.channel_convolution_backward(node, tnames):
            return
        if tgt is aten._assert_tensor_metadata.default:
            return                                       # a trace-time check of dtype/shape: nothing to run, no reason to gather
        if tgt is aten.index_put.default and self.accumulating_index_put(node):
            return
        if tgt in (aten.cat.default, aten.stack.default) and self.joined(node):
            return
        if (tgt in _INDEX_GETS or tgt in _INDEX_PUTS) and self.indexed(node):
            return
        if tgt in POOLS and self.pooled(node, tnames):
            return
        if tgt in BATCHED and self.batched(node, tnames):
            return
        if tgt in DRAWS:
            return self.drawn(node, tnames)
        if tgt in CREATION or (not tnames and not list_args):
            self.spec[node.name] = self.all_r()
            self.steps.append(Step("call", node.name, tgt, self.ref_args(node.args), self.ref_kwargs(node.kwargs)))
            return
        if handled:
            for ax in range(self.na):
                specs = [self.spec[n][ax] for n in tnames]
                res = self.axis_rule(node, tnames, specs, ax, meta)
                if res is None:
                    handled = False
                    break
                w, o = res
                for n, s in zip(tnames, w):
                    if len(wants[n]) <= ax:                  # an operand used twice (x * x) states its want once
                        wants[n].append(s)
                out_specs.append(o)
        if handled:
            # two axes must not shard the same tensor dimension of the output
            dims = [s.dim for s in out_specs if s.kind == "S"]
            if len(dims) != len(set(dims)):
                handled = False
        if not handled:
            self.fallback(node, tnames, list_args)
            return
        new_names = {}
        orig = [a.name for a in flat_args if _is_tensor_node(a)]
        for o, n in zip(orig, tnames):
            new_names[o] = self.reshard(n, tuple(wants[n]))
        self.spec[node.name] = tuple(out_specs)
        args = self.ref_args(node.args, new_names)
        kwargs = self.ref_kwargs(node.kwargs, new_names)
        meta["out_specs"] = tuple(out_specs)
        meta["full_shape"] = _shape(node)
        stack = node.meta.get("nn_module_stack")
        if stack:
            meta["module"] = list(stack.values())[-1][0]          # submodule path the op was traced from
        self.steps.append(Step("call", node.name, tgt, args, kwargs, meta))
        want = self.wanted(node.name)
        if want is not None and want != tuple(out_specs):
            self.renamed[node.name] = self.reshard(node.name, want)      # a stated placement is a constraint

    def axis_rule(self, node, tnames, specs, ax, meta):
        tgt = node.target
        owned = self._owned(specs)
        if owned is not None and tgt not in POINTWISE and tgt not in (aten.mm.default, aten.bmm.default, aten.matmul.default, aten.addmm.default):
            # along this axis every operand is whole on one coordinate (a pipeline stage) or everywhere: the operator
            # runs on that coordinate only, whatever it is
            return [owned if s.kind == "O" else R for s in specs], owned
        if tgt in POINTWISE:
            return self.rule_pointwise(node, tnames, specs, ax)
        if tgt in (aten.mm.default, aten.bmm.default):
            return self.rule_mm(node, tnames, specs, ax, 0 if tgt is aten.mm.default else 1)
        if tgt is aten.matmul.default and len(self.shape[tnames[0]]) == len(self.shape[tnames[1]]) >= 3:
            # products batched over several leading dimensions (batch and heads kept apart, see export.unflatten_products)
            return self.rule_mm(node, tnames, specs, ax, len(self.shape[tnames[0]]) - 2)
        if tgt is aten.matmul.default and len(self.shape[tnames[0]]) >= 3 and len(self.shape[tnames[1]]) == 2:
            # [..., K] x [K, N] (a linear layer whose operand keeps its leading dimensions, export.unflatten_linears):
            # every leading dimension is a row dimension
            return self.rule_rows_mm(node, tnames, specs, ax)
        if tgt is aten.addmm.default:                                   # bias + a @ b
            w, o = self.rule_mm(node, tnames[1:], specs[1:], ax, 0)
            if o.kind == "S" and o.dim == 1:
                bias = Spec("S", len(self.shape[tnames[0]]) - 1, o.counts, o.striped)
            elif o.kind == "P":
                # a row-parallel layer with a bias: every processor adds its partial product, and only the first of the
                # axis adds the bias, so the sum counts it once - the result stays a partial sum (it can still be
                # reduce-scattered by its reader instead of all-reduced here)
                if specs[0].kind != "R" or node.kwargs.get("beta", 1) != 1 or node.kwargs.get("alpha", 1) != 1:
                    return [R, R, R], R
                meta.setdefault("once", (0, []))[1].append(ax)
                bias = R
            else:
                bias = R
            return [bias] + w, o
        if tgt in (aten.view.default, aten._unsafe_view.default, aten.reshape.default):
            res = self.rule_view(node, tnames, specs, ax)
            meta.setdefault("localize", ("shape", 1))
            return res
        if tgt is aten.expand.default:
            s = specs[0]
            ish, osh = self.shape[tnames[0]], _shape(node)
            off = len(osh) - len(ish)
            meta.setdefault("localize", ("shape", 1))
            if s.kind == "S":
                return [s], Spec("S", s.dim + off, s.counts, s.striped)
            return [s], s
        if tgt in (aten.permute.default,):
            s = specs[0]
            if s.kind == "S":
                perm = [p % len(node.args[1]) for p in node.args[1]]
                return [s], Spec("S", perm.index(s.dim), s.counts, s.striped)
            return [s], s
        if tgt is aten.flip.default:
            s = specs[0]
            nd = len(self.shape[tnames[0]])
            if s.kind == "S" and s.dim in {d % nd for d in node.args[1]}:
                return [R], R                                            # reversing along the cut moves rows between processors
            return [s], s
        if tgt is aten.diagonal.default:
            s = specs[0]
            nd = len(self.shape[tnames[0]])
            d1 = (node.args[2] if len(node.args) > 2 else node.kwargs.get("dim1", 0)) % nd
            d2 = (node.args[3] if len(node.args) > 3 else node.kwargs.get("dim2", 1)) % nd
            if s.kind == "S":
                if s.dim in (d1, d2):
                    return [R], R
                return [s], Spec("S", s.dim - sum(1 for d in (d1, d2) if d < s.dim), s.counts, s.striped)
            return [s], s
        if tgt in (aten.transpose.int, aten.t.default):
            s = specs[0]
            nd = len(self.shape[tnames[0]])
            d0, d1 = (0, 1) if tgt is aten.t.default else (node.args[1] % nd, node.args[2] % nd)
            if s.kind == "S":
                nd_ = {d0: d1, d1: d0}.get(s.dim, s.dim)
                return [s], Spec("S", nd_, s.counts, s.striped)
            return [s], s
        if tgt is aten.unsqueeze.default:
            s = specs[0]
            nd = len(self.shape[tnames[0]]) + 1
            d = node.args[1] % nd
            if s.kind == "S":
                return [s], Spec("S", s.dim + (1 if d <= s.dim else 0), s.counts, s.striped)
            return [s], s
        if tgt in (aten.squeeze.dim, aten.squeeze.dims):
            s = specs[0]
            nd = len(self.shape[tnames[0]])
            ds = node.args[1] if isinstance(node.args[1], (list, tuple)) else [node.args[1]]
            ds = sorted(d % nd for d in ds if self.shape[tnames[0]][d % nd] == 1)
            if s.kind == "S":
                if s.dim in ds:
                    return [R], R
                return [s], Spec("S", s.dim - sum(1 for d in ds if d < s.dim), s.counts, s.striped)
            return [s], s
        if tgt in REDUCTIONS:
            return self.rule_reduce(node, tnames, specs, ax, meta)
        if tgt in (aten.argmax.default, aten.argmin.default, aten.logsumexp.default):
            # reductions with no partial form: local when the cut is along a dimension that stays
            s = specs[0]
            nd = len(self.shape[tnames[0]])
            dims = node.args[1] if len(node.args) > 1 else None
            keep = bool(node.args[2]) if len(node.args) > 2 else False
            if dims is None:
                return [R], R
            dims = sorted(d % nd for d in (dims if isinstance(dims, (list, tuple)) else [dims]))
            if s.kind != "S":
                return ([s], s) if s.kind == "R" else ([R], R)
            if s.dim in dims:
                return [R], R
            out_dim = s.dim if keep else s.dim - sum(1 for d in dims if d < s.dim)
            return [s], Spec("S", out_dim, s.counts, s.striped)
        if tgt in SOFTMAX_LIKE:
            pos = SOFTMAX_LIKE[tgt]
            nd = len(self.shape[tnames[0]])
            dim = node.args[pos] if len(node.args) > pos else -1
            dim = dim % max(nd, 1)
            shard = next((s for s in specs if s.kind == "S"), None)
            if isinstance(node.meta.get("val"), (tuple, list)):
                return None
            if shard is not None and shard.dim != dim:
                return [Spec("S", shard.dim, shard.counts, shard.striped) for _ in specs], shard
            return [R for _ in specs], R
        if tgt in (aten.gather.default, aten.scatter_add.default, aten.scatter.src):
            # every tensor operand cut along the same dimension, which is not the indexed one: rows are independent
            nd = len(self.shape[tnames[0]])
            dim = node.args[1] % max(nd, 1)
            shard = next((s for s in specs if s.kind == "S"), None)
            same_rank = all(len(self.shape[n]) == nd for n in tnames)
            if shard is not None and shard.dim != dim and same_rank and all(
                    self.shape[n][shard.dim] == self.shape[tnames[0]][shard.dim] for n in tnames):
                return [Spec("S", shard.dim, shard.counts, shard.striped) for _ in specs], Spec("S", shard.dim, shard.counts, shard.striped)
            return [R for _ in specs], R
        if tgt in (aten.slice_scatter.default, aten.select_scatter.default):
            # (whole, piece, dim, ...): a cut along any other dimension carries through both operands
            nd = len(self.shape[tnames[0]])
            dim = (node.args[2] if len(node.args) > 2 else node.kwargs.get("dim", 0)) % nd
            drop = tgt is aten.select_scatter.default
            whole, piece = specs
            if whole.kind == "S" and whole.dim != dim and not whole.striped:
                d = whole.dim - (1 if drop and whole.dim > dim else 0)
                return [whole, Spec("S", d, whole.counts)], Spec("S", whole.dim, whole.counts)
            if whole.kind == "R" and piece.kind == "S" and not piece.striped:
                d = piece.dim + (1 if drop and piece.dim >= dim else 0)
                if d != dim:
                    return [Spec("S", d, piece.counts), piece], Spec("S", d, piece.counts)
            return [R, R], R
        if tgt is aten.scaled_dot_product_attention.default:
            # q, k, v [batch, heads, tokens, head_dim]: heads (or the batch) cut the same way on all three -> local
            if len(tnames) == 4 and _is_tensor_node(node.args[3] if len(node.args) > 3 else node.kwargs.get("attn_mask")):
                # with a mask tensor [batch | 1, heads | 1, queries, keys]: the mask follows the cut where it spans the
                # cut dimension and stays whole where it broadcasts over it
                res = self._attention_with_mask(node, tnames, specs)
                if res is not None:
                    return res
                return None
            if len(tnames) != 3:
                return None
            q = specs[0]
            same_heads = self.shape[tnames[0]][1] == self.shape[tnames[1]][1] == self.shape[tnames[2]][1]
            if q.kind == "S" and q.dim in (0, 1) and not q.striped and (q.dim == 0 or same_heads):
                want = Spec("S", q.dim, q.counts)
                return [want, want, want], want
            causal = node.kwargs.get("is_causal", node.args[5] if len(node.args) > 5 else False)
            if q.kind == "S" and q.dim == 2 and all(s.kind in ("R", "S") for s in specs[1:]) and (
                    not causal or self.shape[tnames[0]][2] == self.shape[tnames[1]][2]):
                # queries are independent of each other: keep them cut, hold all keys and values; a causal mask is then
                # stated by the executor for the rows this processor holds (their positions in the whole sequence)
                if causal:
                    meta["causal_rows"] = ax
                return [Spec("S", 2, q.counts, q.striped), R, R], Spec("S", 2, q.counts, q.striped)
            kv = next((s for s in specs[1:] if s.kind == "S" and s.dim in (0, 1) and not s.striped), None)
            if q.kind == "R" and kv is not None and (kv.dim == 0 or same_heads):
                want = Spec("S", kv.dim, kv.counts)
                return [want, want, want], want
            return [R, R, R], R
        if tgt is aten.embedding.default:
            w, idx = specs
            if idx.kind == "S" and w.kind == "R":
                return [R, idx], Spec("S", idx.dim, idx.counts, idx.striped)
            if w.kind == "S" and w.dim == 0 and idx.kind == "R" and not w.striped:
                meta["vocab_parallel"] = (ax, w.counts)
                return [w, R], P()
            if w.kind == "S" and w.dim == 1 and idx.kind == "R":
                return [w, R], Spec("S", len(_shape(node)) - 1, w.counts, w.striped)
            return [R, R], R
        if tgt is aten.embedding_dense_backward.default:
            g, idx = specs
            if g.kind == "S" and idx.kind == "S" and g.dim == idx.dim:
                return [g, idx], P()
            if g.kind == "S" and g.dim == len(self.shape[tnames[0]]) - 1 and idx.kind == "R":
                return [g, R], Spec("S", 1, g.counts, g.striped)
            return [R, R], R
        if tgt in (aten.slice.Tensor, aten.select.int, aten.narrow.default, aten.slice_backward.default,
                   aten.select_backward.default):
            s = specs[0]
            if tgt in (aten.slice_backward.default, aten.select_backward.default):
                dim = node.args[2]
                nd = len(node.args[1])
            else:
                dim = node.args[1] if len(node.args) > 1 else 0
                nd = len(self.shape[tnames[0]])
            dim = dim % nd
            if s.kind == "S" and s.dim != dim:
                out_dim = s.dim - (1 if tgt is aten.select.int and dim < s.dim else 0)
                if tgt in (aten.slice_backward.default, aten.select_backward.default):
                    meta.setdefault("localize", ("shape", 1))
                    out_dim = s.dim + (1 if tgt is aten.select_backward.default and dim <= s.dim else 0)
                return [s], Spec("S", out_dim, s.counts, s.striped)
            if s.kind == "S":
                return [R], R
            return [s], s
        if tgt is aten.histc.default:
            # counts of a fixed range of bins: every processor counts its own elements, the counts are partial sums
            lo = node.args[2] if len(node.args) > 2 else node.kwargs.get("min", 0)
            hi = node.args[3] if len(node.args) > 3 else node.kwargs.get("max", 0)
            s = specs[0]
            if s.kind == "S" and lo != hi:                   # (min = max = 0 means the data's own range: a global fact)
                return [s], P()
            return [R], R
        if tgt in (aten.native_layer_norm.default,):
            return None
        return None

    def _attention_with_mask(self, node, tnames, specs):
        q, k, v, mask = specs
        qs, ks, ms = self.shape[tnames[0]], self.shape[tnames[1]], self.shape[tnames[3]]
        if len(ms) != 4 or len(qs) != 4:
            return None
        same_heads = qs[1] == ks[1] == self.shape[tnames[2]][1]
        cut = next((s for s in (q, k, v) if s.kind == "S"), None)
        if any(s.kind not in ("R", "S") for s in specs):
            return [R, R, R, R], R
        if cut is None:
            if mask.kind == "S" and mask.dim in (0, 1, 2) and not mask.striped and ms[mask.dim] == qs[mask.dim] and (mask.dim != 1 or same_heads):
                want = Spec("S", mask.dim, mask.counts)            # only the mask is cut: the others give up all but its rows
                return ([want, want if mask.dim < 2 else R, want if mask.dim < 2 else R, want]), want
            return [R, R, R, R], R
        if cut.dim in (0, 1) and not cut.striped and (cut.dim == 0 or same_heads):
            want = Spec("S", cut.dim, cut.counts)
            return [want, want, want, want if ms[cut.dim] == qs[cut.dim] else R], want
        if q.kind == "S" and q.dim == 2:
            want = Spec("S", 2, q.counts, q.striped)               # queries are independent: their mask rows go with them
            return [want, R, R, want if ms[2] == qs[2] else R], want
        return [R, R, R, R], R

    def rule_reduce(self, node, tnames, specs, ax, meta):
        s = specs[0]
        tgt = node.target
        kind = REDUCTIONS[tgt]
        ish = self.shape[tnames[0]]
        nd = len(ish)
        if tgt in (aten.sum.default, aten.mean.default, aten.any.default, aten.all.default, aten.max.default, aten.min.default):
            dims, keep = list(range(nd)), False
        else:
            d = node.args[1] if len(node.args) > 1 else None
            dims = list(range(nd)) if d is None or d == [] else [x % nd for x in (d if isinstance(d, (list, tuple)) else [d])]
            keep = bool(node.args[2]) if len(node.args) > 2 else False
        if s.kind == "S":
            if s.dim in dims:
                if kind == "mean":
                    total = int(math.prod(ish[d] for d in dims))
                    meta["mean_as_sum"] = total
                    return [s], P("sum")
                return [s], P(kind)
            nd_ = s.dim if keep else s.dim - sum(1 for d in dims if d < s.dim)
            return [s], Spec("S", nd_, s.counts, s.striped)
        if s.kind == "P":
            if kind == "sum" or (kind == "mean"):
                return [s], s
            return [R], R
        return [s], s

    def joined(self, node) -> bool:
        """``cat`` / ``stack`` of tensors that carry the same cut along a dimension other than the joined one (whole
        copies among them give up all but their own rows): every processor joins its own pieces and the result keeps
        the cut (for ``stack``, dimensions at or after the new one move up by one)."""
        parts = list(node.args[0])
        if not parts or not all(_is_tensor_node(p) for p in parts):
            return False
        names = [self.renamed.get(p.name, p.name) for p in parts]
        nd = len(self.shape[names[0]])
        dim = (node.args[1] if len(node.args) > 1 else node.kwargs.get("dim", 0))
        stack = node.target is aten.stack.default
        dim = dim % (nd + 1 if stack else max(nd, 1))
        out_spec, wants = [], {n: [] for n in names}
        for a in range(self.na):
            here = [self.spec[n][a] for n in names]
            if any(o.kind not in ("R", "S") for o in here):
                return False
            sp = next((o for o in here if o.kind == "S"), None)
            if sp is None:
                out_spec.append(R)
                for n in names:
                    if len(wants[n]) <= a:
                        wants[n].append(R)
                continue
            if not stack and sp.dim == dim:
                return False
            extent = self.shape[next(n for n, o in zip(names, here) if o.kind == "S")][sp.dim]
            for n, o in zip(names, here):
                if len(self.shape[n]) != nd or self.shape[n][sp.dim] != extent:
                    return False
                if o.kind == "S" and (o.dim != sp.dim or o.counts != sp.counts or o.striped != sp.striped):
                    return False
                if len(wants[n]) <= a:
                    wants[n].append(Spec("S", sp.dim, sp.counts, sp.striped))      # a whole copy gives up all but its own rows
            d = sp.dim + 1 if (stack and sp.dim >= dim) else sp.dim
            out_spec.append(Spec("S", d, sp.counts, sp.striped))
        if all(s.kind == "R" for s in out_spec):
            return False                                   # nothing to keep: the generic path handles it
        out_spec = tuple(out_spec)
        new_names = {}
        for part, n in zip(parts, names):
            new_names[part.name] = self.reshard(n, tuple(wants[n]))
        self.shape[node.name] = _shape(node)
        v = node.meta.get("val")
        if isinstance(v, torch.Tensor):
            self.dtype[node.name] = v.dtype
        self.spec[node.name] = out_spec
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names),
                               self.ref_kwargs(node.kwargs, new_names), {"out_specs": out_spec, "full_shape": _shape(node)}))
        want = self.wanted(node.name)
        if want is not None and want != out_spec:
            self.renamed[node.name] = self.reshard(node.name, want)
        return True

    def pooled(self, node, tnames) -> bool:
        """2-D and 3-D pooling (and its backward) over an input cut along a spatial dimension where no window straddles a cut:
        stride = kernel, no padding or dilation there, every processor's extent a multiple of the kernel.  Each
        processor pools its own block; the output is cut at the same places, divided by the kernel.  (The indices of a
        max pooling are positions within the local block, which is what its backward, run on the same block, expects.)
        Cuts along the batch or channel dimensions need nothing: they are handled as a batch."""
        info = POOLS[node.target]
        args = list(node.args)

        def arg(key, default):
            pos = info[key]
            v = args[pos] if pos is not None and len(args) > pos else default
            return list(v) if isinstance(v, (list, tuple)) else [v] * k
        k = info.get("spatial", 2)                                     # window dimensions: the trailing ones
        kernel = arg("kernel", None)
        stride = arg("stride", []) or kernel
        padding, dilation = arg("padding", 0), arg("dilation", 1)
        kernel, stride, padding, dilation = (v * k if len(v) == 1 else v for v in (kernel, stride, padding, dilation))
        x = tnames[list(info["inputs"])[0]] if not info["backward"] else tnames[1]
        nd = len(self.shape[x])
        ins = [tnames[i] for i in info["inputs"]]
        outs = [tnames[i] for i in info["outputs"]]
        wants = {n: [] for n in tnames}
        spec_in, spec_out = [], []
        found = False
        for ax in range(self.na):
            sp = self.spec[x][ax]
            if sp.kind == "R":
                others = [self.spec[n][ax] for n in tnames if n != x]
                if any(o.kind != "R" for o in others):
                    return False
                for n in tnames:
                    if len(wants[n]) <= ax:
                        wants[n].append(R)
                spec_in.append(R)
                spec_out.append(R)
                continue
            if sp.kind != "S" or sp.striped:
                return False
            if sp.dim < nd - k:                                        # batch or channel: nothing to check
                small = sp
            else:
                i = sp.dim - (nd - k)
                if stride[i] != kernel[i] or padding[i] or dilation[i] != 1 or any(c % kernel[i] for c in sp.counts):
                    return False
                small = Spec("S", sp.dim, tuple(c // kernel[i] for c in sp.counts))
            found = True
            for n in ins:
                if len(wants[n]) <= ax:
                    wants[n].append(sp)
            for n in outs:
                if len(wants[n]) <= ax:
                    wants[n].append(small)
            spec_in.append(sp)
            spec_out.append(small)
        if not found:
            return False
        new_names = {}
        orig = [a.name for a in node.args if _is_tensor_node(a)]
        for o, n in zip(orig, tnames):
            new_names[o] = self.reshard(n, tuple(wants[n]))
        result = tuple(spec_in if info["backward"] else spec_out)
        val = node.meta.get("val")
        if isinstance(val, (tuple, list)):
            for i in range(len(val)):
                self.spec[(node.name, i)] = result
            self.spec[node.name] = self.all_r()
        else:
            self.spec[node.name] = result
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names),
                               self.ref_kwargs(node.kwargs, new_names), {"out_specs": result, "full_shape": _shape(node)}))
        return True

    def batched(self, node, tnames) -> bool:
        """An operator of ``BATCHED`` whose operands are cut along a batch dimension (one it does not work along):
        every processor runs it on its own problems; outputs keep the cut (or are partial sums where the operator sums
        over the batch).  Handles operators with several outputs, which the per-axis rules do not."""
        shapes = [self.shape[n] for n in tnames]
        info = BATCHED[node.target](node, shapes)
        if info is None:
            return False
        flags, protect, outs = info["batched"], info["protect"], info["outs"]
        wants = {n: [] for n in tnames}
        out_specs = [[] for _ in outs]
        found = False
        for ax in range(self.na):
            specs = [self.spec[n][ax] for n in tnames]
            owned = self._owned(specs)
            if owned is not None:                           # a pipeline stage along this axis: run there
                for n in tnames:
                    if len(wants[n]) <= ax:
                        wants[n].append(owned)
                for o in out_specs:
                    o.append(owned)
                continue
            if any(s.kind not in ("R", "S") for s in specs):
                return False
            cut = next((s for s, f in zip(specs, flags) if f and s.kind == "S"), None)
            if cut is None:
                if any(s.kind != "R" for s in specs):
                    return False                            # an unbatched operand is cut: the generic path gathers it
                for n in tnames:
                    if len(wants[n]) <= ax:
                        wants[n].append(R)
                for o in out_specs:
                    o.append(R)
                continue
            lead = shapes[flags.index(True)][: cut.dim + 1]
            if cut.dim in protect or any(f and tuple(sh[: cut.dim + 1]) != tuple(lead) for f, sh in zip(flags, shapes)):
                return False
            found = True
            same = Spec("S", cut.dim, cut.counts, cut.striped)
            moved = Spec("S", info["out_dim"](cut.dim), cut.counts, cut.striped) if "out_dim" in info else same
            for n, f in zip(tnames, flags):
                if len(wants[n]) <= ax:
                    wants[n].append(same if f else R)
            for o, kind in zip(out_specs, outs):
                o.append(moved if kind == "S" else R if kind == "R" else P())
        if not found:
            return False
        dims = [s.dim for s in out_specs[0] if s.kind == "S"]
        if len(dims) != len(set(dims)):
            return False
        new_names = {}
        orig = [a.name for a in node.args if _is_tensor_node(a)]
        for o, n in zip(orig, tnames):
            new_names[o] = self.reshard(n, tuple(wants[n]))
        val = node.meta.get("val")
        several = isinstance(val, (tuple, list))
        if several:
            for i, sp in enumerate(out_specs[: len(val)]):
                self.spec[(node.name, i)] = tuple(sp)
            self.spec[node.name] = self.all_r()
        else:
            self.spec[node.name] = tuple(out_specs[0])
        meta = {"out_specs": tuple(out_specs[0]), "full_shape": _shape(node)}
        if "batch_arg" in info:
            meta["batch_arg"] = info["batch_arg"]
        stack = node.meta.get("nn_module_stack")
        if stack:
            meta["module"] = list(stack.values())[-1][0]
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names),
                               self.ref_kwargs(node.kwargs, new_names), meta))
        want = self.wanted(node.name)
        if not several and want is not None and want != self.spec[node.name]:
            self.renamed[node.name] = self.reshard(node.name, want)
        return True

    def drawn(self, node, tnames) -> None:
        """A random draw (dropout mask, ``rand`` / ``randn`` and their ``_like`` forms).  It takes the next draw-site
        number (the reference numbers draw sites the same way, compiler/mesh_compiler/export.py:412-507) and the
        placement of its operand: each processor draws exactly the elements it holds."""
        kind = DRAWS[node.target]
        site, self.sites = self.sites, self.sites + 1
        new_names = {}
        if tnames:
            src = tnames[0]
            want = tuple(s if s.kind in ("R", "S") else R for s in self.spec[src])      # partial sums are summed first
            new_names[node.args[0].name] = self.reshard(src, want)
            out_spec = tuple(Spec(s.kind, s.dim, s.counts, s.striped) if s.kind == "S" else R for s in want)
        else:
            out_spec = self.all_r()
        val = node.meta.get("val")
        first = val[0] if isinstance(val, (tuple, list)) else val
        full = tuple(first.shape)
        if isinstance(val, (tuple, list)):
            for i in range(len(val)):
                self.spec[(node.name, i)] = out_spec
        else:
            self.dtype[node.name] = first.dtype
        self.spec[node.name] = out_spec
        self.shape[node.name] = _shape(node)
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names), self.ref_kwargs(node.kwargs, new_names),
                               {"draw": kind, "site": site, "out_specs": out_spec, "full_shape": full, "dtype": first.dtype}))

    def accumulating_index_put(self, node) -> bool:
        """``zeros.index_put(indices, values, accumulate=True)`` with the indices and values cut along the same leading
        dimension (the backward of an embedding or of a gather over sharded tokens): every processor accumulates its
        own rows into a zero buffer; the results are partial sums."""
        base, indices, values = node.args[0], node.args[1], node.args[2]
        accumulate = node.args[3] if len(node.args) > 3 else node.kwargs.get("accumulate", False)
        if not accumulate or not _is_tensor_node(base) or not _is_tensor_node(values):
            return False
        zero_makers = (aten.zeros.default, aten.new_zeros.default, aten.zeros_like.default, aten.full.default, aten.full_like.default)
        if base.op != "call_function" or base.target not in zero_makers:
            return False
        if base.target in (aten.full.default, aten.full_like.default) and base.args[1] != 0:
            return False
        idx_nodes = [i for i in indices if i is not None]
        if not idx_nodes or not all(_is_tensor_node(i) for i in idx_nodes):
            return False
        vname = self.renamed.get(values.name, values.name)
        cut = [(a, sp) for a, sp in enumerate(self.spec[vname]) if sp.kind != "R"]
        if len(cut) != 1 or cut[0][1].kind != "S":
            return False
        ax, sp = cut[0]
        new_names = {}
        for i in idx_nodes:          # the indices follow the values' cut: it must be a dimension the index tensors span
            iname = self.renamed.get(i.name, i.name)
            ish = self.shape[iname]
            if sp.dim >= len(ish) or tuple(ish) != tuple(self.shape[vname][: len(ish)]):
                return False
        for i in idx_nodes:
            iname = self.renamed.get(i.name, i.name)
            want = tuple(Spec("S", sp.dim, sp.counts, sp.striped) if a == ax else R for a in range(self.na))
            new_names[i.name] = self.reshard(iname, want)
        bname = self.renamed.get(base.name, base.name)
        new_names[base.name] = self.reshard(bname, self.all_r())
        out_spec = tuple(P() if a == ax else R for a in range(self.na))
        self.shape[node.name] = _shape(node)
        v = node.meta.get("val")
        if isinstance(v, torch.Tensor):
            self.dtype[node.name] = v.dtype
        self.spec[node.name] = out_spec
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names),
                               self.ref_kwargs(node.kwargs, new_names), {"out_specs": out_spec, "full_shape": _shape(node)}))
        return True

    def indexed(self, node) -> bool:
        """``x[..., i, j, ...]`` (``index.Tensor``) and ``x.index_put((..., i, j, ...), values)`` where ``x`` is cut along
        a dimension that the index tensors leave alone (a ``None`` entry before them, or behind them when they sit
        together): every processor indexes its own block with the whole index tensors."""
        put = node.target in _INDEX_PUTS
        base, indices = node.args[0], list(node.args[1])
        values = node.args[2] if put else None
        if not _is_tensor_node(base) or (put and not _is_tensor_node(values)):
            return False
        bname = self.renamed.get(base.name, base.name)
        bshape = self.shape[bname]
        at = [i for i, ix in enumerate(indices) if ix is not None]
        if not at or not all(_is_tensor_node(indices[i]) for i in at):
            return False
        first, last, together = at[0], at[-1], at[-1] - at[0] + 1 == len(at)
        out_nd = len(_shape(node))
        spread = out_nd - (len(bshape) - len(at))            # dimensions the broadcast index tensors contribute
        vname = self.renamed.get(values.name, values.name) if put else None
        specs = self.spec[bname]
        base_want, out_spec, val_want = [], [], []
        found = False
        if put:
            vshape = self.shape[vname]
            res_nd = len(bshape) - len(at) + max(len(self.shape[self.renamed.get(indices[i].name, indices[i].name)]) for i in at)
        for ax, sp in enumerate(specs):
            if sp.kind == "R" and put and self.spec[vname][ax].kind == "S":
                # a whole base (the zeros a backward accumulates into) under cut values: the base gives up all but the
                # rows of the values' cut when that dimension is one the index tensors leave alone
                vs = self.spec[vname][ax]
                rdim = vs.dim + (res_nd - len(vshape))               # its dimension in the indexed result
                if rdim < first:
                    bdim = rdim
                elif together and rdim >= first + (res_nd - (len(bshape) - len(at))):
                    bdim = rdim - (res_nd - (len(bshape) - len(at))) + len(at)
                else:
                    return False
                if vshape[vs.dim] != bshape[bdim]:
                    return False
                sp = Spec("S", bdim, vs.counts, vs.striped)
            if sp.kind == "R":
                if put and self.spec[vname][ax].kind not in ("R", "P"):
                    return False
                base_want.append(R); out_spec.append(R); val_want.append(R)
                continue
            if sp.kind != "S" or sp.dim in at:
                return False
            if sp.dim < first:
                moved = sp.dim
            elif together and sp.dim > last:
                moved = sp.dim - len(at) + spread
            else:
                return False
            found = True
            base_want.append(sp)
            if put:
                # the values line up with the indexed result (trailing-aligned broadcast): cut them where they span the
                # dimension, keep them whole where they broadcast over it
                res_dim = sp.dim if sp.dim < first else sp.dim - len(at) + (res_nd - (len(bshape) - len(at)))
                vdim = res_dim - (res_nd - len(vshape))
                if vdim >= 0 and vshape[vdim] == bshape[sp.dim]:
                    val_want.append(Spec("S", vdim, sp.counts, sp.striped))
                elif vdim < 0 or vshape[vdim] == 1:
                    val_want.append(R)
                else:
                    return False
                out_spec.append(sp)
            else:
                out_spec.append(Spec("S", moved, sp.counts, sp.striped))
        if not found:
            return False
        new_names = {base.name: self.reshard(bname, tuple(base_want))}
        for i in at:
            iname = self.renamed.get(indices[i].name, indices[i].name)
            new_names[indices[i].name] = self.reshard(iname, self.all_r())
        if put:
            if any(s.kind == "P" for s in self.spec[vname]) and not all(w.kind == "R" for w in val_want):
                pass                                         # reshard below sums partial values first
            new_names[values.name] = self.reshard(vname, tuple(val_want))
        self.spec[node.name] = tuple(out_spec)
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names),
                               self.ref_kwargs(node.kwargs, new_names), {"out_specs": tuple(out_spec), "full_shape": _shape(node)}))
        return True

    def _spatial_cut(self, x: str):
        """``((axis, spec), {axis: batch spec})`` when ``x`` is cut along exactly one spatial dimension (contiguous) and,
        on other grid axes, at most along the batch dimension; ``(None, None)`` otherwise."""
        cut, batch = None, {}
        for a, sp in enumerate(self.spec[x]):
            if sp.kind == "R":
                continue
            if sp.kind == "S" and sp.dim == 0:
                batch[a] = sp
            elif sp.kind == "S" and sp.dim >= 2 and not sp.striped and cut is None:
                cut = (a, sp)
            else:
                return None, None
        return (cut, batch) if cut is not None else (None, None)

    def halo_convolution(self, node, tnames) -> bool:
        """A convolution whose input is cut along one spatial dimension: every processor fetches the rows of its
        neighbours that its windows reach (a neighbour exchange, the reference's halos, placement.py:388-485) and
        convolves its own extended block with no padding along that dimension; the output keeps the input's cut.
        Handled when the windows are 'same'-sized along the cut dimension (stride 1, 2 * padding = dilation *
        (kernel - 1)), the cut is contiguous and the weights are replicated; anything else falls back to gathering."""
        x, w = tnames[0], tnames[1]
        args = list(node.args)
        stride, padding, dilation, transposed, groups = args[3], list(args[4]), args[5], args[6], args[8]
        if transposed or any(self.spec[n][a].kind != "R" for n in tnames[1:] for a in range(self.na)):
            return False
        cut, batch = self._spatial_cut(x)
        if cut is None:
            return False
        ax, sp = cut
        i = sp.dim - 2
        k = self.shape[w][sp.dim]
        reach = dilation[i] * (k - 1)
        halo = self._halo_extent(self.shape[x][sp.dim], _shape(node)[sp.dim], sp.counts, stride[i], padding[i], reach)
        if halo is None:
            return False
        left, right = halo
        small = tuple(c // stride[i] for c in sp.counts)
        src = x
        if left + right and (x, left, right) in self.extended:
            src = self.extended[(x, left, right)]
        elif left + right:
            src = self.fresh(x)
            self.extended[(x, left, right)] = src
            self.channel += 1
            esz = torch.empty((), dtype=self.dtype[x]).element_size() if x in self.dtype else 4
            edge = int(math.prod(self.shape[x])) // max(1, self.shape[x][sp.dim]) * (left + right) * esz
            self.transfers.append(Transfer(self.channel, "permute", "halo", ax, x, sp.dim, tuple(sp.counts), JOIN, edge))
            self.steps.append(Step("collective", src, "halo", (Ref(x),), {},
                                   {"axis": ax, "from": sp, "to": sp, "channel": self.channel, "kind": "permute",
                                    "full_shape": self.shape[x], "left": left, "right": right}))
            self.shape[src] = self.shape[x]
            if x in self.dtype:
                self.dtype[src] = self.dtype[x]
            self.spec[src] = self.spec[x]
        padding[i] = 0
        new_args = list(self.ref_args(node.args, {node.args[0].name: src}))
        new_args[4] = padding
        out_spec = tuple(Spec("S", sp.dim, small) if a == ax else batch.get(a, R) for a in range(self.na))
        self.spec[node.name] = out_spec
        self.steps.append(Step("call", node.name, node.target, tuple(new_args), self.ref_kwargs(node.kwargs),
                               {"out_specs": out_spec, "full_shape": _shape(node), "halo": (left, right)}))
        want = self.wanted(node.name)
        if want is not None and want != out_spec:
            self.renamed[node.name] = self.reshard(node.name, want)
        return True

    @staticmethod
    def _halo_extent(n_in: int, n_out: int, counts, stride: int, padding: int, reach: int):
        """``(left, right)`` rows a processor needs from its neighbours so that it can compute, from its own block of a
        cut dimension, the outputs whose windows start in that block; ``None`` when the outputs do not divide that way.
        They do when every block is a multiple of the stride and the operator makes one output per ``stride`` inputs
        ('same' windows at stride 1, the usual halving convolutions, patch embeddings): output ``o`` reads inputs
        ``o * stride - padding .. + reach``, so a block starting at a multiple of the stride needs ``padding`` rows on
        its left and ``reach - padding - (stride - 1)`` on its right (none when that is negative: its last rows are
        then read by nobody)."""
        if n_in % stride or n_out * stride != n_in or any(c % stride for c in counts):
            return None
        left, right = padding, max(reach - padding - (stride - 1), 0)
        if left + right and min(counts) < max(left, right):
            return None
        return left, right

    def _halo_step(self, x: str, ax: int, sp: Spec, left: int, right: int, verb: str = "halo") -> str:
        """Emit the neighbour exchange of ``x``'s edge rows (or, for ``halo_back``, its adjoint); returns the new value."""
        out = self.fresh(x)
        self.channel += 1
        esz = torch.empty((), dtype=self.dtype[x]).element_size() if x in self.dtype else 4
        full = self.shape[x]
        edge = int(math.prod(full)) // max(1, full[sp.dim]) * (left + right) * esz
        self.transfers.append(Transfer(self.channel, "permute", verb, ax, x, sp.dim, tuple(sp.counts), JOIN, edge))
        self.steps.append(Step("collective", out, verb, (Ref(x),), {},
                               {"axis": ax, "from": sp, "to": sp, "channel": self.channel, "kind": "permute",
                                "full_shape": full, "left": left, "right": right}))
        self.shape[out] = full
        if x in self.dtype:
            self.dtype[out] = self.dtype[x]
        self.spec[out] = self.spec[x]
        return out

    def _channel_axes(self, x: str, w: str, transposed: bool, out_of_grad: bool = False):
        """Per grid axis, how a convolution's channels are cut: ``"out"`` (the weight along its output channels, the
        column-parallel form), ``"in"`` (the input along its channels and the weight, if cut, the same way: the
        row-parallel form, partial sums), ``"batch"``, ``None`` (whole), or ``False`` when the rule does not apply."""
        o_dim, i_dim = (1, 0) if transposed else (0, 1)
        kinds = []
        for a in range(self.na):
            xs, ws = self.spec[x][a], self.spec[w][a]
            if xs.kind not in ("R", "S") or ws.kind not in ("R", "S"):
                return False
            if ws.kind == "S" and ws.dim == o_dim and xs.kind == "R":
                kinds.append(("out", ws))
            elif xs.kind == "S" and xs.dim == 1 and (ws.kind == "R" or (ws.dim == i_dim and ws.counts == xs.counts and ws.striped == xs.striped)):
                kinds.append(("in", xs))
            elif xs.kind == "S" and xs.dim == 0 and ws.kind == "R":
                kinds.append(("batch", xs))
            elif xs.kind == "R" and ws.kind == "R":
                kinds.append((None, None))
            else:
                return False
        if not any(k in ("out", "in") for k, _ in kinds):
            return False                                   # nothing of this rule's: batch cuts have their own
        return kinds

    def attention_operator(self, node, tnames, backward: bool = False) -> bool:
        """``mesh::attention`` and its backward (``compiler/attention_op.py``).  Samples and heads are independent: a
        cut there (the same on every operand, the key / value heads following the query heads' groups) is local.
        Queries cut along the sequence stay cut: every processor attends its queries to all keys and values (gathered
        if they were cut) and states where its queries sit in the whole sequence; in the backward the query gradient is
        cut the same way and the key / value gradients are partial sums over the processors' queries.  An axis on
        which everything is whole on one coordinate (a pipeline stage) runs there."""
        from .attention_op import BACKWARD
        off = 1 if backward else 0
        q, k, v = tnames[off], tnames[off + 1], tnames[off + 2]
        rows = [tnames[0], tnames[4], tnames[5]] if backward else []      # grad, out, lse: laid out like the queries
        qs, ks = self.shape[q], self.shape[k]
        group = qs[1] // ks[1] if ks[1] else 1
        causal = node.args[6 if backward else 3]
        wants = {n: [] for n in tnames}
        like_q, like_kv, outs = [], [], []
        meta = {}
        for ax in range(self.na):
            specs = [self.spec[n][ax] for n in tnames]
            owned = self._owned(specs)
            sq, sk = self.spec[q][ax], self.spec[k][ax]
            cut = next((s for s in specs if s.kind == "S"), None)
            if owned is not None:
                like_q.append(owned); like_kv.append(owned); outs.append((owned, owned, owned))
            elif cut is None:
                like_q.append(R); like_kv.append(R); outs.append((R, R, R))
            elif sq.kind == "S" and sq.dim == 2 and "rows" not in meta and len({q, k, v}) == 3 and (
                    not sq.striped or len(set(sq.counts)) == 1) and (not causal or qs[2] == ks[2]):
                like_q.append(Spec("S", 2, sq.counts, sq.striped)); like_kv.append(R)
                outs.append((like_q[-1], P(), P()))
                meta["rows"] = ax
            elif cut.kind == "S" and cut.dim == 0 and not cut.striped:
                like_q.append(Spec("S", 0, cut.counts)); like_kv.append(like_q[-1]); outs.append((like_q[-1],) * 3)
            elif sq.kind == "S" and sq.dim == 1 and not sq.striped and all(c % group == 0 for c in sq.counts):
                like_q.append(Spec("S", 1, sq.counts)); like_kv.append(Spec("S", 1, tuple(c // group for c in sq.counts)))
                outs.append((like_q[-1], like_kv[-1], like_kv[-1]))
            elif sq.kind == "R" and sk.kind == "S" and sk.dim == 1 and not sk.striped:
                like_kv.append(Spec("S", 1, sk.counts)); like_q.append(Spec("S", 1, tuple(c * group for c in sk.counts)))
                outs.append((like_q[-1], like_kv[-1], like_kv[-1]))
            else:
                like_q.append(R); like_kv.append(R); outs.append((R, R, R))
        new_names = {}
        for arg, n in zip([a for a in node.args if _is_tensor_node(a)], tnames):
            spec = tuple(like_kv) if n in (k, v) and n not in (q,) else tuple(like_q)
            if n in rows and n == tnames[5]:
                spec = tuple(like_q)                         # lse [batch, heads, queries]: the same three leading dimensions
            new_names[arg.name] = self.reshard(n, spec)
        meta["full_shape"] = ()
        if causal and "rows" in meta:
            meta["query_rows"] = (meta["rows"], like_q[meta["rows"]], 8 if backward else 5, qs[2])
        meta.pop("rows", None)
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names), self.ref_kwargs(node.kwargs), meta))
        self.spec[node.name] = self.all_r()
        n_out = 3 if backward else 2
        for j in range(n_out):
            if backward:
                sp = tuple(o[j] for o in outs)
            else:
                sp = tuple(like_q)                           # out and lse follow the queries
            self.spec[(node.name, j)] = sp
        return True

    def channel_norm(self, node, tnames) -> bool:
        """Batch norm (every variant, forward and backward) over an input cut along its channels: channels are normalised
        independently, so every processor works on its own with the matching slices of the per-channel vectors, and
        the per-channel results come out cut the same way.  Instance norm reaches this rule as a batch norm over
        ``[1, samples * channels, ...]`` when the samples are cut."""
        layout = _CHANNEL_NORMS[node.target]
        names = [self.renamed.get(a.name, a.name) if _is_tensor_node(a) else None for a in node.args[: layout["tensors"]]]
        full = [names[i] for i in layout["full"]]
        x = full[0]
        if len(self.shape[x]) < 2:
            return False
        wants = {n: [] for n in names if n is not None}
        big, small = [], []
        found = False
        for a in range(self.na):
            sp = self.spec[x][a]
            others = [self.spec[n][a] for n in names if n is not None and n != x]
            if sp.kind == "S" and sp.dim == 1 and all(o.kind in ("R", "S") for o in others):
                found = True
                big.append(Spec("S", 1, sp.counts, sp.striped)); small.append(Spec("S", 0, sp.counts, sp.striped))
            elif sp.kind == "R" and all(o.kind == "R" for o in others):
                big.append(R); small.append(R)
            else:
                return False
            for i, n in enumerate(names):
                if n is not None and len(wants[n]) <= a:
                    wants[n].append(big[-1] if i in layout["full"] else small[-1])
        if not found:
            return False
        new_names = {}
        for arg, n in zip(node.args[: layout["tensors"]], names):
            if n is not None:
                new_names[arg.name] = self.reshard(n, tuple(wants[n]))
        val = node.meta["val"]
        for j, v in enumerate(val):
            if v is None:
                continue
            kind = layout["outs"][j]
            sp = tuple(big) if kind == "full" else tuple(small) if (kind == "vector" and v.numel()) else self.all_r()
            self.spec[(node.name, j)] = sp
        self.spec[node.name] = self.all_r()
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names),
                               self.ref_kwargs(node.kwargs, new_names), {"out_specs": tuple(big), "full_shape": tuple(self.shape[x])}))
        return True

    def depthwise_convolution(self, node, tnames, backward: bool = False) -> bool:
        """A convolution with one group per input channel, cut along the channels: the groups are independent, so every
        processor convolves its channels with its rows of the weight; the number of groups it passes is the number of
        channels it holds."""
        args = list(node.args)
        off = 1 if backward else 0
        transposed, groups = args[6 + off], args[8 + off]
        x, w = tnames[off], tnames[1 + off]
        cin = self.shape[x][1]
        if transposed or groups != cin or groups == 1 or self.shape[w][1] != 1 or self.shape[w][0] % cin:
            return False
        mult = self.shape[w][0] // cin
        others = tnames[:off] + tnames[2 + off:]
        xs_, ws_, found = [], [], None
        for a in range(self.na):
            sp, wsp = self.spec[x][a], self.spec[w][a]
            if sp.kind == "S" and sp.dim == 1 and not sp.striped and wsp.kind in ("R", "S"):
                if found is not None:
                    return False
                found = (a, tuple(sp.counts))
                xs_.append(sp); ws_.append(Spec("S", 0, tuple(c * mult for c in sp.counts)))
            elif sp.kind == "S" and sp.dim == 0 and wsp.kind == "R":
                xs_.append(sp); ws_.append(R)
            elif sp.kind == "R" and wsp.kind == "R":
                xs_.append(R); ws_.append(R)
            else:
                return False
        if found is None or any(self.spec[n][a].kind not in ("R", "S", "P") for n in others for a in range(self.na)):
            return False
        outs_ = tuple(Spec("S", 1, s.counts) if (s.kind == "S" and s.dim == 0 and a == found[0]) else x_ for a, (s, x_) in enumerate(zip(ws_, xs_)))
        new_names = {node.args[off].name: self.reshard(x, tuple(xs_)), node.args[1 + off].name: self.reshard(w, tuple(ws_))}
        meta = {"groups_local": (8 + off, found[0], found[1]), "full_shape": _shape(node) if not backward else ()}
        if not backward:
            if len(tnames) > 2:
                new_names[node.args[2].name] = self.reshard(tnames[2], tuple(s if s.kind == "S" and s.dim == 0 and a == found[0] else R for a, s in enumerate(ws_)))
            self.spec[node.name] = outs_
            meta["out_specs"] = outs_
            self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names), self.ref_kwargs(node.kwargs), meta))
            want = self.wanted(node.name)
            if want is not None and want != outs_:
                self.renamed[node.name] = self.reshard(node.name, want)
            return True
        mask = list(args[10])
        new_names[node.args[0].name] = self.reshard(tnames[0], outs_)
        if args[3] is not None:
            meta["bias_sizes"] = (found[0], tuple(c * mult for c in found[1]))
        raw = self.fresh(node.name)
        self.steps.append(Step("call", raw, node.target, self.ref_args(node.args, new_names), self.ref_kwargs(node.kwargs), meta))
        vec = tuple(s if (s.kind == "S" and a == found[0]) else (P() if xs_[a].kind == "S" else R) for a, s in enumerate(ws_))
        items = []
        for j, sp in enumerate((tuple(xs_), vec, vec)):
            if not mask[j]:
                items.append(None)
                continue
            item = self.fresh(f"{node.name}_{j}")
            self.steps.append(Step("call", item, operator.getitem, (Ref(raw), j)))
            v = node.meta["val"][j]
            self.shape[item], self.dtype[item] = tuple(v.shape), v.dtype
            self.spec[item] = sp
            self.spec[(node.name, j)] = sp
            items.append(item)
        self.spec[node.name] = self.all_r()
        self.shape[node.name] = ()
        self.steps.append(Step("call", node.name, pack, tuple(Ref(it) if it is not None else None for it in items)))
        return True

    def channel_convolution(self, node, tnames) -> bool:
        """A convolution (or transposed convolution) without groups whose channels are cut.  Output channels cut on the
        weight: every processor computes its own output channels from the whole input (the bias is cut the same way).
        Input channels cut: every processor convolves its channels with the matching slice of the weight and the
        results are partial sums, the bias entering through the first processor of the axis only.  The convolution analogue of column- and row-parallel
        linear layers (the reference derives both from the contraction labels of its rules,
        compiler/mesh_compiler/placement.py:503-517)."""
        args = list(node.args)
        transposed, groups = args[6], args[8]
        if groups != 1:
            return False
        x, w = tnames[0], tnames[1]
        b = tnames[2] if len(tnames) > 2 else None
        kinds = self._channel_axes(x, w, transposed)
        if not kinds:
            return False
        if b is not None and any(sp.kind not in ("R", "S") for sp in self.spec[b]):
            return False
        o_dim, i_dim = (1, 0) if transposed else (0, 1)
        xw, ww, bw, out = [], [], [], []
        for k, sp in kinds:
            if k == "out":
                xw.append(R); ww.append(Spec("S", o_dim, sp.counts, sp.striped)); bw.append(Spec("S", 0, sp.counts, sp.striped))
                out.append(Spec("S", 1, sp.counts, sp.striped))
            elif k == "in":
                xw.append(sp); ww.append(Spec("S", i_dim, sp.counts, sp.striped)); bw.append(R); out.append(P())
            elif k == "batch":
                xw.append(sp); ww.append(R); bw.append(R); out.append(sp)
            else:
                xw.append(R); ww.append(R); bw.append(R); out.append(R)
        new_names = {node.args[0].name: self.reshard(x, tuple(xw)), node.args[1].name: self.reshard(w, tuple(ww))}
        meta = {"out_specs": tuple(out), "full_shape": _shape(node)}
        if b is not None:
            new_names[node.args[2].name] = self.reshard(b, tuple(bw))
            summed = [a for a, o in enumerate(out) if o.kind == "P"]
            if summed:
                meta["once"] = (2, summed)                 # the first processor of a summed axis brings the bias
        self.spec[node.name] = tuple(out)
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names), self.ref_kwargs(node.kwargs), meta))
        want = self.wanted(node.name)
        if want is not None and want != self.spec[node.name]:
            self.renamed[node.name] = self.reshard(node.name, want)
        return True

    def channel_convolution_backward(self, node, tnames) -> bool:
        """The backward of :meth:`channel_convolution`.  Output channels cut: the incoming gradient is cut along its
        channels, the weight and bias gradients come out cut the same way, and the input gradient is a partial sum
        over the output channels.  Input channels cut: the incoming gradient is whole, the input and weight gradients
        are cut along the input channels, and every processor computes the same bias gradient."""
        args = list(node.args)
        transposed, groups, mask = args[7], args[9], list(args[10])
        if groups != 1:
            return False
        g, x, w = tnames[0], tnames[1], tnames[2]
        kinds = self._channel_axes(x, w, transposed)
        if not kinds or any(sp.kind not in ("R", "S", "P") for sp in self.spec[g]):
            return False
        o_dim, i_dim = (1, 0) if transposed else (0, 1)
        gw, xw, ww, dx, dw, db = [], [], [], [], [], []
        local_bias = None
        for a, (k, sp) in enumerate(kinds):
            if k == "out":
                gw.append(Spec("S", 1, sp.counts, sp.striped)); xw.append(R); ww.append(Spec("S", o_dim, sp.counts, sp.striped))
                dx.append(P()); dw.append(Spec("S", o_dim, sp.counts, sp.striped)); db.append(Spec("S", 0, sp.counts, sp.striped))
                local_bias = (a, tuple(sp.counts))
            elif k == "in":
                gw.append(R); xw.append(sp); ww.append(Spec("S", i_dim, sp.counts, sp.striped))
                dx.append(sp); dw.append(Spec("S", i_dim, sp.counts, sp.striped)); db.append(R)
            elif k == "batch":
                gw.append(sp); xw.append(sp); ww.append(R); dx.append(sp); dw.append(P()); db.append(P())
            else:
                gw.append(R); xw.append(R); ww.append(R); dx.append(R); dw.append(R); db.append(R)
        new_names = {node.args[0].name: self.reshard(g, tuple(gw)), node.args[1].name: self.reshard(x, tuple(xw)),
                     node.args[2].name: self.reshard(w, tuple(ww))}
        raw = self.fresh(node.name)
        meta = {"full_shape": ()}
        if local_bias is not None and args[3] is not None:
            meta["bias_sizes"] = local_bias                # the bias extent argument: this processor's channels
        self.steps.append(Step("call", raw, node.target, self.ref_args(node.args, new_names), self.ref_kwargs(node.kwargs), meta))
        items = []
        for j, sp in enumerate((dx, dw, db)):
            if not mask[j]:
                items.append(None)
                continue
            item = self.fresh(f"{node.name}_{j}")
            self.steps.append(Step("call", item, operator.getitem, (Ref(raw), j)))
            val = node.meta["val"][j]
            self.shape[item], self.dtype[item] = tuple(val.shape), val.dtype
            self.spec[item] = tuple(sp)
            self.spec[(node.name, j)] = tuple(sp)
            items.append(item)
        self.spec[node.name] = self.all_r()
        self.shape[node.name] = ()
        self.steps.append(Step("call", node.name, pack, tuple(Ref(it) if it is not None else None for it in items)))
        return True

    def patch_transposed_convolution(self, node, tnames, backward: bool = False) -> bool:
        """A transposed convolution whose windows do not overlap along a cut spatial dimension (stride = kernel there, no
        padding, dilation or output padding: the usual learned upsampling): every input row makes ``stride`` output rows
        of its own, so each processor works on its block alone and the output is cut at the same places times the
        stride.  In the backward the weight and bias gradients are partial sums."""
        off = 1 if backward else 0
        args = list(node.args)
        stride, padding, dilation, transposed, out_pad = args[3 + off], args[4 + off], args[5 + off], args[6 + off], args[7 + off]
        x, w = tnames[off], tnames[1 + off]
        if not transposed or any(self.spec[n][a].kind != "R" for n in tnames[1 + off:] for a in range(self.na)):
            return False
        cut, batch = self._spatial_cut(x)
        if cut is None:
            return False
        ax, sp = cut
        i = sp.dim - 2
        if self.shape[w][sp.dim] != stride[i] or padding[i] or dilation[i] != 1 or out_pad[i]:
            return False
        big = tuple(Spec("S", sp.dim, tuple(c * stride[i] for c in sp.counts)) if a == ax else batch.get(a, R) for a in range(self.na))
        like_input = tuple(Spec("S", sp.dim, sp.counts) if a == ax else batch.get(a, R) for a in range(self.na))
        if not backward:
            self.spec[node.name] = big
            self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args), self.ref_kwargs(node.kwargs),
                                   {"out_specs": big, "full_shape": _shape(node)}))
            want = self.wanted(node.name)
            if want is not None and want != big:
                self.renamed[node.name] = self.reshard(node.name, want)
            return True
        g = tnames[0]
        mask = list(args[10])
        new_names = {node.args[0].name: self.reshard(g, big)}
        raw = self.fresh(node.name)
        self.steps.append(Step("call", raw, node.target, self.ref_args(node.args, new_names), self.ref_kwargs(node.kwargs), {"full_shape": ()}))
        partial = tuple(P() if (a == ax or a in batch) else R for a in range(self.na))
        items = []
        for j in range(3):
            if not mask[j]:
                items.append(None)
                continue
            item = self.fresh(f"{node.name}_{j}")
            self.steps.append(Step("call", item, operator.getitem, (Ref(raw), j)))
            val = node.meta["val"][j]
            self.shape[item], self.dtype[item] = tuple(val.shape), val.dtype
            self.spec[item] = self.spec[(node.name, j)] = like_input if j == 0 else partial
            items.append(item)
        self.spec[node.name] = self.all_r()
        self.shape[node.name] = ()
        self.steps.append(Step("call", node.name, pack, tuple(Ref(it) if it is not None else None for it in items)))
        return True

    def halo_convolution_backward(self, node, tnames) -> bool:
        """The backward of :meth:`halo_convolution`.  Every processor differentiates the convolution of its own extended
        block: the weight and bias gradients are partial sums; the gradient with respect to the extended block has
        rows that belong to the neighbours, which the adjoint of the halo exchange sends back and adds."""
        args = list(node.args)
        g, x, w = tnames[0], tnames[1], tnames[2]
        stride, padding, dilation, transposed, groups, mask = args[4], list(args[5]), args[6], args[7], args[9], list(args[10])
        if transposed or any(self.spec[w][a].kind != "R" for a in range(self.na)):
            return False
        cut, batch = self._spatial_cut(x)
        if cut is None:
            return False
        ax, sp = cut
        i = sp.dim - 2
        k = self.shape[w][sp.dim]
        reach = dilation[i] * (k - 1)
        halo = self._halo_extent(self.shape[x][sp.dim], self.shape[g][sp.dim], sp.counts, stride[i], padding[i], reach)
        if halo is None:
            return False
        left, right = halo
        small = tuple(c // stride[i] for c in sp.counts)
        same = tuple(Spec("S", sp.dim, small) if a == ax else batch.get(a, R) for a in range(self.na))
        g_local = self.reshard(g, same)
        x_ext = x
        if left + right:
            x_ext = self.extended.get((x, left, right)) or self._halo_step(x, ax, sp, left, right)
            self.extended[(x, left, right)] = x_ext
        padding[i] = 0
        new_args = list(self.ref_args(node.args, {node.args[0].name: g_local, node.args[1].name: x_ext}))
        new_args[5] = padding
        raw = self.fresh(node.name)
        self.steps.append(Step("call", raw, node.target, tuple(new_args), self.ref_kwargs(node.kwargs),
                               {"halo": (left, right), "full_shape": ()}))
        partial = tuple(P() if (a == ax or a in batch) else R for a in range(self.na))     # sums over rows and samples
        like_input = tuple(Spec("S", sp.dim, sp.counts) if a == ax else batch.get(a, R) for a in range(self.na))
        items = []
        for j in range(3):
            if not mask[j]:
                items.append(None)
                continue
            item = self.fresh(f"{node.name}_{j}")
            self.steps.append(Step("call", item, operator.getitem, (Ref(raw), j)))
            val = node.meta["val"][j]
            self.shape[item], self.dtype[item] = tuple(val.shape), val.dtype
            self.spec[item] = like_input if j == 0 else partial
            if j == 0 and left + right:
                self.shape[item] = self.shape[x]
                if x in self.dtype:
                    self.dtype[item] = self.dtype[x]
                item = self._halo_step(item, ax, sp, left, right, "halo_back")
            items.append(item)
            self.spec[(node.name, j)] = like_input if j == 0 else partial
        self.spec[node.name] = self.all_r()
        self.shape[node.name] = ()
        self.steps.append(Step("call", node.name, pack, tuple(Ref(it) if it is not None else None for it in items)))
        return True

    def fallback(self, node, tnames, list_args):
        """Rule miss: gather every tensor input and run the op replicated."""
        new_names = {}
        gathered = 0                               # operands that were not whole everywhere: each costs a transfer

        # an axis along which every operand is whole on one coordinate (or everywhere) stays that way: the operator
        # runs on that coordinate; only cut and partial operands are made whole
        every = [self.spec.get(self.renamed.get(x.name, x.name)) for x in
                 [a for a in node.args if _is_tensor_node(a)] + [x for la in list_args for x in la if _is_tensor_node(x)] +
                 [v for v in node.kwargs.values() if _is_tensor_node(v)]]
        every = [sp for sp in every if sp is not None and len(sp) == self.na]
        target = tuple((self._owned([sp[a] for sp in every]) or R) if every else R for a in range(self.na))

        def whole(x):
            nonlocal gathered
            src = self.renamed.get(x.name, x.name)
            gathered += any(s.kind == "S" for s in self.spec.get(src, ()))       # (summing a partial operand is no loss)
            new_names[x.name] = self.reshard(src, target)
        for a in node.args:
            if _is_tensor_node(a):
                whole(a)
        for la in list_args:
            for x in la:
                if _is_tensor_node(x):
                    whole(x)
        for v in node.kwargs.values():
            if _is_tensor_node(v):
                whole(v)
        self.steps.append(Step("call", node.name, node.target, self.ref_args(node.args, new_names),
                               self.ref_kwargs(node.kwargs, new_names), {"fallback": True, "gathered": gathered}))
        self.spec[node.name] = target

    def ref_args(self, args, rename=None):
        rename = rename or {}

        def conv(a):
            if isinstance(a, torch.fx.Node):
                return Ref(rename.get(a.name, self.renamed.get(a.name, a.name)))
            if isinstance(a, (list, tuple)):
                return type(a)(conv(x) for x in a)
            return a
        return tuple(conv(a) for a in args)

    def ref_kwargs(self, kwargs, rename=None):
        rename = rename or {}
        return {k: (Ref(rename.get(v.name, self.renamed.get(v.name, v.name))) if isinstance(v, torch.fx.Node) else v) for k, v in kwargs.items()}


# ----------------------------------------------------------------------------- the public stage
def normalise(stated, node, mesh: Mesh, names_to_axis) -> tuple | None:
    """Turn what the placement callable returned for ``node`` into per-axis Specs."""
    if stated is None:
        return None
    na = len(mesh.shape)
    if isinstance(stated, str):
        rank = mesh.names.index(stated)
        co = mesh.coords(rank)
        return tuple(O(co[a]) for a in range(na))
    dim, procs, units = stated
    shape = _shape(node)
    if isinstance(dim, (tuple, list)):
        dims = list(dim)
        units_l = list(units) if isinstance(units, (tuple, list)) and len(units) == len(dims) and not all(
            isinstance(u, (int, float)) for u in units) else [units] * len(dims)
        specs = [R] * na
        for a, (d, u) in enumerate(zip(dims, units_l)):
            if d is None:
                continue
            if d is Ellipsis:                              # this axis is left to propagation
                specs[a] = None
                continue
            if isinstance(d, str):                         # "@k": whole on coordinate k of this axis (a pipeline stage)
                if not d.startswith("@"):
                    raise ValueError(f"placement of {node.name}: {d!r} is neither a dimension nor '@coordinate'")
                k = int(d[1:])
                if not 0 <= k < mesh.shape[a]:
                    raise ValueError(f"placement of {node.name}: coordinate {k} is outside axis {a} of the grid")
                specs[a] = O(k)
                continue
            d = d % len(shape)
            c = counts(shape[d], u, mesh.shape[a])
            specs[a] = Spec("S", d, tuple(c), u == "striped")
        return tuple(specs)
    procs = tuple(procs)
    axis = names_to_axis(procs)
    d = dim % len(shape)
    c = counts(shape[d], units, len(procs))
    specs = [R] * na
    specs[axis] = Spec("S", d, tuple(c), units == "striped")
    return tuple(specs)


def _walk_refs(obj, out: list) -> None:
    if isinstance(obj, Ref):
        out.append(obj.name)
    elif isinstance(obj, (list, tuple)):
        for o in obj:
            _walk_refs(o, out)
    elif isinstance(obj, dict):
        for o in obj.values():
            _walk_refs(o, out)


def _map_refs(obj, fn):
    if isinstance(obj, Ref):
        return Ref(fn(obj.name))
    if isinstance(obj, (list, tuple)):
        return type(obj)(_map_refs(o, fn) for o in obj)
    if isinstance(obj, dict):
        return {k: _map_refs(v, fn) for k, v in obj.items()}
    return obj


def place(exported, processors: dict, placement: Callable, mesh_shape: tuple | None = None) -> Plan:
    """Propagate the stated placements through the exported graph and insert collectives."""
    names = tuple(processors)
    mesh = Mesh(names, tuple(mesh_shape) if mesh_shape else (len(names),))
    if math.prod(mesh.shape) != len(names):
        raise ValueError("mesh shape does not match the number of processors")

    def names_to_axis(procs: tuple) -> int:
        ranks = tuple(names.index(p) for p in procs)
        for a in range(len(mesh.shape)):
            if any(ranks == mesh.axis_group(r, a) for r in ranks):
                return a
        if len(ranks) == len(names):
            return 0
        raise ValueError(f"processors {procs} are not a line of the mesh")

    stated = {}
    gm = exported.graph_module
    out_node = None
    for node in gm.graph.nodes:
        if node.op == "output":
            out_node = node
            continue
        if node.op in ("placeholder", "call_function", "get_attr") and node.target is not operator.getitem:
            if not isinstance(node.meta.get("val"), torch.Tensor):
                continue
            sp = normalise(placement(node), node, mesh, names_to_axis)
            if sp is not None:
                cut = [s.dim for s in sp if s is not None and s.kind == "S"]
                if len(cut) != len(set(cut)):
                    raise ValueError(f"placement of {node.name}: dimension {cut[0]} is cut along more than one axis of "
                                     f"the processor grid; cut it once, over the processors of both axes as one line")
                stated[node.name] = sp
    # gradients land where their parameter lives (sharded parameters get reduce-scattered gradients)
    if out_node is not None:
        flat = out_node.args[0] if isinstance(out_node.args[0], (tuple, list)) else (out_node.args[0],)
        by_target = {qual: ph for ph, (qual, _) in exported.state.items()}
        for i, (kind, target) in enumerate(exported.outputs):
            if kind == "grad_param" and target in by_target and by_target[target] in stated:
                stated[("output", i)] = stated[by_target[target]]
            elif kind == "grad_input" and target in stated:
                stated[("output", i)] = stated[target]
    order = [n.name for n in gm.graph.nodes if n.op == "placeholder"]
    prop = Propagator(gm, mesh, stated)
    plan = prop.run(order)
    plan.duplicated = getattr(prop, "duplicated", 0)
    # stated placements on intermediate nodes are constraints: applied by resharding right after the node
    return plan
