"""Lowering pass: pairs of (collective, matmul) in a plan become single fused steps.

The placement stage emits the textbook schedule of a tensor-parallel layer over sequence-sharded activations
(compiler/mesh_compiler/placement.py:250-340, :812-834 in the reference): an all-gather of the activations, then the
column-parallel matmul; the row-parallel matmul, then a reduce-scatter of its partial sums.  On the B200 each pair is
one kernel (``mesh_b200/parallel/fused_linear.py``: the transfer runs tile by tile under the tensor-core work), so this
pass rewrites

    X_full = all_gather(X_shard); [view]; Y = mm(X_full, W_t)          ->   Y = fused ag_mm(X_shard, W_t)
    P = mm(H, W_t); [view]; Y_shard = reduce_scatter(P)                ->   Y_shard = fused mm_rs(H, W_t)

when the sharded dimension is the leading one of the flattened operand (rows of rank r are consecutive), the cut is
equal and contiguous, and the intermediate values have no other consumer.  A fused step carries everything the
unfused pair carried, so an executor without the kernels (CPU ranks, odd shapes) runs the pair as before; the report
says how many pairs were found, which is also what the structure tests check.
"""
from __future__ import annotations

import copy
import math

import torch

from .ir import Plan, Ref, Step

aten = torch.ops.aten
_VIEWS = (aten.view.default, aten._unsafe_view.default, aten.reshape.default)


def _uses(plan: Plan) -> dict[str, list[int]]:
    uses: dict[str, list[int]] = {}

    def walk(obj, i):
        if isinstance(obj, Ref):
            uses.setdefault(obj.name, []).append(i)
        elif isinstance(obj, (tuple, list)):
            for o in obj:
                walk(o, i)
        elif isinstance(obj, dict):
            for o in obj.values():
                walk(o, i)
    for i, st in enumerate(plan.steps):
        walk(st.args, i)
        walk(st.kwargs, i)
    for o in plan.outputs:
        if isinstance(o, str):
            uses.setdefault(o, []).append(len(plan.steps))
    return uses


def _leading(shape, dim) -> bool:
    """Is ``dim`` the leading dimension of the flattened tensor (everything before it has size 1)?"""
    return all(s == 1 for s in shape[:dim])


def fuse_plan(plan: Plan) -> tuple[Plan, dict]:
    """Returns a rewritten copy of ``plan`` and a report ``{"ag_mm": n, "mm_rs": n}``."""
    plan = copy.copy(plan)
    steps = list(plan.steps)
    uses = _uses(plan)
    producer = {st.out: i for i, st in enumerate(steps)}
    drop: set[int] = set()
    replace: dict[int, Step] = {}
    report = {"ag_mm": 0, "mm_rs": 0}

    def single_use(name) -> int | None:
        u = uses.get(name, [])
        return u[0] if len(u) == 1 else None

    for i, st in enumerate(steps):
        # ---- all_gather -> (view) -> mm
        if st.op == "collective" and st.target == "all_gather" and i not in drop:
            frm = st.meta["from"]
            if frm.striped or len(set(frm.counts)) != 1 or not _leading(st.meta["full_shape"], frm.dim):
                continue
            j = single_use(st.out)
            chain = [i]
            cur = st.out
            while j is not None and j < len(steps) and steps[j].op == "call" and steps[j].target in _VIEWS:
                chain.append(j)
                cur = steps[j].out
                j = single_use(cur)
            keep = None
            if j is None:
                # several readers (the query, key and value projections share one gather): the first product is fused
                # and hands the gathered rows on to the others, provided every reader is a product with them on the left
                readers = sorted(set(uses.get(cur, [])))
                if readers and readers[-1] < len(steps) and all(
                        steps[r].op == "call" and steps[r].target is aten.mm.default and isinstance(steps[r].args[0], Ref)
                        and steps[r].args[0].name == cur and not (isinstance(steps[r].args[1], Ref) and steps[r].args[1].name == cur)
                        for r in readers):
                    j, keep = readers[0], cur
            if j is None or j >= len(steps):
                continue
            mm = steps[j]
            if mm.op != "call" or mm.target is not aten.mm.default or not isinstance(mm.args[0], Ref) or mm.args[0].name != cur:
                continue
            rows = int(math.prod(st.meta["full_shape"][: frm.dim + 1]))
            k = int(math.prod(st.meta["full_shape"][frm.dim + 1:]))
            meta = dict(mm.meta)
            meta.update({"fused": "ag_mm", "axis": st.meta["axis"], "from": frm, "to": st.meta["to"], "rows": rows, "k": k,
                         "gather_shape": st.meta["full_shape"], "channel": st.meta.get("channel"), "kind": st.meta.get("kind")})
            if keep is not None:
                meta["keep"] = keep                          # the executor binds the gathered rows [rows, k] to this name
            replace[j] = Step("fused", mm.out, "ag_mm", (st.args[0], mm.args[1]), {}, meta)
            drop.update(chain)
            report["ag_mm"] += 1
        # ---- mm -> (view) -> reduce_scatter
        if st.op == "call" and st.target is aten.mm.default and i not in drop and i not in replace:
            j = single_use(st.out)
            chain = []
            cur = st.out
            while j is not None and j < len(steps) and steps[j].op == "call" and steps[j].target in _VIEWS:
                chain.append(j)
                cur = steps[j].out
                j = single_use(cur)
            if j is None or j >= len(steps):
                continue
            rs = steps[j]
            if rs.op != "collective" or rs.target != "reduce_scatter" or rs.args[0].name != cur:
                continue
            to = rs.meta["to"]
            if to.striped or len(set(to.counts)) != 1 or not _leading(rs.meta["full_shape"], to.dim) or rs.meta["from"].op != "sum":
                continue
            meta = dict(rs.meta)
            meta.update({"fused": "mm_rs", "out_shape": rs.meta["full_shape"]})
            replace[j] = Step("fused", rs.out, "mm_rs", (st.args[0], st.args[1]), {}, meta)
            drop.update([i] + chain)
            report["mm_rs"] += 1
    plan.steps = [replace.get(i, st) for i, st in enumerate(steps) if i not in drop]
    return plan, report


def bucket_reductions(plan: Plan) -> tuple[Plan, int]:
    """Gradient all-reduces whose results nothing in the plan reads (they are outputs: the gradients of replicated
    parameters under a batch cut) are marked as members of one bucket per (axis, dtype); the executor holds them back
    and reduces each bucket as one flat message at the end of the step - one launch and one latency instead of one per
    parameter (the reference's planner groups transfers into demands the same way, rdma/mesh-collective.c:1791).
    Returns the rewritten copy and the number of bucketed transfers."""
    plan = copy.copy(plan)
    uses = _uses(plan)
    end = len(plan.steps)
    # which reductions travel together is the planner's decision: its demands (flat messages up to the bucket size,
    # members that exist before the group's earliest reader)
    demand_of: dict = {}
    try:
        from .schedule import planned
        demand_of = {t["channel"]: t["demand"] for t in planned(plan)["transfers"]}
    except Exception:
        demand_of = {}
    steps, count = [], 0
    for st in plan.steps:
        if (st.op == "collective" and st.target == "all_reduce" and st.meta["from"].op == "sum"
                and all(u == end for u in uses.get(st.out, []))):
            meta = dict(st.meta)
            meta["bucket"] = (st.meta["axis"], str(plan.dtypes.get(st.out, plan.dtypes.get(st.args[0].name, "float32"))),
                              demand_of.get(st.meta.get("channel"), 0))
            st = Step(st.op, st.out, st.target, st.args, st.kwargs, meta)
            count += 1
        steps.append(st)
    plan.steps = steps
    return plan, count


def fuse_ring_attention(plan: Plan) -> tuple[Plan, int]:
    """Context parallelism as a ring: attention over queries cut along the sequence whose keys and values were cut the
    same way and gathered for it,

        K = all_gather(k); V = all_gather(v); y = attention(q, K, V)      ->   y = fused ring_attention(q, k, v)

    becomes one step in which the key / value blocks travel around the processors of the axis while every processor
    attends its queries to the block it holds and merges the partial results by their running maximum and sum
    (blockwise attention with ring rotation, the reference's attention operator,
    compiler/mesh_compiler/operations.py:7081-7166).  No processor ever holds the whole keys and values; the bytes on
    the links are those of the two gathers.  A causal mask goes by the positions of the tokens in the whole sequence,
    for contiguous and striped cuts alike; a mask tensor ``[.., queries, keys]`` is read by the rows this processor holds
    and the columns of the block at hand; a block that a causal mask hides entirely is skipped.  Applies when the
    gathered values have no other reader and there is no dropout."""
    sdpa = aten.scaled_dot_product_attention.default
    plan = copy.copy(plan)
    steps = list(plan.steps)
    uses = _uses(plan)
    producer = {st.out: i for i, st in enumerate(steps)}
    drop: set[int] = set()
    replace: dict[int, Step] = {}
    count = 0
    for i, st in enumerate(steps):
        if st.op != "call" or st.target is not sdpa or "out_specs" not in st.meta or len(st.args) < 3:
            continue
        if not all(isinstance(a, Ref) for a in st.args[:3]):
            continue
        opt = dict(zip(("attn_mask", "dropout_p", "is_causal"), st.args[3:6]))
        opt.update(st.kwargs)
        if (opt.get("dropout_p") or 0.0) != 0.0:
            continue
        mask = opt.get("attn_mask")
        if mask is not None and not isinstance(mask, Ref):
            continue
        cut = [(ax, sp) for ax, sp in enumerate(st.meta["out_specs"]) if sp.kind == "S" and sp.dim == 2]
        if len(cut) != 1:
            continue
        ax, sp = cut[0]
        gathers = []
        for ref in st.args[1:3]:
            j = producer.get(ref.name)
            g = steps[j] if j is not None else None
            if g is None or g.op != "collective" or g.target != "all_gather" or g.meta.get("axis") != ax or j in drop:
                break
            frm = g.meta["from"]
            if frm.kind != "S" or frm.dim != 2 or tuple(frm.counts) != tuple(sp.counts) or frm.striped != sp.striped:
                break
            if uses.get(ref.name, []) != [i]:
                break
            gathers.append(j)
        if len(gathers) != 2 or gathers[0] == gathers[1]:
            continue
        kg, vg = steps[gathers[0]], steps[gathers[1]]
        meta = dict(st.meta)
        meta.update({"fused": "ring_attention", "axis": ax, "channel": kg.meta["channel"], "kind": "permute",
                     "causal": bool(opt.get("is_causal", False)) or "causal_rows" in st.meta, "scale": opt.get("scale"),
                     "enable_gqa": bool(opt.get("enable_gqa", False)), "keys": tuple(kg.meta["full_shape"]),
                     "channels": (kg.meta["channel"], vg.meta["channel"])})
        operands = (st.args[0], kg.args[0], vg.args[0]) + ((mask,) if mask is not None else ())
        meta["masked"] = mask is not None
        replace[i] = Step("fused", st.out, "ring_attention", operands, {}, meta)
        drop.update(gathers)
        count += 1
    if count:
        plan.steps = [replace.get(i, st) for i, st in enumerate(steps) if i not in drop]
    return plan, count


def fuse_norms(plan: Plan) -> tuple[Plan, int]:
    """An RMS norm is captured as the chain ``pow(x, 2) -> mean(last dim, keepdim) -> add(eps) -> rsqrt -> mul(x, .)
    [-> mul(., w)]``.  Where every link has that one reader (an inference graph: a training graph keeps the
    intermediates for the backward pass) the chain becomes one ``rms_norm`` step, which the executor runs as the RMSNorm
    kernel on bf16 CUDA operands and as the same PyTorch expression elsewhere.  The reference lowers a norm as one
    normalisation record, not as its pointwise pieces (compiler/mesh_compiler/operations.py:6671-6682).
    Returns the rewritten copy and the number of norms found."""
    plan = copy.copy(plan)
    steps = list(plan.steps)
    uses = _uses(plan)
    at = {st.out: i for i, st in enumerate(steps)}
    drop: set[int] = set()
    replace: dict[int, Step] = {}

    def only_reader(name, target):
        u = uses.get(name, [])
        if len(u) != 1 or u[0] >= len(steps):
            return None
        st = steps[u[0]]
        return u[0] if st.op == "call" and st.target in target else None

    for i, st in enumerate(steps):
        if not (st.op == "call" and st.target is aten.pow.Tensor_Scalar and st.args[1] == 2 and isinstance(st.args[0], Ref)):
            continue
        x = st.args[0]
        shape = plan.full_shapes.get(x.name)
        j = only_reader(st.out, (aten.mean.dim,))
        if j is None:
            continue
        mean = steps[j]
        dims = list(mean.args[1]) if len(mean.args) > 1 else []
        keep = (mean.args[2] if len(mean.args) > 2 else mean.kwargs.get("keepdim", False))
        if len(dims) != 1 or not keep or (dims[0] != -1 and (shape is None or dims[0] != len(shape) - 1)):
            continue
        k = only_reader(mean.out, (aten.add.Tensor, aten.add.Scalar))
        if k is None or isinstance(steps[k].args[1], Ref):
            continue
        eps = float(steps[k].args[1])
        r = only_reader(steps[k].out, (aten.rsqrt.default,))
        if r is None:
            continue
        m1 = only_reader(steps[r].out, (aten.mul.Tensor,))
        if m1 is None:
            continue
        ops = [a.name for a in steps[m1].args if isinstance(a, Ref)]
        if sorted(ops) != sorted([x.name, steps[r].out]):
            continue
        chain, last, w = [i, j, k, r], m1, None
        m2 = only_reader(steps[m1].out, (aten.mul.Tensor,))
        if m2 is not None:
            other = [a for a in steps[m2].args if isinstance(a, Ref) and a.name != steps[m1].out]
            wshape = plan.full_shapes.get(other[0].name) if other else None
            if len(other) == 1 and wshape is not None and len(wshape) == 1:
                chain.append(m1)
                last, w = m2, other[0]
        meta = dict(steps[last].meta)
        meta.update({"fused": "rms_norm", "eps": eps})
        replace[last] = Step("fused", steps[last].out, "rms_norm", (x,) if w is None else (x, w), {}, meta)
        drop.update(chain)
    plan.steps = [replace.get(i, st) for i, st in enumerate(steps) if i not in drop]
    return plan, len(replace)
