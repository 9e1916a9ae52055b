"""Running a scheduled program: ``Program(scheduled)(*args)``.

Two executors share one step interpreter:

* **distributed** — this process is one processor (one process per GPU); collectives go through the
  explicit verbs (the ``mesh`` backend's kernels on CUDA, gloo on CPU);
* **threads** — every processor runs as a thread of this process with in-process queues, which is the
  reference's eager send/recv semantics (compiler/mesh_compiler/ir.py:20-36) and serves as bring-up
  executor and oracle.

Arguments are bound by the captured signature; parameters and buffers are the caller's live tensors,
re-read on every call (compiler/mesh_compiler/runtime.py:42-44); buffer and input mutations are stored
in place into the caller's storage (runtime.py:53-58).  Every processor is handed the full tensors and
reads only the slices its placement names (placement.py:173-180).
"""
from __future__ import annotations

import math
import operator
import os
import threading
import time
from typing import Any

import torch
import torch.distributed as dist
from torch.utils import _pytree as pytree

from .ir import Mesh, Plan, Ref, Scheduled, Spec, Step, TrainingResult
from .placement import local_indices

aten = torch.ops.aten


# ----------------------------------------------------------------------------- collectives back ends
class ThreadWorld:
    """Shared state of the threads that interpret one program."""

    def __init__(self, n: int):
        self.n = n
        self.lock = threading.Lock()
        self.slots: dict[Any, dict] = {}
        self.barriers: dict[Any, threading.Barrier] = {}
        self.timeout = 120.0

    def exchange(self, key, group: tuple, rank: int, value):
        """All ranks of ``group`` deposit ``value``; returns the list in group order."""
        with self.lock:
            slot = self.slots.setdefault((key, group), {})
            bar = self.barriers.setdefault((key, group), threading.Barrier(len(group)))
        slot[rank] = value
        bar.wait(self.timeout)
        out = [slot[r] for r in group]
        bar.wait(self.timeout)
        if rank == group[0]:
            with self.lock:
                self.slots.pop((key, group), None)
                self.barriers.pop((key, group), None)
        return out


class ThreadCollectives:
    def __init__(self, world: ThreadWorld, mesh: Mesh, rank: int, device: torch.device | None = None):
        self.world, self.mesh, self.rank, self.device = world, mesh, rank, device
        self.seq: dict = {}

    def gather_all(self, t, axis):
        # exchanges are numbered per line of processors: a line that sits out a collective (its value lives on another
        # pipeline stage) must not fall out of step with the lines it shares other axes with
        g = self.mesh.axis_group(self.rank, axis)
        self.seq[g] = self.seq.get(g, 0) + 1
        parts = self.world.exchange(self.seq[g], g, self.rank, t)
        if self.device is not None:               # processors on different devices: what arrives is copied to this one
            parts = [v.to(self.device) if isinstance(v, torch.Tensor) and v.device != self.device else v for v in parts]
        return parts, g


class DistCollectives:
    """torch.distributed groups per mesh axis; a 1-D mesh uses the default group / mesh verbs."""

    _groups: dict = {}

    def __init__(self, mesh: Mesh, rank: int):
        self.mesh, self.rank = mesh, rank
        self.seq = 0
        if len(mesh.shape) > 1:
            for a in range(len(mesh.shape)):
                seen = set()
                for r in range(mesh.size):
                    g = mesh.axis_group(r, a)
                    if g in seen:
                        continue
                    seen.add(g)
                    if (mesh.shape, g) not in DistCollectives._groups:
                        DistCollectives._groups[(mesh.shape, g)] = dist.new_group(list(g))

    def group(self, axis):
        g = self.mesh.axis_group(self.rank, axis)
        if len(self.mesh.shape) == 1:
            return None, g
        return DistCollectives._groups[(self.mesh.shape, g)], g

    def gather_all(self, t, axis):
        """Generic fallback used by the uncommon verbs: all-gather of arbitrary (same-dtype) tensors."""
        grp, g = self.group(axis)
        shapes = [None] * len(g)
        dist.all_gather_object(shapes, (tuple(t.shape), t.dtype), group=grp)
        if len({(s, d) for s, d in shapes}) == 1:
            outs = [torch.empty(s, dtype=d, device=t.device) for s, d in shapes]
            dist.all_gather(outs, t.contiguous(), group=grp)
            return outs, g
        # parts of different sizes (an absent value is an empty stand-in): as bytes, padded to the longest
        sizes = [int(math.prod(s)) * torch.empty((), dtype=d).element_size() for s, d in shapes]
        longest = max(max(sizes), 1)
        mine = torch.zeros(longest, dtype=torch.uint8, device=t.device)
        raw = t.contiguous().reshape(-1).view(torch.uint8)
        mine[: raw.numel()] = raw
        bufs = [torch.empty(longest, dtype=torch.uint8, device=t.device) for _ in g]
        dist.all_gather(bufs, mine, group=grp)
        outs = [b[:n].view(d).reshape(s) if n else torch.empty(s, dtype=d, device=t.device) for b, n, (s, d) in zip(bufs, sizes, shapes)]
        return outs, g


# ----------------------------------------------------------------------------- step interpreter
class Executor:
    def __init__(self, plan: Plan, rank: int, coll, device: torch.device):
        self.plan, self.rank, self.coll, self.device = plan, rank, coll, device
        self.mesh = plan.mesh
        self.coords = self.mesh.coords(rank)
        self.dist = isinstance(coll, DistCollectives)
        # with MESH_SYNC_TRACE=1 every collective that actually runs is logged, to be compared with the compiled
        # synchronisation signature (compiler/syncmon.py)
        self.trace = [] if os.environ.get("MESH_SYNC_TRACE", "0") == "1" else None
        # with MESH_OBSERVE=1 every step is timed (device-synchronised on CUDA): what the share solver calls observed
        # costs, and what a person reads to see where a processor's time goes (compiler/observe.py)
        self.times = [] if os.environ.get("MESH_OBSERVE", "0") == "1" else None
        self.seed, self.execution = int(os.environ.get("MESH_SEED", "0")), 0        # random draws: see draw()
        from .kernels import Counter
        self.kernels = Counter()     # products / attention / norms run on this package's kernels vs on PyTorch operators
        self.engine = None           # a HostEngine when this processor is one (compiler/devices.py::is_engine)
        self.engine_report: list = []

    # ---- shards of full tensors
    def shard(self, full: torch.Tensor, specs: tuple) -> torch.Tensor | None:
        t = full
        for ax, s in enumerate(specs):
            if s.kind == "S":
                idx = local_indices(s, self.coords[ax], t.shape[s.dim])
                t = self._index(t, s.dim, idx)
            elif s.kind == "O" and s.owner != self.coords[ax]:
                return None
        return t

    @staticmethod
    def _index(t, dim, idx):
        if isinstance(idx, slice):
            if idx.step in (None, 1):
                return t.narrow(dim, idx.start, max(0, idx.stop - idx.start))
            sl = [slice(None)] * t.dim()
            sl[dim] = idx
            return t[tuple(sl)]
        return t.index_select(dim, torch.tensor(idx, device=t.device, dtype=torch.long))

    # ---- collectives
    def collective(self, step: Step, t):
        m = step.meta
        ax, frm, to, verb = m["axis"], m["from"], m["to"], step.target
        P = self.mesh.shape[ax]
        me = self.coords[ax]
        if self.trace is not None and "channel" in m:
            self.trace.append((verb, m.get("kind"), ax, m["channel"]))
        if P == 1 and verb not in ("halo", "halo_back"):
            return t
        if t is None and frm.kind != "O":
            # the value lives on another coordinate of some other axis (another pipeline stage): so it does for every
            # processor of this axis's line, and none of them takes part
            return None
        if verb == "halo":
            return self._halo(t, ax, frm.dim, m["left"], m["right"], me, P)
        if verb == "halo_back":
            return self._halo_back(t, ax, frm.dim, m["left"], m["right"], me, P)
        if self.dist:
            return self._collective_dist(verb, ax, frm, to, t, m, step.args[0].name if step.args and isinstance(step.args[0], Ref) else None)
        parts, g = self.coll.gather_all(t, ax)
        if verb == "all_reduce" or verb == "reduce":
            out = self._reduce(parts, frm.op)
            if verb == "reduce" and to.owner != me:
                return None
            return out
        if verb == "reduce_scatter":
            out = self._reduce(parts, frm.op)
            return self._index(out, to.dim, local_indices(to, me, out.shape[to.dim])).contiguous()
        if verb == "all_gather" or verb == "gather":
            if verb == "gather" and to.owner != me:
                return None
            return self._assemble(parts, frm, m["full_shape"])
        if verb == "all_to_all":
            full = self._assemble(parts, frm, m["full_shape"])
            return self._index(full, to.dim, local_indices(to, me, full.shape[to.dim])).contiguous()
        if verb == "broadcast":
            return parts[frm.owner]
        if verb == "scatter":
            full = parts[frm.owner]
            return self._index(full, to.dim, local_indices(to, me, full.shape[to.dim])).contiguous()
        if verb == "send_recv":
            return parts[frm.owner] if to.owner == me else None
        raise NotImplementedError(verb)

    def _halo(self, t, ax, dim, left, right, me, P):
        """Extend this processor's block by ``left`` rows of the previous processor's end and ``right`` rows of the
        next one's start (zeros beyond the ends of the whole tensor)."""
        def edge(src, lo, n):
            return src.narrow(dim, lo, n)
        zl = torch.zeros_like(edge(t, 0, left)) if left else None
        zr = torch.zeros_like(edge(t, 0, right)) if right else None
        if P == 1:
            got_l, got_r = zl, zr
        elif self.dist:
            grp, g = self.coll.group(ax)
            got_l, got_r = zl, zr
            ops = []
            if right and me > 0:                                 # my first rows are the previous processor's right halo
                ops.append(dist.P2POp(dist.isend, edge(t, 0, right).contiguous(), g[me - 1], group=grp))
            if left and me < P - 1:
                ops.append(dist.P2POp(dist.isend, edge(t, t.shape[dim] - left, left).contiguous(), g[me + 1], group=grp))
            if left and me > 0:
                got_l = torch.empty_like(zl)
                ops.append(dist.P2POp(dist.irecv, got_l, g[me - 1], group=grp))
            if right and me < P - 1:
                got_r = torch.empty_like(zr)
                ops.append(dist.P2POp(dist.irecv, got_r, g[me + 1], group=grp))
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
        else:
            parts, _ = self.coll.gather_all(t, ax)
            got_l = edge(parts[me - 1], parts[me - 1].shape[dim] - left, left) if (left and me > 0) else zl
            got_r = edge(parts[me + 1], 0, right) if (right and me < P - 1) else zr
        pieces = [p for p in (got_l, t, got_r) if p is not None]
        return torch.cat(pieces, dim=dim) if len(pieces) > 1 else t

    def _halo_back(self, t, ax, dim, left, right, me, P):
        """The adjoint of :meth:`_halo`: ``t`` is a gradient over this processor's extended block.  Its first ``left``
        rows belong to the previous processor's last rows and its last ``right`` rows to the next processor's first
        rows; they are sent there and added, and what the neighbours hold for this block's edges is added here."""
        rows = t.shape[dim] - left - right
        core = t.narrow(dim, left, rows).clone()
        mine_l = t.narrow(dim, 0, left) if left else None                   # for the previous processor
        mine_r = t.narrow(dim, left + rows, right) if right else None       # for the next processor
        got_prev = got_next = None
        if P > 1 and self.dist:
            grp, g = self.coll.group(ax)
            ops = []
            if left and me > 0:
                ops.append(dist.P2POp(dist.isend, mine_l.contiguous(), g[me - 1], group=grp))
            if right and me < P - 1:
                ops.append(dist.P2POp(dist.isend, mine_r.contiguous(), g[me + 1], group=grp))
            if right and me > 0:                                 # the previous processor's right halo covers my first rows
                got_prev = torch.empty_like(core.narrow(dim, 0, right))
                ops.append(dist.P2POp(dist.irecv, got_prev, g[me - 1], group=grp))
            if left and me < P - 1:
                got_next = torch.empty_like(core.narrow(dim, rows - left, left))
                ops.append(dist.P2POp(dist.irecv, got_next, g[me + 1], group=grp))
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
        elif P > 1:
            parts, _ = self.coll.gather_all(t, ax)
            if right and me > 0:
                prev = parts[me - 1]
                got_prev = prev.narrow(dim, prev.shape[dim] - right, right)
            if left and me < P - 1:
                got_next = parts[me + 1].narrow(dim, 0, left)
        if got_prev is not None:
            core.narrow(dim, 0, right).add_(got_prev)
        if got_next is not None:
            core.narrow(dim, rows - left, left).add_(got_next)
        return core

    @staticmethod
    def _reduce(parts, op):
        out = parts[0].clone()
        for p in parts[1:]:
            if op == "max":
                out = torch.maximum(out, p)
            elif op == "min":
                out = torch.minimum(out, p)
            else:
                out = out + p
        return out

    def _assemble(self, parts, spec: Spec, full_shape):
        if not spec.striped:
            return torch.cat(parts, dim=spec.dim)
        n = sum(p.shape[spec.dim] for p in parts)
        shape = list(parts[0].shape)
        shape[spec.dim] = n
        out = torch.empty(shape, dtype=parts[0].dtype, device=parts[0].device)
        for r, p in enumerate(parts):
            idx = local_indices(spec, r, n)
            sl = [slice(None)] * out.dim()
            sl[spec.dim] = idx if isinstance(idx, slice) else torch.tensor(idx, device=out.device)
            out[tuple(sl)] = p
        return out

    def _collective_dist(self, verb, ax, frm, to, t, m, step_name: str | None = None):
        from ..distributed import verbs
        grp, g = self.coll.group(ax)
        me = self.coords[ax]
        if verb == "all_reduce":
            out = t.clone()
            return verbs.all_reduce(out, frm.op, group=grp)
        if verb == "reduce_scatter" and not to.striped:
            return verbs.reduce_scatter(t, to.dim, frm.op, list(to.counts), group=grp)
        if verb == "all_gather" and not frm.striped:
            return verbs.all_gather(t, frm.dim, list(frm.counts), group=grp)
        if verb == "all_to_all" and not frm.striped and not to.striped:
            # cut along the new dim, exchange, join along the old dim
            pieces = [p.contiguous() for p in t.split(list(to.counts), dim=to.dim)]
            moved = [p.movedim(frm.dim, 0).contiguous() for p in pieces]
            # per-destination blocks have different sizes along the new dim, so exchange them as a list
            recv = [torch.empty((frm.counts[r],) + tuple(moved[me].shape[1:]), dtype=t.dtype, device=t.device) for r in range(len(g))]
            dist.all_to_all(recv, moved, group=grp)
            out = torch.cat(recv, dim=0).movedim(0, frm.dim)
            return out.contiguous()
        if verb == "broadcast":
            src = g[frm.owner]
            # the shape first: on a grid the owner may hold a block of the value (cut along other axes), which only it knows
            head = torch.zeros(9, dtype=torch.int64, device=self.device)
            if t is not None:
                head[0] = t.dim()
                head[1:1 + t.dim()] = torch.tensor(list(t.shape), dtype=torch.int64)
            dist.broadcast(head, src=src, group=grp)
            shape = [int(v) for v in head[1:1 + int(head[0])].tolist()]
            buf = t.contiguous() if t is not None else torch.empty(shape, dtype=self.plan.dtypes.get(m.get("value") or step_name or "", torch.float32), device=self.device)
            dist.broadcast(buf, src=src, group=grp)
            return buf
        if verb == "send_recv":
            # a value whole on one coordinate moves to another (a pipeline crossing): point to point, its shape first
            # (the receiver knows the whole shape, not how the other axes cut it on the sender)
            if frm.owner == to.owner:
                return t
            name = m.get("value") or (step_name or "")
            dtype = self.plan.dtypes.get(name, torch.float32)
            if me == frm.owner:
                head = torch.zeros(9, dtype=torch.int64, device=self.device)
                head[0] = t.dim()
                head[1:1 + t.dim()] = torch.tensor(list(t.shape), dtype=torch.int64)
                dist.send(head, g[to.owner], group=grp)
                dist.send(t.contiguous(), g[to.owner], group=grp)
                return None
            if me == to.owner:
                head = torch.zeros(9, dtype=torch.int64, device=self.device)
                dist.recv(head, g[frm.owner], group=grp)
                shape = [int(v) for v in head[1:1 + int(head[0])].tolist()]
                got = torch.empty(shape, dtype=dtype, device=self.device)
                dist.recv(got, g[frm.owner], group=grp)
                return got
            return None
        # uncommon verbs (striped gathers, owner moves): generic gather of the parts
        stand_in = t if t is not None else torch.empty(0, device=self.device)
        parts, _ = self.coll.gather_all(stand_in, ax)
        if verb == "reduce":
            out = self._reduce(parts, frm.op)
            return out if to.owner == me else None
        if verb == "reduce_scatter":
            out = self._reduce(parts, frm.op)
            return self._index(out, to.dim, local_indices(to, me, out.shape[to.dim])).contiguous()
        if verb in ("all_gather", "gather"):
            if verb == "gather" and to.owner != me:
                return None
            return self._assemble(parts, frm, m["full_shape"])
        if verb == "all_to_all":
            full = self._assemble(parts, frm, m["full_shape"])
            return self._index(full, to.dim, local_indices(to, me, full.shape[to.dim])).contiguous()
        if verb == "scatter":
            full = parts[frm.owner]
            return self._index(full, to.dim, local_indices(to, me, full.shape[to.dim])).contiguous()
        if verb == "send_recv":
            return parts[frm.owner] if to.owner == me else None
        raise NotImplementedError(verb)

    def _here(self, t):
        return t.to(self.device) if isinstance(t, torch.Tensor) and t.device != self.device else t

    # ---- one program execution
    def run(self, inputs: dict, consts) -> list:
        env: dict[str, Any] = {}
        pending: dict = {}
        for name, full in inputs.items():
            env[name] = self._here(self.shard(full, self.plan.input_specs[name])) if isinstance(full, torch.Tensor) else full

        def val(a):
            if isinstance(a, Ref):
                return env[a.name]
            if isinstance(a, (list, tuple)):
                return type(a)(val(x) for x in a)
            return a

        # values with a destination are computed straight into the storage of the concatenation that reads them
        from . import destine
        dest = self.__dict__.get("_destinations")
        if dest is None:
            dest = self._destinations = destine.analyse(self.plan) if destine.enabled() else {}
        parents: dict[str, dict] = {}                    # concatenation -> {"buf", "slots", "filled"} for this execution
        self.destined = 0
        for index, st in enumerate(self.plan.steps):
            if self.times is not None:
                if self.device.type == "cuda":
                    torch.cuda.synchronize(self.device)
                t0 = time.perf_counter()
            if st.out in dest and st.op == "call":
                env[st.out] = self._call_into(st, val, dest[st.out], parents)
            elif st.op == "call" and st.out in parents:
                # a concatenation all of whose pieces were written in place: its storage is the result
                rec = parents.pop(st.out)
                if rec["buf"] is not None and rec["filled"] == len(rec["slots"]):
                    env[st.out] = rec["buf"]
                    self.destined += 1
                else:
                    env[st.out] = self.call(st, val)
            elif st.op == "const":
                env[st.out] = self._here(consts(st.target))
            elif st.op == "alias":
                env[st.out] = env[st.args[0].name]
            elif st.op == "slice":
                src = env[st.args[0].name]
                s, ax = st.meta["to"], st.meta["axis"]
                env[st.out] = None if src is None else self._index(src, s.dim, local_indices(s, self.coords[ax], src.shape[s.dim]))
            elif st.op == "collective" and "bucket" in st.meta and env[st.args[0].name] is not None:
                pending.setdefault(st.meta["bucket"], []).append((st, env[st.args[0].name]))     # reduced with its bucket below
                env[st.out] = None
            elif st.op == "collective":
                env[st.out] = self.collective(st, env[st.args[0].name])
            elif st.op == "fused" and st.target == "rms_norm":
                env[st.out] = self.rms_norm(st, env[st.args[0].name], env[st.args[1].name] if len(st.args) > 1 else None)
            elif st.op == "fused":
                env[st.out] = self.fused(st, env[st.args[0].name], env[st.args[1].name], env)
            else:
                env[st.out] = self.call(st, val)
            if self.times is not None:
                if self.device.type == "cuda":
                    torch.cuda.synchronize(self.device)
                self.times.append((index, time.perf_counter() - t0))
        for members in pending.values():
            # one flat all-reduce per bucket, then every member gets its piece back
            first = members[0][0]
            flat = torch.cat([t.reshape(-1) for _, t in members])
            flat = self.collective(Step("collective", first.out, "all_reduce", first.args, {}, first.meta), flat)
            at = 0
            for st, t in members:
                env[st.out] = flat[at:at + t.numel()].view(t.shape)
                at += t.numel()
        out = []
        for o in self.plan.outputs:
            out.append(o[1] if isinstance(o, tuple) else env[o])
        return out

    def run_step(self, st: Step, env: dict, val):
        """One step that is neither a constant, an alias nor a collective, on the values in ``env`` (generated host
        programs call this for the steps they do not spell out, ``compiler/hostgen.py``)."""
        if st.op == "slice":
            src = env.get(st.args[0].name)
            s, ax = st.meta["to"], st.meta["axis"]
            return None if src is None else self._index(src, s.dim, local_indices(s, self.coords[ax], src.shape[s.dim]))
        if st.op == "fused" and st.target == "rms_norm":
            return self.rms_norm(st, env.get(st.args[0].name), env.get(st.args[1].name) if len(st.args) > 1 else None)
        if st.op == "fused":
            return self.fused(st, env.get(st.args[0].name), env.get(st.args[1].name), env)
        return self.call(st, val)

    # ---- fused (collective, matmul) pairs, see compiler/fuse.py
    def _fused_kernels(self, kind: str, a, w_t, rows_total: int):
        """The fused-kernel object for this shape, or None when the pair has to run unfused (CPU ranks, dtypes other
        than bf16, shapes the kernels do not tile, no symmetric heap in this process)."""
        if not (self.dist and a.is_cuda and a.dtype == torch.bfloat16 and w_t.dtype == torch.bfloat16):
            return None
        w = w_t.t()
        P = self.mesh.size
        if len(self.mesh.shape) != 1 or not w.is_contiguous() or rows_total % (P * 128) or w.shape[0] % 64 or w.shape[1] % 64:
            return None
        from ..distributed.context import current_or_none
        ctx = current_or_none()
        if ctx is None or ctx.world != P:
            return None
        cache = self.__dict__.setdefault("_fused_cache", {})
        key = (kind, rows_total, tuple(w.shape))
        if key not in cache:
            from ..parallel.fused_linear import FusedColumnLinear, FusedRowLinear
            cache[key] = (FusedColumnLinear(ctx.heap, rows_total, w.shape[1], w.shape[0]) if kind == "ag_mm"
                          else FusedRowLinear(ctx.heap, rows_total, w.shape[1], w.shape[0]))
        return cache[key]

    def ring_attention(self, st: Step, q, k, v, mask=None):
        """Blockwise attention with the key / value blocks rotating around the axis (``fuse.fuse_ring_attention``).
        Round ``r`` attends this processor's queries to the block that started on processor ``me - r``; partial results
        are merged by running maximum and sum (rows that have seen nothing yet carry weight zero); a causal mask
        compares positions in the whole sequence, whatever the cut.  Accumulates in fp32."""
        m = st.meta
        if q is None or k is None or v is None:
            return None
        ax = m["axis"]
        spec = m["out_specs"][ax]
        P, me = self.mesh.shape[ax], self.coords[ax]
        total = m["full_shape"][2]
        if self.trace is not None:
            self.trace.append(("ring", m.get("kind"), ax, m["channel"]))

        def positions(r):
            idx = local_indices(spec, r, total)
            if isinstance(idx, slice):
                return torch.arange(idx.start or 0, idx.stop, idx.step or 1, device=q.device)
            return torch.as_tensor(list(idx), device=q.device, dtype=torch.long)
        scale = m.get("scale")
        scale = (q.shape[-1] ** -0.5) if scale is None else scale
        qf = q.float() * scale
        group = q.shape[1] // k.shape[1] if k.shape[1] and q.shape[1] != k.shape[1] else 1
        qpos = positions(me)
        if mask is not None and mask.shape[-2] == total and total != q.shape[2]:
            mask = mask.index_select(-2, qpos)               # a whole mask: the rows of this processor's queries
        acc = torch.zeros(*q.shape[:-1], v.shape[-1], dtype=torch.float32, device=q.device)
        top = torch.full((*q.shape[:-1], 1), float("-inf"), dtype=torch.float32, device=q.device)
        den = torch.zeros_like(top)
        threads = None
        if P > 1 and not self.dist:
            threads = (self.coll.gather_all(k, ax)[0], self.coll.gather_all(v, ax)[0])
        kb, vb = k, v
        for r in range(P):
            src = (me - r) % P
            if threads is not None:
                kb, vb = threads[0][src], threads[1][src]
            hidden = bool(m.get("causal")) and kb.shape[2] and qpos.numel() and int(positions(src).min()) > int(qpos.max())
            if kb.shape[2] and not hidden:                   # (a block wholly in these queries' future adds nothing)
                kk, vv = kb.float(), vb.float()
                if group > 1:
                    kk, vv = kk.repeat_interleave(group, 1), vv.repeat_interleave(group, 1)
                s = qf @ kk.transpose(-1, -2)
                if m.get("causal"):
                    s = s.masked_fill(positions(src)[None, :] > qpos[:, None], float("-inf"))
                if mask is not None:
                    cols = mask.index_select(-1, positions(src))
                    s = s.masked_fill(cols.logical_not(), float("-inf")) if cols.dtype == torch.bool else s + cols.float()
                blk = s.amax(-1, keepdim=True)
                new = torch.maximum(top, blk)
                safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)      # rows that still see nothing
                w = torch.exp(s - safe)
                keep = torch.exp(torch.where(torch.isinf(top), torch.full_like(top, float("-inf")), top - safe))
                den = den * keep + w.sum(-1, keepdim=True)
                acc = acc * keep + w @ vv
                top = new
            if r < P - 1 and threads is None and P > 1:
                kb, vb = self._pass_on((kb, vb), ax, [list(x.shape[:2]) + [spec.counts[(src - 1) % P]] + [x.shape[3]] for x in (k, v)])
        out = acc / torch.where(den == 0, torch.ones_like(den), den)
        return out.to(q.dtype)

    def _pass_on(self, blocks, ax, shapes):
        """Send ``blocks`` to the next processor of the axis and receive, with ``shapes``, what the previous one sends."""
        grp, g = self.coll.group(ax)
        P, me = self.mesh.shape[ax], self.coords[ax]
        got = [torch.empty(sh, dtype=b.dtype, device=b.device) for sh, b in zip(shapes, blocks)]
        ops = [dist.P2POp(dist.isend, b.contiguous(), g[(me + 1) % P], group=grp) for b in blocks]
        ops += [dist.P2POp(dist.irecv, t, g[(me - 1) % P], group=grp) for t in got]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        return got

    def fused(self, st: Step, a, w_t, env=None):
        m = st.meta
        if st.target == "ring_attention":
            rest = [None if env is None else env.get(r.name) for r in st.args[2:]]
            if m.get("masked") and rest[1] is None:
                return None
            return self.ring_attention(st, a, w_t, *rest)
        if a is None or w_t is None:
            if "keep" in m and env is not None:
                env[m["keep"]] = None                        # absent here: so are the gathered rows for the other readers
            return None
        if st.target == "ag_mm":
            op = self._fused_kernels("ag_mm", a, w_t, m["rows"])
            if op is not None:
                if self.trace is not None:
                    self.trace.append(("all_gather", m.get("kind"), m["axis"], m["channel"]))
                y, xbuf = op.forward(a.reshape(-1, m["k"]).contiguous(), w_t.t())
                if "keep" in m and env is not None:
                    # other products of the same gathered rows read the kernel's landing zone; it is overwritten two
                    # uses of this shape later, by which time those products have run (stream order)
                    env[m["keep"]] = xbuf.local.view(m["rows"], m["k"])
                return y
            gathered = self.collective(Step("collective", st.out, "all_gather", (), {}, {**m, "full_shape": m["gather_shape"]}), a)
            gathered = gathered.reshape(m["rows"], m["k"])
            if "keep" in m and env is not None:
                env[m["keep"]] = gathered
            return aten.mm.default(gathered, w_t)
        if st.target == "mm_rs":
            shape = list(m["out_shape"])
            op = self._fused_kernels("mm_rs", a, w_t, a.shape[0])
            if op is not None:
                if self.trace is not None:
                    self.trace.append(("reduce_scatter", m.get("kind"), m["axis"], m["channel"]))
                y = op.forward(a.contiguous(), w_t.t())
                to = m["to"]
                shape[to.dim] = to.counts[self.coords[m["axis"]]]
                return y.reshape(shape)
            partial = aten.mm.default(a, w_t).reshape(shape)
            return self.collective(Step("collective", st.out, "reduce_scatter", (), {}, m), partial)
        raise NotImplementedError(st.target)

    def _attention_dropout(self, st: Step, opt: dict, q):
        """The kernel's dropout description for an attention step that drops probabilities, or ``None``: the draw is
        keyed by this program's seed and execution, the step's position in the plan (its site) and the logical head
        (heads cut over processors are offset); a batch cut is left to the PyTorch operator."""
        p = opt.get("dropout_p", 0.0) or 0.0
        if not p:
            return None
        m = st.meta
        head_off, heads_total = 0, q.shape[1]
        for ax, s in enumerate(m.get("out_specs", ())):
            if getattr(s, "kind", "R") == "S":
                if s.dim == 0:
                    return None
                if s.dim == 1:
                    head_off, heads_total = sum(s.counts[:self.coords[ax]]), m["full_shape"][1]
        site = m.get("site", self.plan.steps.index(st) if st in self.plan.steps else 0)
        return {"p": float(p), "seed": self.seed, "execution": self.execution, "site": int(site) & 0xFFFFFFFF,
                "head_off": head_off, "heads_total": heads_total}

    def _on_engine(self, st: Step, tgt, args):
        """A product or a sum placed on an engine processor runs as a batch of the host engine; ``None``: not an
        operation the engine has (it then runs on the PyTorch operator, on the host)."""
        ok = lambda t: isinstance(t, torch.Tensor) and not t.is_cuda and t.dtype in (torch.float32, torch.bfloat16) and t.dim() == 2
        ops = None
        if tgt is aten.mm.default and ok(args[0]) and ok(args[1]) and args[0].dtype == args[1].dtype:
            a = args[0] if args[0].stride(1) == 1 else args[0].contiguous()
            b = args[1].t() if args[1].t().stride(1) == 1 else args[1].t().contiguous()      # the engine takes B as [n, k]
            out = torch.empty((a.shape[0], b.shape[0]), dtype=a.dtype)
            ops = [("gemm_nt", a, b, out)]
        elif tgt is aten.add.Tensor and len(args) == 2 and ok(args[0]) and ok(args[1]) and args[0].shape == args[1].shape \
                and args[0].dtype == args[1].dtype:
            a, b = (t if t.stride(1) == 1 else t.contiguous() for t in args)
            out = torch.empty_like(a, memory_format=torch.contiguous_format)
            ops = [("add", a, b, out)]
        if ops is None:
            return None
        rep = self.engine.wait(self.engine.submit(ops))
        self.engine_report += [{"step": st.out, **r} for r in rep]
        return ops[0][-1]

    def rms_norm(self, st: Step, x, w):
        """One step for the operator chain of an RMS norm (``fuse.fuse_norms``)."""
        if x is None or (len(st.args) > 1 and w is None):
            return None
        if self.engine is not None and w is not None and not x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) \
                and w.dtype == x.dtype:
            x2 = x.reshape(-1, x.shape[-1]).contiguous()
            out = torch.empty_like(x2)
            rep = self.engine.wait(self.engine.submit([("rmsnorm", x2, w.contiguous(), out, float(st.meta["eps"]))]))
            self.engine_report += [{"step": st.out, **r} for r in rep]
            return out.view(x.shape)
        from . import kernels
        if kernels.enabled():
            y = kernels.rms_norm(x, w, st.meta["eps"])
            if y is not None:
                self.kernels.own += 1
                return y
        self.kernels.eager += 1
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + st.meta["eps"])
        return y if w is None else y * w

    def draw(self, m: dict, args):
        """Random numbers for the elements this processor holds, as a function of their positions in the whole tensor
        (Philox4x32-10 keyed by seed, execution and draw site; ``mesh_b200/ops/philox.py``)."""
        from ..ops import philox
        full = m["full_shape"]
        slices = [None] * len(full)
        for ax, s in enumerate(m["out_specs"]):
            if s.kind == "S":
                slices[s.dim] = local_indices(s, self.coords[ax], full[s.dim])
        e = philox.logical_index(full, slices, self.device)
        words = philox.philox4x32((e & philox.MASK, (e >> 32) & philox.MASK, torch.full_like(e, m["site"] & philox.MASK),
                                   torch.full_like(e, self.execution & philox.MASK)),
                                  (self.seed & philox.MASK, (self.seed >> 32) & philox.MASK))
        u = (words[0] >> 8).to(torch.float32) * (1.0 / (1 << 24))                      # [0, 1)
        dtype = m.get("dtype", torch.float32)
        if m["draw"] == "uniform":
            return u.to(dtype)
        if m["draw"] == "normal":                                                       # Box-Muller from two words
            v = (words[1] >> 8).to(torch.float32) * (1.0 / (1 << 24))
            return (torch.sqrt(-2.0 * torch.log1p(-u)) * torch.cos(2 * math.pi * v)).to(dtype)
        x, p = args[0], float(args[1])
        train = args[2] if len(args) > 2 else True
        if train is False or p <= 0:
            return x, torch.ones_like(x, dtype=torch.bool)
        keep = u >= p
        return torch.where(keep, x / (1 - p), torch.zeros((), dtype=x.dtype, device=x.device)), keep

    def _call_into(self, st: Step, val, d, parents: dict):
        """Run a pointwise step whose result is piece ``d.position`` of the concatenation ``d.parent``: the parent's
        storage is laid out when its first piece arrives (every piece's local shape follows from the cut recorded for
        it), and the step writes into its slice through the operator's ``out=`` form.  Whatever does not fit (an operand
        on another processor, a shape that differs from the recorded one) falls back to the plain call, and the
        concatenation then runs as usual."""
        from . import destine
        rec = parents.get(d.parent)
        if rec is None:
            rec = parents[d.parent] = {"buf": None, "slots": None, "filled": 0}
            try:
                metas = [next(s for s in self.plan.steps if s.out == name).meta for name in d.pieces]
                shapes = [destine.local_shape(m, self.coords) for m in metas]
                base = list(shapes[0])
                if all(len(sh) == len(base) and all(a == b for k, (a, b) in enumerate(zip(sh, base)) if k != d.dim) for sh in shapes):
                    base[d.dim] = sum(sh[d.dim] for sh in shapes)
                    rec["buf"] = torch.empty(base, dtype=self.plan.dtypes[d.parent], device=self.device)
                    at, slots = 0, []
                    for sh in shapes:
                        slots.append(rec["buf"].narrow(d.dim, at, sh[d.dim]))
                        at += sh[d.dim]
                    rec["slots"] = slots
            except (StopIteration, KeyError):
                rec["buf"] = None
        if rec["buf"] is None:
            return self.call(st, val)
        args = [val(a) for a in st.args]
        kwargs = {k: val(v) for k, v in st.kwargs.items()}
        if any(a is None for a, r in zip(args, st.args) if isinstance(r, Ref)):
            rec["buf"] = None
            return None
        if "device" in kwargs and kwargs["device"] is not None:
            kwargs["device"] = self.device
        view = rec["slots"][d.position]
        try:
            shape = torch.broadcast_shapes(*[tuple(a.shape) for a in args if isinstance(a, torch.Tensor)])
        except RuntimeError:
            shape = None
        if shape != tuple(view.shape):
            rec["buf"] = None                              # not the recorded shape: no destination for this parent
            return st.target(*args, **kwargs)
        st.target.overloadpacket.out(*args, **kwargs, out=view)
        rec["filled"] += 1
        return view

    def call(self, st: Step, val):
        args = list(val(a) for a in st.args)
        kwargs = {k: val(v) for k, v in st.kwargs.items()}
        if any(a is None for a, r in zip(args, st.args) if isinstance(r, Ref)):
            return None                                   # an operand lives on another processor
        if "device" in kwargs and kwargs["device"] is not None:
            kwargs["device"] = self.device
        tgt = st.target
        m = st.meta
        if "draw" in m:
            return self.draw(m, args)
        if "out_specs" in m and st.out in self.plan.dtypes and m.get("full_shape") and \
                any(isinstance(a, torch.Tensor) and a.numel() == 0 for a in args):
            # this processor's share of a cut operand is empty (more processors than rows, or a share that rounds to
            # nothing).  Operators disagree about empty operands (some refuse them, a convolution over no channels
            # returns the wrong shape), and the result is known anyway: nothing where the cut dimension stays, the
            # reduction's identity where it is summed over.
            shape = list(m["full_shape"])
            pending = None
            for ax, sp in enumerate(m["out_specs"]):
                if sp.kind == "S" and sp.dim < len(shape):
                    shape[sp.dim] = sp.counts[self.coords[ax]]
                elif sp.kind == "P":
                    pending = sp.op
            if pending is not None or 0 in shape:
                dtype = self.plan.dtypes[st.out]
                fill = 0 if pending in (None, "sum") else _identity(pending, dtype)
                return torch.full(shape, fill, dtype=dtype, device=self.device)
        if "items" in m and any(isinstance(a, torch.Tensor) and a.numel() == 0 for a in args):
            # the same for an operator with several results (a convolution's backward, a norm with its statistics, a
            # pooling with its indices): each item by its own placement
            items = [None] * (max(m["items"]) + 1)
            for j, (specs, full, dtype) in m["items"].items():
                shape, pending = list(full), None
                for ax, sp in enumerate(specs):
                    if sp.kind == "S" and sp.dim < len(shape):
                        shape[sp.dim] = sp.counts[self.coords[ax]]
                    elif sp.kind == "P":
                        pending = sp.op
                fill = 0 if pending in (None, "sum") else _identity(pending, dtype)
                items[j] = torch.full(shape, fill, dtype=dtype, device=self.device)
            return tuple(items)
        if "causal_rows" in m:
            # whole attention over this processor's query rows: row i of the whole sequence sees keys 0..i
            ax = m["causal_rows"]
            spec = m["out_specs"][ax]
            q, k = args[0], args[1]
            rows = local_indices(spec, self.coords[ax], m["full_shape"][2])
            from . import kernels
            if kernels.enabled() and isinstance(rows, slice):
                opt = dict(zip(("attn_mask", "dropout_p", "is_causal"), args[3:6]))
                opt.update(kwargs)
                y = kernels.attention(q, k, args[2], causal=True, scale=opt.get("scale"),
                                      row_positions=(rows.start or 0, rows.step or 1),
                                      dropout_p=opt.get("dropout_p", 0.0) or 0.0, mask=opt.get("attn_mask"),
                                      dropout=self._attention_dropout(st, opt, q))
                if y is not None:
                    self.kernels.own += 1
                    return y
            self.kernels.eager += 1
            pos = torch.arange(m["full_shape"][2], device=q.device)[rows] if isinstance(rows, slice) else torch.tensor(rows, device=q.device)
            mask = pos[:, None] >= torch.arange(k.shape[2], device=q.device)[None, :]
            kw = {key: v for key, v in kwargs.items() if key not in ("is_causal", "attn_mask")}
            extra = list(args[3:])
            if len(extra) > 2:
                extra[2] = False                              # positional is_causal
            if extra:
                extra[0] = mask
                return tgt(q, k, args[2], *extra, **kw)
            return tgt(q, k, args[2], attn_mask=mask, is_causal=False, **kw)
        if "query_rows" in m:
            # (grid axis, the queries' cut, position of the row arguments, queries in all): where this processor's
            # queries sit in the whole sequence - a block starts at its offset, a round-robin share at its coordinate
            ax, sp, pos, total = m["query_rows"]
            rows = local_indices(sp, self.coords[ax], total)
            if isinstance(rows, slice):
                args[pos], args[pos + 1] = rows.start or 0, rows.step or 1
            else:
                rows = list(rows)
                args[pos], args[pos + 1] = (rows[0] if rows else 0), ((rows[1] - rows[0]) if len(rows) > 1 else 1)
        if "once" in m:                                    # (argument, axes): a term every processor of those axes holds but
            pos, axes = m["once"]                           # that must enter a partial sum once - the first one brings it
            if any(self.coords[ax] != 0 for ax in axes) and isinstance(args[pos], torch.Tensor):
                args[pos] = torch.zeros_like(args[pos])
        if "groups_local" in m:                            # (argument, grid axis, channels per processor): one group per channel held
            pos, ax, counts = m["groups_local"]
            args[pos] = counts[self.coords[ax]]
        if "bias_sizes" in m:                              # (grid axis, channels per processor): this processor's extent
            ax, counts = m["bias_sizes"]
            args[3] = [counts[self.coords[ax]]]
        if "batch_arg" in m:
            args[m["batch_arg"]] = args[0].shape[0]        # the operator takes the batch size as a number: this shard's
        loc = m.get("localize")
        if loc is not None and "out_specs" in m:
            i = loc[1]
            shape = list(args[i])
            full = m["full_shape"]
            for ax, s in enumerate(m["out_specs"]):
                if s.kind == "S" and len(shape) == len(full):
                    shape[s.dim] = s.counts[self.coords[ax]]
            if -1 in shape and len(shape) == len(full):
                # an inferred extent is ambiguous for an empty shard: state it (a cut dimension was set just above)
                shape = [full[k] if v == -1 else v for k, v in enumerate(shape)]
            args[i] = shape
        if "mean_as_sum" in m:
            a = list(args)
            t = a[0]
            rest = a[1:]
            r = aten.sum.dim_IntList(t, rest[0] if rest else None, *(rest[1:2] if len(rest) > 1 else []))
            if tgt is aten.mean.default:
                r = t.sum()
            return r / m["mean_as_sum"]
        if "vocab_parallel" in m:
            ax, cnts = m["vocab_parallel"]
            start = sum(cnts[:self.coords[ax]])
            w, idx = args[0], args[1]
            local = idx - start
            ok = (local >= 0) & (local < w.shape[0])
            e = aten.embedding.default(w, local.clamp(0, max(w.shape[0] - 1, 0)), *args[2:])
            return e * ok.unsqueeze(-1).to(e.dtype)
        if tgt in (aten.view.default, aten._unsafe_view.default):
            return args[0].reshape(args[1])        # shards and gathered values are not always dense
        if self.engine is not None:
            y = self._on_engine(st, tgt, args)
            if y is not None:
                return y
        # products and whole attention run on this package's kernels where the operands allow it (compiler/kernels.py)
        from . import kernels
        if kernels.enabled():
            y = None
            if tgt is aten.mm.default:
                y = kernels.mm(args[0], args[1])
            elif tgt is aten.matmul.default and args[0].dim() >= 3 and args[1].dim() == 2:
                # a linear layer whose operand keeps its leading dimensions: one product over the merged rows
                y = kernels.mm(args[0].reshape(-1, args[0].shape[-1]), args[1])
                if y is not None:
                    y = y.view(*args[0].shape[:-1], y.shape[-1])
            elif tgt is aten.scaled_dot_product_attention.default:
                # (query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None, enable_gqa=False)
                opt = dict(zip(("attn_mask", "dropout_p", "is_causal"), args[3:6]))
                opt.update(kwargs)
                y = kernels.attention(args[0], args[1], args[2], causal=bool(opt.get("is_causal", False)),
                                      scale=opt.get("scale"), dropout_p=opt.get("dropout_p", 0.0) or 0.0,
                                      mask=opt.get("attn_mask"), dropout=self._attention_dropout(st, opt, args[0]))
            if y is not None:
                self.kernels.own += 1
                return y
        if tgt in _COMPUTE:
            self.kernels.eager += 1
        return tgt(*args, **kwargs)


def _identity(op: str, dtype):
    """The value a reduction starts from: what an empty share contributes."""
    if op == "max":
        return -float("inf") if dtype.is_floating_point else (False if dtype == torch.bool else torch.iinfo(dtype).min)
    if op == "min":
        return float("inf") if dtype.is_floating_point else (True if dtype == torch.bool else torch.iinfo(dtype).max)
    return 0


# operators with a kernel of this package behind them when the operands allow it: the ones counted as "eager" when
# they run on the PyTorch operator instead
_COMPUTE = (aten.mm.default, aten.bmm.default, aten.addmm.default, aten.matmul.default,
            aten.scaled_dot_product_attention.default)


# ----------------------------------------------------------------------------- Program
class Arguments:
    """Binds call arguments to placeholders by the captured signature (runtime.py:18-50 of the reference)."""

    def __init__(self, scheduled: Scheduled):
        self.exported = scheduled.exported
        self.plan = scheduled.plan

    def prepare(self, args, kwargs) -> dict:
        ex = self.exported
        flat, spec = pytree.tree_flatten((tuple(args), dict(kwargs)))
        if spec != ex.in_spec:
            flat = list(ex.in_spec.flatten_up_to((tuple(args), dict(kwargs))))
        if len(flat) != len(ex.user_inputs):
            raise TypeError(f"expected {len(ex.user_inputs)} input leaves, got {len(flat)}")
        bound = {name: (t.detach() if isinstance(t, torch.Tensor) else t) for name, (_, t) in ex.state.items()}
        bound.update(dict(zip(ex.user_inputs, flat)))
        return bound


class Program(Arguments):
    """``Program(scheduled)(*args, **kwargs)`` -> outputs pytree | ``TrainingResult`` | ``None`` on non-owner ranks."""

    def __init__(self, scheduled: Scheduled, entry: str | None = None, device=None, threads: bool | None = None):
        super().__init__(scheduled)
        self.scheduled = scheduled
        self.fusion = {"ag_mm": 0, "mm_rs": 0}
        self.devices = None
        # random draws are a function of (seed, execution, draw site, element): every processor must use the same seed;
        # the execution number advances with every call, so that successive steps draw fresh numbers
        self.seed, self.execution = int(os.environ.get("MESH_SEED", "0")), 0
        if os.environ.get("MESH_FUSE", "1") != "0":
            from .fuse import fuse_norms, fuse_plan
            self.plan, self.fusion = fuse_plan(self.plan)
            self.plan, self.fusion["rms_norm"] = fuse_norms(self.plan)
            if os.environ.get("MESH_RING_ATTENTION", "1") != "0":
                from .fuse import fuse_ring_attention
                self.plan, self.fusion["ring_attention"] = fuse_ring_attention(self.plan)
        self.bucketed = 0
        if os.environ.get("MESH_BUCKET", "0") == "1":
            from .fuse import bucket_reductions
            self.plan, self.bucketed = bucket_reductions(self.plan)
        self.mesh = scheduled.plan.mesh
        distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size() == self.mesh.size
        self.threads = (not distributed) if threads is None else threads
        if not self.threads:
            self.rank = dist.get_rank()
            dev = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and
                             dist.get_backend() != "gloo" else torch.device("cpu"))
            self.device = torch.device(dev)
            self.exec = Executor(self.plan, self.rank, DistCollectives(self.mesh, self.rank), self.device)
        elif device == "processors":
            # every processor on the device its description names (the reference's on_devices stage); values that
            # cross are copied where they arrive
            from .devices import is_engine, on_devices
            self.devices = on_devices(scheduled.processors)
            if any(is_engine(d) for d in scheduled.processors.values()):
                from ..runtime.host_engine import HostEngine
                shared = HostEngine()
                self.engines = [shared if is_engine(d) else None for d in scheduled.processors.values()]
            self.device = self.devices[0 if entry is None else self.mesh.names.index(entry)]
        else:
            self.device = torch.device(device or "cpu")
        self.entry = entry
        self.last_structure = None
        self.engines = getattr(self, "engines", None)

    def _on_device(self, key, t: torch.Tensor) -> torch.Tensor:
        """``t`` on this program's device.  A parameter or constant that lives elsewhere is copied once and again
        only after it has been written (live parameters are re-read on every call, but not re-copied when unchanged)."""
        if t.device == self.device:
            return t
        cache = self.__dict__.setdefault("_device_copies", {})
        stamp = (t._version, t.data_ptr(), tuple(t.shape))
        hit = cache.get(key)
        if hit is None or hit[0] != stamp:
            cache[key] = hit = (stamp, t.detach().to(self.device))
        return hit[1]

    def _consts(self, target):
        gm = self.exported.graph_module
        obj = gm
        for part in str(target).split("."):
            obj = getattr(obj, part)
        return self._on_device(("const", str(target)), obj) if isinstance(obj, torch.Tensor) and not self.devices else obj

    def __call__(self, *args, **kwargs):
        bound = self.prepare(args, kwargs)
        if not self.devices:
            state = self.exported.state
            bound = {k: ((self._on_device(("state", k), v) if k in state else v.to(self.device))
                         if isinstance(v, torch.Tensor) and v.device != self.device else v) for k, v in bound.items()}
        execution, self.execution = self.execution, self.execution + 1
        if not self.threads:
            self.exec.seed, self.exec.execution = self.seed, execution
            flat = self.exec.run(bound, self._consts)
            return self._result(flat, self.exec, bound)
        world = ThreadWorld(self.mesh.size)
        results: list = [None] * self.mesh.size
        errors: list = []
        if self.mesh.size == 1:
            # one processor: run in the calling thread (its current stream, and a CUDA-graph capture if one is open)
            dev = self.devices[0] if self.devices else self.device
            ex = Executor(self.plan, 0, ThreadCollectives(world, self.mesh, 0, dev if self.devices else None), dev)
            ex.seed, ex.execution = self.seed, execution
            results[0] = (ex, ex.run(bound, self._consts))
            self.per_rank = results
            return self._result(results[0][1], ex, bound, results)

        def work(r):
            try:
                dev = self.devices[r] if self.devices else self.device
                ex = Executor(self.plan, r, ThreadCollectives(world, self.mesh, r, dev if self.devices else None), dev)
                ex.seed, ex.execution = self.seed, execution
                ex.engine = self.engines[r] if self.engines else None
                results[r] = (ex, ex.run(bound, self._consts))
            except BaseException as e:  # surfaced to the caller below
                errors.append(e)
                for b in list(world.barriers.values()):
                    b.abort()

        ts = [threading.Thread(target=work, args=(r,), daemon=True) for r in range(self.mesh.size)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        if errors:
            # the first failure aborts the barriers of the others: report the cause, not a bystander's broken barrier
            real = [e for e in errors if not isinstance(e, threading.BrokenBarrierError)]
            raise (real or errors)[0]
        self.per_rank = results
        owner = 0 if self.entry is None else self.mesh.names.index(self.entry)
        ex, flat = results[owner]
        return self._result(flat, ex, bound, results)

    def engine_report(self) -> list:
        """After a call: ``[{processor, step, op, device, seconds}]`` for every operation an engine processor ran."""
        out = []
        for r, res in enumerate(getattr(self, "per_rank", None) or []):
            if res is not None:
                out += [{"processor": self.mesh.names[r], **rec} for rec in res[0].engine_report]
        return out

    def structure(self) -> dict:
        """What the plan was lowered to: fused (collective, product) pairs and norms found, and, after a call, how many
        products / attention / norm steps ran on this package's kernels and how many on PyTorch operators (summed over
        the processors this process ran)."""
        execs = [self.exec] if not self.threads else [r[0] for r in (getattr(self, "per_rank", None) or []) if r is not None]
        own = sum(e.kernels.own for e in execs)
        eager = sum(e.kernels.eager for e in execs)
        return {"fused": dict(self.fusion), "kernels": {"own": own, "eager": eager}, "steps": len(self.plan.steps)}

    def _result(self, flat, ex, bound, all_results=None):
        exp = self.exported
        if all_results is not None:
            # the threaded interpreter sees every processor: a value that lives on another processor (a gradient of a
            # layer placed there) is taken from its owner instead of being reported as absent
            flat = list(flat)
            for i, v in enumerate(flat):
                if v is None:
                    flat[i] = next((r[1][i] for r in all_results if r is not None and r[1][i] is not None), None)
        # in-place stores of buffer / input mutations
        for i, ph in exp.mutations.items():
            if flat[i] is not None and isinstance(bound.get(ph), torch.Tensor):
                target = exp.state[ph][1] if ph in exp.state else bound[ph]
                with torch.no_grad():
                    target.copy_(flat[i].to(target.device))
        returned = [(k, v) for (k, _), v in zip(exp.outputs, flat)]
        if exp.training:
            outs = [v for k, v in returned if k in ("user", "loss")]
            grads_p = {t: v for (k, t), v in zip(exp.outputs, flat) if k == "grad_param"}
            if exp.tied:
                from .export import tied_gradients
                grads_p = tied_gradients(grads_p, exp.tied)
            grads_i = {t: v for (k, t), v in zip(exp.outputs, flat) if k == "grad_input"}
            try:
                outs_tree = pytree.tree_unflatten(outs, exp.out_spec)
            except Exception:
                outs_tree = outs[0] if len(outs) == 1 else tuple(outs)
            return TrainingResult(outs_tree, grads_p, grads_i)
        outs = [v for k, v in returned if k in ("user", "loss")]
        return pytree.tree_unflatten(outs, exp.out_spec)
