"""Synchronisation monitor: what a rank actually did, compared with what the compiler said it would do.

The compiled schedule has a signature: the ordered list of collectives (verb, kind, axis, bytes) and a digest over it
(``schedule.py``).  With ``MESH_SYNC_TRACE=1`` an executor logs every collective it really issues, fused ones
included.  :func:`compare` lines the two up and names the first divergence: a collective that was skipped, one that
was not in the plan, or two that ran in the other order: the bugs that otherwise show up as a bounded wait running out
on some other rank.  The reference checks the same property from outside, with probes on the host's and the GPU's
synchronisation calls compared against the compiled signature (bin/mesh-sync-monitor.py)."""
from __future__ import annotations

import hashlib


_FUSED = {"ag_mm": "all_gather", "mm_rs": "reduce_scatter", "ring_attention": "ring"}


def expected(plan) -> list[tuple]:
    """(verb, kind, axis, channel) of every collective of ``plan``, in program order; a fused step counts as the
    collective it contains."""
    out = []
    for st in plan.steps:
        if st.op == "collective" and "channel" in st.meta:
            out.append((st.target, st.meta.get("kind"), st.meta["axis"], st.meta["channel"]))
        elif st.op == "fused" and "channel" in st.meta:
            out.append((_FUSED[st.target], st.meta.get("kind"), st.meta["axis"], st.meta["channel"]))
    return out


def digest(scheduled, ops: list[tuple]) -> str:
    """Digest of a list of observed operations in the form the schedule's signature uses (bytes looked up by channel)."""
    size = {t.channel: t.nbytes for t in scheduled.plan.transfers}
    h = hashlib.sha256()
    for verb, kind, axis, channel in ops:
        h.update(f"{verb}|{kind}|{axis}|{size.get(channel, 0)};".encode())
    return h.hexdigest()[:16]


def compare(scheduled, observed: list[tuple], plan=None) -> dict:
    """``{"ok", "digest_expected", "digest_observed", "first_divergence", "missing", "unexpected"}``.
    ``plan``: the plan the executor ran when it is not ``scheduled.plan`` itself (the fusion pass moves a gather to
    the position of its matmul, so the order of the fused plan is the one to hold a rank to)."""
    want = expected(plan if plan is not None else scheduled.plan)
    rep = {"ok": True, "count_expected": len(want), "count_observed": len(observed),
           "digest_expected": digest(scheduled, want), "digest_observed": digest(scheduled, observed),
           "first_divergence": None, "missing": [], "unexpected": []}
    for i, (w, o) in enumerate(zip(want, observed)):
        if w != o:
            rep["first_divergence"] = {"index": i, "expected": w, "observed": o}
            break
    if rep["first_divergence"] is None and len(want) != len(observed):
        i = min(len(want), len(observed))
        rep["first_divergence"] = {"index": i, "expected": want[i] if i < len(want) else None,
                                   "observed": observed[i] if i < len(observed) else None}
    seen = {}
    for o in observed:
        seen[o[3]] = seen.get(o[3], 0) + 1
    planned = {w[3] for w in want}
    rep["missing"] = [w for w in want if w[3] not in seen]
    rep["unexpected"] = [o for o in observed if o[3] not in planned]
    rep["ok"] = rep["first_divergence"] is None and rep["digest_expected"] == rep["digest_observed"]
    return rep
