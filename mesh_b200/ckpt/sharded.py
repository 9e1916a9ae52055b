"""Sharded checkpoint: one safetensors file per rank plus a JSON index, re-shardable on load.

The reference archives compiled programs, not model state, and every rank builds the whole module
(compiler/mesh_compiler/archive.py:24-83, placement.py:173-180).  This format adds true sharded state:
``index.json`` records for every tensor the compiler's triple ``(dimension, counts, world)`` — the same
``counts`` / displacement semantics as ``placement.counts`` (compiler/mesh_compiler/placement.py:65-108) — so
a checkpoint written at one world size loads at another, each rank reading only the slices it needs.
Writes follow the journal + atomic-rename discipline of the reference's training continuation notes
(design/TRAINING-CONTINUATION.md:20-45): journal line, data files, fsync, commit line; a step without its
commit line is ignored on load.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch
from safetensors.torch import load_file, save_file

from ..utils.disk import room


def _fsync_dir(d: Path) -> None:
    fd = os.open(str(d), os.O_RDONLY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def save_sharded(directory, step: int, local: dict, layout: dict, rank: int, world: int, extra: dict | None = None,
                 barrier=None) -> Path:
    """``local[name]``: this rank's shard; ``layout[name]`` = ``(dim, counts)`` (``dim`` None = replicated, rank 0
    writes it).  Every rank calls this; ``barrier()`` (if given) separates data from the commit line."""
    d = Path(directory) / f"step-{step:08d}"
    d.mkdir(parents=True, exist_ok=True)
    need = sum(t.numel() * t.element_size() for t in local.values())
    room(d, need)
    journal = Path(directory) / "journal.jsonl"
    if rank == 0:
        with open(journal, "a") as j:
            j.write(json.dumps({"event": "begin", "step": step, "world": world}) + "\n")
            j.flush()
            os.fsync(j.fileno())
    tensors, seen = {}, set()
    for name, t in local.items():
        dim, _ = layout[name]
        if dim is None and rank != 0:
            continue
        t = t.detach().contiguous().cpu()
        if t.untyped_storage().nbytes() != t.numel() * t.element_size() or t.untyped_storage().data_ptr() in seen:
            t = t.clone()                      # a view, or a second name for the same bytes: the file format wants tensors of their own
        seen.add(t.untyped_storage().data_ptr())
        tensors[name] = t
    tmp = d / f"rank{rank}.safetensors.tmp"
    save_file(tensors, str(tmp))
    _fsync_file(tmp)                           # the shard's bytes are durable before its name (and the commit line) is
    os.replace(tmp, d / f"rank{rank}.safetensors")
    if rank == 0:
        index = {"step": step, "world": world, "extra": extra or {},
                 "tensors": {n: {"dim": layout[n][0], "counts": list(layout[n][1]) if layout[n][1] is not None else None,
                                 "dtype": str(local[n].dtype), "shape": list(local[n].shape)} for n in local}}
        tmpi = d / "index.json.tmp"
        tmpi.write_text(json.dumps(index, indent=1))
        _fsync_file(tmpi)
        os.replace(tmpi, d / "index.json")
    _fsync_dir(d)
    if barrier is not None:
        barrier()
    if rank == 0:
        with open(journal, "a") as j:
            j.write(json.dumps({"event": "commit", "step": step}) + "\n")
            j.flush()
            os.fsync(j.fileno())
    if barrier is not None:
        barrier()
    return d


def _fsync_file(path) -> None:
    fd = os.open(str(path), os.O_RDONLY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def latest_step(directory) -> int | None:
    """Highest step whose commit line is in the journal (idempotent replay: uncommitted steps are ignored)."""
    journal = Path(directory) / "journal.jsonl"
    if not journal.exists():
        return None
    best = None
    for line in journal.read_text().splitlines():
        try:
            rec = json.loads(line)
        except json.JSONDecodeError:
            continue                    # a torn last line
        if rec.get("event") == "commit":
            best = rec["step"] if best is None else max(best, rec["step"])
    return best


def load_sharded(directory, step: int | None, rank: int, world: int, new_layout: dict | None = None, device="cpu"):
    """Returns ``(local tensors, extra)`` for ``rank`` of a ``world``-rank job.  ``new_layout[name]`` = ``(dim, counts)``
    for the new world (default: the stored dim with ``torch.chunk`` counts); reads only overlapping old shards."""
    from ..compiler.placement import counts as chunk_counts
    if step is None:
        step = latest_step(directory)
        if step is None:
            raise FileNotFoundError(f"no committed checkpoint in {directory}")
    d = Path(directory) / f"step-{step:08d}"
    index = json.loads((d / "index.json").read_text())
    old_world = index["world"]
    files: dict[int, dict] = {}

    def shard_of(r):
        if r not in files:
            files[r] = load_file(str(d / f"rank{r}.safetensors"))
        return files[r]

    out = {}
    for name, meta in index["tensors"].items():
        dim, old_counts = meta["dim"], meta["counts"]
        if dim is None:
            whole = shard_of(0)[name]
            if new_layout and name in new_layout and new_layout[name][0] is not None:
                ndim, ncounts = new_layout[name]            # stored replicated, wanted cut
                whole = whole.narrow(ndim, sum(ncounts[:rank]), ncounts[rank]).contiguous()
            out[name] = whole.to(device)
            continue
        total = sum(old_counts)
        dtype = getattr(torch, str(meta.get("dtype", "torch.float32")).split(".")[-1])
        if new_layout and name in new_layout:
            ndim, ncounts = new_layout[name]
            if ndim != dim:
                # another dimension (or none: replicated): put the old shards together, then take the new slice
                whole = torch.cat([shard_of(r)[name] for r in range(old_world) if old_counts[r]], dim=dim)
                if ndim is None:
                    out[name] = whole.to(device)
                else:
                    out[name] = whole.narrow(ndim, sum(ncounts[:rank]), ncounts[rank]).contiguous().to(device)
                continue
        else:
            ncounts = chunk_counts(total, None, world)
        lo = sum(ncounts[:rank])
        hi = lo + ncounts[rank]
        pieces, pos = [], 0
        for r in range(old_world):
            a, b = pos, pos + old_counts[r]
            pos = b
            s, e = max(a, lo), min(b, hi)
            if s < e:
                pieces.append(shard_of(r)[name].narrow(dim, s - a, e - s))
        if pieces:
            out[name] = torch.cat(pieces, dim=dim).to(device)
        else:
            shape = list(meta["shape"])
            shape[dim] = 0
            out[name] = torch.empty(shape, dtype=dtype, device=device)
    return out, index.get("extra", {})
