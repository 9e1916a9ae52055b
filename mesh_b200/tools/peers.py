"""Discovery of the node: GPUs, which pairs can map each other's memory, and the link description used by the
roofline model.  ``python -m mesh_b200.tools.peers`` prints it as JSON.

On one NVSwitch node there is nothing to discover over a network (the reference finds its peers by Bonjour and
rebuilds the cable graph from their node-info pages, rdma/peers.py:103-185); what a job needs to know is the peer
matrix and the per-port bandwidth, which come from the driver and from the measured capacity file."""
from __future__ import annotations

import json

from ..utils.bounds import Link, Topology


def discover(n_gpus: int | None = None, can_access=None, capacity: dict | None = None) -> dict:
    """``can_access(a, b) -> bool`` defaults to the CUDA runtime's answer; ``capacity`` to the measured figures."""
    if can_access is None or n_gpus is None:
        import torch
        n_gpus = torch.cuda.device_count() if n_gpus is None else n_gpus
        can_access = can_access or (lambda a, b: bool(torch.cuda.can_device_access_peer(a, b)))
    if capacity is None:
        from ..config import capacity as cap_fn
        capacity = cap_fn()
    matrix = [[a == b or bool(can_access(a, b)) for b in range(n_gpus)] for a in range(n_gpus)]
    return {"gpus": n_gpus, "peer_access": matrix, "p2p_gbs_per_direction": capacity.get("nvlink_p2p_gbs", capacity.get("nvlink_gbs_per_dir", 770.0)),
            "all_connected": all(all(r) for r in matrix)}


def topology(found: dict) -> Topology:
    """Every pair with peer access is joined by a share of the port bandwidth (full bisection through the switch)."""
    n = found["gpus"]
    topo = Topology(set(range(n)))
    per = found["p2p_gbs_per_direction"] * 1e9 * 8 / max(1, n - 1)
    for a in range(n):
        for b in range(a + 1, n):
            if found["peer_access"][a][b] and found["peer_access"][b][a]:
                topo.add(a, b, Link("nvlink5", per, 2e-6))
    return topo


def islands(found: dict) -> list[list[int]]:
    """Groups of GPUs that can all reach each other (a job's tensor-parallel groups must stay inside one)."""
    n, m = found["gpus"], found["peer_access"]
    seen, out = set(), []
    for a in range(n):
        if a in seen:
            continue
        comp, todo = [], [a]
        while todo:
            x = todo.pop()
            if x in seen:
                continue
            seen.add(x)
            comp.append(x)
            todo += [y for y in range(n) if y not in seen and m[x][y] and m[y][x]]
        out.append(sorted(comp))
    return out


def main() -> int:
    f = discover()
    f["islands"] = islands(f)
    print(json.dumps(f))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
