"""Roofline bounds of a placed program on a machine: the four lower bounds on a step's time.

* compute - work over the aggregate rate, and each device's own work over its own rate;
* memory  - bytes over the aggregate memory bandwidth, and each device's own bytes over its own;
* cut     - for every named cut of the machine, the bytes that must cross it over the bandwidth of the links in it;
* path    - a chain of dependent transfers: per hop the link latency plus bytes over the hop's bandwidth.

The largest of them is the time no schedule can beat; benchmark reports quote achieved time against it.  Same model
as the reference's ``bounds()`` (swift/Bounds.swift:26-118) over its ``Topology`` / ``Link`` description
(swift/Topology.swift:4-36); link bandwidth is given in bits per second there and here.  :func:`b200_node` builds the
description of one NVSwitch node from the measured figures of :func:`mesh_b200.config.capacity`.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class Link:
    device: str
    bandwidth: float                      # bits per second, one direction
    latency: float | None = None          # seconds


def _pair(a: int, b: int) -> tuple[int, int]:
    return (a, b) if a <= b else (b, a)


@dataclass
class Topology:
    nodes: set[int] = field(default_factory=set)
    links: dict[tuple[int, int], list[Link]] = field(default_factory=dict)

    def add(self, a: int, b: int, link: Link) -> "Topology":
        self.nodes.update((a, b))
        self.links.setdefault(_pair(a, b), []).append(link)
        return self

    def between(self, a: int, b: int) -> list[Link]:
        return self.links.get(_pair(a, b), [])

    def merging(self, other: "Topology") -> "Topology":
        out = Topology(set(self.nodes) | set(other.nodes), {k: list(v) for k, v in self.links.items()})
        for k, v in other.links.items():
            out.links.setdefault(k, []).extend(v)
        return out


@dataclass(frozen=True)
class Capability:
    rate: float                           # operations per second
    bandwidth: float                      # bytes per second of device memory


@dataclass(frozen=True)
class Work:
    """The whole program: operations and bytes of memory traffic."""
    work: float
    bytes: float


@dataclass(frozen=True)
class Cut:
    links: frozenset                      # pairs (a, b) whose links make up the cut
    bytes: float


@dataclass(frozen=True)
class Hop:
    link: tuple[int, int]
    bytes: float


@dataclass
class Placed:
    """Where the program's work and bytes sit and what crosses which cut (the reference's ``Placement`` record)."""
    owners: list[int] = field(default_factory=list)
    routes: dict[tuple[int, int], list[int]] = field(default_factory=dict)
    work: dict[int, float] = field(default_factory=dict)
    bytes: dict[int, float] = field(default_factory=dict)
    cuts: dict[str, Cut] = field(default_factory=dict)
    path: list[Hop] = field(default_factory=list)


@dataclass(frozen=True)
class Bounds:
    compute: float
    memory: float
    cut: dict
    path: float
    max: float

    def fraction(self, achieved_seconds: float) -> float:
        """Share of the achieved time that the bound explains (1.0 = at the roofline)."""
        return self.max / achieved_seconds if achieved_seconds > 0 else 0.0

    def binding(self) -> str:
        """Name of the bound that equals ``max``."""
        best = max([("compute", self.compute), ("memory", self.memory), ("path", self.path),
                    *[(f"cut:{k}", v) for k, v in self.cut.items()]], key=lambda kv: kv[1])
        return best[0]


def _seconds(amount: float, rate: float) -> float:
    if amount == 0:
        return 0.0
    return float("inf") if rate <= 0 else amount / rate


def bounds(program: Work, placed: Placed, topology: Topology, capability: dict[int, Capability]) -> Bounds:
    rate = sum(c.rate for c in capability.values())
    bw = sum(c.bandwidth for c in capability.values())
    compute = _seconds(program.work, rate)
    memory = _seconds(program.bytes, bw)
    for node, w in placed.work.items():
        compute = max(compute, _seconds(w, capability[node].rate if node in capability else 0.0))
    for node, b in placed.bytes.items():
        memory = max(memory, _seconds(b, capability[node].bandwidth if node in capability else 0.0))
    worst = max(compute, memory)
    cut = {}
    for key, c in placed.cuts.items():
        cap = sum(l.bandwidth / 8 for a, b in c.links for l in topology.between(a, b))
        cut[key] = _seconds(c.bytes, cap)
        worst = max(worst, cut[key])
    path = 0.0
    for hop in placed.path:
        links = topology.between(*hop.link)
        cap = sum(l.bandwidth / 8 for l in links)
        lat = min((l.latency or 0.0 for l in links), default=0.0)
        path += lat + _seconds(hop.bytes, cap)
    return Bounds(compute, memory, cut, path, max(worst, path))


def b200_node(n_gpus: int = 8, cap: dict | None = None) -> tuple[Topology, dict[int, Capability]]:
    """One NVSwitch node: every pair of GPUs joined at the measured peer bandwidth (the switch gives every GPU its
    full bandwidth to every peer; a GPU's total is still bounded by its own port, which :func:`port_cut` states)."""
    if cap is None:
        from ..config import capacity
        cap = capacity()
    p2p = cap.get("nvlink_p2p_gbs", cap.get("nvlink_gbs_per_dir", 770.0)) * 1e9 * 8
    lat = cap.get("nvlink_latency_us", 2.0) * 1e-6
    topo = Topology(set(range(n_gpus)))
    for a in range(n_gpus):
        for b in range(a + 1, n_gpus):
            topo.add(a, b, Link("nvlink5", p2p / max(1, n_gpus - 1), lat))
    caps = {g: Capability(cap.get("bf16_tflops_sustained", 1382.0) * 1e12, cap.get("hbm_gbs", 6529.0) * 1e9)
            for g in range(n_gpus)}
    return topo, caps


def port_cut(gpu: int, n_gpus: int, bytes_out: float) -> Cut:
    """The cut around one GPU's NVLink port: everything it sends to (or receives from) the other GPUs."""
    return Cut(frozenset(_pair(gpu, o) for o in range(n_gpus) if o != gpu), bytes_out)


def tp_ffn_bounds(tokens: int, d_model: int, d_ff: int, world: int, cap: dict | None = None) -> Bounds:
    """Bounds of one sequence-parallel SwiGLU FFN layer, forward and backward, on ``world`` GPUs: three passes of the
    two GEMMs; per pass an all-gather and a reduce-scatter of the activations through every GPU's port."""
    topo, caps = b200_node(world, cap)
    flops = 3 * (2 * tokens * d_model * 2 * d_ff + 2 * tokens * d_ff * d_model)
    weights = 3 * d_model * d_ff * 2
    acts = tokens * d_model * 2
    placed = Placed(work={g: flops / world for g in range(world)},
                    bytes={g: 3 * (weights / world) + 6 * acts for g in range(world)})
    if world > 1:
        per_port = 4 * acts * (world - 1) / world          # AG + RS forward, AG + RS backward (dgrad), per GPU, one way
        placed.cuts = {f"port{g}": port_cut(g, world, per_port) for g in range(world)}
    return bounds(Work(flops, world * placed.bytes[0]), placed, topo, caps)
