"""mesh_b200 — a Blackwell-native (sm_100a) distributed runtime with the capabilities of SQCU/mesh.

Layers, bottom to top:

* ``csrc/``        hand-written CUDA for sm_100a (tcgen05/TMEM GEMMs fed by TMA, fused
                   compute+collective kernels over NVLink peer memory, attention, quantised
                   matmul, norms, RoPE, router) and the C++ host runtime, planner and graph library;
* ``runtime``      symmetric heap, signal pads, status/abort/epoch words, streams and plans;
* ``distributed``  the ``mesh`` ``torch.distributed`` backend and the explicit collective verbs;
* ``ops``          Python entry points and autograd functions over the kernels;
* ``parallel``     TP / SP / DP / EP / CP / PP layer library and placement helpers;
* ``compiler``     GSPMD-style sharding compiler: capture, place, schedule, lower, ``Program``;
* ``models``       the example / benchmark models;
* ``ckpt``         sharded checkpoints with reshard-on-load;
* ``tools``        launcher + watchdog, ``meshctl``, roofline reports.
"""
from __future__ import annotations

__version__ = "0.1.0"

from .config import MeshConfig, config  # noqa: F401
