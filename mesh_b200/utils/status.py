"""Host view of the device status block (csrc/device/status.cuh).

Every kernel in the library reports a failed bounded wait or a failed check by writing one
record here and returning, never by trapping; the host reads the block after a step and
raises.  The codes mirror the reference's ETIMEDOUT / ECANCELED / ESTALE host results
(rdma/mesh.h:15-17) and its GPU status word (rdma/mesh-metal.h:76-80).
"""
from __future__ import annotations

import torch

CODES = {0: "OK", 1: "TIMEOUT", 2: "CANCELED", 3: "STALE", 4: "BOUNDS", 5: "ALIGN", 6: "BAD_ARGUMENT"}
SITES = {0: "none", 1: "smem_full", 2: "smem_empty", 3: "tmem_full", 4: "tmem_empty", 5: "peer_flag",
         6: "local_flag", 7: "barrier", 8: "store_drain", 9: "host_flag", 10: "check"}


class MeshDeviceError(RuntimeError):
    def __init__(self, record: dict):
        self.record = record
        super().__init__(f"mesh device status: {record}")


class MeshTimeout(MeshDeviceError):
    pass


class MeshCanceled(MeshDeviceError):
    pass


_blocks: dict[int, torch.Tensor] = {}


def status_block(device=None) -> torch.Tensor:
    """The per-device 64-byte status block (int32[16]), created on first use."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _blocks.get(idx)
    if t is None:
        t = torch.zeros(16, dtype=torch.int32, device=torch.device("cuda", idx))
        _blocks[idx] = t
    return t


def decode(block: torch.Tensor) -> dict:
    w = block.detach().cpu().tolist()
    u64 = lambda lo, hi: (lo & 0xFFFFFFFF) | ((hi & 0xFFFFFFFF) << 32)
    return {
        "code": CODES.get(w[0], str(w[0])), "site": SITES.get(w[1], str(w[1])), "block": w[2], "thread": w[3],
        "expected": u64(w[4], w[5]), "seen": u64(w[6], w[7]), "aux": u64(w[8], w[9]),
        "count": w[10], "abort": w[11], "epoch": w[12],
    }


def check_status(device=None, clear: bool = True) -> None:
    """Synchronise and raise if any kernel recorded a failure since the last check."""
    blk = status_block(device)
    torch.cuda.synchronize(blk.device)
    rec = decode(blk)
    if rec["code"] == "OK":
        return
    if clear:
        blk[:11].zero_()
    if rec["code"] == "TIMEOUT":
        raise MeshTimeout(rec)
    if rec["code"] == "CANCELED":
        raise MeshCanceled(rec)
    raise MeshDeviceError(rec)


def raise_abort(device=None) -> None:
    """Host-side cancel: bounded device waits observe the flag and return CANCELED."""
    status_block(device)[11] = 1


def clear_abort(device=None) -> None:
    status_block(device)[11] = 0
