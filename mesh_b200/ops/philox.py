"""Philox4x32-10 counter-based random numbers, and dropout masks that do not depend on how a tensor is sharded.

A draw is a pure function of ``(seed, execution, site, element)``: the element index is the element's *logical* index
in the unsharded tensor, so a rank that holds any slice, strided or striped, produces exactly the bits the single
device would (the reference keys its generator the same way, compiler/mesh_compiler/operations.py:7201-7275, and uses
it for attention dropout, :7143-7158).  Counter = (element low, element high, site, execution), key = the 64-bit seed;
Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC 2011.

Stated with 64-bit integer tensor arithmetic, so it runs on CPU and CUDA tensors alike.
"""
from __future__ import annotations

import torch

M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = 0xFFFFFFFF


def _mulhilo(a: int, b: torch.Tensor):
    """32 x 32 -> (hi, lo) without leaving signed 64-bit range."""
    p0 = a * (b & 0xFFFF)
    p1 = a * (b >> 16)
    t = p0 + ((p1 & 0xFFFF) << 16)
    return ((p1 >> 16) + (t >> 32)) & MASK, t & MASK


def philox4x32(counter, key, rounds: int = 10):
    """``counter``: four int64 tensors holding 32-bit words (broadcastable); ``key``: two ints or tensors.
    Returns four int64 tensors of 32-bit words."""
    c0, c1, c2, c3 = (torch.as_tensor(c, dtype=torch.int64) & MASK for c in counter)
    c0, c1, c2, c3 = torch.broadcast_tensors(c0, c1, c2, c3)
    k0, k1 = key
    for _ in range(rounds):
        hi0, lo0 = _mulhilo(M0, c0)
        hi1, lo1 = _mulhilo(M1, c2)
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & MASK, lo1, (hi0 ^ c3 ^ k1) & MASK, lo0
        k0, k1 = (k0 + W0) & MASK, (k1 + W1) & MASK
    return c0, c1, c2, c3


def uniform(elements: torch.Tensor, seed: int, execution: int = 0, site: int = 0) -> torch.Tensor:
    """fp32 numbers in [0, 1), one per entry of ``elements`` (int64 logical element indices)."""
    e = elements.to(torch.int64)
    w0, _, _, _ = philox4x32((e & MASK, (e >> 32) & MASK, torch.full_like(e, site & MASK), torch.full_like(e, execution & MASK)),
                             (seed & MASK, (seed >> 32) & MASK))
    return (w0 >> 8).to(torch.float32) * (1.0 / (1 << 24))


def logical_index(shape, slices=None, device=None) -> torch.Tensor:
    """Logical (row-major, unsharded) element indices of the block ``slices`` of a tensor of ``shape``.
    ``slices``: per dimension ``None`` (all), a ``slice``, or an index tensor (striped shards)."""
    idx = torch.zeros((), dtype=torch.int64, device=device)
    stride = 1
    dims = []
    for d in reversed(range(len(shape))):
        sel = None if slices is None else slices[d]
        if sel is None:
            pos = torch.arange(shape[d], device=device)
        elif isinstance(sel, slice):
            pos = torch.arange(shape[d], device=device)[sel]
        else:
            pos = torch.as_tensor(sel, device=device)
        dims.append((d, pos.to(torch.int64) * stride))
        stride *= shape[d]
    nd = len(shape)
    for d, pos in dims:
        view = [1] * nd
        view[d] = -1
        idx = idx + pos.view(view)
    return idx


def dropout(x: torch.Tensor, p: float, seed: int, execution: int = 0, site: int = 0, *, full_shape=None, slices=None,
            training: bool = True) -> torch.Tensor:
    """Dropout whose keep mask is a function of logical positions: ``x`` is the block ``slices`` of a tensor of
    ``full_shape`` (default: ``x`` is the whole tensor)."""
    if not training or p <= 0:
        return x
    shape = tuple(x.shape) if full_shape is None else tuple(full_shape)
    idx = logical_index(shape, slices, x.device)
    keep = uniform(idx, seed, execution, site) >= p
    return torch.where(keep, x / (1 - p), torch.zeros((), dtype=x.dtype, device=x.device))


def attention_keep_mask(bh: torch.Tensor, qpos: torch.Tensor, kpos: torch.Tensor, p: float, seed: int, site: int = 0,
                        execution: int = 0) -> torch.Tensor:
    """Keep mask of attention dropout as the flash kernels draw it (``csrc/device/philox.cuh``): one Philox call per
    four consecutive key positions, counter ``(kpos >> 2, qpos, batch * heads + head, site)``, key
    ``(seed_lo ^ execution * 0x9E3779B9, seed_hi)``, ``u = (word[kpos & 3] >> 8) * 2^-24``, keep iff ``u >= p``.
    ``bh``, ``qpos``, ``kpos``: broadcastable int64 tensors of logical coordinates.  Returns a bool tensor."""
    bh, qpos, kpos = torch.broadcast_tensors(bh.to(torch.int64), qpos.to(torch.int64), kpos.to(torch.int64))
    k0 = ((seed & MASK) ^ ((execution * 0x9E3779B9) & MASK)) & MASK
    k1 = (seed >> 32) & MASK
    words = philox4x32((kpos >> 2, qpos, bh, torch.full_like(kpos, site & MASK)), (k0, k1))
    sel = kpos & 3
    w = torch.where(sel == 0, words[0], torch.where(sel == 1, words[1], torch.where(sel == 2, words[2], words[3])))
    return (w >> 8).to(torch.float32) * (1.0 / (1 << 24)) >= p
