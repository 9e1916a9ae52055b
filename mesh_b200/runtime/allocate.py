"""Online share allocation between calls (heterogeneous or drifting ranks).

Each rank's time is modelled as ``t = a + b * x`` in its share ``x``; the model is refit after every
call by recursive least squares with a forgetting factor, and the next shares equalise the predicted
finish times on a grain, within lower bounds (the reference's ``Allocator``, rdma/allocate.py:7-46, and
its helpers ``equal_finish`` :49, ``shift`` :92, ``separators`` :129).  Used by the routed-expert planner
example and by unequal tensor-parallel splits.
"""
from __future__ import annotations

import bisect
import math
from fractions import Fraction


def equal_finish(total: int, grain: int, low: list, high: list, a: list, b: list):
    """Shares (multiples of ``grain``, ``low <= s <= high``, summing to ``total``) that make the linear
    times ``a[i] + b[i] * s[i]`` finish together.  Returns ``(integer shares, real-valued shares, finish time)``."""
    n = len(a)
    pinned: dict[int, float] = {}
    while True:
        free = [i for i in range(n) if i not in pinned]
        if free:
            inv = sum(1.0 / b[i] for i in free)
            T = (total - sum(pinned.values()) + sum(a[i] / b[i] for i in free)) / inv
        else:
            T = math.inf
        real = [pinned[i] if i in pinned else (T - a[i]) / b[i] for i in range(n)]
        under = [i for i in free if real[i] < low[i]]
        over = [i for i in free if real[i] > high[i]]
        if not under and not over:
            break
        # pin the side that violates its bounds by more, then re-solve for the rest
        if sum(low[i] - real[i] for i in under) >= sum(real[i] - high[i] for i in over):
            for i in under:
                pinned[i] = float(low[i])
        else:
            for i in over:
                pinned[i] = float(high[i])
    base = [low[i] + grain * math.floor((real[i] - low[i]) / grain) for i in range(n)]
    ints, _ = min_max(total, grain, base, high, [lambda x, i=i: a[i] + b[i] * x for i in range(n)])
    return ints, real, T


def min_max(total: int, grain: int, low: list, high: list, cost: list):
    """Hand out the remaining grains one by one to the rank whose time stays lowest."""
    shares = list(low)
    for _ in range(max(0, (total - sum(low)) // grain)):
        able = [i for i in range(len(shares)) if shares[i] + grain <= high[i]]
        if not able:
            break
        pick = min(able, key=lambda i: (cost[i](shares[i] + grain), i))
        shares[pick] += grain
    return shares, max(cost[i](shares[i]) for i in range(len(shares)))


def shift(shares: list, upper: list, load: list) -> list:
    """Capacity repair: move the excess of over-full ranks to the least loaded ranks with room (Whale-style)."""
    shares = list(shares)
    over = [j for j in range(len(shares)) if shares[j] > upper[j]]
    room = [j for j in range(len(shares)) if shares[j] < upper[j]]
    while over:
        worst = max(over, key=lambda j: shares[j] / upper[j])
        if not room:
            raise ValueError("shift: total capacity is below the total share")
        target = min(room, key=lambda j: load[j](shares[j]))
        excess, space = shares[worst] - upper[worst], upper[target] - shares[target]
        if excess <= space:
            shares[target] += excess
            shares[worst] = upper[worst]
            over.remove(worst)
            if shares[target] >= upper[target]:
                room.remove(target)
        else:
            shares[worst] -= space
            shares[target] = upper[target]
            room.remove(target)
    return shares


def _cuts_for(offsets: list, speeds: list, load) -> list:
    cuts = [0]
    for sp in speeds:
        cuts.append(bisect.bisect_right(offsets, offsets[cuts[-1]] + load * sp) - 1)
    return cuts


def separators(offsets: list, speeds: list) -> list:
    """Cut a ragged tensor's rows (``offsets`` = row starts in elements, len rows+1) into consecutive groups, one
    per rank, minimising the largest ``elements / speed``: exact search over the candidate loads."""
    rows = len(offsets) - 1
    sp = [Fraction(s) for s in speeds]
    ok, bad, first = Fraction(offsets[rows] - offsets[0]) / sp[0], Fraction(-1), 0
    for s in sp:
        lo, hi = first + 1, rows + 1
        while lo < hi:
            mid = (lo + hi) // 2
            load = Fraction(offsets[mid] - offsets[first]) / s
            if bad < load < ok:
                if _cuts_for(offsets, sp, load)[-1] == rows:
                    ok = load
                else:
                    bad = load
            if load >= ok:
                hi = mid
            else:
                lo = mid + 1
        first = lo - 1
    return _cuts_for(offsets, sp, ok)


class Allocator:
    """``shares = allocator(times)`` after every call: refit ``t = a + b x`` per rank, re-split for the next call.

    ``shares``: initial integer shares (multiples of ``grain``); ``low``: lower bounds; ``prior``: per rank
    ``(a, b, var_a, var_b)``; ``floor``: smallest slope believed; ``forget`` in (0, 1]: RLS forgetting factor;
    ``step`` in (0, 1]: how far to move towards the new optimum each call.
    """

    def __init__(self, shares, grain, low, prior, floor, forget=0.9, step=1.0):
        n = len(shares)
        if not (len(low) == len(prior) == len(floor) == n):
            raise ValueError("allocator: one lower bound, prior and floor per rank")
        if any(s % grain or l % grain or l < grain or s < l for s, l in zip(shares, low)) or sum(low) >= sum(shares):
            raise ValueError("allocator: shares and bounds must sit on the grain with room above the bounds")
        if min(floor) <= 0 or not 0 < forget <= 1 or not 0 < step <= 1:
            raise ValueError("allocator: positive floors, forget and step in (0, 1]")
        self.shares, self.grain, self.low, self.floor = list(shares), grain, list(low), list(floor)
        self.total, self.forget, self.step = sum(shares), forget, step
        self.real = [float(s) for s in shares]
        self.a = [float(p[0]) for p in prior]
        self.b = [float(p[1]) for p in prior]
        self.cov = [[float(p[2]), 0.0, float(p[3])] for p in prior]       # [var_a, cov_ab, var_b]
        self.cap = [c[0] + c[2] for c in self.cov]

    def __call__(self, times, scale: float = 1.0, next_scale: float = 1.0):
        n, lam = len(self.shares), self.forget
        target_a, slope = [], []
        for i in range(n):
            x = scale * self.shares[i]
            va, cab, vb = self.cov[i]
            # RLS update with regressor (1, x)
            g0, g1 = va + cab * x, cab + vb * x
            denom = lam + g0 + g1 * x
            k0, k1 = g0 / denom, g1 / denom
            err = times[i] - (self.a[i] + self.b[i] * x)
            self.a[i] += k0 * err
            self.b[i] += k1 * err
            va, cab, vb = (va - k0 * g0) / lam, (cab - k0 * g1) / lam, (vb - k1 * g1) / lam
            if va + vb > self.cap[i]:                      # keep the covariance from winding up
                f = self.cap[i] / (va + vb)
                va, cab, vb = va * f, cab * f, vb * f
            self.cov[i] = [va, cab, vb]
            b = max(self.b[i], self.floor[i])
            predicted = times[i] + b * (next_scale * self.real[i] - x)
            slope.append(b * next_scale)
            target_a.append(self.step * predicted - b * next_scale * self.real[i])
        ints, real, _ = equal_finish(self.total, self.grain, self.low, [math.inf] * n, target_a, slope)
        self.shares, self.real = ints, real
        return list(ints)
