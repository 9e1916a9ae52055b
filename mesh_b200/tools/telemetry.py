"""Per-node telemetry provider: ``python -m mesh_b200.tools.telemetry --port 8101``.

Serves JSON over HTTP: GPU samples (clocks, power, utilisation, memory, throttle reasons) read through NVML at a
fixed rate into a ring buffer, the runtime stats blocks of the node's ranks (launches, collectives, bytes per peer,
liveness), and workload envelopes (FLOP / byte counts per span) that running programs post.  Readers take a *lease*
on a cursor so that a slow reader misses samples instead of holding the ring.  Reading only: the provider changes
no GPU setting.  Counterpart of the reference's node telemetry provider (user/mesh-telemetry.py: powermetrics, GPU
residency, memory bandwidth, bridge counters, workload envelopes, ring buffer with leases) and of rdma/workload.py.

Endpoints: ``/samples?since=<cursor>``, ``/ranks?group=G&world=N``, ``/workloads``, ``POST /workload`` (JSON body),
``/health``.
"""
from __future__ import annotations

import argparse
import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from urllib.parse import parse_qs, urlparse


class Nvml:
    """Thin reader over NVML (``pynvml``); any object with the same ``sample()`` can stand in (tests use a fake)."""

    def __init__(self):
        import pynvml
        self.n = pynvml
        pynvml.nvmlInit()
        self.handles = [pynvml.nvmlDeviceGetHandleByIndex(i) for i in range(pynvml.nvmlDeviceGetCount())]

    def sample(self) -> list[dict]:
        n, out = self.n, []
        for i, h in enumerate(self.handles):
            rec = {"gpu": i}
            for key, fn in (("sm_mhz", lambda: n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)),
                            ("sm_max_mhz", lambda: n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)),
                            ("power_w", lambda: n.nvmlDeviceGetPowerUsage(h) / 1000.0),
                            ("util_pct", lambda: n.nvmlDeviceGetUtilizationRates(h).gpu),
                            ("mem_used_mb", lambda: n.nvmlDeviceGetMemoryInfo(h).used >> 20),
                            ("throttle", lambda: int(n.nvmlDeviceGetCurrentClocksEventReasons(h)))):
                try:
                    rec[key] = fn()
                except Exception:
                    rec[key] = None
            out.append(rec)
        return out


class Ring:
    """Fixed-size ring of samples with monotonically increasing cursors."""

    def __init__(self, size: int = 4096):
        self.size, self.items, self.next = size, [], 0
        self.lock = threading.Lock()

    def push(self, item) -> int:
        with self.lock:
            self.items.append((self.next, item))
            if len(self.items) > self.size:
                self.items.pop(0)
            self.next += 1
            return self.next

    def since(self, cursor: int, limit: int = 1000):
        """Samples with cursor >= ``cursor`` (oldest first), the next cursor, and how many the reader missed."""
        with self.lock:
            first = self.items[0][0] if self.items else self.next
            missed = max(0, first - cursor)
            got = [it for c, it in self.items if c >= cursor][:limit]
            nxt = max(cursor, first) + len(got)
            return got, nxt, missed


class Provider:
    def __init__(self, source=None, interval_s: float = 0.5, ring: int = 4096):
        self.source, self.interval = source, interval_s
        self.samples, self.workloads = Ring(ring), Ring(1024)
        self.run = False
        self.thread = None

    def start(self):
        self.run = True
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self):
        self.run = False
        if self.thread:
            self.thread.join(timeout=2)

    def _loop(self):
        while self.run:
            self.tick()
            time.sleep(self.interval)

    def tick(self):
        if self.source is not None:
            self.samples.push({"t": time.time(), "gpus": self.source.sample()})

    # ---- request handling (also callable without a socket)
    def handle(self, method: str, path: str, body: bytes = b"") -> tuple[int, dict]:
        u = urlparse(path)
        q = {k: v[0] for k, v in parse_qs(u.query).items()}
        if method == "GET" and u.path == "/health":
            return 200, {"ok": True, "samples": self.samples.next, "workloads": self.workloads.next}
        if method == "GET" and u.path == "/samples":
            got, nxt, missed = self.samples.since(int(q.get("since", 0)), int(q.get("limit", 1000)))
            return 200, {"samples": got, "next": nxt, "missed": missed}
        if method == "GET" and u.path == "/workloads":
            got, nxt, missed = self.workloads.since(int(q.get("since", 0)))
            return 200, {"workloads": got, "next": nxt, "missed": missed}
        if method == "POST" and u.path == "/workload":
            try:
                rec = json.loads(body or b"{}")
            except ValueError:
                return 400, {"error": "body is not JSON"}
            rec["t"] = time.time()
            return 200, {"cursor": self.workloads.push(rec)}
        if method == "GET" and u.path == "/ranks":
            from ..runtime import service
            world = int(q.get("world", 8))
            return 200, {"ranks": [service.read(q.get("group", "mesh"), r) for r in range(world)]}
        return 404, {"error": f"no such endpoint {u.path}"}


def serve(provider: Provider, host: str, port: int) -> ThreadingHTTPServer:
    class H(BaseHTTPRequestHandler):
        def _send(self, code, obj):
            data = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def do_GET(self):
            self._send(*provider.handle("GET", self.path))

        def do_POST(self):
            n = int(self.headers.get("Content-Length", 0))
            self._send(*provider.handle("POST", self.path, self.rfile.read(n)))

        def log_message(self, *a):
            pass
    return ThreadingHTTPServer((host, port), H)


def post_workload(url: str, meter) -> None:
    """Send a :class:`~mesh_b200.utils.metrics.WorkloadMeter`'s spans to a provider."""
    import urllib.request
    for span in meter.report():
        req = urllib.request.Request(url.rstrip("/") + "/workload", data=json.dumps(span).encode(), method="POST")
        urllib.request.urlopen(req, timeout=2).read()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mesh-telemetry")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8101)
    ap.add_argument("--interval", type=float, default=0.5)
    a = ap.parse_args(argv)
    try:
        src = Nvml()
    except Exception:
        src = None                      # a node without NVML still serves ranks and workloads
    p = Provider(src, a.interval)
    p.start()
    srv = serve(p, a.host, a.port)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        p.stop()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
