"""Whole-job observer: polls the telemetry providers of several nodes and serves one merged view.

The reference runs a per-node telemetry provider and an aggregator that reaches every node, merges what it reads and
serves a page (viz/serve.py:1-465, bin/mesh-observe.py).  Here a node is one host with up to eight GPUs and its
provider is ``mesh_b200.tools.telemetry``; the observer

* keeps one cursor per provider and reads ``/samples`` and ``/workloads`` since that cursor, each request with a
  deadline, so a node that stopped answering costs one timeout per round and shows as stale instead of blocking;
* merges the latest sample of every node into ``{"nodes": {name: {...}}, "totals": {...}}`` - GPUs, mean utilisation,
  power, memory in use, and the workload envelopes (FLOP and bytes per second) posted since the last round;
* serves it as ``/mesh.json`` and as a plain HTML table at ``/`` (no scripts, no external assets).

    python -m mesh_b200.tools.observe --node a=http://127.0.0.1:8101 --node b=http://10.0.0.2:8101 --port 8110
"""
from __future__ import annotations

import argparse
import html
import json
import threading
import time
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer


def _get(url: str, timeout: float) -> dict:
    with urllib.request.urlopen(url, timeout=timeout) as r:
        return json.loads(r.read())


def _rate(span: dict, key: str) -> float:
    """A workload span carries totals and its duration (``utils/metrics.py``): the rate is their quotient."""
    sec = span.get("seconds") or 0.0
    return float(span.get(key) or 0.0) / sec if sec > 0 else 0.0


class Observer:
    def __init__(self, nodes: dict[str, str], timeout_s: float = 1.0, stale_s: float = 5.0, fetch=_get):
        self.nodes = dict(nodes)
        self.timeout, self.stale, self.fetch = timeout_s, stale_s, fetch
        self.cursor = {n: {"samples": 0, "workloads": 0} for n in nodes}
        self.state = {n: {"url": u, "ok": False, "last_seen": None, "error": "not polled yet", "sample": None,
                          "workloads": [], "missed": 0} for n, u in nodes.items()}
        self.lock = threading.Lock()
        self.rounds = 0

    def poll_one(self, name: str) -> None:
        url, cur = self.nodes[name].rstrip("/"), self.cursor[name]
        try:
            got = self.fetch(f"{url}/samples?since={cur['samples']}&limit=64", self.timeout)
            work = self.fetch(f"{url}/workloads?since={cur['workloads']}", self.timeout)
        except Exception as e:                                  # a node that does not answer is reported, not fatal
            with self.lock:
                self.state[name].update(ok=False, error=f"{type(e).__name__}: {e}")
            return
        cur["samples"], cur["workloads"] = got.get("next", cur["samples"]), work.get("next", cur["workloads"])
        with self.lock:
            st = self.state[name]
            st.update(ok=True, error=None, last_seen=time.time())
            st["missed"] += int(got.get("missed", 0))
            if got.get("samples"):
                st["sample"] = got["samples"][-1]
            st["workloads"] = work.get("workloads", [])

    def poll(self) -> None:
        """One round over all nodes, concurrently (a round takes one timeout at most)."""
        threads = [threading.Thread(target=self.poll_one, args=(n,), daemon=True) for n in self.nodes]
        for t in threads:
            t.start()
        for t in threads:
            t.join(self.timeout * 2 + 1)
        self.rounds += 1

    def merged(self) -> dict:
        now = time.time()
        nodes, totals = {}, {"nodes": 0, "nodes_ok": 0, "gpus": 0, "power_w": 0.0, "memory_used_mib": 0.0, "flops_per_s": 0.0,
                             "bytes_per_s": 0.0}
        with self.lock:
            for name, st in self.state.items():
                gpus = (st["sample"] or {}).get("gpus") or []
                age = None if st["last_seen"] is None else now - st["last_seen"]
                fresh = st["ok"] and age is not None and age <= self.stale
                util = [g.get("util_pct") or 0 for g in gpus]
                rec = {"url": st["url"], "ok": st["ok"], "fresh": fresh, "age_s": None if age is None else round(age, 3),
                       "error": st["error"], "gpus": len(gpus),
                       "mean_util": round(sum(util) / len(util), 2) if util else None,
                       "power_w": round(sum(g.get("power_w") or 0.0 for g in gpus), 1),
                       "memory_used_mib": round(sum(g.get("mem_used_mb") or 0.0 for g in gpus), 1),
                       "missed_samples": st["missed"], "workloads": len(st["workloads"]),
                       "flops_per_s": sum(_rate(w, "flops") for w in st["workloads"]),
                       "bytes_per_s": sum(_rate(w, "hbm_bytes") for w in st["workloads"])}
                nodes[name] = rec
                totals["nodes"] += 1
                totals["nodes_ok"] += int(fresh)
                if fresh:
                    for k in ("gpus", "power_w", "memory_used_mib", "flops_per_s", "bytes_per_s"):
                        totals[k] += rec[k]
        return {"t": now, "rounds": self.rounds, "nodes": nodes, "totals": totals}

    def page(self) -> str:
        m = self.merged()
        cols = ("ok", "fresh", "age_s", "gpus", "mean_util", "power_w", "memory_used_mib", "workloads", "flops_per_s", "error")
        rows = "".join("<tr><td>" + html.escape(n) + "</td>" + "".join(f"<td>{html.escape(str(r[c]))}</td>" for c in cols) + "</tr>"
                       for n, r in sorted(m["nodes"].items()))
        head = "<tr><th>node</th>" + "".join(f"<th>{c}</th>" for c in cols) + "</tr>"
        t = m["totals"]
        return (f"<html><head><meta http-equiv=refresh content=2><title>mesh</title></head><body><h3>{t['nodes_ok']} of "
                f"{t['nodes']} nodes, {t['gpus']} GPUs, {t['power_w']:.0f} W, {t['flops_per_s'] / 1e12:.2f} TFLOP/s</h3>"
                f"<table border=1 cellpadding=4>{head}{rows}</table></body></html>")


def serve(observer: Observer, host: str, port: int) -> ThreadingHTTPServer:
    class H(BaseHTTPRequestHandler):
        def do_GET(self):
            if self.path.startswith("/mesh.json"):
                data, kind = json.dumps(observer.merged()).encode(), "application/json"
            elif self.path in ("/", "/index.html"):
                data, kind = observer.page().encode(), "text/html"
            else:
                self.send_error(404)
                return
            self.send_response(200)
            self.send_header("Content-Type", kind)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def log_message(self, *a):
            pass
    return ThreadingHTTPServer((host, port), H)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mesh-observe")
    ap.add_argument("--node", action="append", default=[], help="name=url of a telemetry provider; repeat per node")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8110)
    ap.add_argument("--interval", type=float, default=1.0)
    ap.add_argument("--once", action="store_true", help="poll one round, print the merged view and exit")
    a = ap.parse_args(argv)
    nodes = dict(n.split("=", 1) for n in a.node) or {"local": "http://127.0.0.1:8101"}
    ob = Observer(nodes)
    if a.once:
        ob.poll()
        print(json.dumps(ob.merged()))
        return 0
    srv = serve(ob, a.host, a.port)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        while True:
            ob.poll()
            time.sleep(a.interval)
    except KeyboardInterrupt:
        pass
    finally:
        srv.shutdown()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
