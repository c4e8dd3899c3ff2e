"""A small command line over the client, for looking at a service without writing a script.

    python -m shadowspill_b200.client --url http://127.0.0.1:8123 info
    python -m shadowspill_b200.client --url ... hardware | components [--kind model]
    python -m shadowspill_b200.client --url ... run SESSION RUN                 # state, workers, plan summary
    python -m shadowspill_b200.client --url ... progress SESSION RUN [--follow]  # the preparation / worker log
    python -m shadowspill_b200.client --url ... metrics SESSION RUN [--after N] [--jsonl PATH]
    python -m shadowspill_b200.client --ssh training-host:8123 info              # through an owned OpenSSH forward

The token comes from ``--token`` or ``SHADOWSPILL_TOKEN``. Everything here only reads; runs are
created and driven from Python (``docs/client_guide.md``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

from .metrics import MetricQueries
from .transport import SSH, HTTPTransport, SSHTunnel


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m shadowspill_b200.client", description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default=os.environ.get("SHADOWSPILL_URL", ""))
    ap.add_argument("--ssh", default="", help="HOST:SERVICE_PORT: reach the service through an OpenSSH forward")
    ap.add_argument("--token", default=os.environ.get("SHADOWSPILL_TOKEN", ""))
    sub = ap.add_subparsers(dest="command", required=True)
    sub.add_parser("info")
    sub.add_parser("hardware")
    comp = sub.add_parser("components")
    comp.add_argument("--kind", default="")
    for name in ("run", "progress", "metrics"):
        p = sub.add_parser(name)
        p.add_argument("session")
        p.add_argument("run")
        if name == "progress":
            p.add_argument("--follow", action="store_true", help="keep printing until the run leaves 'preparing'")
        if name == "metrics":
            p.add_argument("--after", type=int, default=0)
            p.add_argument("--jsonl", default="", help="write the snapshot to this new file instead of printing it")
    a = ap.parse_args(argv)
    tunnel = None
    url = a.url
    if a.ssh:
        host, _, port = a.ssh.rpartition(":")
        tunnel = SSHTunnel(SSH(host, int(port)))
        url = tunnel.open()
    if not url:
        ap.error("give --url (or SHADOWSPILL_URL) or --ssh HOST:PORT")
    t = HTTPTransport(url, a.token)
    out = sys.stdout
    try:
        if a.command == "info":
            json.dump(t.request("GET", "/v1/info")[1], out, indent=1)
        elif a.command == "hardware":
            json.dump(t.request("GET", "/v1/hardware")[1], out, indent=1)
        elif a.command == "components":
            rows = t.request("GET", "/v1/components", query={"kind": a.kind} if a.kind else None)[1]["components"]
            for c in rows:
                out.write(f"{c['kind']:<12} {c['id']:<40} {c['source']['distribution']} {c['source']['version']}\n")
        elif a.command == "run":
            json.dump(t.request("GET", f"/v1/runs/{a.session}/{a.run}")[1], out, indent=1)
        elif a.command == "progress":
            seen = 0
            while True:
                page = t.request("GET", f"/v1/runs/{a.session}/{a.run}/progress", query={"after": seen})[1]
                for line in page.get("lines", ()):
                    out.write(line + "\n")
                seen = int(page.get("next", seen))
                out.flush()
                state = t.request("GET", f"/v1/runs/{a.session}/{a.run}")[1]["state"]
                if not a.follow or state != "preparing":
                    break
                time.sleep(0.5)
        elif a.command == "metrics":
            queries = MetricQueries(t, a.session, a.run)
            if a.jsonl:
                out.write(str(queries.export_jsonl(a.jsonl, after=a.after).result()) + "\n")
            else:
                for rec in queries.snapshot(after=a.after):
                    out.write(json.dumps(rec, sort_keys=True) + "\n")
        out.write("" if a.command in ("components", "progress", "metrics") else "\n")
        return 0
    finally:
        if tunnel is not None:
            tunnel.close()


if __name__ == "__main__":
    sys.exit(main())
