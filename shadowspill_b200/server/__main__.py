"""``python -m shadowspill_b200.server --root DIR [--host H] [--port P] [--token T]``:
run the training service until interrupted. The token defaults to the
``SHADOWSPILL_TOKEN`` environment variable."""
from __future__ import annotations

import argparse
import signal
import threading

from .service import Server


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m shadowspill_b200.server")
    ap.add_argument("--root", required=True, help="service directory (journal, runs, checkpoints)")
    ap.add_argument("--models", default=None, help="directory of pretrained weights, optional")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8123)
    ap.add_argument("--token", default=None)
    a = ap.parse_args(argv)
    stop = threading.Event()
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda *_: stop.set())
    with Server(a.root, a.models, a.host, a.port, a.token) as server:
        print(f"serving on {server.url}", flush=True)
        stop.wait()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
