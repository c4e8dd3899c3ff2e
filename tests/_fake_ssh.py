#!/usr/bin/env python3
"""Stand-in for the OpenSSH client in the tunnel test: understands ``-L bind:port:host:port``,
forwards TCP connections like ``ssh -N -L`` would, and fails the way ssh does for a destination
named ``unreachable``. Nothing is encrypted and nothing leaves this machine."""
import socket
import sys
import threading


def pump(a, b):
    try:
        while True:
            data = a.recv(65536)
            if not data:
                break
            b.sendall(data)
    except OSError:
        pass
    finally:
        for s in (a, b):
            try:
                s.shutdown(socket.SHUT_RDWR)
            except OSError:
                pass


def main():
    args = sys.argv[1:]
    spec = args[args.index("-L") + 1]
    destination = args[-1]
    if "BatchMode=yes" not in args or "--" not in args:
        print("expected a batch-mode invocation", file=sys.stderr)
        return 2
    if destination == "unreachable":
        print("ssh: connect to host unreachable port 22: No route to host", file=sys.stderr)
        return 255
    bind, lport, host, rport = spec.rsplit(":", 3)
    srv = socket.socket()
    srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    srv.bind((bind, int(lport)))
    srv.listen(16)
    while True:
        c, _ = srv.accept()
        up = socket.create_connection((host, int(rport)))
        threading.Thread(target=pump, args=(c, up), daemon=True).start()
        threading.Thread(target=pump, args=(up, c), daemon=True).start()


if __name__ == "__main__":
    sys.exit(main())
