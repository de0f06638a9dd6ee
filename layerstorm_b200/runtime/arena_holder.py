"""Arena holder: a tiny process that keeps the file descriptors of host expert arenas (memfd slabs) open so that their
contents survive an engine restart, plus the client used by the engine and by the operator tool.

Protocol (one JSON line per request over a unix stream socket; descriptors travel as SCM_RIGHTS ancillary data):
    {"op": "put", "name": N, "slot_bytes": B, "n_slots": S, "tag": T}  + fd   -> {"ok": true}
    {"op": "get", "name": N}                                                  -> {"ok": true, "slot_bytes":.., "n_slots":.., "tag":..} + fd
    {"op": "status"}                                                          -> {"ok": true, "arenas": {...}}
    {"op": "wipe", "name": N, "reason": "..."}                                -> {"ok": true}     (drops the descriptor)
    {"op": "shutdown"}
A socket path starting with '@' is an abstract-namespace address (no file system entry).
Reference: tools/arena_holder.cpp (libc-only fd keeper), tools/arena_ctl.cpp (status / reasoned wipe), config section
``memory.arena_attach`` {socket_path, auto_spawn, persist, on_conflict}.
"""
from __future__ import annotations

import json
import os
import socket
import sys
import time
from typing import Dict, Optional, Tuple


def _addr(path: str):
    return "\0" + path[1:] if path.startswith("@") else path


def serve(socket_path: str = "@layerstorm-arena", log=None) -> int:
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    if not socket_path.startswith("@") and os.path.exists(socket_path):
        os.unlink(socket_path)
    srv.bind(_addr(socket_path))
    srv.listen(8)
    arenas: Dict[str, dict] = {}
    wipes = []
    while True:
        conn, _ = srv.accept()
        with conn:
            try:
                msg, fds, _, _ = socket.recv_fds(conn, 65536, 4)
                req = json.loads(msg.decode() or "{}")
                op = req.get("op")
                if op == "put":
                    old = arenas.pop(req["name"], None)
                    if old:
                        os.close(old["fd"])
                    arenas[req["name"]] = {"fd": fds[0], "slot_bytes": req["slot_bytes"], "n_slots": req["n_slots"], "tag": req.get("tag", 0),
                                           "since": time.time()}
                    conn.sendall(b'{"ok": true}')
                elif op == "get":
                    a = arenas.get(req["name"])
                    if a is None:
                        conn.sendall(b'{"ok": false, "error": "no such arena"}')
                    else:
                        socket.send_fds(conn, [json.dumps({"ok": True, "slot_bytes": a["slot_bytes"], "n_slots": a["n_slots"], "tag": a["tag"]}).encode()], [a["fd"]])
                elif op == "status":
                    conn.sendall(json.dumps({"ok": True, "pid": os.getpid(), "wipes": wipes[-8:],
                                             "arenas": {k: {kk: vv for kk, vv in v.items() if kk != "fd"} for k, v in arenas.items()}}).encode())
                elif op == "wipe":
                    a = arenas.pop(req["name"], None)
                    if a:
                        os.close(a["fd"])
                        wipes.append({"name": req["name"], "reason": req.get("reason", ""), "when": time.time()})
                    conn.sendall(json.dumps({"ok": a is not None}).encode())
                elif op == "shutdown":
                    conn.sendall(b'{"ok": true}')
                    break
                else:
                    conn.sendall(b'{"ok": false, "error": "unknown op"}')
                for fd in fds[1:]:
                    os.close(fd)
            except Exception as e:  # noqa: BLE001 - the holder must outlive malformed requests
                try:
                    conn.sendall(json.dumps({"ok": False, "error": str(e)}).encode())
                except OSError:
                    pass
    srv.close()
    return 0


class HolderClient:
    def __init__(self, socket_path: str = "@layerstorm-arena", timeout: float = 5.0):
        self.path, self.timeout = socket_path, timeout

    def _call(self, req: dict, fd: Optional[int] = None) -> Tuple[dict, list]:
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        s.settimeout(self.timeout)
        s.connect(_addr(self.path))
        with s:
            data = json.dumps(req).encode()
            if fd is not None:
                socket.send_fds(s, [data], [fd])
            else:
                s.sendall(data)
            msg, fds, _, _ = socket.recv_fds(s, 65536, 4)
            return json.loads(msg.decode() or "{}"), list(fds)

    def alive(self) -> bool:
        try:
            return bool(self._call({"op": "status"})[0].get("ok"))
        except OSError:
            return False

    def put(self, name: str, arena, tag: int = 0):
        r, _ = self._call({"op": "put", "name": name, "slot_bytes": arena.slot_bytes, "n_slots": arena.n_slots, "tag": tag}, fd=arena.fd)
        if not r.get("ok"):
            raise RuntimeError(r.get("error", "put failed"))

    def get(self, name: str):
        """(HostArena attached to the kept slab, tag) or None."""
        from . import native as rt
        r, fds = self._call({"op": "get", "name": name})
        if not r.get("ok"):
            return None
        try:
            return rt.HostArena(r["slot_bytes"], r["n_slots"], attach_fd=fds[0]), r["tag"]
        finally:
            for fd in fds:
                os.close(fd)

    def status(self) -> dict:
        return self._call({"op": "status"})[0]

    def wipe(self, name: str, reason: str) -> bool:
        if not reason.strip():
            raise ValueError("a wipe needs a reason (it is recorded by the holder)")
        return bool(self._call({"op": "wipe", "name": name, "reason": reason})[0].get("ok"))

    def shutdown(self):
        try:
            self._call({"op": "shutdown"})
        except OSError:
            pass


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="layerstorm_b200.runtime.arena_holder", description="keep expert-arena descriptors alive / inspect them")
    ap.add_argument("command", choices=["serve", "status", "wipe", "shutdown"])
    ap.add_argument("--socket", default="@layerstorm-arena")
    ap.add_argument("--name")
    ap.add_argument("--reason", default="")
    a = ap.parse_args(argv)
    if a.command == "serve":
        return serve(a.socket)
    c = HolderClient(a.socket)
    if a.command == "status":
        print(json.dumps(c.status(), indent=1))
    elif a.command == "wipe":
        print("wiped" if c.wipe(a.name, a.reason) else "no such arena")
    else:
        c.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
