"""ctypes bindings of the native heartbeat / quorum service (``libtt_ft.so``)."""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "_lib", "libtt_ft.so")
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` from the repository root")
        L = ctypes.CDLL(path)
        L.tt_lighthouse_start.restype = ctypes.c_void_p
        L.tt_lighthouse_start.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.tt_lighthouse_port.argtypes = [ctypes.c_void_p]
        L.tt_lighthouse_stop.argtypes = [ctypes.c_void_p]
        L.tt_ft_connect.restype = ctypes.c_void_p
        L.tt_ft_connect.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
        L.tt_ft_set_step.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        L.tt_ft_pause_heartbeat.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.tt_ft_quorum.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_char_p,
                                   ctypes.c_char_p, ctypes.c_int]
        L.tt_ft_status.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
        L.tt_ft_close.argtypes = [ctypes.c_void_p]
        _LIB = L
    return _LIB


class Lighthouse:
    """In-process server. ``heartbeat_timeout_ms``: a replica silent for longer is not waited for;
    ``join_timeout_ms``: how long a forming quorum waits for live replicas that have not asked yet."""

    def __init__(self, port: int = 0, heartbeat_timeout_ms: int = 5000, join_timeout_ms: int = 1000):
        self._h = _lib().tt_lighthouse_start(port, heartbeat_timeout_ms, join_timeout_ms)
        if not self._h:
            raise OSError(f"could not bind the lighthouse to port {port}")
        self.port = _lib().tt_lighthouse_port(self._h)

    @property
    def address(self) -> str:
        return f"127.0.0.1:{self.port}"

    def shutdown(self) -> None:
        if self._h:
            _lib().tt_lighthouse_stop(self._h)
            self._h = None


@dataclass
class Quorum:
    quorum_id: int
    replica_ids: list[str]
    addresses: list[str]
    max_step: int
    max_step_replica: str

    def rank_of(self, replica_id: str) -> int:
        return self.replica_ids.index(replica_id)


class QuorumError(RuntimeError):
    pass


class LighthouseClient:
    def __init__(self, address: str, replica_id: str, heartbeat_interval_ms: int = 100):
        host, port = address.rsplit(":", 1)
        self.replica_id = replica_id
        self._h = _lib().tt_ft_connect(host.encode(), int(port), replica_id.encode(), heartbeat_interval_ms)
        if not self._h:
            raise ConnectionError(f"cannot reach the lighthouse at {address}")

    def set_step(self, step: int) -> None:
        _lib().tt_ft_set_step(self._h, step)

    def pause_heartbeat(self, paused: bool = True) -> None:
        """Test hook: stop (or resume) heartbeats without leaving, to look like a hung replica."""
        _lib().tt_ft_pause_heartbeat(self._h, int(paused))

    def quorum(self, step: int, min_replicas: int = 1, timeout_ms: int = 10000, address: str = "") -> Quorum:
        buf = ctypes.create_string_buffer(1 << 16)
        rc = _lib().tt_ft_quorum(self._h, step, min_replicas, timeout_ms, address.encode(), buf, len(buf))
        line = buf.value.decode()
        if rc != 0:
            raise QuorumError(line or "lighthouse connection lost")
        _, qid, n, ids, addrs, max_step, best = line.split(" ")
        return Quorum(int(qid), ids.split(","), addrs.split(","), int(max_step), best)

    def status(self) -> dict:
        buf = ctypes.create_string_buffer(1024)
        if _lib().tt_ft_status(self._h, buf, len(buf)) != 0:
            raise ConnectionError("lighthouse connection lost")
        return {k: int(v) for k, v in (kv.split("=") for kv in buf.value.decode().split(" ")[1:])}

    def close(self) -> None:
        if self._h:
            _lib().tt_ft_close(self._h)
            self._h = None


def main() -> None:
    """``python -m torchtitan_b200.experiments.ft.lighthouse --port 29510`` runs a stand-alone service."""
    import argparse
    import time

    ap = argparse.ArgumentParser()
    ap.add_argument("--port", type=int, default=29510)
    ap.add_argument("--heartbeat-timeout-ms", type=int, default=5000)
    ap.add_argument("--join-timeout-ms", type=int, default=1000)
    a = ap.parse_args()
    lh = Lighthouse(a.port, a.heartbeat_timeout_ms, a.join_timeout_ms)
    print(f"lighthouse listening on {lh.address}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        lh.shutdown()


if __name__ == "__main__":
    main()
