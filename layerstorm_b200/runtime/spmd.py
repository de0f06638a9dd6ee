"""SPMD control plane for multi-GPU engines: one process per GPU, every rank must issue the same engine calls.

Rank 0 (the leader) owns the orchestrator and the HTTP server; it talks to its engine through ``SpmdLeader``, which
announces every state-changing call (method name + arguments, a few hundred bytes) to the other ranks over a CPU
(gloo) process group before running it locally.  Ranks 1..N-1 run ``follower_loop`` and replay the calls on their own
engine shard, so the in-kernel NVLink collectives of a step always find their peers.  The data plane (activations,
partial sums, expert rows) never goes through this channel.
Reference counterpart: the daemon's command dispatcher driven over IPC by the Python orchestrator
(src/daemon/command_dispatcher.h, python/orchestrator/orchestrator.py) - one command stream, N GPU executors.
"""
from __future__ import annotations

from typing import Any, Optional

# engine methods that change device or sequence state and therefore must run on every rank, in the same order
MIRRORED = ("create_sequence", "free_sequence", "fork_sequence", "rewind", "prefill", "forward_rows", "decode", "generate",
            "enable_kv_tiering", "hibernate", "resume", "configure_expert_cache", "verify_greedy", "anchor", "sample_last_prefill",
            "clear_device_errors")
_STOP = "__stop__"


def control_group():
    """A CPU (gloo) group over all ranks for the command stream; the default group stays free for NCCL bootstrap traffic."""
    import torch.distributed as dist
    return dist.new_group(backend="gloo")


class SpmdLeader:
    """Engine facade for rank 0.  Attribute reads go straight to the engine; mirrored methods are announced first."""

    def __init__(self, engine, group=None, broadcast=None, monitor=None):
        object.__setattr__(self, "_engine", engine)
        object.__setattr__(self, "_group", group)
        object.__setattr__(self, "_broadcast", broadcast or _broadcast_from(0, group))
        object.__setattr__(self, "_monitor", monitor)            # runtime/heartbeat.py RankMonitor: refuse to start a step a dead rank cannot join
        object.__setattr__(self, "calls_announced", 0)

    def __getattr__(self, name: str) -> Any:
        attr = getattr(self._engine, name)
        if name in MIRRORED and callable(attr):
            def mirrored(*args, **kwargs):
                if self._monitor is not None:
                    self._monitor.check()                        # raises RankFailure: nothing is announced, no kernel waits on the dead rank
                self._broadcast([name, args, kwargs])
                object.__setattr__(self, "calls_announced", self.calls_announced + 1)
                return attr(*args, **kwargs)
            return mirrored
        return attr

    def __setattr__(self, name: str, value: Any):
        setattr(self._engine, name, value)

    def shutdown(self):
        self._broadcast([_STOP, (), {}])


def follower_loop(engine, group=None, receive=None, on_error: Optional[callable] = None) -> int:
    """Replay the leader's calls until it shuts down.  Returns the number of calls replayed.  An exception raised by a replayed
    call is passed to ``on_error`` (default: re-raised) - the leader raises the same exception from the same call."""
    receive = receive or _receive_from(0, group)
    n = 0
    while True:
        name, args, kwargs = receive()
        if name == _STOP:
            return n
        try:
            getattr(engine, name)(*args, **kwargs)
        except Exception as e:                      # noqa: BLE001 - mirrored: the leader sees the same failure
            if on_error is None:
                raise
            on_error(name, e)
        n += 1


def _broadcast_from(src: int, group):
    def send(obj):
        import torch.distributed as dist
        dist.broadcast_object_list([obj], src=src, group=group)
    return send


def _receive_from(src: int, group):
    def recv():
        import torch.distributed as dist
        box = [None]
        dist.broadcast_object_list(box, src=src, group=group)
        return box[0]
    return recv
