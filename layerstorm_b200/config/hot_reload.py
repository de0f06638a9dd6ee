"""Configuration hot reload: re-read the config file when it changes and apply the fields a running engine accepts.

Only the fields the schema marks live-changeable are applied; a change of any other field is reported and ignored until
restart, and a file that no longer validates leaves the running configuration untouched.  Listeners receive the list of
``(path, old, new)`` that was applied (the orchestrator uses it for speculation depth, batching and prefetch knobs).
Reference: python/orchestrator/config_hot_reload.py with the generated changeable-field list
(python/orchestrator/_gen_changeable_fields.py).
"""
from __future__ import annotations

import os
import threading
from typing import Any, Callable, List, Optional, Tuple

from .loader import ConfigError, get_path, load_config, set_path
from .schema import leaf_paths, live_changeable_fields

Change = Tuple[str, Any, Any]


def diff_configs(old: dict, new: dict) -> List[Change]:
    out = []
    for path, _ in leaf_paths():
        a, b = get_path(old, path), get_path(new, path)
        if a != b:
            out.append((path, a, b))
    return out


class ConfigHotReloader:
    def __init__(self, path: str, current: dict, overrides: Optional[dict] = None, on_apply: Optional[Callable[[List[Change]], None]] = None):
        self.path, self.cfg, self.overrides = path, current, overrides
        self.listeners: List[Callable[[List[Change]], None]] = [on_apply] if on_apply else []
        self.live = set(live_changeable_fields())
        self._sig = self._signature()
        self.last_error: Optional[str] = None
        self.ignored: List[Change] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _signature(self):
        try:
            st = os.stat(self.path)
            return (st.st_mtime_ns, st.st_size)
        except OSError:
            return None

    def poll(self) -> List[Change]:
        """Check the file once; returns the changes that were applied (empty when nothing changed or the file is invalid)."""
        sig = self._signature()
        if sig is None or sig == self._sig:
            return []
        self._sig = sig
        try:
            new = load_config(self.path, self.overrides)
        except (ConfigError, ValueError, OSError) as e:
            self.last_error = str(e)
            return []
        self.last_error = None
        changes = diff_configs(self.cfg, new)
        applied = [c for c in changes if c[0] in self.live]
        self.ignored = [c for c in changes if c[0] not in self.live]
        if applied:
            for path, _, val in applied:            # in place: holders of the dict see the new values
                set_path(self.cfg, path, val)
            for fn in self.listeners:
                fn(applied)
        return applied

    # ------------------------------------------------------------------ background watcher
    def start(self, interval_s: float = 2.0):
        def loop():
            while not self._stop.wait(interval_s):
                self.poll()
        self._thread = threading.Thread(target=loop, name="config-hot-reload", daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=5)
