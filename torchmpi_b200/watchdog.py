"""Host watchdog: heartbeats through the job's key-value store, and communicator poisoning.

The reference has no failure detection beyond a 10 s spin that raises "looks like a deadlock" when a
worker never releases a resource (lib/resources.cpp:124-132); a lost rank leaves the others blocked in
MPI for ever.  Here every rank runs a small thread that
  * publishes a counter under ``tmpi/<job>/hb/<rank>`` every ``watchdog_interval_ms``,
  * reads the counters of the other ranks and notes when each last moved,
  * declares a rank lost when its counter has stood still for ``watchdog_budget_ms`` (a rank that leaves
    through ``stop()`` says goodbye first and is not reported).
A lost rank, a device-side wait that ran out, or a handle that timed out *poisons* the runtime: every later
collective, barrier or parameter-server call raises ``CommunicatorPoisoned`` at once instead of waiting for
a peer that will not come.  Recovery is a clean error followed by ``stop()``; re-forming the job is out of
scope (the reference has none either).  Failures are only ever injected on the host (a rank that exits or
stalls, a dropped request); nothing here touches a GPU.
"""
from __future__ import annotations

import datetime
import os
import threading
import time
from typing import Optional

from . import config
from .runtime import S


class CommunicatorPoisoned(RuntimeError):
    """A peer was lost or a bounded wait ran out earlier; the communicators of this job are unusable."""


_state = {"reason": None, "thread": None, "stop": None, "paused": False}


def poison(reason: str) -> None:
    """Marks the runtime unusable (first reason wins)."""
    if _state["reason"] is None:
        _state["reason"] = str(reason)


def poisoned() -> Optional[str]:
    return _state["reason"]


def check() -> None:
    """Raises ``CommunicatorPoisoned`` if the runtime has been poisoned."""
    if _state["reason"] is not None:
        raise CommunicatorPoisoned(_state["reason"])


def reset() -> None:
    _state["reason"] = None


def pause(flag: bool = True) -> None:
    """Test hook: stop publishing heartbeats (a rank whose host thread stalls) without stopping the process."""
    _state["paused"] = bool(flag)


def _client_store():
    """A store connection of the watchdog's own (the main thread keeps using the default one)."""
    import torch.distributed as dist
    host, port = os.environ.get("MASTER_ADDR"), os.environ.get("MASTER_PORT")
    if host and port:
        try:
            return dist.TCPStore(host, int(port), is_master=False, timeout=datetime.timedelta(seconds=30),
                                 wait_for_workers=False)
        except Exception:       # fall back to the shared client
            pass
    from torch.distributed import distributed_c10d
    return distributed_c10d._get_default_store()


def start() -> None:
    interval = config.get("watchdog_interval_ms") / 1e3
    if interval <= 0 or S.world <= 1 or _state["thread"] is not None:
        return
    stop_evt = threading.Event()
    prefix = f"tmpi/{S.job_id}/hb/"
    rank, world = S.rank, S.world

    def body():
        try:
            store = _client_store()
        except Exception as e:   # no store, no watchdog
            return
        budget = config.get("watchdog_budget_ms") / 1e3
        seen = {r: (None, time.monotonic()) for r in range(world) if r != rank}
        beat = 0
        while not stop_evt.wait(interval):
            try:
                if not _state["paused"]:
                    beat += 1
                    store.set(prefix + str(rank), str(beat))
                now = time.monotonic()
                for r in list(seen):
                    key = prefix + str(r)
                    if not store.check([key]):
                        val = None
                    else:
                        val = bytes(store.get(key)).decode()
                    last, since = seen[r]
                    if val == "bye":
                        del seen[r]
                        continue
                    if val != last:
                        seen[r] = (val, now)
                    elif now - since > budget:
                        poison(f"rank {r} has not sent a heartbeat for {now - since:.1f} s (budget {budget:.1f} s)")
                        del seen[r]
            except Exception as e:
                # the store itself is gone (rank 0 hosts it): the job cannot go on
                poison(f"the key-value store of the job is unreachable: {e}")
                return

    t = threading.Thread(target=body, name="tmpi-watchdog", daemon=True)
    _state.update(thread=t, stop=stop_evt, paused=False)
    t.start()


def stop(goodbye: bool = True) -> None:
    t, evt = _state["thread"], _state["stop"]
    if t is None:
        return
    evt.set()
    t.join(timeout=5)
    if goodbye:
        try:
            from torch.distributed import distributed_c10d
            distributed_c10d._get_default_store().set(f"tmpi/{S.job_id}/hb/{S.rank}", "bye")
        except Exception:
            pass
    _state.update(thread=None, stop=None)
