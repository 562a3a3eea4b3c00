"""Host-side failure detection and shrink-to-survivors recovery.

The fused collectives wait for their peers on the device; a rank that has died would make
every survivor sit in a bounded wait until its budget runs out, on every bucket.  The monitor
lets survivors learn of a lost peer on the host, before their next launch:

* every rank publishes a heartbeat counter in the rendezvous store from a daemon thread and
  watches its peers' counters; a counter that stops for ``timeout_s`` marks the peer silent;
* a rank that leaves in an orderly way (``leave()``) or catches an exception
  (``report_failure(exc)``, or the ``guard()`` context manager) says so in the store, and
  its peers know within one polling interval instead of after the timeout;
* ``check()`` is what the training loop calls between steps: it only reads state the
  thread keeps up to date (no store round trip on the step's path) and raises
  ``PeerLostError`` naming the ranks and the reason.

``shrink_process_group`` is the recovery half: the survivors agree on the membership through
the store, tear down the old default process group and initialise a new one among themselves
(new ranks = order of the old ones).  ``LowBitGroup.rebind`` then points a low-bit group at
the new process group and re-shards its error-feedback residuals.  The store has to be
hosted by a process that survives (the launcher's agent, or a rank that is not the one lost).

The reference has no failure detection beyond the process-group timeout it forwards to NCCL
(``cpp/include/process_group_lowbit.h:43``, ``cpp/src/process_group_lowbit.cc:375-378``).
"""

from __future__ import annotations

import contextlib
import threading
import time
from typing import Dict, Iterable, List, Optional

import torch.distributed as dist


class PeerLostError(RuntimeError):
    """One or more peers are gone; ``ranks`` maps rank -> reason."""

    def __init__(self, ranks: Dict[int, str]):
        self.ranks = dict(ranks)
        what = ", ".join(f"rank {r}: {why}" for r, why in sorted(self.ranks.items()))
        super().__init__(f"lost peers ({what})")


class HealthMonitor:
    """Heartbeats through a c10d store (``TCPStore``, ``FileStore``, ``HashStore`` ...)."""

    def __init__(self, store, rank: int, world: int, *, interval_s: float = 0.5,
                 timeout_s: float = 5.0, prefix: str = "bitscom/health", start: bool = True):
        if not (0 <= rank < world):
            raise ValueError("rank out of range")
        if timeout_s <= interval_s:
            raise ValueError("timeout_s must exceed interval_s")
        self.store = dist.PrefixStore(prefix, store)
        self.rank, self.world = int(rank), int(world)
        self.interval_s, self.timeout_s = float(interval_s), float(timeout_s)
        self._beats = 0
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        now = time.monotonic()
        self._last_value: Dict[int, bytes] = {}
        self._last_change: Dict[int, float] = {p: now for p in self.peers()}
        self._lost: Dict[int, str] = {}
        self.store_errors = 0
        if start:
            self.start()

    # -- plumbing ---------------------------------------------------------------------------
    def peers(self) -> List[int]:
        return [p for p in range(self.world) if p != self.rank]

    def start(self) -> None:
        if self._thread is not None:
            return
        self.beat()
        self._thread = threading.Thread(target=self._loop, name="bitscom-health", daemon=True)
        self._thread.start()

    def close(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5 * self.interval_s + 1.0)
            self._thread = None

    def _loop(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self.beat()
                self.poll()
            except Exception:  # the store itself is gone: peers will see us fall silent
                self.store_errors += 1

    # -- one round, also callable directly (tests drive it without the thread) ---------------
    def beat(self) -> None:
        self._beats += 1
        self.store.set(f"beat/{self.rank}", str(self._beats))

    def poll(self, now: Optional[float] = None) -> None:
        now = time.monotonic() if now is None else now
        for p in self.peers():
            if p in self._lost and not self._lost[p].startswith("silent"):
                continue  # an explicit message is final
            reason = None
            if self.store.check([f"failed/{p}"]):
                reason = "failed: " + self.store.get(f"failed/{p}").decode(errors="replace")
            elif self.store.check([f"left/{p}"]):
                reason = "left"
            else:
                if self.store.check([f"beat/{p}"]):
                    value = self.store.get(f"beat/{p}")
                    if value != self._last_value.get(p):
                        self._last_value[p] = value
                        self._last_change[p] = now
                quiet = now - self._last_change[p]
                if quiet > self.timeout_s:
                    reason = f"silent for {quiet:.1f} s"
            with self._lock:
                if reason is not None:
                    self._lost[p] = reason
                elif p in self._lost:  # it was only slow: the heartbeat came back
                    del self._lost[p]

    # -- what the training loop uses -------------------------------------------------------------
    def lost(self) -> Dict[int, str]:
        with self._lock:
            return dict(self._lost)

    def alive(self) -> List[int]:
        gone = self.lost()
        return [r for r in range(self.world) if r == self.rank or r not in gone]

    def check(self) -> None:
        """Raise ``PeerLostError`` if a peer has left, failed or fallen silent."""
        gone = self.lost()
        if gone:
            raise PeerLostError(gone)

    def leave(self, wait_release_s: float = 0.0) -> bool:
        """Orderly exit between steps: peers learn of it at their next poll.

        With ``wait_release_s`` > 0 the call then waits (at most that long) until every peer
        that is still alive has called ``release([this rank])``, i.e. has let go of whatever
        it had mapped from this rank (symmetric-memory blocks of the fused collectives), so
        that this process can free that memory and exit without pulling it away under a
        peer.  Returns whether all of them did."""
        self.store.set(f"left/{self.rank}", "1")
        ok = True
        if wait_release_s > 0:
            deadline = time.monotonic() + wait_release_s
            waiting = [p for p in self.peers() if p not in self.lost()]
            while waiting and time.monotonic() < deadline:
                waiting = [p for p in waiting
                           if not self.store.check([f"released/{p}/{self.rank}"])
                           and p not in self.lost()]
                if waiting:
                    time.sleep(min(0.05, self.interval_s))
            ok = not waiting
        self.close()
        return ok

    def release(self, ranks: Iterable[int]) -> None:
        """Tell ranks that have left that this rank no longer holds anything of theirs (call it
        after ``LowBitGroup.rebind`` has dropped the old communicators)."""
        for r in ranks:
            self.store.set(f"released/{self.rank}/{int(r)}", "1")

    def report_failure(self, exc: BaseException) -> None:
        self.store.set(f"failed/{self.rank}", f"{type(exc).__name__}: {exc}"[:500])

    @contextlib.contextmanager
    def guard(self):
        """Publishes an exception that escapes the block, then re-raises it."""
        try:
            yield self
        except PeerLostError:
            raise  # that is news about somebody else
        except BaseException as exc:
            try:
                self.report_failure(exc)
            finally:
                raise


def agree_on_survivors(store, rank: int, candidates: Iterable[int], *, epoch: int,
                       timeout_s: float = 30.0, prefix: str = "bitscom/elastic") -> List[int]:
    """Every survivor publishes the set of ranks it believes alive and waits until all of
    them have published the same set; returns it sorted.  Raises ``PeerLostError`` when the
    views do not converge within ``timeout_s`` (a candidate died during recovery, or two
    ranks saw different losses: call again with ``epoch + 1`` after another ``check()``)."""
    st = dist.PrefixStore(f"{prefix}/{epoch}", store)
    mine = sorted(set(int(c) for c in candidates))
    if rank not in mine:
        raise ValueError("a rank cannot vote itself out")
    text = ",".join(map(str, mine))
    st.set(f"view/{rank}", text)
    deadline = time.monotonic() + timeout_s
    pending = [p for p in mine if p != rank]
    while pending:
        still = []
        for p in pending:
            if not st.check([f"view/{p}"]):
                still.append(p)
                continue
            theirs = st.get(f"view/{p}").decode()
            if theirs != text:
                raise PeerLostError({p: f"disagrees on the survivors ({theirs} vs {text})"})
        pending = still
        if pending:
            if time.monotonic() > deadline:
                raise PeerLostError({p: "did not take part in the recovery" for p in pending})
            time.sleep(0.05)
    return mine


def shrink_process_group(store, old_rank: int, survivors: Iterable[int], *, epoch: int,
                         backend: Optional[str] = None, timeout_s: float = 60.0,
                         device_id=None):
    """Replace the default process group by one over ``survivors`` (old ranks, as returned by
    ``agree_on_survivors``).  Returns ``(new_rank, new_world)``.  Collectives of the old group
    must not be in flight: call it between steps, after ``check()`` raised."""
    import datetime

    members = sorted(set(int(s) for s in survivors))
    if old_rank not in members:
        raise ValueError("this rank is not among the survivors")
    if dist.is_initialized():
        backend = backend or str(dist.get_backend())
        try:
            dist.destroy_process_group()
        except Exception:  # a dead peer can make the orderly teardown fail; the group is gone anyway
            pass
    if backend is None:
        raise ValueError("no backend given and no process group to take it from")
    new_rank, new_world = members.index(old_rank), len(members)
    kwargs = {}
    if device_id is not None:
        kwargs["device_id"] = device_id
    dist.init_process_group(backend, store=dist.PrefixStore(f"bitscom/epoch{epoch}", store),
                            rank=new_rank, world_size=new_world,
                            timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return new_rank, new_world
