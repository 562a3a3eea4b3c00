"""Single-node launcher with restart-based recovery.

    python -m bitscom_b200.launch --nproc 8 --min-nproc 4 --max-restarts 3 -- \
        python -m bitscom_b200.trainer.llama_dp_pp --health_check --output_dir ckpt ...

starts one process per rank with the usual ``RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR /
MASTER_PORT`` environment and watches them.  It also hosts a ``TCPStore`` of its own
(``BITSCOM_AGENT_STORE=host:port`` in the children's environment) that outlives any rank, for
the heartbeats of ``bitscom_b200.utils.health``: ranks learn of a lost peer on the host, stop
between steps (exit code 3 by convention) and leave their checkpoint behind.

When a rank fails, the launcher gives the others ``--grace`` seconds to stop by themselves,
ends what is left (the exact processes it started), and starts a new generation: with the
same number of ranks, or with ``--shrink`` with as many ranks fewer as have failed (never
fewer than ``--min-nproc``).  ``BITSCOM_RESTART_COUNT`` tells the children which generation
they are; resuming from the checkpoint is the program's business.  Exit code: 0 when a
generation ends with every rank returning 0, 1 when the restarts are used up.

The reference is launched with plain ``torchrun`` and has no recovery
(``README.md`` quick start; ``benchmarks/train_llama7b_dp_pp_lowbit.py:203-216``).
"""

from __future__ import annotations

import argparse
import datetime
import json
import os
import signal
import socket
import subprocess
import sys
import time
from typing import Dict, List, Optional

STOPPED_FOR_PEER = 3  # exit code of a rank that stopped because another one was lost


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class Generation:
    """The processes of one start of the job."""

    def __init__(self, command: List[str], world: int, index: int, store_port: int,
                 extra_env: Optional[Dict[str, str]] = None):
        self.world, self.index = world, index
        self.master_port = _free_port()
        self.procs: List[subprocess.Popen] = []
        for rank in range(world):
            env = dict(os.environ)
            env.update(extra_env or {})
            env.update({
                "RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                "LOCAL_WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1",
                "MASTER_PORT": str(self.master_port),
                "BITSCOM_AGENT_STORE": f"127.0.0.1:{store_port}",
                "BITSCOM_RESTART_COUNT": str(index),
            })
            # a session of its own: signals sent to the launcher's group do not hit it twice
            self.procs.append(subprocess.Popen(command, env=env, start_new_session=True))

    def poll(self) -> Dict[int, Optional[int]]:
        return {rank: p.poll() for rank, p in enumerate(self.procs)}

    def stop(self, timeout_s: float = 10.0) -> None:
        """End the processes this generation started that are still running."""
        alive = [p for p in self.procs if p.poll() is None]
        for p in alive:
            try:
                p.send_signal(signal.SIGTERM)
            except ProcessLookupError:
                pass
        deadline = time.monotonic() + timeout_s
        for p in alive:
            try:
                p.wait(timeout=max(0.1, deadline - time.monotonic()))
            except subprocess.TimeoutExpired:
                try:
                    p.kill()
                except ProcessLookupError:
                    pass
                p.wait()


def run(command: List[str], nproc: int, *, min_nproc: Optional[int] = None,
        max_restarts: int = 0, shrink: bool = False, grace_s: float = 30.0,
        poll_s: float = 0.2, log=None) -> int:
    """Run ``command`` on ``nproc`` ranks with restarts; returns the launcher's exit code."""
    import torch.distributed as dist

    log = log or (lambda row: print(json.dumps(row), file=sys.stderr, flush=True))
    min_nproc = nproc if min_nproc is None else max(1, min_nproc)
    store_port = _free_port()
    # the heartbeat store lives in the launcher, so it survives the loss of any rank
    store = dist.TCPStore("127.0.0.1", store_port, is_master=True, wait_for_workers=False,
                          timeout=datetime.timedelta(seconds=300))
    world, restarts = nproc, 0
    try:
        while True:
            gen = Generation(command, world, restarts, store_port)
            log({"launch": "generation started", "generation": restarts, "world": world})
            failed_at = None
            try:
                while True:
                    codes = gen.poll()
                    done = {r: c for r, c in codes.items() if c is not None}
                    bad = {r: c for r, c in done.items() if c != 0}
                    if len(done) == world:
                        break
                    if bad:
                        failed_at = failed_at or time.monotonic()
                        if time.monotonic() - failed_at > grace_s:
                            break
                    time.sleep(poll_s)
            finally:
                gen.stop()
            codes = gen.poll()
            bad = {r: c for r, c in codes.items() if c != 0}
            if not bad:
                log({"launch": "finished", "generation": restarts, "world": world})
                return 0
            # ranks that stopped because somebody else was lost are healthy
            lost = sorted(r for r, c in bad.items() if c != STOPPED_FOR_PEER)
            log({"launch": "generation failed", "generation": restarts, "world": world,
                 "exit_codes": {str(r): c for r, c in sorted(bad.items())}, "lost": lost})
            if restarts >= max_restarts:
                return 1
            restarts += 1
            if shrink:
                world = max(min_nproc, world - max(1, len(lost)))
            store.set("bitscom/launch/generation", str(restarts))
    finally:
        del store


def agent_store(timeout_s: float = 300.0):
    """In a child: a client of the launcher's store, or ``None`` when not started by it."""
    where = os.environ.get("BITSCOM_AGENT_STORE")
    if not where:
        return None
    import torch.distributed as dist

    host, port = where.rsplit(":", 1)
    return dist.TCPStore(host, int(port), is_master=False,
                         timeout=datetime.timedelta(seconds=timeout_s))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--nproc", type=int, required=True, help="ranks (one per GPU)")
    ap.add_argument("--min-nproc", type=int, default=None,
                    help="with --shrink: never restart with fewer ranks than this")
    ap.add_argument("--max-restarts", type=int, default=0)
    ap.add_argument("--shrink", action="store_true",
                    help="restart without the ranks that failed instead of with all of them")
    ap.add_argument("--grace", type=float, default=30.0,
                    help="seconds the other ranks get to stop by themselves after a failure")
    ap.add_argument("command", nargs=argparse.REMAINDER, help="-- program and its arguments")
    args = ap.parse_args(argv)
    command = args.command[1:] if args.command[:1] == ["--"] else args.command
    if not command:
        ap.error("no command given")

    def on_term(signum, frame):  # unwind through run()'s finally, which stops the children
        raise SystemExit(128 + signum)

    signal.signal(signal.SIGTERM, on_term)
    return run(command, args.nproc, min_nproc=args.min_nproc, max_restarts=args.max_restarts,
               shrink=args.shrink, grace_s=args.grace)


if __name__ == "__main__":
    raise SystemExit(main())
