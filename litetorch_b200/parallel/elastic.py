"""Elastic supervision of a single-node job: start the ranks, watch them, and when one fails restart the whole group.

    python -m litetorch_b200.parallel.elastic --nproc 8 --max-restarts 3 train.py --ckpt /data/run1

The launcher starts `nproc` copies of the script with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT set (the
contract of `torch.distributed.run`, so the same script runs under either), plus LT_ELASTIC_ATTEMPT (0 on the first
start) and LT_ELASTIC_STORE_PORT.  A failure is a rank that exits with a non-zero code, or - when the workers called
`start_heartbeat()` - a rank whose heartbeat in the launcher's TCP store is older than `heartbeat_ttl_s` (a hung rank
that would otherwise keep its peers waiting inside a collective until the process-group timeout).  On a failure the
launcher stops the remaining ranks (the exact process groups it started: SIGTERM, then SIGKILL after a few seconds),
picks fresh ports and starts the group again, up to `max_restarts` times; the script is expected to resume from its last
checkpoint (`Trainer.save` / `Trainer.load` write and read one consistent set of per-rank files).

The reference has no counterpart: a short read on one of its sockets throws, its shared-memory barrier spins for ever and
nothing restarts (src/distributed/distributed.cpp:253-266, src/distributed/shm_ipc.cpp:188-192).  Failures are made and
handled on the host only; nothing here touches a GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
from typing import Dict, List, Optional, Sequence

from .process_group import TCPStore, Watchdog


def worker_info() -> Dict[str, int]:
    """What the launcher told this worker: rank, world size, attempt number (0 = first start)."""
    return {"rank": int(os.environ.get("RANK", 0)), "world": int(os.environ.get("WORLD_SIZE", 1)),
            "attempt": int(os.environ.get("LT_ELASTIC_ATTEMPT", 0))}


def start_heartbeat(interval_s: float = 0.25) -> Optional[Watchdog]:
    """Called by a worker: beat in the launcher's store until the process ends (or `.stop()`); None when the process was
    not started by the launcher."""
    port = os.environ.get("LT_ELASTIC_STORE_PORT")
    if not port:
        return None
    store = TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"), int(port), is_server=False)
    return Watchdog(store, int(os.environ.get("RANK", 0)), interval_s=interval_s)


class ElasticLauncher:
    def __init__(self, argv: Sequence[str], nproc: int, max_restarts: int = 3, master_addr: str = "127.0.0.1", base_port: int = 29600,
                 heartbeat_ttl_s: float = 10.0, start_grace_s: float = 120.0, poll_s: float = 0.1, stop_grace_s: float = 5.0,
                 env: Optional[Dict[str, str]] = None, log_dir: Optional[str] = None, shrink_after: int = 0, min_nproc: int = 1,
                 ckpt_dir: Optional[str] = None, tp: int = 1):
        """shrink_after = k > 0: after k failed attempts in a row at the current size the group restarts with half the
        ranks (not below `min_nproc`, and a multiple of `tp`): a job that lost a GPU for good continues on the rest.  With
        `ckpt_dir` the newest trainer checkpoint there is first re-cut for the new world size
        (`checkpoint_tools.reshard`), so the script resumes as usual."""
        self.shrink_after, self.min_nproc, self.ckpt_dir, self.tp = int(shrink_after), max(1, int(min_nproc)), ckpt_dir, max(1, int(tp))
        self.argv, self.nproc, self.max_restarts = list(argv), nproc, max_restarts
        self.addr, self.base_port = master_addr, base_port
        self.ttl, self.start_grace, self.poll, self.stop_grace = heartbeat_ttl_s, start_grace_s, poll_s, stop_grace_s
        self.env = dict(os.environ if env is None else env)
        self.log_dir = log_dir
        self.attempts: List[Dict] = []

    # ------------------------------------------------------------------ one attempt
    def _spawn(self, attempt: int, port: int):
        procs, logs = [], []
        for r in range(self.nproc):
            env = dict(self.env, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(self.nproc), LOCAL_WORLD_SIZE=str(self.nproc),
                       MASTER_ADDR=self.addr, MASTER_PORT=str(port), LT_ELASTIC_ATTEMPT=str(attempt),
                       LT_ELASTIC_STORE_PORT=str(port + 2))
            out = None
            if self.log_dir:
                os.makedirs(self.log_dir, exist_ok=True)
                out = open(os.path.join(self.log_dir, "attempt%d_rank%d.log" % (attempt, r)), "w")
                logs.append(out)
            # its own session: the launcher signals exactly this process group, nothing found by name
            procs.append(subprocess.Popen(self.argv, env=env, stdout=out, stderr=subprocess.STDOUT if out else None,
                                          start_new_session=True))
        return procs, logs

    def _stop(self, procs):
        for p in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except (ProcessLookupError, PermissionError):
                    pass
        t_end = time.monotonic() + self.stop_grace
        for p in procs:
            while p.poll() is None and time.monotonic() < t_end:
                time.sleep(0.05)
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except (ProcessLookupError, PermissionError):
                    pass
                p.wait()

    def _attempt(self, attempt: int) -> Dict:
        port = self.base_port + 4 * attempt            # rendezvous, the job's own store (port + 1), the launcher's store (port + 2)
        store = TCPStore(self.addr, port + 2, is_server=True)
        procs, logs = self._spawn(attempt, port)
        t0 = time.monotonic()
        reason, beating = None, False
        try:
            while reason is None:
                codes = [p.poll() for p in procs]
                bad = [r for r, c in enumerate(codes) if c not in (None, 0)]
                if bad:
                    reason = "rank %d exited with code %d" % (bad[0], codes[bad[0]])
                    break
                if all(c == 0 for c in codes):
                    break
                # heartbeats: only ranks that are still running can be "hung"; a rank that has finished stops beating
                try:
                    running = [r for r, c in enumerate(codes) if c is None]
                    silent_now = set(store.silent_ranks(self.nproc, self.ttl))
                    if len(silent_now) < self.nproc:
                        beating = True                   # somebody beats: the script uses start_heartbeat()
                    if beating:
                        late = [r for r in running if r in silent_now]
                        started = time.monotonic() - t0 >= self.start_grace
                        known_dead = [r for r in running if r in set(store.dead_ranks(self.ttl))]
                        hung = known_dead or (late if started else [])
                        if hung:
                            reason = "rank %d stopped sending heartbeats (ttl %.1f s)" % (hung[0], self.ttl)
                            break
                except Exception:
                    pass
                time.sleep(self.poll)
        finally:
            self._stop(procs)
            store.close()
            for f in logs:
                f.close()
        rec = {"attempt": attempt, "nproc": self.nproc, "returncodes": [p.returncode for p in procs], "reason": reason,
               "seconds": round(time.monotonic() - t0, 3)}
        self.attempts.append(rec)
        return rec

    # ------------------------------------------------------------------ the job
    def _shrink(self) -> bool:
        """Halve the group (a multiple of tp, at least min_nproc) and re-cut the newest checkpoint for it."""
        new = max(self.min_nproc, (self.nproc // 2) // self.tp * self.tp, self.tp)
        if new >= self.nproc:
            return False
        if self.ckpt_dir:
            from .. import checkpoint_tools as tools
            from ..trainer import Trainer
            if Trainer.latest_checkpoint(self.ckpt_dir):
                import shutil
                staged = self.ckpt_dir.rstrip("/") + ".resharded"
                shutil.rmtree(staged, ignore_errors=True)
                tools.reshard(self.ckpt_dir, staged, world=new, tp=self.tp)
                kept = self.ckpt_dir.rstrip("/") + ".world%d" % self.nproc      # the old cut stays beside it
                shutil.rmtree(kept, ignore_errors=True)
                os.replace(self.ckpt_dir, kept)
                os.replace(staged, self.ckpt_dir)
        self.nproc = new
        return True

    def run(self) -> Dict:
        failed_here = 0
        for attempt in range(self.max_restarts + 1):
            rec = self._attempt(attempt)
            if rec["reason"] is None:
                return {"ok": True, "restarts": attempt, "nproc": self.nproc, "attempts": self.attempts}
            failed_here += 1
            if self.shrink_after and failed_here >= self.shrink_after and attempt < self.max_restarts and self._shrink():
                failed_here = 0
        return {"ok": False, "restarts": self.max_restarts, "nproc": self.nproc, "attempts": self.attempts}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--nproc", type=int, required=True)
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--base-port", type=int, default=29600)
    ap.add_argument("--heartbeat-ttl", type=float, default=10.0)
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--shrink-after", type=int, default=0, help="failed attempts at one size before the group is halved (0: never)")
    ap.add_argument("--min-nproc", type=int, default=1)
    ap.add_argument("--ckpt", default=None, help="trainer checkpoint directory to re-cut when the group shrinks")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel width of the job (group sizes stay multiples of it)")
    ap.add_argument("script")
    ap.add_argument("args", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    res = ElasticLauncher([sys.executable, a.script] + a.args, a.nproc, a.max_restarts, a.master_addr, a.base_port, a.heartbeat_ttl,
                          log_dir=a.log_dir, shrink_after=a.shrink_after, min_nproc=a.min_nproc, ckpt_dir=a.ckpt, tp=a.tp).run()
    print(json.dumps(res))
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
