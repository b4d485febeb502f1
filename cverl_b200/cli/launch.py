"""One process per rank, supervised: per-rank logs, failure detection, restart from the latest checkpoint.

    python -m cverl_b200.cli.launch --nproc 8 --max-restarts 2 --log-dir /tmp/run1 -- \
        -m cverl_b200.trainer.ppo_trainer --dp-size 4 --tp-size 2 --checkpoint-dir ckpt --checkpoint-every 50 ...

The reference starts its ranks from a bash loop (``&`` + ``wait``), writes one log per rank and concatenates
them at the end (tools/distributed/run_qwen_pp_tp_ppo_trainer.sh:66-128); a rank that dies leaves its peers
blocked in NCCL and the script waiting for ever.  This launcher keeps the same shape - one child per rank with
``RANK`` / ``LOCAL_RANK`` / ``WORLD_SIZE`` / ``MASTER_ADDR`` / ``MASTER_PORT`` in its environment, one log per
rank - and adds the supervision:

* a child that exits non-zero ends the attempt: its peers get ``--grace-s`` seconds to notice by themselves (the
  trainer's heartbeat watchdog, a process-group timeout), then they are terminated - each by the process group
  this launcher created for it, never by a name pattern;
* ``--stall-timeout-s``: no rank has written to its log for that long (a process that is alive but stuck);
* ``--attempt-timeout-s``: a limit on one attempt as a whole;
* ``--max-restarts``: a failed attempt is started again on a fresh rendezvous port, and when the command names a
  ``--checkpoint-dir`` that holds a complete checkpoint the children get ``--resume-checkpoint <step dir>``.  The
  newest step directory whose manifest is marked complete and whose rank files all exist is chosen, so a
  checkpoint that the failure interrupted half-way is skipped.

With ``--nnodes > 1`` one launcher runs per node (``--node-rank``); each supervises and restarts its own ranks, a
failure on one node reaches the others through their ranks (watchdog, process-group timeout), and attempt ``k``
uses ``--master-port + k * --port-stride`` on every node, so the restarted attempts meet again.

Everything here is host code: no CUDA call, no device state.  The last line printed is a JSON summary of the
attempts.  Exit code: 0 when an attempt finished with every rank at 0, otherwise the first failing rank's code
(124 for a stall or a timeout).
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import threading
import time
from pathlib import Path
from typing import Dict, List, Optional, Sequence

STALL_CODE = 124


def newest_complete_checkpoint(ckpt_dir) -> Optional[Path]:
    """The newest ``step_*`` directory under ``ckpt_dir`` that can be resumed from: ``manifest.json`` parses, is
    marked ``complete`` and every file named in ``rank_files`` exists.  ``latest_checkpoint.txt`` is only a hint
    (it is written last, but a damaged or missing manifest behind it must not stop a restart)."""
    root = Path(ckpt_dir)
    if not root.is_dir():
        return None
    steps = sorted((d for d in root.iterdir() if d.is_dir() and d.name.startswith("step_")), reverse=True)
    for d in steps:
        try:
            manifest = json.loads((d / "manifest.json").read_text())
        except (OSError, ValueError):
            continue
        if not isinstance(manifest, dict) or not manifest.get("complete", False):
            continue
        ok = True
        for entry in manifest.get("rank_files", []):
            names = [entry] if isinstance(entry, str) else [entry.get("param_file"), entry.get("metadata_file")]
            for name in names:
                if name and not (d / name).exists():
                    ok = False
        if ok:
            return d
    return None


def with_option(command: Sequence[str], flag: str, value: str) -> List[str]:
    """``command`` with ``flag value`` set: replaces ``flag X`` / ``flag=X`` when present, else appends."""
    out, i, done = [], 0, False
    while i < len(command):
        tok = command[i]
        if tok == flag and i + 1 < len(command):
            out += [flag, value]
            i, done = i + 2, True
            continue
        if tok.startswith(flag + "="):
            out.append(f"{flag}={value}")
            i, done = i + 1, True
            continue
        out.append(tok)
        i += 1
    return out if done else out + [flag, value]


def option_value(command: Sequence[str], flag: str) -> Optional[str]:
    for i, tok in enumerate(command):
        if tok == flag and i + 1 < len(command):
            return command[i + 1]
        if tok.startswith(flag + "="):
            return tok.split("=", 1)[1]
    return None


def child_argv(program: Sequence[str]) -> List[str]:
    """``-m pkg.mod args`` and ``script.py args`` run under this interpreter; anything else is run as given."""
    if not program:
        raise ValueError("no program given after '--'")
    if program[0] == "-m" or program[0].endswith(".py"):
        return [sys.executable, "-u", *program]
    return list(program)


class _Rank:
    def __init__(self, rank: int, proc: subprocess.Popen, log: Path, handle):
        self.rank, self.proc, self.log, self.handle = rank, proc, log, handle
        self.code: Optional[int] = None


class Attempt:
    """One start of all local ranks.  ``run`` returns a dict: ``ok``, ``cause``, ``rank``, ``code``, ``seconds``."""

    def __init__(self, args, program: Sequence[str], attempt: int, log_dir: Path, out=sys.stdout):
        self.args, self.program, self.attempt, self.log_dir, self.out = args, list(program), attempt, log_dir, out
        self.ranks: List[_Rank] = []
        self._stop_tail = threading.Event()
        self._tail_thread: Optional[threading.Thread] = None
        self._wall0 = 0.0                    # wall clock at start: log mtimes are compared with it

    def _env(self, local_rank: int) -> Dict[str, str]:
        a = self.args
        env = dict(os.environ)
        world = a.nnodes * a.nproc
        env.update({
            "RANK": str(a.node_rank * a.nproc + local_rank), "LOCAL_RANK": str(local_rank), "WORLD_SIZE": str(world),
            "LOCAL_WORLD_SIZE": str(a.nproc), "NODE_RANK": str(a.node_rank), "GROUP_RANK": str(a.node_rank),
            "MASTER_ADDR": a.master_addr, "MASTER_PORT": str(a.master_port + self.attempt * a.port_stride),
            "CVERL_LAUNCH_ATTEMPT": str(self.attempt), "CVERL_LAUNCH_MAX_RESTARTS": str(a.max_restarts),
            "PYTHONUNBUFFERED": "1",
        })
        return env

    def start(self) -> None:
        self.log_dir.mkdir(parents=True, exist_ok=True)
        self._wall0 = time.time()
        argv = child_argv(self.program)
        for lr in range(self.args.nproc):
            log = self.log_dir / f"rank_{self.args.node_rank * self.args.nproc + lr}.log"
            handle = open(log, "wb")
            try:
                proc = subprocess.Popen(argv, env=self._env(lr), stdout=handle, stderr=subprocess.STDOUT,
                                        stdin=subprocess.DEVNULL, start_new_session=True)
            except OSError as exc:             # the program cannot be started at all: end what already runs
                handle.close()
                self.terminate()
                raise RuntimeError(f"cannot start {argv[0]!r}: {exc}") from exc
            self.ranks.append(_Rank(self.args.node_rank * self.args.nproc + lr, proc, log, handle))
        if self.args.tee_rank >= 0:
            for r in self.ranks:
                if r.rank == self.args.tee_rank:
                    self._tail_thread = threading.Thread(target=self._tail, args=(r,), daemon=True)
                    self._tail_thread.start()

    def _tail(self, r: _Rank) -> None:
        with open(r.log, "rb") as f:
            while True:
                line = f.readline()
                if line:
                    self.out.write(line.decode(errors="replace"))
                    self.out.flush()
                    continue
                if self._stop_tail.is_set():
                    return
                time.sleep(0.05)

    def _poll(self) -> None:
        for r in self.ranks:
            if r.code is None:
                r.code = r.proc.poll()

    def _running(self) -> List[_Rank]:
        return [r for r in self.ranks if r.code is None]

    def terminate(self, wait_s: float = 5.0) -> None:
        """Ends what is still running: SIGTERM to each child's own process group, SIGKILL after ``wait_s``."""
        for sig, pause in ((signal.SIGTERM, wait_s), (signal.SIGKILL, 2.0)):
            self._poll()
            alive = self._running()
            if not alive:
                break
            for r in alive:
                try:
                    os.killpg(r.proc.pid, sig)        # the group created by start_new_session: this rank only
                except (ProcessLookupError, PermissionError):
                    pass
            deadline = time.monotonic() + pause
            while self._running() and time.monotonic() < deadline:
                time.sleep(0.05)
                self._poll()
        for r in self.ranks:
            if r.code is None:
                r.code = r.proc.wait()

    def _newest_log_write(self) -> float:
        newest = 0.0
        for r in self.ranks:
            try:
                newest = max(newest, r.log.stat().st_mtime)
            except OSError:
                pass
        return newest

    def run(self) -> dict:
        a = self.args
        t0 = time.monotonic()
        result = {"ok": False, "cause": "", "rank": -1, "code": 0}
        try:
            self.start()
        except RuntimeError as exc:
            for r in self.ranks:
                r.handle.close()
            result.update(cause=str(exc), code=127, seconds=round(time.monotonic() - t0, 3), exit_codes={})
            return result
        try:
            while True:
                self._poll()
                failed = [r for r in self.ranks if r.code not in (None, 0)]
                if failed:
                    first = failed[0]
                    result.update(cause="exit", rank=first.rank, code=first.code if first.code > 0 else 128 - first.code)
                    deadline = time.monotonic() + a.grace_s
                    while self._running() and time.monotonic() < deadline:     # peers may notice by themselves
                        time.sleep(0.05)
                        self._poll()
                    break
                if not self._running():
                    result.update(ok=True, cause="finished")
                    break
                now = time.monotonic()
                if a.attempt_timeout_s > 0 and now - t0 > a.attempt_timeout_s:
                    result.update(cause="attempt-timeout", code=STALL_CODE)
                    break
                if a.stall_timeout_s > 0 and time.time() - max(self._newest_log_write(), self._wall0) > a.stall_timeout_s:
                    result.update(cause="stall", code=STALL_CODE)
                    break
                time.sleep(a.poll_s)
        finally:
            self.terminate()
            self._stop_tail.set()
            if self._tail_thread is not None:
                self._tail_thread.join(timeout=5.0)      # lets the streamed rank's last lines out
            for r in self.ranks:
                r.handle.close()
        result["seconds"] = round(time.monotonic() - t0, 3)
        result["exit_codes"] = {str(r.rank): r.code for r in self.ranks}
        return result

    def log_tails(self, lines: int) -> str:
        """The end of every rank's log, in rank order (what the reference's launcher prints by ``cat``)."""
        parts = []
        for r in self.ranks:
            try:
                text = r.log.read_text(errors="replace").splitlines()[-lines:]
            except OSError:
                text = []
            parts.append(f"===== rank {r.rank} (exit {r.code}) : {r.log} =====\n" + "\n".join(text))
        return "\n".join(parts)


def supervise(args, program: Sequence[str], out=sys.stdout) -> dict:
    log_root = Path(args.log_dir) if args.log_dir else Path(os.environ.get("TMPDIR", "/tmp")) / f"cverl_launch_{os.getpid()}"
    program = list(program)
    ckpt_dir = args.resume_from or option_value(program, "--checkpoint-dir")
    history = []
    current: List[Optional[Attempt]] = [None]

    def on_signal(signum, _frame):
        if current[0] is not None:
            current[0].terminate()
        raise SystemExit(128 + signum)

    old = {}
    if threading.current_thread() is threading.main_thread():
        for s in (signal.SIGTERM, signal.SIGINT):
            old[s] = signal.signal(s, on_signal)
    try:
        for attempt in range(args.max_restarts + 1):
            resumed = None
            if attempt > 0 and ckpt_dir:
                step_dir = newest_complete_checkpoint(ckpt_dir)
                if step_dir is not None:
                    program = with_option(program, "--resume-checkpoint", str(step_dir))
                    resumed = str(step_dir)
            att = Attempt(args, program, attempt, log_root / f"attempt_{attempt}", out=out)
            current[0] = att
            res = att.run()
            res["attempt"], res["resumed_from"] = attempt, resumed
            history.append(res)
            if res["ok"] or res["code"] == 127:        # done, or a program that cannot be started: no point retrying
                if not res["ok"]:
                    print(f"[launch] {res['cause']}", file=out, flush=True)
                break
            print(f"[launch] attempt {attempt} failed: {res['cause']}"
                  + (f" (rank {res['rank']} exit {res['code']})" if res["rank"] >= 0 else "")
                  + (f"; restarting ({args.max_restarts - attempt} left)" if attempt < args.max_restarts else ""),
                  file=out, flush=True)
            if args.tail_lines > 0:
                print(att.log_tails(args.tail_lines), file=out, flush=True)
    finally:
        for s, h in old.items():
            signal.signal(s, h)
    ok = bool(history and history[-1]["ok"])
    return {"ok": ok, "attempts": history, "log_dir": str(log_root),
            "exit_code": 0 if ok else (history[-1]["code"] or 1)}


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="python -m cverl_b200.cli.launch", description=__doc__.split("\n\n")[0],
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--nproc", type=int, default=int(os.environ.get("LOCAL_WORLD_SIZE", "1")), help="ranks on this node")
    ap.add_argument("--nnodes", type=int, default=1)
    ap.add_argument("--node-rank", type=int, default=int(os.environ.get("NODE_RANK", "0")))
    ap.add_argument("--master-addr", default=os.environ.get("MASTER_ADDR", "127.0.0.1"))
    ap.add_argument("--master-port", type=int, default=int(os.environ.get("MASTER_PORT", "29500")))
    ap.add_argument("--port-stride", type=int, default=1, help="attempt k uses master-port + k * stride")
    ap.add_argument("--max-restarts", type=int, default=0)
    ap.add_argument("--grace-s", type=float, default=5.0, help="after a rank failed, time its peers get to exit by themselves")
    ap.add_argument("--stall-timeout-s", type=float, default=0.0, help="> 0: no rank log written for this long ends the attempt")
    ap.add_argument("--attempt-timeout-s", type=float, default=0.0)
    ap.add_argument("--poll-s", type=float, default=0.2)
    ap.add_argument("--log-dir", default="")
    ap.add_argument("--tee-rank", type=int, default=0, help="stream this rank's log to stdout (-1: none)")
    ap.add_argument("--tail-lines", type=int, default=40, help="lines of every rank's log printed after a failed attempt")
    ap.add_argument("--resume-from", default="", help="checkpoint directory for restarts (default: the command's --checkpoint-dir)")
    ap.add_argument("program", nargs=argparse.REMAINDER, help="-- -m module args | -- script.py args | -- executable args")
    return ap


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    program = list(args.program)
    if program and program[0] == "--":
        program = program[1:]
    if not program:
        print("launch: give the program after '--'", file=sys.stderr)
        return 2
    if args.nproc < 1 or args.nnodes < 1 or not (0 <= args.node_rank < args.nnodes) or args.max_restarts < 0:
        print("launch: --nproc / --nnodes >= 1, 0 <= --node-rank < --nnodes, --max-restarts >= 0", file=sys.stderr)
        return 2
    summary = supervise(args, program)
    print(json.dumps({"launch": summary}), flush=True)
    return int(summary["exit_code"])


if __name__ == "__main__":
    sys.exit(main())
