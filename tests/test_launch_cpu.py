"""The supervising launcher and host-side fault injection: a rank that exits, a rank that stalls, a damaged
checkpoint.  Every failure is made on the host, in gloo processes on CPU."""
import csv
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from cverl_b200.cli import launch
from cverl_b200.utils.fault_injection import ATTEMPT_ENV, ENV, HostFault, InjectedFault

ROOT = Path(__file__).resolve().parents[1]
TRAINER = ["-m", "cverl_b200.trainer.ppo_trainer", "--backend", "gloo", "--dtype", "float32", "--lr", "1e-3",
           "--dp", "2", "--micro-batches", "1", "--master-weights"]


def _launch(tmp_path, name, port, *launch_flags, program, fault="", timeout=300):
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=str(ROOT))
    env.pop(ENV, None)
    if fault:
        env[ENV] = fault
    cmd = [sys.executable, "-m", "cverl_b200.cli.launch", "--nproc", "2", "--master-port", str(port),
           "--log-dir", str(tmp_path / name), *launch_flags, "--", *program]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    last = [ln for ln in p.stdout.splitlines() if ln.startswith('{"launch"')]
    assert last, p.stdout[-3000:] + p.stderr[-3000:]
    return p, json.loads(last[-1])["launch"]


def test_command_line_helpers():
    cmd = ["-m", "mod", "--steps", "4", "--checkpoint-dir=ck"]
    assert launch.option_value(cmd, "--steps") == "4" and launch.option_value(cmd, "--checkpoint-dir") == "ck"
    assert launch.option_value(cmd, "--resume-checkpoint") is None
    assert launch.with_option(cmd, "--resume-checkpoint", "x")[-2:] == ["--resume-checkpoint", "x"]
    assert launch.with_option(cmd, "--steps", "9")[2:4] == ["--steps", "9"]
    assert launch.with_option(cmd, "--checkpoint-dir", "d")[-1] == "--checkpoint-dir=d"
    assert launch.child_argv(["-m", "a.b", "1"])[:3] == [sys.executable, "-u", "-m"]
    assert launch.child_argv(["tool.py"])[0] == sys.executable and launch.child_argv(["/bin/true"]) == ["/bin/true"]
    with pytest.raises(ValueError):
        launch.child_argv([])
    assert launch.main(["--nproc", "1"]) == 2                       # no program
    assert launch.main(["--nproc", "0", "--", "/bin/true"]) == 2    # bad geometry


def test_newest_complete_checkpoint_skips_damaged_ones(tmp_path):
    assert launch.newest_complete_checkpoint(tmp_path / "missing") is None

    def make(step, complete=True, files=("rank_0.pt", "rank_0.json")):
        d = tmp_path / f"step_{step:06d}"
        d.mkdir()
        for f in files:
            (d / f).write_bytes(b"x")
        (d / "manifest.json").write_text(json.dumps({
            "complete": complete, "rank_files": [{"param_file": "rank_0.pt", "metadata_file": "rank_0.json"}]}))
        return d
    a = make(2)
    b = make(4)
    assert launch.newest_complete_checkpoint(tmp_path) == b
    (b / "manifest.json").write_text("{ not json")                 # a manifest cut off by the failure
    assert launch.newest_complete_checkpoint(tmp_path) == a
    make(6, complete=False)                                         # written, never marked complete
    make(8, files=("rank_0.json",))                                 # a rank file is missing
    assert launch.newest_complete_checkpoint(tmp_path) == a
    (a / "rank_0.pt").unlink()
    assert launch.newest_complete_checkpoint(tmp_path) is None


def test_fault_specification_and_kinds():
    f = HostFault.parse("rank=1, step=2, kind=exit, code=9, attempt=1")
    assert (f.rank, f.step, f.kind, f.code, f.attempt) == (1, 2, "exit", 9, 1)
    for bad in ("rank=1,step=2", "rank=1,step=2,kind=explode", "rank=1,step=2,kind=exit,when=now", "rank"):
        with pytest.raises(ValueError):
            HostFault.parse(bad)
    assert HostFault.from_env({}) is None and HostFault.from_env({ENV: "rank=0,step=0,kind=raise"}).kind == "raise"
    assert f.due(1, 2, {ATTEMPT_ENV: "1"}) and not f.due(1, 2, {}) and not f.due(0, 2, {ATTEMPT_ENV: "1"})
    order = []
    g = HostFault(rank=0, step=3, kind="raise")
    g.fire(0, 2, sync=lambda: order.append("sync"))                 # not due: nothing happens
    assert order == []
    with pytest.raises(InjectedFault):
        g.fire(0, 3, sync=lambda: order.append("sync"))
    assert order == ["sync"]                                        # the device is drained before the rank leaves
    codes = []
    HostFault(rank=0, step=0, kind="exit", code=5).fire(0, 0, exit_fn=codes.append)
    assert codes == [5]

    class Woke(Exception):
        pass
    naps = []

    def nap(s):
        naps.append(s)
        if len(naps) == 3:
            raise Woke()
    with pytest.raises(Woke):
        HostFault(rank=0, step=0, kind="stall").fire(0, 0, sleep=nap)
    assert len(naps) == 3


def test_restart_resumes_from_the_latest_checkpoint(tmp_path):
    """Rank 1 is killed before step 2 of the first attempt; the job restarts, resumes from the step-2 checkpoint and
    ends with the same loss as a run that was never interrupted."""
    steps = ["--steps", "4", "--checkpoint-every", "1"]
    p0, clean = _launch(tmp_path, "clean", 29911, program=TRAINER + steps + [
        "--checkpoint-dir", str(tmp_path / "ck_clean"), "--metrics-csv", str(tmp_path / "clean.csv")])
    assert p0.returncode == 0 and clean["ok"] and len(clean["attempts"]) == 1
    p1, res = _launch(tmp_path, "faulty", 29921, "--max-restarts", "2", "--grace-s", "3", program=TRAINER + steps + [
        "--checkpoint-dir", str(tmp_path / "ck"), "--metrics-csv", str(tmp_path / "faulty.csv")],
        fault="rank=1,step=2,kind=exit,code=17")
    assert p1.returncode == 0 and res["ok"], p1.stdout[-3000:]
    first, second = res["attempts"]
    assert not first["ok"] and first["cause"] == "exit" and first["exit_codes"]["1"] == 17
    assert all(code is not None for code in first["exit_codes"].values())          # nobody left behind
    assert second["ok"] and second["resumed_from"].endswith("step_000002")
    assert "attempt 0 failed" in p1.stdout and "===== rank 1 (exit 17)" in p1.stdout
    with open(tmp_path / "clean.csv") as f:
        a = list(csv.DictReader(f))
    with open(tmp_path / "faulty.csv") as f:
        b = list(csv.DictReader(f))
    assert [r["step"] for r in a] == ["0", "1", "2", "3"] and [r["step"] for r in b] == ["0", "1", "2", "3"]
    for ra, rb in zip(a, b):
        assert float(ra["loss_sum"]) == pytest.approx(float(rb["loss_sum"]), rel=1e-5, abs=1e-7)
        assert float(ra["global_grad_norm"]) == pytest.approx(float(rb["global_grad_norm"]), rel=1e-4)
    assert (tmp_path / "faulty" / "attempt_0" / "rank_1.log").exists()
    assert (tmp_path / "faulty" / "attempt_1" / "rank_0.log").read_text().count("step=") == 2


def test_a_program_that_cannot_be_started_is_reported_not_retried(tmp_path):
    p, res = _launch(tmp_path, "nope", 29951, "--max-restarts", "3", program=["/no/such/program", "x"])
    assert p.returncode == 127 and not res["ok"] and len(res["attempts"]) == 1
    assert "cannot start" in res["attempts"][0]["cause"] and "cannot start" in p.stdout


def test_failure_without_restarts_returns_the_rank_exit_code(tmp_path):
    p, res = _launch(tmp_path, "once", 29931, "--grace-s", "2", program=TRAINER + ["--steps", "3"],
                     fault="rank=0,step=1,kind=exit,code=23")
    assert p.returncode == 23 and not res["ok"] and len(res["attempts"]) == 1
    assert res["attempts"][0]["rank"] == 0 and res["attempts"][0]["code"] == 23


def test_a_stalled_rank_ends_the_attempt(tmp_path):
    """A rank that is alive but makes no progress: its peer blocks in the next collective, no log moves, the
    supervisor ends both and reports a stall."""
    p, res = _launch(tmp_path, "stall", 29941, "--stall-timeout-s", "20", program=TRAINER + ["--steps", "50"],
                     fault="rank=1,step=1,kind=stall")
    assert p.returncode == launch.STALL_CODE and not res["ok"]
    att = res["attempts"][0]
    assert att["cause"] == "stall" and all(code is not None for code in att["exit_codes"].values())
    assert att["seconds"] < 120
