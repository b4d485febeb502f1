"""The distributed trainer as gloo processes: parallel configurations, PP parity, checkpoint / resume
equality, metrics CSV, and host-side failure detection."""
import csv
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _run(nproc, *flags, port=29650, timeout=240, check=True):
    trainer = ["-m", "cverl_b200.trainer.ppo_trainer", "--backend", "gloo", "--dtype", "float32", "--lr", "1e-3", *flags]
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=str(ROOT))
    if nproc == 1:          # one rank needs no launcher (and no rendezvous): several seconds less per run
        cmd = [sys.executable, *trainer]
        env.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), *trainer]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    if check:
        assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    return p


def _lines(p):
    out = []
    for ln in p.stdout.splitlines():
        if ln.startswith("step="):
            out.append(dict(kv.split("=", 1) for kv in ln.split()))
    return out


@pytest.mark.parametrize("nproc,flags", [
    (4, ["--pp", "2", "--tp", "2", "--micro-batches", "2"]),
    (2, ["--dp", "2", "--micro-batches", "2"]),
    (2, ["--cp", "2"]),
    (2, ["--ep", "2", "--config", "tiny_moe"]),
])
def test_parallel_configs_train(nproc, flags):
    p = _run(nproc, *flags, "--steps", "2", port=29650 + nproc + len(flags))
    rows = _lines(p)
    assert len(rows) == 2
    for r in rows:
        assert r["all_ranks_have_grad"] == "true" and r["all_ranks_updated"] == "true"
        assert "nan" not in r["loss_sum"] and "inf" not in r["global_grad_norm"]
        assert float(r["step_time_s"]) > 0


def test_checkpoint_resume_equality_and_formats(tmp_path):
    ck = tmp_path / "ck"
    csv_a, csv_b = tmp_path / "a.csv", tmp_path / "b.csv"
    base = ["--dp", "2", "--micro-batches", "1", "--master-weights"]
    full = _lines(_run(2, *base, "--steps", "4", "--metrics-csv", str(csv_a), port=29681))
    _run(2, *base, "--steps", "2", "--checkpoint-dir", str(ck), "--checkpoint-every", "2", port=29682)
    step_dir = ck / "step_000002"
    manifest = json.loads((step_dir / "manifest.json").read_text())
    assert manifest["complete"] and manifest["format"] == "cverl_pp_tp_flat_shard_checkpoint_v4"
    # the reference's key names and values (tools/model/qwen3_5_pp_tp_ppo_trainer.cc:1045-1104)
    assert manifest["step"] == 2 and manifest["optimizer_kind"] == "FlatAdamW" and manifest["use_master_weights"]
    assert manifest["model_parameters_saved"] is False and manifest["world_size"] == 2
    assert manifest["data_parallel"] == 2 and manifest["tensor_parallel"] == 1 and manifest["pipeline_parallel"] == 1
    assert manifest["optimizer"]["type"] == "FlatAdamW" and manifest["optimizer"]["step"] == 2
    assert manifest["rank_files"][1] == {"global_rank": 1, "expert_rank": 0, "tensor_rank": 0, "context_rank": 0,
                                         "pipeline_rank": 0, "data_rank": 1, "param_file": "rank_1.pt",
                                         "metadata_file": "rank_1.json"}
    assert (ck / "latest_checkpoint.txt").read_text().strip() == "step_000002"
    meta = json.loads((step_dir / "rank_1.json").read_text())
    fs = meta["flat_parameter_shard"]
    assert fs["shard_end"] - fs["shard_begin"] == fs["numel"] and meta["use_master_weights"] is True
    assert meta["optimizer_kind"] == "FlatAdamW" and meta["optimizer_step"] == 2 and meta["param_file"] == "rank_1.pt"
    assert fs["dtype"] == "Float" and meta["parameters"][0]["dtype"] in ("BFloat16", "Float") and meta["data_rank"] == 1
    assert meta["optimizer_param_indices"] == list(range(len(meta["parameters"])))
    from cverl_b200.utils.checkpoint import load_archive
    arch = load_archive(step_dir / "rank_0.pt")
    assert set(arch) == {"flat_param_shard", "flat_exp_avg", "flat_exp_avg_sq", "optim_step"}
    assert int(arch["optim_step"]) == 2 and arch["flat_param_shard"].dtype == torch.float32
    resumed = _lines(_run(2, *base, "--steps", "4", "--resume-checkpoint", str(ck), "--metrics-csv", str(csv_b),
                          port=29683))
    assert [r["step"] for r in resumed] == ["2", "3"]
    for ra, rb in zip(full[2:], resumed):
        assert float(ra["loss_sum"]) == pytest.approx(float(rb["loss_sum"]), rel=1e-5, abs=1e-7)
        assert float(ra["global_grad_norm"]) == pytest.approx(float(rb["global_grad_norm"]), rel=1e-4)
    with open(csv_a) as f:
        rows = list(csv.DictReader(f))
    assert len(rows) == 4 and rows[0]["dp"] == "2" and "step_time_s" in rows[0]
    # a different topology must be refused
    bad = _run(1, "--steps", "3", "--resume-checkpoint", str(ck), port=29684, check=False)
    assert bad.returncode != 0


def test_reads_an_archive_written_by_libtorch():
    """``tests/fixtures/libtorch_output_archive.pt`` was written by LibTorch's ``OutputArchive`` (tensors stored
    as module parameters; the generating program sits beside it): the reader must return every tensor."""
    from pathlib import Path
    from cverl_b200.utils.checkpoint import c10_dtype_name, load_archive, save_archive
    arch = load_archive(Path(__file__).parent / "fixtures" / "libtorch_output_archive.pt")
    assert set(arch) == {"flat_param_shard", "flat_exp_avg", "flat_exp_avg_sq", "param_0", "optim_step"}
    assert int(arch["optim_step"]) == 3 and arch["flat_param_shard"].dtype == torch.bfloat16
    assert torch.equal(arch["flat_exp_avg"], torch.arange(8).float() * 0.5)
    assert arch["param_0"].shape == (2, 3)
    assert c10_dtype_name(torch.bfloat16) == "BFloat16" and c10_dtype_name(torch.float32) == "Float"
    # and what this package writes has the same container layout: parameters, no buffers
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        save_archive(Path(d) / "a.pt", arch)
        mod = torch.jit.load(str(Path(d) / "a.pt"))
        assert sorted(n for n, _ in mod.named_parameters()) == sorted(arch) and not list(mod.named_buffers())


def test_libtorch_reads_an_archive_written_here(tmp_path):
    """The other direction: ``torch::serialize::InputArchive`` - the reader the reference's trainer resumes with -
    loads a rank archive written by ``save_archive`` and finds every key with its dtype and values.  The small
    reader (``tests/fixtures/read_archive_with_libtorch.cc``) is compiled against the installed LibTorch."""
    import shutil
    from torch.utils import cpp_extension
    from cverl_b200.utils.checkpoint import save_archive
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    tensors = {"flat_param_shard": torch.arange(8).float().mul(0.25).bfloat16(), "flat_exp_avg": torch.arange(8).float() * 0.5,
               "flat_exp_avg_sq": torch.arange(8).float() * 2.0, "optim_step": torch.tensor(3, dtype=torch.int64),
               "param_0": torch.arange(6).float().view(2, 3)}
    save_archive(tmp_path / "rank_0.pt", tensors)
    lib = Path(torch.__file__).parent / "lib"
    exe = tmp_path / "read_archive"
    cmd = ["g++", "-std=c++17", "-O1", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           str(Path(__file__).parent / "fixtures" / "read_archive_with_libtorch.cc"),
           *[f for i in cpp_extension.include_paths() for f in ("-I", i)], "-L", str(lib), "-ltorch", "-ltorch_cpu",
           "-lc10", f"-Wl,-rpath,{lib}", "-o", str(exe)]
    built = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if built.returncode != 0:
        pytest.skip("LibTorch headers / libraries are not usable from g++ here: " + built.stderr[-300:])
    p = subprocess.run([str(exe), str(tmp_path / "rank_0.pt"), *tensors], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr[-1000:]
    rows = {ln.split()[0]: ln.split()[1:] for ln in p.stdout.strip().splitlines()}
    assert rows["flat_param_shard"][0] == "c10::BFloat16" and rows["flat_param_shard"][-2:] == ["8", "7"]
    assert rows["flat_exp_avg"][-2:] == ["8", "14"] and rows["flat_exp_avg_sq"][-2:] == ["8", "56"]
    assert rows["optim_step"][-2:] == ["1", "3"] and "long" in " ".join(rows["optim_step"])
    assert rows["param_0"][-2:] == ["6", "15"]


def test_resume_refuses_damaged_checkpoints(tmp_path):
    """Host-side fault injection on the checkpoint: an incomplete manifest, a manifest whose step disagrees with
    the archive, and a missing rank file must each stop the resume with an error instead of training on."""
    import shutil
    ck = tmp_path / "ck"
    _run(1, "--steps", "2", "--checkpoint-dir", str(ck), "--checkpoint-every", "2", port=29686)
    step_dir = ck / "step_000002"
    good = json.loads((step_dir / "manifest.json").read_text())

    def resume_fails(mutate):
        work = tmp_path / "work"
        if work.exists():
            shutil.rmtree(work)
        shutil.copytree(ck, work)
        mutate(work / "step_000002")
        p = _run(1, "--steps", "3", "--resume-checkpoint", str(work), port=29687, check=False)
        assert p.returncode != 0, p.stdout[-500:]

    resume_fails(lambda d: (d / "manifest.json").write_text(json.dumps(dict(good, complete=False))))
    resume_fails(lambda d: (d / "manifest.json").write_text(
        json.dumps(dict(good, optimizer=dict(good["optimizer"], step=7)))))
    resume_fails(lambda d: (d / "manifest.json").write_text(json.dumps(dict(good, optimizer_kind="flat_adamw"))))
    resume_fails(lambda d: (d / "rank_0.pt").unlink())
    # the untouched checkpoint still resumes
    ok = _lines(_run(1, "--steps", "3", "--resume-checkpoint", str(ck), port=29688))
    assert [r["step"] for r in ok] == ["2"]


def test_sft_jsonl_mode(tmp_path):
    data = tmp_path / "sft.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"q{i}?", "answer": f"a{i}"}) for i in range(8)))
    rows = _lines(_run(1, "--mode", "sft", "--sft-jsonl", str(data), "--steps", "3", "--lr", "5e-3", port=29691))
    losses = [float(r["loss_sum"]) for r in rows]
    assert losses[0] > 0 and losses[-1] < losses[0]


def test_watchdog_detects_silent_and_failed_peers():
    from cverl_b200.utils.watchdog import DictStore, Heartbeat, PeerFailure, Watchdog, guarded
    store = DictStore()
    now = [100.0]
    hbs = [Heartbeat(store, r, 3) for r in range(3)]
    for h in hbs:
        h.beat(0)
    wd = Watchdog(hbs[0], timeout_s=5.0, clock=lambda: now[0])
    wd.check()                                     # everybody alive
    now[0] += 60.0                                 # peers stop beating: a rank that never joins the step
    with pytest.raises(PeerFailure) as e:
        wd.check()
    assert e.value.ranks == [1, 2]
    # silence is judged by the observer's clock: a peer whose own wall clock is far off is fine while it beats
    hbs[1].beat(1)
    hbs[2].beat(1)
    wd.check()
    # a dropped message: rank 2's heartbeat key is lost in the store
    store2 = DictStore()
    store2.dropped.add("cverl/hb/beat/2")
    hb2 = [Heartbeat(store2, r, 3) for r in range(3)]
    for h in hb2:
        h.beat(0)
    t2 = [0.0]
    wd2 = Watchdog(hb2[0], 5.0, clock=lambda: t2[0])
    wd2.check()                                    # inside the grace period a missing first beat is not a failure
    t2[0] = 6.0
    hb2[1].beat(1)                                 # rank 1 is alive and its message arrives; rank 2's never does
    with pytest.raises(PeerFailure) as e:
        wd2.check()
    assert e.value.ranks == [2]
    # a rank that raises publishes the failure before exiting

    @guarded(hbs[1])
    def failing_rank():
        raise ValueError("bad batch")
    with pytest.raises(ValueError):
        failing_rank()
    with pytest.raises(PeerFailure) as e:
        wd.check()
    assert e.value.ranks == [1] and "bad batch" in e.value.reason


def test_watchdog_startup_race_and_long_steps():
    """A peer still building its model has no beat yet: the first check waits for it instead of reporting
    it; and a step far longer than the timeout is not a failure while the peer's host thread keeps beating."""
    import threading
    import time as _t
    from cverl_b200.utils.watchdog import DictStore, Heartbeat, PeerFailure, Watchdog
    store = DictStore()
    hb0, hb1 = Heartbeat(store, 0, 2), Heartbeat(store, 1, 2)
    hb0.beat(0)
    late = threading.Timer(0.3, lambda: hb1.beat(0))          # rank 1 arrives 0.3 s late
    late.start()
    wd = Watchdog(hb0, timeout_s=0.2)
    wd.wait_for_peers(timeout_s=5.0)                            # returns once rank 1 has beaten
    late.join()
    wd.check()
    # rank 1 now runs a "step" of 1 s (5x the timeout) with its background thread beating
    hb1.start_background(0.05)
    _t.sleep(1.0)
    wd.check()
    hb1.stop()
    _t.sleep(0.5)                                               # the thread is gone: now it is silent
    with pytest.raises(PeerFailure) as e:
        wd.check()
    assert e.value.ranks == [1]
    # a peer that never shows up at all is reported by the start-up wait
    store3 = DictStore()
    lone = Watchdog(Heartbeat(store3, 0, 2), timeout_s=0.2)
    with pytest.raises(PeerFailure) as e:
        lone.wait_for_peers(timeout_s=0.3)
    assert e.value.ranks == [1]


def test_simple_grpo_trainer_learns_and_resumes(tmp_path):
    from cverl_b200.trainer.simple_grpo import SimpleGrpoTrainer, SimpleGrpoTrainerConfig
    cfg = SimpleGrpoTrainerConfig(steps=30, prompts_per_batch=8, responses_per_prompt=4, seq_len=6, action_dim=6,
                                  hidden_dim=32, seed=3)
    tr = SimpleGrpoTrainer(cfg)
    ms = tr.train()
    assert ms[-1].step == 30 and tr.current_step() == 30
    assert sum(m.avg_reward for m in ms[-5:]) > sum(m.avg_reward for m in ms[:5])   # it learns the copy task
    prefix = str(tmp_path / "toy")
    tr.save_checkpoint(prefix)
    for suffix in (".model.pt", ".optim.pt", ".meta.pt"):
        assert (tmp_path / ("toy" + suffix)).exists()
    a = tr.train_step()
    tr2 = SimpleGrpoTrainer(cfg)
    tr2.load_checkpoint(prefix)
    assert tr2.current_step() == 30
    b = tr2.train_step()
    assert a.step == b.step == 31
    assert a.loss == pytest.approx(b.loss, rel=1e-5, abs=1e-7) and a.avg_reward == pytest.approx(b.avg_reward)


def test_gsm8k_grpo_cli_tiny_policy(tmp_path, capsys):
    from cverl_b200.trainer import gsm8k_grpo
    data = tmp_path / "gsm.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"What is {i}+{i}?", "answer": f"#### {2 * i}"}) for i in range(6)))
    rc = gsm8k_grpo.main(["--dataset", str(data), "--prompts", "2", "--n", "3", "--steps", "2", "--max-tokens", "8",
                          "--max-response-tokens", "8", "--max-prompt-tokens", "24", "--kl-coef", "0.01",
                          "--kl-penalty", "k3"])
    assert rc == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert lines[0] == gsm8k_grpo.CSV_HEADER and len(lines) == 3
    row = lines[1].split(",")
    assert row[0] == "1" and row[1] == "6"
    assert all(v == v and abs(v) < 1e6 for v in map(float, row[3:]))         # finite metrics


def test_grpo_update_moves_parameters_toward_rewarded_responses():
    from cverl_b200.models.policy import TinyCausalLmPolicy
    from cverl_b200.rollout.rollout_batch import RolloutBatch
    from cverl_b200.trainer.gsm8k_grpo import GrpoUpdateConfig, grpo_update
    torch.manual_seed(0)
    pol = TinyCausalLmPolicy(vocab_size=32, hidden_size=16)
    ref = pol.clone_as_reference()
    opt = torch.optim.AdamW(pol.parameters(), lr=1e-2)
    B, P, R = 8, 5, 6
    batch = RolloutBatch(torch.randint(1, 32, (B, P)), torch.randint(1, 32, (B, R)), torch.ones(B, R),
                         torch.zeros(B, R), torch.zeros(B), torch.arange(B) // 4)
    batch.rewards[::2] = 1.0
    batch.token_rewards[:, -1] = batch.rewards
    before = pol.response_log_probs(batch.prompt_ids, batch.response_ids).detach().sum(-1)
    m = grpo_update(pol, ref, opt, batch, GrpoUpdateConfig(ppo_epochs=3, kl_coef=0.01, kl_penalty="k3"))
    after = pol.response_log_probs(batch.prompt_ids, batch.response_ids).detach().sum(-1)
    assert m["param_delta"] > 0 and m["kl_loss"] >= 0
    assert (after - before)[::2].mean() > (after - before)[1::2].mean()        # rewarded responses gained likelihood


def test_optimizer_modes_agree_and_v2_checkpoint_resumes(tmp_path):
    """Flat ZeRO shard, ZeRO-1 with per-parameter owners and the unsharded bucketed all-reduce are the same
    AdamW: two data-parallel ranks reach the same losses in all three modes; the non-flat mode writes the
    rank-local v2 checkpoint and resumes from it to the same trajectory."""
    base = ["--dp", "2", "--micro-batches", "2", "--steps", "4", "--dp-grad-bucket-mb", "1"]
    flat = _lines(_run(2, *base, port=29701))
    zero1 = _lines(_run(2, *base, "--dp-shard-optimizer", "true", "--dp-flat-shard-optimizer", "false", port=29702))
    dense = _lines(_run(2, *base, "--dp-shard-optimizer", "false", port=29703))
    assert [r["flat_shard_optimizer"] for r in (flat[0], zero1[0], dense[0])] == ["true", "false", "false"]
    assert [r["dp_shard_optimizer"] for r in (flat[0], zero1[0], dense[0])] == ["true", "true", "false"]
    for a, b, c in zip(flat, zero1, dense):
        for other in (b, c):
            assert float(a["loss_sum"]) == pytest.approx(float(other["loss_sum"]), rel=2e-4, abs=1e-6)
            assert float(a["global_grad_norm"]) == pytest.approx(float(other["global_grad_norm"]), rel=1e-3)
    ck = tmp_path / "ck2"
    mode = ["--dp-shard-optimizer", "true", "--dp-flat-shard-optimizer", "false", "--master-weights", "true"]
    full = _lines(_run(2, *base, *mode, port=29704))
    _run(2, *base[:-4], "--steps", "2", "--dp-grad-bucket-mb", "1", *mode, "--checkpoint-dir", str(ck),
         "--checkpoint-every", "2", port=29705)
    d = ck / "step_000002"
    manifest = json.loads((d / "manifest.json").read_text())
    assert manifest["format"] == "cverl_pp_tp_rank_local_checkpoint_v2" and manifest["optimizer"]["type"] == "Fp32MasterAdamW"
    metas = [json.loads((d / f"rank_{r}.json").read_text()) for r in range(2)]
    owned = [set(m["optimizer_param_indices"]) for m in metas]
    assert owned[0] and owned[1] and not (owned[0] & owned[1])          # every parameter has exactly one owner
    assert owned[0] | owned[1] == set(range(len(metas[0]["parameters"])))
    from cverl_b200.utils.checkpoint import load_archive
    arch = load_archive(d / "rank_0.pt")
    assert "param_0" in arch and "optim_exp_avg_0" in arch and int(arch["optim_step"]) == 2
    k = metas[0]["optimizer_param_indices"][0]
    assert arch[f"param_{k}"].dtype == torch.float32                    # the owner's fp32 master copy
    resumed = _lines(_run(2, *base, *mode, "--resume-checkpoint", str(ck), port=29706))
    assert [r["step"] for r in resumed] == ["2", "3"]
    for ra, rb in zip(full[2:], resumed):
        assert float(ra["loss_sum"]) == pytest.approx(float(rb["loss_sum"]), rel=1e-5, abs=1e-7)


def test_rollout_batches_over_a_file_rendezvous_communicator(tmp_path):
    """A rollout source started on its own sends ``GpuRolloutBatch`` to two trainer ranks over a communicator
    that rendezvouses through a file; the trainer reports the batch's reward metrics, and uses the reference
    log-probs it carries for the KL term."""
    idf = tmp_path / "rollout_world.id"
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=str(ROOT))
    src = subprocess.Popen([sys.executable, "-m", "cverl_b200.cli.rollout_batch_source", "--id-file", str(idf),
                            "--rank", "0", "--world-size", "3", "--target-ranks", "1,2", "--steps", "2", "--batch", "4",
                            "--prompt-len", "8", "--response-len", "8", "--backend", "gloo", "--with-ref-log-probs"],
                           cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        p = _run(2, "--dp", "2", "--micro-batches", "2", "--steps", "2", "--rollout-nccl-id-file", str(idf),
                 "--rollout-nccl-world-size", "3", "--rollout-nccl-rank-offset", "1", "--rollout-nccl-source-rank", "0",
                 "--kl-coef", "0.1", "--kl-penalty", "k3", port=29711)
        out, err = src.communicate(timeout=60)
    finally:
        if src.poll() is None:
            src.kill()
    assert src.returncode == 0, out[-1000:] + err[-2000:]
    rows = _lines(p)
    assert len(rows) == 2 and rows[0]["rollout_rows"] == "4"
    assert float(rows[0]["mean_reward"]) == pytest.approx(0.5) and float(rows[0]["success_rate"]) == pytest.approx(0.5)
    assert float(rows[0]["adv_abs_sum"]) == pytest.approx(32.0)          # 4 rows x 8 tokens of +-1
    assert float(rows[0]["kl_loss_sum"]) > 0                             # reference log-probs reached the loss


def test_kl_needs_reference_log_probs():
    p = _run(1, "--steps", "1", "--kl-coef", "0.1", port=29713, check=False)
    assert p.returncode != 0 and "ref_log_probs" in (p.stdout + p.stderr)


def test_zero_stage2_matches_stage1_and_resumes(tmp_path):
    """--zero-stage 2 (per-layer gradient buckets reduced during the backward pass, bucket-sharded optimizer state)
    is the same AdamW as the flat shard: same losses on two data-parallel ranks, and it resumes from its own
    checkpoint onto the same trajectory."""
    base = ["--dp", "2", "--micro-batches", "2", "--steps", "4"]
    flat = _lines(_run(2, *base, port=29711))
    z2 = _lines(_run(2, *base, "--zero-stage", "2", port=29712))
    for a, b in zip(flat, z2):
        assert float(a["loss_sum"]) == pytest.approx(float(b["loss_sum"]), rel=2e-4, abs=1e-6)
        assert float(a["global_grad_norm"]) == pytest.approx(float(b["global_grad_norm"]), rel=1e-3)
        assert b["all_ranks_updated"] == "true"
    ck = tmp_path / "ckz2"
    _run(2, "--dp", "2", "--micro-batches", "2", "--steps", "2", "--zero-stage", "2", "--checkpoint-dir", str(ck),
         "--checkpoint-every", "2", port=29713)
    meta = json.loads((ck / "step_000002" / "rank_1.json").read_text())
    assert meta["flat_parameter_shard"]["layout"] == "bucketed"
    resumed = _lines(_run(2, *base, "--zero-stage", "2", "--resume-checkpoint", str(ck), port=29714))
    assert [r["step"] for r in resumed] == ["2", "3"]
    for ra, rb in zip(z2[2:], resumed):
        assert float(ra["loss_sum"]) == pytest.approx(float(rb["loss_sum"]), rel=1e-5, abs=1e-7)
    bad = _run(2, "--dp", "2", "--dp-flat-shard-optimizer", "false", "--zero-stage", "2", port=29715, check=False)
    assert bad.returncode != 0 and "--zero-stage 2 needs" in (bad.stdout + bad.stderr)


def test_context_parallel_attention_layouts_agree_in_the_trainer():
    """--cp-attn zigzag (resharded, load-balanced ring) and --cp-attn ring (contiguous shards) are the same attention:
    two context-parallel ranks reach the same losses and gradient norms."""
    base = ["--cp", "2", "--steps", "3", "--prompt-len", "8", "--response-len", "8"]
    zig = _lines(_run(2, *base, "--cp-attn", "zigzag", port=29721))
    ring = _lines(_run(2, *base, "--cp-attn", "ring", port=29722))
    assert len(zig) == len(ring) == 3
    for a, b in zip(zig, ring):
        assert float(a["loss_sum"]) == pytest.approx(float(b["loss_sum"]), rel=2e-4, abs=1e-6)
        assert float(a["global_grad_norm"]) == pytest.approx(float(b["global_grad_norm"]), rel=1e-3)


@pytest.mark.parametrize("nproc,flags,port", [
    (2, ["--pp", "2", "--micro-batches", "2"], 29731),
    (2, ["--cp", "2"], 29733),
    (2, ["--dp", "2", "--zero-stage", "2"], 29735),
])
def test_activation_checkpointing_changes_no_number(nproc, flags, port):
    """Layers run again inside the backward pass - under the 1F1B schedule, with the context-parallel exchanges and
    state hand-offs repeated, and with the stage-2 bucket boundaries between the layers: same losses, same norms."""
    plain = _lines(_run(nproc, *flags, "--steps", "2", port=port))
    ckpt = _lines(_run(nproc, *flags, "--steps", "2", "--activation-checkpointing", port=port + 1))
    assert len(plain) == len(ckpt) == 2
    for ra, rb in zip(plain, ckpt):
        assert float(ra["loss_sum"]) == pytest.approx(float(rb["loss_sum"]), rel=1e-6, abs=1e-7)
        assert float(ra["global_grad_norm"]) == pytest.approx(float(rb["global_grad_norm"]), rel=1e-5)
        assert float(ra["grad_norm_sum"]) == pytest.approx(float(rb["grad_norm_sum"]), rel=1e-5)


_ONE_RANK = {}


def _one_rank_sft(tmp_path, moe=False):
    """The one-rank supervised run every layout is compared with (4 micro-batches); run once per model kind."""
    if moe not in _ONE_RANK:
        extra = ["--config", "tiny_moe"] if moe else []
        _ONE_RANK[moe] = _lines(_run(1, *_sft_flags(tmp_path, 4), *extra, port=29791 + int(moe)))
    return _ONE_RANK[moe]


def _sft_flags(tmp_path, micro_batches=4):
    data = tmp_path / "sft.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"Question number {i}: what is {i}+{i}? ",
                                          "answer": f"The answer is {2 * i}."}) for i in range(8)))
    return ["--steps", "3", "--lr", "1e-2", "--max-grad-norm", "0", "--mode", "sft", "--sft-jsonl", str(data),
            "--prompt-len", "16", "--response-len", "16", "--micro-batches", str(micro_batches)]


@pytest.mark.parametrize("nproc,flags,reports", [
    (2, ["--pp", "2"], 1),
    (4, ["--pp", "2", "--cp", "2"], 2),
    (4, ["--pp", "2", "--tp", "2"], 2),
    (4, ["--cp", "2", "--tp", "2"], 4),
])
def test_dense_layouts_reproduce_the_one_rank_losses(tmp_path, nproc, flags, reports):
    """Supervised losses over three real updates: a pipeline (alone, with context parallelism, with tensor
    parallelism) and context x tensor parallelism (a pair the reference refuses) give the one-rank loss at every
    step, reported once per last-stage rank.  Every stage draws the initial values of its tensors from generators
    seeded by the tensor names, so the runs start from the same weights."""
    one = _one_rank_sft(tmp_path)
    many = _lines(_run(nproc, *flags, *_sft_flags(tmp_path), port=29752))
    assert len(one) == len(many) == 3
    for ra, rb in zip(one, many):
        assert float(rb["loss_sum"]) == pytest.approx(reports * float(ra["loss_sum"]), rel=2e-5)
    assert float(one[2]["loss_sum"]) < 0.8 * float(one[0]["loss_sum"])


@pytest.mark.parametrize("nproc,flags,mb,reports", [
    (2, ["--tp", "2"], 4, 2),
    (4, ["--ep", "2", "--tp", "2"], 2, 2),
])
def test_moe_layouts_reproduce_the_one_rank_losses(tmp_path, nproc, flags, mb, reports):
    """Mixture-of-experts under tensor parallelism (alone and with expert parallelism): the supervised loss after
    each of three updates is the one-rank loss.  The routing weights multiply expert outputs that are partial sums
    over the split FFN dimension, so the router's gradient has to be summed over the tensor-parallel group - with
    that sum missing the losses drift apart from the second step on."""
    moe = ["--config", "tiny_moe"]
    one = _one_rank_sft(tmp_path, moe=True)
    many = _lines(_run(nproc, *flags, *_sft_flags(tmp_path, mb), *moe, port=29762))
    assert len(one) == len(many) == 3
    for ra, rb in zip(one, many):
        assert float(rb["loss_sum"]) == pytest.approx(reports * float(ra["loss_sum"]), rel=2e-5)


@pytest.mark.parametrize("flags", [["--dp", "2", "--tp", "2"], ["--dp", "2", "--cp", "2"], ["--dp", "2", "--pp", "2"]])
def test_zero_stage2_with_tensor_or_context_parallelism(tmp_path, flags):
    """Bucketed gradients under model parallelism: the tensor-parallel shares of replicated parameters, the
    context-parallel sum and the two halves of a tied embedding's gradient under a pipeline are formed bucket by
    bucket, just before each bucket's data-parallel reduction - the supervised losses over three updates are the
    one-rank losses."""
    one = _one_rank_sft(tmp_path)
    many = _lines(_run(4, *flags, "--zero-stage", "2", *_sft_flags(tmp_path, 2), port=29772))
    assert len(one) == len(many) == 3
    reports = 1.0 if "--pp" in flags else 2.0            # one last-stage rank per replica reports under a pipeline
    for ra, rb in zip(one, many):
        assert float(rb["loss_sum"]) == pytest.approx(reports * float(ra["loss_sum"]), rel=2e-5)


def test_zero_stage2_with_expert_parallelism(tmp_path):
    """dp 2 x ep 2 on the mixture-of-experts model with bucketed gradients: the non-expert parameters take the
    mean over the expert-parallel group per bucket; one-rank losses over three updates."""
    moe = ["--config", "tiny_moe"]
    one = _one_rank_sft(tmp_path, moe=True)
    many = _lines(_run(4, "--dp", "2", "--ep", "2", "--zero-stage", "2", *_sft_flags(tmp_path, 1), *moe, port=29782))
    assert len(one) == len(many) == 3
    for ra, rb in zip(one, many):
        assert float(rb["loss_sum"]) == pytest.approx(float(ra["loss_sum"]), rel=2e-5)
