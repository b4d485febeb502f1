"""Command-line tools on a synthesized tiny model directory and gloo ranks."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def tiny_dir(tmp_path_factory):
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.hf_io import synthesize_model_dir
    d = tmp_path_factory.mktemp("tiny_model")
    synthesize_model_dir(Qwen35TextConfig.tiny(), d, seed=3, dtype=torch.float32)
    return d


def test_weight_manifest_and_inspect(tiny_dir, capsys):
    from cverl_b200.cli import inspect_hf_model, vllm_weight_manifest
    assert vllm_weight_manifest.main(["--model-dir", str(tiny_dir), "--send-dtype", "bfloat16", "--no-packed"]) == 0
    out = json.loads(capsys.readouterr().out)
    info = out["update_info"]
    assert out["backend"] == "vllm_native_rl_nccl" and info["packed"] is False and not info["is_checkpoint_format"]
    assert len(info["names"]) == len(info["shapes"]) == len(info["dtype_names"]) > 10
    assert set(info["dtype_names"]) == {"bfloat16"} and info["names"][0].endswith("embed_tokens.weight")
    assert inspect_hf_model.main(["--model-dir", str(tiny_dir), "--check", "--tensors"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["check"]["ok"] and rep["num_tensors"] == len(rep["tensors"])
    assert inspect_hf_model.main([str(tiny_dir), "--find", "embed_tokens", "--load-tensor", info["names"][0],
                                  "--load-all"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["match_count"] == 1 and rep["matches"][0]["name"].endswith("embed_tokens.weight")
    assert rep["loaded_tensor"]["shape"] == rep["matches"][0]["shape"] and rep["loaded_tensor"]["nbytes"] > 0
    assert rep["loaded_all"]["tensor_count"] == rep["num_tensors"] and rep["loaded_all"]["nbytes"] == rep["total_bytes"]


def test_forward_dump_and_compare(tiny_dir, tmp_path, capsys):
    from cverl_b200.cli import qwen3_5_forward
    dump = tmp_path / "fwd.pt"
    assert qwen3_5_forward.main(["--model-dir", str(tiny_dir), "--ids", "5,6,7,8,9", "--dump", str(dump)]) == 0
    first = json.loads(capsys.readouterr().out)
    assert first["shape"][:2] == [1, 5] and len(first["argmax"]) == 5
    assert qwen3_5_forward.main(["--model-dir", str(tiny_dir), "--ids", "5,6,7,8,9", "--compare", str(dump)]) == 0
    second = json.loads(capsys.readouterr().out)
    assert second["compare"]["max_abs"] < 1e-5 and second["compare"]["argmax_equal"]
    # the reference's command line: positional model directory, --tokens / --layers / --logits / --save-output
    raw = tmp_path / "logits.bin"
    assert qwen3_5_forward.main([str(tiny_dir), "--tokens", "5,6,7,8,9", "--logits", "--save-output", str(raw)]) == 0
    third = json.loads(capsys.readouterr().out)
    assert third["saved_output"] == str(raw) and len(third["top5_token_ids"]) == 5 and third["tokens"] == 5
    assert raw.read_bytes()[:8] == b"CVTENSR1"
    back = qwen3_5_forward.load_tensor_binary(raw)
    assert list(back.shape) == third["shape"] and abs(float(back.mean()) - third["mean"]) < 1e-6
    assert qwen3_5_forward.main([str(tiny_dir), "--tokens", "5,6,7,8,9", "--compare", str(raw)]) == 0
    assert json.loads(capsys.readouterr().out)["compare"]["max_abs"] < 1e-5
    assert qwen3_5_forward.main([str(tiny_dir), "--tokens", "5,6,7", "--layers", "2", "--hidden"]) == 0
    hid = json.loads(capsys.readouterr().out)
    assert hid["output"] == "hidden" and hid["layers"] == 2 and hid["shape"][:2] == [1, 3] and "top5_token_ids" not in hid


def test_rollout_batch_source_to_receiver_gloo():
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1", MASTER_PORT="29733",
               WORLD_SIZE="2")
    common = [sys.executable, "-m", "cverl_b200.cli.rollout_batch_source", "--backend", "gloo", "--steps", "2",
              "--batch", "4", "--prompt-len", "6", "--response-len", "3"]
    src = subprocess.Popen(common + ["--target-ranks", "1"], env=dict(env, RANK="0", LOCAL_RANK="0"), cwd=ROOT,
                           stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    dst = subprocess.Popen(common + ["--receive-from", "0"], env=dict(env, RANK="1", LOCAL_RANK="0"), cwd=ROOT,
                           stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    so, se = src.communicate(timeout=120)
    do, de = dst.communicate(timeout=120)
    assert src.returncode == 0, se[-2000:]
    assert dst.returncode == 0, de[-2000:]
    assert "rollout source step 2 sent batch=4" in so
    assert "step 2 received batch=4 weight_version=2 reward_sum=2.0" in do


def test_golden_dump_and_replay_through_c_abi(tmp_path, capsys):
    from cverl_b200.cli import golden
    path = tmp_path / "golden.bin"
    assert golden.main(["dump", str(path), "--seed", "7"]) == 0
    assert path.read_bytes()[:8] == b"CVERLGD1"
    assert golden.main(["compare", str(path)]) == 0
    assert "golden replay: ok" in capsys.readouterr().out
    # a corrupted expectation is reported
    raw = bytearray(path.read_bytes())
    import struct
    raw[-4:] = struct.pack("<f", 1234.5)
    bad = tmp_path / "bad.bin"
    bad.write_bytes(bytes(raw))
    assert golden.main(["compare", str(bad)]) == 1


def test_vllm_bridge_policy_update_and_manifest(tiny_dir):
    from cverl_b200.rollout.vllm_bridge import QwenPolicy
    pol = QwenPolicy(str(tiny_dir), device="cpu", param_dtype="float32")
    named = pol.named_parameters()
    info = pol.update_info(packed=True, packed_buffer_size_bytes=1 << 20, packed_num_buffers=3)
    assert [n for n, _ in named] == info["names"] and info["packed_num_buffers"] == 3
    before = named[1][1].detach().clone()
    prompts, answers = ["What is 2+2?", "What is 3+3?"], ["#### 4", "#### 6"]
    responses = ["so #### 4", "hm #### 5", "it is #### 6", "no idea"]
    m = pol.gsm8k_grpo_update(prompts, responses, answers, [0, 0, 1, 1], [0, 1, 0, 1], max_prompt_tokens=16,
                              max_response_tokens=12, ppo_epochs=2, learning_rate=1e-3, kl_coef=0.01,
                              reward_method="flexible", measure_param_delta=True)
    assert m["total_seq"] == 4.0 and m["mean_reward"] == pytest.approx(0.5) and m["success_rate"] == pytest.approx(0.5)
    assert m["param_delta"] > 0 and m["adv_abs_sum"] > 0
    assert not torch.equal(named[1][1], before)          # the named tensors are live views of the weights


@pytest.mark.parametrize("mode,nproc", [("tp", 2), ("dp_tp", 4), ("pp_tp", 4)])
def test_parallel_smokes_gloo(mode, nproc):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(29750 + nproc + len(mode)), "-m", "cverl_b200.cli.parallel_smoke",
           "--mode", mode, "--backend", "gloo"]
    p = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1"),
                       capture_output=True, text=True, timeout=240)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert f"{mode} smoke passed" in p.stdout


def test_static_trainer_rollout_split_gloo():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29771", "-m", "cverl_b200.cli.static_split", "--backend", "gloo",
           "--trainers", "2", "--steps", "2"]
    p = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1"),
                       capture_output=True, text=True, timeout=240)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert "weights_in_sync=True" in p.stdout and "trainer rank 0 step 2" in p.stdout
    assert "rollout rank 2 step 2 sent 16 sequences weight_version=1" in p.stdout     # generated with pushed weights


def test_online_grpo_oracle_dumps_rollouts_that_the_trainer_consumes(tiny_dir, tmp_path, capsys):
    from cverl_b200.cli import online_grpo
    data = tmp_path / "gsm.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"What is {i}+{i}?", "answer": f"#### {2 * i}"}) for i in range(6)))
    rdir = tmp_path / "rollouts"
    rc = online_grpo.main(["--model-dir", str(tiny_dir), "--dataset", str(data), "--rollout", "oracle", "--steps", "2",
                           "--prompts", "2", "--n", "4", "--max-prompt-tokens", "16", "--max-response-tokens", "12",
                           "--lr", "1e-3", "--dump-rollout-dir", str(rdir), "--push-weights"])
    assert rc == 0
    rows = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert [r["step"] for r in rows] == [0, 1] and rows[0]["total_seq"] == 8.0 and rows[0]["pushed_bytes"] > 0
    assert 0.0 < rows[0]["mean_reward"] < 1.0 and rows[0]["param_delta"] > 0
    f0 = json.loads((rdir / "rollout_step_000001.json").read_text())     # 1-based, as the reference numbers them
    assert f0["step"] == 1 and len(f0["responses"]) == 8 and len(f0["prompts"]) == 2
    assert len(f0["sequences"]) == 8 and {"prompt_ids", "response_ids", "advantage"} <= set(f0["sequences"][0])
    # the distributed trainer reads these files step by step
    cmd = [sys.executable, "-m", "cverl_b200.trainer.ppo_trainer", "--backend", "gloo", "--dtype", "float32",
           "--steps", "2", "--rollout-dir", str(rdir), "--prompt-len", "16", "--response-len", "12",
           "--micro-batches", "2", "--micro-batch-seqs", "2"]
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1", MASTER_PORT="29779",
               RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=240)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert p.stdout.count("step=") == 2
    row = dict(kv.split("=", 1) for kv in p.stdout.splitlines()[0].split() if "=" in kv)
    assert 0.0 < float(row["mean_reward"]) < 1.0 and float(row["adv_abs_sum"]) > 0 and row["rollout_rows"] == "8"
    # the same files in the reference's text form (no token-id rows): tokenised, scored and GRPO-normalised here
    tdir = tmp_path / "text_rollouts"
    tdir.mkdir()
    for f in rdir.glob("rollout_step_*.json"):
        doc = json.loads(f.read_text())
        doc.pop("sequences")
        (tdir / f.name).write_text(json.dumps(doc))
    cmd[cmd.index(str(rdir))] = str(tdir)
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=240)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    row2 = dict(kv.split("=", 1) for kv in p.stdout.splitlines()[0].split() if "=" in kv)
    assert float(row2["mean_reward"]) == pytest.approx(float(row["mean_reward"])) and row2["rollout_rows"] == "8"


def test_benchmark_modules_parse_their_flags():
    """The kernel and collective benchmarks import without a GPU and describe their flags."""
    for mod in ("cverl_b200.bench_kernels", "cverl_b200.bench_collectives"):
        p = subprocess.run([sys.executable, "-m", mod, "--help"], cwd=ROOT, env=dict(os.environ, PYTHONPATH=str(ROOT)),
                           capture_output=True, text=True, timeout=120)
        assert p.returncode == 0, p.stderr[-2000:]
        assert "--iters" in p.stdout


def test_env_driven_trainer_launcher_script():
    """examples/run_pp_tp_ppo_trainer.sh maps the reference launcher's environment variables onto the trainer's flags."""
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", DP_SIZE="1", PP_SIZE="1", TP_SIZE="2", LAYERS="2",
               CONFIG="tiny", PROMPT_LEN="8", RESPONSE_LEN="8", DTYPE="float32", ZERO_COMM="nccl", TP_COMM="nccl",
               EP_COMM="nccl", MASTER_PORT="29578", STEPS="2", CLIP_RATIO="0.25", MAX_GRAD_NORM="0.5")
    p = subprocess.run(["bash", str(ROOT / "examples" / "run_pp_tp_ppo_trainer.sh"), "", "--backend", "gloo"], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-2500:]
    steps = [ln for ln in p.stdout.splitlines() if ln.startswith("step=")]
    assert len(steps) == 2 and " tp=2 " in steps[0] and " pp=1 " in steps[0] and "dtype=float32" in steps[0]
    # MAX_RESTARTS / LOG_DIR select the supervising launcher: same flags, one log per rank, a JSON summary
    env.update(MAX_RESTARTS="1", MASTER_PORT="29588")
    p = subprocess.run(["bash", str(ROOT / "examples" / "run_pp_tp_ppo_trainer.sh"), "", "--backend", "gloo"], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-2500:]
    assert len([ln for ln in p.stdout.splitlines() if ln.startswith("step=")]) == 2
    assert json.loads(p.stdout.splitlines()[-1])["launch"]["ok"]


def test_wall_clock_multi_rank_bench_script(tmp_path):
    """examples/run_multigpu_ppo_bench.sh: two 4-rank layouts timed as whole runs, one CSV row each."""
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", CONFIG="tiny", DTYPE="float32", STEPS="2",
               OUT_DIR=str(tmp_path), MASTER_PORT="29861")
    p = subprocess.run(["bash", str(ROOT / "examples" / "run_multigpu_ppo_bench.sh"), "", "--backend", "gloo"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-2500:]
    rows = (tmp_path / "multigpu_ppo_bench.csv").read_text().strip().splitlines()
    assert rows[0].startswith("case,pp,tp,micro_batches,steps") and len(rows) == 3
    a, b = rows[1].split(","), rows[2].split(",")
    assert a[:5] == ["qwen_pp2_tp2_ppo", "2", "2", "2", "2"] and b[:5] == ["qwen_pp4_tp1_ppo", "4", "1", "4", "2"]
    assert float(a[7]) > 0 and float(b[9]) > 0


def test_multi_rank_regression_script(tmp_path):
    """examples/run_multigpu_regression.sh: four layouts, the reference's pass criteria on each log."""
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", CONFIG="tiny", DTYPE="float32", STEPS="2",
               OUT_DIR=str(tmp_path), MASTER_PORT="29851")
    p = subprocess.run(["bash", str(ROOT / "examples" / "run_multigpu_regression.sh"), "", "--backend", "gloo"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-2500:]
    assert "multi-GPU PPO regression passed" in p.stdout
    logs = sorted(f.name for f in tmp_path.glob("*.log"))
    assert logs == ["qwen_dp2_pp1_tp2_ppo.log", "qwen_dp2_pp1_tp2_sharded_optim.log", "qwen_pp2_tp2_ppo.log",
                    "qwen_pp4_tp1_ppo.log"]
    assert "flat_shard_optimizer=false" in (tmp_path / "qwen_dp2_pp1_tp2_ppo.log").read_text()
    assert "flat_shard_optimizer=true" in (tmp_path / "qwen_dp2_pp1_tp2_sharded_optim.log").read_text()
    # a log with a non-finite value fails the run: the check is the script's own grep
    bad = subprocess.run(["bash", "-c", "echo 'step=0 loss_sum=nan all' | grep -Eiq '=(nan|-?inf)( |$)'"])
    assert bad.returncode == 0


def test_rollout_files_to_trainer_script(tiny_dir, tmp_path):
    """examples/run_rollout_to_trainer.sh: the oracle engine writes the step files, the 4-rank trainer reads them."""
    data = tmp_path / "gsm.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"What is {i}+{i}?", "answer": f"#### {2 * i}"}) for i in range(6)))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", DATASET=str(data), ROLLOUT_DIR=str(tmp_path / "r"),
               STEPS="2", PROMPT_LEN="16", RESPONSE_LEN="24", DTYPE="float32", TP_COMM="nccl", ZERO_COMM="nccl",
               MASTER_PORT="29841", LR="1e-4")
    p = subprocess.run(["bash", str(ROOT / "examples" / "run_rollout_to_trainer.sh"), str(tiny_dir), "--backend", "gloo"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-2500:]
    assert sorted(f.name for f in (tmp_path / "r").glob("*.json")) == ["rollout_step_000001.json", "rollout_step_000002.json"]
    steps = [dict(kv.split("=", 1) for kv in ln.split()) for ln in p.stdout.splitlines() if ln.startswith("step=")]
    assert len(steps) == 2 and steps[0]["pp"] == "2" and steps[0]["tp"] == "2" and steps[0]["rollout_rows"] == "4"


def test_vllm_online_grpo_launcher_dry_run_and_oracle(tiny_dir, tmp_path):
    """examples/run_vllm_online_grpo.sh: the command lines it would run, and the whole loop with the oracle engine
    (no server, CPU)."""
    data = tmp_path / "gsm.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"What is {i}+{i}?", "answer": f"#### {2 * i}"}) for i in range(6)))
    script = str(ROOT / "examples" / "run_vllm_online_grpo.sh")
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", MODEL_DIR=str(tiny_dir), DATASET=str(data))
    dry = subprocess.run(["bash", script], cwd=ROOT, env=dict(env, DRY_RUN="1", VLLM_TP_SIZE="2", VLLM_GPUS="0,1"),
                         capture_output=True, text=True, timeout=60)
    assert dry.returncode == 0, dry.stderr
    serve, loop = dry.stdout.strip().splitlines()
    assert "vllm serve" in serve and "--tensor-parallel-size 2" in serve and "--enable-sleep-mode" in serve
    assert "CUDA_VISIBLE_DEVICES=0,1" in serve and "--weight-sync nccl" in loop and "--rollout http" in loop
    static = subprocess.run(["bash", script], cwd=ROOT, env=dict(env, DRY_RUN="1", STATIC_SPLIT="1", ROLLOUT_DIR="/r"),
                            capture_output=True, text=True, timeout=60)
    assert "--skip-train" in static.stdout and "--weight-sync" not in static.stdout and "--dump-rollout-dir /r" in static.stdout
    run = subprocess.run(["bash", script], cwd=ROOT, capture_output=True, text=True, timeout=300,
                         env=dict(env, ROLLOUT_BACKEND="oracle", DEVICE="cpu", PARAM_DTYPE="float32", STEPS="2", N="4",
                                  PROMPTS="2", MAX_PROMPT_TOKENS="16", MAX_RESPONSE_TOKENS="24", LR="1e-3"))
    assert run.returncode == 0, run.stdout[-1500:] + run.stderr[-2500:]
    rows = [json.loads(ln) for ln in run.stdout.strip().splitlines() if ln.startswith("{")]
    assert [r["step"] for r in rows] == [0, 1] and rows[0]["total_seq"] == 8.0


@pytest.mark.parametrize("world", [2, 4])
def test_collectives_smoke_script_on_gloo(world, tmp_path):
    """examples/run_nccl_smoke.sh with the torch backend on CPU: every collective against its closed form, the
    sub-group of the first half of the world, refusals; one log per rank from the supervising launcher."""
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", BACKEND="torch", CPU="1", WORLD_SIZE=str(world),
               MASTER_PORT=str(29820 + world), LOG_DIR=str(tmp_path))
    p = subprocess.run(["bash", str(ROOT / "examples" / "run_nccl_smoke.sh")], cwd=ROOT, env=env, capture_output=True,
                       text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert f"collectives smoke passed: backend=torch world={world}" in p.stdout
    assert "all_to_all" in p.stdout and "sub_group" in p.stdout and "ring_send_recv" in p.stdout
    assert len(list((tmp_path / "attempt_0").glob("rank_*.log"))) == world
