"""Rollout layer on CPU: workers, cached decode, plugin loader, transports, batch builder, weight sync."""
import multiprocessing as mp
import os

import pytest
import torch

from cverl_b200._build import LIB_DIR
from cverl_b200.models.config import Qwen35TextConfig
from cverl_b200.models.policy import (CausalLmPolicyOptions, Qwen3_5CausalLmPolicy, TinyCausalLmPolicy,
                                      make_causal_lm_policy, response_log_probs)
from cverl_b200.models.qwen3_5 import Qwen35Model
from cverl_b200.parallel.collectives import Collectives, ReduceOp, SingleProcessCollectives
from cverl_b200.parallel.weight_sync import (ParameterView, broadcast_parameters_from_root, recv_parameter_shards,
                                             send_parameter_shards)
from cverl_b200.rollout import (CachedQwenRolloutWorker, GenerationConfig, LoopbackRolloutTransport,
                                PolicyRolloutWorker, RolloutRequest, RolloutSample, SharedMemoryRegion,
                                SharedMemoryRolloutTransport, TokenBatch, build_gsm8k_rollout_batch,
                                load_rollout_worker_plugin)
from cverl_b200.rollout.gpu_batch_transport import (GpuBatchReceiver, GpuBatchSender, GpuRolloutBatch,
                                                    TrainerIngressQueue)
from cverl_b200.rollout.transport import (deserialize_request, deserialize_response, serialize_request,
                                          serialize_response)
from cverl_b200.text import ByteTokenizer
from dist_utils import run_ranks


def _batch(B=2, P=5, vocab=50):
    ids = torch.randint(4, vocab, (B, P), generator=torch.Generator().manual_seed(0))
    return TokenBatch(ids, torch.ones_like(ids), torch.full((B,), P))


class DeterministicEosPolicy(TinyCausalLmPolicy):
    """Always predicts eos after `eos_after` generated tokens; counts forwards."""

    def __init__(self, eos=2, eos_after=3):
        super().__init__(vocab_size=16, hidden_size=8)
        self.eos, self.eos_after, self.calls = eos, eos_after, 0

    def forward(self, prompt_ids, response_ids):
        self.calls += 1
        B, R = response_ids.shape
        logits = torch.full((B, R, 16), -10.0)
        tok = self.eos if R > self.eos_after else 5
        logits[:, :, tok] = 10.0
        return logits


def test_policy_worker_greedy_eos_interval():
    pol = DeterministicEosPolicy()
    w = PolicyRolloutWorker(pol)
    out = w.generate(_batch(), GenerationConfig(max_new_tokens=32, temperature=0.0, eos_token_id=2,
                                                eos_check_interval=4))
    assert out.lengths.tolist() == [4, 4]
    assert out.token_ids[0, :4].tolist() == [5, 5, 5, 2]
    assert pol.calls == 4            # stopped at the first interval check after every row finished
    pol2 = DeterministicEosPolicy()
    PolicyRolloutWorker(pol2).generate(_batch(), GenerationConfig(max_new_tokens=12, temperature=0.0, eos_token_id=2,
                                                                  eos_check_interval=0))
    assert pol2.calls == 12          # no host check: runs to max_new_tokens


def test_sampling_top_k_top_p():
    from cverl_b200.rollout import sample_next_tokens
    logits = torch.tensor([[0.0, 1.0, 5.0, 4.0]]).repeat(64, 1)
    g = torch.Generator().manual_seed(1)
    tok, lp = sample_next_tokens(logits, GenerationConfig(top_k=2), g)
    assert set(tok.tolist()) <= {2, 3}
    tok, _ = sample_next_tokens(logits, GenerationConfig(top_p=0.5), g)
    assert set(tok.tolist()) == {2}
    tok, lp = sample_next_tokens(logits, GenerationConfig(temperature=0.0), None)
    assert tok.tolist() == [2] * 64 and torch.allclose(lp, torch.log_softmax(logits, -1)[:, 2])


def test_cached_decode_equals_recompute_generation():
    cfg = Qwen35TextConfig.tiny(layers=4, vocab=64)
    pol = Qwen3_5CausalLmPolicy(cfg, torch.float32)
    pol.model.init_weights(seed=3)
    b = _batch(B=2, P=6, vocab=64)
    gc = GenerationConfig(max_new_tokens=6, temperature=0.0)
    slow = PolicyRolloutWorker(pol).generate(b, gc)
    fast = CachedQwenRolloutWorker(pol.model).generate(b, gc)
    assert torch.equal(slow.token_ids, fast.token_ids)
    torch.testing.assert_close(slow.logprobs, fast.logprobs, rtol=1e-4, atol=1e-4)


def test_tiny_policy_and_reference_clone():
    pol = make_causal_lm_policy(CausalLmPolicyOptions(kind="tiny", vocab_size=32, hidden_size=16))
    p, r = torch.randint(1, 32, (3, 4)), torch.randint(1, 32, (3, 5))
    logits = pol(p, r)
    assert logits.shape == (3, 5, 32)
    # row t must not depend on response tokens >= t
    r2 = r.clone()
    r2[:, 3:] = 7
    torch.testing.assert_close(pol(p, r2)[:, :4], logits[:, :4])
    ref = pol.clone_as_reference()
    assert all(not q.requires_grad for q in ref.parameters())
    lp = response_log_probs(logits, r)
    lp.sum().backward()
    with torch.no_grad():
        for q in pol.parameters():
            q.add_(0.1)
    assert not torch.allclose(ref(p, r), pol(p, r))


def test_qwen_policy_hf_roundtrip(tmp_path):
    from cverl_b200.models.hf_io import synthesize_model_dir
    cfg = Qwen35TextConfig.tiny(layers=2, vocab=64)
    d = synthesize_model_dir(cfg, tmp_path / "m", dtype=torch.float32)
    pol = Qwen3_5CausalLmPolicy.from_model_dir(d)
    p, r = torch.randint(1, 64, (2, 4)), torch.randint(1, 64, (2, 3))
    torch.testing.assert_close(pol.response_log_probs(p, r), response_log_probs(pol(p, r), r), rtol=1e-4, atol=1e-5)
    pol.save_hf_checkpoint(tmp_path / "out")
    again = Qwen3_5CausalLmPolicy.from_model_dir(tmp_path / "out")
    assert torch.equal(again.model.flat.flat, pol.model.flat.flat)
    assert (tmp_path / "out" / "config.json").exists()


def test_plugin_loader_fixture():
    w = load_rollout_worker_plugin(str(LIB_DIR / "libplugin_worker_fixture.so"), '{"vocab": 50, "eos_after": 3}')
    b = TokenBatch(torch.tensor([[0, 5, 7], [1, 2, 3]]), torch.ones(2, 3, dtype=torch.long), torch.tensor([3, 3]))
    o = w.generate(b, GenerationConfig(max_new_tokens=6, eos_token_id=2))
    assert o.token_ids[0].tolist() == [8, 9, 10, 2, 0, 0] and o.lengths.tolist() == [4, 4]
    pv = w.actor_parameters()
    assert pv[0].name == "fixture.weight" and pv[0].tensor.tolist() == [1, 2, 3, 4]
    pv[0].tensor[0] = 9.0                                   # live view into the plugin's memory
    assert w.actor_parameters()[0].tensor[0].item() == 9.0
    with pytest.raises(RuntimeError):
        load_rollout_worker_plugin(str(LIB_DIR / "libcverl.so"))
    with pytest.raises(RuntimeError):
        load_rollout_worker_plugin("/nonexistent/plugin.so")
    with pytest.raises(RuntimeError):
        load_rollout_worker_plugin(str(LIB_DIR / "libplugin_worker_fixture.so"), '{"fail": 1}')


def test_loopback_and_serialization_roundtrip():
    req = RolloutRequest(prompts=["a", "b"], prompt_token_ids=[[1, 2], [3]], n=2, max_tokens=4, temperature=0.5,
                         stop=["x"], model="m", extra_params={"k": "v"}, request_id=7, seed=3)
    assert deserialize_request(serialize_request(req)) == req
    resp = LoopbackRolloutTransport().generate(req)
    assert len(resp.sequences) == 4 and resp.sequences[2].prompt_index == 1
    assert deserialize_response(serialize_response(resp)) == resp
    again = LoopbackRolloutTransport().generate(req)
    assert again.sequences[1].token_ids == resp.sequences[1].token_ids
    with pytest.raises(ValueError):
        deserialize_request(serialize_request(req)[:10])


def _shm_child(name):
    c = SharedMemoryRolloutTransport(name, 1 << 16, create=False, timeout_ms=5000)
    r = c.generate(RolloutRequest(prompts=["hi", "yo"], n=2, max_tokens=4))
    ok = len(r.sequences) == 4 and r.sequences[0].text.startswith("hi")
    try:
        c.generate(RolloutRequest(prompts=["boom"]))
        ok = False
    except RuntimeError:
        pass
    os._exit(0 if ok else 1)


def test_shared_memory_transport_forked_server_and_timeout():
    name = f"/cvb_t_{os.getpid()}"
    srv = SharedMemoryRolloutTransport(name, 1 << 16, create=True, timeout_ms=5000)
    p = mp.get_context("fork").Process(target=_shm_child, args=(name,))
    p.start()

    def handler(req):
        if req.prompts == ["boom"]:
            raise ValueError("handler failure")
        return LoopbackRolloutTransport().generate(req)
    assert srv.serve_one(handler) and srv.serve_one(handler)
    assert srv.serve_one(handler, timeout_ms=100) is False       # nothing pending: timeout, no hang
    p.join(10)
    assert p.exitcode == 0
    cli = SharedMemoryRolloutTransport(name, 1 << 16, create=False, timeout_ms=150)
    with pytest.raises(TimeoutError):
        cli.generate(RolloutRequest(prompts=["nobody listens"]))
    cli.close()
    srv.close()
    with pytest.raises(OSError):
        SharedMemoryRolloutTransport(name, 1 << 16, create=False)


def test_shared_memory_region():
    name = f"/cvb_r_{os.getpid()}"
    with SharedMemoryRegion(name, 4096, create=True) as a:
        a.buffer()[0] = 42
        with SharedMemoryRegion(name) as b:
            assert b.size >= 4096 and b.buffer()[0] == 42
    with pytest.raises(OSError):
        SharedMemoryRegion(name)


def test_build_gsm8k_rollout_batch():
    tok = ByteTokenizer()
    prompts, answers = ["What is 2+2?", "What is 3+3?"], ["#### 4", "6"]
    samples = [RolloutSample(0, "it is #### 4"), RolloutSample(0, "it is #### 5"), RolloutSample(1, "no idea")]
    b = build_gsm8k_rollout_batch(tok, prompts, answers, samples, max_prompt_len=8, max_response_len=16)
    assert b.prompt_ids.shape == (3, 8) and b.response_ids.shape == (3, 16)
    assert tok.decode(b.prompt_ids[0].tolist()) == "What is "     # an over-long prompt keeps its first tokens
    assert b.rewards.tolist() == [1.0, 0.0, 0.0]
    n0 = int(b.response_mask[0].sum())
    assert n0 == len("it is #### 4") + 1 and b.response_ids[0, n0 - 1] == tok.eos_id      # EOS closes the response
    assert b.token_rewards[0, n0 - 1] == 1.0 and b.token_rewards[0].sum() == 1.0
    plain = build_gsm8k_rollout_batch(tok, prompts, answers, samples, 8, 16, add_eos=False)
    assert int(plain.response_mask[0].sum()) == len("it is #### 4")
    full = build_gsm8k_rollout_batch(tok, prompts, answers, [RolloutSample(0, "x" * 40)], 8, 16)
    assert int(full.response_mask[0].sum()) == 16 and full.response_ids[0, 15] == 4 + ord("x")   # no room: no EOS
    assert b.group_ids.tolist() == [0, 0, 1]
    short = build_gsm8k_rollout_batch(tok, ["hi"], ["1"], [RolloutSample(0, "#### 1")], 8, 16)
    assert short.prompt_ids[0, :6].tolist() == [0] * 6            # left padded


@pytest.mark.parametrize("kind", ["byte", "bpe"])
def test_native_batch_builder_equals_the_python_loop(kind):
    """The multi-threaded C++ builder and the Python statement of the rules give the same six tensors: shared and
    unused prompts, responses with and without their own token ids, truncation on both sides, empty responses."""
    from pathlib import Path

    from cverl_b200.reward import Gsm8kRewardOptions
    from cverl_b200.text import HfBpeTokenizer
    tok = ByteTokenizer() if kind == "byte" else HfBpeTokenizer(
        str(Path(__file__).parent / "fixtures" / "synthetic_tokenizer.json"))
    prompts = ["What is 2+2?", "never sampled", "hello world " * 9, ""]
    answers = ["#### 4", "0", "12", "7"]
    samples = [RolloutSample(0, "it is #### 4"), RolloutSample(2, "hello hello #### 12 " * 6), RolloutSample(0, ""),
               RolloutSample(3, "the answer is 7", [5, 6, 7]), RolloutSample(2, "#### 13", list(range(4, 40))),
               RolloutSample(0, "4 #### 4", [])]
    opts = Gsm8kRewardOptions(method="flexible", correct_score=2.0, format_score=0.5, no_answer_score=-1.0)
    ref = build_gsm8k_rollout_batch(tok, prompts, answers, samples, 8, 16, opts, threads=-1)
    for threads in (1, 3):
        got = build_gsm8k_rollout_batch(tok, prompts, answers, samples, 8, 16, opts, threads=threads)
        for f in ref.__dataclass_fields__:
            assert torch.equal(getattr(ref, f), getattr(got, f)), f
    assert ref.rewards.tolist() == [2.0, 2.0, -1.0, 2.0, 0.5, 2.0] and ref.response_mask[4].sum() == 16
    # an empty response is its EOS alone (the reward sits on it); an empty id list means "tokenise the text"
    assert ref.response_mask[2].sum() == 1 and ref.token_rewards[2, 0] == -1.0 and ref.response_mask[5].sum() > 1
    bare = build_gsm8k_rollout_batch(tok, prompts, answers, samples, 8, 16, opts, add_eos=False)
    assert bare.response_mask[2].sum() == 0 and bare.token_rewards[2].sum() == 0
    with pytest.raises(ValueError):
        build_gsm8k_rollout_batch(tok, prompts, answers, [RolloutSample(4, "x")], 8, 16)
    with pytest.raises(ValueError):
        build_gsm8k_rollout_batch(tok, prompts, answers, [RolloutSample(-1, "x")], 8, 16)


class CountingCollectives(SingleProcessCollectives):
    def __init__(self, world=2, rank=1):
        self._w, self._r, self.broadcasts, self.barriers, self.sent = world, rank, 0, 0, []
    def world_size(self): return self._w
    def rank(self): return self._r
    def _check(self, group): pass
    def broadcast(self, tensor, root, group=None):
        self.broadcasts += 1
        return torch.full_like(tensor, 3)
    def barrier(self, group=None): self.barriers += 1
    def send(self, tensor, dst): self.sent.append(tensor.clone())
    def recv_like(self, like, src): return self.sent.pop(0)


def test_weight_sync_buckets_barrier_and_p2p():
    params = [ParameterView(f"p{i}", torch.zeros(1024, dtype=torch.float32)) for i in range(4)]
    params.append(ParameterView("h", torch.zeros(8, dtype=torch.bfloat16)))
    c = CountingCollectives()
    st = broadcast_parameters_from_root(params, c, root=0, group=[0, 1], bucket_bytes=1 << 20)
    assert (st.buckets, c.broadcasts, c.barriers) == (2, 2, 1)      # dtype change splits the bucket
    assert all((p.tensor == 3).all() for p in params)
    c2 = CountingCollectives()
    st2 = broadcast_parameters_from_root(params, c2, 0, [0, 1], bucket_bytes=16, barrier=False)
    assert st2.buckets == 5 and c2.barriers == 0
    single = SingleProcessCollectives()
    assert broadcast_parameters_from_root(params, single, 0, [0]).buckets == 0
    with pytest.raises(ValueError):
        broadcast_parameters_from_root(params, c, root=5, group=[0, 1])
    src = [ParameterView("a", torch.arange(10.0)), ParameterView("b", torch.arange(6.0).view(2, 3))]
    dst = [ParameterView("a", torch.zeros(10)), ParameterView("b", torch.zeros(2, 3))]
    c3 = CountingCollectives()
    send_parameter_shards(src, c3, dst=1, bucket_bytes=32)
    recv_parameter_shards(dst, c3, src=0, bucket_bytes=32)
    assert torch.equal(dst[0].tensor, src[0].tensor) and torch.equal(dst[1].tensor, src[1].tensor)


def _gpu_batch_worker(rank, world, mode):
    from cverl_b200.parallel.collectives import TorchDistCollectives
    os.environ["CVERL_GPU_BATCH_NCCL_MODE"] = mode
    comm = TorchDistCollectives()
    if rank == 0:
        b = GpuRolloutBatch(step=3, weight_version=9, prompt_len=4, response_len=6)
        b.tensors["prompt_ids"] = torch.arange(8).view(2, 4)
        b.tensors["response_ids"] = torch.arange(12).view(2, 6)
        b.tensors["response_mask"] = torch.ones(2, 6)
        b.tensors["rewards"] = torch.tensor([1.0, 0.0])
        GpuBatchSender(comm, "cpu").send(b, 1)
    else:
        got = GpuBatchReceiver(comm, "cpu").recv(0)
        assert (got.step, got.weight_version, got.prompt_len, got.response_len, got.batch) == (3, 9, 4, 6, 2)
        assert list(got.tensors) == ["prompt_ids", "response_ids", "response_mask", "rewards"]
        assert torch.equal(got.tensors["response_ids"], torch.arange(12).view(2, 6))
        q = TrainerIngressQueue(1)
        assert q.push(got) and not q.push(got) and q.pop() is got and q.pop() is None


@pytest.mark.parametrize("mode", ["direct", "slab"])
def test_gpu_batch_transport_over_gloo(mode):
    run_ranks(_gpu_batch_worker, 2, mode)


def test_vllm_control_plane_and_weight_sync_sequence():
    """The control client against a local fake server, and the order of one weight push: engine init on both
    sides, pause, the update manifest in flight while the tensors are sent, resume - with a fake transfer engine
    standing in for vLLM's."""
    import json as _json
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer
    import torch
    from cverl_b200.rollout.vllm_control import VllmControl, VllmNcclSync, normalize_dtype_name
    calls = []
    update_seen = threading.Event()

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def _reply(self, obj):
            body = _json.dumps(obj).encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_POST(self):
            n = int(self.headers.get("Content-Length", "0"))
            payload = _json.loads(self.rfile.read(n) or b"{}")
            calls.append((self.path, payload))
            if self.path == "/update_weights":
                update_seen.set()
            self._reply({"ok": True, "path": self.path})

        def do_GET(self):
            calls.append((self.path, None))
            self._reply({"world_size": 2} if "world_size" in self.path else {"is_sleeping": False})

    server = HTTPServer(("127.0.0.1", 0), Handler)
    t = threading.Thread(target=server.serve_forever, daemon=True)
    t.start()
    try:
        c = VllmControl(f"http://127.0.0.1:{server.server_port}", timeout=10)
        assert c.world_size()["world_size"] == 2 and c.is_sleeping() == {"is_sleeping": False}
        c.sleep(2, "abort")
        c.wake(["weights"])
        assert [p for p, _ in calls[-2:]] == ["/sleep?level=2&mode=abort", "/wake_up?tags=weights"]
        calls.clear()

        sent = []

        class FakeEngine:
            @staticmethod
            def trainer_init(info):
                sent.append(("init", dict(info)))
                return "group"

            @staticmethod
            def trainer_send_weights(it, args):
                assert update_seen.wait(5.0)              # the manifest request is in flight while tensors move
                sent.append(("send", [n for n, _ in it], args))

        params = [("model.a.weight", torch.zeros(4, 2)), ("model.b.weight", torch.zeros(3, dtype=torch.bfloat16))]
        info = {"names": [n for n, _ in params], "dtype_names": ["torch.float32", "BFloat16".lower()],
                "shapes": [[4, 2], [3]], "packed": True}
        sync = VllmNcclSync(c, "127.0.0.1", 29999, 3, engine=FakeEngine, send_args=lambda **kw: kw)
        out = sync.sync(params, info)
        assert out["sent"] == 2 and out["bytes"] == 4 * 2 * 4 + 3 * 2 and out["server"]["ok"]
        paths = [p for p, _ in calls]
        assert paths == ["/init_weight_transfer_engine", "/pause?mode=wait", "/update_weights", "/resume"]
        assert calls[0][1]["init_info"] == {"master_address": "127.0.0.1", "master_port": 29999, "rank_offset": 1,
                                            "world_size": 3}
        upd = calls[2][1]["update_info"]
        assert upd["dtype_names"] == ["float32", "bfloat16"] and upd["is_checkpoint_format"] is True
        assert sent[0] == ("init", {"master_address": "127.0.0.1", "master_port": 29999, "world_size": 3})
        assert sent[1][1] == ["model.a.weight", "model.b.weight"] and sent[1][2]["group"] == "group"
        assert sent[1][2]["packed_buffer_size_bytes"] == 1 << 30 and sent[1][2]["packed_num_buffers"] == 2
        calls.clear()
        update_seen.clear()
        sync.sync(params, info)                               # the group is opened once
        assert [p for p, _ in calls] == ["/pause?mode=wait", "/update_weights", "/resume"]
        assert normalize_dtype_name("torch.bfloat16") == "bfloat16" and normalize_dtype_name("Float") == "float32"
        # the server's side handled elsewhere: no init request, no update request - the engine is still driven
        calls.clear()
        sent.clear()
        update_seen.set()
        bare = VllmNcclSync(c, "127.0.0.1", 29998, 3, engine=FakeEngine, send_args=lambda **kw: kw, pause=False,
                            server_init=False, update_metadata=False, packed=False)
        out = bare.sync(params, info)
        assert calls == [] and out["server"] is None and out["sent"] == 2
        assert sent[0][0] == "init" and sent[1][0] == "send" and sent[1][2]["packed"] is False
    finally:
        server.shutdown()


def test_bridge_module_name_of_the_reference():
    import inspect
    import _cverl_vllm_bridge as bridge
    from cverl_b200.rollout.vllm_bridge import QwenPolicy
    assert bridge.QwenPolicy is QwenPolicy
    sig = inspect.signature(QwenPolicy.gsm8k_grpo_update)
    assert list(sig.parameters)[1:6] == ["prompts", "responses", "answers", "prompt_indices", "sample_indices"]
    assert sig.parameters["learning_rate"].default == 3.0e-6 and sig.parameters["reward_method"].default == "flexible"
    assert list(inspect.signature(QwenPolicy.__init__).parameters)[1:] == ["model_dir", "tokenizer_path", "device",
                                                                          "param_dtype", "max_layers"]


def test_transport_messages_round_trip_for_arbitrary_content():
    """Property test of the wire format: any request / response - empty lists, non-ASCII and NUL-bearing text,
    extreme integers, special floats - comes back equal, and every proper prefix of a message is refused."""
    hyp = pytest.importorskip("hypothesis")
    st = pytest.importorskip("hypothesis.strategies")
    from cverl_b200.rollout.transport import RolloutRequest, RolloutResponse, RolloutSequence
    i64 = st.integers(min_value=-2 ** 63, max_value=2 ** 63 - 1)
    u31 = st.integers(min_value=0, max_value=2 ** 31 - 1)
    text = st.text(max_size=20)
    flt = st.floats(allow_nan=False, width=64)
    requests = st.builds(RolloutRequest, prompts=st.lists(text, max_size=3),
                         prompt_token_ids=st.lists(st.lists(i64, max_size=5), max_size=3), n=u31, max_tokens=u31,
                         temperature=flt, top_p=flt, top_k=u31, stop=st.lists(text, max_size=2), flags=u31, seed=i64,
                         model=text, extra_params=st.dictionaries(text, text, max_size=3), request_id=i64)
    sequences = st.builds(RolloutSequence, prompt_index=u31, sample_index=u31, text=text,
                          token_ids=st.lists(i64, max_size=6), logprobs=st.lists(flt, max_size=6), finish_reason=text)
    responses = st.builds(RolloutResponse, sequences=st.lists(sequences, max_size=3),
                          metrics=st.dictionaries(text, flt, max_size=3))

    @hyp.settings(max_examples=150, deadline=None)
    @hyp.given(requests, responses, st.data())
    def check(req, resp, data):
        raw = serialize_request(req)
        assert deserialize_request(raw) == req
        out = serialize_response(resp)
        assert deserialize_response(out) == resp
        if len(raw) > 1:
            cut = data.draw(st.integers(min_value=0, max_value=len(raw) - 1))
            with pytest.raises(Exception):
                deserialize_request(raw[:cut])
    check()
