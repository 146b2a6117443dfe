"""HTTP contract of the serving layer (CPU): health / models / topology, SSE framing with x_telemetry and x_summary,
backend selection, the vLLM proxy against a fake HTTP response, Prometheus spec counters, and the real engine
streaming real router selections."""
import io
import json

import pytest
from fastapi.testclient import TestClient

from inferencehackathon_b200.serve import backends as bk
from inferencehackathon_b200.serve.app import create_app
from inferencehackathon_b200.serve.mock_engine import ENGINE_PROFILES, mock_stream
from inferencehackathon_b200.serve.optimization_telemetry import B200X8, floor_breakdown, summary_fields
from inferencehackathon_b200.serve.schemas import ChatMessage, ChatRequest, sse, sse_done
from inferencehackathon_b200.serve.spec_metrics import accept_stats, cumulative_accept, parse_spec_counters
from inferencehackathon_b200.serve.topology import build_topology


def _frames(text):
    return [f[6:] for f in text.split("\n\n") if f.startswith("data: ")]


def test_health_models_topology():
    c = TestClient(create_app(bk.MockBackend()))
    assert c.get("/health").json()["status"] == "ok"
    assert c.get("/v1/models").json()["data"][0]["id"] == "qwen3-235b-a22b"
    t = c.get("/v1/topology").json()
    assert len(t["gpus"]) == 8 and t["num_layers"] == 94 and t["experts_per_layer"] == 128
    assert t["placement"]["3"]["17"] == 17 % 8 and t["placement_source"] in ("round-robin", "optimized")
    assert set(t["gpus"][0]) == {"id", "name", "mem_total_mb", "mem_used_mb", "utilization_pct", "temp_c"}


def test_sse_contract_with_mock_backend():
    c = TestClient(create_app(bk.MockBackend()))
    body = {"messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6, "stream": True}
    r = c.post("/v1/chat/completions", json=body)
    assert r.headers["content-type"].startswith("text/event-stream")
    frames = _frames(r.text)
    assert frames[-1] == "[DONE]"
    summary = json.loads(frames[-2])["x_summary"]
    chunks = [json.loads(f) for f in frames[:-2]]
    assert len(chunks) == 6 and all(ch["object"] == "chat.completion.chunk" for ch in chunks)
    for i, ch in enumerate(chunks):
        tel = ch["x_telemetry"]
        assert tel["token_index"] == i and len(tel["experts"]) == 8
        assert all(0 <= e["gpu"] < 8 and e["layer"] == i % 94 for e in tel["experts"])
        assert tel["spec"]["accepted"] <= tel["spec"]["proposed"]
    for key in ("ttft_ms", "decode_tok_per_s", "prefill_tokens", "completion_tokens", "spec_accept_rate", "engine",
                "spec_enabled", "floor_breakdown_ms", "regime", "next_lever", "pct_of_ceiling", "pct_of_roofline"):
        assert key in summary
    assert summary["prefill_tokens"] == 2 and summary["completion_tokens"] == 6
    r2 = c.post("/v1/chat/completions", json={**body, "stream": False, "engine": "vllm"})
    assert r2.json()["object"] == "chat.completion" and r2.json()["choices"][0]["message"]["content"]


def test_mock_is_deterministic_and_profiles_differ():
    req = ChatRequest(messages=[ChatMessage(role="user", content="x")], max_tokens=5)
    topo = build_topology()
    assert list(mock_stream(req, topo)) == list(mock_stream(req, topo))
    v = list(mock_stream(ChatRequest(messages=req.messages, max_tokens=5, engine="vllm"), topo))[-1]["x_summary"]
    a = list(mock_stream(req, topo))[-1]["x_summary"]
    assert a["decode_tok_per_s"] > v["decode_tok_per_s"] and a["spec_enabled"] and not v["spec_enabled"]
    assert set(ENGINE_PROFILES) == {"conifer", "vllm"}
    assert sse({"a": 1}) == 'data: {"a": 1}\n\n' and sse_done() == "data: [DONE]\n\n"


def test_optimization_telemetry_blocks():
    bd = floor_breakdown(11.7, "bf16", "bf16", 17.0, 512)
    assert bd["weight"] == pytest.approx(1.61, abs=0.01) and bd["comms"] == pytest.approx(3.196, abs=1e-3)
    assert bd["overhead"] == pytest.approx(11.7 - bd["weight"] - bd["comms"] - bd["kv"], abs=2e-3)
    s = summary_fields(11.7, 85.7, "bf16")
    assert s["regime"] == "floor-bound" and 0 < s["pct_of_roofline"] < 100
    w = summary_fields(0.9, 1100.0, "fp8", collective_us=0.1)
    assert w["regime"] == "weight-bound"
    assert summary_fields(2.0, 500.0, "fp8", profile=B200X8)["floor_breakdown_ms"]["weight"] < bd["weight"] / 2


def test_backend_selection(monkeypatch):
    monkeypatch.setenv("BACKEND", "mock")
    assert isinstance(bk.get_backend(), bk.MockBackend)
    monkeypatch.delenv("BACKEND")
    monkeypatch.setattr(bk, "_vllm_healthy", lambda url=None: True)
    assert isinstance(bk.get_backend(), bk.VLLMBackend)
    monkeypatch.setattr(bk, "_vllm_healthy", lambda url=None: False)
    assert isinstance(bk.get_backend(), bk.MockBackend)


class _FakeResponse(io.BytesIO):
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def test_vllm_proxy_reframes_and_summarises(monkeypatch):
    words = ["Hi", " there", " friend"]
    payload = b"".join(b"data: " + json.dumps({"choices": [{"delta": {"content": w}}]}).encode() + b"\n\n" for w in words)
    payload += b"data: [DONE]\n\n"
    monkeypatch.setattr(bk.urllib.request, "urlopen", lambda *a, **k: _FakeResponse(payload))
    out = list(bk.VLLMBackend(scrape_spec=False).stream(
        ChatRequest(messages=[ChatMessage(role="user", content="one two three")], max_tokens=8), build_topology()))
    assert [c["choices"][0]["delta"]["content"] for c in out[:-1]] == words
    assert all(len(c["x_telemetry"]["experts"]) == 8 for c in out[:-1])
    assert out[-1]["x_summary"]["completion_tokens"] == 3 and out[-1]["x_summary"]["prefill_tokens"] == 3


def test_spec_metrics_parsing():
    before = '# HELP x\nvllm:spec_decode_num_accepted_tokens_total{model="m"} 100\nvllm:spec_decode_num_drafts_total{model="m"} 50\n'
    after = 'vllm:spec_decode_num_accepted_tokens_total{model="m"} 160\nvllm:spec_decode_num_drafts_total{model="m"} 90\n'
    assert parse_spec_counters(before) == {"accepted": 100.0, "drafts": 50.0}
    st = accept_stats(before, after)
    assert st["accepted"] == 60 and st["drafts"] == 40 and st["tau"] == pytest.approx(2.5) and st["accept_rate"] == 1.0
    assert accept_stats(after, after)["tau"] == 1.0
    assert cumulative_accept("")["accept_rate"] == 0.0


def test_engine_backend_streams_real_routes():
    from inferencehackathon_b200 import TINY
    from inferencehackathon_b200.runtime.engine import InferenceEngine
    eng = InferenceEngine.build("tiny", weights="fp32", max_seq=128)
    backend = bk.EngineBackend(eng)
    c = TestClient(create_app(backend))
    t = c.get("/v1/topology").json()
    assert t["num_layers"] == TINY.n_layers and t["experts_per_layer"] == TINY.n_experts and t["placement_source"] == "engine"
    body = {"messages": [{"role": "user", "content": "route me"}], "max_tokens": 5, "temperature": 0.0}
    frames = _frames(c.post("/v1/chat/completions", json=body).text)
    chunks = [json.loads(f) for f in frames[:-2]]
    assert frames[-1] == "[DONE]" and len(chunks) == 5
    for i, ch in enumerate(chunks):
        ex = ch["x_telemetry"]["experts"]
        assert len(ex) == TINY.top_k and len({e["expert_id"] for e in ex}) == TINY.top_k
        assert all(e["layer"] == i % TINY.n_layers and 0 <= e["expert_id"] < TINY.n_experts for e in ex)
        assert ch["x_telemetry"]["t_ms"] > 0
    again = [json.loads(f) for f in _frames(c.post("/v1/chat/completions", json=body).text)[:-2]]
    assert [a["choices"][0]["delta"]["content"] for a in again] == [b["choices"][0]["delta"]["content"] for b in chunks]
    summ = json.loads(frames[-2])["x_summary"]
    assert summ["completion_tokens"] == 5 and summ["prefill_tokens"] == len("route me") and summ["decode_tok_per_s"] > 0
    assert "qwen3" in c.get("/v1/models").json()["data"][0]["id"]
    from server.main import app as shim_app     # the reference's import path
    assert shim_app.title == "multi-gpu-inference-console"


def test_engine_backend_with_speculative_driver_streams_same_text():
    from inferencehackathon_b200.runtime.engine import InferenceEngine
    from inferencehackathon_b200.spec.driver import SpecDriver
    from inferencehackathon_b200.spec.ngram import NGramDrafter
    eng = InferenceEngine.build("tiny", weights="fp32", max_seq=256)
    body = {"messages": [{"role": "user", "content": "abcabcabcabcabcabc"}], "max_tokens": 12, "temperature": 0.0}
    plain = [json.loads(f) for f in _frames(TestClient(create_app(bk.EngineBackend(eng))).post(
        "/v1/chat/completions", json=body).text)[:-2]]
    spec_backend = bk.EngineBackend(eng, spec_driver=SpecDriver(eng, NGramDrafter(2), depth=4, width=1, floor_fraction=1.0))
    frames = _frames(TestClient(create_app(spec_backend)).post("/v1/chat/completions", json=body).text)
    spec = [json.loads(f) for f in frames[:-2]]
    text = lambda cs: [c["choices"][0]["delta"]["content"] for c in cs]
    assert text(spec) == text(plain) and len(spec) == 12
    summ = json.loads(frames[-2])["x_summary"]
    assert summ["spec_enabled"] is True and 0.0 <= summ["spec_accept_rate"] <= 1.0
    assert all("spec" in c["x_telemetry"] for c in spec)


def test_metrics_endpoint_counts_tokens_and_speculation():
    from fastapi.testclient import TestClient
    from inferencehackathon_b200.serve.app import create_app
    from inferencehackathon_b200.serve import backends as bk
    from inferencehackathon_b200.serve.spec_metrics import parse_spec_counters
    c = TestClient(create_app(bk.MockBackend()))
    before = c.get("/metrics").text
    assert "ihb:requests_total 0.0" in before and "# TYPE ihb:generation_tokens_total counter" in before
    body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 12, "temperature": 0.0}
    frames = [f[6:] for f in c.post("/v1/chat/completions", json=body).text.split("\n\n") if f.startswith("data: ")]
    n_tokens = sum(1 for f in frames if f != "[DONE]" and "x_telemetry" in f)
    text = c.get("/metrics").text
    vals = {l.split()[0]: float(l.split()[1]) for l in text.splitlines() if l and not l.startswith("#")}
    assert vals["ihb:requests_total"] == 1.0 and vals["ihb:generation_tokens_total"] == float(n_tokens) > 0
    assert vals["ihb:ttft_seconds_count"] == 1.0 and vals["ihb:ttft_seconds_sum"] > 0 and vals["ihb:backend_healthy"] == 1.0
    # the scraper written for a vLLM server reads the same counters here
    spec = parse_spec_counters(text)
    assert spec["accepted"] == vals["ihb:spec_decode_num_accepted_tokens_total"]
    assert spec["drafts"] == vals["ihb:spec_decode_num_drafts_total"]
    # non-streaming requests are counted too
    c.post("/v1/chat/completions", json=dict(body, stream=False))
    assert "ihb:requests_total 2.0" in c.get("/metrics").text


def test_engine_backend_can_run_on_an_e4m3_kv_cache(monkeypatch):
    """``ENGINE_KV=fp8`` builds the served engine with e4m3 KV rows (scale per position); the stream still carries real
    router ids."""
    from inferencehackathon_b200.serve import backends as bk
    monkeypatch.setenv("ENGINE_MODEL", "tiny")
    monkeypatch.setenv("ENGINE_DEVICE", "cpu")
    monkeypatch.setenv("ENGINE_KV", "fp8")
    be = bk._build_engine_backend()
    assert be.engine.cfg.quant.kv == "fp8" and be.engine.cache.fp8


def test_engine_backend_reports_route_prediction_when_the_pipeline_is_on(monkeypatch):
    """``ROUTE_PIPELINE=1``: the routing of every streamed token drives the native Markov predictor and prefetch
    scheduler, and the turn's summary says how many predicted experts were really selected."""
    from fastapi.testclient import TestClient
    from inferencehackathon_b200 import TINY
    from inferencehackathon_b200.runtime.engine import InferenceEngine
    from inferencehackathon_b200.serve.app import create_app
    eng = InferenceEngine.build("tiny", weights="fp32", max_seq=128)
    body = {"messages": [{"role": "user", "content": "route me"}], "max_tokens": 12, "temperature": 0.0}
    plain = json.loads(_frames(TestClient(create_app(bk.EngineBackend(eng))).post("/v1/chat/completions", json=body).text)[-2])
    assert "route_prediction" not in plain["x_summary"]
    monkeypatch.setenv("ROUTE_PIPELINE", "1")
    backend = bk.EngineBackend(eng)
    frames = _frames(TestClient(create_app(backend)).post("/v1/chat/completions", json=body).text)
    rp = json.loads(frames[-2])["x_summary"]["route_prediction"]
    assert rp["tokens"] == 12 and rp["records"] == 12 * TINY.n_layers
    assert rp["prefetched"] > 0 and 0.0 <= rp["prefetch_hit_rate"] <= 1.0 and rp["hits"] <= rp["prefetched"]


def test_served_engine_can_use_a_hugging_face_tokenizer_directory(tmp_path, monkeypatch):
    """``ENGINE_TOKENIZER`` points at a tokenizer directory; a tiny word-level tokenizer is built here, offline."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    words = ["[UNK]", "route", "me", "to", "the", "experts", "please"]
    t = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="[UNK]"))
    t.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=t, unk_token="[UNK]").save_pretrained(str(tmp_path))
    monkeypatch.setenv("ENGINE_MODEL", "tiny")
    monkeypatch.setenv("ENGINE_DEVICE", "cpu")
    monkeypatch.setenv("ENGINE_TOKENIZER", str(tmp_path))
    be = bk._build_engine_backend()
    assert be.tok.encode("route me please") == [1, 2, 6] and be.tok.decode([3, 4, 5]).split() == ["to", "the", "experts"]
    from fastapi.testclient import TestClient
    from inferencehackathon_b200.serve.app import create_app
    frames = _frames(TestClient(create_app(be)).post("/v1/chat/completions", json={
        "messages": [{"role": "user", "content": "route me to the experts"}], "max_tokens": 4, "temperature": 0.0}).text)
    summ = json.loads(frames[-2])["x_summary"]
    assert summ["prefill_tokens"] == 5 and summ["completion_tokens"] == 4


def test_served_engine_loads_a_safetensors_checkpoint_directory(tmp_path, monkeypatch):
    """``ENGINE_CHECKPOINT``: the served engine reads Hugging Face safetensors shards instead of drawing random weights."""
    import torch
    from safetensors.torch import save_file
    from inferencehackathon_b200.config import get_model_config
    from inferencehackathon_b200.models.weights import random_state_dict
    from inferencehackathon_b200.runtime.engine import InferenceEngine
    sd = random_state_dict(get_model_config("tiny"), 11)
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    monkeypatch.setenv("ENGINE_MODEL", "tiny")
    monkeypatch.setenv("ENGINE_DEVICE", "cpu")
    monkeypatch.setenv("ENGINE_CHECKPOINT", str(tmp_path))
    be = bk._build_engine_backend()
    ref = InferenceEngine.build("tiny", weights="fp32", state_dict=sd)
    other = InferenceEngine.build("tiny", weights="fp32")                  # seed 0: another model
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    got = be.engine.prefill(prompt, return_logits=True).logits
    assert torch.equal(got, ref.prefill(prompt, return_logits=True).logits)
    assert not torch.equal(got, other.prefill(prompt, return_logits=True).logits)


def test_package_command_line_generates_and_reports(capsys):
    from inferencehackathon_b200.__main__ import main
    assert main(["generate", "--model", "tiny", "--prompt", "abc", "--max-new", "6", "--kv", "fp8", "--json"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["prompt_tokens"] == 3 and out["new_tokens"] == 6 and out["kv"] == "fp8" and out["backend"] == "torch"
    assert out["ttft_ms"] > 0 and out["decode_tok_per_s"] > 0 and isinstance(out["text"], str)
    assert main(["generate", "--prompt", "x" * 40, "--max-seq", "32"]) == 2          # no room left: refused with a reason
    capsys.readouterr()
    assert main(["info"]) == 0
    info = json.loads(capsys.readouterr().out)
    assert set(info["native_libraries"]) == {"libihb_kernels.so", "libihb_ctrl.so"}
    assert info["presets"]["qwen3-235b-a22b"]["experts"] == 128 and info["presets"]["tiny"]["layers"] == 4


from hypothesis import given, settings, strategies as st   # noqa: E402


@settings(max_examples=150, deadline=None)
@given(st.text(max_size=300), st.text(max_size=300))
def test_metric_scrape_parser_never_raises_and_keeps_rates_in_range(before, after):
    """Arbitrary scrape text (truncated lines, odd numbers, binary junk) around the counters: the parser returns finite
    numbers, an accept rate in [0, 1] and tau >= 1."""
    import math
    from inferencehackathon_b200.serve.spec_metrics import accept_stats, cumulative_accept
    head = 'vllm:spec_decode_num_accepted_tokens_total{model="m"} 12\nvllm:spec_decode_num_drafts_total 20\n'
    for b, a in ((before, after), (head + before, head + after), (before, head + after)):
        for r in (accept_stats(b, a), cumulative_accept(a)):
            assert all(math.isfinite(float(v)) for v in r.values())
            assert 0.0 <= r["accept_rate"] <= 1.0 and r["tau"] >= 1.0 and r["accepted"] >= 0.0 and r["drafts"] >= 0.0


_json_values = st.recursive(st.none() | st.booleans() | st.integers(-5, 20) | st.floats(allow_nan=False, allow_infinity=True) | st.text(max_size=4),
                            lambda c: st.lists(c, max_size=3) | st.dictionaries(st.sampled_from(["0", "1", "2", "placement", "x"]), c, max_size=4),
                            max_leaves=12)


@settings(max_examples=120, deadline=None)
@given(_json_values)
def test_placement_file_of_any_shape_yields_a_complete_in_range_table(tmp_path_factory, doc):
    """Whatever JSON the placement file holds (another model's table, wrong types, GPUs that are not there), the topology
    has one GPU in range for every (layer, expert); valid entries are kept, the rest fall back to round robin."""
    from pathlib import Path
    from inferencehackathon_b200.serve.topology import _load_placement
    path = Path(tmp_path_factory.mktemp("pl")) / "placement.json"
    path.write_text(json.dumps({"placement": doc}) if not isinstance(doc, float) else json.dumps({"placement": None}))
    table = _load_placement(3, 4, 2, path)
    assert sorted(table) == ["0", "1", "2"]
    for L, row in table.items():
        assert sorted(row) == ["0", "1", "2", "3"] and all(isinstance(g, int) and 0 <= g < 2 for g in row.values())
    if isinstance(doc, dict) and isinstance(doc.get("1"), dict) and doc["1"].get("2") in (0, 1) and not isinstance(doc["1"].get("2"), bool):
        assert table["1"]["2"] == doc["1"]["2"]
