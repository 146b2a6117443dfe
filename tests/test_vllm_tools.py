"""Tooling around a vLLM baseline server (routing feed, gate hook, all-reduce replacement, launcher) on CPU, against
stand-in modules: no vLLM process and no GPU are involved."""
import os
import time
import types

import torch

from inferencehackathon_b200.serve import vllm_tools as vt


def _wait(cond, timeout=5.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if cond():
            return True
        time.sleep(0.01)
    return False


class _Gate(torch.nn.Module):
    """Returns (logits, None) like vLLM's replicated linear layer."""

    def __init__(self, h, e, seed):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.w = torch.nn.Parameter(torch.randn(e, h, generator=g))

    def forward(self, x):
        return x @ self.w.t(), None


class _Block(torch.nn.Module):
    def __init__(self, seed):
        super().__init__()
        self.gate = _Gate(16, 32, seed)

    def forward(self, hidden_states):
        logits, _ = self.gate(hidden_states)
        return hidden_states + logits.sum(-1, keepdim=True) * 0.0


def test_feed_round_trip_and_telemetry(tmp_path):
    path = str(tmp_path / "r.sock")
    feed = vt.RoutingFeed(path).start()
    assert feed.send({"token": 0, "layer": 0, "experts": [1]}) is False and feed.dropped == 1     # nobody listens yet
    reader = vt.RoutingFeedReader(path, retry_s=0.02)
    assert _wait(feed.connected)
    for tok in range(2):
        for layer in range(3):
            assert feed.send({"token": tok, "layer": layer, "experts": [tok + layer, 10 + layer]})
    feed.send({"layer": "broken"})                                        # a malformed line is skipped by the reader
    assert _wait(lambda: reader.records == 6)
    assert reader.latest_token() == 1
    assert reader.layers_of() == {0: [1, 10], 1: [2, 11], 2: [3, 12]}
    assert reader.layers_of(0)[2] == [2, 12]
    topo = {"placement": {"1": {"2": 5, "11": 6}}}
    tel = vt.telemetry_from_feed(reader, 4, 12.345, topo)                  # token 4 shows layer 4 % 3 = 1
    assert tel["token_index"] == 4 and tel["t_ms"] in (12.34, 12.35)
    assert tel["experts"] == [{"layer": 1, "expert_id": 2, "gpu": 5}, {"layer": 1, "expert_id": 11, "gpu": 6}]
    full = vt.telemetry_from_feed(reader, 0, 0.0, topo, all_layers=True)
    assert [e["layer"] for e in full["experts"]] == [0, 0, 1, 1, 2, 2]
    reader.close()
    feed.close()
    assert not os.path.exists(path)


def test_feed_starts_listening_in_the_process_that_sends(tmp_path):
    path = str(tmp_path / "lazy.sock")
    feed = vt.RoutingFeed(path)                                            # not started: as inherited by a forked worker
    assert not os.path.exists(path)
    assert feed.send({"token": 0, "layer": 0, "experts": [1]}) is False     # the first record opens the listener
    assert os.path.exists(path)
    reader = vt.RoutingFeedReader(path, retry_s=0.02)
    assert _wait(feed.connected)
    assert feed.send({"token": 0, "layer": 1, "experts": [2]})
    assert _wait(lambda: reader.layers_of() == {1: [2]})
    reader.close()
    feed.close()


def test_empty_feed_gives_no_telemetry(tmp_path):
    reader = vt.RoutingFeedReader(str(tmp_path / "absent.sock"), retry_s=0.02)
    assert vt.telemetry_from_feed(reader, 0, 0.0, {}) is None
    reader.close()


def test_gate_hook_reports_the_routers_own_choices():
    blocks = [_Block(s) for s in range(3)]
    sent = []
    uninstall = vt.install_routing_hook(_Block, sent.append, top_k=4)
    xs = [torch.randn(2, 16, generator=torch.Generator().manual_seed(7 + t)) for t in range(2)]
    for x in xs:                                                            # two decode steps through the three layers
        for b in blocks:
            b(x)
    assert [(r["token"], r["layer"]) for r in sent] == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1), (1, 2)]
    uninstall()                                                             # the gates below must not report again
    n = len(sent)
    for r in sent:
        logits, _ = blocks[r["layer"]].gate(xs[r["token"]])
        assert r["experts"] == torch.topk(logits[0], 4).indices.tolist()     # first row = the token being decoded
    blocks[0](xs[0])
    assert len(sent) == n


def test_all_reduce_replacement_dispatches_by_shape():
    calls = {"orig": 0, "fused": 0}

    def orig(t, *a, **k):
        calls["orig"] += 1
        return t

    class Fused:
        def accepts(self, t):
            return t.dim() == 2 and t.shape[0] <= 4

        def __call__(self, t):
            calls["fused"] += 1
            return t * 2

    mod = types.SimpleNamespace(tensor_model_parallel_all_reduce=orig)
    unpatch = vt.patch_tensor_parallel_all_reduce(mod, Fused())
    assert torch.equal(mod.tensor_model_parallel_all_reduce(torch.ones(2, 8)), 2 * torch.ones(2, 8))
    mod.tensor_model_parallel_all_reduce(torch.ones(64, 8))                 # a prompt-sized tensor keeps the original path
    mod.tensor_model_parallel_all_reduce(torch.ones(2, 8), "extra")          # an unknown calling form too
    assert calls == {"orig": 2, "fused": 1}
    unpatch()
    assert mod.tensor_model_parallel_all_reduce is orig


def test_all_reduce_replacement_rebinds_modules_that_imported_the_function(monkeypatch):
    import sys

    def orig(t):
        return t

    class Fused:
        def accepts(self, t):
            return True

        def __call__(self, t):
            return t + 1

    home = types.ModuleType("fakellm.comm")
    user = types.ModuleType("fakellm.models.moe")
    other = types.ModuleType("elsewhere.mod")
    for m in (home, user, other):
        m.tensor_model_parallel_all_reduce = orig
        monkeypatch.setitem(sys.modules, m.__name__, m)
    unpatch = vt.patch_tensor_parallel_all_reduce(home, Fused(), importers_prefix="fakellm")
    assert float(user.tensor_model_parallel_all_reduce(torch.zeros(1, 4)).sum()) == 4.0
    assert other.tensor_model_parallel_all_reduce is orig                   # outside the prefix: untouched
    unpatch()
    assert home.tensor_model_parallel_all_reduce is orig and user.tensor_model_parallel_all_reduce is orig


def test_fused_all_reduce_refuses_what_the_kernel_cannot_take():
    f = vt.FusedSmallAllReduce()
    assert not f.accepts(torch.ones(2, 8))                                  # host tensor
    assert not f.accepts(torch.ones(2, 8, 3))


def test_launcher_command_line(capsys):
    argv = vt.build_serve_argv("/models/q", tp=4, port=9000, extra=["--enforce-eager"])
    assert argv[:3] == ["vllm", "serve", "/models/q"] and argv.count("--enforce-eager") == 1
    assert "--enforce-eager" in vt.build_serve_argv("/m") and "--enforce-eager" not in vt.build_serve_argv("/m", eager=False)
    assert argv[argv.index("--tensor-parallel-size") + 1] == "4" and argv[argv.index("--port") + 1] == "9000"
    assert vt.main(["--model", "/models/q", "--tp", "2", "--print-only", "--max-model-len", "4096"]) == 0
    out = capsys.readouterr().out
    assert "vllm serve /models/q" in out and "--max-model-len 4096" in out


def test_vllm_backend_uses_the_feed_when_it_has_records(tmp_path):
    from inferencehackathon_b200.serve import backends as bk
    path = str(tmp_path / "b.sock")
    feed = vt.RoutingFeed(path).start()
    be = bk.VLLMBackend(scrape_spec=False, routing_sock=path)
    topo = {"num_layers": 94, "experts_per_layer": 128, "placement": {}}
    assert len(be._telemetry(0, 1.0, topo)["experts"]) == 8                 # nothing fed yet: the synthetic cycle
    assert _wait(feed.connected)
    feed.send({"token": 0, "layer": 0, "experts": [3, 9]})
    assert _wait(lambda: be.feed.records == 1)
    assert be._telemetry(1, 2.0, topo)["experts"] == [{"layer": 0, "expert_id": 3, "gpu": 3}, {"layer": 0, "expert_id": 9, "gpu": 1}]
    be.feed.close()
    feed.close()


def test_fed_routing_drives_the_prediction_pipeline(tmp_path, monkeypatch):
    from inferencehackathon_b200.serve import backends as bk
    monkeypatch.setenv("ROUTE_PIPELINE", "1")
    monkeypatch.setenv("VLLM_NUM_LAYERS", "4")
    monkeypatch.setenv("VLLM_NUM_EXPERTS", "16")
    path = str(tmp_path / "p.sock")
    feed = vt.RoutingFeed(path).start()
    be = bk.VLLMBackend(scrape_spec=False, routing_sock=path)
    assert _wait(feed.connected)
    for tok in range(12):                                                   # every layer shifts the experts by one
        for layer in range(4):
            feed.send({"token": tok, "layer": layer, "experts": [(tok + layer + j) % 16 for j in range(8)]})
    assert _wait(lambda: be.pipeline.records == 48)
    st = be.pipeline.stats()
    assert st["tokens"] == 12 and st["prefetched"] > 0 and st["prefetch_hit_rate"] > 0.5
    be.feed.close()
    feed.close()


def test_reader_survives_any_line():
    """Lines that are not records (JSON of another shape, numbers that do not fit, binary junk) are skipped."""
    from hypothesis import given, settings, strategies as st

    reader = vt.RoutingFeedReader("/nonexistent/never.sock", retry_s=10.0)

    @settings(max_examples=200, deadline=None)
    @given(st.one_of(st.binary(max_size=60), st.sampled_from([b"[1,2]", b"3", b"null", b'"x"', b'{"layer":1}',
                                                                b'{"layer":"a","experts":[1]}', b'{"layer":1,"experts":7}',
                                                                b'{"layer":1e999,"experts":[1]}', b'{"layer":1,"experts":[[]]}',
                                                                b'{"token":null,"layer":2,"experts":[1]}'])))
    def feed(line):
        before = reader.records
        reader._take(line)
        assert reader.records in (before, before + 1)

    feed()
    reader._take(b'{"token": 3, "layer": 1, "experts": [4, 5]}')
    assert reader.layers_of(3) == {1: [4, 5]}
    reader.close()
