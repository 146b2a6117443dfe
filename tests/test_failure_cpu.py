"""Failure handling without a GPU: (a) a device-side wait that gives up surfaces as an exception of the decode
pipeline; the engine marks itself unhealthy, rebuilds the cache on the PyTorch + collectives reference path from
the tokens fed so far and keeps generating the same tokens; the serving layer turns an unrecoverable error into an
in-stream error chunk. (b) A host-side model of the cross-GPU slot / arrival-counter protocol of the fused
all-reduce (double-buffered slots by round parity, monotonic counter, bounded waits) is run under random
interleavings and never reads a slot of the wrong round; a rank that stops arriving ends the others' waits with an
error status instead of a hang."""
import json
import random

import pytest
import torch

from inferencehackathon_b200.runtime.engine import InferenceEngine


class _FailingDecoder:
    """Stands in for the CUDA decoder: works for ``ok_steps`` decode steps, then reports a timed-out device wait."""

    def __init__(self, inner: InferenceEngine, ok_steps: int, prefill_fails: bool = False):
        self.inner, self.ok_steps, self.prefill_fails = inner, ok_steps, prefill_fails
        self.max_seq = inner.cache.max_seq
        self.steps = 0

    def reset(self):
        self.inner.reset()

    @property
    def seq_len(self):
        return self.inner.seq_len

    def prefill(self, toks, sampler, return_logits):
        if self.prefill_fails:
            raise RuntimeError("device-side wait gave up: peer barrier time-out")
        out = self.inner.prefill(toks.tolist(), return_logits)
        return out.next_token, out.logits

    def decode_step(self, tok, sampler, want_routes=True):
        if self.steps >= self.ok_steps:
            raise RuntimeError("device-side wait gave up: peer barrier time-out")
        self.steps += 1
        st = self.inner.decode_step(tok)
        return st.token_id, st.seconds, st.routes

    def last_routes(self):
        return list(self.inner.model.last_routes)

    def check_error(self):
        pass


def _engines():
    eng = InferenceEngine.build("tiny", weights="fp32", max_seq=128)
    shadow = InferenceEngine.build("tiny", weights="fp32", max_seq=128)
    return eng, shadow


@pytest.mark.parametrize("ok_steps,prefill_fails", [(3, False), (0, False), (0, True)])
def test_engine_falls_back_to_reference_path_and_keeps_its_tokens(ok_steps, prefill_fails):
    prompt = torch.randint(0, 2048, (12,), generator=torch.Generator().manual_seed(1)).tolist()
    want = InferenceEngine.build("tiny", weights="fp32", max_seq=128).generate(prompt, 10).tokens
    eng, shadow = _engines()
    eng.gpu = _FailingDecoder(shadow, ok_steps, prefill_fails)
    got = eng.generate(prompt, 10).tokens
    assert got == want
    assert eng.healthy is False and eng.gpu is None and eng.backend == "torch"
    assert len(eng.failures) == 1 and "time-out" in eng.failures[0]
    # the next request runs on the fallback path from the start
    assert eng.generate(prompt, 6).tokens == want[:6]


def test_fallback_can_be_disabled_and_server_reports_in_stream():
    from fastapi.testclient import TestClient
    from inferencehackathon_b200.serve import backends as bk
    from inferencehackathon_b200.serve.app import create_app
    eng, shadow = _engines()
    eng.gpu = _FailingDecoder(shadow, 2)
    eng.fallback_enabled = False
    backend = bk.EngineBackend(eng)
    c = TestClient(create_app(backend))
    body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 8, "temperature": 0.0}
    frames = [f[6:] for f in c.post("/v1/chat/completions", json=body).text.split("\n\n") if f.startswith("data: ")]
    objs = [json.loads(f) for f in frames if f != "[DONE]"]
    assert any("error" in o and o["error"]["type"] == "engine_error" for o in objs)
    assert backend.healthy is False and frames[-1] == "[DONE]"


# ---- protocol model ---------------------------------------------------------------------------------------------------------
class _Rank:
    def __init__(self, r, n):
        self.r, self.n = r, n
        self.epoch = 0
        self.pc = "push"
        self.out = []
        self.err = None
        self.spins = 0


def _run_protocol(n_ranks, rounds, seed, dead_rank=None, dead_after=None, spin_limit=200):
    """Slots [parity][rank] and one arrival counter per GPU. Each rank: push value(round) into slot[parity][self] of
    every GPU, arrive on every GPU's counter, wait until the own counter reaches (epoch + 1) * n, read all slots of
    the parity, next round. The scheduler picks which rank advances one step."""
    rng = random.Random(seed)
    slots = [[[None] * n_ranks for _ in range(2)] for _ in range(n_ranks)]
    counter = [0] * n_ranks
    ranks = [_Rank(r, n_ranks) for r in range(n_ranks)]
    live = list(range(n_ranks))
    while live:
        r = rng.choice(live)
        k = ranks[r]
        if dead_rank == r and k.epoch >= dead_after and k.pc == "push":
            live.remove(r)                       # stops between rounds, nothing in flight
            continue
        par = k.epoch & 1
        if k.pc == "push":
            for g in range(n_ranks):
                slots[g][par][r] = (k.epoch, r)
            k.pc = "arrive"
        elif k.pc == "arrive":
            for g in range(n_ranks):
                counter[g] += 1
            k.pc = "wait"
        elif k.pc == "wait":
            if counter[r] >= (k.epoch + 1) * n_ranks:
                k.pc = "read"
                k.spins = 0
            else:
                k.spins += 1
                if k.spins > spin_limit:         # bounded wait: status, not a hang
                    k.err = "peer barrier time-out"
                    live.remove(r)
        else:
            got = list(slots[r][par])
            assert all(v is not None and v[0] == k.epoch for v in got), (r, k.epoch, got)
            k.out.append(sum(v[1] for v in got))
            k.epoch += 1
            k.pc = "push"
            if k.epoch == rounds:
                live.remove(r)
    return ranks


@pytest.mark.parametrize("n_ranks", [2, 4, 8])
def test_slot_protocol_never_reads_a_stale_or_future_round(n_ranks):
    for seed in range(20):
        ranks = _run_protocol(n_ranks, rounds=12, seed=seed)
        want = [sum(range(n_ranks))] * 12
        assert all(k.out == want and k.err is None for k in ranks)


def test_slot_protocol_with_single_buffer_would_break():
    """The same schedule with ONE slot set (parity ignored) lets a fast rank overwrite a slot a slow rank has not
    read yet: the double buffer is what makes one barrier per round enough."""
    def run(seed):
        rng = random.Random(seed)
        n = 2
        slots = [[None] * n for _ in range(n)]
        counter = [0] * n
        st = [dict(epoch=0, pc="push") for _ in range(n)]
        for _ in range(400):
            r = rng.randrange(n)
            k = st[r]
            if k["epoch"] >= 6:
                continue
            if k["pc"] == "push":
                for g in range(n):
                    slots[g][r] = k["epoch"]
                k["pc"] = "arrive"
            elif k["pc"] == "arrive":
                for g in range(n):
                    counter[g] += 1
                k["pc"] = "wait"
            elif k["pc"] == "wait":
                if counter[r] >= (k["epoch"] + 1) * n:
                    k["pc"] = "read"
            else:
                if any(v != k["epoch"] for v in slots[r]):
                    return True
                k["epoch"] += 1
                k["pc"] = "push"
        return False
    assert any(run(seed) for seed in range(200))


def test_rank_that_stops_arriving_gives_the_others_a_status_not_a_hang():
    ranks = _run_protocol(4, rounds=10, seed=3, dead_rank=2, dead_after=4)
    for k in ranks:
        if k.r == 2:
            assert k.epoch == 4 and k.err is None
        else:
            assert k.err == "peer barrier time-out" and 4 <= k.epoch <= 5
            assert k.out == [6] * k.epoch


# ---- tagged-slot protocol (the persistent kernel's all-reduce and phase hand-over) ----------------------------------------------
def _run_tagged(n_ranks, n_ctas, rounds, seed, n_parities=2, dead=None, spin_limit=400):
    """Every (rank, CTA) is an agent. Round n (tag n + 1): the agent pushes ITS element of its rank's partial sum as
    one {value, tag} store to every GPU - the stores to different GPUs land one at a time, in any order, at any later
    step - then reads all ranks x CTAs elements of the round from its own GPU, retrying an element until it carries
    the tag. No counter, no barrier. Returns (agents, violations): a violation is a read that accepted a value of
    another round."""
    rng = random.Random(seed)
    E = n_ctas                                              # elements per rank: one per CTA
    mem = [[[[(0, None)] * E for _ in range(n_ranks)] for _ in range(n_parities)] for _ in range(n_ranks)]
    inflight = []                                           # (gpu, parity, rank, elem, tag, value)
    agents = [dict(r=r, c=c, rnd=0, pc="push", todo=None, acc=0, out=[], err=None, spins=0)
              for r in range(n_ranks) for c in range(n_ctas)]
    live = list(range(len(agents)))
    violations = 0
    while live or inflight:
        if inflight and (not live or rng.random() < 0.5):
            g, p, r, e, tag, val = inflight.pop(rng.randrange(len(inflight)))
            mem[g][p][r][e] = (tag, val)
            continue
        i = rng.choice(live)
        a = agents[i]
        if dead is not None and (a["r"], a["c"]) == dead[0] and a["rnd"] >= dead[1] and a["pc"] == "push":
            live.remove(i)                                   # leaves between rounds with nothing in flight
            continue
        tag, par = a["rnd"] + 1, a["rnd"] % n_parities
        if a["pc"] == "push":
            for g in range(n_ranks):
                inflight.append((g, par, a["r"], a["c"], tag, (a["rnd"], a["r"], a["c"])))
            a["pc"], a["todo"], a["acc"] = "read", [(r, e) for r in range(n_ranks) for e in range(E)], 0
        else:
            r, e = a["todo"][0]
            t, val = mem[a["r"]][par][r][e]
            if t == tag:
                if val != (a["rnd"], r, e):
                    violations += 1
                a["acc"] += 1
                a["todo"].pop(0)
                a["spins"] = 0
                if not a["todo"]:
                    a["out"].append(a["acc"])
                    a["rnd"] += 1
                    a["pc"] = "push"
                    if a["rnd"] == rounds:
                        live.remove(i)
            else:
                a["spins"] += 1
                if a["spins"] > spin_limit:                  # bounded wait: status, not a hang
                    a["err"] = "tag time-out"
                    live.remove(i)
    return agents, violations


@pytest.mark.parametrize("n_ranks,n_ctas", [(1, 4), (2, 3), (4, 2), (8, 2)])
def test_tagged_slots_need_no_barrier_and_two_parities_suffice(n_ranks, n_ctas):
    for seed in range(10):
        agents, bad = _run_tagged(n_ranks, n_ctas, rounds=8, seed=seed)
        assert bad == 0
        assert all(a["err"] is None and a["out"] == [n_ranks * n_ctas] * 8 for a in agents)


def test_tagged_slots_with_one_parity_can_lose_a_round():
    """With a single slot set a fast agent's store of round n + 1 may land before a slow reader has taken round n:
    the reader then never sees tag n (a time-out in the model, a wrong wait in the kernel). Two parities exclude it,
    because a store of round n + 2 needs its author to have read ALL of round n + 1, which every agent pushed only
    after reading round n."""
    lost = 0
    for seed in range(60):
        agents, bad = _run_tagged(2, 2, rounds=6, seed=seed, n_parities=1, spin_limit=150)
        assert bad == 0                                      # a tag never validates another round's value
        lost += any(a["err"] for a in agents)
    assert lost > 0


def test_tagged_slots_dead_agent_gives_status_not_hang():
    agents, bad = _run_tagged(2, 2, rounds=6, seed=1, dead=((1, 0), 3), spin_limit=120)
    assert bad == 0
    for a in agents:
        if (a["r"], a["c"]) == (1, 0):
            assert a["rnd"] == 3 and a["err"] is None
        else:
            assert a["err"] == "tag time-out" and 3 <= a["rnd"] <= 4


# ---- counted-accumulation protocol (the persistent kernel's all-reduce) -----------------------------------------------------------
def _run_counted(n_ranks, n_ctas, layers, seed, n_parities=8, clear_after_barrier=True):
    """Model of the all-reduce of the persistent decode kernel. Every (rank, CTA) is an agent that owns ONE channel.
    A round: the agent adds its rank's partial of its channel into the round's slot on every GPU (the adds to different
    GPUs land one at a time, at any later step, in any order), then reads all channels of the round on its own GPU,
    waiting on each slot until it has counted n_ranks contributions. Two rounds per layer (attention, experts); after
    the first read of a layer the agent arrives at its GPU's grid barrier and, once the barrier is complete, clears its
    own channel in the slots of all rounds it has read since the last clearing; then it pushes the second round. Slots
    are reused every n_parities rounds. Returns the number of violations: a read that found more contributions than
    ranks or a sum that mixes rounds, and the agents."""
    rng = random.Random(seed)
    rounds = 2 * layers
    # mem[gpu][parity][channel] = [count, sum]
    mem = [[[[0, 0] for _ in range(n_ctas)] for _ in range(n_parities)] for _ in range(n_ranks)]
    inflight = []                                            # (gpu, parity, channel, value)
    arrivals = [0] * n_ranks
    agents = [dict(r=r, c=c, rnd=0, pc="push", todo=None, clr_lo=0, waits=0, spins=0, err=None)
              for r in range(n_ranks) for c in range(n_ctas)]
    live = list(range(len(agents)))
    bad = 0

    def value(rnd, rank, chan):                              # distinct per round: a mixed sum cannot look right
        return (rnd + 1) * 1000 + rank * 10 + chan

    def want(rnd, chan):
        return sum(value(rnd, r, chan) for r in range(n_ranks))

    while live or inflight:
        if inflight and (not live or rng.random() < 0.5):
            g, p, ch, v = inflight.pop(rng.randrange(len(inflight)))
            mem[g][p][ch][0] += 1
            mem[g][p][ch][1] += v
            continue
        i = rng.choice(live)
        a = agents[i]
        r, c, rnd = a["r"], a["c"], a["rnd"]
        par = rnd % n_parities
        if a["pc"] == "push":
            for g in range(n_ranks):
                inflight.append((g, par, c, value(rnd, r, c)))
            a["pc"], a["todo"] = "read", list(range(n_ctas))
        elif a["pc"] == "read":
            ch = a["todo"][0]
            cnt, tot = mem[r][par][ch]
            if cnt > n_ranks:
                bad += 1
            if cnt >= n_ranks:
                if tot != want(rnd, ch):
                    bad += 1
                a["todo"].pop(0)
                a["spins"] = 0
                if not a["todo"]:
                    a["rnd"] += 1
                    if a["rnd"] % 2 == 1:                     # first round of a layer read: arrive, later wait + clear
                        arrivals[r] += 1
                        a["waits"] += 1
                        a["pc"] = "barrier"
                    elif a["rnd"] == rounds:
                        live.remove(i)
                    else:
                        a["pc"] = "push"
            else:
                a["spins"] += 1
                if a["spins"] > 3000:                         # bounded wait: status, not a hang
                    a["err"] = "slot time-out"
                    live.remove(i)
        else:                                                 # barrier: complete when every CTA of this GPU has arrived
            if arrivals[r] >= a["waits"] * n_ctas:
                if clear_after_barrier:
                    for q in range(a["clr_lo"], a["rnd"]):
                        mem[r][q % n_parities][c] = [0, 0]
                    a["clr_lo"] = a["rnd"]
                a["pc"] = "push"
    return bad, agents


@pytest.mark.parametrize("n_ranks,n_ctas", [(1, 3), (2, 3), (4, 2), (8, 2)])
def test_counted_slots_are_complete_exact_and_reusable(n_ranks, n_ctas):
    for seed in range(8):
        bad, agents = _run_counted(n_ranks, n_ctas, layers=10, seed=seed)
        assert bad == 0
        assert all(a["err"] is None and a["rnd"] == 20 for a in agents)


def test_counted_slots_with_too_few_parities_lose_or_mix_contributions():
    """With two parities a fast GPU's add of round n + 2 can land in a slot that a slow CTA of this GPU has not read or
    cleared yet: the model then sees a mixed sum, a count above the number of ranks, or a wait that never ends."""
    broken = 0
    for seed in range(40):
        bad, agents = _run_counted(2, 3, layers=6, seed=seed, n_parities=2)
        broken += int(bad > 0 or any(a["err"] for a in agents))
    assert broken > 0


def test_counted_slots_without_clearing_cannot_be_reused():
    bad, agents = _run_counted(2, 2, layers=6, seed=0, n_parities=4, clear_after_barrier=False)
    assert bad > 0 or any(a["err"] for a in agents)


# ---- counted accumulation as a stand-alone launch (ar_counted_kernel) -----------------------------------------------------------
def _run_standalone_counted(n_ranks, n_rows, row_counts, seed, n_parities=4, dead_rank=None, dead_after=0):
    """Model of the small-message all-reduce kernel that the window path launches per collective. An agent is one
    (rank, row): in every call that covers its row it adds its partial into the row's word on every GPU (the adds land
    one at a time, at any later step, in any order), polls ITS OWN GPU's word until it has counted n_ranks
    contributions, checks the sum, clears the word (it is the word's only reader) and bumps the row's call count, which
    selects the parity of the row's next call. ``row_counts[k]`` rows take part in call k (the same sequence on every
    rank). Rows progress independently here; on the GPU the calls of a rank are ordered by the stream, which only removes
    interleavings. Returns (violations, agents)."""
    rng = random.Random(seed)
    mem = [[[[0, 0] for _ in range(n_rows)] for _ in range(n_parities)] for _ in range(n_ranks)]   # [gpu][parity][row]
    inflight = []
    agents = []
    for r in range(n_ranks):
        for t in range(n_rows):
            mine = [k for k, T in enumerate(row_counts) if T > t]          # the calls this row takes part in
            agents.append(dict(r=r, t=t, calls=mine, done=0, pc="push", spins=0, err=None))
    live = [i for i, a in enumerate(agents) if a["calls"]]
    bad = 0

    def value(k, rank, row):
        return (k + 1) * 1000 + rank * 10 + row

    while live or inflight:
        if inflight and (not live or rng.random() < 0.5):
            g, p, t, v = inflight.pop(rng.randrange(len(inflight)))
            mem[g][p][t][0] += 1
            mem[g][p][t][1] += v
            continue
        i = rng.choice(live)
        a = agents[i]
        r, t = a["r"], a["t"]
        k = a["calls"][a["done"]]                                           # global index of the row's current call
        par = a["done"] % n_parities                                        # the row's own call count picks the parity
        if a["pc"] == "push":
            if dead_rank == r and a["done"] >= dead_after:
                live.remove(i)                                              # this rank makes no further calls
                continue
            for g in range(n_ranks):
                inflight.append((g, par, t, value(k, r, t)))
            a["pc"] = "read"
        else:
            cnt, tot = mem[r][par][t]
            if cnt > n_ranks:
                bad += 1
            if cnt >= n_ranks:
                if tot != sum(value(k, q, t) for q in range(n_ranks)):
                    bad += 1
                mem[r][par][t] = [0, 0]
                a["done"] += 1
                a["spins"] = 0
                a["pc"] = "push"
                if a["done"] == len(a["calls"]):
                    live.remove(i)
            else:
                a["spins"] += 1
                if a["spins"] > 4000:                                       # bounded wait: an error status, not a hang
                    a["err"] = "peer time-out"
                    live.remove(i)
    return bad, agents


@pytest.mark.parametrize("n_ranks", [1, 2, 4, 8])
def test_standalone_counted_all_reduce_with_changing_row_counts(n_ranks):
    """Every call is complete and exact although the number of rows changes from call to call, the adds of a fast rank
    land while a slow rank still reads the previous call, and nothing but the words themselves synchronises the ranks."""
    for seed in range(6):
        rng = random.Random(100 + seed)
        row_counts = [rng.choice([1, 2, 5]) for _ in range(12)]
        bad, agents = _run_standalone_counted(n_ranks, 5, row_counts, seed)
        assert bad == 0
        assert all(a["err"] is None and a["done"] == len(a["calls"]) for a in agents)


def test_standalone_counted_all_reduce_needs_more_than_one_parity():
    """With a single slot per row a fast rank's add of call n + 1 lands in the word a slow rank has not read yet: the
    model sees a count above the number of ranks, a mixed sum, or a contribution wiped by the late clear (a wait that
    runs out). Two parities are already safe for this protocol (a rank adds call n + 2 only after every rank has
    contributed n + 1, i.e. has read and cleared n); the kernel keeps four."""
    broken = 0
    for seed in range(30):
        bad, agents = _run_standalone_counted(2, 2, [2] * 8, seed, n_parities=1)
        broken += int(bad > 0 or any(a["err"] for a in agents))
    assert broken > 0
    for seed in range(10):
        bad, agents = _run_standalone_counted(4, 2, [2] * 8, seed, n_parities=2)
        assert bad == 0 and all(a["err"] is None for a in agents)


def test_standalone_counted_all_reduce_with_a_rank_that_stops_calling_ends_with_a_status():
    bad, agents = _run_standalone_counted(4, 2, [2] * 6, seed=1, dead_rank=2, dead_after=3)
    assert bad == 0
    for a in agents:
        if a["r"] == 2:
            assert a["done"] == 3 and a["err"] is None
        else:
            assert a["err"] == "peer time-out" and a["done"] == 3          # all calls before the stop completed everywhere
