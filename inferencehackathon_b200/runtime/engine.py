"""The inference engine: prefill, single-token decode, generation loop, device-timed steps and per-token
expert-routing telemetry.

Two backends share this front end: ``torch`` runs the functional PyTorch model (CPU/gloo configuration, and
the oracle on GPU), ``cuda`` runs the sm_100a kernel pipeline of :mod:`..runtime.gpu_decoder` under a CUDA
graph. The reference has no engine object: its drivers are ``main()`` functions that replay one layer of dummy
weights 94 times, never append to the KV cache across steps and have no sampler beyond argmax
(kernels/decode_step_tp8.cu:50-54, 1155-1184).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from ..config import EngineConfig, ModelConfig, ParallelConfig, QuantConfig, env_flag, get_model_config
from ..models.qwen3_moe import Qwen3MoE, RouteRecord
from ..models.weights import (DeviceRandomStateDict, ModelWeights, random_sharded_weights, random_state_dict,
                              shard_state_dict)
from ..parallel.collectives import Collectives
from ..utils.timing import StepTimer
from .sampler import Sampler, SamplingParams


class _nvtx:
    """NVTX range around a device-side stage (prefill, decode step, verify window): shows up in timeline tools, costs a
    few hundred nanoseconds otherwise. A no-op on the CPU."""

    def __init__(self, name: str, device):
        self.name, self.on = name, torch.device(device).type == "cuda"

    def __enter__(self):
        if self.on:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.on:
            torch.cuda.nvtx.range_pop()
        return False


@dataclass
class PrefillOutput:
    n_prompt_tokens: int
    seconds: float
    next_token: int
    logits: Optional[torch.Tensor] = None


@dataclass
class StepOutput:
    index: int
    token_id: int
    seconds: float
    routes: List[RouteRecord] = field(default_factory=list)


@dataclass
class GenerationResult:
    prompt_tokens: int
    tokens: List[int]
    ttft_s: float
    step_seconds: List[float]
    routes: List[List[RouteRecord]]
    spec_proposed: int = 0
    spec_accepted: int = 0

    @property
    def decode_tok_per_s(self) -> float:
        t = sum(self.step_seconds)
        return (len(self.step_seconds) / t) if t > 0 else 0.0


def expert_gpu(expert_id: int, cfg: ModelConfig, par: ParallelConfig) -> int:
    """GPU that serves an expert: its owner under expert parallelism; under pure tensor parallelism every rank
    holds a slice of every expert and the home convention ``expert % world`` of the reference server is kept
    (server/topology.py:45-64)."""
    if par.ep > 1:
        return expert_id // (cfg.n_experts // par.ep)
    return expert_id % max(par.world, 1)


class InferenceEngine:
    """One rank of the engine. All ranks of a parallel run call the same methods in the same order."""

    def __init__(self, cfg: EngineConfig, weights: ModelWeights, comm: Optional[Collectives] = None,
                 device=None):
        self.cfg = cfg
        self.weights = weights
        self.device = torch.device(device if device is not None else weights.embed.device)
        self.comm = comm if comm is not None else Collectives(cfg.parallel)
        backend = cfg.backend
        if backend == "auto":
            backend = "cuda" if self.device.type == "cuda" else "torch"
        self.backend = backend
        self.model = Qwen3MoE(weights, self.comm)
        kv_dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp8": torch.float8_e4m3fn}[cfg.quant.kv]
        self.gpu = None
        if backend == "cuda":
            from .gpu_decoder import GpuDecoder            # imports the compiled kernels; fails loudly if absent
            self.gpu = GpuDecoder(cfg, weights, self.comm, self.device)
            self.cache = None
        else:
            self.cache = self.model.new_cache(cfg.max_seq, kv_dtype, self.device)
        # expert parallel on GPUs: multi-token windows exchange rows through peer memory (one kernel per exchange)
        par = cfg.parallel
        if self.device.type == "cuda" and par.ep > 1 and par.world > 1 and env_flag("IHB_A2A", 1):
            from ..parallel.a2a import PeerRowExchange
            window = min(cfg.max_seq, 1024)
            self.comm.fast_a2a = PeerRowExchange(self.device, (cfg.model.hidden + 2 + 3) // 4 * 4,
                                                 -(-window // par.world) * cfg.model.top_k)
        self.sampler = Sampler()
        self._last_token: Optional[int] = None
        self._index = 0
        self._timer = StepTimer(self.device)
        # failure handling: tokens fed so far (to rebuild the cache on the fallback path) and the health record
        self._history: List[int] = []
        self.healthy = True
        self.fallback_enabled = True
        self.failures: List[str] = []

    # construction ------------------------------------------------------------------------------------------
    @classmethod
    def build(cls, model: str = "tiny", *, tp: int = 1, ep: int = 1, rank: int = 0, world: Optional[int] = None,
              weights: str = "fp32", kv: Optional[str] = None, device="cpu", backend: str = "auto",
              max_seq: int = 2048, seed: int = 0, n_layers: Optional[int] = None, distinct_layers: int = 0,
              state_dict=None, checkpoint: Optional[str] = None, comm: str = "auto",
              use_graph: bool = True, same_weights_in_every_layout: bool = False,
              kv_seq_split: bool = False) -> "InferenceEngine":
        """Public constructor. Weight source, in order: ``state_dict`` (HF names), ``checkpoint`` (safetensors
        directory), else random init (host-side and layout-independent for small models, streamed on the
        device otherwise: per-rank random streams, fast, but a sharded engine then holds other numbers than the
        one-GPU engine; ``same_weights_in_every_layout`` generates every full tensor on the device from a seed derived
        from its name and slices it, for comparisons across layouts). ``kv_seq_split`` (PyTorch path): the ranks that
        share a KV head split its cache rows between them instead of replicating them."""
        mcfg = get_model_config(model, n_layers)
        world = world if world is not None else max(tp, ep)
        share = tp // mcfg.n_kv_heads if (kv_seq_split and tp > mcfg.n_kv_heads) else 1
        par = ParallelConfig(tp=tp, ep=ep, rank=rank, world=world, kv_share=share)
        par.validate(mcfg)
        q = QuantConfig(weights=weights, kv=kv or ("fp32" if weights == "fp32" else "bf16"))
        ecfg = EngineConfig(model=mcfg, parallel=par, quant=q, max_seq=max_seq, seed=seed, backend=backend,
                            distinct_layers=distinct_layers, comm=comm, use_graph=use_graph)
        if state_dict is not None or checkpoint is not None:
            w = shard_state_dict(state_dict if state_dict is not None else checkpoint, mcfg, par, q, device=device)
        elif mcfg.total_params() <= 300_000_000:
            w = shard_state_dict(random_state_dict(mcfg, seed), mcfg, par, q, device=device)
        elif same_weights_in_every_layout:
            w = shard_state_dict(DeviceRandomStateDict(mcfg, seed, device), mcfg, par, q, device=device)
        else:
            w = random_sharded_weights(mcfg, par, q, device, seed, distinct_layers)
        return cls(ecfg, w, device=device)

    # state ---------------------------------------------------------------------------------------------------
    @property
    def seq_len(self) -> int:
        return self.gpu.seq_len if self.gpu is not None else self.cache.len

    def reset(self) -> None:
        if self.gpu is not None:
            self.gpu.reset()
        else:
            self.cache.reset()
        self._last_token = None
        self._index = 0
        self._history = []

    def set_sampling(self, params: SamplingParams) -> None:
        self.sampler = Sampler(params)

    # forward passes ------------------------------------------------------------------------------------------
    def prefill(self, token_ids: Sequence[int], return_logits: bool = False) -> PrefillOutput:
        """Process the prompt, fill the KV cache, return the first generated token (device-timed)."""
        toks = torch.as_tensor(list(token_ids), dtype=torch.long, device=self.device)
        self._history += [int(t) for t in token_ids]
        self._timer.start()
        if self.gpu is not None:
            try:
                with _nvtx("ihb.prefill", self.device):
                    nxt, logits = self.gpu.prefill(toks, self.sampler, return_logits)
            except RuntimeError as e:
                self._fall_back(e, drop=len(toks))
                return self.prefill_torch(toks, return_logits)
        else:
            hidden = self.model.forward_hidden(toks, self.cache)
            nxt, logits = self._pick(hidden[-1:], return_logits)
        seconds = self._timer.stop()
        self._last_token = int(nxt)
        self._index = 0
        return PrefillOutput(len(toks), seconds, int(nxt), logits)

    def prefill_torch(self, toks: torch.Tensor, return_logits: bool) -> PrefillOutput:
        self._timer.start()
        hidden = self.model.forward_hidden(toks, self.cache)
        nxt, logits = self._pick(hidden[-1:], return_logits)
        seconds = self._timer.stop()
        self._last_token = int(nxt)
        self._index = 0
        return PrefillOutput(len(toks), seconds, int(nxt), logits)

    # failure handling --------------------------------------------------------------------------------------------
    def _fall_back(self, err: Exception, drop: int = 0) -> None:
        """A device-side wait gave up (a peer stopped answering, a poisoned error word, ...): the fused pipeline is
        abandoned, the engine is marked unhealthy and continues on the PyTorch + NCCL reference path. The KV cache of
        that path is rebuilt from the tokens fed so far (``drop`` = tokens of the failed call, which the caller
        re-runs)."""
        self.failures.append(f"{type(err).__name__}: {err}")
        self.healthy = False
        if not self.fallback_enabled or self.gpu is None:
            raise err
        if self.weights.layers and self.weights.layers[0].wqkv.data.device.type == "meta":
            raise RuntimeError("no fallback: the plain weight copies were released for the tiled layout") from err
        kv_dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp8": torch.float8_e4m3fn}[self.cfg.quant.kv]
        max_seq = self.gpu.max_seq
        self.gpu = None
        self.backend = "torch"
        self.cache = self.model.new_cache(max_seq, kv_dtype, self.device)
        done = self._history[: len(self._history) - drop]
        if done:
            self.model.forward_hidden(torch.as_tensor(done, dtype=torch.long, device=self.device), self.cache)

    def _pick(self, hidden_last: torch.Tensor, return_logits: bool):
        if self.sampler.params.greedy and not return_logits:
            return int(self.model.greedy(hidden_last)[0]), None
        logits = self.model.logits(hidden_last)
        tok = self.sampler.sample(logits[0])
        if self.cfg.parallel.world > 1 and not self.sampler.params.greedy:
            # all ranks must continue with the same token: rank 0's draw wins
            t = tok.reshape(1).clone()
            torch.distributed.broadcast(t, src=0)
            tok = t[0]
        return int(tok), (logits if return_logits else None)

    def decode_step(self, token: Optional[int] = None, return_logits: bool = False,
                    want_routes: bool = True) -> StepOutput:
        """Feed one token (default: the previously generated one) and produce the next."""
        tok = self._last_token if token is None else token
        if tok is None:
            raise RuntimeError("decode_step before prefill")
        self._history.append(int(tok))
        if self.gpu is not None:
            try:
                with _nvtx("ihb.decode_step", self.device):
                    out_tok, seconds, routes = self.gpu.decode_step(tok, self.sampler, want_routes=want_routes)
            except RuntimeError as e:
                self._fall_back(e, drop=1)
        if self.gpu is None:
            t = torch.tensor([tok], dtype=torch.long, device=self.device)
            self._timer.start()
            hidden = self.model.forward_hidden(t, self.cache)
            out_tok, _ = self._pick(hidden, return_logits)
            seconds = self._timer.stop()
            routes = list(self.model.last_routes)
        self._last_token = int(out_tok)
        i = self._index
        self._index += 1
        return StepOutput(i, int(out_tok), seconds, routes)

    def decode_many(self, n: int, per_launch: int = 8) -> List[int]:
        """``n`` greedy tokens with ONE host synchronisation: the persistent kernel produces ``per_launch`` tokens per
        cooperative launch, feeding its own arg-max back, and logs them in a device ring (no per-token host round
        trip, no routing telemetry). Other pipelines, samplers and the PyTorch path fall back to ``decode_step``."""
        if (self.gpu is None or not self.gpu.use_mega or not self.sampler.params.greedy or self._last_token is None
                or n < 1):
            return [self.decode_step(want_routes=False).token_id for _ in range(n)]
        try:
            with _nvtx("ihb.decode_many", self.device):
                toks = self.gpu.decode_many(n, per_launch)
        except RuntimeError as e:
            self._fall_back(e, drop=0)
            return [self.decode_step(want_routes=False).token_id for _ in range(n)]
        self._history += [int(self._last_token)] + [int(t) for t in toks[:-1]]
        self._last_token = int(toks[-1])
        self._index += n
        return [int(t) for t in toks]

    def logits_for(self, tokens: Sequence[int], commit: bool = True, tree_mask=None, positions=None,
                   aux_layers=()) -> torch.Tensor:
        """Logits ``[T, V]`` of a window of new tokens (speculative verify, chains and token trees)."""
        if self.gpu is not None:
            with _nvtx("ihb.verify_window" if not commit or tree_mask is not None else "ihb.window", self.device):
                logits = self.gpu.logits_for(tokens, commit=commit, tree_mask=tree_mask, positions=positions,
                                             aux_layers=tuple(aux_layers))
            self.model.aux_taps = getattr(self.gpu.window(), "aux_taps", {})
            return logits
        t = torch.as_tensor(list(tokens), dtype=torch.long, device=self.device)
        hidden = self.model.forward_hidden(t, self.cache, positions=positions, tree_mask=tree_mask,
                                           commit=commit, aux_layers=tuple(aux_layers))
        return self.model.logits(hidden)

    def rollback(self, seq_len: int) -> None:
        """Drop KV rows beyond ``seq_len`` (rejected draft tokens)."""
        if self.gpu is not None:
            self.gpu.rollback(seq_len)
        else:
            self.cache.len = seq_len

    # generation ----------------------------------------------------------------------------------------------
    def generate(self, prompt_ids: Sequence[int], max_new_tokens: int, *, eos: Optional[int] = None,
                 sampling: Optional[SamplingParams] = None,
                 on_token: Optional[Callable[[StepOutput], None]] = None) -> GenerationResult:
        if sampling is not None:
            self.set_sampling(sampling)
        self.reset()
        pre = self.prefill(prompt_ids)
        tokens = [pre.next_token]
        secs: List[float] = []
        routes: List[List[RouteRecord]] = [list(self.model.last_routes) if self.gpu is None else self.gpu.last_routes()]
        if on_token is not None:
            on_token(StepOutput(-1, pre.next_token, pre.seconds, routes[0]))
        while len(tokens) < max_new_tokens and (eos is None or tokens[-1] != eos):
            st = self.decode_step()
            tokens.append(st.token_id)
            secs.append(st.seconds)
            routes.append(st.routes)
            if on_token is not None:
                on_token(st)
        return GenerationResult(len(prompt_ids), tokens, pre.seconds, secs, routes)
