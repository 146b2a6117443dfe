"""Tooling around a vLLM server used as the serving baseline on the same GPUs.

Three parts, each usable on its own:

* **Routing feed.** The MoE blocks of a running vLLM report the experts their router picked for the token being decoded
  as newline-delimited JSON over a Unix socket, ``{"token": t, "layer": L, "experts": [..top_k ids..]}``
  (:class:`RoutingFeed`, :func:`install_routing_hook`). The demo server reads the feed (:class:`RoutingFeedReader`) and
  puts real expert ids into ``x_telemetry`` instead of a synthetic cycle (``VLLM_ROUTING_SOCK`` in
  ``serve/backends.py``). The hook listens on the block's own gate module, so the router runs once per layer; the
  reference re-computes the gate inside a replaced ``forward`` (tools/vllm_routing_hook.py:62-140,
  tools/start_vllm.py:79-112).
* **All-reduce replacement.** :func:`patch_tensor_parallel_all_reduce` swaps vLLM's tensor-parallel all-reduce for this
  package's counted NVSwitch kernel (one one-way trip through the switch, no barrier) for decode-sized messages and
  leaves every other call with vLLM's own path. The reference builds a multicast object in a coordinator process and
  imports it into every worker by file descriptor (tools/patch_vllm_nvls.py:222-480); here the workers' own process group
  carries the rendezvous of torch symmetric memory, so no coordinator is needed.
* **Launcher.** ``python -m inferencehackathon_b200.serve.vllm_tools --model /path --tp 8`` starts the feed, installs the
  hook (and the all-reduce replacement with ``--fused-allreduce``) and hands over to vLLM's ``serve`` command line
  (tools/start_vllm.py:118-137).

Nothing here runs without a vLLM install and model weights; the parts are tested on CPU against stand-in modules.
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import socket
import sys
import threading
import time
from typing import Callable, Deque, Dict, List, Optional

import torch

DEFAULT_SOCK = os.environ.get("VLLM_ROUTING_SOCK", "/tmp/vllm_routing.sock")


# ---- producer side: inside the vLLM process ---------------------------------------------------------------------------------------
class RoutingFeed:
    """Unix-socket server that streams routing records to ONE reader (the newest connection wins). Records sent while
    nobody listens are dropped: the feed must never slow the decode loop down. The listener belongs to the process that
    sends: ``send`` (re)starts it when called from another process than the one that started it, so a feed created in a
    launcher and inherited by a forked model worker listens in the worker, where the records are made."""

    def __init__(self, path: str = DEFAULT_SOCK):
        self.path = path
        self._srv: Optional[socket.socket] = None
        self._client: Optional[socket.socket] = None
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._pid = -1
        self.sent = 0
        self.dropped = 0

    def start(self) -> "RoutingFeed":
        self._lock = threading.Lock()                  # a lock copied by fork may be held by a thread that no longer exists
        self._stop = threading.Event()
        self._client = None
        self._pid = os.getpid()
        if os.path.exists(self.path):
            os.unlink(self.path)
        srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        srv.bind(self.path)
        srv.listen(1)
        srv.settimeout(0.2)
        self._srv = srv
        threading.Thread(target=self._accept_loop, name="routing-feed", daemon=True).start()
        return self

    def _accept_loop(self) -> None:
        while not self._stop.is_set():
            try:
                conn, _ = self._srv.accept()
            except socket.timeout:
                continue
            except OSError:
                return
            conn.setblocking(False)
            with self._lock:
                if self._client is not None:
                    try:
                        self._client.close()
                    except OSError:
                        pass
                self._client = conn

    def connected(self) -> bool:
        with self._lock:
            return self._client is not None

    def send(self, record: Dict) -> bool:
        if self._pid != os.getpid():
            self.start()
        data = (json.dumps(record, separators=(",", ":")) + "\n").encode()
        with self._lock:
            if self._client is None:
                self.dropped += 1
                return False
            try:
                self._client.sendall(data)
                self.sent += 1
                return True
            except (BlockingIOError, BrokenPipeError, ConnectionResetError, OSError):
                # a reader that went away or fell behind loses records; it does not stall the model
                try:
                    self._client.close()
                except OSError:
                    pass
                self._client = None
                self.dropped += 1
                return False

    def close(self) -> None:
        self._stop.set()
        with self._lock:
            for s in (self._client, self._srv):
                if s is not None:
                    try:
                        s.close()
                    except OSError:
                        pass
            self._client = None
        if os.path.exists(self.path):
            try:
                os.unlink(self.path)
            except OSError:
                pass


def _is_rank0() -> bool:
    try:
        import torch.distributed as dist
        return (not dist.is_available()) or (not dist.is_initialized()) or dist.get_rank() == 0
    except Exception:                                                   # noqa: BLE001 - telemetry must not break serving
        return True


def install_routing_hook(block_cls, send: Callable[[Dict], object], top_k: int = 8, gate_attr: str = "gate",
                         rank0_only: bool = True) -> Callable[[], None]:
    """Make every instance of the sparse-MoE block class ``block_cls`` report the experts of the FIRST token of each
    forward (B = 1 decode: the token being generated). The block's ``forward`` is wrapped only to attach, on an
    instance's first call, a forward hook to its gate module; the gate's own output is what gets ranked, so the layer
    does no extra matmul. Layers are numbered in the order their blocks first run; the token counter advances when
    layer 0 runs again. Returns a function that restores the class."""
    original = block_cls.forward
    state = {"layers": {}, "token": -1, "lock": threading.Lock(), "handles": []}

    def gate_hook(layer: int):
        def hook(_module, _inputs, output):
            if rank0_only and not _is_rank0():
                return
            logits = output[0] if isinstance(output, (tuple, list)) else output
            if not torch.is_tensor(logits) or logits.numel() == 0:
                return
            if logits.is_cuda and torch.cuda.is_current_stream_capturing():
                return                                  # reading the ids back would end a CUDA-graph capture
            with torch.no_grad():
                row = logits.reshape(-1, logits.shape[-1])[0]
                ids = torch.topk(row.float(), k=min(top_k, row.numel())).indices.tolist()
            with state["lock"]:
                if layer == 0:
                    state["token"] += 1
                tok = max(state["token"], 0)
            send({"token": tok, "layer": layer, "experts": ids})
        return hook

    def forward(self, *args, **kwargs):
        key = id(self)
        if key not in state["layers"]:
            with state["lock"]:
                if key not in state["layers"]:
                    layer = len(state["layers"])
                    state["layers"][key] = layer
                    gate = getattr(self, gate_attr, None)
                    if gate is not None and hasattr(gate, "register_forward_hook"):
                        state["handles"].append(gate.register_forward_hook(gate_hook(layer)))
        return original(self, *args, **kwargs)

    block_cls.forward = forward

    def uninstall() -> None:
        block_cls.forward = original
        for h in state["handles"]:
            h.remove()
        state["handles"].clear()

    return uninstall


# ---- consumer side: inside the demo server ---------------------------------------------------------------------------------------
class RoutingFeedReader:
    """Reads the feed in a background thread and keeps the records of the most recent tokens. Connects lazily and keeps
    retrying: the server may start before vLLM does."""

    def __init__(self, path: str = DEFAULT_SOCK, keep_tokens: int = 64, retry_s: float = 0.5,
                 on_record: Optional[Callable[[int, int, List[int]], None]] = None):
        self.path, self.retry_s = path, retry_s
        self.on_record = on_record                 # called in the reader thread with (token, layer, experts) of every record
        self._by_token: "collections.OrderedDict[int, Dict[int, List[int]]]" = collections.OrderedDict()
        self._keep = keep_tokens
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._recent: Deque[Dict] = collections.deque(maxlen=1024)
        self.records = 0
        self._thread = threading.Thread(target=self._run, name="routing-reader", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        while not self._stop.is_set():
            s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            try:
                s.connect(self.path)
            except OSError:
                s.close()
                self._stop.wait(self.retry_s)
                continue
            s.settimeout(0.2)
            buf = b""
            try:
                while not self._stop.is_set():
                    try:
                        chunk = s.recv(65536)
                    except socket.timeout:
                        continue
                    if not chunk:
                        break
                    buf += chunk
                    while b"\n" in buf:
                        line, buf = buf.split(b"\n", 1)
                        self._take(line)
            except OSError:
                pass
            finally:
                s.close()

    def _take(self, line: bytes) -> None:
        try:
            rec = json.loads(line)
            if not isinstance(rec, dict):
                return
            tok, layer, experts = int(rec.get("token", 0)), int(rec["layer"]), [int(e) for e in rec["experts"]]
        except (ValueError, KeyError, TypeError, OverflowError, RecursionError):
            return                              # a malformed line must not end the reader thread
        with self._lock:
            self.records += 1
            self._recent.append({"token": tok, "layer": layer, "experts": experts})
            row = self._by_token.setdefault(tok, {})
            row[layer] = experts
            while len(self._by_token) > self._keep:
                self._by_token.popitem(last=False)
        if self.on_record is not None:
            self.on_record(tok, layer, experts)

    def latest_token(self) -> Optional[int]:
        with self._lock:
            return next(reversed(self._by_token)) if self._by_token else None

    def layers_of(self, token: Optional[int] = None) -> Dict[int, List[int]]:
        """{layer: expert ids} of ``token`` (default: the newest token seen)."""
        with self._lock:
            if not self._by_token:
                return {}
            if token is None or token not in self._by_token:
                token = next(reversed(self._by_token))
            return dict(self._by_token[token])

    def close(self) -> None:
        self._stop.set()


def telemetry_from_feed(reader: RoutingFeedReader, token_index: int, t_ms: float, topo: dict,
                        all_layers: bool = False) -> Optional[dict]:
    """``x_telemetry`` record built from the newest token of the feed, None while the feed is empty. One layer per token
    (cycling with the token index, like the engine backend) unless ``all_layers``."""
    layers = reader.layers_of()
    if not layers:
        return None
    placement = topo.get("placement", {})
    order = sorted(layers)
    pick = order if all_layers else [order[token_index % len(order)]]
    experts = []
    for L in pick:
        row = placement.get(str(L), {})
        experts += [{"layer": L, "expert_id": e, "gpu": row.get(str(e), e % 8)} for e in layers[L]]
    return {"token_index": token_index, "t_ms": round(t_ms, 2), "experts": experts, "spec": {"proposed": 0, "accepted": 0}}


# ---- all-reduce replacement ------------------------------------------------------------------------------------------------------
class FusedSmallAllReduce:
    """Sum over the ranks of the default process group with this package's counted kernel: up to ``ARC_MAX_ROWS`` rows of
    at most 8192 channels, fp32 or bf16. The symmetric buffer is built on first use (a collective: every rank reaches its
    first small all-reduce at the same point of the model)."""

    def __init__(self, max_hidden: int = 8192, group_fn: Optional[Callable[[], object]] = None):
        self.max_hidden = max_hidden
        self.group_fn = group_fn                   # returns the process group to reduce over (default: the world group)
        self.hidden: Optional[int] = None          # the slot layout depends on the row width: fixed by the first call
        self._ready = False
        self.n_calls = 0
        self.check_every = 256                     # calls between two reads of the device error word (a read synchronises)

    def _setup(self, device: torch.device) -> None:
        import torch.distributed as dist
        from ..config import ParallelConfig
        from ..ops import lib as K
        from ..parallel.symm import SymmetricComm
        group = self.group_fn() if self.group_fn is not None else None
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        par = ParallelConfig(tp=world, ep=1, rank=rank, world=world)
        nbytes = 4 * K.ARC_MAX_ROWS * self.max_hidden * 8
        self.K = K
        self.comm = SymmetricComm(par, device, slot_floats=1024, group=group, extra_bytes=nbytes)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.counter = torch.zeros(8, dtype=torch.int32, device=device)
        self.calls = torch.zeros(K.ARC_MAX_ROWS, dtype=torch.int32, device=device)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self.comm.extra(nbytes).zero_()
        self.comm.barrier_host()
        self.cm = self.comm.comm_block(self.epoch, slot_offset_bytes=self.comm.extra_off)
        self._ready = True

    def accepts(self, t: torch.Tensor) -> bool:
        from ..ops import lib as K
        return (t.is_cuda and t.dim() == 2 and t.is_contiguous() and t.dtype in (torch.float32, torch.bfloat16)
                and 1 <= t.shape[0] <= K.ARC_MAX_ROWS and t.shape[1] <= self.max_hidden and t.shape[1] % 4 == 0
                and (self.hidden is None or t.shape[1] == self.hidden))

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        if not self._ready:
            self._setup(t.device)
            self.hidden = int(t.shape[1])
        out = torch.empty(t.shape, dtype=torch.float32, device=t.device)
        self.K.allreduce_counted(self.cm, t, out, self.counter, self.calls, self.err)
        self.n_calls += 1
        if self.n_calls % self.check_every == 0:
            self.check()
        return out if t.dtype == torch.float32 else out.to(t.dtype)

    def check(self) -> None:
        """Raise if a bounded device-side wait gave up (a rank that stopped calling): the sums since then are not valid."""
        if self._ready:
            code = int(self.err.item())
            if code:
                raise RuntimeError(f"fused all-reduce: device-side wait gave up ({self.K.ERR_NAMES.get(code, code)})")


def patch_tensor_parallel_all_reduce(target, fused=None, name: str = "tensor_model_parallel_all_reduce",
                                     importers_prefix: Optional[str] = None) -> Callable[[], None]:
    """Replace ``target.<name>`` (vLLM: ``vllm.distributed.communication_op``) by a function that sends decode-sized
    tensors through ``fused`` and everything else through the original. Model files bind the function by
    ``from ... import``; with ``importers_prefix`` (``"vllm"``) every loaded module of that prefix that holds the original
    under the same name is rebound too. ``fused`` needs ``accepts(tensor) -> bool`` and ``__call__(tensor) -> tensor``;
    default :class:`FusedSmallAllReduce`. Returns a function that restores every binding."""
    original = getattr(target, name)
    fused = fused if fused is not None else FusedSmallAllReduce()

    def all_reduce(tensor, *args, **kwargs):
        if not args and not kwargs and fused.accepts(tensor):
            return fused(tensor)
        return original(tensor, *args, **kwargs)

    all_reduce.__wrapped__ = original
    rebound = [target]
    setattr(target, name, all_reduce)
    if importers_prefix:
        for mod_name, mod in list(sys.modules.items()):
            if mod is None or mod is target or not mod_name.startswith(importers_prefix):
                continue
            if getattr(mod, name, None) is original:
                setattr(mod, name, all_reduce)
                rebound.append(mod)

    def unpatch() -> None:
        for mod in rebound:
            setattr(mod, name, original)

    return unpatch


# ---- launcher -----------------------------------------------------------------------------------------------------------------------
def build_serve_argv(model: str, tp: int = 8, port: int = 8001, extra: Optional[List[str]] = None,
                     eager: bool = True) -> List[str]:
    """Command line handed to vLLM's ``serve`` (the flags the reference launcher passes, tools/start_vllm.py:124-132).
    ``eager``: add ``--enforce-eager``; the gate hook reads expert ids back to the host, which neither a compiled graph
    nor a CUDA-graph capture allows (under capture the hook stays silent)."""
    extra = list(extra or [])
    argv = ["vllm", "serve", model, "--tensor-parallel-size", str(tp), "--port", str(port),
            "--chat-template-content-format", "string"]
    if eager and "--enforce-eager" not in extra:
        argv.append("--enforce-eager")
    return argv + extra


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Start vLLM with the routing feed (and optionally the fused all-reduce) installed")
    ap.add_argument("--model", default=os.environ.get("VLLM_MODEL_PATH", ""))
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--port", type=int, default=8001)
    ap.add_argument("--sock", default=DEFAULT_SOCK)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--fused-allreduce", action="store_true", help="decode-sized tensor-parallel all-reduces go through this "
                    "package's counted NVSwitch kernel")
    ap.add_argument("--graphs", action="store_true", help="do not add --enforce-eager (the routing feed then only reports "
                    "steps that run outside CUDA graphs)")
    ap.add_argument("--print-only", action="store_true", help="print the vLLM command line and exit")
    a, extra = ap.parse_known_args(argv)
    if not a.model:
        ap.error("--model (or VLLM_MODEL_PATH) is required")
    serve_argv = build_serve_argv(a.model, a.tp, a.port, extra, eager=not a.graphs)
    if a.print_only:
        print(" ".join(serve_argv))
        return 0
    try:
        from vllm.model_executor.models.qwen3_moe import Qwen3MoeSparseMoeBlock
    except Exception as e:                                              # noqa: BLE001 - report and stop: nothing to serve with
        print(f"vllm is not usable here: {type(e).__name__}: {e}", file=sys.stderr)
        return 2
    # the model runs in worker processes: fork them, so that they inherit the patched classes; the feed starts
    # listening in the worker that sends the first record (rank 0 of the tensor-parallel group)
    os.environ.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "fork")
    feed = RoutingFeed(a.sock)
    install_routing_hook(Qwen3MoeSparseMoeBlock, feed.send, top_k=a.top_k)
    if a.fused_allreduce:
        import vllm.distributed.communication_op as comm_op

        def tp_group():
            from vllm.distributed.parallel_state import get_tp_group
            return get_tp_group().device_group

        patch_tensor_parallel_all_reduce(comm_op, FusedSmallAllReduce(group_fn=tp_group), importers_prefix="vllm")
    sys.argv = serve_argv
    print(f"[routing] feed on {a.sock}; starting: {' '.join(serve_argv)}", flush=True)
    from vllm.entrypoints.cli.main import main as vllm_main
    t0 = time.time()
    try:
        vllm_main()
    finally:
        feed.close()
        print(f"[routing] vLLM ended after {time.time() - t0:.0f} s; records sent {feed.sent}, dropped {feed.dropped}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
