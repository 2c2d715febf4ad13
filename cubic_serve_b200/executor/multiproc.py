"""Process-per-GPU execution: a controller-side executor proxy and the rank worker loop.

Shape of the reference's controller / worker split (``runtime/performance.py:8813-9247`` ``_ProcessController``,
``runtime/quantized_graph.py:263`` worker there): the controller process owns HTTP, tokenisation, scheduling
and the page pool; one spawned worker per GPU owns the weights shard, the KV cache and the captured graphs.
A step is broadcast to every rank over pipes (all ranks execute the same batch), the sampler rank answers with
the token ids.  Liveness: a worker that exits, or a result that does not arrive within the watchdog period,
poisons the executor (fail closed) with a message that names the rank and decodes the exit signal.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import signal
import socket
import time
from dataclasses import dataclass

import numpy as np


class WorkerFailure(RuntimeError):
    pass


@dataclass
class WorkerSpec:
    model: str                   # checkpoint dir or random:<config>
    devices: list[int]
    tp: int
    k_bits: int
    v_bits: int
    max_rows: int
    token_budget: int
    max_model_len: int
    num_pages: int | None
    tp_comm: str = "fused"
    seed: int = 0
    gpu_reserve_gib: float = 4.0
    pp: int = 1                  # pipeline stages; rank = stage * tp + tensor rank
    kv_rotation: bool = False    # Walsh-Hadamard rotation of q / k / v before the cache write

    @property
    def world(self) -> int:
        return self.tp * self.pp


def describe_exit(code: int | None) -> str:
    """Human-readable reason for a child exit code (negative = killed by that signal)."""
    if code is None:
        return "still running"
    if code == 0:
        return "exited normally"
    if code < 0:
        try:
            name = signal.Signals(-code).name
        except ValueError:
            name = f"signal {-code}"
        hint = {"SIGSEGV": " (memory fault in native code)", "SIGKILL": " (killed, often by the out-of-memory killer)",
                "SIGBUS": " (bus error, often a full /dev/shm)"}.get(name, "")
        return f"terminated by {name}{hint}"
    return f"exited with status {code}"


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_main(rank: int, spec: WorkerSpec, port: int, conn) -> None:
    """Rank process: build everything, report readiness, then serve commands until told to close."""
    import torch
    import torch.distributed as dist

    from ..models.config import NAMED_CONFIGS
    from ..models.decoder import DecoderRunner, random_decoder_weights
    from ..contracts.execution import ParallelTopology
    from ..parallel.pp import PipelineStage
    from ..parallel.tp import TensorParallel
    from ..runtime.serving import plan_kv_pages
    from .gpu_executor import GpuExecutor
    try:
        dev = torch.device("cuda", spec.devices[rank])
        torch.cuda.set_device(dev)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        topo = ParallelTopology.single_node(spec.devices, spec.tp, spec.pp)
        place = topo.placement(rank)
        tp = pp = tp_group = None
        if spec.world > 1:
            dist.init_process_group("nccl", rank=rank, world_size=spec.world, device_id=dev)
            tp_group = dist.group.WORLD
            if spec.pp > 1 and spec.tp > 1:                   # every rank creates every stage's group, in order
                for stage in range(spec.pp):
                    g = dist.new_group(list(range(stage * spec.tp, (stage + 1) * spec.tp)))
                    if stage == place.stage:
                        tp_group = g
        conn.send(("progress", rank, "process group up"))
        t_rank = place.tensor_rank
        if spec.model.startswith("random:"):
            cfg = NAMED_CONFIGS[spec.model.split(":", 1)[1]]()
            layers = topo.layer_range(place.stage, cfg.num_layers)
            weights = random_decoder_weights(cfg, dev, spec.seed, t_rank, spec.tp, layer_range=layers)
        elif spec.model.endswith(".gguf"):
            import gguf

            from ..models.gguf import config_from_gguf, load_gguf_decoder_weights
            layers = topo.layer_range(place.stage, config_from_gguf(gguf.GGUFReader(spec.model)).num_layers)
            cfg, weights = load_gguf_decoder_weights(spec.model, dev, t_rank, spec.tp, layer_range=layers)
        else:
            from ..models.checkpoint import admit_checkpoint, load_decoder_weights
            ck = admit_checkpoint(spec.model)
            cfg = ck.cfg
            layers = topo.layer_range(place.stage, cfg.num_layers)
            weights = load_decoder_weights(ck, dev, t_rank, spec.tp, layer_range=layers)
        conn.send(("progress", rank, "weights loaded"))
        if spec.pp > 1:
            pp = PipelineStage.from_topology(topo, rank, dist.group.WORLD)
        if spec.tp > 1:
            tp = TensorParallel(tp_group, dev, mode="nccl" if spec.pp > 1 else spec.tp_comm, hidden=cfg.hidden_size,
                                max_tokens=spec.token_budget, rows_max=max(512, spec.max_rows))
        pages = spec.num_pages
        # models with recurrent layers keep as many state snapshot rows as request rows, for prefix caching
        snapshots = spec.max_rows if cfg.is_hybrid else 0
        if pages is None:
            free, _ = torch.cuda.mem_get_info(dev)
            pages = plan_kv_pages(free, int(spec.gpu_reserve_gib * 2 ** 30) + (2 << 30), cfg, spec.tp, spec.k_bits,
                                  spec.v_bits, spec.max_model_len, spec.max_rows, layers=layers[1] - layers[0],
                                  state_snapshots=snapshots)
        if spec.world > 1:
            # every rank runs the same code on the same model; the KV pool is the smallest any rank can hold
            import dataclasses

            from ..contracts.implementation import digest_of, identity
            from ..runtime.preparation import consensus
            agreed = consensus({"implementation": identity().digest, "model": digest_of(dataclasses.asdict(cfg)),
                                "tp": spec.tp, "pp": spec.pp, "kv_bits": [spec.k_bits, spec.v_bits],
                                "fixed_pages": spec.num_pages, "pages": pages}, minimum=("pages",))
            pages = int(agreed["pages"])
        runner = DecoderRunner(cfg, weights, num_pages=pages, max_tokens=spec.token_budget, k_bits=spec.k_bits,
                               v_bits=spec.v_bits, tp=tp, pp=pp, max_requests=spec.max_rows,
                               state_checkpoints=snapshots, kv_rotation=spec.kv_rotation)
        from ..runtime.serving import _tokenizer_for, reasoning_end_tokens
        think = reasoning_end_tokens(_tokenizer_for(spec.model, cfg.vocab_size))
        if think is not None:
            runner.enable_reasoning_budget(*think)      # every rank runs the same budget state machine
        ex = GpuExecutor(runner, max_rows=spec.max_rows, max_prefill_tokens=spec.token_budget,
                         max_model_len=spec.max_model_len)
        caps = ex.capture_decode_graphs()
        conn.send(("ready", rank, {"pages": pages, "capacities": caps, "vocab": cfg.vocab_size, "name": cfg.name,
                                   "reasoning_end_id": ex.reasoning_end_id, "hybrid": cfg.is_hybrid,
                                   "state_rows": list(ex.state_checkpoint_rows)}))
        while True:
            cmd = conn.recv()
            if cmd[0] == "execute":
                ids = ex.execute(cmd[1])
                runner.ws.check_status()
                if rank == 0:
                    conn.send(("result", ids, ex.kernel_launches_last))
            elif cmd[0] == "copy":
                ex.copy_pages(cmd[1])
                ex.invalidate_page_rows(cmd[2])
            elif cmd[0] == "copy_state":
                ex.copy_state(cmd[1])                   # recurrent-state rows: snapshot taken / snapshot restored
            elif cmd[0] == "close":
                break
        if spec.world > 1:
            dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001 - reported to the controller, which fails closed
        try:
            conn.send(("error", rank, f"{type(exc).__name__}: {exc}"))
        except Exception:  # noqa: BLE001
            pass
        raise


class MultiprocExecutor:
    """Controller-side proxy with the executor contract (``execute`` / ``copy_pages``)."""

    def __init__(self, spec: WorkerSpec, startup_timeout: float = 1800.0, result_timeout: float = 600.0,
                 worker_target=_worker_main, start: bool = True) -> None:
        self.spec = spec
        self.result_timeout = result_timeout
        self.startup_timeout = startup_timeout
        self.poisoned = False
        self.info: dict = {}
        self.h2d_bytes_last = self.d2h_bytes_last = self.kernel_launches_last = 0
        self._procs: list = []
        self._conns: list = []
        if start:
            self._spawn(worker_target)
            self._await_ready()

    def _spawn(self, target) -> None:
        ctx = mp.get_context("spawn")
        port = _free_port()
        for r in range(self.spec.world):
            parent, child = ctx.Pipe()
            p = ctx.Process(target=target, args=(r, self.spec, port, child), name=f"cubic-rank-{r}", daemon=True)
            p.start()
            child.close()
            self._procs.append(p)
            self._conns.append(parent)

    def _fail(self, message: str) -> None:
        self.poisoned = True
        raise WorkerFailure(message)

    def _check_alive(self) -> None:
        for r, p in enumerate(self._procs):
            if not p.is_alive():
                self._fail(f"rank {r} {describe_exit(p.exitcode)}")

    def _await_ready(self) -> None:
        """Each rank must report readiness; any validated progress message renews that rank's lease."""
        deadline = [time.time() + self.startup_timeout] * len(self._conns)
        ready = [False] * len(self._conns)
        while not all(ready):
            for r, c in enumerate(self._conns):
                if ready[r]:
                    continue
                if c.poll(0.05):
                    try:
                        msg = c.recv()
                    except EOFError:
                        self._check_alive()
                        self._fail(f"rank {r} closed its pipe during start-up")
                    if msg[0] == "ready":
                        ready[r] = True
                        self.info = self.info or msg[2]
                        if msg[2]["pages"] != self.info["pages"]:
                            self._fail("ranks disagree on the number of KV pages")
                    elif msg[0] == "progress":
                        deadline[r] = time.time() + self.startup_timeout
                    elif msg[0] == "error":
                        self._fail(f"rank {r} failed during start-up: {msg[2]}")
                elif time.time() > deadline[r]:
                    self._fail(f"rank {r} made no start-up progress for {self.startup_timeout:.0f} s")
            self._check_alive()

    # ------------------------------------------------------------- executor API
    @property
    def reasoning_end_id(self) -> int | None:
        return self.info.get("reasoning_end_id")

    @property
    def cfg(self):
        """Properties of the served model that the engine reads: recurrent layers (prefix caching then needs state
        snapshots) and the vocabulary size (width of the allowed-token masks of constrained requests)."""
        from types import SimpleNamespace
        return SimpleNamespace(is_hybrid=bool(self.info.get("hybrid", False)), vocab_size=int(self.info.get("vocab", 0)))

    @property
    def state_checkpoint_rows(self) -> tuple[int, ...]:
        """Snapshot rows of the workers' recurrent-state arrays (empty for models without recurrent layers)."""
        return tuple(self.info.get("state_rows", ()))

    def copy_state(self, pairs) -> None:
        if pairs:
            for c in self._conns:
                c.send(("copy_state", list(pairs)))

    def execute(self, segs) -> np.ndarray:
        if self.poisoned:
            raise WorkerFailure("executor is poisoned")
        if any(getattr(s, "mask_fn", None) is not None for s in segs):
            # the review-mask callbacks of speculative rounds are closures over the controller's grammar matchers:
            # they do not cross the pipe (the workers run plain steps, which use Segment.mask)
            from dataclasses import replace
            segs = [replace(s, mask_fn=None) if s.mask_fn is not None else s for s in segs]
        for c in self._conns:
            c.send(("execute", segs))
        c0 = self._conns[0]
        t0 = time.time()
        while not c0.poll(0.01):
            self._check_alive()
            if time.time() - t0 > self.result_timeout:
                self._fail(f"no result from the sampler rank within {self.result_timeout:.0f} s")
        try:
            msg = c0.recv()
        except EOFError:
            self._check_alive()
            self._fail("sampler rank closed its pipe")
        if msg[0] == "error":
            self._fail(f"rank {msg[1]} failed: {msg[2]}")
        self.kernel_launches_last = msg[2]
        return msg[1]

    def copy_pages(self, pairs) -> None:
        for c in self._conns:
            c.send(("copy", pairs, []))

    def invalidate_page_rows(self, slots) -> None:
        for c in self._conns:
            c.send(("copy", [], list(slots)))

    def close(self) -> None:
        for c in self._conns:
            try:
                c.send(("close",))
            except (OSError, BrokenPipeError):
                pass
        for p in self._procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()


def _check_partition(model: str, tp: int, pp: int) -> None:
    """Refuse a split the model does not admit before any worker is spawned (the planner names what does not divide)."""
    from ..models.config import NAMED_CONFIGS, ModelConfig
    from ..models.parallel_weights import PartitionError, plan_partition
    from pathlib import Path
    if model.startswith("random:"):
        cfg = NAMED_CONFIGS[model.split(":", 1)[1]]()
    elif (Path(model) / "config.json").exists():
        cfg = ModelConfig.from_hf_config(Path(model) / "config.json")
    else:
        return
    try:
        plan_partition(cfg, tp, pp, tp if cfg.is_moe else 1)      # experts are owned whole: EP over the TP ranks
    except PartitionError as exc:
        raise SystemExit(f"--tp-size {tp} --pp-size {pp} does not fit {cfg.name}: {exc}") from exc


def build_multiproc_backend(args, devices, tp, spec_cfg, k_bits, v_bits):
    from ..runtime.async_engine import TokenChatBackend
    from ..runtime.engine import LLMEngine
    from ..runtime.scheduler import SchedulerConfig
    from ..runtime.serving import _tokenizer_for
    max_len = args.max_model_len or 8192
    _check_partition(args.model, tp, args.pp_size)
    spec = WorkerSpec(args.model, devices, tp, k_bits, v_bits, args.max_running_requests, args.token_budget, max_len,
                      None, args.tp_comm, args.seed, args.gpu_reserve_gib, args.pp_size,
                      bool(getattr(args, "enable_kv_cache_rotation", False)))
    ex = MultiprocExecutor(spec)
    sched = SchedulerConfig(max_running_requests=args.max_running_requests, max_batched_tokens=args.token_budget,
                            prefill_chunk_tokens=min(args.prefill_chunk_tokens, args.token_budget), max_model_len=max_len,
                            enable_prefix_cache=args.prefix_cache)
    tok = _tokenizer_for(args.model, ex.info["vocab"])
    engine = LLMEngine(ex, num_pages=ex.info["pages"], scheduler_config=sched, eos_token_id=getattr(tok, "eos_token_id", None))
    return TokenChatBackend(engine, tok, default_thinking=args.thinking), ((args.served_model_name if isinstance(args.served_model_name, str) else (args.served_model_name or [None])[0])
                                                                                 or ex.info["name"])
