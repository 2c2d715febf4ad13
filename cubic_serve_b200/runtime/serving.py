"""Assemble a serving stack from CLI arguments and run it behind an HTTP server.

``build_backend`` follows the reference's start-up order (``cli.py:1074`` ``_serve_model`` /
``runtime/quantized_graph.py:263`` worker there): read the device memory budget, admit the checkpoint, load
rank-local weights, size the KV page pool from the memory that is left, capture the decode graph buckets
(largest first), then open the door.
"""
from __future__ import annotations

import logging
import threading
import time
from pathlib import Path

log = logging.getLogger("cubic.serve")


def _tokenizer_for(model: str, vocab_size: int):
    path = Path(model)
    if path.is_dir() and any((path / f).exists() for f in ("tokenizer.json", "tokenizer_config.json")):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(str(path))
    if path.suffix == ".gguf" and path.exists():
        # the file carries its tokenizer as metadata; a file without one falls through to the byte tokenizer
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(str(path.parent), gguf_file=path.name)
        except Exception as exc:  # noqa: BLE001
            log.warning("no tokenizer could be built from %s (%s): using the byte tokenizer", path.name, type(exc).__name__)
    from ..inputs.chat import ByteTokenizer
    tok = ByteTokenizer()
    if tok.vocab_size > vocab_size:
        raise SystemExit("the built-in byte tokenizer needs a vocabulary of at least 259 entries")
    return tok


def reasoning_end_tokens(tok) -> tuple[int, list[int]] | None:
    """``(closing token id, forced end sequence)`` of the tokenizer's ``</think>`` marker, or None when the marker is
    not a single token.  The forced sequence is what ends a reasoning block whose budget is used up: the marker
    framed by line breaks when that tokenizes to at most four tokens, else the marker alone."""
    try:
        ids = tok.encode("</think>", add_special_tokens=False)
    except TypeError:
        ids = tok.encode("</think>")
    if len(ids) != 1:
        return None
    end = int(ids[0])
    try:
        framed = [int(t) for t in tok.encode("\n</think>\n\n", add_special_tokens=False)]
    except TypeError:
        framed = [int(t) for t in tok.encode("\n</think>\n\n")]
    return end, (framed if end in framed and len(framed) <= 4 else [end])


def plan_kv_pages(free_bytes: int, reserve_bytes: int, cfg, tp: int, k_bits: int, v_bits: int, max_model_len: int,
                  max_running: int, layers: int | None = None, state_snapshots: int = 0) -> int:
    """Pages that fit in the remaining device memory (one page = 16 tokens of every local layer's rank-local KV
    heads; ``layers`` = decoder layers held by this pipeline stage, default all)."""
    from ..contracts.model import CacheSpec, ModelSpec, StateSpec
    n_layers = layers or cfg.num_layers
    n_gdn = sum(cfg.layer_is_gdn(i) for i in range(cfg.num_layers)) if layers is None else 0
    from ..models.config import kv_heads_of_rank
    cache = CacheSpec(n_layers - n_gdn, kv_heads_of_rank(cfg.num_kv_heads, 0, tp)[1], cfg.head_dim, k_bits, v_bits)
    # Gated DeltaNet layers keep, per request, one 128 x 128 fp32 state per value head and three conv inputs
    state = StateSpec(n_gdn, cfg.gdn_k_heads // tp, cfg.gdn_v_heads // tp) if n_gdn else None
    return ModelSpec(cfg.name, cfg.family, "", cache, state).kv_pages(free_bytes, reserve_bytes, max_model_len, max_running,
                                                                      state_snapshots)


def build_backend(args, devices: list[int], tp: int, spec, k_bits: int, v_bits: int):
    import torch

    from ..models.config import NAMED_CONFIGS
    from ..runtime.async_engine import TokenChatBackend
    from ..runtime.engine import LLMEngine
    from ..runtime.scheduler import SchedulerConfig
    if tp != 1 or args.pp_size != 1:
        from ..executor.multiproc import build_multiproc_backend
        for flag in ("startup_numerical_audit", "tune_launch_plans"):
            if getattr(args, flag, False):
                log.warning("--%s applies to single-process serving; the rank workers of this deployment start without it "
                            "(run `cubic qualify` on one GPU of the node instead)", flag.replace("_", "-"))
        return build_multiproc_backend(args, devices, tp, spec, k_bits, v_bits)
    model = args.model
    eager = args.execution_mode != "cuda" or not torch.cuda.is_available()
    gguf_weights = None
    if model.startswith("random:"):
        cfg = NAMED_CONFIGS[model.split(":", 1)[1]]()
        ck = None
        if getattr(cfg, "family", "") == "qwen4_exp":
            return _build_qwen4_exp_backend(args, cfg, None, spec)
    elif _model_type_of(model) == "qwen4_exp":
        return _build_qwen4_exp_backend(args, None, model, spec)
    elif model.endswith(".gguf") and _gguf_architecture(model) == "qwen4exp":
        return _build_qwen4_exp_backend(args, None, model, spec)
    elif model.endswith(".gguf"):
        import gguf

        from ..models.gguf import config_from_gguf
        cfg = config_from_gguf(gguf.GGUFReader(model))
        ck = None
        gguf_weights = model
    else:
        from ..models.checkpoint import admit_checkpoint
        ck = admit_checkpoint(model)
        cfg = ck.cfg
    max_len = args.max_model_len or min(cfg.max_position, 8192)
    sched = SchedulerConfig(max_running_requests=args.max_running_requests, max_batched_tokens=args.token_budget,
                            prefill_chunk_tokens=min(args.prefill_chunk_tokens, args.token_budget), max_model_len=max_len,
                            enable_prefix_cache=args.prefix_cache)
    if eager:
        from ..executor.eager_executor import EagerPagedExecutor
        from ..models.reference import dense_weights_from_checkpoint, random_dense_weights
        if gguf_weights is not None:
            raise SystemExit("eager execution mode serves checkpoint directories and random:<config> models")
        pages = 4096
        if cfg.is_moe or cfg.is_hybrid or cfg.qkv_bias:
            # the families beyond the dense full-attention decoder (experts, shared experts, Gated DeltaNet layers,
            # projection biases, any head width) run on the eager family model with per-request state
            from ..models.eager_family import EagerFamilyExecutor, family_weights_from_checkpoint, random_family_weights
            fw = family_weights_from_checkpoint(ck) if ck is not None else random_family_weights(cfg, args.seed)
            depth = getattr(spec, "num_speculative_tokens", 0) if spec is not None and getattr(spec, "method", "") == "mtp" else 0
            if depth and not cfg.mtp_layers:
                raise SystemExit("this checkpoint carries no MTP head (no mtp.* tensors)")
            executor = EagerFamilyExecutor(cfg, fw, kv_bits=(k_bits, v_bits), speculative_depth=depth)
        else:
            dense = dense_weights_from_checkpoint(ck) if ck is not None else random_dense_weights(cfg, args.seed)
            executor = EagerPagedExecutor(cfg, dense, pages, kv_bits=(k_bits, v_bits))
    else:
        from ..executor.gpu_executor import GpuExecutor
        dev = torch.device("cuda", devices[0])
        torch.cuda.set_device(dev)
        from ..models import registry as model_registry
        if getattr(args, "model_adapter", None):
            model_registry.load_adapter(args.model_adapter)          # audited, then registered (may replace a family)
        if getattr(args, "startup_numerical_audit", False):
            from ..guardrail.qualify import qualify_with_receipt
            report, reused = qualify_with_receipt(devices[0], quick=True, evidence_dir=getattr(args, "evidence_dir", None))
            if not report["ok"]:
                bad = [r["kernel"] for r in report["results"] if r["class"] == "mismatch"]
                raise SystemExit(f"start-up qualification failed on this GPU: {bad}")
            log.info("start-up qualification: %d checks passed (%s receipt)", len(report["results"]), "reused" if reused else "new")
        defn = model_registry.get(cfg.family)
        if gguf_weights is not None:
            from ..models.gguf import load_gguf_decoder_weights
            cfg, weights = load_gguf_decoder_weights(gguf_weights, dev)
        else:
            weights = defn.load_weights(ck, dev) if ck is not None else defn.random_weights(cfg, dev, args.seed)
        free, _total = torch.cuda.mem_get_info(dev)
        if args.gpu_memory_gib:
            free = min(free, int(args.gpu_memory_gib * 2 ** 30) - torch.cuda.memory_allocated(dev))
        # models with recurrent layers resume a cached prefix from a snapshot of the state taken at its last page
        # boundary: as many snapshot rows as request rows
        snapshots = args.max_running_requests if cfg.is_hybrid and args.prefix_cache else 0
        pages = plan_kv_pages(free, int(args.gpu_reserve_gib * 2 ** 30) + (2 << 30), cfg, 1, k_bits, v_bits, max_len,
                              args.max_running_requests, state_snapshots=snapshots)
        runner = defn.build_runner(cfg, weights, num_pages=pages, max_tokens=args.token_budget, k_bits=k_bits, v_bits=v_bits,
                                   max_requests=args.max_running_requests, state_checkpoints=snapshots,
                                   kv_rotation=bool(getattr(args, "enable_kv_cache_rotation", False)))
        depth = getattr(spec, "num_speculative_tokens", 0) if spec is not None else 0
        if depth and getattr(spec, "method", "mtp") == "ngram":
            # prompt-lookup drafts: no draft model; steps without a draft replay the decode graphs
            from ..executor.spec_executor import NgramSpeculativeGpuExecutor
            executor = NgramSpeculativeGpuExecutor(runner, depth, max_rows=args.max_running_requests,
                                                   max_prefill_tokens=args.token_budget, max_model_len=max_len)
            caps = executor.capture_decode_graphs()
            log.info("n-gram speculative decoding: depth %d; decode graphs %s; %d KV pages", depth, caps, pages)
        elif depth:
            # MTP speculative decoding (--speculative-config): draft head + review rounds instead of graph decode
            from ..executor.spec_executor import SpeculativeGpuExecutor
            from ..models.mtp import MtpRunner, random_mtp_weights
            if ck is not None and not cfg.mtp_layers or gguf_weights is not None:
                raise SystemExit("this checkpoint carries no MTP head (no mtp.* tensors): use "
                                 '--speculative-config \'{"method":"ngram",...}\' or a checkpoint with the head')
            if ck is not None:
                from ..models.checkpoint import load_mtp_weights
                mtp_weights = load_mtp_weights(ck, dev)
            else:
                mtp_weights = random_mtp_weights(cfg, dev, args.seed + 1)
            mtp = MtpRunner(runner, mtp_weights)
            executor = SpeculativeGpuExecutor(runner, mtp, depth, max_rows=args.max_running_requests,
                                              max_prefill_tokens=args.token_budget, max_model_len=max_len)
            log.info("MTP speculative decoding: depth %d, %s draft length; %d KV pages", depth, spec.mode, pages)
        else:
            think = reasoning_end_tokens(_tokenizer_for(model, cfg.vocab_size))
            if think is not None:
                runner.enable_reasoning_budget(*think)       # thinking-token budgets are enforced on the device
            executor = GpuExecutor(runner, max_rows=args.max_running_requests, max_prefill_tokens=args.token_budget,
                                   max_model_len=max_len)
            if getattr(args, "tune_launch_plans", False):
                # measured launch form per (projection, decode capacity); kept as start-up evidence, so measured once
                from ..contracts.implementation import identity
                from ..ops import autotune
                from .preparation import EvidenceStore, StartupPreparation, device_description
                prep = StartupPreparation(EvidenceStore(getattr(args, "evidence_dir", None)), identity(),
                                          device_description(devices[0]))
                rows = [c for c in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512) if c <= args.max_running_requests]
                n = autotune.install(autotune.prepare(cfg, rows, dev, prep))
                log.info("launch plans: %d measured entries replace the rules (%s)", n, "cached" if prep.hits else "measured now")
            caps = executor.capture_decode_graphs()
            log.info("captured decode graphs for capacities %s; %d KV pages", caps, pages)
    tok = _tokenizer_for(model, cfg.vocab_size)
    from ..models.protocol import check_executor
    log.info("executor %s: %s", type(executor).__name__, check_executor(executor))
    engine = LLMEngine(executor, num_pages=pages, scheduler_config=sched, eos_token_id=getattr(tok, "eos_token_id", None))
    if spec is not None and getattr(spec, "mode", "fixed") == "dynamic" and getattr(executor, "speculative_depth", 0):
        from .speculative import DraftPolicyConfig
        engine.enable_dynamic_draft(DraftPolicyConfig.from_dict(spec.policy) if spec.policy else None)
    processor = None
    if ck is not None and ck.vision is not None:
        processor = build_media_processor(args, ck, tok, executor, max_len)
    backend = TokenChatBackend(engine, tok, default_thinking=args.thinking, processor=processor)
    return backend, (_first_name(args.served_model_name) or cfg.name)


def _first_name(names):
    """``--served-model-name`` takes one or several names; the first is the one responses carry."""
    if not names:
        return None
    return names if isinstance(names, str) else names[0]


def _gguf_architecture(path: str) -> str | None:
    import gguf
    f = gguf.GGUFReader(str(path)).fields.get("general.architecture")
    return None if f is None else bytes(f.parts[f.data[0]]).decode()


def _model_type_of(model: str) -> str | None:
    import json
    from pathlib import Path
    p = Path(model) / "config.json"
    try:
        return json.loads(p.read_text()).get("model_type") if p.is_file() else None
    except (OSError, ValueError):
        return None


def _build_qwen4_exp_backend(args, cfg, path, spec=None):
    """The qwen4_exp family is served by its eager executor (explicit per-request state, no prefix sharing); with
    ``--speculative-config '{"method":"mtp",...}'`` and a checkpoint that carries the draft head, decode steps of greedy
    requests run as draft / review rounds."""
    from ..models.qwen4_exp import Qwen4ExpEagerExecutor, admit_qwen4_exp_checkpoint, random_qwen4_exp_weights
    from ..runtime.async_engine import TokenChatBackend
    from ..runtime.engine import LLMEngine
    from ..runtime.scheduler import SchedulerConfig
    if args.execution_mode == "cuda":
        log.warning("the qwen4_exp family runs on the eager executor; --execution-mode cuda has no native runner for it")
    store = None
    depth = getattr(spec, "num_speculative_tokens", 0) if spec is not None and getattr(spec, "method", "") == "mtp" else 0
    if spec is not None and getattr(spec, "method", "none") == "ngram":
        raise SystemExit("the qwen4_exp executor runs draft-head rounds (method mtp); n-gram drafts are not wired to it")
    if path is not None and str(path).endswith(".gguf"):
        from ..models.qwen4_exp_gguf import load_qwen4_exp_gguf
        cfg, weights = load_qwen4_exp_gguf(path)
        if depth:
            raise SystemExit("the draft head of this format lives in a file of its own, which is not read: serve without "
                             "--speculative-config")
    elif path is not None:
        cfg, weights, store = admit_qwen4_exp_checkpoint(path)
        if depth and "mtp.fc_hidden.weight" not in weights:
            raise SystemExit("this checkpoint carries no draft head (no mtp.* tensors)")
    else:
        weights = random_qwen4_exp_weights(cfg, args.seed, draft_head=depth > 0)
    max_len = args.max_model_len or min(cfg.max_position, 8192)
    sched = SchedulerConfig(max_running_requests=args.max_running_requests, max_batched_tokens=args.token_budget,
                            prefill_chunk_tokens=min(args.prefill_chunk_tokens, args.token_budget), max_model_len=max_len,
                            enable_prefix_cache=False)
    executor = Qwen4ExpEagerExecutor(cfg, weights, speculative_depth=depth)
    tok = _tokenizer_for(path or "random:qwen4-exp-tiny", cfg.vocab_size)
    engine = LLMEngine(executor, num_pages=max(4096, args.max_running_requests * (max_len // 16 + 1)), scheduler_config=sched,
                       eos_token_id=getattr(tok, "eos_token_id", None))
    processor = None
    if store is not None and cfg.vision is not None:
        import json
        from pathlib import Path
        from types import SimpleNamespace
        # the same builder as for the other multimodal checkpoints: tower, feature store, media policy
        ck = SimpleNamespace(vision=cfg.vision, vision_prefix="model.visual.", store=store, cfg=cfg,
                             raw_config=json.loads((Path(path) / "config.json").read_text()))
        processor = build_media_processor(args, ck, tok, executor, max_len)
    return (TokenChatBackend(engine, tok, default_thinking=args.thinking, processor=processor),
            (_first_name(args.served_model_name) or cfg.name))


def build_media_processor(args, ck, tok, executor, max_len: int):
    """The input processor of a multimodal checkpoint: vision tower (on the executor's device when it has one), encoded
    feature store, media policy.  Executors that take no feature rows serve such a checkpoint as text only."""
    import torch
    if ck.vision.deepstack_visual_indexes and not getattr(executor, "accepts_deepstack", False):
        log.warning("the vision tower feeds intermediate layers into the decoder (deepstack), which the decoders of this "
                    "execution mode does not consume (--execution-mode eager does): the checkpoint is served as text only")
        return None
    if not getattr(executor, "accepts_features", False):
        log.warning("the checkpoint has a vision tower, but this execution mode serves text only "
                    "(--execution-mode eager serves image and video parts)")
        return None
    from ..executor.vision import EncodedFeatureStore, VisionService
    from ..inputs.media import MediaPolicy, MediaResolver
    from ..inputs.multimodal import MultimodalChatProcessor, VisionTokens
    from ..models.checkpoint import load_vision_weights
    from ..models.vision import VisionEncoder
    device = getattr(executor, "device", "cpu")
    dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
    encoder = VisionEncoder(ck.vision, load_vision_weights(ck, device, dtype))
    service = VisionService(encoder, EncodedFeatureStore(getattr(args, "feature_store_mib", 1024) << 20),
                            memory_bytes=int(getattr(args, "encoder_memory_gib", 2.0) * 2 ** 30),
                            max_prompt_tokens=max_len - 1, identity=ck.cfg.name.encode(),
                            graph_buckets=tuple(int(c) for c in str(getattr(args, "encoder_graph_buckets", "") or "").split(",")
                                                if c.strip()))
    policy = MediaPolicy(file_roots=tuple(getattr(args, "media_file_root", ()) or ()),
                         http_hosts=tuple(getattr(args, "media_http_host", ()) or ()))
    log.info("vision tower: %d layers, %d patches per encoder call, feature store %d MiB", ck.vision.depth,
             service.plan.max_patches_per_call, getattr(args, "feature_store_mib", 1024))
    return MultimodalChatProcessor(tok, service, VisionTokens.from_hf(ck.raw_config), resolver=MediaResolver(policy),
                                   default_thinking=args.thinking, max_model_len=max_len,
                                   max_items=getattr(args, "max_media_items", 16),
                                   video_max_frames=getattr(args, "video_max_frames", 768),
                                   preprocess_workers=getattr(args, "mm_preprocess_workers", 2))


class StatusReporter(threading.Thread):
    """``[STATUS]`` line every 10 s of activity (reference: ``runtime/logging.py:316``)."""

    def __init__(self, backend, period: float = 10.0) -> None:
        super().__init__(daemon=True, name="cubic-status")
        self.backend, self.period = backend, period
        self._last_tokens = 0

    def run(self) -> None:
        while self.backend.ready:
            time.sleep(self.period)
            eng = self.backend.engine
            s = eng.stats()
            tokens = self.backend.stats["tokens"]
            rate = (tokens - self._last_tokens) / self.period
            self._last_tokens = tokens
            if s["running"] or s["waiting"] or rate:
                log.info("[STATUS] n_req=%d waiting=%d kv=%.0f%% prefix=%.0f%% decode=%.1f tok/s", s["running"],
                         s["waiting"], 100 * s["kv_used_frac"], 100 * s["prefix_hit_rate"], rate)


def run_http_server(backend, model_name: str, args) -> int:
    import uvicorn

    from ..api.server import CubicASGIApp
    from .logging import LogConfig, close_logging, serve_logging
    handles = serve_logging(LogConfig.from_file(getattr(args, "log_config", None)))
    from ..inputs.normalize import sampling_defaults_from_generation_config
    defaults = sampling_defaults_from_generation_config(Path(args.model) / "generation_config.json")
    if defaults:
        log.info("sampling defaults from generation_config.json: %s", defaults)
    app = CubicASGIApp(backend, model_name, args.served_model_name, args.api_key, sampling_defaults=defaults)
    StatusReporter(backend).start()
    config = uvicorn.Config(app, host=args.host, port=args.port, log_level="warning",
                            timeout_keep_alive=args.http_keep_alive_seconds, lifespan="on")
    try:
        uvicorn.Server(config).run()
    finally:
        close_logging(handles)
    return 0
