"""``cubic`` command line: ``serve``, ``inspect-model``, ``qualify``, ``check-install``, ``audit-checkpoint``,
``quantize``, ``trace``.

Flag surface follows the reference CLI (``cli.py:281-528`` there): Server / Model and generation / Devices and
parallelism / Memory and cache / Scheduling / Advanced groups, JSON sub-configs for speculative decoding
(``--speculative-config '{"method":"mtp","num_speculative_tokens":3,"mode":"dynamic"}'``) and structured
outputs, cache dtypes chosen independently for K and V.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from dataclasses import dataclass

KV_DTYPES = ("auto", "bfloat16", "float16", "fp8", "int8", "int6", "int4")
KV_BITS = {"auto": 8, "int8": 8, "int6": 6, "int4": 4, "fp8": 8, "bfloat16": 16, "float16": 16}


@dataclass(frozen=True)
class SpeculativeConfig:
    method: str = "none"
    num_speculative_tokens: int = 0
    mode: str = "fixed"            # fixed | dynamic
    max_tokens: int = 0
    policy: dict | None = None


def parse_speculative_config(text: str | None) -> SpeculativeConfig:
    if not text:
        return SpeculativeConfig()
    try:
        cfg = json.loads(text)
    except ValueError as exc:
        raise argparse.ArgumentTypeError(f"--speculative-config is not valid JSON: {exc}") from exc
    if not isinstance(cfg, dict) or cfg.get("method") not in ("mtp", "ngram"):
        raise argparse.ArgumentTypeError('--speculative-config needs {"method": "mtp" | "ngram", ...}')
    n = cfg.get("num_speculative_tokens")
    if not isinstance(n, int) or not 1 <= n <= 7:
        raise argparse.ArgumentTypeError("num_speculative_tokens must be an integer in [1, 7]")
    mode = cfg.get("mode", "fixed")
    if mode not in ("fixed", "dynamic"):
        raise argparse.ArgumentTypeError("mode must be fixed or dynamic")
    if cfg["method"] == "ngram" and mode != "fixed":
        raise argparse.ArgumentTypeError("n-gram drafts have no planned length: a request without a match drafts nothing")
    return SpeculativeConfig(cfg["method"], n, mode, int(cfg.get("max_tokens", n)), cfg.get("policy"))


def parse_devices(text: str | None) -> list[int]:
    if not text:
        return [0]
    out: list[int] = []
    for part in text.split(","):
        part = part.strip()
        if ".." in part or "-" in part:
            a, b = part.replace("..", "-").split("-")
            out.extend(range(int(a), int(b) + 1))
        elif part:
            out.append(int(part))
    if len(set(out)) != len(out) or not out:
        raise argparse.ArgumentTypeError("--devices must list distinct device ids")
    return out


def validate_topology(devices: list[int], tp: int, pp: int, ep: int, spec: SpeculativeConfig) -> None:
    if pp not in (1, 2):
        raise SystemExit("--pp-size must be 1 or 2")
    if tp * pp != len(devices):
        raise SystemExit(f"--tp-size x --pp-size = {tp * pp} must equal the number of devices ({len(devices)})")
    if ep < 1 or tp % ep:
        raise SystemExit("--ep-size must divide --tp-size")
    if spec.method == "mtp" and pp != 1:
        raise SystemExit("MTP speculative decoding requires --pp-size 1")
    if spec.method in ("mtp", "ngram") and tp * pp != 1:
        raise SystemExit("speculative decoding runs in the single-process executor: use one device")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="cubic", description="Blackwell-native quantized LLM serving")
    from . import __version__ as version
    ap.add_argument("--version", action="version", version=f"%(prog)s {version}")
    sub = ap.add_subparsers(dest="command", required=True)

    ins = sub.add_parser("inspect-model", help="print the architecture, quantization and tensor inventory of a checkpoint")
    ins.add_argument("model")
    ins.add_argument("--json", action="store_true")
    ins.add_argument("--tp", type=int, default=1, help="also print what each rank of this split would own")
    ins.add_argument("--pp", type=int, default=1)
    ins.add_argument("--ep", type=int, default=1)

    q = sub.add_parser("qualify", help="run the numerical witness checks of the native kernels on this GPU")
    q.add_argument("--device", type=int, default=0)
    q.add_argument("--quick", action="store_true")
    q.add_argument("--evidence-dir", help="directory of start-up receipts (default: $CUBIC_EVIDENCE_DIR or the user cache)")
    q.add_argument("--reuse", action="store_true", help="accept a passing receipt made by the same code on the same GPU model")
    q.add_argument("--save", help="write the report (verdict, error and result digest of every check) to this JSON file")
    q.add_argument("--against", help="compare with a report saved earlier: which checks kept their bits, which changed")
    q.add_argument("--operators", action="store_true",
                   help="audit the plain PyTorch operators of one decoder layer against the enclosures of their own inputs "
                        "(needs no GPU: checks that this torch build honours the arithmetic contract the kernels are held to)")

    rf = sub.add_parser("reference", help="greedy-decode a prompt of token ids with the eager fp32 reference decoder "
                                          "(the oracle the native kernels are qualified against)")
    rf.add_argument("model", help="checkpoint directory or random:<config>")
    rf.add_argument("--prompt-ids", "--input-ids", dest="prompt_ids", required=True, help="comma-separated token ids")
    rf.add_argument("--max-tokens", "--max-new-tokens", dest="max_tokens", type=int, default=16)
    rf.add_argument("--kv", default="16,16", help="simulated K,V cache bits (16 = unquantized)")
    rf.add_argument("--seed", type=int, default=0)

    ci = sub.add_parser("check-install", help="check python modules, the native library and the GPUs")
    ci.add_argument("--build", action="store_true", help="(re)build the native library first")
    ci.add_argument("--json", action="store_true")
    au = sub.add_parser("audit-checkpoint", help="inventory, shard digests, decode statistics and (with --reference) "
                                                 "quantization error of a checkpoint")
    au.add_argument("checkpoint")
    au.add_argument("--reference", help="the unquantized checkpoint this one was made from")
    au.add_argument("--no-digests", action="store_true")
    au.add_argument("--json", action="store_true")
    au.add_argument("--verbose", action="store_true")
    qz = sub.add_parser("quantize", help="quantize an unquantized checkpoint into a registered weight format "
                                         "(round to nearest; check the result with audit-checkpoint --reference)")
    qz.add_argument("source")
    qz.add_argument("destination")
    qz.add_argument("--format", default="cubic")
    qz.add_argument("--bits", type=int, default=4)
    qz.add_argument("--group-size", type=int, default=128)
    qz.add_argument("--shard-gib", type=float, default=4.0)
    tr = sub.add_parser("trace", help="record an execution trace of synthetic requests, or replay a recorded trace and "
                                      "report the first token that differs (another build, execution mode or topology)")
    tr.add_argument("action", choices=("record", "replay"))
    tr.add_argument("trace", help="trace file (JSON lines)")
    tr.add_argument("--check-lifecycle", action="store_true",
                    help="replay: also compare pages in use, prefix-cache contents and cached-prefix lengths step by step "
                         "(same scheduler flags and cache size as the recording)")
    tr.add_argument("model", help="checkpoint directory, .gguf file, or random:<named-config>")
    tr.add_argument("--requests", type=int, default=8, help="record: number of synthetic requests")
    tr.add_argument("--max-tokens", type=int, default=16)
    tr.add_argument("--serve-args", default="", help="further `cubic serve` flags for the engine, one string "
                                                     "(e.g. \"--execution-mode eager --max-running-requests 8\")")
    s = sub.add_parser("serve", help="serve a checkpoint over OpenAI / Anthropic compatible HTTP")
    s.add_argument("model", help="checkpoint directory, .gguf file, or random:<named-config>")
    g = s.add_argument_group("Server")
    g.add_argument("--served-model-name", nargs="+", metavar="NAME",
                   help="public model name(s): requests may use any of them, responses carry the first")
    g.add_argument("--host", default="127.0.0.1")
    g.add_argument("--port", type=int, default=8000)
    g.add_argument("--api-key", default=os.environ.get("CUBIC_API_KEY"))
    g.add_argument("--http-keep-alive-seconds", type=int, default=5)
    g.add_argument("--log-config")
    g = s.add_argument_group("Model and generation")
    g.add_argument("--compute-mode", choices=("wna16", "wna8"), default="wna16",
                   help="wna16: packed weights, 16-bit activations (the only mode of this build; wna8 is refused)")
    g.add_argument("--dtype", choices=("bfloat16",), default="bfloat16")
    g.add_argument("--max-model-len", type=int)
    g.add_argument("--chat-template")
    g.add_argument("--reasoning-parser", default="auto")
    g.add_argument("--tool-call-parser", default="hermes")
    g.add_argument("--thinking", action=argparse.BooleanOptionalAction, default=None)
    g.add_argument("--structured-outputs-config")
    g.add_argument("--speculative-config")
    g = s.add_argument_group("Devices and parallelism")
    g.add_argument("--devices", "--device", dest="devices")
    g.add_argument("--tp-size", type=int, default=None)
    g.add_argument("--pp-size", type=int, default=1)
    g.add_argument("--ep-size", type=int, default=1)
    g.add_argument("--tp-comm", choices=("fused", "nccl"), default="fused")
    g = s.add_argument_group("Memory and cache")
    g.add_argument("--gpu-memory-gib", type=float)
    g.add_argument("--gpu-reserve-gib", type=float, default=4.0)
    g.add_argument("--k-cache-dtype", choices=KV_DTYPES, default="auto")
    g.add_argument("--v-cache-dtype", choices=KV_DTYPES, default="auto")
    g.add_argument("--enable-kv-cache-rotation", action="store_true")
    g.add_argument("--prefix-cache", action=argparse.BooleanOptionalAction, default=True)
    g = s.add_argument_group("Scheduling")
    g.add_argument("--max-running-requests", type=int, default=256)
    g.add_argument("--token-budget", type=int, default=8192)
    g.add_argument("--cuda-graph-max-tokens", default="auto")
    g.add_argument("--prefill-chunk-tokens", type=int, default=4096)
    g = s.add_argument_group("Multimodal input")
    g.add_argument("--encoder-memory-gib", "--multimodal-memory-gib", dest="encoder_memory_gib", type=float, default=2.0,
                   help="transient memory one call of the vision tower may use; larger items are cut at frame boundaries "
                        "or refused")
    g.add_argument("--feature-store-mib", type=int, default=1024, help="host memory for encoded media, reused by content")
    g.add_argument("--mm-feature-cache-gib", type=float, default=None,
                   help="the same budget in GiB (overrides --feature-store-mib; 0 keeps nothing)")
    g.add_argument("--media-file-root", "--allowed-local-media-path", dest="media_file_root", action="append", default=[],
                   help="directory file: media may be read from")
    g.add_argument("--mm-preprocess-workers", type=int, default=2,
                   help="threads that fetch, decode and cut the media of one request into patches")
    g.add_argument("--mm-worker-layout", choices=("colocated", "separate"), default="colocated",
                   help="colocated: the vision tower shares the first GPU (the only layout of this build)")
    g.add_argument("--video-fps", type=float, default=2.0,
                   help="accepted for compatibility: clips arrive as decoded frames (no container decoding)")
    g.add_argument("--video-max-frames", type=int, default=768, help="frames a clip may carry")
    g.add_argument("--media-http-host", action="append", default=[], help="host name http(s): media may be fetched from")
    g.add_argument("--max-media-items", type=int, default=16)
    g.add_argument("--encoder-graph-buckets", default="",
                   help="comma-separated patch capacities (e.g. 1024,4096): encode calls that fit replay a CUDA graph of the "
                        "vision tower captured for the smallest bucket that holds them (off by default: eager calls)")
    g = s.add_argument_group("Advanced")
    g.add_argument("--execution-mode", choices=("cuda", "eager", "debug"), default="cuda")
    g.add_argument("--recurrent-state-dtype", "--mamba-ssm-cache-dtype", dest="recurrent_state_dtype",
                   choices=("auto", "float32", "bfloat16"), default="float32",
                   help="storage of the Gated DeltaNet state: float32 (this build keeps the recurrent matrices in fp32; "
                        "bfloat16 is refused)")
    for flag in ("--activation-dtype", "--attention-dtype", "--softmax-dtype"):
        g.add_argument(flag, choices=("auto", "fp32"), default=None,
                       help="auto: bf16 operands with fp32 accumulation and fp32 softmax (the native kernels); fp32 selects "
                            "the eager execution mode, whose arithmetic is fp32 throughout")
    g.add_argument("--startup-numerical-audit", action="store_true",
                   help="qualify the kernels against their oracles before serving (a passing receipt of the same code on "
                        "the same GPU model is reused); a failure refuses to serve")
    g.add_argument("--evidence-dir", help="directory of start-up receipts and cached plans")
    g.add_argument("--tune-launch-plans", action="store_true",
                   help="time the launch forms of every weight GEMM of the model at every decode capacity at start-up "
                        "(cached as start-up evidence) instead of using the built-in rules")
    g.add_argument("--model-adapter", help="Python file defining MODEL_DEFINITION (loaded after a source-policy audit)")
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--operator-config", help="JSON file with launch policies of the native kernels (ops/strategies.py)")
    return ap


def _kv_bits(name: str) -> int:
    bits = KV_BITS[name]
    if bits not in (8, 6, 4):
        raise SystemExit(f"KV cache dtype {name} is not available in this build (int8, int6 and int4 are)")
    return bits


def _reference(args) -> int:
    """``cubic reference``: greedy decoding of a prompt of token ids on the eager models (the reference's
    ``reference-qwen3-5`` subcommand for every family of this build: dense decoders on the reference decoder, experts /
    hybrid layers / biases / wide heads on the family model, ``qwen4_exp`` on its own)."""
    import torch

    from .models.config import NAMED_CONFIGS
    from .runtime.serving import _model_type_of
    kb, vb = (int(b) for b in args.kv.split(","))
    kv_bits = None if kb >= 16 and vb >= 16 else (kb, vb)
    ck = None
    if args.model.startswith("random:"):
        cfg = NAMED_CONFIGS[args.model.split(":", 1)[1]]()
    elif _model_type_of(args.model) == "qwen4_exp":
        cfg = None
    else:
        from .models.checkpoint import admit_checkpoint
        ck = admit_checkpoint(args.model)
        cfg = ck.cfg
    stateful = None
    if cfg is None or getattr(cfg, "family", "") == "qwen4_exp":
        from .models.qwen4_exp import Qwen4ExpModel, admit_qwen4_exp_checkpoint, random_qwen4_exp_weights
        if cfg is None:
            cfg, weights, _ = admit_qwen4_exp_checkpoint(args.model)
        else:
            weights = random_qwen4_exp_weights(cfg, args.seed)
        stateful = Qwen4ExpModel(cfg, weights)
    elif cfg.is_moe or cfg.is_hybrid or cfg.qkv_bias:
        from .models.eager_family import EagerFamilyModel, family_weights_from_checkpoint, random_family_weights
        stateful = EagerFamilyModel(cfg, family_weights_from_checkpoint(ck) if ck is not None
                                    else random_family_weights(cfg, args.seed), kv_bits)
    ids = [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    if not ids or any(t < 0 or t >= cfg.vocab_size for t in ids):
        raise SystemExit(f"prompt ids must lie in [0, {cfg.vocab_size})")
    if stateful is not None:
        logits, state = stateful.forward(ids, last_only=True)
        out = []
        for _ in range(args.max_tokens):
            out.append(int(logits[0].argmax()))
            if len(out) < args.max_tokens:
                logits, state = stateful.forward([out[-1]], state, last_only=True)
    else:
        from .models.reference import EagerDecoder, dense_weights_from_checkpoint, random_dense_weights
        weights = dense_weights_from_checkpoint(ck) if ck is not None else random_dense_weights(cfg, args.seed)
        tokens, _ = EagerDecoder(cfg, weights, kv_bits=kv_bits).generate(torch.tensor([ids]), args.max_tokens)
        out = [int(t) for t in tokens[0]]
    print(json.dumps({"model": cfg.name, "family": getattr(cfg, "family", "?"), "prompt_ids": ids, "output_ids": out}))
    return 0


def _serve(args) -> int:
    from .runtime.serving import build_backend, run_http_server
    if args.compute_mode != "wna16":
        raise SystemExit("--compute-mode wna8 (INT8 activations) is not available in this build: packed weights run "
                         "with 16-bit activations (wna16)")
    if args.recurrent_state_dtype == "bfloat16":
        raise SystemExit("--recurrent-state-dtype bfloat16 is not available: the Gated DeltaNet state is kept in float32")
    if any(getattr(args, n) == "fp32" for n in ("activation_dtype", "attention_dtype", "softmax_dtype")) \
            and args.execution_mode == "cuda":
        print("fp32 arithmetic requested: using --execution-mode eager", file=sys.stderr)
        args.execution_mode = "eager"
    if args.mm_worker_layout != "colocated":
        raise SystemExit("--mm-worker-layout separate is not available: the vision tower runs on the first GPU")
    if args.mm_feature_cache_gib is not None:
        args.feature_store_mib = int(args.mm_feature_cache_gib * 1024)
    if args.video_max_frames < 4:
        raise SystemExit("--video-max-frames must be at least 4")
    spec = parse_speculative_config(args.speculative_config)
    devices = parse_devices(args.devices)
    tp = args.tp_size or max(1, len(devices) // args.pp_size)
    validate_topology(devices, tp, args.pp_size, args.ep_size, spec)
    if args.operator_config:
        # through the environment as well, so that spawned rank workers install the same policies
        from .ops import strategies
        ctx = strategies.launch_context(args.model, tp, devices[0])
        strategies.install(strategies.load_operator_config(args.operator_config, ctx))
        os.environ["CUBIC_OPERATOR_CONFIG"] = os.path.abspath(args.operator_config)
        os.environ["CUBIC_OPERATOR_CONTEXT"] = json.dumps(ctx)
    os.environ.setdefault("OMP_NUM_THREADS", "4")
    os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
    sys.setswitchinterval(0.001)
    backend, model_name = build_backend(args, devices, tp, spec, _kv_bits(args.k_cache_dtype), _kv_bits(args.v_cache_dtype))
    return run_http_server(backend, model_name, args)


def _trace(args) -> int:
    """``cubic trace record|replay``: the engine is built exactly as ``cubic serve`` builds it (same flags)."""
    import shlex

    import numpy as np

    from .guardrail.replay import TraceRecorder, replay_trace
    from .runtime.scheduler import SamplingParams
    from .runtime.serving import build_backend
    sargs = build_parser().parse_args(["serve", args.model, *shlex.split(args.serve_args)])
    spec = parse_speculative_config(sargs.speculative_config)
    devices = parse_devices(sargs.devices)
    tp = sargs.tp_size or max(1, len(devices) // sargs.pp_size)
    validate_topology(devices, tp, sargs.pp_size, sargs.ep_size, spec)
    backend, _name = build_backend(sargs, devices, tp, spec, _kv_bits(sargs.k_cache_dtype), _kv_bits(sargs.v_cache_dtype))
    engine = backend.engine
    backend.close()                                 # stop the serving thread: this command steps the engine itself
    try:
        if args.action == "record":
            rec = TraceRecorder(engine)
            rng = np.random.default_rng(sargs.seed)
            vocab = min(engine.executor.cfg.vocab_size if hasattr(engine.executor, "cfg") else 256, 50000)
            for i in range(args.requests):
                prompt = rng.integers(1, vocab, int(rng.integers(4, 48))).tolist()
                rec.add_request(prompt, SamplingParams(max_tokens=args.max_tokens, ignore_eos=True), f"trace-{i}")
                if i % 3 == 2:
                    rec.step()                      # arrivals spread over steps: prefill and decode rows mix
            rec.run()
            rec.save(args.trace)
            tokens = sum(len(t) for r in rec.records if r["kind"] == "step" for t in r["emitted"].values())
            print(json.dumps({"recorded": args.trace, "requests": args.requests, "tokens": tokens}))
            return 0
        report = replay_trace(args.trace, engine, check_lifecycle=getattr(args, "check_lifecycle", False))
        print(report.to_json())
        return 0 if report.ok else 1
    finally:
        stop = getattr(engine.executor, "close", None)      # multi-process executors own worker processes
        if stop:
            stop()


def _inspect(args) -> int:
    from .models.checkpoint import inspect_checkpoint
    if args.model.startswith("random:"):
        from .models.config import NAMED_CONFIGS
        cfg = NAMED_CONFIGS[args.model.split(":", 1)[1]]()
        info = {"model": cfg.name, "family": cfg.family, "layers": cfg.num_layers, "hidden": cfg.hidden_size,
                "quantization": f"{cfg.quant.method} {cfg.quant.bits}-bit group {cfg.quant.group_size}"}
    else:
        info = inspect_checkpoint(args.model)
        cfg = None
    if args.tp * args.pp * args.ep > 1:
        from pathlib import Path

        from .models.config import ModelConfig
        from .models.parallel_weights import PartitionError, plan_partition
        if cfg is None and (Path(args.model) / "config.json").exists():
            cfg = ModelConfig.from_hf_config(Path(args.model) / "config.json")
        if cfg is not None:
            try:
                info["partition"] = plan_partition(cfg, args.tp, args.pp, args.ep).summary()
            except PartitionError as exc:
                info["partition_error"] = str(exc)
            else:
                # the communication calls every rank issues per step, and the proof that they cannot block each other
                from .contracts.execution import ParallelTopology
                from .guardrail.collective_schedule import check_schedules, decoder_step_schedule
                topo = ParallelTopology.single_node(range(args.tp * args.pp), tp=args.tp, pp=args.pp, ep=args.ep)
                sch = {r: decoder_step_schedule(cfg, topo, r, rows=1) for r in range(topo.world_size)}
                problems = check_schedules(topo, sch)
                info["collectives_per_step"] = {f"rank {r}": len(s) for r, s in sch.items()}
                info["collective_schedule"] = "every group agrees, transfers match, the step runs to its end" \
                    if not problems else problems
    if args.json:
        print(json.dumps(info, indent=1, default=str))
    else:
        for k, v in info.items():
            print(f"{k}: {v}")
    return 0


def _qualify(args) -> int:
    if args.operators:
        from .guardrail.enclosure import audit_layer_operators
        rows = [{"operator": n, "ok": r.ok, "outside": r.outside, "of": r.total, "worst_excess_ulps": r.worst_excess_ulps}
                for seed in range(2 if args.quick else 8) for n, r in audit_layer_operators(seed=seed)]
        ok = all(r["ok"] for r in rows)
        print(json.dumps({"ok": ok, "checks": len(rows), "failed": [r for r in rows if not r["ok"]]}, indent=1))
        return 0 if ok else 1
    from .guardrail.qualify import qualify_with_receipt
    report, reused = qualify_with_receipt(args.device, quick=args.quick, evidence_dir=args.evidence_dir, force=not args.reuse)
    report = dict(report, receipt="reused" if reused else "new")
    if args.save:
        from pathlib import Path
        Path(args.save).write_text(json.dumps(report, indent=1))
    if args.against:
        from pathlib import Path

        from .guardrail.qualify import compare_reports
        diff = compare_reports(json.loads(Path(args.against).read_text()), report)
        print(json.dumps(diff, indent=1))
        return 0 if diff["ok"] else 1
    print(json.dumps(report, indent=1))
    return 0 if report["ok"] else 1


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "serve":
        return _serve(args)
    if args.command == "inspect-model":
        return _inspect(args)
    if args.command == "qualify":
        return _qualify(args)
    if args.command == "quantize":
        from .utils.quantize_checkpoint import quantize_checkpoint
        print(json.dumps(quantize_checkpoint(args.source, args.destination, args.format, args.bits, args.group_size,
                                             int(args.shard_gib * 2 ** 30))))
        return 0
    if args.command == "trace":
        return _trace(args)
    if args.command == "audit-checkpoint":
        from .utils.audit_checkpoint import audit_checkpoint, format_report as format_audit
        report = audit_checkpoint(args.checkpoint, args.reference, digests=not args.no_digests)
        print(json.dumps(report, indent=1) if args.json else format_audit(report, args.verbose))
        return 0 if report["ok"] else 1
    if args.command == "reference":
        return _reference(args)
    if args.command == "check-install":
        from .utils.check_install import format_report, run_checks
        report = run_checks(build=args.build)
        print(json.dumps(report, indent=1) if args.json else format_report(report))
        return 0 if report["ok"] else 1
    return 2


if __name__ == "__main__":
    raise SystemExit(main())
