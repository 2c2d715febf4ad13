"""The public SSE benchmark client against the real ASGI app served by uvicorn on a loopback port (CPU toy model)."""
import asyncio
import socket
import threading
import time

import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_chat_stream_benchmark_against_live_server():
    uvicorn = pytest.importorskip("uvicorn")
    pytest.importorskip("aiohttp")
    from cubic_serve_b200.api.server import CubicASGIApp
    from cubic_serve_b200.benchmarks.chat_stream import run_level, synthetic_prompt
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.models.config import ModelConfig
    from cubic_serve_b200.models.reference import random_dense_weights
    from cubic_serve_b200.runtime.async_engine import TokenChatBackend
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig

    assert synthetic_prompt(5, 1) != synthetic_prompt(5, 2) and len(synthetic_prompt(7, 3).split()) == 7
    tok = ByteTokenizer()
    cfg = ModelConfig(num_layers=1, hidden_size=64, num_q_heads=2, num_kv_heads=1, head_dim=32, intermediate_size=128,
                      vocab_size=tok.vocab_size)
    eng = LLMEngine(EagerPagedExecutor(cfg, random_dense_weights(cfg, 0), 128), 128,
                    SchedulerConfig(max_running_requests=4, max_model_len=512, max_batched_tokens=256))
    port = _free_port()
    box = {}

    def serve():
        loop = asyncio.new_event_loop()
        asyncio.set_event_loop(loop)
        backend = TokenChatBackend(eng, tok, default_max_tokens=8)
        app = CubicASGIApp(backend, "toy", api_key="k")
        server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error", lifespan="off"))
        box["server"], box["backend"] = server, backend
        loop.run_until_complete(server.serve())

    th = threading.Thread(target=serve, daemon=True)
    th.start()
    for _ in range(100):
        if box.get("server") is not None and box["server"].started:
            break
        time.sleep(0.05)
    try:
        s = asyncio.run(run_level(f"http://127.0.0.1:{port}", "toy", concurrency=3, requests=5, max_tokens=6,
                                  prompt_tokens=4, api_key="k", timeout_s=60, temperature=0.0, telemetry=False))
        assert s.failed == 0 and s.requests == 5, s.errors
        assert s.output_tokens == 5 * 6 and s.total_tok_s > 0 and s.ttft_p50_ms > 0 and s.rate_p50_tok_s > 0
        bad = asyncio.run(run_level(f"http://127.0.0.1:{port}", "toy", 1, 1, 4, 4, "wrong-key", 30, 0.0, False))
        assert bad.failed == 1
    finally:
        box["server"].should_exit = True
        th.join(timeout=10)
        box["backend"].close()
