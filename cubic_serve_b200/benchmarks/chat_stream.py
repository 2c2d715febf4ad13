"""Public-API streaming benchmark: total output tokens/s, TTFT and per-request rate over OpenAI-compatible SSE.

What the reference's headline numbers are measured with (``tools/benchmarks/chat_stream.py`` there): C concurrent
``POST /v1/chat/completions`` streams with ``stream_options.include_usage``, a fixed number of output tokens per
request, total tokens/s over the wall time of the level, and per request ``(tokens - 1) / (last_SSE - first_SSE)``.
GPU telemetry (SM clock, power, throttle reasons) is sampled with ``nvidia-smi`` while a level runs when asked.

    python -m cubic_serve_b200.benchmarks.chat_stream --url http://127.0.0.1:8000 --model dense-8b \\
        --concurrency 1,4,16,64,256 --max-tokens 1024 --prompt-tokens 1024

Prints one JSON line per concurrency level.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import statistics
import subprocess
import time
from dataclasses import dataclass, field


@dataclass
class StreamResult:
    ok: bool
    status: int = 0
    ttft_s: float = 0.0               # request sent -> first content / reasoning delta
    first_s: float = 0.0              # absolute times of the first and last delta
    last_s: float = 0.0
    chunks: int = 0
    completion_tokens: int = 0        # from the usage frame when the server sends one, else the delta count
    error: str = ""


def synthetic_prompt(tokens: int, seed: int) -> str:
    """About ``tokens`` whitespace-separated pseudo-words, different per request (defeats prefix caching unless
    ``--shared-prefix`` asks for a common head)."""
    words, x = [], (seed * 2654435761) & 0xFFFFFFFF
    for _ in range(max(1, tokens)):
        x = (1103515245 * x + 12345) & 0x7FFFFFFF
        words.append("w%x" % (x % 65521))
    return " ".join(words)


async def one_stream(session, url: str, body: dict, headers: dict, timeout_s: float) -> StreamResult:
    import aiohttp
    t0 = time.perf_counter()
    res = StreamResult(False)
    try:
        async with session.post(url, json=body, headers=headers, timeout=aiohttp.ClientTimeout(total=timeout_s)) as resp:
            res.status = resp.status
            if resp.status != 200:
                res.error = (await resp.text())[:200]
                return res
            buf = b""
            async for chunk in resp.content.iter_any():
                buf += chunk
                while b"\n\n" in buf:
                    frame, buf = buf.split(b"\n\n", 1)
                    if not frame.startswith(b"data: "):
                        continue
                    data = frame[6:]
                    if data == b"[DONE]":
                        continue
                    obj = json.loads(data)
                    usage = obj.get("usage")
                    if usage:
                        res.completion_tokens = int(usage.get("completion_tokens", 0))
                    for ch in obj.get("choices", ()):
                        delta = ch.get("delta", {})
                        if delta.get("content") or delta.get("reasoning_content") or delta.get("tool_calls"):
                            now = time.perf_counter()
                            if not res.chunks:
                                res.ttft_s, res.first_s = now - t0, now
                            res.last_s = now
                            res.chunks += 1
            res.ok = res.chunks > 0
            if not res.completion_tokens:
                res.completion_tokens = res.chunks
    except Exception as exc:  # noqa: BLE001 - a benchmark reports failures, it does not raise them
        res.error = f"{type(exc).__name__}: {exc}"
    return res


class Telemetry:
    """``nvidia-smi`` sampler for the duration of a level (no-op when the tool is missing)."""
    QUERY = "index,clocks.sm,power.draw,clocks_event_reasons.sw_power_cap,clocks_event_reasons.hw_slowdown"

    def __init__(self, enabled: bool) -> None:
        self.proc = None
        if enabled:
            try:
                self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                              "-lms", "500"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            except OSError:
                self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            return {}
        sm, power, capped, slow = [], [], 0, 0
        for ln in out.splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 5:
                continue
            try:
                sm.append(float(f[1]))
                power.append(float(f[2]))
            except ValueError:
                continue
            capped += f[3].lower().startswith("active")
            slow += f[4].lower().startswith("active")
        if not sm:
            return {}
        return {"sm_mhz_median": statistics.median(sm), "power_w_max": max(power), "sw_power_cap_samples": capped,
                "hw_slowdown_samples": slow, "samples": len(sm)}


@dataclass
class LevelSummary:
    concurrency: int
    requests: int
    failed: int
    wall_s: float
    output_tokens: int
    total_tok_s: float
    ttft_p50_ms: float
    ttft_p99_ms: float
    rate_p50_tok_s: float            # per-request (tokens - 1) / (last - first)
    tpot_p50_ms: float
    telemetry: dict = field(default_factory=dict)
    errors: list = field(default_factory=list)


def summarize(concurrency: int, results: list[StreamResult], wall_s: float, telemetry: dict) -> LevelSummary:
    good = [r for r in results if r.ok]
    toks = sum(r.completion_tokens for r in good)
    ttft = sorted(r.ttft_s for r in good) or [0.0]
    rates = [(r.completion_tokens - 1) / (r.last_s - r.first_s) for r in good
             if r.completion_tokens > 1 and r.last_s > r.first_s] or [0.0]
    p = lambda xs, q: xs[min(len(xs) - 1, int(q * len(xs)))]       # noqa: E731
    rate50 = statistics.median(rates)
    return LevelSummary(concurrency, len(results), len(results) - len(good), round(wall_s, 4), toks,
                        round(toks / wall_s, 2) if wall_s > 0 else 0.0, round(1e3 * p(ttft, 0.5), 2),
                        round(1e3 * p(ttft, 0.99), 2), round(rate50, 2), round(1e3 / rate50, 3) if rate50 else 0.0,
                        telemetry, sorted({r.error for r in results if r.error})[:3])


async def run_level(url: str, model: str, concurrency: int, requests: int, max_tokens: int, prompt_tokens: int,
                    api_key: str | None, timeout_s: float, temperature: float, telemetry: bool,
                    shared_prefix: int = 0) -> LevelSummary:
    import aiohttp
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    endpoint = url.rstrip("/") + "/v1/chat/completions"
    sem = asyncio.Semaphore(concurrency)
    head = synthetic_prompt(shared_prefix, 0) + " " if shared_prefix else ""

    async def guarded(i: int, session):
        body = {"model": model, "stream": True, "stream_options": {"include_usage": True}, "max_tokens": max_tokens,
                "temperature": temperature, "ignore_eos": True,
                "messages": [{"role": "user", "content": head + synthetic_prompt(prompt_tokens - shared_prefix, i + 1)}]}
        async with sem:
            return await one_stream(session, endpoint, body, headers, timeout_s)

    tele = Telemetry(telemetry)
    conn = aiohttp.TCPConnector(limit=0)
    async with aiohttp.ClientSession(connector=conn) as session:
        t0 = time.perf_counter()
        results = await asyncio.gather(*(guarded(i, session) for i in range(requests)))
        wall = time.perf_counter() - t0
    return summarize(concurrency, list(results), wall, tele.stop())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", required=True)
    ap.add_argument("--concurrency", default="1,4,16,64,256", help="comma-separated levels")
    ap.add_argument("--requests-per-level", type=int, default=0, help="default: one request per concurrent stream")
    ap.add_argument("--max-tokens", type=int, default=1024)
    ap.add_argument("--prompt-tokens", type=int, default=1024)
    ap.add_argument("--shared-prefix", type=int, default=0, help="words of prompt head common to all requests")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--api-key")
    ap.add_argument("--timeout", type=float, default=3600.0)
    ap.add_argument("--telemetry", action="store_true", help="sample nvidia-smi clocks / power during each level")
    args = ap.parse_args(argv)
    for level in (int(x) for x in args.concurrency.split(",")):
        n = args.requests_per_level or level
        s = asyncio.run(run_level(args.url, args.model, level, n, args.max_tokens, args.prompt_tokens, args.api_key,
                                  args.timeout, args.temperature, args.telemetry, args.shared_prefix))
        print(json.dumps(s.__dict__), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
