import json

from cubic_serve_b200.runtime.profiling import StepProfile, nvtx_range


def test_step_profile_window_and_percentiles():
    lines = []
    p = StepProfile(window_steps=3, sink=lines.append)
    for i in range(3):
        with p.phase("schedule_cpu_ms"):
            pass
        for v in (1.0, 2.0, 10.0):
            p.record("gpu_step_ms", v + i)
        out = p.end_step()
    assert out is not None and len(lines) == 1
    s = json.loads(lines[0])["feeding_profile"]
    assert s["gpu_step_ms"]["count"] == 9 and s["gpu_step_ms"]["p50_ms"] == 3.0 and s["gpu_step_ms"]["p95_ms"] == 12.0
    assert s["schedule_cpu_ms"]["count"] == 3 and p.steps == 0 and not p.samples
    with nvtx_range("x"):
        pass
