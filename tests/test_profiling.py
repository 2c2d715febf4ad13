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


def test_serve_logging_file_rotation_and_fd_relay(tmp_path):
    import json
    import logging
    import os
    import subprocess
    import sys
    # run in a child process: the relay rewires the process's file descriptors
    cfg = tmp_path / "log.json"
    logfile = tmp_path / "logs" / "serve.log"
    cfg.write_text(json.dumps({"level": "DEBUG", "file": str(logfile), "rotate_bytes": 2000, "backups": 2, "relay_fds": True,
                               "loggers": {"cubic.noisy": "WARNING"}}))
    code = (
        "import logging, os, sys\n"
        "from cubic_serve_b200.runtime.logging import LogConfig, serve_logging, close_logging\n"
        f"h = serve_logging(LogConfig.from_file({str(cfg)!r}))\n"
        "log = logging.getLogger('cubic.test')\n"
        "for i in range(60): log.info('line %03d of the test run', i)\n"
        "logging.getLogger('cubic.noisy').info('dropped')\n"
        "os.write(1, b'written to fd 1 by native code\\n')\n"
        "os.write(2, b'written to fd 2 by a child\\n')\n"
        "close_logging(h)\n")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=60,
                         env={**os.environ, "PYTHONPATH": os.getcwd()})
    assert out.returncode == 0, out.stderr
    files = sorted(p.name for p in logfile.parent.iterdir())
    assert files[0] == "serve.log" and 2 <= len(files) <= 3            # rotated, at most two backups kept
    text = "".join(p.read_text() for p in logfile.parent.iterdir())
    assert "line 059" in text and "dropped" not in text
    assert "cubic.stdout: written to fd 1 by native code" in text and "WARNING cubic.stderr: written to fd 2" in text
    assert "written to fd 2 by a child" in out.stderr                  # the console still shows it, formatted
    import pytest
    from cubic_serve_b200.runtime.logging import LogConfig
    bad = tmp_path / "bad.json"
    bad.write_text('{"colour": true}')
    with pytest.raises(ValueError):
        LogConfig.from_file(bad)
