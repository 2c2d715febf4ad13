"""Serving log set-up: one format for console and file, size-based rotation, and a relay that brings what native code
and child processes write to the process's stdout / stderr file descriptors into the same log.

``--log-config`` takes a JSON file: ``{"level": "INFO", "file": "/var/log/cubic/serve.log", "rotate_bytes":
50000000, "backups": 5, "relay_fds": true, "loggers": {"cubic.scheduler": "DEBUG"}}``; every key is optional.

Reference counterpart: ``runtime/logging.py:80`` (``serve_logging``: loguru sink with rotation, fd-level stdout /
stderr relay) -- done here with the standard library.
"""
from __future__ import annotations

import json
import logging
import logging.handlers
import os
import threading
from dataclasses import dataclass, field
from pathlib import Path

FORMAT = "%(asctime)s %(levelname)s %(name)s: %(message)s"


@dataclass(frozen=True)
class LogConfig:
    level: str = "INFO"
    file: str | None = None
    rotate_bytes: int = 50_000_000
    backups: int = 5
    relay_fds: bool = False
    loggers: dict = field(default_factory=dict)

    @staticmethod
    def from_file(path: str | Path | None) -> "LogConfig":
        if not path:
            return LogConfig()
        raw = json.loads(Path(path).read_text())
        unknown = set(raw) - set(LogConfig.__dataclass_fields__)
        if unknown:
            raise ValueError(f"unknown log configuration keys: {sorted(unknown)}")
        return LogConfig(**raw)


class FdRelay(threading.Thread):
    """Redirects a file descriptor (1 or 2) into a pipe and logs every line read from it.  The original descriptor is
    kept for the console handler, so console output still appears once, formatted."""

    def __init__(self, fd: int, logger: logging.Logger, level: int) -> None:
        super().__init__(daemon=True, name=f"cubic-fd{fd}-relay")
        self.fd, self.logger, self.level = fd, logger, level
        self.saved = os.dup(fd)
        self._r, w = os.pipe()
        os.dup2(w, fd)
        os.close(w)

    def run(self) -> None:
        with os.fdopen(self._r, "r", errors="replace") as pipe:
            for line in pipe:
                line = line.rstrip()
                if line:
                    self.logger.log(self.level, line)

    def restore(self) -> None:
        os.dup2(self.saved, self.fd)          # closes the pipe's write end: the reader sees EOF and ends


def serve_logging(cfg: LogConfig | None = None) -> list:
    """Install the handlers; returns the objects to ``close_logging`` at shutdown."""
    cfg = cfg or LogConfig()
    root = logging.getLogger()
    root.setLevel(getattr(logging, cfg.level.upper()))
    for h in list(root.handlers):
        root.removeHandler(h)
    fmt = logging.Formatter(FORMAT)
    opened: list = []
    relays: list[FdRelay] = []
    console_stream = None
    if cfg.relay_fds:
        relays = [FdRelay(1, logging.getLogger("cubic.stdout"), logging.INFO),
                  FdRelay(2, logging.getLogger("cubic.stderr"), logging.WARNING)]
        console_stream = os.fdopen(os.dup(relays[1].saved), "w", buffering=1)     # the real stderr
        opened.append(console_stream)
    console = logging.StreamHandler(console_stream)
    console.setFormatter(fmt)
    root.addHandler(console)
    opened.append(console)
    if cfg.file:
        Path(cfg.file).parent.mkdir(parents=True, exist_ok=True)
        fh = logging.handlers.RotatingFileHandler(cfg.file, maxBytes=cfg.rotate_bytes, backupCount=cfg.backups)
        fh.setFormatter(fmt)
        root.addHandler(fh)
        opened.append(fh)
    for name, level in cfg.loggers.items():
        logging.getLogger(name).setLevel(getattr(logging, str(level).upper()))
    for r in relays:
        r.start()
    return opened + relays


def close_logging(handles: list) -> None:
    """Undo ``serve_logging``: the relays first (descriptor restored, reader drained), then handlers, then streams."""
    root = logging.getLogger()
    relays = [h for h in handles if isinstance(h, FdRelay)]
    for r in relays:
        r.restore()
    for r in relays:
        r.join(timeout=5)
    for h in handles:
        if isinstance(h, logging.Handler):
            root.removeHandler(h)
            h.close()
    for h in handles:
        if not isinstance(h, (FdRelay, logging.Handler)):
            try:
                h.close()
            except OSError:
                pass
    for r in relays:
        try:
            os.close(r.saved)
        except OSError:
            pass
