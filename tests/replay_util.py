"""Drives bin/trace_run as a user would: steps on stdin, `done <step>` on stdout, .f32 files."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
TRACE_RUN = ROOT / "bin" / "trace_run"


class Trace:
    """One run of trace_run.  ``step`` sends a step and waits for its `done` line."""

    def __init__(self, model_dir, dtype: str, out_dir, max_tokens: int):
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.proc = subprocess.Popen(
            [sys.executable, str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype,
             "--out", str(self.out_dir), "--max-tokens", str(max_tokens)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=str(ROOT),
            env={**os.environ, "PYTHONDONTWRITEBYTECODE": "1"})
        self.n = 0
        self.vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]

    def step(self, entries, end=()) -> torch.Tensor | None:
        """entries: [(id, tokens, want)].  Returns the logits written for this step, if any."""
        rec = {"step": self.n,
               "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {self.n}":
            self.proc.kill()
            raise RuntimeError(f"trace_run answered {line!r} to step {self.n} "
                               f"(exit code {self.proc.poll()})")
        path = self.out_dir / f"{self.n}.f32"
        wanted = sum(len(w) for _, _, w in entries)
        self.n += 1
        if wanted == 0:
            assert not path.exists()
            return None
        arr = np.fromfile(path, dtype="<f4")
        assert arr.size == wanted * self.vocab, (arr.size, wanted, self.vocab)
        return torch.from_numpy(arr.reshape(wanted, self.vocab))

    def close(self) -> int:
        self.proc.stdin.close()
        code = self.proc.wait(timeout=120)
        return code

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if self.proc.poll() is None:
            try:
                code = self.close()
            except Exception:
                self.proc.kill()
                raise
            if exc[0] is None:
                assert code == 0, f"trace_run exited with {code}"
