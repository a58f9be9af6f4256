"""Builds replay traces in the four ways of cutting the work, drives ``bin/trace_run`` with them
and gathers the logits it writes by (request, position)."""

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


def round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class Trace:
    """Steps of a trace plus, for every wanted row, which (request, position) it is."""

    def __init__(self, keep=None):
        """``keep``: of the places that "all" names, only those whose absolute position it accepts are wanted (large
        vocabularies: a row of logits is half a megabyte)."""
        self.keep = keep
        self.steps: list[dict] = []
        self.rows: dict[int, list[tuple[str, int]]] = {}
        self._fed: dict[str, int] = {}
        self.peak_tokens = 0
        self._live: dict[str, int] = {}

    def add_step(self, entries: list[tuple[str, list[int], str | list[int]]], end: list[str] = ()):
        """``entries``: (request, its next tokens, "all" | "last" | "none" | explicit places)."""
        step = len(self.steps)
        rec_entries, rows = [], []
        for req, tokens, want in entries:
            start = self._fed.get(req, 0)
            if want == "all":
                want = [i for i in range(len(tokens)) if self.keep is None or self.keep(start + i)]
            elif want == "last":
                want = [len(tokens) - 1]
            elif want == "none":
                want = []
            rec_entries.append({"id": req, "tokens": list(tokens), "want": list(want)})
            rows += [(req, start + w) for w in want]
            self._fed[req] = start + len(tokens)
            self._live[req] = self._fed[req]
        self.peak_tokens = max(self.peak_tokens, sum(round_up(n, 64) for n in self._live.values()))
        for req in end:
            self._live.pop(req, None)
            self._fed.pop(req, None)
        self.steps.append({"step": step, "entries": rec_entries, "end": list(end)})
        if rows:
            self.rows[step] = rows

    def extend(self, other: "Trace") -> None:
        """Append another trace's steps (its requests must have ended or differ in name)."""
        base = len(self.steps)
        for s in other.steps:
            self.steps.append({**s, "step": base + s["step"]})
        for k, v in other.rows.items():
            self.rows[base + k] = v
        self.peak_tokens = max(self.peak_tokens, other.peak_tokens)


def whole(name: str, tokens: list[int], keep=None) -> Trace:
    t = Trace(keep)
    t.add_step([(name, tokens, "all")], end=[name])
    return t


def decode_tail(name: str, tokens: list[int], tail: int = 32, keep=None) -> Trace:
    """Most of it in one step, the last ``tail`` tokens one by one."""
    t = Trace(keep)
    head = max(1, len(tokens) - tail)
    t.add_step([(name, tokens[:head], "all")])
    for i in range(head, len(tokens)):
        t.add_step([(name, [tokens[i]], "all")], end=[name] if i == len(tokens) - 1 else [])
    if head == len(tokens):
        t.steps[-1]["end"] = [name]
    return t


def portions(name: str, tokens: list[int], sizes=(7, 2, 16, 3, 5, 2, 1, 9), keep=None) -> Trace:
    """Portions of changing size, down to two tokens (and one)."""
    t = Trace(keep)
    i, k = 0, 0
    while i < len(tokens):
        n = min(sizes[k % len(sizes)], len(tokens) - i)
        i += n
        t.add_step([(name, tokens[i - n : i], "all")], end=[name] if i == len(tokens) else [])
        k += 1
    return t


def mixed(requests: dict[str, list[int]], prefill: dict[str, int], chunk: int = 16, live: int = 4, stagger: int = 2, keep=None) -> Trace:
    """Up to ``live`` requests at a time: each is first fed ``prefill[name]`` tokens in portions
    of at most ``chunk`` and then its remaining tokens one by one, beside the others; a request
    starts ``stagger`` steps after the one before it, or when a place becomes free."""
    t = Trace(keep)
    waiting = list(requests)
    active: dict[str, int] = {}
    steps_since_start = stagger
    while waiting or active:
        if waiting and len(active) < live and steps_since_start >= stagger:
            active[waiting.pop(0)] = 0
            steps_since_start = 0
        entries, end = [], []
        for name, fed in list(active.items()):
            tokens = requests[name]
            n = min(chunk, prefill[name] - fed) if fed < prefill[name] else 1
            n = min(n, len(tokens) - fed)
            entries.append((name, tokens[fed : fed + n], "all"))
            active[name] = fed + n
            if active[name] == len(tokens):
                end.append(name)
                del active[name]
        t.add_step(entries, end=end)
        steps_since_start += 1
    return t


def run_trace(model_dir, dtype: str, trace: Trace, out_dir, max_tokens: int | None = None, page_size: int | None = None,
              env: dict | None = None, timeout: float = 900.0) -> dict[tuple[str, int], np.ndarray]:
    """Run ``bin/trace_run`` over the trace, step by step (the next step is sent only after
    ``done <step>``), and return the logits row of every wanted (request, position)."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cmd = [sys.executable, str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
           "--max-tokens", str(max_tokens if max_tokens is not None else trace.peak_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                            env={**os.environ, **(env or {})})
    try:
        for s in trace.steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            if line != f"done {s['step']}":
                proc.stdin.close()
                err = proc.stderr.read()
                raise AssertionError(f"trace_run answered {line!r} to step {s['step']}\n{err[-4000:]}")
        proc.stdin.close()
        code = proc.wait(timeout=timeout)
        assert code == 0, f"trace_run exited with {code}\n{proc.stderr.read()[-4000:]}"
    finally:
        if proc.poll() is None:
            proc.kill()
    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    vocab = cfg["vocab_size"]
    got: dict[tuple[str, int], np.ndarray] = {}
    for s in trace.steps:
        rows = trace.rows.get(s["step"])
        f = out_dir / f"{s['step']}.f32"
        if not rows:
            assert not f.exists(), f"step {s['step']} wanted nothing but wrote {f.name}"
            continue
        data = np.fromfile(f, dtype="<f4").reshape(len(rows), vocab)
        for key, row in zip(rows, data):
            assert key not in got, f"{key} was asked for twice"
            got[key] = row
    return got


def compare(got: dict, expected: dict[str, torch.Tensor], atol_of) -> None:
    """Every wanted row against the plain implementation's; on failure, name the first wrong
    (request, position) so that what is special about its place can be asked."""
    worst = (0.0, None)
    for (req, pos), row in sorted(got.items()):
        ref = expected[req][pos].numpy()
        diff = float(np.abs(row - ref).max())
        tol = atol_of(ref)
        assert np.isfinite(row).all(), f"non-finite logits at request {req!r} position {pos}"
        assert diff <= tol, f"first wrong row: request {req!r} position {pos}: max |diff| {diff:.3e} > {tol:.3e}"
        if diff / tol > worst[0]:
            worst = (diff / tol, (req, pos, diff))
    return worst


def run_trace_inprocess(model_dir, dtype: str, trace: Trace, out_dir, device: str = "cpu", max_tokens=None, page_size=None):
    """The same through ``replay.main`` in this process (used with the plain operations patched in)."""
    import io

    from llmserve_triton_kernels_b200 import replay

    out_dir = Path(out_dir)
    argv = ["--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir), "--device", device,
            "--max-tokens", str(max_tokens if max_tokens is not None else trace.peak_tokens)]
    if page_size is not None:
        argv += ["--page-size", str(page_size)]
    stdin, stdout = sys.stdin, sys.stdout
    sys.stdin, sys.stdout = io.StringIO("".join(json.dumps(s) + "\n" for s in trace.steps)), io.StringIO()
    try:
        assert replay.main(argv) == 0
        said = sys.stdout.getvalue().split("\n")
    finally:
        sys.stdin, sys.stdout = stdin, stdout
    assert [l for l in said if l] == [f"done {s['step']}" for s in trace.steps]
    vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    got = {}
    for s in trace.steps:
        rows = trace.rows.get(s["step"])
        if rows:
            data = np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(len(rows), vocab)
            got.update(dict(zip(rows, data)))
    return got
