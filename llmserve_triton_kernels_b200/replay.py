"""Trace replay: feeds given token ids through a model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
    bin/trace_run --random PRESET [--seed S] ...        (random weights of a named configuration, no folder)

It samples nothing and has no forward pass, cache or loader of its own: it drives the same
model, step function, cache manager and kernels that generation uses.  Steps are read from
standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch.  For a step in which something is wanted the logits at
the wanted places, in the order of the entries and of ``want``, are written to
``<out>/<step>.f32`` as little-endian float32 ``[wanted, vocab]``.  Requests named in ``end``
give their pages back after the step.  After every step a line ``done <step>`` is printed and
flushed.  The cache pool holds ``--max-tokens`` tokens (rounded up to whole pages), so pages
are used again as requests end.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids step by step and write logits")
    ap.add_argument("--model", help="folder with config.json and model.safetensors")
    ap.add_argument("--random", metavar="PRESET", help="instead of --model: random weights of a named configuration (config/presets.py)")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights (with --random)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens that live requests hold at any time")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per page of the cache")
    ap.add_argument("--max-requests", type=int, default=16, help="most requests alive at a time")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if (args.model is None) == (args.random is None):
        ap.error("give a model folder with --model, or a configuration's name with --random")
    return args


def main(argv=None) -> int:
    args = parse_args(argv)
    from . import models as _models  # noqa: F401
    from . import ops
    from .cache import CacheManager
    from .engine.batch import StepEntry
    from .engine.step import StepFunction
    from .config.presets import PRESETS
    from .config.registry import architecture_of
    from .models.load import load_model, random_model, resolve_dtype

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    device = torch.device(args.device)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    dtype = resolve_dtype(args.dtype)
    if args.random is not None:
        if args.random not in PRESETS:
            raise SystemExit(f"trace_run: no configuration named {args.random!r}; known: {sorted(PRESETS)}")
        cfg_dict = PRESETS[args.random]
        model = random_model(architecture_of(cfg_dict).config_class.from_dict(cfg_dict), args.seed, dtype, device)
    else:
        model, _ = load_model(args.model, dtype, device)
    num_pages = max(1, -(-args.max_tokens // args.page_size))
    cache = CacheManager(
        model.cache_specs(), model.plan.schedule, page_size=args.page_size, num_pages=num_pages,
        max_requests=args.max_requests, dtype=dtype, device=device,
    )
    step_function = StepFunction(model, cache)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [
            StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
            for e in record.get("entries", [])
        ]
        if entries:
            logits = step_function(entries)
            if logits.shape[0]:
                host = logits.to("cpu", torch.float32).contiguous().numpy()
                host.astype("<f4", copy=False).tofile(out_dir / f"{step}.f32")
            elif device.type == "cuda":
                torch.cuda.synchronize(device)
            ops.check_device_errors()  # the host has just waited for the device: a kernel whose wait gave up has said so
        for req in record.get("end", []):
            if cache.has_request(req):
                cache.free_request(req)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
