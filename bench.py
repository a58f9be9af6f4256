"""Measures decode and prefill throughput of the engine on one B200 and prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The model has the layer sizes of TinyLlama 1.1B (22 layers, hidden 2048, 32 heads, 4 key/value
heads, head size 64, feed-forward 5632, vocabulary 32000) with random weights N(0, 0.02) and
seeded random token ids.  A "step" is one decode step of a batch of 8 requests whose prompts of
512 tokens were prefilled before the clock starts.  ``value`` is decoded tokens a second over
exactly K steps, timed on the device with CUDA events; ``e2e`` is the same through the Python
entry point ``LLM.generate`` (host token ids in, host token ids out, every step's descriptor
copied from pinned memory and its tokens read back).  ``prefill`` is one prompt of 2,048
tokens; ``roofline`` relates the bytes a decode step has to read (every weight once, and the
cache of the live requests) to its time; ``points`` holds decode at batch 1 and 64.
Peaks come from MEASURED_PEAKS.json beside this file when present, else from an earlier
measurement on the same pool (and the line says which).

``python bench.py --sweep [--steps K]`` prints no JSON line but two tables: decode steps over batch sizes and
context lengths, and prefills over prompt lengths, timed the same way.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
MODEL = "tinyllama-1.1b"
PROMPT_LEN, NEW_TOKENS, PREFILL_TOKENS = 512, 256, 2048


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            d = json.loads(path.read_text())
            flat = {}

            def walk(x):
                if isinstance(x, dict):
                    for k, v in x.items():
                        if isinstance(v, (int, float)) and k in FALLBACK_PEAKS:
                            flat[k] = float(v)
                        else:
                            walk(v)

            walk(d)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return {**FALLBACK_PEAKS, **flat}, "measured"
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.proc = None
        self.lines: list[tuple[float, str]] = []
        self.window = [0.0, float("inf")]  # only samples taken while the timed region ran are counted

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def begin(self):
        self.window[0] = time.time()

    def end(self):
        self.window[1] = time.time()

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for stamp, line in self.lines:
            if not self.window[0] <= stamp <= self.window[1] + 0.02:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> int:
    """The unmodified reference from ``baseline/_ref`` through its own public API."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "llmserve").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref (pip install --no-index --target baseline/_ref failed or was not run)"}))
        return 0
    sys.path.insert(0, str(ref))
    try:
        import torch
        from llmserve.config import ModelConfig
        from llmserve.datatypes import SamplingParams as RefParams
        from llmserve.kvcache.paged import PagedKVCache
        from llmserve.scheduler.engine import ContinuousBatchingEngine
        from llmserve.weights import random_model as ref_random_model
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"the reference does not import here: {type(e).__name__}: {e}"[:300]}))
        return 0
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device"}))
        return 0
    batch, steps, warmup = 8, args.steps, args.warmup
    cfg = ModelConfig()  # the reference's defaults are TinyLlama 1.1B's sizes
    model = ref_random_model(cfg, seed=0, device="cuda", dtype=torch.bfloat16, std=0.02)
    total_new = warmup + steps + 1
    cache = PagedKVCache(cfg, num_blocks=batch * (-(-(PROMPT_LEN + total_new) // 16) + 1) + 8, block_size=16, device="cuda", dtype=torch.bfloat16)
    engine = ContinuousBatchingEngine(model, cache, max_batch_size=batch, max_prefill_tokens=batch * PROMPT_LEN)
    g = torch.Generator().manual_seed(1)
    for _ in range(batch):
        engine.add_request(torch.randint(0, cfg.vocab_size, (PROMPT_LEN,), generator=g).tolist(), RefParams(max_new_tokens=total_new))
    engine.step()  # prefill of all eight, first token
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    with ClockSampler() as clocks:
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()  # one decode pass; ends in a host read of the tokens
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    value = batch * steps / dt
    print(json.dumps({
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "clocks": clocks.summary(),
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": batch * 8},
        "config": {"model": "TinyLlama-1.1B sizes, random weights", "global_batch": batch, "seq_len": 2048, "prompt_len": PROMPT_LEN,
                   "parallelism": "single GPU", "api": "ContinuousBatchingEngine.step", "timing": "wall clock around K engine steps"},
    }))
    return 0


def model_numbers(cfg) -> dict:
    h, L, H, KV, D = cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    I, V = cfg.intermediate_size, cfg.vocab_size
    layer_params = h * (H + 2 * KV) * D + H * D * h + 3 * h * I
    return {"layer_params": layer_params, "head_params": V * h, "kv_bytes_per_token": 2 * L * KV * D * 2, "L": L, "H": H, "D": D}


def prefill_flops(cfg, tokens: int) -> float:
    m = model_numbers(cfg)
    gemm = 2.0 * tokens * m["layer_params"] * m["L"] + 2.0 * m["head_params"]
    attention = m["L"] * 4.0 * m["H"] * m["D"] * tokens * (tokens + 1) / 2.0
    return gemm + attention


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (recorded in config)")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64 and the end-to-end run")
    ap.add_argument("--sweep", action="store_true",
                    help="instead of the one line: a table of decode steps over batch sizes and context lengths and of prefills over prompt lengths")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)

    import torch

    from llmserve_triton_kernels_b200 import LLM, SamplingParams, ops
    from llmserve_triton_kernels_b200.config.presets import PRESETS
    from llmserve_triton_kernels_b200.engine.batch import StepEntry

    peaks, peaks_from = load_peaks()
    cfg_dict = dict(PRESETS[MODEL])
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    device = "cuda:0"
    steps, warmup = args.steps, args.warmup
    total_new = warmup + steps + 1
    if PROMPT_LEN + total_new > cfg_dict["max_position_embeddings"]:
        print(f"bench.py: {PROMPT_LEN} prompt tokens + {total_new} new tokens exceed the context of {cfg_dict['max_position_embeddings']}")
        return 2
    page_size = 16

    def tokens_for(batch: int, length: int, seed: int):
        g = torch.Generator().manual_seed(seed)
        return [torch.randint(0, cfg_dict["vocab_size"], (length,), generator=g).tolist() for _ in range(batch)]

    llm = LLM(cfg_dict, dtype="bfloat16", device=device, seed=0, block_size=page_size,
              num_blocks=64 * (-(-((1536 if args.sweep else PROMPT_LEN) + max(NEW_TOKENS, total_new) + 64) // page_size)) + 256, max_batch_size=64,
              max_num_batched_tokens=8192)
    cfg = llm.config
    numbers = model_numbers(cfg)
    weight_bytes = llm.model.weight_bytes()
    flush = torch.empty(256 * 2**20, dtype=torch.uint8, device=device)  # larger than the 126 MB L2

    def decode_run(batch: int, k: int, w: int, prompt_len: int = PROMPT_LEN) -> dict:
        """Prefill ``batch`` prompts (untimed), then w warm-up and k timed decode steps through the
        step function and the device sampler; the next token never leaves the device between steps
        except for the read that the engine itself does."""
        llm.cache.reset()
        step, sampler = llm.step_function, llm.sampler
        names = [f"b{i}" for i in range(batch)]
        prompts = tokens_for(batch, prompt_len, seed=1)
        greedy = [SamplingParams()] * batch
        per_step = max(1, 4096 // prompt_len)  # prefill eight prompts of 512 tokens at a time
        for i in range(0, batch, per_step):
            step([StepEntry(n, p, []) for n, p in zip(names[i : i + per_step], prompts[i : i + per_step])])
        tokens = [p[-1] for p in prompts]
        launches0 = ops.launch_count()

        # As the scheduler does it: a step's chosen tokens stay on the device and feed the next step, which is launched
        # before the host reads them (through pinned memory, one step late); every token reaches the host in the loop.
        ahead = None  # (tokens on the device, the same in pinned host memory, event after the kernel that wrote both)

        def one_step():
            nonlocal tokens, ahead
            if ahead is None:
                logits = step([StepEntry(n, [t], [0]) for n, t in zip(names, tokens)])
            else:
                logits = step.decode_ahead(names, ahead[0])
            host = torch.empty((batch,), dtype=torch.int32, pin_memory=True)
            chosen = sampler.on_device(logits, greedy, [0] * batch, [0] * batch, host_out=host)
            copied = torch.cuda.Event()
            copied.record()
            if ahead is not None:
                ahead[2].synchronize()
                tokens = ahead[1].tolist()
            ahead = (chosen, host, copied)

        gc.collect()  # the prefill left garbage behind; a full collection (tens of ms) must not fall into the timed steps
        for _ in range(w):
            one_step()
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler() as clocks:
            time.sleep(0.3)  # nvidia-smi is up and sampling before the timed region starts
            flush.fill_(1)
            torch.cuda.synchronize()
            clocks.begin()
            start.record()
            for _ in range(k):
                one_step()
            ahead[2].synchronize()  # the last step's tokens reach the host inside the timed region too
            tokens = ahead[1].tolist()
            end.record()
            torch.cuda.synchronize()
            clocks.end()
        ms = start.elapsed_time(end)
        context = prompt_len + w + (k + 1) / 2.0  # mean number of cached tokens a timed step reads per request
        bytes_per_step = weight_bytes + batch * context * numbers["kv_bytes_per_token"]
        out = {
            "tokens_per_s": batch * k / (ms / 1e3), "ms_per_step": ms / k, "bytes_per_step": bytes_per_step,
            "gbs": bytes_per_step / (ms / k / 1e3) / 1e9, "launches": ops.launch_count() - launches0,
            "clocks": clocks.summary(), "h2d": step.h2d_bytes, "d2h": sampler.d2h_bytes,
        }
        for n in names:
            llm.cache.free_request(n)
        return out

    def prefill_run(n_tokens: int = PREFILL_TOKENS) -> dict:
        llm.cache.reset()
        prompt = tokens_for(1, n_tokens, seed=2)[0]
        times = []
        for i in range(3 + 3):
            flush.fill_(1)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            logits = llm.step_function([StepEntry("p", prompt, [n_tokens - 1])])
            ops.argmax(logits)
            end.record()
            torch.cuda.synchronize()
            llm.cache.free_request("p")
            if i >= 3:
                times.append(start.elapsed_time(end))
        ms = statistics.median(times)
        flops = prefill_flops(cfg, n_tokens)
        return {"value": n_tokens / (ms / 1e3), "tokens": n_tokens, "ms": ms,
                "frac": flops / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), "tflops": flops / (ms / 1e3) / 1e12}

    def e2e_run(batch: int) -> dict:
        """Through ``LLM.generate``: host token ids in, host token ids out."""
        llm.cache.reset()
        prompts = tokens_for(batch, PROMPT_LEN, seed=3)
        llm.generate(prompts[:2], SamplingParams(max_new_tokens=4))  # warm-up of the whole path
        torch.cuda.synchronize()
        outs = llm.generate(prompts, SamplingParams(max_new_tokens=NEW_TOKENS))
        first = max(o.ttft_s for o in outs)
        last = max(o.total_s for o in outs)
        decoded = sum(len(o.token_ids) - 1 for o in outs)
        return {"value": decoded / (last - first), "unit": "tokens/s", "h2d_bytes_per_step": llm.step_function.h2d_bytes,
                "d2h_bytes_per_step": llm.sampler.d2h_bytes, "ttft_ms": first * 1e3, "new_tokens": NEW_TOKENS}

    if args.sweep:
        print(f"decode steps (bf16, {cfg.num_hidden_layers} layers, {steps} steps each; bytes = weights + cache of the live requests; peak {peaks['hbm_gbs']:.0f} GB/s {peaks_from})")
        print("| requests | cached tokens each | ms/step | tokens/s | GB/s | of peak |")
        print("|---:|---:|---:|---:|---:|---:|")
        for batch in (1, 8, 16, 32, 64):
            for prompt_len in (128, 512, 1536):
                if prompt_len + total_new > cfg.max_position_embeddings:
                    continue
                r = decode_run(batch, steps, warmup, prompt_len)
                print(f"| {batch} | {prompt_len + warmup}-{prompt_len + total_new - 1} | {r['ms_per_step']:.3f} | {r['tokens_per_s']:.0f} | {r['gbs']:.0f} | {r['gbs'] / peaks['hbm_gbs']:.2f} |")
        print(f"prefill of one prompt (peak {peaks['bf16_tflops']:.0f} TFLOP/s {peaks_from})")
        print("| tokens | ms | tokens/s | TFLOP/s | of peak |")
        print("|---:|---:|---:|---:|---:|")
        for n_tokens in (128, 512, 1024, 2048):
            r = prefill_run(n_tokens)
            print(f"| {n_tokens} | {r['ms']:.3f} | {r['value']:.0f} | {r['tflops']:.0f} | {r['frac']:.2f} |")
        return 0
    main_run = decode_run(8, steps, warmup)
    clocks = main_run["clocks"]
    rejected = [r for r in clocks["reasons"] if r != "sw_power_cap"]
    if rejected:  # measured once more, as the timing rules ask
        main_run = decode_run(8, steps, warmup)
        clocks = main_run["clocks"]
    prefill = prefill_run()
    points, e2e = {}, None
    if not args.skip_points:
        points = {"decode_b1": decode_run(1, steps, warmup)["tokens_per_s"], "decode_b64": decode_run(64, steps, warmup)["tokens_per_s"]}
        e2e = e2e_run(8)
    line = {
        "metric": "decode_tokens_per_s", "value": main_run["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "TinyLlama-1.1B sizes, random weights N(0,0.02) seed 0", "global_batch": 8, "seq_len": cfg.max_position_embeddings,
            "prompt_len": PROMPT_LEN, "new_tokens": NEW_TOKENS, "parallelism": "single GPU", "layers": cfg.num_hidden_layers,
            "layers_of_config": full_layers, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
            "vocab": cfg.vocab_size, "page_size": page_size, "l2": "256 MiB buffer written before each timed region; weights of 2.2 GB exceed L2",
            "peaks": peaks_from,
        },
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": main_run["launches"],
        "prefill": {k: prefill[k] for k in ("value", "tokens", "ms", "frac")},
        "roofline": {"bound": "hbm", "achieved": main_run["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": main_run["gbs"] / peaks["hbm_gbs"], "bytes_per_step": main_run["bytes_per_step"], "of": peaks_from},
        "points": points,
        "kernels_library": ops.loaded_library_path(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
