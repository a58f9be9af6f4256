"""Command line:  python -m llmserve_triton_kernels_b200.cli --model DIR --prompt "..."

Option names and meanings follow the reference's demo (src/llmserve/cli.py:17-26: ``--model
--prompt --max-new-tokens --mode --temperature --device --dtype``; ``--model tiny`` runs random
weights on token ids 10..25 with ids printed, src/llmserve/cli.py:31-33) and, for the engine, its
server launcher (src/llmserve/server/__main__.py:26-31: ``--block-size --num-blocks --kv-mem-mib
--max-batch-size --policy``).  The last line has the reference's form:
``[kv_cache] ttft=… ms | decode=… tok/s | peak mem=… MiB`` (src/llmserve/cli.py:48-53).
"""

from __future__ import annotations

import argparse

import torch

from .config.presets import PRESETS
from .engine.llm import LLM
from .sampling import SamplingParams


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="llmserve_triton_kernels_b200.cli", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help=f"model folder (config.json + safetensors), or a preset for random weights: {sorted(PRESETS)}")
    ap.add_argument("--prompt", default="Explain KV caching in one paragraph.")
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids instead of --prompt")
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--mode", choices=["kv_cache"], default="kv_cache", help="the reference's no-cache 'naive' mode is not built; its role is the tests' plain implementation")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=None, help="sampling seed (and the weights' seed for a preset; default 0 there)")
    ap.add_argument("--device", default="cuda", help="a CUDA device; there is no CPU path")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-blocks", type=int, default=None)
    ap.add_argument("--kv-mem-mib", type=float, default=None, help="size the cache by memory instead of --num-blocks")
    ap.add_argument("--max-batch-size", type=int, default=8)
    ap.add_argument("--max-num-batched-tokens", type=int, default=4096)
    ap.add_argument("--chunk-size", type=int, default=None, help="most prompt tokens of one request per step")
    ap.add_argument("--policy", choices=["continuous", "static"], default="continuous")
    return ap.parse_args(argv)


def main(argv=None) -> None:
    args = parse_args(argv)
    device = "cuda:0" if args.device == "cuda" else args.device
    llm = LLM(
        args.model, dtype=args.dtype, device=device, seed=args.seed or 0, block_size=args.block_size,
        num_blocks=args.num_blocks, kv_mem_mib=args.kv_mem_mib, max_batch_size=args.max_batch_size,
        max_num_batched_tokens=args.max_num_batched_tokens, chunk_size=args.chunk_size, policy=args.policy,
    )
    tok = llm.tokenizer
    if args.prompt_ids is not None:
        prompt = [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    elif tok is None:
        prompt = [t % llm.config.vocab_size for t in range(10, 26)]
    else:
        prompt = tok(args.prompt).input_ids
    eos = tok.eos_token_id if tok is not None else None
    params = SamplingParams(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, max_new_tokens=args.max_new_tokens,
        eos_token_id=eos, seed=args.seed,
    )
    if llm.device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(llm.device)
    result = llm.generate([prompt], params)[0]
    peak = torch.cuda.max_memory_allocated(llm.device) if llm.device.type == "cuda" else 0
    print(result.text if tok is not None else result.token_ids)
    print(
        f"\n[{args.mode}] ttft={result.ttft_s * 1e3:.1f} ms | "
        f"decode={result.decode_tokens_per_s:.1f} tok/s | "
        f"peak mem={peak / 2**20:.0f} MiB"
    )


if __name__ == "__main__":
    main()
