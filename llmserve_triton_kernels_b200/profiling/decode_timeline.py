"""A timeline of one decode step, from the global timer as the kernels read it.

    python -m llmserve_triton_kernels_b200.profiling.decode_timeline [--batch 8] [--prompt 512] [--first 20] [--last 32]

The serving build has no stamps.  This program compiles a second copy of the kernel library with ``-DLLM_TIMELINE``
(``csrc/timeline.cuh``; into a folder of its own under the system's temporary folder, never beside the serving build), in which thread 0 of every CTA of
the decode products and of the decode attention stamps the global timer when the CTA enters, when it has asked for
all that does not depend on the kernel in front, when ``griddepcontrol.wait`` has let it go, when its inputs lie in
shared memory (products) or its key tiles are done (attention), and when it ends.  One captured decode step is replayed
once and the records are printed kernel by kernel, every time relative to the end of the last CTA of the kernel in
front: so a line reads "entered 1.9 us before the kernel in front had ended, was let go 0.1 us after it, had its input
0.9 us later, ended 2.8 us after that".  The reference's counterpart is its table of operator times
(benchmarks/profile_decode.py:55-73); kernels that overlap under programmatic dependent launch need stamps from
inside instead.

The stamps cost a few hundred nanoseconds per kernel: the step is slower here than in the serving build, and no number
of this program is a benchmark value.
"""

from __future__ import annotations

import argparse
import ctypes
import os


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", default="tinyllama-1.1b", help="a preset's name (random weights)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=512, help="tokens each request holds before the timed step")
    ap.add_argument("--first", type=int, default=20, help="first kernel of the step to print")
    ap.add_argument("--last", type=int, default=32, help="one past the last kernel to print")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--sections", action="store_true", help="also print, for every product, where warp 0's cycles inside its loop went")
    args = ap.parse_args()

    os.environ["LLMSERVE_B200_TIMELINE"] = "1"
    import numpy as np
    import torch

    from .. import ops
    from ..config.presets import PRESETS
    from ..engine.batch import StepEntry
    from ..engine.llm import LLM

    cfg = dict(PRESETS[args.config])
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    B, page = args.batch, 16
    pages = B * (-(-(args.prompt + 32) // page)) + 8
    llm = LLM(cfg, dtype="bfloat16", device="cuda:0", seed=0, block_size=page, num_blocks=pages, max_batch_size=B,
              max_num_batched_tokens=max(8192, args.prompt))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg["vocab_size"], (args.prompt,), generator=g).tolist() for _ in range(B)]
    names = [f"r{i}" for i in range(B)]
    step = llm.step_function
    per_step = max(1, 8192 // args.prompt)
    for i in range(0, B, per_step):
        step([StepEntry(n, p, []) for n, p in zip(names[i : i + per_step], prompts[i : i + per_step])])
    tokens = [p[-1] for p in prompts]
    for _ in range(6):
        logits = step([StepEntry(n, [t], [0]) for n, t in zip(names, tokens)])
        tokens = ops.argmax(logits).tolist()
    torch.cuda.synchronize()

    lib = ops.library()
    record = np.dtype([("t", "<u8", 6), ("kernel", "<i4"), ("launch", "<i4"), ("block", "<i4"), ("sm", "<i4"), ("a", "<i4"), ("b", "<i4")])

    def read(reader: str) -> np.ndarray:
        buf = np.zeros(1 << 16, dtype=record)
        n = getattr(lib, reader)(ctypes.c_void_p(buf.ctypes.data), ctypes.c_uint(1 << 16))
        return buf[:n]

    read("llm_timeline_read_linear"), read("llm_timeline_read_attention")  # what warm-up left
    graph = step.graphs[B]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.graph.replay()
    end.record()
    torch.cuda.synchronize()
    ops.check_device_errors()
    print(f"{args.config}, {B} requests of {args.prompt + 6} cached tokens; one replay of the step's graph with stamps: "
          f"{start.elapsed_time(end) * 1e3:.1f} us")
    lin, att = read("llm_timeline_read_linear"), read("llm_timeline_read_attention")
    t0 = min(lin["t"][:, 0].min(), att["t"][:, 0].min())
    mode = {0: "product", 1: "gate/up + SwiGLU", 2: "product into the stream", 3: "q/k/v + rotary + cache"}
    rows = []
    for key in sorted(set(zip(lin["kernel"].tolist(), lin["launch"].tolist())), key=lambda k: k[1]):
        r = lin[(lin["kernel"] == key[0]) & (lin["launch"] == key[1])]
        rows.append((f"{mode[key[0]]} [{r['a'][0]} x {r['b'][0]}]", r["t"].astype(np.int64) - t0, True, r["t"]))
    if len(att):
        a = att[np.argsort(att["t"][:, 0])]
        t = a["t"].astype(np.int64) - t0
        first = 0
        for i in range(1, len(a) + 1):
            if i == len(a) or t[i, 0] - t[i - 1, 0] > 2500:  # launches are several microseconds apart
                rows.append((f"attention, {a['kernel'][first] - 100} key warps", t[first:i], False, None))
                first = i
    rows.sort(key=lambda row: row[1][:, 0].min())
    print("times in us from the end of the last CTA of the kernel in front; medians over the CTAs that had work")
    print(f"{'#':>3} {'kernel':44s} {'CTAs':>4} {'entered':>8} {'let go':>7} {'inputs in':>9} {'ended':>6} {'last end':>8} {'span':>6}")
    previous_end = None
    for i, (label, t, is_product, raw) in enumerate(rows):
        busy = t[(t[:, 4] - t[:, 0]) > 1000] if is_product else t[t[:, 2] > -10**12]
        if not len(busy):
            busy = t
        last = int(t[:, 4].max())
        ref = previous_end if previous_end is not None else int(t[:, 0].min())
        if args.first <= i < args.last:
            f = lambda x: f"{(float(x) - ref) / 1e3:.2f}"
            print(f"{i:3d} {label:44s} {len(busy):4d} {f(np.median(busy[:, 0])):>8} {f(np.median(busy[:, 2])):>7} "
                  f"{f(np.median(busy[:, 3])):>9} {f(np.median(busy[:, 4])):>6} {f(last):>8} {(last - int(t[:, 0].min())) / 1e3:6.2f}")
            if args.sections and raw is not None:
                # warp 0 of every CTA: SM cycles inside the product's loop over weight boxes, by what they were spent on
                live = raw[(raw[:, 4] - raw[:, 0]) > 1000] if ((raw[:, 4] - raw[:, 0]) > 1000).any() else raw
                sec, n = live[:, 1], np.maximum(live[:, 3] & 0xFF, 1)
                wait, load, arm, mma = (sec >> 48) & 0xFFFF, (sec >> 32) & 0xFFFF, (sec >> 16) & 0xFFFF, sec & 0xFFFF
                loop, meet, whole = live[:, 5] >> 40, (live[:, 5] >> 20) & 0xFFFFF, live[:, 5] & 0xFFFFF
                m = lambda v: float(np.median(v))
                print(f"      warp 0: {m(n):.0f} boxes; cycles a box: wait for it {m(wait / n):.0f}, shared loads {m(load / n):.0f}, "
                      f"next request {m(arm / n):.0f}, products {m(mma / n):.0f}; loop {m(loop):.0f}, to the team's meeting {m(meet):.0f}, "
                      f"to the end {m(whole):.0f} cycles")
        previous_end = last
    print(f"first entry to last end: {(rows[-1][1][:, 4].max() - rows[0][1][:, 0].min()) / 1e3:.1f} us over {len(rows)} kernels")


if __name__ == "__main__":
    main()
