"""The Python entry point: ``LLM(model).generate(prompts, params)``.

The reference's call is the free function ``generate(model, prompt_ids, params, device=)``
returning tokens and timings (src/llmserve/engine/generate.py:16-58,
src/llmserve/datatypes.py:16-27); its engine options are the server launcher's
``--block-size --num-blocks --kv-mem-mib --max-batch-size --policy``
(src/llmserve/server/__main__.py:26-31).  Here one object holds the model, the cache, the step
function and the scheduler, and serves many prompts at once through them.
"""

from __future__ import annotations

import gc
from dataclasses import dataclass, field
from pathlib import Path
from time import perf_counter

import torch

from .. import models as _models  # noqa: F401  registers the built-in architecture
from ..cache import CacheManager, num_pages_for_budget
from ..config.presets import PRESETS
from ..config.registry import architecture_of
from ..models.load import load_model, random_model, resolve_dtype
from ..parts.base import PagedKVSpec
from ..sampling import Sampler, SamplingParams
from .scheduler import Scheduler
from .step import StepFunction


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: list[int]
    token_ids: list[int]
    finish_reason: str | None
    text: str | None = None
    ttft_s: float = 0.0  # arrival to first token
    step_latencies_s: list[float] = field(default_factory=list)  # between consecutive tokens
    total_s: float = 0.0
    num_preemptions: int = 0

    @property
    def decode_tokens_per_s(self) -> float:
        total = sum(self.step_latencies_s)
        return len(self.step_latencies_s) / total if total > 0 else 0.0


class LLM:
    def __init__(
        self,
        model: str | Path | dict,
        *,
        dtype: str | torch.dtype = "bfloat16",
        device: str = "cuda:0",
        seed: int = 0,
        block_size: int = 16,
        num_blocks: int | None = None,
        kv_mem_mib: float | None = None,
        max_batch_size: int = 8,
        max_num_batched_tokens: int = 4096,
        chunk_size: int | None = None,
        policy: str = "continuous",
        tokenizer=None,
        freeze_gc: bool = True,
    ):
        """``model``: a folder with config.json and ``*.safetensors``; or the name of a preset or a
        config.json dictionary, for random weights drawn from ``seed``.

        ``freeze_gc``: once the engine stands, collect garbage and move everything that is alive to the collector's
        permanent generation (``gc.freeze()``).  A full collection otherwise walks the some 170,000 objects that the
        imported libraries keep, about 50 ms in which no step is launched; afterwards it walks a thousand."""
        self.device = torch.device(device)
        self.dtype = resolve_dtype(dtype)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        if isinstance(model, dict) or (isinstance(model, str) and model in PRESETS and not Path(model).exists()):
            cfg_dict = PRESETS[model] if isinstance(model, str) else model
            self.config = architecture_of(cfg_dict).config_class.from_dict(cfg_dict)
            self.model = random_model(self.config, seed, self.dtype, self.device)
        else:
            self.model, self.config = load_model(model, self.dtype, self.device)
            if tokenizer is None:
                tokenizer = _maybe_tokenizer(model)
        self.tokenizer = tokenizer
        specs = self.model.cache_specs()
        element = torch.empty(0, dtype=self.dtype).element_size()
        if num_blocks is None:
            if kv_mem_mib is not None:
                num_blocks = num_pages_for_budget(specs, block_size, element, int(kv_mem_mib * 2**20))
            else:  # room for every request slot at the model's full length, within a quarter of the free memory
                want = max_batch_size * -(-self.model.plan.max_positions // block_size)
                cap = want
                if self.device.type == "cuda":
                    free, _ = torch.cuda.mem_get_info(self.device)
                    groups = {s for s in specs if isinstance(s, PagedKVSpec)}
                    cap = num_pages_for_budget(specs, block_size, element, free // 4) // max(1, len(groups))
                num_blocks = max(1, min(want, cap))
        self.cache = CacheManager(
            specs, self.model.plan.schedule, page_size=block_size, num_pages=num_blocks,
            max_requests=max_batch_size, dtype=self.dtype, device=self.device,
        )
        self.step_function = StepFunction(self.model, self.cache)
        self.sampler = Sampler(self.device)
        self.scheduler = Scheduler(
            self.step_function, self.cache, self.sampler, max_position=self.model.plan.max_positions,
            max_batch_size=max_batch_size, max_num_batched_tokens=max_num_batched_tokens, chunk_size=chunk_size,
            policy=policy,
        )
        if freeze_gc:
            gc.collect()
            gc.freeze()

    def generate(self, prompts, params: SamplingParams | list[SamplingParams] | None = None) -> list[RequestOutput]:
        """Serve every prompt (a list of token ids, or a string when the folder has a tokenizer) to
        completion through the scheduler; outputs are in the order of the prompts."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if params is None:
            params = SamplingParams()
        per_prompt = params if isinstance(params, list) else [params] * len(prompts)
        if len(per_prompt) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        start = perf_counter()
        ids = []
        for prompt, p in zip(prompts, per_prompt):
            if isinstance(prompt, str):
                if self.tokenizer is None:
                    raise ValueError("a text prompt needs a tokenizer; this model folder has none (pass token ids)")
                prompt = self.tokenizer(prompt).input_ids
            ids.append(self.scheduler.add_request(list(prompt), p, arrival_time=start))
        self.scheduler.run_until_complete()
        outputs = []
        for rid in ids:
            r = self.scheduler.finished.pop(rid)
            times = r.token_times
            outputs.append(
                RequestOutput(
                    request_id=rid,
                    prompt_token_ids=r.prompt_ids,
                    token_ids=r.generated,
                    finish_reason=r.finish_reason,
                    text=self.tokenizer.decode(r.generated, skip_special_tokens=True) if self.tokenizer else None,
                    ttft_s=(times[0] - r.arrival_time) if times else 0.0,
                    step_latencies_s=[b - a for a, b in zip(times, times[1:])],
                    total_s=(r.finish_time or perf_counter()) - r.arrival_time,
                    num_preemptions=r.num_preemptions,
                )
            )
        return outputs


def _maybe_tokenizer(model_dir):
    path = Path(model_dir)
    if not any((path / f).exists() for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")):
        return None
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(path)
