"""A small, whole inference engine for the Llama architecture on one B200 (sm_100a).

``LLM(model_folder).generate(prompts, SamplingParams(...))`` is the Python entry point,
``python -m llmserve_triton_kernels_b200.cli`` the command line, ``bin/trace_run`` the replay
program.
"""

from .sampling.params import SamplingParams  # noqa: F401


def __getattr__(name):
    if name in ("LLM", "RequestOutput"):
        from .engine import llm

        return getattr(llm, name)
    raise AttributeError(name)
