"""The Python entry point: a model folder and prompts (token ids) in, generated
token ids out.

In the reference a user builds ``NativeGPT2(weights_dir, library_path,
backend, EngineOptions)`` and drives sessions or the batch API
(pytorch/src/mini_llm/native.py:169-233, batch_api.py:44-70); its scheduler
sits above that (pytorch/src/mini_llm/scheduler.py).  Here ``LLM`` holds the
engine and a scheduler, and ``generate`` runs the requests to completion with
continuous batching.
"""

from __future__ import annotations

from dataclasses import dataclass

from .engine.engine import Engine
from .engine.scheduler import Request, Scheduler
from .sampling import request_seed


@dataclass
class EngineOptions:
    """Options of the engine and its scheduler (the reference's counterpart:
    ``EngineOptions{use_kv_cache, max_sessions, fp16_decode}``, native.py:31-38)."""

    dtype: str = "bfloat16"               # "bfloat16" or "float32"
    device: str = "cuda:0"
    page_size: int = 64
    cache_tokens: int | None = None       # tokens the page pool holds; default: max_sessions full contexts
    max_sessions: int = 64                # most requests live at a time
    max_tokens_per_step: int = 2048       # token budget of one batch
    max_prefill_chunk: int | None = None  # longest prompt portion in one batch
    plain_kernels: bool = False
    cuda_graphs: bool = True
    run_ahead: bool = True                # launch a step before the host has read the step before it


class LLM:
    def __init__(self, model_dir: str, options: EngineOptions | None = None, **overrides):
        options = options or EngineOptions()
        for key, value in overrides.items():
            if not hasattr(options, key):
                raise TypeError(f"unknown engine option '{key}'")
            setattr(options, key, value)
        self.options = options
        self.engine = Engine(model_dir, dtype=options.dtype, device=options.device, page_size=options.page_size,
                             cache_tokens=options.cache_tokens, max_requests=options.max_sessions,
                             max_tokens_per_step=options.max_tokens_per_step, plain_kernels=options.plain_kernels,
                             cuda_graphs=options.cuda_graphs)
        self.scheduler = Scheduler(self.engine, options.max_tokens_per_step, options.max_prefill_chunk,
                                   options.max_sessions, run_ahead=options.run_ahead)

    @property
    def eos_token_id(self):
        return self.engine.spec.eos_token_id

    def generate(self, prompts, max_new_tokens: int = 64, temperature: float = 0.0, top_p: float = 1.0,
                 seed: int = 0, eos_token_id: int | None = None, on_token=None, return_requests: bool = False):
        """Generate for every prompt (a list of token ids).  Returns one list of
        new token ids per prompt; raises if a request failed.  ``temperature <= 0``
        is greedy.  ``eos_token_id=None`` ends on nothing but length and context
        (pass ``llm.eos_token_id`` to stop at the model's end-of-text token).
        ``seed``: one number for the call (request i then draws with
        ``request_seed(seed, i)``) or a list with one seed per prompt.
        ``on_token(index, token, finish_reason)`` is called for every token."""
        requests = []
        prompts = list(prompts)
        if isinstance(seed, (list, tuple)):
            if len(seed) != len(prompts):
                raise ValueError("one seed per prompt is needed when seeds are given as a list")
            seeds = [int(s) for s in seed]
        else:
            seeds = [request_seed(seed, index) for index in range(len(prompts))]
        for index, prompt in enumerate(prompts):
            emit = None
            if on_token is not None:
                emit = (lambda token, reason, i=index: on_token(i, token, reason))
            request = Request(list(int(t) for t in prompt), max_new_tokens, eos_token_id, float(temperature),
                              float(top_p), seeds[index], emit)
            requests.append(request)
            self.scheduler.submit(request)
        self.scheduler.run()
        if return_requests:
            return requests
        for index, request in enumerate(requests):
            if request.error is not None:
                raise RuntimeError(f"request {index} failed: {request.error}")
        return [list(r.generated) for r in requests]


def generate(model_dir: str, prompts, max_new_tokens: int = 64, temperature: float = 0.0, top_p: float = 1.0,
             seed: int = 0, eos_token_id: int | None = None, **engine_options):
    """One call: load ``model_dir``, generate for ``prompts``, return the new token ids."""
    return LLM(model_dir, **engine_options).generate(prompts, max_new_tokens, temperature, top_p, seed, eos_token_id)
