"""``LLM``: the synchronous entry point, prompts in and generated tokens out.

Mirrors tinyvllm/serving/llm.py:56-147: ``LLM(EngineConfig)``, ``generate(prompts,
SamplingParams)``, ``close()``, context manager, and an output record with
``finish_reason`` in {"stop", "length", "cancelled"} (:12-53).  The engine is
token-in, token-out: a prompt is a sequence of token ids.  Text prompts work
when a tokenizer is given (any object with ``encode(str) -> list[int]`` and
``decode(list[int]) -> str``) or the model folder holds a ``tokenizer.json``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

from ..config.engine import EngineConfig
from ..sampling.params import SamplingParams
from .engine import Engine, GenerateRequest


@dataclass(frozen=True)
class TextOutput:
    request_id: int
    text: str
    output_token_ids: tuple[int, ...]
    prompt_token_count: int
    finish_reason: str

    @property
    def completion_token_count(self) -> int:
        return len(self.output_token_ids)

    @property
    def total_token_count(self) -> int:
        return self.prompt_token_count + self.completion_token_count


class _JsonTokenizer:
    def __init__(self, path) -> None:
        from tokenizers import Tokenizer

        self._tokenizer = Tokenizer.from_file(str(path))

    def encode(self, text: str) -> list[int]:
        return self._tokenizer.encode(text).ids

    def decode(self, ids) -> str:
        return self._tokenizer.decode(list(ids))


class LLM:
    """One caller owns an instance at a time."""

    def __init__(self, config: EngineConfig, *, tokenizer=None) -> None:
        self.config = config
        self.tokenizer = tokenizer
        if tokenizer is None and (config.model / "tokenizer.json").is_file():
            self.tokenizer = _JsonTokenizer(config.model / "tokenizer.json")
        self._engine: Engine | None = Engine.from_config(config)

    @property
    def engine(self) -> Engine:
        if self._engine is None:
            raise RuntimeError("LLM is closed")
        return self._engine

    def _encode(self, prompt) -> tuple[int, ...]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer; give token ids, pass "
                                 "tokenizer=..., or put tokenizer.json into the model folder")
            return tuple(self.tokenizer.encode(prompt))
        return tuple(prompt)

    def generate(self, prompts, sampling: SamplingParams | None = None) -> list[TextOutput]:
        """``prompts``: one prompt or a sequence of prompts, each a string or a sequence
        of token ids.  All prompts share ``sampling``."""
        engine = self.engine
        sampling = SamplingParams() if sampling is None else sampling
        if not isinstance(sampling, SamplingParams):
            raise TypeError("sampling must be SamplingParams")
        if isinstance(prompts, str) or (isinstance(prompts, Sequence) and prompts
                                        and isinstance(prompts[0], int)):
            prompts = (prompts,)
        token_batches = [self._encode(prompt) for prompt in prompts]   # all before any is submitted
        outputs = engine.generate([GenerateRequest(tokens, sampling) for tokens in token_batches])
        results = []
        for output in outputs:
            text = self.tokenizer.decode(output.output_token_ids) if self.tokenizer is not None else ""
            results.append(TextOutput(output.request_id, text, output.output_token_ids,
                                      output.prompt_token_count, output.finish_reason))
        return results

    def stream(self, prompts, sampling: SamplingParams | None = None):
        """Like :meth:`generate`, but a generator: yields (index of the prompt, token id) as the
        tokens come (after every decode step) and, when a request has ended, (index, TextOutput).
        The engine has to be idle."""
        engine = self.engine
        sampling = SamplingParams() if sampling is None else sampling
        if not isinstance(sampling, SamplingParams):
            raise TypeError("sampling must be SamplingParams")
        if engine.has_unfinished():
            raise RuntimeError("stream() needs an idle engine")
        if isinstance(prompts, str) or (isinstance(prompts, Sequence) and prompts
                                        and isinstance(prompts[0], int)):
            prompts = (prompts,)
        token_batches = [self._encode(prompt) for prompt in prompts]
        index_of = {engine.submit(tokens, sampling): index for index, tokens in enumerate(token_batches)}
        while engine.has_unfinished() or index_of:
            events = engine.step()
            for request_id, token in events.tokens:
                yield index_of[request_id], token
            for output in events.finished:
                text = self.tokenizer.decode(output.output_token_ids) if self.tokenizer is not None else ""
                yield index_of.pop(output.request_id), TextOutput(
                    output.request_id, text, output.output_token_ids, output.prompt_token_count,
                    output.finish_reason)

    def close(self) -> None:
        if self._engine is not None:
            self._engine.close()
            self._engine = None

    def __enter__(self) -> "LLM":
        self.engine
        return self

    def __exit__(self, exc_type, exc, traceback) -> None:
        self.close()
