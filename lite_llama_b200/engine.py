"""Continuous-batching engine: request queue, per-step scheduling, greedy sampling.

The role of the reference's ``ContinuousBatchingEngine`` (lite_llama/engine/continuous_engine.py:157-419: admit
while slots are free, prefill, then decode the running set every step) on top of ``ModelRunner``:

* models that serve RAGGED steps (``runner.ragged_steps``: the layer-list decoders) get one flat batch per step: one
  token of every running request plus prompt PORTIONS of the requests still reading their prompt, under a token
  budget per step, so a long prompt never stalls the decoding requests;
* the uniform rotary decoders keep the reference's scheme on the slot layout (``SlotBatch``): a new request's whole
  prompt is one prefill step, the running set decodes together.

Sampling is greedy through the library's ``argmax_rows`` kernel (the temperature-0 branch of
lite_llama/engine/sampler.py).  Admission reserves a request's worst case (prompt + new tokens) against the KV pool,
so a step never runs out of rows.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Sequence

import torch

from .executor.model_runner import ModelRunner, RequestState
from .kernels import argmax_rows


@dataclass
class GenerationRequest:
    rid: int
    prompt: list[int]
    max_new_tokens: int
    eos_token_id: int | None = None
    output: list[int] = field(default_factory=list)
    fed: int = 0                                   # prompt tokens already in the cache / state
    state: RequestState | None = None              # ragged models
    slot: int = -1                                 # slot-layout models
    finished: bool = False

    @property
    def reserve(self) -> int:
        return len(self.prompt) + self.max_new_tokens


class Engine:
    def __init__(self, runner: ModelRunner, max_step_tokens: int = 2048, max_portion: int = 512,
                 decode_graphs: bool = True) -> None:
        """``decode_graphs``: capture the ragged-step models' decode steps as CUDA graphs (one per batch width and
        context bucket) when the engine starts on a runner with no live request; pure decode steps then replay."""
        self.runner = runner
        self.max_step_tokens = max(1, max_step_tokens)
        self.max_portion = max(1, max_portion)
        self.waiting: deque[GenerationRequest] = deque()
        self.running: list[GenerationRequest] = []
        self.done: dict[int, GenerationRequest] = {}
        self._next_id = 0
        self._reserved = 0
        self.steps = 0
        if runner.ragged_steps:
            self._slots_free = runner.max_request_num
            self._pool = runner.kv_cache_manager.max_num_tokens
            if decode_graphs and hasattr(runner, "enable_ragged_decode_graphs"):
                runner.enable_ragged_decode_graphs()
        else:
            self._sb = runner.enable_slot_kv_cache()
            self._free_slots = list(range(self._sb.num_slots - 1, -1, -1))
            self._slots_free = len(self._free_slots)
            self._pool = None

    # ------------------------------------------------------------------------------------------------- requests #
    def add_request(self, prompt: Sequence[int], max_new_tokens: int, eos_token_id: int | None = None) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt or max_new_tokens < 1:
            raise ValueError("a request needs a non-empty prompt and at least one new token")
        if len(prompt) + max_new_tokens > self.runner.max_seq_len:
            raise ValueError(f"prompt + new tokens exceed max_seq_len {self.runner.max_seq_len}")
        if self._pool is not None and self._rows(len(prompt) + max_new_tokens) > self._pool:
            raise ValueError("the request alone exceeds the KV pool")
        rid = self._next_id
        self._next_id += 1
        self.waiting.append(GenerationRequest(rid, prompt, max_new_tokens, eos_token_id))
        return rid

    def _rows(self, tokens: int) -> int:
        """Pool rows a sequence of ``tokens`` holds at most: all of them, or -- when every cached layer has a sliding
        window and the runner gives unseen rows back on the way -- what the windows keep plus one portion."""
        keep = getattr(self.runner, "keep_positions", 0)
        return min(tokens, keep + self.max_portion) if keep else tokens

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _admit(self) -> None:
        while self.waiting and self._slots_free > 0:
            req = self.waiting[0]
            if self._pool is not None and self._reserved + self._rows(req.reserve) > self._pool:
                break
            self.waiting.popleft()
            self._slots_free -= 1
            self._reserved += self._rows(req.reserve)
            if self.runner.ragged_steps:
                req.state = self.runner.open_request()
            else:
                req.slot = self._free_slots.pop()
            self.running.append(req)

    def _retire(self, req: GenerationRequest) -> None:
        req.finished = True
        if self.runner.ragged_steps:
            self.runner.close_request(req.state)
            req.state = None
        else:
            self._free_slots.append(req.slot)
        self._slots_free += 1
        self._reserved -= self._rows(req.reserve)
        self.running.remove(req)
        self.done[req.rid] = req

    def _accept(self, req: GenerationRequest, token: int, produced: list[tuple[int, int]]) -> None:
        req.output.append(token)
        produced.append((req.rid, token))
        if len(req.output) >= req.max_new_tokens or (req.eos_token_id is not None and token == req.eos_token_id):
            self._retire(req)

    # ---------------------------------------------------------------------------------------------------- steps #
    def step(self) -> list[tuple[int, int]]:
        """One scheduling round; returns the ``(request id, token)`` pairs sampled in it."""
        self._admit()
        if not self.running:
            return []
        self.steps += 1
        return self._step_ragged() if self.runner.ragged_steps else self._step_slots()

    def _step_ragged(self) -> list[tuple[int, int]]:
        budget = self.max_step_tokens
        entries, samplers, want, at = [], [], [], 0
        # one token of every decoding request first, then prompt portions with what is left of the budget
        for req in self.running:
            if req.fed == len(req.prompt) and budget > 0:
                entries.append((req.state, [req.output[-1]]))
                at += 1
                budget -= 1
                want.append(at - 1)
                samplers.append(req)
        for req in self.running:
            if req.fed < len(req.prompt) and budget > 0:
                n = min(len(req.prompt) - req.fed, self.max_portion, budget)
                entries.append((req.state, req.prompt[req.fed:req.fed + n]))
                req.fed += n
                at += n
                budget -= n
                if req.fed == len(req.prompt):
                    want.append(at - 1)
                    samplers.append(req)
        logits = self.runner.forward_ragged(entries, want)
        produced: list[tuple[int, int]] = []
        if samplers:
            tokens = argmax_rows(logits).tolist()
            for req, tok in zip(samplers, tokens):
                self._accept(req, tok, produced)
        return produced

    def _step_slots(self) -> list[tuple[int, int]]:
        runner, dev = self.runner, self.runner.device
        produced: list[tuple[int, int]] = []
        fresh = next((r for r in self.running if r.fed == 0), None)
        if fresh is not None:                      # whole prompt of one new request
            n = len(fresh.prompt)
            self._sb.begin_prefill([fresh.slot], [n])
            ids = torch.tensor([fresh.prompt], dtype=torch.int64, device=dev)
            pos = torch.arange(n, dtype=torch.int64, device=dev).view(1, n)
            logits = runner.forward(ids, pos, last_token_index=torch.tensor([n - 1], device=dev))
            fresh.fed = n
            self._accept(fresh, int(argmax_rows(logits[:, -1, :].contiguous()).item()), produced)
            return produced
        batch = list(self.running)
        lens = [len(r.prompt) + len(r.output) for r in batch]
        width = self._sb.begin_decode([r.slot for r in batch], lens)
        ids = torch.zeros((width, 1), dtype=torch.int64)
        pos = torch.zeros((width, 1), dtype=torch.int64)
        for i, (r, n) in enumerate(zip(batch, lens)):
            ids[i, 0], pos[i, 0] = r.output[-1], n - 1
        for i in range(len(batch), width):
            pos[i, 0] = max(lens) - 1
        logits = runner.forward(ids.to(dev), pos.to(dev))
        tokens = argmax_rows(logits[: len(batch), -1, :].contiguous()).tolist()
        for r, tok in zip(batch, tokens):
            self._accept(r, tok, produced)
        return produced

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                 eos_token_id: int | None = None) -> list[list[int]]:
        """Greedy continuations of ``prompts`` (token ids), in order."""
        ids = [self.add_request(p, max_new_tokens, eos_token_id) for p in prompts]
        while self.has_work():
            self.step()
        return [self.done.pop(i).output for i in ids]
