"""Request bookkeeping and batching over a model's ``step``: named requests mapped onto the model's request slots and
cache pages, explicit steps (a caller-made schedule) and a continuous-batching greedy scheduler.

A step is a ragged batch: every live request that takes part contributes its next tokens -- a portion of its prompt or
the one token it decoded last -- and all of them run as one forward pass.  Finished requests give their pages and
slot back at once, so later requests reuse them.
"""
from __future__ import annotations

from collections import deque


class Engine:
    def __init__(self, model):
        self.model = model
        self.slots: dict[str, int] = {}  # request name -> model request id

    # -- explicit schedule
    def step(self, entries, end=()):
        """``entries``: [(name, tokens, want offsets)]; a name seen for the first time is admitted.  ``end``: names whose state is
        released after the step.  Returns fp32 logits [sum of wanted rows, vocab] in entry order."""
        batch, want = [], []
        for name, tokens, w in entries:
            if name not in self.slots:
                self.slots[name] = self.model.alloc_request()
            if len(tokens) == 0:  # admitted, nothing to run for it in this step
                continue
            batch.append((self.slots[name], tokens))
            want.append(list(w))
        try:
            if not batch:
                import torch
                return torch.empty((0, 0), dtype=torch.float32)
            return self.model.step(batch, want)
        finally:
            for name in end:
                self.release(name)

    def release(self, name) -> None:
        rid = self.slots.pop(name, None)
        if rid is not None:
            self.model.drop_request(rid)

    # -- scheduler: greedy generation of many prompts with continuous batching
    def generate(self, prompts, max_new_tokens: int, max_live: int = 4, token_budget: int = 256, stop_ids=()):
        """Greedy continuation of every prompt.  Each step carries one token of every request that is decoding and fills the rest of
        ``token_budget`` with prompt portions of admitted requests (first come, first served; at most ``max_live`` live)."""
        waiting = deque(range(len(prompts)))
        out = [[] for _ in prompts]
        live = {}  # index -> [tokens fed so far, pending token or None]
        stop = set(stop_ids)
        while waiting or live:
            while waiting and len(live) < max_live:
                i = waiting.popleft()
                live[i] = [0, None]
            entries, kinds, budget = [], [], token_budget
            for i, (fed, pending) in live.items():
                if pending is not None:
                    entries.append((f"g{i}", [pending], [0]))
                    kinds.append((i, "decode"))
                    budget -= 1
            for i, (fed, pending) in live.items():
                if pending is None and budget > 0:
                    part = prompts[i][fed:fed + budget]
                    last = fed + len(part) == len(prompts[i])
                    entries.append((f"g{i}", part, [len(part) - 1] if last else []))
                    kinds.append((i, "last" if last else "part"))
                    live[i][0] = fed + len(part)
                    budget -= len(part)
            batch = []
            for n, t, _ in entries:
                if n not in self.slots:
                    self.slots[n] = self.model.alloc_request()
                batch.append((self.slots[n], t))
            _, sampled = self.model.step(batch, [w for _, _, w in entries], sample=True, logits=False)
            row = 0
            for (i, kind) in kinds:
                if kind == "part":
                    continue
                tok = sampled[row]
                row += 1
                out[i].append(tok)
                live[i][1] = tok
                if len(out[i]) >= max_new_tokens or tok in stop:
                    del live[i]
                    self.release(f"g{i}")
        return out
