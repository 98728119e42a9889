"""Batch generation driver on top of `Engine`: page allocation, chunked prefill, greedy decode loop.

This is the smallest public entry point that runs the model end to end (`generate(engine, prompts, n_new)`);
the serving scheduler (`serving.scheduler`) drives the same `Engine` methods with continuous batching,
prefix reuse and speculation.  Every step copies its inputs host-to-device from pinned memory and reads the
selected tokens back device-to-host, so timing this loop is an end-to-end measurement.
"""
from __future__ import annotations

import torch

from .engine import Engine, StepShape
from .kv import PAGE, PagePool, SeqKV


class BatchGenerator:
    def __init__(self, engine: Engine, pool: PagePool | None = None, prefill_chunk: int = 4096):
        self.eng = engine
        self.pool = pool or PagePool(engine.n_pages)
        self.prefill_chunk = prefill_chunk
        self.seqs: list[SeqKV] = []
        self.last: list[int] = []
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._tok_host = None

    def _readback(self, lane, n: int) -> list[int]:
        if self._tok_host is None or self._tok_host.numel() < n:
            self._tok_host = torch.zeros(max(n, 64), dtype=torch.int32).pin_memory()
        self._tok_host[:n].copy_(lane.next_tok[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * n
        return self._tok_host[:n].tolist()

    def _page_rows(self, seqs):
        return [s.pages for s in seqs]

    def prefill(self, prompts: list[list[int]], use_graph: bool = False) -> list[int]:
        """Runs every prompt through the model (chunked), returns the first generated token of each."""
        eng = self.eng
        self.seqs = [SeqKV() for _ in prompts]
        self.hist = [list(p) for p in prompts]           # tokens whose rows are in the cache (the n-gram memory looks three back)
        for s, p in zip(self.seqs, prompts):
            s.ensure(self.pool, len(p) + 1)
        eng.reset_state_slots(range(len(prompts)))       # hybrid stacks: sequence i owns recurrent-state slot i
        first = [0] * len(prompts)
        # sequences are prefetched one chunk at a time, several sequences per step while rows fit
        pending = [(i, 0) for i in range(len(prompts))]
        while pending:
            rows, batch = 0, []
            while pending and rows < self.prefill_chunk:
                i, off = pending.pop(0)
                take = min(len(prompts[i]) - off, self.prefill_chunk - rows)
                batch.append((i, off, take))
                rows += take
                if off + take < len(prompts[i]):
                    pending.insert(0, (i, off + take))
                    break
            tokens, positions, slots, logit_rows, kv_len, q_start, q_len, seqs = [], [], [], [], [], [], [], []
            finals = []
            for i, off, take in batch:
                s = self.seqs[i]
                q_start.append(len(tokens))
                tokens += prompts[i][off:off + take]
                positions += list(range(off, off + take))
                slots += [s.slot(p) for p in range(off, off + take)]
                kv_len.append(off + take)
                q_len.append(take)
                seqs.append(s)
                if off + take == len(prompts[i]):
                    finals.append((i, len(logit_rows)))
                    logit_rows.append(len(tokens) - 1)
            self.h2d_bytes += eng.set_inputs(tokens, positions, slots, logit_rows, kv_len, q_start, q_len, self._page_rows(seqs),
                                             state_slots=[i for i, _, _ in batch],
                                             **({"engram_ctx": [prompts[i][max(0, off - 3):off] for i, off, _ in batch]} if getattr(eng, "engram", None) is not None else {}))
            sh = StepShape(T=len(tokens), n_seq=len(batch), max_q_len=max(q_len), n_logits=len(logit_rows), attn_splits=1)
            lane = eng.run(sh, use_graph=use_graph)
            if finals:
                toks = self._readback(lane, len(logit_rows))
                for i, r in finals:
                    first[i] = toks[r]
            for i, off, take in batch:
                self.seqs[i].length = off + take
        self.last = first
        return first

    def plan_decode(self) -> StepShape:
        """Stages the inputs of one greedy decode step (one token per live sequence) and returns its shape."""
        eng, n = self.eng, len(self.seqs)
        tokens, positions, slots, kv_len = [], [], [], []
        for s, t in zip(self.seqs, self.last):
            s.ensure(self.pool, s.length + 1)
            tokens.append(t)
            positions.append(s.length)
            slots.append(s.slot(s.length))
            kv_len.append(s.length + 1)
        self.h2d_bytes += eng.set_inputs(tokens, positions, slots, list(range(n)), kv_len, list(range(n)), [1] * n,
                                         self._page_rows(self.seqs),
                                         **({"engram_ctx": [h[-3:] for h in self.hist]} if getattr(eng, "engram", None) is not None else {}))
        splits = eng.attn_splits_for(n, 1, max(kv_len))
        return StepShape(T=n, n_seq=n, max_q_len=1, n_logits=n, attn_splits=splits, uniform=True)

    def commit_decode(self, lane) -> list[int]:
        toks = self._readback(lane, len(self.seqs))
        for s in self.seqs:
            s.length += 1
        if getattr(self, "hist", None):
            for h, t in zip(self.hist, self.last):
                h.append(t)
        self.last = toks
        return toks

    def decode_step(self, use_graph: bool = True) -> list[int]:
        """One greedy token for every live sequence (feeds `self.last`)."""
        sh = self.plan_decode()
        return self.commit_decode(self.eng.run(sh, use_graph=use_graph))

    def plan_prefill_all(self, prompts: list[list[int]]) -> StepShape:
        """Stages ONE step that ingests every prompt whole (short prompts; `prefill` chunks long ones)."""
        eng = self.eng
        self.seqs = [SeqKV() for _ in prompts]
        eng.reset_state_slots(range(len(prompts)))
        tokens, positions, slots, logit_rows, kv_len, q_start, q_len = [], [], [], [], [], [], []
        for s, p in zip(self.seqs, prompts):
            s.ensure(self.pool, len(p) + 1)
            q_start.append(len(tokens))
            tokens += p
            positions += list(range(len(p)))
            slots += [s.slot(i) for i in range(len(p))]
            kv_len.append(len(p))
            q_len.append(len(p))
            logit_rows.append(len(tokens) - 1)
        self._prompt_lens = [len(p) for p in prompts]
        self.hist = [list(p) for p in prompts]
        self.h2d_bytes += eng.set_inputs(tokens, positions, slots, logit_rows, kv_len, q_start, q_len, self._page_rows(self.seqs),
                                         **({"engram_ctx": [[] for _ in prompts]} if getattr(eng, "engram", None) is not None else {}))
        return StepShape(T=len(tokens), n_seq=len(prompts), max_q_len=max(q_len), n_logits=len(logit_rows), attn_splits=1)

    def commit_prefill_all(self, lane) -> list[int]:
        toks = self._readback(lane, len(self.seqs))
        for s, n in zip(self.seqs, self._prompt_lens):
            s.length = n
        self.last = toks
        return toks

    def release(self):
        for s in self.seqs:
            s.release(self.pool)
        self.seqs = []


def generate(engine: Engine, prompts: list[list[int]], n_new: int, use_graph: bool = True) -> list[list[int]]:
    """Greedy-generate `n_new` tokens for every prompt.  Returns the new tokens per prompt."""
    g = BatchGenerator(engine)
    out = [[t] for t in g.prefill(prompts)]
    for _ in range(n_new - 1):
        for o, t in zip(out, g.decode_step(use_graph)):
            o.append(t)
    engine.check_status()
    g.release()
    return out
