"""MTP drafter for the serving scheduler: proposes draft tokens with the model's own multi-token-prediction module.

The scheduler asks `propose(state, n)` before each decode round.  The drafter keeps, per sequence, the target hidden
state of the last verified position; the runner records the hidden rows of every step (`EngineRunner.keep_hidden`), and
`propose` first (re)writes the draft layer's KV rows of all positions verified since the last call - pairing each
token with the target hidden of the position before it - and then drafts `n` tokens by feeding the module its own
output.  Rows written from draft hiddens are provisional and are rewritten by the next call, so the drafts stay exact
with respect to `engine.mtp.MtpSpeculator` / the oracle; verification in the scheduler keeps the output lossless.
(Reference: native MTP drafter of the MiMo / DeepSeek families, families/mimo_v2/engine.rs, shared/draft/.)
"""
from __future__ import annotations

import torch

from ..engine.engine import StepShape

CHUNK = 2048


class MtpDrafter:
    def __init__(self, runner, depth: int = 0):
        if not runner.eng.weights.mtp:
            raise ValueError("this model has no MTP module")
        self.runner, self.eng, self.depth = runner, runner.eng, depth
        runner.keep_hidden = True
        self.last_h: dict = {}          # id(state) -> hidden of the last verified position
        self.proposed = 0
        self._host = torch.zeros(64, dtype=torch.int32)
        if torch.cuda.is_available():
            self._host = self._host.pin_memory()

    def _step(self, st, rows, want_token: bool):
        eng, seq = self.eng, st.seq
        tokens = [t for t, _, _ in rows]
        positions = [p for _, p, _ in rows]
        slots = [seq.slot(p - 1) for p in positions]
        T = len(rows)
        eng.set_inputs(tokens, positions, slots, [T - 1] if want_token else [], [positions[-1]], [0], [T], [seq.pages])
        sh = StepShape(T=T, n_seq=1, max_q_len=T, n_logits=1 if want_token else 0, attn_splits=eng.attn_splits_for(1, T, positions[-1]))
        lane = eng.mtp_forward(self.depth, sh, torch.stack([h for _, _, h in rows]))
        h = lane.x[T - 1].clone()
        tok = None
        if want_token:
            self._host[:1].copy_(lane.next_tok[:1], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            tok = int(self._host[0])
        return tok, h

    def propose(self, st, n: int) -> list[int]:
        key = id(st)
        recs = self.runner.records.pop(key, [])
        carried = self.last_h.get(key)
        pend = []
        for start, toks, hid in recs:
            valid = min(len(toks), st.seq.length - start)
            for i in range(max(valid, 0)):
                pos = start + i
                prev = hid[i - 1] if i > 0 else carried
                if pos >= 1 and prev is not None:
                    pend.append((toks[i], pos, prev))
            if valid > 0:
                carried = hid[valid - 1]
        if carried is None or st.pending is None or n <= 0:
            self.last_h[key] = carried
            return []
        self.last_h[key] = carried
        pend.append((st.pending, st.seq.length, carried))
        st.seq.ensure(self.runner.pool, st.seq.length + n + 1)
        tok = h = None
        for c in range(0, len(pend), CHUNK):                  # long prompts: the draft layer prefetches in chunks
            part = pend[c:c + CHUNK]
            tok, h = self._step(st, part, want_token=c + CHUNK >= len(pend))
        drafts = [tok]
        for d in range(1, n):
            tok, h = self._step(st, [(drafts[-1], st.seq.length + d, h)], True)
            drafts.append(tok)
        self.proposed += len(drafts)
        if len(self.last_h) > 4096:                           # forget sequences that are gone
            self.last_h.clear()
        return drafts
