"""Speculative greedy decoding with the model's own multi-token-prediction (MTP) module as the drafter.

Protocol (the oracle's `RefModel.generate_speculative`; reference: MTP draft/verify rounds,
families/deepseek_v4/engine.rs:2047-2133, mtp_protocol_ref.py:6-19, lossless acceptance in
cuteafd-core/src/verify.rs):

  * the MTP module pairs the TARGET hidden state of position q-1 with the token at position q, runs one decoder
    layer of its own (own KV rows) and projects with the shared LM head: its output at position q predicts q+1;
  * a round drafts `n_draft` tokens by feeding the module its own output hidden, verifies anchor + drafts in ONE
    target step of 1 + n_draft rows per sequence, and accepts the longest prefix the target agrees with, plus the
    target's own next token (so every round emits at least one token and the output equals plain greedy decoding);
  * MTP rows written from draft hiddens are provisional: the next round first rewrites the rows of the accepted
    positions from the verified target hiddens ("pending rows"), and the last of them yields the next first draft, so
    one MTP step both repairs the draft cache and starts the next round.

The MTP layer's KV rows live in extra layers of the engine's paged KV store and reuse the sequence's pages; because
there is no MTP row for position 0, the row of position q sits in the slot of position q-1.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import ops
from .engine import Engine, StepShape
from .kv import PagePool, SeqKV


@dataclass
class _Seq:
    kv: SeqKV
    length: int = 0                 # verified tokens whose target KV is in the cache
    anchor: int = 0                 # last emitted token (not yet in the cache)
    out: list = field(default_factory=list)
    pending: list = field(default_factory=list)   # [(token, position, hidden row tensor [H])] MTP rows to (re)write
    accepted: list = field(default_factory=list)  # drafts accepted per round


class MtpSpeculator:
    def __init__(self, engine: Engine, pool: PagePool | None = None, n_draft: int = 3, depth: int = 0, use_graph: bool = False):
        if not engine.weights.mtp:
            raise ValueError("this model has no MTP module")
        if getattr(engine, "lin_layers", None):
            raise NotImplementedError("speculation needs recurrent-state snapshots per draft row: not wired for linear-attention stacks")
        self.eng, self.pool, self.n_draft, self.depth = engine, pool or PagePool(engine.n_pages), n_draft, depth
        self.seqs: list[_Seq] = []
        self.rounds = 0
        self.seconds_drafting = self.seconds_verifying = 0.0     # host clock, split at the last draft token's read-back
        self._host = None
        self._acc = None
        self.use_graph = use_graph       # replay draft and verify steps from CUDA graphs (steady-state serving / benchmarks)

    # ------------------------------------------------------------------ helpers
    def _read(self, dev_tokens: torch.Tensor, n: int) -> list[int]:
        if self._host is None or self._host.numel() < n:
            self._host = torch.zeros(max(n, 256), dtype=torch.int32).pin_memory()
        self._host[:n].copy_(dev_tokens[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._host[:n].tolist()

    def _read_many(self, parts: list) -> list:
        """Several device int32 tensors -> host lists with one synchronisation."""
        total = sum(n for _, n in parts)
        if self._host is None or self._host.numel() < total:
            self._host = torch.zeros(max(total, 256), dtype=torch.int32).pin_memory()
        o = 0
        for t, n in parts:
            self._host[o:o + n].copy_(t[:n], non_blocking=True)
            o += n
        torch.cuda.current_stream().synchronize()
        out, o = [], 0
        for _, n in parts:
            out.append(self._host[o:o + n].tolist())
            o += n
        return out

    def _mtp_step(self, rows_per_seq: list[list], want_logits: bool):
        """One MTP step.  rows_per_seq[i] = [(token, position, hidden)], possibly empty.  Returns (first-draft token
        per participating sequence, output hidden of its last row) for the sequences that had rows."""
        eng = self.eng
        live = [(s, rows) for s, rows in zip(self.seqs, rows_per_seq) if rows]
        tokens, positions, slots, kv_len, q_start, q_len, logit_rows, hid = [], [], [], [], [], [], [], []
        for s, rows in live:
            q_start.append(len(tokens))
            for tok, pos, h in rows:
                tokens.append(tok); positions.append(pos); slots.append(s.kv.slot(pos - 1)); hid.append(h)
            q_len.append(len(rows))
            kv_len.append(rows[-1][1])                    # MTP rows exist for positions 1..pos: `pos` rows
            logit_rows.append(len(tokens) - 1)
        T = len(tokens)
        eng.set_inputs(tokens, positions, slots, logit_rows if want_logits else [], kv_len, q_start, q_len, [s.kv.pages for s, _ in live])
        prev = torch.stack(hid)
        mq = max(q_len)
        sh = StepShape(T=T, n_seq=len(live), max_q_len=mq, n_logits=len(live) if want_logits else 0,
                       attn_splits=eng.attn_splits_for(len(live), mq, max(kv_len)))
        lane = eng.mtp_run(self.depth, sh, prev, self.use_graph)
        last = torch.tensor(logit_rows, device=lane.x.device)
        h_out = lane.x[:T].index_select(0, last).clone()
        toks = self._read(lane.next_tok, len(live)) if want_logits else [0] * len(live)
        return live, toks, h_out

    # ------------------------------------------------------------------ API
    def prefill(self, prompts: list[list[int]]):
        """Target prefill (one step per prompt), leaving every prompt row's MTP input pending."""
        eng = self.eng
        self.seqs = []
        for p in prompts:
            s = _Seq(kv=SeqKV())
            s.kv.ensure(self.pool, len(p) + 2 + self.n_draft)
            n = len(p)
            eng.set_inputs(p, list(range(n)), [s.kv.slot(q) for q in range(n)], [n - 1], [n], [0], [n], [s.kv.pages])
            lane = eng.run(StepShape(T=n, n_seq=1, max_q_len=n, n_logits=1, attn_splits=1), use_graph=False)
            hidden = lane.x[:n].clone()
            s.anchor = self._read(lane.next_tok, 1)[0]
            s.length = n
            s.out = [s.anchor]
            s.pending = [(p[q], q, hidden[q - 1]) for q in range(1, n)] + [(s.anchor, n, hidden[n - 1])]
            self.seqs.append(s)

    def round(self):
        """One draft/verify round for every sequence."""
        eng, nd = self.eng, self.n_draft
        import time as _time
        t_start = _time.perf_counter()
        for s in self.seqs:
            s.kv.ensure(self.pool, s.length + nd + 2)
        # drafts: the pending rows first (repairs the draft cache, last row = first draft), then one row at a time
        live, toks, h = self._mtp_step([s.pending for s in self.seqs], True)
        drafts = [[t] for t in toks]
        for d in range(1, nd):
            rows = [[(drafts[i][-1], s.length + d, h[i])] for i, s in enumerate(self.seqs)]
            _, toks, h = self._mtp_step(rows, True)
            for i, t in enumerate(toks):
                drafts[i].append(t)
        t_drafted = _time.perf_counter()         # every draft step ends with a token read-back, so host clocks bracket device work
        # verify anchor + drafts in one target step
        tokens, positions, slots, kv_len, q_start, q_len = [], [], [], [], [], []
        for s, dr in zip(self.seqs, drafts):
            q_start.append(len(tokens))
            inputs = [s.anchor] + dr
            tokens += inputs
            positions += list(range(s.length, s.length + len(inputs)))
            slots += [s.kv.slot(q) for q in range(s.length, s.length + len(inputs))]
            kv_len.append(s.length + len(inputs))
            q_len.append(len(inputs))
        T = len(tokens)
        eng.set_inputs(tokens, positions, slots, list(range(T)), kv_len, q_start, q_len, [s.kv.pages for s in self.seqs])
        sh = StepShape(T=T, n_seq=len(self.seqs), max_q_len=nd + 1, n_logits=T, attn_splits=eng.attn_splits_for(len(self.seqs), nd + 1, max(kv_len)),
                       uniform=True)
        lane = eng.run(sh, use_graph=self.use_graph)
        # acceptance on the device (longest draft prefix the target agrees with, per sequence), read back with the target's
        # tokens in one transfer; `ref.ops.greedy_verify` is the host statement of the same rule
        n = len(self.seqs)
        if self._acc is None or self._acc.numel() < 2 * n:
            self._acc = torch.zeros(2 * max(n, 64), dtype=torch.int32, device=lane.next_tok.device)
        acc_dev, emit_dev = self._acc[:n], self._acc[n:2 * n]
        ops.verify_accept(eng.md["tokens"][:T].view(n, nd + 1), lane.next_tok[:T].view(n, nd + 1), None, acc_dev, emit_dev)
        both = self._read_many([(lane.next_tok, T), (self._acc, 2 * n)])
        target, acc_host, emit_host = both[0], both[1][:n], both[1][n:2 * n]
        vh = lane.x[:T].clone()
        for i, (s, dr) in enumerate(zip(self.seqs, drafts)):
            a0 = q_start[i]
            inputs = [s.anchor] + dr
            accepted = acc_host[i]
            emitted = target[a0:a0 + emit_host[i]]
            s.accepted.append(accepted - 1)
            s.out += emitted
            s.pending = [(inputs[j], s.length + j, vh[a0 + j - 1]) for j in range(1, accepted)]
            s.pending.append((emitted[-1], s.length + accepted, vh[a0 + accepted - 1]))
            s.length += accepted
            s.anchor = emitted[-1]
        self.rounds += 1
        t_end = _time.perf_counter()
        self.seconds_drafting += t_drafted - t_start
        self.seconds_verifying += t_end - t_drafted

    def generate(self, prompts: list[list[int]], n_new: int) -> list[list[int]]:
        self.prefill(prompts)
        while min(len(s.out) for s in self.seqs) < n_new:
            self.round()
        self.eng.check_status()
        out = [s.out[:n_new] for s in self.seqs]
        return out

    def release(self):
        for s in self.seqs:
            s.kv.release(self.pool)
        self.seqs = []
