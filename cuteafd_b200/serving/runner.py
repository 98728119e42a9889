"""`ModelRunner` implementations: the GPU engine adapter and a deterministic fake for CPU tests.

`EngineRunner.run(rows)` packs the rows of a scheduler round into one engine step (one host-to-device copy of the
step inputs, CUDA-graph replay for decode-shaped steps), selects tokens on the device (greedy argmax, or the exact
sampler / masked argmax for rows that ask for it) and reads only token ids back.
`FakeRunner` computes "the model's" next token as a pure function of the token prefix, so scheduler, prefix-cache
and speculation tests are exact without a GPU (reference: cuteafd-bench/examples/fake_server.rs:1-10,
cuteafd-transport/src/synthetic.rs:128-131).
"""
from __future__ import annotations

import bisect
import hashlib

import torch

from .scheduler import Row


class FakeRunner:
    def __init__(self, vocab: int = 1000, max_rows: int = 4096, eos_every: int = 0):
        self.vocab, self._max_rows, self.calls, self.rows_seen, self.fail_next = vocab, max_rows, 0, 0, None
        self.kv: dict = {}           # (id(seq), position) -> token: lets tests check that cached KV is really reused

    @property
    def max_rows(self) -> int:
        return self._max_rows

    def next_token(self, prefix: list[int]) -> int:
        h = hashlib.blake2b(repr(prefix[-8:]).encode() + len(prefix).to_bytes(4, "little"), digest_size=4).digest()
        return int.from_bytes(h, "little") % self.vocab

    def run(self, rows: list[Row]) -> list[list[int]]:
        self.calls += 1
        if self.fail_next:
            msg, self.fail_next = self.fail_next, None
            raise RuntimeError(msg)
        out = []
        for r in rows:
            self.rows_seen += len(r.tokens)
            history = r.state.tokens[:r.start_pos]       # tokens whose KV must already be cached
            assert len(history) == r.start_pos, "scheduler asked to run a row at a position beyond its history"
            toks = []
            for i in r.want_logits:
                prefix = history + r.tokens[:i + 1]
                t = self.next_token(prefix)
                c = getattr(r.state.req, "constraint", None)
                m = c.mask(prefix) if c is not None else None
                if m is not None:                        # grammar mask: the fake model's pick moves to an allowed token
                    w = m.to("cpu").tolist()
                    allowed = [j for j in range(self.vocab) if (w[j >> 5] >> (j & 31)) & 1]
                    if allowed and t not in allowed:
                        t = allowed[t % len(allowed)]
                toks.append(t)
            out.append(toks)
        return out


class EngineRunner:
    def __init__(self, engine, max_rows: int = 4096):
        self.eng, self._max_rows = engine, max_rows
        self.h2d_bytes = self.d2h_bytes = 0
        # with `keep_hidden` every step leaves, per sequence, (start position, input tokens, target hidden rows): what an
        # MTP drafter pairs with the next tokens (serving.mtp_drafter)
        self.keep_hidden = False
        self.records: dict = {}
        # hybrid stacks (linear-attention layers): every live sequence owns one recurrent-state slot of the engine
        self._recurrent = bool(getattr(engine, "lin_layers", None))
        self._state_slot: dict = {}
        self._state_pos: dict = {}
        self._deferred = None             # (step shape, [(state id, start position, rows)]) of a speculative step awaiting `commit`
        self._free_slots = list(range(getattr(engine, "max_seqs", 0)))[::-1] if self._recurrent else []
        self._tok_host = torch.zeros(max(64, max_rows), dtype=torch.int32)
        if torch.cuda.is_available():
            self._tok_host = self._tok_host.pin_memory()

    @property
    def max_rows(self) -> int:
        return self._max_rows

    def forget(self, state):
        """The scheduler finished this sequence: its recurrent-state slot and hidden records are free again."""
        slot = self._state_slot.pop(id(state), None)
        self._state_pos.pop(id(state), None)
        if slot is not None:
            self._free_slots.append(slot)
        self.records.pop(id(state), None)

    def _slots_of(self, rows: list[Row]) -> list[int]:
        out, fresh = [], []
        for r in rows:
            slot = self._state_slot.get(id(r.state))
            if slot is None or r.start_pos == 0:
                if slot is None:
                    if r.start_pos != 0:
                        raise RuntimeError("a linear-attention stack cannot resume a sequence from cached pages: run it without the prefix cache")
                    if not self._free_slots:
                        raise RuntimeError("more live sequences than recurrent-state slots (engine max_seqs)")
                    slot = self._state_slot[id(r.state)] = self._free_slots.pop()
                fresh.append(slot)
            elif r.start_pos != self._state_pos.get(id(r.state)):      # the recurrent state sits at another position
                raise RuntimeError("a linear-attention stack cannot step back (was a speculative step left uncommitted?)")
            self._state_pos[id(r.state)] = r.start_pos + len(r.tokens)
            out.append(slot)
        self.eng.reset_state_slots(fresh)
        return out

    def commit(self, accepted: list):
        """The scheduler verified a speculative step: `accepted` = [(sequence state, accepted input rows)].  Stacks with recurrent
        layers now absorb exactly those rows (the step itself left their state untouched)."""
        if self._deferred is None:
            return
        sh, order = self._deferred
        self._deferred = None
        by_state = {id(st): n for st, n in accepted}
        counts = []
        for sid, start, n in order:
            k = by_state.get(sid, n)
            counts.append(k)
            if sid in self._state_pos:
                self._state_pos[sid] = start + k
        self.eng.commit_state(sh, counts)

    def run(self, rows: list[Row]) -> list[list[int]]:
        from ..engine.engine import StepShape
        from .. import ops
        eng = self.eng
        if self._deferred is not None:
            raise RuntimeError("the previous speculative step of a linear-attention stack was not committed")
        tokens, positions, slots, logit_rows, kv_len, q_start, q_len, pages = [], [], [], [], [], [], [], []
        over_rows, over_vals = [], []           # step rows whose embedding is an image row of the request
        for r in rows:
            seq = r.state.seq
            q_start.append(len(tokens))
            n = len(r.tokens)
            emb = getattr(r.state.req, "embeds", None)
            if emb is not None and r.start_pos <= emb["positions"][-1]:
                pos = emb["positions"]
                lo, hi = bisect.bisect_left(pos, r.start_pos), bisect.bisect_left(pos, r.start_pos + n)
                if hi > lo:
                    over_rows += [len(tokens) + p - r.start_pos for p in pos[lo:hi]]
                    over_vals.append(emb["rows"][lo:hi])
            seq.ensure(eng_pool(self), r.start_pos + n)
            for i, t in enumerate(r.tokens):
                tokens.append(t)
                positions.append(r.start_pos + i)
                slots.append(seq.slot(r.start_pos + i))
            logit_rows += [q_start[-1] + i for i in r.want_logits]
            kv_len.append(r.start_pos + n)
            q_len.append(n)
            pages.append(seq.pages)
        extra = {"state_slots": self._slots_of(rows)} if self._recurrent else {}
        if getattr(eng, "engram", None) is not None:          # n-gram memory: the three tokens before each row run
            extra["engram_ctx"] = [r.state.tokens[max(0, r.start_pos - 3):r.start_pos] for r in rows]
        self.h2d_bytes += eng.set_inputs(tokens, positions, slots, logit_rows, kv_len, q_start, q_len, pages, **extra)
        max_q = max(q_len)
        decode_like = max_q <= 8
        # regular decode / verify rounds (every sequence the same number of rows, logits for every row or none) may be cut into
        # micro-batches by a multi-GPU engine
        uniform = decode_like and all(q == max_q for q in q_len) and (not logit_rows or logit_rows == list(range(len(tokens))))
        # drafted rows over recurrent layers: the step leaves their state alone, `commit` absorbs what the scheduler accepts
        defer = self._recurrent and decode_like and any(len(r.tokens) > 1 and len(r.want_logits) == len(r.tokens) for r in rows)
        sh = StepShape(T=len(tokens), n_seq=len(rows), max_q_len=max_q, n_logits=len(logit_rows),
                       attn_splits=eng.attn_splits_for(len(rows), max_q, max(kv_len)) if decode_like else 1, uniform=uniform, defer_state=defer)
        if over_rows:
            eng.set_input_embeds(over_rows, torch.cat(over_vals) if len(over_vals) > 1 else over_vals[0])
        lane = eng.run(sh, use_graph=decode_like and not over_rows)
        pending = (sh, [(id(r.state), r.start_pos, len(r.tokens)) for r in rows]) if defer else None
        if self.keep_hidden:
            for r, qs, ql in zip(rows, q_start, q_len):
                recs = self.records.setdefault(id(r.state), [])
                recs.append((r.start_pos, list(r.tokens), lane.x[qs:qs + ql].clone()))
                if len(recs) > 256:          # nobody is consuming them (a request that never drafts): keep the tail only
                    del recs[:-64]
        n = len(logit_rows)
        # rows that sample or carry a grammar mask are re-selected from their logits row on the device
        special = []
        base = 0
        for r in rows:
            st = r.state
            if r.want_logits and (not st.req.sampling.greedy or st.req.constraint is not None):
                special.append((base, r))
            base += len(r.want_logits)
        for off, r in special:
            self._select_special(lane, off, r)
        if n:
            self._tok_host[:n].copy_(lane.next_tok[:n], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            self.d2h_bytes += 4 * n
        eng.check_status()
        flat = self._tok_host[:n].tolist()
        out, base = [], 0
        for r in rows:
            out.append(flat[base:base + len(r.want_logits)])
            base += len(r.want_logits)
        self._deferred = pending          # only a step that completed waits for its commit
        return out

    def _select_special(self, lane, off: int, r: Row):
        from .. import ops
        from ..ref import sampler as ref_sampler
        st = r.state
        k = len(r.want_logits)
        logits = lane.logits[off:off + k]
        mask = None
        if st.req.constraint is not None:
            # one mask per row: row i follows the sequence's history plus the step's inputs up to i (drafts included)
            history = st.tokens[:r.start_pos]
            ms = [st.req.constraint.mask(history + list(r.tokens[:i + 1])) for i in r.want_logits]
            if any(m is not None for m in ms):
                ref = next(m for m in ms if m is not None)
                ms = [m if m is not None else torch.full_like(ref, -1) for m in ms]
                mask = torch.stack([m.view(-1) for m in ms]).to(logits.device).contiguous()
        p = st.req.sampling
        if p.greedy:
            ops.argmax_rows(logits, lane.next_tok[off:off + k], masks=mask, status=lane.tok_status[off:off + k])
        elif 1 <= p.top_k <= 1024:
            pos = [len(st.tokens) + i for i in range(k)]
            par = ops.pack_sample_params([p] * k, pos).to(logits.device)
            ops.sample_rows(logits, par, lane.next_tok[off:off + k], lane.tok_status[off:off + k], masks=mask)
        else:   # unbounded candidate sets go through the exact host sampler on the logits row
            host = logits.float().cpu()
            for i in range(k):
                mk = None
                if mask is not None:
                    bits = mask[i].cpu()
                    mk = torch.tensor([(int(bits[j >> 5]) >> (j & 31)) & 1 for j in range(host.shape[1])], dtype=torch.bool)
                lane.next_tok[off + i] = ref_sampler.sample(host[i], p, len(st.tokens) + i, mk)


def eng_pool(runner: EngineRunner):
    return runner.pool


def attach_pool(runner: EngineRunner, pool):
    runner.pool = pool
    return runner
