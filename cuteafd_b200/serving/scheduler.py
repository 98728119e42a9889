"""Continuous-batching scheduler: admission with prefix reuse, chunked prefill with a decode time share,
speculative decode with lossless verification, per-request isolation, stats.

One `step()` = admit -> (one prefill round | one decode/verify round).  The scheduler talks to the model through a
small `ModelRunner` interface (`run(rows) -> tokens`), implemented by `EngineRunner` over the GPU engine and by
`FakeRunner` for CPU tests - the same split the reference uses between its serve loop and `Engine`
(families/deepseek_v4/serve.rs:610-983: admission :641-767, prefill round :768-898, speculative step :389-537,
verify budget of 64 rows, failure isolation :932-940).
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Protocol

from ..engine.kv import PAGE, OutOfPages, PagePool, SeqKV
from ..ref.ops import greedy_verify
from ..ref.sampler import SamplingParams
from ..utils.trace import PhaseProfile, SpeculationTrace
from .draft_policy import DraftPolicy, SimpleDraftPolicy
from .prefix import PrefixCache

VERIFY_ROWS = 64


@dataclass
class Request:
    rid: str
    prompt: list[int]
    max_tokens: int = 128
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: tuple = ()
    eos_id: int | None = None
    on_token: Callable[[list[int], bool, str | None], None] | None = None   # (new tokens, finished, reason)
    constraint: object | None = None        # object with .mask(prefix_tokens) -> allowed-token bitmask or None
    use_cache: bool = True
    allow_drafts: bool = True
    embeds: dict | None = None              # {"positions": sorted prompt positions, "rows": bf16 [n, hidden]}: image rows of a vision tower
    arrived: float = field(default_factory=time.time)


@dataclass
class SeqState:
    req: Request
    seq: SeqKV
    prefilled: int = 0              # prompt tokens whose KV is in the cache
    out: list = field(default_factory=list)
    pending: int | None = None      # last emitted token whose KV is not written yet (the next anchor)
    cache_hit: int = 0
    ttft: float | None = None
    finished: bool = False
    reason: str | None = None
    cancelled: bool = False

    @property
    def tokens(self) -> list[int]:
        return self.req.prompt + self.out


@dataclass
class Row:
    """One sequence's contribution to a model step."""
    state: SeqState
    tokens: list[int]
    start_pos: int
    want_logits: list[int]          # indices into `tokens` whose next-token choice is needed


class ModelRunner(Protocol):
    def run(self, rows: list[Row]) -> list[list[int]]: ...
    @property
    def max_rows(self) -> int: ...


class Drafter(Protocol):
    def propose(self, state: SeqState, n: int) -> list[int]: ...


class NgramDrafter:
    """Copy-continuation drafts: if the last `k` tokens occurred before, propose what followed them
    (the reference mixes such copy drafts with neural ones; serve.rs:446-465)."""

    def __init__(self, k: int = 3):
        self.k = k

    def propose(self, state: SeqState, n: int) -> list[int]:
        toks = state.tokens
        for k in range(min(self.k, len(toks) - 1), 0, -1):
            tail = toks[-k:]
            for s in range(len(toks) - k - 1, -1, -1):
                if toks[s:s + k] == tail:
                    cont = toks[s + k:s + k + n]
                    if cont:
                        return cont
        return []


class Scheduler:
    def __init__(self, runner: ModelRunner, pool: PagePool, *, max_seqs: int = 16, prefill_chunk: int = 4096, decode_share: float = 0.2,
                 prefix: PrefixCache | None = None, drafter: Drafter | None = None, policy: DraftPolicy | None = None,
                 max_draft: int = 3, queue_limit: int = 64, queue_wait_s: float | None = None):
        self.runner, self.pool = runner, pool
        self.max_seqs, self.prefill_chunk, self.decode_share = max_seqs, prefill_chunk, decode_share
        self.prefix = prefix
        self.drafter, self.policy, self.max_draft = drafter, policy or SimpleDraftPolicy(max_draft), max_draft
        self.queue: deque[Request] = deque()
        self.queue_limit = queue_limit
        self.queue_wait_s = queue_wait_s                      # admission wait budget: a request queued longer than this is answered "busy"
        self.active: list[SeqState] = []
        self.fatal: str | None = None
        self._prefill_debt = 0.0
        self.stats = {"requests": 0, "finished": 0, "generated": 0, "prefill_tokens": 0, "steps": 0, "verify_rows": 0,
                      "drafted": 0, "accepted": 0, "failed": 0, "deferred": 0, "rejected": 0}
        # observability: host phases of a step, draft acceptance by draft position, a ring of recent events for the
        # console (only filled while somebody watches), the speculation trace file when the environment names one
        self.profile = PhaseProfile()
        self.accept_by_pos = [[0, 0] for _ in range(8)]          # [offered, accepted] per draft position
        self.events: deque = deque(maxlen=512)
        self.watchers = 0
        self.spec_trace = SpeculationTrace()
        self.recent: deque = deque(maxlen=32)

    # ------------------------------------------------------------------ intake
    def submit(self, req: Request) -> bool:
        if self.fatal:
            self._finish_unadmitted(req, "unavailable: " + self.fatal)
            return False
        if len(self.queue) >= self.queue_limit:
            self.stats["rejected"] += 1
            self._finish_unadmitted(req, "queue full")
            return False
        req.queued_at = time.monotonic()
        self.queue.append(req)
        self.stats["requests"] += 1
        return True

    def cancel(self, rid: str):
        for s in self.active:
            if s.req.rid == rid:
                s.cancelled = True
        self.queue = deque(r for r in self.queue if r.rid != rid)

    def _finish_unadmitted(self, req: Request, reason: str):
        if req.on_token:
            req.on_token([], True, reason)

    def fail_all(self, cause: str):
        """A terminal engine/transport failure: every admitted and queued client hears about it
        (reference: mimo_v2/serve_failures.rs:14-40)."""
        self.fatal = cause
        for s in self.active:
            self._finish(s, "error: " + cause, capture=False)
        self.active = []
        while self.queue:
            self._finish_unadmitted(self.queue.popleft(), "error: " + cause)

    # ------------------------------------------------------------------ admission
    def _admit(self):
        if self.queue_wait_s is not None:
            now = time.monotonic()
            while self.queue and now - getattr(self.queue[0], "queued_at", now) > self.queue_wait_s:
                self.stats["rejected"] += 1
                self._finish_unadmitted(self.queue.popleft(), "busy: admission wait budget exceeded")
        while self.queue and len(self.active) < self.max_seqs:
            req = self.queue[0]
            if not req.prompt:
                self.queue.popleft()
                self._finish_unadmitted(req, "error: empty prompt")
                continue
            try:
                if self.prefix is not None and req.use_cache:
                    adm = self.prefix.admit(req.prompt, reserve_new=req.max_tokens + self.max_draft + 1)
                    st = SeqState(req, adm.seq, prefilled=adm.hit_tokens, cache_hit=adm.hit_tokens)
                else:
                    seq = SeqKV()
                    need = seq.pages_needed(len(req.prompt) + req.max_tokens + self.max_draft + 1)
                    if not self.pool.can_alloc(need):
                        raise OutOfPages("pool")
                    seq.ensure(self.pool, len(req.prompt) + req.max_tokens + self.max_draft + 1)
                    st = SeqState(req, seq)
            except OutOfPages:
                self.stats["deferred"] += 1      # KV pressure defers, it does not reject
                if not self.active:
                    self.queue.popleft()
                    self._finish_unadmitted(req, "error: prompt does not fit the KV pool")
                    continue
                break
            except Exception as e:                # anything else is this request's failure, never the scheduler's
                self.queue.popleft()
                self.stats["rejected"] += 1
                self._finish_unadmitted(req, f"error: admission failed ({type(e).__name__}: {e})")
                continue
            self.queue.popleft()
            self.active.append(st)

    # ------------------------------------------------------------------ rounds
    def _prefill_round(self, states: list[SeqState]):
        rows, budget = [], min(self.prefill_chunk, self.runner.max_rows)
        for st in states:
            if budget <= 0:
                break
            take = min(len(st.req.prompt) - st.prefilled, budget)
            last = st.prefilled + take == len(st.req.prompt)
            rows.append(Row(st, st.req.prompt[st.prefilled:st.prefilled + take], st.prefilled, [take - 1] if last else []))
            budget -= take
        outs = self._run(rows)
        if outs is None:
            return
        for row, toks in zip(rows, outs):
            st = row.state
            st.prefilled += len(row.tokens)
            st.seq.length = st.prefilled
            self.stats["prefill_tokens"] += len(row.tokens)
            if st.cancelled:
                if self.prefix is not None:
                    self.prefix.park(st.req.prompt, st.seq)
                self._finish(st, "cancelled", capture=False)
                continue
            if row.want_logits:
                st.ttft = time.time() - st.req.arrived
                if self.prefix is not None and st.req.use_cache:
                    self.prefix.capture(st.req.prompt, st.seq, kind="prompt")
                self._emit(st, [toks[0]])

    def _decode_round(self, states: list[SeqState]):
        rows, budget = [], min(VERIFY_ROWS, self.runner.max_rows)
        plan = []
        plan_round = getattr(self.policy, "plan_round", None)      # policies that choose all requests' lengths jointly
        if plan_round is not None and self.drafter is not None:
            drafting = [st for st in states if st.req.allow_drafts]
            plan_round([st.req.rid for st in drafting], budget - (len(states) - len(drafting)),
                       room={st.req.rid: st.req.max_tokens - len(st.out) - 1 for st in drafting})
        for st in states:
            drafts = []
            # Sampled requests verify too: every verify row is sampled with the (seed, position) generator, and a draft is accepted
            # when it equals its row's sample.  With deterministic proposals that is exact speculative sampling - P(accept) = p(draft),
            # and a rejection emits a sample of p given "not the draft" - and it reproduces the undrafted token stream.
            # A grammar constraint masks every verify row with the state its own prefix (drafts included) leads to, so a draft the
            # grammar forbids simply fails to match.
            if self.drafter is not None and st.req.allow_drafts:
                width = self.policy.width(st.req.rid, budget - (len(states) - len(plan)))
                room = st.req.max_tokens - len(st.out) - 1
                if width > 0 and room > 0:
                    drafts = self.drafter.propose(st, min(width, room))
            if budget - (1 + len(drafts)) < len(states) - len(plan) - 1:
                drafts = []
            inputs = [st.pending] + drafts
            budget -= len(inputs)
            plan.append((st, inputs))
            rows.append(Row(st, inputs, st.seq.length, list(range(len(inputs)))))
        t0 = time.perf_counter()
        outs = self._run(rows)
        if outs is None:
            return
        step_ms = (time.perf_counter() - t0) * 1e3
        verified = []
        for (st, inputs), target in zip(plan, outs):
            remaining = st.req.max_tokens - len(st.out)
            accepted, emitted, _, _ = greedy_verify(inputs, target, st.req.eos_id, max(1, remaining))
            verified.append((st, accepted))
            st.seq.length += accepted
            self.stats["verify_rows"] += len(inputs)
            self.stats["drafted"] += len(inputs) - 1
            self.stats["accepted"] += accepted - 1
            for pos in range(min(len(inputs) - 1, len(self.accept_by_pos))):
                self.accept_by_pos[pos][0] += 1
                self.accept_by_pos[pos][1] += 1 if pos < accepted - 1 else 0
            if len(inputs) > 1:
                self.spec_trace.record(st.req.rid, len(inputs) - 1, accepted - 1, step_ms)
            self.policy.observe(st.req.rid, len(inputs) - 1, accepted - 1)
            self._emit(st, emitted)
        observe_round = getattr(self.policy, "observe_round", None)
        if observe_round is not None:
            observe_round(len(plan), sum(len(i) for _, i in plan), step_ms, widths={st.req.rid: len(i) - 1 for st, i in plan})
        commit = getattr(self.runner, "commit", None)
        if commit is not None:              # engines with recurrent layers absorb exactly the accepted rows now
            commit(verified)
        self._event("decode", rows=sum(len(i) for _, i in plan), seqs=len(plan), ms=round(step_ms, 3))

    def _run(self, rows: list[Row]):
        if not rows:
            return []
        try:
            self.stats["steps"] += 1
            with self.profile.phase("run"):
                return self.runner.run(rows)
        except Exception as e:  # a failed step fails the sequences in it, the server keeps going
            for r in rows:
                self.stats["failed"] += 1
                self._finish(r.state, f"error: {e}", capture=False)
            return None

    # ------------------------------------------------------------------ bookkeeping
    def _emit(self, st: SeqState, toks: list[int]):
        new = []
        for t in toks:
            if st.finished:
                break
            st.out.append(t)
            new.append(t)
            st.pending = t
            self.stats["generated"] += 1
            if st.req.eos_id is not None and t == st.req.eos_id:
                self._finish(st, "stop", new)
            elif t in st.req.stop_ids:
                self._finish(st, "stop", new)
            elif len(st.out) >= st.req.max_tokens:
                self._finish(st, "length", new)
        if not st.finished and st.cancelled:
            self._finish(st, "cancelled", new)
        elif not st.finished and new and st.req.on_token:
            try:
                st.req.on_token(new, False, None)
            except Exception as e:          # a broken client stream fails one request, never the batch
                self._finish(st, f"error: stream: {e}", capture=False)

    def _finish(self, st: SeqState, reason: str, new: list | None = None, capture: bool = True):
        if st.finished:
            return
        st.finished, st.reason = True, reason
        if capture and self.prefix is not None and st.req.use_cache and not reason.startswith("error"):
            toks = st.tokens[:st.seq.length]
            self.prefix.capture(toks, st.seq, kind="turn")
        if self.prefix is not None:
            self.prefix.release(st.seq)
        else:
            st.seq.release(self.pool)
        forget = getattr(self.runner, "forget", None)
        if forget is not None:
            forget(st)
        forget = getattr(self.policy, "forget", None)
        if forget is not None:
            forget(st.req.rid)
        self.stats["finished"] += 1
        self.recent.append({"rid": st.req.rid, "prompt": len(st.req.prompt), "generated": len(st.out), "cache_hit": st.cache_hit, "reason": reason})
        self._event("finish", rid=st.req.rid, reason=reason, generated=len(st.out))
        if st.req.on_token:
            try:
                st.req.on_token(new or [], True, reason)
            except Exception:
                pass

    def step(self) -> bool:
        """Returns False when there was nothing to do."""
        if self.fatal:
            return False
        with self.profile.phase("admit"):
            self._admit()
        self.active = [s for s in self.active if not s.finished]
        for s in self.active:
            if s.cancelled and s.prefilled == len(s.req.prompt):
                self._finish(s, "cancelled")
        self.active = [s for s in self.active if not s.finished]
        prefilling = [s for s in self.active if s.prefilled < len(s.req.prompt)]
        decoding = [s for s in self.active if s.prefilled == len(s.req.prompt) and s.pending is not None]
        if not prefilling and not decoding:
            return False
        # decode keeps a time share while prompts are being ingested (reference: prefill_share.rs:1-19)
        if prefilling and (not decoding or self._prefill_debt <= 0):
            self._prefill_round(prefilling)
            self._prefill_debt += self.decode_share / max(1e-6, 1.0 - self.decode_share)
        else:
            self._decode_round(decoding)
            self._prefill_debt -= 1.0
        self.active = [s for s in self.active if not s.finished]
        if self.prefix is not None:
            self.prefix.tick()
        return True

    def run_until_idle(self, max_steps: int = 100000):
        n = 0
        while n < max_steps and (self.step() or self.queue):
            n += 1
        return n

    def _event(self, kind: str, **fields):
        """Console events cost nothing while nobody watches (docs/dashboard.md:1-24 in the reference: producers skip
        work when there are no viewers)."""
        if self.watchers > 0:
            self.events.append(dict(fields, kind=kind, t=round(time.time(), 3), seq=self.stats["steps"]))

    def snapshot(self) -> dict:
        census = getattr(getattr(self.runner, "eng", None), "census", None)
        from ..utils.memory_ledger import LEDGER
        return dict(self.stats, active=len(self.active), queued=len(self.queue),
                    prefilling=sum(1 for s in self.active if s.prefilled < len(s.req.prompt)),
                    prefix=self.prefix.snapshot() if self.prefix else None, draft_policy=self.policy.snapshot(),
                    free_pages=self.pool.n_free, fatal=self.fatal, phases=self.profile.snapshot(), memory=LEDGER.report(),
                    draft_acceptance_by_position=[round(a / o, 3) if o else None for o, a in self.accept_by_pos],
                    graphs=census.snapshot() if census is not None else None)
