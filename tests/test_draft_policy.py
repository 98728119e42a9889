"""Online resource-priced draft policy: the fits, the joint choice of verification lengths, calibration, skipping and the scheduler hooks."""
import random

from cuteafd_b200.engine.kv import PagePool
from cuteafd_b200.serving.draft_policy import OnlineDraftPolicy, _Fit, concurrency_bucket
from cuteafd_b200.serving.runner import FakeRunner
from cuteafd_b200.serving.scheduler import NgramDrafter, Request, Scheduler


def test_buckets_and_fit_recover_a_cost_model_and_shrug_off_outliers():
    assert [concurrency_bucket(n) for n in (1, 2, 4, 5, 8, 9, 64)] == [0, 1, 1, 2, 2, 3, 3]
    rng = random.Random(0)
    fit = _Fit((20.0, 0.05, 0.5))
    for i in range(400):
        rows, mb = rng.randint(1, 64), rng.uniform(0, 40)
        y = 8.0 + 0.2 * rows + 0.1 * mb + rng.gauss(0, 0.05)
        if i % 50 == 49:
            y += 200.0                               # a stall: one sample in fifty is far off
        fit.update((1.0, float(rows), mb), y)
    assert abs(fit.theta[0] - 8.0) < 1.5 and abs(fit.theta[1] - 0.2) < 0.03 and abs(fit.theta[2] - 0.1) < 0.03
    assert abs(fit.predict((1.0, 32.0, 10.0)) - (8.0 + 6.4 + 1.0)) < 1.0


def _warm(policy, n_requests, rows, ms, rounds=16):
    for _ in range(rounds):
        policy.observe_round(n_requests, rows, ms)


def test_lengths_follow_acceptance_and_cost():
    cheap = OnlineDraftPolicy(max_width=6, prior_ms=(20.0, 0.05, 0.0))
    _warm(cheap, 2, 2, 20.1)
    _warm(cheap, 2, 14, 20.7)
    plan = cheap.plan_round(["a", "b"], 64)
    assert plan == {"a": 6, "b": 6}                     # rows are nearly free next to the fixed cost: draft as far as allowed
    dear = OnlineDraftPolicy(max_width=6, prior_ms=(1.0, 4.0, 0.0), prior_accept=0.3)
    for _ in range(8):
        dear.observe_round(2, 2, 9.0)
        dear.observe_round(2, 8, 33.0)
    assert sum(dear.plan_round(["a", "b"], 64).values()) <= 1      # every row costs as much as the round: drafting loses
    # a request whose drafts are accepted drafts longer than one whose drafts fail, inside the same round
    mixed = OnlineDraftPolicy(max_width=6, prior_ms=(10.0, 0.6, 0.0))
    _warm(mixed, 2, 2, 11.2)
    _warm(mixed, 2, 10, 16.0)
    for _ in range(6):
        mixed.observe("good", 4, 4)
        mixed.observe("bad", 4, 1)
        mixed.observe_round(2, 10, 16.0)
    plan = mixed.plan_round(["good", "bad"], 64, room={"good": 10, "bad": 10})
    assert plan["good"] > plan["bad"]
    assert mixed.plan_round(["good", "bad"], 64, room={"good": 2, "bad": 10})["good"] <= 2       # never past what the request may emit
    assert sum(mixed.plan_round(["good", "bad"], 4).values()) <= 2                                 # the shared row budget binds


def test_requests_that_keep_failing_are_skipped_and_probed():
    p = OnlineDraftPolicy(max_width=4, prior_ms=(20.0, 0.05, 0.0), explore_skips=4)
    _warm(p, 1, 1, 20.0)
    _warm(p, 1, 5, 20.3)
    for _ in range(5):
        p.observe("r", 4, 0)
        p.observe_round(1, 5, 20.3)
    widths = [p.plan_round(["r"], 64)["r"] for _ in range(8)]
    assert widths.count(0) == 6 and sum(1 for w in widths if w > 0) == 2          # one probe every four rounds
    p.observe("r", 2, 2)
    p.observe("r", 2, 2)
    p.observe("r", 2, 2)
    assert p.plan_round(["r"], 64)["r"] > 0                                        # accepted probes bring the request back
    p.forget("r")
    assert "r" not in p.recent and "r" not in p.skips


def test_route_forecast_prices_shared_experts_once():
    p = OnlineDraftPolicy(max_width=4, n_experts=16, top_k=2, slice_mb=10.0, group_rows=16, prior_ms=(5.0, 0.0, 1.0))
    p.observe_routes("a", [{1, 2}] * 8)
    p.observe_routes("b", [{1, 2}] * 8)
    p.observe_routes("c", [{i % 16, (i + 5) % 16} for i in range(8)])
    same = p.expert_megabytes({"a": 3, "b": 3})            # both requests keep hitting experts 1 and 2: two slices, read once
    assert same == 20.0
    spread = p.expert_megabytes({"a": 3, "c": 3})
    assert spread > same
    assert p.expert_megabytes({"zzz": 3}) == 0.0           # no route history: the term is off
    _warm(p, 2, 2, 25.0, rounds=13)
    # with traffic priced, lengthening the request that wanders over the experts costs more than lengthening the one that stays put
    base = {"a": 1, "c": 1}
    assert p.predict_ms({"a": 1, "c": 3}) > p.predict_ms({"a": 3, "c": 1})
    assert base == {"a": 1, "c": 1}


def test_scheduler_drives_the_policy_and_stays_lossless():
    def build(policy=None, drafter=None):
        runner = FakeRunner(vocab=64)
        runner.next_token = lambda prefix: (prefix[-1] * 7 + prefix[-2] * 3 + 1) % 11          # a short cycle: n-gram drafts hit often
        return Scheduler(runner, PagePool(256), max_seqs=4, drafter=drafter, policy=policy, max_draft=6)

    def run(sched, prompts, n):
        out = {}
        for i, p in enumerate(prompts):
            sched.submit(Request(f"r{i}", p, max_tokens=n, on_token=lambda t, d, r, i=i: out.setdefault(i, []).extend(t)))
        sched.run_until_idle()
        return [out[i] for i in range(len(prompts))]

    prompts = [[1, 2, 3, 4, 5], [5, 4, 3], [2, 2, 9, 1]]
    want = run(build(), prompts, 60)
    policy = OnlineDraftPolicy(max_width=6, warm_rounds=4)
    sched = build(policy, NgramDrafter())
    got = run(sched, prompts, 60)
    assert got == want
    snap = policy.snapshot()
    assert snap["rounds"] > 4 and snap["drafted"] > 0 and sched.stats["drafted"] == snap["drafted"]
    assert any(f["samples"] > 0 for f in snap["fit"]) and not policy.recent           # finished requests were forgotten
    assert sched.snapshot()["draft_policy"]["kind"] == "online-resource-priced"
