"""N-gram memory on the GPU: the module's kernels against the oracle, and the decoder stack with engram layers end to end."""
import numpy as np
import pytest
import torch

from cuteafd_b200.config import tiny_spec
from cuteafd_b200.engine.engine import Engine
from cuteafd_b200.engine.generate import BatchGenerator, generate
from cuteafd_b200.models.weights import DeviceWeights
from cuteafd_b200.ref.engram import EngramAddressing, EngramSpec, context_hashes, engram_apply, init_engram_weights
from cuteafd_b200.ref.model import RefCache, RefModel, init_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("tables", ["device", "host"])
def test_engram_module_matches_oracle(tables):
    """Gather + dequantise (tables in device memory, or read in place from pinned host memory), projection, gate over four streams;
    masked (image) rows stay untouched."""
    from cuteafd_b200.models.engram import EngramModule
    spec = EngramSpec(layers=(1, 5), vocab=300, row_dim=256, prime_floor=150, streams=4, hidden=256)
    w = init_engram_weights(spec, 2)
    mod = EngramModule(spec, w, DEV, cap=64, tables=tables)
    assert mod.nbytes()["tables_on_device"] == (tables == "device")
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 300, (40,), generator=g).tolist()
    hashes = context_hashes(EngramAddressing(spec), toks[:3], toks[3:])           # 37 rows
    T = hashes.shape[1]
    mask = torch.ones(T, dtype=torch.bool)
    mask[5] = mask[20] = False
    x = (torch.randn(T, 4, 256, generator=g)).bfloat16()
    mod.set_hashes(hashes, mask)
    for e in range(2):
        xd = x.to(DEV).reshape(T, -1).contiguous()
        mod.apply(e, xd, T)
        torch.cuda.synchronize()
        mod.check_status()
        want = engram_apply(spec, w["layers"][e], x.float(), hashes[e], mask)
        got = xd.float().cpu().reshape(T, 4, 256)
        assert torch.equal(got[5], x[5].float()) and torch.equal(got[20], x[20].float())
        delta, wd = got - x.float(), want - x.float()
        err = float((delta - wd).norm() / wd.norm())
        assert err < 0.03, f"layer {e}: rel err of the added memory {err}"


def test_stack_with_engram_layers_matches_oracle_prefill_decode_and_graphs():
    spec = tiny_spec().replace(n_layers=3, engram_layers=(0, 2), engram_row_dim=64, engram_prime_floor=200)
    masters = init_weights(spec, 8)
    dw = DeviceWeights.from_masters(spec, masters, DEV)
    assert dw.engram is not None
    eng = Engine(dw, n_pages=32, max_seqs=8, max_pages_per_seq=4)
    ref = RefModel(spec, dw.dequantized_masters())
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (40, 27)]
    gen = BatchGenerator(eng, prefill_chunk=32)                   # chunk borders inside both prompts: the lookback crosses them
    gen.prefill(prompts)
    lane = eng.lane(32)
    torch.cuda.synchronize()
    eng.check_status()
    gen.release()
    out = generate(eng, prompts, 10)                              # decode steps replay a captured graph with fresh addresses each step
    plain = RefModel(spec.replace(engram_layers=()), dw.dequantized_masters())
    differs = False
    for i, p in enumerate(prompts):
        want, rows = ref.generate_greedy(torch.tensor(p), 10)
        other, _ = plain.generate_greedy(torch.tensor(p), 10)
        differs |= other != want
        for j, (a, b) in enumerate(zip(out[i], want)):
            if a != b:
                top2 = rows[j].topk(2).values
                assert float(top2[0] - top2[1]) < 0.05, f"prompt {i} step {j}: {a} != {b}"
                break
    assert differs, "the memory should change what this model generates"
    # teacher-forced logits of a whole prompt in one eager step
    gen = BatchGenerator(eng)
    gen.prefill([prompts[0]])
    torch.cuda.synchronize()
    rl, _ = ref.forward(torch.tensor(prompts[0]), 0, RefCache())
    got = eng.lane(len(prompts[0])).logits[0].float().cpu()
    assert float((got - rl[-1]).norm() / rl[-1].norm()) < 0.05
    gen.release()


def test_scheduler_serves_a_model_with_an_ngram_memory_with_drafts_and_prefix_reuse():
    from cuteafd_b200.engine.kv import PagePool
    from cuteafd_b200.serving.prefix import PrefixCache
    from cuteafd_b200.serving.runner import EngineRunner, attach_pool
    from cuteafd_b200.serving.scheduler import NgramDrafter, Request, Scheduler
    spec = tiny_spec().replace(engram_layers=(1,), engram_row_dim=64, engram_prime_floor=200)
    masters = init_weights(spec, 9)

    def build(drafter=None, prefix=False):
        eng = Engine(DeviceWeights.from_masters(spec, masters, DEV), n_pages=64, max_seqs=8, max_pages_per_seq=8)
        pool = PagePool(64)
        runner = attach_pool(EngineRunner(eng, max_rows=256), pool)
        return eng, Scheduler(runner, pool, max_seqs=4, prefill_chunk=48, drafter=drafter, prefix=PrefixCache(pool, min_tokens=64) if prefix else None)

    def run(sched, prompts, n):
        res = {}
        for i, p in enumerate(prompts):
            sched.submit(Request(f"r{i}", p, max_tokens=n, on_token=lambda t, d, r, i=i: res.setdefault(i, []).extend(t)))
        sched.run_until_idle()
        return [res[i] for i in range(len(prompts))]

    g = torch.Generator().manual_seed(13)
    base = torch.randint(0, spec.vocab, (10,), generator=g).tolist()
    shared = torch.randint(0, spec.vocab, (70,), generator=g).tolist()
    prompts = [base * 5, shared + base, shared + base[:4]]
    ref_eng, _ = build()
    want = generate(ref_eng, prompts, 12, use_graph=False)
    _, sched = build(drafter=NgramDrafter(), prefix=True)
    got = run(sched, prompts[:2], 12) + run(sched, prompts[2:], 12)          # the third request restores the shared prefix from the cache
    assert got == want
    assert sched.stats["drafted"] > 0 and sched.prefix.stats["hits"] >= 1
