"""Gated delta-rule linear attention (GDN: one decay per head; KDA: one per key channel) and the width-4 causal convolution in
front of it, against the fp32 statements in `ref.ops`: decode steps that continue a prefilled state, verify runs with
per-token state snapshots, ragged batches over state slots."""
import pytest
import torch

from cuteafd_b200.ops.native import call, ptr, stream
from cuteafd_b200.ref import ops as rops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("per_channel", [False, True])
def test_gated_delta_rule_matches_reference(per_channel):
    g = torch.Generator().manual_seed(8 + per_channel)
    H, n_slots = 3, 5
    lens = [9, 1, 4]                      # a short prefill run, a decode token, a verify run
    slots = [4, 0, 2]
    T = sum(lens)
    q = torch.nn.functional.normalize(torch.randn(T, H, 128, generator=g), dim=-1) * 128 ** -0.5
    k = torch.nn.functional.normalize(torch.randn(T, H, 128, generator=g), dim=-1)
    v = torch.randn(T, H, 128, generator=g)
    gate = torch.rand(T, H, 128, generator=g) * 0.3 + 0.7 if per_channel else torch.rand(T, H, generator=g) * 0.3 + 0.7
    beta = torch.rand(T, H, generator=g)
    state0 = torch.randn(n_slots, H, 128, 128, generator=g) * 0.1
    b16 = lambda t: t.to(torch.bfloat16)
    d = lambda t: t.to(DEV).contiguous()
    qd, kd, vd = d(b16(q)), d(b16(k)), d(b16(v))
    state = d(state0.clone())
    out = torch.zeros(T, H, 128, dtype=torch.bfloat16, device=DEV)
    snaps = torch.zeros(T, H, 128, 128, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    starts = [0, lens[0], lens[0] + lens[1]]
    i32 = lambda v_: torch.tensor(v_, dtype=torch.int32, device=DEV)
    d_slots, d_starts, d_lens = i32(slots), i32(starts), i32(lens)
    gd, bd = d(gate), d(beta)
    call("cuteafd_gated_delta_step", ptr(qd), ptr(kd), ptr(vd), ptr(gd), ptr(bd), ptr(state), ptr(d_slots), ptr(d_starts), ptr(d_lens),
         ptr(out), ptr(snaps), len(lens), H, 1 if per_channel else 0, n_slots, ptr(status), stream())
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    for s, (t0, n, slot) in enumerate(zip(starts, lens, slots)):
        rows = slice(t0, t0 + n)
        want, final, sn = rops.gated_delta_rule(b16(q[rows]).float(), b16(k[rows]).float(), b16(v[rows]).float(), gate[rows], beta[rows], state0[slot])
        got = out[rows].float().cpu()
        assert float((got - want).abs().max()) < 2e-2 * float(want.abs().max()) + 1e-3, f"sequence {s}"
        assert torch.allclose(state[slot].cpu(), final, atol=1e-4, rtol=1e-4)
        assert torch.allclose(snaps[t0 + n - 1].cpu(), final, atol=1e-4, rtol=1e-4) and torch.allclose(snaps[t0].cpu(), sn[0], atol=1e-4, rtol=1e-4)
    untouched = [i for i in range(n_slots) if i not in slots]
    assert torch.equal(state[untouched].cpu(), state0[untouched])


def test_short_conv4_carries_its_history():
    g = torch.Generator().manual_seed(3)
    C, n_slots = 384, 3
    x1, x2 = torch.randn(7, C, generator=g), torch.randn(2, C, generator=g)
    w = torch.randn(C, 4, generator=g) * 0.5
    b16 = lambda t: t.to(torch.bfloat16)
    carry = torch.zeros(n_slots, 3, C, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    i32 = lambda v_: torch.tensor(v_, dtype=torch.int32, device=DEV)
    wd = w.to(DEV)
    want1, c1 = rops.short_conv4(b16(x1).float(), w)
    want2, _ = rops.short_conv4(b16(x2).float(), w, b16(c1).float())
    for x, want in ((x1, want1), (x2, want2)):       # two calls on slot 1: the second continues from the carried inputs
        xd = b16(x).to(DEV)
        y = torch.zeros(x.shape[0], C, dtype=torch.bfloat16, device=DEV)
        d_slot, d_start, d_len = i32([1]), i32([0]), i32([x.shape[0]])
        call("cuteafd_short_conv4", ptr(xd), ptr(wd), ptr(carry), ptr(d_slot), ptr(d_start), ptr(d_len), ptr(y), 1, C, C, n_slots, ptr(status), stream())
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        assert float((y.float().cpu() - want).abs().max()) < 2e-2
    assert bool((carry[0] == 0).all()) and bool((carry[2] == 0).all())
