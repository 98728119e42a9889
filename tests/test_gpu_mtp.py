"""MTP speculative decoding on the GPU engine: lossless (same tokens as plain greedy decoding) and equal to the oracle."""
import pytest
import torch

from cuteafd_b200.config import tiny_spec
from cuteafd_b200.ref.model import RefModel, init_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _engine(spec, masters):
    from cuteafd_b200.engine.engine import Engine
    from cuteafd_b200.models.weights import DeviceWeights
    dw = DeviceWeights.from_masters(spec, masters, DEV)
    return dw, Engine(dw, n_pages=24, max_seqs=4, max_pages_per_seq=6)


@pytest.mark.parametrize("n_draft", [1, 3])
def test_mtp_speculative_equals_greedy_and_oracle(n_draft):
    from cuteafd_b200.engine.generate import generate
    from cuteafd_b200.engine.mtp import MtpSpeculator
    spec = tiny_spec().replace(mtp_layers=1)
    masters = init_weights(spec, seed=5)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (9, 17)]
    n_new = 12
    dw, eng = _engine(spec, masters)
    greedy = generate(eng, prompts, n_new, use_graph=False)
    spec_dec = MtpSpeculator(eng, n_draft=n_draft)
    out = spec_dec.generate(prompts, n_new)
    spec_dec.release()
    assert out == greedy
    assert all(len(s) == n_new for s in out)
    # oracle on the weights the GPU computes with
    ref = RefModel(spec, dw.dequantized_masters())
    for p, o in zip(prompts, out):
        want, _ = ref.generate_speculative(torch.tensor(p), n_new, n_draft)
        assert o == want
