"""Where the reference tree is present (the development container), the oracle restatement and the
package's eager module definitions are compared with the UNMODIFIED reference modules on fresh seeded
inputs (beyond the committed golden vectors).  Skipped elsewhere."""
import pytest
import torch

from oracle import clt_oracle as O
from oracle import ref_import

pytestmark = pytest.mark.skipif(not ref_import.available(), reason="reference tree not present")


@pytest.fixture(scope="module")
def ref():
    return ref_import.load()


def test_selections_match(ref):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(7, 3, 40, generator=g)
    assert torch.equal(O.per_layer_topk(x, 6), ref.topk.PerLayerTopK(k=6)(x))
    r = ref.topk.BatchTopK(k=4, e=0.2)
    out, thr = O.batch_topk(x, 4, torch.zeros(1), 0.2)
    assert torch.equal(out, r(x)) and torch.allclose(thr, r.threshold)
    r = ref.topk.PerLayerBatchTopK(k=4, e=0.2, n_layers=3)
    out, thr = O.per_layer_batch_topk(x, 4, torch.zeros(3), 0.2)
    assert torch.equal(out, r(x)) and torch.allclose(thr, r.threshold)


def test_jumprelu_forward_backward_match(ref):
    g = torch.Generator().manual_seed(6)
    x = (torch.randn(9, 2, 16, generator=g) * 0.5).requires_grad_(True)
    x2 = x.detach().clone().requires_grad_(True)
    jr = ref.jumprelu.JumpReLU(theta=0.1, bandwidth=0.7, n_layers=2, d_features=16)
    theta = jr.theta.detach().clone().requires_grad_(True)
    w = torch.randn(9, 2, 16, generator=g)
    (jr(x) * w).sum().backward()
    (O.jumprelu(x2, theta, 0.7) * w).sum().backward()
    assert torch.equal(x.grad, x2.grad)
    assert torch.allclose(jr.theta.grad, theta.grad)


@pytest.mark.parametrize("cross", [True, False])
def test_package_modules_match_reference_forward(ref, cross):
    import crosslayer_transcoder_b200.model as M

    L, D, F, B = 3, 12, 20, 17
    torch.manual_seed(3)
    batch = torch.randn(B, 2, L, D) * 2 + 0.5
    rdec = (ref.clt.CrosslayerDecoder if cross else ref.clt.Decoder)(D, F, L)
    rm = ref.clt.CrossLayerTranscoder(ref.jumprelu.JumpReLU(0.05, 1.0, L, F), ref.clt.Encoder(D, F, L), rdec,
                                      ref.standardize.DimensionwiseInputStandardizer(L, D),
                                      ref.standardize.DimensionwiseOutputStandardizer(L, D))
    mine = M.CrossLayerTranscoder(M.JumpReLU(0.05, 1.0, L, F), M.Encoder(D, F, L),
                                  (M.CrosslayerDecoder if cross else M.Decoder)(D, F, L),
                                  M.DimensionwiseInputStandardizer(L, D), M.DimensionwiseOutputStandardizer(L, D))
    mine.load_state_dict(rm.state_dict())                     # same keys and shapes
    rm.initialize_standardizers(batch)
    mine.initialize_standardizers(batch)
    for a, b in zip(rm(batch[:, 0]), mine(batch[:, 0])):
        assert torch.allclose(a, b, rtol=1e-6, atol=1e-6)
    rm.fold()
    mine.fold()
    for (ka, a), (kb, b) in zip(rm.state_dict().items(), mine.state_dict().items()):
        assert ka == kb and torch.allclose(a, b, rtol=1e-6, atol=1e-7), ka
