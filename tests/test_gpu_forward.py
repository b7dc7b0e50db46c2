"""The inference forward (``module.forward`` without gradients) on the contraction kernels against the
model's own PyTorch forward, which follows the reference's ``CrossLayerTranscoder.forward``
(crosslayer_transcoder/model/clt.py:403-425)."""
import pytest
import torch

from crosslayer_transcoder_b200 import synthetic

from helpers import build_module, rel_err, spec_inputs

pytestmark = pytest.mark.gpu

CASES = [
    # name, L, D, F, B, crosslayer, kind, k
    ("clt_jumprelu", 3, 64, 192, 136, True, "jumprelu", 0),
    ("plt_jumprelu", 2, 96, 256, 77, False, "jumprelu", 0),
    ("clt_topk", 3, 64, 128, 50, True, "topk", 8),
    ("clt_batchtopk", 2, 64, 128, 64, True, "batchtopk", 4),
]


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
@pytest.mark.parametrize("name,L,D,F,B,cross,kind,k", CASES)
def test_kernel_forward_matches_model_forward(name, L, D, F, B, cross, kind, k, prec):
    bf16 = prec == "bf16"
    if bf16 and kind != "jumprelu":
        pytest.skip("selection sets of a bf16 run depend on the accumulation order; covered in fp32")
    dev = torch.device("cuda:0")
    spec = synthetic.WorkloadSpec(name, L, D, F, B, kind, cross, bf16, rank_u=8, n_outlier=1, k=k, k_aux=0)
    batch, w, la = spec_inputs(spec)
    mod = build_module(spec, w, dev, last_active=la)
    mod.model.initialize_standardizers(batch.to(dev))
    acts = batch[:, 0].to(dev)
    tol = 2e-2 if bf16 else 1e-4
    with torch.no_grad():
        got = mod(acts)
        if bf16:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                want = mod.model(acts)
        else:
            want = mod.model(acts)
    mod._engine.check_status("kernel forward")
    assert mod._engine.launches >= 2
    names = ("pre_actvs", "features", "recons_norm", "recons")
    for n, a, b in zip(names, got, want):
        assert a.shape == b.shape, n
        if n == "features" and bf16:
            # a pre-activation within rounding distance of its threshold may land on either side
            frac = float(((a > 0) != (b > 0)).float().mean())
            assert frac < 2e-3, (n, frac)
            continue
        assert rel_err(a.float(), b.float()) < tol, (n, rel_err(a.float(), b.float()))


def test_kernel_forward_needs_cuda_without_grad():
    """With gradients enabled, or on CPU tensors, forward is the model's differentiable PyTorch code."""
    dev = torch.device("cuda:0")
    spec = synthetic.WorkloadSpec("g", 2, 32, 64, 16, "jumprelu", True, False, rank_u=8, n_outlier=1)
    batch, w, la = spec_inputs(spec)
    mod = build_module(spec, w, dev, last_active=la)
    mod.model.initialize_standardizers(batch.to(dev))
    n0 = mod._engine.launches
    out = mod(batch[:, 0].to(dev))
    assert mod._engine.launches == n0 and out[3].requires_grad


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
@pytest.mark.parametrize("cross", [True, False], ids=["crosslayer", "per_layer"])
def test_forward_layer_runs_on_the_kernels(cross, prec):
    """``encoder(x, layer=i)`` / ``decoder(features, layer=i)`` (what the reference's replacement-model metric
    calls, crosslayer_transcoder/model/clt.py:134-145, 216-231, 304-317) on the contraction kernels against the
    eager definitions, with the reference's [batch, seq, ...] shapes."""
    bf16 = prec == "bf16"
    dev = torch.device("cuda:0")
    L, D, F = 3, 64, 192
    spec = synthetic.WorkloadSpec("fl", L, D, F, 8, "jumprelu", cross, bf16, rank_u=8, n_outlier=1)
    batch, w, la = spec_inputs(spec)
    mod = build_module(spec, w, dev, last_active=la)
    enc, dec = mod.model.encoder, mod.model.decoder
    g = torch.Generator().manual_seed(4)
    x = torch.randn(5, 7, D, generator=g).to(dev)
    tol = 2e-2 if bf16 else 1e-4
    n0 = mod._engine.launches
    for layer in (0, L - 1):
        got = enc(x, layer=layer)
        want = x @ enc.W[layer] + enc.b[layer]
        assert got.shape == want.shape and rel_err(got, want) < tol
        if cross:
            feats = torch.relu(torch.randn(5, 7, layer + 1, F, generator=g)).to(dev)
            want = torch.einsum("bqsf,sfd->bqd", feats, dec.get_parameter(f"W_{layer}")) + dec.b[layer]
        else:
            feats = torch.relu(torch.randn(5, 7, L, F, generator=g)).to(dev)
            want = feats[:, :, layer, :] @ dec.W[layer] + dec.b[layer]
        got = dec(feats, layer=layer)
        assert got.shape == want.shape and rel_err(got, want) < tol
    assert mod._engine.launches >= n0 + 10      # 2 layers x (3 encoder-side + 2 decoder-side) launches
    mod._engine.check_status("forward_layer")
    assert torch.equal(enc.cpu()(x.cpu(), layer=0), x.cpu() @ enc.W[0] + enc.b[0])      # CPU tensors: eager definition
