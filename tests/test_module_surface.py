"""The module surface mirrors the reference's: selection semantics (reference tests/test_topk.py),
standardizer folding algebra (tests/test_standardization_folding.py), config / checkpoint round trip
(tests/test_save_to_pretrained.py, tests/test_load_from_pretrained.py).  CPU only: these are the eager
definitions used for inference-style calls and export, not the fused training step."""
import pytest
import torch

import crosslayer_transcoder_b200.model as M


@pytest.fixture(params=[(3, 4, 5), (1, 1, 5), (2, 8, 10), (1, 12, 768), (10, 1, 3)])
def features(request):
    return torch.rand(*request.param) + 0.1


def test_topk_counts_and_shapes(features):
    B, L, F = features.shape
    assert M.PerLayerTopK(k=3)(features).shape == features.shape
    assert int((M.PerLayerTopK(k=3)(features)[0, 0] != 0).sum()) == 3
    out = M.BatchTopK(k=3, e=0.1)(features)
    assert int((out != 0).sum()) == 3 * B * L
    out = M.PerLayerBatchTopK(k=3, e=0.1, n_layers=L)(features)
    for l in range(L):
        assert int((out[:, l] != 0).sum()) == 3 * B


def test_topk_known_answers():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]])
    assert torch.equal(M.PerLayerTopK(k=3)(x), torch.tensor([[[0.0, 0.0, 3.0, 4.0, 5.0]]]))
    y = torch.arange(1.0, 21.0).reshape(2, 2, 5)
    out = M.BatchTopK(k=3, e=0.1)(y)
    assert int((out != 0).sum()) == 12 and out.max() == 20 and (out == 19).any()


def test_topk_edges(features):
    B, L, F = features.shape
    for mod in (M.PerLayerTopK(k=0), M.BatchTopK(k=0, e=0.1), M.PerLayerBatchTopK(k=0, e=0.1, n_layers=L)):
        assert torch.equal(mod(features), torch.zeros_like(features))
    for mod in (M.PerLayerTopK(k=F), M.BatchTopK(k=F, e=0.1), M.PerLayerBatchTopK(k=F, e=0.1, n_layers=L)):
        assert torch.allclose(mod(features), features)
    for mod in (M.PerLayerTopK(k=F + 1), M.BatchTopK(k=F + 1, e=0.1), M.PerLayerBatchTopK(k=F + 1, e=0.1, n_layers=L)):
        with pytest.raises(AssertionError):
            mod(features)
    neg = -features
    for mod in (M.PerLayerTopK(k=2), M.BatchTopK(k=2, e=0.1), M.PerLayerBatchTopK(k=2, e=0.1, n_layers=L)):
        assert (mod(neg) >= 0).all()
    f = features.clone().requires_grad_(True)
    M.BatchTopK(k=2, e=0.1)(f).sum().backward()
    assert f.grad is not None


def test_batchtopk_inference_threshold():
    nl = M.BatchTopK(k=2, e=0.5)
    x = torch.rand(4, 3, 16) + 0.1
    nl(x)
    thr = float(nl.threshold)
    assert thr > 0
    out = nl(x, layer=1)
    assert torch.equal(out, torch.where(x > thr, x, torch.zeros_like(x)))


DT = torch.float64
B, D, F, L = 100, 48, 32, 5


def _model(decoder_cls):
    torch.manual_seed(0)
    m = M.CrossLayerTranscoder(M.ReLU(), M.Encoder(D, F, L), decoder_cls(D, F, L),
                               M.DimensionwiseInputStandardizer(L, D), M.DimensionwiseOutputStandardizer(L, D)).to(DT)
    with torch.no_grad():
        m.encoder.b.normal_()
        m.decoder.b.normal_()
    return m


@pytest.mark.parametrize("decoder_cls", [M.Decoder, M.CrosslayerDecoder])
def test_fold_equals_unfolded(decoder_cls):
    batch = torch.randn(B, 2, L, D, dtype=DT) * 3 + 1
    m = _model(decoder_cls)
    m.initialize_standardizers(batch)
    pre, feat, rn, recons = m(batch[:, 0])
    m.fold()
    assert m.input_standardizer is None and m._is_folded
    pre2, feat2, rn2, recons2 = m(batch[:, 0])
    assert torch.allclose(pre, pre2, rtol=1e-7, atol=1e-9)
    assert torch.allclose(recons, recons2, rtol=1e-7, atol=1e-9)     # folded decoder emits de-standardised output
    m.fold()                                                           # idempotent


def test_uninitialised_standardizer_raises():
    s = M.DimensionwiseInputStandardizer(2, 4)
    with pytest.raises(ValueError, match="Standardizer not initialized"):
        s(torch.zeros(3, 2, 4))


@pytest.mark.parametrize("decoder_cls", [M.Decoder, M.CrosslayerDecoder])
@pytest.mark.parametrize("nl", ["jumprelu", "relu", "topk", "batchtopk", "perlayer_batchtopk"])
def test_save_and_load_pretrained(tmp_path, decoder_cls, nl):
    nls = {"jumprelu": lambda: M.JumpReLU(theta=0.03, bandwidth=1.0, n_layers=3, d_features=16), "relu": M.ReLU,
           "topk": lambda: M.PerLayerTopK(k=4), "batchtopk": lambda: M.BatchTopK(k=4, e=0.1),
           "perlayer_batchtopk": lambda: M.PerLayerBatchTopK(k=4, e=0.1, n_layers=3)}
    m = M.CrossLayerTranscoder(nls[nl](), M.Encoder(8, 16, 3), decoder_cls(8, 16, 3),
                               M.DimensionwiseInputStandardizer(3, 8), M.DimensionwiseOutputStandardizer(3, 8))
    m.initialize_standardizers(torch.randn(20, 2, 3, 8))
    m.save_pretrained(tmp_path / "ckpt", fold_standardizers=False)
    assert (tmp_path / "ckpt" / "config.yaml").exists() and (tmp_path / "ckpt" / "checkpoint.safetensors").exists()
    m2 = M.CrossLayerTranscoder.from_pretrained(tmp_path / "ckpt")
    sd, sd2 = m.state_dict(), m2.state_dict()
    assert list(sd) == list(sd2)
    for k_ in sd:
        assert sd[k_].shape == sd2[k_].shape and torch.equal(sd[k_], sd2[k_]), k_
    names = set(sd)
    assert {"encoder.W", "encoder.b", "decoder.b"} <= names
    assert ("decoder.W_2" in names) == (decoder_cls is M.CrosslayerDecoder)
    cfg = m.to_config()
    assert cfg["class_path"].endswith("clt.CrossLayerTranscoder")
    assert cfg["init_args"]["encoder"]["init_args"] == {"d_acts": 8, "d_features": 16, "n_layers": 3}


def test_training_module_surface():
    m = M.CrossLayerTranscoder(M.JumpReLU(0.03, 1.0, 2, 8), M.Encoder(4, 8, 2), M.CrosslayerDecoder(4, 8, 2),
                               M.DimensionwiseInputStandardizer(2, 4), M.DimensionwiseOutputStandardizer(2, 4))
    mod = M.JumpReLUCrossLayerTranscoderModule(model=m, lambda_sparsity=1e-3, c_sparsity=0.5, pre_actv_loss=1e-5,
                                               learning_rate=1e-3, optimizer="adamw", beta1=0.8)
    assert mod.last_active.shape == (2, 8) and mod.last_active.dtype == torch.long
    assert [n for n, _ in mod.named_parameters()] == ["model.encoder.W", "model.encoder.b", "model.decoder.W_0",
                                                      "model.decoder.W_1", "model.decoder.b",
                                                      "model.nonlinearity.theta"]
    mod.optimizer = "sgd"
    with pytest.raises(ValueError, match="not supported"):
        mod.configure_optimizers()
    mod.optimizer, mod.warmup_steps = "adam", 10
    out = mod.configure_optimizers()
    assert out["lr_scheduler"]["name"] == "warmup" and out["lr_scheduler"]["interval"] == "step"
    with pytest.raises(RuntimeError):                       # no CPU fallback for the training step
        mod.training_step(torch.randn(6, 2, 2, 4), 0)
