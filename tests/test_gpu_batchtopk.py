"""Parity of the fused CUDA BatchTopK step (one batch-wide threshold from a histogram select,
per-layer entry lists, sparse decoder) with the reference: golden vectors and the CPU oracle."""
import pytest
import torch

from crosslayer_transcoder_b200 import synthetic
from oracle import clt_oracle as O
from tests.helpers import (build_module, golden_grad_list, load_golden, module_grad_list, oracle_for_spec, rel_err,
                           spec_inputs)

pytestmark = pytest.mark.gpu
TOL = {"fp32": 1e-4, "bf16": 2e-2}


def run_step(mod, batch, idx=1):
    loss = mod.training_step(batch, idx)
    loss.backward()
    mod._engine.check_status("after backward")
    return loss


def dense_from_lists(mod, B):
    """[B, L, F] dense features rebuilt from the engine's per-layer entry lists."""
    ws = mod._engine.ws.buf
    idx, val, tok = ws["bt_idx"].long().cpu(), ws["bt_val"].cpu(), ws["bt_tok"].long().cpu()
    L = idx.shape[0]
    F = mod.model.encoder.d_features
    dense = torch.zeros(B, L, F)
    for l in range(L):
        m = val[l] != 0
        dense[tok[l][m], l, idx[l][m]] = val[l][m]
    return dense


def engine_pre(mod):
    z = mod._engine.ws.buf["z"].float().cpu()
    return (z + mod.model.encoder.b.detach().cpu().unsqueeze(1)).permute(1, 0, 2).contiguous()


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
def test_golden_batchtopk_step(prec):
    g = load_golden(f"batchtopk_clt_{prec}")
    spec = synthetic.WorkloadSpec(**g["spec"])
    dev = torch.device("cuda:0")
    mod = build_module(spec, g["weights"], dev)
    batch = g["batch"].to(dev)
    mod.model.initialize_standardizers(batch)
    loss = run_step(mod, batch)
    tol = TOL[prec]
    feat = dense_from_lists(mod, spec.batch)
    n_keep = spec.k * spec.batch * spec.n_layers
    if prec == "fp32":
        assert int((feat != 0).sum()) == n_keep                      # exactly k B L survivors (tests/test_topk.py:63-74)
        assert torch.equal(feat > 0, g["feat"] > 0)
        assert rel_err(feat, g["feat"]) < tol
    else:
        ref_sel, _ = O.batch_topk(engine_pre(mod), spec.k, torch.zeros(1), spec.e)
        assert torch.equal(feat > 0, ref_sel > 0)                    # same selector on this path's pre-activations
    assert rel_err(mod.model.nonlinearity.threshold.cpu(), g["threshold_out"]) < tol
    assert torch.equal(mod.last_active.cpu(), g["last_active_out"])
    assert rel_err(loss.cpu(), g["loss"]) < tol
    for a, b in zip(module_grad_list(mod), golden_grad_list(g)):
        assert rel_err(a.cpu(), b) < tol


CASES = [
    # name, L, D, F, B, crosslayer, k
    ("clt", 4, 128, 1024, 300, True, 4),
    ("plt", 3, 192, 768, 200, False, 6),
    ("clt_k1", 2, 64, 4096, 100, True, 1),
]


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
@pytest.mark.parametrize("name,L,D,F,B,cross,k", CASES)
def test_oracle_batchtopk_step(name, L, D, F, B, cross, k, prec):
    spec = synthetic.WorkloadSpec(name, L, D, F, B, "batchtopk", cross, prec == "bf16", rank_u=16, n_outlier=2, k=k,
                                  e=0.05, lr=1e-3)
    batch, w, la = spec_inputs(spec)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    ref, ref_grads = O.step_with_grads(P, batch, stats, H, **kw)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    loss = run_step(mod, batch.to(dev), idx=0)
    tol = TOL[prec]
    feat = dense_from_lists(mod, B)
    if prec == "fp32":
        assert torch.equal(feat > 0, ref.feat > 0)
    else:
        ref_sel, _ = O.batch_topk(engine_pre(mod), k, torch.zeros(1), spec.e)
        assert torch.equal(feat > 0, ref_sel > 0)
    assert rel_err(mod.model.nonlinearity.threshold.cpu(), ref.threshold) < tol
    assert rel_err(loss.cpu(), ref.loss) < tol
    for a, b in zip(module_grad_list(mod), ref_grads):
        assert rel_err(a.cpu(), b) < tol
    # a second step moves the threshold's running average on; its first histogram pass starts from half of
    # the previous threshold
    thr1 = float(mod.model.nonlinearity.threshold)
    run_step(mod, batch.to(dev), idx=1)
    assert float(mod.model.nonlinearity.threshold) > thr1
    sel, _ = O.batch_topk(engine_pre(mod), k, torch.zeros(1), spec.e)
    assert torch.equal(dense_from_lists(mod, B) > 0, sel > 0)
    # a much quieter batch: the guessed floor is now too high and the selection must fall back to the full range
    run_step(mod, (0.2 * batch).to(dev), idx=2)
    sel, _ = O.batch_topk(engine_pre(mod), k, torch.zeros(1), spec.e)
    got = dense_from_lists(mod, B)
    assert int((got != 0).sum()) == k * B * L
    assert torch.equal(got > 0, sel > 0)


def test_batchtopk_edge_cases():
    """k = 0 keeps nothing (reference tests/test_topk.py:137-148); more slots than positive values keeps
    every positive one and leaves the threshold's running average fed with 0."""
    dev = torch.device("cuda:0")
    spec = synthetic.WorkloadSpec("k0", 2, 64, 256, 50, "batchtopk", True, False, rank_u=8, n_outlier=1, k=0, e=0.1)
    batch, w, la = spec_inputs(spec)
    mod = build_module(spec, w, dev)
    loss = run_step(mod, batch.to(dev), idx=0)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    ref, _ = O.step_with_grads(P, batch, stats, H, **kw)
    assert rel_err(loss.cpu(), ref.loss) < 1e-4
    spec = synthetic.scaled(spec, name="kall", k=200)                 # 200 of 256 per row: more than the positives
    mod = build_module(spec, w, dev)
    loss = run_step(mod, batch.to(dev), idx=0)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    ref, ref_grads = O.step_with_grads(P, batch, stats, H, **kw)
    assert torch.equal(dense_from_lists(mod, spec.batch) > 0, ref.feat > 0)
    assert rel_err(loss.cpu(), ref.loss) < 1e-4
    assert float(mod.model.nonlinearity.threshold) == 0.0
    for a, b in zip(module_grad_list(mod), ref_grads):
        assert rel_err(a.cpu(), b) < 1e-4


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
def test_oracle_perlayer_batchtopk_step(prec):
    """PerLayerBatchTopK (reference topk.py:99-133): the same selection, one threshold per layer."""
    L, B, F, k = 4, 150, 1024, 3
    spec = synthetic.WorkloadSpec("plbtk", L, 128, F, B, "perlayer_batchtopk", True, prec == "bf16", rank_u=16,
                                  n_outlier=2, k=k, e=0.05, lr=1e-3)
    batch, w, la = spec_inputs(spec)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    ref, ref_grads = O.step_with_grads(P, batch, stats, H, **kw)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    loss = run_step(mod, batch.to(dev), idx=0)
    tol = TOL[prec]
    feat = dense_from_lists(mod, B)
    if prec == "fp32":
        assert torch.equal(feat > 0, ref.feat > 0)
        for l in range(L):
            assert int((feat[:, l] != 0).sum()) == k * B            # k B survivors in every layer
    else:
        ref_sel, _ = O.per_layer_batch_topk(engine_pre(mod), k, torch.zeros(L), spec.e)
        assert torch.equal(feat > 0, ref_sel > 0)
    assert rel_err(mod.model.nonlinearity.threshold.cpu(), ref.threshold) < tol
    assert rel_err(loss.cpu(), ref.loss) < tol
    for a, b in zip(module_grad_list(mod), ref_grads):
        assert rel_err(a.cpu(), b) < tol
