"""Parity of the fused CUDA TopK step (exact per-row selection, sparse decoder, auxiliary
dead-feature loss) with the reference: golden vectors and the CPU oracle.
Active-index sets must be bit-exact (away from exact value ties); losses and gradients
within 1e-4 relative in fp32 and 2e-2 in bf16."""
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


def dense_from_selection(mod):
    """[B, L, F] dense features rebuilt from the engine's (idx, val) lists."""
    ws = mod._engine.ws.buf
    idx, val = ws["idx"].long().cpu(), ws["val"].cpu()
    L, B, k = idx.shape
    F = mod.model.encoder.d_features
    dense = torch.zeros(L, B, F)
    dense.scatter_add_(2, idx, val)
    return dense.permute(1, 0, 2).contiguous()


def engine_pre(mod):
    """Pre-activations the selection saw: stored contraction output + bias, as [B, L, F] fp32."""
    z = mod._engine.ws.buf["z"].float().cpu()
    return (z + mod.model.encoder.b.detach().cpu().unsqueeze(1)).permute(1, 0, 2).contiguous()


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
def test_golden_topk_step(prec):
    g = load_golden(f"topk_clt_{prec}")
    spec = synthetic.WorkloadSpec(**g["spec"])
    dev = torch.device("cuda:0")
    mod = build_module(spec, g["weights"], dev, last_active=g["last_active_in"])
    batch = g["batch"].to(dev)
    mod.model.initialize_standardizers(batch)
    loss = run_step(mod, batch)
    tol = TOL[prec]
    feat = dense_from_selection(mod)
    if prec == "fp32":
        assert torch.equal(feat > 0, g["feat"] > 0)                   # index sets, bit-exact
        assert rel_err(feat, g["feat"]) < tol
    else:
        # same selector on the pre-activations this path produced: sets must agree exactly
        assert torch.equal(feat > 0, O.per_layer_topk(engine_pre(mod), spec.k) > 0)
        assert ((feat > 0) != (g["feat"] > 0)).float().mean() < 1e-3  # and almost always with the reference's
    assert torch.equal(mod.last_active.cpu(), g["last_active_out"])
    assert rel_err(loss.cpu(), g["loss"]) < tol
    assert rel_err(mod.logged["training/aux_loss"].cpu(), g["logged"]["training/aux_loss"]) < tol
    assert rel_err(mod.logged["metrics/dead_features"].cpu(), g["logged"]["metrics/dead_features"]) < 1e-6
    for a, b in zip(module_grad_list(mod), golden_grad_list(g)):
        assert rel_err(a.cpu(), b) < tol
    if prec == "fp32":
        opt = mod.configure_optimizers()
        opt.step()
        torch.cuda.synchronize()
        after = g["params_after_adam"]
        # the first Adam step moves every weight by about lr * sign(g); gradients near eps amplify rounding noise
        assert rel_err(mod.model.encoder.W.detach().cpu(), after["model.encoder.W"]) < 1e-4
        for t, w in enumerate(mod.model.decoder.blocks()):
            assert rel_err(w.detach().cpu(), after[f"model.decoder.W_{t}"]) < 1e-4


CASES = [
    # name, L, D, F, B, crosslayer, k, k_aux, dead_fraction
    ("clt", 4, 128, 1024, 300, True, 8, 32, 0.2),
    ("plt", 3, 192, 768, 200, False, 5, 16, 0.3),
    ("clt_no_dead", 2, 64, 256, 129, True, 4, 8, 0.0),
    ("clt_few_dead", 3, 64, 512, 150, True, 16, 64, 0.05),      # fewer dead features than k_aux
    ("clt_no_aux", 2, 64, 256, 100, True, 4, 0, 0.0),
    ("clt_wide", 2, 64, 4096, 130, True, 32, 64, 0.1),          # one warp per row, k = 32
    ("clt_wider", 2, 64, 16384, 70, True, 32, 64, 0.05),        # one CTA per row: the two-sweep selection path
]


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
@pytest.mark.parametrize("name,L,D,F,B,cross,k,k_aux,dead", CASES)
def test_oracle_topk_step(name, L, D, F, B, cross, k, k_aux, dead, prec):
    spec = synthetic.WorkloadSpec(name, L, D, F, B, "topk", cross, prec == "bf16", rank_u=16, n_outlier=2, k=k,
                                  k_aux=k_aux, aux_loss_scale=1 / 32, tokens_till_dead=1000, dead_fraction=dead,
                                  lr=1e-3)
    batch, w, la = spec_inputs(spec)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    ref, ref_grads = O.step_with_grads(P, batch, stats, H, **kw)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev, last_active=la)
    if k_aux == 0:
        mod.topk_aux.k = 0
    loss = run_step(mod, batch.to(dev), idx=0)
    tol = TOL[prec]
    feat = dense_from_selection(mod)
    if prec == "fp32":
        assert torch.equal(feat > 0, ref.feat > 0)
    else:
        assert torch.equal(feat > 0, O.per_layer_topk(engine_pre(mod), k) > 0)
    assert torch.equal(mod.last_active.cpu(), ref.last_active)
    assert rel_err(loss.cpu(), ref.loss) < tol
    for a, b in zip(module_grad_list(mod), ref_grads):
        assert rel_err(a.cpu(), b) < tol


def test_selection_edge_cases():
    """k = F keeps every positive value; all-negative rows keep nothing; k > F is an AssertionError
    (reference tests/test_topk.py:137-224)."""
    from crosslayer_transcoder_b200._lib import lib, stream_ptr

    dev = torch.device("cuda:0")
    lib().check_device()
    for L, B, F, ks in ((2, 5, 96, (1, 7, 96)), (2, 5, 4096, (1, 32, 256, 300, 4096)), (2, 9, 16384, (1, 32, 256, 300))):
        _check_selection(dev, L, B, F, ks)
    spec = synthetic.WorkloadSpec("kbig", 2, 64, 64, 16, "topk", True, False, rank_u=8, n_outlier=1, k=65, k_aux=0)
    batch, w, la = spec_inputs(spec)
    mod = build_module(spec, w, dev, last_active=la)
    with pytest.raises(AssertionError):
        mod.training_step(batch.to(dev), 0)


def _check_selection(dev, L, B, F, ks):
    from crosslayer_transcoder_b200._lib import lib, stream_ptr

    g = torch.Generator().manual_seed(0)
    z = torch.randn(L, B, F, generator=g)
    # a bias with a few large entries, in multiples of 2^-10 so that z = c - bias gives pre-activations exactly
    # equal to c
    bias_h = torch.round(0.05 * torch.randn(L, F, generator=g) * 1024) / 1024
    bias_h[:, ::97] += 0.75
    bias_h[0, 1] = -3.0
    z[1, 3] = -z[1, 3].abs() - 1.5                                   # an all-negative row, bias included
    z[0, 1, F // 2:] = -2.0                                          # positives in half of the row only
    z[0, 2] = torch.where(z[0, 2] > 0, 0.5 - bias_h[0], z[0, 2] - 1.0)   # masses of equal pre-activations
    zb = z.to(dev)
    bias = bias_h.to(dev)
    pre = z + bias_h.unsqueeze(1)
    for k in ks:
        idx = torch.empty(L, B, k, dtype=torch.int32, device=dev)
        val = torch.empty(L, B, k, device=dev)
        lib().call("clt_select_topk", zb, bias, idx, val, None, B, L, F, k, 0, stream_ptr())
        dense = torch.zeros(L, B, F).scatter_add_(2, idx.long().cpu(), val.cpu())
        ref = O.per_layer_topk(pre.permute(1, 0, 2).contiguous(), k).permute(1, 0, 2)
        tie_row = torch.zeros(L, B, dtype=torch.bool)
        tie_row[0, 2] = True                                         # which of the equal values win is unspecified
        assert torch.equal(dense[~tie_row], ref[~tie_row])
        assert torch.equal(dense[tie_row].sort(dim=-1).values, ref[tie_row].sort(dim=-1).values)
        assert (dense >= 0).all() and float(dense[1, 3].abs().sum()) == 0.0
        if F >= 2048 and k <= 256 and (F > 8192 or k > 64):
            # the one-sweep kernel hands the entries out as torch.topk does: largest value first (equal values
            # by feature), unused slots (value 0) last
            v, f = val.cpu(), idx.cpu()
            assert bool(((v[..., 1:] < v[..., :-1]) | ((v[..., 1:] == v[..., :-1]) &
                                                      ((f[..., 1:] > f[..., :-1]) | (v[..., 1:] == 0)))).all())
            tv, ti = torch.topk(pre[0, 0], k)
            assert torch.equal(v[0, 0], tv) and torch.equal(f[0, 0].long(), ti)
