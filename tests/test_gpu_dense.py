"""Parity of the fused CUDA training step (JumpReLU / ReLU, dense decoder) with the
reference: golden vectors made from the unmodified reference, and the CPU oracle on
larger seeded cases.  Tolerances are the parity bar: 1e-4 relative in fp32, 2e-2 in bf16."""
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


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
@pytest.mark.parametrize("case", ["jumprelu_clt", "jumprelu_plt"])
def test_golden_step(case, prec):
    g = load_golden(f"{case}_{prec}")
    spec = synthetic.WorkloadSpec(**g["spec"])
    dev = torch.device("cuda:0")
    mod = build_module(spec, g["weights"], dev)
    mod.fuse_activation = True
    batch = g["batch"].to(dev)
    mod.model.initialize_standardizers(batch)
    for name, ref in (("mean", g["stats"]["mu_in"]), ("std", g["stats"]["sd_in"])):
        assert rel_err(getattr(mod.model.input_standardizer, name).cpu(), ref) < 1e-5
    loss = run_step(mod, batch)
    tol = TOL[prec]
    assert rel_err(loss.cpu(), g["loss"]) < tol
    for name, a, b in zip(["W_enc", "b_enc"] + ["W_dec"] * len(mod.model.decoder.blocks()) + ["b_dec", "theta"],
                          module_grad_list(mod), golden_grad_list(g)):
        assert a is not None, name
        assert rel_err(a.cpu(), b) < tol, name
    assert torch.equal(mod.last_active.cpu(), g["last_active_out"])     # dead-feature counters, bit-exact
    if prec == "fp32":
        opt = mod.configure_optimizers()
        opt.step()
        torch.cuda.synchronize()
        after = g["params_after_adam"]
        assert rel_err(mod.model.encoder.W.detach().cpu(), after["model.encoder.W"]) < 1e-5
        assert rel_err(mod.model.nonlinearity.theta.detach().cpu(), after["model.nonlinearity.theta"]) < 1e-5
        for t, w in enumerate(mod.model.decoder.blocks()):
            key = f"model.decoder.W_{t}" if spec.crosslayer else "model.decoder.W"
            assert rel_err(w.detach().cpu(), after[key]) < 1e-5


SPECS = [
    # name, L, D, F, B, crosslayer, lambda, pre_actv
    ("clt_ragged", 4, 128, 512, 300, True, 4e-4, 3e-6),
    ("plt_ragged", 3, 192, 768, 333, False, 2e-4, 3e-6),
    ("clt_nolambda", 2, 64, 256, 129, True, 0.0, 0.0),
]


@pytest.mark.parametrize("fuse", [True, False], ids=["fused_epilogue", "split_activation"])
@pytest.mark.parametrize("prec", ["fp32", "bf16"])
@pytest.mark.parametrize("name,L,D,F,B,cross,lam,pal", SPECS)
def test_oracle_step(name, L, D, F, B, cross, lam, pal, prec, fuse):
    spec = synthetic.WorkloadSpec(name, L, D, F, B, "jumprelu", cross, prec == "bf16", rank_u=16, n_outlier=2,
                                  lambda_sparsity=lam, pre_actv_loss=pal, lr=1e-3)
    batch, w, la = spec_inputs(spec)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    ref, ref_grads = O.step_with_grads(P, batch, stats, H, **kw)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    mod.fuse_activation = fuse                          # both forms of the (Jump)ReLU: in the epilogues or streamed
    loss = run_step(mod, batch.to(dev), idx=0)          # idx 0: the step initialises the standardizers itself
    tol = TOL[prec]
    assert rel_err(loss.cpu(), ref.loss) < tol
    terms = mod._engine.last_terms.cpu()
    assert rel_err(terms[0], ref.terms["mse"]) < tol
    if lam:
        assert rel_err(terms[1], ref.terms["sparsity"]) < tol
    if pal:
        assert rel_err(terms[2], ref.terms["pre_actv"]) < tol
    for a, b in zip(module_grad_list(mod), ref_grads):
        assert rel_err(a.cpu(), b) < tol


def test_relu_kind_matches_oracle():
    spec = synthetic.WorkloadSpec("relu", 2, 64, 256, 150, "relu", True, False, rank_u=16, n_outlier=2, lr=1e-3)
    batch, w, la = spec_inputs(spec)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    H.kind = "relu"
    ref, ref_grads = O.step_with_grads(P, batch, stats, H)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    loss = run_step(mod, batch.to(dev), idx=0)
    assert rel_err(loss.cpu(), ref.loss) < 1e-4
    for a, b in zip(module_grad_list(mod), ref_grads):
        assert rel_err(a.cpu(), b) < 1e-4


def test_fp16_batch_and_two_steps_train():
    """A half-precision batch (the reference's activation dtype) and two full steps: the loss goes down
    and the bf16 operand copy follows the optimizer."""
    spec = synthetic.WorkloadSpec("two_steps", 3, 64, 256, 200, "jumprelu", True, True, rank_u=16, n_outlier=2,
                                  lambda_sparsity=1e-4, pre_actv_loss=3e-6, lr=1e-2)
    batch, w, la = spec_inputs(spec)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    opt = mod.configure_optimizers()
    b16 = batch.to(dev).half()
    losses = []
    for i in range(3):
        opt.zero_grad()
        loss = mod.training_step(b16, i)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    mod._engine.check_status()
    assert losses[2] < losses[0]
    fp = mod._engine.flat
    assert rel_err(fp.shadow.float().cpu(), fp.flat.cpu()) < 1e-2
    # the reference keeps the dead-feature counters for every module kind
    assert int(mod.last_active.max()) <= 3 * spec.batch


def test_missing_gpu_path_raises():
    spec = synthetic.WorkloadSpec("cpu", 2, 64, 64, 8, "jumprelu", True, False, rank_u=8, n_outlier=1)
    batch, w, la = spec_inputs(spec)
    mod = build_module(spec, w, torch.device("cpu"))
    with pytest.raises(RuntimeError):
        mod.training_step(batch, 0)
