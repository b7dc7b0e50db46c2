"""Optimizer and loss-scaling behaviour of the fused step on the GPU: AdamW and the LR schedules of the
reference's configure_optimizers (clt_lightning.py:333-392) against torch.optim on the CPU, and a scaled
backward (what a GradScaler does) against the unscaled one."""
import pytest
import torch

from crosslayer_transcoder_b200 import synthetic
from tests.helpers import build_module, module_grad_list, rel_err, spec_inputs

pytestmark = pytest.mark.gpu


def _spec(**kw):
    return synthetic.WorkloadSpec("opt", 2, 64, 256, 120, "jumprelu", True, False, rank_u=8, n_outlier=1,
                                  lambda_sparsity=1e-4, pre_actv_loss=3e-6, lr=1e-2, **kw)


@pytest.mark.parametrize("optimizer", ["adam", "adamw"])
def test_three_steps_match_torch_optim(optimizer):
    spec = _spec()
    batch, w, la = spec_inputs(spec)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    mod.optimizer, mod.lr_decay_step, mod.lr_decay_factor = optimizer, 2, 0.1      # one LR drop after step 2
    cfg = mod.configure_optimizers()
    opt, sched = cfg["optimizer"], cfg["lr_scheduler"]["scheduler"]
    # CPU twin driven by the gradients the fused step produced
    twins = [p.detach().cpu().clone().requires_grad_(True) for p in mod.parameters()]
    topt = (torch.optim.AdamW if optimizer == "adamw" else torch.optim.Adam)(twins, lr=spec.lr, betas=(0.9, 0.999))
    tsched = torch.optim.lr_scheduler.MultiStepLR(topt, milestones=[2], gamma=0.1)
    b = batch.to(dev)
    for i in range(3):
        opt.zero_grad()
        loss = mod.training_step(b, i)
        loss.backward()
        for t, p in zip(twins, mod.parameters()):
            t.grad = p.grad.detach().cpu().clone()
        opt.step()
        sched.step()
        topt.step()
        tsched.step()
    assert opt.param_groups[0]["lr"] == pytest.approx(spec.lr * 0.1)
    for t, p in zip(twins, mod.parameters()):
        assert rel_err(p.detach().cpu(), t.detach()) < 1e-5


def test_scaled_backward_scales_every_gradient():
    spec = _spec()
    batch, w, la = spec_inputs(spec)
    dev = torch.device("cuda:0")
    b = batch.to(dev)
    grads = []
    for scale in (1.0, 1024.0):
        mod = build_module(spec, w, dev)
        loss = mod.training_step(b, 0)
        (loss * scale).backward()
        grads.append([g.detach().cpu().clone() for g in module_grad_list(mod)])
    for g1, g2 in zip(*grads):
        assert rel_err(g2 / 1024.0, g1) < 1e-5


def test_gradient_accumulation_keeps_earlier_gradients():
    """A second backward on ANOTHER batch without zero_grad adds to the first.  After the first backward
    every .grad is its slice of the flat gradient buffer, which the second backward's kernels overwrite:
    the step must carry the earlier values over."""
    spec = _spec()
    batch, w, la = spec_inputs(spec)
    batch2, _, _ = spec_inputs(spec, seed=77)
    dev = torch.device("cuda:0")
    b1, b2 = batch.to(dev), batch2.to(dev)
    singles = []
    for b in (b1, b2):
        mod = build_module(spec, w, dev)
        mod.model.initialize_standardizers(b1)
        mod.training_step(b, 1).backward()
        singles.append([g.detach().clone() for g in module_grad_list(mod)])
    assert rel_err(singles[1][0], singles[0][0]) > 1e-2          # the two batches give different gradients
    mod = build_module(spec, w, dev)
    mod.model.initialize_standardizers(b1)
    mod.training_step(b1, 1).backward()
    mod.training_step(b2, 2).backward()
    for a, g1, g2 in zip(module_grad_list(mod), *singles):
        assert rel_err(a, g1 + g2) < 1e-5
    # the accumulated gradients still sit in the flat buffer, so the one-launch Adam path stays available
    opt = mod.configure_optimizers()
    assert opt._flat_ready(opt.param_groups[0])


def test_zero_grad_in_place_does_not_double_count():
    """zero_grad(set_to_none=False) leaves zero-filled .grad tensors that alias the flat buffer; the next
    backward must produce G, not 2 G."""
    spec = _spec()
    batch, w, la = spec_inputs(spec)
    dev = torch.device("cuda:0")
    b = batch.to(dev)
    mod = build_module(spec, w, dev)
    opt = mod.configure_optimizers()
    mod.training_step(b, 0).backward()
    g1 = [g.detach().clone() for g in module_grad_list(mod)]
    opt.zero_grad(set_to_none=False)
    mod.training_step(b, 1).backward()
    for a, g in zip(module_grad_list(mod), g1):
        assert rel_err(a, g) < 1e-5
