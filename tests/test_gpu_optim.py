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


def test_a_second_optimizer_starts_from_zero_moments():
    """configure_optimizers() called again on a module that has trained: the new optimizer must not inherit the
    moments the first one left in the flat buffers (torch.optim.Adam's would not either)."""
    spec = _spec()
    batch, w, la = spec_inputs(spec)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    b = batch.to(dev)
    opt = mod.configure_optimizers()
    for i in range(2):
        opt.zero_grad()
        mod.training_step(b, i).backward()
        opt.step()
    opt2 = mod.configure_optimizers()
    opt2.zero_grad()
    mod.training_step(b, 2).backward()
    grads = [p.grad.detach().clone() for p in mod.parameters()]
    opt2.step()
    for p, g in zip(mod.parameters(), grads):
        st = opt2.state[p]
        assert int(st["step"]) == 1
        assert rel_err(st["exp_avg"], 0.1 * g) < 1e-5               # (1 - beta1) g: nothing carried over
        assert rel_err(st["exp_avg_sq"], 0.001 * g * g) < 1e-4


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


FUSED_CASES = [
    # kind, precision, d_acts  (a decoder row is split into 256-column parts; 520 and 2056 leave the last one ragged)
    ("topk", "fp32", 64), ("topk", "bf16", 64), ("batchtopk", "fp32", 64), ("batchtopk", "bf16", 64),
    ("topk", "fp32", 520), ("topk", "fp32", 2056), ("topk", "bf16", 2048), ("batchtopk", "bf16", 2048),
]


@pytest.mark.parametrize("kind,prec,D", FUSED_CASES)
def test_fused_optimizer_equals_separate_kernels(kind, prec, D):
    """module.fuse_optimizer applies Adam to the decoder inside the sparse backward.  After ONE step the
    decoder's parameters, moments and bf16 operand copy must be where the separate backward + optimizer
    kernels leave them to rounding (its gradient does not depend on the order of any atomic addition:
    dead features with an auxiliary gradient and features nobody selected included); after three steps
    everything must still agree to the accuracy the optimizer allows (the encoder gradient is summed by
    atomics whose order differs from run to run, and Adam turns differences of gradients near eps into
    differences of about lr / 100)."""
    bf16 = prec == "bf16"
    if kind == "topk":
        spec = synthetic.WorkloadSpec("fo", 3, D, 256, 90, "topk", True, bf16, rank_u=8, n_outlier=1, k=4, k_aux=16,
                                      aux_loss_scale=1 / 32, tokens_till_dead=500, dead_fraction=0.25, lr=1e-2)
    else:
        spec = synthetic.WorkloadSpec("fo", 3, D, 256, 90, "batchtopk", True, bf16, rank_u=8, n_outlier=1, k=3, e=0.1,
                                      lr=1e-2)
    batch, w, la = spec_inputs(spec)
    dev = torch.device("cuda:0")
    b = batch.to(dev)
    runs = []
    for fuse in (False, True):
        mod = build_module(spec, w, dev, last_active=la)
        mod.optimizer = "adamw" if D == 64 and kind == "topk" else "adam"
        mod.fuse_optimizer = fuse
        opt = mod.configure_optimizers()
        losses, first = [], None
        for i in range(3):
            opt.zero_grad()
            loss = mod.training_step(b, i)
            loss.backward()
            if fuse:
                assert all(wb.grad is None for wb in mod.model.decoder.blocks())
                assert mod.model.encoder.W.grad is not None
            opt.step()
            losses.append(float(loss.detach()))
            if i == 0:
                fp = mod._engine.flat
                o0 = fp.offsets[id(mod.model.decoder.blocks()[0])]
                o1 = o0 + sum(x.numel() for x in mod.model.decoder.blocks())
                first = dict(p=fp.flat[o0:o1].clone(), m=fp.exp_avg[o0:o1].clone(), v=fp.exp_avg_sq[o0:o1].clone(),
                             sh=None if fp.shadow is None else fp.shadow[o0:o1].float().clone())
        mod._engine.check_status()
        fp = mod._engine.flat
        runs.append(dict(losses=losses, first=first, p=fp.flat.clone(), m=fp.exp_avg.clone(), v=fp.exp_avg_sq.clone(),
                         sh=None if fp.shadow is None else fp.shadow.float().clone(),
                         la=mod.last_active.clone(), steps=[opt.state[p]["step"] for p in mod.parameters()]))
    a, f = runs
    # the decoder after one step: moments to rounding; parameters to what Adam allows (where |g| is near eps
    # the step lr g / (|g| + eps) turns the last bits of g into a visible difference, between two runs of
    # the separate kernels just as much)
    for key in ("m", "v"):          # (the order of a feature's entries, hence of the fp32 sums, varies from run to run)
        assert rel_err(f["first"][key], a["first"][key]) < (1e-4 if bf16 else 1e-5), key
    dp = (f["first"]["p"] - a["first"]["p"]).abs()
    assert float(dp.max()) < 5e-3 * spec.lr and float((dp > 1e-7).float().mean()) < 0.05
    assert a["losses"] == pytest.approx(f["losses"], rel=1e-5)
    assert torch.equal(a["la"], f["la"]) and a["steps"] == f["steps"] == [3] * len(a["steps"])
    for key in ("p", "m", "v"):
        assert rel_err(f[key], a[key]) < (1e-2 if bf16 else 1e-3), key
    if bf16:
        assert torch.equal(f["sh"], f["p"].bfloat16().float())      # the operand copy follows the master weights


def test_fused_optimizer_refuses_a_second_backward():
    spec = synthetic.WorkloadSpec("fo2", 2, 64, 256, 50, "topk", True, False, rank_u=8, n_outlier=1, k=4, k_aux=0)
    batch, w, la = spec_inputs(spec)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev, last_active=la)
    mod.topk_aux.k = 0
    mod.fuse_optimizer = True
    opt = mod.configure_optimizers()
    mod.training_step(batch.to(dev), 0).backward()
    with pytest.raises(RuntimeError, match="twice"):
        mod.training_step(batch.to(dev), 1).backward()
    opt.step()
    mod.training_step(batch.to(dev), 2).backward()      # after the optimizer step the next backward is fine
    opt.step()


def test_fp16_mixed_with_grad_scaler_runs_on_the_bf16_path():
    """The reference's default precision is ``16-mixed`` (fp16 autocast + GradScaler).  Under fp16 autocast the
    fused step computes with bf16 operands.  Against the reference arithmetic run in fp16 the loss must agree
    to the bf16 bar and the unscaled gradients to the bf16 rounding level (the two roundings differ, so their
    errors do not cancel as they do between two bf16 runs: 6e-2 of the largest entry); the scaler must find
    no inf / nan, and the step must train."""
    from oracle import clt_oracle as O
    from tests.helpers import oracle_for_spec

    spec = synthetic.WorkloadSpec("amp16", 3, 128, 512, 200, "jumprelu", True, True, rank_u=16, n_outlier=2,
                                  lambda_sparsity=4e-4, pre_actv_loss=3e-6, lr=1e-3)
    batch, w, la = spec_inputs(spec)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    H.bf16 = "fp16"
    ref, ref_grads = O.step_with_grads(P, batch, stats, H, **kw)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    mod.precision = "auto"
    opt = mod.configure_optimizers()
    scaler = torch.amp.GradScaler("cuda", init_scale=1024.0)
    b = batch.to(dev).half()
    before = mod.model.encoder.W.detach().clone()
    with torch.autocast("cuda", dtype=torch.float16):
        loss = mod.training_step(b, 0)
    scaler.scale(loss).backward()
    scaler.unscale_(opt)
    assert rel_err(loss.detach().cpu(), ref.loss) < 2e-2
    for a, g in zip(module_grad_list(mod), ref_grads):
        assert rel_err(a.cpu(), g) < 6e-2
    scaler.step(opt)
    scaler.update()
    assert scaler.get_scale() == 1024.0                       # no inf / nan was found
    assert not torch.equal(mod.model.encoder.W.detach(), before)
    mod._engine.check_status()
