"""Generate the golden vectors under ``tests/golden/`` by running the UNMODIFIED
reference modules (imported with ``oracle/ref_import.py``) on seeded inputs.

Run where the reference tree is present:

    python tests/golden/make_golden.py

Each ``<case>.pt`` holds the case's spec, its inputs (batch, weights, state) and
what the reference's ``training_step`` + ``backward`` + one ``Adam`` step gave:
loss, pre-activations, features, normalised reconstruction, every parameter's
gradient and the parameters after the optimizer step.
"""
from __future__ import annotations

import contextlib
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from crosslayer_transcoder_b200 import synthetic  # noqa: E402
from oracle import ref_import  # noqa: E402  (only main() needs the reference)
from oracle.ref_step import build_reference_module  # noqa: E402

HERE = Path(__file__).resolve().parent


def cases():
    base = dict(n_layers=3, d_acts=64, d_features=64, batch=136, rank_u=8, n_outlier=2)
    S = synthetic.WorkloadSpec
    out = []
    for bf16 in (False, True):
        sfx = "bf16" if bf16 else "fp32"
        out += [
            S(f"jumprelu_clt_{sfx}", kind="jumprelu", crosslayer=True, bf16=bf16, lambda_sparsity=4e-4,
              pre_actv_loss=3e-6, lr=1e-3, **base),
            S(f"jumprelu_plt_{sfx}", kind="jumprelu", crosslayer=False, bf16=bf16, lambda_sparsity=2e-4,
              c_sparsity=0.5, pre_actv_loss=3e-6, lr=1e-3, **base),
            S(f"topk_clt_{sfx}", kind="topk", crosslayer=True, bf16=bf16, k=4, k_aux=8, aux_loss_scale=1 / 32,
              tokens_till_dead=1000, dead_fraction=0.3, lr=1e-3, **base),
            S(f"batchtopk_clt_{sfx}", kind="batchtopk", crosslayer=True, bf16=bf16, k=3, e=0.1, lr=1e-3, **base),
        ]
    return out


def case_inputs(spec):
    """Inputs of a golden case, regenerated from fixed seeds (also used by the tests)."""
    batch = synthetic.make_batch(spec, seed=11)
    weights = synthetic.make_weights(spec, seed=12)
    # non-zero biases so that every term of the arithmetic is exercised
    g = torch.Generator().manual_seed(13)
    weights["b_enc"] = 0.02 * torch.randn(weights["b_enc"].shape, generator=g)
    weights["b_dec"] = 0.02 * torch.randn(weights["b_dec"].shape, generator=g)
    last_active = synthetic.make_last_active(spec, seed=14)
    return batch, weights, last_active


def checksum(batch, weights):
    ts = [batch, weights["W_enc"], weights["b_enc"], weights["b_dec"]]
    ts += list(weights["W_dec"]) if isinstance(weights["W_dec"], list) else [weights["W_dec"]]
    return torch.stack([torch.stack([t.double().sum(), t.double().abs().sum()]) for t in ts])


def run_case(ref, spec):
    batch, weights, last_active = case_inputs(spec)
    mod = build_reference_module(ref, spec, weights, last_active)
    mod.model.initialize_standardizers(batch)
    ctx = torch.autocast("cpu", dtype=torch.bfloat16) if spec.bf16 else contextlib.nullcontext()
    with ctx:
        # the forward tuple, for the intermediate tensors
        pre, feat, recons_norm, recons = mod.forward(batch[:, 0])
    thr0 = mod.model.nonlinearity.threshold.clone() if spec.kind == "batchtopk" else None
    if thr0 is not None:
        mod.model.nonlinearity.threshold = torch.zeros(1)     # undo the forward's EMA update
    with ctx:
        loss = mod.training_step(batch, 1)
    loss.backward()
    names = [n for n, _ in mod.named_parameters()]
    grads = {n: (p.grad.detach().clone() if p.grad is not None else torch.zeros_like(p))
             for n, p in mod.named_parameters()}
    opt = mod.configure_optimizers()
    opt.step()
    after = {n: p.detach().clone() for n, p in mod.named_parameters()}
    out = {
        "spec": dict(spec.__dict__),
        "input_checksum": checksum(batch, weights),
        "names": names,
        "loss": loss.detach(), "pre": pre.detach().float(), "feat": feat.detach().float(),
        "recons_norm": recons_norm.detach().float(),
        "grads": grads, "params_after_adam": after if not spec.bf16 else None,
        "logged": {k: (v.detach().clone() if torch.is_tensor(v) else v) for k, v in mod.logged.items()},
        "last_active_out": mod.last_active.clone(),
        "stats": {"mu_in": mod.model.input_standardizer.mean.clone(), "sd_in": mod.model.input_standardizer.std.clone(),
                  "mu_out": mod.model.output_standardizer.mean.clone(), "sd_out": mod.model.output_standardizer.std.clone()},
    }
    if spec.kind == "batchtopk":
        out["threshold_out"] = mod.model.nonlinearity.threshold.detach().clone()
    return out


def main():
    ref = ref_import.load(with_lightning=True)
    torch.set_num_threads(1)          # fixed reduction order
    for spec in cases():
        out = run_case(ref, spec)
        torch.save(out, HERE / f"{spec.name}.pt")
        print(f"{spec.name}: loss={out['loss'].item():.6f}  nnz={int((out['feat'] > 0).sum())}")


if __name__ == "__main__":
    main()
