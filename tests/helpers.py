"""Shared helpers of the test-suite: golden-vector loading and error measures."""
from pathlib import Path

import torch

from oracle import clt_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = ["jumprelu_clt", "jumprelu_plt", "topk_clt", "batchtopk_clt"]


def load_golden(name):
    return torch.load(GOLDEN / f"{name}.pt", weights_only=False)


def rel_err(a, b):
    """max |a-b| over max |b|: the relative error measure of the parity bar."""
    a, b = a.double(), b.double()
    den = b.abs().max().clamp_min(1e-30)
    return float((a - b).abs().max() / den)


def oracle_inputs(g):
    """(Params, Hyper, stats, extra kwargs) of the oracle for one golden case."""
    s = g["spec"]
    w = g["weights"]
    P = O.Params(w["W_enc"], w["b_enc"], w["W_dec"], w["b_dec"], w.get("theta"))
    H = O.Hyper(kind=s["kind"], bf16=s["bf16"], bandwidth=s["bandwidth"], lambda_sparsity=s["lambda_sparsity"],
                c_sparsity=s["c_sparsity"], use_tanh=s["use_tanh"], pre_actv_loss=s["pre_actv_loss"], k=s["k"],
                k_aux=s["k_aux"], aux_loss_scale=s["aux_loss_scale"], tokens_till_dead=s["tokens_till_dead"], e=s["e"])
    st = g["stats"]
    stats = (st["mu_in"], st["sd_in"], st["mu_out"], st["sd_out"])
    kw = {}
    if s["kind"] == "topk":
        kw["last_active"] = g["last_active_in"]
    if s["kind"] == "batchtopk":
        kw["threshold"] = torch.zeros(1)
    return P, H, stats, kw


def golden_grad_list(g):
    """Reference gradients in ``Params.tensors()`` order."""
    s = g["spec"]
    gr = g["grads"]
    out = [gr["model.encoder.W"], gr["model.encoder.b"]]
    if s["crosslayer"]:
        out += [gr[f"model.decoder.W_{t}"] for t in range(s["n_layers"])]
    else:
        out.append(gr["model.decoder.W"])
    out.append(gr["model.decoder.b"])
    if s["kind"] == "jumprelu":
        out.append(gr["model.nonlinearity.theta"])
    return out
