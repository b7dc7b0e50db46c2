"""Shared helpers of the test-suite: golden-vector loading and error measures."""
from pathlib import Path

import torch

from oracle import clt_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = ["jumprelu_clt", "jumprelu_plt", "topk_clt", "batchtopk_clt"]


def load_golden(name):
    """Golden outputs plus the case's inputs, regenerated from the fixed seeds the generator used."""
    import importlib.util

    from crosslayer_transcoder_b200 import synthetic

    g = torch.load(GOLDEN / f"{name}.pt", weights_only=False)
    spec_ = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    mg = importlib.util.module_from_spec(spec_)
    spec_.loader.exec_module(mg)
    spec = synthetic.WorkloadSpec(**g["spec"])
    g["batch"], g["weights"], g["last_active_in"] = mg.case_inputs(spec)
    assert torch.allclose(mg.checksum(g["batch"], g["weights"]), g["input_checksum"], rtol=1e-9), \
        "seeded inputs differ from the ones the golden vectors were made with"
    return g


def rel_err(a, b):
    """max |a-b| over max |b|: the relative error measure of the parity bar."""
    a, b = a.detach().double(), b.detach().double()
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


# --------------------------------------------------------------------------- #
# building the CUDA-side module from a workload spec
# --------------------------------------------------------------------------- #
def build_module(spec, weights, device, last_active=None, precision=None):
    """The package's training module for ``spec`` with ``weights`` copied in."""
    import crosslayer_transcoder_b200.model as M

    L, D = spec.n_layers, spec.d_acts
    F = weights["W_enc"].shape[-1]
    enc = M.Encoder(D, F, L)
    dec = (M.CrosslayerDecoder if spec.crosslayer else M.Decoder)(D, F, L)
    if spec.kind == "jumprelu":
        nl = M.JumpReLU(theta=spec.theta, bandwidth=spec.bandwidth, n_layers=L, d_features=F)
    elif spec.kind == "relu":
        nl = M.ReLU()
    elif spec.kind == "topk":
        nl = M.PerLayerTopK(k=spec.k)
    elif spec.kind == "perlayer_batchtopk":
        nl = M.PerLayerBatchTopK(k=spec.k, e=spec.e, n_layers=L)
    else:
        nl = M.BatchTopK(k=spec.k, e=spec.e)
    model = M.CrossLayerTranscoder(nl, enc, dec, M.DimensionwiseInputStandardizer(L, D),
                                   M.DimensionwiseOutputStandardizer(L, D))
    with torch.no_grad():
        enc.W.copy_(weights["W_enc"])
        enc.b.copy_(weights["b_enc"])
        dec.b.copy_(weights["b_dec"])
        if spec.crosslayer:
            for t, w in enumerate(dec.blocks()):
                w.copy_(weights["W_dec"][t])
        else:
            dec.W.copy_(weights["W_dec"])
        if spec.kind == "jumprelu" and "theta" in weights:
            nl.theta.copy_(weights["theta"])
    common = dict(model=model, learning_rate=spec.lr)
    if spec.kind in ("jumprelu", "relu"):
        mod = M.JumpReLUCrossLayerTranscoderModule(lambda_sparsity=spec.lambda_sparsity, c_sparsity=spec.c_sparsity,
                                                   use_tanh=spec.use_tanh, pre_actv_loss=spec.pre_actv_loss, **common)
        mod.trainer.max_steps = 1
        mod.global_step = 1
    elif spec.kind == "topk":
        mod = M.TopKCrossLayerTranscoderModule(topk_aux=M.PerLayerTopK(k=spec.k_aux),
                                               tokens_till_dead=spec.tokens_till_dead,
                                               aux_loss_scale=spec.aux_loss_scale, **common)
    else:
        mod = M.CrossLayerTranscoderModule(tokens_till_dead=spec.tokens_till_dead, **common)
    if last_active is not None:
        mod.last_active.copy_(last_active)
    mod.precision = precision or ("bf16" if spec.bf16 else "fp32")
    return mod.to(device)


def module_grad_list(mod):
    """Gradients of the package's module in ``Params.tensors()`` order."""
    m = mod.model
    out = [m.encoder.W.grad, m.encoder.b.grad] + [w.grad for w in m.decoder.blocks()] + [m.decoder.b.grad]
    if hasattr(m.nonlinearity, "theta"):
        out.append(m.nonlinearity.theta.grad)
    return out


def spec_inputs(spec, seed=21, bias_scale=0.02):
    """Seeded batch / weights / counters for an arbitrary spec (non-zero biases)."""
    from crosslayer_transcoder_b200 import synthetic

    batch = synthetic.make_batch(spec, seed=seed)
    w = synthetic.make_weights(spec, seed=seed + 1)
    g = torch.Generator().manual_seed(seed + 2)
    w["b_enc"] = bias_scale * torch.randn(w["b_enc"].shape, generator=g)
    w["b_dec"] = bias_scale * torch.randn(w["b_dec"].shape, generator=g)
    la = synthetic.make_last_active(spec, seed=seed + 3)
    return batch, w, la


def oracle_for_spec(spec, batch, w, la):
    P = O.Params(w["W_enc"], w["b_enc"], w["W_dec"], w["b_dec"], w.get("theta"))
    H = O.Hyper(kind=spec.kind, bf16=spec.bf16, bandwidth=spec.bandwidth, lambda_sparsity=spec.lambda_sparsity,
                c_sparsity=spec.c_sparsity, use_tanh=spec.use_tanh, pre_actv_loss=spec.pre_actv_loss, k=spec.k,
                k_aux=spec.k_aux, aux_loss_scale=spec.aux_loss_scale, tokens_till_dead=spec.tokens_till_dead, e=spec.e)
    stats = O.standardizer_stats(batch)
    kw = {}
    if spec.kind == "topk":
        kw["last_active"] = la
    if spec.kind == "batchtopk":
        kw["threshold"] = torch.zeros(1)
    if spec.kind == "perlayer_batchtopk":
        kw["threshold"] = torch.zeros(spec.n_layers)
    return P, H, stats, kw
