"""Parity at the benchmark configurations' own contraction lengths and tile counts.

Every case keeps d_acts, d_features and the batch size of one benchmark configuration and cuts only the
number of layers, so that the persistent tensor-core kernel runs with dozens of output tiles per CTA (both
accumulators, many reuses), the selection kernels see full-length rows and the sparse kernels see the real
row lengths — against the CPU oracle on the same seeded inputs.  Tolerances: 2e-2 relative (bf16 arithmetic);
TopK / BatchTopK index sets bit-exact against the reference selector applied to this path's own
pre-activations, and the disagreements with the oracle's own run (different accumulation order before the
bf16 rounding) must lie within one bf16 step of the row's k-th value."""
import pytest
import torch

from crosslayer_transcoder_b200 import synthetic
from oracle import clt_oracle as O
from tests.helpers import build_module, module_grad_list, oracle_for_spec, rel_err, spec_inputs

pytestmark = pytest.mark.gpu
TOL = 2e-2


_ORACLE_CACHE = {}


def _oracle(spec, key, **inputs_kw):
    """Seeded inputs and the oracle's step for ``spec`` (computed once per case: the CPU step takes tens of
    seconds at these sizes)."""
    if key not in _ORACLE_CACHE:
        batch, w, la = spec_inputs(spec, **inputs_kw)
        _ORACLE_CACHE[key] = (batch, w, la)
    return _ORACLE_CACHE[key]


def _step(mod, batch_dev):
    loss = mod.training_step(batch_dev, 0)
    loss.backward()
    torch.cuda.synchronize()
    mod._engine.check_status("after backward")
    return loss


def _check_grads(mod, ref_grads):
    names = ["W_enc", "b_enc"] + [f"W_dec[{i}]" for i in range(len(mod.model.decoder.blocks()))] + ["b_dec", "theta"]
    for name, a, b in zip(names, module_grad_list(mod), ref_grads):
        assert a is not None, name
        e = rel_err(a.cpu(), b)
        assert e < TOL, f"{name}: {e}"


def _pre_of(mod):
    z = mod._engine.ws.buf["z"].float().cpu()
    return (z + mod.model.encoder.b.detach().cpu().unsqueeze(1)).permute(1, 0, 2).contiguous()      # [B, L, F]


@pytest.mark.parametrize("fuse", [False, True], ids=["split_activation", "fused_epilogue"])
def test_c2_slice_per_layer_jumprelu(fuse):
    """configs[1] cut to 2 layers: D=768, F=24576, B=4000 (96 x 32 output tiles per layer)."""
    spec = synthetic.scaled(synthetic.WORKLOADS["c2_plt_bf16"], n_layers=2, name="c2_slice")
    batch, w, la = _oracle(spec, "c2", bias_scale=0.01)
    if "c2_ref" not in _ORACLE_CACHE:
        P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
        _ORACLE_CACHE["c2_ref"] = O.step_with_grads(P, batch, stats, H, **kw)
    ref, ref_grads = _ORACLE_CACHE["c2_ref"]
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    mod.fuse_activation = fuse
    loss = _step(mod, batch.to(dev))
    assert rel_err(loss.cpu(), ref.loss) < TOL
    terms = mod._engine.last_terms.cpu()
    assert rel_err(terms[0], ref.terms["mse"]) < TOL and rel_err(terms[2], ref.terms["pre_actv"]) < TOL
    _check_grads(mod, ref_grads)


def test_c5_slice_crosslayer_jumprelu():
    """configs[4] cut to 2 layers: D=2304, F=16384, B=4096, tanh sparsity + pre-activation loss."""
    spec = synthetic.scaled(synthetic.WORKLOADS["c5_clt_jumprelu_bf16"], n_layers=2, name="c5_slice")
    batch, w, la = spec_inputs(spec, bias_scale=0.01)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    ref, ref_grads = O.step_with_grads(P, batch, stats, H, **kw)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev)
    loss = _step(mod, batch.to(dev))
    assert rel_err(loss.cpu(), ref.loss) < TOL
    terms = mod._engine.last_terms.cpu()
    assert rel_err(terms[1], ref.terms["sparsity"]) < TOL and rel_err(terms[2], ref.terms["pre_actv"]) < TOL
    _check_grads(mod, ref_grads)


def _ulp_report(pre_here, feat_here, feat_ref, k_rows):
    """Fraction of selected-set disagreements and how many of them lie within one bf16 step of the row's
    k-th largest value (``k_rows``: [B, L] thresholds of this path's own selection)."""
    diff = (feat_here > 0) != (feat_ref > 0)
    n_diff = int(diff.sum())
    if n_diff == 0:
        return 0.0, 1.0
    thr = k_rows.unsqueeze(-1).expand_as(pre_here)
    step = thr.abs() * 2.0 ** -7                                  # one bf16 step at the threshold's magnitude
    near = ((pre_here - thr).abs() <= step) & diff
    return n_diff / float(max(1, int((feat_ref > 0).sum()))), float(near.sum()) / n_diff


def test_c3_slice_crosslayer_topk_with_aux():
    """configs[2] cut to 3 layers (6 decoder blocks): D=768, F=32768, B=4000, k=32, k_aux=512, 10 % dead."""
    spec = synthetic.scaled(synthetic.WORKLOADS["c3_clt_topk_bf16"], n_layers=3, name="c3_slice", lr=1e-3)
    batch, w, la = spec_inputs(spec, bias_scale=0.01)
    dead = la > spec.tokens_till_dead
    w["b_enc"][dead] = -1.0                     # dead features stay out of the top-k, as in the benchmark
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    ref, ref_grads = O.step_with_grads(P, batch, stats, H, **kw)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev, last_active=la)
    loss = _step(mod, batch.to(dev))
    ws = mod._engine.ws.buf
    idx, val = ws["idx"].long().cpu(), ws["val"].cpu()
    Ln, B, k = idx.shape
    feat = torch.zeros(Ln, B, spec.d_features).scatter_add_(2, idx, val).permute(1, 0, 2).contiguous()
    pre = _pre_of(mod)
    assert torch.equal(feat > 0, O.per_layer_topk(pre, spec.k) > 0)          # bit-exact on the same pre-activations
    kth = torch.topk(pre, spec.k, dim=-1).values[..., -1]
    frac, near = _ulp_report(pre, feat, ref.feat, kth)
    print(f"c3 slice: {frac:.2e} of the selected entries differ from the oracle's run; {near:.3f} of those lie "
          f"within one bf16 step of the k-th value")
    assert frac < 2e-3 and near > 0.95
    assert rel_err(loss.cpu(), ref.loss) < TOL
    assert rel_err(mod.logged["training/aux_loss"].cpu(), ref.terms["aux"]) < TOL
    # dead-feature counters: a feature whose only activations are the near-tie entries may differ
    assert (mod.last_active.cpu() != ref.last_active).float().mean() < 1e-3
    # Features are sparse here (a few activations each), so ONE near-tie entry that falls the other way
    # changes that feature's whole gradient column.  Gradients are therefore compared on the features
    # whose selections (main and auxiliary) agree in every token, which must be almost all of them; the
    # loss, the decoder bias gradient and the counters above cover the rest.
    aux = mod._engine._last_ctx["aux"]
    a_aux, dl, nd = aux["a_aux"].float().cpu(), aux["dead_list"].long().cpu(), aux["n_dead"].cpu()
    aux_here = torch.zeros(Ln, B, spec.d_features)
    for l in range(Ln):
        n = int(nd[l])
        aux_here[l, :, dl[l, :n]] = a_aux[l, :, :n]
    aux_here = aux_here.permute(1, 0, 2)
    differs = (((feat > 0) != (ref.feat > 0)) | ((aux_here > 0) != (ref.aux_feat > 0))).any(dim=0)      # [L, F]
    print(f"c3 slice: {int(differs.sum())} of {differs.numel()} features have a selection that differs in some token")
    assert differs.float().mean() < 2e-3
    same = ~differs
    g_here, names = module_grad_list(mod), ["W_enc", "b_enc"] + [f"W_dec[{t}]" for t in range(Ln)] + ["b_dec"]
    for name, a, b in zip(names, g_here, ref_grads):
        a = a.cpu()
        if name == "W_enc":                      # [L, D, F]: feature columns
            m = same.unsqueeze(1).expand_as(b)
        elif name == "b_enc":                    # [L, F]
            m = same
        elif name.startswith("W_dec"):           # [(t+1), F, D]: rows of the source layers' features
            m = same[: b.shape[0]].unsqueeze(-1).expand_as(b)
        else:
            m = torch.ones_like(b, dtype=torch.bool)
        e = float((a - b)[m].abs().max() / b[m].abs().max())
        assert e < TOL, f"{name}: {e}"


def test_c4_slice_crosslayer_batchtopk():
    """configs[3] cut to 2 layers and a quarter of the batch: D=2048, F=16384, B=2048, batch-global top 4 B L."""
    spec = synthetic.scaled(synthetic.WORKLOADS["c4_clt_batchtopk_bf16"], n_layers=2, batch=2048, name="c4_slice",
                            lr=1e-3)
    batch, w, la = spec_inputs(spec, bias_scale=0.01)
    P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
    ref, ref_grads = O.step_with_grads(P, batch, stats, H, **kw)
    dev = torch.device("cuda:0")
    mod = build_module(spec, w, dev, last_active=la)
    loss = _step(mod, batch.to(dev))
    ws = mod._engine.ws.buf
    idx, val, tok = ws["bt_idx"].long().cpu(), ws["bt_val"].cpu(), ws["bt_tok"].long().cpu()
    Ln, npl = idx.shape
    B, F = spec.batch, spec.d_features
    feat = torch.zeros(Ln, B * F)
    live = val > 0
    for l in range(Ln):
        feat[l].scatter_add_(0, (tok[l] * F + idx[l])[live[l]], val[l][live[l]])
    feat = feat.view(Ln, B, F).permute(1, 0, 2).contiguous()
    pre = _pre_of(mod)
    here, _ = O.batch_topk(pre, spec.k, torch.zeros(1), spec.e)
    n_keep = spec.k * B * Ln
    assert int((feat > 0).sum()) == n_keep
    # same set as the reference selector on these pre-activations, except among values equal to the threshold
    thr = float(torch.topk(pre.flatten(), n_keep).values[-1])
    assert torch.equal((feat > 0) & (pre != thr), (here > 0) & (pre != thr))
    frac, near = _ulp_report(pre, feat, ref.feat, torch.full(pre.shape[:2], thr))
    print(f"c4 slice: {frac:.2e} of the selected entries differ from the oracle's run; {near:.3f} of those lie "
          f"within one bf16 step of the threshold")
    assert frac < 2e-3 and near > 0.95
    assert rel_err(loss.cpu(), ref.loss) < TOL
    assert rel_err(mod.model.nonlinearity.threshold.cpu(), ref.threshold) < TOL
    _check_grads(mod, ref_grads)
