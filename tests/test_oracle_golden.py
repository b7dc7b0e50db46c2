"""The CPU oracle against the golden vectors made from the unmodified reference."""
import pytest
import torch

from oracle import clt_oracle as O
from tests.helpers import CASES, golden_grad_list, load_golden, oracle_inputs, rel_err


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
@pytest.mark.parametrize("case", CASES)
def test_step_matches_reference(case, prec):
    g = load_golden(f"{case}_{prec}")
    P, H, stats, kw = oracle_inputs(g)
    st = O.standardizer_stats(g["batch"])
    for a, b in zip(st, stats):
        assert torch.allclose(a, b, rtol=1e-6, atol=1e-7)
    out, grads = O.step_with_grads(P, g["batch"], stats, H, **kw)
    tol = 1e-5 if prec == "fp32" else 2e-3
    assert rel_err(out.loss, g["loss"]) < tol
    assert rel_err(out.pre, g["pre"]) < tol
    assert torch.equal(out.feat > 0, g["feat"] > 0)          # active sets bit-exact
    assert rel_err(out.feat, g["feat"]) < tol
    assert rel_err(out.recons_norm, g["recons_norm"]) < tol
    for a, b in zip(grads, golden_grad_list(g)):
        assert a.shape == b.shape
        assert rel_err(a, b) < tol
    if case == "topk_clt":
        assert torch.equal(out.last_active, g["last_active_out"])
    if case == "batchtopk_clt":
        assert rel_err(out.threshold, g["threshold_out"]) < tol


@pytest.mark.parametrize("case", CASES)
def test_adam_matches_reference(case):
    g = load_golden(f"{case}_fp32")
    s = g["spec"]
    for name, p1 in g["params_after_adam"].items():
        key = name
        w = g["weights"]
        lookup = {"model.encoder.W": w["W_enc"], "model.encoder.b": w["b_enc"], "model.decoder.b": w["b_dec"]}
        if s["crosslayer"]:
            lookup.update({f"model.decoder.W_{t}": w["W_dec"][t] for t in range(s["n_layers"])})
        else:
            lookup["model.decoder.W"] = w["W_dec"]
        if "theta" in w:
            lookup["model.nonlinearity.theta"] = w["theta"]
        p0, gr = lookup[key], g["grads"][key]
        p, m, v = O.adam_step(p0, gr, torch.zeros_like(p0), torch.zeros_like(p0), 1, s["lr"])
        assert torch.allclose(p, p1, rtol=1e-6, atol=1e-7), name


def test_topk_known_answers():
    # literal cases of the reference's own selection tests (tests/test_topk.py:77-113)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]])
    assert torch.equal(O.per_layer_topk(x, 3), torch.tensor([[[0.0, 0.0, 3.0, 4.0, 5.0]]]))
    assert torch.equal(O.per_layer_topk(x, 0), torch.zeros_like(x))
    assert torch.equal(O.per_layer_topk(x, 5), x)
    with pytest.raises(AssertionError):
        O.per_layer_topk(x, 6)
    neg = -torch.rand(2, 3, 7) - 0.1
    assert (O.per_layer_topk(neg, 3) >= 0).all()
    y = torch.arange(1.0, 21.0).reshape(2, 2, 5)
    f, thr = O.batch_topk(y, 3, torch.zeros(1), 0.1)
    assert int((f != 0).sum()) == 12 and f.max() == 20 and (f == 19).any()
    assert torch.allclose(thr, torch.tensor([0.9]))
