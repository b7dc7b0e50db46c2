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
    state = mod._engine.ws.buf["bt_state"]
    assert int(state[0, 6]) == 16                    # first step: no floor yet, full sweeps of z
    run_step(mod, batch.to(dev), idx=1)
    assert int(state[0, 6]) == 0                     # second step: one sweep, the rest on the candidate list
    assert float(mod.model.nonlinearity.threshold) > thr1
    sel, _ = O.batch_topk(engine_pre(mod), k, torch.zeros(1), spec.e)
    assert torch.equal(dense_from_lists(mod, B) > 0, sel > 0)
    # a much quieter batch: the guessed floor is now too high and the selection must fall back to the full range
    run_step(mod, (0.2 * batch).to(dev), idx=2)
    assert int(state[0, 6]) == 16
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


# ---------------------------------------------------------------------------------------------------------
# the candidate-list path of the selection against its full-sweep path, through the C ABI
# ---------------------------------------------------------------------------------------------------------
def _select(z, b_enc, n_keep, groups, floor, use_list, cap=None):
    """One BatchTopK selection of z [L, B, F] (fp32) with state[:, 7] = key(floor).  Returns the survivors as a
    dense [L, B, F] tensor, the per-row entry lists and state[:, 6]."""
    from crosslayer_transcoder_b200._lib import lib, stream_ptr

    L, B, F = z.shape
    dev = z.device
    s = stream_ptr()
    state = torch.zeros(groups, 8, dtype=torch.int64, device=dev)
    if floor > 0:
        state[:, 7] = int(torch.tensor(floor, dtype=torch.float32).view(torch.int32))
    nh = groups * 2048
    hbuf = torch.zeros(nh + 8, dtype=torch.int64, device=dev)
    hist, inval = hbuf[:nh], hbuf[nh:]
    npl = min(n_keep, B * F)
    idx = torch.zeros(L, npl, dtype=torch.int32, device=dev)
    val = torch.zeros(L, npl, device=dev)
    tok = torch.zeros(L, npl, dtype=torch.int32, device=dev)
    row_start = torch.zeros(L, B, dtype=torch.int32, device=dev)
    row_cnt = torch.zeros(L, B, dtype=torch.int32, device=dev)
    fill = torch.zeros(L, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    if use_list:
        cap = cap or L * B * F
        cf = torch.zeros(cap, dtype=torch.int32, device=dev)
        cv = torch.zeros(cap, device=dev)
        cr = torch.zeros(cap, dtype=torch.int32, device=dev)
        cfill = torch.zeros(1, dtype=torch.int32, device=dev)
        cs = torch.zeros(L, B, dtype=torch.int32, device=dev)
        cc = torch.zeros(L, B, dtype=torch.int32, device=dev)
        lib().call("clt_batchtopk_candidates", z, b_enc, state, cf, cv, cr, cfill, cs, cc, inval, groups, B, L, F, cap,
                   0, s)
    for level, retry in ((0, 0), (0, 1), (1, 0), (2, 0)):
        lib().call("clt_batchtopk_hist", z, b_enc, state, hist, inval if use_list else None, level, retry, groups, B, L,
                   F, 0, s)
        if use_list and not retry:
            lib().call("clt_batchtopk_hist_list", cv, cr, cfill, state, hist, inval, level, groups, B, cap, s)
        lib().call("clt_batchtopk_pick", hist, None, state, inval if use_list else None, level, retry, groups,
                   n_keep // groups, s)
    lib().call("clt_batchtopk_collect", z, b_enc, state, None, idx, val, tok, row_start, row_cnt, fill, None, groups, B,
               L, F, npl, 0, status, s)
    if use_list:
        lib().call("clt_batchtopk_filter", cf, cv, cs, cc, state, None, idx, val, tok, row_start, row_cnt, fill, None,
                   groups, B, L, F, npl, status, s)
    torch.cuda.synchronize()
    assert int(status) == 0
    dense = torch.zeros(L, B, F, device=dev)
    for l in range(L):
        n = int(fill[l])
        dense[l, tok[l, :n].long(), idx[l, :n].long()] = val[l, :n]
    return dense, (idx, val, tok, row_start, row_cnt, fill), state[:, 6].clone()


def _check_rows_sorted(lists, L, B):
    idx, val, tok, row_start, row_cnt, fill = [t.cpu() for t in lists]
    for l in range(L):
        assert int(row_cnt[l].sum()) == int(fill[l])
        for b in range(0, B, max(1, B // 16)):
            s0, c = int(row_start[l, b]), int(row_cnt[l, b])
            seg = idx[l, s0:s0 + c].long()
            assert bool((tok[l, s0:s0 + c] == b).all())
            # a fixed order: ascending 32-bit hash of the feature, salted with the row
            h = (seg * 2654435761 + (l * B + b) * 0x9E3779B1) % (1 << 32)
            assert bool((h[1:] > h[:-1]).all())


@pytest.mark.parametrize("groups", [1, 3])
def test_candidate_list_matches_full_sweeps(groups):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    L, B, F, k = 3, 64, 4096, 6
    z = torch.randn(L, B, F, generator=g).to(dev)
    b_enc = 0.1 * torch.randn(L, F, generator=g)
    b_enc[:, ::61] += 0.8                              # a few large biases
    b_enc = b_enc.to(dev)
    n_keep = k * B * L
    full, _, code_full = _select(z, b_enc, n_keep, groups, 0.0, False)
    assert int((full != 0).sum()) == n_keep and bool((code_full == 16).all())
    thr = float(full[full != 0].min())
    # a floor a little below the threshold: the list path runs (bit 4 clear) and gives the same survivors
    got, lists, code = _select(z, b_enc, n_keep, groups, 0.9 * thr, True)
    assert bool((code == 0).all())
    assert torch.equal(got, full)
    _check_rows_sorted(lists, L, B)
    # no floor yet: full sweeps
    got, _, code = _select(z, b_enc, n_keep, groups, 0.0, True)
    assert bool((code == 16).all()) and torch.equal(got, full)
    # a floor above the threshold: too few candidates, retry on full sweeps
    got, _, code = _select(z, b_enc, n_keep, groups, 1.5 * float(full.max()), True)
    assert bool((code == 16).all()) and torch.equal(got, full)
    # a list that is too small for the candidates: flagged invalid, full sweeps
    got, _, code = _select(z, b_enc, n_keep, groups, 0.9 * thr, True, cap=n_keep // 2)
    assert bool((code == 16).all()) and torch.equal(got, full)


def test_candidate_list_row_overflow_and_ties():
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(6)
    L, B, F = 2, 40, 8192
    z = torch.randn(L, B, F, generator=g).to(dev)
    z[1, 7] = z[1, 7].abs() + 3.0                 # one row holds 8192 values above any sensible floor
    b_enc = torch.zeros(L, F, device=dev)
    n_keep = 3000
    full, _, _ = _select(z, b_enc, n_keep, 1, 0.0, False)
    thr = float(full[full != 0].min())
    got, _, code = _select(z, b_enc, n_keep, 1, 0.9 * thr, True)
    assert bool((code == 16).all()) and torch.equal(got, full)       # more than 2048 candidates in that row
    # ties at the threshold: exactly n_keep survivors on both paths (which of the tied ones is not fixed)
    z = torch.randn(L, B, F, generator=g).to(dev).clamp_(max=1.5)     # thousands of elements equal to 1.5
    n_keep = int((z == 1.5).sum()) - 100
    full, _, _ = _select(z, b_enc, n_keep, 1, 0.0, False)
    got, lists, code = _select(z, b_enc, n_keep, 1, 1.2, True)
    assert bool((code == 0).all())
    assert int((got != 0).sum()) == n_keep == int((full != 0).sum())
    assert bool((got[got != 0] == 1.5).all())
    _check_rows_sorted(lists, L, B)
