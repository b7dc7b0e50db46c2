"""Interchange with the reference project on the CPU: configs / checkpoints written by either side load on
the other (class paths are mapped), and the fused optimizer's state survives a checkpoint round trip in
``torch.optim.Adam``'s own layout."""
import pytest
import torch

import crosslayer_transcoder_b200.model as M
from crosslayer_transcoder_b200.engine import FlatParams, FusedAdam
from crosslayer_transcoder_b200.model import serializable_module as SM
from oracle import ref_import

L, D, F = 3, 8, 16


def _ours(nl=None):
    torch.manual_seed(3)
    m = M.CrossLayerTranscoder(nl or M.JumpReLU(0.03, 1.0, L, F), M.Encoder(D, F, L), M.CrosslayerDecoder(D, F, L),
                               M.DimensionwiseInputStandardizer(L, D), M.DimensionwiseOutputStandardizer(L, D))
    with torch.no_grad():
        m.encoder.b.normal_()
    return m


def test_reference_class_paths_resolve_to_this_package():
    assert SM._resolve("crosslayer_transcoder.model.clt.Encoder") is M.Encoder
    assert SM._resolve("crosslayer_transcoder.model.topk.BatchTopK") is M.BatchTopK
    assert SM._resolve("crosslayer_transcoder_b200.model.jumprelu.JumpReLU") is M.JumpReLU
    cfg = _ours().config_for_export(reference_class_paths=True)
    assert cfg["class_path"] == "crosslayer_transcoder.model.clt.CrossLayerTranscoder"
    assert cfg["init_args"]["encoder"]["class_path"] == "crosslayer_transcoder.model.clt.Encoder"
    assert _ours().to_config()["class_path"].startswith("crosslayer_transcoder_b200.")       # default unchanged
    again = M.CrossLayerTranscoder.from_config(cfg)                                          # and it loads back here
    assert isinstance(again.encoder, M.Encoder) and again.encoder.W.shape == (L, D, F)


@pytest.mark.skipif(not ref_import.available(), reason="needs the reference source tree")
@pytest.mark.parametrize("nl_name", ["JumpReLU", "PerLayerTopK", "BatchTopK"])
def test_checkpoints_load_both_ways(tmp_path, nl_name):
    ref = ref_import.load()

    def make(ns_clt, ns_jr, ns_topk, ns_std):
        if nl_name == "JumpReLU":
            nl = ns_jr.JumpReLU(0.03, 1.0, L, F)
        else:
            nl = getattr(ns_topk, nl_name)(k=4, e=0.1, n_layers=L)
        return ns_clt.CrossLayerTranscoder(nl, ns_clt.Encoder(D, F, L), ns_clt.CrosslayerDecoder(D, F, L),
                                           ns_std.DimensionwiseInputStandardizer(L, D),
                                           ns_std.DimensionwiseOutputStandardizer(L, D))

    import crosslayer_transcoder_b200.model.clt as oc
    import crosslayer_transcoder_b200.model.jumprelu as oj
    import crosslayer_transcoder_b200.model.standardize as os_
    import crosslayer_transcoder_b200.model.topk as ot

    # reference -> here
    torch.manual_seed(5)
    rm = make(ref.clt, ref.jumprelu, ref.topk, ref.standardize)
    rm.save_pretrained(tmp_path / "from_ref", fold_standardizers=False)
    mine = M.CrossLayerTranscoder.from_pretrained(tmp_path / "from_ref")
    assert type(mine.encoder) is M.Encoder and type(mine.nonlinearity).__name__ == nl_name
    for k, v in rm.state_dict().items():
        assert _same_bits(mine.state_dict()[k], v), k
    # here -> reference
    torch.manual_seed(6)
    om = make(oc, oj, ot, os_)
    om.save_pretrained(tmp_path / "to_ref", fold_standardizers=False, reference_class_paths=True)
    theirs = ref.clt.CrossLayerTranscoder.from_pretrained(tmp_path / "to_ref")
    assert type(theirs.encoder) is ref.clt.Encoder
    for k, v in om.state_dict().items():
        assert _same_bits(theirs.state_dict()[k], v), k


def _same_bits(a, b):
    """Equality that also holds for uninitialised standardizer buffers (which may contain NaN patterns)."""
    return a.shape == b.shape and a.dtype == b.dtype and torch.equal(a.reshape(-1).contiguous().view(torch.uint8),
                                                                      b.reshape(-1).contiguous().view(torch.uint8))


class _FakeEngine:
    """Just the attributes FusedAdam touches outside a kernel launch."""

    def __init__(self, module):
        self.flat = FlatParams(module, torch.device("cpu"), want_bf16=False)


def test_fused_adam_state_round_trip_relinks_the_flat_moments():
    """What a checkpoint resume does: ``state_dict()`` of an optimizer that has stepped is loaded into a
    fresh one.  The step count and both moments must arrive in the flat buffers the kernel reads (and
    ``state`` must point into them), in the layout of ``torch.optim.Adam``."""
    m1 = _ours()
    e1 = _FakeEngine(m1)
    o1 = FusedAdam(m1.parameters(), e1, lr=1e-3)
    e1.flat.ensure_moments()
    torch.manual_seed(9)
    e1.flat.exp_avg.normal_()
    e1.flat.exp_avg_sq.uniform_()
    o1._link_state(e1.flat)
    o1._step = 2
    for p in m1.parameters():
        o1.state[p]["step"] = 2
    sd = o1.state_dict()
    assert set(sd["state"][0]) == {"exp_avg", "exp_avg_sq", "step"}
    # the same dict loads into torch's own Adam (layout compatibility)
    twin = torch.optim.Adam([torch.nn.Parameter(p.detach().clone()) for p in m1.parameters()], lr=1e-3)
    sd_t = {"state": {i: {**st, "step": torch.tensor(float(st["step"]))} for i, st in sd["state"].items()},
            "param_groups": twin.state_dict()["param_groups"]}
    twin.load_state_dict(sd_t)
    # resume: fresh module + optimizer, flat buffers already built
    m2 = _ours()
    e2 = _FakeEngine(m2)
    o2 = FusedAdam(m2.parameters(), e2, lr=1e-3)
    o2.load_state_dict(sd)
    assert o2._step == 2
    def same_moments(fa, ma, fb, mb):          # per parameter: the alignment gaps between them carry nothing
        return all(torch.equal(fa.view_of(pa, getattr(fa, n)), fb.view_of(pb, getattr(fb, n)))
                   for pa, pb in zip(ma.parameters(), mb.parameters()) for n in ("exp_avg", "exp_avg_sq"))

    assert same_moments(e2.flat, m2, e1.flat, m1)
    for p in m2.parameters():
        assert o2.state[p]["exp_avg"].data_ptr() == e2.flat.view_of(p, e2.flat.exp_avg).data_ptr()
    # resume before the flat buffers exist (the usual order in a trainer): linked at the first step
    m3 = _ours()
    e3 = _FakeEngine(m3)
    flat3, e3.flat = e3.flat, None
    o3 = FusedAdam(m3.parameters(), e3, lr=1e-3)
    o3.load_state_dict(sd_t)                       # torch's layout (tensor step counts) is accepted too
    assert o3._step == 2 and o3._linked_to is None
    e3.flat = flat3
    o3._link_state(flat3)
    assert same_moments(flat3, m3, e1.flat, m1)
