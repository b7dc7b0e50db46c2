"""The allocation-free counting sort (`clt_csc_build_static`) against the ordinary entry point.

Some hosts of this library cannot let it allocate: their device memory is pre-reserved by their own
pool, or a cudaMalloc in the loop would stall the device.  For them the sort's scratch lives inside
the library image.  This test calls both entry points through the C ABI on the same selections, twice
in a row (the second call finds the first call's leftovers in the shared scratch), and requires
identical outputs.  Entries of one feature may come out in any order (they are placed with atomics),
so they are compared as sorted groups; everything else is compared bit for bit.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _selection(L, B, F, k, seed, dev):
    g = torch.Generator().manual_seed(seed)
    idx = torch.stack([torch.stack([torch.randperm(F, generator=g)[:k] for _ in range(B)]) for _ in range(L)])
    val = torch.rand(L, B, k, generator=g) + 0.1
    val[torch.rand(L, B, k, generator=g) < 0.2] = 0.0           # unused slots
    return idx.to(torch.int32).to(dev), val.to(dev)


def _canonical(col_ptr, ent, L, F):
    """Entries of every (layer, feature) group sorted, so that the atomic placement order does not matter."""
    cp, e = col_ptr.cpu(), ent.cpu()
    out = []
    for l in range(L):
        row = e[l].clone()
        for f in range(F):
            a, b = int(cp[l, f]), int(cp[l, f + 1])
            row[a:b] = row[a:b].sort().values
        out.append(row[: int(cp[l, F])])
    return out


def test_static_scratch_matches_caller_scratch_twice():
    from crosslayer_transcoder_b200._lib import lib, stream_ptr

    dev = torch.device("cuda:0")
    L_ = lib()
    L_.check_device()
    for seed, (L, B, F, k) in enumerate([(3, 50, 96, 4), (2, 70, 160, 8)]):      # two calls in a row, different shapes
        idx, val = _selection(L, B, F, k, seed, dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        cp_a = torch.empty(L, F + 1, dtype=torch.int32, device=dev)
        cp_b = torch.empty_like(cp_a)
        ent_a = torch.full((L, B * k), -1, dtype=torch.int32, device=dev)
        ent_b = torch.full_like(ent_a, -1)
        cursor = torch.empty(L, F, dtype=torch.int32, device=dev)
        L_.call("clt_csc_build", idx, val, cp_a, cursor, ent_a, B * k, L, F, status, stream_ptr())
        L_.call("clt_csc_build_static", idx, val, cp_b, ent_b, B * k, L, F, status, stream_ptr())
        torch.cuda.synchronize()
        assert int(status) == 0
        assert torch.equal(cp_a, cp_b)
        assert int(cp_a[:, -1].sum()) == int((val != 0).sum())
        for a, b in zip(_canonical(cp_a, ent_a, L, F), _canonical(cp_b, ent_b, L, F)):
            assert torch.equal(a, b)


def test_static_scratch_rejects_oversize():
    from crosslayer_transcoder_b200._lib import CltError, lib, stream_ptr

    dev = torch.device("cuda:0")
    L_ = lib()
    L_.check_device()
    t = torch.zeros(8, dtype=torch.int32, device=dev)
    with pytest.raises(CltError, match="exceeds the built-in scratch"):
        L_.call("clt_csc_build_static", t, t.float(), t, t, 1, 2, (1 << 20), None, stream_ptr())
