"""Device status word: kernels that read feature indices from memory compare them with the feature count
before any access that uses them, skip the bad entry, and report code 0x20 through the caller's status
word instead of faulting.  Exercised through the C ABI on the two entry points that take caller-supplied
index lists."""
import pytest
import torch

from crosslayer_transcoder_b200._lib import CltError, check_status, lib, stream_ptr

pytestmark = pytest.mark.gpu


def _lists(dev, L=2, B=7, k=4, F=64):
    g = torch.Generator().manual_seed(0)
    idx = torch.stack([torch.stack([torch.randperm(F, generator=g)[:k] for _ in range(B)]) for _ in range(L)]).int()
    val = torch.rand(L, B, k, generator=g) + 0.1
    return idx.to(dev), val.to(dev)


@pytest.mark.parametrize("short_rows", [0, 1])
def test_sparse_decoder_skips_out_of_range_index_and_reports_it(short_rows):
    dev = torch.device("cuda:0")
    lib().check_device()
    L, B, k, F, D = 2, 7, 4, 64, 64
    idx, val = _lists(dev, L, B, k, F)
    W = torch.randn(L * (L + 1) // 2, F, D, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def run(ix):
        recon = torch.full((B, L, D), 7.0, device=dev)
        lib().call("clt_sparse_decoder_fwd", ix, val, None, None, B * k, W, None, recon, B, L, D, F, k, 1, short_rows, 0,
                   status, stream_ptr())
        torch.cuda.synchronize()
        return recon

    good = run(idx)
    assert int(status) == 0
    bad = idx.clone()
    bad[0, 2, 1] = F + 5                # beyond the feature axis
    bad[1, 4, 0] = -1                   # negative
    out = run(bad)
    assert int(status) == 0x20
    with pytest.raises(CltError, match="out of range"):
        check_status(status, "test")
    assert int(status) == 0             # reported once, then cleared
    # the rest of the result is what the valid entries give: only rows that lost an entry differ
    val_fixed = val.clone()
    val_fixed[0, 2, 1] = 0.0
    val_fixed[1, 4, 0] = 0.0
    dense = torch.zeros(L, B, F, device=dev).scatter_add_(2, idx.long(), val_fixed)
    ref = torch.zeros(B, L, D, device=dev)
    for t in range(L):
        for s in range(t + 1):
            ref[:, t] += dense[s] @ W[t * (t + 1) // 2 + s]
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5)
    assert not torch.allclose(out, good)


def test_csc_build_skips_out_of_range_index_and_reports_it():
    dev = torch.device("cuda:0")
    lib().check_device()
    L, B, k, F = 2, 7, 4, 64
    idx, val = _lists(dev, L, B, k, F)
    bad = idx.clone()
    bad[1, 3, 2] = F                    # first index past the end
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    col_ptr = torch.full((L, F + 1), -3, dtype=torch.int32, device=dev)
    cursor = torch.empty(L, F, dtype=torch.int32, device=dev)
    ent = torch.full((L, B * k), -3, dtype=torch.int32, device=dev)
    lib().call("clt_csc_build", bad, val, col_ptr, cursor, ent, B * k, L, F, status, stream_ptr())
    torch.cuda.synchronize()
    assert int(status) == 0x20
    status.zero_()
    # the bad entry is in no feature's list; every other entry is listed exactly once under its feature
    assert int(col_ptr[0, F]) == B * k and int(col_ptr[1, F]) == B * k - 1
    for l in range(L):
        n = int(col_ptr[l, F])
        listed = ent[l, :n].long().cpu()
        assert len(set(listed.tolist())) == n and (ent[l, n:] == -3).all()
        feats = bad[l].reshape(-1).cpu()[listed]
        cp = col_ptr[l].cpu()
        for f in range(F):
            assert (feats[cp[f]:cp[f + 1]] == f).all()
    assert (3 * k + 2) not in ent[1, :int(col_ptr[1, F])].tolist()
