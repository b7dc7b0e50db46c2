"""The entry points of the exchange that is fused into the kernels (`*_push`, `clt_sum_slots`), on ONE GPU:
the "ranks" are several buffers on the same device, so the ownership and slot arithmetic and the multi-
destination stores are checked against the plain entry points without needing peers.  The 2-GPU run of
the same kernels over NVLink is tests/test_gpu_multi.py."""
import pytest
import torch

from tests.helpers import rel_err

pytestmark = pytest.mark.gpu


def _bases(bufs):
    return torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64)


@pytest.mark.parametrize("short_rows", [0, 1])
@pytest.mark.parametrize("bf16", [0, 1])
def test_sparse_decoder_push_matches_plain(bf16, short_rows):
    from crosslayer_transcoder_b200._lib import lib, stream_ptr

    dev = torch.device("cuda:0")
    lib().check_device()
    g = torch.Generator().manual_seed(0)
    B, L, D, F, k, R = 77, 3, 128, 256, 6, 3
    P = L * (L + 1) // 2
    T = torch.bfloat16 if bf16 else torch.float32
    idx = torch.randint(0, F, (L, B, k), generator=g, dtype=torch.int32).to(dev)
    val = (torch.rand(L, B, k, generator=g) + 0.1).to(dev)
    val[:, :, k - 2:] = 0.0                                     # unused slots come last
    W = (torch.randn(P, F, D, generator=g) * 0.1).to(dev).to(T)
    bias = torch.randn(L, D, generator=g).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    recon = torch.empty(B, L, D, device=dev)
    lib().call("clt_sparse_decoder_fwd", idx, val, None, None, B * k, W, bias, recon, B, L, D, F, k, 1, short_rows,
               bf16, status, stream_ptr())
    rpr = (B + R - 1) // R
    bufs = [torch.zeros(R, rpr, L, D, device=dev) for _ in range(R)]      # owner buffers: one slot per source
    lib().call("clt_sparse_decoder_fwd_push", idx, val, None, None, B * k, W, bias, _bases(bufs), rpr, R, 1, 0, B, L, D,
               F, k, 1, short_rows, bf16, status, stream_ptr())
    torch.cuda.synchronize()
    assert int(status) == 0
    got = torch.cat([b[1] for b in bufs], 0)                    # slot 1 of every owner
    assert torch.equal(got[:B], recon)
    assert float(got[B:].abs().sum()) == 0.0                    # rows past B stay untouched
    assert all(float(b[0].abs().sum()) == 0.0 and float(b[2].abs().sum()) == 0.0 for b in bufs)   # other slots too
    # a second source fills another slot; the owner's sum of its slots is the reduced reconstruction
    lib().call("clt_sparse_decoder_fwd_push", idx, val, None, None, B * k, W, None, _bases(bufs), rpr, R, 2, 0, B, L, D,
               F, k, 1, short_rows, bf16, status, stream_ptr())
    own = [torch.empty(rpr, L, D, device=dev) for _ in range(R)]
    for b, o in zip(bufs, own):
        lib().call("clt_sum_slots", b, o, R, rpr * L * D, 0, stream_ptr())
    torch.cuda.synchronize()
    assert torch.allclose(torch.cat(own, 0)[:B], 2 * recon - bias, rtol=1e-6, atol=1e-6)
    # bf16 slots: the same partial rows rounded to bf16 (half the bytes), summed in fp32 by the owner
    hb = [torch.zeros(R, rpr, L, D, device=dev, dtype=torch.bfloat16) for _ in range(R)]
    for slot, bb in ((0, bias), (2, None)):
        lib().call("clt_sparse_decoder_fwd_push", idx, val, None, None, B * k, W, bb, _bases(hb), rpr, R, slot, 1, B, L,
                   D, F, k, 1, short_rows, bf16, status, stream_ptr())
    for b, o in zip(hb, own):
        lib().call("clt_sum_slots", b, o, R, rpr * L * D, 1, stream_ptr())
    torch.cuda.synchronize()
    assert int(status) == 0
    assert torch.equal(torch.cat([b[0] for b in hb], 0)[:B], recon.bfloat16())
    second = torch.cat([b[2] for b in hb], 0)[:B].float()           # partial rows without the bias
    assert rel_err(second, recon - bias) < 1e-2                     # (one bf16 rounding)
    want = recon.bfloat16().float() + second
    assert torch.allclose(torch.cat(own, 0)[:B], want, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("bf16", [0, 1])
def test_dense_decoder_push_matches_plain(bf16):
    from crosslayer_transcoder_b200._lib import lib, stream_ptr

    dev = torch.device("cuda:0")
    lib().check_device()
    g = torch.Generator().manual_seed(1)
    B, L, D, F, R = 200, 3, 128, 192, 3
    P = L * (L + 1) // 2
    T = torch.bfloat16 if bf16 else torch.float32
    feat = torch.relu(torch.randn(L, B, F, generator=g)).to(dev).to(T)
    W = (torch.randn(P, F, D, generator=g) * 0.1).to(dev).to(T)
    bias = torch.randn(L, D, generator=g).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    recon = torch.empty(B, L, D, device=dev)
    lib().call("clt_decoder_dense_fwd", feat, W, bias, recon, B, L, D, F, 1, bf16, status, stream_ptr())
    rpr = (B + R - 1) // R
    bufs = [torch.zeros(R, rpr, L, D, device=dev) for _ in range(R)]
    lib().call("clt_decoder_dense_fwd_push", feat, W, bias, _bases(bufs), rpr, R, 2, 0, B, L, D, F, 1, bf16, status,
               stream_ptr())
    torch.cuda.synchronize()
    assert int(status) == 0
    got = torch.cat([b[2] for b in bufs], 0)
    assert torch.equal(got[:B], recon)
    assert float(got[B:].abs().sum()) == 0.0
    assert all(float(b[0].abs().sum()) == 0.0 and float(b[1].abs().sum()) == 0.0 for b in bufs)


@pytest.mark.parametrize("with_aux", [False, True])
@pytest.mark.parametrize("bf16", [0, 1])
def test_loss_bwd_push_matches_plain(bf16, with_aux):
    from crosslayer_transcoder_b200._lib import DTYPE_CODE, lib, stream_ptr

    dev = torch.device("cuda:0")
    lib().check_device()
    g = torch.Generator().manual_seed(2)
    B, L, D, R = 90, 3, 64, 4
    T = torch.bfloat16 if bf16 else torch.float32
    batch = torch.randn(B, 2, L, D, generator=g).half().to(dev)
    recon = torch.randn(B, L, D, generator=g).to(dev)
    aux = torch.randn(B, L, D, generator=g).to(dev) if with_aux else None
    mu, sd = torch.randn(L, D, generator=g).to(dev), (torch.rand(L, D, generator=g) + 0.5).to(dev)
    gs = torch.full((1,), 0.7, device=dev)
    code = DTYPE_CODE[batch.dtype]
    drecon = torch.empty(L, B, D, dtype=T, device=dev)
    daux = torch.empty(L, B, D, dtype=T, device=dev) if with_aux else None
    db = torch.zeros(L, D, device=dev)
    lib().call("clt_loss_bwd", recon, aux, batch, code, mu, sd, gs, 0.25 if with_aux else 0.0, drecon, daux, bf16, db, B,
               L, D, stream_ptr())
    rpr = (B + R - 1) // R
    dsts = [torch.full((L, B, D), float("nan"), dtype=T, device=dev) for _ in range(R)]
    adsts = [torch.full((L, B, D), float("nan"), dtype=T, device=dev) for _ in range(R)] if with_aux else None
    db2 = torch.zeros(L, D, device=dev)
    for r in range(R):                                          # every "rank" pushes its own rows to all buffers
        lo = min(B, r * rpr)
        cnt = max(0, min(B, lo + rpr) - lo)
        lib().call("clt_loss_bwd_push", recon[lo:lo + cnt].contiguous(), aux[lo:lo + cnt].contiguous() if with_aux else None,
                   batch, code, mu, sd, gs, 0.25 if with_aux else 0.0, _bases(dsts), _bases(adsts) if with_aux else None,
                   R, bf16, db2, B, lo, cnt, L, D, stream_ptr())
    torch.cuda.synchronize()
    for d_ in dsts:
        assert torch.equal(d_, drecon)
    if with_aux:
        for d_ in adsts:
            assert torch.equal(d_, daux)
    assert torch.allclose(db2, db, rtol=1e-5, atol=1e-7)
