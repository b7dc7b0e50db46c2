"""The feature-sharding exchange steps on CPU ranks (gloo, world size 2): partial reconstructions
summed by all-reduce, and the TopK threshold derived from the all-gathered per-shard candidates,
both against the unsharded oracle."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    from crosslayer_transcoder_b200 import parallel, synthetic
    from oracle import clt_oracle as O

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        spec = synthetic.WorkloadSpec("gloo", 3, 32, 64, 40, "topk", True, False, rank_u=8, n_outlier=1, k=4)
        batch = synthetic.make_batch(spec, seed=3)
        w = synthetic.make_weights(spec, seed=4)
        lo, hi = parallel.feature_shard(spec.d_features, rank, world)
        ws = synthetic.make_weights(spec, seed=4, f_lo=lo, f_hi=hi)          # this rank's slice, drawn independently
        assert torch.equal(ws["W_enc"], w["W_enc"][:, :, lo:hi])
        assert all(torch.equal(a, b[:, lo:hi]) for a, b in zip(ws["W_dec"], w["W_dec"]))
        stats = O.standardizer_stats(batch)
        xn = (batch[:, 0] - stats[0]) / stats[1]
        full = O.Params(w["W_enc"], w["b_enc"], w["W_dec"], w["b_dec"])
        part = O.Params(ws["W_enc"], ws["b_enc"], ws["W_dec"], torch.zeros_like(ws["b_dec"]))
        pre_full = O.encoder_fwd(xn, full, False)
        feat_full = O.per_layer_topk(pre_full, spec.k)
        # --- selection across shards: all-gather the k best values per row, threshold, filter
        pre = O.encoder_fwd(xn, part, False)
        vals = torch.topk(pre, spec.k, dim=-1).values.clamp_min(0).permute(1, 0, 2).contiguous()    # [L, B, k]
        allv = torch.empty(world, *vals.shape)
        parallel.all_gather(allv, vals, dist.group.WORLD)
        merged = allv.permute(1, 2, 0, 3).reshape(*vals.shape[:2], -1)                              # [L, B, R k]
        thr = torch.topk(merged, spec.k, dim=-1).values[..., -1].permute(1, 0).unsqueeze(-1)        # [B, L, 1]
        feat = torch.where((pre >= thr) & (pre > 0), pre, torch.zeros_like(pre))
        assert torch.equal(feat, feat_full[:, :, lo:hi])
        # --- partial reconstructions: sum over shards == unsharded decoder
        recon = O.decoder_fwd(feat, part, False).contiguous()
        parallel.all_reduce_sum(recon, dist.group.WORLD)
        recon = recon + w["b_dec"]
        ref = O.decoder_fwd(feat_full, full, False)
        assert torch.allclose(recon, ref, rtol=1e-5, atol=1e-6)
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_exchange():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29611, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(v == "ok" for _, v in res), res


def test_feature_shard_bounds():
    from crosslayer_transcoder_b200 import parallel
    import pytest

    assert parallel.feature_shard(32768, 3, 8) == (12288, 16384)
    with pytest.raises(ValueError):
        parallel.feature_shard(100, 0, 8)


def _ckpt_worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    import crosslayer_transcoder_b200.model as M
    from crosslayer_transcoder_b200 import parallel

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, D, F = 3, 8, 16
        torch.manual_seed(7)
        full = M.JumpReLUCrossLayerTranscoderModule(model=M.CrossLayerTranscoder(
            M.JumpReLU(0.03, 1.0, L, F), M.Encoder(D, F, L), M.CrosslayerDecoder(D, F, L),
            M.DimensionwiseInputStandardizer(L, D), M.DimensionwiseOutputStandardizer(L, D)))
        full.last_active.copy_(torch.arange(L * F).reshape(L, F))
        ref_sd = {k: v.clone() for k, v in full.state_dict().items()}
        lo, hi = parallel.feature_shard(F, rank, world)
        shard = M.JumpReLUCrossLayerTranscoderModule(model=M.CrossLayerTranscoder(
            M.JumpReLU(0.03, 1.0, L, hi - lo), M.Encoder(D, hi - lo, L), M.CrosslayerDecoder(D, hi - lo, L),
            M.DimensionwiseInputStandardizer(L, D), M.DimensionwiseOutputStandardizer(L, D)))
        shard.load_state_dict(parallel.shard_state_dict(ref_sd, rank, world))      # reference layout -> this rank's slice
        assert shard.model.encoder.W.shape == (L, D, hi - lo)
        back = parallel.gather_state_dict(shard)                                   # and back
        assert list(back) == list(ref_sd)
        for k in ref_sd:
            # (standardizer buffers are uninitialised memory here and may hold NaN patterns)
            assert back[k].shape == ref_sd[k].shape and torch.equal(back[k].nan_to_num(), ref_sd[k].nan_to_num()), k
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_sharded_checkpoint_round_trip_in_reference_layout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ckpt_worker, args=(r, 2, 29613, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(v == "ok" for _, v in res), res


def _configure_worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    import crosslayer_transcoder_b200.model as M
    from crosslayer_transcoder_b200 import parallel

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, D, F = 3, 8, 16
        for decoder_cls, nl in ((M.CrosslayerDecoder, M.JumpReLU(0.03, 1.0, L, F)), (M.Decoder, M.PerLayerTopK(k=2))):
            torch.manual_seed(11)
            full = M.CrossLayerTranscoderModule(model=M.CrossLayerTranscoder(
                nl, M.Encoder(D, F, L), decoder_cls(D, F, L),
                M.DimensionwiseInputStandardizer(L, D), M.DimensionwiseOutputStandardizer(L, D)))
            full.last_active.copy_(torch.arange(L * F).reshape(L, F))
            ref_sd = {k: v.clone() for k, v in full.state_dict().items()}
            full.trainer.num_devices = world
            full.configure_model()                       # the reference shards here (clt_lightning.py:106-119)
            assert full.tp_world == world and full.tp_rank == rank and not full.tp_fused
            lo, hi = parallel.feature_shard(F, rank, world)
            assert full.model.encoder.d_features == hi - lo and full.model.decoder.d_features == hi - lo
            want = parallel.shard_state_dict(ref_sd, rank, world)
            got = full.state_dict()
            assert list(got) == list(want)
            for k in want:
                if "standardizer" in k:
                    continue                             # uninitialised buffers
                assert got[k].shape == want[k].shape and torch.equal(got[k], want[k]), k
            assert all(p.requires_grad for p in full.parameters())
            full.configure_model()                       # a second call leaves the shard alone
            assert full.model.encoder.W.shape == (L, D, hi - lo)
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback

        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def test_configure_model_shards_an_unsharded_module():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_configure_worker, args=(r, 2, 29615, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(v == "ok" for _, v in res), res
