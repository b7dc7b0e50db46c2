"""Worker of the multi-GPU parity test: one process per GPU (launched by torch.distributed.run),
each holding one feature shard; rank 0 compares the gathered result with the unsharded CPU oracle."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from crosslayer_transcoder_b200 import parallel, synthetic  # noqa: E402
from oracle import clt_oracle as O  # noqa: E402
from tests.helpers import build_module, oracle_for_spec, rel_err, spec_inputs  # noqa: E402


def shard_weights(w, lo, hi, crosslayer):
    out = {"W_enc": w["W_enc"][:, :, lo:hi].contiguous(), "b_enc": w["b_enc"][:, lo:hi].contiguous(),
           "b_dec": w["b_dec"]}
    out["W_dec"] = [x[:, lo:hi].contiguous() for x in w["W_dec"]] if crosslayer else w["W_dec"][:, lo:hi].contiguous()
    if "theta" in w:
        out["theta"] = w["theta"][:, :, lo:hi].contiguous()
    return out


def uploader_case(mod, spec, batch, dev, join):
    """Three training steps fed by ``parallel.ShardedBatchUploader`` (every rank uploads its own token rows and
    copies their input halves to the peers) against the same steps fed with whole device batches: same losses,
    same parameters afterwards.  ``join``: "early" = ordered by the step's own last collective, "late" = by the
    uploader's own all-reduce at the end of backward."""
    import copy

    if join == "late":
        parallel.ShardedBatchUploader.late_join_bytes = 0
    g = torch.Generator().manual_seed(123)
    host = [(batch * (1.0 + 0.1 * i) + 0.01 * torch.randn(batch.shape, generator=g)).half().pin_memory()
            for i in range(3)]
    state0 = copy.deepcopy(mod.state_dict())
    la0 = mod.last_active.clone() if hasattr(mod, "last_active") else None

    def run(feed):
        mod.load_state_dict(state0)
        if la0 is not None:
            mod.last_active.copy_(la0)
        opt = mod.configure_optimizers()
        losses = []
        for i in range(3):
            b = feed(i)
            opt.zero_grad(set_to_none=True)
            loss = mod.training_step(b, i)
            loss.backward()
            opt.step()
            losses.append(float(loss))
            feed.done()
        mod._engine.check_status("uploader case")
        return losses, [p.detach().clone() for p in mod.parameters()]

    class Whole:
        def __call__(self, i):
            return host[i].to(dev)

        def done(self):
            pass

    class Uploaded:
        def __init__(self):
            self.up = parallel.ShardedBatchUploader(mod, host[0].shape, host[0].dtype, dev)
            assert self.up.late_join == (join == "late")
            self.up.upload(host[0], full=True)
            self.up.fence()

        def __call__(self, i):
            b = self.up.take()
            if i + 1 < len(host):
                self.up.upload(host[i + 1])
            return b

        def done(self):
            self.up.release()

    want_l, want_p = run(Whole())
    feed = Uploaded()
    got_l, got_p = run(feed)
    feed.up.detach()
    # Sums taken with atomics differ in their last bits from run to run, and Adam turns such a difference into a
    # step of up to lr wherever a gradient is at the rounding level (two runs of the SAME feed differ that way
    # too): the losses of all three steps must agree to 1e-4 — a wrong or stale row would move them by percents —
    # and no parameter may differ by more than a few steps of lr.
    ok = all(abs(a - b) <= 1e-4 * abs(b) for a, b in zip(got_l, want_l))
    worst = max(float((a - b).abs().max()) for a, b in zip(got_p, want_p))
    ok = ok and worst <= 3 * spec.lr
    if not ok:
        print("uploader case FAILED", got_l, want_l, "max |dp|", worst)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) else 1)


def main():
    kind, prec = sys.argv[1], sys.argv[2]
    mode = sys.argv[3] if len(sys.argv) > 3 else "nccl"     # "fused": exchange fused into the kernels over peer memory
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    dev = torch.device(f"cuda:{local}")
    bf16 = prec == "bf16"
    if kind == "jumprelu":
        spec = synthetic.WorkloadSpec("mp_jr", 3, 128, 512, 200, "jumprelu", True, bf16, rank_u=16, n_outlier=2,
                                      lambda_sparsity=4e-4, pre_actv_loss=3e-6, lr=1e-3)
    elif kind == "batchtopk":
        spec = synthetic.WorkloadSpec("mp_btk", 3, 128, 1024, 200, "batchtopk", True, bf16, rank_u=16, n_outlier=2, k=4,
                                      e=0.05, lr=1e-3)
    else:
        spec = synthetic.WorkloadSpec("mp_topk", 3, 128, 1024, 200, "topk", True, bf16, rank_u=16, n_outlier=2, k=8,
                                      k_aux=32, aux_loss_scale=1 / 32, tokens_till_dead=1000, dead_fraction=0.2,
                                      lr=1e-3)
    batch, w, la = spec_inputs(spec)
    lo, hi = parallel.feature_shard(spec.d_features, rank, world)
    mod = build_module(spec, shard_weights(w, lo, hi, spec.crosslayer), dev, last_active=la[:, lo:hi].contiguous())
    parallel.attach(mod, fused=(mode == "fused"))
    assert mod.tp_fused == (mode == "fused")
    if mode == "fused" and len(sys.argv) > 4:
        return uploader_case(mod, spec, batch, dev, sys.argv[4])
    loss = mod.training_step(batch.to(dev), 0)
    loss.backward()
    mod._engine.check_status("multi-GPU step")
    m = mod.model
    thr_after_first = m.nonlinearity.threshold.clone() if kind == "batchtopk" else None
    if mode == "fused":
        # a second step on the same weights reuses the peer buffers: it must reproduce the first one
        first = [p.grad.clone() for p in mod.parameters() if p.grad is not None]
        la_first = mod.last_active.clone()
        mod.last_active.copy_(la[:, lo:hi].to(dev))
        for p in mod.parameters():
            p.grad = None
        loss2 = mod.training_step(batch.to(dev), 1)
        loss2.backward()
        second = [p.grad for p in mod.parameters() if p.grad is not None]
        same = abs(float(loss2) - float(loss)) <= 1e-6 * abs(float(loss)) and all(
            rel_err(a, b) < 1e-5 for a, b in zip(second, first)) and torch.equal(mod.last_active, la_first)
        assert same, "the second step on the same weights differs from the first"
    # gather the feature-sharded gradients on every rank
    def gather(t, dim):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return torch.cat(parts, dim=dim).cpu()

    g_enc = gather(m.encoder.W.grad, 2)
    g_benc = gather(m.encoder.b.grad, 1)
    g_dec = [gather(x.grad, 1) for x in m.decoder.blocks()]
    g_bdec = m.decoder.b.grad.cpu()
    la_out = gather(mod.last_active, 1)
    ok = True
    if rank == 0:
        P, H, stats, kw = oracle_for_spec(spec, batch, w, la)
        ref, rg = O.step_with_grads(P, batch, stats, H, **kw)
        tol = 2e-2 if bf16 else 1e-4
        errs = {"loss": rel_err(loss.detach().cpu(), ref.loss), "W_enc": rel_err(g_enc, rg[0]),
                "b_enc": rel_err(g_benc, rg[1]), "b_dec": rel_err(g_bdec, rg[2 + len(g_dec)])}
        for t, g in enumerate(g_dec):
            errs[f"W_dec{t}"] = rel_err(g, rg[2 + t])
        bad = {k: v for k, v in errs.items() if not v < tol}
        if kind == "topk" and not torch.equal(la_out, ref.last_active):
            bad["last_active"] = 1.0
        if kind == "batchtopk":
            errs["threshold"] = rel_err(thr_after_first.cpu(), ref.threshold)
            if not errs["threshold"] < tol:
                bad["threshold"] = errs["threshold"]
        print("errors", errs)
        ok = not bad
        if bad:
            print("FAILED", bad)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) else 1)


if __name__ == "__main__":
    main()
