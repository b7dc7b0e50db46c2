"""Time the UNMODIFIED reference training step (``training_step`` -> ``backward`` -> the optimizer the
reference's ``configure_optimizers`` returns).  TEST / BENCHMARK INFRASTRUCTURE ONLY.

Used by the benchmark's reference arm and by ``tests/golden/make_golden.py``.  The reference modules
are imported as they are by ``oracle/ref_import.py`` (crosslayer_transcoder/model/clt_lightning.py:290-312,
420-475, 519-567 are the steps that run; crosslayer_transcoder/model/clt_lightning.py:333-392 the optimizer).

Run as a program it prints one JSON object:

    python -m oracle.ref_step --workload c3_clt_topk_bf16 --steps 1 --warmup 1 [--device cpu|cuda]
                              [--override n_layers=2] [--mem-limit-gb G]

``--mem-limit-gb`` caps the process's address space so that a shape that does not fit the host ends in a
``MemoryError`` (exit code 3) instead of the machine running out of memory.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import resource
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from crosslayer_transcoder_b200 import synthetic  # noqa: E402
from oracle import ref_import  # noqa: E402


def build_reference_module(ref, spec, weights=None, last_active=None, device="cpu"):
    """The reference's Lightning module for ``spec``.  ``weights`` (a dict as ``synthetic.make_weights``
    returns) are copied in when given; otherwise the parameters are drawn in place from the benchmark
    configurations' distributions (same bounds, seeded), which avoids holding a second copy of a
    multi-GB model."""
    clt, jr, tk, st, cl = ref.clt, ref.jumprelu, ref.topk, ref.standardize, ref.clt_lightning
    L, D, F = spec.n_layers, spec.d_acts, spec.d_features
    with torch.device(device):
        enc = clt.Encoder(D, F, L)
        dec = (clt.CrosslayerDecoder if spec.crosslayer else clt.Decoder)(D, F, L)
        if spec.kind == "jumprelu":
            nl = jr.JumpReLU(theta=spec.theta, bandwidth=spec.bandwidth, n_layers=L, d_features=F)
        elif spec.kind == "topk":
            nl = tk.PerLayerTopK(k=spec.k)
        else:
            nl = tk.BatchTopK(k=spec.k, e=spec.e)
        model = clt.CrossLayerTranscoder(nl, enc, dec, st.DimensionwiseInputStandardizer(L, D),
                                         st.DimensionwiseOutputStandardizer(L, D))
    with torch.no_grad():
        if weights is not None:
            enc.W.copy_(weights["W_enc"])
            enc.b.copy_(weights["b_enc"])
            dec.b.copy_(weights["b_dec"])
            if spec.crosslayer:
                for t in range(L):
                    dec.get_parameter(f"W_{t}").copy_(weights["W_dec"][t])
            else:
                dec.W.copy_(weights["W_dec"])
        else:
            g = torch.Generator(device=device).manual_seed(1234)
            enc.W.uniform_(-D ** -0.5, D ** -0.5, generator=g)
            enc.b.zero_()
            dec.b.zero_()
            bound = (L * F) ** -0.5 if spec.crosslayer else F ** -0.5
            for name, p in dec.named_parameters():
                if name != "b":
                    p.uniform_(-bound, bound, generator=g)
    common = dict(model=model, learning_rate=spec.lr, log_metrics_every=10 ** 9)
    if spec.kind == "jumprelu":
        mod = cl.JumpReLUCrossLayerTranscoderModule(lambda_sparsity=spec.lambda_sparsity, c_sparsity=spec.c_sparsity,
                                                    use_tanh=spec.use_tanh, pre_actv_loss=spec.pre_actv_loss, **common)
        mod.trainer.max_steps = 1
        mod.global_step = 1          # lambda ramp factor global_step / max_steps = 1
    elif spec.kind == "topk":
        mod = cl.TopKCrossLayerTranscoderModule(topk_aux=tk.PerLayerTopK(k=spec.k_aux),
                                                tokens_till_dead=spec.tokens_till_dead,
                                                aux_loss_scale=spec.aux_loss_scale, **common)
        if last_active is not None:
            mod.last_active.copy_(last_active)
    else:
        mod = cl.CrossLayerTranscoderModule(**common)
    return mod.to(device)


def time_reference(spec, steps: int, warmup: int, device: str = "cpu", threads: int = 0) -> dict:
    """Wall-clock seconds per step of the reference module on ``device`` (all host cores for "cpu")."""
    ref = ref_import.load(with_lightning=True)
    cores = threads or os.cpu_count() or 1
    torch.set_num_threads(cores)
    dev = torch.device(device)
    batch = synthetic.make_batch(spec, seed=0, device=device if dev.type == "cuda" else "cpu")
    la = None
    if spec.kind == "topk":
        la = synthetic.make_last_active(spec)
    mod = build_reference_module(ref, spec, None, la, device=device)
    if spec.kind == "topk" and la is not None:
        with torch.no_grad():       # seeded dead features stay dead (same device as the benchmark's own arm)
            mod.model.encoder.b[(la > spec.tokens_till_dead).to(dev)] = -1.0
    opt = mod.configure_optimizers()
    if isinstance(opt, dict):
        opt = opt["optimizer"]
    if spec.bf16:
        ctx = lambda: torch.autocast(dev.type, dtype=torch.bfloat16)
    else:
        ctx = contextlib.nullcontext
    times, loss = [], None
    mod.model.initialize_standardizers(batch)       # what training_step does at batch_idx 0
    for i in range(1, warmup + steps + 1):          # (batch_idx 0 would also run the heavy metrics block)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        with ctx():
            loss = mod.training_step(batch, i)
        loss.backward()
        opt.step()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if i > warmup:
            times.append(dt)
    times.sort()
    med = times[len(times) // 2]
    return {"step_s": med, "steps": steps, "warmup": warmup, "tokens_per_s": spec.batch / med, "cores": cores,
            "device": device, "loss": float(loss), "maxrss_gb": resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 1e6}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", required=True)
    ap.add_argument("--override", default="")
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--mem-limit-gb", type=float, default=0.0)
    a = ap.parse_args()
    if a.mem_limit_gb > 0:
        lim = int(a.mem_limit_gb * 1e9)
        resource.setrlimit(resource.RLIMIT_AS, (lim, lim))
    spec = synthetic.WORKLOADS[a.workload]
    if a.override:
        over = {}
        for kv in a.override.split(","):
            k, v = kv.split("=")
            over[k] = type(getattr(spec, k))(v)
        spec = synthetic.scaled(spec, **over)
    try:
        r = time_reference(spec, a.steps, a.warmup, a.device)
    except (MemoryError, RuntimeError) as e:
        msg = str(e).splitlines()[0] if str(e) else type(e).__name__
        if isinstance(e, MemoryError) or "alloc" in msg.lower() or "out of memory" in msg.lower():
            print(json.dumps({"error": "out of memory", "detail": msg[:200]}))
            sys.exit(3)
        raise
    print(json.dumps(r))


if __name__ == "__main__":
    main()
