"""Benchmark of the crosslayer-transcoder training step (forward + backward + Adam).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line (rank 0).  ``value`` is training tokens/s with the batch already
resident in HBM; ``e2e`` is the same metric through the public module API with the batch
copied from pinned host memory and the loss read back every step; ``roofline`` describes
the kernel with the largest share of the timed region; ``cpu_baseline`` is the reference's own
training step (unmodified modules, CPU PyTorch) timed on this host on a bounded sample.

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N bench.py --gpus N``:
the feature axis is sharded over the ranks, every rank sees the same batch (strong scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from crosslayer_transcoder_b200 import synthetic  # noqa: E402

METRIC = "clt_train_tokens_per_s"
UNIT = "tokens/s"
DEFAULT_WORKLOAD = "c3_clt_topk_bf16"

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernels from
# the ncu captures summarised under profiles/; None where no capture has been taken.
# Adam: 29.83 B/parameter (profiles/adam_kernel_c3_4layer.md), scaled by the parameter count at run time.
# Fused decoder backward + Adam: 26.45 B/decoder parameter (profiles/sparse_bwd_dec_adam_kernel_c3_4layer.md).
NCU_TRAFFIC_PER_UNIT = {"clt_adam_step": 29.83, "clt_sparse_bwd_dec_adam": 26.45}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------
# workload construction
# --------------------------------------------------------------------------------------
STATIONARY_TOKENS_TILL_DEAD = 10 ** 12      # no live feature can cross this during a benchmark run


def bench_spec(spec):
    """The workload as the benchmark runs it: the TopK configuration's seeded dead features stay dead and no
    live feature dies during the run (``tokens_till_dead`` far beyond the tokens of the run), so every step
    does the same work."""
    if spec.kind == "topk":
        return synthetic.scaled(spec, tokens_till_dead=STATIONARY_TOKENS_TILL_DEAD)
    return spec


def draw_weights(mod_enc, mod_dec, spec, dev, lo: int, hi: int):
    """Seeded weights of the benchmark configurations, identical for every number of ranks: each encoder
    layer and each decoder block is drawn whole from its own seed on the device and this rank keeps its
    feature slice ``[lo, hi)``.  (The loss after the same number of steps therefore agrees across 1/2/4/8
    GPUs up to summation order.)"""
    L, D, F = spec.n_layers, spec.d_acts, spec.d_features
    g = torch.Generator(device=dev)
    with torch.no_grad():
        for l in range(L):
            g.manual_seed(1234 + l)
            full = (torch.rand(D, F, device=dev, generator=g) * 2 - 1) / D ** 0.5
            mod_enc.W[l].copy_(full[:, lo:hi])
        bound = (L * F) ** -0.5 if spec.crosslayer else F ** -0.5
        p = 0
        for w in mod_dec.blocks():
            for s_ in range(w.shape[0]):
                g.manual_seed(100_000 + p)
                full = (torch.rand(F, D, device=dev, generator=g) * 2 - 1) * bound
                w[s_].copy_(full[lo:hi])
                p += 1
        del full


def build_on_device(spec: synthetic.WorkloadSpec, dev, rank: int, world: int, exchange: str = "auto"):
    """The package's training module for this rank's feature shard, weights drawn on the device."""
    import crosslayer_transcoder_b200.model as M
    from crosslayer_transcoder_b200 import parallel

    L, D, F = spec.n_layers, spec.d_acts, spec.d_features
    lo, hi = parallel.feature_shard(F, rank, world)
    Fl = hi - lo
    with torch.device(dev):
        enc = M.Encoder(D, Fl, L)
        dec = (M.CrosslayerDecoder if spec.crosslayer else M.Decoder)(D, Fl, L)
        if spec.kind == "jumprelu":
            nl = M.JumpReLU(theta=spec.theta, bandwidth=spec.bandwidth, n_layers=L, d_features=Fl)
        elif spec.kind == "topk":
            nl = M.PerLayerTopK(k=spec.k)
        else:
            nl = M.BatchTopK(k=spec.k, e=spec.e)
        model = M.CrossLayerTranscoder(nl, enc, dec, M.DimensionwiseInputStandardizer(L, D),
                                       M.DimensionwiseOutputStandardizer(L, D))
    draw_weights(enc, dec, spec, dev, lo, hi)
    common = dict(model=model, learning_rate=spec.lr, tokens_till_dead=spec.tokens_till_dead,
                  log_metrics_every=0)      # the metrics block is not part of the timed step
    if spec.kind == "jumprelu":
        mod = M.JumpReLUCrossLayerTranscoderModule(lambda_sparsity=spec.lambda_sparsity, c_sparsity=spec.c_sparsity,
                                                   use_tanh=spec.use_tanh, pre_actv_loss=spec.pre_actv_loss, **common)
        mod.trainer.max_steps = 1
        mod.global_step = 1
    elif spec.kind == "topk":
        mod = M.TopKCrossLayerTranscoderModule(topk_aux=M.PerLayerTopK(k=spec.k_aux),
                                               aux_loss_scale=spec.aux_loss_scale, **common)
        la = synthetic.make_last_active(spec, f_lo=lo, f_hi=hi)
        mod.last_active.copy_(la)
        # Features marked dead get an encoder bias of -1: like dead features in a real run they stay out of
        # the top-k (so they stay dead) while a few per cent of their pre-activations are still positive,
        # which is what the auxiliary loss works on.  With the plain random weights every "dead" feature
        # would fire within a step and the auxiliary path would see almost no dead features.
        with torch.no_grad():
            enc.b[(la > spec.tokens_till_dead).to(enc.b.device)] = -1.0
    else:
        mod = M.CrossLayerTranscoderModule(**common)
    mod = mod.to(dev)
    mod.precision = "bf16" if spec.bf16 else "fp32"
    if world > 1:
        parallel.attach(mod, fused={"nccl": False, "fused": True, "auto": "auto"}[exchange])
    return mod


def algorithmic_work(spec, world: int, Fl: int, n_params: int, batch_bytes_per_elem: int, nd_pad: int = 0,
                     fused_exchange: bool = False, candidate_list: bool = True):
    """Per-launch algorithmic FLOPs / bytes of every entry point ON THIS RANK (feature shard Fl = F / world).
    Dense contractions: 2 M N K.  HBM-bound kernels: the bytes the operation has to move once.  Gathers have
    two figures: the token-major count (every fetched row counted, L2 hits included) and the lower bound
    with perfect row reuse, min(rows fetched, rows that exist); the fraction reported is of the lower bound.
    Returns {entry point: (bound, amount)} or (bound, amount, token_major_amount)."""
    B, L, D = spec.batch, spec.n_layers, spec.d_acts
    P = L * (L + 1) // 2 if spec.crosslayer else L
    e = 2 if spec.bf16 else 4
    Fd = nd_pad if spec.kind == "topk" else Fl        # width of the dense decoder-side contractions
    enc = 2.0 * B * L * D * Fl
    dec = 2.0 * B * P * Fd * D
    bld = float(B) * L * D
    own = bld / world if fused_exchange else bld       # rows whose loss this rank computes
    k = max(spec.k, 1)
    rows = float(B) * k * P / world                    # decoder rows fetched by the sparse forward (expected per shard)
    rows_unique = min(rows, float(P) * Fl)
    ent = float(L) * B * k / world                     # selected entries on this shard (expected)
    aux = 1 if spec.k_aux else 0
    sparse_fwd = ("hbm", rows_unique * D * e + bld * 4, rows * D * e + bld * 4)
    work = {
        "clt_encoder_fwd_act": ("tensor", enc), "clt_encoder_fwd_store": ("tensor", enc),
        # the auxiliary path's own encoder contraction over the compact dead columns, and the gather that builds
        # its operand (touches most sectors of the encoder weights: counted as one read of them)
        "clt_encoder_fwd_store[dead]": ("tensor", 2.0 * B * L * D * nd_pad),
        "clt_gather_enc_cols": ("hbm", float(L) * D * Fl * e + float(L) * D * nd_pad * e),
        "clt_encoder_dense_bwd_dw": ("tensor", 2.0 * B * L * D * Fd if spec.kind == "topk" else enc),
        "clt_decoder_dense_fwd": ("tensor", dec), "clt_decoder_dense_fwd_push": ("tensor", dec),
        "clt_decoder_dense_bwd_dfeat": ("tensor", dec), "clt_decoder_dense_bwd_dw": ("tensor", dec),
        "clt_decoder_dense_bwd_dfeat_raw": ("tensor", dec),
        "clt_act_fwd": ("hbm", float(B) * L * Fl * e * 2), "clt_act_bwd": ("hbm", float(B) * L * Fl * e * 3),
        "clt_adam_step": ("hbm", n_params * (28.0 + (2 if spec.bf16 else 0))),      # n_params: see the caller
        "clt_prep_input": ("hbm", bld * (batch_bytes_per_elem + e)),
        "clt_loss_fwd": ("hbm", own * (4 + batch_bytes_per_elem + 4 * aux)),
        "clt_loss_bwd": ("hbm", bld * (4 + batch_bytes_per_elem + e + (4 + e) * aux)),
        # owned rows read locally; the gradient rows written once into every rank's buffer
        "clt_loss_bwd_push": ("hbm", own * (4 + batch_bytes_per_elem + 4 * aux) + own * world * e * (1 + aux)),
        # the owner reads its R slots (bf16 on the bf16 path, fp32 otherwise) and writes the fp32 sum
        "clt_sum_slots": ("hbm", own * (e * world + 4)),
        "clt_dec_norms": ("hbm", float(P) * Fl * D * 4),
        "clt_select_topk": ("hbm", float(L) * B * Fl * e + float(L) * B * k * 8),
        "clt_select_aux": ("hbm", float(L) * B * nd_pad * e * 2),
        "clt_aux_count": ("hbm", float(L) * B * nd_pad * e),
        "clt_topk_threshold": ("hbm", float(L) * B * k * 4 * world + float(L) * B * 4),
        "clt_topk_apply_threshold": ("hbm", float(L) * B * k * 8 * 2),
        "clt_sparse_decoder_fwd": sparse_fwd, "clt_sparse_decoder_fwd_push": sparse_fwd,
        "clt_sparse_bwd_dec": ("hbm", float(P) * Fl * D * (e + 4)),
        # read p, m, v; write p, m, v (+ the bf16 copy): the gradient and the operand copy never touch memory
        "clt_sparse_bwd_dec_adam": ("hbm", float(P) * Fl * D * (24 + (2 if spec.bf16 else 0))),
        "clt_sparse_bwd_enc": ("hbm", float(L) * D * Fl * 4 + ent * D * e),
        "clt_gather_rows": ("hbm", float(P) * nd_pad * D * e * 2),
        "clt_scatter_rows": ("hbm", float(P) * nd_pad * D * 4 * 3),
        "clt_csc_build": ("hbm", float(L) * B * k * 8 * 2 + float(L) * Fl * 4 * 3),
        # the one sweep of the selection's steady state; the full-sweep entry points (clt_batchtopk_hist,
        # clt_batchtopk_collect) are enqueued every step and return at once unless a step falls back to them,
        # so they carry no work model when the candidate list is in use
        "clt_batchtopk_candidates": ("hbm", float(L) * B * Fl * e),
        "clt_batchtopk_hist": ("hbm", float(L) * B * Fl * e),
        "clt_batchtopk_collect": ("hbm", float(L) * B * Fl * e + float(L) * B * k * 12),
    }
    if candidate_list:
        del work["clt_batchtopk_hist"], work["clt_batchtopk_collect"]
    return work


# --------------------------------------------------------------------------------------
# CPU arm: the reference's own training step on the host cores
# --------------------------------------------------------------------------------------
def dense_flops(s) -> float:
    """Dense work of the REFERENCE's step (it runs every decoder product densely; the TopK module runs the
    decoder a second time for the auxiliary loss): what its step time scales with."""
    Pn = s.n_layers * (s.n_layers + 1) // 2 if s.crosslayer else s.n_layers
    passes = 2.0 if (s.kind == "topk" and s.k_aux) else 1.0
    return 4.0 * s.batch * s.n_layers * s.d_acts * s.d_features + passes * 6.0 * s.batch * Pn * s.d_features * s.d_acts


def time_cpu_port(spec, steps: int = 1, warmup: int = 1):
    """Fallback when the reference modules are not on this machine: the oracle restatement of the step
    (``oracle/clt_oracle.py``) on the same 2-layer sample."""
    from oracle import clt_oracle as O

    sample = synthetic.scaled(spec, n_layers=2, name=spec.name + "_cpu_sample")
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    batch = synthetic.make_batch(sample, seed=5)
    g = torch.Generator().manual_seed(6)
    L, D, F = sample.n_layers, sample.d_acts, sample.d_features
    W_enc = (torch.rand(L, D, F, generator=g) * 2 - 1) / D ** 0.5
    if sample.crosslayer:
        W_dec = [(torch.rand(t + 1, F, D, generator=g) * 2 - 1) / (spec.n_layers * F) ** 0.5 for t in range(L)]
    else:
        W_dec = (torch.rand(L, F, D, generator=g) * 2 - 1) / F ** 0.5
    theta = torch.full((1, L, F), sample.theta) if sample.kind == "jumprelu" else None
    P = O.Params(W_enc, torch.zeros(L, F), W_dec, torch.zeros(L, D), theta)
    H = O.Hyper(kind=sample.kind, bf16=sample.bf16, bandwidth=sample.bandwidth,
                lambda_sparsity=sample.lambda_sparsity, c_sparsity=sample.c_sparsity, use_tanh=sample.use_tanh,
                pre_actv_loss=sample.pre_actv_loss, k=sample.k, k_aux=sample.k_aux,
                aux_loss_scale=sample.aux_loss_scale, tokens_till_dead=sample.tokens_till_dead, e=sample.e)
    stats = O.standardizer_stats(batch)
    kw = {}
    if sample.kind == "topk":
        kw["last_active"] = synthetic.make_last_active(sample)
    if sample.kind == "batchtopk":
        kw["threshold"] = torch.zeros(1)
    state = [(torch.zeros_like(t), torch.zeros_like(t)) for t in P.tensors()]
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        out, grads = O.step_with_grads(P, batch, stats, H, **kw)
        new = []
        for t, gr, (m, v) in zip(P.tensors(), grads, state):
            p2, m2, v2 = O.adam_step(t, gr, m, v, i + 1, sample.lr)
            t.copy_(p2)
            new.append((m2, v2))
        state = new
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    scale = dense_flops(spec) / dense_flops(sample)
    t_med = statistics.median(times)
    return {"cores": cores, "kind": "port", "sample_step_s": t_med, "scale": scale, "full": False,
            "tokens_per_s": spec.batch / (t_med * scale), "step_s": t_med, "steps": steps, "warmup": warmup,
            "sample": f"CPU restatement of the reference step (the reference modules are not on this machine); "
                      f"2 of {spec.n_layers} layers at full B/D/F timed ({t_med:.2f} s per step), step time scaled "
                      f"by the dense-work ratio {scale:.1f} (extrapolated)"}


def _run_ref_step(workload: str, override: str, steps: int, warmup: int, mem_limit_gb: float, timeout_s: float):
    """One run of ``oracle/ref_step.py`` in a child process (its own address-space limit and time limit);
    returns its JSON, or {"error": ...}."""
    cmd = [sys.executable, "-m", "oracle.ref_step", "--workload", workload, "--steps", str(steps), "--warmup",
           str(warmup), "--device", "cpu"]
    if override:
        cmd += ["--override", override]
    if mem_limit_gb > 0:
        cmd += ["--mem-limit-gb", f"{mem_limit_gb:.1f}"]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, cwd=str(ROOT))
    except subprocess.TimeoutExpired:
        return {"error": f"no result within {timeout_s:.0f} s"}
    for ln in reversed(r.stdout.strip().splitlines()):
        if ln.startswith("{"):
            return json.loads(ln)
    return {"error": f"exit code {r.returncode}: {r.stderr.strip().splitlines()[-1] if r.stderr.strip() else ''}"[:300]}


def host_mem_available_gb() -> float:
    try:
        for ln in Path("/proc/meminfo").read_text().splitlines():
            if ln.startswith("MemAvailable:"):
                return float(ln.split()[1]) / 1e6
    except OSError:
        pass
    return 0.0


def time_cpu_reference(spec, workload: str, override: str, full_budget_s: float):
    """The unmodified reference step on the host cores.  First a bounded sample (2 layers, everything else
    as in the workload; one warm-up step and one timed step).  If the sample predicts that ONE full-shape
    step fits ``full_budget_s`` and the host has the memory, the full workload is timed as it is (no
    extrapolation); otherwise the sample's step time is scaled by the dense-work ratio and labelled so."""
    from oracle import ref_import

    kind = "reference"
    if not ref_import.available():
        return time_cpu_port(spec)
    over = (override + "," if override else "") + "n_layers=2"
    sample_spec = synthetic.scaled(spec, n_layers=2)
    s = _run_ref_step(workload, over, 1, 1, 0.0, 600)
    if "error" in s:
        return {"error": "sample: " + s["error"]}
    scale = dense_flops(spec) / dense_flops(sample_spec)
    predicted = s["step_s"] * scale
    out = {"cores": s["cores"], "kind": kind, "sample_step_s": s["step_s"], "scale": scale, "full": False,
           "tokens_per_s": spec.batch / predicted, "step_s": s["step_s"], "steps": 1, "warmup": 1,
           "sample": f"unmodified reference modules; 2 of {spec.n_layers} layers at full B/D/F timed "
                     f"({s['step_s']:.2f} s per step), step time scaled by the dense-work ratio {scale:.1f} "
                     f"(extrapolated)"}
    # memory of the full shape: fp32 p/g/m/v, plus the sample's activation footprint grown with the layer
    # count (dense [B, L, F] intermediates) and the block count (per-target operand copies); errs high
    def n_par(sp):
        Pn = sp.n_layers * (sp.n_layers + 1) // 2 if sp.crosslayer else sp.n_layers
        return sp.n_layers * sp.d_acts * sp.d_features + Pn * sp.d_features * sp.d_acts

    Pf = spec.n_layers * (spec.n_layers + 1) // 2 if spec.crosslayer else spec.n_layers
    act_sample = max(0.0, s["maxrss_gb"] - 16.0 * n_par(sample_spec) / 1e9)
    need_gb = 16.0 * n_par(spec) / 1e9 + act_sample * (0.5 * spec.n_layers / 2 + 0.5 * Pf / (3 if spec.crosslayer else 2))
    avail = host_mem_available_gb()
    if full_budget_s > 0 and spec.n_layers > 2 and predicted <= full_budget_s and need_gb < 0.8 * avail:
        wu = 1 if 2 * predicted <= full_budget_s else 0
        k = max(1, min(3, int(full_budget_s / max(predicted, 1e-3)) - wu))
        f = _run_ref_step(workload, override, k, wu, 0.9 * avail, 1.6 * full_budget_s + 60)
        if "error" not in f:
            out.update(full=True, tokens_per_s=f["tokens_per_s"], step_s=f["step_s"], steps=k, warmup=wu,
                       sample=f"unmodified reference modules at the full workload shape, median of {k} step(s) "
                              f"after {wu} warm-up ({f['step_s']:.2f} s per step, no extrapolation)")
        else:
            out["sample"] += f"; the full-shape run gave: {f['error']}"
    return out


# --------------------------------------------------------------------------------------
def time_ingest(spec, dev, batches: int = 10) -> dict:
    """Batch ingestion from the reference's activation store, both ways, on this machine: the reference's own
    consumer (``SharedActivationBuffer.get_activations`` on one CPU thread, then the upload of the pageable
    batch it returns) against the device-side consumer (``data.SharedBufferBatches``: the GPU gathers the
    same choice of rows from the registered shared mapping).  ms per batch of ``spec.batch`` rows."""
    import faulthandler
    import gc
    import shutil

    from crosslayer_transcoder_b200 import data
    from oracle import ref_import

    faulthandler.enable()           # a crash in native code names the Python frame it came from
    shm_mod = ref_import.load_shared_memory()
    if shm_mod is None:
        return {"unavailable": "the reference's shared_memory.py is not present (oracle/_ref missing)"}
    B, L, D = spec.batch, spec.n_layers, spec.d_acts
    n = 3 * B
    need = n * 2 * L * D * 2
    if shutil.disk_usage("/dev/shm").free < need + (256 << 20):
        return {"unavailable": f"/dev/shm has less than {need >> 20} MiB free"}
    store = shm_mod.SharedActivationBuffer(buffer_size=n, n_in_out=2, n_layers=L, activation_dim=D,
                                           dtype=torch.float16, generation_batch_size=1, max_sequence_length=64,
                                           batch_size=B)
    try:
        chunk = torch.randn(500, 2, L, D).half()
        for i in range(0, n, 500):
            store.buffer_tensor[i:i + 500] = chunk[: min(500, n - i)]
        store.validity_tensor.fill_(True)
        t_get, t_all = [], []
        for _ in range(batches):
            t0 = time.perf_counter()
            x = store.get_activations(B)
            t1 = time.perf_counter()
            x.to(dev)
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            t_get.append(t1 - t0)
            t_all.append(t2 - t0)
            store.validity_tensor.fill_(True)
        t_get.sort()
        t_all.sort()
        out = {"rows_per_batch": B, "bytes_per_batch": B * 2 * L * D * 2,
               "reference_get_activations_ms": 1e3 * t_get[len(t_get) // 2],
               "reference_with_upload_ms": 1e3 * t_all[len(t_all) // 2]}
        for mode in ("mapped", "staged"):
            src = data.SharedBufferBatches(store, B, device=dev, depth=2, mode=mode)
            try:
                for _ in range(3):
                    next(src)
                    store.validity_tensor.fill_(True)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(batches):
                    next(src)
                    store.validity_tensor.fill_(True)
                torch.cuda.synchronize()
                out[f"device_consumer_{mode}_ms"] = 1e3 * (time.perf_counter() - t0) / batches
                src.gather.check()
            finally:
                src.close()
                del src
                gc.collect()
        out["mapped_gather_GBps"] = out["bytes_per_batch"] / out["device_consumer_mapped_ms"] / 1e6
        return out
    finally:
        store.cleanup()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0,
                    help="timed steps; 0 (default) = as many as fill about 3 s of device time")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(synthetic.WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"],
                    help="ours: this package; reference: the unmodified reference step on the host cores; "
                         "reference-gpu: the same unmodified reference modules on cuda:0 (eager PyTorch)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", choices=["nccl", "fused", "auto"], default="auto",
                    help="feature shards: sum the partial reconstructions with NCCL, or fused into the kernels "
                         "over peer memory; auto = fused where available")
    ap.add_argument("--override", default="", help="comma-separated field=value changes to the workload "
                    "(reduced shapes for profiler captures; the result is then not a benchmark value)")
    ap.add_argument("--no-fuse-optimizer", action="store_true",
                    help="TopK / BatchTopK workloads: keep the decoder's Adam update in the optimizer kernel "
                         "instead of applying it inside the sparse decoder backward (module.fuse_optimizer)")
    ap.add_argument("--gather-form", choices=["auto", "warp", "cta"], default="auto",
                    help="form of the token-major decoder gather (module.decoder_gather_warp); auto = the engine's rule")
    ap.add_argument("--ingest", action="store_true",
                    help="1 GPU: also time batch ingestion from the reference's shared-memory activation store "
                         "(its own consumer vs the device-side one) and add an `ingest` object to the line")
    ap.add_argument("--ref-full-budget-s", type=float, default=150.0,
                    help="--impl reference: time the full workload shape if one step is predicted to fit this")
    args = ap.parse_args()
    spec = synthetic.WORKLOADS[args.workload]
    if args.override:
        over = {}
        for kv in args.override.split(","):
            k, v = kv.split("=")
            over[k] = type(getattr(spec, k))(v)
        spec = synthetic.scaled(spec, name=spec.name + "[" + args.override + "]", **over)
    spec = bench_spec(spec)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": spec.name, "kind": spec.kind, "decoder": "crosslayer" if spec.crosslayer else "per-layer",
              "n_layers": spec.n_layers, "d_acts": spec.d_acts, "d_features": spec.d_features,
              "batch_tokens": spec.batch, "sharding": f"d_features/{world}",
              "l2": "inputs_larger_than_l2 (batch and activations are hundreds of MB to GB per step)",
              "weights": "seeded per layer / decoder block, identical for every number of GPUs"}
    if spec.kind == "topk":
        config["dead_features"] = (f"{spec.dead_fraction:.0%} seeded dead (last_active beyond tokens_till_dead), their "
                                   "encoder bias set to -1 so they stay dead; b_enc = 0 elsewhere; no feature dies "
                                   "during the run (stationary work per step)")
    dtype_name = "bf16" if spec.bf16 else "fp32"

    if args.impl in ("reference", "reference-gpu"):
        if rank != 0:
            return
        base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic", "config": config}
        if args.impl == "reference-gpu":
            from oracle import ref_step

            try:
                r = ref_step.time_reference(spec, steps=max(1, min(args.steps or 3, 5)), warmup=1, device="cuda:0")
            except Exception as e:          # typically torch.OutOfMemoryError at the full shapes
                print(json.dumps({"impl": "reference", "unavailable": f"reference on cuda:0: {type(e).__name__}: "
                                  f"{str(e).splitlines()[0][:160]}"}))
                return
            base.update(value=r["tokens_per_s"], steps=r["steps"], warmup=r["warmup"], ms_per_step=1e3 * r["step_s"],
                        reference_device="cuda:0 (eager PyTorch, bf16 autocast, torch.optim.Adam(fused=True))",
                        last_loss=r["loss"])
            print(json.dumps(base))
            return
        r = time_cpu_reference(spec, args.workload, args.override, args.ref_full_budget_s)
        if r is None or "error" in r:
            why = "the reference modules are not available (oracle/_ref missing)" if r is None else r["error"]
            print(json.dumps({"impl": "reference", "unavailable": why}))
            return
        base.update(value=r["tokens_per_s"], steps=r["steps"], warmup=r["warmup"], ms_per_step=1e3 * r["step_s"],
                    cpu_baseline={"value": r["tokens_per_s"], "unit": UNIT, "cores": r["cores"], "kind": r["kind"],
                                  "sample": r["sample"], "full_shape": r["full"]},
                    e2e={"value": r["tokens_per_s"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        if not r["full"]:
            base["note"] = ("ms_per_step is the timed 2-layer sample's step; value = batch_tokens / (ms_per_step x "
                            f"{r['scale']:.1f})")
        print(json.dumps(base))
        return

    import torch.distributed as dist

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    mod = build_on_device(spec, dev, rank, world, args.exchange)
    fused_exchange = bool(getattr(mod, "tp_fused", False))
    if world > 1:
        config["exchange"] = "fused into the kernels over peer memory" if fused_exchange else "nccl"
    if spec.kind in ("topk", "batchtopk") and not args.no_fuse_optimizer:
        mod.fuse_optimizer = True
        config["optimizer"] = ("Adam; the decoder's update is applied inside the sparse decoder backward "
                               "(module.fuse_optimizer=True: same result as the separate optimizer kernel, the "
                               "decoder gradient is never stored), the other parameters in the optimizer kernel")
    else:
        config["optimizer"] = "Adam, one kernel over the flat parameter buffer"
    if args.gather_form != "auto":
        mod.decoder_gather_warp = args.gather_form == "warp"
        config["decoder_gather"] = args.gather_form
    opt = mod.configure_optimizers()
    eng = mod._engine
    # fp16 activations (the reference's storage dtype), drawn on the device (same on every rank), with a pinned
    # host copy for the end-to-end arm
    batch_dev = synthetic.make_batch(spec, seed=0, dtype=torch.float16, device=dev)
    batch_host = torch.empty(batch_dev.shape, dtype=batch_dev.dtype).pin_memory()
    batch_host.copy_(batch_dev)
    torch.cuda.synchronize()

    def step(b, idx):
        opt.zero_grad(set_to_none=True)
        loss = mod.training_step(b, idx)
        loss.backward()
        opt.step()
        return loss

    warmup = max(args.warmup, 3)
    for i in range(warmup):
        step(batch_dev, i)
    eng.check_status("warm-up")
    steps = args.steps
    if steps <= 0:
        # as many steps as fill about 3 s: time two more (untimed for the result) to size the region
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for i in range(2):
            step(batch_dev, 50 + i)
        c1.record()
        torch.cuda.synchronize()
        t = torch.tensor([c0.elapsed_time(c1) / 2], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        steps = int(min(2000, max(20, 3000.0 / max(float(t), 1e-3))))

    # host time to ENQUEUE a step, over two steps from an empty launch queue (from the third step on, the TopK
    # step waits for the sizes the step before last copied to the host, i.e. for the device): if this approaches
    # ms_per_step the run is bound by the host's launch path, not by the device
    barrier()
    h0 = time.perf_counter()
    for i in range(2):
        step(batch_dev, 60 + i)
    host_issue_ms = (time.perf_counter() - h0) * 1e3 / 2
    torch.cuda.synchronize()

    # ---- device-resident timing, per-kernel events collected in the same region --------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = eng.launches
    eng.profile = {}
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(batch_dev, 100 + i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    prof = eng.profile_summary()
    eng.profile = None
    launches = eng.launches - launches0
    nd_pad = int(getattr(eng, "last_nd_pad", 0))      # width of the compacted dead-feature operands in those launches
    clocks = sampler.stop() if rank == 0 else None
    eng.check_status("timed region")
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)

    # ---- end to end: pinned host batch -> device every step (prefetched on a copy stream), loss read back
    loss_host = torch.zeros(2, dtype=torch.float32).pin_memory()
    loss_ready = [torch.cuda.Event(), torch.cuda.Event()]
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    last = 0.0
    row_bytes = batch_host[0].numel() * batch_host.element_size()
    if world > 1 and eng.has_fused_exchange():
        # every rank uploads its own token rows and copies their input halves into the peers' buffers;
        # the step's last collective orders the copies (parallel.ShardedBatchUploader)
        from crosslayer_transcoder_b200 import parallel

        up = parallel.ShardedBatchUploader(mod, batch_host.shape, batch_host.dtype, dev)
        h2d_bytes = (up.hi - up.lo) * row_bytes
        config["upload"] = ("each rank uploads B/N token rows and copies their input halves to the peers (NVLink); "
                            + ("joined at the end of backward" if up.late_join else "joined at the step's last collective"))
        for _ in range(2):                         # untimed: maps the pinned pages, touches both buffers
            up.upload(batch_host, full=True)
            up.fence()
            up.take()
            up.release()
        barrier()
        t0.record()
        up.upload(batch_host)                      # the first step's batch: ordered by an explicit fence
        up.fence()
        for i in range(steps):
            slot = i & 1
            b = up.take()
            if i + 1 < steps:
                up.upload(batch_host)
            loss = step(b, 200 + i)
            up.release()
            loss_host[slot:slot + 1].copy_(loss.detach().reshape(1), non_blocking=True)   # device -> host, every step
            loss_ready[slot].record()
            if i > 0:
                loss_ready[slot ^ 1].synchronize()
                last = float(loss_host[slot ^ 1])
        up.detach()
    else:
        copy_stream = torch.cuda.Stream()
        if world > 1:
            from crosslayer_transcoder_b200 import parallel

            # NCCL form: every rank needs the whole batch; each uploads 1/N of the rows and the slices are
            # all-gathered over NVLink on the step's communicator
            upload_group = dist.group.WORLD
            chunk = (spec.batch + world - 1) // world
            shape = (world * chunk, *batch_dev.shape[1:])
            bufs = [torch.empty(shape, dtype=batch_dev.dtype, device=dev) for _ in range(2)]
            h2d_bytes = chunk * row_bytes
            config["upload"] = "each rank uploads B/N token rows, NCCL all-gather of the slices"
        else:
            bufs = [torch.empty_like(batch_dev), torch.empty_like(batch_dev)]
            h2d_bytes = spec.batch * row_bytes
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        freed = [torch.cuda.Event(), torch.cuda.Event()]
        views = [None, None]

        def upload(slot):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(freed[slot])
                if world > 1:
                    views[slot] = parallel.upload_batch(batch_host, bufs[slot], upload_group)
                else:
                    bufs[slot].copy_(batch_host, non_blocking=True)
                    views[slot] = bufs[slot]
                ready[slot].record(copy_stream)

        for f in freed:
            f.record()
        # untimed: one upload per slot, so that the pinned pages are mapped
        upload(0)
        upload(1)
        torch.cuda.synchronize()
        barrier()
        t0.record()
        upload(0)
        # the loss of every step is copied to pinned host memory inside the timed region; the host looks at a
        # step's value one step later, so that reading it does not drain the launch queue
        for i in range(steps):
            slot = i & 1
            if i + 1 < steps:
                upload(slot ^ 1)
            torch.cuda.current_stream().wait_event(ready[slot])
            loss = step(views[slot], 200 + i)
            freed[slot].record()
            loss_host[slot:slot + 1].copy_(loss.detach().reshape(1), non_blocking=True)   # device -> host, every step
            loss_ready[slot].record()
            if i > 0:
                loss_ready[slot ^ 1].synchronize()
                last = float(loss_host[slot ^ 1])
    loss_ready[(steps - 1) & 1].synchronize()
    last = float(loss_host[(steps - 1) & 1])
    t1.record()
    barrier()
    e2e_ms = t0.elapsed_time(t1)
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t)
    eng.check_status("end-to-end region")

    if rank == 0:
        peaks = load_peaks()
        Fl = spec.d_features // world
        n_adam = eng.flat.numel
        n_dec_params = sum(w.numel() for w in mod.model.decoder.blocks())
        if getattr(mod, "fuse_optimizer", False):
            # the optimizer kernel runs twice per step, before and after the decoder blocks; its per-launch
            # average covers half of the remaining parameters
            n_dec = sum((w.numel() + 63) // 64 * 64 for w in mod.model.decoder.blocks())
            n_adam = (eng.flat.numel - n_dec) / 2.0
        work = algorithmic_work(spec, world, Fl, n_adam, batch_host.element_size(), nd_pad=nd_pad,
                                fused_exchange=fused_exchange,
                                candidate_list=bool(getattr(mod, "batchtopk_candidates", True)))
        kernels = {}
        flags = []
        for name, st in prof.items():
            w = work.get(name)
            entry = {"launches": st["launches"], "ms_avg": round(st["ms_avg"], 4),
                     "share": round(st["ms_total"] / ms, 4)}
            if w is not None:
                bound, amount = w[0], w[1]
                per_s = amount / (st["ms_avg"] * 1e-3)
                if bound == "tensor":
                    ach, peak, unit, limit = per_s / 1e12, peaks["bf16_tflops"], "TFLOP/s", 1.4
                else:
                    ach, peak, unit, limit = per_s / 1e9, peaks["hbm_gbs"], "GB/s", 1.2
                entry.update(bound=bound, achieved=round(ach, 1), unit=unit, frac=round(ach / peak, 4))
                if len(w) > 2:      # gathers: the figure above counts every distinct row once
                    tm = w[2] / (st["ms_avg"] * 1e-3) / 1e9
                    entry["counts"] = "each distinct decoder row once (lower bound with perfect reuse)"
                    entry["token_major"] = {"achieved": round(tm, 1), "unit": "GB/s", "frac": round(tm / peak, 4),
                                            "counts": "every fetched row, L2 hits included"}
                if ach / peak > limit:
                    flags.append(f"{name}: {ach / peak:.2f} of peak exceeds {limit}")
            kernels[name] = entry
        top = max((k for k in kernels if "bound" in kernels[k]), key=lambda k: kernels[k]["share"])
        tk = kernels[top]
        roofline = {"kernel": top, "bound": tk["bound"], "achieved": tk["achieved"],
                    "peak": peaks["bf16_tflops"] if tk["bound"] == "tensor" else peaks["hbm_gbs"],
                    "unit": tk["unit"], "frac": tk["frac"], "peak_source": peaks["source"],
                    "traffic": (NCU_TRAFFIC_PER_UNIT[top] * (n_dec_params if top == "clt_sparse_bwd_dec_adam" else n_adam)
                                if top in NCU_TRAFFIC_PER_UNIT else None)}
        line = {"metric": METRIC, "value": spec.batch * steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
                "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": dtype_name, "data": "synthetic", "config": config,
                "clocks": clocks,
                "e2e": {"value": spec.batch * steps / (e2e_ms * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": h2d_bytes,
                        "d2h_bytes_per_step": 8, "last_loss": last},
                "last_loss": last, "gpu_launches": launches, "host_issue_ms_per_step": host_issue_ms,
                "roofline": roofline, "kernels": kernels,
                "accounting_ok": not flags}
        if flags:
            line["accounting_flags"] = flags
            print("bench.py: work-model check failed: " + "; ".join(flags), file=sys.stderr)
        if world == 1 and not args.no_cpu_baseline:
            r = time_cpu_reference(spec, args.workload, args.override, 0.0)       # the bounded sample only
            if r is not None and "error" not in r:
                line["cpu_baseline"] = {"value": r["tokens_per_s"], "unit": UNIT, "cores": r["cores"], "kind": r["kind"],
                                        "sample": r["sample"], "sample_step_s": r["sample_step_s"]}
            else:
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                                        "sample": "unavailable: " + ("oracle/_ref missing" if r is None else r["error"])}
        if world == 1 and args.ingest:
            try:
                line["ingest"] = time_ingest(spec, dev)
            except Exception as e:
                line["ingest"] = {"unavailable": f"{type(e).__name__}: {str(e).splitlines()[0][:160]}"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
