#!/usr/bin/env python
"""Decode-attention benchmark of the Fourier-compressed KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default ``llama31_8b_32k``): Llama-3.1-8B attention geometry (32 layers, 32 query / 8 KV heads,
head_dim 128), bf16, batch 8, a 32768-token synthetic prompt per sequence (Gaussian K/V, rotary-embedded
keys), 96 of 128 dims per KV head compressed (seeded tables), 4 sinks, a 1024-token window, M = 512
spectral coefficients.  One *step* is one decode step of the hot path over all layers: per layer a cache
``update`` with the new token (window slide, eviction into the coefficients, verbatim append) followed by
the fused decode attention of one query token.  tokens/s = batch / step time.

With N > 1 (launched by torchrun, one rank per GPU) the KV heads are sharded N ways, no communication on
the data path; the reported time is the maximum over ranks.

One JSON line is printed by rank 0.  ``--impl reference`` times the CPU oracle (a numpy restatement of the
reference's PyTorch path) on the host cores instead, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # BASELINE config 2: the configuration the headline metric is quoted on
    "llama31_8b_32k": dict(layers=32, B=8, Hq=32, Hkv=8, D=128, ctx=32768, S=4, W=1024, M=512, ncomp=96,
                           dtype="bf16", new_tokens=256),
    # BASELINE config 3
    "llama32_3b_16k": dict(layers=28, B=32, Hq=24, Hkv=8, D=128, ctx=16384, S=4, W=512, M=256, ncomp=80,
                           dtype="bf16", new_tokens=256),
    # BASELINE config 1 (single layer, fp16)
    "single_layer_8k": dict(layers=1, B=1, Hq=32, Hkv=8, D=128, ctx=8192, S=4, W=1024, M=256, ncomp=96,
                            dtype="fp16", new_tokens=64),
    # a small case for profiler captures (a few hundred MB on the device, still larger than L2)
    "profile_small": dict(layers=2, B=8, Hq=32, Hkv=8, D=128, ctx=32768, S=4, W=1024, M=512, ncomp=96,
                          dtype="bf16", new_tokens=256),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback"


def algorithmic_bytes(w, n_mid, heads_frac=1.0):
    """Bytes one decode step must move per layer and sequence (2-byte elements, fp32 coefficients):
    e*[2(S+W)F + n_mid(Mn_k+Mn_v) + 2 Hq D] + 4*2N*(Mc_k+Mc_v) + 2*6*Mc; returns (whole op, part the
    main kernel streams)."""
    F = w["Hkv"] * w["D"]
    Mc = w["Hkv"] * w["ncomp"]
    Mn = F - Mc
    e = 2
    rows = e * (2 * (w["S"] + w["W"]) * F + n_mid * 2 * Mn + 2 * w["Hq"] * w["D"])
    coef = 4 * w["M"] * 2 * Mc + 2 * 6 * Mc
    return (rows + coef) * heads_frac, rows * heads_frac


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop_all(self):
        """Fallback when the timed region was shorter than the sampling period: use every sample taken
        since the sampler started (warm-up included)."""
        return self.stop(None, None)

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        if self.proc.poll() is None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ts, line in self.lines:
            if t0 is not None and not (t0 <= ts <= t1 + 0.2):
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm and t0 is not None:
            return self.stop_all()
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle on the host cores
# ------------------------------------------------------------------------------------------------
def run_cpu_oracle(w, steps, warmup, seed=1234):
    """Times ``steps`` sample steps; one sample step = the hot path (cache update + attention, the
    reference's PyTorch-path arithmetic) for ONE layer and ONE sequence of the workload.  Returns
    (seconds per sample step, description)."""
    import numpy as np
    from oracle import fourier_oracle as fo
    tables = fo.make_splithead_tables(1, w["Hkv"], w["D"], w["ncomp"], seed)
    total_new = warmup + steps
    oc = fo.OracleCache([fo.DimTables(tables["Layer_0"])], w["S"], w["W"], w["M"], w["new_tokens"],
                        1 << 30, w["dtype"])
    k, v = fo.synth_kv(seed, 1, w["Hkv"], w["ctx"] + total_new, w["D"], w["dtype"])
    rng = np.random.default_rng(seed + 1)
    qs = fo.rnd(rng.standard_normal((total_new, 1, w["Hq"] * w["D"])).astype(np.float32), w["dtype"])
    P = w["ctx"]
    oc.update(k[:, :, :P], v[:, :, :P], 0)
    t0 = None
    for s in range(total_new):
        if s == warmup:
            t0 = time.perf_counter()
        oc.update(k[:, :, P + s:P + s + 1], v[:, :, P + s:P + s + 1], 0)
        oc.attend(qs[s], 0, w["Hq"], w["Hkv"], faithful=True)
    dt = (time.perf_counter() - t0) / steps
    return dt, f"{steps} decode steps of 1 layer x 1 sequence (of {w['layers']} x {w['B']}), numpy oracle, float32 rebuild"


def reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    t, sample = run_cpu_oracle(w, max(1, args.steps), max(0, args.warmup))
    step_s = t * w["layers"] * w["B"]           # one full step = every layer and sequence
    val = w["B"] / step_s
    line = {"impl": "reference", "metric": "decode-attn tokens/s", "value": val, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic", "config": workload_config(args, w),
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(args, w):
    n_mid = w["ctx"] - w["S"] - w["W"]
    return {"workload": args.workload, "layers": w["layers"], "batch": w["B"], "context": w["ctx"],
            "q_heads": w["Hq"], "kv_heads": w["Hkv"], "head_dim": w["D"], "sinks": w["S"], "window": w["W"],
            "coefficients_M": w["M"], "compressed_dims_per_head": w["ncomp"], "n_mid": n_mid,
            "sharding": f"kv-heads/{args.gpus}" if args.gpus > 1 else "none",
            "cache_flush": "inputs larger than L2 (the step streams the whole cache, far above 126 MB)"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def ours_arm(args, w):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import fourierattention_b200 as pkg
    from fourierattention_b200 import ops, synth

    assert w["Hkv"] % world == 0, "KV heads must divide across ranks"
    hk = w["Hkv"] // world
    h0, h1 = rank * hk, (rank + 1) * hk
    R = w["Hq"] // w["Hkv"]
    hq_l = hk * R
    tdt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    W_, K_ = args.warmup, args.steps
    total_new = 2 * (W_ + K_) + 1
    new_tokens = max(w["new_tokens"], total_new)

    tables = synth.make_splithead_tables(w["layers"], w["Hkv"], w["D"], w["ncomp"], seed=2024)
    tf = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
    json.dump(tables, tf); tf.close()
    cfg = types.SimpleNamespace(numinittokens=w["S"], maxlocallen=w["W"], maxmidstates=w["M"],
                                non_critical_dims_path=tf.name, max_position_embeddings=1 << 30,
                                num_key_value_heads=w["Hkv"], max_new_tokens=new_tokens, model_type="llama")
    cache = pkg.DynamicCache(cfg, device=dev, kv_head_range=(h0, h1) if world > 1 else None)
    os.unlink(tf.name)

    gen = torch.Generator(device=dev); gen.manual_seed(99 + rank)
    B, D, L = w["B"], w["D"], w["layers"]
    t_setup = time.time()
    for layer in range(L):
        k, v = synth.rope_kv(B, hk, w["ctx"], D, tdt, dev, gen)
        cache.update(k, v, layer)
        del k, v
    torch.cuda.synchronize()
    setup_s = time.time() - t_setup

    def make_inputs(n, pinned):
        shape_q, shape_kv = (n, L, B, hq_l * D), (n, L, B, hk, 1, D)
        if pinned:
            g = torch.Generator(); g.manual_seed(7 + rank)
            mk = lambda s: torch.randn(s, generator=g, dtype=torch.float32).to(tdt).pin_memory()
        else:
            mk = lambda s: torch.randn(s, device=dev, dtype=torch.float32, generator=gen).to(tdt)
        return mk(shape_q), mk(shape_kv), mk(shape_kv)

    def step_device(q, k, v, s, events=None, main_only=False):
        # main_only: record just the two events that bracket the main kernel (the timed steps), so that the
        # timed region carries as few extra stream operations as the roofline measurement needs
        for layer in range(L):
            cache.update(k[s, layer], v[s, layer], layer)
            ev = None
            if events is not None:
                ev = events[s][layer]
                if main_only:
                    ev = [None, ev[1], ev[2], None, None] if layer % 4 == 0 else None
            cache.fourier_attention(q[s, layer], layer, hq_l, phase_events=ev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- leg 1: inputs resident in HBM -------------------------------------------------------
    q, k, v = make_inputs(W_ + K_, pinned=False)
    events = [[[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(L)] for _ in range(W_ + K_)]
    for s_ in events:
        for l_ in s_:
            for e in l_:
                e.record()
    for s in range(W_):
        step_device(q, k, v, s, events)      # warm-up steps also give the per-call split (all five events)
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ops.launch_count
    wall0 = time.time()
    ev0.record()
    for s in range(W_, W_ + K_):
        step_device(q, k, v, s, events, main_only=True)
    ev1.record()
    barrier()
    wall1 = time.time()
    clocks = sampler.stop(wall0, wall1)
    launches = ops.launch_count - launches0
    ms = ev0.elapsed_time(ev1)
    main_ms, call_ms = [], []
    for s in range(W_, W_ + K_):
        for layer in range(0, L, 4):             # every fourth layer's main kernel is bracketed by events
            e = events[s][layer]
            main_ms.append(e[1].elapsed_time(e[2]))
    for s in range(1, W_):                       # the whole attention call, from the warm-up steps
        for layer in range(L):
            e = events[s][layer]
            call_ms.append(e[0].elapsed_time(e[4]))
    main_avg = sum(main_ms) / len(main_ms)
    call_avg = sum(call_ms) / len(call_ms) if call_ms else float("nan")
    del q, k, v

    # ---- leg 2: end to end through the public API with host buffers --------------------------
    qh, kh, vh = make_inputs(W_ + K_, pinned=True)
    out_h = torch.empty((L, B, hq_l, 1, D), dtype=torch.float32).pin_memory()

    out_d = torch.empty((L, B, hq_l, 1, D), dtype=torch.float32, device=dev)

    def step_host(s):
        # the step's inputs (all layers) come up from pinned host memory in three copies, its outputs go
        # back in one; both inside the timed region
        qd = qh[s].to(dev, non_blocking=True)
        kd = kh[s].to(dev, non_blocking=True)
        vd = vh[s].to(dev, non_blocking=True)
        for layer in range(L):
            cache.update(kd[layer], vd[layer], layer)
            out_d[layer].copy_(cache.fourier_attention(qd[layer], layer, hq_l))
        out_h.copy_(out_d, non_blocking=True)
        torch.cuda.synchronize()        # the step's result is read on the host

    for s in range(W_):
        step_host(s)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(W_, W_ + K_):
        step_host(s)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)

    if world > 1:
        t = torch.tensor([ms, ms_e2e, main_avg, call_avg], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e, main_avg, call_avg = [float(x) for x in t.tolist()]

    if rank == 0:
        n_mid = cache.curr_tokennum[0]
        step_ms = ms / K_
        val = B / (step_ms * 1e-3)
        e2e_val = B / (ms_e2e / K_ * 1e-3)
        peak, peak_src = peaks()
        frac_heads = 1.0 / world
        op_bytes, main_bytes = algorithmic_bytes(w, n_mid, frac_heads)
        achieved = main_bytes * B / (main_avg * 1e-3) / 1e9
        step_bytes = op_bytes * B * L
        # DRAM read+write bytes of one launch from the committed ncu captures of `profile_small`, whose
        # launches have this workload's per-launch shape (algorithmic bytes 294.1 MB)
        fast = ops.last_decode_path in (1, 2)
        kernel_name = {0: "decode_main_kernel", 1: "decode_main_fast_kernel", 2: "decode_main_ws_kernel"}[ops.last_decode_path]
        traffic, traffic_src = None, None
        if fast and world == 1 and args.workload in ("llama31_8b_32k", "profile_small"):
            traffic = 307.7e6 if ops.last_decode_path == 2 else 303.7e6
            traffic_src = "ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch of profile_small " \
                          f"(profiles/{kernel_name}.profile_small.md)"
        h2d = L * B * (hq_l * D + 2 * hk * D) * 2
        d2h = L * B * hq_l * D * 4
        line = {
            "metric": "decode-attn tokens/s", "value": val, "unit": "tokens/s", "n_gpus": world, "steps": K_,
            "warmup": W_, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic", "config": workload_config(args, w),
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                         "traffic_source": traffic_src, "peak_source": peak_src,
                         "kernel_ms": main_avg, "bytes_per_launch": main_bytes * B,
                         "attention_call_ms": call_avg,
                         "step_bytes": step_bytes, "step_gbs": step_bytes / (step_ms * 1e-3) / 1e9,
                         "step_frac": step_bytes / (step_ms * 1e-3) / 1e9 / peak,
                         "step_frac_of_8TBs": step_bytes / (step_ms * 1e-3) / 1e9 / 8000.0},
            "setup_s": setup_s,
        }
        if world == 1 and not args.no_cpu:
            try:
                t, sample = run_cpu_oracle(w, 4, 1)
                cpu_step = t * L * B
                line["cpu_baseline"] = {"value": B / cpu_step, "unit": "tokens/s", "cores": os.cpu_count() or 1,
                                        "kind": "port", "sample": sample}
            except Exception as ex:  # the GPU result stands even if the host baseline cannot run
                line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": os.cpu_count() or 1,
                                        "kind": "port", "sample": f"failed: {ex}"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def compress_sweep(args):
    """BASELINE config 4: the prefill projection alone, bf16, one layer, 8 KV heads x 128 dims of which 96 per
    head are compressed (Mc = 768), K/V ~ N(0,1) x per-dim scale ~ LogUniform(0.1, 10); spans 4096..131072,
    M in {256, 512, 1024}.  Prints one JSON line with TFLOP/s (algorithmic FLOPs 2*M*K*Mc of the compressed
    columns only) against the measured bf16 tensor peak, and the coefficient error against a float64
    evaluation of 24 sampled columns."""
    import math
    import torch
    from fourierattention_b200 import ops, synth, compress_period
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev); gen.manual_seed(4)
    Hkv, D, ncomp = 8, 128, 96
    F, Mc = Hkv * D, Hkv * ncomp
    tables = synth.make_splithead_tables(1, Hkv, D, ncomp, seed=44)["Layer_0"]
    idx = torch.tensor(tables["kc_list"], dtype=torch.int32, device=dev)
    peak = 1682.2
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = float(json.load(open(pk))["bf16_tflops"])
    rows = []
    for span in (4096, 16384, 65536, 131072):
        scale = torch.exp(torch.empty(F, device=dev).uniform_(math.log(0.1), math.log(10.0), generator=gen))
        x = (torch.randn((1, span, F), device=dev, generator=gen) * scale).to(torch.bfloat16)
        for M in (256, 512, 1024):
            N = M // 2
            T = span + 256
            T_c = compress_period(T)
            for _ in range(3):
                coef = ops.compress(x, idx, N, T_c, 0)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            e0.record()
            for _ in range(reps):
                coef = ops.compress(x, idx, N, T_c, 0)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            flops = 2.0 * M * span * Mc
            # float64 check on sampled columns and frequencies
            cols = idx[torch.arange(0, Mc, Mc // 24, device=dev)[:24]].long()
            xs = x[0][:, cols].double()
            n = torch.arange(0, N, max(1, N // 16), device=dev)
            k = torch.arange(span, device=dev, dtype=torch.int64)
            ph = (k[:, None] * n[None, :]) % T_c
            ang = ph.double() * (2 * math.pi / T_c)
            ref_c = torch.cos(ang).T @ xs
            ref_s = torch.sin(ang).T @ xs
            pos = torch.arange(0, Mc, Mc // 24, device=dev)[:24]
            got_c = coef[0][n][:, pos].double()
            got_s = coef[0][N + n][:, pos].double()
            err = max(float((got_c - ref_c).abs().max()), float((got_s - ref_s).abs().max()))
            rms = float(torch.cat([ref_c, ref_s]).pow(2).mean().sqrt())
            rows.append({"span": span, "M": M, "ms": ms, "tflops": flops / ms / 1e9, "frac_of_peak": flops / ms / 1e9 / peak,
                         "max_abs_err": err, "coef_rms": rms, "rel_err": err / rms, "T": T, "T_c": T_c})
    print(json.dumps({"metric": "compression TFLOP/s (algorithmic)", "unit": "TFLOP/s", "n_gpus": 1, "dtype": "bf16",
                      "data": "synthetic", "config": {"workload": "compress_sweep", "Mc": Mc, "source_columns": F},
                      "roofline": {"bound": "tensor", "peak": peak, "unit": "TFLOP/s",
                                   "note": "the kernel also multiplies the 256 uncompressed columns and uses 3 bf16 "
                                           "terms per basis value, so its executed FLOPs are 4x the algorithmic ones"},
                      "rows": rows}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama31_8b_32k", choices=list(WORKLOADS) + ["compress_sweep"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the host-core baseline leg")
    args = ap.parse_args()
    if args.workload == "compress_sweep":
        return compress_sweep(args)
    w = dict(WORKLOADS[args.workload])
    if args.impl == "reference":
        reference_arm(args, w)
    else:
        ours_arm(args, w)


if __name__ == "__main__":
    main()
