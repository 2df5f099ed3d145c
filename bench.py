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
    # the headline workload: full Llama-3.1-8B attention geometry, batch 8, 32k-token prompts, 256 decode steps
    "llama31_8b_32k": dict(layers=32, B=8, Hq=32, Hkv=8, D=128, ctx=32768, S=4, W=1024, M=512, ncomp=96,
                           dtype="bf16", new_tokens=256),
    # Llama-3.2-3B attention geometry, batch 32, 16k-token prompts
    "llama32_3b_16k": dict(layers=28, B=32, Hq=24, Hkv=8, D=128, ctx=16384, S=4, W=512, M=256, ncomp=80,
                           dtype="bf16", new_tokens=256),
    # one layer, one sequence, fp16, 8k context, 64 decode steps
    "single_layer_8k": dict(layers=1, B=1, Hq=32, Hkv=8, D=128, ctx=8192, S=4, W=1024, M=256, ncomp=96,
                            dtype="fp16", new_tokens=64),
    # one long sequence, one layer, 2048-token window, M = 1024; with --gpus N the middle span is split by
    # sequence over the N ranks and the partial results are merged by log-sum-exp over NCCL
    "long_131k": dict(layers=1, B=1, Hq=32, Hkv=8, D=128, ctx=131072, S=4, W=2048, M=1024, ncomp=96,
                      dtype="bf16", new_tokens=256, seq_split=True),
    "long_262k": dict(layers=1, B=1, Hq=32, Hkv=8, D=128, ctx=262144, S=4, W=2048, M=1024, ncomp=96,
                      dtype="bf16", new_tokens=256, seq_split=True),
    "long_524k": dict(layers=1, B=1, Hq=32, Hkv=8, D=128, ctx=524288, S=4, W=2048, M=1024, ncomp=96,
                      dtype="bf16", new_tokens=256, seq_split=True),
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
                                          "-lms", "20", "-i", str(self.gpu)], stdout=subprocess.PIPE,
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
    steps = max(1, args.steps)
    t, sample = run_cpu_oracle(w, steps, max(0, args.warmup))
    scale = w["layers"] * w["B"]                # one full step = every layer and sequence
    step_s = t * scale
    val = w["B"] / step_s
    line = {"impl": "reference", "metric": "decode-attn tokens/s", "value": val, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic", "config": workload_config(args, w),
            # what was timed is one layer x one sequence; the full step is that time x layers x batch
            "extrapolated": True, "sampled_s": t * steps, "sampled_ms_per_sample_step": t * 1e3, "scale": scale,
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
                             "extrapolated": True, "sampled_s": t * steps, "scale": scale},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def triton_arm(args, w):
    """Context number, not a target: the reference's own GPU path -- its unmodified ``DynamicCache.update`` and
    ``triton_fourier_attn`` (fourier_triton_valid4_v2.py:684-779), JIT-compiled by the installed Triton -- timed
    on ONE layer of the workload after warm-up; the full step is that time x layers.  It needs a checkout of the
    reference (``--reference-dir`` or FA_REFERENCE_DIR, the directory that holds ``fourier_attn_triton/``);
    without one, or if its modules do not import or run on this box, the line says ``unavailable`` and why."""
    ref = args.reference_dir or os.environ.get("FA_REFERENCE_DIR") or ""
    base = {"impl": "triton", "metric": "decode-attn tokens/s", "unit": "tokens/s", "n_gpus": 1,
            "config": workload_config(args, w)}
    src = os.path.join(ref, "fourier_attn_triton")
    if not ref or not os.path.isdir(src):
        print(json.dumps(dict(base, unavailable=f"no reference checkout at {src!r}")), flush=True)
        return
    try:
        import torch
        for name in ("matplotlib", "matplotlib.pyplot"):          # imported at the top of the kernel module, unused
            sys.modules.setdefault(name, types.ModuleType(name))
        sys.path.insert(0, src)
        import fourier_triton_valid4_v2 as km
        sys.modules["lxr_fourier_triton_valid4_v2"] = km
        import cache_utils_fourier as cu
        from fourierattention_b200 import synth                      # seeded inputs only; none of its kernels run here
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        tdt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
        W_, K_ = max(2, args.warmup), args.steps
        tables = synth.make_splithead_tables(1, w["Hkv"], w["D"], w["ncomp"], seed=2024)
        tf = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
        json.dump(tables, tf); tf.close()
        cfg = types.SimpleNamespace(numinittokens=w["S"], maxlocallen=w["W"], maxmidstates=w["M"],
                                    non_critical_dims_path=tf.name, max_position_embeddings=1 << 30,
                                    num_key_value_heads=w["Hkv"], max_new_tokens=max(w["new_tokens"], W_ + K_ + 1),
                                    model_type="llama")
        cache = cu.DynamicCache(cfg)
        os.unlink(tf.name)
        B, D, Hq, Hkv = w["B"], w["D"], w["Hq"], w["Hkv"]
        gen = torch.Generator(device=dev); gen.manual_seed(99)
        k, v = synth.rope_kv(B, Hkv, w["ctx"], D, tdt, dev, gen)
        cache.update(k.contiguous().transpose(1, 2).contiguous().transpose(1, 2), v.contiguous().transpose(1, 2).contiguous().transpose(1, 2), 0)
        del k, v
        mk = lambda s_: torch.randn(s_, device=dev, dtype=torch.float32, generator=gen).to(tdt)
        n = W_ + K_
        q, kn, vn = mk((n, B, 1, Hq * D)), mk((n, B, 1, Hkv, D)), mk((n, B, 1, Hkv, D))

        def step(s_):
            ks, vs = cache.update(kn[s_].transpose(1, 2), vn[s_].transpose(1, 2), 0)
            return km.triton_fourier_attn(
                q=q[s_].contiguous(), k_il=torch.cat([ks["k_init"], ks["k_local"]], dim=1).contiguous(),
                v_il=torch.cat([vs["v_init"], vs["v_local"]], dim=1).contiguous(),
                k_mc=ks["k_compressed"], v_mc=vs["v_compressed"], k_mn=ks["k_uncompressed"], v_mn=vs["v_uncompressed"],
                avg_k_u=cache.k_layer_average[0], avg_k_d=cache.kd_layer_average[0], scale_k=cache.k_scale[0],
                avg_v_u=cache.v_layer_average[0], avg_v_d=cache.vd_layer_average[0], scale_v=cache.v_scale[0],
                kc_list=cache.k_non_critical_dims[0], kc_h_list=cache.k_non_critical_head_dims[0],
                kn_list=cache.k_critical_dims[0], kn_h_list=cache.k_critical_head_dims[0],
                vc_list=cache.v_non_critical_dims[0], vc_h_list=cache.v_non_critical_head_dims[0],
                vn_list=cache.v_critical_dims[0], vn_h_list=cache.v_critical_head_dims[0],
                num_head_q=Hq, num_head_kv=Hkv, seq_len_m=ks["k_uncompressed"].size(1),
                T=cache.maxtokens - cache.numinittokens - cache.maxlocallen)
        for s_ in range(W_):
            out = step(s_)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s_ in range(W_, W_ + K_):
            out = step(s_)
        e1.record()
        torch.cuda.synchronize()
        layer_ms = e0.elapsed_time(e1) / K_
        step_ms = layer_ms * w["layers"]
        # The reference kernel takes the span length as a compile-time constant (N_m: tl.constexpr,
        # fourier_triton_valid4_v2.py:477), so every decode step -- the span grows by one row -- is compiled anew.
        # The same attention call repeated on an unchanged cache shows the kernel alone.
        ks, vs = cache.key_cache[0], cache.value_cache[0]

        def attend_again():
            return km.triton_fourier_attn(
                q=q[0].contiguous(), k_il=torch.cat([ks["k_init"], ks["k_local"]], dim=1).contiguous(),
                v_il=torch.cat([vs["v_init"], vs["v_local"]], dim=1).contiguous(),
                k_mc=ks["k_compressed"], v_mc=vs["v_compressed"], k_mn=ks["k_uncompressed"], v_mn=vs["v_uncompressed"],
                avg_k_u=cache.k_layer_average[0], avg_k_d=cache.kd_layer_average[0], scale_k=cache.k_scale[0],
                avg_v_u=cache.v_layer_average[0], avg_v_d=cache.vd_layer_average[0], scale_v=cache.v_scale[0],
                kc_list=cache.k_non_critical_dims[0], kc_h_list=cache.k_non_critical_head_dims[0],
                kn_list=cache.k_critical_dims[0], kn_h_list=cache.k_critical_head_dims[0],
                vc_list=cache.v_non_critical_dims[0], vc_h_list=cache.v_non_critical_head_dims[0],
                vn_list=cache.v_critical_dims[0], vn_h_list=cache.v_critical_head_dims[0],
                num_head_q=Hq, num_head_kv=Hkv, seq_len_m=ks["k_uncompressed"].size(1),
                T=cache.maxtokens - cache.numinittokens - cache.maxlocallen)
        attend_again()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(4):
            attend_again()
        e1.record()
        torch.cuda.synchronize()
        kernel_ms = e0.elapsed_time(e1) / 4
        print(json.dumps(dict(base, value=B / (step_ms * 1e-3), ms_per_step=step_ms, steps=K_, warmup=W_,
                              higher_is_better=True, dtype=w["dtype"], data="synthetic", extrapolated=w["layers"] > 1,
                              sampled_ms_per_layer=layer_ms, scale=w["layers"],
                              attention_only_ms_per_layer_compiled=kernel_ms,
                              finite=bool(torch.isfinite(out.float()).all()),
                              note="the reference's Triton path on this GPU, one layer timed, for context only; a decode "
                                   "step recompiles its kernel because the span length is a compile-time constant, "
                                   "attention_only_ms_per_layer_compiled repeats one call on an unchanged cache")),
              flush=True)
    except Exception as ex:      # the context arm must never take the benchmark down
        print(json.dumps(dict(base, unavailable=f"{type(ex).__name__}: {ex}"[:400])), flush=True)


KERNEL_SOURCES = ("decode.cu", "decode_fast.cuh", "decode_il.cuh", "decode_ws.cuh", "decode_ws2.cuh", "common.cuh")


def kernel_source_sha16():
    """Digest of the decode kernel sources: a recorded DRAM-traffic figure is only quoted while the sources it was
    measured on are unchanged."""
    import hashlib
    h = hashlib.sha256()
    for name in KERNEL_SOURCES:
        with open(os.path.join(ROOT, "fourierattention_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def recorded_traffic(kernel_name, workload):
    """DRAM read + write bytes of one launch of ``kernel_name`` from the ncu capture summarised under profiles/
    (``<kernel>.traffic.json``, written next to the summary it was read from).  Returns (bytes or None, note)."""
    path = os.path.join(ROOT, "profiles", f"{kernel_name}.traffic.json")
    if not os.path.exists(path):
        return None, "no ncu capture recorded for this kernel"
    with open(path) as f:
        rec = json.load(f).get(workload)
    if rec is None:
        return None, "no ncu capture recorded for this workload"
    if rec.get("source_sha16") != kernel_source_sha16():
        return None, f"the kernel sources changed since the capture of {rec.get('captured')}: figure withheld"
    return float(rec["dram_bytes"]), rec.get("source", "")


def main_kernel_name(path):
    """Name of the middle-span kernel a decode path runs (fa_decode_path: 0 exact, 1 tensor-core pass, 2 the
    warp-specialised form, 3 its variant with the spectral accumulator in tensor memory)."""
    if path in (2, 3):
        return "decode_main_ws2_kernel" if path == 3 else "decode_main_ws_kernel"
    return {0: "decode_main_kernel", 1: "decode_main_fast_kernel"}.get(path)


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

    if w.get("seq_split"):
        return seq_split_arm(args, w, world, rank, dev)
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
        fast = ops.last_decode_path in (1, 2, 3)
        kernel_name = main_kernel_name(ops.last_decode_path)
        # DRAM bytes of one launch as ncu measured them on `profile_small`, whose launches have this workload's
        # per-launch shape; scaled by the share of the KV heads a rank holds (traffic grows with the row width)
        traffic, traffic_src = None, None
        if args.workload in ("llama31_8b_32k", "profile_small"):
            traffic, traffic_src = recorded_traffic(kernel_name, "profile_small")
            if traffic is not None:
                traffic *= frac_heads
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
                                        "kind": "port", "sample": sample, "extrapolated": True,
                                        "sampled_s": t * 4, "scale": L * B}
            except Exception as ex:  # the GPU result stands even if the host baseline cannot run
                line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": os.cpu_count() or 1,
                                        "kind": "port", "sample": f"failed: {ex}"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def seq_split_arm(args, w, world, rank, dev):
    """One long sequence, one layer: the middle span is split by sequence over the ranks (every rank keeps an
    equal slice of the verbatim rows, the coefficients are replicated, rank 0 also attends sinks + window); a
    step is ``update`` + attention, whose partial results travel in one all_gather of Hq*(D+2) floats per
    rank and are merged by log-sum-exp on every rank.  Reports tokens/s, the bytes each GPU streams per step
    as GB/s, and the share of a step that the exchange (all_gather + merge) takes, measured as the difference
    to the same steps without it."""
    import torch
    import torch.distributed as dist
    import fourierattention_b200 as pkg
    from fourierattention_b200 import ops, synth
    tdt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    W_, K_ = args.warmup, args.steps
    total_new = 2 * (W_ + K_) + 1
    new_tokens = max(w["new_tokens"], total_new)
    tables = synth.make_splithead_tables(1, w["Hkv"], w["D"], w["ncomp"], seed=2024)
    tf = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
    json.dump(tables, tf); tf.close()
    cfg = types.SimpleNamespace(numinittokens=w["S"], maxlocallen=w["W"], maxmidstates=w["M"],
                                non_critical_dims_path=tf.name, max_position_embeddings=1 << 30,
                                num_key_value_heads=w["Hkv"], max_new_tokens=new_tokens, model_type="llama")
    cache = pkg.DynamicCache(cfg, device=dev, seq_shard=(rank, world) if world > 1 else None)
    os.unlink(tf.name)
    B, D, Hq, Hkv = w["B"], w["D"], w["Hq"], w["Hkv"]
    gen = torch.Generator(device=dev); gen.manual_seed(99)          # every rank sees the same sequence
    k, v = synth.rope_kv(B, Hkv, w["ctx"], D, tdt, dev, gen)
    cache.update(k, v, 0)
    del k, v
    torch.cuda.synchronize()
    n = 2 * (W_ + K_)
    mk = lambda s_: torch.randn(s_, device=dev, dtype=torch.float32, generator=gen).to(tdt)
    q, kn, vn = mk((n, B, Hq * D)), mk((n, B, Hkv, 1, D)), mk((n, B, Hkv, 1, D))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run(s0, count, merged):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for s_ in range(s0, s0 + count):
            cache.update(kn[s_], vn[s_], 0)
            if merged or world == 1:
                cache.fourier_attention(q[s_], 0, Hq)
            else:
                cache.partial_attention(q[s_], 0, Hq)
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    run(0, W_, True)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    time.sleep(0.2)
    launches0 = ops.launch_count
    wall0 = time.time()
    ms = run(W_, K_, True)
    wall1 = time.time()
    launches = ops.launch_count - launches0
    clocks = sampler.stop(wall0, wall1)
    run(W_ + K_, W_, False)
    ms_nox = run(2 * W_ + K_, K_, False)
    if world > 1:
        t = torch.tensor([ms, ms_nox], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_nox = [float(x) for x in t.tolist()]
    if rank == 0:
        st = cache._state[0]
        F = Hkv * D
        Mc = Hkv * w["ncomp"]
        Mn = F - Mc
        n_mid_total = cache.curr_tokennum[0]
        rows_rank0 = st.n_mid
        # bytes rank 0 streams per step: its slice of the verbatim rows, sinks + window, the replicated coefficients
        rank_bytes = 2 * (rows_rank0 * 2 * Mn + 2 * (w["S"] + w["W"]) * F) + 4 * w["M"] * 2 * Mc
        total_bytes = 2 * (n_mid_total * 2 * Mn + 2 * (w["S"] + w["W"]) * F) + 4 * w["M"] * 2 * Mc
        step_ms = ms / K_
        peak, peak_src = peaks()
        line = {"metric": "decode-attn tokens/s", "value": B / (step_ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
                "steps": K_, "warmup": W_, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
                "config": dict(workload_config(args, w), sharding=f"sequence/{world}" if world > 1 else "none",
                               n_mid=n_mid_total),
                "gpu_launches": launches, "clocks": clocks,
                "roofline": {"bound": "hbm", "kernel": main_kernel_name(ops.last_decode_path),
                             "per_gpu_bytes_per_step": rank_bytes, "per_gpu_gbs": rank_bytes / (step_ms * 1e-3) / 1e9,
                             "achieved": total_bytes / (step_ms * 1e-3) / 1e9, "peak": peak * world, "unit": "GB/s",
                             "frac": total_bytes / (step_ms * 1e-3) / 1e9 / (peak * world), "traffic": None,
                             "peak_source": peak_src},
                "exchange": {"ms_per_step_without": ms_nox / K_, "share_of_step": max(0.0, 1.0 - ms_nox / ms),
                             "bytes_per_rank_per_step": B * Hq * (D + 2) * 4}}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def compress_sweep(args):
    """The prefill projection alone (the compression sweep configuration): bf16, one layer, 8 KV heads x 128 dims of which 96 per
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
            # the reference's own projection of the same columns: complex64 FFT of length T_c, first N bins
            # (fourier_triton_valid4_v2.py:857-865); its error against float64 is the floor the contract is defined on
            fq = torch.fft.fft(x[0][:, cols].to(torch.complex64), n=T_c, dim=0)[:N][n]
            fft_c, fft_s = fq.real.double(), -fq.imag.double()
            fft_err = max(float((fft_c - ref_c).abs().max()), float((fft_s - ref_s).abs().max()))
            vs_fft = max(float((got_c - fft_c).abs().max()), float((got_s - fft_s).abs().max()))
            rows.append({"span": span, "M": M, "ms": ms, "tflops": flops / ms / 1e9, "frac_of_peak": flops / ms / 1e9 / peak,
                         "max_abs_err": err, "coef_rms": rms, "rel_err": err / rms, "T": T, "T_c": T_c,
                         "reference_fft_max_abs_err": fft_err, "max_abs_diff_to_reference_fft": vs_fft})
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
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "triton"])
    ap.add_argument("--reference-dir", default=None, help="checkout of the reference, for --impl triton")
    ap.add_argument("--workload", default="llama31_8b_32k", choices=list(WORKLOADS) + ["compress_sweep"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the host-core baseline leg")
    ap.add_argument("--print-source-sha", action="store_true", help="print the digest of the decode kernel sources")
    args = ap.parse_args()
    if args.print_source_sha:
        print(kernel_source_sha16())
        return
    if args.workload == "compress_sweep":
        return compress_sweep(args)
    w = dict(WORKLOADS[args.workload])
    if args.impl == "reference":
        reference_arm(args, w)
    elif args.impl == "triton":
        triton_arm(args, w)
    else:
        ours_arm(args, w)


if __name__ == "__main__":
    main()
