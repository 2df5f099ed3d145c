"""Generate the golden fixtures in this directory from the reference's own Python code.

Run once, in a container that has the reference checkout (read-only) next to this repository:

    python tests/golden/make_golden.py --reference /path/to/FourierAttention

The reference's cache (``DynamicCache.__init__`` / ``update``), its prefill compressor
(``MultiDimHiPPO2.forward``, FFT branch) and its PyTorch attention path
(``torch_fourier_attn`` / ``mat_fourier_inv_torch``) are executed UNMODIFIED on CPU.
Five things have to be patched around them because they need a GPU or a missing package:

* ``matplotlib`` (imported, never used) is stubbed;
* ``torch.Tensor.cuda`` becomes the identity and the module-level ``DEVICE`` becomes cpu;
* ``flash_attn_func`` is replaced by a float32 softmax attention whose output is cast to the
  input dtype (one query row sees every key under bottom-right causal alignment);
* the three Triton entry points that the cache calls (``mat_avg_std_triton``,
  ``mat_fourier_avg_std_triton``, ``mat_fourier_triton``) are replaced by float32 PyTorch
  code that follows the arithmetic of their kernels line by line (same angle formula, same
  order of roundings, same output dtypes).  Tensor-core TF32 rounding inside ``tl.dot`` is not
  emulated.

Inputs are seeded (``oracle.fourier_oracle.synth_kv`` / ``make_splithead_tables``) so the
fixtures store outputs only, plus a checksum of the inputs.
"""
import argparse
import hashlib
import json
import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import fourier_oracle as fo  # noqa: E402

CASES = {
    # name: geometry.  P = prompt length, steps = decode steps, mpe = max_position_embeddings
    "toy_fp16_ragged": dict(B=2, Hq=4, Hkv=2, D=8, S=4, W=6, M=8, P=40, steps=5, mpe=4096,
                            dtype="fp16", ncomp=6, ragged=True, seed=11),
    "small_fp16": dict(B=1, Hq=8, Hkv=2, D=32, S=4, W=16, M=16, P=200, steps=6, mpe=4096,
                       dtype="fp16", ncomp=24, ragged=False, seed=12),
    # P + steps - S - W = 93 and int(1/(1/93)) == 92: the two periods differ
    "small_bf16_tc": dict(B=2, Hq=6, Hkv=2, D=16, S=2, W=5, M=8, P=97, steps=3, mpe=4096,
                          dtype="bf16", ncomp=12, ragged=False, seed=13),
    "mid_fp16": dict(B=1, Hq=8, Hkv=2, D=128, S=4, W=64, M=64, P=600, steps=4, mpe=131072,
                     dtype="fp16", ncomp=96, ragged=False, seed=14),
    "mid_bf16_ragged": dict(B=2, Hq=8, Hkv=4, D=64, S=4, W=32, M=32, P=300, steps=4, mpe=131072,
                            dtype="bf16", ncomp=48, ragged=True, seed=15),
    # max_position_embeddings clamps maxtokens below P + steps (CU:542)
    "clamp_fp16": dict(B=1, Hq=4, Hkv=2, D=16, S=4, W=8, M=8, P=100, steps=3, mpe=101,
                       dtype="fp16", ncomp=12, ragged=False, seed=16),
    # prompt not longer than S + M + W: never compressed (CU:598-611, CU:681-686)
    "short_fp16": dict(B=2, Hq=4, Hkv=2, D=8, S=4, W=6, M=8, P=18, steps=3, mpe=4096,
                       dtype="fp16", ncomp=6, ragged=False, seed=17),
}


def load_reference(ref_root):
    mpl = types.ModuleType("matplotlib"); plt = types.ModuleType("matplotlib.pyplot")
    mpl.pyplot = plt
    sys.modules["matplotlib"] = mpl; sys.modules["matplotlib.pyplot"] = plt
    sys.path.insert(0, os.path.join(ref_root, "fourier_attn_triton"))
    import fourier_triton_valid4_v2 as km
    sys.modules["lxr_fourier_triton_valid4_v2"] = km
    km.DEVICE = torch.device("cpu")

    def avg_std(a):                      # arithmetic of _mean_max_dev_one_pass_kernel
        a32 = a.to(torch.float32)
        K = a32.shape[1]
        avg = a32.sum(dim=1) / K
        dev = torch.maximum(a32.max(dim=1).values - avg, avg - a32.min(dim=1).values)
        return avg.to(a.dtype), dev.to(a.dtype)

    def fourier_avg_std(c, K, T):        # arithmetic of mat_fourier_avg_std_triton(_kernel)
        B, N2, M = c.shape
        N = N2 // 2
        k = torch.arange(K, dtype=torch.int32); n = torch.arange(N, dtype=torch.int32)
        arg = (torch.tensor(2.0 * np.pi / T, dtype=torch.float32) * k[:, None].to(torch.float32)) \
            * n[None, :].to(torch.float32)
        a = torch.cos(arg) @ c[:, :N].float() + torch.sin(arg) @ c[:, N:].float()
        a = a / N
        avg = a.sum(dim=1) / K
        dev = torch.maximum(a.max(dim=1).values - avg, avg - a.min(dim=1).values)
        return avg.to(torch.float16), dev.to(torch.float16)

    def fourier_fwd(a, N, T, K_start=0):  # arithmetic of mat_fourier_kernel
        B, K, M = a.shape
        k = torch.arange(K, dtype=torch.float32) + K_start
        n = torch.arange(N, dtype=torch.float32)
        F = torch.tensor(2.0 * 3.14159265359, dtype=torch.float32) * k[None, :] * n[:, None] / T
        a32 = a.to(torch.float32)
        return torch.cat([torch.cos(F) @ a32, torch.sin(F) @ a32], dim=1)

    def flash_standin(q, k, v, softmax_scale=None, causal=True):
        B, Lq, Hq, D = q.shape
        Hkv = k.shape[2]
        assert Lq == 1
        scale = softmax_scale if softmax_scale is not None else D ** -0.5
        qf = q.float().view(B, Hkv, Hq // Hkv, D)
        kf = k.float().permute(0, 2, 1, 3)           # B,Hkv,L,D
        vf = v.float().permute(0, 2, 1, 3)
        s = torch.einsum("bgrd,bgld->bgrl", qf, kf) * scale
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("bgrl,bgld->bgrd", p, vf).reshape(B, 1, Hq, D)
        return o.to(q.dtype)

    km.mat_avg_std_triton = avg_std
    km.mat_fourier_avg_std_triton = fourier_avg_std
    km.mat_fourier_triton = fourier_fwd
    km.flash_attn_func = flash_standin
    torch.Tensor.cuda = lambda self, *a, **k: self
    import cache_utils_fourier as cu
    sys.modules["lxr_cache_utils_fourier"] = cu
    return km, cu


def tt(x, dtype):
    return torch.from_numpy(np.ascontiguousarray(x)).to(torch.float16 if dtype == "fp16" else torch.bfloat16)


def run_case(km, cu, name, g, out_dir):
    tables = fo.make_splithead_tables(1, g["Hkv"], g["D"], g["ncomp"], g["seed"], ragged=g["ragged"])
    with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as f:
        json.dump(tables, f)
        path = f.name
    cfg = types.SimpleNamespace(numinittokens=g["S"], maxlocallen=g["W"], maxmidstates=g["M"],
                                non_critical_dims_path=path, max_position_embeddings=g["mpe"],
                                num_key_value_heads=g["Hkv"], max_new_tokens=g["steps"], model_type="llama")
    cache = cu.DynamicCache(cfg)
    os.unlink(path)
    B, Hq, Hkv, D, P = g["B"], g["Hq"], g["Hkv"], g["D"], g["P"]
    dt = g["dtype"]
    k, v = fo.synth_kv(g["seed"], B, Hkv, P + g["steps"], D, dt)
    rng = np.random.default_rng(g["seed"] + 1000)
    qs = fo.rnd(rng.standard_normal((g["steps"], B, Hq * D)).astype(np.float32), dt)
    h = hashlib.sha256(); h.update(k.tobytes()); h.update(v.tobytes()); h.update(qs.tobytes())
    out = {"input_sha256": np.frombuffer(h.digest(), dtype=np.uint8)}

    def as_update_arg(x):                      # (B,Hkv,L,D) view of (B,L,Hkv,D) memory (CU:529-534)
        return tt(x.transpose(0, 2, 1, 3), dt).transpose(1, 2)

    kd, vd = cache.update(as_update_arg(k[:, :, :P]), as_update_arg(v[:, :, :P]), 0)
    assert kd["k_init"] is None and kd["k_local"].shape[1] == P
    compressed = P > g["S"] + g["M"] + g["W"]
    out["maxtokens"] = np.int64(cache.maxtokens)
    out["curr_tokennum_prefill"] = np.int64(cache.curr_tokennum[0])
    if compressed:
        kc, vc = cache.key_cache[0], cache.value_cache[0]
        out["pre_k_compressed"] = kc["k_compressed"].numpy()
        out["pre_v_compressed"] = vc["v_compressed"].numpy()
        out["pre_k_uncompressed"] = kc["k_uncompressed"].float().numpy()
        out["pre_v_uncompressed"] = vc["v_uncompressed"].float().numpy()
        for nm in ("k_scale", "v_scale", "k_layer_average", "v_layer_average",
                   "kd_layer_average", "vd_layer_average"):
            t = getattr(cache, nm)[0]
            out[nm] = t.float().numpy()
            out[nm + "_dtype"] = np.array(str(t.dtype))
    for s in range(g["steps"]):
        kd, vd = cache.update(as_update_arg(k[:, :, P + s:P + s + 1]), as_update_arg(v[:, :, P + s:P + s + 1]), 0)
        out[f"seq_len_{s}"] = np.int64(cache.get_seq_length(0))
        if kd["k_init"] is None:
            out[f"local_len_{s}"] = np.int64(kd["k_local"].shape[1])
            continue
        T = cache.maxtokens - cache.numinittokens - cache.maxlocallen
        o = km.torch_fourier_attn(
            q=tt(qs[s], dt).view(B, 1, Hq * D),
            k_il=torch.cat([kd["k_init"], kd["k_local"]], dim=1).contiguous(),
            v_il=torch.cat([vd["v_init"], vd["v_local"]], dim=1).contiguous(),
            k_mc=kd["k_compressed"], v_mc=vd["v_compressed"],
            k_mn=kd["k_uncompressed"], v_mn=vd["v_uncompressed"],
            avg_k_u=cache.k_layer_average[0], avg_k_d=cache.kd_layer_average[0], scale_k=cache.k_scale[0],
            avg_v_u=cache.v_layer_average[0], avg_v_d=cache.vd_layer_average[0], scale_v=cache.v_scale[0],
            kc_list=cache.k_non_critical_dims[0], kc_h_list=cache.k_non_critical_head_dims[0],
            kn_list=cache.k_critical_dims[0], kn_h_list=cache.k_critical_head_dims[0],
            vc_list=cache.v_non_critical_dims[0], vc_h_list=cache.v_non_critical_head_dims[0],
            vn_list=cache.v_critical_dims[0], vn_h_list=cache.v_critical_head_dims[0],
            num_head_q=Hq, num_head_kv=Hkv, seq_len_m=kd["k_uncompressed"].size(1), T=T)
        out[f"attn_{s}"] = o.float().numpy()
        out[f"attn_{s}_dtype"] = np.array(str(o.dtype))
    if compressed:
        kc, vc = cache.key_cache[0], cache.value_cache[0]
        out["fin_k_compressed"] = kc["k_compressed"].numpy()
        out["fin_v_compressed"] = vc["v_compressed"].numpy()
        out["fin_k_uncompressed_tail"] = kc["k_uncompressed"][:, -g["steps"]:].float().numpy()
        out["fin_v_uncompressed_tail"] = vc["v_uncompressed"][:, -g["steps"]:].float().numpy()
        out["fin_k_local"] = kc["k_local"].float().numpy()
        out["fin_v_local"] = vc["v_local"].float().numpy()
        out["fin_k_init"] = kc["k_init"].float().numpy()
        out["curr_tokennum_final"] = np.int64(cache.curr_tokennum[0])
    out["geometry"] = np.array(json.dumps(g))
    np.savez_compressed(os.path.join(out_dir, name + ".npz"), **out)
    print(name, "written;", {k_: getattr(v_, "shape", None) for k_, v_ in out.items() if k_.startswith(("pre_k_c", "attn_0"))})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=HERE)
    a = ap.parse_args()
    km, cu = load_reference(a.reference)
    for name, g in CASES.items():
        run_case(km, cu, name, g, a.out)


if __name__ == "__main__":
    main()
