"""Helpers shared by the GPU tests: numpy <-> device conversion, cache construction."""
import json
import os
import tempfile
import types

import numpy as np
import torch

from oracle import fourier_oracle as fo

TDT = {"fp16": torch.float16, "bf16": torch.bfloat16}


def dev(x, dtype=None, device="cuda"):
    t = torch.from_numpy(np.ascontiguousarray(x)).to(device)
    return t.to(TDT[dtype]) if dtype in TDT else t


def host(t):
    return t.detach().float().cpu().numpy()


def write_tables(tables):
    f = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
    json.dump(tables, f)
    f.close()
    return f.name


def make_config(g, path):
    return types.SimpleNamespace(numinittokens=g["S"], maxlocallen=g["W"], maxmidstates=g["M"],
                                 non_critical_dims_path=path, max_position_embeddings=g["mpe"],
                                 num_key_value_heads=g["Hkv"], max_new_tokens=g["steps"], model_type="llama")


def update_arg(x, dtype):
    """(B,Hkv,L,D) numpy -> tensor with (B,L,Hkv,D) memory order, as the attention forward hands it over."""
    return dev(x.transpose(0, 2, 1, 3), dtype).transpose(1, 2)


def oracle_cache(g, tables):
    return fo.OracleCache([fo.DimTables(tables["Layer_0"])], g["S"], g["W"], g["M"], g["steps"], g["mpe"], g["dtype"])


def decode_inputs_from_oracle(oc, dtype, pad_rows=True):
    """Device tensors for ops.decode_attn from an OracleCache state (layer 0)."""
    import fourierattention_b200.ops as ops
    kc, vc = oc.key_cache[0], oc.value_cache[0]
    tb = oc.tables[0]
    f32 = lambda a: dev(np.asarray(a, np.float32))

    def store(a):
        a = np.asarray(a, np.float32)
        if not pad_rows:
            return dev(a, dtype)
        B, L, Mn = a.shape
        buf = torch.zeros((B, L + 3, (Mn + 7) // 8 * 8 + 8), dtype=TDT[dtype], device="cuda")
        buf[:, :L, :Mn] = dev(a, dtype)
        return buf[:, :L, :Mn]
    tabs = ops.DecodeTables(tb.kc, tb.kc_h, tb.kn, tb.kn_h, tb.vc, tb.vc_h, tb.vn, tb.vn_h, device="cuda")
    return dict(k_sink=dev(kc["k_init"], dtype), v_sink=dev(vc["v_init"], dtype),
                k_win=dev(kc["k_local"], dtype), v_win=dev(vc["v_local"], dtype),
                k_mn=store(kc["k_uncompressed"]), v_mn=store(vc["v_uncompressed"]),
                k_coef=f32(kc["k_compressed"]), v_coef=f32(vc["v_compressed"]),
                avg_k_u=f32(oc.k_layer_average[0]), avg_k_d=f32(oc.kd_layer_average[0]), scale_k=f32(oc.k_scale[0]),
                avg_v_u=f32(oc.v_layer_average[0]), avg_v_d=f32(oc.vd_layer_average[0]), scale_v=f32(oc.v_scale[0]),
                tables=tabs)
