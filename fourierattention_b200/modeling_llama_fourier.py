"""Drop-in for the attention forward of ``fourier_attn_triton/modeling_llama_fourier.py``.

Only ``LlamaSdpaAttention.forward`` (modeling_llama_fourier.py:565-667) belongs to the Fourier path; the
rest of that file is stock Llama.  To stay independent of any ``transformers`` version this module
carries a small self-contained Llama (RMSNorm, rotary embedding, SwiGLU MLP, decoder layer, model, LM
head) with the usual parameter names, so that checkpoints in the HuggingFace layout load with
``load_state_dict``.
"""
import math
from types import SimpleNamespace
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as Fnn

from .cache_utils_fourier import Cache, DynamicCache, StaticCache  # noqa: F401  (re-exported names)

__all__ = ["LlamaConfig", "LlamaRMSNorm", "LlamaRotaryEmbedding", "LlamaMLP", "LlamaAttention",
           "LlamaSdpaAttention", "LLAMA_ATTENTION_CLASSES", "LlamaDecoderLayer", "LlamaModel", "LlamaForCausalLM",
           "apply_rotary_pos_emb", "rotate_half"]


class LlamaConfig(SimpleNamespace):
    """Attribute bag with Llama defaults (Llama-3.1-8B geometry)."""

    def __init__(self, **kw):
        d = dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=8, head_dim=None, rms_norm_eps=1e-5,
                 rope_theta=500000.0, max_position_embeddings=131072, attention_bias=False, mlp_bias=False,
                 initializer_range=0.02, _attn_implementation="sdpa")
        d.update(kw)
        if d["head_dim"] is None:
            d["head_dim"] = d["hidden_size"] // d["num_attention_heads"]
        super().__init__(**d)


class LlamaRMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x):
        dt = x.dtype
        x = x.to(torch.float32)
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
        return self.weight * x.to(dt)


class LlamaRotaryEmbedding(nn.Module):
    def __init__(self, config):
        super().__init__()
        dim = config.head_dim
        inv = 1.0 / (config.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        self.register_buffer("inv_freq", inv, persistent=False)

    @torch.no_grad()
    def forward(self, x, position_ids):
        f = position_ids[:, :, None].float() * self.inv_freq[None, None, :].to(x.device)
        emb = torch.cat((f, f), dim=-1)
        return emb.cos().to(x.dtype), emb.sin().to(x.dtype)


def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    return (q * cos) + (rotate_half(q) * sin), (k * cos) + (rotate_half(k) * sin)


class LlamaMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=config.mlp_bias)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=config.mlp_bias)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=config.mlp_bias)

    def forward(self, x):
        return self.down_proj(Fnn.silu(self.gate_proj(x)) * self.up_proj(x))


class LlamaAttention(nn.Module):
    """Projections and geometry shared by the attention variants."""

    def __init__(self, config, layer_idx: Optional[int] = None):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = config.head_dim
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        b = config.attention_bias
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=b)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=b)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=b)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=b)
        self.rotary_emb = LlamaRotaryEmbedding(config)


def _dense_causal(q, k, v, num_kv_heads, head_dim):
    """Causal attention over uncompressed keys in float16, as the reference's prefill branch does with
    ``flash_attn_func(q.half(), k.half(), v.half(), causal=True)`` (modeling_llama_fourier.py:627-633).
    q: (B, q_len, Hq, D); k, v: (B, L, F).  Library call (scaled_dot_product_attention)."""
    B, L = k.shape[0], k.shape[1]
    kh = k.reshape(B, L, num_kv_heads, head_dim).half().transpose(1, 2)
    vh = v.reshape(B, L, num_kv_heads, head_dim).half().transpose(1, 2)
    qh = q.half().transpose(1, 2)
    q_len = qh.shape[2]
    if q_len == L:
        o = Fnn.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=True)
    else:                      # bottom-right aligned mask: the q rows are the last q_len positions
        mask = torch.ones(q_len, L, dtype=torch.bool, device=q.device).tril(diagonal=L - q_len)
        o = Fnn.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, enable_gqa=True)
    return o.transpose(1, 2)


class LlamaSdpaAttention(LlamaAttention):
    """Attention forward with the Fourier KV cache (reference: modeling_llama_fourier.py:547-667)."""

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value: Optional[Cache] = None,
                output_attentions: bool = False, use_cache: bool = False, cache_position=None,
                position_embeddings: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, **kwargs):
        if output_attentions:
            raise NotImplementedError("output_attentions=True is not available on the Fourier path")
        bsz, q_len, _ = hidden_states.size()
        q = self.q_proj(hidden_states).view(bsz, q_len, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        if position_embeddings is None:
            cos, sin = self.rotary_emb(v, position_ids)
        else:
            cos, sin = position_embeddings
        q, k = apply_rotary_pos_emb(q, k, cos, sin)

        if past_key_value is None:
            kd = {"k_init": None, "k_compressed": None, "k_uncompressed": None,
                  "k_local": k.transpose(1, 2).reshape(bsz, q_len, -1)}
            vd = {"v_local": v.transpose(1, 2).reshape(bsz, q_len, -1)}
        else:
            kd, vd = past_key_value.update(k, v, self.layer_idx, {"sin": sin, "cos": cos,
                                                                   "cache_position": cache_position})
        if kd["k_init"] is None and kd["k_compressed"] is None and kd["k_uncompressed"] is None:
            attn = _dense_causal(q.transpose(1, 2), kd["k_local"], vd["v_local"], self.num_key_value_heads,
                                 self.head_dim)
        else:
            qf = q.transpose(1, 2).reshape(bsz, q_len, self.num_heads * self.head_dim)
            if isinstance(past_key_value, DynamicCache):
                attn = past_key_value.fourier_attention(qf, self.layer_idx, self.num_heads)
            else:   # a foreign cache that follows the reference's dict contract
                from .fourier_triton_valid4_v2 import triton_fourier_attn
                c, L = past_key_value, self.layer_idx
                attn = triton_fourier_attn(
                    q=qf.contiguous(), k_il=torch.cat([kd["k_init"], kd["k_local"]], dim=1).contiguous(),
                    v_il=torch.cat([vd["v_init"], vd["v_local"]], dim=1).contiguous(),
                    k_mc=kd["k_compressed"], v_mc=vd["v_compressed"], k_mn=kd["k_uncompressed"],
                    v_mn=vd["v_uncompressed"], avg_k_u=c.k_layer_average[L], avg_k_d=c.kd_layer_average[L],
                    scale_k=c.k_scale[L], avg_v_u=c.v_layer_average[L], avg_v_d=c.vd_layer_average[L],
                    scale_v=c.v_scale[L], kc_list=c.k_non_critical_dims[L], kc_h_list=c.k_non_critical_head_dims[L],
                    kn_list=c.k_critical_dims[L], kn_h_list=c.k_critical_head_dims[L],
                    vc_list=c.v_non_critical_dims[L], vc_h_list=c.v_non_critical_head_dims[L],
                    vn_list=c.v_critical_dims[L], vn_h_list=c.v_critical_head_dims[L],
                    num_head_q=self.num_heads, num_head_kv=self.num_key_value_heads,
                    seq_len_m=kd["k_uncompressed"].size(1), T=c.maxtokens - c.numinittokens - c.maxlocallen)
            attn = attn.transpose(1, 2).contiguous()
        attn = attn.reshape(bsz, q_len, -1).to(q.dtype)
        return self.o_proj(attn), None, past_key_value


LLAMA_ATTENTION_CLASSES = {"eager": LlamaSdpaAttention, "flash_attention_2": LlamaSdpaAttention,
                           "sdpa": LlamaSdpaAttention}


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.self_attn = LLAMA_ATTENTION_CLASSES[config._attn_implementation](config=config, layer_idx=layer_idx)
        self.mlp = LlamaMLP(config)
        self.input_layernorm = LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden_states, past_key_value=None, position_embeddings=None, **kwargs):
        h, _, _ = self.self_attn(self.input_layernorm(hidden_states), past_key_value=past_key_value,
                                 position_embeddings=position_embeddings, **kwargs)
        hidden_states = hidden_states + h
        return hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))


class LlamaModel(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([LlamaDecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.norm = LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.rotary_emb = LlamaRotaryEmbedding(config)

    def forward(self, input_ids, past_key_values=None, position_ids=None, use_cache=True):
        h = self.embed_tokens(input_ids)
        if position_ids is None:
            past = past_key_values._seen_tokens if past_key_values is not None else 0
            position_ids = torch.arange(past, past + input_ids.shape[1], device=input_ids.device)[None].expand(
                input_ids.shape[0], -1)
        pe = self.rotary_emb(h, position_ids)
        for layer in self.layers:
            h = layer(h, past_key_value=past_key_values, position_embeddings=pe)
        return self.norm(h)


class LlamaForCausalLM(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.model = LlamaModel(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        std = config.initializer_range
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                m.weight.data.normal_(mean=0.0, std=std)
                if getattr(m, "bias", None) is not None:
                    m.bias.data.zero_()

    def forward(self, input_ids, past_key_values=None, use_cache=True, num_logits_to_keep: int = 1, **kwargs):
        h = self.model(input_ids, past_key_values=past_key_values)
        logits = self.lm_head(h[:, -num_logits_to_keep:, :])
        return SimpleNamespace(logits=logits, past_key_values=past_key_values)
