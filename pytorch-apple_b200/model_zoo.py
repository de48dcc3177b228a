"""Seeded, offline builders for the two model families the CUDA path serves:
torchvision-topology ResNet-18/50 and Qwen2.5-1.5B-architecture prefill/decode.

The Qwen wrappers present the same calling convention as the reference's
extraction wrappers (examples/extract_qwen_ir.py:39-131): positional inputs
``input_ids, attention_mask, position_ids, cache_position[, *past_kv_flat]`` and
outputs ``(logits, k0, v0, k1, v1, ...)``; decode writes the new K/V rows into
fixed-shape ``[B, kv_heads, max_cache_len, head_dim]`` buffers with an
out-of-place ``index_copy`` along dim 2.  No checkpoint is read: weights are drawn
from a seeded generator, which stands in for the published checkpoint.
"""

from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn as nn

QWEN25_1P5B = dict(
    vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
    num_attention_heads=12, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
)


# --------------------------------------------------------------------------
# Qwen2
# --------------------------------------------------------------------------
def qwen2_config(num_layers: int | None = None, **overrides):
    from transformers import Qwen2Config

    kw = dict(QWEN25_1P5B)
    kw.update(overrides)
    if num_layers is not None:
        kw["num_hidden_layers"] = num_layers
    kw.pop("head_dim", None)
    cfg = Qwen2Config(max_position_embeddings=32768, tie_word_embeddings=True, attention_dropout=0.0, **kw)
    cfg._attn_implementation = "eager"
    return cfg


def qwen2_model(cfg, device: str = "meta", dtype=torch.bfloat16) -> nn.Module:
    from transformers import Qwen2ForCausalLM

    with torch.device(device):
        model = Qwen2ForCausalLM(cfg)
    model = model.to(dtype).eval()
    # ``.to(dtype)`` also narrows the rotary ``inv_freq`` buffers; checkpoints loaded the
    # usual way keep them in fp32, and the graphs compute the angle in fp32.
    rot = model.model.rotary_emb
    rot.inv_freq = rot.inv_freq.float() if device == "meta" else _inv_freq(cfg).to(device)
    rot.original_inv_freq = rot.inv_freq.clone() if device != "meta" else rot.inv_freq
    return model


def _inv_freq(cfg) -> torch.Tensor:
    hd = cfg.hidden_size // cfg.num_attention_heads
    theta = getattr(cfg, "rope_theta", None) or cfg.rope_parameters["rope_theta"]
    return 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.int64).to(torch.float32) / hd))


class _StaticKV:
    """Fixed-shape KV store updated with out-of-place ``index_copy`` (dim 2)."""

    def __init__(self, flat, num_layers, cache_position):
        self.keys = [flat[2 * i] for i in range(num_layers)]
        self.values = [flat[2 * i + 1] for i in range(num_layers)]
        self._pos = cache_position

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        self.keys[layer_idx] = self.keys[layer_idx].index_copy(2, self._pos, key_states)
        self.values[layer_idx] = self.values[layer_idx].index_copy(2, self._pos, value_states)
        return self.keys[layer_idx], self.values[layer_idx]

    def get_seq_length(self, layer_idx=0):
        return self.keys[0].shape[-2]

    def get_mask_sizes(self, cache_position, layer_idx=0):
        return self.keys[0].shape[-2], 0

    def __len__(self):
        return len(self.keys)


class QwenPrefillWrapper(nn.Module):
    def __init__(self, model):
        super().__init__()
        self.model = model

    def forward(self, input_ids, attention_mask, position_ids, cache_position):
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                         cache_position=cache_position, use_cache=True)
        flat = [out.logits]
        cache = out.past_key_values
        for i in range(len(cache.layers)):
            flat += [cache.layers[i].keys, cache.layers[i].values]
        return tuple(flat)


class QwenDecodeWrapper(nn.Module):
    def __init__(self, model, num_layers):
        super().__init__()
        self.model = model
        self.num_layers = num_layers

    def forward(self, input_ids, attention_mask, position_ids, cache_position, *past_kv_flat):
        cache = _StaticKV(past_kv_flat, self.num_layers, cache_position)
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                         cache_position=cache_position, past_key_values=cache, use_cache=True)
        flat = [out.logits]
        for i in range(self.num_layers):
            flat += [cache.keys[i], cache.values[i]]
        return tuple(flat)


def qwen2_example_inputs(cfg, batch: int, seq: int, cache_len: int | None, device="meta", dtype=torch.bfloat16):
    """Example tensors for export.  ``cache_len=None`` -> prefill of ``seq`` tokens,
    else a decode step (``seq`` must be 1) over a ``cache_len``-row cache."""
    kvh = cfg.num_key_value_heads
    hd = cfg.hidden_size // cfg.num_attention_heads
    with torch.device(device):
        ids = torch.zeros(batch, seq, dtype=torch.long)
        pos = torch.zeros(batch, seq, dtype=torch.long)
        cpos = torch.zeros(seq, dtype=torch.long)
        if cache_len is None:
            mask = torch.zeros(batch, 1, seq, seq, dtype=dtype)
            return (ids, mask, pos, cpos)
        mask = torch.zeros(batch, 1, seq, cache_len, dtype=dtype)
        kv = tuple(torch.zeros(batch, kvh, cache_len, hd, dtype=dtype) for _ in range(2 * cfg.num_hidden_layers))
    return (ids, mask, pos, cpos) + kv


def qwen2_weights(cfg, seed: int = 0, dtype=torch.bfloat16, device="cpu", prefix: str = "model.") -> dict[str, torch.Tensor]:
    """State dict drawn from ``seed``: projections, biases and embeddings ~N(0, 0.02),
    RMSNorm gains ~N(1, 0.02); tied ``lm_head``; ``inv_freq`` for the config's theta.
    Keys carry ``prefix`` because the export wrappers hold the network as ``.model``."""
    g = torch.Generator(device=device).manual_seed(seed)
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    hd = H // cfg.num_attention_heads
    kvd = cfg.num_key_value_heads * hd

    def normal(*shape, mean=0.0):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * 0.02 + mean).to(dtype)

    sd: dict[str, torch.Tensor] = {}
    sd["model.embed_tokens.weight"] = normal(V, H)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = normal(H, H)
        sd[p + "self_attn.q_proj.bias"] = normal(H)
        sd[p + "self_attn.k_proj.weight"] = normal(kvd, H)
        sd[p + "self_attn.k_proj.bias"] = normal(kvd)
        sd[p + "self_attn.v_proj.weight"] = normal(kvd, H)
        sd[p + "self_attn.v_proj.bias"] = normal(kvd)
        sd[p + "self_attn.o_proj.weight"] = normal(H, H)
        sd[p + "mlp.gate_proj.weight"] = normal(I, H)
        sd[p + "mlp.up_proj.weight"] = normal(I, H)
        sd[p + "mlp.down_proj.weight"] = normal(H, I)
        sd[p + "input_layernorm.weight"] = normal(H, mean=1.0)
        sd[p + "post_attention_layernorm.weight"] = normal(H, mean=1.0)
    sd["model.norm.weight"] = normal(H, mean=1.0)
    sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    inv = _inv_freq(cfg)
    sd["model.rotary_emb.inv_freq"] = inv.to(device)
    sd["model.rotary_emb.original_inv_freq"] = inv.to(device).clone()
    return {prefix + k: v for k, v in sd.items()}


def causal_mask(batch: int, q_len: int, kv_len: int, valid_len, dtype=torch.bfloat16) -> torch.Tensor:
    """Additive mask ``[B,1,q_len,kv_len]``: 0 where key j <= query position, else
    the dtype's most negative finite value (what transformers emits).  ``valid_len``
    is the number of cache rows already filled before these ``q_len`` queries."""
    neg = torch.finfo(dtype).min
    j = torch.arange(kv_len)[None, :]
    i = torch.arange(q_len)[:, None] + int(valid_len)
    m = torch.where(j <= i, 0.0, neg).to(dtype)
    return m[None, None].expand(batch, 1, q_len, kv_len).contiguous()


# --------------------------------------------------------------------------
# ResNet
# --------------------------------------------------------------------------
def resnet(depth: int, seed: int = 0, device: str = "cpu") -> nn.Module:
    """torchvision ResNet-18/50 topology with seeded statistics: conv Kaiming-normal
    (fan_out), fc default init, BN gamma~U(.5,1.5), beta~N(0,.1), running_mean~N(0,.1),
    running_var~U(.5,1.5).  Returned in eval mode, fp32."""
    import torchvision

    torch.manual_seed(seed)
    ctor = {18: torchvision.models.resnet18, 50: torchvision.models.resnet50}[depth]
    if device == "meta":
        with torch.device("meta"):
            return ctor(weights=None).eval()
    model = ctor(weights=None)
    g = torch.Generator().manual_seed(seed)
    for m in model.modules():
        if isinstance(m, nn.Conv2d):
            fan_out = m.out_channels * m.kernel_size[0] * m.kernel_size[1]
            with torch.no_grad():
                m.weight.copy_(torch.randn(m.weight.shape, generator=g) * math.sqrt(2.0 / fan_out))
        elif isinstance(m, nn.BatchNorm2d):
            with torch.no_grad():
                m.weight.copy_(torch.rand(m.weight.shape, generator=g) + 0.5)
                m.bias.copy_(torch.randn(m.bias.shape, generator=g) * 0.1)
                m.running_mean.copy_(torch.randn(m.running_mean.shape, generator=g) * 0.1)
                m.running_var.copy_(torch.rand(m.running_var.shape, generator=g) + 0.5)
        elif isinstance(m, nn.Linear):
            with torch.no_grad():
                bound = 1.0 / math.sqrt(m.in_features)
                m.weight.copy_((torch.rand(m.weight.shape, generator=g) * 2 - 1) * bound)
                m.bias.copy_((torch.rand(m.bias.shape, generator=g) * 2 - 1) * bound)
    return model.eval()


def state_dict_numpy(sd: dict[str, torch.Tensor]) -> dict[str, np.ndarray]:
    """torch state dict -> numpy dict; bf16 tensors become ``ml_dtypes.bfloat16`` views."""
    import ml_dtypes

    out = {}
    for k, t in sd.items():
        t = t.detach().cpu()
        if t.dtype == torch.bfloat16:
            out[k] = t.contiguous().view(torch.uint16).numpy().view(ml_dtypes.bfloat16)
        elif t.ndim == 0:
            out[k] = np.asarray(t.item())
        else:
            out[k] = t.contiguous().numpy()
    return out
