"""Named configurations, as config.json dicts.

The reference keeps its models' sizes as constructor presets (crates/burn-lm-llama/src/nn/llama/
base.rs:73-139: llama3_2_1b, llama3_2_3b, llama3_1_8b, ...); here the same sizes are written with the
keys a Llama model folder's config.json carries, so a preset and a folder go through one reader.
Stop ids follow the reference's tokenizer: 256 special tokens after 128,000 ranks, of which
<|end_of_text|> is the 2nd, <|eom_id|> the 9th and <|eot_id|> the 10th
(crates/burn-lm-llama/src/tokenizer/tiktoken.rs:17-30,126-132).

The two tiny ones differ from each other in every size and option (layers, width, heads and groups,
head size, inner size, vocabulary, theta, scaling, eps, tied or untied head, positions); tests and the
smoke run use them with random weights.
"""
from __future__ import annotations

import copy


def _llama3(layers, width, heads, kv_heads, head_dim, inner, factor, tied, positions=131072):
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": layers, "hidden_size": width, "num_attention_heads": heads,
        "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inner,
        "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": tied, "max_position_embeddings": positions,
        "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
        "bos_token_id": 128000, "eos_token_id": [128001, 128008, 128009],
    }


_PRESETS = {
    # base.rs:106-115
    "llama3_2_1b": _llama3(16, 2048, 32, 8, 64, 8192, 32.0, True),
    # base.rs:75-86
    "llama3_2_3b": _llama3(28, 3072, 24, 8, 128, 8192, 32.0, True),
    # base.rs:117-123 (default width 4096, 32 layers, 32 heads: base.rs:43-52; default scaling factor 8)
    "llama3_1_8b": _llama3(32, 4096, 32, 8, 128, 14336, 8.0, False),
    "tiny_a": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
        "head_dim": 16, "intermediate_size": 160, "vocab_size": 256, "rope_theta": 10000.0,
        "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
        "max_position_embeddings": 128, "hidden_act": "silu",
    },
    "tiny_b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 1,
        "head_dim": 32, "intermediate_size": 512, "vocab_size": 384, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 64},
        "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256,
        "hidden_act": "silu", "eos_token_id": [7, 11],
    },
}


def _fobilorn_layer(heads, kv_heads, dim, vdim, window, keep_first, mlp, v_mix=True):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "v_mix": v_mix,
                      "mask": {"size": window, "keep_first": keep_first}}}


def _moe(experts, top, ff, shared_ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": {"ff": shared_ff} if shared_ff else None}


# a small Fobilorn decoder that uses every branch of the design: a dense and two mixture-of-experts layers (one
# without a shared expert), a layer without a feed-forward, layers inside and outside the blending of values,
# one and several kv heads, values wider and narrower than the keys
_PRESETS["fobilorn_tiny"] = {
    "architecture": "Fobilorn", "vocab": 384, "width": 96,
    "embedding": {"bigram": {"buckets": 211, "mul_prev": 13, "mul_cur": 29}}, "norm": {"eps": 1e-5},
    "layers": [
        _fobilorn_layer(4, 2, 24, 16, 40, 6, {"kind": "dense", "ff": 160}),
        _fobilorn_layer(6, 1, 16, 40, 24, 0, _moe(6, 2, 48, 64), v_mix=False),
        _fobilorn_layer(4, 2, 32, 16, 70, 3, None),
        _fobilorn_layer(2, 2, 24, 16, 33, 9, _moe(5, 1, 32, None)),
    ],
}


def _nufolix_parallel(heads, kv_heads, dim, vdim, rot_dims, r_heads, r_qk_heads, r_dim, r_vdim, r_conv, ff, left_scale=0.5,
                      right_scale=1.25, softcap=15.0, base=10000.0, scale=None):
    return {"type": "parallel", "mlp": {"kind": "dense", "ff": ff} if ff else None,
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
                               "softcap": softcap, "rot": {"dims": rot_dims, "base": base}},
                      "right": {"heads": r_heads, "kv_heads": r_qk_heads, "dim": r_dim, "vdim": r_vdim, "conv": r_conv},
                      "left_scale": left_scale, "right_scale": right_scale}}


def _nufolix_mamba2(heads, vdim, state, groups, conv, norm_groups, ff):
    return {"type": "mamba2", "mlp": {"kind": "dense", "ff": ff} if ff else None,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


# a small Nufolix decoder that uses every branch of the design: both kinds of mixer with and without a feed-forward,
# several query heads a key/value head on both sides of the parallel mixer, a rotation of some of a head's lanes,
# state-space heads that share their B and C in groups, a norm in several parts
_PRESETS["nufolix_tiny"] = {
    "architecture": "Nufolix", "vocab": 320, "width": 96, "embedding": {"scale": 9.797958971132712}, "norm": {"eps": 1e-5},
    "residual_mult": 0.8,
    "layers": [
        _nufolix_mamba2(6, 16, 24, 2, 4, 3, None),
        _nufolix_parallel(4, 2, 24, 16, 16, 4, 2, 16, 24, 3, 160),
        _nufolix_mamba2(4, 24, 16, 4, 3, 1, 128),
        _nufolix_parallel(6, 3, 16, 32, 8, 2, 1, 32, 16, 4, None),
    ],
}


def _ridopel_experts(n, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": n, "top": top}}


def _ridopel_latent(heads, dim, rot_dim, rot_dims, vdim, rank, scale, base, mlp):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"dims": rot_dims, "base": base}}}


# a small Ridopel decoder that uses every branch of the design: the three kinds of mixer with and without a
# feed-forward, a loop over two layers of different kinds that starts behind the first layer, fewer turning lanes than
# rotated ones, values wider and narrower than the keys, a cap on the logits
_PRESETS["ridopel_tiny"] = {
    "architecture": "Ridopel", "vocab": 352, "width": 96, "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "logit_softcap": 20.0,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        {"type": "hgrn2", "mixer": {"heads": 3, "dim": 16, "vdim": 32}, "mlp": _ridopel_experts(8, 2, 48, 1.5)},
        _ridopel_latent(4, 24, 16, 8, 20, 40, 0.17, 10000.0, _ridopel_experts(6, 3, 32, 1.0)),
        {"type": "wkv", "mixer": {"heads": 3, "dim": 32}, "mlp": None},
        _ridopel_latent(2, 16, 8, 8, 48, 24, 0.2, 5000.0, None),
        {"type": "hgrn2", "mixer": {"heads": 2, "dim": 24, "vdim": 16}, "mlp": None},
        {"type": "wkv", "mixer": {"heads": 2, "dim": 16}, "mlp": _ridopel_experts(4, 1, 64, 2.0)},
    ],
}


def _marinex_experts(n, top, ff, groups, keep):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": n, "top": top, "groups": {"count": groups, "keep": keep}}}


def _marinex_attention(heads, kv_heads, dim, vdim, rot_dims, scale, softcap, base, mlp):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
                      "rot": {"dims": rot_dims, "base": base}}}


def _marinex_latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, scale, base, mlp, rot_dims=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
                      "mask": {"size": window}, "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}}


# a small Marinex decoder that uses every branch of the design: both kinds of mixer with and without a feed-forward,
# several query heads a key/value head and one, values wider and narrower than the keys, some and all of a head's lanes
# turning, a window inside a cache page and one across a page border, groups of experts of which some are left out
_PRESETS["marinex_tiny"] = {
    "architecture": "Marinex", "vocab": 288, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        _marinex_attention(4, 2, 24, 16, 12, 0.2, 15.0, 10000.0, _marinex_experts(8, 2, 48, 4, 2)),
        _marinex_latent(4, 16, 16, 24, 48, 32, 20, 0.18, 10000.0, None),
        _marinex_attention(6, 6, 16, 32, 16, 0.25, 8.0, 500000.0, _marinex_experts(6, 3, 32, 2, 1)),
        _marinex_latent(2, 32, 8, 16, 24, 48, 70, 0.16, 5000.0, _marinex_experts(4, 1, 64, 1, 1)),
        _marinex_attention(2, 1, 32, 32, 8, 0.18, 30.0, 10000.0, None),
    ],
}


def preset_names() -> list:
    return sorted(_PRESETS)


def preset(name: str) -> dict:
    """The config.json content of a named configuration (a fresh copy)."""
    from .reader import ConfigError
    key = name.lower().replace("-", "_").replace(".", "_")
    if key not in _PRESETS:
        raise ConfigError(f"no preset named {name!r}; presets: {preset_names()}")
    return copy.deepcopy(_PRESETS[key])


def llama3_2_1b() -> dict:
    return preset("llama3_2_1b")


def llama3_2_3b() -> dict:
    return preset("llama3_2_3b")


def llama3_1_8b() -> dict:
    return preset("llama3_1_8b")


def tiny_a() -> dict:
    return preset("tiny_a")


def tiny_b() -> dict:
    return preset("tiny_b")
