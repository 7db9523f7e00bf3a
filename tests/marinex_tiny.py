"""Small configurations of the Marinex decoder for the tests, differing in every size and option, with helpers.

The folders are written here, not by the package's random-weights mode: matrices are drawn with a spread of
gain / sqrt(inputs), so that attention weights are far from equal, scores reach their cap, sinks and gates spread over
their range and the groups of experts matter; a fault in a rotation, a window or a choice of experts then moves the
logits by far more than rounding does.
"""
import json
import os

import numpy as np

from burn_lm_b200.config import preset


def experts(n, top, ff, groups=1, keep=1):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": n, "top": top, "groups": {"count": groups, "keep": keep}}}


def attention(heads, kv_heads, dim, vdim, mlp, rot_dims=None, base=10000.0, scale=None, softcap=20.0):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "softcap": softcap,
                      "rot": {"dims": dim if rot_dims is None else rot_dims, "base": base}}}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, mlp, rot_dims=None, base=10000.0, scale=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": scale or (dim + rot_dim) ** -0.5, "mask": {"size": window},
                      "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}}


def model(vocab, width, layers, eps=1e-5):
    return {"architecture": "Marinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# every branch (see the preset): both mixers with and without a feed-forward, groups that are left out, windows inside a
# page and across a page border, some and all lanes turning
MAR_A = preset("marinex_tiny")
# values that a model may happen to make equal or 1: one head everywhere, keys as wide as values, every lane turning and
# none, one expert, as many chosen as there are, one group and all groups kept, a window of one and of two tokens, a
# scale of 1, latents as wide as each other
MAR_B = model(131, 64, [
    attention(1, 1, 32, 32, experts(1, 1, 64), scale=1.0, softcap=1.0),
    latent(1, 32, 32, 32, 32, 32, 1, experts(3, 3, 32, 3, 3), scale=1.0),
    attention(2, 2, 16, 16, None, rot_dims=0),
    latent(2, 16, 16, 16, 16, 16, 2, None, rot_dims=0),
])
# sizes that are no multiples of 8 or of a warp: five heads on one key/value head, heads of 12 and 20 lanes of which 6
# turn, three heads of 12 + 6 lanes on a latent of 36, a width of 72, six experts in three groups of which two are kept
MAR_C = model(257, 72, [
    latent(3, 12, 6, 20, 20, 36, 33, experts(6, 3, 40, 3, 2), base=500.0, scale=0.31),
    attention(5, 1, 12, 20, experts(5, 2, 24, 5, 3), rot_dims=6, base=500.0, softcap=5.0),
    attention(3, 3, 20, 12, None, rot_dims=10, scale=0.3),
    latent(5, 12, 12, 4, 28, 20, 100, None, rot_dims=4),
], eps=1e-6)
# heads of 64 and 128 lanes, latents of 128 and 256 lanes, eight query heads a key/value head: the sizes of large models;
# one latent layer whose keys are wider than the prompt kernels take, windows beyond two pages
MAR_D = model(300, 128, [
    attention(4, 1, 128, 128, experts(16, 4, 64, 4, 2), rot_dims=64, base=1e6, softcap=30.0),
    latent(4, 128, 64, 128, 192, 256, 200, experts(8, 2, 128, 2, 1), base=1e6),
    attention(8, 1, 64, 64, None, rot_dims=32, softcap=50.0),
    latent(4, 64, 32, 64, 96, 128, 130, None, rot_dims=16),
])

CONFIGS = {"mar_a": MAR_A, "mar_b": MAR_B, "mar_c": MAR_C, "mar_d": MAR_D}


def _values(rng, name, shape, lively=True):
    """A tensor's values by its stored name's ending; not `lively`: every matrix with a gain of one and corrections two
    apart, which decide the choice of experts alone (scores lie between 0 and 1), for the comparisons in bfloat16, where a
    close call between two experts would otherwise be decided by rounding; the weights still follow the scores."""
    last = name.split(".")[-1]
    if last in ("norm", "norm1", "norm2"):
        return 1.0 + 0.2 * rng.normal(size=shape)
    if last == "temp":
        return rng.uniform(0.5, 2.0, size=shape)
    if last == "sink":
        return rng.normal(size=shape) * 1.5
    if last == "correction":
        return 0.1 * rng.normal(size=shape) if lively else 2.0 * rng.permutation(shape[0])
    if name == "embed":
        return rng.normal(size=shape)
    gain = {"router": 3.0, "q": 2.0, "k": 2.0, "uq": 2.0, "dkv": 2.0, "up": 2.0, "g": 2.0}.get(last, 1.0) if lively else 1.0
    return gain * rng.normal(size=shape) / np.sqrt(shape[-1])


def make_folder(tmp_path, name, seed=0, config=None, lively=True):
    """A model folder for CONFIGS[name] (or `config`), stored in bfloat16."""
    import torch
    from safetensors.torch import save_file
    from burn_lm_b200.model import tensor_specs_of

    cfg = config if config is not None else CONFIGS[name]
    folder = os.path.join(str(tmp_path), f"{name}-{seed}-{'lively' if lively else 'calm'}")
    if os.path.exists(os.path.join(folder, "model.safetensors")):
        return folder
    os.makedirs(folder, exist_ok=True)
    rng = np.random.default_rng(seed)
    tensors = {}
    for spec in tensor_specs_of(cfg):
        tensors[spec.name] = torch.tensor(_values(rng, spec.name, tuple(spec.shape), lively), dtype=torch.float32).to(torch.bfloat16).contiguous()
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder


def random_tokens(seed, n, vocab):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=n)]


def row_error(got, want):
    """max |got - want| of every row, relative to the row's largest |want|."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return np.abs(got - want).max(axis=-1) / np.abs(want).max(axis=-1)
