"""Small configurations of the Ridopel decoder for the tests, differing in every size and option, with helpers.

The folders are written here, not by the package's random-weights mode: matrices are drawn with a spread of
gain / sqrt(inputs), so that projections are of size one, attention weights are far from equal, gates and decays
spread over their whole range and the experts' clamps bite; a fault in a rotation, a decay or a choice of experts then
moves the logits by far more than rounding does.
"""
import json
import os

import numpy as np

from burn_lm_b200.config import preset


def experts(n, top, ff, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": n, "top": top}}


def latent(heads, dim, rot_dim, vdim, rank, mlp, rot_dims=None, base=10000.0, scale=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                      "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}}


def hgrn2(heads, dim, vdim, mlp):
    return {"type": "hgrn2", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def wkv(heads, dim, mlp):
    return {"type": "wkv", "mlp": mlp, "mixer": {"heads": heads, "dim": dim}}


def model(vocab, width, layers, taps=3, loop=None, cap=None, eps=1e-5):
    cfg = {"architecture": "Ridopel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    if cap is not None:
        cfg["logit_softcap"] = cap
    return cfg


# every branch (see the preset): all three mixers with and without a feed-forward, a loop in the middle of the model
# over two kinds of mixer, fewer turning lanes than rotated ones, a cap on the logits
RID_A = preset("ridopel_tiny")
# values that a model may happen to make equal or 1: one head everywhere, keys as wide as values, one expert, as many
# chosen as there are, one chosen, a convolution of one tap (nothing carried), a loop that runs once, over the first layer
# only, no cap, a scale of 1
RID_B = model(131, 64, [
    latent(1, 32, 32, 32, 32, experts(1, 1, 64), scale=1.0),
    hgrn2(1, 32, 32, experts(3, 3, 32)),
    wkv(1, 64, experts(4, 1, 48)),
    latent(2, 16, 16, 16, 16, None, rot_dims=0),
], taps=1, loop=(0, 1, 1))
# sizes that are no multiples of 8 or of a warp: five heads of 12 + 6 lanes, a latent of 36, values of 20, heads of 20
# and 12 lanes in the scans, a width of 72, five taps, five experts of which three are chosen; the loop runs the whole
# model three times
RID_C = model(257, 72, [
    wkv(5, 12, None),
    latent(5, 12, 6, 20, 36, experts(5, 3, 40, limit=0.7), base=500.0, scale=0.31),
    hgrn2(3, 20, 12, experts(7, 2, 24, limit=3.0)),
], taps=5, loop=(0, 3, 3), cap=12.0, eps=1e-6)
# heads of 64 and 128 lanes, a latent of 256 lanes, states of 64 x 64 and 128 x 64: the sizes of large models; no loop key
RID_D = model(300, 128, [
    latent(4, 128, 64, 128, 256, experts(32, 8, 64), base=1e6),
    wkv(2, 64, experts(8, 2, 128)),
    hgrn2(2, 128, 64, None),
    latent(2, 64, 32, 64, 192, None, rot_dims=16),
], taps=2, cap=50.0)

CONFIGS = {"rid_a": RID_A, "rid_b": RID_B, "rid_c": RID_C, "rid_d": RID_D}

DECAY_RANK = 6      # the inner size of the decays' projection, which no configuration key names


def _values(rng, name, shape, lively=True):
    """A tensor's values by its stored name's ending; not `lively`: every matrix with a gain of one and corrections two
    apart, which decide the choice of experts alone (scores lie between 0 and 1), for the comparisons in bfloat16, where a
    close call between two experts would otherwise be decided by rounding; the weights still follow the scores."""
    last = name.split(".")[-1]
    if name.endswith(("norm", "norm1", "norm2")):
        return 1.0 + 0.2 * rng.normal(size=shape)
    if ".mu." in name or last == "lower":
        return rng.uniform(0.05, 0.95, size=shape)
    if last == "canon1":
        return 0.4 * rng.normal(size=shape)
    if last == "w0":
        return rng.uniform(-5.0, 0.5, size=shape)            # decays from 0.993 a token down to 0.19
    if last == "u":
        return rng.normal(size=shape)
    if last == "b":
        return rng.normal(size=shape) + 1.0
    if last == "correction":
        return 0.1 * rng.normal(size=shape) if lively else 2.0 * rng.permutation(shape[0])
    if name == "embed":
        return rng.normal(size=shape)
    gain = {"router": 3.0, "q": 2.0, "dkv": 2.0, "w2": 2.0, "gate": 2.5, "up": 2.5, "f": 2.0}.get(last, 1.0) if lively else 1.0
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
        shape = tuple(DECAY_RANK if d == -1 else d for d in spec.shape)
        tensors[spec.name] = torch.tensor(_values(rng, spec.name, shape, lively), dtype=torch.float32).to(torch.bfloat16).contiguous()
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
