"""The Marinex decoder without a GPU: its configuration, its plan and stored names, what its runs keep in the cache,
and the plain implementation's mechanisms against closed forms."""
import copy
import math

import numpy as np
import pytest

from plain import marinex_plain as P
from marinex_tiny import CONFIGS, MAR_A, make_folder, random_tokens


def test_configuration_round_trip_and_errors():
    from burn_lm_b200.config import ConfigError, MarinexConfig
    for cfg in CONFIGS.values():
        typed = MarinexConfig.from_dict(cfg)
        assert MarinexConfig.from_dict(typed.to_dict()) == typed and typed.to_dict() == cfg
        assert len(typed.layers) == len(cfg["layers"])
    for path, value, key in ((("layers", 0, "type"), "conv", "layers[0].type"),
                             (("layers", 0, "mixer", "rot", "dims"), 7, "layers[0].mixer.rot.dims"),
                             (("layers", 0, "mixer", "rot", "dims"), 26, "layers[0].mixer.rot.dims"),
                             (("layers", 0, "mixer", "kv_heads"), 3, "layers[0].mixer.heads"),
                             (("layers", 0, "mixer", "softcap"), 0.0, "layers[0].mixer.softcap"),
                             (("layers", 1, "mixer", "kv_rank"), 0, "layers[1].mixer.kv_rank"),
                             (("layers", 1, "mixer", "q_rank"), None, "layers[1].mixer.q_rank"),
                             (("layers", 1, "mixer", "mask", "size"), 0, "layers[1].mixer.mask.size"),
                             (("layers", 1, "mixer", "rot", "dims"), 18, "layers[1].mixer.rot.dims"),
                             (("layers", 0, "mlp", "router", "top"), 5, "layers[0].mlp.router.top"),
                             (("layers", 0, "mlp", "router", "groups", "count"), 3, "layers[0].mlp.router.groups.count"),
                             (("layers", 0, "mlp", "router", "groups", "keep"), 5, "layers[0].mlp.router.groups.keep"),
                             (("layers", 0, "mlp", "kind"), "dense", "layers[0].mlp.kind"),
                             (("layers", 0, "mlp", "expert", "ff"), None, "layers[0].mlp.expert.ff"),
                             (("norm", "eps"), "x", "norm.eps"), (("width",), 0, "width")):
        bad = copy.deepcopy(MAR_A)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=key.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
            MarinexConfig.from_dict(bad)


def test_the_plan_names_the_stored_tensors():
    from burn_lm_b200.model import plan_of, tensor_specs_of
    arch, typed, plan = plan_of(MAR_A)
    assert arch.name == "Marinex" and plan.head.tensors == {"weight": "head"} and plan.embedding.tensors == {"table": "embed"}
    assert [lp.block for lp in plan.layers] == ["postnorm"] * 5 and [e.layer for e in plan.schedule] == [0, 1, 2, 3, 4]
    assert [lp.part("mixer").kind for lp in plan.layers] == ["normed_attention", "latent_attention"] * 2 + ["normed_attention"]
    names = {s.name: tuple(s.shape) for s in tensor_specs_of(MAR_A)}
    assert names["embed"] == (288, 96) and names["head"] == (288, 96) and names["final.norm"] == (96,)
    assert names["l0.mix.q"] == (96, 96) and names["l0.mix.k"] == (48, 96) and names["l0.mix.v"] == (32, 96) and names["l0.mix.o"] == (96, 64)
    assert names["l0.mix.q.norm"] == (24,) and names["l0.mix.k.norm"] == (24,) and names["l0.mix.temp"] == (4,) and names["l0.norm1"] == (96,)
    assert names["l1.mix.dq"] == (48, 96) and names["l1.mix.dq.norm"] == (48,) and names["l1.mix.uq"] == (4 * 32, 48)
    assert names["l1.mix.dkv"] == (48, 96) and names["l1.mix.dkv.norm"] == (32,) and names["l1.mix.uk"] == (64, 32) and names["l1.mix.uv"] == (96, 32)
    assert names["l1.mix.g"] == (4, 96) and names["l1.mix.sink"] == (4,) and names["l1.mix.o"] == (96, 96)
    assert names["l0.mlp.router"] == (8, 96) and names["l0.mlp.correction"] == (8,) and names["l0.mlp.e7.up"] == (48, 96) and names["l0.mlp.e7.down"] == (96, 48)
    assert "l0.mlp.e0.gate" not in names and "l0.mlp.e8.up" not in names and "l1.norm2" not in names and "l1.mlp.router" not in names
    assert "l1.mix.q" not in names and "l4.norm2" not in names and names["l3.norm2"] == (96,)


def test_what_the_runs_keep():
    import torch
    from burn_lm_b200.model import Model, plan_of
    from burn_lm_b200.parts.base import Runtime
    _, _, plan = plan_of(MAR_A)
    model = Model(plan, Runtime(torch.float32, "cpu"), MAR_A)
    needs = model.cache_needs()
    assert [n.kind for n in needs] == ["kv", "rows", "kv", "rows", "kv"]
    assert (needs[0].n_kv_heads, needs[0].head_dim, needs[0].value_dim, needs[0].window) == (2, 24, 16, None)
    assert (needs[1].head_dim, needs[1].window) == (32 + 16, 20) and (needs[3].head_dim, needs[3].window) == (48 + 8, 70)
    # the block reads the stream itself: what stands where its first norm would takes a pending normed output
    assert model.layers[0].block.first_norm().takes_post_normed
    assert sorted(model.kernel_modules()) == ["attention_latent", "attention_sink", "elementwise", "gemm", "moe", "stream_ops"]


def test_folders_hold_what_the_plain_implementation_reads(tmp_path):
    folder = make_folder(tmp_path, "mar_c")
    cfg, tensors = P.read_model_folder(folder)
    after = []
    logits = P.forward(cfg, tensors, random_tokens(0, 40, cfg["vocab"]), after)
    assert logits.shape == (40, cfg["vocab"]) and len(after) == 4 and np.isfinite(logits).all()
    # causal: a later token changes nothing before it
    again = P.forward(cfg, tensors, random_tokens(0, 40, cfg["vocab"])[:35] + [3, 1, 4, 1, 5])
    assert np.abs(again[:35] - logits[:35]).max() < 1e-12 and np.abs(again[35:] - logits[35:]).max() > 1e-3
    # the package's random-weights mode writes the same names and shapes
    from burn_lm_b200 import write_random_model
    other = write_random_model(str(tmp_path / "r"), cfg, seed=1, dtype="float32")
    _, drawn = P.read_model_folder(other)
    assert set(drawn) == set(tensors) and all(drawn[k].shape == tensors[k].shape for k in tensors)
    assert np.isfinite(P.forward(cfg, drawn, [1, 2, 3])).all()


# the plain implementation's mechanisms against closed forms --------------------------------------------------
def test_plain_norm_has_the_epsilon_inside_the_root():
    assert np.allclose(P.rms(np.full((1, 4), 1e-3), 1e-2), 1e-3 / np.sqrt(1e-6 + 1e-2))
    assert np.allclose(P.rms_norm(np.array([[3.0, -4.0]]), np.array([2.0, 0.5]), 0.0), [[3.0 / np.sqrt(12.5) * 2, -4.0 / np.sqrt(12.5) * 0.5]])


def test_plain_activation_is_the_exact_one():
    z = np.array([-3.0, -0.5, 0.0, 0.7, 4.0])
    assert np.allclose(P.gelu_erf(z), [x * 0.5 * math.erfc(-x / math.sqrt(2.0)) for x in z])
    tanh_form = 0.5 * z * (1 + np.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    assert 1e-5 < np.abs(P.gelu_erf(z) - tanh_form).max() < 1e-3          # close to the other form, and not it


@pytest.mark.parametrize("turn", [P.rotate_neighbours, P.rotate_halves])
def test_plain_rotations_depend_on_the_distance_only(turn):
    rng = np.random.default_rng(1)
    q, k = rng.normal(size=(1, 1, 12)), rng.normal(size=(1, 1, 12))
    at = lambda p: np.array([float(p)])
    dots = [float((turn(q, at(i), 8, 100.0) * turn(k, at(j), 8, 100.0)).sum()) for i, j in ((5, 2), (13, 10), (103, 100))]
    assert np.allclose(dots, dots[0])
    assert np.array_equal(turn(q, at(9), 8, 100.0)[..., 8:], q[..., 8:]) and np.array_equal(turn(q, at(0), 8, 100.0), q)


def test_plain_rotations_pair_different_lanes():
    x = np.zeros((1, 8))
    x[0, 0] = 1.0
    a, b = P.rotate_neighbours(x, np.array([1.0]), 8, 10.0), P.rotate_halves(x, np.array([1.0]), 8, 10.0)
    assert np.allclose(a[0, :2], [np.cos(1.0), np.sin(1.0)]) and np.allclose(a[0, 2:], 0)
    assert np.allclose(b[0, [0, 4]], [np.cos(1.0), np.sin(1.0)]) and np.allclose(b[0, [1, 2, 3, 5, 6, 7]], 0)
    x = np.zeros((1, 8))
    x[0, 3] = 1.0                       # the second lane of pair 1, or the first lane of pair 3
    f = P.frequencies(8, 10.0)
    assert np.allclose(P.rotate_neighbours(x, np.array([2.0]), 8, 10.0)[0, [2, 3]], [-np.sin(2 * f[1]), np.cos(2 * f[1])])
    assert np.allclose(P.rotate_halves(x, np.array([2.0]), 8, 10.0)[0, [3, 7]], [np.cos(2 * f[3]), np.sin(2 * f[3])])


def test_plain_softmax_with_a_sink():
    s = np.log(np.array([[1.0, 2.0, 5.0]]))
    see = np.array([[True, True, False]])
    assert np.allclose(P.softmax_with_sink(s, see, 0.0), [[0.25, 0.5, 0.0]])                 # 1 + 1 + 2 in the denominator
    assert np.allclose(P.softmax_with_sink(s, see, np.log(7.0)), [[0.1, 0.2, 0.0]])
    assert np.allclose(P.softmax_with_sink(s + 700.0, see, 0.0), [[1 / 3, 2 / 3, 0.0]])      # no overflow; the sink vanishes
    assert np.allclose(P.softmax_with_sink(s - 700.0, see, 0.0), 0.0)                        # the sink takes everything


def test_plain_windows():
    assert P.window(5, 2).astype(int).tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 1, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 1, 1]]
    assert np.array_equal(P.window(4, 1), np.eye(4, dtype=bool)) and np.array_equal(P.window(4, 9), P.causal(4))


def test_plain_attention_written_out():
    """One head at a time with explicit loops: the norms before the turn, the head's number, the cap, the sink of score 0."""
    rng = np.random.default_rng(3)
    T, D, H, G, dk, dv, eps = 6, 10, 4, 2, 4, 3, 1e-5
    h = rng.normal(size=(T, D))
    w = {"q": rng.normal(size=(H * dk, D)), "k": rng.normal(size=(G * dk, D)), "v": rng.normal(size=(G * dv, D)), "q.norm": rng.normal(size=dk),
         "k.norm": rng.normal(size=dk), "temp": rng.uniform(0.5, 2, size=H), "o": np.eye(H * dv)}
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": 0.7, "softcap": 2.0, "rot": {"dims": 2, "base": 10.0}}
    got = P.attention(h, w, m, eps, "")
    unit = lambda x: x / np.sqrt((x * x).mean() + eps)
    turn = lambda x, p: np.concatenate([[x[0] * np.cos(p) - x[1] * np.sin(p), x[1] * np.cos(p) + x[0] * np.sin(p)], x[2:]])
    for t in range(T):
        for i in range(H):
            g = i // 2
            q = turn(unit((w["q"] @ h[t])[i * dk:(i + 1) * dk]) * w["q.norm"], t)
            ks = [turn(unit((w["k"] @ h[s])[g * dk:(g + 1) * dk]) * w["k.norm"], s) for s in range(t + 1)]
            vs = [unit((w["v"] @ h[s])[g * dv:(g + 1) * dv]) for s in range(t + 1)]
            e = np.exp([2.0 * np.tanh(0.7 * w["temp"][i] * (q @ k) / 2.0) for k in ks])
            assert np.allclose(got[t, i * dv:(i + 1) * dv], sum(p * v for p, v in zip(e / (1.0 + e.sum()), vs)))


def test_plain_latent_attention_is_attention_over_up_projected_keys():
    """Written out per head with keys [W_uk c | shared turned part] and values W_uv c, a window of three, a sink and a gate."""
    rng = np.random.default_rng(4)
    T, D, H, dk, dr, dv, R, Q, eps = 7, 10, 2, 4, 2, 3, 5, 6, 1e-5
    h = rng.normal(size=(T, D))
    w = {"dq": rng.normal(size=(Q, D)), "dq.norm": rng.normal(size=Q), "uq": rng.normal(size=(H * (dk + dr), Q)), "dkv": rng.normal(size=(R + dr, D)),
         "dkv.norm": rng.normal(size=R), "uk": rng.normal(size=(H * dk, R)), "uv": rng.normal(size=(H * dv, R)), "g": rng.normal(size=(H, D)),
         "sink": rng.normal(size=H), "o": np.eye(H * dv)}
    m = {"heads": H, "dim": dk, "rot_dim": dr, "vdim": dv, "kv_rank": R, "q_rank": Q, "scale": 0.4, "mask": {"size": 3}, "rot": {"dims": 2, "base": 10.0}}
    got = P.latent_attention(h, w, m, eps, "")
    unit = lambda x: x / np.sqrt((x * x).mean() + eps)
    turn = lambda x, p: np.array([x[0] * np.cos(p) - x[1] * np.sin(p), x[1] * np.cos(p) + x[0] * np.sin(p)])
    down = h @ w["dkv"].T
    c = np.stack([unit(down[s, :R]) * w["dkv.norm"] for s in range(T)])
    for t in range(T):
        q_all = w["uq"] @ (unit(w["dq"] @ h[t]) * w["dq.norm"])
        for i in range(H):
            q = q_all[i * (dk + dr):(i + 1) * (dk + dr)]
            seen = range(max(0, t - 2), t + 1)
            e = np.exp([0.4 * (q[:dk] @ (w["uk"][i * dk:(i + 1) * dk] @ c[s]) + turn(q[dk:], t) @ turn(down[s, R:], s)) for s in seen])
            o = sum(p * (w["uv"][i * dv:(i + 1) * dv] @ c[s]) for p, s in zip(e / (np.exp(w["sink"][i]) + e.sum()), seen))
            assert np.allclose(got[t, i * dv:(i + 1) * dv], o * P.sigmoid(w["g"][i] @ h[t]))


def test_plain_routing_by_groups():
    f = {"router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}}
    logit = lambda p: np.log(p / (1 - p))
    scores = np.array([0.9, 0.1, 0.6, 0.6, 0.2, 0.8])                   # marks of the groups: 1.0, 1.2, 1.0
    w = {"router": logit(scores)[:, None], "correction": np.zeros(6)}
    ids, wt = P.route(np.ones((1, 1)), w, f, "")
    assert ids.tolist() == [[2, 3]] and np.allclose(wt, [[0.6, 0.6]])   # the best expert of all lies in a group that is left out
    w["correction"] = np.array([0.0, 0.5, 0.0, 0.0, 0.0, 0.0])          # the first group's mark is 1.5 now
    ids, wt = P.route(np.ones((1, 1)), w, f, "")
    assert ids.tolist() == [[0, 1]] and np.allclose(wt, [[0.9, 0.1]])   # chosen with the correction, weighed without it
    w["correction"] = np.array([-5.0, -5.0, -5.0, -5.0, -5.5, -5.0])    # negative choice scores: a left-out group counts as minus infinity, not 0
    f["router"]["groups"]["keep"] = 2
    ids, _ = P.route(np.ones((1, 1)), w, f, "")
    assert ids.tolist() == [[0, 2]]                                     # groups 0 (-9.0) and 1 (-8.8) are kept; expert 5 (-4.2) is not among them
    f["router"]["groups"] = {"count": 1, "keep": 1}
    assert P.route(np.ones((1, 1)), w, f, "")[0].tolist() == [[0, 5]]


def test_plain_layer_norms_the_sublayers_output_only():
    """x <- x + norm(mixer(x)): the stream itself is never normed on its way into a sublayer."""
    rng = np.random.default_rng(5)
    cfg = {"type": "attention", "mlp": None, "mixer": {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "softcap": 9.0, "rot": {"dims": 0, "base": 10.0}}}
    w = {"l0.mix." + k: rng.normal(size=s) for k, s in (("q", (4, 6)), ("k", (4, 6)), ("v", (4, 6)), ("o", (6, 4)), ("q.norm", (4,)), ("k.norm", (4,)), ("temp", (1,)))}
    w["l0.norm1"] = rng.normal(size=6)
    x = rng.normal(size=(5, 6))
    out = P.layer(x, w, cfg, 1e-5, 0)
    assert np.allclose(out - x, P.rms_norm(P.attention(x, w, cfg["mixer"], 1e-5, "l0.mix."), w["l0.norm1"], 1e-5))
    # queries, keys and values are all normed head by head: the mixer's output is blind to the scale of v's weight and
    # (up to eps) to the scale of the stream it reads, while the stream itself passes unscaled
    w2 = dict(w)
    w2["l0.mix.v"] = 3.0 * w["l0.mix.v"]
    assert np.allclose(P.layer(x, w2, cfg, 1e-5, 0), out, atol=1e-4)
    assert np.allclose(P.layer(2 * x, w, cfg, 1e-5, 0) - 2 * x, out - x, atol=1e-3)
