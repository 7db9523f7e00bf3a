"""The Ridopel decoder without a GPU: its configuration, its plan, schedule and stored names, the cache of a run that
keeps rows of a latent beside a state, and the plain implementation's mechanisms against closed forms."""
import copy

import numpy as np
import pytest

from plain import ridopel_plain as P
from ridopel_tiny import CONFIGS, RID_A, RID_C, make_folder, random_tokens


def test_configuration_round_trip_and_errors():
    from burn_lm_b200.config import ConfigError, RidopelConfig
    for cfg in CONFIGS.values():
        typed = RidopelConfig.from_dict(cfg)
        assert RidopelConfig.from_dict(typed.to_dict()) == typed
        assert len(typed.layers) == len(cfg["layers"])
    assert RidopelConfig.from_dict(CONFIGS["rid_d"]).loop is None and RidopelConfig.from_dict(CONFIGS["rid_b"]).logit_softcap is None
    for path, value, key in ((("layers", 0, "type"), "conv", "layers[0].type"),
                             (("layers", 1, "mixer", "rot", "dims"), 7, "layers[1].mixer.rot.dims"),
                             (("layers", 1, "mixer", "rot", "dims"), 18, "layers[1].mixer.rot.dims"),
                             (("layers", 1, "mixer", "kv_rank"), 0, "layers[1].mixer.kv_rank"),
                             (("layers", 1, "mlp", "router", "top"), 7, "layers[1].mlp.router.top"),
                             (("layers", 0, "mlp", "kind"), "dense", "layers[0].mlp.kind"),
                             (("layers", 0, "mlp", "expert", "limit"), None, "layers[0].mlp.expert.limit"),
                             (("layers", 2, "mixer", "heads"), 0, "layers[2].mixer.heads"),
                             (("loop", "stop"), 9, "loop"), (("loop", "times"), 0, "loop.times"),
                             (("canon", "taps"), 0, "canon.taps"), (("norm", "eps"), "x", "norm.eps")):
        bad = copy.deepcopy(RID_A)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=key.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
            RidopelConfig.from_dict(bad)


def test_the_plan_names_the_stored_tensors_and_orders_the_runs():
    from burn_lm_b200.architectures.ridopel import run_order
    from burn_lm_b200.model import plan_of, tensor_specs_of
    arch, typed, plan = plan_of(RID_A)
    assert arch.name == "Ridopel" and plan.head.tensors["weight"] == "head" and plan.embedding.tensors == {"table": "embed", "norm": "embed.norm"}
    names = {s.name: tuple(s.shape) for s in tensor_specs_of(RID_A)}
    assert names["embed"] == (352, 96) and names["head"] == (352, 96) and names["loop.in"] == (96, 192) and names["final.norm"] == (96,)
    assert names["l0.canon1"] == (96, 4) and names["l0.mix.f.b"] == (48,) and names["l0.mix.lower"] == (48,) and names["l0.mix.norm"] == (32,)
    assert names["l1.mix.q"] == (4 * 40, 96) and names["l1.mix.dkv"] == (56, 96) and names["l1.mix.dkv.norm"] == (40,)
    assert names["l1.mix.uk"] == (96, 40) and names["l1.mix.uv"] == (80, 40) and names["l1.mix.g"] == (80, 96) and names["l1.mix.o"] == (96, 80)
    assert names["l2.mix.mu.w"] == (96,) and names["l2.mix.w1"] == (-1, 96) and names["l2.mix.w2"] == (96, -1) and names["l2.mix.u"] == (3, 32)
    assert names["l1.mlp.router"] == (6, 96) and names["l1.mlp.correction"] == (6,) and names["l1.mlp.e5.down"] == (96, 32)
    assert "l2.norm2" not in names and "l2.mlp.router" not in names and "l5.mlp.e3.gate" in names and "l5.mlp.e4.gate" not in names
    # the runs: the looped span twice in a row, the stream rewritten in front of each pass, every run with a cache line of its own
    assert [(e.layer, e.before, e.cache_of) for e in plan.schedule] == [(0, None, None), (1, 0, None), (2, None, None), (1, 0, None),
                                                                        (2, None, None), (3, None, None), (4, None, None), (5, None, None)]
    assert run_order(3, None) == [(0, False), (1, False), (2, False)]
    assert [i for i, _ in run_order(4, typed.loop.__class__(0, 4, 2))] == [0, 1, 2, 3, 0, 1, 2, 3]
    assert [i for i, _ in run_order(4, typed.loop.__class__(3, 4, 3))] == [0, 1, 2, 3, 3, 3]
    assert P.run_order(RID_A) == run_order(6, typed.loop) and P.run_order(RID_C) == [(i, i == 0) for _ in range(3) for i in range(3)]
    # without a loop the stream is never rewritten and the stored matrix for it is not wanted
    _, _, flat = plan_of(CONFIGS["rid_d"])
    assert flat.stream_parts == () and "loop.in" not in {s.name for s in tensor_specs_of(CONFIGS["rid_d"])}


def test_a_run_that_keeps_rows_of_a_latent_and_a_state():
    import torch
    from burn_lm_b200.cache import Cache
    from burn_lm_b200.parts.base import CacheNeed
    from burn_lm_b200.plan import ScheduleEntry
    rows = CacheNeed("rows", n_kv_heads=1, head_dim=20)
    carried = CacheNeed("state", state_shape=(2, 12))
    scan = CacheNeed("state", state_shape=(2, 12 + 64))
    cache = Cache([(rows, carried), scan, (rows, carried)], [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2)], 256, 3, 256,
                  torch.float32, "cpu")
    v0, v1, v2 = cache.view(0), cache.view(1), cache.view(2)
    assert v0.kind == "rows+state" and tuple(v0.pool.shape[1:]) == (64, 20) and tuple(v0.state.shape) == (3, 2, 12) and v1.kind == "state"
    assert v0.block_table is v2.block_table and v0.pool.data_ptr() != v2.pool.data_ptr() and v0.state.data_ptr() != v2.state.data_ptr()
    slot = cache.acquire()
    v0.state[slot] += 1.0
    v1.state[slot] += 1.0
    cache.reserve([(slot, 70)])
    cache.release(slot)
    assert cache.acquire() == slot and float(v0.state[slot].abs().sum()) == 0.0 and float(v1.state[slot].abs().sum()) == 0.0


def test_the_filtered_block_puts_the_filters_inputs_in_front_of_the_mixers_state():
    from burn_lm_b200.model import Model, plan_of
    from burn_lm_b200.parts.base import Runtime
    import torch
    _, _, plan = plan_of(RID_A)
    model = Model(plan, Runtime(torch.float32, "cpu"), RID_A)
    carried = 3 * 96
    needs = [layer.block.cache_need() for layer in model.layers]
    assert needs[0].kind == "state" and needs[0].state_shape == (2, carried + 3 * 16 * 32)                   # hgrn2: 3 heads of 16 x 32
    assert [n.kind for n in needs[1]] == ["rows", "state"] and needs[1][0].head_dim == 56 and needs[1][1].state_shape == (2, carried)
    assert needs[2].state_shape == (2, carried + 96 + 3 * 32 * 32)                                           # wkv: the last input, 3 heads of 32 x 32


def test_folders_hold_what_the_plain_implementation_reads(tmp_path):
    folder = make_folder(tmp_path, "rid_c")
    cfg, tensors = P.read_model_folder(folder)
    logits, after = P.forward(cfg, tensors, random_tokens(0, 12, cfg["vocab"]), return_layers=True)
    assert logits.shape == (12, cfg["vocab"]) and len(after) == 9 and np.isfinite(logits).all() and np.abs(logits).max() < 12.0
    # causal: a later token changes nothing before it
    again = P.forward(cfg, tensors, random_tokens(0, 12, cfg["vocab"])[:7] + [3, 1, 4, 1, 5])
    assert np.abs(again[:7] - logits[:7]).max() < 1e-12 and np.abs(again[7:] - logits[7:]).max() > 1e-3
    # the package's random-weights mode writes the same names and shapes
    from burn_lm_b200 import write_random_model
    other = write_random_model(str(tmp_path / "r"), cfg, seed=1, dtype="float32")
    _, drawn = P.read_model_folder(other)
    assert set(drawn) == set(tensors) and all(drawn[k].shape == tensors[k].shape or k.endswith(("w1", "w2")) for k in tensors)
    assert np.isfinite(P.forward(cfg, drawn, [1, 2, 3])).all()


# the plain implementation's mechanisms against closed forms --------------------------------------------------
def test_plain_input_convolution():
    rng = np.random.default_rng(0)
    x, w = rng.normal(size=(9, 2)), rng.normal(size=(2, 4))
    y = P.input_convolution(x, w)
    for c in range(2):
        assert np.allclose(y[:, c], x[:, c] + np.convolve(x[:, c], w[c, ::-1])[:9])
    assert np.allclose(P.input_convolution(x, w[:, 3:]), x * (1 + w[:, 3]))           # one tap: the current token's
    assert np.allclose(P.input_convolution(x, np.array([[1.0, 0.0], [1.0, 0.0]]))[1:], x[1:] + x[:-1])     # the first tap is the oldest


def test_plain_norm_has_the_epsilon_inside_the_root():
    assert np.allclose(P.rms(np.full((1, 4), 1e-3), 1e-2), 1e-3 / np.sqrt(1e-6 + 1e-2))
    assert np.allclose(P.rms_norm(np.array([[3.0, -4.0]]), np.array([2.0, 0.5]), 0.0), [[3.0 / np.sqrt(12.5) * 2, -4.0 / np.sqrt(12.5) * 0.5]])


def test_plain_scans_against_sums_written_out():
    rng = np.random.default_rng(2)
    T, dk, dv = 6, 3, 2
    r, k, v, w, u = rng.normal(size=(T, dk)), rng.normal(size=(T, dk)), rng.normal(size=(T, dv)), rng.uniform(0.2, 1, size=(T, dk)), rng.normal(size=dk)
    o = P.wkv_scan(r, k, v, w, u)
    for t in range(T):        # o_t = sum_(s<t) (r_t . (w_(s+1) ... w_(t-1) k_s)) v_s + (r_t . (u k_t)) v_t
        want = (r[t] * u * k[t]).sum() * v[t] + sum((r[t] * np.prod(w[s + 1: t], axis=0) * k[s]).sum() * v[s] for s in range(t))
        assert np.allclose(o[t], want)
    q, f = rng.normal(size=(T, dk)), rng.uniform(0.1, 0.9, size=(T, dk))
    o = P.hgrn2_scan(q, f, v)
    for t in range(T):        # o_t = sum_(s<=t) (q_t . (f_(s+1) ... f_t (1 - f_s))) v_s: the current token is in it
        assert np.allclose(o[t], sum((q[t] * np.prod(f[s + 1: t + 1], axis=0) * (1 - f[s])).sum() * v[s] for s in range(t + 1)))
    # a gate that is shut (f = 1) writes nothing and keeps everything; one that is open (f = 0) keeps the last value only
    assert np.allclose(P.hgrn2_scan(np.ones((3, 2)), np.array([[0.0, 0.0], [1.0, 1.0], [1.0, 1.0]]), v[:3]), 2 * v[0])
    assert np.allclose(P.hgrn2_scan(np.ones((3, 2)), np.zeros((3, 2)), v[:3]), 2 * v[:3])


def test_plain_rotation_depends_on_the_distance_only():
    rng = np.random.default_rng(1)
    q, k = rng.normal(size=(1, 1, 12)), rng.normal(size=(1, 1, 12))
    dots = [float((P.rotate_pairs(q, [i], 8, 100.0) * P.rotate_pairs(k, [j], 8, 100.0)).sum()) for i, j in ((5, 2), (13, 10), (103, 100))]
    assert np.allclose(dots, dots[0])
    assert np.array_equal(P.rotate_pairs(q, [9], 8, 100.0)[..., 8:], q[..., 8:]) and np.array_equal(P.rotate_pairs(q, [0], 8, 100.0), q)


def test_plain_latent_attention_is_attention_over_up_projected_keys():
    """Written out per head with keys [W_uk c | shared rotated part] and values W_uv c."""
    rng = np.random.default_rng(3)
    T, D, H, dk, dr, dv, R, eps = 7, 10, 2, 4, 2, 3, 5, 1e-5
    h = rng.normal(size=(T, D))
    w = {"q": rng.normal(size=(H * (dk + dr), D)), "dkv": rng.normal(size=(R + dr, D)), "dkv.norm": rng.normal(size=R), "uk": rng.normal(size=(H * dk, R)),
         "uv": rng.normal(size=(H * dv, R)), "g": rng.normal(size=(H * dv, D)), "o": np.eye(H * dv)}
    m = {"heads": H, "dim": dk, "rot_dim": dr, "vdim": dv, "kv_rank": R, "scale": 0.4, "rot": {"dims": 2, "base": 10.0}}
    got = P.latent_attention(h, w, m, eps)
    down = h @ w["dkv"].T
    c = down[:, :R] / np.sqrt((down[:, :R] ** 2).mean(-1, keepdims=True) + eps) * w["dkv.norm"]
    turn = lambda x, p: np.array([x[0] * np.cos(p) - x[1] * np.sin(p), x[1] * np.cos(p) + x[0] * np.sin(p)])
    for t in range(T):
        for i in range(H):
            q = (w["q"] @ h[t])[i * (dk + dr): (i + 1) * (dk + dr)]
            scores = [0.4 * (q[:dk] @ (w["uk"][i * dk: (i + 1) * dk] @ c[s]) + turn(q[dk:], t) @ turn(down[s, R:], s)) for s in range(t + 1)]
            p = np.exp(scores) / np.sum(np.exp(scores))
            o = sum(p[s] * (w["uv"][i * dv: (i + 1) * dv] @ c[s]) for s in range(t + 1))
            assert np.allclose(got[t, i * dv: (i + 1) * dv], o * P.sigmoid(w["g"] @ h[t])[i * dv: (i + 1) * dv])


def test_plain_routing():
    s = np.log(np.array([[0.1, 0.2, 0.3, 0.4]]))                       # softmax gives these back
    ids, w = P.route(np.eye(1), s.T, np.array([0.5, 0.0, 0.0, 0.0]), 2)
    assert ids.tolist() == [[0, 3]] and np.allclose(w, [[0.2, 0.8]])   # chosen with the correction, weighed without it
    ids, w = P.route(np.eye(1), s.T, np.zeros(4), 4)
    assert ids.tolist() == [[3, 2, 1, 0]] and np.allclose(w.sum(), 1.0)
