"""The Marinex decoder in the engine against the plain implementation (tests/plain/marinex_plain.py): every
mechanism alone (its part and kernels on a cache of the test's own), then whole models through the step function, the
cache, the scheduler and generation."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import marinex_plain as P
from marinex_tiny import CONFIGS, attention, experts, latent, make_folder, model, random_tokens, row_error

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 6e-2
PAGE = 64
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(x, dtype=torch.float32):
    return torch.tensor(np.asarray(x), dtype=dtype, device="cuda")


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device="cuda")


def bf(x):
    """What a bfloat16 tensor holds of x, in float64: weights and inputs that both dtypes read alike."""
    return torch.tensor(np.asarray(x), dtype=torch.float32).to(torch.bfloat16).to(torch.float64).numpy()


class Scratch:
    def scratch(self, name, n):
        return torch.empty(max(n, 1), dtype=torch.float32, device="cuda")


def step_of(portions, slots, starts):
    """A step that brings portions[s] tokens of the sequence in slots[s], which has starts[s] tokens already."""
    seq_of, pos, cu = [], [], [0]
    for s, (k, st) in enumerate(zip(portions, starts)):
        seq_of += [s] * k
        pos += list(range(st, st + k))
        cu.append(cu[-1] + k)
    return SimpleNamespace(token_seq=ints(seq_of), token_pos=ints(pos), slot_of_seq=ints(slots), cu_seqlens=ints(cu),
                           start_pos=ints(starts), n_tokens=len(seq_of), n_seqs=len(slots), max_q_len=max(portions),
                           max_kv_len=max(s + k for s, k in zip(starts, portions)), workspace=Scratch(), memo={}, host={}, handoff=None)


def engine_for(folder, dtype, max_tokens=4096, **kw):
    from burn_lm_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def rows_ok(err, dtype, tol):
    """float32: nineteen rows in twenty within tol and none beyond 10 tol.  bfloat16: rounding may decide a close call
    between two experts, which moves a row and what follows it by far more than rounding itself; so half of the rows
    within tol / 2 and nine in ten within tol."""
    err = np.atleast_1d(np.asarray(err))
    if dtype == "float32":
        ok = np.quantile(err, 0.95) < tol and err.max() < 10 * tol
    else:
        ok = np.median(err) < tol / 2 and np.quantile(err, 0.9) < tol
    if not ok:
        print(f"{dtype}: median {np.median(err):.3g}, nine in ten {np.quantile(err, 0.9):.3g}, largest {err.max():.3g} of {len(err)} rows")
    return ok


def folder_for(tmp_path, name, dtype, **kw):
    """Lively weights for the sharp comparison in float32, calm ones for bfloat16 (see rows_ok)."""
    return make_folder(tmp_path, name, lively=dtype == "float32", **kw)


# ---------------------------------------------------------------------------------------------------------
# a mixer alone: the part with weights of the test's own, on a paged cache of the test's own
# ---------------------------------------------------------------------------------------------------------
def build_mixer(entry, width, weights, dtype, eps=1e-5):
    """The mixer part the architecture plans for one layer entry, bound to `weights` (stored name -> array)."""
    from burn_lm_b200.model import plan_of
    from burn_lm_b200.parts.base import Runtime
    from burn_lm_b200.registry import part_class
    _, _, plan = plan_of(model(16, width, [entry], eps=eps))
    pp = plan.layers[0].part("mixer")
    part = part_class("mixer", pp.kind)(pp.spec, pp.tensors, Runtime(DTYPES[dtype], torch.device("cuda")))
    part.bind({name: dev(weights[name], DTYPES[dtype]) for name in (s.name for s in part.tensor_specs())})
    return part


def mixer_weights(entry, width, rng, gain=1.5):
    from burn_lm_b200.model import plan_of
    from burn_lm_b200.parts.base import Runtime
    from burn_lm_b200.registry import part_class
    _, _, plan = plan_of(model(16, width, [entry]))
    pp = plan.layers[0].part("mixer")
    part = part_class("mixer", pp.kind)(pp.spec, pp.tensors, Runtime(torch.float32, torch.device("cpu")))
    w = {}
    for s in part.tensor_specs():
        last = s.name.split(".")[-1]
        if last == "norm":
            w[s.name] = bf(1.0 + 0.3 * rng.normal(size=s.shape))
        elif last == "temp":
            w[s.name] = bf(rng.uniform(0.4, 2.0, size=s.shape))
        elif last == "sink":
            w[s.name] = bf(1.5 * rng.normal(size=s.shape))
        else:
            w[s.name] = bf((gain if last != "o" else 1.0) * rng.normal(size=s.shape) / np.sqrt(s.shape[-1]))
    return w


class OwnCache:
    """Pages of one run, handed out in a shuffled order; rubbish (NaN) wherever nothing was written."""

    def __init__(self, part, dtype, n_slots=4, pages_each=24, seed=0):
        need = part.cache_need()
        n_pages = n_slots * pages_each + 3
        shape = (n_pages, PAGE, need.head_dim) if need.kind == "rows" else (n_pages, need.n_kv_heads * PAGE * (need.head_dim + (need.value_dim or need.head_dim)))
        self.pool = torch.full(shape, float("nan"), dtype=DTYPES[dtype], device="cuda")
        order = np.random.default_rng(seed).permutation(n_pages)[:n_slots * pages_each]
        self.block_table = ints(order).view(n_slots, pages_each).contiguous()
        self.writes = True


def run_mixer(part, cache, hs, slots, schedule, dtype):
    """Feeds sequences hs[s] ([T_s, D] arrays) side by side, schedule = list of per-sequence portions; returns every
    sequence's output rows [T_s, D]."""
    at, outs = [0] * len(hs), [[] for _ in hs]
    for portion in schedule:
        live = [s for s, k in enumerate(portion) if k > 0]
        st = step_of([portion[s] for s in live], [slots[s] for s in live], [at[s] for s in live])
        x = dev(np.concatenate([hs[s][at[s]:at[s] + portion[s]] for s in live]), DTYPES[dtype])
        y = part.forward(x, st, cache).float().cpu().numpy()
        row = 0
        for s in live:
            outs[s].append(y[row:row + portion[s]])
            row += portion[s]
            at[s] += portion[s]
    assert at == [len(h) for h in hs]
    return [np.concatenate(o) for o in outs]


SCHEDULES = {
    "whole": lambda a, b: [(a, b)],
    "portions": lambda a, b: [(1, 1), (2, 1), (1, 2), (61, 3), (2, 0), (a - 100, b - 7), (33, 0)],
    "twos": lambda a, b: [(a - 40, b)] + [(2, 0)] * 20,
    "single tokens": lambda a, b: [(a - 30, b - 3)] + [(1, 1)] * 3 + [(1, 0)] * 27,
}

ATTENTION_SHAPES = {      # heads, kv heads, dim, vdim, turning lanes
    "small heads": (4, 2, 24, 16, 12),
    "one head": (1, 1, 32, 32, 32),
    "no multiples of eight": (5, 1, 12, 20, 6),
    "heads of 128": (4, 1, 128, 128, 64),
    "sixteen heads a group, values of 160": (16, 1, 64, 160, 0),
    "seventeen heads a group": (17, 1, 16, 16, 8),
}


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2.5e-2)])
@pytest.mark.parametrize("shape", sorted(ATTENTION_SHAPES))
@pytest.mark.parametrize("schedule", sorted(SCHEDULES))
def test_attention_alone(shape, schedule, dtype, tol):
    H, G, dk, dv, rot = ATTENTION_SHAPES[shape]
    rng = np.random.default_rng(H + dk)
    width = 48
    entry = attention(H, G, dk, dv, None, rot_dims=rot, base=300.0, scale=1.7 / np.sqrt(dk), softcap=6.0)
    w = mixer_weights(entry, width, rng)
    hs = [bf(rng.normal(size=(n, width))) for n in (200, 9)]
    want = [P.attention(h, {"m." + k.split("mix.")[1]: v for k, v in w.items()}, entry["mixer"], 1e-5, "m.") for h in hs]
    part = build_mixer(entry, width, w, dtype)
    got = run_mixer(part, OwnCache(part, dtype), hs, [2, 0], SCHEDULES[schedule](200, 9), dtype)
    for g, wnt in zip(got, want):
        assert np.abs(g - wnt).max() < tol * np.abs(wnt).max()


LATENT_SHAPES = {         # heads, dim, rot_dim, vdim, q_rank, kv_rank, window, turning lanes
    "small": (4, 16, 16, 24, 48, 32, 20, 16),
    "one head, a window of one": (1, 32, 32, 32, 32, 32, 1, 32),
    "no multiples of eight": (3, 12, 6, 20, 20, 36, 33, 4),
    "keys wider than 128": (4, 128, 64, 128, 96, 256, 150, 64),
    "a window beyond the sequence": (2, 64, 32, 64, 64, 128, 1000, 32),
    "no turning lane, a window of a page": (2, 16, 16, 16, 16, 48, 64, 0),
}


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2.5e-2)])
@pytest.mark.parametrize("shape", sorted(LATENT_SHAPES))
@pytest.mark.parametrize("schedule", sorted(SCHEDULES))
def test_latent_attention_alone(shape, schedule, dtype, tol):
    H, dk, dr, dv, Q, R, window, rot = LATENT_SHAPES[shape]
    rng = np.random.default_rng(H + dk + window)
    width = 48
    entry = latent(H, dk, dr, dv, Q, R, window, None, rot_dims=rot, base=300.0, scale=1.7 / np.sqrt(dk + dr))
    w = mixer_weights(entry, width, rng)
    hs = [bf(rng.normal(size=(n, width))) for n in (200, 9)]
    want = [P.latent_attention(h, {"m." + k.split("mix.")[1]: v for k, v in w.items()}, entry["mixer"], 1e-5, "m.") for h in hs]
    part = build_mixer(entry, width, w, dtype)
    got = run_mixer(part, OwnCache(part, dtype), hs, [1, 3], SCHEDULES[schedule](200, 9), dtype)
    for g, wnt in zip(got, want):
        assert np.abs(g - wnt).max() < tol * np.abs(wnt).max()


def test_latent_attention_written_out_and_on_the_latent_agree():
    """Long bfloat16 portions write out every head's keys and values; short ones work on the latent itself."""
    from burn_lm_b200.parts import latent_attention as L
    rng = np.random.default_rng(9)
    entry = latent(4, 32, 16, 40, 64, 64, 90, None, base=300.0)
    w = mixer_weights(entry, 64, rng)
    hs = [bf(rng.normal(size=(170, 64)))]
    part = build_mixer(entry, 64, w, "bfloat16")
    assert part.expands
    a = run_mixer(part, OwnCache(part, "bfloat16"), hs, [1], [(170,)], "bfloat16")[0]
    kept, L.EXPAND_TOKENS = L.EXPAND_TOKENS, 10 ** 9
    try:
        b = run_mixer(part, OwnCache(part, "bfloat16"), hs, [1], [(170,)], "bfloat16")[0]
    finally:
        L.EXPAND_TOKENS = kept
    want = P.latent_attention(hs[0], {"m." + k.split("mix.")[1]: v for k, v in w.items()}, entry["mixer"], 1e-5, "m.")
    assert np.abs(a - b).max() < 2.5e-2 * np.abs(want).max() and np.abs(a - want).max() < 2.5e-2 * np.abs(want).max()


# one key made to stand out among hundreds ----------------------------------------------------------------
def planted_attention(n, j, dk=32, dv=24):
    """One head; the query reads the first half of the input's lanes and the key the second half, so that the last token's
    query points along the key of token j and along no other token's (its own too); the values are a random map."""
    rng = np.random.default_rng(n + j)
    width = 2 * dk
    entry = attention(1, 1, dk, dv, None, rot_dims=0, scale=1.0, softcap=200.0)
    zero, eye = np.zeros((dk, dk)), np.eye(dk)
    w = {"l0.mix.q": np.hstack([eye, zero]), "l0.mix.k": np.hstack([zero, eye]), "l0.mix.v": bf(rng.normal(size=(dv, width))),
         "l0.mix.o": np.eye(dv), "l0.mix.q.norm": np.ones(dk), "l0.mix.k.norm": np.ones(dk), "l0.mix.temp": np.ones(1)}
    h = bf(rng.normal(size=(n, width)))
    u = bf(rng.normal(size=dk))
    h[n - 1, :dk] = u
    h[j, dk:] = u
    return entry, width, w, h


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("n,j", [(300, 0), (300, 1), (300, 63), (300, 64), (300, 127), (300, 298), (65, 0), (129, 64), (2, 0)])
def test_a_key_far_back_at_page_borders_and_among_the_first_tokens(n, j, decoded, dtype, tol):
    entry, width, w, h = planted_attention(n, j)
    want = P.attention(h, {"m." + k.split("mix.")[1]: v for k, v in w.items()}, entry["mixer"], 1e-5, "m.")
    v_j = P.rms(w["l0.mix.v"] @ h[j], 1e-5)
    assert np.abs(want[-1] - v_j).max() < 1e-3            # the test is sharp: the last token reads token j's value and nothing else
    part = build_mixer(entry, width, w, dtype)
    schedule = [(n - 1,), (1,)] if decoded else [(n,)]
    got = run_mixer(part, OwnCache(part, dtype, seed=j), [h], [3], schedule, dtype)[0]
    assert np.abs(got[-1] - want[-1]).max() < tol and np.abs(got - want).max() < tol * 3


def planted_latent(n, j, window, dr=16, R=32, dv=24):
    """One head whose turned key part does not turn (no turning lane): token j's shared key part is made a large multiple
    of the last token's query part, whatever the other weights are."""
    rng = np.random.default_rng(n + j)
    width = 48
    entry = latent(1, 16, dr, dv, 24, R, window, None, rot_dims=0, scale=0.2)
    w = mixer_weights(entry, width, rng, gain=1.0)
    w["l0.mix.o"] = np.eye(dv)
    w["l0.mix.sink"] = np.zeros(1)
    h = bf(rng.normal(size=(n, width)))
    cq = P.rms_norm(h[-1] @ w["l0.mix.dq"].T, w["l0.mix.dq.norm"], 1e-5)
    q_turn = (cq @ w["l0.mix.uq"].T)[16:]
    h[j] = bf(np.linalg.lstsq(w["l0.mix.dkv"][R:], 400.0 * q_turn / (q_turn @ q_turn), rcond=None)[0])     # its score: 0.2 * 400 + small
    return entry, width, w, h


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("n,window,back", [(300, 75, 74), (300, 75, 75), (300, 64, 63), (300, 64, 64), (300, 65, 64), (300, 65, 65),
                                           (300, 1, 0), (300, 2, 1), (300, 2, 2), (70, 200, 69), (130, 129, 128), (130, 128, 128)])
def test_a_key_just_inside_and_just_outside_the_window(n, window, back, decoded, dtype, tol):
    j = n - 1 - back
    entry, width, w, h = planted_latent(n, j, window)
    wp = {"m." + k.split("mix.")[1]: v for k, v in w.items()}
    want = P.latent_attention(h, wp, entry["mixer"], 1e-5, "m.")
    inside = back < window
    c = P.rms_norm((h[j] @ w["l0.mix.dkv"].T)[:32], w["l0.mix.dkv.norm"], 1e-5)
    v_j = (c @ w["l0.mix.uv"].T) * P.sigmoid(h[-1] @ w["l0.mix.g"].T)
    if back > 0:          # (the last token itself is not made to stand out)
        assert (np.abs(want[-1] - v_j).max() < 1e-3) == inside          # the test is sharp: all or nothing of token j's value
    part = build_mixer(entry, width, w, dtype)
    schedule = [(n - 1,), (1,)] if decoded else [(n,)]
    got = run_mixer(part, OwnCache(part, dtype, seed=j), [h], [2], schedule, dtype)[0]
    assert np.abs(got[-1] - want[-1]).max() < tol * max(1.0, np.abs(want[-1]).max())


def test_a_head_whose_number_is_negative_and_scores_beyond_the_cap():
    """A negative number per head turns the order of the scores round (the largest raw score is the smallest score);
    a small cap flattens the scores that lie beyond it."""
    rng = np.random.default_rng(11)
    entry = attention(4, 2, 32, 32, None, rot_dims=16, scale=2.0, softcap=1.5)
    w = mixer_weights(entry, 64, rng, gain=3.0)
    w["l0.mix.temp"] = np.array([-1.5, 0.25, 3.0, -0.125])
    h = bf(rng.normal(size=(150, 64)))
    wp = {"m." + k.split("mix.")[1]: v for k, v in w.items()}
    want = P.attention(h, wp, entry["mixer"], 1e-5, "m.")
    free = P.attention(h, wp, dict(entry["mixer"], softcap=1e6), 1e-5, "m.")
    assert np.abs(free - want).max() > 0.1 * np.abs(want).max()
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 2.5e-2)):
        part = build_mixer(entry, 64, w, dtype)
        for schedule in ([(150,)], [(140,)] + [(1,)] * 10, [(3,), (147,)]):
            got = run_mixer(part, OwnCache(part, dtype), [h], [1], schedule, dtype)[0]
            assert np.abs(got - want).max() < tol * np.abs(want).max(), (dtype, schedule)


# the stream, the norm behind a sublayer --------------------------------------------------------------------
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_the_norm_behind_a_sublayer_joins_the_stream_which_is_handed_on_as_it_is(out_dtype):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(2)
    n, d, eps = 37, 72, 1e-6
    x, a, g = rng.normal(size=(n, d)), 5.0 * rng.normal(size=(n, d)), 1.0 + 0.3 * rng.normal(size=d)
    for delta_dtype in (torch.float32, torch.bfloat16):
        resid, delta = dev(x), dev(a, delta_dtype)
        out = torch.empty((n, d), dtype=out_dtype, device="cuda")
        K.sandwich_norm(resid, delta, dev(g), 1.0, eps, None, 0.0, out)
        want = x.astype(np.float32).astype(np.float64) + P.rms_norm(delta.double().cpu().numpy(), g.astype(np.float32).astype(np.float64), eps)
        assert np.abs(resid.cpu().numpy() - want).max() < 1e-5
        assert torch.equal(out, resid.to(out_dtype))


# the experts ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n_experts,top,groups,keep", [(12, 3, 3, 2), (8, 2, 4, 2), (6, 3, 2, 1), (5, 2, 5, 3), (4, 4, 1, 1), (16, 4, 8, 2), (1, 1, 1, 1), (6, 2, 3, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routing_by_groups_and_experts_without_a_gate(n_experts, top, groups, keep, dtype):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(n_experts + top)
    n, width, ff = 45, 40, 24
    f = experts(n_experts, top, ff, groups, keep)
    hp = bf(rng.normal(size=(n, width)))
    w = {"m.router": bf(3.0 * rng.normal(size=(n_experts, width)) / np.sqrt(width)), "m.correction": bf(0.3 * rng.normal(size=n_experts) - 0.4)}
    for e in range(n_experts):
        w[f"m.e{e}.up"], w[f"m.e{e}.down"] = bf(2.0 * rng.normal(size=(ff, width)) / np.sqrt(width)), bf(rng.normal(size=(width, ff)) / np.sqrt(ff))
    want_ids, want_w = P.route(hp, w, f, "m.")
    ids, weights = K.moe_route(dev(hp, dtype), dev(w["m.router"]), top, correction=dev(w["m.correction"]), n_groups=groups, keep_groups=keep)
    assert np.array_equal(ids.cpu().numpy(), want_ids) and np.allclose(weights.cpu().numpy(), want_w, atol=1e-6)
    if keep < groups and n_experts // groups > 1:      # (with one expert a group the best experts lie in the best groups)
        free, _ = P.route(hp, w, experts(n_experts, top, ff, 1, 1), "m.")
        assert not np.array_equal(free, want_ids)                     # the groups matter
    up = dev(np.stack([w[f"m.e{e}.up"] for e in range(n_experts)]), dtype)
    down = dev(np.stack([w[f"m.e{e}.down"] for e in range(n_experts)]), dtype)
    got = K.moe_experts(dev(hp, dtype), ids, weights, up, down, weight_on_input=False, out_dtype=torch.float32, unit=K.UNIT_GELU)
    want = P.experts(hp, w, f, "m.")
    assert np.abs(got.cpu().numpy() - want).max() < (2e-5 if dtype == torch.float32 else 3e-2) * np.abs(want).max()
    tanh_form = K.moe_experts(dev(hp, dtype), ids, weights, up, down, weight_on_input=False, out_dtype=torch.float32, unit=K.UNIT_GELU_TANH)
    if dtype == torch.float32:       # the other form of the activation is close, and not the same
        assert 1e-6 < np.abs(tanh_form.cpu().numpy() - want).max() / np.abs(want).max() < 5e-3


def test_experts_of_odd_sizes_and_of_large_ones():
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(5)
    for width, ff, dtype in ((36, 20, torch.bfloat16), (128, 256, torch.bfloat16), (128, 256, torch.float32)):
        f = experts(6, 2, ff, 3, 2)
        hp = bf(rng.normal(size=(150, width)))
        w = {"m.router": bf(rng.normal(size=(6, width))), "m.correction": 2.0 * rng.permutation(6).astype(np.float64)}
        for e in range(6):
            w[f"m.e{e}.up"], w[f"m.e{e}.down"] = bf(2.0 * rng.normal(size=(ff, width)) / np.sqrt(width)), bf(rng.normal(size=(width, ff)) / np.sqrt(ff))
        ids, weights = K.moe_route(dev(hp, dtype), dev(w["m.router"]), 2, correction=dev(w["m.correction"]), n_groups=3, keep_groups=2)
        up = dev(np.stack([w[f"m.e{e}.up"] for e in range(6)]), dtype)
        down = dev(np.stack([w[f"m.e{e}.down"] for e in range(6)]), dtype)
        got = K.moe_experts(dev(hp, dtype), ids, weights, up, down, weight_on_input=False, out_dtype=torch.float32, unit=K.UNIT_GELU)
        want = P.experts(hp, w, f, "m.")
        assert np.abs(got.cpu().numpy() - want).max() < (2e-5 if dtype == torch.float32 else 3e-2) * np.abs(want).max()


@pytest.mark.parametrize("n,width,ff,n_experts,top", [(700, 136, 72, 4, 2), (1100, 64, 264, 3, 1), (520, 128, 128, 2, 2)])
def test_experts_with_many_tokens_an_expert(n, width, ff, n_experts, top):
    """Prompts run other kernels than single tokens do (larger tiles); with and without a gate, against the plain
    implementation and against the 32-bit kernels."""
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(n)
    f = experts(n_experts, top, ff, 1, 1)
    hp = bf(rng.normal(size=(n, width)))
    w = {"m.router": bf(2.0 * rng.normal(size=(n_experts, width)) / np.sqrt(width)), "m.correction": np.zeros(n_experts)}
    for e in range(n_experts):
        w[f"m.e{e}.up"], w[f"m.e{e}.down"] = bf(2.0 * rng.normal(size=(ff, width)) / np.sqrt(width)), bf(rng.normal(size=(width, ff)) / np.sqrt(ff))
    gate = bf(2.0 * rng.normal(size=(n_experts, ff, width)) / np.sqrt(width))
    want = P.experts(hp, w, f, "m.")
    outs = {}
    for dtype in (torch.float32, torch.bfloat16):
        ids, weights = K.moe_route(dev(hp, dtype), dev(w["m.router"]), top)
        up = dev(np.stack([w[f"m.e{e}.up"] for e in range(n_experts)]), dtype)
        down = dev(np.stack([w[f"m.e{e}.down"] for e in range(n_experts)]), dtype)
        got = K.moe_experts(dev(hp, dtype), ids, weights, up, down, weight_on_input=False, out_dtype=torch.float32, unit=K.UNIT_GELU)
        assert np.abs(got.cpu().numpy() - want).max() < (2e-5 if dtype == torch.float32 else 3e-2) * np.abs(want).max()
        gate_up = torch.cat([dev(gate, dtype), up], dim=1).contiguous()
        for on_input in (False, True):
            outs[dtype, on_input] = K.moe_experts(dev(hp, dtype), ids, weights, gate_up, down, weight_on_input=on_input,
                                                  out_dtype=torch.float32).cpu().numpy()
    for on_input in (False, True):
        exact = outs[torch.float32, on_input]
        assert np.abs(outs[torch.bfloat16, on_input] - exact).max() < 3e-2 * np.abs(exact).max()


def test_a_gate_per_head():
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(6)
    o, g = rng.normal(size=(9, 5 * 12)), rng.normal(size=(9, 7))
    wide = dev(g)
    out = torch.empty((9, 60), device="cuda")
    K.sigmoid_gate(dev(o), wide[:, 1:6], out, share=12)
    want = o.reshape(9, 5, 12) * P.sigmoid(g[:, 1:6])[:, :, None]
    assert np.abs(out.cpu().numpy() - want.reshape(9, 60)).max() < 1e-6


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------
def _logits(engine, tokens, want, portions=None):
    from burn_lm_b200 import StepEntry
    slot = engine.acquire()
    rows, at = [], 0
    for k in portions or [len(tokens)]:
        w = [p - at for p in want if at <= p < at + k]
        out = engine.step([StepEntry(slot, tokens[at: at + k], w)])
        if w:
            rows.append(out.cpu().numpy().copy())
        at += k
    engine.release(slot)
    return np.concatenate(rows)


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype,tol", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompts_portions_and_single_tokens(tmp_path, name, dtype, tol):
    folder = folder_for(tmp_path, name, dtype)
    cfg, tensors = P.read_model_folder(folder)
    tokens = random_tokens(1, 250, cfg["vocab"])
    want = P.forward(cfg, tensors, tokens)
    engine = engine_for(folder, dtype)
    every = list(range(len(tokens)))
    assert rows_ok(row_error(_logits(engine, tokens, every), want), dtype, tol)
    for portions in ([64, 64, 122], [1, 2, 61, 1, 1, 2, 2, 17, 63, 100], [200] + [1] * 50, [2] * 125):
        assert rows_ok(row_error(_logits(engine, tokens, every, portions), want), dtype, tol), portions
    # the first tokens alone, one at a time from an empty sequence
    assert rows_ok(row_error(_logits(engine, tokens[:9], list(range(9)), [1] * 9), want[:9]), dtype, tol)
    engine.verify()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_stream_after_every_layer(tmp_path, name):
    from burn_lm_b200 import StepEntry
    from burn_lm_b200.parts.norm import PostRMSNorm
    folder = make_folder(tmp_path, name)
    cfg, tensors = P.read_model_folder(folder)
    tokens = random_tokens(2, 40, cfg["vocab"])
    after = []
    P.forward(cfg, tensors, tokens, after)
    engine = engine_for(folder, "float32")
    engine.use_graphs = False
    seen, kept = [], []
    for layer in engine.model.layers:
        block = layer.block

        def watched(resid, delta, step, view, next_norm=None, plain=block.forward):
            pending = plain(resid, delta, step, view, next_norm=next_norm)
            whole = resid.clone()
            if pending is not None:                 # what the layer's last sublayer returned is still to join the stream
                PostRMSNorm.add(whole, pending)
            seen.append(whole.cpu().numpy())
            return pending

        kept.append((block, block.forward))
        block.forward = watched
    try:
        slot = engine.acquire()
        engine.step([StepEntry(slot, tokens, [0])])
        engine.release(slot)
    finally:
        for block, plain in kept:
            block.forward = plain
    assert len(seen) == len(after)
    for i, (got, want) in enumerate(zip(seen, after)):
        assert np.abs(got[:len(tokens)] - want).max() < 1e-4 * np.abs(want).max(), i


@pytest.mark.parametrize("name", ["mar_a", "mar_c", "mar_d"])
@pytest.mark.parametrize("dtype,tol", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_unequal_requests_together_through_used_slots_and_pages(tmp_path, name, dtype, tol):
    from burn_lm_b200 import StepEntry
    folder = folder_for(tmp_path, name, dtype)
    cfg, tensors = P.read_model_folder(folder)
    engine = engine_for(folder, dtype, max_tokens=1024)
    errs = []
    for set_no in range(3):              # the same slots and pages serve three sets of requests
        lengths = [[1, 70, 230], [65, 3, 64, 120], [228, 2]][set_no]
        reqs = [random_tokens(10 * set_no + i, n + 12, cfg["vocab"]) for i, n in enumerate(lengths)]
        want = [P.forward(cfg, tensors, r) for r in reqs]
        slots = [engine.acquire() for _ in reqs]
        out = engine.step([StepEntry(s, r[:n], [0, n - 1]) for s, r, n in zip(slots, reqs, lengths)]).cpu().numpy()
        for i, n in enumerate(lengths):
            errs += [row_error(out[2 * i], want[i][0]), row_error(out[2 * i + 1], want[i][n - 1])]
            assert dtype != "float32" or max(errs[-2:]) < tol, (set_no, i)
        live = list(range(len(reqs)))
        for t in range(12):
            if t == 5:                      # the shortest request ends early
                gone = live.pop(int(np.argmin([lengths[i] for i in live])))
                engine.release(slots[gone])
            out = engine.step([StepEntry(slots[i], [reqs[i][lengths[i] + t]], [0]) for i in live]).cpu().numpy().copy()
            for j, i in enumerate(live):
                errs.append(row_error(out[j], want[i][lengths[i] + t]))
                assert dtype != "float32" or errs[-1] < tol, (set_no, i, t)
        for i in live:
            engine.release(slots[i])
    engine.verify()
    assert rows_ok(errs, dtype, tol)


@pytest.mark.parametrize("name", ["mar_a", "mar_c"])
def test_long_decoding_while_the_windows_give_pages_back(tmp_path, name):
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, name)
    cfg, tensors = P.read_model_folder(folder)
    tokens = random_tokens(5, 400, cfg["vocab"])
    want = P.forward(cfg, tensors, tokens)
    engine = engine_for(folder, "float32", max_tokens=640)       # room for the keys of every position and little else
    slot = engine.acquire()
    engine.step([StepEntry(slot, tokens[:30], [])])
    for p in range(30, len(tokens)):
        row = engine.step([StepEntry(slot, [tokens[p]], [0])]).cpu().numpy()[0]
        assert row_error(row, want[p]) < FP32_TOL, p
    engine.release(slot)
    engine.verify()


@pytest.mark.parametrize("name", ["mar_a", "mar_b"])
def test_greedy_generation_through_the_entry_point(tmp_path, name):
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, name)
    cfg, tensors = P.read_model_folder(folder)
    prompts = [random_tokens(20 + i, n, cfg["vocab"]) for i, n in enumerate([5, 70, 17])]
    want = [P.greedy(cfg, tensors, p, 10) for p in prompts]
    lm = blm.load(folder, dtype="float32", max_seq_len=256, max_batch=3)
    assert lm.generate(prompts, sample_len=10, ignore_stop=True).tokens == want
    assert lm.generate(prompts[::-1], sample_len=10, ignore_stop=True).tokens == want[::-1]      # used slots, another order


def test_the_device_side_decode_loop(tmp_path):
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, "mar_a")
    cfg, tensors = P.read_model_folder(folder)
    prompts = [random_tokens(30 + i, n, cfg["vocab"]) for i, n in enumerate([33, 64])]
    want = [P.greedy(cfg, tensors, p, 12) for p in prompts]
    engine = engine_for(folder, "float32", max_tokens=1024)
    slots = [engine.acquire() for _ in prompts]
    first = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).argmax(dim=-1).tolist()
    assert first == [w[0] for w in want]
    more = engine.decode_run(slots, first, 8).cpu().numpy()
    assert more.T.tolist() == [w[1:9] for w in want]
    again = engine.decode_run(slots, [w[8] for w in want], 3)       # the captured graph once more, from where it stopped
    assert again.cpu().numpy().T.tolist() == [w[9:] for w in want]


def test_sampling_with_a_temperature_runs_inside_the_captured_step(tmp_path):
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, "mar_a")
    lm = blm.load(folder, dtype="bfloat16", max_seq_len=256, max_batch=2)
    prompts = [random_tokens(50, 20, 288), random_tokens(51, 66, 288)]
    a = lm.generate(prompts, sample_len=12, temperature=0.8, seed=7, ignore_stop=True).tokens
    b = lm.generate(prompts, sample_len=12, temperature=0.8, seed=7, ignore_stop=True).tokens
    assert a == b and all(len(t) == 12 for t in a)          # the same draws from the same seed, through used slots


def test_the_trace_runner_as_a_child_process(tmp_path):
    cfg = CONFIGS["mar_c"]
    a, b = random_tokens(40, 115, cfg["vocab"]), random_tokens(41, 9, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:110], "want": [0, 109]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[110]], "want": []}, {"id": "b", "tokens": [b[5]], "want": [0]}], "end": []}]
    steps += [{"step": 2 + t, "entries": [{"id": "a", "tokens": [a[111 + t]], "want": [0]}] + ([{"id": "b", "tokens": [b[6 + t]], "want": [0]}] if t < 3 else []),
               "end": ["b"] if t == 2 else []} for t in range(4)]
    out = tmp_path / "out"
    for dtype, tol in (("float32", FP32_TOL), ("bfloat16", BF16_TOL)):
        folder = folder_for(tmp_path, "mar_c", dtype)
        cfg, tensors = P.read_model_folder(folder)
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
                               "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
        wa, wb = P.forward(cfg, tensors, a), P.forward(cfg, tensors, b)
        read = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        want = {0: [wa[0], wa[109], wb[4]], 1: [wb[5]]}
        want.update({2 + t: [wa[111 + t]] + ([wb[6 + t]] if t < 3 else []) for t in range(4)})
        errs = [e for n, w in want.items() for e in row_error(read(n), np.stack(w))]
        assert len(errs) == 11 and rows_ok(errs, dtype, tol), errs


def test_the_command_line_on_the_preset(tmp_path):
    program = [sys.executable, os.path.join(ROOT, "bin", "burn-lm")]
    folder = str(tmp_path / "n")
    r = subprocess.run(program + ["random", folder, "--preset", "marinex_tiny", "--seed", "4", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and f"wrote {folder}" in r.stdout, r.stderr
    cfg, tensors = P.read_model_folder(folder)
    prompt = random_tokens(5, 23, cfg["vocab"])
    want = P.greedy(cfg, tensors, prompt, 12)
    r = subprocess.run(program + ["run", folder, "--dtype", "float32", "--sample-len", "12", "--max-seq-len", "128",
                                  ",".join(map(str, prompt))], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert lines[0].split() == [str(t) for t in want], (lines[0], want)


@pytest.mark.parametrize("kinds", ["attention only", "latent only", "no feed-forward at all", "latent first and last"])
def test_models_of_one_kind_of_layer_and_other_orders(tmp_path, kinds):
    e = experts(6, 2, 32, 3, 2)
    layers = {
        "attention only": [attention(4, 2, 16, 8, e, rot_dims=8), attention(2, 2, 24, 24, None)],
        "latent only": [latent(2, 16, 8, 16, 24, 24, 50, e), latent(3, 8, 8, 16, 16, 16, 7, None, rot_dims=4)],
        "no feed-forward at all": [attention(2, 1, 24, 16, None), latent(2, 8, 16, 8, 32, 32, 65, None), attention(3, 3, 8, 16, None, rot_dims=0)],
        "latent first and last": [latent(2, 16, 8, 16, 24, 24, 64, e), attention(2, 1, 16, 16, e), attention(4, 4, 8, 8, e), latent(1, 16, 16, 48, 8, 8, 128, e)],
    }[kinds]
    cfg = model(97, 48, layers)
    tokens = random_tokens(7, 190, 97)
    for dtype, tol in (("float32", FP32_TOL), ("bfloat16", BF16_TOL)):
        folder = folder_for(tmp_path, "m", dtype, seed=3, config=cfg)
        pcfg, tensors = P.read_model_folder(folder)
        want = P.forward(pcfg, tensors, tokens)
        engine = engine_for(folder, dtype)
        assert rows_ok(row_error(_logits(engine, tokens, list(range(190)), [170] + [1] * 20), want), dtype, tol)
        assert rows_ok(row_error(_logits(engine, tokens, list(range(190)), [3, 64, 2, 121]), want), dtype, tol)
