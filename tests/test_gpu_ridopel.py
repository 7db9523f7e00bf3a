"""The Ridopel decoder in the engine against the plain implementation (tests/plain/ridopel_plain.py): every
mechanism's kernels alone, then whole models through the step function, the cache, the scheduler and generation."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import ridopel_plain as P
from ridopel_tiny import CONFIGS, experts, hgrn2, latent, make_folder, model, random_tokens, row_error, wkv

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 6e-2
PAGE = 64
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def dev(x, dtype=torch.float32):
    return torch.tensor(np.asarray(x), dtype=dtype, device="cuda")


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device="cuda")


def f32(x):
    """What a float32 tensor holds of x, in float64."""
    return np.asarray(x).astype(np.float32).astype(np.float64)


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
                           max_kv_len=max(s + k for s, k in zip(starts, portions)), workspace=Scratch())


def engine_for(folder, dtype, max_tokens=4096, **kw):
    from burn_lm_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def close(got, want, tol):
    want = np.asarray(want)
    return np.abs(np.asarray(got, dtype=np.float64) - want).max() <= tol * max(1.0, np.abs(want).max())


def rows_ok(err, dtype, tol):
    """float32: nineteen rows in twenty within tol and none beyond 10 tol (a loop that runs the same layers four times
    enlarges what rounding leaves in a row or two).  bfloat16: rounding may decide a close call between two experts, which
    moves a row and what follows it by far more than rounding itself; so half of the rows within tol / 2 and nine in ten
    within tol."""
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


PORTIONS = [(1, 1), (2, 1), (1, 2), (33, 3), (2, 1), (31, 1)]      # of two sequences of 70 and 9 tokens


def in_portions(lengths, slots, run):
    """Feeds two sequences side by side in PORTIONS; run(step, rows of sequence s = (s, lo, hi) list) returns the step's
    output rows, which are handed back per sequence in order."""
    at, outs = [0] * len(lengths), [[] for _ in lengths]
    for portion in PORTIONS:
        st = step_of(portion, slots, at)
        spans = [(s, at[s], at[s] + k) for s, k in enumerate(portion)]
        y = run(st, spans, max(portion) == 1)
        row = 0
        for s, k in enumerate(portion):
            outs[s].append(y[row: row + k])
            row += k
            at[s] += k
    assert at == list(lengths)
    return [np.concatenate(o) for o in outs]


# ---------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("taps", [1, 2, 3, 6])
def test_input_convolution_adds_its_input_and_carries_the_last_ones(taps):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(0)
    channels, lengths = 45, [70, 9]
    xs, w = [rng.normal(size=(n, channels)) for n in lengths], rng.normal(size=(channels, taps))
    want = [P.input_convolution(f32(x), f32(w)) for x in xs]
    floats = 5 + max(1, (taps - 1) * channels)
    state = torch.full((4, 2, floats), float("nan"), device="cuda")       # rubbish: a sequence's start must not read it

    def run(st, spans, single):
        x = dev(np.concatenate([xs[s][lo:hi] for s, lo, hi in spans]))
        y = torch.empty_like(x)
        rounded = torch.empty(x.shape, dtype=torch.bfloat16, device="cuda")
        for again in range(2 if single else 1):        # a step of single tokens may run twice
            K.causal_conv(x, 0, channels, dev(w), None, y, 0, st, state, 5, silu=False, out_bf16=rounded, residual=True)
        assert torch.equal(rounded, y.to(torch.bfloat16))
        return y.cpu().numpy()

    got = in_portions(lengths, [3, 1], run)
    for g, wnt in zip(got, want):
        assert close(g, wnt, 1e-5)
    # the slot of the first sequence goes to a new one: nothing of the old is seen
    x2 = rng.normal(size=(6, channels))
    y = torch.empty((6, channels), device="cuda")
    K.causal_conv(dev(x2), 0, channels, dev(w), None, y, 0, step_of((6,), [3], [0]), state, 5, silu=False, residual=True)
    assert close(y.cpu().numpy(), P.input_convolution(f32(x2), f32(w)), 1e-5)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_token_shift_mixes_with_the_token_before(out_dtype):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(1)
    channels, lengths, n_mixes = 52, [70, 9], 5
    xs, mu = [rng.normal(size=(n, channels)) for n in lengths], rng.uniform(size=(n_mixes, channels))
    want = []
    for x in xs:
        prev = np.concatenate([np.zeros((1, channels)), f32(x)[:-1]])
        want.append(np.stack([f32(x) + (prev - f32(x)) * f32(m) for m in mu], axis=1))          # [T, S, C]
    state = torch.full((3, 2, 9 + channels), float("nan"), device="cuda")

    def run(st, spans, single):
        x = dev(np.concatenate([xs[s][lo:hi] for s, lo, hi in spans]))
        out = torch.empty((n_mixes, x.shape[0], channels), dtype=out_dtype, device="cuda")
        for again in range(2 if single else 1):
            K.shift_mix(x, dev(mu), out, st, state, 9)
        return out.float().cpu().numpy().transpose(1, 0, 2)

    for g, wnt in zip(in_portions(lengths, [2, 0], run), want):
        assert close(g, wnt, 1e-6 if out_dtype == torch.float32 else 1e-2)


DECAY_SHAPES = [  # heads, key lanes, value lanes
    (3, 16, 16), (1, 64, 64), (5, 12, 12), (2, 48, 48), (2, 128, 128), (3, 20, 12), (4, 16, 32), (1, 5, 40), (2, 128, 64), (2, 64, 100)]


@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("heads,dk,dv", DECAY_SHAPES)
def test_wkv_scan_in_portions(heads, dk, dv, wide):
    """The bonus counts for the current token only and the state is read before it is written; decays from nearly 1
    to nearly 0 in one head."""
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(2)
    lengths = [70, 9]
    w0, u = rng.uniform(-6.0, 1.0, size=heads * dk), rng.normal(size=(heads, dk))
    seqs, want = [], []
    for n in lengths:
        r, k, v, a = (rng.normal(size=(n, heads, d)) for d in (dk, dk, dv, dk))
        seqs.append((r, k, v, a))
        decay = np.exp(-np.exp(f32(a) + f32(w0).reshape(heads, dk)))
        want.append(np.stack([P.wkv_scan(f32(r)[:, h], f32(k)[:, h], f32(v)[:, h], decay[:, h], f32(u)[h]) for h in range(heads)], axis=1).reshape(n, -1))
    floats = 3 + K.scan_state_floats(heads, dk, dv)
    state = torch.full((3, 2, floats), float("nan"), device="cuda")

    def run(st, spans, single):
        r, k, v, a = (dev(np.concatenate([seqs[s][i][lo:hi].reshape(hi - lo, -1) for s, lo, hi in spans])) for i in range(4))
        wide_in = torch.cat([torch.zeros((r.shape[0], 2), device="cuda"), r, k], dim=1)         # column ranges of a wider tensor
        y = torch.zeros((r.shape[0], heads * dv), device="cuda")
        for again in range(2 if single else 1):
            K.decay_scan(wide_in, 2, wide_in, 2 + heads * dk, v, 0, a, 0, dev(w0), dev(u.reshape(-1)), y, heads, dk, dv, K.DECAY_EXP_EXP, True,
                         st, state, 3, wide_sums=wide)
        return y.cpu().numpy()

    for g, wnt in zip(in_portions(lengths, [2, 0], run), want):
        assert close(g, wnt, 2e-6 if wide else 3e-5)


@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("heads,dk,dv", DECAY_SHAPES)
def test_hgrn2_scan_in_portions(heads, dk, dv, wide):
    """The forget gate never falls below its bound, writes 1 - itself, and the state is read after the write."""
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(3)
    lengths = [70, 9]
    bias, low = rng.normal(size=heads * dk), rng.uniform(0.0, 1.0, size=heads * dk)
    low[:2] = [0.0, 0.999]
    seqs, want = [], []
    for n in lengths:
        q, a, v = rng.normal(size=(n, heads, dk)), 2.0 * rng.normal(size=(n, heads, dk)), rng.normal(size=(n, heads, dv))
        seqs.append((q, a, v))
        lo = f32(low).reshape(heads, dk)
        f = lo + (1.0 - lo) * P.sigmoid(f32(a) + f32(bias).reshape(heads, dk))
        want.append(np.stack([P.hgrn2_scan(P.silu(f32(q)[:, h]), f[:, h], f32(v)[:, h]) for h in range(heads)], axis=1).reshape(n, -1))
    state = torch.full((3, 2, K.scan_state_floats(heads, dk, dv)), float("nan"), device="cuda")

    def run(st, spans, single):
        q, a, v = (dev(np.concatenate([seqs[s][i][lo:hi].reshape(hi - lo, -1) for s, lo, hi in spans])) for i in range(3))
        proj = torch.cat([q, a, v], dim=1)
        y = torch.zeros((q.shape[0], heads * dv), device="cuda")
        for again in range(2 if single else 1):
            K.decay_scan(proj, 0, None, 0, proj, 2 * heads * dk, proj, heads * dk, dev(bias), dev(low), y, heads, dk, dv, K.DECAY_LOWER_BOUND,
                         False, st, state, 0, wide_sums=wide)
        return y.cpu().numpy()

    for g, wnt in zip(in_portions(lengths, [1, 2], run), want):
        assert close(g, wnt, 2e-6 if wide else 3e-5)


def test_a_slow_decay_keeps_a_token_from_hundreds_back():
    """One early token writes a value through a channel whose decay is 0.9999 a token; 600 tokens later, through portions
    and single tokens, a query on that channel alone reads it back, shrunk by the decays between."""
    from burn_lm_b200 import kernels as K
    heads, dk, dv, n = 2, 16, 8, 640
    rng = np.random.default_rng(4)
    r, k, v = np.zeros((n, heads, dk)), np.zeros((n, heads, dk)), rng.normal(size=(n, heads, dv))
    a = np.full((n, heads, dk), 2.0)                                   # exp(-exp(2)): everything else is forgotten at once
    a[:, 1, 5] = np.log(1e-4)
    k[7, 1, 5], r[n - 1, 1, 5] = 1.0, 1.0
    k[300:, 0, :] = 1.0                                                 # noise in the other head
    u = np.zeros(heads * dk)
    state = torch.zeros((1, 2, K.scan_state_floats(heads, dk, dv)), device="cuda")
    at, last = 0, None
    for portion in (250, 1, 1, 2, 300, 64, 21, 1):
        st = step_of((portion,), [0], [at])
        rows = [dev(t[at: at + portion].reshape(portion, -1)) for t in (r, k, v, a)]
        y = torch.zeros((portion, heads * dv), device="cuda")
        K.decay_scan(rows[0], 0, rows[1], 0, rows[2], 0, rows[3], 0, dev(np.zeros(heads * dk)), dev(u), y, heads, dk, dv, K.DECAY_EXP_EXP, True, st, state, 0)
        at, last = at + portion, y[-1].cpu().numpy()
    want = f32(v)[7, 1] * np.exp(-np.float64(np.float32(1e-4))) ** (n - 1 - 8)
    assert close(last[dv:], want, 1e-4) and np.abs(want).max() > 0.5


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_head_norms_with_a_shared_weight_and_with_a_gate(out_dtype):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(5)
    n, heads, dv, eps = 7, 3, 20, 1e-5
    y, gate = rng.normal(size=(n, heads, dv)) * 30, rng.normal(size=(n, heads * dv))
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    shared, whole = rng.normal(size=dv) + 1, rng.normal(size=heads * dv) + 1
    out = torch.empty((n, heads * dv), dtype=out_dtype, device="cuda")
    K.gated_group_norm(dev(y.reshape(n, -1)), None, 0, dev(shared), dv, K.GATE_NONE, eps, out)
    assert close(out.float().cpu().numpy(), P.rms_norm(f32(y), f32(shared), eps).reshape(n, -1), tol)
    wide = torch.cat([torch.zeros((n, 3), device="cuda"), dev(gate)], dim=1)
    K.gated_group_norm(dev(y.reshape(n, -1)), wide, 3, dev(whole), dv, K.GATE_SILU_LAST, eps, out)
    assert close(out.float().cpu().numpy(), P.rms(f32(y), eps).reshape(n, -1) * f32(whole) * P.silu(f32(gate)), tol)
    tiny = np.full((1, 1, dv), 1e-4)                                    # the epsilon sits inside the root
    o1 = torch.empty((1, dv), dtype=torch.float32, device="cuda")
    K.gated_group_norm(dev(tiny.reshape(1, -1)), None, 0, dev(np.ones(dv)), dv, K.GATE_NONE, 1e-3, o1)
    assert close(o1.cpu().numpy(), np.full((1, dv), 1e-4 / np.sqrt(1e-8 + 1e-3)), 1e-5)


# ---------------------------------------------------------------------------------------------------------
# latent attention
# ---------------------------------------------------------------------------------------------------------
def _plain_latent(H, dk, dr, dv, R, rot_dims, base, scale, eps, q_proj, down, c_weight, uk, uv):
    """The plain mixer on inputs that are the projections themselves: h = [q_proj | down], Wq and Wdkv pick their columns,
    the gate is sigmoid(0) and the output projection 2 I."""
    nq, nd = q_proj.shape[1], down.shape[1]
    h = np.concatenate([q_proj, down], axis=1)
    w = {"q": np.eye(nq, nq + nd), "dkv": np.eye(nd, nq + nd, k=nq), "dkv.norm": c_weight, "uk": uk, "uv": uv,
         "g": np.zeros((H * dv, nq + nd)), "o": 2.0 * np.eye(H * dv)}
    m = {"heads": H, "dim": dk, "rot_dim": dr, "vdim": dv, "kv_rank": R, "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    return P.latent_attention(h, w, m, eps)


def _latent(dtype, H, dk, dr, dv, R, rot_dims, base, scale, eps, q_proj, down, c_weight, uk, uv, portions, pages=None, splits=1,
            out_dtype=None, expand_from=0):
    """One sequence through prepare, the product with the keys' up-projection, attention over the cached latent and the
    values' up-projection, in portions; pages: the sequence's pages in the pool, in order.  Portions of `expand_from`
    tokens or more (when it is not 0) take the other route: whole keys and values of every head, written out for the
    portion from the gathered latents, under the grouped-query attention kernels."""
    from burn_lm_b200 import kernels as K
    T = q_proj.shape[0]
    n_pages = (T + PAGE - 1) // PAGE
    pages = list(pages) if pages is not None else list(range(n_pages))
    pool = torch.full((max(pages) + 2, PAGE, R + dr), float("nan"), dtype=dtype, device="cuda")
    table = torch.full((2, len(pages) + 1), -1, dtype=torch.int32, device="cuda")
    table[1, :len(pages)] = ints(pages)
    freq = torch.tensor([base ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)], dtype=torch.float64, device="cuda") if rot_dims else None
    uk_t = dev(uk, dtype).view(H, dk, R).transpose(1, 2).contiguous()
    uv_d = dev(uv, dtype).view(H, dv, R).contiguous()
    outs, at = [], 0
    for k in portions:
        st = step_of((k,), [1], [at])
        if expand_from and k >= expand_from:
            hd = 64 if dk + dr <= 64 else 128
            q = torch.empty((k, H, hd), dtype=dtype, device="cuda")
            K.latent_prepare(dev(q_proj[at: at + k]), dev(down[at: at + k]), dev(c_weight), eps, freq, rot_dims, None, None, pool, table, st,
                             H, dk, dr, R, q_full=q)
            each = (at + k + PAGE - 1) // PAGE
            gathered = torch.full((each * PAGE, R + dr), float("nan"), dtype=dtype, device="cuda")
            K.latent_gather(pool, table, st, gathered, each, R + dr)
            kv = gathered[:, :R] @ torch.cat([dev(uk, dtype), dev(uv, dtype)]).t()
            whole = torch.full((each, 2, H, PAGE, hd), float("nan"), dtype=dtype, device="cuda")
            K.latent_expand(kv, gathered, whole, H, dk, dr, dv, R)
            o = torch.zeros((k, H * hd), dtype=dtype, device="cuda")
            K.attention(q, H * hd, whole, ints(list(range(each))).view(1, each), st.cu_seqlens, ints([0]), st.start_pos, o, k, 1, k, H, H, hd,
                        scale, max_kv_len=at + k)
            outs.append(o.view(k, H, hd)[:, :, :dv].reshape(k, H * dv).float().cpu().numpy())
            at += k
            continue
        q_nope = torch.empty((H, k, dk), dtype=dtype, device="cuda")
        q_rot = torch.empty((k, H, dr), dtype=torch.float32, device="cuda")
        K.latent_prepare(dev(q_proj[at: at + k]), dev(down[at: at + k]), dev(c_weight), eps, freq, rot_dims, q_nope, q_rot, pool, table, st,
                         H, dk, dr, R)
        q_lat = K.batched_product(q_nope, uk_t, out_dtype=torch.float32)
        mixed = torch.zeros((H, k, R), dtype=out_dtype or dtype, device="cuda")
        partial = torch.empty(K.latent_attention_scratch_floats(k, H, R, splits), device="cuda") if splits > 1 else None
        K.latent_attention(q_lat, q_rot, pool, table, st, mixed, H, R, dr, scale, n_splits=splits, partial=partial)
        heads = K.batched_product(mixed.to(dtype), uv_d, out_dtype=torch.float32)           # [H, k, dv]
        outs.append(heads.transpose(0, 1).reshape(k, H * dv).cpu().numpy())
        at += k
    assert at == T
    return np.concatenate(outs)


LATENT_SHAPES = [  # heads, unrotated, rotated, turning, value lanes, latent
    (4, 24, 16, 8, 20, 40), (1, 32, 32, 32, 32, 32), (5, 12, 6, 6, 20, 36), (8, 64, 32, 32, 64, 256), (2, 16, 16, 0, 16, 16),
    (3, 128, 64, 64, 128, 512), (17, 8, 4, 2, 8, 24)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dr,rot,dv,R", LATENT_SHAPES)
def test_latent_attention_in_prompts_portions_and_single_tokens(dtype, H, dk, dr, rot, dv, R):
    rng = np.random.default_rng(6)
    T, eps, scale, base = 150, 1e-5, 1.7 * (dk + dr) ** -0.5, 300.0
    q_proj, down = rng.normal(size=(T, H * (dk + dr))), 1.5 * rng.normal(size=(T, R + dr))
    c_weight, uk, uv = rng.normal(size=R) + 1, rng.normal(size=(H * dk, R)) / np.sqrt(R), rng.normal(size=(H * dv, R)) / np.sqrt(R)
    args = (H, dk, dr, dv, R, rot, base, scale, eps, q_proj, down, c_weight, uk, uv)
    rounded = (H, dk, dr, dv, R, rot, base, scale, eps, f32(q_proj), f32(down), f32(c_weight), *(dev(t, dtype).double().cpu().numpy() for t in (uk, uv)))
    want = _plain_latent(*rounded)
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    for portions, pages, splits in (((150,), None, 1), ((63, 1, 1, 2, 70, 5, 1, 1, 1, 1, 1, 1, 1, 1), [4, 0, 2], 1), ((100, 50), [1, 5, 3], 3),
                                    ((140,) + (1,) * 10, None, 2), ((2,) * 75, [2, 1, 0], 1)):
        got = _latent(dtype, *args, portions, pages=pages, splits=splits)
        assert close(got, want, tol), (portions, splits)


@pytest.mark.parametrize("H,dk,dr,rot,dv,R", [s for s in LATENT_SHAPES if s[1] + s[2] <= 128])
def test_latent_attention_with_the_heads_written_out_for_long_portions(H, dk, dr, rot, dv, R):
    rng = np.random.default_rng(8)
    dtype, T, eps, scale, base = torch.bfloat16, 333, 1e-5, 1.7 * (dk + dr) ** -0.5, 300.0
    q_proj, down = rng.normal(size=(T, H * (dk + dr))), 1.5 * rng.normal(size=(T, R + dr))
    c_weight, uk, uv = rng.normal(size=R) + 1, rng.normal(size=(H * dk, R)) / np.sqrt(R), rng.normal(size=(H * dv, R)) / np.sqrt(R)
    args = (H, dk, dr, dv, R, rot, base, scale, eps, q_proj, down, c_weight, uk, uv)
    rounded = (H, dk, dr, dv, R, rot, base, scale, eps, f32(q_proj), f32(down), f32(c_weight), *(dev(t, dtype).double().cpu().numpy() for t in (uk, uv)))
    want = _plain_latent(*rounded)
    for portions, pages in (((333,), None), ((200, 1, 1, 16, 17, 64, 2, 32), [4, 0, 2, 7, 1, 3]), ((64, 64, 128, 77), [5, 4, 3, 2, 1, 0]),
                            ((130, 3, 200), None)):
        got = _latent(dtype, *args, portions, pages=pages, expand_from=16)
        assert close(got, want, 4e-2), portions


@pytest.mark.parametrize("dr,R", [(4, 16), (16, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_key_far_back_at_page_borders_and_the_diagonal(dtype, dr, R):
    """All scores are zero but one pair's, planted in a rotated lane that does not turn: the query's output is that
    position's value if it may see it, and the mean of what it sees otherwise.  The key sits at the sequence's start, on
    both sides of page borders, on the diagonal, and one position after the query."""
    H, dk, dv, T = 2, 8, 8, 400
    rng = np.random.default_rng(7)
    c_weight, uk, uv = np.ones(R), rng.normal(size=(H * dk, R)), rng.normal(size=(H * dv, R))
    for key_at in (0, 63, 64, 127, 128, 255, 256, 320, 398, 399):
        for query_at in sorted({key_at - 1, key_at, min(key_at + 1, T - 1), T - 1} - {-1}):
            q_proj, down = np.zeros((T, H, dk + dr)), np.concatenate([rng.normal(size=(T, R)), np.zeros((T, dr))], axis=1)
            down[key_at, R + 3] = 8.0
            q_proj[query_at, :, dk + 3] = 8.0                       # score 64 on the planted pair, 0 elsewhere
            args = (H, dk, dr, dv, R, 2, 100.0, 1.0, 1e-5, q_proj.reshape(T, -1), down, c_weight, uk, uv)
            rounded = args[:9] + (f32(args[9]), f32(down), c_weight, *(dev(t, dtype).double().cpu().numpy() for t in (uk, uv)))
            want = _plain_latent(*rounded)
            values = P.rms(f32(down[:, :R]), 1e-5) @ rounded[-1].T
            seen = key_at <= query_at
            assert close(want[query_at], values[key_at] if seen else values[:query_at + 1].mean(axis=0), 1e-6)
            for portions, splits in (((T,), 1), ((T,), 4), ((key_at + 1,) + (1,) * (T - key_at - 1), 2) if key_at > 300 else ((200, 200), 3)):
                got = _latent(dtype, *args, portions, splits=splits)
                assert close(got[query_at], want[query_at], 1e-4 if dtype == torch.float32 else 3e-2), (key_at, query_at, portions)


def test_the_rotation_pairs_neighbouring_lanes_and_depends_on_the_distance():
    """Query and keys are one fixed vector in the first turning pair (frequency 1): the score is 36 cos(distance), so
    the weights sit on the distances 0, 6, 13, 19, 25 ... (multiples of 2 pi, nearly); a position one off, a pairing of lane i
    with lane i + dims / 2, or a sign of the sine the other way round gives other weights.  Far positions: the angle is
    taken exactly."""
    H, dk, dr, dv, R = 1, 4, 8, 4, 8
    rng = np.random.default_rng(8)
    for T in (200,):
        q_proj, down = np.zeros((T, dk + dr)), np.concatenate([rng.normal(size=(T, R)), np.zeros((T, dr))], axis=1)
        q_proj[:, dk: dk + 4] = [6.0, 0.0, 0.5, -0.5]
        down[:, R: R + 4] = [6.0, 0.0, -0.5, 0.5]
        q_proj[:, dk + 6], down[:, R + 6] = 1.0, rng.normal(size=T)        # a lane that does not turn
        args = (H, dk, dr, dv, R, 4, 7.0, 1.0, 1e-5, q_proj, down, np.ones(R), rng.normal(size=(dk, R)), np.eye(dv, R))
        want = _plain_latent(*args[:9], f32(q_proj), f32(down), *args[11:])
        for portions in ((T,), (130,) + (1,) * 70, (64, 64, 72)):
            got = _latent(torch.float32, *args, portions)
            assert close(got, want, 1e-4), portions
    # the plain rotation itself: lane 0 with lane 1, by position * base^(-2i / dims)
    one = P.rotate_pairs(np.array([[1.0, 0.0, 1.0, 0.0, 5.0]]), [3], 4, 100.0)[0]
    assert np.allclose(one, [np.cos(3.0), np.sin(3.0), np.cos(0.3), np.sin(0.3), 5.0])


def test_latent_rows_of_two_sequences_in_one_step_share_nothing():
    """Two sequences of different lengths appended and attended in one step, their pages interleaved in the pool."""
    from burn_lm_b200 import kernels as K
    H, dk, dr, dv, R, rot = 3, 16, 8, 16, 24, 8
    rng = np.random.default_rng(9)
    lengths, eps, scale = [130, 67], 1e-5, 0.3
    c_weight, uk, uv = rng.normal(size=R) + 1, rng.normal(size=(H * dk, R)) / 4, rng.normal(size=(H * dv, R)) / 4
    data = [(rng.normal(size=(n, H * (dk + dr))), rng.normal(size=(n, R + dr))) for n in lengths]
    want = [_plain_latent(H, dk, dr, dv, R, rot, 50.0, scale, eps, f32(q), f32(d), f32(c_weight), f32(uk), f32(uv)) for q, d in data]
    pool = torch.full((8, PAGE, R + dr), float("nan"), device="cuda")
    table = ints([0, 2, 4, 6, 5, 3, 1, 7]).view(2, 4)
    freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64, device="cuda")
    uk_t, uv_d = dev(uk).view(H, dk, R).transpose(1, 2).contiguous(), dev(uv).view(H, dv, R).contiguous()
    at = [0, 0]
    for portion in [(100, 60), (1, 1), (29, 6)]:
        st = step_of(portion, [1, 0], at)
        n = sum(portion)
        q = dev(np.concatenate([data[s][0][at[s]: at[s] + k] for s, k in enumerate(portion)]))
        d = dev(np.concatenate([data[s][1][at[s]: at[s] + k] for s, k in enumerate(portion)]))
        q_nope, q_rot = torch.empty((H, n, dk), device="cuda"), torch.empty((n, H, dr), device="cuda")
        K.latent_prepare(q, d, dev(c_weight), eps, freq, rot, q_nope, q_rot, pool, table, st, H, dk, dr, R)
        mixed = torch.zeros((H, n, R), device="cuda")
        K.latent_attention(K.batched_product(q_nope, uk_t), q_rot, pool, table, st, mixed, H, R, dr, scale)
        got = K.batched_product(mixed, uv_d).transpose(0, 1).reshape(n, -1).cpu().numpy()
        row = 0
        for s, k in enumerate(portion):
            assert close(got[row: row + k], want[s][at[s]: at[s] + k], 3e-5), (portion, s)
            row += k
            at[s] += k


def test_the_output_gate():
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(10)
    o, g = rng.normal(size=(5, 44)), 4 * rng.normal(size=(5, 50))
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        out = torch.empty((5, 44), dtype=dtype, device="cuda")
        K.sigmoid_gate(dev(o, dtype), dev(g)[:, 3:47], out)
        assert close(out.float().cpu().numpy(), dev(o, dtype).double().cpu().numpy() * P.sigmoid(f32(g)[:, 3:47]), tol)


# ---------------------------------------------------------------------------------------------------------
# the experts, the cap
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_experts,top,ff,limit", [(8, 2, 48, 1.5), (1, 1, 40, 0.5), (5, 5, 24, 3.0), (33, 7, 16, 1.0), (16, 4, 96, 100.0)])
def test_softmax_routing_with_a_correction_and_the_clamped_unit(dtype, n_experts, top, ff, limit):
    """The correction decides who is chosen and stays out of the weights; the weights sum to one; the unit clamps the gate
    from above only and the other half on both sides, and adds one to it."""
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(11)
    n, d = 77, 56
    h = dev(rng.normal(size=(n, d)), dtype)
    hp = h.double().cpu().numpy()
    w = {"router": rng.normal(size=(n_experts, d)) * 0.5, "correction": rng.normal(size=n_experts) * 0.3}
    for e in range(n_experts):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (dev(rng.normal(size=s) * 0.4, dtype).double().cpu().numpy() for s in ((ff, d), (ff, d), (d, ff)))
    ids, weights = K.moe_route(h, dev(w["router"]), top, softmax=True, correction=dev(w["correction"]), renormalise=True)
    want_ids, want_w = P.route(hp, f32(w["router"]), f32(w["correction"]), top)
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert np.abs(weights.cpu().numpy() - want_w).max() < 1e-5 and np.allclose(weights.sum(dim=1).cpu().numpy(), 1.0, atol=1e-5)
    if 1 < top < n_experts:        # without the correction others are chosen somewhere, and the weights are those of the scores alone
        plain_ids, _ = P.route(hp, f32(w["router"]), 0.0, top)
        assert not np.array_equal(plain_ids, want_ids)
        s = P.softmax(hp @ f32(w["router"]).T)
        picked = np.take_along_axis(s, want_ids, axis=1)
        assert np.allclose(want_w, picked / picked.sum(axis=1, keepdims=True))
    gate_up = dev(np.stack([np.concatenate([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(n_experts)]), dtype)
    down = dev(np.stack([w[f"e{e}.down"] for e in range(n_experts)]), dtype)
    got = K.moe_experts(h, ids, weights, gate_up, down, weight_on_input=False, clamp_limit=limit, clamp_alpha=1.702, out_dtype=torch.float32)
    want = P.experts_feed_forward(hp, {k: (f32(v) if k in ("router", "correction") else v) for k, v in w.items()},
                                  {"router": {"top": top}, "expert": {"limit": limit}})
    assert np.abs(got.cpu().numpy() - want).max() < (2e-5 if dtype == torch.float32 else 3e-2) * np.abs(want).max()
    if limit < 2.0:                # the clamps bite: the unclamped unit gives something else
        free = P.experts_feed_forward(hp, w, {"router": {"top": top}, "expert": {"limit": 1e9}})
        assert np.abs(free - want).max() > 0.05 * np.abs(want).max()


def test_the_plain_expert_unit_at_its_clamps():
    one = lambda g, u, limit: P.expert(np.array([[g, u]]), np.array([[1.0, 0.0]]), np.array([[0.0, 1.0]]), np.array([[1.0]]), limit)[0, 0]
    assert np.isclose(one(5.0, 0.0, 2.0), 2.0 * P.sigmoid(1.702 * 2.0))              # the gate is cut from above
    assert np.isclose(one(-5.0, 0.0, 2.0), -5.0 * P.sigmoid(1.702 * -5.0))           # and not from below
    assert np.isclose(one(1.0, 9.0, 2.0), P.sigmoid(1.702) * 3.0) and np.isclose(one(1.0, -9.0, 2.0), -P.sigmoid(1.702))
    assert np.isclose(one(1.0, -1.0, 2.0), 0.0)                                       # up + 1


def test_the_cap_on_the_logits():
    from burn_lm_b200 import kernels as K
    z = np.array([[-1e4, -40.0, -1.0, 0.0, 1e-3, 7.0, 29.0, 300.0]])
    x = dev(z)
    K.softcap(x, 12.5)
    assert close(x.cpu().numpy(), 12.5 * np.tanh(z / 12.5), 1e-6)


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
    tokens = random_tokens(1, 150, cfg["vocab"])
    want = P.forward(cfg, tensors, tokens)
    engine = engine_for(folder, dtype)
    every = list(range(len(tokens)))
    assert rows_ok(row_error(_logits(engine, tokens, every), want), dtype, tol)
    for portions in ([64, 64, 22], [1, 2, 61, 1, 1, 2, 2, 17, 63], [100] + [1] * 50, [2] * 75):
        assert rows_ok(row_error(_logits(engine, tokens, every, portions), want), dtype, tol), portions
    # the first tokens alone, one at a time from an empty sequence
    assert rows_ok(row_error(_logits(engine, tokens[:9], list(range(9)), [1] * 9), want[:9]), dtype, tol)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_stream_after_every_layer_run(tmp_path, name):
    """A looped layer counts every time it runs; the stream is rewritten before each pass."""
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, name)
    cfg, tensors = P.read_model_folder(folder)
    tokens = random_tokens(2, 40, cfg["vocab"])
    _, after = P.forward(cfg, tensors, tokens, return_layers=True)
    assert len(after) == len(P.run_order(cfg))
    engine = engine_for(folder, "float32")
    engine.use_graphs = False
    seen, kept = [], []
    for layer in engine.model.layers:
        block = layer.block

        def watched(resid, delta, step, view, next_norm=None, plain=block.forward):
            out = plain(resid, delta, step, view, next_norm=next_norm)
            seen.append((resid.clone() + (out.float() if out is not None else 0.0)).cpu().numpy())
            return out

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
        assert np.abs(got - want).max() < 1e-4 * np.abs(want).max(), i


@pytest.mark.parametrize("name", ["rid_a", "rid_c", "rid_d"])
@pytest.mark.parametrize("dtype,tol", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_unequal_requests_together_through_used_slots_and_pages(tmp_path, name, dtype, tol):
    from burn_lm_b200 import StepEntry
    folder = folder_for(tmp_path, name, dtype)
    cfg, tensors = P.read_model_folder(folder)
    engine = engine_for(folder, dtype, max_tokens=1024)
    errs = []
    for set_no in range(3):              # the same slots and pages serve three sets of requests
        lengths = [[1, 70, 130], [65, 3, 64, 20], [128, 2]][set_no]
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


@pytest.mark.parametrize("name", ["rid_a", "rid_c"])
def test_long_decoding(tmp_path, name):
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, name)
    cfg, tensors = P.read_model_folder(folder)
    tokens = random_tokens(5, 330, cfg["vocab"])
    want = P.forward(cfg, tensors, tokens)
    engine = engine_for(folder, "float32")
    slot = engine.acquire()
    engine.step([StepEntry(slot, tokens[:30], [])])
    for p in range(30, len(tokens)):
        row = engine.step([StepEntry(slot, [tokens[p]], [0])]).cpu().numpy()[0]
        assert row_error(row, want[p]) < FP32_TOL, p
    engine.release(slot)


@pytest.mark.parametrize("name", ["rid_a", "rid_b"])
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
    """Steps replayed as a graph without the host, after a warm-up step that runs the first one twice: the carried inputs
    and states of a sequence are read from where that step found them."""
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, "rid_a")
    cfg, tensors = P.read_model_folder(folder)
    prompts = [random_tokens(30 + i, n, cfg["vocab"]) for i, n in enumerate([33, 64])]
    want = [P.greedy(cfg, tensors, p, 9) for p in prompts]
    engine = engine_for(folder, "float32", max_tokens=1024)
    slots = [engine.acquire() for _ in prompts]
    first = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).argmax(dim=-1).tolist()
    assert first == [w[0] for w in want]
    more = engine.decode_run(slots, first, 8).cpu().numpy()
    assert more.T.tolist() == [w[1:] for w in want]
    again = engine.decode_run(slots, [w[-1] for w in want], 3)       # the captured graph once more, from where it stopped
    longer = [P.greedy(cfg, tensors, p, 12) for p in prompts]
    assert again.cpu().numpy().T.tolist() == [w[9:] for w in longer]


def test_the_trace_runner_as_a_child_process(tmp_path):
    cfg = CONFIGS["rid_c"]
    a, b = random_tokens(40, 75, cfg["vocab"]), random_tokens(41, 9, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[70]], "want": []}, {"id": "b", "tokens": [b[5]], "want": [0]}], "end": []}]
    steps += [{"step": 2 + t, "entries": [{"id": "a", "tokens": [a[71 + t]], "want": [0]}] + ([{"id": "b", "tokens": [b[6 + t]], "want": [0]}] if t < 3 else []),
               "end": ["b"] if t == 2 else []} for t in range(4)]
    out = tmp_path / "out"
    for dtype, tol in (("float32", FP32_TOL), ("bfloat16", BF16_TOL)):
        folder = folder_for(tmp_path, "rid_c", dtype)
        cfg, tensors = P.read_model_folder(folder)
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
                               "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
        wa, wb = P.forward(cfg, tensors, a), P.forward(cfg, tensors, b)
        read = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        want = {0: [wa[0], wa[69], wb[4]], 1: [wb[5]]}
        want.update({2 + t: [wa[71 + t]] + ([wb[6 + t]] if t < 3 else []) for t in range(4)})
        if dtype == "bfloat16":
            # the runner adds no arithmetic: the same steps through an engine in this process give the same rows, up to what
            # another choice of kernels for another cache size rounds differently (the short request's second token is a
            # close call between two experts in bfloat16, so the plain rows judge float32 and the long request only)
            from burn_lm_b200 import StepEntry
            engine = engine_for(folder, dtype, max_tokens=256)
            slot = {}
            for s in steps:
                for e in s["entries"]:
                    if e["id"] not in slot:
                        slot[e["id"]] = engine.acquire()
                rows = engine.step([StepEntry(slot[e["id"]], e["tokens"], e["want"]) for e in s["entries"]])
                if any(e["want"] for e in s["entries"]):
                    assert row_error(read(s["step"]), rows.cpu().numpy().astype(np.float64)).max() < tol / 2, s["step"]
                for name in s["end"]:
                    engine.release(slot.pop(name))
            a_rows = [row_error(read(n)[:1], np.stack(w[:1]))[0] for n, w in want.items() if n != 1]
            assert rows_ok(a_rows, dtype, tol), a_rows
            continue
        errs = [e for n, w in want.items() for e in row_error(read(n), np.stack(w))]
        assert len(errs) == 11 and rows_ok(errs, dtype, tol), errs


def test_the_command_line_on_the_preset(tmp_path):
    program = [sys.executable, os.path.join(ROOT, "bin", "burn-lm")]
    folder = str(tmp_path / "n")
    r = subprocess.run(program + ["random", folder, "--preset", "ridopel_tiny", "--seed", "4", "--dtype", "float32"],
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


def test_sampling_with_a_temperature_runs_inside_the_captured_step(tmp_path):
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, "rid_a")
    lm = blm.load(folder, dtype="bfloat16", max_seq_len=256, max_batch=2)
    prompts = [random_tokens(50, 20, 352), random_tokens(51, 66, 352)]
    a = lm.generate(prompts, sample_len=12, temperature=0.8, seed=7, ignore_stop=True).tokens
    b = lm.generate(prompts, sample_len=12, temperature=0.8, seed=7, ignore_stop=True).tokens
    assert a == b and all(len(t) == 12 for t in a)          # the same draws from the same seed, through used slots


@pytest.mark.parametrize("kinds", ["wkv only", "hgrn2 only", "latent only", "no feed-forward at all", "the loop last"])
def test_models_of_one_kind_of_layer_and_other_loops(tmp_path, kinds):
    """No pages at all, no state of a scan at all, no experts at all, and a loop over the model's last layers."""
    e = experts(6, 2, 32)
    layers, loop = {
        "wkv only": ([wkv(2, 16, e), wkv(4, 8, None)], (1, 2, 2)),
        "hgrn2 only": ([hgrn2(2, 16, 8, None), hgrn2(1, 24, 48, e)], (0, 2, 2)),
        "latent only": ([latent(2, 16, 8, 16, 24, e), latent(3, 8, 8, 16, 16, None, rot_dims=4)], None),
        "no feed-forward at all": ([wkv(2, 24, None), latent(2, 8, 16, 8, 32, None), hgrn2(3, 8, 16, None)], (1, 3, 3)),
        "the loop last": ([latent(2, 16, 8, 16, 24, e), hgrn2(2, 16, 8, e), wkv(2, 16, e), latent(1, 16, 16, 48, 8, e)], (2, 4, 4)),
    }[kinds]
    cfg = model(97, 48, layers, taps=3, loop=loop, cap=25.0 if kinds != "latent only" else None)
    tokens = random_tokens(7, 90, 97)
    for dtype, tol in (("float32", FP32_TOL), ("bfloat16", BF16_TOL)):
        folder = folder_for(tmp_path, "m", dtype, seed=3, config=cfg)
        pcfg, tensors = P.read_model_folder(folder)
        want = P.forward(pcfg, tensors, tokens)
        engine = engine_for(folder, dtype)
        assert rows_ok(row_error(_logits(engine, tokens, list(range(90)), [70] + [1] * 20), want), dtype, tol)
        assert rows_ok(row_error(_logits(engine, tokens, list(range(90)), [3, 64, 2, 21]), want), dtype, tol)
