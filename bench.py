"""Decode and prefill throughput of the Llama-3.2-1B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--config 1b|3b|8b]
    python bench.py --compare fobilorn|nufolix|ridopel|marinex [--size 1b-layers|8b-layers]     (another design beside this one, see run_compare)

A "step" is one decode step of the whole batch.  The default run has the layer sizes of the 1B
configuration (16 layers, width 2048, 32 heads on 8 kv heads of 64, inner 8192, vocabulary 128256,
llama3 rotary scaling, tied head), bfloat16 random weights N(0, 0.02), a batch of 8 sequences with
512-token random prompts in a context of 4096, and prints ONE JSON line:

  value      decoded tokens a second: K steps run back to back on the device (captured CUDA graph,
             greedy token fed back by a kernel), timed with CUDA events
  e2e        the same through the Python entry point `LanguageModel.generate`: every step copies its
             inputs from pinned host memory and reads the sampled tokens back
  prefill    one 2,048-token prompt in one step
  roofline   the decode step against the HBM bandwidth: bytes it has to read / its time
  points     decode at batch 1 and 64

--config 3b: the Llama-3.2-3B shape, 16 prompts of 64 to 4,096 tokens prefilled together, 128 greedy steps,
context 8192.  --config 8b: the Llama-3.1-8B shape, 32 prompts of 128 to 2,048 tokens, 256 steps at temperature
0.7 (the draw runs inside the captured step; the host launches every step), and a 2,048-token prefill.
Models are built with random weights drawn on the device (`load_random`), no folder in between.

Peaks come from MEASURED_PEAKS.json beside this file when it is there.  The weights (2.47 GB) are
far larger than the L2, so nothing is flushed between steps.  For --gpus N > 1 it says that this
library runs on one GPU and exits with 2.  The reference arm is unavailable: tracel-ai/burn-lm is a
Rust workspace and neither cargo nor its git dependency `burn` can be had offline.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The workloads, by the name --config takes.  "1b" is the headline and the default; "3b" and "8b" are the two
# larger shapes with the batches their configurations state.  `prompts`: ("equal", n) or ("uniform", lo, hi).
WORKLOADS = {
    "1b": {"preset": "llama3_2_1b", "model": "llama-3.2-1b-shape-random", "context": 4096, "batch": 8,
           "prompts": ("equal", 512), "steps": 256, "temperature": 0.0, "prefill": ("one", 2048), "points": (1, 64)},
    "3b": {"preset": "llama3_2_3b", "model": "llama-3.2-3b-shape-random", "context": 8192, "batch": 16,
           "prompts": ("uniform", 64, 4096), "steps": 128, "temperature": 0.0, "prefill": ("batch",), "points": ()},
    "8b": {"preset": "llama3_1_8b", "model": "llama-3.1-8b-shape-random", "context": 8192, "batch": 32,
           "prompts": ("uniform", 128, 2048), "steps": 256, "temperature": 0.7, "prefill": ("one", 2048), "points": ()},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read only) while a region runs."""

    def __init__(self, period=0.004):
        self.period, self.samples, self.reasons = period, [], set()
        self._stop = threading.Event()
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            idx = int(os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or 0)
            try:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    _NAMES = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
              0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
              0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self._NAMES.items():
                    if r & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._loop, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self.nv is not None:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def weight_bytes(cfg):
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    h, kv, hd, layers = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    per_layer = d * (h + 2 * kv) * hd + h * hd * d + 3 * d * i + 2 * d
    head = v * d if cfg.get("tie_word_embeddings") else 2 * v * d      # untied: the table is stored beside the head
    return 2 * (layers * per_layer + head + d)      # bf16


def decode_step_bytes(cfg, live_tokens):
    """What a decode step has to read: every weight it uses once (the embedding table only as far as it is
    the head: a step gathers a handful of its rows) and the cache of the live sequences."""
    d, v = cfg["hidden_size"], cfg["vocab_size"]
    used = weight_bytes(cfg) - (0 if cfg.get("tie_word_embeddings") else 2 * v * d)
    return used + live_tokens * kv_bytes_per_token(cfg)


def kv_bytes_per_token(cfg):
    return 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, lengths):
    """Flops of one prompt step over prompts of these lengths: the products over all tokens, attention within
    each prompt (the causal half of QK^T and PV), the head on one row per prompt."""
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    h, kv, hd, layers = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    per_layer = d * (h + 2 * kv) * hd + h * hd * d + 3 * d * i
    total = sum(lengths)
    gemm = 2.0 * total * layers * per_layer + 2.0 * v * d * len(lengths)
    attn = layers * 2.0 * h * hd * sum(t * t for t in lengths)
    return gemm + attn


def make_prompts(spec, n, vocab, seed):
    """`spec`: ("equal", length) or ("uniform", lo, hi); ids uniform over the vocabulary, seeded."""
    import numpy as np
    rng = np.random.default_rng(seed)
    if spec[0] == "equal":
        lengths = [spec[1]] * n
    else:
        lengths = [int(x) for x in rng.integers(spec[1], spec[2] + 1, size=n)]
    return [[int(x) for x in rng.integers(0, vocab, size=length)] for length in lengths]


def prefill_in_parts(engine, slots, prompts, most=8192):
    """Prompts go in a few at a time to keep the prefill's activations small."""
    from burn_lm_b200 import StepEntry
    group, held = [], 0
    for s, p in zip(slots, prompts):
        if group and held + len(p) > most:
            engine.step([StepEntry(a, b, []) for a, b in group])
            group, held = [], 0
        group.append((s, p))
        held += len(p)
    if group:
        engine.step([StepEntry(a, b, []) for a, b in group])


def device_decode(engine, prompts, steps, warmup, sample_clocks=False, temperature=0.0):
    """Prefill the prompts, then time `steps` decode steps.  Greedy: the steps run back to back on the device
    (captured graph, the argmax token fed back by a kernel).  With a temperature: every step is the captured
    graph with the draw inside it, launched by the host with the step's tokens (the draw needs the host's counters)."""
    import torch
    from burn_lm_b200 import kernels
    from burn_lm_b200.sampling import SamplingParams
    batch = len(prompts)
    lengths = [len(p) for p in prompts]
    slots = [engine.acquire() for _ in range(batch)]
    try:
        prefill_in_parts(engine, slots, prompts)
        first = [p[-1] for p in prompts]
        params = SamplingParams(temperature, 0.9, 1234) if temperature > 0 else None

        def run(n):
            if params is None:
                return engine.decode_run(slots, first, n)
            toks = list(first)
            for k in range(n):
                toks = engine.decode_sampled(slots, toks, params, list(range(batch)), [k] * batch)
                assert toks is not None, "this engine does not capture its decode steps"
            return toks

        sampled_per_step = 0
        if params is not None:                                   # the first drawn step runs plainly, then is captured
            count0 = kernels.launch_count()
            run(1)
            sampled_per_step = (kernels.launch_count() - count0) // 2
        run(max(warmup, 3))                                      # warm-up: captures the graph, W steps
        for s, n in zip(slots, lengths):                         # rewind: the timed run decodes from the prompts' ends
            engine.cache.set_length(s, n)
        torch.cuda.synchronize()
        before = kernels.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.__enter__()
        torch.cuda.synchronize()
        start.record()
        run(steps)
        stop.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.__exit__()
        ms = start.elapsed_time(stop)
        g = engine.decode_graph(batch, max(lengths) + steps)
        per_step = sampled_per_step or g.launches_per_step or 0
        launches = per_step * steps + (kernels.launch_count() - before)
        engine.verify()        # no kernel gave up a bounded wait
        return {"ms_per_step": ms / steps, "tokens_per_s": batch * steps / (ms / 1e3), "launches": launches,
                "clocks": sampler.summary() if sampler else None, "graph": g}
    finally:
        for s in slots:
            engine.release(s)


def time_prefill(engine, prompts, reps=5):
    """Median time of one prefill step over `prompts`, the last logits of each wanted."""
    import torch
    from burn_lm_b200 import StepEntry
    times = []
    for r in range(reps + 2):
        slots = [engine.acquire() for _ in prompts]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        stop.record()
        torch.cuda.synchronize()
        for s in slots:
            engine.release(s)
        if r >= 2:
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def sweep(engine, cfg, pk):
    """Decode and prefill at further batch sizes and context lengths, one JSON line each, with the
    fraction of the measured peak (bytes a step has to read, or flops) beside the time."""
    vocab = cfg["vocab_size"]
    for prompt_len in (512, 2048, 3840):
        for b in (1, 8, 64):
            steps = 128
            r = device_decode(engine, make_prompts(("equal", prompt_len), b, vocab, seed=b), steps, 3)
            gbs = decode_step_bytes(cfg, b * (prompt_len + steps / 2.0)) / (r["ms_per_step"] / 1e3) / 1e9
            print(json.dumps({"decode": {"batch": b, "context": prompt_len, "ms_per_step": round(r["ms_per_step"], 4),
                                         "tokens_per_s": round(r["tokens_per_s"], 1), "gb_per_s": round(gbs, 1),
                                         "frac_hbm": round(gbs / pk["hbm_gbs"], 3)}}), flush=True)
    for n_prompts, tokens in ((1, 128), (1, 512), (1, 2048), (1, 4096), (8, 512), (16, 1024)):
        prompts = make_prompts(("equal", tokens), n_prompts, vocab, seed=99)
        ms = time_prefill(engine, prompts, reps=3)
        flops = prefill_flops(cfg, [tokens] * n_prompts)
        print(json.dumps({"prefill": {"prompts": n_prompts, "tokens_each": tokens, "ms": round(ms, 3),
                                      "tokens_per_s": round(n_prompts * tokens / (ms / 1e3), 1),
                                      "frac_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3)}}), flush=True)


# ---------------------------------------------------------------------------------------------------------
# --compare fobilorn: the Fobilorn decoder beside the dense Llama decoder at equal layer sizes
# ---------------------------------------------------------------------------------------------------------
COMPARE_SIZES = {
    # name: width, heads, kv heads, head size, inner size, layers, vocabulary, window, kept first, experts, top
    "1b-layers": dict(width=2048, heads=32, kv=8, hd=64, inner=8192, layers=4, vocab=32000, window=1024, keep=64, experts=16, top=2),
    "8b-layers": dict(width=4096, heads=32, kv=8, hd=128, inner=14336, layers=2, vocab=32000, window=1024, keep=64, experts=16, top=2),
}


def compare_configs(z):
    """(llama, fobilorn with dense feed-forwards, fobilorn with experts) of one size.  The experts' layers keep the
    inner size a token uses: `top` experts of inner / (2 top) each beside a shared one of inner / 2."""
    llama = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": z["layers"], "hidden_size": z["width"],
             "num_attention_heads": z["heads"], "num_key_value_heads": z["kv"], "head_dim": z["hd"], "intermediate_size": z["inner"],
             "vocab_size": z["vocab"], "rope_theta": 500000.0, "rope_scaling": None, "rms_norm_eps": 1e-5,
             "tie_word_embeddings": False, "max_position_embeddings": 8192, "hidden_act": "silu"}

    def fob(mlp):
        layer = {"type": "attention", "mlp": mlp,
                 "mixer": {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["hd"], "vdim": z["hd"], "scale": z["hd"] ** -0.5,
                           "v_mix": True, "mask": {"size": z["window"], "keep_first": z["keep"]}}}
        return {"architecture": "Fobilorn", "vocab": z["vocab"], "width": z["width"],
                "embedding": {"bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 17}}, "norm": {"eps": 1e-6},
                "layers": [layer] * z["layers"]}
    each = z["inner"] // (2 * z["top"])
    return {"llama": llama, "fobilorn-dense": fob({"kind": "dense", "ff": z["inner"]}),
            "fobilorn-experts": fob({"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": each},
                                     "shared": {"ff": z["inner"] // 2}})}


def _time(fn, reps=10):
    import torch
    for _ in range(3):
        fn()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps


def compare_kernels(z, pk):
    """The new design's kernels alone beside the like kernels of the dense decoder, CUDA events, back to back: prompt
    attention (one 2,048-token prompt), decode attention (64 sequences of 1,088 tokens) and the feed-forward of a
    token's share of experts beside the dense products of the same inner size (2,048 and 64 tokens)."""
    import torch
    from types import SimpleNamespace
    from burn_lm_b200 import kernels as K
    dev, bf = "cuda", torch.bfloat16
    H, G, hd, d = z["heads"], z["kv"], z["hd"], z["width"]
    out = {}
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)

    def attention_case(n_seqs, new, cached):
        total = cached + new
        pages_each = -(-total // K.PAGE)
        n = n_seqs * new
        bt = torch.arange(n_seqs * pages_each, dtype=torch.int32, device=dev).reshape(n_seqs, pages_each)
        seq = [s for s in range(n_seqs) for _ in range(new)]
        pos = [cached + t for _ in range(n_seqs) for t in range(new)]
        st = SimpleNamespace(token_seq=i32(seq), token_pos=i32(pos), slot_of_seq=i32(list(range(n_seqs))),
                             cu_seqlens=i32([new * s for s in range(n_seqs + 1)]), start_pos=i32([cached] * n_seqs))
        q = torch.randn((n, H * hd), dtype=bf, device=dev)
        # the dense decoder's kernel: window as the new design's, no kept first tokens
        pool5 = torch.randn((n_seqs * pages_each, 2, G, K.PAGE, hd), dtype=bf, device=dev)
        o = torch.empty_like(q)
        splits = 1
        ms_llama = _time(lambda: K.attention(q, q.shape[1], pool5, bt, st.cu_seqlens, st.slot_of_seq, st.start_pos, o, n, n_seqs, new,
                                             H, G, hd, hd ** -0.5, window=z["window"], n_splits=splits, max_kv_len=total))
        pool = pool5.reshape(n_seqs * pages_each, -1)
        gate = torch.randn((n, H), dtype=torch.float32, device=dev)
        ms_new = _time(lambda: K.attention_sink(q, st, pool, bt, o, H, G, hd, hd, hd ** -0.5, z["window"], z["keep"], sink=True,
                                                gate=gate, gate_stride=H, max_q_len=new))
        return ms_llama, ms_new, n, total

    # prompt: flops of the visible pairs (window and causal), both products
    ms_l, ms_n, n, total = attention_case(1, 2048, 0)
    pairs = sum(min(t + 1, z["window"]) for t in range(2048))
    flops = 4.0 * H * hd * pairs
    out["attention_prefill_2048"] = {"llama_ms": round(ms_l, 4), "fobilorn_ms": round(ms_n, 4),
                                     "llama_frac_bf16": round(flops / (ms_l / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                                     "fobilorn_frac_bf16": round(flops / (ms_n / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    ms_l, ms_n, n, total = attention_case(64, 1, 1087)
    seen = min(total, z["window"])
    nbytes = 64 * G * seen * 2 * hd * 2
    out["attention_decode_b64"] = {"llama_ms": round(ms_l, 4), "fobilorn_ms": round(ms_n, 4), "keys_seen": seen,
                                   "llama_frac_hbm": round(nbytes / (ms_l / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                                   "fobilorn_frac_hbm": round(nbytes / (ms_n / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    # feed-forward: a token's experts beside dense products of the inner size they make together
    E, top = z["experts"], z["top"]
    each = z["inner"] // (2 * top)
    gate_up = torch.randn((E, 2 * each, d), dtype=bf, device=dev) * 0.02
    down = torch.randn((E, d, each), dtype=bf, device=dev) * 0.02
    router = torch.randn((E, d), dtype=torch.float32, device=dev)
    w1 = torch.randn((2 * top * each, d), dtype=bf, device=dev) * 0.02
    w2 = torch.randn((d, top * each), dtype=bf, device=dev) * 0.02
    for n in (2048, 64):
        h = torch.randn((n, d), dtype=bf, device=dev)
        ids, weights = K.moe_route(h, router, top)
        ms_moe = _time(lambda: K.moe_experts(h, ids, weights, gate_up, down))
        a = torch.empty((n, top * each), dtype=bf, device=dev)

        def dense():
            gu = torch.mm(h, w1.t())
            K.swiglu(gu, a)
            return torch.mm(a, w2.t())
        ms_dense = _time(dense)
        flops = 2.0 * n * top * 3 * each * d
        wbytes = 2.0 * 3 * each * d * min(E, n * top)             # the weights of the experts that get a token
        out[f"experts_{n}_tokens"] = {
            "fobilorn_ms": round(ms_moe, 4), "dense_same_inner_ms": round(ms_dense, 4),
            "fobilorn_frac_bf16": round(flops / (ms_moe / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
            "dense_frac_bf16": round(flops / (ms_dense / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
            "fobilorn_frac_hbm": round(wbytes / (ms_moe / 1e3) / 1e9 / pk["hbm_gbs"], 4),
            "dense_frac_hbm": round(2.0 * 3 * top * each * d / (ms_dense / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    return out


def nufolix_configs(z):
    """(llama, nufolix) of one size: half of the new design's layers are state-space scans without a feed-forward, half hold
    sigmoid attention beside a gated delta rule and a dense feed-forward of the same inner size as the dense decoder's."""
    llama = compare_configs(z)["llama"]
    hd, d = z["hd"], z["width"]
    par = {"type": "parallel", "mlp": {"kind": "dense", "ff": z["inner"]},
           "mixer": {"left": {"heads": z["heads"], "kv_heads": z["kv"], "dim": hd, "vdim": hd, "scale": hd ** -0.5, "softcap": 30.0,
                              "rot": {"dims": hd, "base": 500000.0}},
                     "right": {"heads": d // 128, "kv_heads": d // 256, "dim": 128, "vdim": 128, "conv": 4},
                     "left_scale": 0.7, "right_scale": 0.7}}
    ssm = {"type": "mamba2", "mlp": None,
           "mixer": {"heads": 2 * d // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8}}
    nuf = {"architecture": "Nufolix", "vocab": z["vocab"], "width": d, "embedding": {"scale": d ** 0.5}, "norm": {"eps": 1e-6},
           "residual_mult": 0.7, "layers": [par if i % 2 == 0 else ssm for i in range(z["layers"])]}
    return {"llama": llama, "nufolix": nuf}


def nufolix_kernels(z, pk):
    """The new design's kernels alone, CUDA events, back to back, beside the like kernel of the dense decoder where it has
    one: attention over one 2,048-token prompt and over 64 sequences of 1,088 tokens, the two scans over the same rows."""
    import torch
    from types import SimpleNamespace
    from burn_lm_b200 import kernels as K
    dev, bf = "cuda", torch.bfloat16
    H, G, hd, d = z["heads"], z["kv"], z["hd"], z["width"]
    out = {}
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)

    def step(n_seqs, new, cached):
        seq = [s for s in range(n_seqs) for _ in range(new)]
        pos = [cached + t for _ in range(n_seqs) for t in range(new)]
        return SimpleNamespace(token_seq=i32(seq), token_pos=i32(pos), slot_of_seq=i32(list(range(n_seqs))),
                               cu_seqlens=i32([new * s for s in range(n_seqs + 1)]), start_pos=i32([cached] * n_seqs),
                               n_tokens=n_seqs * new, n_seqs=n_seqs, max_q_len=new, max_kv_len=cached + new)

    def attention_case(n_seqs, new, cached):
        total = cached + new
        # the key ranges the mixer takes at this size (parts.sigmoid_attention.SigmoidAttention._ranges)
        tiles, sms = n_seqs * (-(-new // 16)), K.sm_count()
        ranges = max(1, min(-(-(4 if new == 1 else 2) * sms // tiles), total // (K.PAGE if new == 1 else 256), 64))
        pages_each = -(-total // K.PAGE)
        n = n_seqs * new
        bt = torch.arange(n_seqs * pages_each, dtype=torch.int32, device=dev).reshape(n_seqs, pages_each)
        st = step(n_seqs, new, cached)
        q = torch.randn((n, H * hd), dtype=bf, device=dev)
        pool5 = torch.randn((n_seqs * pages_each, 2, G, K.PAGE, hd), dtype=bf, device=dev)
        o = torch.empty_like(q)
        ms_llama = _time(lambda: K.attention(q, q.shape[1], pool5, bt, st.cu_seqlens, st.slot_of_seq, st.start_pos, o, n, n_seqs, new,
                                             H, G, hd, hd ** -0.5, window=0, n_splits=1, max_kv_len=total))
        pool = pool5.reshape(n_seqs * pages_each, -1)
        talk = torch.randn((H, H), dtype=torch.float32, device=dev) * 0.2
        pb = torch.randn(H, dtype=torch.float32, device=dev) - 3.0
        partial = torch.empty(ranges * n * H * hd, dtype=torch.float32, device=dev) if ranges > 1 else None
        ms_new = _time(lambda: K.sigmoid_attention(q, pool, bt, st, o, H, G, hd, hd, hd ** -0.5, softcap=30.0, talk=talk, head_bias=pb,
                                                   ranges=ranges, partial=partial), reps=3)
        return ms_llama, ms_new, total, ranges

    ms_l, ms_n, total, ranges = attention_case(1, 2048, 0)
    pairs = 2048 * 2049 / 2
    flops = 4.0 * H * hd * pairs
    mix = 2.0 * H * H * pairs                      # the heads' mix: fp32 multiply-adds outside the tensor cores
    out["attention_prefill_2048"] = {"llama_ms": round(ms_l, 4), "nufolix_ms": round(ms_n, 4), "key_ranges": ranges, "mix_gflop_fp32": round(mix / 1e9, 1),
                                     "llama_frac_bf16": round(flops / (ms_l / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                                     "nufolix_frac_bf16": round(flops / (ms_n / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    ms_l, ms_n, total, ranges = attention_case(64, 1, 1087)
    nbytes = 64 * G * total * 2 * hd * 2
    out["attention_decode_b64"] = {"llama_ms": round(ms_l, 4), "nufolix_ms": round(ms_n, 4), "keys_seen": total, "key_ranges": ranges,
                                   "llama_frac_hbm": round(nbytes / (ms_l / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                                   "nufolix_frac_hbm": round(nbytes / (ms_n / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    # the scans: prompts read and write rows (a pass over their inputs and outputs), single tokens the states
    for name, heads, groups, rows, dv in (("ssm", 2 * d // 64, 8, 128, 64), ("delta", d // 128, d // 256, 128, 128)):
        inner = heads * dv
        for n_seqs, new, cached in ((1, 2048, 0), (64, 1, 1087)):
            st = step(n_seqs, new, cached)
            n = st.n_tokens
            floats = K.scan_state_floats(heads, rows, dv)
            state = torch.zeros((n_seqs, 2, floats), dtype=torch.float32, device=dev)
            y = torch.zeros((n, inner), dtype=torch.float32, device=dev)
            if name == "ssm":
                xbc = torch.randn((n, inner + 2 * groups * rows), dtype=torch.float32, device=dev)
                dt = torch.randn((n, heads), dtype=torch.float32, device=dev)
                one = torch.zeros(heads, dtype=torch.float32, device=dev)
                ms = _time(lambda: K.ssm_scan(xbc, 0, inner, inner + groups * rows, dt, 0, one, one, one, y, heads, groups, rows, dv, st, state, 0), reps=3)
                row_bytes = 4.0 * n * (2 * inner + 2 * groups * rows + heads)
            else:
                qkv = torch.randn((n, 2 * groups * rows + inner), dtype=torch.float32, device=dev)
                b = torch.randn((n, heads), dtype=torch.float32, device=dev)
                a = torch.randn((n, heads * rows), dtype=torch.float32, device=dev)
                bias, alog = torch.zeros(heads * rows, dtype=torch.float32, device=dev), torch.zeros(heads, dtype=torch.float32, device=dev)
                ms = _time(lambda: K.delta_scan(qkv, 0, qkv, groups * rows, qkv, 2 * groups * rows, b, 0, a, 0, bias, alog, y, heads, groups, rows, dv, st, state, 0), reps=3)
                row_bytes = 4.0 * n * (2 * inner + 2 * groups * rows + heads * rows + heads)
            state_bytes = 2.0 * 4 * n_seqs * floats          # read and written once a step
            flops = (4.0 if name == "ssm" else 8.0) * n * heads * rows * dv
            out[f"{name}_scan_{n_seqs}x{new}"] = {"ms": round(ms, 4), "frac_hbm": round((row_bytes + state_bytes) / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                                                  "gflop_fp32_per_s": round(flops / (ms / 1e3) / 1e9, 1)}
    return out


def ridopel_configs(z):
    """(llama, ridopel) of one size.  The new design's layers take turns: attention over a cached latent (Llama's head count
    and head size, half of a head's key lanes rotated, a latent of 4 heads' width), WKV and HGRN2 with heads of Llama's size,
    each with `experts` experts of which a token uses `top`, whose inner sizes make Llama's together."""
    llama = compare_configs(z)["llama"]
    hd, d, H = z["hd"], z["width"], z["heads"]
    mlp = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["inner"] // z["top"], "limit": 7.0}}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": H, "dim": hd // 2, "rot_dim": hd // 2, "vdim": hd, "kv_rank": 4 * hd, "scale": hd ** -0.5,
                        "rot": {"dims": hd // 2, "base": 500000.0}}}
    wkv = {"type": "wkv", "mlp": mlp, "mixer": {"heads": d // hd, "dim": hd}}
    hgrn = {"type": "hgrn2", "mlp": mlp, "mixer": {"heads": d // hd, "dim": hd, "vdim": hd}}
    turn = (latent, wkv, hgrn, latent)
    rid = {"architecture": "Ridopel", "vocab": z["vocab"], "width": d, "norm": {"eps": 1e-6}, "canon": {"taps": 4}, "logit_softcap": 30.0,
           "layers": [turn[i % 4] for i in range(z["layers"])]}
    return {"llama": llama, "ridopel": rid}


def ridopel_kernels(z, pk):
    """The new design's kernels alone, CUDA events, back to back: attention over the latent beside the dense decoder's
    attention (one 2,048-token prompt; 64 sequences of 1,088 tokens), the two decay scans over the same rows, and the clamped
    experts beside dense products of the inner size a token uses."""
    import torch
    from types import SimpleNamespace
    from burn_lm_b200 import kernels as K
    dev, bf = "cuda", torch.bfloat16
    H, G, hd, d = z["heads"], z["kv"], z["hd"], z["width"]
    R, dr = 4 * hd, hd // 2
    out = {}
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)

    def step(n_seqs, new, cached):
        seq = [s for s in range(n_seqs) for _ in range(new)]
        pos = [cached + t for _ in range(n_seqs) for t in range(new)]
        return SimpleNamespace(token_seq=i32(seq), token_pos=i32(pos), slot_of_seq=i32(list(range(n_seqs))),
                               cu_seqlens=i32([new * s for s in range(n_seqs + 1)]), start_pos=i32([cached] * n_seqs),
                               n_tokens=n_seqs * new, n_seqs=n_seqs, max_q_len=new, max_kv_len=cached + new)

    def attention_case(n_seqs, new, cached):
        total = cached + new
        pages_each = -(-total // K.PAGE)
        n = n_seqs * new
        bt = torch.arange(n_seqs * pages_each, dtype=torch.int32, device=dev).reshape(n_seqs, pages_each)
        st = step(n_seqs, new, cached)
        q = torch.randn((n, H * hd), dtype=bf, device=dev)
        pool5 = torch.randn((n_seqs * pages_each, 2, G, K.PAGE, hd), dtype=bf, device=dev)
        o = torch.empty_like(q)
        ms_llama = _time(lambda: K.attention(q, q.shape[1], pool5, bt, st.cu_seqlens, st.slot_of_seq, st.start_pos, o, n, n_seqs, new,
                                             H, G, hd, hd ** -0.5, window=0, n_splits=1, max_kv_len=total))
        # the key shares the mixer takes at this size (parts.latent_attention.LatentAttention._splits)
        tile = K.latent_attention_tile_rows(bf, H, R, dr, new)
        tiles = (new * H + tile - 1) // tile * n_seqs
        splits = max(1, min(2 * K.sm_count() // tiles, total // (2 * K.PAGE), 32))
        pool = torch.randn((n_seqs * pages_each, K.PAGE, R + dr), dtype=bf, device=dev)
        q_lat = torch.randn((H, n, R), dtype=torch.float32, device=dev) * 0.1
        q_rot = torch.randn((n, H, dr), dtype=torch.float32, device=dev)
        mixed = torch.empty((H, n, R), dtype=bf, device=dev)
        partial = None
        if splits > 1:
            partial = torch.empty(K.latent_attention_scratch_floats(n, H, R, splits), dtype=torch.float32, device=dev)
        ms_new = _time(lambda: K.latent_attention(q_lat, q_rot, pool, bt, st, mixed, H, R, dr, hd ** -0.5, n_splits=splits,
                                                  partial=partial), reps=3)
        if new < 16:
            return ms_llama, ms_new, total, splits, None
        # long portions: every head's keys and values written out for the step, under the dense decoder's kernel
        dk = hd - dr
        rows = n_seqs * pages_each * K.PAGE
        gathered = torch.empty((rows, R + dr), dtype=bf, device=dev)
        up = torch.randn((H * dk + H * hd, R), dtype=bf, device=dev) * R ** -0.5
        whole = torch.empty((n_seqs * pages_each, 2, H, K.PAGE, hd), dtype=bf, device=dev)
        qf = torch.randn((n, H * hd), dtype=bf, device=dev)

        def written_out():
            K.latent_gather(pool, bt, st, gathered, pages_each, R + dr)
            kv = torch.mm(gathered[:, :R], up.t())
            K.latent_expand(kv, gathered, whole, H, dk, dr, hd, R)
            K.attention(qf, qf.shape[1], whole, bt, st.cu_seqlens, st.slot_of_seq, st.start_pos, o, n, n_seqs, new, H, H, hd, hd ** -0.5,
                        max_kv_len=total)
        return ms_llama, _time(written_out), total, splits, ms_new

    ms_l, ms_n, total, splits, ms_lat = attention_case(1, 2048, 0)
    pairs = 2048 * 2049 / 2
    flops_l = 4.0 * H * hd * pairs
    flops_n = flops_l + 2.0 * 2048 * R * H * (hd - dr + hd)                        # the same pairs and the heads' keys and values
    out["attention_prefill_2048"] = {"llama_ms": round(ms_l, 4), "ridopel_ms": round(ms_n, 4),
                                     "ridopel_on_the_latent_ms": round(ms_lat, 4), "key_shares_on_the_latent": splits,
                                     "llama_gflop": round(flops_l / 1e9, 1), "ridopel_gflop": round(flops_n / 1e9, 1),
                                     "llama_frac_bf16": round(flops_l / (ms_l / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                                     "ridopel_frac_bf16": round(flops_n / (ms_n / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    ms_l, ms_n, total, splits, _ = attention_case(64, 1, 1087)
    bytes_l, bytes_n = 64 * G * total * 2 * hd * 2, 64 * total * (R + dr) * 2
    out["attention_decode_b64"] = {"llama_ms": round(ms_l, 4), "ridopel_ms": round(ms_n, 4), "keys_seen": total, "key_shares": splits,
                                   "llama_mb": round(bytes_l / 1e6, 1), "ridopel_mb": round(bytes_n / 1e6, 1),
                                   "llama_frac_hbm": round(bytes_l / (ms_l / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                                   "ridopel_frac_hbm": round(bytes_n / (ms_n / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    # the scans: prompts read and write rows, single tokens the states
    heads = d // hd
    for name, kind, first in (("wkv", K.DECAY_EXP_EXP, True), ("hgrn2", K.DECAY_LOWER_BOUND, False)):
        for n_seqs, new, cached in ((1, 2048, 0), (64, 1, 1087)):
            st = step(n_seqs, new, cached)
            n = st.n_tokens
            floats = K.scan_state_floats(heads, hd, hd)
            state = torch.zeros((n_seqs, 2, floats), dtype=torch.float32, device=dev)
            rows = torch.randn((n, 4 * heads * hd), dtype=torch.float32, device=dev)
            bias, extra = torch.zeros(heads * hd, dtype=torch.float32, device=dev), torch.full((heads * hd,), 0.5, dtype=torch.float32, device=dev)
            y = torch.zeros((n, heads * hd), dtype=torch.float32, device=dev)
            ms = _time(lambda: K.decay_scan(rows, 0, rows if first else None, heads * hd, rows, 2 * heads * hd, rows, 3 * heads * hd, bias,
                                            extra, y, heads, hd, hd, kind, first, st, state, 0), reps=3)
            row_bytes = 4.0 * n * heads * hd * (5 if first else 4)
            state_bytes = 2.0 * 4 * n_seqs * floats
            flops = 4.0 * n * heads * hd * hd
            out[f"{name}_scan_{n_seqs}x{new}"] = {"ms": round(ms, 4), "frac_hbm": round((row_bytes + state_bytes) / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                                                  "gflop_fp32_per_s": round(flops / (ms / 1e3) / 1e9, 1)}
    # feed-forward: a token's experts with the clamped unit beside dense products of the inner size they make together
    E, top = z["experts"], z["top"]
    each = z["inner"] // top
    gate_up = torch.randn((E, 2 * each, d), dtype=bf, device=dev) * 0.02
    down = torch.randn((E, d, each), dtype=bf, device=dev) * 0.02
    router = torch.randn((E, d), dtype=torch.float32, device=dev)
    correction = torch.randn(E, dtype=torch.float32, device=dev) * 0.05
    w1 = torch.randn((2 * top * each, d), dtype=bf, device=dev) * 0.02
    w2 = torch.randn((d, top * each), dtype=bf, device=dev) * 0.02
    for n in (2048, 64):
        h = torch.randn((n, d), dtype=bf, device=dev)
        ms_route = _time(lambda: K.moe_route(h, router, top, softmax=True, correction=correction, renormalise=True))
        ids, weights = K.moe_route(h, router, top, softmax=True, correction=correction, renormalise=True)
        ms_moe = _time(lambda: K.moe_experts(h, ids, weights, gate_up, down, weight_on_input=False, clamp_limit=7.0, clamp_alpha=1.702,
                                             out_dtype=torch.float32))
        a = torch.empty((n, top * each), dtype=bf, device=dev)

        def dense():
            gu = torch.mm(h, w1.t())
            K.swiglu(gu, a)
            return torch.mm(a, w2.t())
        ms_dense = _time(dense)
        flops = 2.0 * n * top * 3 * each * d
        wbytes = 2.0 * 3 * each * d * min(E, n * top)
        out[f"experts_{n}_tokens"] = {
            "route_ms": round(ms_route, 4), "ridopel_ms": round(ms_moe, 4), "dense_same_inner_ms": round(ms_dense, 4),
            "ridopel_frac_bf16": round(flops / (ms_moe / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
            "dense_frac_bf16": round(flops / (ms_dense / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
            "ridopel_frac_hbm": round(wbytes / (ms_moe / 1e3) / 1e9 / pk["hbm_gbs"], 4),
            "dense_frac_hbm": round(2.0 * 3 * top * each * d / (ms_dense / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    return out


def marinex_configs(z):
    """(llama, marinex) of one size.  The new design's layers take turns between grouped-query attention (Llama's head counts
    and head size, half of a head's lanes turning, capped scores) and attention over a cached latent (Llama's head count,
    half of a head's key lanes rotated, a latent of 4 heads' width, a query latent of half the width, a window of 1,024);
    every layer has 8 experts without gates in 4 groups of which a token uses 2 from the best 2 groups, whose inner sizes
    give a token the dense feed-forward's work (two matrices of 3/4 of the inner size where the dense one has three)."""
    llama = compare_configs(z)["llama"]
    hd, d, H = z["hd"], z["width"], z["heads"]
    mlp = {"kind": "moe", "expert": {"ff": 3 * z["inner"] // (2 * z["top"])},
           "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": 4, "keep": 2}}}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": H, "kv_heads": z["kv"], "dim": hd, "vdim": hd, "scale": hd ** -0.5, "softcap": 30.0,
                     "rot": {"dims": hd // 2, "base": 500000.0}}}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": H, "dim": hd // 2, "rot_dim": hd // 2, "vdim": hd, "q_rank": d // 2, "kv_rank": 4 * hd, "scale": hd ** -0.5,
                     "mask": {"size": z["window"]}, "rot": {"dims": hd // 2, "base": 500000.0}}}
    mar = {"architecture": "Marinex", "vocab": z["vocab"], "width": d, "norm": {"eps": 1e-6},
           "layers": [att if i % 2 == 0 else lat for i in range(z["layers"])]}
    return {"llama": llama, "marinex": mar}


def marinex_kernels(z, pk):
    """The new design's kernels alone, CUDA events, back to back, beside the like kernel of the dense decoder: attention with
    a number per head, a cap and a sink (one 2,048-token prompt; 64 sequences of 1,088 tokens), windowed attention over the
    latent (the same two cases), what stands between the projection and the attention, the kernel that joins a normed
    sublayer output to the stream, and the experts without gates beside dense products of the work a token gets."""
    import torch
    from types import SimpleNamespace
    from burn_lm_b200 import kernels as K
    dev, bf = "cuda", torch.bfloat16
    H, G, hd, d, W = z["heads"], z["kv"], z["hd"], z["width"], z["window"]
    R, dr = 4 * hd, hd // 2
    dk = hd - dr
    out = {}
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    frac_bf16 = lambda flops, ms: round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)
    frac_hbm = lambda nbytes, ms: round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    def step(n_seqs, new, cached):
        seq = [s for s in range(n_seqs) for _ in range(new)]
        pos = [cached + t for _ in range(n_seqs) for t in range(new)]
        return SimpleNamespace(token_seq=i32(seq), token_pos=i32(pos), slot_of_seq=i32(list(range(n_seqs))),
                               cu_seqlens=i32([new * s for s in range(n_seqs + 1)]), start_pos=i32([cached] * n_seqs),
                               n_tokens=n_seqs * new, n_seqs=n_seqs, max_q_len=new, max_kv_len=cached + new)

    temp = torch.rand(H, dtype=torch.float32, device=dev) + 0.5
    sink = torch.randn(H, dtype=torch.float32, device=dev)

    def attention_case(n_seqs, new, cached):
        total = cached + new
        pages_each = -(-total // K.PAGE)
        n = n_seqs * new
        bt = torch.arange(n_seqs * pages_each, dtype=torch.int32, device=dev).reshape(n_seqs, pages_each)
        st = step(n_seqs, new, cached)
        q = torch.randn((n, H * hd), dtype=bf, device=dev)
        pool5 = torch.randn((n_seqs * pages_each, 2, G, K.PAGE, hd), dtype=bf, device=dev)
        o = torch.empty_like(q)
        ms_llama = _time(lambda: K.attention(q, q.shape[1], pool5, bt, st.cu_seqlens, st.slot_of_seq, st.start_pos, o, n, n_seqs, new,
                                             H, G, hd, hd ** -0.5, window=0, n_splits=1, max_kv_len=total))
        pool = pool5.reshape(n_seqs * pages_each, -1)
        ms_new = _time(lambda: K.attention_sink(q, st, pool, bt, o, H, G, hd, hd, hd ** -0.5, 1 << 30, 0, sink=True, max_q_len=new,
                                                head_scale=temp, softcap=30.0))
        ms_plain = _time(lambda: K.attention_sink(q, st, pool, bt, o, H, G, hd, hd, hd ** -0.5, 1 << 30, 0, sink=True, max_q_len=new))
        # over the latent, with the window: single tokens on the latent itself, portions on keys and values written out
        tile = K.latent_attention_tile_rows(bf, H, R, dr, new)
        tiles = (new * H + tile - 1) // tile * n_seqs
        seen = min(total, W + new)
        splits = max(1, min(2 * K.sm_count() // tiles, seen // (2 * K.PAGE), 32))
        lpool = torch.randn((n_seqs * pages_each, K.PAGE, R + dr), dtype=bf, device=dev)
        if new < 16:
            q_lat = torch.randn((H, n, R), dtype=torch.float32, device=dev) * 0.1
            q_rot = torch.randn((n, H, dr), dtype=torch.float32, device=dev)
            mixed = torch.empty((H, n, R), dtype=bf, device=dev)
            partial = torch.empty(max(1, K.latent_attention_scratch_floats(n, H, R, splits)), dtype=torch.float32, device=dev)
            ms_lat = _time(lambda: K.latent_attention(q_lat, q_rot, lpool, bt, st, mixed, H, R, dr, hd ** -0.5, n_splits=splits,
                                                      partial=partial if splits > 1 else None, window=W, sink=sink), reps=5)
            return ms_llama, ms_new, ms_plain, ms_lat, total, splits
        rows = n_seqs * pages_each * K.PAGE
        gathered = torch.empty((rows, R + dr), dtype=bf, device=dev)
        up = torch.randn((H * dk + H * hd, R), dtype=bf, device=dev) * R ** -0.5
        whole = torch.empty((n_seqs * pages_each, 2, H, K.PAGE, hd), dtype=bf, device=dev)

        def written_out():
            K.latent_gather(lpool, bt, st, gathered, pages_each, R + dr, window=W)
            kv = torch.mm(gathered[:, :R], up.t())
            K.latent_expand(kv, gathered, whole, H, dk, dr, hd, R)
            K.attention_sink(q, st, whole, bt, o, H, H, hd, hd, hd ** -0.5, W, 0, sink=True, sink_logit=sink, max_q_len=new)
        return ms_llama, ms_new, ms_plain, _time(written_out), total, splits

    ms_l, ms_n, ms_p, ms_lat, total, _ = attention_case(1, 2048, 0)
    flops = 4.0 * H * hd * 2048 * 2049 / 2
    flops_w = 4.0 * H * hd * sum(min(t + 1, W) for t in range(2048)) + 2.0 * 2048 * R * H * (dk + hd)
    out["attention_prefill_2048"] = {"llama_ms": round(ms_l, 4), "marinex_ms": round(ms_n, 4), "marinex_without_cap_and_numbers_ms": round(ms_p, 4),
                                     "llama_frac_bf16": frac_bf16(flops, ms_l), "marinex_frac_bf16": frac_bf16(flops, ms_n),
                                     "marinex_latent_window_ms": round(ms_lat, 4), "marinex_latent_frac_bf16": frac_bf16(flops_w, ms_lat)}
    ms_l, ms_n, ms_p, ms_lat, total, splits = attention_case(64, 1, 1087)
    nbytes = 64 * G * total * 2 * hd * 2
    lbytes = 64 * min(total, W) * (R + dr) * 2
    out["attention_decode_b64"] = {"llama_ms": round(ms_l, 4), "marinex_ms": round(ms_n, 4), "marinex_without_cap_and_numbers_ms": round(ms_p, 4),
                                   "keys_seen": total, "llama_frac_hbm": frac_hbm(nbytes, ms_l), "marinex_frac_hbm": frac_hbm(nbytes, ms_n),
                                   "marinex_latent_window_ms": round(ms_lat, 4), "latent_keys_seen": min(total, W), "latent_key_shares": splits,
                                   "marinex_latent_frac_hbm": frac_hbm(lbytes, ms_lat)}
    # between the projection and the attention: norms over heads, the turn, unit values and the append, beside the dense
    # decoder's turn and append; and the kernel that joins a normed output to the stream beside the dense decoder's add + norm
    for n_seqs, new, cached in ((1, 2048, 0), (64, 1, 1087)):
        st = step(n_seqs, new, cached)
        n = st.n_tokens
        pages_each = -(-(cached + new) // K.PAGE)
        bt = torch.arange(n_seqs * pages_each, dtype=torch.int32, device=dev).reshape(n_seqs, pages_each)
        cols = (H + 2 * G) * hd
        proj = torch.randn((n, cols), dtype=torch.float32, device=dev)
        qkv = torch.randn((n, cols), dtype=bf, device=dev)
        pool5 = torch.empty((n_seqs * pages_each, 2, G, K.PAGE, hd), dtype=bf, device=dev)
        q = torch.empty((n, H * hd), dtype=bf, device=dev)
        wq = torch.ones(hd, dtype=torch.float32, device=dev)
        freq = torch.tensor([500000.0 ** (-2.0 * i / (hd // 2)) for i in range(hd // 4)], dtype=torch.float64, device=dev)
        freq_l = torch.tensor([500000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device=dev)
        ms_new = _time(lambda: K.head_norm_rope_append(proj, st, pool5.view(n_seqs * pages_each, -1), bt, q, H, G, hd, hd, q_weight=wq, k_weight=wq,
                                                       eps=1e-6, value_norm=True, freq=freq, rotary_dims=hd // 2))
        ms_llama = _time(lambda: K.rope_append(qkv, st.token_seq, st.token_pos, st.slot_of_seq, bt, freq_l, hd, K.PAIRS_HALVES, pool5, H, G, hd,
                                               write_cache=True, max_position=cached + new - 1))
        resid = torch.randn((n, d), dtype=torch.float32, device=dev)
        delta = torch.randn((n, d), dtype=torch.float32, device=dev)
        gamma = torch.ones(d, dtype=torch.float32, device=dev)
        x = torch.empty((n, d), dtype=bf, device=dev)
        ms_join = _time(lambda: K.sandwich_norm(resid, delta, gamma, 1.0, 1e-6, None, 0.0, x))
        ms_norm = _time(lambda: K.add_rmsnorm(resid, delta, gamma.to(bf), 1e-6, x))
        out[f"between_{n_seqs}x{new}"] = {"marinex_norms_turn_append_ms": round(ms_new, 4), "llama_turn_append_ms": round(ms_llama, 4),
                                          "marinex_frac_hbm": frac_hbm(n * cols * 6.0, ms_new), "llama_frac_hbm": frac_hbm(n * cols * 4.0, ms_llama),
                                          "marinex_join_stream_ms": round(ms_join, 4), "llama_add_norm_ms": round(ms_norm, 4),
                                          "marinex_join_frac_hbm": frac_hbm(n * d * 14.0, ms_join), "llama_add_norm_frac_hbm": frac_hbm(n * d * 14.0, ms_norm)}
    # feed-forward: a token's experts without gates beside dense products of the same work
    E, top = z["experts"], z["top"]
    each = 3 * z["inner"] // (2 * top)
    up = torch.randn((E, each, d), dtype=bf, device=dev) * 0.02
    down = torch.randn((E, d, each), dtype=bf, device=dev) * 0.02
    router = torch.randn((E, d), dtype=torch.float32, device=dev)
    correction = torch.randn(E, dtype=torch.float32, device=dev) * 0.05
    w1 = torch.randn((2 * z["inner"], d), dtype=bf, device=dev) * 0.02
    w2 = torch.randn((d, z["inner"]), dtype=bf, device=dev) * 0.02
    for n in (2048, 64):
        h = torch.randn((n, d), dtype=bf, device=dev)
        ms_route = _time(lambda: K.moe_route(h, router, top, correction=correction, n_groups=4, keep_groups=2))
        ids, weights = K.moe_route(h, router, top, correction=correction, n_groups=4, keep_groups=2)
        ms_moe = _time(lambda: K.moe_experts(h, ids, weights, up, down, weight_on_input=False, out_dtype=torch.float32, unit=K.UNIT_GELU))
        a = torch.empty((n, z["inner"]), dtype=bf, device=dev)

        def dense():
            gu = torch.mm(h, w1.t())
            K.swiglu(gu, a)
            return torch.mm(a, w2.t())
        ms_dense = _time(dense)
        flops = 2.0 * n * top * 2 * each * d
        wbytes = 2.0 * 2 * each * d * min(E, n * top)
        out[f"experts_{n}_tokens"] = {
            "route_ms": round(ms_route, 4), "marinex_ms": round(ms_moe, 4), "dense_same_work_ms": round(ms_dense, 4),
            "marinex_frac_bf16": frac_bf16(flops, ms_moe), "dense_frac_bf16": frac_bf16(flops, ms_dense),
            "marinex_frac_hbm": frac_hbm(wbytes, ms_moe), "dense_frac_hbm": frac_hbm(2.0 * 3 * z["inner"] * d, ms_dense)}
    return out


def run_compare(args):
    """One JSON line per size and model: prefill of one 2,048-token prompt and decode at batch 8 and 64 after 512-token
    prompts, for the dense Llama decoder and the named design (Fobilorn with dense feed-forwards and with experts, Nufolix,
    Ridopel) at equal layer sizes with random weights; then a line with the kernels alone."""
    import torch
    import burn_lm_b200 as blm
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: burn-lm_b200 has no CPU path"}))
        return 1
    pk = peaks()
    for size, z in COMPARE_SIZES.items():
        if args.size and size != args.size:
            continue
        if args.compare in ("ridopel", "marinex"):
            z = dict(z, experts=8)          # 8 experts of half the dense inner size each: four times the dense layer's weights
        configs = {"nufolix": nufolix_configs, "ridopel": ridopel_configs, "marinex": marinex_configs}.get(args.compare, compare_configs)(z)
        for name, cfg in configs.items():
            vocab = z["vocab"]
            lm = blm.load_random(cfg, seed=0, dtype="bfloat16", max_seq_len=4096, max_batch=64, max_tokens=64 * 1024)
            engine = lm.engine
            line = {"compare": size, "model": name, "layers": z["layers"]}
            ms = time_prefill(engine, make_prompts(("equal", 2048), 1, vocab, seed=99), reps=3)
            line["prefill_2048_ms"] = round(ms, 3)
            line["prefill_tokens_per_s"] = round(2048 / (ms / 1e3), 1)
            for b in (8, 64):
                r = device_decode(engine, make_prompts(("equal", 512), b, vocab, seed=b), args.steps or 64, 3)
                line[f"decode_b{b}_ms_per_step"] = round(r["ms_per_step"], 4)
                line[f"decode_b{b}_tokens_per_s"] = round(r["tokens_per_s"], 1)
                line[f"decode_b{b}_launches_per_step"] = r["graph"].launches_per_step
            print(json.dumps(line), flush=True)
            del lm, engine
            torch.cuda.empty_cache()
        alone = {"nufolix": nufolix_kernels, "ridopel": ridopel_kernels, "marinex": marinex_kernels}.get(args.compare, compare_kernels)(z, pk)
        print(json.dumps({"compare": size, "kernels": alone, "peaks": pk["source"]}), flush=True)
    return 0


def run_ours(args):
    import torch
    import burn_lm_b200 as blm
    from burn_lm_b200 import kernels

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: burn-lm_b200 has no CPU path"}))
        return 1
    pk = peaks()
    w = WORKLOADS[args.config]
    cfg = blm.preset(w["preset"])
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or full_layers
    context = w["context"]
    batch = args.batch or w["batch"]
    steps, warmup = args.steps or w["steps"], max(args.warmup, 3)
    vocab = cfg["vocab_size"]
    most = max((batch,) + tuple(w["points"]))
    lm = blm.load_random(cfg, seed=0, dtype="bfloat16", max_seq_len=context, max_batch=most, max_tokens=most * context)
    engine = lm.engine
    prompts = make_prompts(w["prompts"], batch, vocab, seed=batch)
    lengths = [len(p) for p in prompts]
    if max(lengths) + steps + 1 > context:
        print(f"--steps {steps} does not fit the context of {context} after a {max(lengths)}-token prompt")
        return 2
    one_prompt = make_prompts(("equal", w["prefill"][1]), 1, vocab, seed=99) if w["prefill"][0] == "one" else None

    if args.only == "decode":      # a short run of one workload, for profilers
        r = device_decode(engine, prompts, steps, warmup, temperature=w["temperature"])
        print(json.dumps({"only": "decode", "batch": batch, "ms_per_step": round(r["ms_per_step"], 4)}))
        return 0
    if args.only == "prefill":
        if args.prompt_tokens:
            one_prompt = make_prompts(("equal", args.prompt_tokens), 1, vocab, seed=99)
        ms = time_prefill(engine, one_prompt or prompts, reps=1)
        print(json.dumps({"only": "prefill", "tokens": sum(len(p) for p in (one_prompt or prompts)), "ms": round(ms, 3)}))
        return 0
    if args.only == "sweep":
        sweep(engine, cfg, pk)
        return 0
    main = device_decode(engine, prompts, steps, warmup, sample_clocks=True, temperature=w["temperature"])
    points = {}
    for b in w["points"]:
        r = device_decode(engine, make_prompts(w["prompts"], b, vocab, seed=b), min(steps, 128), warmup)
        points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)

    # end to end through the Python entry point: host tokens in and out every step
    options = dict(ignore_stop=True, temperature=w["temperature"], seed=1234)
    lm.generate(prompts, sample_len=warmup + 2, **options)                  # warm-up (captures the graph)
    out = lm.generate(prompts, sample_len=steps + 1, **options)             # steps decode steps after the prefill
    st = out.stats
    e2e_value = batch * st.decode_steps / st.decode_seconds
    h2d = main["graph"].bytes_in_per_step() + (8 * batch if w["temperature"] > 0 else 0)      # + the draws' counters

    pre_prompts = one_prompt or prompts
    prefill_ms = time_prefill(engine, pre_prompts, reps=5 if one_prompt else 3)
    pre_tokens = sum(len(p) for p in pre_prompts)
    flops = prefill_flops(cfg, [len(p) for p in pre_prompts])

    live = sum(lengths) + batch * steps / 2.0
    achieved = decode_step_bytes(cfg, live) / (main["ms_per_step"] / 1e3) / 1e9
    rs = cfg["rope_scaling"]
    plen = w["prompts"]
    line = {
        "metric": f"decode tokens/s, {w['model'].replace('-shape-random', '')} shape, bf16, batch {batch} "
                  f"({'%d-token prompts' % plen[1] if plen[0] == 'equal' else 'prompts of %d to %d tokens' % plen[1:]}, context {context})",
        "value": round(main["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": w["model"], "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
            "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"], "vocab_size": vocab,
            "tied_head": bool(cfg["tie_word_embeddings"]), "rope": f"theta {cfg['rope_theta']:g}, llama3 x{rs['factor']:g}",
            "global_batch": batch, "seq_len": context,
            "prompt_len": plen[1] if plen[0] == "equal" else f"uniform {plen[1]}..{plen[2]} (mean {sum(lengths) // batch})",
            "parallelism": "single-gpu", "weights": "random N(0,0.02) bf16",
            "l2": f"inputs ({weight_bytes(cfg) / 1e9:.2f} GB of weights) exceed the 126 MB L2; no flush",
            "sampling": "greedy" if w["temperature"] == 0 else f"temperature {w['temperature']}, top-p 0.9, host-launched steps",
            "peaks": pk["source"],
        },
        "clocks": main["clocks"],
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * batch, "ms_per_step": round(1e3 * st.decode_seconds / st.decode_steps, 4)},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(pre_tokens / (prefill_ms / 1e3), 1), "tokens": pre_tokens,
                    "ms": round(prefill_ms, 3), "frac": round(flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                    "peak_tflops": pk["bf16_tflops"], "prompts": len(pre_prompts)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "impl": "ours",
        "kernel_modules": kernels.loaded_modules(),
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="decode steps to time (default: the workload's: 256, 128, 256)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="1b", choices=sorted(WORKLOADS),
                    help="the workload: 1b (the headline, default), 3b or 8b")
    ap.add_argument("--batch", type=int, default=0, help="sequences decoded together (default: the workload's)")
    ap.add_argument("--only", default=None, choices=["decode", "prefill", "sweep"],
                    help="run one workload briefly (for profilers), or a sweep over batch sizes and context lengths")
    ap.add_argument("--prompt-tokens", type=int, default=0, help="with --only prefill: one prompt of this many tokens instead of the workload's")
    ap.add_argument("--compare", default=None, choices=["fobilorn", "nufolix", "ridopel", "marinex"],
                    help="instead of the workload: the named design beside the dense Llama decoder at equal layer sizes "
                         "(prefill and decode throughput, then its kernels alone), one JSON line each")
    ap.add_argument("--size", default=None, choices=sorted(COMPARE_SIZES), help="with --compare: one of the sizes only")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (both numbers are named in config)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "tracel-ai/burn-lm is a Rust workspace: no cargo/rustc here, its `burn` dependency is a git "
                          "branch that cannot be fetched offline, and pip finds neither setup.py nor pyproject.toml"}))
        return 0
    if args.gpus != 1:
        print(f"burn-lm_b200 generates on ONE GPU; --gpus {args.gpus} is not built (no multi-GPU path)")
        return 2
    if args.compare:
        return run_compare(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
