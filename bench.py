#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Hunyuan-1.8B layer
sizes with random weights (bfloat16), printed as ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192]
                    [--layers L] [--impl reference]

A step is one decode step of the whole batch.  ``value`` is decoded tokens per
second with the K steps timed on the device (CUDA events); ``e2e`` is the same
through the Python entry point (``LLMEngine.step``: host token ids in, sampled
token ids out, every step).  The cache of every request is first filled to the
context length with random keys and values, so the step reads what a real
request of that length would read; inputs (weights and cache, far more than the
126 MB of L2) are larger than L2, so nothing is flushed between steps.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = {
    "architectures": ["HunYuanDenseV1ForCausalLM"], "model_type": "hunyuan_v1_dense",
    "vocab_size": 120818, "hidden_size": 2048, "intermediate_size": 6144, "num_hidden_layers": 32,
    "num_attention_heads": 16, "num_key_value_heads": 4, "head_dim": 128, "hidden_act": "silu",
    "max_position_embeddings": 32768, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "rope_scaling": {"alpha": 1000.0, "type": "dynamic"}, "use_qk_norm": True,
    "tie_word_embeddings": True, "attention_bias": False,
}
# the other layer sizes of the baseline's configurations, for --sizes (the default run keeps 1.8B)
OTHER_SIZES = {
    "4b": {"hidden_size": 3072, "intermediate_size": 8192, "num_attention_heads": 32, "num_key_value_heads": 8},
    "7b": {"hidden_size": 4096, "intermediate_size": 14336, "num_attention_heads": 32, "num_key_value_heads": 8,
           "vocab_size": 128167, "tie_word_embeddings": False},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in d.items() if k in out and v})
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(int(float(r[0]))); mx = max(mx, int(float(r[1])))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def param_bytes(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * i + 2 * h + 2 * cfg["head_dim"]
    head = v * h if cfg["tie_word_embeddings"] else 2 * v * h     # tied: the table is read once as the head
    return 2 * (layers * per_layer + head), 2 * layers * per_layer


def decode_bytes(cfg, layers, batch, context):
    weights, _ = param_bytes(cfg, layers)
    kv_per_token = 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    return weights + batch * context * kv_per_token


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * i
    gemm = 2 * tokens * layers * per_layer + 2 * v * h            # the head runs on the last row only
    attn = layers * 4 * q * tokens * tokens / 2                    # causal: half of QK^T and PV
    return gemm + attn


def build_model(cfg, engine_opts, seed=0, dtype="bf16"):
    """Random weights drawn and rounded to bfloat16; ``dtype`` "fp32" loads the
    same rounded values into the true 32-bit path."""
    import torch
    from crane_b200.generation import ModelForCausalLM
    from crane_b200.weights.random_init import model_manifest_for, random_tensors
    tensors = random_tensors(model_manifest_for(cfg), seed, torch.bfloat16, "cuda:0")
    return ModelForCausalLM.from_tensors(cfg, tensors, dtype, **engine_opts)


def fill_cache(model, batch, context, seed=1):
    """Admits `batch` requests and gives each `context` cached positions of
    random keys and values, without running a prefill."""
    import torch
    g = torch.Generator(device="cuda:0"); g.manual_seed(seed)
    for top in model.runner.pools.layers:
        for lc in (top,) + tuple(top.parts):      # a mixer that keeps pages and a state has them as parts
            if lc.k is not None:
                lc.k.normal_(0.0, 1.0, generator=g)
                lc.v.normal_(0.0, 1.0, generator=g)
    ids = list(range(1000, 1000 + batch))
    for rid in ids:
        model.runner.table.admit(rid)
        model.runner.table.extend(rid, context)
    return ids


def check_decode_logits(model, cfg, ids, context, vocab, page):
    """One decode step of the live requests `ids` (cache filled to `context`) on
    the serving path against the same step on the engine's true 32-bit path (no
    tensor cores, plain kernels): same weights, same cached keys and values, same
    tokens.  Outside every timed region.  Returns the largest difference relative
    to the largest logit, and how many rows pick the same token."""
    import numpy as np
    import torch
    from crane_b200.engine import StepEntry
    batch = len(ids)
    ref = build_model(cfg, dict(page_size=page, num_pages=batch * (context // page + 2) + 8,
                                max_concurrent=max(batch, 1), max_seq_len=context + 1024,
                                max_batched_tokens=max(batch, 64), use_cuda_graphs=False), dtype="fp32")
    r16, r32 = model.runner, ref.runner
    blocks = (context + page - 1) // page
    for rid in ids:
        r32.table.admit(rid)
        r32.table.extend(rid, context)
    pages = {}                                    # per layer group: (pages here, pages there) of all requests
    for lc16, lc32 in zip(r16.pools.layers, r32.pools.layers):
        if lc16.k is None:
            continue
        if lc16.group not in pages:
            src = np.concatenate([r16.table.block_table(rid, lc16.group, blocks) for rid in ids])
            dst = np.concatenate([r32.table.block_table(rid, lc32.group, blocks) for rid in ids])
            pages[lc16.group] = (torch.from_numpy(src).to("cuda:0", torch.long),
                                 torch.from_numpy(dst).to("cuda:0", torch.long))
        src, dst = pages[lc16.group]
        lc32.k[dst] = lc16.k[src].float()
        lc32.v[dst] = lc16.v[src].float()
    toks = [(5 * i + 2) % vocab for i in range(batch)]
    entries = [StepEntry(r, [t], [0]) for r, t in zip(ids, toks)]
    got = r16.step(entries).float().clone()
    want = r32.step(entries).float()
    r16.rt.check_errors()
    r32.rt.check_errors()
    err = float((got - want).abs().max() / want.abs().max())
    same = int((got.argmax(dim=1) == want.argmax(dim=1)).sum())
    del ref, r32, want
    torch.cuda.empty_cache()
    return err, same


def time_decode(model, ids, steps, warmup, vocab, mark=False):
    """K decode steps of the whole batch, timed on the device.  `mark`: the
    timed steps lie between cudaProfilerStart and cudaProfilerStop."""
    import torch
    from crane_b200.engine import StepEntry
    from crane_b200.sampling import SamplingParams
    runner, sampler = model.runner, model.engine.sampler
    greedy = [SamplingParams() for _ in ids]
    toks = [(7 * i + 3) % vocab for i in range(len(ids))]

    def one():
        logits = runner.step([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)])
        return sampler.sample_device(logits, greedy)
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    launches0 = runner.rt.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if mark:
        torch.cuda.profiler.start()
    start.record()
    for _ in range(steps):
        one()
    stop.record()
    torch.cuda.synchronize()
    if mark:
        torch.cuda.profiler.stop()
    runner.rt.check_errors()
    return start.elapsed_time(stop) / steps, (runner.rt.launches - launches0) // steps


def time_decode_e2e(model, batch, context, steps, warmup, vocab):
    """The same through the entry point: requests added with host token ids,
    every step plans on the host, copies its inputs from pinned memory and
    reads the sampled ids back."""
    import torch
    eng = model.engine
    runner = model.runner
    ids = []
    for b in range(batch):
        rid = eng.add_request([(11 * b + 5) % vocab], None, max_new_tokens=steps + warmup + 8,
                              eos_token_ids=[])
        ids.append(rid)
    eng.step()                                    # the one-token prompts
    for rid in ids:                               # then stretch every request to the context length
        runner.table.extend(rid, context - runner.table.length(rid))
    for _ in range(warmup):
        eng.step()
    eng.flush()                                   # nothing in flight when the clock starts
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = 0
    for _ in range(steps):
        n += len(eng.step())
    n += len(eng.flush())                         # the last step's tokens are read inside the clock
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for rid in ids:
        eng.cancel(rid)
    eng.finished.clear()
    m = runner.meta
    return n / dt, m.total * 4, batch * 4


def time_prefill(model, tokens, vocab, reps=3, mark=False):
    """`mark`: the last repetition lies between cudaProfilerStart and cudaProfilerStop."""
    import torch
    from crane_b200.engine import StepEntry
    runner = model.runner
    prompt = [(13 * i + 1) % vocab for i in range(tokens)]
    times = []
    for r in range(reps + 1):
        rid = 5000 + r
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if mark and r == reps:
            torch.cuda.profiler.start()
        start.record()
        runner.step([StepEntry(rid, prompt, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        if mark and r == reps:
            torch.cuda.profiler.stop()
        runner.end(rid)
        if r > 0:                                 # the first run warms up
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]                 # the median


def time_prefill_chunked(model, tokens, chunk, vocab, reps=2):
    """One prompt of `tokens` tokens in portions of `chunk`, one step each, as the
    scheduler cuts a long prompt under its token budget; the whole prompt timed."""
    import torch
    from crane_b200.engine import StepEntry
    runner = model.runner
    prompt = [(13 * i + 1) % vocab for i in range(tokens)]
    times = []
    for r in range(reps + 1):
        rid = 7000 + r
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for a in range(0, tokens, chunk):
            b = min(tokens, a + chunk)
            runner.step([StepEntry(rid, prompt[a:b], [b - a - 1] if b == tokens else [])])
        stop.record()
        torch.cuda.synchronize()
        runner.end(rid)
        if r > 0:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def serve_workload(model, cfg, args, pk):
    """The serving mix: `--requests` requests with seeded prompt lengths between
    `--prompt-min` and `--prompt-max` and `--new-tokens` generated tokens each, all
    added at once, through the engine's scheduler (continuous batching, prompt
    portions beside decoded tokens under the token budget).  Reports the running
    averages the reference's engine keeps (crane-serve/src/engine/stats.rs:41-54:
    prompt tokens over the time of steps that held prompt tokens, decoded tokens
    over the time of pure decode steps), the whole job's tokens per second, the
    steps' wall-time percentiles and the share of mixed steps."""
    import numpy as np
    import torch
    from crane_b200.sampling import SamplingParams
    eng = model.engine
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(args.seed)
    lengths = rng.integers(args.prompt_min, args.prompt_max + 1, args.requests)
    prompts = [rng.integers(0, vocab, int(n)).tolist() for n in lengths]
    # warm-up: a short mix that touches the step shapes' kernels
    for p in prompts[:4]:
        eng.add_request(p[:300], SamplingParams(temperature=0.7, seed=1), 8, [])
    eng.run_until_done()
    for k in eng.timers:
        eng.timers[k] = 0 if isinstance(eng.timers[k], int) else 0.0
    launches0 = model.runner.rt.launches
    for i, p in enumerate(prompts):
        eng.add_request(p, SamplingParams(temperature=0.7, seed=100 + i), args.new_tokens, [])
    kinds, times = [], []
    torch.cuda.synchronize()
    t_all = time.perf_counter()
    with ClockSampler() as clocks:
        while eng.has_work():
            t0 = time.perf_counter()
            eng.step()
            times.append(time.perf_counter() - t0)
            kinds.append(eng.last_step_kind)
        torch.cuda.synchronize()
    wall = time.perf_counter() - t_all
    model.runner.rt.check_errors()
    done = eng.finished
    generated = sum(len(o.generated) for o in done.values())
    prompt_tokens = int(lengths.sum())
    st = eng.stats()
    ms = np.asarray(times) * 1e3
    by_kind = {k: ms[[i for i, x in enumerate(kinds) if x == k]] for k in ("decode", "prefill", "mixed")}
    pct = lambda a: {"n": int(a.size), "p50": round(float(np.percentile(a, 50)), 3),
                     "p90": round(float(np.percentile(a, 90)), 3),
                     "p99": round(float(np.percentile(a, 99)), 3)} if a.size else {"n": 0}
    return {
        "workload": "serve", "requests": args.requests, "prompt_tokens": prompt_tokens,
        "prompt_len_min": int(lengths.min()), "prompt_len_max": int(lengths.max()),
        "generated_tokens": generated, "wall_s": round(wall, 3),
        "total_tokens_per_s": round((prompt_tokens + generated) / wall, 1),
        "generated_tokens_per_s": round(generated / wall, 1),
        "avg_prefill_tokens_per_sec": round(st["avg_prefill_tokens_per_sec"], 1),
        "avg_decode_tokens_per_sec": round(st["avg_decode_tokens_per_sec"], 1),
        "steps": len(times), "mixed_step_share": round(kinds.count("mixed") / max(1, len(kinds)), 3),
        "step_ms": {k: pct(v) for k, v in by_kind.items()},
        "preemptions": st.get("preemptions", 0), "gpu_launches": model.runner.rt.launches - launches0,
        "graph_replays": model.runner.graph_replays, "clocks": clocks.summary(),
    }


def mixed_step_workload(model, cfg, args):
    """What a step of `--batch` decoded tokens at `--context` beside one prompt
    portion of `--portion` tokens costs, against a pure decode step plus the
    portion alone, with the single tokens on the split-KV decode kernel (the
    engine's choice at such contexts) and with everything on the prefill kernel."""
    import torch
    from crane_b200.engine import StepEntry
    runner = model.runner
    vocab = cfg["vocab_size"]
    ids = fill_cache(model, args.batch, args.context)
    toks = [(7 * i + 3) % vocab for i in range(len(ids))]
    portion = [(13 * i + 1) % vocab for i in range(args.portion)]
    nxt = [9000]

    def timed(make_entries, reps, after=None):
        out = []
        for r in range(reps + 2):
            entries = make_entries()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            runner.step(entries)
            b.record()
            torch.cuda.synchronize()
            if after:
                after(entries)
            if r >= 2:
                out.append(a.elapsed_time(b))
        out.sort()
        return out[len(out) // 2]

    def decode_entries():
        return [StepEntry(r, [t], [0]) for r, t in zip(ids, toks)]

    def portion_entry():
        nxt[0] += 1
        return StepEntry(nxt[0], portion, [len(portion) - 1])

    def end_portion(entries):
        runner.end(entries[-1].request_id)
    reps = max(3, args.steps // 8)
    res = {"workload": "mixed-step", "batch": args.batch, "context": args.context, "portion": args.portion}
    res["decode_ms"] = round(timed(decode_entries, reps), 4)
    res["portion_ms"] = round(timed(lambda: [portion_entry()], reps, end_portion), 4)
    res["mixed_ms"] = round(timed(lambda: decode_entries() + [portion_entry()], reps, end_portion), 4)
    keep = runner.cfg.mixed_decode_min_keys
    runner.cfg.mixed_decode_min_keys = 1 << 60
    res["mixed_prefill_kernel_only_ms"] = round(timed(lambda: decode_entries() + [portion_entry()], reps, end_portion), 4)
    runner.cfg.mixed_decode_min_keys = keep
    res["mixed_over_sum"] = round(res["mixed_ms"] / (res["decode_ms"] + res["portion_ms"]), 3)
    runner.rt.check_errors()
    return res


def radorax_config(like, layers):
    """A Radorax model with the width, head count, layer count and vocabulary of the Hunyuan
    configuration `like` and about its number of parameters per layer: heads of 128 + 32 (rotated)
    query/key and 128 value elements, a latent of 192, feed-forward 1.5 x the other's (two matrices
    instead of three), every layer with a cache of its own."""
    h, heads = like["hidden_size"], like["num_attention_heads"]
    mixer = {"heads": heads, "dim": 128, "rot_dim": 32, "vdim": 128, "kv_rank": 192, "scale": 160 ** -0.5,
             "rot": {"dims": 32, "base": 10000.0,
                     "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    layer = {"type": "latent_attention", "mixer": mixer,
             "mlp": {"kind": "dense", "ff": like["intermediate_size"] * 3 // 2}}
    return {"architecture": "Radorax", "vocab": like["vocab_size"], "width": h, "norm": {"eps": 1e-5},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 7919}},
            "layers": [layer] * layers}


def _median_ms(fn, reps=9, flush=None):
    import torch
    for _ in range(3):
        fn()
    out = []
    for _ in range(reps):
        if flush is not None:
            flush.add_(1.0)                      # 512 MB written: L2 holds none of the kernel's inputs
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    out.sort()
    return out[len(out) // 2]


def radorax_kernel_table(rcfg, hcfg, pk, tokens, batch, context):
    """Every kernel that only Radorax runs beside the kernel of Hunyuan Dense that does the like
    job, each alone on synthetic operands of the two models' layer sizes (L2 flushed between
    repetitions), with the fraction of its roofline: algorithmic bytes over the measured copy
    rate, or FLOPs over the measured bf16 rate, whichever takes longer."""
    import numpy as np
    import torch
    from crane_b200.kernels import get_kernels
    from crane_b200.parts.latent_attention import latent_attention_kernel
    K = get_kernels([hcfg["head_dim"]])
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    W, H = rcfg["width"], rcfg["layers"][0]["mixer"]["heads"]
    m = rcfg["layers"][0]["mixer"]
    dim, rot, vd, r = m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    ffr, ffh = rcfg["layers"][0]["mlp"]["ff"], hcfg["intermediate_size"]
    d, nq, nkv = hcfg["head_dim"], hcfg["num_attention_heads"], hcfg["num_key_value_heads"]
    hbm, peak = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = []

    def add(name, like, ms, nbytes, flops, like_ms, like_bytes, like_flops):
        def frac(ms_, b, f):
            return round(max(b / hbm, f / peak) / (ms_ * 1e-3), 3)
        rows.append({"kernel": name, "ms": round(ms, 4), "frac": frac(ms, nbytes, flops), "like": like,
                     "like_ms": round(like_ms, 4) if like_ms else None,
                     "like_frac": frac(like_ms, like_bytes, like_flops) if like_ms else None})

    T = tokens
    rnd = lambda *shape, dt=bf: torch.randn(*shape, device=dev, dtype=torch.float32).to(dt)
    # the additions and norms between layers, at mid depth (16 earlier results in the average)
    n_hist = min(17, len(rcfg["layers"]) + 1)
    x, hist = rnd(T, W, dt=torch.float32), rnd(n_hist, T, W, dt=torch.float32)
    a, f, o1, o2 = rnd(T, W), rnd(T, W), torch.empty(T, W, device=dev, dtype=bf), torch.empty(T, W, device=dev, dtype=bf)
    w = [rnd(W, dt=torch.float32) for _ in range(4)]
    dwa = rnd(n_hist, dt=torch.float32)
    t_r = _median_ms(lambda: K.combine_layernorm(x, hist, n_hist, a, f, dwa, None, w[0], w[1], o1, w[2], w[3], o2, 1e-5),
                     flush=flush)
    t_h = _median_ms(lambda: K.add_rmsnorm(x, a, w[0], 1e-5, o1), flush=flush)
    add(f"combine_layernorm (average of {n_hist})", "add_rmsnorm", t_r, T * W * (4 * (n_hist + 2) + 2 + 2 + 4), 0,
        t_h, T * W * (4 + 4 + 2 + 2), 0)
    del hist
    # activation
    up, act = rnd(T, ffr), torch.empty(T, ffr, device=dev, dtype=bf)
    pq = torch.tensor([0.3, -0.2], device=dev)
    gu, act_h = rnd(T, 2 * ffh), torch.empty(T, ffh, device=dev, dtype=bf)
    t_r = _median_ms(lambda: K.xielu(up, act, pq), flush=flush)
    t_h = _median_ms(lambda: K.silu_mul(gu, act_h, False), flush=flush)
    add("xielu", "silu_mul", t_r, T * ffr * 4, 0, t_h, T * ffh * 6, 0)
    del up, act, gu, act_h
    # attention: one prompt of T tokens, and `batch` decoded tokens at `context`
    ps = 64
    for kind, n_req, q_len, kv in (("prefill", 1, T, T), ("decode", batch, 1, context)):
        blocks = -(-kv // ps)
        pages = n_req * blocks
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(n_req, blocks)
        cu = np.arange(n_req + 1, dtype=np.int32) * q_len
        kvl = np.full(n_req, kv, dtype=np.int32)
        cu_d, kv_d = torch.from_numpy(cu).to(dev), torch.from_numpy(kvl).to(dev)
        n = n_req * q_len
        pos = torch.from_numpy(np.concatenate([np.arange(kv - q_len, kv, dtype=np.int32)] * n_req)).to(dev)
        ent = torch.from_numpy(np.repeat(np.arange(n_req, dtype=np.int32), q_len)).to(dev)
        pool = rnd(pages, 1, ps, r + rot)
        q_abs, o_lat = rnd(n, H * (r + rot)), torch.empty(n, H * r, device=dev, dtype=bf)
        t_r = _median_ms(lambda: latent_attention_kernel(K, q_abs, o_lat, pool, pos, ent, cu_d, kv_d, cu, kvl, table,
                                                         ps, H, r, rot, 0.08, err, False), flush=flush)
        k_pool, v_pool = rnd(pages, nkv, ps, d), rnd(pages, nkv, ps, d)
        qh, oh = rnd(n, nq * d), torch.empty(n, nq * d, device=dev, dtype=bf)
        if kind == "prefill":
            tiles = -(-T // 128)
            t_h = _median_ms(lambda: K.prefill_attention_tc(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, tiles, nq,
                                                            nkv, d, 0, d ** -0.5, err), flush=flush)
            pairs = T * T / 2
            add("latent_attention_mma (prefill)", "prefill_attn_tc", t_r, 0, pairs * H * 2 * (2 * r + rot),
                t_h, 0, pairs * nq * 4 * d)
            # and beside the engine's own warp-level flash attention (the kernel of the same kind)
            tiles64 = -(-T // 64)
            t_w = _median_ms(lambda: K.paged_prefill_attention(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, tiles64,
                                                               nq, nkv, d, 0, d ** -0.5, err), flush=flush)
            add("latent_attention_mma (prefill)", "paged_prefill_attn (warp-level MMA)", t_r, 0,
                pairs * H * 2 * (2 * r + rot), t_w, 0, pairs * nq * 4 * d)
        else:
            splits = K.decode_splits(n_req, nkv, 148, 64, max_keys=kv)
            po = torch.empty(n_req * nq * splits, d, device=dev)
            pml = torch.empty(n_req * nq * splits, 2, device=dev)
            t_h = _median_ms(lambda: K.paged_decode_attention(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, nq, nkv,
                                                              d, 0, d ** -0.5, splits, po, pml, err), flush=flush)
            add("latent_attention_mma (decode)", "paged_decode_attn", t_r, n_req * kv * (r + rot) * 2, 0,
                t_h, n_req * kv * nkv * d * 2 * 2, 0)
        # the two per-head products around the attention (no counterpart: Hunyuan's heads come out of its q/k/v product)
        if kind == "prefill":
            cols = H * (dim + rot) + H * vd + r + rot
            proj = rnd(n, cols)
            uk, uv_t = rnd(H, dim, r), rnd(H, r, vd)
            o = torch.empty(n, H * vd, device=dev, dtype=bf)
            t_q = _median_ms(lambda: K.head_linear(proj, cols, 0, dim + rot, uk, dim, r, q_abs, H * (r + rot), r + rot, H),
                             flush=flush)
            t_v = _median_ms(lambda: K.head_linear(o_lat, H * r, 0, r, uv_t, r, vd, o, H * vd, vd, H, gate=proj,
                                                   g_cols=cols, g_off=H * (dim + rot)), flush=flush)
            add("head_linear (query into the latent space)", None, t_q, n * H * (dim + r) * 2, 2.0 * n * H * dim * r, 0, 0, 0)
            add("head_linear (latent output to values, gate)", None, t_v, n * H * (r + 2 * vd) * 2, 2.0 * n * H * r * vd, 0, 0, 0)
            del proj
        del pool, k_pool, v_pool
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    return rows


def radorax_workload(args, pk):
    """Prefill and decode throughput of Radorax at the layer sizes of --sizes beside Hunyuan Dense
    (the engine's closest model) at the same width, heads, layers and vocabulary, random weights,
    and the kernels of the two side by side."""
    import gc
    import torch
    hcfg = dict(MODEL)
    hcfg.update(OTHER_SIZES.get(args.sizes, {}))
    layers = args.layers or hcfg["num_hidden_layers"]
    hcfg["num_hidden_layers"] = layers
    hcfg["max_position_embeddings"] = max(hcfg["max_position_embeddings"], args.context + 2048)
    rcfg = radorax_config(hcfg, layers)
    page, pt = 64, args.prefill_tokens
    out = {"workload": "radorax", "sizes": args.sizes, "layers": layers, "batch": args.batch,
           "context": args.context, "prefill_tokens": pt, "dtype": "bf16", "data": "synthetic", "models": {}}
    for name, cfg, vocab in (("radorax", rcfg, rcfg["vocab"]), ("hunyuan_dense", hcfg, hcfg["vocab_size"])):
        opts = dict(page_size=page, num_pages=(args.batch * (args.context + args.steps + args.warmup + 64) + pt) // page + 64,
                    max_concurrent=max(64, args.batch), max_seq_len=max(args.context, pt) + 1024,
                    max_batched_tokens=max(2048, pt), chunk_size=max(2048, pt))
        model = build_model(cfg, opts)
        pms = time_prefill(model, pt, vocab, reps=3)
        ids = fill_cache(model, args.batch, args.context)
        dms, launches = time_decode(model, ids, args.steps, args.warmup, vocab)
        weights = sum(t.numel() * t.element_size() for t in _model_tensors(model))
        out["models"][name] = {"prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(pt * 1000.0 / pms, 1),
                               "decode_ms_per_step": round(dms, 4),
                               "decode_tokens_per_s": round(args.batch * 1000.0 / dms, 1),
                               "launches_per_decode_step": launches, "weight_bytes": weights}
        del model
        gc.collect()
        torch.cuda.empty_cache()
    out["kernels"] = radorax_kernel_table(rcfg, hcfg, pk, pt, args.batch, args.context)
    out["peaks"] = pk
    return out


def vodelix_config(like, layers):
    """A Vodelix model with the width, layer count and vocabulary of the Hunyuan configuration `like`:
    of every four layers one attends (the other's head counts, heads of 128) and three run the delta
    rule (heads of 64 across the width); every other layer has a dense feed-forward of the other's
    inner size, the rest eight experts of a quarter of it, two chosen, and a shared one; layers 1 and
    2 run twice; a token input of 64 per layer."""
    h, heads, kv = like["hidden_size"], like["num_attention_heads"], like["num_key_value_heads"]
    ff = like["intermediate_size"]
    att = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5}
    delta = {"heads": h // 64, "dim": 64, "decay_rank": 64}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": ff // 4}, "shared": {"ff": ff // 4}}
    ls = [{"type": "attention" if i % 4 == 1 else "general_delta", "mixer": att if i % 4 == 1 else delta,
           "mlp": dense if i % 2 == 0 else moe} for i in range(layers)]
    cfg = {"architecture": "Vodelix", "vocab": like["vocab_size"], "width": h, "norm": {"eps": 1e-5},
           "token_side": {"dim": 64}, "layers": ls}
    if layers >= 3:
        cfg["loop"] = {"start": 1, "stop": 3, "times": 2}
    return cfg


def vodelix_kernel_table(vcfg, hcfg, pk, tokens, batch, context):
    """Every kernel that only Vodelix runs beside the kernel of Hunyuan Dense that does the like job,
    each alone on synthetic operands of the two models' layer sizes (L2 flushed between repetitions),
    with the fraction of its roofline: algorithmic bytes over the measured copy rate, or FLOPs over
    the measured bf16 rate, whichever takes longer."""
    import math
    import numpy as np
    import torch
    from crane_b200.kernels import get_kernels
    K = get_kernels([hcfg["head_dim"]])
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    W = vcfg["width"]
    dl = next(l["mixer"] for l in vcfg["layers"] if l["type"] == "general_delta")
    H, dd, R = dl["heads"], dl["dim"], dl["decay_rank"]
    ffh = hcfg["intermediate_size"]
    d, nq, nkv = hcfg["head_dim"], hcfg["num_attention_heads"], hcfg["num_key_value_heads"]
    hbm, peak = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = []

    def add(name, like, ms, nbytes, flops, like_ms, like_bytes, like_flops):
        def frac(ms_, b, f):
            return round(max(b / hbm, f / peak) / (ms_ * 1e-3), 4)
        rows.append({"kernel": name, "ms": round(ms, 4), "frac": frac(ms, nbytes, flops), "like": like,
                     "like_ms": round(like_ms, 4) if like_ms else None,
                     "like_frac": frac(like_ms, like_bytes, like_flops) if like_ms else None})

    T = tokens
    rnd = lambda *shape, dt=bf: torch.randn(*shape, device=dev, dtype=torch.float32).to(dt)
    # a normed result joins the stream and the next norm reads it
    x, a = rnd(T, W, dt=torch.float32), rnd(T, W)
    o1 = torch.empty(T, W, device=dev, dtype=bf)
    w = [rnd(W, dt=torch.float32) for _ in range(2)]
    t_v = _median_ms(lambda: K.add_normed_norm(x, a, w[0], 1e-5, w[1], 1e-5, o1), flush=flush)
    t_h = _median_ms(lambda: K.add_rmsnorm(x, a, w[0], 1e-5, o1), flush=flush)
    add("add_normed_norm", "add_rmsnorm", t_v, T * W * (4 + 4 + 2 + 2), 0, t_h, T * W * (4 + 4 + 2 + 2), 0)
    # activations: the routed feed-forward's (erf gelu times routing weight) and the dense one's
    moe = next(l["mlp"] for l in vcfg["layers"] if l["mlp"]["kind"] == "moe")
    E, F = moe["router"]["experts"], moe["expert"]["ff"]
    cols = E * F + moe["shared"]["ff"]
    up, act = rnd(T, cols), torch.empty(T, cols, device=dev, dtype=bf)
    route = torch.rand(T, E, device=dev)
    gu, act_h = rnd(T, 2 * ffh), torch.empty(T, ffh, device=dev, dtype=bf)
    t_h = _median_ms(lambda: K.silu_mul(gu, act_h, False), flush=flush)
    t_v = _median_ms(lambda: K.ffn_activation(up, act, "gelu", route, F, E * F), flush=flush)
    add("ffn_activation (gelu x routing weight)", "silu_mul", t_v, T * cols * 4, 0, t_h, T * ffh * 6, 0)
    up2, act2 = rnd(T, ffh), torch.empty(T, ffh, device=dev, dtype=bf)
    t_v = _median_ms(lambda: K.ffn_activation(up2, act2, "relu2"), flush=flush)
    add("ffn_activation (squared relu)", "silu_mul", t_v, T * ffh * 4, 0, t_h, T * ffh * 6, 0)
    logits = rnd(T, E, dt=torch.float32)
    idx, wt = torch.empty(T, 2, dtype=torch.int32, device=dev), torch.empty(T, 2, device=dev)
    t_v = _median_ms(lambda: K.route_topk(logits, route, idx, wt), flush=flush)
    add("route_topk", None, t_v, T * E * 8, 0, 0, 0, 0)
    del up, act, gu, act_h, up2, act2
    ps = 64
    for kind, n_req, q_len, kv in (("prefill", 1, T, T), ("decode", batch, 1, context)):
        blocks = -(-kv // ps)
        pages = n_req * blocks
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(n_req, blocks)
        cu = np.arange(n_req + 1, dtype=np.int32) * q_len
        kvl = np.full(n_req, kv, dtype=np.int32)
        cu_d, kv_d = torch.from_numpy(cu).to(dev), torch.from_numpy(kvl).to(dev)
        n = n_req * q_len
        pos = torch.from_numpy(np.concatenate([np.arange(kv - q_len, kv, dtype=np.int32)] * n_req)).to(dev)
        ent = torch.from_numpy(np.repeat(np.arange(n_req, dtype=np.int32), q_len)).to(dev)
        slots = torch.arange(n_req, dtype=torch.int32, device=dev)
        # the recurrence and what prepares it
        hd = H * dd
        pcols = 5 * hd + R
        proj = rnd(n, pcols)
        w2, w0, ab, nw = rnd(R, hd), rnd(hd, dt=torch.float32), rnd(hd, dt=torch.float32), rnd(hd, dt=torch.float32)
        aux = torch.empty(n, 3 * hd, device=dev)
        state = torch.zeros(n_req, H, dd, dd, device=dev)
        od = torch.empty(n, hd, device=dev, dtype=bf)
        t_p = _median_ms(lambda: K.delta_rule_prep(proj, pcols, ent, w2, w0, ab, aux, H, dd, math.exp(-0.5), 1e-6, bf),
                         flush=flush)
        K.delta_rule_prep(proj, pcols, ent, w2, w0, ab, aux, H, dd, math.exp(-0.5), 1e-6, bf)
        o_raw = torch.empty(n, hd, device=dev) if kind == "prefill" else None      # a prompt alone: four CTAs a head
        t_s = _median_ms(lambda: K.delta_rule_scan(proj, pcols, aux, cu_d, kv_d, slots, state, nw, 1e-5, od, H, dd, err,
                                                   col_blocks=4, o_raw=o_raw, tok_entry=ent), flush=flush)
        # attention of the other model, and this one's (the warp-level kernels with the sink)
        k_pool, v_pool = rnd(pages, nkv, ps, d), rnd(pages, nkv, ps, d)
        qh, oh = rnd(n, nq * d), torch.empty(n, nq * d, device=dev, dtype=bf)
        qkv = rnd(n, (nq + 2 * nkv) * d)
        qw, kw = rnd(nq * d, dt=torch.float32), rnd(nkv * d, dt=torch.float32)
        cos = sin = torch.ones(max(kv, 1) + 1, d // 2, device=dev)
        t_c = _median_ms(lambda: K.projection_norm_cache(qkv, qkv.shape[1], pos, ent, table, ps, qw, kw, 1e-5, qh, k_pool,
                                                         v_pool, nq, nkv, d, d, err), flush=flush)
        qn, kn = rnd(d, dt=torch.float32), rnd(d, dt=torch.float32)
        t_rc = _median_ms(lambda: K.rope_norm_cache(qkv, qkv.shape[1], bf, pos, ent, table, cos, sin, qn, kn, 1e-5, qh,
                                                    k_pool, v_pool, ps, nq, nkv, d, True, True, err), flush=flush)
        io = n * (nq + 2 * nkv) * d * 2
        add(f"projection_norm_cache ({kind})", "rope_norm_cache", t_c, io + n * (nq + 2 * nkv) * d * 2, 0, t_rc,
            io + n * (nq + 2 * nkv) * d * 2, 0)
        add(f"delta_rule_prep ({kind})", "rope_norm_cache", t_p, n * (3 * hd + R) * 2 + n * 3 * hd * 4, 0, t_rc,
            io + n * (nq + 2 * nkv) * d * 2, 0)
        if kind == "prefill":
            tiles = -(-T // 128)
            t_h = _median_ms(lambda: K.prefill_attention_tc(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, tiles, nq,
                                                            nkv, d, 0, d ** -0.5, err), flush=flush)
            tiles64 = -(-T // 64)
            t_w = _median_ms(lambda: K.paged_prefill_attention(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, tiles64,
                                                               nq, nkv, d, 0, d ** -0.5, err, sink=True), flush=flush)
            pairs = T * T / 2
            add("sink attention, prompt (paged_prefill_attn with the sink)", "prefill_attn_tc", t_w, 0, pairs * nq * 4 * d,
                t_h, 0, pairs * nq * 4 * d)
            # the recurrence: per token and head 3 d^2 multiply-adds in 32-bit; its roofline is the FP32 rate,
            # reported here against the bytes it must move (inputs, outputs) as the other kernels are
            add("delta_rule_scan, prompt", "prefill_attn_tc", t_s, n * (4 * hd * 2 + 3 * hd * 4 + hd * 2), 0,
                t_h, 0, pairs * nq * 4 * d)
        else:
            splits = K.decode_splits(n_req, nkv, 148, 64, max_keys=kv)
            po = torch.empty(n_req * nq * splits, d, device=dev)
            pml = torch.empty(n_req * nq * splits, 2, device=dev)
            t_h = _median_ms(lambda: K.paged_decode_attention(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, nq, nkv,
                                                              d, 0, d ** -0.5, splits, po, pml, err), flush=flush)
            t_w = _median_ms(lambda: K.paged_decode_attention(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, nq, nkv,
                                                              d, 0, d ** -0.5, splits, po, pml, err, sink=True), flush=flush)
            add("sink attention, decoded tokens (paged_decode_attn with the sink)", "paged_decode_attn", t_w,
                n_req * kv * nkv * d * 2 * 2, 0, t_h, n_req * kv * nkv * d * 2 * 2, 0)
            add("delta_rule_scan, decoded tokens", "paged_decode_attn", t_s, n_req * H * dd * dd * 4 * 2, 0,
                t_h, n_req * kv * nkv * d * 2 * 2, 0)
        del proj, aux, state, k_pool, v_pool, qkv
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    return rows


def vodelix_workload(args, pk):
    """Prefill and decode throughput of Vodelix at the layer sizes of --sizes beside Hunyuan Dense
    (the engine's closest model) at the same width, layers and vocabulary, random weights, and the
    kernels of the two side by side."""
    import gc
    import torch
    hcfg = dict(MODEL)
    hcfg.update(OTHER_SIZES.get(args.sizes, {}))
    layers = args.layers or 16
    hcfg["num_hidden_layers"] = layers
    hcfg["max_position_embeddings"] = max(hcfg["max_position_embeddings"], args.context + 2048)
    vcfg = vodelix_config(hcfg, layers)
    page, pt = 64, args.prefill_tokens
    out = {"workload": "vodelix", "sizes": args.sizes, "layers": layers, "batch": args.batch,
           "context": args.context, "prefill_tokens": pt, "dtype": "bf16", "data": "synthetic", "models": {}}
    for name, cfg, vocab in (("vodelix", vcfg, vcfg["vocab"]), ("hunyuan_dense", hcfg, hcfg["vocab_size"])):
        opts = dict(page_size=page, num_pages=(args.batch * (args.context + args.steps + args.warmup + 64) + pt) // page + 64,
                    max_concurrent=max(64, args.batch), max_seq_len=max(args.context, pt) + 1024,
                    max_batched_tokens=max(2048, pt), chunk_size=max(2048, pt))
        model = build_model(cfg, opts)
        pms = time_prefill(model, pt, vocab, reps=3)
        ids = fill_cache(model, args.batch, args.context)
        dms, launches = time_decode(model, ids, args.steps, args.warmup, vocab)
        weights = sum(t.numel() * t.element_size() for t in _model_tensors(model))
        out["models"][name] = {"prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(pt * 1000.0 / pms, 1),
                               "decode_ms_per_step": round(dms, 4),
                               "decode_tokens_per_s": round(args.batch * 1000.0 / dms, 1),
                               "launches_per_decode_step": launches, "weight_bytes": weights,
                               "layer_runs": len(model.runner.spec.schedule)}
        del model
        gc.collect()
        torch.cuda.empty_cache()
    out["kernels"] = vodelix_kernel_table(vcfg, hcfg, pk, pt, args.batch, args.context)
    out["peaks"] = pk
    return out


def mufevik_config(like, layers):
    """A Mufevik model with the width, layer count and vocabulary of the Hunyuan configuration `like`:
    of every three layers one runs the gated delta rule (heads of 64 across the width, half as many
    query/key heads, a convolution of four taps) and two run attention whose heads exchange their
    weights (the other's head counts, heads of 128, half of each rotated) beside gated linear
    attention (keys of 64, values of 128); every layer has eight experts of a quarter of the other's
    inner size in four groups, two groups kept and two experts chosen, and a shared one; three streams."""
    h, heads, kv = like["hidden_size"], like["num_attention_heads"], like["num_key_value_heads"]
    ff = like["intermediate_size"]
    left = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "rot": {"dims": 64, "base": 10000.0}}
    right = {"heads": max(1, h // 256), "dim": 64, "vdim": 128, "tau": 16.0, "decay_rank": 64}
    delta = {"heads": h // 64, "kv_heads": max(1, h // 128), "dim": 64, "vdim": 64, "conv": 4}
    moe = {"kind": "moe", "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}},
           "expert": {"ff": ff // 4}, "shared": {"ff": ff // 4}}
    ls = [{"type": "delta" if i % 3 == 0 else "parallel",
           "mixer": delta if i % 3 == 0 else {"left": left, "right": right}, "mlp": moe} for i in range(layers)]
    return {"architecture": "Mufevik", "vocab": like["vocab_size"], "width": h, "norm": {"eps": 1e-5},
            "streams": 3, "logit_scale": 1.0, "layers": ls}


def mufevik_kernel_table(mcfg, vcfg, hcfg, pk, tokens, batch, context):
    """Every kernel that only Mufevik runs beside the kernel of Vodelix (the engine's closest model)
    that does the like job, each alone on synthetic operands of the two models' layer sizes (L2
    flushed between repetitions), with the fraction of its roofline: algorithmic bytes over the
    measured copy rate, or FLOPs over the measured bf16 rate, whichever takes longer."""
    import math
    from types import SimpleNamespace
    import numpy as np
    import torch
    from crane_b200.kernels import get_kernels
    K = get_kernels([128])
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    W, R = mcfg["width"], mcfg["streams"]
    dl = next(l["mixer"] for l in mcfg["layers"] if l["type"] == "delta")
    par = next(l["mixer"] for l in mcfg["layers"] if l["type"] == "parallel")
    lt, rg = par["left"], par["right"]
    vd = next(l["mixer"] for l in vcfg["layers"] if l["type"] == "general_delta")
    hbm, peak = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = []

    def add(name, like, ms, nbytes, flops, like_ms=0, like_bytes=0, like_flops=0):
        def frac(ms_, b, f):
            return round(max(b / hbm, f / peak) / (ms_ * 1e-3), 4)
        rows.append({"kernel": name, "ms": round(ms, 4), "frac": frac(ms, nbytes, flops), "like": like,
                     "like_ms": round(like_ms, 4) if like_ms else None,
                     "like_frac": frac(like_ms, like_bytes, like_flops) if like_ms else None})

    T = tokens
    rnd = lambda *shape, dt=bf: torch.randn(*shape, device=dev, dtype=torch.float32).to(dt)
    f32 = torch.float32
    # a sublayer's result joins the streams and the next norm reads them / the single stream's like
    streams, y, o1 = rnd(R, T, W, dt=f32), rnd(T, W), torch.empty(T, W, device=dev, dtype=bf)
    mix, outw, inw, g = rnd(R, R, dt=f32), rnd(R, dt=f32), rnd(R, dt=f32), rnd(1, dt=f32)
    x, w = rnd(T, W, dt=f32), [rnd(W, dt=f32) for _ in range(2)]
    t_m = _median_ms(lambda: K.streams_norm(streams, None, y, mix, outw, inw, g, 1e-5, o1), flush=flush)
    t_v = _median_ms(lambda: K.add_normed_norm(x, y, w[0], 1e-5, w[1], 1e-5, o1), flush=flush)
    add(f"streams_norm ({R} streams)", "add_normed_norm", t_m, T * W * (8 * R + 4), 0, t_v, T * W * 12, 0)
    a2, b2 = rnd(T, W), rnd(T, W)
    t_m = _median_ms(lambda: K.pair_norm_mean(a2, b2, w[0], w[1], 1e-5, o1), flush=flush)
    add("pair_norm_mean", "add_normed_norm", t_m, T * W * 6, 0, t_v, T * W * 12, 0)
    del streams, x, a2, b2
    # the router and the activation between the experts' two products
    moe = mcfg["layers"][0]["mlp"]
    E, F, Fs = moe["router"]["experts"], moe["expert"]["ff"], moe["shared"]["ff"]
    top, gc, gk = moe["router"]["top"], moe["router"]["groups"]["count"], moe["router"]["groups"]["keep"]
    cols = E * F + Fs
    z, corr = rnd(T, E + 1, dt=f32), rnd(E, dt=f32)
    route = torch.empty(T, E + 1, device=dev)
    t_m = _median_ms(lambda: K.route_grouped(z, corr, route, E, top, gc, gk, True), flush=flush)
    idx, wt = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, device=dev)
    route_v = torch.rand(T, E, device=dev)
    t_v = _median_ms(lambda: K.route_topk(z[:, :E].contiguous(), route_v, idx, wt), flush=flush)
    add("route_grouped", "route_topk", t_m, T * (E + 1) * 8, 0, t_v, T * E * 8, 0)
    gu, act = rnd(T, 2 * cols), torch.empty(T, cols, device=dev, dtype=bf)
    up = rnd(T, cols)
    t_m = _median_ms(lambda: K.gated_activation(gu, act, route, E, F, E * F, True), flush=flush)
    t_v = _median_ms(lambda: K.ffn_activation(up, act, "gelu", route_v, F, E * F), flush=flush)
    add("gated_activation (silu gate x up x routing weight)", "ffn_activation (gelu x routing weight)", t_m,
        T * cols * 6, 0, t_v, T * cols * 4, 0)
    del gu, act, up
    ps = 64
    H, G, d = lt["heads"], lt["kv_heads"], lt["dim"]
    dH, dG, dk, dv, taps = dl["heads"], dl["kv_heads"], dl["dim"], dl["vdim"], dl["conv"]
    gH, gk_, gv_, rank = rg["heads"], rg["dim"], rg["vdim"], rg["decay_rank"]
    vH, vdd, vR = vd["heads"], vd["dim"], vd["decay_rank"]
    for kind, n_req, q_len, kv in (("prefill", 1, T, T), ("decode", batch, 1, context)):
        blocks = -(-kv // ps)
        pages = n_req * blocks
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(n_req, blocks)
        cu_d = torch.from_numpy(np.arange(n_req + 1, dtype=np.int32) * q_len).to(dev)
        kv_d = torch.from_numpy(np.full(n_req, kv, dtype=np.int32)).to(dev)
        n = n_req * q_len
        pos = torch.from_numpy(np.concatenate([np.arange(kv - q_len, kv, dtype=np.int32)] * n_req)).to(dev)
        ent = torch.from_numpy(np.repeat(np.arange(n_req, dtype=np.int32), q_len)).to(dev)
        slots = torch.arange(n_req, dtype=torch.int32, device=dev)
        ctx = SimpleNamespace(tok_entry=ent, cu_q=cu_d, kv_len=kv_d, slots=slots)
        # Vodelix: what prepares its recurrence, and the recurrence
        hd = vH * vdd
        pcols = 5 * hd + vR
        proj = rnd(n, pcols)
        w2, w0, ab, nw = rnd(vR, hd), rnd(hd, dt=f32), rnd(hd, dt=f32), rnd(hd, dt=f32)
        aux = torch.empty(n, 3 * hd, device=dev)
        vstate = torch.zeros(n_req, vH, vdd, vdd, device=dev)
        od = torch.empty(n, hd, device=dev, dtype=bf)
        prep_v = lambda: K.delta_rule_prep(proj, pcols, ent, w2, w0, ab, aux, vH, vdd, math.exp(-0.5), 1e-6, bf)
        t_pv = _median_ms(prep_v, flush=flush)
        prep_v()
        o_raw_v = torch.empty(n, hd, device=dev) if kind == "prefill" else None
        t_sv = _median_ms(lambda: K.delta_rule_scan(proj, pcols, aux, cu_d, kv_d, slots, vstate, nw, 1e-5, od, vH, vdd,
                                                    err, col_blocks=4, o_raw=o_raw_v, tok_entry=ent), flush=flush)
        b_pv = n * (3 * hd + vR) * 2 + n * 3 * hd * 4
        b_sv = (n * (4 * hd * 2 + 3 * hd * 4 + hd * 2)) if kind == "prefill" else n_req * vH * vdd * vdd * 8
        del proj, aux, vstate, od
        # the gated delta rule: convolutions and unit vectors, then the recurrence, then head norm and gate
        C = 2 * dG * dk + dH * dv
        pc = C + dH * dv + 2 * dH
        proj = rnd(n, pc)
        rws, lanes = K.matrix_state_plan(dk)
        conv_off = dH * rws * lanes * dv
        state = torch.zeros(n_req, conv_off + (taps - 1) * C, device=dev)
        conv_w, a_log, dtb = rnd(C, taps, dt=f32), rnd(dH, dt=f32), rnd(dH, dt=f32)
        aux = torch.empty(n, C + 2 * dH, device=dev)
        prep = lambda: K.conv_delta_prep(proj, pc, ctx, state, conv_off, conv_w, taps, a_log, dtb, aux, dH, dG, dk, dv,
                                         1e-6, dk ** -0.5, err, bf)
        t_p = _median_ms(prep, flush=flush)
        prep()
        o_raw = torch.empty(n, dH * dv, device=dev)
        gd = dG * dk
        t_s = _median_ms(lambda: K.matrix_state_scan(aux, (0, gd, 2 * gd, C, C + dH), False, True, dH // dG, ctx, state,
                                                     o_raw, dH, dk, dv, err), flush=flush)
        o = torch.empty(n, dH * dv, device=dev, dtype=bf)
        nwm = rnd(dv, dt=f32)
        t_n = _median_ms(lambda: K.head_norm_gate(o_raw, proj, pc, C, ent, nwm, 1e-5, o, dH, dv), flush=flush)
        add(f"conv_delta_prep ({kind})", "delta_rule_prep", t_p, n * C * (2 + 4), 0, t_pv, b_pv, 0)
        b_s = n * (C + 2 * dH + dH * dv) * 4 if kind == "prefill" else n_req * dH * dk * dv * 8
        add(f"matrix_state_scan, delta rule ({kind})", "delta_rule_scan", t_s, b_s, 0, t_sv, b_sv, 0)
        add(f"head_norm_gate ({kind})", "delta_rule_prep", t_n, n * dH * dv * (4 + 2 + 2), 0, t_pv, b_pv, 0)
        del proj, state, aux, o_raw, o
        # gated linear attention: the decay per key channel, then the same recurrence without correction
        ghd, ghv = gH * gk_, gH * gv_
        pc = 2 * ghd + 2 * ghv + rank
        proj = rnd(n, pc)
        a2t, bias = rnd(rank, ghd, dt=f32), rnd(ghd, dt=f32)
        aux = torch.empty(n, 3 * ghd + ghv, device=dev)
        rws, lanes = K.matrix_state_plan(gk_)
        state = torch.zeros(n_req, gH * rws * lanes * gv_, device=dev)
        prep = lambda: K.decay_gate_prep(proj, pc, ent, a2t, bias, 1.0 / rg["tau"], gk_ ** -0.5, aux, gH, gk_, gv_, bf)
        t_p = _median_ms(prep, flush=flush)
        prep()
        o_raw = torch.empty(n, ghv, device=dev)
        t_s = _median_ms(lambda: K.matrix_state_scan(aux, (0, ghd, 2 * ghd, 2 * ghd + ghv, 0), True, False, 1, ctx, state,
                                                     o_raw, gH, gk_, gv_, err), flush=flush)
        add(f"decay_gate_prep ({kind})", "delta_rule_prep", t_p, n * (2 * ghd + ghv + rank) * 2 + n * (3 * ghd + ghv) * 4,
            0, t_pv, b_pv, 0)
        b_s = n * (3 * ghd + 2 * ghv) * 4 if kind == "prefill" else n_req * gH * gk_ * gv_ * 8
        add(f"matrix_state_scan, decay per channel ({kind})", "delta_rule_scan", t_s, b_s, 0, t_sv, b_sv, 0)
        del proj, state, aux, o_raw
        # attention whose heads exchange their weights, beside the like kernels with the sink
        k_pool, v_pool = rnd(pages, G, ps, d), rnd(pages, G, ps, d)
        qh, oh = rnd(n, H * d), torch.empty(n, H * d, device=dev, dtype=bf)
        cross = torch.empty(n, H * G * d, device=dev)
        talk = rnd(H, H, dt=f32)
        t_x = _median_ms(lambda: K.head_talk_mix(cross, talk, ent, oh, H, G, d, d), flush=flush)
        add(f"head_talk_mix ({kind})", None, t_x, n * H * d * (4 * G + 2), 0)
        if kind == "prefill":
            tiles = -(-T // 64)
            t_m = _median_ms(lambda: K.paged_prefill_attention(qh, cross, k_pool, v_pool, cu_d, kv_d, table, ps, tiles, H, G,
                                                               d, 0, d ** -0.5, err, cross=True), flush=flush)
            t_v = _median_ms(lambda: K.paged_prefill_attention(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, tiles, H, G,
                                                               d, 0, d ** -0.5, err, sink=True), flush=flush)
            pairs = T * T / 2
            add("attention for every pair of heads, prompt (paged_prefill_attn, cross)", "paged_prefill_attn with the sink",
                t_m, 0, pairs * H * G * 4 * d, t_v, 0, pairs * H * 4 * d)
        else:
            sp_v = K.decode_splits(n_req, G, 148, 64, max_keys=kv)
            sp_m = max(1, min(32, (2 * 148) // max(1, n_req * G * G)))
            po = torch.empty(n_req * H * G * max(sp_v, sp_m), d, device=dev)
            pml = torch.empty(n_req * H * G * max(sp_v, sp_m), 2, device=dev)
            t_m = _median_ms(lambda: K.paged_decode_attention(qh, cross, k_pool, v_pool, cu_d, kv_d, table, ps, H, G, d, 0,
                                                              d ** -0.5, sp_m, po, pml, err, cross=True), flush=flush)
            t_v = _median_ms(lambda: K.paged_decode_attention(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, H, G, d, 0,
                                                              d ** -0.5, sp_v, po, pml, err, sink=True), flush=flush)
            kvb = n_req * kv * G * d * 2 * 2
            add("attention for every pair of heads, decoded tokens (paged_decode_attn, cross)",
                "paged_decode_attn with the sink", t_m, kvb, 0, t_v, kvb, 0)
        del k_pool, v_pool, cross
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    return rows


def mufevik_workload(args, pk):
    """Prefill and decode throughput of Mufevik at the layer sizes of --sizes beside Vodelix (the
    engine's closest model: a delta rule, experts with a shared one, attention on the warp-level
    kernels) at the same width, layers and vocabulary, random weights, and the kernels of the two
    side by side."""
    import gc
    import torch
    hcfg = dict(MODEL)
    hcfg.update(OTHER_SIZES.get(args.sizes, {}))
    layers = args.layers or 12
    hcfg["num_hidden_layers"] = layers
    vcfg = vodelix_config(hcfg, layers)
    vcfg.pop("loop", None)                       # every layer once, as in the other model
    mcfg = mufevik_config(hcfg, layers)
    page, pt = 64, args.prefill_tokens
    out = {"workload": "mufevik", "sizes": args.sizes, "layers": layers, "batch": args.batch,
           "context": args.context, "prefill_tokens": pt, "dtype": "bf16", "data": "synthetic", "models": {}}
    for name, cfg in (("mufevik", mcfg), ("vodelix", vcfg)):
        opts = dict(page_size=page, num_pages=(args.batch * (args.context + args.steps + args.warmup + 64) + pt) // page + 64,
                    max_concurrent=max(64, args.batch), max_seq_len=max(args.context, pt) + 1024,
                    max_batched_tokens=max(2048, pt), chunk_size=max(2048, pt))
        model = build_model(cfg, opts)
        pms = time_prefill(model, pt, cfg["vocab"], reps=3)
        ids = fill_cache(model, args.batch, args.context)
        dms, launches = time_decode(model, ids, args.steps, args.warmup, cfg["vocab"])
        weights = sum(t.numel() * t.element_size() for t in _model_tensors(model))
        out["models"][name] = {"prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(pt * 1000.0 / pms, 1),
                               "decode_ms_per_step": round(dms, 4),
                               "decode_tokens_per_s": round(args.batch * 1000.0 / dms, 1),
                               "launches_per_decode_step": launches, "weight_bytes": weights,
                               "layer_runs": len(model.runner.spec.schedule)}
        del model
        gc.collect()
        torch.cuda.empty_cache()
    out["kernels"] = mufevik_kernel_table(mcfg, vcfg, hcfg, pk, pt, args.batch, args.context)
    out["peaks"] = pk
    return out


def zudarax_config(like, layers):
    """A Zudarax model with the width, layer count, head counts and vocabulary of the Hunyuan configuration
    `like`: layers take turns between the three mixers (softmax attention behind convolutions of four taps
    with half of each head rotated, squashed scores and blocks of 1,024 positions; differential attention with
    two maps of 64 per head and values of 128; sigmoid attention behind the convolutions with YaRN), all with
    heads stored at 128; norms in eight groups; the feed-forward's inner size one and a half times the
    other's, which has three matrices where this one has two."""
    h, heads, kv = like["hidden_size"], like["num_attention_heads"], like["num_key_value_heads"]
    ff = like["intermediate_size"] * 3 // 2
    soft = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "conv": 4,
            "rot": {"dims": 64, "base": 10000.0}, "softcap": 50.0, "mask": {"size": 1024}}
    diff = {"heads": heads, "kv_heads": kv, "dim": 64, "vdim": 128, "scale": 64 ** -0.5, "diff": 0.5,
            "rot": {"dims": 32, "base": 10000.0}}
    sig = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "conv": 4,
           "rot": {"dims": 128, "base": 1000000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}
    kinds = (("attention", soft), ("attention_2", diff), ("attention_3", sig))
    ls = [{"type": kinds[i % 3][0], "mixer": kinds[i % 3][1], "mlp": {"kind": "dense", "ff": ff}} for i in range(layers)]
    return {"architecture": "Zudarax", "vocab": like["vocab_size"], "width": h, "norm": {"eps": 1e-5, "groups": 8},
            "layers": ls}


def zudarax_kernel_table(zcfg, hcfg, pk, tokens, batch, context):
    """Every kernel that only Zudarax runs beside the kernel of Hunyuan Dense (the engine's closest model:
    attention layers only, a dense feed-forward) that does the like job, each alone on synthetic operands of
    the two models' layer sizes (L2 flushed between repetitions), with the fraction of its roofline:
    algorithmic bytes over the measured copy rate, or FLOPs over the measured bf16 rate, whichever takes
    longer."""
    from types import SimpleNamespace
    import numpy as np
    import torch
    from crane_b200.kernels import get_kernels
    K = get_kernels([128])
    dev, bf, f32 = "cuda:0", torch.bfloat16, torch.float32
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    W, groups = zcfg["width"], zcfg["norm"]["groups"]
    ffz, ffh = zcfg["layers"][0]["mlp"]["ff"], hcfg["intermediate_size"]
    d, nq, nkv = hcfg["head_dim"], hcfg["num_attention_heads"], hcfg["num_key_value_heads"]
    hbm, peak = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = []

    def add(name, like, ms, nbytes, flops, like_ms=0, like_bytes=0, like_flops=0):
        def frac(ms_, b, f):
            return round(max(b / hbm, f / peak) / (ms_ * 1e-3), 4)
        rows.append({"kernel": name, "ms": round(ms, 4), "frac": frac(ms, nbytes, flops), "like": like,
                     "like_ms": round(like_ms, 4) if like_ms else None,
                     "like_frac": frac(like_ms, like_bytes, like_flops) if like_ms else None})

    T = tokens
    rnd = lambda *shape, dt=bf: torch.randn(*shape, device=dev, dtype=torch.float32).to(dt)
    for n in (T, batch):
        tag = "prompt" if n == T else f"{batch} tokens"
        # two results join the stream and the next norm reads it / one result and the plain norm
        x, a, f = rnd(n, W, dt=f32), rnd(n, W), rnd(n, W)
        o1, w = torch.empty(n, W, device=dev, dtype=bf), rnd(W, dt=f32)
        t_z = _median_ms(lambda: K.add_group_rmsnorm(x, a, f, w, groups, 1e-5, o1), flush=flush)
        t_h = _median_ms(lambda: K.add_rmsnorm(x, a, w, 1e-5, o1), flush=flush)
        add(f"add_group_rmsnorm ({tag})", "add_rmsnorm", t_z, n * W * (4 + 4 + 2 + 2 + 2), 0, t_h, n * W * (4 + 4 + 2 + 2), 0)
        # the activation between the feed-forward's two products
        up, act = rnd(n, ffz), torch.empty(n, ffz, device=dev, dtype=bf)
        coef = rnd(4, dt=f32)
        gu, act_h = rnd(n, 2 * ffh), torch.empty(n, ffh, device=dev, dtype=bf)
        t_z = _median_ms(lambda: K.poly_norm(up, coef, 1e-5, act), flush=flush)
        t_h = _median_ms(lambda: K.silu_mul(gu, act_h, False), flush=flush)
        add(f"poly_norm ({tag})", "silu_mul", t_z, n * ffz * 4, 0, t_h, n * ffh * 6, 0)
        del x, a, f, up, act, gu, act_h
    ps = 64
    kinds = {l["type"]: l["mixer"] for l in zcfg["layers"]}
    for kind, n_req, q_len, kv in (("prompt", 1, T, T), (f"{batch} tokens", batch, 1, context)):
        blocks = -(-kv // ps)
        pages = n_req * blocks
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(n_req, blocks)
        cu_d = torch.from_numpy(np.arange(n_req + 1, dtype=np.int32) * q_len).to(dev)
        kv_d = torch.from_numpy(np.full(n_req, kv, dtype=np.int32)).to(dev)
        n = n_req * q_len
        pos = torch.from_numpy(np.concatenate([np.arange(kv - q_len, kv, dtype=np.int32)] * n_req)).to(dev)
        ent = torch.from_numpy(np.repeat(np.arange(n_req, dtype=np.int32), q_len)).to(dev)
        slots = torch.arange(n_req, dtype=torch.int32, device=dev)
        ctx = SimpleNamespace(positions=pos, tok_entry=ent, cu_q=cu_d, kv_len=kv_d, slots=slots)
        # the like kernels of Hunyuan Dense
        k_pool, v_pool = rnd(pages, nkv, ps, d), rnd(pages, nkv, ps, d)
        qkv_h = rnd(n, (nq + 2 * nkv) * d)
        qh, oh = rnd(n, nq * d), torch.empty(n, nq * d, device=dev, dtype=bf)
        cos, sin = torch.rand(kv, d // 2, device=dev), torch.rand(kv, d // 2, device=dev)
        nw = rnd(d, dt=f32)
        t_rope = _median_ms(lambda: K.rope_norm_cache(qkv_h, (nq + 2 * nkv) * d, bf, pos, ent, table, cos, sin, nw, nw, 1e-5,
                                                      qh, k_pool, v_pool, ps, nq, nkv, d, True, True, err), flush=flush)
        b_rope = n * (nq + 2 * nkv) * d * 2 * 2
        pairs = T * T / 2
        if q_len > 1:
            tiles64 = -(-T // 64)
            t_like = _median_ms(lambda: K.paged_prefill_attention(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, tiles64, nq,
                                                                  nkv, d, 0, d ** -0.5, err), flush=flush)
            t_tc = _median_ms(lambda: K.prefill_attention_tc(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, -(-T // 128),
                                                             nq, nkv, d, 0, d ** -0.5, err), flush=flush)
            add("(the like kernel beside the tcgen05 one)", "prefill_attn_tc (tcgen05)", t_like, 0, pairs * nq * 4 * d,
                t_tc, 0, pairs * nq * 4 * d)
        else:
            sp = K.decode_splits(n_req, nkv, 148, 64, max_keys=kv)
            po, pml = torch.empty(n_req * nq * sp, d, device=dev), torch.empty(n_req * nq * sp, 2, device=dev)
            t_like = _median_ms(lambda: K.paged_decode_attention(qh, oh, k_pool, v_pool, cu_d, kv_d, table, ps, nq, nkv, d, 0,
                                                                 d ** -0.5, sp, po, pml, err), flush=flush)
        kvb = n_req * kv * nkv * d * 2 * 2
        for name, m in kinds.items():
            H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            maps = 2 if name == "attention_2" else 1
            taps = m.get("conv", 0)
            D, dpad = 128, 128 // maps
            cq, ck, cv = H * maps * dim, G * maps * dim, G * vd
            C = cq + ck + cv
            cols = C + (H if maps == 2 else 0)
            proj = rnd(n, cols)
            conv_w = rnd(taps, C, dt=f32) if taps else None
            tails = torch.zeros(n_req, (taps - 1) * C, device=dev) if taps > 1 else None
            qn, kn = (rnd(cq, dt=f32), rnd(ck, dt=f32)) if name == "attention" else (None, None)
            rot = m["rot"]["dims"]
            cz, sz = torch.rand(kv, rot // 2, device=dev), torch.rand(kv, rot // 2, device=dev)
            q = torch.empty(n, H * D, device=dev, dtype=bf)
            gate = torch.empty(n, H, device=dev) if maps == 2 else None
            t_p = _median_ms(lambda: K.scored_prep(proj, cols, ctx, table, tails, conv_w, max(taps, 1), ps, qn, kn, 1e-5, q,
                                                   k_pool, v_pool, H, G, maps, dim, vd, dpad, cz, sz, rot, gate, C, err),
                             flush=flush)
            add(f"scored_prep, {name} ({kind})", "rope_norm_cache", t_p, n * C * 2 * 2 + (n * C * 2 * (taps - 1) if taps and
                q_len == 1 else 0), 0, t_rope, b_rope, 0)
            finish = maps == 2
            mod = K.ScoreMod(softcap=m.get("softcap", 0.0), chunk=(m.get("mask") or {}).get("size", 0),
                             sigmoid=name == "attention_3", head_bias=rnd(H, dt=f32) if name == "attention_3" else None,
                             maps=maps, lam=0.4, head_norm=finish, norm_scale=0.5, eps=1e-5, gate=gate, dv=vd, compact=finish)
            o = torch.empty(n, H * (vd if finish else D), device=dev, dtype=bf)
            q.copy_(rnd(n, H * D))
            if q_len > 1:
                t_a = _median_ms(lambda: K.scored_prefill_attention(q, o, k_pool, v_pool, cu_d, kv_d, table, ps, -(-T // 64),
                                                                    H, G, D, 0, m["scale"], mod, err), flush=flush)
                blk = mod.chunk or T
                seen = T * min(blk, T) / 2 if blk < T else pairs          # (query, key) pairs that are visible
                add(f"scored_prefill_attn, {name} (prompt)", "paged_prefill_attn (warp-level MMA)", t_a, 0,
                    seen * H * (2 * D + 2 * D * maps), t_like, 0,
                    pairs * nq * 4 * d)
            else:
                sp = max(1, min(32, ((3 if maps == 2 else 2) * 148) // max(1, n_req * G)))
                po = torch.empty(n_req * H * maps * sp, D, device=dev)
                pml = torch.empty(n_req * H * maps * sp, 2, device=dev)
                t_a = _median_ms(lambda: K.scored_decode_attention(q, o, k_pool, v_pool, cu_d, kv_d, table, ps, H, G, D, 0,
                                                                   m["scale"], sp, po, pml, mod, err), flush=flush)
                blk = mod.chunk or kv
                read = min(kv, (kv - 1) % blk + 1)                        # keys a token at position kv - 1 sees
                add(f"scored_decode_attn + merge, {name} ({kind})", "paged_decode_attn", t_a, n_req * read * G * D * 2 * 2, 0,
                    t_like, kvb, 0)
            del proj, q, o
        del k_pool, v_pool, qkv_h, qh, oh
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    return rows


def zudarax_workload(args, pk):
    """Prefill and decode throughput of Zudarax at the layer sizes of --sizes beside Hunyuan Dense (the
    engine's closest model) at the same width, heads, layers and vocabulary, random weights, and the
    kernels of the two side by side."""
    import gc
    import torch
    hcfg = dict(MODEL)
    hcfg.update(OTHER_SIZES.get(args.sizes, {}))
    layers = args.layers or 12
    hcfg["num_hidden_layers"] = layers
    zcfg = zudarax_config(hcfg, layers)
    page, pt = 64, args.prefill_tokens
    out = {"workload": "zudarax", "sizes": args.sizes, "layers": layers, "batch": args.batch,
           "context": args.context, "prefill_tokens": pt, "dtype": "bf16", "data": "synthetic", "models": {}}
    for name, cfg in (("zudarax", zcfg), ("hunyuan_dense", hcfg)):
        opts = dict(page_size=page, num_pages=(args.batch * (args.context + args.steps + args.warmup + 64) + pt) // page + 64,
                    max_concurrent=max(64, args.batch), max_seq_len=max(args.context, pt) + 1024,
                    max_batched_tokens=max(2048, pt), chunk_size=max(2048, pt))
        vocab = cfg.get("vocab") or cfg["vocab_size"]
        model = build_model(cfg, opts)
        pms = time_prefill(model, pt, vocab, reps=3)
        ids = fill_cache(model, args.batch, args.context)
        dms, launches = time_decode(model, ids, args.steps, args.warmup, vocab)
        weights = sum(t.numel() * t.element_size() for t in _model_tensors(model))
        out["models"][name] = {"prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(pt * 1000.0 / pms, 1),
                               "decode_ms_per_step": round(dms, 4),
                               "decode_tokens_per_s": round(args.batch * 1000.0 / dms, 1),
                               "launches_per_decode_step": launches, "weight_bytes": weights,
                               "layer_runs": len(model.runner.spec.schedule)}
        del model
        gc.collect()
        torch.cuda.empty_cache()
    out["kernels"] = zudarax_kernel_table(zcfg, hcfg, pk, pt, args.batch, args.context)
    out["peaks"] = pk
    return out


def _model_tensors(model):
    seen, out = set(), []
    parts = [model.runner.model.embed, model.runner.model.final_norm, model.runner.model.head]
    for b in model.runner.model.blocks:
        parts += list(b.parts())
    import torch
    for p in parts:
        for v in vars(p).values():
            if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                seen.add(v.data_ptr())
                out.append(v)
    return out


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "cryptomilk/Crane is a Rust workspace on Candle; there is no cargo or rustc "
                      "in this image and no vendored crates, so it cannot be built or installed offline"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--impl", default="crane_b200")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill measurements")
    ap.add_argument("--only-prefill", action="store_true",
                    help="measure the 2,048-token prefill alone (for profiling); prints its record only")
    ap.add_argument("--prefill-tokens", type=int, default=2048,
                    help="with --only-prefill: another prompt length than the contract's 2,048 (one step)")
    ap.add_argument("--sizes", default="1.8b", choices=["1.8b", "4b", "7b"],
                    help="layer sizes: Hunyuan 1.8B (the default, the headline configuration), 4B or 7B")
    ap.add_argument("--prefill-chunk", type=int, default=0,
                    help="with --only-prefill: also time the prompt in portions of this many tokens, a step each")
    ap.add_argument("--workload", default="", choices=["", "serve", "mixed-step", "radorax", "vodelix", "mufevik", "zudarax"],
                    help="serve: a mix of requests through the scheduler; mixed-step: decoded tokens beside "
                         "one prompt portion in one step; radorax: prefill and decode of Radorax beside Hunyuan "
                         "Dense at equal layer sizes, and their kernels side by side; vodelix: the same for Vodelix; "
                         "each prints its own record only")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=4096)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--portion", type=int, default=512)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-check", action="store_true",
                    help="skip the comparison of one decode step's logits with the 32-bit path")
    ap.add_argument("--only-decode", action="store_true",
                    help="measure the decode step alone (for profiling: the timed steps lie between "
                         "cudaProfilerStart and cudaProfilerStop); prints its record only")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    args.warmup = max(args.warmup, 3)

    if args.workload == "zudarax":
        print(json.dumps(zudarax_workload(args, peaks())))
        return 0
    if args.workload == "mufevik":
        print(json.dumps(mufevik_workload(args, peaks())))
        return
    if args.workload == "vodelix":
        print(json.dumps(vodelix_workload(args, peaks())))
        return 0
    if args.workload == "radorax":
        print(json.dumps(radorax_workload(args, peaks())))
        return 0

    import torch
    cfg = dict(MODEL)
    cfg.update(OTHER_SIZES.get(args.sizes, {}))
    full_layers = cfg["num_hidden_layers"]
    # a context beyond the configuration's limit: the same layer sizes with a longer position table
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], args.context + 2048,
                                         args.prefill_tokens + 2048)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers, vocab = cfg["num_hidden_layers"], cfg["vocab_size"]
    pk = peaks()
    page = 64
    need_tokens = 64 * (args.context + args.steps + args.warmup + 64) if not args.no_points else \
        args.batch * (args.context + args.steps + args.warmup + 64)
    need_tokens = max(need_tokens, args.batch * (args.context + args.steps + args.warmup + 64))
    opts = dict(page_size=page, num_pages=need_tokens // page + 64, max_concurrent=max(64, args.batch),
                max_seq_len=args.context + 1024, max_batched_tokens=2048, chunk_size=2048)
    if args.only_prefill:
        pt = args.prefill_tokens
        opts.update(num_pages=pt // page + 8, max_concurrent=4, max_seq_len=pt + 1024,
                    max_batched_tokens=max(2048, pt), chunk_size=max(2048, pt))
    if args.only_decode:
        opts.update(num_pages=args.batch * (args.context + args.steps + args.warmup + 64) // page + 64)
    if args.workload == "serve":
        per = args.prompt_max + args.new_tokens + page
        cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], per + 64)
        opts.update(num_pages=args.requests * per // page + 64, max_concurrent=args.requests,
                    max_seq_len=per, max_batched_tokens=2048, chunk_size=2048)
    if args.workload == "mixed-step":
        opts.update(num_pages=(args.batch * (args.context + 256) + 4 * args.portion) // page + 64,
                    max_concurrent=args.batch + 2, max_batched_tokens=max(2048, args.batch + args.portion))
    model = build_model(cfg, opts)
    runner = model.runner
    if args.workload == "serve":
        print(json.dumps(dict(serve_workload(model, cfg, args, pk), sizes=args.sizes, layers=layers)))
        return 0
    if args.workload == "mixed-step":
        print(json.dumps(dict(mixed_step_workload(model, cfg, args), sizes=args.sizes, layers=layers)))
        return 0
    if args.only_prefill:
        pms = time_prefill(model, pt, vocab, reps=max(1, args.steps), mark=True)
        flops = prefill_flops(cfg, layers, pt)
        rec = {"value": round(pt * 1000.0 / pms, 1), "tokens": pt, "ms": round(pms, 3), "layers": layers,
               "sizes": args.sizes, "tflops": round(flops / (pms * 1e-3) / 1e12, 1),
               "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        if args.prefill_chunk:
            cms = time_prefill_chunked(model, pt, args.prefill_chunk, vocab)
            rec["chunked"] = {"chunk": args.prefill_chunk, "value": round(pt * 1000.0 / cms, 1),
                              "ms": round(cms, 3),
                              "frac": round(flops / (cms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        print(json.dumps({"prefill": rec}))
        return 0

    def decode_point(batch):
        ids = fill_cache(model, batch, args.context)
        ms, launches = time_decode(model, ids, args.steps, args.warmup, vocab, mark=args.only_decode)
        for rid in ids:
            runner.end(rid)
        return ms, launches

    if args.only_decode:
        ms, launches = decode_point(args.batch)
        gbs = decode_bytes(cfg, layers, args.batch, args.context + args.warmup + args.steps // 2) / (ms * 1e-3) / 1e9
        print(json.dumps({"decode": {"value": round(args.batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 4),
                                     "layers": layers, "sizes": args.sizes, "batch": args.batch,
                                     "context": args.context, "launches_per_step": launches,
                                     "gbs": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4)}}))
        return 0

    check = None
    if not args.no_check:
        # the serving path's logits at the headline shape against the 32-bit path, before anything is timed
        ids = fill_cache(model, args.batch, args.context)
        err, same = check_decode_logits(model, cfg, ids, args.context, vocab, page)
        for rid in ids:
            runner.end(rid)
        check = {"against": "float32 path of the same engine, one decode step", "max_rel_err": round(err, 5),
                 "same_argmax": same, "rows": args.batch}
        # Rounding of the bfloat16 activations adds up over the layers: measured at this shape with 1,
        # 2, 4, 8, 16 and 32 layers, 0.0057, 0.0079, 0.0105, 0.0138, 0.0181 and 0.0316 of the largest
        # logit, that is 0.0057 * sqrt(layers).  Twice that is the bound; a key slice left out in one
        # layer moves the logits by several times as much.
        check["bound"] = round(1.2e-2 * layers ** 0.5, 5)
        if not err < check["bound"]:
            print(json.dumps({"error": "the serving path's logits differ from the 32-bit path's", "check": check}))
            return 1

    with ClockSampler() as clocks:
        ms, launches = decode_point(args.batch)
    clock = clocks.summary()
    value = args.batch * 1000.0 / ms
    bytes_step = decode_bytes(cfg, layers, args.batch, args.context + args.warmup + args.steps // 2)
    achieved = bytes_step / (ms * 1e-3) / 1e9
    e2e_value, h2d, d2h = time_decode_e2e(model, args.batch, args.context, args.steps, args.warmup, vocab)

    out = {
        "metric": "decode tokens/s (Hunyuan-%s sizes, batch %d, context %d)" % (args.sizes.upper(), args.batch, args.context),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": "Hunyuan-%s-sized, random weights" % args.sizes.upper(), "layers": layers,
                   "layers_of_model": full_layers, "hidden": cfg["hidden_size"],
                   "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": vocab, "global_batch": args.batch, "seq_len": args.context,
                   "page_size": page, "parallelism": "none", "l2": "inputs larger than L2",
                   "cuda_graphs": bool(runner.graph_replays)},
        "clocks": clock,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                     "peaks": pk["source"]},
    }
    if check is not None:
        out["check"] = check
    if not args.no_points:
        # the prefill first: right after the batch-64 point the power cap holds the SM clock down
        # for a moment, which says nothing about the prefill
        tokens = 2048
        pms = time_prefill(model, tokens, vocab, reps=5)
        flops = prefill_flops(cfg, layers, tokens)
        out["prefill"] = {"value": round(tokens * 1000.0 / pms, 1), "tokens": tokens,
                          "ms": round(pms, 3),
                          "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        points = {}
        for b in (1, 64):
            pms, _ = decode_point(b)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
