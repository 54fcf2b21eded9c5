#!/usr/bin/env python3
"""Measurement of the library's headline metric on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl own|reference]

A "step" is one decode step of the batch.  The default run has the layer sizes
of SmolLM2-1.7B (random weights, bfloat16), a batch of 8 and sequences that end
at a context of 8192 tokens.  It prints ONE JSON line:

  value      decoded tokens a second, device time of K replayed decode steps
             (the sampled tokens feed the next step on the device)
  e2e        the same through the public entry point DecodeBatch.step_host:
             every step uploads the tokens it feeds from pinned host memory and
             downloads the tokens it sampled
  prefill    one prompt of 2,048 tokens through step(), its token ids handed over
             as an array (the figure reported; `ms_from_list` is the same with a
             Python list of ints): tokens a second, and the step's flops / time /
             the bfloat16 matrix peak
  roofline   the decode step against HBM: bytes it has to read (every weight
             once, the cache of the live sequences) / its time / the copy peak
  points     decode tokens a second at batch 1 and 64 (same context), and
             decode_b{1,8,64}_u2048: batches whose prompts, of lengths drawn
             uniformly from [128, 2048] (seeded), were really prefilled through
             step() before the timed decode steps; points_ms and points_roofline
             give every point's milliseconds per step and its fraction of the
             HBM roofline at its own context lengths
  cpu_baseline  for context only: the plain NumPy implementation of tests/ on the
             host, tiny-llama-A, tokens a second

With --design ropovik it measures the Ropovik design instead (see `run_design`):
prefill and decode of a looped stack of Mamba-2 and attention layers at the
layer sizes of two real models, beside the Llama decoder at equal width, depth
and heads, and every kernel the design added beside the like kernel of the
Llama path, each against the copy peak.  With --design senupel it does the same
for the Senupel design (attention through a latent, dense and routed
feed-forwards; see `senupel_shape`), and with --design zotolix for the Zotolix
design (four copies of the hidden state, attention within stretches of
positions, squared-relu experts; see `zotolix_shape`), and with --design megerax
for the Megerax design (attention with convolved projections, capped scores and
a gate on all channels, attention through a latent with sinks, the gated delta
rule; see `megerax_shape`).  The default run is not changed by any of them.

Peaks come from MEASURED_PEAKS.json beside this file if present, else from the
fallback figures of an earlier measurement on the same pool.  Inputs are larger
than L2 (3.4 GB of weights and 1.6 GB of cache per sequence against 126 MB), so
no flush is needed between steps.  For --gpus N > 1 it prints a line that says
so and exits with 2: this library runs on one GPU.
"""
import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SMOLLM2_1P7B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 49152,
    "rope_theta": 130000.0, "rope_scaling": None, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 8192,
}
LLAMA3_SCALING = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                  "original_max_position_embeddings": 8192}
# The other shapes the reference's engine names, for measurements beside the default.
LLAMA_3P2_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0, "rope_scaling": dict(LLAMA3_SCALING, factor=32.0), "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
LLAMA_3P1_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rope_theta": 500000.0, "rope_scaling": dict(LLAMA3_SCALING, factor=8.0), "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 131072,
}
SHAPES = {"smollm2-1.7b": ("SmolLM2-1.7B", SMOLLM2_1P7B), "llama-3.2-1b": ("Llama-3.2-1B", LLAMA_3P2_1B),
          "llama-3.1-8b": ("Llama-3.1-8B", LLAMA_3P1_8B)}
FULL_LAYERS = SMOLLM2_1P7B["num_hidden_layers"]
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs.  The
    query polls every 20 ms from before the warm-up on; `mark()` at the start of the
    timed region separates the samples.  The summary is taken over the timed region
    when it is long enough to hold three samples, else over warm-up and timed region
    together (`window` says which)."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.proc = None
        self.marked_at = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark(self):
        """The timed region begins now (samples carry nvidia-smi's own time stamps)."""
        self.marked_at = datetime.datetime.now()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.03)                        # let the sample that covers the region's end be taken
        ended_at = datetime.datetime.now()
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        rows = []
        for line in out.splitlines():
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 7:
                continue
            try:
                when = datetime.datetime.strptime(cells[0], "%Y/%m/%d %H:%M:%S.%f")
                rows.append((when, float(cells[1]), float(cells[2]),
                             [n for n, c in zip(self.NAMES, cells[3:7]) if c.lower().startswith("active")]))
            except ValueError:
                continue
        timed = [r for r in rows if self.marked_at is not None and self.marked_at <= r[0] <= ended_at]
        window = "timed region"
        if len(timed) < 3:
            timed, window = rows, "warm-up and timed region"
        sm, mx = [r[1] for r in timed], [r[2] for r in timed]
        reasons = sorted({n for r in timed for n in r[3]})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "window": window, "poll_ms": 20}


def decode_bytes(cfg, n_layers, batch, context):
    """Bytes a decode step has to read: every weight it uses once (bfloat16) and
    the keys and values of the live sequences."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * H + H * q + 3 * H * I + 2 * H
    # a tied head reads the embedding table; a separate one is read instead of it (a
    # decode step reads only a few rows of the table itself)
    weights = 2 * (n_layers * per_layer + V * H + H)
    cache = batch * context * n_layers * 2 * kv * 2
    return weights + cache, weights, cache


def prefill_flops(cfg, n_layers, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, hd = cfg["num_attention_heads"], cfg["head_dim"]
    q, kv = nh * hd, cfg["num_key_value_heads"] * hd
    gemm = 2 * T * ((q + 2 * kv) * H + H * q + 3 * H * I)
    attn = 2 * T * T * hd * nh          # causal: half of QK^T and half of PV
    return n_layers * (gemm + attn) + 2 * V * H


def kernel_breakdown(run, repeats, what, n_layers):
    """Where a step's time goes: for every kernel the time it ADDS to the step (its end
    minus the end of the kernel before it; kernels of a step overlap their starts under
    programmatic dependent launch, so durations would count some time twice), summed per
    kernel name; a kernel launched several times per layer (the products) is split by
    its position among those launches (#0, #1, ... in launch order)."""
    import collections
    import torch
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(repeats):
            run()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda e: e.time_range.start)
    def short(name):
        name = name.replace("(anonymous namespace)::", "").replace("void ", "")
        return name.split("(")[0][:60]
    per_step = collections.Counter(short(e.name) for e in events)
    per_layer = {k: (v // repeats) // n_layers if (v // repeats) % n_layers == 0 else 1 for k, v in per_step.items()}
    seen = collections.Counter()
    added = collections.defaultdict(lambda: [0, 0.0])
    last_end = None
    for e in events:
        begin, end = e.time_range.start, e.time_range.end
        name = short(e.name)
        if per_layer[name] > 1:
            k = seen[name]
            seen[name] = k + 1
            name = f"{name} #{k % per_layer[name]}"
        if last_end is not None:
            gain = max(0.0, end - last_end) if begin - last_end < 50 else end - begin   # a gap: another step begins
            row = added[name]
            row[0] += 1
            row[1] += gain
        last_end = end if last_end is None else max(last_end, end)
    total = sum(t for _, t in added.values())
    print(f"# {what}: time added per kernel, microseconds per step (sum {total / repeats:.1f})")
    for name, (count, t) in sorted(added.items(), key=lambda kv: -kv[1][1]):
        print(f"# {t / repeats:9.1f} us  {100 * t / total:5.1f} %  {count / repeats:6.1f} launches  {name}")


def prefill_only(args, model, cache, vocab, gen):
    """For profilers: `warmup` + `steps` prefills of one 2,048-token prompt."""
    import torch
    from go_tinygrad_b200.engine import StepEntry, step
    prompt = torch.randint(0, vocab, (2048,), generator=gen).tolist()
    times = []
    for i in range(args.warmup + args.steps):
        slot = cache.open_sequence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step(model, cache, [StepEntry(slot, prompt, [2047])])
        b.record()
        torch.cuda.synchronize()
        if i >= args.warmup:
            times.append(a.elapsed_time(b))
        cache.close_sequence(slot)
    if args.breakdown:
        def once():
            slot = cache.open_sequence()
            step(model, cache, [StepEntry(slot, prompt, [2047])])
            cache.close_sequence(slot)
        kernel_breakdown(once, 3, "prefill of 2,048 tokens", args.layers)
    print(json.dumps({"only": "prefill", "ms": round(statistics.median(times), 3)}))
    return 0


def run_own(args):
    import torch
    import go_tinygrad_b200 as lib
    from go_tinygrad_b200.engine import StepEntry, step
    from go_tinygrad_b200.engine.decode import DecodeBatch
    from go_tinygrad_b200.kernels import ops

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    shape_name, shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    cfg = dict(shape, num_hidden_layers=args.layers)
    pk = peaks()
    model = lib.Model.random(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02)
    context, vocab = args.context, cfg["vocab_size"]
    if args.only != "all":
        args.points = False
    biggest = max([args.batch] + ([1, 64] if args.points else []))
    cache = model.new_cache(max_tokens=biggest * context + 64 * 40, max_slots=biggest + 1)
    for grp in cache.groups:                       # synthetic keys and values of unit scale
        grp.storage.normal_(0.0, 1.0)
    gen = torch.Generator().manual_seed(0)

    kv_row = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * args.layers     # cache bytes of one token, all layers
    weight_bytes = decode_bytes(cfg, args.layers, 0, 0)[1]
    # at least this much untimed device work before a timed region (not in the --only modes,
    # which are for profilers and want few launches before the captured ones)
    WARM_MS = 300.0 if args.only == "all" else 0.0

    def decode_run(batch, steps, warmup, host, prompts=None):
        """`steps` timed decode steps of `batch` sequences.  Without `prompts` the
        sequences are equal and end at `context` tokens over synthetic keys and values;
        with them (token lists) every sequence is really prefilled through step(),
        eight prompts a step, and decoding goes on from what the model sampled.
        Returns tokens a second, ms per step, the clock record, launches per step and
        the bytes a timed step reads on average."""
        slots = [cache.open_sequence() for _ in range(batch)]
        if prompts is not None:
            prompts = sorted(prompts, key=len, reverse=True)     # longest first, as the generation loop orders a batch
        if prompts is None:
            starts = [context] * batch
            est_ms = (weight_bytes + batch * context * kv_row) / (pk["hbm_gbs"] * 1e6)
        else:
            starts = [len(p) for p in prompts]
            est_ms = (weight_bytes + sum(starts) * kv_row) / (pk["hbm_gbs"] * 1e6)
        # the clocks settle under load: warm up for `warmup` steps and for WARM_MS at least
        warm = max(warmup, int(WARM_MS / est_ms) + 1)
        if prompts is None:
            warm = max(warmup, min(warm, context - steps - 8))
        total = warm + steps + (6 if args.breakdown else 0)
        sampler = ClockSampler()
        sampler.start()
        if prompts is None:
            for s in slots:
                cache.reserve(s, context)
                cache.advance(s, context - total)
            cache.flush_tables()
            tokens = torch.randint(0, vocab, (batch,), generator=gen).tolist()
        else:
            tokens = []
            for lo in range(0, batch, 8):
                part = list(zip(slots[lo:lo + 8], prompts[lo:lo + 8]))
                logits = step(model, cache, [StepEntry(s, p, [len(p) - 1]) for s, p in part])
                tokens += logits.argmax(dim=1).tolist()
            for s, n in zip(slots, starts):
                cache.reserve(s, n + total)
            cache.flush_tables()
        db = DecodeBatch(model, cache, slots, list(range(batch)), lib.Sampler(0.0, 0),
                         use_graph=not args.eager, chained=not args.no_chain)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches_before = ops.launch_count()
        if host:
            out = db.step_host(tokens, [0] * batch)      # eager: loads and configures kernels
            per_step = ops.launch_count() - launches_before
            for i in range(1, warm):
                out = db.step_host(out, [i] * batch)
            torch.cuda.synchronize()
            first = [cache.length(s) for s in slots]
            sampler.mark()
            start.record()
            for i in range(steps):
                out = db.step_host(out, [warm + i] * batch)
            stop.record()
        else:
            db.set_state(tokens, [0] * batch)
            db._launch()                                 # eager: loads and configures kernels
            per_step = ops.launch_count() - launches_before
            for _ in range(warm - 1):
                db.step_device()
            torch.cuda.synchronize()
            first = [cache.length(s) for s in slots]
            sampler.mark()
            start.record()
            for _ in range(steps):
                db.step_device()
            stop.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = start.elapsed_time(stop) / steps
        # a timed step attends over its sequences' keys: their lengths at the middle of the region
        read_bytes = weight_bytes + sum(n + steps // 2 for n in first) * kv_row
        if args.breakdown and not host:
            kernel_breakdown(db.step_device, 6, f"decode step, batch {batch}, mean context {sum(first) / batch:.0f}", args.layers)
        for s in slots:
            cache.close_sequence(s)
        return {"value": batch / (ms * 1e-3), "ms": ms, "clocks": clocks, "launches": per_step + 1,   # +1: the kernel that feeds tokens back
                "bytes": read_bytes, "mean_context": sum(first) / batch + steps / 2}

    def u2048_prompts(n):
        """The decode workload as the benchmark description words it: prompts of lengths
        uniform in [128, 2048], ids uniform in the vocabulary (seeded)."""
        g = torch.Generator().manual_seed(1)
        lengths = torch.randint(128, 2049, (64,), generator=g).tolist()
        prompts = [torch.randint(0, vocab, (k,), generator=g).tolist() for k in lengths]
        if n > 64:                      # more sequences than the named points use: the same draw goes on
            more = torch.randint(128, 2049, (n - 64,), generator=g).tolist()
            prompts += [torch.randint(0, vocab, (k,), generator=g).tolist() for k in more]
        return prompts[:n]

    if args.only == "decode":          # for profilers: the decode steps and nothing else
        r = decode_run(args.batch, args.steps, args.warmup, host=False,
                       prompts=u2048_prompts(args.batch) if args.workload == "u2048" else None)
        print(json.dumps({"only": "decode", "value": round(r["value"], 1), "ms_per_step": round(r["ms"], 4),
                          "launches_per_step": r["launches"], "eager": args.eager}))
        return 0
    if args.only == "prefill":
        return prefill_only(args, model, cache, vocab, gen)
    main_run = decode_run(args.batch, args.steps, args.warmup, host=False)
    e2e_run = decode_run(args.batch, args.steps, args.warmup, host=True)
    points, points_ms, points_roofline, points_context = {}, {}, {}, {}

    def point(name, r):
        points[name] = round(r["value"], 1)
        points_ms[name] = round(r["ms"], 4)
        points_roofline[name] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        points_context[name] = round(r["mean_context"], 1)
    if args.points:
        few = max(3, args.steps // 2)
        for b in (1, 64):
            point(f"decode_b{b}", decode_run(b, few, args.warmup, host=False))
        prompts = u2048_prompts(64)            # really prefilled, then decoded
        for b in (1, 8, 64):
            point(f"decode_b{b}_u2048", decode_run(b, few if b != args.batch else args.steps, args.warmup,
                                                   host=False, prompts=prompts[:b]))

    # prefill of one 2,048-token prompt through the step function: its ids as an array
    # (the figure reported) and as a Python list of ints (what build_context then converts)
    T = 2048
    prompt = torch.randint(0, vocab, (T,), generator=gen)
    pre = {}
    for kind, tokens in (("array", prompt.numpy()), ("list", prompt.tolist())):
        times = []
        for i in range(3 + 5):
            slot = cache.open_sequence()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            step(model, cache, [StepEntry(slot, tokens, [T - 1])])
            b.record()
            torch.cuda.synchronize()
            if i >= 3:
                times.append(a.elapsed_time(b))
            cache.close_sequence(slot)
        pre[kind] = statistics.median(times)
    pre_ms = pre["array"]
    flops = prefill_flops(cfg, args.layers, T)

    ms = main_run["ms"]
    achieved = main_run["bytes"] / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch}, context {context} ({shape_name} shape)",
        "value": round(main_run["value"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": f"{shape_name} shape, random weights", "layers": args.layers,
            "layers_of_model": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "rope_theta": cfg["rope_theta"], "tied_head": bool(cfg["tie_word_embeddings"]),
            "global_batch": args.batch, "seq_len": context,
            "prefill_tokens": T, "parallelism": "single GPU", "l2": "inputs larger than L2",
            "peaks": pk["source"], "graph": "decode step replayed as a CUDA graph",
            "warmup_floor_ms": WARM_MS,
        },
        "clocks": main_run["clocks"],
        "e2e": {"value": round(e2e_run["value"], 1), "unit": "tokens/s", "ms_per_step": round(e2e_run["ms"], 4),
                "h2d_bytes_per_step": 3 * 4 * args.batch, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": main_run["launches"] * args.steps,
        "prefill": {"value": round(T / (pre_ms * 1e-3), 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "tokens_given_as": "array", "ms_from_list": round(pre["list"], 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                     "weight_gb": round(weight_bytes / 1e9, 3),
                     "cache_gb": round((main_run["bytes"] - weight_bytes) / 1e9, 3)},
        "points": points, "points_ms": points_ms, "points_roofline": points_roofline,
        "points_context": points_context,
        "cpu_baseline": cpu_baseline(),
    }
    print(json.dumps(line))
    return 0



# ------------------------------------------------------------------ --design ropovik
def ropovik_shape(width, heads, kv_heads, dim, ff, m_heads, m_dim, m_state, m_groups, vocab=32000):
    """Four layers (recurrence, attention, recurrence, attention, each with a dense
    feed-forward) that run twice: eight layer runs and two loop projections."""
    attn = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                      "rot": {"dims": dim, "base": 10000.0,
                              "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}}
    mamba = {"type": "mamba2", "mlp": {"kind": "dense", "ff": ff},
             "mixer": {"heads": m_heads, "vdim": m_dim, "state": m_state, "groups": m_groups, "conv": 4,
                       "norm_groups": m_groups}}
    return {"architecture": "Ropovik", "vocab": vocab, "width": width, "logit_softcap": 30.0, "norm": {"eps": 1e-5},
            "loop": {"start": 0, "stop": 4, "times": 2}, "layers": [mamba, attn, mamba, attn]}


def senupel_shape(width, heads, ff, experts, expert_ff, top, window=4096, vocab=32000):
    """Eight layers of attention through a latent (heads of 128 unrotated and 64 rotated
    channels, values of 128, a latent of 512, the sizes latent attention is used with);
    the even ones have a down projection and a dense feed-forward, the odd ones read
    the latents of the layer before and route each token to `top` of `experts` experts
    (together as wide as the dense feed-forward)."""
    def mixer(i):
        m = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
             "mask": {"size": window},
             "rot": {"dims": 64, "base": 10000.0, "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}
        if i % 2:
            m["kv_from"] = i - 1
        return m
    dense = {"kind": "dense", "ff": ff}
    routed = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}}
    return {"architecture": "Senupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [{"type": "latent_attention", "mixer": mixer(i), "mlp": routed if i % 2 else dense} for i in range(8)]}


def zotolix_shape(width, heads, kv_heads, dim, experts, expert_ff, top, vocab=32000):
    """Eight layers, unit-norm attention and gated attention in turn, keys seen within
    stretches of 1,024 positions in the even layers and of 8,192 in the odd ones, half of a head
    rotating, every layer's values blended with the first layer's; each token goes to `top` of
    `experts` squared-relu experts; four copies of the hidden state."""
    def mixer(i):
        return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "v_mix": True,
                "mask": {"size": 8192 if i % 2 else 1024}, "rot": {"dims": dim // 2, "base": 500000.0}}
    routed = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}}
    return {"architecture": "Zotolix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
            "residual_mult": 0.8, "streams": 4,
            "layers": [{"type": "attention_2" if i % 2 else "attention", "mixer": mixer(i), "mlp": routed} for i in range(8)]}


def megerax_shape(width, heads, kv_heads, dim, ff, l_heads, l_rank, l_qrank, d_heads, vocab=32000):
    """Eight layers: attention with keys of its own (a causal convolution of four taps over q, k and v, weighted head
    norms, half of a head rotating under wavelength scaling, scores capped at 30, a window of 1,024, the gate on all
    channels), attention through a latent with a query latent and sinks, the gated delta rule (heads of 128 x 128),
    and attention that reads the first layer's keys; twice.  Every layer has a gated gelu feed-forward."""
    rot = {"dims": dim // 2, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    att = lambda src: {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "conv": 4, "rot": rot,
                       "softcap": 30.0, "mask": {"size": 1024}, **({"kv_from": src} if src is not None else {})}
    lat = {"heads": l_heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": l_rank, "q_rank": l_qrank, "scale": 192 ** -0.5,
           "rot": {"dims": 64, "base": 10000.0}}
    dlt = {"heads": d_heads, "kv_heads": d_heads, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 128, "gate_rank": 128}
    mlp = {"kind": "dense", "ff": ff}
    four = lambda at: [{"type": "attention", "mixer": att(None), "mlp": mlp}, {"type": "latent_attention", "mixer": lat, "mlp": mlp},
                       {"type": "channel_delta", "mixer": dlt, "mlp": mlp}, {"type": "attention", "mixer": att(at), "mlp": mlp}]
    return {"architecture": "Megerax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
            "layers": four(0) + four(4)}


DESIGN_SIZES = {
    # the layer sizes of Llama-3.2-1B / SmolLM2 (width 2048) and of Llama-3.1-8B (width 4096); the
    # recurrence has twice the width in its inner size, heads of 64 and a state of 128, as Mamba-2 models do
    "w2048": (ropovik_shape(2048, 32, 8, 64, 8192, 64, 64, 128, 8), dict(LLAMA_3P2_1B, num_hidden_layers=8, vocab_size=32000)),
    "w4096": (ropovik_shape(4096, 32, 8, 128, 14336, 128, 64, 128, 8), dict(LLAMA_3P1_8B, num_hidden_layers=8, vocab_size=32000)),
}


SENUPEL_SIZES = {
    # the same two widths; 16 experts of a quarter of the dense feed-forward's size, four to a token
    "w2048": (senupel_shape(2048, 16, 8192, 16, 2048, 4), dict(LLAMA_3P2_1B, num_hidden_layers=8, vocab_size=32000)),
    "w4096": (senupel_shape(4096, 32, 14336, 16, 3584, 4), dict(LLAMA_3P1_8B, num_hidden_layers=8, vocab_size=32000)),
}
ZOTOLIX_SIZES = {
    # the same two widths and heads as the Llama layers beside them; 16 experts of a quarter of the dense
    # feed-forward's size, four to a token: as many multiplications a token as the dense feed-forward's up and down
    "w2048": (zotolix_shape(2048, 32, 8, 64, 16, 2048, 4), dict(LLAMA_3P2_1B, num_hidden_layers=8, vocab_size=32000)),
    "w4096": (zotolix_shape(4096, 32, 8, 128, 16, 3584, 4), dict(LLAMA_3P1_8B, num_hidden_layers=8, vocab_size=32000)),
}
MEGERAX_SIZES = {
    # the same two widths, heads and feed-forward sizes as the Llama layers beside them; the latent layers keep 512
    # channels a token, the delta layers as many value channels as the width
    "w2048": (megerax_shape(2048, 32, 8, 64, 8192, 16, 512, 768, 16), dict(LLAMA_3P2_1B, num_hidden_layers=8, vocab_size=32000)),
    "w4096": (megerax_shape(4096, 32, 8, 128, 14336, 32, 512, 1536, 32), dict(LLAMA_3P1_8B, num_hidden_layers=8, vocab_size=32000)),
}
DESIGNS = {
    "megerax": (MEGERAX_SIZES, "8 layers: attention with convolved projections, capped scores, a window of 1024 and a gate on all "
                               "channels (two with keys of their own, two reading theirs), attention through a latent with sinks, "
                               "the gated delta rule with heads of 128 x 128; a gated gelu feed-forward each; beside 8 Llama layers "
                               "of equal width, heads and feed-forward size; vocabulary 32000"),
    "zotolix": (ZOTOLIX_SIZES, "8 layers of attention within stretches of 1024 and 8192 positions (unit-norm and gated in turn, biased "
                               "projections, values blended with the first layer's), mixtures of 16 squared-relu experts (4 to a token, "
                               "the router's sigmoid on the input), four copies of the hidden state, beside 8 Llama layers of equal "
                               "width, heads and feed-forward size; vocabulary 32000"),
    "ropovik": (DESIGN_SIZES, "4 layers (mamba2, attention, mamba2, attention, a dense feed-forward each) run twice, "
                              "beside 8 Llama layers of equal width, heads and feed-forward size; vocabulary 32000"),
    "senupel": (SENUPEL_SIZES, "8 layers of attention through a latent (a window of 4096), dense gated feed-forwards with biases "
                               "and mixtures of 16 experts (4 to a token) in turn, odd layers reading the even layers' latents, "
                               "beside 8 Llama layers of equal width and feed-forward size; vocabulary 32000"),
}


def run_design(args):
    """Prefill and decode throughput of a design beside the Llama decoder at
    equal width, depth and heads (random weights, bfloat16), and its own kernels one
    by one against the copy peak beside the like kernel of the Llama path.  One JSON line."""
    import torch
    import go_tinygrad_b200 as lib
    from go_tinygrad_b200.engine import StepEntry, step
    from go_tinygrad_b200.engine.decode import DecodeBatch
    from go_tinygrad_b200.kernels import ops

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    pk = peaks()
    gen = torch.Generator().manual_seed(0)
    T, prompt_len = 2048, 1024
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # larger than the L2

    def timed(fn, repeats=10, warm=3):
        """Median device time of fn() in ms, the L2 flushed before every call."""
        times = []
        for i in range(warm + repeats):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= warm:
                times.append(a.elapsed_time(b))
        return statistics.median(times)

    def model_numbers(cfg):
        model = lib.Model.random(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02)
        vocab = model.plan.vocab_size
        cache = model.new_cache(max_tokens=64 * (prompt_len + 256) + T + 64, max_slots=65)
        out = {}
        prompt = torch.randint(0, vocab, (T,), generator=gen).numpy()

        def prefill():
            slot = cache.open_sequence()
            step(model, cache, [StepEntry(slot, prompt, [T - 1])])
            cache.close_sequence(slot)
        ms = timed(prefill, repeats=5)
        out["prefill_2048"] = {"ms": round(ms, 3), "tokens_per_s": round(T / ms * 1e3, 1)}
        for batch in (8, 64):
            slots = [cache.open_sequence() for _ in range(batch)]
            prompts = [torch.randint(0, vocab, (prompt_len,), generator=gen).numpy() for _ in range(batch)]
            tokens = []
            for lo in range(0, batch, 8):
                logits = step(model, cache, [StepEntry(s, p, [prompt_len - 1]) for s, p in zip(slots[lo:lo + 8], prompts[lo:lo + 8])])
                tokens += logits.argmax(dim=1).tolist()
            steps, warm = args.steps, max(args.warmup, 10)
            for s in slots:
                cache.reserve(s, prompt_len + steps + warm + 2)
            cache.flush_tables()
            db = DecodeBatch(model, cache, slots, list(range(batch)), lib.Sampler(0.0, 0))
            db.set_state(tokens, [0] * batch)
            before = ops.launch_count()
            db._launch()
            launches = ops.launch_count() - before + 1
            for _ in range(warm):
                db.step_device()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                db.step_device()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / steps
            out[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3, 1),
                                       "context": prompt_len, "launches_per_step": launches}
            for s in slots:
                cache.close_sequence(s)
        out["weight_gb"] = round(model.weight_bytes() / 1e9, 3)
        del model, cache
        torch.cuda.empty_cache()
        return out

    def senupel_kernel_table(cfg):
        """Each kernel the Senupel design added, alone, at this size: a prompt of T tokens
        and a decode step of 64 sequences after 1,024 tokens; the bytes it has to move
        against the copy peak and, for the products, its FLOPs against the matrix peak.
        Beside each the like kernel of the Llama path at the same rows."""
        from go_tinygrad_b200.cache import Cache, KVRequest
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        m = cfg["layers"][0]["mixer"]
        ex = cfg["layers"][1]["mlp"]
        H, heads, dim, rot, vdim, rank, window = cfg["width"], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["mask"]["size"]
        ff, E, eff, top = cfg["layers"][0]["mlp"]["ff"], ex["router"]["experts"], ex["expert"]["ff"], ex["router"]["top"]
        row = rank + rot
        rows = []

        def add(name, rows_n, ms, nbytes, flops=0, like=None):
            rows.append({"kernel": name, "rows": rows_n, "us": round(ms * 1e3, 2), "mb": round(nbytes / 1e6, 2),
                         "of_copy_peak": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3),
                         **({"tflops": round(flops / ms / 1e9, 1), "of_matrix_peak": round(flops / ms / 1e9 / pk["bf16_tflops"], 3)} if flops else {}),
                         **({"like": like} if like else {})})
        rnd = lambda *shape, dtype=bf: torch.randn(*shape, device=dev, dtype=f32).to(dtype)
        for n, n_seqs, ctx_len, tag in ((T, 1, 0, "prompt"), (64, 64, prompt_len, "decode")):
            per = n // n_seqs
            rt = lib.parts.Runtime(dev, bf)
            cache = Cache([[KVRequest(1, row, window, planes=1)], [KVRequest(heads // 2, 128, None)]], [None, None],
                          max_tokens=64 * ((ctx_len + per + 63) // 64) * n_seqs, max_slots=n_seqs, dtype=bf, device=dev)
            slot_list = [cache.open_sequence() for _ in range(n_seqs)]
            cache.reserve_many([(s, ctx_len + per) for s in slot_list]); cache.flush_tables()
            for g in cache.groups:
                g.storage.normal_()
            kv, kv_like = cache.handles[0].kv, cache.handles[1].kv
            cu = torch.arange(0, n + 1, per, dtype=i32, device=dev)
            seq = torch.arange(n, dtype=i32, device=dev) // per
            slots = torch.tensor(slot_list, dtype=i32, device=dev)
            start = torch.full((n_seqs,), ctx_len, dtype=i32, device=dev)
            pos = (start[seq.long()] + (torch.arange(n, device=dev) % per)).to(i32)
            # the norm on a sublayer's output, beside the norm before a sublayer
            res, upd, w = rnd(n, H, dtype=f32), rnd(n, H), rnd(H, dtype=f32)
            image, out = torch.empty(n, H, dtype=bf, device=dev), torch.empty(n, H, dtype=bf, device=dev)
            add(f"rmsnorm_add ({tag})", n, timed(lambda: ops.rmsnorm_add(upd, w, 1e-5, res, image)), n * H * (2 + 4 + 4 + 2))
            add(f"add_rmsnorm ({tag})", n, timed(lambda: ops.add_rmsnorm(res, upd, w, 1e-5, out)), n * H * (4 + 4 + 2 + 2), like="rmsnorm_add")
            # latent norm, rotation and cache store, beside rotation and store of ordinary heads
            q, dkv = rnd(n, heads * (dim + rot)), rnd(n, row)
            cs, nw = rnd(n, rot // 2, 2, dtype=f32), rnd(rank, dtype=f32)
            folded = torch.empty(n, heads * row, dtype=bf, device=dev)
            add(f"latent_prepare ({tag})", n, timed(lambda: ops.latent_prepare(q, dkv, cs, nw, 1e-5, kv, seq, slots, pos, folded, heads, dim, rot, rank)),
                n * (row * 4 + heads * rot * 4))
            qkv, cs2 = rnd(n, (heads + heads) * 128), rnd(n, 64, 2, dtype=f32)
            add(f"rope_kv_store ({tag})", n, timed(lambda: ops.rope_kv_store(qkv, cs2, heads, heads // 2, 128, kv_like, seq, slots, pos)),
                n * (heads * 128 * 4 + heads * 128 * 3), like="latent_prepare")
            # the products per head, beside one product of the same size
            w_uk, w_uv = rnd(heads, rank, dim), rnd(heads, vdim, rank)
            att, hd, gate = rnd(n, heads * rank), torch.empty(n, heads * vdim, dtype=bf, device=dev), rnd(n, heads * vdim)
            fl = 2 * n * heads * dim * rank
            add(f"linear_heads fold ({tag})", n, timed(lambda: ops.linear_heads(q.view(n, heads, dim + rot)[:, :, :dim], w_uk, folded.view(n, heads, row)[:, :, :rank])),
                w_uk.numel() * 2 + n * heads * (dim + rank) * 2, fl)
            add(f"linear_heads values + gate ({tag})", n, timed(lambda: ops.linear_heads(att.view(n, heads, rank), w_uv, hd.view(n, heads, vdim), gate.view(n, heads, vdim))),
                w_uv.numel() * 2 + n * heads * (rank + 2 * vdim) * 2, fl)
            wl, xl, ol = rnd(rank, heads * dim), rnd(n, heads * dim), torch.empty(n, rank, dtype=bf, device=dev)
            add(f"linear, as many FLOPs ({tag})", n, timed(lambda: ops.linear(xl, wl, ol)), wl.numel() * 2 + n * (heads * dim + rank) * 2, fl, like="linear_heads")
            # attention
            keys = (ctx_len + per) * n_seqs if per == 1 else sum(min(i + 1, window) for i in range(per))
            splits, floats = ops.latent_attention_plan(n_seqs, per, heads, row, rank, ctx_len + per, window)
            runs = torch.empty(max(1, n * floats), dtype=f32, device=dev)
            add(f"latent_attention, keys in {splits} run(s) ({tag}{', as a portion would run' if per > 1 else ''})", n,
                timed(lambda: ops.latent_attention_bf16(folded, att, kv, cu, slots, start, n_seqs, per, heads, rank, 0.07, window, splits, runs)),
                n * heads * (row + rank) * 2 + (n_seqs * (ctx_len + per)) * row * 2, 2 * heads * keys * (row + rank))
            if per > 1:
                # a whole prompt: its rows expanded per head by one product, and attention over those
                per_head = dim + vdim + rot
                w_exp, lat = rnd(heads * per_head, rank), rnd(n, row)
                runs = torch.empty(n, heads * per_head, dtype=bf, device=dev)
                add(f"linear, the prompt's rows per head ({tag})", n, timed(lambda: ops.linear(lat[:, :rank], w_exp, runs)),
                    w_exp.numel() * 2 + n * (rank + heads * per_head) * 2, 2 * n * heads * per_head * rank)
                add(f"latent_spread ({tag})", n, timed(lambda: ops.latent_spread(lat[:, rank:], runs, heads, dim + vdim)), n * (heads + 1) * rot * 2)
                add(f"expanded_attention ({tag})", n,
                    timed(lambda: ops.expanded_attention_bf16(q, runs, hd, cu, n_seqs, per, heads, dim, rot, vdim, 0.07, window)),
                    n * heads * (dim + rot + per_head + vdim) * 2, 2 * heads * keys * (dim + rot + vdim))
            ql, ml = rnd(n, heads * 128), torch.empty(n, heads * 128, dtype=bf, device=dev)
            if per == 1:
                splits, chunk, ring = ops.attention_decode_plan(n, heads, heads // 2, 128, ctx_len + 1, 0, n * (ctx_len + 1))
                scratch = torch.empty(max(1, ops.attention_decode_scratch_floats(n, heads, 128, splits)), dtype=f32, device=dev)
                fn = lambda: ops.attention_decode_bf16(ql, ml, kv_like, slots, pos, heads, 0.09, 0, splits, scratch, chunk_pages=chunk, ring_pages=ring)
            else:
                fn = lambda: ops.attention_prefill_tcgen05(ql, ml, kv_like, cu, slots, start, n_seqs, per, heads, 0.09, 0)
            add(f"attention, {heads} heads of 128 on {heads // 2} key heads ({tag})", n, timed(fn),
                n * heads * 128 * 4 + n_seqs * (ctx_len + per) * (heads // 2) * 128 * 4, 2 * heads * keys * 256, like="latent_attention")
            # biases
            sums, bg, act = rnd(n, 2 * ff, dtype=f32), rnd(ff, dtype=f32), torch.empty(n, ff, dtype=bf, device=dev)
            add(f"swiglu_bias ({tag})", n, timed(lambda: ops.swiglu_bias(sums, bg, bg, act)), n * ff * (8 + 2))
            gu = rnd(n, 2 * ff)
            add(f"swiglu ({tag})", n, timed(lambda: ops.swiglu(gu, act)), n * ff * 6, like="swiglu_bias")
            ys, bd = rnd(n, H, dtype=f32), rnd(H, dtype=f32)
            add(f"add_bias ({tag})", n, timed(lambda: ops.add_bias(ys, bd, out)), n * H * 6)
            # routed experts
            x, router, rb = rnd(n, H), rnd(E, H, dtype=f32), rnd(E, dtype=f32)
            chosen, wts = torch.empty(n, top, dtype=i32, device=dev), torch.empty(n, top, dtype=f32, device=dev)
            add(f"moe_route ({tag})", n, timed(lambda: ops.moe_route(x, router, rb, chosen, wts)), n * H * 2 + E * H * 4)
            tile = 128 if n * top >= 128 * E else 64
            tiles = ops.moe_tiles_cap(n * top, E, tile)
            row_item, item_row = torch.empty(tiles * tile, dtype=i32, device=dev), torch.empty(n * top, dtype=i32, device=dev)
            tile_expert = torch.empty(tiles, dtype=i32, device=dev)
            add(f"moe_arrange ({tag})", n, timed(lambda: ops.moe_arrange(chosen, E, row_item, item_row, tile_expert, tile)), n * top * 12)
            wgu, wd = rnd(E, 2 * eff, H), rnd(E, H, eff)
            acts, y = torch.empty(tiles * tile, eff, dtype=bf, device=dev), torch.empty(tiles * tile, H, dtype=f32, device=dev)
            used = min(E, n * top)
            if tile == 128:
                # as the part does for prompts: the inputs copied into arranged order, then the product over them
                gathered = torch.empty(tiles * tile, H, dtype=bf, device=dev)
                add(f"moe_gather ({tag})", n, timed(lambda: ops.moe_gather(x, row_item, top, gathered)), n * H * 2 + n * top * H * 2)
                add(f"moe_product gate, up, silu ({tag})", n, timed(lambda: ops.moe_product(gathered, row_item, 0, wgu, tile_expert, acts, epilogue="swiglu")),
                    used * 2 * eff * H * 2 + n * top * (H + eff) * 2, 2 * n * top * 2 * eff * H)
            else:
                add(f"moe_product gate, up, silu ({tag})", n, timed(lambda: ops.moe_product(x, row_item, top, wgu, tile_expert, acts, epilogue="swiglu")),
                    used * 2 * eff * H * 2 + n * H * 2 + n * top * eff * 2, 2 * n * top * 2 * eff * H)
            add(f"moe_product down ({tag})", n, timed(lambda: ops.moe_product(acts, row_item, 0, wd, tile_expert, y)),
                used * eff * H * 2 + n * top * (eff * 2 + H * 4), 2 * n * top * eff * H)
            wg2, a2 = rnd(2 * eff * top, H), torch.empty(n, eff * top, dtype=bf, device=dev)
            add(f"linear gate, up, silu of {top} experts' width ({tag})", n, timed(lambda: ops.linear(x, wg2, a2, epilogue="swiglu")),
                wg2.numel() * 2 + n * (H + eff * top) * 2, 2 * n * top * 2 * eff * H, like="moe_product")
            add(f"moe_combine ({tag})", n, timed(lambda: ops.moe_combine(y, item_row, wts, out)), n * top * H * 4 + n * H * 2)
            del cache
        return rows

    def megerax_kernel_table(cfg):
        """Each kernel the Megerax design added or extended, alone, at this size: a prompt of T tokens
        and a decode step of 64 sequences after 1,024 tokens; the bytes it has to move against the copy
        peak and, for products and attention, its FLOPs against the matrix peak.  Beside each the like
        kernel of the Llama path (of the Ropovik path for the recurrence) at the same rows."""
        from go_tinygrad_b200.cache import Cache, KVRequest
        from go_tinygrad_b200.parts.base import StepContext
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        a, d = cfg["layers"][0]["mixer"], cfg["layers"][2]["mixer"]
        H, heads, n_kv, hd, taps, window, cap = cfg["width"], a["heads"], a["kv_heads"], a["dim"], a["conv"], a["mask"]["size"], a["softcap"]
        ff = cfg["layers"][0]["mlp"]["ff"]
        dh, dd, dv, dtaps = d["heads"], d["dim"], d["vdim"], d["conv"]
        rows = []

        def add(name, rows_n, ms, nbytes, flops=0, like=None):
            rows.append({"kernel": name, "rows": rows_n, "us": round(ms * 1e3, 2), "mb": round(nbytes / 1e6, 2),
                         "of_copy_peak": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3),
                         **({"tflops": round(flops / ms / 1e9, 1), "of_matrix_peak": round(flops / ms / 1e9 / pk["bf16_tflops"], 3)} if flops else {}),
                         **({"like": like} if like else {})})
        rnd = lambda *shape, dtype=bf: torch.randn(*shape, device=dev, dtype=f32).to(dtype)
        for n, n_seqs, ctx_len, tag in ((T, 1, 0, "prompt"), (64, 64, prompt_len, "decode")):
            per = n // n_seqs
            rt = lib.parts.Runtime(dev, bf)
            cache = Cache([[KVRequest(n_kv, hd, None, value_dim=hd)]], [None],
                          max_tokens=64 * ((ctx_len + per + 63) // 64) * n_seqs, max_slots=n_seqs, dtype=bf, device=dev)
            slot_list = [cache.open_sequence() for _ in range(n_seqs)]
            cache.reserve_many([(s, ctx_len + per) for s in slot_list]); cache.flush_tables()
            for g in cache.groups:
                g.storage.normal_()
            kv = cache.handles[0].kv
            cu = torch.arange(0, n + 1, per, dtype=i32, device=dev)
            seq = torch.arange(n, dtype=i32, device=dev) // per
            slots = torch.tensor(slot_list, dtype=i32, device=dev)
            start = torch.full((n_seqs,), ctx_len, dtype=i32, device=dev)
            pos = (start[seq.long()] + (torch.arange(n, device=dev) % per)).to(i32)
            ctx = StepContext(rt=rt, n_tokens=n, n_seqs=n_seqs, tokens=seq, positions=pos, token_seq=seq, cu_seqlens=cu, slots=slots,
                              start_pos=start, max_q_len=per, max_kv_len=ctx_len + per, is_decode=per == 1, total_kv_len=n_seqs * (ctx_len + per))
            # the norm behind the embedding, beside the norm before a sublayer
            res, upd, w = rnd(n, H, dtype=f32), rnd(n, H), rnd(H, dtype=f32)
            out = torch.empty(n, H, dtype=bf, device=dev)
            add(f"rmsnorm_rows ({tag})", n, timed(lambda: ops.rmsnorm_rows(res, w, 1e-5)), n * H * 8)
            add(f"add_rmsnorm ({tag})", n, timed(lambda: ops.add_rmsnorm(res, upd, w, 1e-5, out)), n * H * (4 + 4 + 2 + 2), like="rmsnorm_rows")
            # bias, convolution, head norms, rotation and cache store, beside rotation and store alone
            C = (heads + 2 * n_kv) * hd
            sums, bias, cw = rnd(n, C + heads * hd, dtype=f32), rnd(C, dtype=f32), rnd(taps, C, dtype=f32)
            state = torch.zeros(n_seqs, taps - 1, C, dtype=f32, device=dev)
            nq, nk, cs = rnd(hd, dtype=f32), rnd(hd, dtype=f32), rnd(n, hd // 4, 2, dtype=f32)
            q = torch.empty(n, heads * hd, dtype=bf, device=dev)
            add(f"qkv_conv_finish ({tag})", n, timed(lambda: ops.qkv_conv_finish(sums, bias, cw, state, cu, nq, nk, 1e-5, cs, True, heads, n_kv, hd, hd, kv, q, seq, slots, pos, one_token_each=per == 1)),
                n * C * (4 + 2))
            add(f"conv_state_update ({tag})", n, timed(lambda: ops.conv_state_update(sums[:, :C], state, cu, slots, n_seqs)), n_seqs * (taps - 1) * C * 8)
            qkv, cs2 = rnd(n, C), rnd(n, hd // 2, 2, dtype=f32)
            kv_plain = Cache([[KVRequest(n_kv, hd, None)]], [None], max_tokens=64 * ((ctx_len + per + 63) // 64) * n_seqs, max_slots=n_seqs, dtype=bf, device=dev)
            for s in slot_list:
                kv_plain.open_sequence()
            kv_plain.reserve_many([(s, ctx_len + per) for s in slot_list]); kv_plain.flush_tables()
            kv_plain.groups[0].storage.normal_()
            kvl = kv_plain.handles[0].kv
            add(f"rope_kv_store ({tag})", n, timed(lambda: ops.rope_kv_store(qkv, cs2, heads, n_kv, hd, kvl, seq, slots, pos)), n * C * (2 + 2), like="qkv_conv_finish")
            # attention with capped scores, the window and the gate on all channels, beside attention over all keys
            mixed = torch.empty(n, heads * hd, dtype=bf, device=dev)
            logits = sums[:, C:]
            keys = n_seqs * min(ctx_len + 1, window) if per == 1 else sum(min(i + 1, window) for i in range(per))
            add(f"attention, capped, window {window}, gated ({tag})", n,
                timed(lambda: ops.attention_general(q, mixed, kv, ctx, heads, hd ** -0.5, window=window, softcap=cap, gate_logits=logits)),
                n * heads * hd * (2 + 2 + 4) + n_seqs * n_kv * min(ctx_len + per, window + per) * hd * 4, 4 * heads * keys * hd)
            add(f"attention, window {window} alone ({tag})", n,
                timed(lambda: ops.attention_general(q, mixed, kv, ctx, heads, hd ** -0.5, window=window)),
                n * heads * hd * 4 + n_seqs * n_kv * min(ctx_len + per, window + per) * hd * 4, 4 * heads * keys * hd, like="attention, capped")
            if per == 1:
                splits, chunk, ring = ops.attention_decode_plan(n, heads, n_kv, hd, ctx_len + 1, window, n * (ctx_len + 1))
                scratch = torch.empty(max(1, ops.attention_decode_scratch_floats(n, heads, hd, splits)), dtype=f32, device=dev)
                fn = lambda: ops.attention_decode_bf16(q, mixed, kvl, slots, pos, heads, hd ** -0.5, window, splits, scratch, chunk_pages=chunk, ring_pages=ring)
                add(f"split-KV decode attention, window {window} ({tag})", n, timed(fn),
                    n * heads * hd * 4 + n_seqs * n_kv * min(ctx_len + per, window + per) * hd * 4, 4 * heads * keys * hd, like="attention, capped")
            # the delta rule: convolution with silu, preparation, recurrence, norm and gate; beside the state-space recurrence
            W = 2 * dh * dd + dh * dv
            dsums, dcw = rnd(n, W + dh, dtype=f32), rnd(dtaps, W, dtype=f32)
            dstate = torch.zeros(n_seqs, dtaps - 1, W, dtype=f32, device=dev)
            qkv_f = torch.empty(n, W, dtype=f32, device=dev)
            add(f"causal_conv_silu, float ({tag})", n,
                timed(lambda: ops.causal_conv_silu(dsums[:, :W], dcw, None, dstate, qkv_f, seq, cu, slots, n_seqs=n_seqs, update_state=True, one_token_each=per == 1)),
                n * W * 8)
            decay, beta = rnd(n, dh * dd, dtype=f32), torch.empty(n, dh, dtype=f32, device=dev)
            dtb, alog = rnd(dh * dd, dtype=f32), rnd(dh, dtype=f32)
            raw = decay.clone()
            def prep():
                decay.copy_(raw)
                ops.delta_prepare(qkv_f, decay, dtb, alog, dsums[:, W:], beta, dh, dh, dd, 1e-6, dd ** -0.5)
            add(f"delta_prepare, with a copy of the decays before it ({tag})", n, timed(prep), n * (2 * dh * dd * 8 + dh * dd * 16))
            S = torch.zeros(n_seqs, dh, dd, dv, dtype=f32, device=dev)
            y = torch.empty(n, dh * dv, dtype=f32, device=dev)
            add(f"delta_scan ({tag})", n, timed(lambda: ops.delta_scan(qkv_f, qkv_f[:, 2 * dh * dd:], decay, beta, S, y, cu, slots, n_seqs, dh, dh, dd, dv)),
                n * (3 * dh * dd + 2 * dh * dv) * 4 + n_seqs * dh * dd * dv * 8)
            gate_l, nw = rnd(n, dh * dv, dtype=f32), rnd(dv, dtype=f32)
            outd = torch.empty(n, dh * dv, dtype=bf, device=dev)
            add(f"head_norm_gate ({tag})", n, timed(lambda: ops.head_norm_gate(y, gate_l, nw, 1e-5, outd, dh)), n * dh * dv * (4 + 4 + 2))
            # the like kernels of the state-space path at equal inner size: heads of 64, a state of 128
            mh, mp, ms_, mg = dh * dv // 64, 64, 128, 8
            xs, bc = rnd(n, mh * mp), rnd(n, mg * ms_, 2, dtype=f32)
            dt_raw, dtb2, alog2, skip = rnd(n, mh), rnd(mh, dtype=f32), rnd(mh, dtype=f32), rnd(mh, dtype=f32)
            S2 = torch.zeros(n_seqs, mh, ms_, mp, dtype=f32, device=dev)
            y2 = torch.empty(n, mh * mp, dtype=f32, device=dev)
            add(f"ssm_scan ({tag})", n, timed(lambda: ops.ssm_scan(xs, bc, dt_raw, dtb2, alog2, skip, S2, y2, cu, slots, n_seqs, mh, mg, ms_, mp, one_token_each=per == 1)),
                n * (mh * mp * 6 + mg * ms_ * 8) + n_seqs * mh * ms_ * mp * 8, like="delta_scan")
            z, gw = rnd(n, mh * mp), rnd(mh * mp, dtype=f32)
            og = torch.empty(n, mh * mp, dtype=bf, device=dev)
            add(f"gated_rmsnorm ({tag})", n, timed(lambda: ops.gated_rmsnorm(y2, z, gw, 1e-5, og, mg)), n * mh * mp * (4 + 2 + 2), like="head_norm_gate")
            # the gated feed-forward's first product with gelu on the gate in its epilogue, beside silu
            x, wgu = rnd(n, H), rnd(2 * ff, H)
            act = torch.empty(n, ff, dtype=bf, device=dev)
            fl = 2 * n * 2 * ff * H
            add(f"gate/up product, gelu on the gate ({tag})", n, timed(lambda: ops.linear(x, wgu, act, epilogue="gated_gelu_tanh")), wgu.numel() * 2 + n * (H + ff) * 2, fl)
            add(f"gate/up product, silu on the gate ({tag})", n, timed(lambda: ops.linear(x, wgu, act, epilogue="swiglu")), wgu.numel() * 2 + n * (H + ff) * 2, fl, like="gelu on the gate")
            del cache, kv_plain
        return rows

    def zotolix_kernel_table(cfg):
        """Each kernel the Zotolix design added or extended, alone, at this size: a prompt of T
        tokens and a decode step of 64 sequences at the last place of a stretch; the bytes it has to move
        against the copy peak and, for products and attention, its FLOPs against the matrix
        peak.  Beside each the like kernel of the Llama path (of the Senupel path for the
        experts) at the same rows."""
        from go_tinygrad_b200.cache import Cache, KVRequest
        from go_tinygrad_b200.parts.base import StepContext
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        m, ex = cfg["layers"][0]["mixer"], cfg["layers"][0]["mlp"]
        H, heads, n_kv, hd, vd, chunk, S = cfg["width"], m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"], cfg["streams"]
        E, eff, top = ex["router"]["experts"], ex["expert"]["ff"], ex["router"]["top"]
        rows = []

        def add(name, rows_n, ms, nbytes, flops=0, like=None):
            rows.append({"kernel": name, "rows": rows_n, "us": round(ms * 1e3, 2), "mb": round(nbytes / 1e6, 2),
                         "of_copy_peak": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3),
                         **({"tflops": round(flops / ms / 1e9, 1), "of_matrix_peak": round(flops / ms / 1e9 / pk["bf16_tflops"], 3)} if flops else {}),
                         **({"like": like} if like else {})})
        rnd = lambda *shape, dtype=bf: torch.randn(*shape, device=dev, dtype=f32).to(dtype)
        # the decode step stands at the last place of a stretch, where it sees the most keys
        for n, n_seqs, ctx_len, tag in ((T, 1, 0, "prompt"), (64, 64, max(prompt_len, chunk) // chunk * chunk - 1, "decode")):
            per = n // n_seqs
            rt = lib.parts.Runtime(dev, bf)
            cache = Cache([[KVRequest(n_kv, hd, None, value_dim=vd, chunk=chunk)], [KVRequest(n_kv, hd, None)],
                           [KVRequest(n_kv, hd, None, value_dim=hd // 2, chunk=chunk)]], [None, None, None],
                          max_tokens=64 * ((ctx_len + per + 63) // 64) * n_seqs, max_slots=n_seqs, dtype=bf, device=dev)
            slot_list = [cache.open_sequence() for _ in range(n_seqs)]
            cache.reserve_many([(s, ctx_len + per) for s in slot_list]); cache.flush_tables()
            for g in cache.groups:
                g.storage.normal_()
            kv, kv_like, kv_narrow = (h.kv for h in cache.handles)
            cu = torch.arange(0, n + 1, per, dtype=i32, device=dev)
            seq = torch.arange(n, dtype=i32, device=dev) // per
            slots = torch.tensor(slot_list, dtype=i32, device=dev)
            start = torch.full((n_seqs,), ctx_len, dtype=i32, device=dev)
            pos = (start[seq.long()] + (torch.arange(n, device=dev) % per)).to(i32)
            ctx = StepContext(rt=rt, n_tokens=n, n_seqs=n_seqs, tokens=seq, positions=pos, token_seq=seq, cu_seqlens=cu, slots=slots,
                              start_pos=start, max_q_len=per, max_kv_len=ctx_len + per, is_decode=per == 1,
                              total_kv_len=n_seqs * (ctx_len + per))
            # the copies of the hidden state: update, read and norm in one pass, beside add + norm of one copy
            copies, upd, w = rnd(n, S, H, dtype=f32), rnd(n, H, dtype=f32), rnd(H, dtype=f32)
            mix, ow, iw = rnd(S, S, dtype=f32), rnd(S, dtype=f32), rnd(S, dtype=f32)
            out = torch.empty(n, H, dtype=bf, device=dev)
            add(f"hyper_norm, {S} copies ({tag})", n, timed(lambda: ops.hyper_norm(copies, w, 1e-5, out, update=upd, mix=mix, out_w=ow, in_w=iw)),
                n * H * (8 * S + 4 + 2))
            res, pend = rnd(n, H, dtype=f32), rnd(n, H)
            add(f"add_rmsnorm ({tag})", n, timed(lambda: ops.add_rmsnorm(res, pend, w, 1e-5, out)), n * H * (4 + 4 + 2 + 2), like="hyper_norm")
            # what stands between projection and attention, beside rotation and store of the Llama path
            width = heads * hd + n_kv * (hd + vd) + heads
            sums, bias = rnd(n, (width + 7) // 8 * 8, dtype=f32), rnd(width - heads, dtype=f32)
            cs = rnd(n, m["rot"]["dims"] // 2, 2, dtype=f32)
            q, gate = torch.empty(n, heads * hd, dtype=bf, device=dev), torch.empty(n, heads, dtype=f32, device=dev)
            vf = rnd(n, n_kv * vd, dtype=f32)
            add(f"qkv_finish ({tag})", n, timed(lambda: ops.qkv_finish(sums, bias, cs, heads, kv, q, seq, slots, pos, unit_norm=True, eps=1e-5,
                                                                       v_first=vf, blend=0.3, gate_out=gate)),
                n * (width * 4 + heads * hd * 2 + n_kv * (hd + vd) * 2 + n_kv * vd * 4))
            qkv, cs2 = rnd(n, (heads + 2 * n_kv) * hd), rnd(n, hd // 2, 2, dtype=f32)
            add(f"rope_kv_store ({tag})", n, timed(lambda: ops.rope_kv_store(qkv, cs2, heads, n_kv, hd, kv_like, seq, slots, pos)),
                n * (heads + 2 * n_kv) * hd * 4, like="qkv_finish")
            # attention within stretches, as the mixer runs it, beside the Llama path's at the same heads
            keys = sum(min(i % chunk + 1, i + 1) for i in range(ctx_len, ctx_len + per)) * n_seqs
            seen = min(ctx_len + per, chunk if per > 1 else ((ctx_len) % chunk + 1))
            mixed = torch.empty(n, heads * vd, dtype=bf, device=dev)
            att_bytes = n * heads * (hd + vd) * 2 + n_seqs * seen * n_kv * (hd + vd) * 2
            add(f"attention within stretches of {chunk} ({tag})", n,
                timed(lambda: ops.attention_general(q, mixed, kv, ctx, heads, hd ** -0.5, chunk=chunk, gate=gate)), att_bytes, 2 * heads * keys * (hd + vd))
            narrow = torch.empty(n, heads * (hd // 2), dtype=bf, device=dev)
            add(f"the same with values of {hd // 2} channels: attention_masked ({tag})", n,
                timed(lambda: ops.attention_general(q, narrow, kv_narrow, ctx, heads, hd ** -0.5, chunk=chunk, gate=gate)),
                n * heads * (hd + hd // 2) * 2 + n_seqs * seen * n_kv * (hd + hd // 2) * 2, 2 * heads * keys * (hd + hd // 2))
            ql, ml = rnd(n, heads * hd), torch.empty(n, heads * hd, dtype=bf, device=dev)
            if per == 1:
                splits, chunk_pages, ring = ops.attention_decode_plan(n, heads, n_kv, hd, ctx_len + 1, 0, n * (ctx_len + 1))
                scratch = torch.empty(max(1, ops.attention_decode_scratch_floats(n, heads, hd, splits)), dtype=f32, device=dev)
                fn = lambda: ops.attention_decode_bf16(ql, ml, kv_like, slots, pos, heads, hd ** -0.5, 0, splits, scratch, chunk_pages=chunk_pages, ring_pages=ring)
                like_keys, like_seen = n_seqs * (ctx_len + 1), ctx_len + 1
            else:
                fn = lambda: ops.attention_prefill_tcgen05(ql, ml, kv_like, cu, slots, start, n_seqs, per, heads, hd ** -0.5, 0)
                like_keys, like_seen = per * (per + 1) // 2, per
            add(f"attention over all keys, the Llama path ({tag})", n, timed(fn),
                n * heads * hd * 4 + n_seqs * like_seen * n_kv * hd * 4, 2 * heads * like_keys * 2 * hd, like="attention within stretches")
            # the experts, beside the gated experts of the Senupel path
            x, router = rnd(n, H), rnd(E, H, dtype=f32)
            chosen, wts = torch.empty(n, top, dtype=i32, device=dev), torch.empty(n, top, dtype=f32, device=dev)
            add(f"moe_route, sigmoid scores ({tag})", n, timed(lambda: ops.moe_route(x, router, None, chosen, wts, "sigmoid")), n * H * 2 + E * H * 4)
            add(f"moe_route, softmax over the chosen ({tag})", n, timed(lambda: ops.moe_route(x, router, None, chosen, wts)), n * H * 2 + E * H * 4, like="moe_route")
            ops.moe_route(x, router, None, chosen, wts, "sigmoid")
            tile = 128 if n * top >= 128 * E else 64
            tiles = ops.moe_tiles_cap(n * top, E, tile)
            row_item, item_row = torch.empty(tiles * tile, dtype=i32, device=dev), torch.empty(n * top, dtype=i32, device=dev)
            tile_expert = torch.empty(tiles, dtype=i32, device=dev)
            ops.moe_arrange(chosen, E, row_item, item_row, tile_expert, tile)
            gathered = torch.empty(tiles * tile, H, dtype=bf, device=dev)
            add(f"moe_gather, rows times their scores ({tag})", n, timed(lambda: ops.moe_gather(x, row_item, top, gathered, weights=wts)), n * H * 2 + n * top * H * 2)
            add(f"moe_gather ({tag})", n, timed(lambda: ops.moe_gather(x, row_item, top, gathered)), n * H * 2 + n * top * H * 2, like="moe_gather")
            wu, wgu, wd = rnd(E, eff, H), rnd(E, 2 * eff, H), rnd(E, H, eff)
            acts, y = torch.empty(tiles * tile, eff, dtype=bf, device=dev), torch.empty(tiles * tile, H, dtype=f32, device=dev)
            used = min(E, n * top)
            add(f"moe_product up, squared relu ({tag})", n, timed(lambda: ops.moe_product(gathered, row_item, 0, wu, tile_expert, acts, epilogue="relu2")),
                used * eff * H * 2 + n * top * (H + eff) * 2, 2 * n * top * eff * H)
            add(f"moe_product gate, up, silu ({tag})", n, timed(lambda: ops.moe_product(gathered, row_item, 0, wgu, tile_expert, acts, epilogue="swiglu")),
                used * 2 * eff * H * 2 + n * top * (H + eff) * 2, 2 * n * top * 2 * eff * H, like="moe_product up")
            add(f"moe_product down ({tag})", n, timed(lambda: ops.moe_product(acts, row_item, 0, wd, tile_expert, y)),
                used * eff * H * 2 + n * top * (eff * 2 + H * 4), 2 * n * top * eff * H)
            outf = torch.empty(n, H, dtype=f32, device=dev)
            add(f"moe_combine, plain sum ({tag})", n, timed(lambda: ops.moe_combine(y, item_row, None, outf)), n * top * H * 4 + n * H * 4)
            add(f"moe_combine, weighted ({tag})", n, timed(lambda: ops.moe_combine(y, item_row, wts, outf)), n * top * H * 4 + n * H * 4, like="moe_combine")
            del cache
        return rows

    def kernel_table(cfg):
        """Each kernel the design added, alone, at this size: a prompt of T tokens and a
        decode step of 64 sequences; bytes it has to move / time / the copy peak.  Beside
        each the like kernel of the Llama path at the same rows."""
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        m = cfg["layers"][0]["mixer"]
        at = cfg["layers"][1]["mixer"]
        H, heads, P, N, G, taps = cfg["width"], m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
        inner, conv_dim = heads * P, heads * P + 2 * G * N
        ff = cfg["layers"][0]["mlp"]["ff"]
        rows = []

        def add(name, rows_n, ms, nbytes, like=None):
            rows.append({"kernel": name, "rows": rows_n, "us": round(ms * 1e3, 2), "mb": round(nbytes / 1e6, 2),
                         "gbs": round(nbytes / ms / 1e6, 1), "of_copy_peak": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3),
                         **({"like": like} if like else {})})
        rnd = lambda *shape, dtype=bf: torch.randn(*shape, device=dev, dtype=f32).to(dtype)
        for n, n_seqs, tag in ((T, 1, "prompt"), (64, 64, "decode")):
            per = n // n_seqs
            cu = torch.arange(0, n + 1, per, dtype=i32, device=dev)
            seq = torch.arange(n, dtype=i32, device=dev) // per
            slots = torch.arange(n_seqs, dtype=i32, device=dev)
            one = per == 1
            # norms
            res, pend, w, b = rnd(n, H, dtype=f32), rnd(n, H), rnd(H, dtype=f32), rnd(H, dtype=f32)
            out = torch.empty(n, H, dtype=bf, device=dev)
            add(f"add_layernorm ({tag})", n, timed(lambda: ops.add_layernorm(res, pend, w, b, 1e-5, out)), n * H * (4 + 4 + 2 + 2))
            add(f"add_rmsnorm ({tag})", n, timed(lambda: ops.add_rmsnorm(res, pend, w, 1e-5, out)), n * H * (4 + 4 + 2 + 2), like="add_layernorm")
            # activation beside the unfused gate of the Llama path
            act, gate_up, half = rnd(n, ff), rnd(n, 2 * ff), torch.empty(n, ff, dtype=bf, device=dev)
            add(f"activation relu2 ({tag})", n, timed(lambda: ops.activation(act, "relu2")), n * ff * 4)
            add(f"swiglu ({tag})", n, timed(lambda: ops.swiglu(gate_up, half)), n * ff * 6, like="activation")
            # the hidden state beside the embedding output
            other, both = rnd(n, H, dtype=f32), torch.empty(n, 2 * H, dtype=bf, device=dev)
            add(f"hidden_concat ({tag})", n, timed(lambda: ops.hidden_concat(res, pend, other, both)), n * H * (4 + 2 + 4 + 4))
            # convolution and recurrence
            proj = rnd(n, inner + conv_dim + heads)
            conv_in, z, dt_raw = proj[:, inner:inner + conv_dim], proj[:, :inner], proj[:, inner + conv_dim:]
            cw, cb = rnd(taps, conv_dim, dtype=f32), rnd(conv_dim, dtype=f32)
            cstate = torch.zeros(n_seqs, taps - 1, conv_dim, device=dev)
            xs, bc = torch.empty(n, inner, dtype=bf, device=dev), torch.empty(n, G * N, 2, device=dev)
            add(f"causal_conv_silu + state ({tag})", n,
                timed(lambda: ops.causal_conv_silu(conv_in, cw, cb, cstate, xs, seq, cu, slots, n_seqs=n_seqs,
                                                   update_state=True, one_token_each=one, pairs=bc)),
                n * (conv_dim * 2 + inner * 2 + 2 * G * N * 4) + (2 * n_seqs * (taps - 1) * conv_dim * 4 if one else 0))
            dtb, al, sk = rnd(heads, dtype=f32) - 2.0, rnd(heads, dtype=f32), rnd(heads, dtype=f32)
            sstate = torch.zeros(n_seqs, heads, N, P, device=dev)
            y = torch.empty(n, inner, dtype=f32, device=dev)
            scan_bytes = n * (inner * 2 + 2 * G * N * 4 + inner * 4) + 2 * n_seqs * heads * N * P * 4
            add(f"ssm_scan ({tag})", n,
                timed(lambda: ops.ssm_scan(xs, bc, dt_raw, dtb, al, sk, sstate, y, cu, slots, n_seqs, heads, G, N, P,
                                           one_token_each=one)), scan_bytes)
            gated, norm_w = torch.empty(n, inner, dtype=bf, device=dev), torch.ones(inner, device=dev)
            add(f"gated_rmsnorm ({tag})", n, timed(lambda: ops.gated_rmsnorm(y, z, norm_w, 1e-5, gated, G)),
                n * inner * (4 + 2 + 2))
        return rows

    sampler = ClockSampler()
    sampler.start()
    sampler.mark()
    sizes = {}
    design_sizes, what = DESIGNS[args.design]
    table = {"senupel": senupel_kernel_table, "zotolix": zotolix_kernel_table, "megerax": megerax_kernel_table}.get(args.design, kernel_table)
    for name in (args.sizes.split(",") if args.sizes else list(design_sizes)):
        design_cfg, llama_cfg = design_sizes[name]
        sizes[name] = {args.design: model_numbers(design_cfg), "llama": model_numbers(llama_cfg),
                       "kernels": table(design_cfg)}
    clocks = sampler.stop()
    print(json.dumps({"design": args.design, "dtype": "bf16", "data": "synthetic (random weights and token ids)",
                      "what": what,
                      "peaks": pk, "l2": "flushed before every timed prefill and kernel; decode steps read more than the L2 holds",
                      "steps": args.steps, "clocks": clocks, "sizes": sizes}))
    return 0


def cpu_baseline():
    """For context only: the plain NumPy implementation that the tests use as their
    oracle, on the host, at tiny-llama-A (three prompts of 5, 17 and 32 tokens, 16
    greedy tokens each; it recomputes the whole sequence for every token).  The
    reference itself is a Go program that cannot be built here; it reports tokens a
    second the same way, new tokens over wall time (cmd/llmgen/main.go:121-133)."""
    import tempfile
    import numpy as np
    import go_tinygrad_b200 as lib
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    try:
        import plain_llama
    except ImportError:
        return {"unavailable": "tests/plain_llama.py not found"}
    tiny = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2,
            "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
            "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
            "tie_word_embeddings": True, "max_position_embeddings": 128}
    with tempfile.TemporaryDirectory() as folder:
        lib.write_random_model(folder, tiny, seed=0, dtype="float32", std=0.02, norm_std=0.01)
        cfg, w = plain_llama.read_model(folder)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 256, n).tolist() for n in (5, 17, 32)]
    t0 = time.time()
    new = sum(len(plain_llama.generate(cfg, w, p, 16)) for p in prompts)
    elapsed = time.time() - t0
    return {"what": "plain NumPy implementation on the host CPU, tiny-llama-A, float32, no cache",
            "value": round(new / elapsed, 1), "unit": "tokens/s", "tokens": new}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=SMOLLM2_1P7B["max_position_embeddings"])
    ap.add_argument("--shape", default="smollm2-1.7b", choices=sorted(SHAPES),
                    help="the model shape; the default is the one the headline numbers are quoted on")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has, where memory or time needs it")
    ap.add_argument("--no-points", dest="points", action="store_false",
                    help="skip the batch-1 and batch-64 decode points")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only and print a short line (for profilers)")
    ap.add_argument("--workload", default="context", choices=["context", "u2048"],
                    help="with --only decode: equal sequences at --context over synthetic keys, or prompts of "
                         "lengths uniform in [128, 2048] that are really prefilled")
    ap.add_argument("--breakdown", action="store_true",
                    help="with --only: also print, as comment lines, the time each kernel adds to a step")
    ap.add_argument("--eager", action="store_true",
                    help="launch the decode step kernel by kernel instead of replaying a graph")
    ap.add_argument("--design", default=None, choices=sorted(DESIGNS),
                    help="measure this design beside the Llama decoder at equal size instead of the default workload")
    ap.add_argument("--sizes", default="", help="with --design: which of its sizes, comma separated (default: all)")
    ap.add_argument("--no-chain", action="store_true",
                    help="decode kernels wait for their predecessor to finish before they are launched")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Go program (go.mod, purego); no Go toolchain is installed "
                          "and pip cannot build it, so it cannot be run here"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"--gpus {args.gpus}: this library runs on one GPU; "
                                   f"there is no multi-GPU path to measure", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.design:
        return run_design(args)
    return run_own(args)


if __name__ == "__main__":
    sys.exit(main())
