"""Throughput of the engine on one B200: decoded tokens a second at the sizes of Llama-3.2-1B with
random weights (the metric and configuration of BASELINE.json's configs[2]).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--config 2|3|4]

Prints ONE JSON line.  ``value``: decoded tokens a second at batch 8, each request holding a
2,048-token prompt in the cache, timed on the device with CUDA events around K decode steps
(each step: the host builds the batch, one pinned copy to the device, the model, the sampler; the
sampled tokens stay on the device); the block of K steps is repeated (at least five blocks and
half a second in all while the context budget allows, ``block_ms``) and the median block is reported.  ``e2e``: the same through the Python entry point
(``Engine.step``: scheduler, pinned host-to-device copy of the step's inputs, model, sampler,
device-to-host read of the sampled tokens; the engine launches step t+1 before it reads step t, so
each call reads the step before the one it launches), by the wall clock.  ``prefill``: one 2,048-token
prompt in one step.  ``roofline``: bytes a decode step has to read (every weight it uses once, and
the cache of the live requests) over its time, against the measured copy bandwidth.  ``points``:
decode at batch 1, 8 and 64 over the 256 generated tokens that the metric names (with each point's
fraction of the HBM roofline), batch 8 without CUDA graphs, and the prompt in four portions of 512.
``breakdown``: CUDA-event time of each kind of kernel in one decode step.  The weights (2.5 GB) are larger than the L2 cache (126 MB), so every
step reads them from HBM; nothing is flushed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def load_baseline_config() -> dict:
    """Sizes of BASELINE.json's configs[2] (Llama-3.2-1B), as config.json keys."""
    return dict(
        architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=16, hidden_size=2048,
        num_attention_heads=32, num_key_value_heads=8, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0,
        rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192),
        rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)


def load_other_config(index: int) -> dict:
    """Sizes of BASELINE.json's configs[3] (Llama-3.2-3B) and configs[4] (Llama-3.1-8B), as config.json keys."""
    cfg = load_baseline_config()
    if index == 3:
        cfg.update(num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8,
                   intermediate_size=8192)
    elif index == 4:
        cfg.update(num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                   intermediate_size=14336, tie_word_embeddings=False)
        cfg["rope_scaling"] = dict(cfg["rope_scaling"], factor=8.0)
    else:
        raise ValueError(f"no configuration {index}")
    return cfg


def load_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            peaks = dict(FALLBACK_PEAKS)
            for k in peaks:
                if isinstance(d.get(k), (int, float)):
                    peaks[k] = float(d[k])
            return peaks, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.proc = None
        self.lines: list[tuple[float, str]] = []
        self.t0 = 0.0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark(self):
        """The timed region starts now: samples taken before (nvidia-smi needs a moment to start) do not count."""
        self.t0 = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for when, line in self.lines:
            if when < self.t0:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def model_numbers(cfg: dict, layers: int):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = H // nh
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * H * I
    return dict(H=H, I=I, V=V, nh=nh, nkv=nkv, hd=hd, per_layer_params=per_layer, head_params=V * H, layers=layers)


def decode_bytes(m: dict, batch: int, ctx_len: float, elt: int = 2) -> float:
    weights = (m["layers"] * m["per_layer_params"] + m["head_params"]) * elt + (2 * m["layers"] + 1) * m["H"] * 4
    kv = batch * ctx_len * 2 * m["nkv"] * m["hd"] * elt * m["layers"]
    return weights + kv


def prefill_flops(m: dict, T: int, rows: int = 1) -> float:
    L = m["layers"]
    attn_proj = (m["nh"] + 2 * m["nkv"]) * m["hd"] * m["H"]
    rest = m["per_layer_params"] - attn_proj  # o, gate, up, down: only `rows` rows in the last layer
    linear = 2.0 * T * (L * attn_proj + (L - 1) * rest) + 2.0 * rows * rest + 2.0 * rows * m["head_params"]
    attention = L * m["nh"] * m["hd"] * 4.0 * T * (T + 1) / 2
    return linear + attention


TIMED_OPS = ("embed_gather", "add_rmsnorm", "rope_kv_write", "rope_kv_write_partials", "linear_decode", "linear_smallm",
             "linear_smallm_gated", "silu_mul", "gather_rows", "attn_decode_mma", "attn_decode_rope_mma", "attn_prefill_mma",
             "attn_prefill_tc", "sample", "gemm_tcgen05", "linear_tc_decode", "linear")


def kernel_breakdown(ops, torch, run_step, reps: int = 5) -> dict:
    """CUDA-event time of each kind of kernel in one eager step (microseconds, summed over the step's calls of that
    kind, median of ``reps`` steps).  Products are told apart by their weight's shape.  The whole step is put into the
    stream behind a kernel that keeps the GPU busy for a few milliseconds, so that no event waits for the host;
    the events between the kernels keep a kernel from starting under the one before it, so the sum is a little above
    a step's time as a graph replays it: read the shares."""
    records: list[tuple[str, object, object]] = []
    saved = {}

    def wrap(name, fn):
        def timed(*a, **k):
            label = name
            if name.startswith(("linear", "gemm_")) and len(a) >= 2 and hasattr(a[1], "shape"):
                label = f"{name}[{a[1].shape[0]}x{a[1].shape[1]}]"
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **k)
            e1.record()
            records.append((label, e0, e1))
            return out
        return timed

    for name in TIMED_OPS:
        if hasattr(ops, name):
            saved[name] = getattr(ops, name)
    runs = []
    try:
        for name, fn in saved.items():
            # the inner calls of ops.linear_few_rows / ops.linear go through the module's globals: wrap only what
            # the parts call, and let a wrapped function's own calls of other wrapped functions count once
            setattr(ops, name, wrap(name, fn))
        for _ in range(reps):
            records.clear()
            torch.cuda.synchronize()
            torch.cuda._sleep(int(6e6))  # a few milliseconds of spinning: the step's launches queue up behind it
            run_step()
            torch.cuda.synchronize()
            per = {}
            for label, e0, e1 in records:
                per[label] = per.get(label, 0.0) + e0.elapsed_time(e1) * 1e3
            runs.append(per)
    finally:
        for name, fn in saved.items():
            setattr(ops, name, fn)
    labels = sorted({k for r in runs for k in r})
    out = {k: round(statistics.median(r.get(k, 0.0) for r in runs), 1) for k in labels}
    out["sum_us"] = round(sum(v for k, v in out.items()), 1)
    return out


def run_ours(args) -> dict:
    import numpy as np
    import torch

    from tokasaurus_b200.engine.batch import StepEntry
    from tokasaurus_b200.engine.engine import Engine
    from tokasaurus_b200.kernels import ops
    from tokasaurus_b200.sampling.params import SamplingParams

    cfg = load_baseline_config()
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    peaks, peak_src = load_peaks()
    prompt_len, context_len, page_size, generated = 2048, 4096, 16, 256
    max_batch = max(args.batch, 64 if not args.skip_points else args.batch)
    pool_tokens = max_batch * context_len
    eng = Engine(config_dict=cfg, random_weights=0, dtype="bfloat16", page_size=page_size,
                 kv_cache_num_tokens=pool_tokens, max_tokens_per_forward=8192, max_seqs_per_forward=max(64, max_batch),
                 device="cuda:0")
    runner, cache, sampler = eng.runner, eng.runner.cache, eng.sampler
    m = model_numbers(cfg, layers)
    g = torch.Generator().manual_seed(0)
    dev = runner.rt.device

    def tokens(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()

    def event_ms(fn, reps):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    # ---------------------------------------------------------------- prefill: 2,048 tokens in one step, and in 4 of 512
    pf_tokens = tokens(prompt_len)

    def prefill_once(chunk=prompt_len):
        """The prompt in portions of ``chunk`` tokens, each run as the engine runs such a step: as a step graph
        where it keeps graphs for steps of that size, else kernel by kernel."""
        cache.admit("pf")
        cache.ensure_capacity("pf", prompt_len)
        for at in range(0, prompt_len, chunk):
            last = at + chunk >= prompt_len
            entries = [StepEntry("pf", pf_tokens[at:at + chunk], at, [chunk - 1] if last else [])]
            rows = 1 if last else 0
            extra = dict(temperature=np.zeros(rows, dtype=np.float32), stream_key=np.zeros(rows, dtype=np.int64),
                         sample_pos=np.full(rows, at + chunk, dtype=np.int32),
                         row_slot=np.full(rows, cache.slot("pf"), dtype=np.int32))
            prep = None
            if eng.graphs is not None and eng.graphs.usable_general(entries):
                prep = eng.graphs.prepare_general(entries, extra)
            if prep is not None:
                eng.graphs.launch(prep)
            else:
                runner.step(entries, extra)
        cache.free("pf")

    for _ in range(max(3, args.warmup // 2)):
        prefill_once()
    pf_ms = statistics.median(event_ms(prefill_once, 3) for _ in range(5))
    pf_flops = prefill_flops(m, prompt_len)
    prefill = dict(value=round(prompt_len / (pf_ms / 1e3), 1), tokens=prompt_len, ms=round(pf_ms, 3),
                   frac=round(pf_flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4),
                   frac_of_sustained=round(pf_flops / (pf_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12), 4), of=peak_src)
    points = {}
    if not args.skip_points:
        for _ in range(3):
            prefill_once(512)
        ch_ms = statistics.median(event_ms(lambda: prefill_once(512), 3) for _ in range(5))
        points["prefill_chunked_4x512"] = round(prompt_len / (ch_ms / 1e3), 1)

    # ---------------------------------------------------------------- decode at a batch size, on the device
    def fill(batch, tag):
        ids = [f"{tag}{i}" for i in range(batch)]
        for chunk in range(0, batch, 4):
            entries = []
            for rid in ids[chunk:chunk + 4]:
                cache.admit(rid)
                cache.ensure_capacity(rid, prompt_len)
                entries.append(StepEntry(rid, tokens(prompt_len), 0, [prompt_len - 1]))
            logits = runner.step(entries)
            rows = len(entries)
            slots = torch.tensor([cache.slot(e.request) for e in entries], dtype=torch.int32, device=dev)
            sampler.sample(logits, torch.zeros(rows, device=dev), None, None, slots, cache.last_token)
        torch.cuda.synchronize()
        return ids

    class Decoder:
        """A batch of requests with their prompts in the cache; ``one`` runs one decode step (host batch building,
        one pinned copy, model, sampler; the sampled ids stay on the device)."""

        def __init__(self, batch, tag, graphs=True):
            self.ids = fill(batch, tag)
            self.length = {rid: prompt_len for rid in self.ids}
            self.zeros = np.zeros(batch, dtype=np.float32)
            self.keys = np.zeros(batch, dtype=np.int64)
            self.graphs = graphs

        def one(self):
            entries = []
            for rid in self.ids:
                cache.ensure_capacity(rid, self.length[rid] + 1)
                entries.append(StepEntry(rid, None, self.length[rid], [0]))
                self.length[rid] += 1
            pos = np.asarray([self.length[r] for r in self.ids], dtype=np.int32)
            slot = np.asarray([cache.slot(r) for r in self.ids], dtype=np.int32)
            extra = dict(temperature=self.zeros, stream_key=self.keys, sample_pos=pos, row_slot=slot)
            if self.graphs and eng.graphs is not None and eng.graphs.usable(entries):
                eng.graphs.run(entries, extra)
                return
            logits = runner.step(entries, extra)
            ex = runner.last_context.extra
            sampler.sample(logits, ex["temperature"], ex["stream_key"], ex["sample_pos"], ex["row_slot"], cache.last_token)

        def context(self):
            return next(iter(self.length.values()))

        def close(self):
            runner.check_status()
            for rid in self.ids:
                cache.free(rid)

    def decode_point(batch, steps, warmup, tag, graphs=True):
        d = Decoder(batch, tag, graphs)
        for _ in range(warmup):
            d.one()
        ms = event_ms(d.one, steps)
        d.close()
        return ms

    # the headline: blocks of --steps steps, the median block; at least five blocks and 150 ms in all
    clocks = ClockSampler()
    clocks.start()
    d = Decoder(args.batch, "d")
    for _ in range(args.warmup):
        d.one()
    clocks.mark()
    ops.LAUNCHES = 0
    first_ctx = d.context()
    blocks = [event_ms(d.one, args.steps)]
    launches = ops.LAUNCHES
    room = context_len - d.context() - args.steps - 8
    while ((len(blocks) < 5 or sum(blocks) * args.steps < 500.0) and room >= args.steps
           and len(blocks) < (args.max_blocks or 60)):
        blocks.append(event_ms(d.one, args.steps))
        room -= args.steps
    clock_info = clocks.stop()
    mean_ctx = (first_ctx + d.context()) / 2
    ms = statistics.median(blocks)
    # where the step's time goes: each kind of kernel, timed with events in an eager step of the same requests
    breakdown = None if args.skip_points else kernel_breakdown(ops, torch, lambda: (setattr(d, "graphs", False), d.one(),
                                                                                      setattr(d, "graphs", True)))
    d.close()
    value = args.batch * 1e3 / ms
    nbytes = decode_bytes(m, args.batch, mean_ctx)
    achieved = nbytes / (ms / 1e3) / 1e9
    roofline = dict(bound="hbm", achieved=round(achieved, 1), peak=peaks["hbm_gbs"], unit="GB/s",
                    frac=round(achieved / peaks["hbm_gbs"], 4), of=peak_src)

    if not args.skip_points:
        # the metric's own shape: 2,048 prompt tokens, then 256 generated tokens, at batch 1, 8 and 64
        for b in (1, args.batch, 64):
            pms = decode_point(b, generated, max(3, args.warmup // 2), f"p{b}_")
            points[f"decode_b{b}" if b != args.batch else f"decode_b{b}_256"] = round(b * 1e3 / pms, 1)
            bytes_b = decode_bytes(m, b, prompt_len + generated / 2)
            points[f"hbm_frac_b{b}"] = round(bytes_b / (pms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        pms = decode_point(args.batch, 32, 3, "ng", graphs=False)
        points[f"decode_b{args.batch}_no_graphs"] = round(args.batch * 1e3 / pms, 1)

    # ---------------------------------------------------------------- end to end through the entry point
    e2e_steps = args.steps * len(blocks)
    prompts = [tokens(prompt_len) for _ in range(args.batch)]
    for p in prompts:
        eng.add_request(p, SamplingParams(temperature=0.0), max_num_tokens=args.warmup + e2e_steps + 8, ignore_eos=True)
    while eng.scheduler.prefilling or eng.scheduler.queued:
        eng.step()
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    h2d = d2h = 0
    e2e_blocks = []
    for _ in range(len(blocks)):
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.step()
            h2d += eng.last_step_bytes["h2d"]
            d2h += eng.last_step_bytes["d2h"]
        torch.cuda.synchronize()
        e2e_blocks.append((time.perf_counter() - t0) * 1e3 / args.steps)
    e2e_ms = statistics.median(e2e_blocks)
    e2e = dict(value=round(args.batch * 1e3 / e2e_ms, 1), unit="tokens/s",
               h2d_bytes_per_step=h2d // e2e_steps, d2h_bytes_per_step=d2h // e2e_steps,
               ms_per_step=round(e2e_ms, 4))

    if not args.skip_points:
        # many requests through the entry point: 256 requests of 512 + 128 tokens, all of them admitted at once
        # (prompt portions under the token budget, then decode steps of up to 256 requests from step graphs)
        n_req, n_prompt, n_gen = 256, 512, 128
        del eng
        serve = Engine(config_dict=cfg, random_weights=0, dtype="bfloat16", page_size=page_size,
                       kv_cache_num_tokens=n_req * (n_prompt + n_gen + 64), max_tokens_per_forward=8192,
                       max_seqs_per_forward=n_req, cudagraph_max_size=n_req)
        many = [tokens(n_prompt) for _ in range(n_req)]
        greedy = SamplingParams(temperature=0.0)
        serve.warm_up()  # the decode graphs of every batch size, as a server records them when it starts
        serve.generate(many, greedy, max_num_tokens=4, ignore_eos=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        serve.generate(many, greedy, max_num_tokens=n_gen, ignore_eos=True)
        torch.cuda.synchronize()
        points["engine_256_requests_512p128_total"] = round(n_req * (n_prompt + n_gen) / (time.perf_counter() - t0), 1)
        cuda_graphs = serve.graphs is not None
        del serve
    else:
        cuda_graphs = eng.graphs is not None

    out = {
        "metric": "decode tokens/s (Llama-3.2-1B sizes, batch 8, 2,048-token prompts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids (seeded uniform), random weights N(0, 0.02)",
        "impl": "ours",
        "config": {
            "model": "Llama-3.2-1B sizes", "global_batch": args.batch, "seq_len": prompt_len, "context_len": context_len,
            "parallelism": "1 GPU", "layers": layers, "layers_full": full_layers, "hidden": m["H"], "heads": m["nh"],
            "kv_heads": m["nkv"], "head_dim": m["hd"], "intermediate": m["I"], "vocab": m["V"], "page_size": page_size,
            "tied_embeddings": True, "rope": "llama3 factor 32", "l2": "inputs (2.5 GB of weights) larger than L2; no flush",
            "cuda_graphs": cuda_graphs, "timed_blocks": len(blocks),
        },
        "e2e": e2e, "gpu_launches": launches, "clocks": clock_info, "prefill": prefill, "roofline": roofline,
        "points": points, "block_ms": [round(b, 4) for b in blocks],
    }
    if breakdown is not None:
        out["breakdown"] = breakdown
    return out


def run_further(args) -> dict:
    """The further workloads BASELINE.json names, with the same kind of line: configs[3], one mixed step at
    Llama-3.2-3B sizes (32 requests that decode at contexts of 1,024 to 4,096 beside the second 2,048-token
    portion of a 4,096-token prompt), and configs[4], decode at batch 64 with every request at context 8,192 at
    Llama-3.1-8B sizes (64 x 8,192 tokens of keys and values: 68.7 GB beside 16 GB of weights).  All layers by
    default (the random weights are drawn on the device); ``--layers`` runs fewer, and ``config`` names both numbers."""
    import numpy as np
    import torch

    from tokasaurus_b200.engine.batch import StepEntry
    from tokasaurus_b200.engine.engine import Engine
    from tokasaurus_b200.kernels import ops

    cfg = load_other_config(args.config)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    peaks, peak_src = load_peaks()
    page_size = 16
    g = torch.Generator().manual_seed(0)
    rng = np.random.default_rng(0)
    if args.config == 3:
        batch, chunk = 32, 2048
        contexts = [int(c) for c in rng.integers(1024, 4097, size=batch)]
        pool_tokens = sum(-(-(c + 1) // page_size) * page_size for c in contexts) + 4096 + 64 * page_size
    else:
        batch, chunk = 64, 0
        contexts = [8192] * batch
        pool_tokens = batch * (8192 + 512)
    eng = Engine(config_dict=cfg, random_weights=0, dtype="bfloat16", page_size=page_size,
                 kv_cache_num_tokens=pool_tokens, max_tokens_per_forward=8192, max_seqs_per_forward=max(64, batch + 1),
                 device="cuda:0")
    runner, cache, sampler = eng.runner, eng.runner.cache, eng.sampler
    m = model_numbers(cfg, layers)
    dev = runner.rt.device

    def tokens(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()

    def sample_rows(logits, entries):
        slots = torch.tensor([cache.slot(e.request) for e in entries], dtype=torch.int32, device=dev)
        sampler.sample(logits, torch.zeros(len(entries), device=dev), None, None, slots, cache.last_token)

    # the requests' contexts go into the cache through the step function, up to 8,192 tokens a step
    ids = [f"d{i}" for i in range(batch)]
    done = {rid: 0 for rid in ids}
    want = dict(zip(ids, contexts))
    for rid in ids:
        cache.admit(rid)
        cache.ensure_capacity(rid, want[rid] + 1)
    while any(done[r] < want[r] for r in ids):
        entries, room = [], 8192
        for rid in ids:
            n = min(want[rid] - done[rid], room)
            if n > 0:
                last = done[rid] + n == want[rid]
                entries.append(StepEntry(rid, tokens(n), done[rid], [n - 1] if last else []))
                done[rid] += n
                room -= n
        logits = runner.step(entries)
        finishing = [e for e in entries if e.want]
        if finishing:
            sample_rows(logits, finishing)
    torch.cuda.synchronize()

    def event_ms(fn, reps):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    zeros = np.zeros(batch + (1 if chunk else 0), dtype=np.float32)
    keys = np.zeros(len(zeros), dtype=np.int64)
    if args.config == 3:
        # the mixed step, repeated as it is: the same positions are computed and written again
        cache.admit("pf")
        cache.ensure_capacity("pf", 2 * chunk)
        runner.step([StepEntry("pf", tokens(chunk), 0, [])])
        pf_tokens = tokens(chunk)

        def one():
            entries = [StepEntry("pf", pf_tokens, chunk, [chunk - 1])]
            entries += [StepEntry(rid, None, want[rid], [0]) for rid in ids]
            pos = np.asarray([2 * chunk] + [want[r] + 1 for r in ids], dtype=np.int32)
            slot = np.asarray([cache.slot(e.request) for e in entries], dtype=np.int32)
            logits = runner.step(entries, dict(temperature=zeros, stream_key=keys, sample_pos=pos, row_slot=slot))
            ex = runner.last_context.extra
            sampler.sample(logits, ex["temperature"], ex["stream_key"], ex["sample_pos"], ex["row_slot"], cache.last_token)

        step_tokens = batch + chunk
        rows = batch + 1
        flops = prefill_flops(m, chunk, rows) + 2.0 * batch * (layers - 1) * m["per_layer_params"] \
            + layers * m["nh"] * m["hd"] * 4.0 * (chunk * chunk + sum(contexts))  # the chunk's queries see 2,048 keys more
        nbytes = decode_bytes(m, batch, sum(contexts) / batch) + decode_bytes(m, 1, 2 * chunk) - decode_bytes(m, 0, 0)
        metric = "tokens/s of a mixed step (Llama-3.2-3B sizes: 32 decoding requests beside a 2,048-token prompt portion)"
    else:
        length = dict(want)

        def one():
            entries = []
            for rid in ids:
                cache.ensure_capacity(rid, length[rid] + 1)
                entries.append(StepEntry(rid, None, length[rid], [0]))
                length[rid] += 1
            pos = np.asarray([length[r] for r in ids], dtype=np.int32)
            slot = np.asarray([cache.slot(r) for r in ids], dtype=np.int32)
            extra = dict(temperature=zeros, stream_key=keys, sample_pos=pos, row_slot=slot)
            if eng.graphs is not None and eng.graphs.usable(entries):
                eng.graphs.run(entries, extra)
                return
            logits = runner.step(entries, extra)
            ex = runner.last_context.extra
            sampler.sample(logits, ex["temperature"], ex["stream_key"], ex["sample_pos"], ex["row_slot"], cache.last_token)

        step_tokens = batch
        flops = 2.0 * batch * (layers * m["per_layer_params"] + m["head_params"])
        nbytes = decode_bytes(m, batch, 8192 + args.warmup + args.steps / 2)
        metric = "decode tokens/s (Llama-3.1-8B sizes, batch 64, every request at context 8,192)"

    clocks = ClockSampler()
    clocks.start()
    for _ in range(args.warmup):
        one()
    clocks.mark()
    ops.LAUNCHES = 0
    reps = max(1, int(0.5e3 / max(1e-3, event_ms(one, 1)) / args.steps))  # the timed block repeated to half a second
    ms = statistics.median(event_ms(one, args.steps) for _ in range(min(reps, 20)))
    launches = ops.LAUNCHES
    clock_info = clocks.stop()
    runner.check_status()
    achieved = nbytes / (ms / 1e3) / 1e9
    return {
        "metric": metric, "value": round(step_tokens * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids (seeded uniform), random weights N(0, 0.02)",
        "impl": "ours",
        "config": {
            "model": "Llama-3.2-3B sizes" if args.config == 3 else "Llama-3.1-8B sizes", "baseline_config": args.config,
            "global_batch": batch, "prompt_portion": chunk, "context_mean": round(sum(contexts) / batch, 1),
            "parallelism": "1 GPU", "layers": layers, "layers_full": full_layers, "hidden": m["H"], "heads": m["nh"],
            "kv_heads": m["nkv"], "head_dim": m["hd"], "intermediate": m["I"], "vocab": m["V"], "page_size": page_size,
            "l2": "weights and cache larger than L2; no flush",
        },
        "gpu_launches": launches, "clocks": clock_info,
        "roofline": dict(bound="hbm", achieved=round(achieved, 1), peak=peaks["hbm_gbs"], unit="GB/s",
                         frac=round(achieved / peaks["hbm_gbs"], 4), of=peak_src),
        "compute": dict(tflops=round(flops / (ms / 1e3) / 1e12, 1), peak=peaks["bf16_tflops"],
                        frac=round(flops / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4), of=peak_src),
    }


def run_reference(args) -> dict:
    """The reference arm: baseline/reference_arm.py in a process of its own (it imports nothing of this
    repository's package), which drives the unmodified reference installed under baseline/_ref.  Its JSON line
    is passed on; if it cannot run, the line says why."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "tokasaurus")):
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref (pip install "
                "--no-index --no-deps --target baseline/_ref from a copy of the reference's tree)"}
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--steps", str(args.steps), "--warmup",
           str(args.warmup), "--batch", str(args.batch)]
    if args.layers:
        cmd += ["--layers", str(args.layers)]
    if args.skip_points:
        cmd += ["--skip-points"]
    env = dict(os.environ)
    env.pop("PYTHONPATH", None)
    clocks = ClockSampler()
    clocks.start()
    try:
        proc = subprocess.run(cmd, cwd=os.path.join(ROOT, "baseline"), env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True, timeout=args.reference_timeout)
    except subprocess.TimeoutExpired:
        clocks.stop()
        return {"impl": "reference", "unavailable": f"the reference arm did not finish in {args.reference_timeout} s"}
    clock_info = clocks.stop()
    line = None
    for text in reversed(proc.stdout.splitlines()):
        if text.startswith("{") and '"impl"' in text:
            line = text
            break
    if proc.returncode != 0 or line is None:
        tail = " | ".join((proc.stderr or proc.stdout).strip().splitlines()[-3:])[-400:]
        return {"impl": "reference", "unavailable": f"the reference arm exited with {proc.returncode}: {tail}"}
    out = json.loads(line)
    out.setdefault("clocks", clock_info)  # the arm samples its own timed region; this one covers the whole process
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch-1 and batch-64 points")
    ap.add_argument("--max-blocks", type=int, default=0,
                    help="at most this many timed blocks of --steps steps (0: at least five and half a second's worth); "
                         "1 keeps a profiler's capture short")
    ap.add_argument("--reference-timeout", type=int, default=1500, help="seconds the reference arm may take")
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4],
                    help="2: the headline metric (default); 3 and 4: the further workloads, see run_further")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0
    print(json.dumps(run_ours(args) if args.config == 2 else run_further(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
