"""The reference arm of bench.py: the UNMODIFIED reference (installed under baseline/_ref) on the metric and
configuration of bench.py's own arm: decode tokens a second at Llama-3.2-1B sizes with random weights, batch 8,
2,048-token prompts, bfloat16, page size 16.

    python baseline/reference_arm.py --steps K --warmup W [--batch 8] [--skip-points]

What runs is the reference's stock one-GPU model worker path, driven the way its own benchmark does
(tokasaurus/benchmarks/bench_model.py:119-283) and its worker loop does (tokasaurus/model/basic_worker.py:40-160):

    make_model -> ModelRunner (+ record_graphs) -> per step: seqs_to_input -> calc_padding ->
    make_input_batch_state -> ModelRunner.plan -> move_batch_state -> last-token lookup ->
    add_decoding_ids_to_batch_state -> ModelRunner.run -> unpad_output_batch_state -> last-token update

with the manager's page accounting (BlockAllocator.allocate_with_prefix_match / allocate_up_to_length) and its
sequence counters (tokasaurus/manager/scheduler.py:640-684).  The requests' prompts really are prefilled through
the model first.  Nothing of this repository's engine, models or kernels is imported.

What is not the reference's: stand-ins for four third-party packages this image lacks (baseline/stubs: pydra,
accelerate, art, statsd), an adapter for two FlashInfer arguments renamed since the version the reference pins
(baseline/flashinfer_compat.py), and the random-weight model folder written here (config.json and
model.safetensors in bfloat16 under HF tensor names).

Prints ONE JSON line with bench.py's keys (``impl`` = "reference").  ``value``: K decode steps timed on the
device with CUDA events, each step with its host-side batch building and FlashInfer planning, as in the other arm;
``e2e``: the same by the wall clock with the sampled ids read back to the host every step, the work of step t+1
prepared while step t runs, as the reference's worker loop does (run_overlapped_loop, model/utils.py:267-318).
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def llama_1b_config() -> dict:
    """config.json of the benchmark model: the sizes of Llama-3.2-1B (BASELINE.json configs[2])."""
    return dict(
        architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=16, hidden_size=2048,
        num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256,
        rope_theta=500000.0, hidden_act="silu", attention_bias=False, mlp_bias=False,
        rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192),
        rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072, torch_dtype="bfloat16",
        bos_token_id=128000, eos_token_id=128001)


def write_model_folder(folder: str, cfg: dict, seed: int = 0) -> None:
    """Random weights N(0, 0.02), norm weights 1, bfloat16, under the HF names the reference loads by
    (tokasaurus/model/llama.py:824-847)."""
    import torch
    from safetensors.torch import save_file

    g = torch.Generator(device="cuda").manual_seed(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = H // nh

    def matrix(rows, cols):
        return (torch.randn(rows, cols, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()

    tensors = {"model.embed_tokens.weight": matrix(V, H), "model.norm.weight": torch.ones(H, dtype=torch.bfloat16)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        tensors[p + "input_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        tensors[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        tensors[p + "self_attn.q_proj.weight"] = matrix(nh * hd, H)
        tensors[p + "self_attn.k_proj.weight"] = matrix(nkv * hd, H)
        tensors[p + "self_attn.v_proj.weight"] = matrix(nkv * hd, H)
        tensors[p + "self_attn.o_proj.weight"] = matrix(H, nh * hd)
        tensors[p + "mlp.gate_proj.weight"] = matrix(I, H)
        tensors[p + "mlp.up_proj.weight"] = matrix(I, H)
        tensors[p + "mlp.down_proj.weight"] = matrix(H, I)
    if not cfg["tie_word_embeddings"]:
        tensors["lm_head.weight"] = matrix(V, H)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})


def native_libraries() -> list[str]:
    """Shared objects mapped into this process that are not part of the Python installation's own tree."""
    found = set()
    try:
        with open("/proc/self/maps") as f:
            for line in f:
                path = line.rsplit(" ", 1)[-1].strip()
                if path.endswith(".so") and ("flashinfer" in path or "tokasaurus" in path or "/csrc/" in path):
                    found.add(path)
    except OSError:
        pass
    return sorted(found)


def run(args) -> dict:
    import transformers  # noqa: F401  (before the accelerate stand-in becomes importable)

    sys.path.insert(0, os.path.join(HERE, "stubs"))
    sys.path.insert(0, REF)
    sys.path.insert(0, HERE)
    import flashinfer_compat

    flashinfer_compat.install()

    import torch
    from tokasaurus.common_types import ServerConfig
    from tokasaurus.manager.allocator import BlockAllocator
    from tokasaurus.manager.manager import seqs_to_input
    from tokasaurus.manager.types import Sequence
    from tokasaurus.model.utils import (
        ModelRunner,
        add_decoding_ids_to_batch_state,
        make_input_batch_state,
        make_model,
        move_batch_state,
        run_overlapped_loop,
        unpad_output_batch_state,
    )
    from tokasaurus.server.types import SamplingParams

    import random

    random.seed(0)
    torch.manual_seed(0)
    device = "cuda:0"
    torch.cuda.set_device(device)
    dtype = torch.bfloat16
    cfg = llama_1b_config()
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    prompt_len, context_len, page_size = 2048, 4096, 16
    max_batch = max(args.batch, args.batch if args.skip_points else 64)

    folder = tempfile.mkdtemp(prefix="ref_arm_model_")
    try:
        write_model_folder(folder, cfg)
        config = ServerConfig()
        config.model = folder
        config.page_size = page_size
        config.kv_cache_num_tokens = max_batch * context_len
        config.max_tokens_per_forward = 8192
        config.max_seqs_per_forward = max(64, max_batch)
        config.use_cudagraphs = True
        t0 = time.perf_counter()
        with torch.inference_mode():
            model = make_model(config, device=device, dtype=dtype)
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    runner = ModelRunner(config=config, model=model)
    runner.record_graphs("reference_arm")
    setup_s = time.perf_counter() - t0

    num_pages = config.kv_cache_num_blocks()
    allocator = BlockAllocator(num_pages, page_size)
    last_token = torch.zeros(config.max_batch_index(), dtype=torch.long, device=device)
    greedy = SamplingParams(temperature=0.0, top_p=1.0)
    vocab = cfg["vocab_size"]
    counter = [0]

    def tokens(n):
        return [random.randint(0, vocab - 1) for _ in range(n)]

    # -- one step of the model worker, as basic_worker.py's preprocess / run_model do it --------------------
    class Work:
        pass

    def preprocess(decoding, prefilling):
        counter[0] += 1
        inp = seqs_to_input(decoding, prefilling, schedule_id=f"s{counter[0]}", page_size=page_size,
                            starting_prefill_offset=0)
        batch_indices = torch.tensor(inp.batch_indices, dtype=torch.long)
        pad_total, pad_lm = runner.calc_padding(num_prefill_tokens=inp.num_prefill_tokens(),
                                                num_decode_tokens=inp.num_decode_tokens(),
                                                num_lm_head_tokens=inp.num_lm_head_tokens())
        state = make_input_batch_state(inp, num_total_padding=pad_total, num_lm_head_padding=pad_lm)
        runner.plan(state, non_blocking=True)
        move_batch_state(input_batch_state=state, device=device, non_blocking=True)
        w = Work()
        w.inp, w.state, w.batch_indices = inp, state, batch_indices.to(device, non_blocking=True)
        return w

    def run_model(w):
        decoding_ids = last_token[w.batch_indices[w.inp.decode_start_pos():]]
        add_decoding_ids_to_batch_state(input_batch_state=w.state, decoding_input_ids=decoding_ids)
        out = runner.run(w.state, non_blocking=True)
        unpad_output_batch_state(output_batch_state=out, model_input=w.inp)
        rows = w.state.raw_lm_head_indices if w.state.raw_lm_head_indices is not None else w.state.lm_head_indices
        idx = w.batch_indices[rows]
        if len(idx) > 0:
            last_token[idx] = out.outputs.output_ids
        w.out = out

    # -- the manager's bookkeeping for a request (manager.py:451-473, scheduler.py:640-684) --------------------
    def admit(name, slot):
        seq = Sequence(id=name, completion_total=1 << 30, input_ids=tokens(prompt_len), sampling_params=greedy,
                       batch_index=slot)
        seq.kv_indices, cached = allocator.allocate_with_prefix_match(seq.id, seq.input_ids)
        seq.prompt_scheduled = cached
        return seq

    def after_prefill(seq, n):
        seq.prompt_scheduled += n
        if seq.prompt_scheduled == seq.prompt_total():
            seq.completion_scheduled += 1

    def grow(seqs):
        for seq in seqs:
            seq.kv_indices.extend(allocator.allocate_up_to_length(seq.id, seq.kv_indices, seq.total_scheduled()))

    def release(seqs):
        for seq in seqs:
            allocator.free_and_update(seq.id, seq.kv_indices, seq.input_ids)

    def event_ms(fn, reps):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    # -- prefill: one 2,048-token prompt in one step -------------------------------------------------------
    def prefill_once():
        seq = admit(f"pf{counter[0]}", 0)
        w = preprocess([], [(seq, prompt_len - seq.prompt_scheduled)])
        run_model(w)
        release([seq])

    for _ in range(max(3, args.warmup // 2)):
        prefill_once()
    pf_ms = event_ms(prefill_once, 5)

    # -- decode at a batch size -----------------------------------------------------------------------------
    def fill(batch, tag):
        seqs = [admit(f"{tag}{i}", i) for i in range(batch)]
        for i in range(0, batch, 4):
            chunk = seqs[i:i + 4]
            run_model(preprocess([], [(s, prompt_len - s.prompt_scheduled) for s in chunk]))
            for s in chunk:
                after_prefill(s, prompt_len - s.prompt_scheduled)
        grow(seqs)
        torch.cuda.synchronize()
        return seqs

    def decode_step(seqs):
        w = preprocess(seqs, [])
        run_model(w)
        for s in seqs:
            s.completion_scheduled += 1
        grow(seqs)
        return w

    def decode_run(batch, steps, warmup, tag, repeats=1):
        seqs = fill(batch, tag)
        for _ in range(warmup):
            decode_step(seqs)
        samples = [event_ms(lambda: decode_step(seqs), steps) for _ in range(repeats)]
        return seqs, statistics.median(samples), samples

    sys.path.insert(0, os.path.dirname(HERE))
    from bench import ClockSampler  # nvidia-smi in a thread; bench.py imports nothing of this repository's package

    clocks = ClockSampler()
    clocks.start()
    seqs = fill(args.batch, "d")
    for _ in range(args.warmup):
        decode_step(seqs)
    clocks.mark()
    samples = [event_ms(lambda: decode_step(seqs), args.steps) for _ in range(args.repeats)]
    ms = statistics.median(samples)
    clock_info = clocks.stop()

    # -- the device's share alone: one planned decode step replayed from its CUDA graph, no host work between
    #    (what bench_model.py graph=True plan_before=True times, utils.py:254-309) ------------------------------
    w = preprocess(seqs, [])
    run_model(w)
    graph_index = runner.match_state_to_graph(w.state)
    replay_ms = None
    if graph_index is not None:
        graph = runner.graphs[graph_index].graph
        replay_ms = event_ms(graph.replay, max(10, args.steps))

    # -- end to end: the same requests go on, ids read back every step, next step prepared meanwhile --------
    todo = [args.warmup + args.steps]
    host_ids = []
    d2h = [0]

    def e2e_preprocess():
        if todo[0] == 0:
            return None
        todo[0] -= 1
        w = preprocess(seqs, [])
        for s in seqs:  # the manager counts a step as scheduled when it submits it (scheduler.py:640-684)
            s.completion_scheduled += 1
        grow(seqs)
        return w

    def e2e_synchronize(w):
        torch.cuda.synchronize()
        w.cpu = w.out.outputs.to("cpu")

    def e2e_postprocess(w):
        host_ids.append(w.cpu.output_ids.tolist())
        d2h[0] += w.cpu.output_ids.numel() * w.cpu.output_ids.element_size()
        if w.cpu.chosen_logprobs is not None:
            d2h[0] += w.cpu.chosen_logprobs.numel() * w.cpu.chosen_logprobs.element_size()

    with torch.inference_mode():
        todo[0] = args.warmup
        run_overlapped_loop(e2e_preprocess, run_model, e2e_synchronize, e2e_postprocess, max_iters=args.warmup)
        torch.cuda.synchronize()
        host_ids.clear()
        d2h[0] = 0
        todo[0] = args.steps
        t0 = time.perf_counter()
        run_overlapped_loop(e2e_preprocess, run_model, e2e_synchronize, e2e_postprocess, max_iters=args.steps)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    w = preprocess(seqs, [])
    h2d = sum(t.numel() * t.element_size() for t in (
        w.state.position_ids, w.state.attention_info.append_kv_token_indices, w.state.lm_head_indices,
        w.batch_indices) if t is not None)
    info = w.state.attention_info.decode_info
    for name in ("kv_indptr", "kv_indices", "kv_last_page_len"):
        t = getattr(info, name, None)
        if t is not None:
            h2d += t.numel() * t.element_size()
    release(seqs)

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            pseqs, pms, _ = decode_run(b, max(10, args.steps // 2), max(3, args.warmup // 2), f"p{b}_")
            points[f"decode_b{b}"] = round(b * 1e3 / pms, 1)
            release(pseqs)

    layers = cfg["num_hidden_layers"]
    return {
        "metric": "decode tokens/s (Llama-3.2-1B sizes, batch 8, 2,048-token prompts)",
        "value": round(args.batch * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids (seeded uniform), random weights N(0, 0.02)",
        "impl": "reference",
        "config": {
            "model": "Llama-3.2-1B sizes", "global_batch": args.batch, "seq_len": prompt_len, "context_len": context_len,
            "parallelism": "1 GPU", "layers": layers, "layers_full": 16, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": 64,
            "intermediate": cfg["intermediate_size"], "vocab": vocab, "page_size": page_size, "tied_embeddings": True,
            "rope": "llama3 factor 32", "l2": "inputs (2.5 GB of weights) larger than L2; no flush",
            "cuda_graphs": True, "timed_blocks": args.repeats,
        },
        "e2e": dict(value=round(args.batch * args.steps / e2e_s, 1), unit="tokens/s", h2d_bytes_per_step=h2d,
                    d2h_bytes_per_step=d2h[0] // max(1, args.steps), ms_per_step=round(e2e_s * 1e3 / args.steps, 4)),
        "prefill": dict(value=round(prompt_len / (pf_ms / 1e3), 1), tokens=prompt_len, ms=round(pf_ms, 3)),
        "clocks": clock_info, "points": points, "graph_replay_ms": None if replay_ms is None else round(replay_ms, 4), "block_ms": [round(s, 4) for s in samples], "setup_s": round(setup_s, 1),
        "path": "make_model -> ModelRunner (CUDA graphs) -> seqs_to_input / plan / run, FlashInfer "
                + __import__("flashinfer").__version__,
        "native_so_loaded": native_libraries(),
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--repeats", type=int, default=5, help="timed blocks of --steps steps; the median is reported")
    ap.add_argument("--skip-points", action="store_true")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    print(json.dumps(run(args)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
