"""Compare the plain implementation (tests/plain_llama.py) ONCE with the reference's own model
code on a tiny random model, on the CPU, and store the reference's logits as a golden file.

Run by hand:  python tests/golden/make_reference_golden.py <path of the tokasaurus checkout>

What runs of the reference: ``tokasaurus.model.llama.LlamaForCausalLM`` in float32 (its RMSNorm,
projections, rotary tables and application, cache append indexing, residual order, last-layer row
restriction, head and weight tying) with inputs built by its own ``PageInformationBuilder`` /
``AttentionInfoBuilder`` / ``BatchState``.  What cannot run on a CPU and is replaced here: the
FlashInfer attention call (a plain paged softmax attention stands in) and the FlashInfer sampling
call (the float32 logits are captured instead).  Packages the reference imports but this image
lacks (pydra, accelerate, art, statsd) are stubbed.  The attention inner product and the sampling
therefore rest on the formulas, not on the reference's code.

Outputs (committed), for each of the two tiny test configurations i = 0 (tied head, plain rotary, two kv heads, pages
of 16) and 1 (own head, llama3 rotary scaling, one kv head, pages of 8): tests/golden/reference_cfg<i>_logits.npy
(float32 [tokens, vocab]: the prompt rows from a whole-prompt step and 1 row from a decode step) and
reference_cfg<i>_meta.json.
"""

import contextlib
import json
import math
import sys
import tempfile
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(HERE.parent))
if len(sys.argv) < 2:
    sys.exit("usage: make_reference_golden.py <folder of the reference's source tree>")
REF = sys.argv[1]
sys.path.insert(0, REF)


def stub_missing_packages():
    pydra = types.ModuleType("pydra")

    class Config:
        def __init__(self):
            pass

        def finalize(self):
            pass

    pydra.Config = Config
    pydra.run = lambda f: None
    pydra.main = lambda c: (lambda f: f)
    pydra.Alias = lambda x: x
    pydra.apply_overrides = lambda c, o: None
    sys.modules["pydra"] = pydra
    import transformers  # noqa: F401  (must be imported before accelerate is stubbed)

    acc = types.ModuleType("accelerate")

    @contextlib.contextmanager
    def init_empty_weights(include_buffers=False):
        yield

    acc.init_empty_weights = init_empty_weights
    sys.modules["accelerate"] = acc
    art = types.ModuleType("art")
    art.text2art = lambda s: s
    sys.modules["art"] = art
    statsd = types.ModuleType("statsd")
    statsd.StatsClient = object
    sys.modules["statsd"] = statsd


def main():
    stub_missing_packages()
    import tokasaurus.model.llama as L
    from tokasaurus.model.kv_cache import LayerKVCache
    from tokasaurus.model.types import (AttentionInfoBuilder, BatchSamplingParams, BatchState, ExtraModelConfig,
                                        ModelOutputTensors, PageInformationBuilder)
    from transformers import LlamaConfig

    from plain_llama import PlainLlama, tiny_configs, rope_inv_freq, rope_tables
    from tokasaurus_b200.weights import write_model_folder
    from safetensors import safe_open

    from plain_llama import TINY_WEIGHTS

    for index in (0, 1):
        golden_for(index, L, LayerKVCache, AttentionInfoBuilder, BatchSamplingParams, BatchState, ExtraModelConfig,
                   ModelOutputTensors, PageInformationBuilder, LlamaConfig, PlainLlama, tiny_configs()[index],
                   TINY_WEIGHTS[index], rope_inv_freq, rope_tables, write_model_folder, safe_open)


def golden_for(index, L, LayerKVCache, AttentionInfoBuilder, BatchSamplingParams, BatchState, ExtraModelConfig,
               ModelOutputTensors, PageInformationBuilder, LlamaConfig, PlainLlama, cfgd, wopt, rope_inv_freq,
               rope_tables, write_model_folder, safe_open):
    tmp = Path(tempfile.mkdtemp())
    folder = write_model_folder(tmp / f"cfg{index}", cfgd, seed=wopt["seed"], std=wopt["std"],
                                norm_init=wopt["norm_init"], store_dtype="float32")

    hf_cfg = LlamaConfig(**{k: v for k, v in cfgd.items() if k not in ("architectures", "model_type")})
    torch.set_default_dtype(torch.float32)
    model = L.LlamaForCausalLM(hf_cfg, ExtraModelConfig())
    tensors = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    # the reference's own mapping from checkpoint names to its parameter names
    name_map = model.make_name_to_hf_name()
    sd = {internal: tensors[hf] for internal, hf in name_map.items()}
    model.load_state_dict(sd, strict=False, assign=True)

    # 1. rotary tables: reference buffers against the plain formula
    hd = cfgd["hidden_size"] // cfgd["num_attention_heads"]
    inv = rope_inv_freq(hd, cfgd["rope_theta"], cfgd["rope_scaling"])
    cos, sin = rope_tables(torch.arange(cfgd["max_position_embeddings"]), inv)
    rope_diff = max((cos - model.model.rope_cos).abs().max().item(), (sin - model.model.rope_sin).abs().max().item())

    # 2. forward on the CPU with the attention and sampling library calls replaced
    ps = wopt["page_size"]

    def cpu_attention(ragged_q, ragged_k, ragged_v, k_cache, v_cache, attn_info, wrappers):
        from tokasaurus.model.attention_utils import append_to_kv_cache
        append_to_kv_cache(attn_info.append_kv_token_indices, ragged_k, ragged_v, k_cache, v_cache)

        def run(info, q):
            o = torch.empty_like(q)
            qpos = 0
            for s in range(info.num_seqs):
                pages = info.kv_indices[info.kv_indptr[s]:info.kv_indptr[s + 1]].tolist()
                kvlen = (len(pages) - 1) * ps + int(info.kv_last_page_len[s])
                K = torch.cat([k_cache[p] for p in pages])[:kvlen]
                V = torch.cat([v_cache[p] for p in pages])[:kvlen]
                nq = int(info.qo_indptr[s + 1] - info.qo_indptr[s]) if info.qo_indptr is not None else 1
                Q = q[qpos:qpos + nq]
                g = Q.shape[1] // K.shape[1]
                Kx = K.repeat_interleave(g, dim=1)
                Vx = V.repeat_interleave(g, dim=1)
                sc = torch.einsum("qhd,khd->hqk", Q.float(), Kx.float()) / math.sqrt(Q.shape[-1])
                qabs = torch.arange(kvlen - nq, kvlen).view(-1, 1)
                kabs = torch.arange(kvlen).view(1, -1)
                sc = sc.masked_fill(kabs > qabs, float("-inf"))
                o[qpos:qpos + nq] = torch.einsum("hqk,khd->qhd", sc.softmax(-1), Vx.float()).to(q.dtype)
                qpos += nq
            return o

        pq, _hq, dq = attn_info.split_q(ragged_q)
        return torch.cat([run(attn_info.prefill_info, pq), run(attn_info.decode_info, dq)], 0)

    L.tokasaurus_attention = cpu_attention
    torch.cuda.is_current_stream_capturing = lambda: False
    for layer in model.model.modules():
        if isinstance(layer, L.LlamaAttention):
            layer.layer_cache = LayerKVCache(head_dim=layer.head_dim(), num_kv_heads=layer.num_kv_heads, num_pages=8,
                                             page_size=ps, device="cpu", dtype=torch.float32)
            layer.wrapper_collection = object()
    captured = []

    def fake_calc(logits, temperature, greedy_mask, config):
        captured.append(logits.clone())
        return ModelOutputTensors(output_ids=logits.argmax(-1))

    L.calc_tokens_and_logprobs = fake_calc

    def step(ids, start, pages, lm_idx, decode=False):
        n = len(ids)
        pb, db = PageInformationBuilder(), PageInformationBuilder()
        (db if decode else pb).add_sequence(kv_indices=pages, kv_seq_len=start + n, num_qtokens=n, page_size=ps)
        ai = AttentionInfoBuilder(page_size=ps,
                                  append_kv_token_indices=[pages[i // ps] * ps + i % ps for i in range(start, start + n)],
                                  prefill_builder=pb, decode_builder=db).build()
        model.set_attention_info(ai)
        bs = BatchState(input_ids=ids, position_ids=torch.arange(start, start + n), attention_info=ai,
                        lm_head_indices=torch.tensor(lm_idx),
                        sampling_params=BatchSamplingParams(temperature=torch.ones(len(lm_idx)),
                                                            greedy_mask=torch.ones(len(lm_idx), dtype=torch.bool)))
        with torch.inference_mode():
            return model(bs)

    g = torch.Generator().manual_seed(3)
    n_ids = 12 if index == 1 else 21  # the prompt crosses a page edge in both
    ids = torch.randint(0, cfgd["vocab_size"], (n_ids,), generator=g)
    step(ids[:n_ids - 1], 0, [3, 5], list(range(n_ids - 1)))
    whole = captured[-1]
    step(ids[n_ids - 1:], n_ids - 1, [3, 5], [0], decode=True)
    dec = captured[-1]
    ref_logits = torch.cat([whole, dec], 0).float().numpy()

    plain32 = PlainLlama(folder, torch.float32).logits(ids.tolist()).float().numpy()
    plain64 = PlainLlama(folder, torch.float64).logits(ids.tolist()).double().numpy()
    d32 = float(np.abs(plain32 - ref_logits).max())
    d64 = float(np.abs(plain64 - ref_logits).max())
    np.save(HERE / f"reference_cfg{index}_logits.npy", ref_logits.astype(np.float32))
    meta = dict(config=cfgd, seed=wopt["seed"], std=wopt["std"], norm_init=wopt["norm_init"], store_dtype="float32", token_ids=ids.tolist(),
                rope_table_max_abs_diff=rope_diff, plain32_vs_reference_max_abs=d32, plain64_vs_reference_max_abs=d64,
                logits_abs_max=float(np.abs(ref_logits).max()), torch=torch.__version__,
                weights_checksum=float(sum(t.double().sum().item() for t in tensors.values())))
    with open(HERE / f"reference_cfg{index}_meta.json", "w") as f:
        json.dump(meta, f, indent=1)
    print(json.dumps({k: v for k, v in meta.items() if k != "config"}, indent=1))


if __name__ == "__main__":
    main()
