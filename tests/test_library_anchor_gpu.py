"""The attention formula and the sampler's distribution, pinned on the library that the reference calls.

The plain implementation's attention (``plain_llama.causal_gqa_attention``: scale 1/sqrt(head_dim), query i of a
portion of n tokens whose request holds m keys sees keys 0 .. m - n + i, query head j reads kv head j // group) is
a reading of FlashInfer's defaults.  Here FlashInfer's paged wrappers are called the way the reference calls them
(``plan`` as in tokasaurus/model/llama.py:716-764, wrappers made as in tokasaurus/model/attention_utils.py:25-47
with ``use_tensor_cores`` from the group size, ``run`` on the (k_cache, v_cache) pair of layout [page, slot, kv head,
head_dim] as in attention_utils.py:137-149) and compared with the plain function; the only change is the keyword
``head_dim``, which the installed FlashInfer calls ``head_dim_qk``.  The sampler: the reference draws from
softmax(logits / T) with ``flashinfer.sampling_from_probs`` (llama.py:362-397); this engine draws by the Gumbel-max
rule; both must follow the same distribution.  Test code only: nothing of this is on the product path.
Skipped where FlashInfer is not installed."""

import math

import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu
flashinfer = pytest.importorskip("flashinfer")
DEV = "cuda:0"


def paged(keys: torch.Tensor, page_size: int, pages: list[int], pool: torch.Tensor):
    """Write [T, nkv, hd] keys (or values) into the pages of a pool [P, page_size, nkv, hd]."""
    for t in range(keys.shape[0]):
        pool[pages[t // page_size], t % page_size] = keys[t]


@pytest.mark.parametrize("nh,nkv", [(3, 1), (8, 2), (4, 4)])
def test_flashinfer_paged_attention_equals_the_plain_formula(nh, nkv):
    hd, ps, n_pages = 64, 16, 64
    g = torch.Generator().manual_seed(nh * 10 + nkv)
    lengths = [(70, 23), (200, 200), (45, 1), (129, 2)]  # (keys held after the step, tokens the step brings)
    perm = torch.randperm(n_pages, generator=g).tolist()
    k_cache = torch.zeros(n_pages, ps, nkv, hd, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    seqs = []
    for m, n in lengths:
        q = torch.randn(m, nh, hd, generator=g).to(torch.bfloat16)
        k = torch.randn(m, nkv, hd, generator=g).to(torch.bfloat16)
        v = torch.randn(m, nkv, hd, generator=g).to(torch.bfloat16)
        k[m // 3] *= 6.0  # one far key stands out
        pages = [perm.pop() for _ in range(-(-m // ps))]
        paged(k.to(DEV), ps, pages, k_cache)
        paged(v.to(DEV), ps, pages, v_cache)
        want = plain.causal_gqa_attention(q.double(), k.double(), v.double())[m - n:]
        seqs.append(dict(m=m, n=n, q=q[m - n:], pages=pages, want=want))
    work = torch.empty(128 * 1024 * 1024, dtype=torch.uint8, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)  # noqa: E731

    def csr(which):
        indptr, indices, last = [0], [], []
        for s in which:
            indices += s["pages"]
            indptr.append(len(indices))
            last.append((s["m"] - 1) % ps + 1)
        return i32(indptr), i32(indices), i32(last)

    # portions: the prefill wrapper with causal=True over the request's pages, its keys including the portion
    pre = [s for s in seqs if s["n"] > 1]
    kv_indptr, kv_indices, kv_last = csr(pre)
    qo_indptr = i32(np.concatenate([[0], np.cumsum([s["n"] for s in pre])]))
    wrapper = flashinfer.BatchPrefillWithPagedKVCacheWrapper(work)
    wrapper.plan(qo_indptr=qo_indptr, paged_kv_indptr=kv_indptr, paged_kv_indices=kv_indices,
                 paged_kv_last_page_len=kv_last, num_kv_heads=nkv, num_qo_heads=nh, head_dim_qk=hd, page_size=ps,
                 q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16, causal=True, non_blocking=False)
    out = wrapper.run(q=torch.cat([s["q"] for s in pre]).to(DEV), paged_kv_cache=(k_cache, v_cache)).double().cpu()
    at = 0
    for s in pre:
        got = out[at:at + s["n"]]
        at += s["n"]
        assert (got - s["want"]).abs().max() < 0.02 * s["want"].abs().max(), ("portion", s["m"], s["n"])
    # single tokens: the decode wrapper, tensor cores from a group of four on as the reference chooses
    dec = [s for s in seqs if s["n"] == 1]
    kv_indptr, kv_indices, kv_last = csr(dec)
    wrapper = flashinfer.BatchDecodeWithPagedKVCacheWrapper(work, use_tensor_cores=(nh // nkv) >= 4)
    wrapper.plan(indptr=kv_indptr, indices=kv_indices, last_page_len=kv_last, num_kv_heads=nkv, num_qo_heads=nh,
                 head_dim=hd, page_size=ps, q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16, non_blocking=False)
    out, _lse = wrapper.run_return_lse(q=torch.cat([s["q"] for s in dec]).to(DEV), paged_kv_cache=(k_cache, v_cache))
    for i, s in enumerate(dec):
        got = out[i:i + 1].double().cpu()
        assert (got - s["want"]).abs().max() < 0.02 * s["want"].abs().max(), ("single token", s["m"])


def test_gumbel_max_and_the_library_sampler_follow_the_same_distribution():
    """20,000 draws each from softmax(logits / T) at T = 0.7 over 11 entries: the reference's way (probabilities,
    then ``flashinfer.sampling_from_probs``) and this engine's (Gumbel-max over the logits), both against the
    probabilities by chi-square, and against each other."""
    from tokasaurus_b200.kernels import ops

    V, N, T = 11, 20000, 0.7
    logits = torch.tensor([1.2, 0.1, -0.7, 2.1, 0.0, -3.0, 1.4, 0.6, -1.1, 0.9, 0.3], device=DEV)
    rows = logits.repeat(N, 1).contiguous()
    probs = torch.softmax(rows / T, dim=-1)  # tokasaurus/model/llama.py:377-384
    theirs = flashinfer.sampling_from_probs(probs).long().cpu()
    ids = torch.zeros(N, dtype=torch.int32, device=DEV)
    ops.sample(rows, torch.full((N,), T, device=DEV), torch.arange(N, dtype=torch.int64, device=DEV) * 104729 + 5,
               torch.zeros(N, dtype=torch.int32, device=DEV), None, ids, None, None)
    ours = ids.long().cpu()
    p = probs[0].double().cpu()
    limit = 29.6  # 99.9 % point of chi-square with 10 degrees of freedom
    for name, draws in (("library", theirs), ("gumbel-max", ours)):
        counts = torch.bincount(draws, minlength=V).double()
        chi2 = (((counts - N * p) ** 2) / (N * p)).sum().item()
        assert chi2 < limit, (name, chi2)
    a, b = torch.bincount(theirs, minlength=V).double(), torch.bincount(ours, minlength=V).double()
    chi2 = (((a - b) ** 2) / (a + b).clamp(min=1)).sum().item()
    assert chi2 < limit, ("library against gumbel-max", chi2)
