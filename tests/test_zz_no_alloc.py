"""The allocation-free decode attention entry point (attention_decode_static.cu), called through
its exported C symbol the way a program without torch's allocator would call it: inputs and the
output are the caller's, the scratch between the two kernels is the library's fixed device
array.  Its result must equal the engine's usual entry point, which gets its scratch from torch,
on two calls in a row (the second call finds the first call's leftovers in the array).

This file is named so that it is collected last: a run that stops at the first failure has then
already run every other test.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(x):
    return torch.tensor(np.asarray(x, dtype=np.int32), device=DEV)


def make_case(seed, lens_kv, nh, nkv, hd, ps):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-L // ps) for L in lens_kv) + 3
    kc = torch.randn(n_pages, nkv, ps, hd, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(n_pages, nkv, ps, hd, generator=g).to(torch.bfloat16).to(DEV)
    perm = torch.randperm(n_pages, generator=g).tolist()
    indptr, pages = [0], []
    for L in lens_kv:
        pages += [perm.pop() for _ in range(-(-L // ps))]
        indptr.append(len(pages))
    qkv = torch.randn(len(lens_kv), (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16).to(DEV)
    return kc, vc, i32(indptr), i32(pages), qkv


def test_static_scratch_entry_point_matches_the_usual_one():
    from tokasaurus_b200.kernels import build, ops
    from tokasaurus_b200.parts.attention import plan_attention

    nh, nkv, hd, ps = 32, 8, 64, 16
    lib = build.load_module("attention_decode_static.cu", {"TKB_HD": hd})
    fn = lib.tkb_attn_decode_static_scratch_bf16
    fn.restype = c_int
    lib.tkb_attn_decode_static_scratch_capacity.restype = ctypes.c_longlong
    capacity = lib.tkb_attn_decode_static_scratch_capacity()
    assert capacity == 2 * 1024 * 1024

    def ptr(t):
        return c_void_p(t.data_ptr())

    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    for call, lens_kv in enumerate(([1, 300, 2049, 77, 1024], [513, 5, 1500])):
        kc, vc, indptr, pages, qkv = make_case(call, lens_kv, nh, nkv, hd, ps)
        B = len(lens_kv)
        plan = plan_attention(SimpleNamespace(seq_q_len=np.ones(B, dtype=np.int32),
                                              seq_kv_len=np.asarray(lens_kv, dtype=np.int32)), None)
        n_items, n_dec = int(plan["counts"][0]), int(plan["counts"][1])
        counts, items = i32(plan["counts"]), i32(plan["items"])
        dec_seqs, dec_start = i32(plan["dec_seqs"]), i32(plan["dec_item_start"])
        q_start, kv_len = i32(list(range(B))), i32(lens_kv)
        scale = 1 / math.sqrt(hd)
        want = torch.zeros(B, nh * hd, dtype=torch.bfloat16, device=DEV)
        ops.attn_decode_mma(qkv, kc, vc, q_start, kv_len, indptr, pages, items, counts[0:1], n_items, dec_seqs, dec_start,
                            counts[1:2], n_dec, want, nh, nkv, hd, ps, scale, None)
        got = torch.zeros_like(want)
        stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        before = torch.cuda.memory_allocated()
        rc = fn(ptr(qkv), c_int(qkv.shape[1]), ptr(kc), ptr(vc), ptr(q_start), ptr(kv_len), ptr(indptr), ptr(pages),
                ptr(items), ptr(counts[0:1]), c_int(n_items), ptr(dec_seqs), ptr(dec_start), ptr(counts[1:2]),
                c_int(n_dec), ptr(got), c_int(got.shape[1]), c_int(nh), c_int(nkv), c_int(ps), c_float(scale), c_int(0),
                c_int(kc.shape[0]), ptr(status), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=1e-2)
        assert torch.equal(got, want)  # same kernels, same order of sums: the same bits

    # a call that would not fit the built-in scratch is refused and launches nothing
    too_many = capacity // (nh * (hd + 2)) + 1
    rc = fn(ptr(qkv), c_int(qkv.shape[1]), ptr(kc), ptr(vc), ptr(q_start), ptr(kv_len), ptr(indptr), ptr(pages),
            ptr(items), ptr(counts[0:1]), c_int(too_many), ptr(dec_seqs), ptr(dec_start), ptr(counts[1:2]), c_int(n_dec),
            ptr(got), c_int(got.shape[1]), c_int(nh), c_int(nkv), c_int(ps), c_float(scale), c_int(0),
            c_int(kc.shape[0]), ptr(status), stream)
    assert rc == -4
    torch.cuda.synchronize()
    assert int(status) == 0
    # a block table that names a page beyond the caller's cache: the status bit is set, zeros stand in for the page,
    # nothing outside the cache is read
    bad = pages.clone()
    bad[0] = kc.shape[0] + 7
    rc = fn(ptr(qkv), c_int(qkv.shape[1]), ptr(kc), ptr(vc), ptr(q_start), ptr(kv_len), ptr(indptr), ptr(bad),
            ptr(items), ptr(counts[0:1]), c_int(n_items), ptr(dec_seqs), ptr(dec_start), ptr(counts[1:2]), c_int(n_dec),
            ptr(got), c_int(got.shape[1]), c_int(nh), c_int(nkv), c_int(ps), c_float(scale), c_int(0),
            c_int(kc.shape[0]), ptr(status), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status) & 2
