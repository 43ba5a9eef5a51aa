"""Plain PyTorch statements of what each kernel computes, with the signatures of
``tokasaurus_b200.kernels.ops``.  The GPU tests compare every kernel with these; the CPU tests
put them in the kernels' place (``install_cpu_kernels``) so that the step function, the cache
manager and the scheduler can be exercised together on a machine without a GPU.  They are test
code: the engine itself has no such path.
"""

from __future__ import annotations

import math

import numpy as np
import torch


def embed_gather(table, ids, token_seq, seq_slot, last_token, x_out, status):
    n = x_out.shape[0]
    for t in range(n):
        s = int(token_seq[t])
        if s < 0:
            x_out[t] = 0
            continue
        i = int(ids[t])
        if i < 0:
            i = int(last_token[int(seq_slot[s])])
        if not 0 <= i < table.shape[0]:
            status |= 1
            x_out[t] = 0
        else:
            x_out[t] = table[i].float()


def add_rmsnorm(x, delta, weight, eps, out):
    if delta is not None and delta.dim() == 3:
        x += delta.double().sum(0).float()
    elif delta is not None:
        x += delta.float()
    var = x.double().pow(2).mean(-1, keepdim=True)
    out.copy_((x.double() * torch.rsqrt(var + eps) * weight.double()).to(out.dtype))


def rope_kv_write(qkv, positions, token_seq, page_indptr, page_ids, inv_freq, kcache, vcache, n_heads, n_kv_heads,
                  head_dim, rotary_dim, page_size, write_cache, status, bias=None, qk_norm=None, norm_eps=0.0):
    """The element-wise stage before the rotation: ``bias`` [C] is added to the row and the sum rounded to the
    row's type; ``qk_norm`` [2, head_dim] RMS-normalises every q head and every k head (rounded to the row's type)."""
    T = qkv.shape[0]
    nh, nkv, hd = n_heads, n_kv_heads, head_dim
    half = rotary_dim // 2
    for t in range(T):
        s = int(token_seq[t])
        if s < 0:
            continue
        p = int(positions[t])
        row = qkv[t].float()
        if bias is not None:
            row = (row + bias.float().to(row.device)).to(qkv.dtype).float()
        q = row[: nh * hd].view(nh, hd).clone()
        k = row[nh * hd:(nh + nkv) * hd].view(nkv, hd).clone()
        v = row[(nh + nkv) * hd:].view(nkv, hd).to(qkv.dtype)
        if qk_norm is not None:
            w = qk_norm.float().to(row.device)
            q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + norm_eps) * w[0]).to(qkv.dtype).float()
            k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + norm_eps) * w[1]).to(qkv.dtype).float()
        if rotary_dim:
            ang = torch.tensor(float(p), dtype=torch.float32) * inv_freq.float().cpu()
            c, sn = ang.cos().to(row.device), ang.sin().to(row.device)

            def rot(x):
                x1, x2 = x[:, :half].clone(), x[:, half:rotary_dim].clone()
                x[:, :half] = x1 * c - x2 * sn
                x[:, half:rotary_dim] = x2 * c + x1 * sn
                return x
            q, k = rot(q), rot(k)
        qkv[t, : nh * hd] = q.reshape(-1).to(qkv.dtype)
        if not write_cache:
            continue
        page = int(page_ids[int(page_indptr[s]) + p // page_size])
        if not 0 <= page < kcache.shape[0]:
            status |= 2
            continue
        kcache[page, :, p % page_size, :] = k.to(kcache.dtype)
        vcache[page, :, p % page_size, :] = v


def silu_mul(gate_up, out, interleave=0):
    I = out.shape[1]
    if interleave:
        v = gate_up.view(gate_up.shape[0], I // 8, 2, 8)
        g, u = v[:, :, 0].reshape(-1, I).float(), v[:, :, 1].reshape(-1, I).float()
    else:
        g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def gather_rows(src, rows, out):
    out.copy_(src[rows.long()])


def sgemm_tn(a, w, out):
    out.copy_((a.double() @ w.double().T).float())


def attn_paged(q, q_stride, out, kcache, vcache, token_seq, positions, page_indptr, page_ids, rows, n_rows, n_heads,
               n_kv_heads, head_dim, page_size, scale, window, status=None):
    group = n_heads // n_kv_heads
    for r in range(n_rows):
        t = int(rows[r]) if rows is not None else r
        s = int(token_seq[t])
        if s < 0:
            continue
        p = int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        table = page_ids[int(page_indptr[s]):]
        keys = list(range(lo, p + 1))
        pg = torch.tensor([int(table[j // page_size]) for j in keys], dtype=torch.long, device=kcache.device)
        sl = torch.tensor([j % page_size for j in keys], dtype=torch.long, device=kcache.device)
        K = kcache[pg, :, sl, :].double()  # [keys, nkv, hd]
        V = vcache[pg, :, sl, :].double()
        qv = q[t, : n_heads * head_dim].double().view(n_heads, head_dim)
        for h in range(n_heads):
            kv = h // group
            sc = (K[:, kv, :] @ qv[h]) * scale
            pr = torch.softmax(sc, dim=0)
            out[r, h * head_dim:(h + 1) * head_dim] = (pr @ V[:, kv, :]).to(out.dtype)


def philox4x32_10(ctr: np.ndarray, key: np.ndarray) -> np.ndarray:
    """ctr uint32 [n, 4], key uint32 [2] -> uint32 [n, 4]."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c = ctr.astype(np.uint64)
    k0, k1 = int(key[0]), int(key[1])
    for _ in range(10):
        p0 = M0 * c[:, 0]
        p1 = M1 * c[:, 2]
        hi0, lo0 = p0 >> 32, p0 & 0xFFFFFFFF
        hi1, lo1 = p1 >> 32, p1 & 0xFFFFFFFF
        c = np.stack([hi1 ^ c[:, 1] ^ k0, lo1, hi0 ^ c[:, 3] ^ k1, lo0], axis=1)
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return c.astype(np.uint32)


def uniform_open(bits: np.ndarray) -> np.ndarray:
    """32 random bits -> a float32 inside (0, 1), with the kernel's float32 operations: 23 bits plus one half
    are exact in a 24-bit significand (24 bits plus one half are not: the largest would round up to 1)."""
    return ((bits.astype(np.uint32) >> np.uint32(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)


def gumbel_noise(vocab: int, stream_key: int, pos: int) -> np.ndarray:
    """The Gumbel noise the sampling kernel adds to row logits / T (the uniform in float32 as in the kernel,
    the logarithms in float64)."""
    groups = (vocab + 3) // 4
    ctr = np.zeros((groups, 4), dtype=np.uint32)
    ctr[:, 0] = np.arange(groups, dtype=np.uint32)
    ctr[:, 1] = np.uint32(pos)
    key = np.array([stream_key & 0xFFFFFFFF, (stream_key >> 32) & 0xFFFFFFFF], dtype=np.uint32)
    r = philox4x32_10(ctr, key).reshape(-1)[:vocab]
    u = uniform_open(r).astype(np.float64)
    return -np.log(-np.log(u))


def sample(logits, temperature, stream_key, sample_pos, row_slot, out_ids, out_logprob, last_token):
    R, V = logits.shape
    for r in range(R):
        T = float(temperature[r]) if temperature is not None else 0.0
        z = logits[r].double().cpu().numpy() / (T if T > 0 else 1.0)
        score = z
        if T > 0:
            key = int(stream_key[r]) & 0xFFFFFFFFFFFFFFFF if stream_key is not None else 0
            score = z + gumbel_noise(V, key, int(sample_pos[r]) if sample_pos is not None else 0)
        c = int(np.argmax(score))
        out_ids[r] = c
        if out_logprob is not None:
            m = z.max()
            out_logprob[r] = float(z[c] - (m + math.log(np.exp(z - m).sum())))
        if last_token is not None and row_slot is not None and int(row_slot[r]) >= 0:
            last_token[int(row_slot[r])] = c


def topk_logprobs(logits, temperature, k, out_idx, out_lp):
    R, V = logits.shape
    for r in range(R):
        T = float(temperature[r]) if temperature is not None else 0.0
        z = logits[r].double() / (T if T > 0 else 1.0)
        lp = torch.log_softmax(z, dim=0)
        order = sorted(range(V), key=lambda i: (-float(z[i]), i))[:k]
        for j, i in enumerate(order):
            out_idx[r, j] = i
            out_lp[r, j] = float(lp[i])


def linear(a, w, out_dtype=None):
    out = a.double() @ w.double().T
    return out.to(out_dtype or a.dtype)


def install_cpu_kernels(monkeypatch):
    """Put the plain statements above in the place of the kernels (CPU tests only)."""
    from tokasaurus_b200.engine import runner
    from tokasaurus_b200.kernels import ops

    for name in ("embed_gather", "add_rmsnorm", "rope_kv_write", "silu_mul", "gather_rows", "sgemm_tn", "attn_paged",
                 "sample", "topk_logprobs", "linear"):
        monkeypatch.setattr(ops, name, globals()[name])
    monkeypatch.setattr(ops, "prepare", lambda *a, **k: None)
    monkeypatch.setattr(runner, "require_cuda", lambda device: None)
