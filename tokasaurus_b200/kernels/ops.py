"""Tensor-level entry points of the hand-written kernels.

Each function checks its arguments, then launches one kernel on the current CUDA stream through
the ctypes library built by ``tokasaurus_b200.kernels.build``.  There is no other
implementation behind these functions: a tensor that is not on a CUDA device, or a library
that cannot be built or loaded, raises.
"""

from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import torch

from tokasaurus_b200.kernels import build


class KernelError(RuntimeError):
    pass


_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}


def _suffix(dtype: torch.dtype) -> str:
    try:
        return _SUFFIX[dtype]
    except KeyError:
        raise KernelError(f"kernels exist for float32 and bfloat16 activations, not {dtype}") from None


def _ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current CUDA stream of the current device as a raw handle (the direct binding where torch has
    it: ``torch.cuda.current_stream()`` costs more on the host than a kernel launch)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(
                "this engine runs on CUDA devices only; got a tensor on " + str(t.device)
            )


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


LAUNCHES = 0  # kernels of this engine launched so far (the benchmark reads and resets it)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        if code > 0:
            raise KernelError(f"{what}: CUDA launch failed with error {code}")
        reason = {-2: "sizes not supported", -3: "grid too large", -4: "size beyond the built-in scratch"}.get(
            code, "refused"
        )
        raise KernelError(f"{what}: {reason} (code {code})")


def _fn(lib: ctypes.CDLL, name: str):
    f = lib.__dict__.get(name)  # ctypes keeps a function it has looked up once as an attribute of the library
    if f is not None:
        return f
    try:
        f = getattr(lib, name)
    except AttributeError:
        raise KernelError(f"compiled kernel library lacks the symbol {name}") from None
    f.restype = c_int
    return f


class _Libs:
    def __init__(self) -> None:
        self._cache: dict[tuple, ctypes.CDLL] = {}

    def get(self, source: str, **defines) -> ctypes.CDLL:
        key = (source, tuple(defines.items())) if len(defines) < 2 else (source, tuple(sorted(defines.items())))
        lib = self._cache.get(key)
        if lib is None:
            lib = build.load_module(source, defines or None)
            self._cache[key] = lib
        return lib


_libs = _Libs()


def check_head_dim(hd: int) -> None:
    if hd % 16 or not 16 <= hd <= 256:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 up to 256, not {hd}")


def prepare(head_dims=(), dtype: torch.dtype = torch.bfloat16) -> None:
    """Build and load everything a model with these head sizes needs (first call compiles)."""
    from tokasaurus_b200.kernels.modules import all_modules

    for hd in head_dims:
        check_head_dim(hd)
    name = {torch.float32: "float32", torch.bfloat16: "bfloat16"}.get(dtype)
    for source, defines in all_modules(head_dims, name):
        _libs.get(source, **(defines or {}))


# ---------------------------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, token_seq: torch.Tensor, seq_slot: torch.Tensor,
                 last_token: torch.Tensor, x_out: torch.Tensor, status: torch.Tensor) -> None:
    """x_out[t] = table[ids[t]] as float32; ids[t] < 0 takes last_token[seq_slot[token_seq[t]]]."""
    _need_cuda(table, ids, token_seq, seq_slot, last_token, x_out, status)
    n, H = x_out.shape
    V = table.shape[0]
    _need(table.shape[1] == H and table.is_contiguous() and x_out.is_contiguous(), "embed_gather: bad table/x shapes")
    _need(x_out.dtype == torch.float32, "embed_gather: the residual stream is float32")
    _need(ids.dtype == torch.int32 and ids.numel() >= n and token_seq.numel() >= n, "embed_gather: ids int32 [T]")
    f = _fn(_libs.get("elementwise.cu"), f"tkb_embed_gather_{_suffix(table.dtype)}")
    _check(f(_ptr(table), _ptr(ids), _ptr(token_seq), _ptr(seq_slot), _ptr(last_token), _ptr(x_out), c_int(n),
             c_int(H), c_int(V), _ptr(status), _stream()), "embed_gather")


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """x += delta (float32, in place) if delta is given; out = rmsnorm(x) * weight in out's dtype.

    ``delta`` is [rows, H] in out's dtype, or float32 [slices, rows, H]: the slices of a split matrix
    product (``linear_smallm``), added in slice order."""
    _need_cuda(x, delta, weight, out)
    rows, H = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "add_rmsnorm: x must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == H, "add_rmsnorm: weight must be float32 [H]")
    _need(out.shape == x.shape and out.is_contiguous(), "add_rmsnorm: out shape")
    partials, n_part, stride = None, 0, 0
    if delta is not None and delta.dim() == 3:
        _need(delta.dtype == torch.float32 and tuple(delta.shape[1:]) == (rows, H) and delta.is_contiguous(),
              "add_rmsnorm: partial sums must be contiguous float32 [slices, rows, H]")
        partials, n_part, stride, delta = delta, delta.shape[0], rows * H, None
    elif delta is not None:
        _need(delta.shape == x.shape and delta.dtype == out.dtype and delta.is_contiguous(), "add_rmsnorm: delta")
    f = _fn(_libs.get("elementwise.cu"), f"tkb_add_rmsnorm_{_suffix(out.dtype)}")
    _check(f(_ptr(x), _ptr(delta), _ptr(partials), c_int(n_part), ctypes.c_longlong(stride), _ptr(weight), _ptr(out),
             c_float(eps), c_int(rows), c_int(H), _stream()), "add_rmsnorm")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor, page_indptr: torch.Tensor,
                  page_ids: torch.Tensor, inv_freq: torch.Tensor | None, kcache: torch.Tensor, vcache: torch.Tensor,
                  n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                  write_cache: bool, status: torch.Tensor, bias: torch.Tensor | None = None,
                  qk_norm: torch.Tensor | None = None, norm_eps: float = 0.0) -> None:
    """Rotate q (in place) and k by position, write rotated k and v into the request's pages.

    kcache/vcache: [pages, n_kv_heads, page_size, head_dim].  The element-wise stage before the rotation:
    ``bias`` float32 [C] is added to the row; ``qk_norm`` float32 [2, head_dim] RMS-normalises every q head (first
    row of weights) and every k head (second row) over the head size, with ``norm_eps``."""
    _need_cuda(qkv, positions, token_seq, page_indptr, page_ids, inv_freq, kcache, vcache, status, bias, qk_norm)
    _check_qkv_stage(bias, qk_norm, (n_heads + 2 * n_kv_heads) * head_dim, head_dim)
    n = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim, "rope_kv_write: qkv shape")
    _need(kcache.is_contiguous() and vcache.is_contiguous() and kcache.dtype == qkv.dtype, "rope_kv_write: cache")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "rope_kv_write: cache layout")
    _need(0 <= rotary_dim <= head_dim and rotary_dim % 2 == 0, "rope_kv_write: rotary_dim")
    if rotary_dim:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
              "rope_kv_write: inv_freq must be float32 [rotary_dim/2]")
    f = _fn(_libs.get("elementwise.cu"), f"tkb_rope_kv_write_{_suffix(qkv.dtype)}")
    _check(f(_ptr(qkv), _ptr(positions), _ptr(token_seq), _ptr(page_indptr), _ptr(page_ids), _ptr(inv_freq),
             _ptr(kcache), _ptr(vcache), c_int(n), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
             c_int(rotary_dim), c_int(page_size), c_int(kcache.shape[0]), c_int(1 if write_cache else 0),
             _ptr(status), _ptr(bias), _ptr(qk_norm), c_float(norm_eps), _stream()), "rope_kv_write")


def _check_qkv_stage(bias: torch.Tensor | None, qk_norm: torch.Tensor | None, C: int, head_dim: int) -> None:
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C, "q|k|v bias: float32 [C]")
    if qk_norm is not None:
        _need(qk_norm.dtype == torch.float32 and qk_norm.is_contiguous() and tuple(qk_norm.shape) == (2, head_dim),
              "q/k norm weights: float32 [2, head_dim]")


SMALL_M_MAX = 16   # above this many rows the library product is as fast or faster (measured on B200)
GATED_M_MAX = 8    # the gated small-batch product wins only up to this many rows
DECODE_M_MAX = 16
_EPILOGUES = {"bf16": 0, "add": 1, "gated": 2, "f32": 3}


def can_use_linear_decode(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (w.dtype == torch.bfloat16 and a.dtype in (torch.bfloat16, torch.float32) and 0 < a.shape[0] <= DECODE_M_MAX
            and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1)


def linear_decode(a: torch.Tensor, w: torch.Tensor, epilogue: str = "bf16", norm_weight: torch.Tensor | None = None,
                  eps: float = 0.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Fused product for at most 16 rows: ``prologue(a) @ w^T`` with the epilogue applied in the same kernel.

    ``a``: bfloat16 [M, K], or the float32 residual stream [M, K] with ``norm_weight`` (an RMS norm is
    folded in).  ``epilogue``: "bf16" store; "f32" store; "add" adds into the float32 ``out`` [M, N] in place;
    "gated": ``w`` interleaves gate/up rows (``interleave_gate_up``), result silu(gate)*up [M, N/2]."""
    _need_cuda(a, w, norm_weight, out)
    _need(can_use_linear_decode(a, w), "linear_decode: at most 16 rows, bfloat16 weights, K a multiple of 8")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K, "linear_decode: shapes")
    pro = 1 if a.dtype == torch.float32 else 0
    _need((pro == 1) == (norm_weight is not None), "linear_decode: a float32 input goes with a norm weight")
    if pro:
        _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == K, "linear_decode: norm weight float32 [K]")
    epi = _EPILOGUES[epilogue]
    if epilogue == "add":
        _need(out is not None and out.dtype == torch.float32 and tuple(out.shape) == (M, N) and out.stride(1) == 1,
              "linear_decode: 'add' needs the float32 stream [M, N]")
    elif epilogue == "gated":
        _need(N % 16 == 0, "linear_decode: gated weights come in groups of 16 rows")
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    else:
        out = torch.empty((M, N), dtype=torch.bfloat16 if epilogue == "bf16" else torch.float32, device=a.device)
    _check(_fn(_libs.get("linear_decode.cu"), "tkb_linear_decode_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(norm_weight), c_float(eps), _ptr(w), c_int(w.stride(0)), _ptr(out),
        c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(pro), c_int(epi), _stream()), "linear_decode")
    return out


def can_use_smallm(a: torch.Tensor, w: torch.Tensor, max_rows: int | None = None) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < a.shape[0] <= (max_rows or SMALL_M_MAX)
            and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def linear_smallm(a: torch.Tensor, w: torch.Tensor, max_slices: int = 8) -> torch.Tensor:
    """a[M, K] @ w[N, K]^T for M <= 64 in bfloat16, as float32 slices [slices, M, N] of a K-split
    product (the consumer adds the slices).  ``max_slices=1`` gives the whole product as [1, M, N]."""
    _need_cuda(a, w)
    _need(can_use_smallm(a, w, 64), "linear_smallm: bfloat16, M <= 64, K a multiple of 8")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and a.stride(1) == 1 and w.stride(1) == 1, "linear_smallm: shapes")
    lib = _libs.get("linear_smallm.cu")
    slices = lib.tkb_linear_smallm_slices(c_int(N), c_int(K), c_int(max_slices))
    out = torch.empty((slices, M, N), dtype=torch.float32, device=a.device)
    _check(_fn(lib, "tkb_linear_smallm_bf16")(_ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out),
                                              c_int(M), c_int(N), c_int(K), c_int(slices), _stream()), "linear_smallm")
    return out


def linear_smallm_gated(a: torch.Tensor, w_interleaved: torch.Tensor) -> torch.Tensor:
    """silu(a @ gate^T) * (a @ up^T) as bfloat16 [M, I] for M <= 64; ``w_interleaved`` [2I, K] holds gate
    and up rows in groups of 8 (``interleave_gate_up``)."""
    _need_cuda(a, w_interleaved)
    _need(can_use_smallm(a, w_interleaved, 64) and w_interleaved.shape[0] % 16 == 0, "linear_smallm_gated: operands")
    M, K = a.shape
    N = w_interleaved.shape[0]
    out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    _check(_fn(_libs.get("linear_smallm.cu"), "tkb_linear_smallm_gated_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(w_interleaved), c_int(w_interleaved.stride(0)), _ptr(out), c_int(M), c_int(N),
        c_int(K), _stream()), "linear_smallm_gated")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2I, K]: for every 8 features, their 8 gate rows then their 8 up rows.  I must be a multiple of 8."""
    I, K = gate.shape
    _need(I % 8 == 0 and up.shape == gate.shape, "interleave_gate_up: I must be a multiple of 8")
    return torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


def rope_kv_write_partials(partials: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                           token_seq: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor,
                           inv_freq: torch.Tensor | None, kcache: torch.Tensor, vcache: torch.Tensor, n_heads: int,
                           n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int, write_cache: bool,
                           status: torch.Tensor, bias: torch.Tensor | None = None,
                           qk_norm: torch.Tensor | None = None, norm_eps: float = 0.0) -> None:
    """``rope_kv_write`` for q|k|v that arrive as float32 slices [slices, T, C] of a split product: the
    slices are added, q is rotated into ``q_out`` [T, n_heads*head_dim] (bfloat16), k and v go to the cache."""
    _need_cuda(partials, q_out, positions, token_seq, page_indptr, page_ids, inv_freq, kcache, vcache, status, bias,
               qk_norm)
    S, T, C = partials.shape
    _check_qkv_stage(bias, qk_norm, C, head_dim)
    _need(partials.dtype == torch.float32 and partials.is_contiguous() and C == (n_heads + 2 * n_kv_heads) * head_dim,
          "rope_kv_write_partials: partials")
    _need(q_out.dtype == torch.bfloat16 and q_out.is_contiguous() and tuple(q_out.shape) == (T, n_heads * head_dim),
          "rope_kv_write_partials: q_out")
    _need(kcache.dtype == torch.bfloat16 and tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim),
          "rope_kv_write_partials: cache layout")
    _need((C + max(rotary_dim, 2)) * 4 <= 160 * 1024, "rope_kv_write_partials: row too wide for shared memory")
    f = _fn(_libs.get("elementwise.cu"), "tkb_rope_kv_write_partials_bf16")
    _check(f(_ptr(partials), c_int(S), ctypes.c_longlong(T * C), _ptr(q_out), _ptr(positions), _ptr(token_seq),
             _ptr(page_indptr), _ptr(page_ids), _ptr(inv_freq), _ptr(kcache), _ptr(vcache), c_int(T), c_int(n_heads),
             c_int(n_kv_heads), c_int(head_dim), c_int(rotary_dim), c_int(page_size), c_int(kcache.shape[0]),
             c_int(1 if write_cache else 0), _ptr(status), _ptr(bias), _ptr(qk_norm), c_float(norm_eps), _stream()),
           "rope_kv_write_partials")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> None:
    """out[t, i] = silu(gate[t, i]) * up[t, i].  interleave 0: gate_up = [gate | up]; interleave 8: columns in
    groups of 16, 8 gate columns then the 8 up columns of the same features."""
    _need_cuda(gate_up, out)
    rows, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape == (rows, two_i // 2), "silu_mul: shapes")
    _need(gate_up.is_contiguous() and out.is_contiguous() and out.dtype == gate_up.dtype, "silu_mul: layout")
    f = _fn(_libs.get("elementwise.cu"), f"tkb_silu_mul_{_suffix(out.dtype)}")
    _check(f(_ptr(gate_up), _ptr(out), c_int(rows), c_int(two_i // 2), c_int(interleave), _stream()), "silu_mul")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = src[rows[r]]."""
    _need_cuda(src, rows, out)
    _need(src.is_contiguous() and out.is_contiguous() and src.dtype == out.dtype, "gather_rows: layout")
    _need(rows.dtype == torch.int32 and out.shape[0] == rows.numel() and out.shape[1:] == src.shape[1:],
          "gather_rows: shapes")
    row_bytes = src[0].numel() * src.element_size() if src.shape[0] else 0
    f = _fn(_libs.get("elementwise.cu"), "tkb_gather_rows")
    _check(f(_ptr(src), _ptr(out), _ptr(rows), c_int(rows.numel()), c_int(row_bytes), _stream()), "gather_rows")


def sgemm_tn(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FP32 FMA, fixed summation order)."""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "sgemm_tn: shapes")
    _need(a.dtype == w.dtype == out.dtype == torch.float32, "sgemm_tn: float32 only")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "sgemm_tn: rows must be contiguous")
    f = _fn(_libs.get("sgemm.cu"), "tkb_sgemm_tn_f32")
    _check(f(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0) if M > 1 else K),
             c_int(w.stride(0) if N > 1 else K), c_int(out.stride(0) if M > 1 else N), _stream()), "sgemm_tn")


def attn_paged(q: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
               token_seq: torch.Tensor, positions: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor,
               rows: torch.Tensor | None, n_rows: int, n_heads: int, n_kv_heads: int, head_dim: int,
               page_size: int, scale: float, window: int | None, status: torch.Tensor | None = None) -> None:
    """Causal GQA attention over the paged cache on the FP32 pipes (any mix of portions and single tokens).

    q: first n_heads*head_dim columns of each row of a [T, q_stride] buffer; out: [n_rows, n_heads*head_dim].
    ``status``: the device status word; a page id beyond the pool sets its bit 2 and its keys count for nothing."""
    _need_cuda(q, out, kcache, vcache, token_seq, positions, page_indptr, page_ids, rows, status)
    check_head_dim(head_dim)
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim and out.shape[0] >= n_rows, "attn_paged: out")
    _need(kcache.dtype == q.dtype == out.dtype, "attn_paged: dtypes")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "attn_paged: cache layout")
    f = _fn(_libs.get("attention_simt.cu", TKB_HD=head_dim), f"tkb_attn_paged_simt_{_suffix(q.dtype)}")
    _check(f(_ptr(q), c_int(q_stride), _ptr(out), c_int(out.shape[1]), _ptr(kcache), _ptr(vcache), _ptr(token_seq),
             _ptr(positions), _ptr(page_indptr), _ptr(page_ids), _ptr(rows), c_int(n_rows), c_int(n_heads),
             c_int(n_kv_heads), c_int(page_size), c_float(scale), c_int(window or 0), c_int(kcache.shape[0]), _ptr(status),
             _stream()), "attn_paged")


_COUNTERS: dict = {}
_COUNTER_INTS = 1 << 20


def _decode_counters(device: torch.device, dec_cap: int, n_heads: int, n_kv_heads: int) -> torch.Tensor | None:
    """Arrival counters of the split-key kernel's in-kernel merge: one fixed zero-initialised array per device
    (every launch leaves it zero again).  None if a launch would need more than it holds."""
    group = n_heads // n_kv_heads
    need = dec_cap * n_kv_heads * ((group + 15) // 16)
    if need > _COUNTER_INTS:
        return None
    key = (device.type, device.index)
    t = _COUNTERS.get(key)
    if t is None:
        t = torch.zeros((_COUNTER_INTS,), dtype=torch.int32, device=device)
        _COUNTERS[key] = t
    return t


def attn_decode_mma(qkv: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, seq_q_start: torch.Tensor,
                    seq_kv_len: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor, items: torch.Tensor,
                    n_items: torch.Tensor, items_cap: int, dec_seqs: torch.Tensor, dec_item_start: torch.Tensor,
                    n_dec: torch.Tensor, dec_cap: int, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                    page_size: int, scale: float, window: int | None,
                    out_row_of: torch.Tensor | None = None, item_entry: torch.Tensor | None = None,
                    tma: bool = True, status: torch.Tensor | None = None) -> None:
    """bfloat16 split-key attention for requests that bring one token: ``items`` are (request row,
    first key, number of keys) triples, computed into float32 partial results and merged into
    ``out`` [T, n_heads*head_dim] at each request's token row (or at row ``out_row_of[request]``).
    ``n_items``/``n_dec`` are device counters; the launch grids are sized by ``items_cap``/``dec_cap``.
    ``tma``: some work item is longer than three tiles (the kernel variant that fetches tiles by TMA pays)."""
    _need_cuda(qkv, kcache, vcache, seq_q_start, seq_kv_len, page_indptr, page_ids, items, n_items, dec_seqs,
               dec_item_start, n_dec, out, status)
    check_head_dim(head_dim)
    _need(qkv.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attn_decode_mma: bfloat16 only")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "attn_decode_mma: cache layout")
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim, "attn_decode_mma: out")
    _need(items.numel() >= 3 * items_cap and dec_item_start.numel() >= dec_cap + 1, "attn_decode_mma: plan arrays")
    lib = _libs.get("attention_mma.cu", TKB_HD=head_dim)
    part_o = torch.empty((items_cap, n_heads, head_dim), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((items_cap, n_heads, 2), dtype=torch.float32, device=qkv.device)
    counters = _decode_counters(qkv.device, dec_cap, n_heads, n_kv_heads) if item_entry is not None else None
    if counters is not None:
        # the merge of the splits happens inside the attention kernel
        _check(_fn(lib, "tkb_attn_decode_merged_bf16")(
            _ptr(qkv), c_int(qkv.shape[1]), _ptr(None), c_int(0), ctypes.c_longlong(0), _ptr(kcache), _ptr(vcache),
            _ptr(seq_q_start), _ptr(seq_kv_len), _ptr(page_indptr), _ptr(page_ids), _ptr(items), _ptr(n_items),
            c_int(items_cap), _ptr(part_o), _ptr(part_ml), c_int(n_heads), c_int(n_kv_heads), c_int(page_size),
            c_float(scale), c_int(window or 0), c_int(0), _ptr(None), c_int(0), c_int(0), c_int(kcache.shape[0]),
            c_int(1 if tma else 0), _ptr(status), _ptr(counters), _ptr(item_entry), _ptr(dec_item_start),
            _ptr(out_row_of if out_row_of is not None else seq_q_start), _ptr(out), c_int(out.shape[1]), _ptr(None),
            _ptr(None), c_float(0.0), _stream()), "attn_decode_merged")
        return
    _check(_fn(lib, "tkb_attn_decode_mma_bf16")(
        _ptr(qkv), c_int(qkv.shape[1]), _ptr(kcache), _ptr(vcache), _ptr(seq_q_start), _ptr(seq_kv_len),
        _ptr(page_indptr), _ptr(page_ids), _ptr(items), _ptr(n_items), c_int(items_cap), _ptr(part_o), _ptr(part_ml),
        c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale), c_int(window or 0),
        c_int(kcache.shape[0]), _ptr(status), _stream()), "attn_decode_mma")
    _check(_fn(lib, "tkb_attn_decode_merge_bf16")(
        _ptr(part_o), _ptr(part_ml), _ptr(dec_seqs), _ptr(dec_item_start), _ptr(n_dec), c_int(dec_cap),
        _ptr(out_row_of if out_row_of is not None else seq_q_start), _ptr(out), c_int(out.shape[1]), c_int(n_heads),
        _stream()), "attn_decode_merge")


def attn_decode_rope_mma(qkv: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, seq_q_start: torch.Tensor,
                         seq_kv_len: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor,
                         items: torch.Tensor, n_items: torch.Tensor, items_cap: int, dec_seqs: torch.Tensor,
                         dec_item_start: torch.Tensor, n_dec: torch.Tensor, dec_cap: int, out: torch.Tensor,
                         n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                         window: int | None, inv_freq: torch.Tensor | None, rotary_dim: int,
                         write_cache: bool, status: torch.Tensor, item_entry: torch.Tensor | None = None,
                         tma: bool = True, bias: torch.Tensor | None = None, qk_norm: torch.Tensor | None = None,
                         norm_eps: float = 0.0) -> None:
    """``attn_decode_mma`` with rotary encoding and the cache write folded in: ``qkv`` holds the step's
    un-rotated q|k|v rows of requests that bring one token each, as bfloat16 [T, C] or as the float32 slices
    [slices, T, C] of a K-split product (``linear_smallm``); C = (n_heads + 2 n_kv_heads) * head_dim."""
    _need_cuda(qkv, kcache, vcache, seq_q_start, seq_kv_len, page_indptr, page_ids, items, n_items, dec_seqs,
               dec_item_start, n_dec, out, inv_freq, status, bias, qk_norm)
    check_head_dim(head_dim)
    C = (n_heads + 2 * n_kv_heads) * head_dim
    _check_qkv_stage(bias, qk_norm, C, head_dim)
    _need(kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "attn_decode_rope_mma: bfloat16 only")
    _need(qkv.is_contiguous() and qkv.shape[-1] == C, "attn_decode_rope_mma: qkv")
    if qkv.dim() == 3:
        _need(qkv.dtype == torch.float32, "attn_decode_rope_mma: slices are float32")
        parts, n_parts, part_stride, qkv_ptr = qkv, qkv.shape[0], qkv.shape[1] * C, None
    else:
        _need(qkv.dtype == torch.bfloat16, "attn_decode_rope_mma: rows are bfloat16")
        parts, n_parts, part_stride, qkv_ptr = None, 0, 0, qkv
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "attn_decode_rope_mma: cache layout")
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim, "attn_decode_rope_mma: out")
    _need(rotary_dim % 4 == 0 and 0 <= rotary_dim <= head_dim, "attn_decode_rope_mma: rotary_dim")
    if rotary_dim:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
              "attn_decode_rope_mma: inv_freq")
    lib = _libs.get("attention_mma.cu", TKB_HD=head_dim)
    part_o = torch.empty((items_cap, n_heads, head_dim), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((items_cap, n_heads, 2), dtype=torch.float32, device=qkv.device)
    counters = _decode_counters(qkv.device, dec_cap, n_heads, n_kv_heads) if item_entry is not None else None
    if counters is not None:
        _check(_fn(lib, "tkb_attn_decode_merged_bf16")(
            _ptr(qkv_ptr), c_int(C), _ptr(parts), c_int(n_parts), ctypes.c_longlong(part_stride), _ptr(kcache),
            _ptr(vcache), _ptr(seq_q_start), _ptr(seq_kv_len), _ptr(page_indptr), _ptr(page_ids), _ptr(items),
            _ptr(n_items), c_int(items_cap), _ptr(part_o), _ptr(part_ml), c_int(n_heads), c_int(n_kv_heads),
            c_int(page_size), c_float(scale), c_int(window or 0), c_int(1), _ptr(inv_freq),
            c_int(rotary_dim), c_int(1 if write_cache else 0), c_int(kcache.shape[0]), c_int(1 if tma else 0),
            _ptr(status), _ptr(counters),
            _ptr(item_entry), _ptr(dec_item_start), _ptr(seq_q_start), _ptr(out), c_int(out.shape[1]), _ptr(bias),
            _ptr(qk_norm), c_float(norm_eps), _stream()), "attn_decode_merged")
        return
    _check(_fn(lib, "tkb_attn_decode_rope_mma_bf16")(
        _ptr(qkv_ptr), c_int(C), _ptr(parts), c_int(n_parts), ctypes.c_longlong(part_stride), _ptr(kcache),
        _ptr(vcache), _ptr(seq_q_start), _ptr(seq_kv_len),
        _ptr(page_indptr), _ptr(page_ids), _ptr(items), _ptr(n_items), c_int(items_cap), _ptr(part_o), _ptr(part_ml),
        c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale), c_int(window or 0),
        _ptr(inv_freq), c_int(rotary_dim), c_int(1 if write_cache else 0), c_int(kcache.shape[0]),
        c_int(1 if tma else 0), _ptr(status), _ptr(bias), _ptr(qk_norm), c_float(norm_eps), _stream()),
        "attn_decode_rope_mma")
    _check(_fn(lib, "tkb_attn_decode_merge_bf16")(
        _ptr(part_o), _ptr(part_ml), _ptr(dec_seqs), _ptr(dec_item_start), _ptr(n_dec), c_int(dec_cap),
        _ptr(seq_q_start), _ptr(out), c_int(out.shape[1]), c_int(n_heads), _stream()), "attn_decode_merge")


def attn_prefill_mma(qkv: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                     seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, seq_kv_len: torch.Tensor,
                     page_indptr: torch.Tensor, page_ids: torch.Tensor, tiles: torch.Tensor, n_tiles: torch.Tensor,
                     tiles_cap: int, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                     window: int | None, status: torch.Tensor | None = None) -> None:
    """bfloat16 causal attention for prompt portions: ``tiles`` are (request row, first query of a
    64-query tile within the portion) pairs; results go to ``out`` [T, n_heads*head_dim] at the token rows."""
    _need_cuda(qkv, out, kcache, vcache, seq_q_start, seq_q_len, seq_kv_len, page_indptr, page_ids, tiles, n_tiles)
    check_head_dim(head_dim)
    _need(qkv.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attn_prefill_mma: bfloat16 only")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "attn_prefill_mma: cache layout")
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim, "attn_prefill_mma: out")
    _need(tiles.numel() >= 2 * tiles_cap, "attn_prefill_mma: plan arrays")
    lib = _libs.get("attention_mma.cu", TKB_HD=head_dim)
    _check(_fn(lib, "tkb_attn_prefill_mma_bf16")(
        _ptr(qkv), c_int(qkv.shape[1]), _ptr(out), c_int(out.shape[1]), _ptr(kcache), _ptr(vcache), _ptr(seq_q_start),
        _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(page_indptr), _ptr(page_ids), _ptr(tiles), _ptr(n_tiles),
        c_int(tiles_cap), c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale), c_int(window or 0),
        c_int(kcache.shape[0]), _ptr(status), _stream()), "attn_prefill_mma")


ATTN_PREFILL_TC = True  # portions of prompts on the tcgen05 kernels where one takes the head size
# head size -> (source, compile-time constants, entry point).  Both accumulate the output in tensor memory; head
# size 64 has 128-key tiles and one S tile a head (the faster of the two there), head size 128 64-key tiles and two.
ATTN_PREFILL_TC_KERNELS = {
    64: ("attention_tc.cu", {}, "tkb_attn_prefill_tc_bf16"),
    128: ("attention_tc_acc.cu", {"TKB_HD": 128}, "tkb_attn_prefill_acc_bf16"),
}


def can_use_attn_prefill_tc(head_dim: int) -> bool:
    return ATTN_PREFILL_TC and head_dim in ATTN_PREFILL_TC_KERNELS


def attn_prefill_tc(qkv: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                    seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, seq_kv_len: torch.Tensor,
                    page_indptr: torch.Tensor, page_ids: torch.Tensor, tiles: torch.Tensor, n_tiles: torch.Tensor,
                    tiles_cap: int, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                    window: int | None, status: torch.Tensor, single_heads: bool = False) -> None:
    """bfloat16 causal attention for prompt portions on tcgen05 tensor cores (head sizes 64 and 128): ``tiles`` are
    (request row, first query of a 128-query tile within the portion) pairs; results go to ``out``
    [T, n_heads*head_dim] at the token rows.  ``status`` collects a wait that ran out.  A block takes two query
    heads of a kv head; ``single_heads``: one (twice the blocks, for steps whose tiles are too few to give every
    SM a pair)."""
    _need_cuda(qkv, out, kcache, vcache, seq_q_start, seq_q_len, seq_kv_len, page_indptr, page_ids, tiles, n_tiles,
               status)
    _need(head_dim in ATTN_PREFILL_TC_KERNELS,
          f"attn_prefill_tc: head sizes {sorted(ATTN_PREFILL_TC_KERNELS)} only, got {head_dim}")
    _need(qkv.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attn_prefill_tc: bfloat16 only")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim) and kcache.is_contiguous()
          and vcache.shape == kcache.shape and vcache.is_contiguous(), "attn_prefill_tc: cache layout")
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim, "attn_prefill_tc: out")
    _need(qkv.stride(1) == 1 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0,
          "attn_prefill_tc: rows of q must start on 16-byte boundaries")
    _need(tiles.numel() >= 2 * tiles_cap, "attn_prefill_tc: plan arrays")
    source, defines, entry = ATTN_PREFILL_TC_KERNELS[head_dim]
    _check(_fn(_libs.get(source, **defines), entry)(
        _ptr(qkv), c_int(qkv.stride(0)), _ptr(out), c_int(out.shape[1]), _ptr(kcache), _ptr(vcache),
        c_int(kcache.shape[0]), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(page_indptr), _ptr(page_ids),
        _ptr(tiles), _ptr(n_tiles), c_int(tiles_cap), c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale),
        c_int(window or 0), c_int(1 if single_heads else 0), _ptr(status), _stream()), "attn_prefill_tc")


def sample(logits: torch.Tensor, temperature: torch.Tensor | None, stream_key: torch.Tensor | None,
           sample_pos: torch.Tensor | None, row_slot: torch.Tensor | None, out_ids: torch.Tensor,
           out_logprob: torch.Tensor | None, last_token: torch.Tensor | None) -> None:
    """Greedy (temperature <= 0) or Gumbel-max temperature sampling of one id per row of logits [R, V]."""
    _need_cuda(logits, temperature, stream_key, sample_pos, row_slot, out_ids, out_logprob, last_token)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits must be contiguous float32")
    _need(out_ids.dtype == torch.int32 and out_ids.numel() >= R, "sample: out_ids int32 [R]")
    if stream_key is not None:
        _need(stream_key.dtype == torch.int64, "sample: stream_key int64 [R]")
    lib = _libs.get("sampling.cu")
    nch = lib.tkb_sample_chunks(c_int(R), c_int(V))
    if nch > 1:
        # few rows, large vocabulary: chunks of the vocabulary in parallel, then a fold in chunk order
        part = torch.empty((R, nch, 4), dtype=torch.float32, device=logits.device)
        _check(_fn(lib, "tkb_sample_two_stage")(
            _ptr(logits), _ptr(temperature), _ptr(stream_key), _ptr(sample_pos), _ptr(row_slot), _ptr(out_ids),
            _ptr(out_logprob), _ptr(last_token), _ptr(part), c_int(nch), c_int(R), c_int(V), _stream()), "sample")
        return
    f = _fn(lib, "tkb_sample")
    _check(f(_ptr(logits), _ptr(temperature), _ptr(stream_key), _ptr(sample_pos), _ptr(row_slot), _ptr(out_ids),
             _ptr(out_logprob), _ptr(last_token), c_int(R), c_int(V), _stream()), "sample")


def noise_of_bits(bits: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The uniform number in (0, 1) and the Gumbel value the sampling kernels make of 32 random bits each
    (``bits``: int32 holding the bit patterns).  For tests of the extremes."""
    _need_cuda(bits)
    _need(bits.dtype == torch.int32 and bits.is_contiguous(), "noise_of_bits: bits must be contiguous int32")
    u = torch.empty(bits.numel(), dtype=torch.float32, device=bits.device)
    g = torch.empty_like(u)
    _check(_fn(_libs.get("sampling.cu"), "tkb_noise_of_bits")(_ptr(bits), _ptr(u), _ptr(g), c_int(bits.numel()), _stream()),
           "noise_of_bits")
    return u, g


def topk_logprobs(logits: torch.Tensor, temperature: torch.Tensor | None, k: int, out_idx: torch.Tensor,
                  out_lp: torch.Tensor) -> None:
    _need_cuda(logits, temperature, out_idx, out_lp)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "topk_logprobs: logits")
    _need(out_idx.shape == (R, k) and out_lp.shape == (R, k) and out_idx.dtype == torch.int32, "topk_logprobs: outs")
    f = _fn(_libs.get("sampling.cu"), "tkb_topk_logprobs")
    _check(f(_ptr(logits), _ptr(temperature), _ptr(out_idx), _ptr(out_lp), c_int(R), c_int(V), c_int(k), _stream()),
           "topk_logprobs")


TCGEN05_M_MIN = 128  # from this many rows on the gated tcgen05 product beats library product + activation kernel


def can_use_tcgen05(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and a.shape[1] % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor, gated: bool = False) -> torch.Tensor:
    """a[M, K] @ w[N, K]^T in bfloat16 on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory).
    ``gated``: ``w`` interleaves gate/up rows (``interleave_gate_up``); the result is silu(gate)*up [M, N/2].
    ``status``: the device status word; a bounded wait that runs out sets its bit 4."""
    _need_cuda(a, w, status)
    _need(can_use_tcgen05(a, w), "gemm_tcgen05: bfloat16 operands, K and strides multiples of 8, 16-byte aligned")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and (not gated or N % 16 == 0), "gemm_tcgen05: shapes")
    out = torch.empty((M, N // 2 if gated else N), dtype=torch.bfloat16, device=a.device)
    _check(_fn(_libs.get("gemm_tcgen05.cu"), "tkb_gemm_tcgen05_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(M), c_int(N),
        c_int(K), c_int(1 if gated else 0), _ptr(status), _stream()), "gemm_tcgen05")
    return out


TC_DECODE_M_MAX = 64


def linear_tc_decode(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor, max_slices: int = 16,
                     gated: bool = False) -> torch.Tensor:
    """a[M, K] @ w[N, K]^T for M <= 64 on the tcgen05 tensor cores with the weights on the 128-row side
    (TMA-fed ten-stage ring).  Returns float32 slices [slices, M, N] of a K-split product, or with ``gated``
    (``w`` from ``interleave_gate_up``) silu(gate)*up as bfloat16 [M, N/2]."""
    _need_cuda(a, w, status)
    _need(can_use_tcgen05(a, w) and 0 < a.shape[0] <= TC_DECODE_M_MAX, "linear_tc_decode: bfloat16, M <= 64, K % 8 == 0")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and (not gated or N % 16 == 0), "linear_tc_decode: shapes")
    lib = _libs.get("gemm_tcgen05_decode.cu")
    slices = 1 if gated else lib.tkb_linear_tcgen05_decode_slices(c_int(N), c_int(K), c_int(max_slices))
    if gated:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    else:
        out = torch.empty((slices, M, N), dtype=torch.float32, device=a.device)
    _check(_fn(lib, "tkb_linear_tcgen05_decode_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(M), c_int(N), c_int(K),
        c_int(slices), c_int(1 if gated else 0), _ptr(status), _stream()), "linear_tc_decode")
    return out


FEW_ROWS_MAX = 16  # measured on B200: from 17 rows on, library products + separate kernels are faster than the K-split path
# ... except for the attention block's two products, whose weights are small (the library's kernels take 10 us each
# for 2 us worth of bytes at 64 rows) and whose slices the attention kernel and the norm add on their way anyway:
# measured at Llama-3.2-1B sizes, batch 32: 24.2 k -> 25.5 k tok/s, batch 64: 38.1 k -> 38.6 k
ATTN_FEW_ROWS_MAX = 64


def can_use_few_rows(a: torch.Tensor, w: torch.Tensor, max_rows: int | None = None) -> bool:
    """Steps with few rows (decode) use K-split products whose float32 slices the consumer adds."""
    if a.shape[0] <= SMALL_M_MAX:
        return can_use_smallm(a, w)
    return a.shape[0] <= (max_rows or FEW_ROWS_MAX) and can_use_tcgen05(a, w)


def linear_few_rows(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor | None) -> torch.Tensor:
    """Float32 slices [slices, M, N] of a[M, K] @ w[N, K]^T: the mma.sync kernel up to 16 rows (measured
    faster there), the tcgen05 kernel above (if ``FEW_ROWS_MAX`` is raised)."""
    if a.shape[0] <= SMALL_M_MAX:
        return linear_smallm(a, w)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=a.device)
    return linear_tc_decode(a, w, status)


def linear_few_rows_gated(a: torch.Tensor, w_interleaved: torch.Tensor, status: torch.Tensor | None) -> torch.Tensor:
    """silu(gate) * up [M, I] for at most 64 rows: mma.sync kernel up to 8 rows, tcgen05 kernel above."""
    if a.shape[0] <= GATED_M_MAX:
        return linear_smallm_gated(a, w_interleaved)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=a.device)
    return linear_tc_decode(a, w_interleaved, status, gated=True)


def linear(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """a[M, K] @ w[N, K]^T.  float32: this engine's FP32 kernel (no tf32).  bfloat16: the library
    matrix product (cuBLAS through torch), float32 accumulation, output bfloat16 or float32."""
    _need_cuda(a, w)
    M = a.shape[0]
    N = w.shape[0]
    if a.dtype == torch.float32:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
        sgemm_tn(a, w, out)
        return out
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear: operands must share the engine dtype")
    if out_dtype is None or out_dtype == torch.bfloat16:
        return torch.mm(a, w.t())
    return torch.mm(a, w.t(), out_dtype=out_dtype)


def softmax_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
