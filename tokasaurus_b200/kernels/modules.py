"""The list of kernel modules (source file, compile-time constants) that exist, and which of them a model of given
head sizes and precision needs: what is compiled at a first call is what that model runs."""

from __future__ import annotations

# every precision: embedding, norms, rotary + cache write, activation, row gather; sampling
SHARED = [("elementwise.cu", None), ("sampling.cu", None)]
# float32: the FP32-FMA product; attention on the FP32 pipes (per head size, below)
FLOAT32 = [("sgemm.cu", None)]
# bfloat16: small-batch products (mma.sync and tcgen05), the tcgen05 product for many rows
BFLOAT16 = [("linear_smallm.cu", None), ("gemm_tcgen05.cu", None), ("gemm_tcgen05_decode.cu", None)]
# tested alternatives that no model needs: built by the build check, loaded by whoever calls them
EXTRA = [("linear_decode.cu", None)]


def head_dim_modules(head_dim: int, dtype: str | None = None) -> list[tuple[str, dict | None]]:
    mods = [("attention_simt.cu", {"TKB_HD": head_dim})]  # float32; in bfloat16 steps whose planner declines
    if dtype in (None, "bfloat16"):
        mods.append(("attention_mma.cu", {"TKB_HD": head_dim}))
        if head_dim == 64:
            mods.append(("attention_tc.cu", None))  # tcgen05 kernel for prompt portions
        if head_dim == 128:
            mods.append(("attention_tc_acc.cu", {"TKB_HD": 128}))  # the same with the output in tensor memory
    return mods


def optional_modules(head_dim: int) -> list[tuple[str, dict | None]]:
    """Built by the build check, loaded only by callers that ask for them."""
    return EXTRA + [("attention_decode_static.cu", {"TKB_HD": head_dim})]


def all_modules(head_dims, dtype: str | None = None) -> list[tuple[str, dict | None]]:
    """``dtype`` "float32" or "bfloat16": what an engine of that precision needs; None: everything."""
    mods = list(SHARED)
    if dtype in (None, "float32"):
        mods += FLOAT32
    if dtype in (None, "bfloat16"):
        mods += BFLOAT16
    for hd in head_dims:
        mods += head_dim_modules(hd, dtype)
    return mods
