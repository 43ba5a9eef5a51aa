"""The list of kernel modules (source file, compile-time constants) that exist."""

from __future__ import annotations


def common_modules() -> list[tuple[str, dict | None]]:
    return [("elementwise.cu", None), ("sgemm.cu", None), ("sampling.cu", None), ("linear_smallm.cu", None), ("linear_decode.cu", None), ("gemm_tcgen05.cu", None), ("gemm_tcgen05_decode.cu", None)]


def head_dim_modules(head_dim: int) -> list[tuple[str, dict | None]]:
    mods = [("attention_simt.cu", {"TKB_HD": head_dim}), ("attention_mma.cu", {"TKB_HD": head_dim})]
    if head_dim == 64:
        mods.append(("attention_tc.cu", None))  # tcgen05 kernel for prompt portions
    if head_dim == 128:
        mods.append(("attention_tc_acc.cu", {"TKB_HD": 128}))  # the same with the output in tensor memory
    return mods


def optional_modules(head_dim: int) -> list[tuple[str, dict | None]]:
    """Built by the build check, loaded only by callers that ask for them."""
    return [("attention_decode_static.cu", {"TKB_HD": head_dim})]


def all_modules(head_dims) -> list[tuple[str, dict | None]]:
    mods = common_modules()
    for hd in head_dims:
        mods += head_dim_modules(hd)
    return mods
