"""Engine options, named as the reference names them where it has them.

The reference's ``ServerConfig`` (tokasaurus/common_types.py:52-126) is filled by the
``toka key=value`` command line through pydra (tokasaurus/entry.py:139-143).  The options
that matter on one GPU without a server keep their names and meanings here; the command
line grammar (``key=value``, ``key=T``/``key=F``, ``key='(2*1024)'``) is parsed by
``parse_overrides`` below.  Options of this engine that the reference has no name for
(the reference takes prompts over HTTP) are listed last.
"""

from __future__ import annotations

import ast
import json
from dataclasses import dataclass, fields
from typing import Any


class OptionError(ValueError):
    pass


@dataclass
class EngineConfig:
    # --- names and defaults of tokasaurus/common_types.py:52-126 ---
    model: str | None = None
    dtype: str = "bfloat16"
    rope_scaling: str | None = None  # JSON text that replaces config.json's rope_scaling
    enable_chosen_logprobs: bool = True
    max_topk_logprobs: int | None = None
    log_level: str = "INFO"  # of the logger "tokasaurus_b200"
    stats_report_seconds: float = 5.0  # a line of counts and rates at level INFO this often
    page_size: int = 16
    kv_cache_num_tokens: int = 1024 * 128
    max_tokens_per_forward: int = 8192
    max_seqs_per_forward: int = 1024
    prefill_round_up_multiple: int = 16  # of the paced prompt tokens a step (greedy_prefill=F)
    scheduling_steps_ahead: int = 2  # decode steps launched before the current one's results are read (0: none; reference: 8)
    max_num_tokens_per_request: int | None = None
    greedy_prefill: bool = True
    use_cudagraphs: bool = True
    cudagraph_max_size: int = 128
    cudagraph_step: int = 16
    cudagraph_max_kv_indices_per_seq: int = 32768  # a request with more pages keeps its step out of the graphs
    allocator_sanity_checks: bool = False
    bump_city_population_me: bool = False
    # --- this engine's own options ---
    random_weights: int | None = None  # seed: build weights from the configuration instead of reading them
    device: str = "cuda:0"

    def kv_cache_num_blocks(self) -> int:
        # tokasaurus/common_types.py:130-132
        if self.kv_cache_num_tokens % self.page_size:
            raise OptionError(
                f"kv_cache_num_tokens={self.kv_cache_num_tokens} is not a multiple of page_size={self.page_size}"
            )
        return self.kv_cache_num_tokens // self.page_size

    def finalize(self, max_position_embeddings: int | None = None) -> "EngineConfig":
        if self.dtype not in ("bfloat16", "float32"):
            raise OptionError(f"dtype={self.dtype!r}: this engine runs 'bfloat16' or 'float32'")
        for name in ("page_size", "kv_cache_num_tokens", "max_tokens_per_forward", "max_seqs_per_forward",
                     "prefill_round_up_multiple", "cudagraph_step", "cudagraph_max_size"):
            if getattr(self, name) <= 0:
                raise OptionError(f"{name} must be positive")
        self.kv_cache_num_blocks()
        if self.max_num_tokens_per_request is None and max_position_embeddings is not None:
            # tokasaurus/common_types.py:162-166
            self.max_num_tokens_per_request = min(max_position_embeddings, self.kv_cache_num_tokens)
        return self


def _parse_value(text: str, typ: Any) -> Any:
    t = text.strip()
    if t in ("None", "none", "null"):
        return None
    base = typ
    if isinstance(typ, str):
        base = typ.replace(" ", "").replace("|None", "").replace("None|", "")
        base = {"int": int, "float": float, "bool": bool, "str": str}.get(base, str)
    if base is bool:
        if t in ("T", "True", "true", "1"):
            return True
        if t in ("F", "False", "false", "0"):
            return False
        raise OptionError(f"cannot read {text!r} as a boolean (use T or F)")
    if base in (int, float):
        if t.startswith("(") and t.endswith(")"):
            v = _eval_arith(t)
        else:
            try:
                v = ast.literal_eval(t)
            except (ValueError, SyntaxError) as e:
                raise OptionError(f"cannot read {text!r} as a number") from e
        if base is int:
            if isinstance(v, float) and not v.is_integer():
                raise OptionError(f"{text!r} is not an integer")
            return int(v)
        return float(v)
    return t


def _eval_arith(expr: str) -> float | int:
    """Evaluate a parenthesised arithmetic expression such as ``(1024*128)``."""
    tree = ast.parse(expr, mode="eval")
    allowed = (ast.Expression, ast.BinOp, ast.UnaryOp, ast.Constant, ast.Add, ast.Sub, ast.Mult, ast.Div,
               ast.FloorDiv, ast.Pow, ast.Mod, ast.USub, ast.UAdd)
    for node in ast.walk(tree):
        if not isinstance(node, allowed):
            raise OptionError(f"only arithmetic is allowed in {expr!r}")
        if isinstance(node, ast.Constant) and not isinstance(node.value, (int, float)):
            raise OptionError(f"only numbers are allowed in {expr!r}")
    return eval(compile(tree, "<option>", "eval"), {"__builtins__": {}}, {})


def parse_overrides(argv: list[str], config_cls: type = EngineConfig, extra: dict[str, Any] | None = None):
    """Read ``key=value`` words into an instance of ``config_cls``.

    ``extra`` maps further option names to their types (for example the command line's
    prompt options); their values are returned as a second dictionary.
    """
    cfg = config_cls()
    types = {f.name: f.type for f in fields(config_cls)}
    extra = extra or {}
    extra_values: dict[str, Any] = {}
    for word in argv:
        if "=" not in word:
            raise OptionError(f"expected key=value, got {word!r}")
        key, _, text = word.partition("=")
        key = key.strip()
        if key in types:
            setattr(cfg, key, _parse_value(text, types[key]))
        elif key in extra:
            extra_values[key] = _parse_value(text, extra[key])
        else:
            raise OptionError(f"unknown option {key!r}; known: {sorted(list(types) + list(extra))}")
    return cfg, extra_values


def parse_rope_scaling_override(text: str | None) -> dict[str, Any] | None:
    """The ``rope_scaling`` option holds JSON (tokasaurus/model/utils.py:353-354)."""
    if text is None:
        return None
    try:
        d = json.loads(text)
    except json.JSONDecodeError as e:
        raise OptionError(f"rope_scaling option is not JSON: {e}") from e
    if not isinstance(d, dict):
        raise OptionError("rope_scaling option must be a JSON object")
    return d
