"""The step function, batch builder and cache manager together on the CPU, with the plain
statements of the kernels (tests/kernel_refs.py) in the kernels' place.  This checks the
bookkeeping (positions, block tables, wanted rows, page reuse), not the kernels: those are
compared on the GPU."""

import numpy as np
import pytest
import torch

import cuttings
import kernel_refs
from plain_llama import TINY_WEIGHTS, tiny_configs


@pytest.fixture()
def cpu_kernels(monkeypatch):
    kernel_refs.install_cpu_kernels(monkeypatch)


def _replay(model_dir, steps, page_size):
    from tokasaurus_b200.engine.trace import TraceReplayer

    rp = TraceReplayer(str(model_dir), "float32", cuttings.max_live_tokens(steps), page_size=page_size, device="cpu")
    outs = []
    for st in steps:
        outs.append(rp.run_step(st))
        rp.runner.cache.check()
    assert not rp.runner.cache.requests
    return cuttings.collect(steps, outs)


@pytest.mark.parametrize("cfg_index", [0, 1])
@pytest.mark.parametrize("cut", ["whole", "changing_portions", "mixed"])
def test_replay_on_cpu_matches_plain(cpu_kernels, tiny_model_dirs, cfg_index, cut):
    cfg = tiny_configs()[cfg_index]
    lengths = [40, 9, 33, 1, 24] if cfg_index == 0 else [37, 2, 17, 41, 8]
    reqs = {f"r{i}": cuttings.random_tokens(n, cfg["vocab_size"], 7 * cfg_index + i) for i, n in enumerate(lengths)}
    steps = getattr(cuttings, cut)(reqs)
    got = _replay(tiny_model_dirs[cfg_index], steps, TINY_WEIGHTS[cfg_index]["page_size"])
    want = cuttings.plain_logits(tiny_model_dirs[cfg_index], reqs, torch.float64)
    for rid in reqs:
        err = np.abs(got[rid] - want[rid]).max(axis=1)
        assert err.max() < 1e-4 * max(1.0, np.abs(want[rid]).max()), (rid, int(err.argmax()), float(err.max()))


def test_graph_eligibility_of_a_step():
    """Which steps may run as CUDA graphs (host-side rule, no GPU needed): single tokens that want their logits,
    no more requests than the largest recorded batch, and no request beyond ``cudagraph_max_kv_indices_per_seq``
    pages."""
    from types import SimpleNamespace

    from tokasaurus_b200.engine.batch import StepEntry
    from tokasaurus_b200.engine.graphs import DecodeGraphs

    runner = SimpleNamespace(model=SimpleNamespace(graph_safe=True), cache=SimpleNamespace(pages_for=lambda n: -(-n // 16)))
    g = DecodeGraphs(runner, None, max_size=8, step=4, max_tokens=64, max_pages_per_request=10)
    assert g.sizes == [1, 2, 4, 8]
    one = lambda rid, start: StepEntry(rid, None, start, [0])  # noqa: E731
    assert g.usable([one("a", 5), one("b", 159)])            # 160 tokens: 10 pages
    assert not g.usable([one("a", 5), one("b", 160)])        # 161 tokens: 11 pages
    assert not g.usable([one(i, 3) for i in range(9)])       # more requests than the largest graph
    assert not g.usable([StepEntry("a", [1, 2], 0, [1])])    # a prompt portion
    assert not g.usable([StepEntry("a", [1], 0, [])])        # nothing wanted
    assert g.usable_general([StepEntry("a", [1, 2, 3], 0, [2]), one("b", 7)])
    assert not g.usable_general([StepEntry("a", list(range(65)), 0, [64])])   # more tokens than graph_max_tokens
    assert not g.usable_general([StepEntry("a", [1, 2, 3], 158, [2])])        # 161 tokens: 11 pages
    unlimited = DecodeGraphs(runner, None, max_size=8, step=4, max_tokens=0)
    assert unlimited.usable([one("b", 10 ** 6)]) and not unlimited.usable_general([StepEntry("a", [1, 2], 0, [1])])


def test_uniform_of_random_bits_stays_inside_the_open_interval():
    """The plain statement of the sampler's uniform number, in float32 as the kernel computes it: all bits set
    gives a number below 1 and a finite Gumbel value, no bit set a number above 0."""
    import numpy as np

    import kernel_refs as ref

    bits = np.array([0xFFFFFFFF, 0, 0xFFFFFE00, 0x1FF], dtype=np.uint32)
    u = ref.uniform_open(bits)
    assert u.dtype == np.float32 and (u > 0).all() and (u < 1).all()
    assert u[0] == np.float32(8388607.5 / 8388608.0) and u[1] == np.float32(0.5 / 8388608.0)
    g = -np.log(-np.log(u.astype(np.float64)))
    assert np.isfinite(g).all()
    # the form with 24 random bits, which the kernel must not use: it rounds up to exactly 1
    assert (np.float32(0xFFFFFF) + np.float32(0.5)) * np.float32(1.0 / 16777216.0) == np.float32(1.0)
