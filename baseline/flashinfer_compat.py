"""Argument adapter between the reference's FlashInfer calls (written for flashinfer 0.2.0) and the FlashInfer
that this image has (0.6.x).  Two entry points changed their arguments; nothing else is touched, and no file of
the reference is edited:

* ``BatchPrefillWithPagedKVCacheWrapper.plan(head_dim=...)`` is now ``plan(head_dim_qk=...)``
  (the reference calls it in tokasaurus/model/llama.py:716-729);
* ``sampling_from_probs(probs, uniform_samples)`` no longer takes the uniform numbers, it draws its own
  (the reference calls it in tokasaurus/model/llama.py:362-368).

``install()`` must run before ``tokasaurus.model.llama`` is imported, because that module binds
``sampling_from_probs`` by name at import time.
"""

from __future__ import annotations

import functools


def install() -> None:
    import flashinfer

    prefill = flashinfer.BatchPrefillWithPagedKVCacheWrapper
    if not getattr(prefill.plan, "_takes_head_dim", False):
        plan = prefill.plan

        @functools.wraps(plan)
        def plan_with_head_dim(self, *args, head_dim=None, **kwargs):
            if head_dim is not None:
                kwargs["head_dim_qk"] = head_dim
            return plan(self, *args, **kwargs)

        plan_with_head_dim._takes_head_dim = True
        prefill.plan = plan_with_head_dim

    if not getattr(flashinfer.sampling_from_probs, "_drops_uniform", False):
        sample = flashinfer.sampling_from_probs

        def sampling_from_probs(probs, uniform_samples=None, **kwargs):
            return sample(probs, **kwargs)

        sampling_from_probs._drops_uniform = True
        flashinfer.sampling_from_probs = sampling_from_probs
