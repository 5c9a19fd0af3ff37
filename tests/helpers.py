"""Shared helpers of the tests: building an engine over a kernel set, random prompts."""
from __future__ import annotations

import random
from typing import List

import torch


def make_runner(folder: str, kernels, *, dtype: str, device: str, page_size: int, num_pages: int,
                max_slots: int = 4, max_tokens_per_step: int = 512, max_tokens_per_request: int = 512):
    from kvcache_b200.cache import CacheManager
    from kvcache_b200.engine.loading import load_model
    from kvcache_b200.engine.runner import ModelRunner
    model = load_model(folder, dtype=dtype, device=device, max_positions=max_tokens_per_request)
    cache = CacheManager(model.cache_entries(), page_size=page_size, num_pages=num_pages, max_slots=max_slots,
                         max_tokens_per_request=max_tokens_per_request, dtype=dtype, device=device)
    return ModelRunner(model, cache, kernels, max_tokens_per_step=max_tokens_per_step)


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def paged_scenario(segments, *, num_kv_heads: int, head_dim: int, page_size: int, dtype, device,
                   window=None, seed: int = 0, extra_pages: int = 3, fill_history: bool = True,
                   tc_min_key_tiles: int = 16):
    """A step's metadata and a paged cache with shuffled pages, made by hand for kernel tests.

    `segments`: list of (tokens already cached, new tokens).  Returns (StepBatch, PagedKVView);
    pages hold random keys and values for the cached part when `fill_history`.
    """
    import numpy as np
    from kvcache_b200.parts.base import PagedKVSpec, PagedKVView, StepBatch
    g = torch.Generator().manual_seed(seed)
    S = len(segments)
    T = sum(n for _, n in segments)
    max_len = max(s + n for s, n in segments)
    width = (max_len + page_size - 1) // page_size + 1
    total_pages = sum((s + n + page_size - 1) // page_size for s, n in segments) + extra_pages
    order = torch.randperm(total_pages, generator=g).tolist()      # shuffled physical pages
    table = np.full((S, width), -1, dtype=np.int32)
    at = 0
    for i, (s, n) in enumerate(segments):
        for j in range((s + n + page_size - 1) // page_size):
            table[i, j] = order[at]
            at += 1
    shape = (total_pages, num_kv_heads, page_size, head_dim)
    k_pages = torch.randn(shape, generator=g) if fill_history else torch.zeros(shape)
    v_pages = torch.randn(shape, generator=g) if fill_history else torch.zeros(shape)
    pos = np.concatenate([np.arange(s, s + n) for s, n in segments]).astype(np.int32)
    row_seg = np.concatenate([np.full(n, i) for i, (s, n) in enumerate(segments)]).astype(np.int32)
    q_start = np.cumsum([0] + [n for _, n in segments[:-1]]).astype(np.int32)
    dev = lambda a: torch.tensor(np.array(a), dtype=torch.int32).to(device)
    from kvcache_b200.kernels.attention_plan import PagedAttentionPlanner, plan_prefill_units
    from kvcache_b200.parts.base import StepPlan
    arrays, counts = PagedAttentionPlanner().plan(np.asarray([s for s, _ in segments]), np.asarray([n for _, n in segments]))
    if tc_min_key_tiles != 16 and "tc_units" in arrays:
        tc, counts["tc_tiles"] = plan_prefill_units([(i, s, n) for i, (s, n) in enumerate(segments) if n > 1], 128, tc_min_key_tiles)
        arrays["tc_units"], counts["tc_units"] = tc.reshape(-1), len(tc)
    batch = StepBatch(
        plans={PagedAttentionPlanner.name: StepPlan({k: dev(v) for k, v in arrays.items()}, counts)},
        num_tokens=T, num_segments=S, num_wanted=0, token_ids=dev(np.zeros(T)), positions=dev(pos),
        row_segment=dev(row_seg), seg_q_start=dev(q_start), seg_q_len=dev([n for _, n in segments]),
        seg_kv_len=dev([s + n for s, n in segments]), seg_slot=dev(np.arange(S)), wanted_rows=dev([]),
        max_q_len=max(n for _, n in segments), max_kv_len=max_len)
    kv = PagedKVView(spec=PagedKVSpec(num_kv_heads, head_dim, window), k_pages=k_pages.to(dtype).to(device),
                     v_pages=v_pages.to(dtype).to(device), block_table=dev(table), page_size=page_size, writes=True)
    return batch, kv


def clone_kv(kv, device=None):
    from kvcache_b200.parts.base import PagedKVView
    to = (lambda t: t.clone().to(device)) if device else (lambda t: t.clone())
    return PagedKVView(spec=kv.spec, k_pages=to(kv.k_pages), v_pages=to(kv.v_pages), block_table=to(kv.block_table),
                       page_size=kv.page_size, writes=kv.writes)


def batch_to(batch, device):
    import dataclasses
    from kvcache_b200.parts.base import StepPlan
    changes = {f.name: getattr(batch, f.name).to(device) for f in dataclasses.fields(batch)
               if isinstance(getattr(batch, f.name), torch.Tensor)}
    # The planners' work lists are read by the kernels too: they move with the rest.
    changes["plans"] = {name: StepPlan({k: v.to(device) for k, v in plan.arrays.items()}, dict(plan.counts))
                        for name, plan in batch.plans.items()}
    return dataclasses.replace(batch, **changes)


def assert_close(got: torch.Tensor, want: torch.Tensor, rel: float, what: str = ""):
    """max |got - want| <= rel * max(|want|) (the tolerance scales with the reference's size)."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    scale = max(want.abs().max().item(), 1e-30)
    err = (got - want).abs().max().item()
    assert err <= rel * scale, f"{what}: max abs error {err:.3e} > {rel:g} * {scale:.3e}"


def reference_attention_case():
    """The case of the reference's own numpy attention (ref/ref_attn.py): q [8, 64], K and V [8, 128, 64] drawn from
    numpy's default_rng(0) as that script draws them, and its output as committed under tests/golden (made by
    tests/golden/make_ref_attn_golden.py).  The inputs are checked against the digests recorded with the output."""
    import hashlib
    import json
    import os
    import numpy as np
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    with open(os.path.join(golden, "ref_attn.json"), "r", encoding="utf-8") as fh:
        meta = json.load(fh)
    H, S, D = meta["heads"], meta["keys"], meta["head_dim"]
    rng = np.random.default_rng(meta["seed"])
    q = rng.standard_normal((H, D)).astype(np.float32)
    K = rng.standard_normal((H, S, D)).astype(np.float32)
    V = rng.standard_normal((H, S, D)).astype(np.float32)
    for name, arr in (("q", q), ("K", K), ("V", V)):
        assert hashlib.sha256(arr.tobytes()).hexdigest() == meta["inputs_sha256"][name], f"{name} is not what the reference drew"
    out = np.fromfile(os.path.join(golden, "ref_attn_out.f32"), dtype="<f4").reshape(H, D)
    return torch.from_numpy(q), torch.from_numpy(K), torch.from_numpy(V), torch.from_numpy(out.copy())
