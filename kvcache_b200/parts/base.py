"""Interfaces of the parts a model is put together from, and the context a step hands them.

A part knows its own sizes and constants and nothing about the model around it.
It declares the checkpoint tensors it wants (`tensor_specs`), takes them
(`bind`), and runs on the rows of one step (`forward`).  The kinds of part:

* `Norm`            - `add_norm(h, delta, out, ctx)`: folds `delta` into the float32 residual
                      stream `h` and writes the normalised rows in the compute type.
* `PositionEncoding`- `on_embed(h, ctx)` for encodings added to the embedding and
                      `rotation()` for encodings that rotate queries and keys.
* `Mixer`           - `forward(x, ctx) -> delta`; declares the cache it needs with
                      `cache_spec()` (pages of keys and values) and `state_spec()`
                      (per-request state of fixed size, one tensor or several by name),
                      and the work lists its kernels want with `step_planners()`.
* `FeedForward`     - `forward(x, ctx) -> delta`.
* `Block`           - the arrangement of the four in one layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple

import torch

from ..weights.loader import TensorSpec

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass(frozen=True)
class PagedKVSpec:
    """Pages of keys and values: `[pages, num_kv_heads, page_size, head_dim]` for K and for V.

    `window`: how many keys, its own included, a query sees (None: all of them).
    Layers whose specs are equal share a group: one block table, one page id
    for all of them, as the reference uses one table for its 24 layers
    (apps/qwen_serve.cu:99-100).
    """
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: one `shape`-sized tensor per live request, zeroed at admission.
    A mixer with several states (a convolution's tail beside a recurrent state) returns a dict of them by name."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass
class PagedKVView:
    """The cache one layer call reads and writes."""
    spec: PagedKVSpec
    k_pages: torch.Tensor            # [pages, num_kv_heads, page_size, head_dim]
    v_pages: torch.Tensor
    block_table: torch.Tensor        # int32 [segments capacity, pages per request]; -1 where no page is held
    page_size: int
    writes: bool = True              # False: the call reads what another call wrote


class StepPlanner:
    """Work lists a kernel wants for every step, made on the host from the lengths of the step's segments.

    Kernels that cut a step's rows into tiles, units or chunks of their own size need lists that say which block
    does what.  The step function knows nothing of those sizes: the kernel set hands the mixers that use it a
    planner, the runner calls `plan` once a step, packs the arrays into the step's metadata with everything else
    (one copy to the device) and hands the device views back in `StepBatch.plans[name]`.

    `sections(T, S)`: the most int32 words each named list can take in a step of T tokens in S segments (the
    layout of the metadata buffer depends on T, S and nothing else, so that a recorded CUDA graph finds every list
    where it was).  `plan(starts, counts)`: for segments that have `starts[i]` tokens cached and bring `counts[i]`,
    the lists (flat int32 arrays) and the counts that fix the launches' shapes - those counts are part of the key
    under which the step's launches may be replayed.
    """
    name: str = ""

    def sections(self, num_tokens: int, num_segments: int) -> Dict[str, int]:
        raise NotImplementedError

    def plan(self, starts, counts) -> Tuple[Dict[str, Any], Dict[str, int]]:
        raise NotImplementedError


@dataclass
class StepPlan:
    """A planner's lists for one step, on the device, and the counts that go with them."""
    arrays: Dict[str, torch.Tensor]
    counts: Dict[str, int]


@dataclass
class StepBatch:
    """The rows of one step, on the device.  Row r is one token; a segment is the run of
    rows that one request brings (a portion of a prompt, or one decoded token)."""
    num_tokens: int
    num_segments: int
    num_wanted: int
    token_ids: torch.Tensor          # int32 [T]
    positions: torch.Tensor          # int32 [T]   absolute position of the row in its request
    row_segment: torch.Tensor        # int32 [T]   which segment the row belongs to
    seg_q_start: torch.Tensor        # int32 [S]   first row of the segment
    seg_q_len: torch.Tensor          # int32 [S]
    seg_kv_len: torch.Tensor         # int32 [S]   tokens of the request cached after this step
    seg_slot: torch.Tensor           # int32 [S]   the request's state slot
    wanted_rows: torch.Tensor        # int32 [R]   rows whose logits are returned
    token_src: Optional[torch.Tensor] = None     # int32 [T]: >= 0: the row's token is last_tokens[token_src[r]]
    last_tokens: Optional[torch.Tensor] = None   # int32: tokens the previous step sampled, still on the device
    # Work lists that kernels asked for (see StepPlanner), by the planner's name.
    plans: Dict[str, "StepPlan"] = field(default_factory=dict)
    max_q_len: int = 1               # host copies, for launch shapes
    max_kv_len: int = 1
    host: Dict[str, Any] = field(default_factory=dict)


@dataclass
class LayerContext:
    """What a part may touch during one layer call."""
    batch: StepBatch
    kernels: Any                     # the kernel set (see kvcache_b200.kernels.api)
    workspace: Any                   # named scratch buffers that outlive the step
    kv: Optional[PagedKVView] = None
    state: Any = None                # [slots, *StateSpec.shape], or a dict of such tensors by the states' names
    call_index: int = 0


class Part:
    """Base of all parts: checkpoint tensors in, device buffers held."""

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def init_kinds(self) -> Dict[str, str]:
        """Random-weights mode: `{name: "normal" | "ones_plus_normal" | "skip"}` for non-default tensors."""
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        """Takes this part's tensors (CPU, as stored) and places what it needs on the device."""

    def weight_bytes(self) -> int:
        """Bytes of device weights one step has to read (for rooflines)."""
        return 0



class Norm(Part):
    def add_norm(self, h: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
                 ctx: LayerContext, rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError

    def fold_params(self) -> Optional[Tuple[torch.Tensor, float]]:
        """(weight, eps) if this norm is y = v * rsqrt(mean(v^2) + eps) * weight, so that a matrix product that follows
        it can apply it on the way in (see `Mixer.forward_folded`); None for norms that cannot be folded."""
        return None


@dataclass(frozen=True)
class Rotation:
    """Rotate-half rotation of the first `2 * cos.shape[1]` dimensions of each head:
    dimension t pairs with t + rotary_dim/2, angle table[pos, t]."""
    cos: torch.Tensor                # float32 [positions, rotary_dim / 2], on the device
    sin: torch.Tensor


class PositionEncoding(Part):
    def on_embed(self, h: torch.Tensor, ctx: LayerContext) -> None:
        """Encodings that are added to the embedded rows act here; default: nothing."""

    def rotation(self) -> Optional[Rotation]:
        """Encodings that rotate queries and keys return their table; default: none."""
        return None


class Mixer(Part):
    def cache_spec(self) -> Optional[PagedKVSpec]:
        return None

    def state_spec(self):
        """None, one `StateSpec`, or `{name: StateSpec}` for a mixer that keeps several states per request."""
        return None

    def step_planners(self, kernels: Any) -> Sequence[StepPlanner]:
        """The planners whose work lists this mixer's kernels read (asked of the kernel set, which owns the tiling)."""
        return ()

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        raise NotImplementedError

    # The folded form, which a part may offer for steps of few rows: it takes the residual stream itself (`h`, float32,
    # and `h16`, the same rounded to the compute type), applies `norm` inside its first matrix product and adds its
    # result into `h` and `h16` inside its last - two kernels and two round trips through memory fewer per part.
    def supports_fold(self, norm: "Norm", kernels: Any, num_rows: int) -> bool:
        return False

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, norm: "Norm", ctx: LayerContext) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        raise NotImplementedError

    def supports_fold(self, norm: "Norm", kernels: Any, num_rows: int) -> bool:
        """See `Mixer.supports_fold`."""
        return False

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, norm: "Norm", ctx: LayerContext) -> None:
        raise NotImplementedError


class Block(Part):
    """One layer.  `forward` receives the residual stream `h` (float32, updated in place)
    and the delta the previous layer has not yet added to it, and returns its own."""

    mixer: Mixer

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx: LayerContext) -> Optional[torch.Tensor]:
        raise NotImplementedError

    def supports_fold(self, kernels: Any, num_rows: int) -> bool:
        """Whether every part of the layer offers its folded form for a step of `num_rows` rows."""
        return False

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, ctx: LayerContext) -> None:
        """The layer on `h` and `h16` in place; nothing is left pending."""
        raise NotImplementedError
