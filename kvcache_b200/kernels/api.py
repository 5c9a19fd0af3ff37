"""The kernel set: the contract every operator of a step goes through, and its CUDA form.

`KernelSet` states what each operator computes; `CudaKernels` launches the
hand-written sm_100a kernels of `kvcache_b200/csrc` through ctypes on the
current CUDA stream.  The parts of a model call nothing else for device work
(matrix products included: `linear`).  There is no CPU implementation in the
package; `CudaKernels` raises if the device or the compiler is missing.
"""
from __future__ import annotations

import contextlib
import ctypes
from collections import Counter
from typing import Dict, Optional, Sequence

import torch

from ..parts.base import PagedKVView, StepBatch
from . import build
from .attention_plan import PagedAttentionPlanner

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

DEVICE_ERRORS = {8: "a wait inside a kernel ran out (a pipeline stalled); the step's results are not valid",
                 1: "a token id outside the vocabulary",
                 2: "a key or value was needed from a page the block table does not hold",
                 4: "a position beyond the rotation table (longer than the model's maximum length)"}


class KernelError(RuntimeError):
    pass


class KernelSet:
    """Operators of a step.  Shapes: T rows, H width, all tensors contiguous.

    embed(table[V,H], ids[T], src[T], last) -> h[T,H] float32; row r takes last[src[r]] instead of ids[r] where src[r] >= 0
    add_rmsnorm(h, delta, weight, eps, out, rows):
        rows is None: h[r] += delta[r] (if delta is given); out[r] = h[r] * rsqrt(mean(h[r]^2) + eps) * weight
        rows given:   v = h[rows[i]] + delta[rows[i]];      out[i] = v * rsqrt(mean(v^2) + eps) * weight
    linear(x[M,K], w[N,K], out[M,N], bias[N] float32 or None): out = x . w^T + bias
    qkv_rope_append(qkv[T,(Hq+2Hkv)D], bias, cos, sin, batch, kv, q_out[T,Hq*D]):
        adds the bias, rotates queries and keys by the row's position, writes the queries to
        q_out and, if kv.writes, keys and values into their cache pages
    paged_attention(q[T,Hq*D], batch, kv, out[T,Hq*D], scale): causal (windowed if kv.spec.window)
        softmax(scale * q.k) v over the keys of the row's request, from the pages
    rope_append_attention(qkv, bias, cos, sin, batch, kv, out, num_heads, scale, workspace) -> bool   (optional)
        both of the above in one launch where the set has a kernel for the step at hand; False: nothing was
        done and the caller makes the two calls
    silu_mul(gate_up[T,2I], out[T,I]): out = silu(gate_up[:, :I]) * gate_up[:, I:]
    sample(logits[R,V], temperature[R], seeds[R], counters[R]) -> tokens[R] int32
    """

    def check_errors(self) -> None:
        """Raises if a kernel has flagged bad input since the last check (synchronises)."""


def _dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return 0
    if t == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t}")


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    if t is None:
        return _c_void_p(0)
    if not t.is_contiguous():
        raise KernelError("kernels take contiguous tensors")
    if not t.is_cuda:
        raise KernelError("kernels take tensors on the device; a host tensor's address means nothing there")
    return _c_void_p(t.data_ptr())


_RETURN_CODES = {-1: "unsupported dtype", -2: "unsupported shape", -3: "misaligned operand", -4: "size beyond the kernel's limit"}


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: refused ({_RETURN_CODES.get(code, code)})")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_SIGNATURES = {
    "elementwise": {
        "kvb_embed": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
        "kvb_add_rmsnorm": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_float, _c_void_p],
        "kvb_silu_mul": [_c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    },
    "rope_append": {
        "kvb_qkv_rope_append": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p,
                                _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    },
    "attention_generic": {
        "kvb_paged_attention_generic": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                                        _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                        _c_float, _c_void_p, _c_void_p],
    },
    "gemm_simt": {
        "kvb_gemm_simt": [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    },
    "gemm_skinny": {
        "kvb_gemm_skinny": [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_gemm_skinny_norm_act": [_c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_gemm_skinny_residual": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_gemm_skinny_qkv": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int, _c_void_p,
                                _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                                _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    },
    "gemm_wstream": {
        "kvb_gemm_wstream": [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    },
    "gemm_tcgen05": {
        "kvb_gemm_tcgen05": [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    },
    "attention_flash": {
        "kvb_flash_head_dim": [],
        "kvb_flash_decode": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                             _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                             _c_void_p],
        "kvb_flash_decode_cluster": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                     _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                     _c_void_p],
        "kvb_flash_decode_tma_max_clusters": [_c_int],
        "kvb_flash_decode_tma": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int,
                                 _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                 _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                                 _c_void_p, _c_void_p],
        "kvb_flash_prefill": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                              _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    },
    "attention_tc": {
        "kvb_attention_tc_head_dim": [],
        "kvb_attention_tc": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                             _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                             _c_void_p, _c_void_p],
    },
    "primitive_costs": {
        "kvb_primitive_costs_count": [],
        "kvb_primitive_costs": [_c_void_p, _c_void_p, _c_void_p, _c_void_p],
    },
    "wait_probe": {
        "kvb_wait_probe": [_c_void_p, _c_void_p, _c_void_p],
    },
    "sampling": {
        "kvb_sample_parts": [_c_int],
        "kvb_sample": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    },
}


_OPTIONAL = {"kvb_flash_decode_tma", "kvb_flash_decode_tma_max_clusters"}      # only in attention_flash variants for head sizes 64 and 128


class _Library:
    """A lazily built and loaded kernel module with typed entry points."""

    def __init__(self, module: str, variant: str = "", flags: Sequence[str] = ()):
        self.module, self.variant, self.flags = module, variant, tuple(flags)
        self._lib = None

    def __getattr__(self, name: str):
        if self._lib is None:
            lib = build.load_module(self.module, self.variant, self.flags)
            for fname, argtypes in _SIGNATURES[self.module].items():
                try:
                    fn = getattr(lib, fname)
                except AttributeError:
                    if fname in _OPTIONAL:
                        continue              # a variant compiled for a size that has no such entry point
                    raise
                fn.argtypes = argtypes
                fn.restype = _c_int
            self._lib = lib
        return getattr(self._lib, name)


class CudaKernels(KernelSet):
    def __init__(self, device: torch.device | str = "cuda:0", bf16_gemm: str = "auto"):
        """`bf16_gemm`: which kernel multiplies bfloat16 matrices of more than SKINNY_MAX_ROWS rows:
        "tcgen05" (the tensor-memory kernel of csrc/gemm_tcgen05.cu), "cublas" (the library, as the
        reference uses it), "simt" (CUDA cores), or "auto": the tensor-memory kernel for the gate/up
        projection with its fused activation where 256 x 256 two-SM tiles fill the machine (measured
        30.8 us against 28.4 + 13.6 us for library product + activation kernel at 2,048 x 9,728 x 896),
        the library for plain products, where it is still ahead (28.4 against 33.7 us at that size)."""
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError("kvcache_b200 runs on a CUDA device (sm_100a) only; no device is available")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"kernels are built for sm_100a; device {self.device} is sm_{major}{minor}")
        if bf16_gemm not in ("auto", "tcgen05", "cublas", "simt"):
            raise KernelError(f"unknown bf16_gemm '{bf16_gemm}'")
        self.bf16_gemm = bf16_gemm
        self._elementwise = _Library("elementwise")
        self._rope = _Library("rope_append")
        self._attn_generic = _Library("attention_generic")
        self._gemm_simt = _Library("gemm_simt")
        self._sampling = _Library("sampling")
        self._gemm_skinny = _Library("gemm_skinny")
        self._gemm_tc = _Library("gemm_tcgen05")
        self._gemm_ws = _Library("gemm_wstream")
        self.wstream_gemm = True             # bfloat16, 16 < M <= WSTREAM_MAX_ROWS, K % 8 == 0: weights streamed through tcgen05
        self.skinny_gemm = True              # bfloat16, M <= 64, K % 32 == 0: weight-streaming kernel
        self._flash: Dict[int, _Library] = {}
        self._attn_tc: Dict[int, _Library] = {}
        # Portions of prompts with at least this many rows go through the tensor-memory attention kernel
        # (bfloat16, head size 64 or 128, pages of 8..64 tokens); None turns it off.  Measured on 24 layers of the
        # 0.5B shape: the mma.sync kernel is ahead at 128 and 256 rows (1.09 / 1.24 ms a step against 1.14 / 1.28),
        # the tensor-memory kernel from 512 rows on (1.56 against 1.69 ms).
        self.tc_attention_min_rows: Optional[int] = 384
        self.flash_attention = True          # bfloat16, head sizes 16..128: tensor-core kernels
        # Decode steps of at least this many requests: bias, rotation and append inside the TMA decode kernel (None: never).
        # Measured on 24 layers of the 0.5B shape at 4,096 tokens of context, a step with the kernel against a step with
        # the separate rotation kernel: 1 % slower at 1 and 8 requests (the queries reach the tensor cores a trip through
        # shared memory later, which costs what the saved launch gains), 1.4 % faster at 16, 3 % at 64.
        self.fused_rope_min_requests: Optional[int] = 16
        # Decode attention splits the keys of a request over blocks.  "cluster": the splits (at most 8) are a
        # thread-block cluster and merge through distributed shared memory; "tma": the same with keys and values
        # brought by TMA (head sizes 64 and 128, pages of 8..64 tokens; otherwise it falls back to "cluster");
        # "ticket": up to 32 splits leave partial results in scratch and the last one to finish merges them.
        self.decode_merge = "tma"
        self.decode_cluster_max = 8          # the kernel's limit
        self.decode_pow2_splits = True
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.decode_ctas_wanted = 2 * self.sm_count    # the split over the keys aims at this many blocks in flight
        self.decode_min_tiles = 4            # ... but gives a split at least this many 64-key tiles
        # Most clusters one (request, kv head) is given by the TMA kernel (0: always one).  The clusters meet through memory,
        # which costs about 5 us; it pays where there are fewer blocks than SMs and each block still keeps eight 64-key tiles -
        # one request: 10.5 -> 8.9 us a layer at 8,192 tokens, 18.0 -> 10.9 at 16,000, 34.6 -> 11.8 at 32,000 - and not where
        # the blocks fill the GPU already (8 requests at 8,192 tokens: 11.7 -> 17.3 us).
        self.decode_superclusters = 16
        self.decode_super_min_tiles = 8
        self.error_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0
        self.launch_counts: Counter = Counter()      # launches by kernel, as issued from the host (a replayed graph adds none)
        self._pinned_stream: Optional[_c_void_p] = None
        self._tma_cluster_capacity: Dict[tuple, int] = {}
        self._timing = None
        self._attention_planner: Optional[PagedAttentionPlanner] = None

    # ---- helpers -----------------------------------------------------------
    def _count(self, kernel: str) -> None:
        """One launch of `kernel` (while a graph is being recorded: one launch of every later replay)."""
        self.launches += 1
        self.launch_counts[kernel] += 1

    def _stream(self) -> _c_void_p:
        if self._pinned_stream is not None:
            return self._pinned_stream
        return _c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    @contextlib.contextmanager
    def on_current_stream(self):
        """Within the block every launch goes to the stream that is current now (asked for once, not per launch)."""
        saved = self._pinned_stream
        self._pinned_stream = _c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        try:
            yield
        finally:
            self._pinned_stream = saved

    def start_timing(self, hold_ms: float = 4.0) -> None:
        """From now on every operator is bracketed by CUDA events and filed under its class (kernels/timing.py).
        For steps launched kernel by kernel: graphs cannot hold the events.  `hold_ms`: how long the GPU is kept busy
        before each step so that the host can queue the step's launches (0: not at all)."""
        from .timing import KernelTiming
        if self._timing is None:
            self._timing = KernelTiming(self, hold_ms)
            self._timing.start()

    def stop_timing(self) -> Dict[str, dict]:
        """Ends timing; returns {class: {"us", "bytes", "calls", "launches"}} summed over the calls since `start_timing`."""
        timing, self._timing = self._timing, None
        return timing.stop() if timing is not None else {}

    def check_errors(self) -> None:
        word = int(self.error_word.item())
        if word:
            self.error_word.zero_()
            reasons = [text for bit, text in DEVICE_ERRORS.items() if word & bit]
            raise KernelError("a kernel flagged bad input: " + "; ".join(reasons))

    def probe_wait_timeout(self) -> int:
        """Runs a kernel whose only wait cannot end (csrc/wait_probe.cu: the bounded mbarrier wait of the TMA and tcgen05
        kernels, on a barrier nothing arrives on, with a short poll limit).  The kernel gives up, sets the time-out bit of
        the error word and returns; the next `check_errors()` raises.  Returns the number of polls it made."""
        outcome = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._count("wait_probe")
        _check(_Library("wait_probe").kvb_wait_probe(_ptr(self.error_word), _ptr(outcome), self._stream()), "wait_probe")
        gave_up, polls = (int(v) for v in outcome.tolist())
        if gave_up != 2:
            raise KernelError("the wait of the probe kernel ended although nothing arrived on its barrier")
        return polls

    PRIMITIVE_NAMES = ("wait on a completed mbarrier, all lanes", "the same, one lane asks and the warp meets again", "shuffle",
                       "vote and population count", "expect_tx by one lane and the warp meets again",
                       "tcgen05.mma 128 x 64 x 16, operands in shared memory", "tcgen05.mma 128 x 128 x 16, operands in shared memory",
                       "tcgen05.mma 128 x 64 x 16, A in tensor memory", "tcgen05.commit", "TMA copy of one page (16 rows of 128 bytes)",
                       "tcgen05.ld of 32 columns and its wait", "mma.sync m16n8k16 (bfloat16), eight accumulators in turn",
                       "mma.sync m16n8k16, each needing the one before")

    def primitive_costs(self) -> Dict[str, float]:
        """Clocks per primitive of the warp-specialised kernels on an otherwise idle SM (csrc/primitive_costs.cu)."""
        lib = _Library("primitive_costs")
        count = lib.kvb_primitive_costs_count()
        zeros = torch.zeros(4 << 20, dtype=torch.uint8, device=self.device)
        out = torch.zeros(count + 1, dtype=torch.float32, device=self.device)
        for _ in range(2):          # the second run finds the code and the tensor map cached
            self._count("primitive_costs")
            _check(lib.kvb_primitive_costs(_ptr(zeros), _ptr(out), _ptr(self.error_word), self._stream()), "primitive_costs")
        self.check_errors()
        return dict(zip(self.PRIMITIVE_NAMES, out[:count].tolist()))

    def paged_attention_planner(self) -> PagedAttentionPlanner:
        """The work lists `paged_attention` and `rope_append_attention` read from `StepBatch.plans` (one planner for all layers)."""
        if self._attention_planner is None:
            self._attention_planner = PagedAttentionPlanner()
        return self._attention_planner

    # ---- operators ---------------------------------------------------------
    def embed(self, table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, src: Optional[torch.Tensor] = None,
              last: Optional[torch.Tensor] = None, out16: Optional[torch.Tensor] = None) -> None:
        """out[r] = table[ids[r]], or table[last[src[r]]] where src[r] >= 0 (a token still on the device);
        `out16`: the same rows in bfloat16 as well."""
        T, H = out.shape
        self._count("embed")
        _check(self._elementwise.kvb_embed(_dtype_code(table.dtype), _ptr(table), _ptr(ids), _ptr(src), _ptr(last), _ptr(out),
                                           _ptr(out16), T, H, table.shape[0], _ptr(self.error_word), self._stream()), "embed")

    # ---- the folded chain of a decode layer ------------------------------------------------------------------
    # For steps of few rows a layer can run as five launches instead of eight: the norm before a product inside that
    # product (x holds the residual stream in bfloat16, not normalised), the add after a product inside it
    # (`linear_into_residual`), and bias, rotation and cache append inside the q/k/v projection.  Off by default: measured
    # on 24 layers of the 0.5B shape at 8 requests and 4,096 tokens of context the folded chain takes 32 us a layer against
    # 26 - each folded product takes as long as the kernels it replaces together (q/k/v 5.6 us against 2.5 + 1.9 + 1.4),
    # and the products that add into the residual stream 5.0 us against 2.5, because the kernel after them, which streams
    # many megabytes of weights before its own wait, now crowds their loads instead of a norm kernel's that has few.
    fold_norms = False

    @property
    def fold_key(self) -> tuple:
        """The switches `can_fold` depends on (a model caches its answer per value of this)."""
        return (self.fold_norms, self.skinny_gemm, self.wstream_gemm, self.bf16_gemm)

    def can_fold(self, dtype: torch.dtype, rows: int, K: int, N: int) -> bool:
        """Whether a product of `rows` rows with a [N, K] weight can take the folded forms (the register kernel's)."""
        return self.fold_norms and self._skinny(dtype, rows, K, N)

    def norm_gate_up_act(self, x16: torch.Tensor, w_gate_up: torch.Tensor, norm_w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        """out[M, I] = silu(g) * u with [g | u] = rmsnorm(x16; norm_w, eps) . w_gate_up^T (rows interleaved in eights)."""
        M, K = x16.shape
        self._count("gemm_skinny_norm_act")
        _check(self._gemm_skinny.kvb_gemm_skinny_norm_act(_ptr(x16), _ptr(w_gate_up), _ptr(norm_w), float(eps), _ptr(out), M,
                                                          w_gate_up.shape[0], K, self._stream()), "norm_gate_up_act")

    def linear_into_residual(self, x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, h16: torch.Tensor,
                             bias: Optional[torch.Tensor] = None) -> None:
        """h += x . w^T + bias (float32, in place); h16 = bfloat16(h)."""
        M, K = x.shape
        self._count("gemm_skinny_residual")
        _check(self._gemm_skinny.kvb_gemm_skinny_residual(_ptr(x), _ptr(w), _ptr(bias), _ptr(h), _ptr(h16), M, w.shape[0], K,
                                                          self._stream()), "linear_into_residual")

    def norm_qkv_rope_append(self, x16: torch.Tensor, w_paired: torch.Tensor, bias_paired: Optional[torch.Tensor],
                             norm_w: torch.Tensor, eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                             batch: StepBatch, kv: PagedKVView, q_out: torch.Tensor, num_heads: int) -> None:
        """The q/k/v projection of rmsnorm(x16) with bias, rotation and append: `qkv_rope_append` after `linear` after the
        norm, in one launch.  `w_paired` / `bias_paired`: rows permuted within each head so that rows 16 j + i and
        16 j + 8 + i (i < 8) are dimensions 8 j + i and D / 2 + 8 j + i (see `pair_rotation_rows`)."""
        M, K = x16.shape
        spec = kv.spec
        if cos is not None and cos.shape[1] * 2 != spec.head_dim:
            raise KernelError("the folded q/k/v projection rotates whole heads only")
        self._count("gemm_skinny_qkv")
        _check(self._gemm_skinny.kvb_gemm_skinny_qkv(
            _ptr(x16), _ptr(w_paired), _ptr(bias_paired), _ptr(norm_w), float(eps), _ptr(cos), _ptr(sin),
            0 if cos is None else cos.shape[0], _ptr(batch.positions), _ptr(batch.row_segment), _ptr(kv.block_table),
            kv.block_table.shape[1], _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(q_out), M, K, num_heads, spec.num_kv_heads,
            spec.head_dim, kv.page_size, 1 if kv.writes else 0, _ptr(self.error_word), self._stream()), "norm_qkv_rope_append")

    @staticmethod
    def pair_rotation_rows(num_heads_total: int, head_dim: int) -> torch.Tensor:
        """The row order `norm_qkv_rope_append` wants: for every head, tiles of 16 rows holding dimensions
        8 j .. 8 j + 7 and D / 2 + 8 j .. D / 2 + 8 j + 7.  Returns the source row of each row of the permuted matrix."""
        half = head_dim // 2
        within = torch.cat([torch.cat([torch.arange(8 * j, 8 * j + 8), torch.arange(half + 8 * j, half + 8 * j + 8)])
                            for j in range(head_dim // 16)])
        return (torch.arange(num_heads_total)[:, None] * head_dim + within[None, :]).reshape(-1)

    def add_rmsnorm(self, h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                    out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        n_out, H = out.shape
        self._count("add_rmsnorm")
        _check(self._elementwise.kvb_add_rmsnorm(_dtype_code(out.dtype), _ptr(h), _ptr(delta), _ptr(weight),
                                                 _ptr(out), _ptr(rows), n_out, H, float(eps), self._stream()),
               "add_rmsnorm")

    def silu_mul(self, gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
        T, I = out.shape
        self._count("silu_mul")
        _check(self._elementwise.kvb_silu_mul(_dtype_code(out.dtype), _ptr(gate_up), _ptr(out), T, I,
                                              1 if interleaved else 0, self._stream()), "silu_mul")

    def gate_up_act(self, x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, workspace, interleaved: bool) -> None:
        """out[M, I] = silu(x Wg^T) * (x Wu^T); `w_gate_up` [2 I, K] holds gate and up rows one after the
        other, or interleaved in eights (see csrc/gemm_skinny.cu)."""
        M, K = x.shape
        I = out.shape[1]
        if interleaved and self._skinny(x.dtype, M, K, 2 * I):
            self._count("gemm_skinny")
            _check(self._gemm_skinny.kvb_gemm_skinny(_dtype_code(out.dtype), 1, _ptr(x), _ptr(w_gate_up), _ptr(None),
                                                     _ptr(out), M, 2 * I, K, self._stream()), "gate_up_act (skinny)")
            return
        if interleaved and self._wstream(x.dtype, M, K):
            self._count("gemm_wstream")
            _check(self._gemm_ws.kvb_gemm_wstream(_dtype_code(out.dtype), 1, _ptr(x), _ptr(w_gate_up), _ptr(None), _ptr(out), M,
                                                  2 * I, K, _ptr(self.error_word), self._stream()), "gate_up_act (wstream)")
            return
        if interleaved and self._tcgen05(x, w_gate_up, out, fused=True):
            self._count("gemm_tcgen05")
            _check(self._gemm_tc.kvb_gemm_tcgen05(_dtype_code(out.dtype), 1, _ptr(x), _ptr(w_gate_up), _ptr(None), _ptr(out), M,
                                                  2 * I, K, _ptr(self.error_word), self._stream()), "gate_up_act (tcgen05)")
            return
        gate_up = workspace.buffer("ffn.gate_up", (M, 2 * I), out.dtype)
        self.linear(x, w_gate_up, gate_up)
        self.silu_mul(gate_up, out, interleaved)

    SKINNY_MAX_ROWS = 16     # above this the weight-streaming tcgen05 product takes over
    WSTREAM_MAX_ROWS = 32    # measured on 24 layers of the 0.5B shape: 11 % faster steps than the library at 17 and 32 rows, equal at 40, slower at 128

    # Products with K >= 4 N (the feed-forward's way down) up to this many rows: the library splits K too little for
    # them - 8.4 us against 5.8 at 64 x 896 x 4864; steps of 40, 48 and 64 requests are 4 % faster for it.
    WSTREAM_DEEP_MAX_ROWS = 64

    def _wstream(self, dtype: torch.dtype, M: int, K: int, N: int = 0) -> bool:
        rows = self.WSTREAM_DEEP_MAX_ROWS if K >= 4 * N > 0 else self.WSTREAM_MAX_ROWS
        return self.wstream_gemm and dtype == torch.bfloat16 and self.bf16_gemm == "auto" and M <= rows and K % 8 == 0

    # Weights of at least this many bytes go through the weight-streaming tcgen05 kernel at any number of rows up to its
    # limit: TMA keeps more bytes in flight per SM than register loads do.  Measured at 8 rows: the 7B model's gate/up
    # (272 MB) 45 against 64 us, its way down (136 MB) 25 against 40 us, output heads (272 MB .. 1.1 GB) at 6.6-7.0
    # against 5.1-6.0 TB/s; below it the register kernel is ahead (1.5B gate/up, 55 MB: 10.5 against 13.2 us).
    WSTREAM_MIN_WEIGHT_BYTES = 96 << 20

    def _skinny(self, dtype: torch.dtype, M: int, K: int, N: int = 0) -> bool:
        if 2 * N * K >= self.WSTREAM_MIN_WEIGHT_BYTES and self._wstream(dtype, M, K, N):
            return False
        return self.skinny_gemm and dtype == torch.bfloat16 and M <= self.SKINNY_MAX_ROWS and K % 32 == 0

    def _tcgen05(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, fused: bool = False) -> bool:
        """The tensor-memory kernel takes bfloat16 operands whose rows are multiples of 16 bytes."""
        if x.dtype != torch.bfloat16 or w.shape[1] % 8 != 0 or (x.data_ptr() | w.data_ptr() | out.data_ptr()) % 16 != 0:
            return False
        if self.bf16_gemm == "auto":
            return fused and -(-x.shape[0] // 256) * -(-w.shape[0] // 256) >= self.sm_count
        return self.bf16_gemm == "tcgen05"

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """out = x . w^T + bias."""
        M = x.shape[0]
        N, K = w.shape
        if x.shape[1] != K or tuple(out.shape) != (M, N):
            raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not fit")
        if self._skinny(x.dtype, M, K, N):
            self._count("gemm_skinny")
            _check(self._gemm_skinny.kvb_gemm_skinny(_dtype_code(out.dtype), 0, _ptr(x), _ptr(w), _ptr(bias),
                                                     _ptr(out), M, N, K, self._stream()), "linear (skinny)")
            return
        if self._wstream(x.dtype, M, K, N):
            self._count("gemm_wstream")
            _check(self._gemm_ws.kvb_gemm_wstream(_dtype_code(out.dtype), 0, _ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K,
                                                  _ptr(self.error_word), self._stream()), "linear (wstream)")
            return
        if self._tcgen05(x, w, out):
            self._count("gemm_tcgen05")
            _check(self._gemm_tc.kvb_gemm_tcgen05(_dtype_code(out.dtype), 0, _ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K,
                                                  _ptr(self.error_word), self._stream()), "linear (tcgen05)")
            return
        if x.dtype == torch.bfloat16 and self.bf16_gemm != "simt":
            # Library matrix product, as the reference's cublasGemmEx (apps/qwen_serve.cu:27-39).
            self._count("gemm_library")
            if out.dtype == torch.bfloat16:
                torch.matmul(x, w.t(), out=out)
            else:
                torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
            if bias is not None:
                out.add_(bias)
            return
        self._count("gemm_simt")
        _check(self._gemm_simt.kvb_gemm_simt(_dtype_code(x.dtype), _dtype_code(out.dtype), _ptr(x), _ptr(w),
                                             _ptr(bias), _ptr(out), M, N, K, self._stream()), "linear")

    def qkv_rope_append(self, qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                        sin: Optional[torch.Tensor], batch: StepBatch, kv: PagedKVView, q_out: torch.Tensor,
                        num_heads: int) -> None:
        T = qkv.shape[0]
        spec = kv.spec
        rot_half = 0 if cos is None else cos.shape[1]
        table_len = 0 if cos is None else cos.shape[0]
        self._count("rope_append")
        _check(self._rope.kvb_qkv_rope_append(
            _dtype_code(qkv.dtype), _ptr(qkv), _ptr(bias), _ptr(cos), _ptr(sin), rot_half, table_len,
            _ptr(batch.positions), _ptr(batch.row_segment), _ptr(kv.block_table), kv.block_table.shape[1],
            _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(q_out), T, num_heads, spec.num_kv_heads, spec.head_dim,
            kv.page_size, 1 if kv.writes else 0, _ptr(self.error_word), self._stream()), "qkv_rope_append")

    def _tma_clusters(self, lib, head_dim: int, nsplit: int) -> int:
        key = (head_dim, nsplit)
        found = self._tma_cluster_capacity.get(key)
        if found is None:
            found = int(lib.kvb_flash_decode_tma_max_clusters(nsplit)) or 1 << 30     # unknown: no limit
            self._tma_cluster_capacity[key] = found
        return found

    def _flash_library(self, head_dim: int) -> _Library:
        lib = self._flash.get(head_dim)
        if lib is None:
            lib = _Library("attention_flash", f"d{head_dim}", [f"-DKVB_HEAD_DIM={head_dim}"])
            self._flash[head_dim] = lib
        return lib

    def _cluster_splits(self, n: int, Hkv: int, tiles: int) -> int:
        nsplit = max(1, min(self.decode_cluster_max, self.decode_ctas_wanted // (n * Hkv), tiles // self.decode_min_tiles))
        if self.decode_pow2_splits:
            nsplit = 1 << (nsplit.bit_length() - 1)     # clusters of 3, 5, 6, 7 blocks place badly
        return nsplit

    def _tma_decode(self, D: int, kv: PagedKVView) -> bool:
        return self.decode_merge == "tma" and D % 64 == 0 and 8 <= kv.page_size <= 64

    def _fit_clusters(self, lib, D: int, clusters: int, nsplit: int) -> int:
        # All clusters at once: a grid with more clusters than the GPU holds runs in waves.
        while nsplit > 1 and clusters > self._tma_clusters(lib, D, nsplit):
            nsplit //= 2
        return nsplit

    def rope_append_attention(self, qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                              sin: Optional[torch.Tensor], batch: StepBatch, kv: PagedKVView, out: torch.Tensor,
                              num_heads: int, scale: float, workspace=None) -> bool:
        """`qkv_rope_append` and `paged_attention` in one launch, where one kernel does both: a step in which every
        request brings one token, bfloat16, through the TMA decode kernel, into a cache that this call writes.  Returns
        False (and does nothing) otherwise; the caller then makes the two calls."""
        spec = kv.spec
        D, Hkv, n = spec.head_dim, spec.num_kv_heads, batch.num_segments
        plan = batch.plans.get(PagedAttentionPlanner.name)
        if not (self.fused_rope_min_requests is not None and n >= self.fused_rope_min_requests
                and self.flash_attention and qkv.dtype == torch.bfloat16 and kv.writes and plan is not None
                and batch.num_tokens == n and plan.counts["decode_items"] == n and num_heads // Hkv <= 16
                and self._tma_decode(D, kv) and (cos is None or cos.shape[1] <= D // 2)):
            return False
        lib = self._flash_library(D)
        tiles = -(-(kv.block_table.shape[1] * kv.page_size) // 64)
        nsplit = self._fit_clusters(lib, D, n * Hkv, self._cluster_splits(n, Hkv, tiles))
        self._count("flash_decode_tma_fused")
        _check(lib.kvb_flash_decode_tma(
            None, _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), kv.k_pages.shape[0], _ptr(kv.block_table),
            kv.block_table.shape[1], None, n, _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len),
            num_heads, Hkv, kv.page_size, spec.window or 0, nsplit, float(scale), _ptr(qkv), _ptr(bias), _ptr(cos), _ptr(sin),
            0 if cos is None else cos.shape[1], 0 if cos is None else cos.shape[0], 1, None, None, _ptr(self.error_word),
            self._stream()), "flash_decode_tma (rotation and append fused)")
        return True

    def paged_attention(self, q: torch.Tensor, batch: StepBatch, kv: PagedKVView, out: torch.Tensor,
                        num_heads: int, scale: float, workspace=None) -> None:
        T = q.shape[0]
        spec = kv.spec
        D, Hkv = spec.head_dim, spec.num_kv_heads
        plan = batch.plans.get(PagedAttentionPlanner.name)
        if (self.flash_attention and q.dtype == torch.bfloat16 and D % 16 == 0 and D <= 128 and num_heads // Hkv <= 16
                and workspace is not None and plan is not None):
            lib = self._flash_library(D)
            counts, lists = plan.counts, plan.arrays
            if (counts["tc_units"] and self.tc_attention_min_rows is not None and D in (64, 128)
                    and 8 <= kv.page_size <= 64 and batch.max_q_len >= self.tc_attention_min_rows):
                tc = self._attn_tc.get(D)
                if tc is None:
                    tc = self._attn_tc[D] = _Library("attention_tc", f"d{D}", [f"-DKVB_HEAD_DIM={D}"])
                units = counts["tc_units"]
                scratch = workspace.buffer("attn.tc_scratch", (units * num_heads * 128 * (D + 2),), torch.float32)
                # Two counters of the kernel's work queue, then a ticket per (tile, head); the kernel leaves all of them zero.
                tickets = workspace.zeros("attn.tc_tickets", (2 + max(counts["tc_tiles"], 1) * num_heads,), torch.int32)
                self._count("attention_tc")
                _check(tc.kvb_attention_tc(
                    _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), kv.k_pages.shape[0], _ptr(kv.block_table),
                    kv.block_table.shape[1], _ptr(lists["tc_units"]), units, _ptr(scratch), _ptr(tickets),
                    _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len), T, num_heads, Hkv, kv.page_size,
                    spec.window or 0, float(scale), _ptr(self.error_word), self._stream()), "attention_tc")
            elif counts["prefill_units"]:
                units = counts["prefill_units"]
                scratch = workspace.buffer("attn.prefill_scratch", (units * num_heads * 64 * (D + 2),), torch.float32)
                tickets = workspace.zeros("attn.prefill_tickets", (max(counts["prefill_tiles"], 1) * num_heads,), torch.int32)
                self._count("flash_prefill")
                _check(lib.kvb_flash_prefill(
                    _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table), kv.block_table.shape[1],
                    _ptr(lists["prefill_units"]), units, _ptr(batch.seg_q_start), _ptr(batch.seg_q_len),
                    _ptr(batch.seg_kv_len), _ptr(scratch), _ptr(tickets), num_heads, Hkv, kv.page_size, spec.window or 0,
                    float(scale), self._stream()), "flash_prefill")
            n = counts["decode_items"]
            items = lists["decode_items"]
            if n:
                # Sized by the longest request the block table allows, not by this step's lengths, so that the
                # split (and with it the rounding) is the same in every step and under a CUDA graph.
                tiles = -(-(kv.block_table.shape[1] * kv.page_size) // 64)
                if self.decode_merge in ("cluster", "tma"):
                    nsplit = self._cluster_splits(n, Hkv, tiles)
                    if self._tma_decode(D, kv):
                        self._count("flash_decode_tma")
                        # Few requests with many keys: several clusters for each (request, kv head), each with a run of
                        # the keys, so that the whole GPU streams them; their sums meet in scratch, the last to finish
                        # adds them in cluster order.  Like the split itself this follows from the block table's
                        # capacity and the number of requests, never from the lengths of the moment.
                        nsuper = 1
                        if nsplit > 1 and self.decode_superclusters:
                            nsuper = max(1, min(self.decode_superclusters, self.sm_count // (n * Hkv * nsplit),
                                                tiles // (max(self.decode_min_tiles, self.decode_super_min_tiles) * nsplit)))
                            while nsuper > 1 and n * Hkv * nsuper > self._tma_clusters(lib, D, nsplit):
                                nsuper -= 1
                        nsplit = self._fit_clusters(lib, D, n * Hkv * nsuper, nsplit)
                        if nsplit == 1:
                            nsuper = 1
                        scratch = tickets = None
                        if nsuper > 1:
                            scratch = workspace.buffer("attn.decode_super", (n * Hkv * nsuper * 16 * (D + 2),), torch.float32)
                            tickets = workspace.zeros("attn.decode_super_tickets", (n * Hkv * 8,), torch.int32)
                        _check(lib.kvb_flash_decode_tma(
                            _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), kv.k_pages.shape[0],
                            _ptr(kv.block_table), kv.block_table.shape[1],
                            _ptr(None if n == batch.num_segments else items), n,   # every segment, in order: no list
                            _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len), num_heads, Hkv,
                            kv.page_size, spec.window or 0, nsplit, float(scale), None, None, None, None, 0, 0,
                            nsuper, _ptr(scratch), _ptr(tickets), _ptr(self.error_word), self._stream()), "flash_decode_tma")
                        return
                    self._count("flash_decode_cluster")
                    _check(lib.kvb_flash_decode_cluster(
                        _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table),
                        kv.block_table.shape[1], _ptr(items), n, _ptr(batch.seg_q_start),
                        _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len), num_heads, Hkv, kv.page_size, spec.window or 0,
                        nsplit, float(scale), self._stream()), "flash_decode_cluster")
                    return
                nsplit = max(1, min(32, 2 * self.decode_ctas_wanted // (n * Hkv), tiles // self.decode_min_tiles))
                scratch = workspace.buffer("attn.decode_scratch", (n * Hkv * nsplit * 16 * (D + 2),), torch.float32)
                tickets = workspace.zeros("attn.decode_tickets", (n * Hkv,), torch.int32)
                self._count("flash_decode_ticket")
                _check(lib.kvb_flash_decode(
                    _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table), kv.block_table.shape[1],
                    _ptr(items), n, _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len),
                    _ptr(scratch), _ptr(tickets), num_heads, Hkv, kv.page_size, spec.window or 0, nsplit, float(scale),
                    self._stream()), "flash_decode")
            return
        self._count("attention_generic")
        _check(self._attn_generic.kvb_paged_attention_generic(
            _dtype_code(q.dtype), _ptr(q), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table),
            kv.block_table.shape[1], _ptr(batch.positions), _ptr(batch.row_segment), _ptr(out), T, num_heads,
            spec.num_kv_heads, spec.head_dim, kv.page_size, spec.window or 0, float(scale),
            _ptr(self.error_word), self._stream()), "paged_attention")

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
               out: torch.Tensor, scratch_val: torch.Tensor, scratch_idx: torch.Tensor) -> None:
        R, V = logits.shape
        self._count("sample")
        _check(self._sampling.kvb_sample(_ptr(logits), R, V, _ptr(temperature), _ptr(seeds), _ptr(counters),
                                         _ptr(scratch_val), _ptr(scratch_idx), _ptr(out), self._stream()), "sample")

    def sample_parts(self, vocab: int) -> int:
        return int(self._sampling.kvb_sample_parts(vocab))
