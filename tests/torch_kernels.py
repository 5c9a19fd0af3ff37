"""Plain PyTorch statement of every operator of the kernel set, over the same paged
layouts.  Two uses: the per-kernel reference that each CUDA kernel is compared with, and
a stand-in kernel set that lets the engine's host logic (cache, step function, scheduler)
run in tests on a machine without a GPU.  It is test code: the package has no CPU path.
"""
from __future__ import annotations

from typing import Optional

import torch

from plain_qwen2 import gumbel_scores


class TorchKernels:
    """Same operator signatures as kvcache_b200.kernels.api.CudaKernels; math in float32
    (or float64 when `wide` is set), stores in the tensors' own types."""

    def __init__(self, wide: bool = False):
        self.f = torch.float64 if wide else torch.float32
        self.launches = 0

    def check_errors(self) -> None:
        pass

    def embed(self, table, ids, out, src=None, last=None):
        ids = ids.long()
        if src is not None:
            ids = torch.where(src >= 0, last[src.clamp(min=0).long()].long(), ids)
        out.copy_(table[ids].to(torch.float32))

    def add_rmsnorm(self, h, delta, weight, eps, out, rows=None):
        f = self.f
        if rows is None:
            if delta is not None:
                h.add_(delta.to(torch.float32))
            v = h.to(f)
        else:
            v = h[rows.long()].to(f)
            if delta is not None:
                v = (h[rows.long()] + delta[rows.long()].to(torch.float32)).to(f)
        inv = torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + eps)
        out.copy_((v * inv * weight.to(f)).to(out.dtype))

    def linear(self, x, w, out, bias=None):
        y = x.to(self.f) @ w.to(self.f).t()
        if bias is not None:
            y = y + bias.to(self.f)
        out.copy_(y.to(out.dtype))

    def qkv_rope_append(self, qkv, bias, cos, sin, batch, kv, q_out, num_heads):
        f = self.f
        T = qkv.shape[0]
        Hq, Hkv, D = num_heads, kv.spec.num_kv_heads, kv.spec.head_dim
        x = qkv.to(f)
        if bias is not None:
            x = x + bias.to(f)
        x = x.view(T, Hq + 2 * Hkv, D).clone()
        pos = batch.positions.long()
        if cos is not None:
            half = cos.shape[1]
            c, s = cos[pos].to(f)[:, None, :], sin[pos].to(f)[:, None, :]
            qk = x[:, :Hq + Hkv, :]
            x1, x2 = qk[..., :half].clone(), qk[..., half:2 * half].clone()
            qk[..., :half] = x1 * c - x2 * s
            qk[..., half:2 * half] = x2 * c + x1 * s
        q_out.copy_(x[:, :Hq, :].reshape(T, Hq * D).to(q_out.dtype))
        if kv.writes:
            seg = batch.row_segment.long()
            page = kv.block_table[seg, pos // kv.page_size].long()
            assert bool((page >= 0).all()), "append into a page the block table does not hold"
            slot = pos % kv.page_size
            kv.k_pages[page, :, slot, :] = x[:, Hq:Hq + Hkv, :].to(kv.k_pages.dtype)
            kv.v_pages[page, :, slot, :] = x[:, Hq + Hkv:, :].to(kv.v_pages.dtype)

    def paged_attention(self, q, batch, kv, out, num_heads, scale, workspace=None):
        f = self.f
        T = q.shape[0]
        Hq, Hkv, D = num_heads, kv.spec.num_kv_heads, kv.spec.head_dim
        group = Hq // Hkv
        window = kv.spec.window
        qf = q.to(f).view(T, Hq, D)
        result = torch.zeros(T, Hq, D, dtype=f, device=q.device)
        for r in range(T):
            p = int(batch.positions[r])
            seg = int(batch.row_segment[r])
            lo = max(0, p - window + 1) if window else 0
            js = torch.arange(lo, p + 1, device=q.device)
            pages = kv.block_table[seg, js // kv.page_size].long()
            assert bool((pages >= 0).all()), "a needed key lies in a page the block table does not hold"
            keys = kv.k_pages[pages, :, js % kv.page_size, :].to(f)     # [n, Hkv, D]
            vals = kv.v_pages[pages, :, js % kv.page_size, :].to(f)
            for h in range(Hq):
                s = (keys[:, h // group, :] @ qf[r, h]) * scale
                result[r, h] = torch.softmax(s, dim=0) @ vals[:, h // group, :]
        out.copy_(result.view(T, Hq * D).to(out.dtype))

    def silu_mul(self, gate_up, out, interleaved=False):
        I = out.shape[1]
        if interleaved:
            pairs = gate_up.view(gate_up.shape[0], I // 8, 2, 8)
            g, u = pairs[:, :, 0, :].reshape(-1, I).to(self.f), pairs[:, :, 1, :].reshape(-1, I).to(self.f)
        else:
            g, u = gate_up[:, :I].to(self.f), gate_up[:, I:].to(self.f)
        out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))

    def gate_up_act(self, x, w_gate_up, out, workspace, interleaved):
        gate_up = torch.empty(x.shape[0], w_gate_up.shape[0], dtype=out.dtype, device=out.device)
        self.linear(x, w_gate_up, gate_up)
        self.silu_mul(gate_up, out, interleaved)

    def sample_parts(self, vocab):
        return 1

    def sample(self, logits, temperature, seeds, counters, out, scratch_val=None, scratch_idx=None):
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t > 0:
                scores = gumbel_scores(logits[r].cpu(), t, int(seeds[r]), int(counters[r]))
                out[r] = int(torch.argmax(scores))
            else:
                out[r] = int(torch.argmax(logits[r]))
