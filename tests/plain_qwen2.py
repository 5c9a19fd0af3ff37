"""Plain, slow implementation of the Qwen2 dense decoder: whole sequences, no cache, one
function for each part, float64 by default.  It shares no code with `kvcache_b200`
(it reads the model folder with the `safetensors` package and `json`).

It rests on the reference's formulas, not on running the reference: kimxinw/kvcache's
model code is CUDA + cuBLAS with the sizes of one checkpoint compiled in
(apps/qwen_serve.cu:20-23) and cannot be imported or run on a CPU.  Each function
cites the lines it restates.  What of the reference does run on a CPU is its numpy
attention of one query over 128 keys (ref/ref_attn.py): its output lies under
tests/golden with the script that made it, and `attention` is held to it in
tests/test_plain.py.  The window keys have no counterpart in the reference
(it has no windowed layers); their meaning here is the one of the checkpoint's own
config.json: layers at index >= max_window_layers see `sliding_window` keys, their
own included, when use_sliding_window is true.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


def read_folder(folder: str, dtype: torch.dtype = torch.float64):
    """config.json as a dict and every tensor of model.safetensors widened to `dtype`."""
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
        config = json.load(fh)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return config, weights


def embed(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """x[r, :] = E[ids[r], :]  (src/qwen_kernels.cu:14-20)."""
    return table[torch.as_tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, row by row  (src/qwen_kernels.cu:26-40)."""
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * inv * weight


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T (+ b), W stored [out, in]  (apps/qwen_serve.cu:27-31; bias src/qwen_kernels.cu:46-49)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half on [T, heads, D]: pairs (t, t + D/2), inv_t = theta^(-2t/D), a = pos * inv_t,
    x'_t = x_t cos a - x_{t+D/2} sin a, x'_{t+D/2} = x_{t+D/2} cos a + x_t sin a
    (src/qwen_kernels.cu:65-78; per-row positions :253-264)."""
    D = x.shape[-1]
    half = D // 2
    t = torch.arange(half, dtype=torch.float64)
    inv = torch.exp(-math.log(theta) * (2.0 * t / D))
    ang = positions.to(torch.float64)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.  q [T, Hq, D], k, v [T, Hkv, D].
    Query at position p, head h uses kv head h // (Hq / Hkv) and keys 0..p, scores scaled by
    1/sqrt(D) after the dot product, softmax, weighted sum of values
    (src/qwen_kernels.cu:148-176; scale apps/qwen_serve.cu:53).  With a window w the keys are
    max(0, p - w + 1)..p."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    scale = 1.0 / math.sqrt(D)
    out = torch.zeros_like(q)
    for h in range(Hq):
        hk = h // group
        scores = (q[:, h, :] @ k[:, hk, :].t()) * scale            # [T, T]
        pos = torch.arange(T)
        visible = pos[None, :] <= pos[:, None]
        if window is not None:
            visible &= pos[None, :] > pos[:, None] - window
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ v[:, hk, :]
    return out


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """(g / (1 + e^-g) * u) Wd^T with g = x Wg^T, u = x Wu^T  (apps/qwen_serve.cu:112-115;
    src/qwen_kernels.cu:102-105)."""
    g = linear(x, w_gate)
    u = linear(x, w_up)
    return linear(g / (1.0 + torch.exp(-g)) * u, w_down)


def layer_window(config: dict, layer: int) -> Optional[int]:
    if config.get("use_sliding_window") and layer >= config.get("max_window_layers", config["num_hidden_layers"]):
        return config["sliding_window"]
    return None


def block(x: torch.Tensor, weights: Dict[str, torch.Tensor], config: dict, layer: int,
          positions: torch.Tensor, shared_kv=None, kv_out: Optional[list] = None) -> torch.Tensor:
    """One layer in the reference's order (apps/qwen_serve.cu:101-116): norm, q/k/v with bias,
    rotation of q and k, attention, o_proj, residual, norm, gated feed-forward, residual.
    `shared_kv`: (k, v) of another layer call to attend to instead of this call's own;
    `kv_out`: a list that receives this call's rotated keys and values."""
    p = f"model.layers.{layer}."
    Hq, Hkv = config["num_attention_heads"], config.get("num_key_value_heads", config["num_attention_heads"])
    D = config.get("head_dim") or config["hidden_size"] // Hq
    eps, theta = config["rms_norm_eps"], config["rope_theta"]
    T = x.shape[0]
    n = rms_norm(x, weights[p + "input_layernorm.weight"], eps)
    q = linear(n, weights[p + "self_attn.q_proj.weight"], weights[p + "self_attn.q_proj.bias"]).view(T, Hq, D)
    k = linear(n, weights[p + "self_attn.k_proj.weight"], weights[p + "self_attn.k_proj.bias"]).view(T, Hkv, D)
    v = linear(n, weights[p + "self_attn.v_proj.weight"], weights[p + "self_attn.v_proj.bias"]).view(T, Hkv, D)
    q, k = rope(q, positions, theta), rope(k, positions, theta)
    if kv_out is not None:
        kv_out.append((k, v))
    if shared_kv is not None:
        k, v = shared_kv
    a = attention(q, k, v, layer_window(config, layer)).reshape(T, Hq * D)
    x = x + linear(a, weights[p + "self_attn.o_proj.weight"])
    n = rms_norm(x, weights[p + "post_attention_layernorm.weight"], eps)
    return x + swiglu(n, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                      weights[p + "mlp.down_proj.weight"])


def logits_of(config: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int],
              layer_order: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence (apps/qwen_serve.cu:97-119:
    embedding, layers, model.norm, lm_head - the embedding table when tied,
    tools/dump_weights.py:23-26)."""
    x = embed(weights["model.embed_tokens.weight"], tokens)
    positions = torch.arange(len(tokens))
    for layer in (layer_order if layer_order is not None else range(config["num_hidden_layers"])):
        x = block(x, weights, config, layer, positions)
    x = rms_norm(x, weights["model.norm.weight"], config["rms_norm_eps"])
    head = weights["model.embed_tokens.weight"] if config.get("tie_word_embeddings") else weights["lm_head.weight"]
    return linear(x, head)


def greedy_generate(config: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int], max_new: int,
                    eos: Sequence[int] = ()) -> List[int]:
    """Greedy decoding by recomputing the whole sequence for every token; the lowest index
    wins a tie.  Stops after `max_new` tokens or after an end token, which is kept
    (apps/qwen_serve.cu:182-190)."""
    tokens = list(prompt)
    out: List[int] = []
    for _ in range(max_new):
        nxt = int(torch.argmax(logits_of(config, weights, tokens)[-1]).item())
        out.append(nxt)
        tokens.append(nxt)
        if nxt in eos:
            break
    return out


# ---- the sampler's random numbers, restated ---------------------------------------------

def philox4x32_10(counter, key):
    """Philox4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3")."""
    M0, M1, W0, W1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c3 ^ k1) & mask, p0 & mask
        k0, k1 = (k0 + W0) & mask, (k1 + W1) & mask
    return c0, c1, c2, c3


def gumbel_scores(logits: torch.Tensor, temperature: float, seed: int, counter: int) -> torch.Tensor:
    """logit_i / temperature + g_i with g_i = -log(-log(u_i)), u_i = ((bits_i >> 8) + 0.5) / 2^24 and
    bits_i the first word of Philox(counter = (i, counter, 0, 0), key = seed)."""
    V = logits.shape[0]
    key = (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    u = torch.tensor([((philox4x32_10((i, counter, 0, 0), key)[0] >> 8) + 0.5) / 16777216.0 for i in range(V)],
                     dtype=torch.float64)
    return logits.to(torch.float64) / temperature - torch.log(-torch.log(u))
