"""A toy architecture defined here, in the test: a mixer with per-request state of its own, a feed-forward that
routes every row to one of several experts, another position encoding, a layer of each kind - registered, built
from a folder and stepped with no change to the framework."""
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Mapping

import pytest
import torch

from helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _define():
    from kvcache_b200.config.base import KeyReader, ModelConfig
    from kvcache_b200.parts import (DecoderModel, FeedForward, GatedMLP, GQAAttention, LayerCall, Mixer, PositionEncoding,
                                    PreNormBlock, RMSNorm, StateSpec, StepPlanner)
    from kvcache_b200.weights import TensorSpec

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        width: int
        vocab: int
        inner: int
        decay: float
        eps: float

        @classmethod
        def from_dict(cls, data, where="config.json"):
            r = KeyReader(data, where)
            out = cls("ToyRunningMeanLM", r.integer("width"), r.integer("vocab"), r.integer("inner"), r.number("decay"),
                      r.number("eps"))
            r.finish()
            return out

        def to_dict(self) -> Dict[str, Any]:
            return {"architectures": [self.architecture], "width": self.width, "vocab": self.vocab, "inner": self.inner,
                    "decay": self.decay, "eps": self.eps}

    class FirstRows(StepPlanner):
        """A work list of the toy mixer's own: the first row of every segment, and the longest segment as the count
        that fixes how many passes the mixer makes.  The runner packs it like the attention kernels' lists."""
        name = "toy_first_rows"

        def sections(self, num_tokens, num_segments):
            return {"first_rows": num_segments}

        def plan(self, starts, counts):
            import numpy as np
            first = np.zeros(len(counts), dtype=np.int32)
            np.cumsum(np.asarray(counts)[:-1], out=first[1:])
            return {"first_rows": first}, {"longest": int(max(counts))}

    class RunningMean(Mixer):
        """delta[r] = W . (s[r] / n[r]) with s[r] = decay * s[r - 1] + x[r] and n[r] = decay * n[r - 1] + 1 over the
        request's rows: two states of fixed size that have to survive from step to step, in the slot the cache manager
        gave the request.  Everything runs on the device from the step's device arrays, so that a step can be recorded
        in a CUDA graph and replayed."""

        def __init__(self, width, decay, prefix, dtype):
            self.width, self.decay, self.prefix, self.dtype = width, decay, prefix, dtype
            self.w = None

        def tensor_specs(self):
            return {self.prefix + "mix.weight": TensorSpec((self.width, self.width))}

        def bind(self, tensors: Mapping[str, torch.Tensor], device):
            self.w = tensors[self.prefix + "mix.weight"].to(torch.float32).to(device)

        def state_spec(self):
            return {"sum": StateSpec((self.width,), "float32"), "weight": StateSpec((1,), "float32")}

        def step_planners(self, kernels):
            return (FirstRows(),)

        def forward(self, x, ctx):
            b, plan = ctx.batch, ctx.batch.plans["toy_first_rows"]
            T = x.shape[0]
            slots = b.seg_slot.long()
            s, n = ctx.state["sum"].index_select(0, slots), ctx.state["weight"].index_select(0, slots)
            xf = torch.cat([x.float(), x.new_zeros((1, self.width), dtype=torch.float32)])
            out = torch.zeros((T + 1, self.width), dtype=torch.float32, device=x.device)     # row T takes what no segment owns
            first = plan.arrays["first_rows"].long()
            for j in range(plan.counts["longest"]):
                live = (b.seg_q_len > j)[:, None]
                rows = torch.where(live[:, 0], first + j, torch.full_like(first, T))
                s = torch.where(live, self.decay * s + xf[rows], s)
                n = torch.where(live, self.decay * n + 1.0, n)
                out.index_copy_(0, rows, (s / n.clamp(min=1e-30)) @ self.w.t())
            ctx.state["sum"].index_copy_(0, slots, s)
            ctx.state["weight"].index_copy_(0, slots, n)
            return out[:T].to(x.dtype)

    class TopOneExperts(FeedForward):
        """delta[r] = p_e * Wout_e relu(Win_e x[r]) with e = argmax of the router's logits (float32) and p_e its
        softmax weight: a feed-forward with routing, its sizes (experts, inner width) given as parameters."""

        def __init__(self, width, inner, experts, prefix, dtype):
            self.width, self.inner, self.experts, self.prefix, self.dtype = width, inner, experts, prefix, dtype
            self.router = self.w_in = self.w_out = None

        def tensor_specs(self):
            p = self.prefix
            return {p + "router.weight": TensorSpec((self.experts, self.width)),
                    p + "in.weight": TensorSpec((self.experts, self.inner, self.width)),
                    p + "out.weight": TensorSpec((self.experts, self.width, self.inner))}

        def bind(self, tensors: Mapping[str, torch.Tensor], device):
            p = self.prefix
            self.router = tensors[p + "router.weight"].to(torch.float32).to(device)
            self.w_in = tensors[p + "in.weight"].to(torch.float32).to(device)
            self.w_out = tensors[p + "out.weight"].to(torch.float32).to(device)

        def forward(self, x, ctx):
            xf = x.float()
            prob = torch.softmax(xf @ self.router.t(), dim=-1)
            chosen = prob.argmax(dim=-1, keepdim=True)                                  # [T, 1]
            # Every expert on every row, then the chosen one is picked: shapes that do not depend on the routing, so
            # that the step can be recorded in a CUDA graph.
            hidden = torch.relu(torch.einsum("tw,eiw->tei", xf, self.w_in))
            every = torch.einsum("tei,ewi->tew", hidden, self.w_out)
            picked = every.gather(1, chosen[:, :, None].expand(-1, 1, self.width)).squeeze(1)
            return (prob.gather(1, chosen) * picked).to(x.dtype)

    class AddedSinusoid(PositionEncoding):
        """Adds sin(pos / 10) to every element of the embedded row: an encoding that acts at the embedding."""

        def on_embed(self, h, ctx):
            h.add_(torch.sin(ctx.batch.positions.float() / 10.0)[:, None])

    def build(config, dtype="float32", device="cuda:0", max_positions=None):
        c = config
        blocks = [
            PreNormBlock(c.width, RMSNorm(c.width, c.eps, "l0.n1"), RunningMean(c.width, c.decay, "l0.", dtype),
                         RMSNorm(c.width, c.eps, "l0.n2"), GatedMLP(c.width, c.inner, activation="silu", prefix="l0.f.", dtype=dtype), dtype),
            PreNormBlock(c.width, RMSNorm(c.width, c.eps, "l1.n1"),
                         GQAAttention(c.width, 2, 1, c.width // 2, qkv_bias=False, out_bias=False, position=None, window=None,
                                      prefix="l1.a.", dtype=dtype),
                         RMSNorm(c.width, c.eps, "l1.n2"), TopOneExperts(c.width, c.inner, 3, "l1.moe.", dtype), dtype),
        ]
        return DecoderModel(config=c, dtype=dtype, vocab_size=c.vocab, width=c.width, embed_name="emb", head_name=None,
                            blocks=blocks, schedule=[LayerCall(0, 0), LayerCall(1, 1)],
                            final_norm=RMSNorm(c.width, c.eps, "final"), position=AddedSinusoid())

    return ToyConfig, build


def _plain(config, w, tokens):
    """The toy model on one whole sequence, in float64."""
    import plain_qwen2 as plain
    W = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    x = W["emb"][torch.tensor(tokens)] + torch.sin(torch.arange(T).double() / 10.0)[:, None]
    n = plain.rms_norm(x, W["l0.n1"], config["eps"])
    s, weight, mixed = torch.zeros(config["width"], dtype=torch.float64), 0.0, []
    for r in range(T):
        s = config["decay"] * s + n[r]
        weight = config["decay"] * weight + 1.0
        mixed.append(W["l0.mix.weight"] @ (s / weight))
    x = x + torch.stack(mixed)
    x = x + plain.swiglu(plain.rms_norm(x, W["l0.n2"], config["eps"]), W["l0.f.gate_proj.weight"], W["l0.f.up_proj.weight"],
                         W["l0.f.down_proj.weight"])
    n = plain.rms_norm(x, W["l1.n1"], config["eps"])
    D = config["width"] // 2
    q = plain.linear(n, W["l1.a.q_proj.weight"]).view(T, 2, D)
    k = plain.linear(n, W["l1.a.k_proj.weight"]).view(T, 1, D)
    v = plain.linear(n, W["l1.a.v_proj.weight"]).view(T, 1, D)
    x = x + plain.linear(plain.attention(q, k, v).reshape(T, 2 * D), W["l1.a.o_proj.weight"])
    n = plain.rms_norm(x, W["l1.n2"], config["eps"])
    prob = torch.softmax(n @ W["l1.moe.router.weight"].t(), dim=-1)
    routed = []
    for r in range(T):
        e = int(prob[r].argmax())
        routed.append(prob[r, e] * (W["l1.moe.out.weight"][e] @ torch.relu(W["l1.moe.in.weight"][e] @ n[r])))
    x = x + torch.stack(routed)
    return plain.linear(plain.rms_norm(x, W["final"], config["eps"]), W["emb"])


@pytest.mark.parametrize("use_graphs", [False, True])
def test_toy_architecture_with_state_runs_through_the_unchanged_engine(tmp_path, use_graphs):
    from safetensors.torch import load_file
    from kvcache_b200.config import EngineOptions, register_architecture, unregister_architecture
    from kvcache_b200.engine.core import EngineCore
    from kvcache_b200.engine.runner import StepEntry
    from kvcache_b200.weights import write_random_model
    ToyConfig, build = _define()
    register_architecture("ToyRunningMeanLM", ToyConfig, build)
    try:
        data = {"architectures": ["ToyRunningMeanLM"], "width": 32, "vocab": 50, "inner": 40, "decay": 0.8, "eps": 1e-5}
        folder = write_random_model(os.path.join(tmp_path, "toy"), ToyConfig.from_dict(data), seed=1, dtype=torch.float32)
        with open(os.path.join(folder, "config.json")) as fh:
            assert json.load(fh)["architectures"] == ["ToyRunningMeanLM"]
        weights = load_file(os.path.join(folder, "model.safetensors"))
        core = EngineCore(folder, EngineOptions(dtype="float32", page_size=8, num_pages=16, max_running=2,
                                                max_tokens_per_step=64, max_model_len=64, use_graphs=use_graphs))
        core.runner.graph_after_sightings = 1          # a portion's launches are recorded the first time its shape comes
        entries = core.model.cache_entries()
        assert entries[0].kv is None and set(entries[0].state) == {"sum", "weight"}   # the toy mixer: two states, no pages
        assert entries[1].kv is not None and entries[1].state is None                 # attention: pages, no state
        assert core.cache.states[0]["sum"].shape == (2, 32) and core.cache.states[0]["weight"].shape == (2, 1)
        assert [p.name for p in core.runner.planners] == ["toy_first_rows", "paged_attention"]
        a = [3, 14, 15, 9, 2, 6, 5, 35, 8, 9, 7, 9, 3, 2, 38, 4, 6]
        b = [27, 18, 28, 18, 2, 8, 4, 5, 9, 0, 45]
        want_a, want_b = _plain(data, weights, a), _plain(data, weights, b)
        sa, sb = core.cache.admit(), core.cache.admit()
        got_a, got_b = [], []
        step = lambda entries: core.runner.step(entries).clone()
        # a in portions and then token by token, b beside it: the state has to be carried in a's slot.
        out = step([StepEntry(sa, a[:5], range(5)), StepEntry(sb, b[:3], range(3))])
        got_a.append(out[:5]); got_b.append(out[5:])
        out = step([StepEntry(sb, b[3:], range(8)), StepEntry(sa, a[5:7], range(2))])
        got_b.append(out[:8]); got_a.append(out[8:])
        # One token a step, sampled on the device: with graphs the first of these steps records the launches (and
        # runs once), the others replay them.
        for i in range(7, len(a)):
            got_a.append(core.runner.step([StepEntry(sa, a[i:i + 1], [0])], sample=True)[0].clone())
        assert_close(torch.cat(got_a), want_a, 1e-4, "a")
        assert_close(torch.cat(got_b), want_b, 1e-4, "b")
        if use_graphs:
            assert core.runner.graph_replays == len(a) - 7 - 1
        # A slot that is used again starts from a zeroed state.
        core.cache.release(sa)
        sc = core.cache.admit()
        assert sc == sa and all(float(t[sc].abs().sum()) == 0.0 for t in core.cache.states[0].values())
        again = step([StepEntry(sc, b, range(len(b)))])                     # one portion of one prompt: recorded as it runs
        assert_close(again, want_b, 1e-4, "b in a's old slot")
        core.cache.release(sc)
        sd = core.cache.admit()
        replayed = step([StepEntry(sd, b, range(len(b)))])                  # the same shape again: replayed
        assert_close(replayed, want_b, 1e-4, "b again, replayed")
        if use_graphs:
            assert core.runner.graph_replays == len(a) - 7 - 1 + 1
        core.kernels.check_errors()
    finally:
        unregister_architecture("ToyRunningMeanLM")
