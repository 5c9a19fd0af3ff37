"""Each part of a model alone on the GPU against the plain implementation's function for it, at sizes
the engine tests do not use; and the model as data: a layer run twice, a call that reads another call's cache."""
import pytest
import torch

import plain_qwen2 as plain
from helpers import assert_close, batch_to, clone_kv, paged_scenario, random_tokens
from tiny_configs import make_model_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL = {"float32": 2e-5, "bfloat16": 2e-2}
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def kernels():
    from kvcache_b200.kernels.api import CudaKernels
    return CudaKernels(DEV)


def _ctx(kernels, batch=None, kv=None):
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.base import LayerContext
    return LayerContext(batch=batch, kernels=kernels, workspace=Workspace(DEV), kv=kv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rms_norm_part(kernels, dtype):
    from kvcache_b200.parts.norm import RMSNorm
    g = torch.Generator().manual_seed(0)
    T, H, eps = 7, 200, 2e-5
    w = (1 + 0.2 * torch.randn(H, generator=g)).to(torch.bfloat16)
    part = RMSNorm(H, eps, "n.weight")
    assert part.tensor_specs()["n.weight"].shape == (H,) and part.init_kinds() == {"n.weight": "ones_plus_normal"}
    part.bind({"n.weight": w}, torch.device(DEV))
    assert part.weight.dtype == torch.float32
    h = torch.randn(T, H, generator=g) * 2
    delta = torch.randn(T, H, generator=g).to(TORCH[dtype])
    hd, out = h.clone().to(DEV), torch.empty(T, H, dtype=TORCH[dtype], device=DEV)
    part.add_norm(hd, delta.to(DEV), out, _ctx(kernels))
    want_h = h.double() + delta.double()
    assert_close(hd, want_h, 1e-6)
    assert_close(out, plain.rms_norm(want_h, w.double(), eps), REL[dtype])


def test_rotary_tables_match_the_plain_rotation():
    from kvcache_b200.parts.position import RotaryHalf
    part = RotaryHalf(48, 50000.0, 300)
    part.bind({}, torch.device("cpu"))
    rot = part.rotation()
    assert rot.cos.shape == (300, 24) and rot.cos.dtype == torch.float32
    x = torch.randn(5, 2, 48, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    pos = torch.tensor([0, 1, 17, 255, 299])
    c, s = rot.cos[pos].double()[:, None, :], rot.sin[pos].double()[:, None, :]
    mine = torch.cat([x[..., :24] * c - x[..., 24:] * s, x[..., 24:] * c + x[..., :24] * s], dim=-1)
    assert torch.allclose(mine, plain.rope(x, pos, 50000.0), atol=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_alone(kernels, dtype, window):
    """A whole sequence run as one segment through the mixer: projections with bias, rotation, cache append,
    attention over the pages it just wrote, output projection."""
    from kvcache_b200.parts.attention import GQAAttention
    from kvcache_b200.parts.position import RotaryHalf
    g = torch.Generator().manual_seed(2)
    T, H, Hq, Hkv, D, theta = 23, 72, 6, 3, 16, 777.0
    names = {"q": (Hq * D, H), "k": (Hkv * D, H), "v": (Hkv * D, H)}
    w = {f"a.{n}_proj.weight": (torch.randn(shape, generator=g) * 0.2).to(torch.bfloat16) for n, shape in names.items()}
    w.update({f"a.{n}_proj.bias": (torch.randn(shape[0], generator=g) * 0.2).to(torch.bfloat16) for n, shape in names.items()})
    w["a.o_proj.weight"] = (torch.randn(H, Hq * D, generator=g) * 0.2).to(torch.bfloat16)
    rope = RotaryHalf(D, theta, 64)
    rope.bind({}, torch.device(DEV))
    part = GQAAttention(H, Hq, Hkv, D, qkv_bias=True, out_bias=False, position=rope, window=window, prefix="a.", dtype=dtype)
    assert set(part.tensor_specs()) == set(w) and part.cache_spec().window == window and part.state_spec() is None
    part.bind(w, torch.device(DEV))
    x = torch.randn(T, H, generator=g).to(TORCH[dtype])
    batch, kv = paged_scenario([(0, T)], num_kv_heads=Hkv, head_dim=D, page_size=8, dtype=TORCH[dtype], device="cpu",
                               window=window, seed=3, fill_history=False)
    out = part.forward(x.to(DEV), _ctx(kernels, batch_to(batch, DEV), clone_kv(kv, DEV)))
    wd = {k: v.double() for k, v in w.items()}
    xd, pos = x.double(), torch.arange(T)
    q = plain.rope(plain.linear(xd, wd["a.q_proj.weight"], wd["a.q_proj.bias"]).view(T, Hq, D), pos, theta)
    k = plain.rope(plain.linear(xd, wd["a.k_proj.weight"], wd["a.k_proj.bias"]).view(T, Hkv, D), pos, theta)
    v = plain.linear(xd, wd["a.v_proj.weight"], wd["a.v_proj.bias"]).view(T, Hkv, D)
    want = plain.linear(plain.attention(q, k, v, window).reshape(T, Hq * D), wd["a.o_proj.weight"])
    assert_close(out, want, REL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H,I", [(5, 72, 136), (40, 64, 100), (3, 40, 77)])
def test_feed_forward_part_alone(kernels, dtype, T, H, I):
    from kvcache_b200.parts.feedforward import GatedMLP
    g = torch.Generator().manual_seed(4)
    w = {"m.gate_proj.weight": torch.randn(I, H, generator=g) * 0.3, "m.up_proj.weight": torch.randn(I, H, generator=g) * 0.3,
         "m.down_proj.weight": torch.randn(H, I, generator=g) * 0.3}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    part = GatedMLP(H, I, activation="silu", prefix="m.", dtype=dtype)
    part.bind(w, torch.device(DEV))
    assert part.interleaved == (I % 8 == 0)
    x = torch.randn(T, H, generator=g).to(TORCH[dtype])
    out = part.forward(x.to(DEV), _ctx(kernels))
    want = plain.swiglu(x.double(), *(w[f"m.{n}_proj.weight"].double() for n in ("gate", "up", "down")))
    assert_close(out, want, REL[dtype])
    with pytest.raises(ValueError, match="activation"):
        GatedMLP(H, I, activation="gelu", prefix="m.", dtype=dtype)


def _model_with_schedule(folder, schedule, dtype="float32"):
    """The tiny model of `folder` with another order of layer calls."""
    from kvcache_b200.cache import CacheManager
    from kvcache_b200.config.registry import load_config
    from kvcache_b200.engine.runner import ModelRunner
    from kvcache_b200.kernels.api import CudaKernels
    from kvcache_b200.models.qwen2 import build_qwen2
    from kvcache_b200.parts.model import DecoderModel
    from kvcache_b200.weights.loader import load_tensors
    base = build_qwen2(load_config(folder), dtype=dtype, max_positions=256)
    model = DecoderModel(config=base.config, dtype=dtype, vocab_size=base.vocab_size, width=base.width,
                         embed_name=base.embed_name, head_name=base.head_name, blocks=base.blocks, schedule=schedule,
                         final_norm=base.final_norm, position=base.position)
    model.bind(load_tensors(folder, model.tensor_specs()), torch.device(DEV))
    cache = CacheManager(model.cache_entries(), page_size=8, num_pages=32, max_slots=2, max_tokens_per_request=256,
                         dtype=dtype, device=DEV)
    return ModelRunner(model, cache, CudaKernels(DEV), max_tokens_per_step=128), model


def test_a_layer_may_run_twice(tmp_path):
    from kvcache_b200.engine.runner import StepEntry
    from kvcache_b200.parts.model import LayerCall
    folder = make_model_folder(tmp_path, "B", dtype=torch.bfloat16)
    config, weights = plain.read_folder(folder)
    runner, model = _model_with_schedule(folder, [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 3)])
    assert len(model.cache_entries()) == 4
    tokens = random_tokens(config["vocab_size"], 30, 5)
    want = plain.logits_of(config, weights, tokens, layer_order=[0, 1, 0, 2])
    slot = runner.cache.admit()
    got = [runner.step([StepEntry(slot, tokens[:19], list(range(19)))]).clone()]
    for i in range(19, 30):                           # the second call of layer 0 has a cache of its own
        got.append(runner.step([StepEntry(slot, tokens[i:i + 1], [0])]).clone())
    assert_close(torch.cat(got), want, 1e-4)


def test_a_call_may_read_another_calls_cache(tmp_path):
    from kvcache_b200.engine.runner import StepEntry
    from kvcache_b200.parts.model import LayerCall
    folder = make_model_folder(tmp_path, "B", dtype=torch.bfloat16)
    config, weights = plain.read_folder(folder)
    runner, model = _model_with_schedule(folder, [LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 0, writes_cache=False)])
    assert len(model.cache_entries()) == 2
    tokens = random_tokens(config["vocab_size"], 26, 6)
    # Plain: layer 2 attends with its own queries to the keys and values layer 0 made.
    x = plain.embed(weights["model.embed_tokens.weight"], tokens)
    pos, kv0 = torch.arange(len(tokens)), []
    x = plain.block(x, weights, config, 0, pos, kv_out=kv0)
    x = plain.block(x, weights, config, 1, pos)
    x = plain.block(x, weights, config, 2, pos, shared_kv=kv0[0])
    want = plain.linear(plain.rms_norm(x, weights["model.norm.weight"], config["rms_norm_eps"]), weights["lm_head.weight"])
    slot = runner.cache.admit()
    got = [runner.step([StepEntry(slot, tokens[:9], list(range(9)))]).clone(),
           runner.step([StepEntry(slot, tokens[9:24], list(range(15)))]).clone()]
    for i in range(24, 26):
        got.append(runner.step([StepEntry(slot, tokens[i:i + 1], [0])]).clone())
    assert_close(torch.cat(got), want, 1e-4)


def test_schedule_is_checked():
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.models.qwen2 import build_qwen2
    from kvcache_b200.parts.model import DecoderModel, LayerCall
    from tiny_configs import TINY_A
    base = build_qwen2(config_from_dict(TINY_A), dtype="float32")
    make = lambda schedule: DecoderModel(config=base.config, dtype="float32", vocab_size=base.vocab_size, width=base.width,
                                         embed_name=base.embed_name, head_name=None, blocks=base.blocks, schedule=schedule,
                                         final_norm=base.final_norm, position=base.position)
    with pytest.raises(ValueError, match="names layer"):
        make([LayerCall(5, 0)])
    with pytest.raises(ValueError, match="written by two"):
        make([LayerCall(0, 0), LayerCall(1, 0)])
    with pytest.raises(ValueError, match="before any call writes"):
        make([LayerCall(0, 1, writes_cache=False)])
