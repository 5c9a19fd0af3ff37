"""The plain implementation checked against independent statements of the same formulas,
so that what every other test compares with is itself sound."""
import math

import torch

import plain_qwen2 as plain
from tiny_configs import make_model_folder


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    inv = 1.0 / math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(plain.rms_norm(x, w, 1e-6), torch.tensor([[3 * inv * 2, 4 * inv * 0.5]], dtype=torch.float64))


def test_rope_is_a_rotation_of_pairs_by_complex_multiplication():
    T, H, D, theta = 6, 2, 8, 10000.0
    x = torch.randn(T, H, D, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    pos = torch.tensor([0, 1, 2, 50, 51, 1000])
    got = plain.rope(x, pos, theta)
    for t in range(D // 2):
        angle = pos.double() * theta ** (-2.0 * t / D)
        z = torch.complex(x[..., t], x[..., t + D // 2]) * torch.polar(torch.ones(T, dtype=torch.float64), angle)[:, None]
        assert torch.allclose(got[..., t], z.real) and torch.allclose(got[..., t + D // 2], z.imag)
    assert torch.equal(plain.rope(x, torch.zeros(T, dtype=torch.long), theta), x)          # position 0: identity
    # Scores depend on the distance of positions only.
    q, k = torch.randn(1, 1, D, dtype=torch.float64), torch.randn(1, 1, D, dtype=torch.float64)
    s1 = (plain.rope(q, torch.tensor([7]), theta) * plain.rope(k, torch.tensor([3]), theta)).sum()
    s2 = (plain.rope(q, torch.tensor([104]), theta) * plain.rope(k, torch.tensor([100]), theta)).sum()
    assert abs(s1 - s2) < 1e-9


def _attention_by_loops(q, k, v, window):
    T, Hq, D = q.shape
    group = Hq // k.shape[1]
    out = torch.zeros_like(q)
    for p in range(T):
        lo = max(0, p - window + 1) if window else 0
        for h in range(Hq):
            m, l, acc = -float("inf"), 0.0, torch.zeros(D, dtype=q.dtype)
            for j in range(lo, p + 1):          # the reference's online form, src/qwen_kernels.cu:159-176
                s = float(q[p, h] @ k[j, h // group]) / math.sqrt(D)
                m_new = max(m, s)
                c, e = math.exp(m - m_new), math.exp(s - m_new)
                l, acc, m = l * c + e, acc * c + e * v[j, h // group], m_new
            out[p, h] = acc / l
    return out


def test_attention_matches_the_online_loop_with_and_without_window():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(11, n, 8, dtype=torch.float64, generator=g) for n in (6, 2, 2))
    for window in (None, 1, 4, 11, 50):
        assert torch.allclose(plain.attention(q, k, v, window), _attention_by_loops(q, k, v, window), atol=1e-12)


def test_window_edge_is_exact():
    """A key that takes all the weight is seen at distance window - 1 and not at distance window."""
    T, D, W = 12, 4, 5
    q = torch.zeros(T, 1, D, dtype=torch.float64)
    k = torch.zeros(T, 1, D, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64)[:, None, None].expand(T, 1, D).clone()
    k[3, 0, 0] = 100.0
    q[:, 0, 0] = 100.0
    out = plain.attention(q, k, v, W)[:, 0, 0]
    assert abs(out[7] - 3.0) < 1e-9            # 7 - 3 = 4 = W - 1: still inside
    assert abs(out[8] - 6.0) < 1e-9            # 8 - 3 = 5 = W: outside; keys 4..8 share the weight
    assert abs(plain.attention(q, k, v, None)[11, 0, 0] - 3.0) < 1e-9


def test_attention_equals_the_references_own_numpy_attention():
    """The one piece of the reference's arithmetic that runs on a CPU, ref/ref_attn.py: one query per head over 128
    keys.  Here it is the last position of a sequence of 128 (it sees every key); eight heads with a kv head each."""
    from helpers import reference_attention_case
    q, K, V, want = reference_attention_case()
    H, S, D = K.shape
    queries = torch.zeros(S, H, D, dtype=torch.float64)
    queries[-1] = q.double()
    got = plain.attention(queries, K.double().transpose(0, 1).contiguous(), V.double().transpose(0, 1).contiguous())[-1]
    assert (got - want.double()).abs().max().item() < 2e-6


def test_swiglu_by_hand():
    x = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    wg, wu, wd = (torch.tensor(m, dtype=torch.float64) for m in ([[1.0, 0.0]], [[0.0, 1.0]], [[3.0], [1.0]]))
    g, u = 1.0, -2.0
    a = g / (1 + math.exp(-g)) * u
    assert torch.allclose(plain.swiglu(x, wg, wu, wd), torch.tensor([[3 * a, a]], dtype=torch.float64))


def test_logits_are_causal_and_the_tied_head_is_the_embedding(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    config, w = plain.read_folder(folder)
    tokens = [5, 17, 3, 200, 41, 7, 99]
    full = plain.logits_of(config, w, tokens)
    assert torch.allclose(full[:4], plain.logits_of(config, w, tokens[:4]), atol=1e-12)
    assert config["tie_word_embeddings"] and "lm_head.weight" not in w
    out = plain.greedy_generate(config, w, tokens, 3)
    assert out[0] == int(torch.argmax(full[-1]))


def test_philox_known_answers():
    """Known-answer vectors of Philox4x32-10 from the Random123 distribution."""
    cases = [((0, 0, 0, 0), (0, 0), "6627e8d5 e169c58d bc57ac4c 9b00dbd8"),
             ((0xffffffff,) * 4, (0xffffffff,) * 2, "408f276d 41c83b0e a20bc7c6 6d5451fd"),
             ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0), "d16cfe09 94fdcceb 5001e420 24126ea1")]
    for counter, key, want in cases:
        assert " ".join("%08x" % x for x in plain.philox4x32_10(counter, key)) == want


def test_gumbel_sampling_follows_the_softmax():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0], dtype=torch.float64)
    counts = torch.zeros(4)
    n = 3000
    for c in range(n):
        counts[int(torch.argmax(plain.gumbel_scores(logits, 0.8, seed=42, counter=c)))] += 1
    want = torch.softmax(logits / 0.8, dim=0)
    assert (counts / n - want).abs().max() < 0.03
