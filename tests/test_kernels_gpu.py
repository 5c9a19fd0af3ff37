"""Each CUDA kernel alone against its plain PyTorch reference (float64 math on the same
inputs), at sizes other than the engine tests use: head sizes in steps of 16, odd head
counts and groups, widths and vocabularies that are no power of two, shuffled pages."""
import pytest
import torch

from helpers import assert_close, batch_to, clone_kv, paged_scenario
from torch_kernels import TorchKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL = {torch.float32: 2e-5, torch.bfloat16: 1e-2}
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def kernels():
    from kvcache_b200.kernels.api import CudaKernels
    return CudaKernels(DEV)


REF = TorchKernels(wide=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,V", [(1, 64, 100), (7, 896, 1531), (33, 120, 331)])
def test_embed(kernels, dtype, T, H, V):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(V, H, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    out = torch.empty(T, H, dtype=torch.float32, device=DEV)
    kernels.embed(table.to(DEV), ids.to(DEV), out)
    assert torch.equal(out.cpu(), table[ids.long()].float())


def test_embed_flags_bad_token(kernels):
    from kvcache_b200.kernels.api import KernelError
    table = torch.randn(10, 16, device=DEV)
    out = torch.empty(2, 16, device=DEV)
    kernels.embed(table, torch.tensor([3, 10], dtype=torch.int32, device=DEV), out)
    with pytest.raises(KernelError, match="token id"):
        kernels.check_errors()
    kernels.check_errors()   # the word was cleared


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,eps", [(1, 64, 1e-6), (5, 896, 1e-6), (19, 120, 1e-5), (3, 3584, 1e-6), (4, 50, 1e-3),
                                     (300, 896, 1e-6), (257, 5000, 1e-5), (261, 120, 1e-6),    # many rows, rows longer than the registers keep
                                     (259, 1536, 1e-6), (256, 2048, 1e-5), (300, 1028, 1e-6), (258, 516, 1e-6)])
def test_add_rmsnorm(kernels, dtype, T, H, eps):
    g = torch.Generator().manual_seed(1)
    h = torch.randn(T, H, generator=g) * 3
    delta = torch.randn(T, H, generator=g).to(dtype)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    for use_delta in (True, False):
        h_ref, out_ref = h.clone(), torch.empty(T, H, dtype=dtype)
        REF.add_rmsnorm(h_ref, delta if use_delta else None, w, eps, out_ref)
        h_dev, out = h.clone().to(DEV), torch.empty(T, H, dtype=dtype, device=DEV)
        kernels.add_rmsnorm(h_dev, delta.to(DEV) if use_delta else None, w.to(DEV), eps, out)
        assert_close(h_dev, h_ref, 1e-6, "residual stream")
        assert_close(out, out_ref, REL[dtype], "normalised rows")
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32)
    out_ref = torch.empty(3, H, dtype=dtype)
    REF.add_rmsnorm(h.clone(), delta, w, eps, out_ref, rows)
    h_dev, out = h.clone().to(DEV), torch.empty(3, H, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(h_dev, delta.to(DEV), w.to(DEV), eps, out, rows.to(DEV))
    assert torch.equal(h_dev.cpu(), h), "with rows the residual stream is left alone"
    assert_close(out, out_ref, REL[dtype], "gathered rows")
    if T >= 256:                                             # a long gather
        rows = torch.arange(T - 1, -1, -1, dtype=torch.int32)
        out_ref = torch.empty(T, H, dtype=dtype)
        REF.add_rmsnorm(h.clone(), delta, w, eps, out_ref, rows)
        h_dev, out = h.clone().to(DEV), torch.empty(T, H, dtype=dtype, device=DEV)
        kernels.add_rmsnorm(h_dev, delta.to(DEV), w.to(DEV), eps, out, rows.to(DEV))
        assert torch.equal(h_dev.cpu(), h)
        assert_close(out, out_ref, REL[dtype], "many gathered rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [896, 120, 1536, 2048, 516])
def test_add_rmsnorm_does_not_depend_on_the_row_count(kernels, dtype, H):
    """Launches of many rows take a kernel with a warp per row, launches of few rows one with a block per row; a row's
    numbers are the same bit for bit, so a prompt gives the same logits whole and in portions."""
    T = 300
    g = torch.Generator().manual_seed(4)
    h = (torch.randn(T, H, generator=g) * 3).to(DEV)
    delta = torch.randn(T, H, generator=g).to(dtype).to(DEV)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(DEV)
    h_all, out_all = h.clone(), torch.empty(T, H, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(h_all, delta, w, 1e-6, out_all)
    h_few, out_few = h.clone(), torch.empty(T, H, dtype=dtype, device=DEV)
    for a in range(0, T, 100):
        kernels.add_rmsnorm(h_few[a:a + 100], delta[a:a + 100], w, 1e-6, out_few[a:a + 100])
    assert torch.equal(h_all, h_few)
    assert torch.equal(out_all, out_few)
    rows = torch.arange(T - 1, -1, -1, dtype=torch.int32, device=DEV)
    gathered, few = torch.empty(T, H, dtype=dtype, device=DEV), torch.empty(T, H, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(h.clone(), delta, w, 1e-6, gathered, rows)
    for a in range(0, T, 100):
        kernels.add_rmsnorm(h.clone(), delta, w, 1e-6, few[a:a + 100], rows[a:a + 100])
    assert torch.equal(gathered, few)
    assert torch.equal(gathered.flip(0), out_all)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 128), (9, 4864), (31, 200), (2, 77)])
def test_silu_mul(kernels, dtype, T, I):
    gu = (torch.randn(T, 2 * I, generator=torch.Generator().manual_seed(2)) * 4).to(dtype)
    for interleaved in ([False, True] if I % 8 == 0 else [False]):
        ref = torch.empty(T, I, dtype=dtype)
        REF.silu_mul(gu, ref, interleaved)
        out = torch.empty(T, I, dtype=dtype, device=DEV)
        kernels.silu_mul(gu.to(DEV), out, interleaved)
        assert_close(out, ref, REL[dtype])


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                                (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (5, 331, 120), (70, 130, 77), (64, 1152, 896), (129, 64, 333)])
def test_gemm_simt(kernels, in_dtype, out_dtype, M, N, K):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).to(in_dtype)
    w = torch.randn(N, K, generator=g).to(in_dtype)
    bias = torch.randn(N, generator=g)
    for b in (None, bias):
        ref = torch.empty(M, N, dtype=out_dtype)
        REF.linear(x, w, ref, b)
        out = torch.empty(M, N, dtype=out_dtype, device=DEV)
        saved = kernels.bf16_gemm
        kernels.bf16_gemm = "simt"
        try:
            kernels.linear(x.to(DEV), w.to(DEV), out, b.to(DEV) if b is not None else None)
        finally:
            kernels.bf16_gemm = saved
        assert_close(out, ref, REL[out_dtype])


@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (3, 331, 96), (8, 1152, 896), (8, 896, 4864), (9, 40, 32), (16, 9728, 896),
                                   (17, 1000, 320), (33, 151936, 64), (64, 1152, 896), (64, 200, 4864), (5, 20000, 128),
                                   (2, 48, 1024), (5, 100, 736)])     # K over a cluster of 8; uneven shares of K
def test_gemm_skinny(kernels, request, M, N, K):
    g = torch.Generator().manual_seed(16)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    bias = torch.randn(N, generator=g)
    saved_rows = kernels.SKINNY_MAX_ROWS
    kernels.SKINNY_MAX_ROWS = 64
    request.addfinalizer(lambda: setattr(kernels, 'SKINNY_MAX_ROWS', saved_rows))
    assert kernels._skinny(torch.bfloat16, M, K)
    for out_dtype in (torch.bfloat16, torch.float32):
        for b in (None, bias):
            ref = torch.empty(M, N, dtype=out_dtype)
            REF.linear(x, w, ref, b)
            out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
            kernels.linear(x.to(DEV), w.to(DEV), out, b.to(DEV) if b is not None else None)
            assert_close(out, ref, REL[out_dtype])


@pytest.mark.parametrize("M,I,K", [(1, 128, 64), (8, 4864, 896), (13, 200, 96), (64, 320, 128), (70, 200, 120), (5, 77, 64)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_up_act(kernels, request, dtype, M, I, K):
    saved_rows = kernels.SKINNY_MAX_ROWS
    kernels.SKINNY_MAX_ROWS = 64
    request.addfinalizer(lambda: setattr(kernels, 'SKINNY_MAX_ROWS', saved_rows))
    """Gate/up projection with the activation: fused into the skinny kernel's output, or as
    library product + activation kernel; interleaved rows where the width allows."""
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.feedforward import GatedMLP
    g = torch.Generator().manual_seed(18)
    x = torch.randn(M, K, generator=g).to(dtype)
    wg, wu = torch.randn(I, K, generator=g).to(dtype), torch.randn(I, K, generator=g).to(dtype)
    gate, up = x.double() @ wg.double().t(), x.double() @ wu.double().t()
    want = gate / (1 + torch.exp(-gate)) * up
    name = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
    ffn = GatedMLP(K, I, activation="silu", prefix="m.", dtype=name)
    ffn.bind({"m.gate_proj.weight": wg, "m.up_proj.weight": wu, "m.down_proj.weight": torch.zeros(K, I)}, torch.device(DEV))
    assert ffn.interleaved == (I % 8 == 0)
    out = torch.full((M, I), float("nan"), dtype=dtype, device=DEV)
    kernels.gate_up_act(x.to(DEV), ffn.w_gate_up, out, Workspace(DEV), ffn.interleaved)
    # bfloat16: gate and up are rounded before the activation on the unfused path.
    assert_close(out, want, 2e-5 if dtype == torch.float32 else 2e-2)


def test_gemm_skinny_rows_do_not_depend_on_the_batch(kernels, request):
    saved_rows = kernels.SKINNY_MAX_ROWS
    kernels.SKINNY_MAX_ROWS = 64
    request.addfinalizer(lambda: setattr(kernels, 'SKINNY_MAX_ROWS', saved_rows))
    g = torch.Generator().manual_seed(17)
    x = torch.randn(64, 896, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(1152, 896, generator=g).to(torch.bfloat16).to(DEV)
    full = torch.empty(64, 1152, dtype=torch.bfloat16, device=DEV)
    kernels.linear(x, w, full)
    for M in (1, 7, 8, 20, 33):
        part = torch.empty(M, 1152, dtype=torch.bfloat16, device=DEV)
        kernels.linear(x[:M].contiguous(), w, part)
        assert torch.equal(part, full[:M]), M


TC_SHAPES = [(128, 128, 64), (128, 128, 128), (2048, 1152, 896), (300, 896, 4864), (17, 331, 120), (129, 130, 72),
             (1, 64, 8), (250, 9728, 896), (64, 151936, 896), (1000, 200, 200),
             (2048, 9728, 896), (2100, 9800, 904), (4096, 5000, 136),        # enough 256 x 256 tiles for two SMs per tile
             (2048, 4736, 200), (2048, 6144, 136), (4000, 2440, 264)]        # ... of 192 columns, of 256, of 192 with ragged edges


@pytest.mark.parametrize("M,N,K", [(17, 1152, 896), (64, 896, 4864), (100, 896, 896), (128, 1000, 320), (33, 331, 120),
                                   (40, 136, 72), (128, 200, 64), (31, 9728, 896), (65, 2560, 128)])
def test_gemm_wstream(kernels, request, M, N, K):
    """The weight-streaming tensor-memory product (17..128 rows) against float64 on the same bfloat16 inputs: K over
    a cluster of 1, 2, 4, 8 blocks, ragged N and K, every padded row count."""
    g = torch.Generator().manual_seed(31)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    bias = torch.randn(N, generator=g)
    saved = kernels.WSTREAM_MAX_ROWS
    kernels.WSTREAM_MAX_ROWS = 128                        # the kernel takes up to 128 rows; the engine gives it fewer
    request.addfinalizer(lambda: setattr(kernels, "WSTREAM_MAX_ROWS", saved))
    assert kernels._wstream(torch.bfloat16, M, K) and not kernels._skinny(torch.bfloat16, M, K)
    xd, wd = x.to(DEV), w.to(DEV)
    for out_dtype in (torch.bfloat16, torch.float32):
        for b in (None, bias):
            out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
            kernels.linear(xd, wd, out, b.to(DEV) if b is not None else None)
            kernels.check_errors()
            want = x.double() @ w.double().t() + (b.double() if b is not None else 0)
            assert_close(out, want, REL[out_dtype])
    # Rows do not depend on how many rows there are beside them.
    full = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels.linear(xd, wd, full)
    part = torch.empty(17, N, dtype=torch.bfloat16, device=DEV)
    kernels.linear(xd[:17].contiguous(), wd, part)
    assert torch.equal(part, full[:17])


@pytest.mark.parametrize("M,I,K", [(17, 64, 64), (64, 4864, 896), (128, 200, 120), (50, 4872, 200)])
def test_gemm_wstream_gated(kernels, request, M, I, K):
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.feedforward import GatedMLP
    saved = kernels.WSTREAM_MAX_ROWS
    kernels.WSTREAM_MAX_ROWS = 128
    request.addfinalizer(lambda: setattr(kernels, "WSTREAM_MAX_ROWS", saved))
    g = torch.Generator().manual_seed(32)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    wg, wu = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16), (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    gate, up = x.double() @ wg.double().t(), x.double() @ wu.double().t()
    want = gate / (1 + torch.exp(-gate)) * up
    ffn = GatedMLP(K, I, activation="silu", prefix="m.", dtype="bfloat16")
    ffn.bind({"m.gate_proj.weight": wg, "m.up_proj.weight": wu, "m.down_proj.weight": torch.zeros(K, I)}, torch.device(DEV))
    assert ffn.interleaved and kernels._wstream(torch.bfloat16, M, K)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gate_up_act(x.to(DEV), ffn.w_gate_up, out, Workspace(DEV), ffn.interleaved)
    kernels.check_errors()
    assert_close(out, want, 1e-2)


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tcgen05(M, N, K):
    """The tensor-memory kernel against float64 on the same bfloat16 inputs: whole tiles, ragged edges in M, N
    and K, one row, many K blocks (more than the ring has stages)."""
    from kvcache_b200.kernels.api import CudaKernels
    k = CudaKernels(DEV, bf16_gemm="tcgen05")
    k.skinny_gemm = False
    g = torch.Generator().manual_seed(19)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    bias = torch.randn(N, generator=g)
    xd, wd = x.to(DEV), w.to(DEV)
    for out_dtype in (torch.bfloat16, torch.float32):
        for b in (None, bias):
            if N > 100000 and b is not None:
                continue
            out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
            assert k._tcgen05(xd, wd, out)
            k.linear(xd, wd, out, b.to(DEV) if b is not None else None)
            k.check_errors()
            want = x.double() @ w.double().t() + (b.double() if b is not None else 0)
            assert_close(out, want, REL[out_dtype])


@pytest.mark.parametrize("M,I,K", [(128, 64, 64), (300, 4864, 896), (77, 200, 120), (2048, 320, 96), (2048, 4864, 896),
                                   (2500, 4872, 200), (2048, 2368, 136), (2048, 3072, 72)])    # tiles of 224, 224, 192 and 256 columns
def test_gemm_tcgen05_gated(M, I, K):
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.kernels.api import CudaKernels
    from kvcache_b200.parts.feedforward import GatedMLP
    k = CudaKernels(DEV, bf16_gemm="tcgen05")
    k.skinny_gemm = False
    g = torch.Generator().manual_seed(20)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    wg, wu = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16), (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    gate, up = x.double() @ wg.double().t(), x.double() @ wu.double().t()
    want = gate / (1 + torch.exp(-gate)) * up
    ffn = GatedMLP(K, I, activation="silu", prefix="m.", dtype="bfloat16")
    ffn.bind({"m.gate_proj.weight": wg, "m.up_proj.weight": wu, "m.down_proj.weight": torch.zeros(K, I)}, torch.device(DEV))
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gate_up_act(x.to(DEV), ffn.w_gate_up, out, Workspace(DEV), ffn.interleaved)
    k.check_errors()
    assert_close(out, want, 1e-2)


@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (8, 1152, 896), (70, 136, 80), (200, 331, 120)])
def test_linear_bf16_library(kernels, M, N, K):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    for out_dtype in (torch.bfloat16, torch.float32):
        ref = torch.empty(M, N, dtype=out_dtype)
        REF.linear(x, w, ref)
        out = torch.empty(M, N, dtype=out_dtype, device=DEV)
        saved = kernels.skinny_gemm, kernels.bf16_gemm
        kernels.skinny_gemm, kernels.bf16_gemm = False, "cublas"
        try:
            kernels.linear(x.to(DEV), w.to(DEV), out)
        finally:
            kernels.skinny_gemm, kernels.bf16_gemm = saved
        assert_close(out, ref, REL[out_dtype])


SCENARIOS = [
    # (segments (cached, new), Hq, Hkv, D, page, window)
    ([(0, 5)], 4, 2, 16, 16, None),
    ([(0, 40), (17, 1), (63, 2)], 6, 2, 48, 8, None),
    ([(130, 1), (0, 33), (31, 1), (200, 3)], 14, 2, 64, 16, None),
    ([(300, 1)], 3, 1, 32, 8, None),
    ([(0, 70), (90, 1), (41, 6)], 8, 8, 80, 16, 25),
    ([(515, 2), (127, 1)], 5, 1, 128, 32, 128),
    ([(0, 9)], 2, 2, 256, 4, None),
]
# Steps of many rows take the kernel that handles four rows per block (a count of rows that four does not divide).
ROPE_SCENARIOS = SCENARIOS + [([(40, 301), (3, 1), (0, 61)], 6, 2, 64, 16, None), ([(0, 258)], 3, 1, 48, 8, 100)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("scenario", ROPE_SCENARIOS)
def test_qkv_rope_append(kernels, dtype, scenario):
    segments, Hq, Hkv, D, page, window = scenario
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=dtype, device="cpu",
                               window=window, seed=5)
    T = batch.num_tokens
    g = torch.Generator().manual_seed(6)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g).to(dtype)
    bias = torch.randn((Hq + 2 * Hkv) * D, generator=g)
    from kvcache_b200.parts.position import RotaryHalf
    rope = RotaryHalf(D, 10000.0, 1024)
    rope.bind({}, torch.device("cpu"))
    rot = rope.rotation()
    for b in (bias, None):
        kv_ref, q_ref = clone_kv(kv), torch.empty(T, Hq * D, dtype=dtype)
        REF.qkv_rope_append(qkv, b, rot.cos, rot.sin, batch, kv_ref, q_ref, Hq)
        kv_dev, q_out = clone_kv(kv, DEV), torch.empty(T, Hq * D, dtype=dtype, device=DEV)
        kernels.qkv_rope_append(qkv.to(DEV), b.to(DEV) if b is not None else None, rot.cos.to(DEV), rot.sin.to(DEV),
                                batch_to(batch, DEV), kv_dev, q_out, Hq)
        assert_close(q_out, q_ref, REL[dtype], "queries")
        assert_close(kv_dev.k_pages, kv_ref.k_pages, REL[dtype], "key pages")
        assert_close(kv_dev.v_pages, kv_ref.v_pages, REL[dtype], "value pages")
    kernels.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("scenario", SCENARIOS)
def test_paged_attention_generic(kernels, dtype, scenario):
    segments, Hq, Hkv, D, page, window = scenario
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=dtype, device="cpu",
                               window=window, seed=7)
    T = batch.num_tokens
    q = torch.randn(T, Hq * D, generator=torch.Generator().manual_seed(8)).to(dtype)
    ref = torch.empty(T, Hq * D, dtype=dtype)
    REF.paged_attention(q, batch, kv, ref, Hq, D ** -0.5)
    out = torch.empty(T, Hq * D, dtype=dtype, device=DEV)
    kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), out, Hq, D ** -0.5)
    assert_close(out, ref, REL[dtype])
    kernels.check_errors()


FLASH_SCENARIOS = SCENARIOS[:6] + [
    ([(4000, 1), (64, 1), (63, 1), (0, 1), (129, 1)], 14, 2, 64, 16, None),     # decode only, split over the keys
    ([(0, 200), (300, 130), (1000, 1)], 14, 2, 64, 16, None),                   # several tiles per segment
    ([(0, 150), (700, 1), (90, 70)], 4, 4, 96, 8, 33),                          # window shorter than a key tile
    ([(2500, 1), (100, 1)], 16, 1, 128, 64, 1000),                              # group of 16, large pages
    ([(50, 3), (64, 2)], 2, 1, 112, 16, None),
    ([(0, 1500), (3000, 70)], 6, 2, 64, 16, None),                              # long tiles cut into units and merged
    ([(900, 700)], 4, 1, 64, 32, 300),                                          # units of a windowed layer: some hold no keys
    ([(1000, 1), (70, 2), (5, 1), (2047, 1)], 8, 2, 64, 8, 200),                # decode by TMA: small pages, a window that gave pages back
    ([(777, 1), (3000, 1), (15, 1)], 8, 4, 128, 32, None),                      # decode by TMA: head size 128, splits without keys
    ([(130, 1), (64, 2)], 3, 3, 64, 64, 100),                                   # decode by TMA: a page is a whole key tile
]


@pytest.mark.parametrize("scenario", FLASH_SCENARIOS)
def test_paged_attention_flash(kernels, request, scenario):
    from kvcache_b200.engine.workspace import Workspace
    segments, Hq, Hkv, D, page, window = scenario
    dtype = torch.bfloat16
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=dtype, device="cpu",
                               window=window, seed=12)
    T = batch.num_tokens
    q = torch.randn(T, Hq * D, generator=torch.Generator().manual_seed(13)).to(dtype)
    ref = torch.empty(T, Hq * D, dtype=dtype)
    REF.paged_attention(q, batch, kv, ref, Hq, D ** -0.5)
    if window:                                           # as the cache manager does: pages behind the window are not held
        for i, (cached, new) in enumerate(segments):
            kv.block_table[i, :max(0, cached - window + 1) // page] = -1
    ws = Workspace(DEV)
    saved_tc = kernels.tc_attention_min_rows
    kernels.tc_attention_min_rows = None                 # this test is about the mma.sync kernels
    request.addfinalizer(lambda: setattr(kernels, "tc_attention_min_rows", saved_tc))
    saved = (kernels.decode_merge, kernels.decode_ctas_wanted, kernels.decode_min_tiles)
    request.addfinalizer(lambda: [setattr(kernels, n, v) for n, v in
                                  zip(("decode_merge", "decode_ctas_wanted", "decode_min_tiles"), saved)])
    for merge in ("tma", "cluster", "ticket"):           # the splits as a cluster (keys by TMA, or by cp.async), or through scratch
        kernels.decode_merge = merge
        # default; one split; as many as allowed; a number of splits that does not divide the rows
        for wanted, min_tiles in ((saved[1], saved[2]), (3, 4), (100000, 1), (5 * len(segments) * Hkv, 1)):
            kernels.decode_ctas_wanted, kernels.decode_min_tiles = wanted, min_tiles
            out = torch.full((T, Hq * D), float("nan"), dtype=dtype, device=DEV)
            kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), out, Hq, D ** -0.5, ws)
            assert_close(out, ref, REL[dtype], f"decode_merge={merge} decode_ctas_wanted={wanted}")
    for name in ("attn.decode_tickets", "attn.prefill_tickets"):
        if name in ws._buffers:
            assert int(ws._buffers[name].sum()) == 0, name
    kernels.check_errors()


FUSED_DECODE_SCENARIOS = [
    # (cached tokens of each request (each brings one more), Hq, Hkv, D, page, window, rotated dimensions)
    ([4000, 64, 63, 0, 129, 127, 128], 14, 2, 64, 16, None, 64),     # new keys first and last of a tile, of a page, of the cache
    ([1000, 5, 2047, 15, 16], 8, 2, 64, 8, 200, 32),                 # small pages, a window that gave pages back, half the head rotated
    ([777, 3000, 15, 63, 64], 8, 4, 128, 32, None, 128),             # head size 128, splits without keys
    ([130, 64, 0], 3, 3, 64, 64, 100, 0),                            # a page is a whole key tile; no rotation
    ([2500, 100], 16, 1, 128, 64, 1000, 96),                         # group of 16
]


@pytest.mark.parametrize("scenario", FUSED_DECODE_SCENARIOS)
def test_rope_append_attention_fused_decode(kernels, request, scenario):
    """Bias, rotation, append and attention of a decode step in one kernel, against the plain rotation + append followed
    by the plain attention: the attention's output, and the pages with the new keys and values in them."""
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.position import RotaryHalf
    cached, Hq, Hkv, D, page, window, rotated = scenario
    dtype = torch.bfloat16
    segments = [(c, 1) for c in cached]
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=dtype, device="cpu",
                               window=window, seed=21)
    T = batch.num_tokens
    g = torch.Generator().manual_seed(22)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g).to(dtype)
    bias = torch.randn((Hq + 2 * Hkv) * D, generator=g)
    cos = sin = None
    if rotated:
        rope = RotaryHalf(rotated, 10000.0, 4200)
        rope.bind({}, torch.device("cpu"))
        cos, sin = rope.rotation().cos, rope.rotation().sin
    if window:                                           # as the cache manager does: pages behind the window are not held
        for i, c in enumerate(cached):
            kv.block_table[i, :max(0, c - window + 1) // page] = -1
    ws = Workspace(DEV)
    saved = (kernels.decode_ctas_wanted, kernels.decode_min_tiles, kernels.fused_rope_min_requests)
    request.addfinalizer(lambda: [setattr(kernels, n, v) for n, v in
                                  zip(("decode_ctas_wanted", "decode_min_tiles", "fused_rope_min_requests"), saved)])
    kernels.fused_rope_min_requests = 1
    to = lambda t: None if t is None else t.to(DEV)
    for b in (bias, None):
        kv_ref, q_ref, ref = clone_kv(kv), torch.empty(T, Hq * D, dtype=dtype), torch.empty(T, Hq * D, dtype=dtype)
        REF.qkv_rope_append(qkv, b, cos, sin, batch, kv_ref, q_ref, Hq)
        REF.paged_attention(q_ref, batch, kv_ref, ref, Hq, D ** -0.5)
        for wanted, min_tiles in ((saved[0], saved[1]), (3, 4), (100000, 1), (5 * T * Hkv, 1)):
            kernels.decode_ctas_wanted, kernels.decode_min_tiles = wanted, min_tiles
            kv_dev = clone_kv(kv, DEV)
            out = torch.full((T, Hq * D), float("nan"), dtype=dtype, device=DEV)
            assert kernels.rope_append_attention(qkv.to(DEV), to(b), to(cos), to(sin), batch_to(batch, DEV), kv_dev, out, Hq,
                                                 D ** -0.5, ws)
            assert_close(out, ref, REL[dtype], f"attention, decode_ctas_wanted={wanted}")
            assert_close(kv_dev.k_pages, kv_ref.k_pages, REL[dtype], "key pages")
            assert_close(kv_dev.v_pages, kv_ref.v_pages, REL[dtype], "value pages")
    # what the kernel does not take is left to the two calls
    kv_dev = clone_kv(kv, DEV)
    kv_dev.writes = False
    assert not kernels.rope_append_attention(qkv.to(DEV), to(bias), to(cos), to(sin), batch_to(batch, DEV), kv_dev,
                                             torch.empty(T, Hq * D, dtype=dtype, device=DEV), Hq, D ** -0.5, ws)
    kernels.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_kernels_equal_the_references_own_numpy_attention(kernels, request, dtype):
    """ref/ref_attn.py of the reference (one query per head over 128 keys, eight heads with a kv head each; output
    committed under tests/golden): its keys and values laid into shuffled pages, the query as a decode step's only row.
    float32 through the generic kernel; bfloat16 through the TMA, cluster and ticket decode kernels."""
    from helpers import reference_attention_case
    from kvcache_b200.engine.workspace import Workspace
    q, K, V, want = reference_attention_case()
    H, S, D = K.shape
    for page in (16, 8):
        batch, kv = paged_scenario([(S - 1, 1)], num_kv_heads=H, head_dim=D, page_size=page, dtype=dtype, device="cpu", seed=3)
        for pos in range(S):
            slot = int(kv.block_table[0, pos // page])
            kv.k_pages[slot, :, pos % page, :] = K[:, pos, :].to(dtype)
            kv.v_pages[slot, :, pos % page, :] = V[:, pos, :].to(dtype)
        saved = kernels.decode_merge
        request.addfinalizer(lambda: setattr(kernels, "decode_merge", saved))
        for merge in (("tma", "cluster", "ticket") if dtype == torch.bfloat16 else (saved,)):
            kernels.decode_merge = merge
            out = torch.full((1, H * D), float("nan"), dtype=dtype, device=DEV)
            kernels.paged_attention(q.reshape(1, H * D).to(dtype).to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), out, H,
                                    D ** -0.5, Workspace(DEV))
            # float32: summation order only.  bfloat16: q, K, V, the probabilities and the output are rounded to 8 bits
            # of mantissa (rounding the inputs and the output alone gives 3.5e-3 here).
            assert_close(out.reshape(H, D), want, REL[dtype], f"page {page}, {merge}")
    kernels.check_errors()


TC_SCENARIOS = [
    # (segments (cached, new), Hq, Hkv, D, page, window, least key tiles of a unit)
    ([(0, 128)], 2, 1, 64, 16, None, 8),
    ([(0, 300)], 4, 2, 64, 16, None, 8),
    ([(0, 700), (100, 70), (515, 2)], 14, 2, 64, 16, None, 8),
    ([(1000, 130), (0, 64)], 4, 4, 128, 16, None, 8),
    ([(0, 520)], 3, 1, 128, 64, None, 8),
    ([(300, 400)], 6, 2, 64, 8, 150, 8),                    # window: pages behind it are not held
    ([(0, 257)], 2, 2, 64, 64, 64, 8),
    ([(0, 1100), (2000, 300)], 4, 2, 64, 16, None, 16),     # tiles cut into units over the keys and merged
    ([(0, 700), (100, 70)], 6, 2, 64, 32, None, 1),         # units of a single key tile
    ([(900, 700)], 4, 1, 128, 32, 300, 2),                  # units of a windowed layer: some hold no keys
    # one-row segments beside long ones: the tensor-memory kernel and the decode kernel in one call
    ([(700, 1), (100, 450), (30, 1), (2000, 1)], 14, 2, 64, 16, None, 16),
    ([(515, 1), (200, 400), (64, 1)], 12, 2, 128, 16, None, 16),
    ([(400, 1), (350, 390)], 7, 1, 64, 32, 300, 16),
    # many more pieces of work than the GPU holds blocks: every block takes several from the queue, its pipeline's
    # bookkeeping running on from piece to piece (two blocks a SM at head size 64, one at 128)
    ([(0, 1500)], 14, 2, 64, 16, None, 1),
    ([(200, 900), (0, 130)], 8, 2, 128, 16, None, 1),
    ([(700, 1200)], 10, 2, 64, 16, 500, 2),
]


@pytest.mark.parametrize("scenario", TC_SCENARIOS)
def test_paged_attention_tc(kernels, request, scenario):
    """The tensor-memory prefill attention against float64 on the same bfloat16 inputs.  Pages behind a window
    are dropped from the block table, as the cache manager does, so the kernel must not touch them."""
    from kvcache_b200.engine.workspace import Workspace
    segments, Hq, Hkv, D, page, window, min_key_tiles = scenario
    dtype = torch.bfloat16
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=dtype, device="cpu",
                               window=window, seed=22, tc_min_key_tiles=min_key_tiles)
    T = batch.num_tokens
    q = torch.randn(T, Hq * D, generator=torch.Generator().manual_seed(23)).to(dtype)
    ref = torch.empty(T, Hq * D, dtype=dtype)
    REF.paged_attention(q, batch, kv, ref, Hq, D ** -0.5)
    if window:
        for i, (cached, new) in enumerate(segments):
            gone = max(0, cached - window + 1) // page
            kv.block_table[i, :gone] = -1
    saved = kernels.tc_attention_min_rows
    kernels.tc_attention_min_rows = 2
    request.addfinalizer(lambda: setattr(kernels, "tc_attention_min_rows", saved))
    ws = Workspace(DEV)
    rows = torch.arange(T)                                    # every row: segments of one row go through the decode kernel
    for _ in range(2):                                        # twice: the tickets of the first call must be zero again
        out = torch.full((T, Hq * D), float("nan"), dtype=dtype, device=DEV)
        kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), out, Hq, D ** -0.5, ws)
        kernels.check_errors()
        assert_close(out[rows], ref[rows], REL[dtype])
    if "attn.tc_tickets" in ws._buffers:
        assert int(ws._buffers["attn.tc_tickets"].sum()) == 0


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_paged_attention_random_shapes(kernels, request, seed):
    """Random mixes of segments (one token, a few, hundreds), group sizes, page sizes, windows and unit sizes through the
    tensor-memory prefill kernel and the TMA decode kernel, against float64 on the same bfloat16 inputs."""
    import random
    from kvcache_b200.engine.workspace import Workspace
    rng = random.Random(seed)
    saved = kernels.tc_attention_min_rows
    kernels.tc_attention_min_rows = 2
    request.addfinalizer(lambda: setattr(kernels, "tc_attention_min_rows", saved))
    ws = Workspace(DEV)
    for it in range(8):
        D, Hkv, G = rng.choice([64, 128]), rng.choice([1, 2, 4]), rng.choice([1, 2, 3, 7])
        page, window = rng.choice([8, 16, 32, 64]), rng.choice([None, None, rng.randint(40, 900)])
        segments = [(rng.randint(0, 1500), rng.choice([1, 2, rng.randint(2, 200), rng.randint(100, 900)]))
                    for _ in range(rng.randint(1, 4))]
        batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=torch.bfloat16, device="cpu",
                                   window=window, seed=100 * seed + it, tc_min_key_tiles=rng.choice([1, 2, 4, 16]))
        T, Hq = batch.num_tokens, Hkv * G
        q = torch.randn(T, Hq * D, generator=torch.Generator().manual_seed(it)).to(torch.bfloat16)
        ref = torch.empty(T, Hq * D, dtype=torch.bfloat16)
        REF.paged_attention(q, batch, kv, ref, Hq, D ** -0.5)
        if window:
            for i, (cached, new) in enumerate(segments):
                kv.block_table[i, :max(0, cached - window + 1) // page] = -1
        out = torch.full((T, Hq * D), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), out, Hq, D ** -0.5, ws)
        kernels.check_errors()
        assert_close(out, ref, REL[torch.bfloat16], f"{segments}, Hq {Hq}, Hkv {Hkv}, D {D}, page {page}, window {window}")


def test_flash_attention_sees_one_far_key_and_the_window_edge(kernels):
    """bfloat16 tensor-core path: a single key that takes all the weight is found among
    thousands (another page, another split); with a window it is seen at distance
    window - 1 and not at distance window."""
    from kvcache_b200.engine.workspace import Workspace
    Hq, Hkv, D, page = 4, 2, 64, 16
    ws = Workspace(DEV)
    for cached, far, window, seen in [(3000, 1234, None, True), (3000, 3000 - 99, 100, True), (3000, 3000 - 100, 100, False)]:
        batch, kv = paged_scenario([(cached, 1)], num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=torch.bfloat16,
                                   device="cpu", window=window, seed=14)
        q = torch.randn(1, Hq * D, generator=torch.Generator().manual_seed(15)).to(torch.bfloat16)
        p = int(kv.block_table[0, far // page])
        for hk in range(Hkv):
            qh = q.view(Hq, D)[hk * 2].float()
            kv.k_pages[p, hk, far % page] = (60.0 * qh / qh.norm() ** 2).to(torch.bfloat16)
            kv.v_pages[p, hk, far % page] = 7.0
        out = torch.empty(1, Hq * D, dtype=torch.bfloat16, device=DEV)
        kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), out, Hq, 1.0, ws)
        ref = torch.empty(1, Hq * D, dtype=torch.bfloat16)
        REF.paged_attention(q, batch, kv, ref, Hq, 1.0)
        assert_close(out, ref, 1e-2)
        got = out.view(Hq, D)[0].float().cpu()
        assert ((got - 7.0).abs().max() < 0.1) == seen


def test_attention_sees_one_far_key(kernels):
    """One key among hundreds, on another page, scaled so that it takes all the weight: the
    output must be that key's value."""
    Hq, Hkv, D, page = 4, 2, 32, 16
    batch, kv = paged_scenario([(700, 1)], num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=torch.float32,
                               device="cpu", seed=9)
    q = torch.randn(1, Hq * D, generator=torch.Generator().manual_seed(10))
    far = 37
    p = int(kv.block_table[0, far // page])
    for hk in range(Hkv):
        kv.k_pages[p, hk, far % page] = 40.0 * q.view(Hq, D)[hk * 2] / q.view(Hq, D)[hk * 2].norm()
    out = torch.empty(1, Hq * D, device=DEV)
    kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), out, Hq, 1.0)
    ref = torch.empty(1, Hq * D)
    REF.paged_attention(q, batch, kv, ref, Hq, 1.0)
    assert_close(out, ref, 2e-5)
    got = out.view(Hq, D)[0].cpu()
    assert (got - kv.v_pages[p, 0, far % page]).abs().max() < 1e-3


@pytest.mark.parametrize("R,V", [(1, 256), (3, 331), (5, 151936), (64, 4099)])
def test_sample(kernels, R, V):
    from plain_qwen2 import gumbel_scores
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(R, V, generator=g)
    logits[0, V // 2] = logits[0].max() + 1
    if V > 40:
        logits[0, 7] = logits[0, V // 2]           # a tie: the lowest index wins
    temperature = torch.tensor([0.0 if r % 2 == 0 else 0.7 for r in range(R)])
    seeds = torch.tensor([1234567890123 + r for r in range(R)], dtype=torch.int64)
    counters = torch.tensor([r * 3 for r in range(R)], dtype=torch.int32)
    parts = kernels.sample_parts(V)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    kernels.sample(logits.to(DEV), temperature.to(DEV), seeds.to(DEV), counters.to(DEV), out,
                   torch.empty(R * parts, device=DEV), torch.empty(R * parts, dtype=torch.int32, device=DEV))
    out = out.cpu()
    for r in range(min(R, 6)):
        if temperature[r] == 0:
            assert int(out[r]) == int(torch.argmax(logits[r])) or logits[r, out[r]] == logits[r].max()
            assert int(out[r]) == int((logits[r] == logits[r].max()).nonzero()[0])
        elif V <= 5000:
            scores = gumbel_scores(logits[r], 0.7, int(seeds[r]), int(counters[r]))
            assert scores[int(out[r])] >= scores.max() - 1e-4


def test_a_wait_that_runs_out_reaches_the_host_as_an_error(kernels):
    """Every mbarrier wait of the TMA and tensor-memory kernels is bounded.  A kernel whose wait cannot end (nothing
    arrives on its barrier) gives up after its poll limit, sets the time-out bit of the error word and returns: the host
    reads the error, and the device goes on working."""
    from kvcache_b200.kernels.api import KernelError
    kernels.check_errors()
    polls = kernels.probe_wait_timeout()
    assert 0 < polls < 1 << 20
    with pytest.raises(KernelError, match="a wait inside a kernel ran out"):
        kernels.check_errors()
    kernels.check_errors()                                    # read and cleared: the next check is clean
    x = torch.randn(4, 64, device=DEV).to(torch.bfloat16)
    w = torch.randn(32, 64, device=DEV).to(torch.bfloat16)
    out = torch.empty(4, 32, dtype=torch.bfloat16, device=DEV)
    kernels.linear(x, w, out)                                 # the context is as usable as before
    assert_close(out, x.float() @ w.float().t(), 2e-2)
    kernels.check_errors()


# ---- the folded forms of the register product (decode steps of up to 16 rows) -------------------------------------------

FOLD_SHAPES = [(1, 96), (5, 896), (8, 1536), (13, 224), (16, 896)]      # (rows, width)


@pytest.mark.parametrize("M,K", FOLD_SHAPES)
def test_norm_folded_into_the_gated_product(kernels, M, K):
    """out = silu(g) * u with [g | u] = rmsnorm(x) . W^T, the norm applied inside the product: against the norm, the
    product and the activation one after the other in float64."""
    g = torch.Generator().manual_seed(40 + M)
    I = 136 if K < 500 else 1216
    x16 = (torch.randn(M, K, generator=g) * 2).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=g) * 0.05).to(torch.bfloat16)
    norm_w, eps = 1 + 0.1 * torch.randn(K, generator=g), 1e-5
    normed = torch.empty(M, K, dtype=torch.float64)
    REF.add_rmsnorm(x16.float(), None, norm_w, eps, normed)
    want = torch.empty(M, I, dtype=torch.float64)
    REF.gate_up_act(normed, w.double(), want, None, True)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.norm_gate_up_act(x16.to(DEV), w.to(DEV), norm_w.to(DEV), eps, out)
    assert_close(out, want, REL[torch.bfloat16])
    kernels.check_errors()


@pytest.mark.parametrize("M,K", FOLD_SHAPES)
def test_product_added_into_the_residual_stream(kernels, M, K):
    """h += x . W^T and h16 = bfloat16(h) inside the product, for a weight with few rows (K split over a cluster) and
    one with many."""
    g = torch.Generator().manual_seed(50 + M)
    for N in (K, 4 * K if K < 500 else 1152):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
        h = torch.randn(M, N, generator=g) * 3
        want = h.double() + x.double() @ w.double().t()
        h_dev, h16 = h.clone().to(DEV), torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.linear_into_residual(x.to(DEV), w.to(DEV), h_dev, h16)
        assert_close(h_dev, want, 1e-5, f"residual stream, N={N}")          # float32 sums, float32 add
        assert torch.equal(h16, h_dev.to(torch.bfloat16)), "the rounded copy is the stream's own rounding"
    kernels.check_errors()


FOLD_QKV = [
    # (segments (cached, new), Hq, Hkv, D, page, width)
    ([(130, 1), (31, 1), (200, 1), (0, 1), (15, 1), (16, 1), (4095, 1), (77, 1)], 14, 2, 64, 16, 896),
    ([(300, 1)], 3, 1, 32, 8, 96),
    ([(5, 1), (63, 1), (64, 1)], 12, 2, 128, 32, 1536),
    ([(0, 3), (40, 2), (9, 1)], 4, 4, 16, 4, 224),                       # short portions take the same path
    ([(i * 7, 1) for i in range(16)], 6, 2, 48, 16, 288),
]


@pytest.mark.parametrize("rotate", [True, False])
@pytest.mark.parametrize("scenario", FOLD_QKV)
def test_norm_bias_rotation_and_append_folded_into_the_qkv_product(kernels, scenario, rotate):
    """The q/k/v projection of rmsnorm(x) with bias, rotation and append in one launch, from row-paired weights, against
    the norm, the product and `qkv_rope_append` one after the other on the weights in their natural order."""
    from kvcache_b200.kernels.api import CudaKernels
    from kvcache_b200.parts.position import RotaryHalf
    segments, Hq, Hkv, D, page, K = scenario
    dtype = torch.bfloat16
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=dtype, device="cpu", seed=61)
    T = batch.num_tokens
    g = torch.Generator().manual_seed(62)
    N = (Hq + 2 * Hkv) * D
    x16 = (torch.randn(T, K, generator=g) * 1.5).to(dtype)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
    bias = torch.randn(N, generator=g)
    norm_w, eps = 1 + 0.1 * torch.randn(K, generator=g), 1e-6
    cos = sin = None
    if rotate:
        rope = RotaryHalf(D, 1000000.0, 4200)
        rope.bind({}, torch.device("cpu"))
        cos, sin = rope.rotation().cos, rope.rotation().sin
    normed = torch.empty(T, K, dtype=torch.float64)
    REF.add_rmsnorm(x16.float(), None, norm_w, eps, normed)
    qkv = torch.empty(T, N, dtype=torch.float64)
    REF.linear(normed, w.double(), qkv)
    for b in (bias, None):
        kv_ref, q_ref = clone_kv(kv), torch.empty(T, Hq * D, dtype=dtype)
        REF.qkv_rope_append(qkv, b, cos, sin, batch, kv_ref, q_ref, Hq)
        order = CudaKernels.pair_rotation_rows(Hq + 2 * Hkv, D)
        kv_dev, q_out = clone_kv(kv, DEV), torch.full((T, Hq * D), float("nan"), dtype=dtype, device=DEV)
        to = lambda t: None if t is None else t.to(DEV)
        kernels.norm_qkv_rope_append(x16.to(DEV), w[order].contiguous().to(DEV), to(b[order].contiguous()) if b is not None else None,
                                     norm_w.to(DEV), eps, to(cos), to(sin), batch_to(batch, DEV), kv_dev, q_out, Hq)
        assert_close(q_out, q_ref, REL[dtype], "queries")
        assert_close(kv_dev.k_pages, kv_ref.k_pages, REL[dtype], "key pages")
        assert_close(kv_dev.v_pages, kv_ref.v_pages, REL[dtype], "value pages")
    # A call that only reads the cache another call wrote leaves the pages alone.
    kv_dev = clone_kv(kv, DEV)
    kv_dev.writes = False
    before = kv_dev.k_pages.clone()
    kernels.norm_qkv_rope_append(x16.to(DEV), w[order].contiguous().to(DEV), None, norm_w.to(DEV), eps, to(cos), to(sin),
                                 batch_to(batch, DEV), kv_dev, q_out, Hq)
    assert torch.equal(kv_dev.k_pages, before)
    kernels.check_errors()


def test_primitive_costs_probe(kernels):
    """The probe that the helper warps' layout rests on (csrc/primitive_costs.cu) runs to its end, flags nothing, and
    reports a cost for each primitive."""
    costs = kernels.primitive_costs()
    assert len(costs) == len(kernels.PRIMITIVE_NAMES)
    for name, clocks in costs.items():
        assert 1.0 < clocks < 20000.0, (name, clocks)
    kernels.check_errors()
