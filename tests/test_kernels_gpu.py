"""Each kernel alone against a plain PyTorch float32/float64 restatement of the same
operation, at sizes other than the engine's tiny models use."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P
from sampler_cases import CASES

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def K():
    from rustyllm_b200 import kernels
    return kernels


def _rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)


# ----------------------------------------------------------------------------- random weights
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mean", [0.0, 1.0])
def test_random_fill_gives_the_hosts_numbers_bit_for_bit(dtype, mean):
    from rustyllm_b200.weights.random_init import normal_values
    n, seed = 100003, (1 << 62) + 12345
    out = torch.empty(n, dtype=dtype, device=DEV)
    K().random_fill(out, seed, mean, 0.02)
    host = torch.from_numpy(normal_values(seed, n, mean, 0.02)).to(dtype)
    assert torch.equal(out.cpu(), host)


# ----------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_gathers_rows_and_flags_bad_ids(dtype):
    table = _rand(1000, 100, dtype=dtype)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 100, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    K().embedding(table, ids, out, flag)
    assert torch.equal(out, table[ids.long()].float()) and flag.item() == 0
    K().embedding(table, torch.tensor([1000], dtype=torch.int32, device=DEV), out[:1], flag)
    assert flag.item() == 1


@pytest.mark.parametrize("d", [7, 100, 4096, 5000])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(d, out_dtype):
    x = _rand(9, d, seed=1, scale=3.0)
    w = _rand(d, seed=2) + 1.0
    out = torch.empty(9, d, dtype=out_dtype, device=DEV)
    K().rmsnorm(x, w, out, 1e-6)
    ref = P.rms_norm(x.double().cpu(), w.double().cpu(), 1e-6)
    torch.testing.assert_close(out.double().cpu(), ref, **(dict(rtol=1e-2, atol=1e-2) if out_dtype == torch.bfloat16 else dict(rtol=2e-6, atol=2e-6)))
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, d, dtype=out_dtype, device=DEV)
    K().rmsnorm(x, w, out2, 1e-6, rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I", [172, 256, 14336])
def test_swiglu(dtype, I):
    gu = _rand(13, 2 * I, dtype=dtype, seed=3, scale=2.0)
    out = torch.empty(13, I, dtype=dtype, device=DEV)
    K().swiglu(gu, out)
    g, u = gu[:, :I].double().cpu(), gu[:, I:].double().cpu()
    torch.testing.assert_close(out.double().cpu(), P.swiglu(g, u), **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I", [100, 50, 51])
def test_swiglu_interleaved(dtype, I):
    gu = _rand(7, 2 * I, dtype=dtype, seed=3, scale=2.0)
    out = torch.empty(7, I, dtype=dtype, device=DEV)
    K().swiglu(gu, out, interleaved=True)
    torch.testing.assert_close(out.double().cpu(), P.swiglu(gu[:, 0::2].double().cpu(), gu[:, 1::2].double().cpu()), **_tol(dtype))


@pytest.mark.parametrize("M,N,K_,parts", [(1, 256, 128, 0), (8, 28672, 512, 0), (8, 1024, 4096, 8), (40, 400, 72, 0), (64, 512, 1024, 4),
                                          (300, 344, 264, 0), (17, 130, 104, 2), (100, 640, 2048, 0), (130, 344, 1024, 4),
                                          (256, 512, 512, 2)])
def test_gemm_tc_swiglu_epilogue(M, N, K_, parts):
    k = K()
    a = _rand(M, K_, dtype=torch.bfloat16, seed=24)
    w = _rand(N, K_, dtype=torch.bfloat16, seed=25, scale=0.1)
    bias = _rand(N, seed=26, scale=0.1)
    out = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gemm_tc(a, w, out, k.OUT_SWIGLU, bias, force_splits=parts)
    k.check_device_errors()
    y = a.double().cpu() @ w.double().cpu().T + bias.double().cpu()
    torch.testing.assert_close(out.double().cpu(), P.swiglu(y[:, 0::2], y[:, 1::2]), rtol=2e-2, atol=2e-2)


def test_convert_rounds_to_nearest_even():
    # SimonWaldherr/RustyLLM src/simd.rs:88-96 (f32_to_bf16) and its tests at 9203-9225
    x = torch.tensor([1.0, 1.00390625, 1.005859375, 1.01171875, -2.5, 3.0e38, 1e-40], device=DEV)
    out = torch.empty(7, dtype=torch.bfloat16, device=DEV)
    K().convert(x, out)
    assert torch.equal(out, x.to(torch.bfloat16))
    assert out[1].item() == 1.0 and out[3].item() == 1.015625   # ties go to the even mantissa
    back = torch.empty(7, device=DEV)
    K().convert(out, back)
    assert torch.equal(back, out.float())


# ----------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (3, 96, 96), (17, 130, 172), (64, 64, 64), (65, 300, 33),
                                    (200, 257, 100), (8, 1000, 256)])
def test_gemm_simt_all_modes(dtype, M, N, K_):
    k = K()
    a = _rand(M, K_, dtype=dtype, seed=4)
    w = _rand(N, K_, dtype=dtype, seed=5)
    bias = _rand(N, seed=6)
    ref = a.double().cpu() @ w.double().cpu().T
    tol = dict(rtol=1e-2, atol=1e-2 * math.sqrt(K_)) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=2e-5 * math.sqrt(K_))
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    k.gemm_simt(a, w, out, k.OUT_SAME)
    torch.testing.assert_close(out.double().cpu(), ref, **tol)
    out32 = torch.empty(M, N, device=DEV)
    k.gemm_simt(a, w, out32, k.OUT_F32, bias)
    torch.testing.assert_close(out32.double().cpu(), ref + bias.double().cpu(), rtol=1e-5, atol=2e-5 * math.sqrt(K_))
    res = _rand(M, N, seed=7)
    acc = res.clone()
    k.gemm_simt(a, w, acc, k.OUT_ADD_F32)
    torch.testing.assert_close(acc.double().cpu(), ref + res.double().cpu(), rtol=1e-5, atol=2e-5 * math.sqrt(K_))


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    k = K()
    a = _rand(130, 172, seed=8)
    w = _rand(96, 172, seed=9)
    full = torch.empty(130, 96, device=DEV)
    k.gemm_simt(a, w, full, k.OUT_F32)
    for rows in ([5], [0, 64, 129], list(range(20, 60))):
        sub = torch.empty(len(rows), 96, device=DEV)
        k.gemm_simt(a[rows].contiguous(), w, sub, k.OUT_F32)
        assert torch.equal(sub, full[rows]), "bit-equal whatever else is in the batch"
    # strided rows of A (a column block of a wider buffer)
    wide = _rand(10, 300, seed=10)
    sub = torch.empty(10, 96, device=DEV)
    k.gemm_simt(wide[:, 100:272], w, sub, k.OUT_F32)
    ref = torch.empty(10, 96, device=DEV)
    k.gemm_simt(wide[:, 100:272].contiguous(), w, ref, k.OUT_F32)
    assert torch.equal(sub, ref)


# ----------------------------------------------------------------------------- tensor-core GEMM
@pytest.mark.parametrize("M,N,K_", [(1, 128, 64), (1, 4096, 4096), (5, 96, 96), (16, 256, 128), (17, 130, 104),
                                    (33, 1000, 264), (64, 512, 1024), (100, 384, 4096), (129, 300, 72),
                                    (300, 2048, 512), (1000, 768, 320)])
def test_gemm_tc_all_modes(M, N, K_):
    k = K()
    a = _rand(M, K_, dtype=torch.bfloat16, seed=4)
    w = _rand(N, K_, dtype=torch.bfloat16, seed=5)
    bias = _rand(N, seed=6)
    assert k.gemm_tc_supported(a, w, None)
    ref = (a.float() @ w.float().T).double().cpu() if M * N * K_ > 1e8 else a.double().cpu() @ w.double().cpu().T
    scale = math.sqrt(K_)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    k.gemm_tc(a, w, out, k.OUT_SAME)
    torch.testing.assert_close(out.double().cpu(), ref, rtol=1e-2, atol=1e-2 * scale)
    out32 = torch.empty(M, N, device=DEV)
    k.gemm_tc(a, w, out32, k.OUT_F32, bias)
    torch.testing.assert_close(out32.double().cpu(), ref + bias.double().cpu(), rtol=1e-4, atol=2e-5 * scale * 4)
    res = _rand(M, N, seed=7)
    acc = res.clone()
    k.gemm_tc(a, w, acc, k.OUT_ADD_F32)
    torch.testing.assert_close(acc.double().cpu(), ref + res.double().cpu(), rtol=1e-4, atol=2e-5 * scale * 4)
    k.check_device_errors()
    # the same product on the CUDA cores agrees to float accumulation order
    simt = torch.empty(M, N, device=DEV)
    k.gemm_simt(a, w, simt, k.OUT_F32, bias)
    torch.testing.assert_close(out32, simt, rtol=1e-4, atol=2e-5 * scale * 4)


@pytest.mark.parametrize("M,N,K_", [(1, 4096, 4096), (8, 6144, 4096), (8, 4096, 14336), (8, 512, 512), (64, 1024, 4096),
                                    (33, 300, 1096), (16, 128, 256),
                                    # more than 64 tokens, few tiles: 128- and 256-token tiles in parts as well
                                    (128, 4096, 4096), (100, 520, 2048), (200, 640, 1096), (256, 256, 1024), (300, 1100, 640),
                                    (512, 4096, 4096), (700, 4096, 1024)])
def test_gemm_tc_split_k_is_deterministic_and_matches_the_unsplit_product(M, N, K_):
    k = K()
    a = _rand(M, K_, dtype=torch.bfloat16, seed=14)
    w = _rand(N, K_, dtype=torch.bfloat16, seed=15)
    bias = _rand(N, seed=16)
    res = _rand(M, N, seed=17)
    whole = res.clone()
    k.gemm_tc(a, w, whole, k.OUT_ADD_F32, bias, force_splits=1)
    runs = []
    for parts in (0, 0, 0, 2, 4, 8):
        o = res.clone()
        k.gemm_tc(a, w, o, k.OUT_ADD_F32, bias, force_splits=parts)
        runs.append(o)
    for o in runs[3:]:
        torch.testing.assert_close(o, whole, rtol=1e-4, atol=1e-4 * math.sqrt(K_))
    k.check_device_errors()
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])        # fixed order of the parts
    torch.testing.assert_close(runs[0], whole, rtol=1e-4, atol=1e-4 * math.sqrt(K_))
    ref = a.double().cpu() @ w.double().cpu().T + bias.double().cpu() + res.double().cpu()
    torch.testing.assert_close(runs[0].double().cpu(), ref, rtol=1e-4, atol=1e-4 * math.sqrt(K_))
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    k.gemm_tc(a, w, out, k.OUT_SAME)
    torch.testing.assert_close(out.double().cpu(), ref - bias.double().cpu() - res.double().cpu(), rtol=1e-2, atol=1e-2 * math.sqrt(K_))
    if (M, N, K_) in [(1, 4096, 4096), (8, 6144, 4096), (8, 4096, 14336), (128, 4096, 4096), (100, 520, 2048), (200, 640, 1096)]:
        assert k.gemm_tc_splits(M, N, K_) > 1
    if (M, N, K_) == (512, 4096, 4096):
        assert k.gemm_tc_splits(M, N, K_) == 2      # 64 tiles of 256 tokens: two parts fill most of the SMs
    if (M, N, K_) == (700, 4096, 1024):
        assert k.gemm_tc_splits(M, N, K_) == 1      # 96 tiles: the persistent kernel takes them whole


@pytest.mark.parametrize("M,N,K_,parts", [(8, 384, 512, 0), (8, 384, 512, 1), (5, 200, 256, 4), (40, 136, 192, 2),
                                          (64, 512, 1024, 8), (33, 264, 320, 0), (64, 520, 128, 1)])
def test_gemm_tc_starts_the_norm_of_the_updated_residual(M, N, K_, parts):
    """Add-into-residual epilogue with the next RMSNorm riding along: the residual times
    the norm weight in bf16, and the rows' sums of squares in pieces."""
    k = K()
    a = _rand(M, K_, dtype=torch.bfloat16, seed=31)
    w = _rand(N, K_, dtype=torch.bfloat16, seed=32, scale=0.2)
    bias = _rand(N, seed=33)
    g = (_rand(N, seed=34) * 0.3 + 1.0)
    res = _rand(M, N, seed=35, scale=3.0)
    out = res.clone()
    xg = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    sumsq = torch.full((M, k.norm_pieces(N)), float("nan"), device=DEV)
    k.gemm_tc(a, w, out, k.OUT_ADD_F32, bias, force_splits=parts, norm_weight=g, norm_out=xg, norm_sumsq=sumsq)
    k.check_device_errors()
    plain = res.clone()
    k.gemm_tc(a, w, plain, k.OUT_ADD_F32, bias, force_splits=parts)
    assert torch.equal(out, plain)                                   # the residual itself is what it was without the norm
    assert torch.equal(xg, (out * g).to(torch.bfloat16))             # float product, rounded once
    want = (out.double() ** 2).sum(1)
    torch.testing.assert_close(sumsq.double().sum(1), want, rtol=1e-5, atol=0)
    assert not torch.isnan(sumsq).any()


@pytest.mark.parametrize("mode", ["same", "f32", "add", "swiglu"])
@pytest.mark.parametrize("M,N,K_,parts", [(8, 384, 512, 0), (8, 384, 512, 1), (5, 200, 256, 4), (40, 136, 192, 2),
                                          (33, 264, 320, 0), (64, 520, 128, 1), (17, 4096, 4096, 0)])
def test_gemm_tc_finishes_a_norm_of_its_input(M, N, K_, parts, mode):
    """The input is x * norm weight; the epilogue multiplies row m by rsqrt(mean(x_m^2) + eps),
    the mean coming as sums of squares in pieces: the result is the product with RMSNorm(x)."""
    k = K()
    eps = 1e-3
    x = _rand(M, K_, seed=41, scale=5.0) * (1 + torch.arange(M, device=DEV).float()[:, None])    # rows of very different size
    g = _rand(K_, seed=42) * 0.3 + 1.0
    xg = (x * g).to(torch.bfloat16)
    w = _rand(N, K_, dtype=torch.bfloat16, seed=43, scale=0.2)
    bias = _rand(N, seed=44)
    pieces = 7
    cut = torch.rand(M, pieces, device=DEV) + 0.1
    sumsq = ((x.double() ** 2).sum(1, keepdim=True) * (cut / cut.sum(1, keepdim=True)).double()).float().contiguous()
    r = 1.0 / torch.sqrt((x.double().cpu() ** 2).mean(1, keepdim=True) + eps)
    y = (xg.double().cpu() @ w.double().cpu().T) * r + bias.double().cpu()
    res = _rand(M, N, seed=45)
    tol = dict(rtol=1e-4, atol=2e-5 * math.sqrt(K_) * 4)
    if mode == "same":
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        k.gemm_tc(xg, w, out, k.OUT_SAME, bias, force_splits=parts, row_sumsq=sumsq, row_eps=eps)
        torch.testing.assert_close(out.double().cpu(), y, rtol=1e-2, atol=1e-2)
    elif mode == "f32":
        out = torch.empty(M, N, device=DEV)
        k.gemm_tc(xg, w, out, k.OUT_F32, bias, force_splits=parts, row_sumsq=sumsq, row_eps=eps)
        torch.testing.assert_close(out.double().cpu(), y, **tol)
    elif mode == "add":
        out = res.clone()
        k.gemm_tc(xg, w, out, k.OUT_ADD_F32, bias, force_splits=parts, row_sumsq=sumsq, row_eps=eps)
        torch.testing.assert_close(out.double().cpu(), y + res.double().cpu(), **tol)
    else:
        if N % 2:
            pytest.skip("the SwiGLU epilogue needs an even number of rows")
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
        k.gemm_tc(xg, w, out, k.OUT_SWIGLU, bias, force_splits=parts, row_sumsq=sumsq, row_eps=eps)
        torch.testing.assert_close(out.double().cpu(), P.swiglu(y[:, 0::2], y[:, 1::2]), rtol=2e-2, atol=2e-2)
    k.check_device_errors()


def test_gemm_tc_strided_rows_and_refusals():
    k = K()
    # a norm rides along for up to 64 tokens only
    with pytest.raises(k.KernelError, match="up to 64 tokens"):
        k.gemm_tc(_rand(65, 64, dtype=torch.bfloat16), _rand(128, 64, dtype=torch.bfloat16), torch.empty(65, 128, device=DEV),
                  k.OUT_F32, row_sumsq=torch.ones(65, 4, device=DEV), row_eps=1e-5)
    wide = _rand(40, 640, dtype=torch.bfloat16, seed=8)
    w = _rand(200, 256, dtype=torch.bfloat16, seed=9)
    a = wide[:, 128:384]
    assert k.gemm_tc_supported(a, w, None)
    out = torch.empty(40, 200, device=DEV)
    k.gemm_tc(a, w, out, k.OUT_F32)
    torch.testing.assert_close(out.double().cpu(), a.double().cpu() @ w.double().cpu().T, rtol=1e-4, atol=1e-3)
    k.check_device_errors()
    # K = 172: rows of 344 bytes are no multiple of 16 bytes, TMA cannot address them
    assert not k.gemm_tc_supported(_rand(4, 172, dtype=torch.bfloat16), _rand(8, 172, dtype=torch.bfloat16), None)
    assert not k.gemm_tc_supported(wide[:, 4:260], w, None)      # base not 16-byte aligned
    with pytest.raises(k.KernelError, match="not supported"):
        k.gemm_tc(_rand(4, 172, dtype=torch.bfloat16), _rand(8, 172, dtype=torch.bfloat16),
                  torch.empty(4, 8, device=DEV), k.OUT_F32)


# ----------------------------------------------------------------------------- rope + cache write
def _paged(G, hd, n_pages, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    k_pool = torch.randn(n_pages, G, PAGE, hd, generator=g).to(dtype).to(DEV)   # stale contents on purpose
    v_pool = torch.randn(n_pages, G, PAGE, hd, generator=g).to(dtype).to(DEV)
    return k_pool, v_pool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,rot,interleaved", [(4, 2, 16, 16, False), (3, 1, 32, 32, True), (5, 5, 48, 24, False),
                                                    (8, 2, 128, 128, False), (2, 2, 256, 64, True), (6, 3, 80, 0, False)])
def test_rope_kv_write(dtype, H, G, hd, rot, interleaved):
    k = K()
    M = 11
    qkv = _rand(M, (H + 2 * G) * hd + 8, dtype=dtype, seed=11)[:, :(H + 2 * G) * hd + 8]   # padded row stride
    positions = torch.tensor([0, 1, 63, 64, 65, 200, 5, 6, 7, 130, 131], dtype=torch.int32, device=DEV)
    slot_of_token = torch.tensor([0, 0, 0, 0, 0, 0, 2, 2, 2, 2, 2], dtype=torch.int32, device=DEV)
    page_table = torch.tensor([[7, 3, 1, 9], [0, 0, 0, 0], [2, 8, 4, 5]], dtype=torch.int32, device=DEV)
    inv = torch.tensor([1.0 / (10000.0 ** (2 * i / max(rot, 2))) for i in range(max(rot // 2, 1))], device=DEV)
    k_pool, v_pool = _paged(G, hd, 10, dtype)
    k_before, v_before = k_pool.clone(), v_pool.clone()
    src = qkv.clone()
    k.rope_kv_write(qkv, positions, slot_of_token, page_table, inv, H, G, hd, rot, interleaved, k_pool, v_pool)

    x = src[:, :(H + 2 * G) * hd].double().cpu()
    q, kk, v = x[:, :H * hd].view(M, H, hd), x[:, H * hd:(H + G) * hd].view(M, G, hd), x[:, (H + G) * hd:].view(M, G, hd)
    if rot:
        sin, cos = P.rope_angles(positions.cpu(), inv.cpu())
        f = P.apply_rope_interleaved if interleaved else P.apply_rope_half
        q = torch.cat([f(q[..., :rot], sin, cos), q[..., rot:]], -1)
        kk = torch.cat([f(kk[..., :rot], sin, cos), kk[..., rot:]], -1)
    tol = _tol(dtype)
    torch.testing.assert_close(qkv[:, :H * hd].double().cpu().view(M, H, hd), q, **tol)
    touched = torch.zeros(10, PAGE, dtype=torch.bool)
    for m in range(M):
        p = int(positions[m]); page = int(page_table[int(slot_of_token[m]), p // PAGE]); off = p % PAGE
        touched[page, off] = True
        torch.testing.assert_close(k_pool[page, :, off].double().cpu(), kk[m], **tol)
        assert torch.equal(v_pool[page, :, off].double().cpu(), v[m])
    # nothing else in the pools moved
    keep = ~touched.to(DEV)
    assert torch.equal(k_pool.permute(0, 2, 1, 3)[keep], k_before.permute(0, 2, 1, 3)[keep])
    assert torch.equal(v_pool.permute(0, 2, 1, 3)[keep], v_before.permute(0, 2, 1, 3)[keep])


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("M,H,G,K_,normed,store", [(1, 3, 1, 1024, False, True), (8, 3, 1, 1024, True, True),
                                                  (11, 2, 2, 2048, False, True), (33, 4, 2, 512, True, True),
                                                  (11, 3, 1, 1024, False, False), (64, 32, 8, 2048, True, True)])
def test_gemm_tc_qkv_rope_is_the_product_then_the_rotation_and_the_cache_write(M, H, G, K_, normed, store, interleaved, hd):
    """The QKV product with rotation and cache write in its epilogue, against float64:
    product, (finished norm,) bias, rotation of query and key heads, keys and values at
    their tokens' places of the paged cache, nothing else in the pools touched."""
    k = K()
    N = (H + 2 * G) * hd              # head size 64: two heads a tile of 128 columns; 5 heads leave the last tile half empty
    x = _rand(M, K_, seed=51, scale=2.0)
    g = _rand(K_, seed=52) * 0.3 + 1.0
    a = (x * g).to(torch.bfloat16) if normed else x.to(torch.bfloat16)
    w = _rand(N, K_, dtype=torch.bfloat16, seed=53, scale=0.05)
    bias = _rand(N, seed=54, scale=0.5)
    assert k.gemm_tc_qkv_rope_supported(a, w, H, G, hd, hd)
    assert not k.gemm_tc_qkv_rope_supported(a, w, H, G, hd, hd // 2)     # partial rotation: the separate kernel
    positions = torch.tensor(([0, 1, 63, 64, 65, 200, 5, 6, 7, 130, 131] * 3 + list(range(31)))[:M], dtype=torch.int32, device=DEV)
    slot_of_token = torch.tensor(([0, 0, 0, 0, 0, 0, 2, 2, 2, 2, 2] + [1] * 11 + [3] * 11 + [4] * 31)[:M], dtype=torch.int32, device=DEV)
    page_table = torch.tensor([[7, 3, 1, 9], [10, 11, 12, 13], [2, 8, 4, 5], [14, 15, 16, 17], [0, 6, 6, 6]], dtype=torch.int32, device=DEV)
    inv = torch.tensor([1.0 / (10000.0 ** (2 * i / hd)) for i in range(hd // 2)], device=DEV)
    k_pool, v_pool = _paged(G, hd, 18, torch.bfloat16)
    k_before, v_before = k_pool.clone(), v_pool.clone()
    eps = 1e-5
    kw = {}
    y = a.double().cpu() @ w.double().cpu().T
    if normed:
        sumsq = ((x.double() ** 2).sum(1, keepdim=True) * torch.tensor([[0.25, 0.5, 0.25]], device=DEV).double()).float().contiguous()
        kw = dict(row_sumsq=sumsq, row_eps=eps)
        y = y / torch.sqrt((x.double().cpu() ** 2).mean(1, keepdim=True) + eps)
    y = y + bias.double().cpu()
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gemm_tc_qkv_rope(a, w, out, bias, positions, slot_of_token, page_table, inv, interleaved, H, G,
                       k_pool if store else None, v_pool if store else None, **kw)
    k.check_device_errors()
    q, kk, v = y[:, :H * hd].view(M, H, hd), y[:, H * hd:(H + G) * hd].view(M, G, hd), y[:, (H + G) * hd:].view(M, G, hd)
    sin, cos = P.rope_angles(positions.cpu(), inv.cpu())
    f = P.apply_rope_interleaved if interleaved else P.apply_rope_half
    q, kk = f(q, sin, cos), f(kk, sin, cos)
    tol = dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out[:, :H * hd].double().cpu().view(M, H, hd), q, **tol)
    if not store:
        assert torch.equal(k_pool, k_before) and torch.equal(v_pool, v_before)
        return
    touched = torch.zeros(18, PAGE, dtype=torch.bool)
    for m in range(M):
        p = int(positions[m]); page = int(page_table[int(slot_of_token[m]), p // PAGE]); off = p % PAGE
        touched[page, off] = True
        torch.testing.assert_close(k_pool[page, :, off].double().cpu(), kk[m], **tol)
        torch.testing.assert_close(v_pool[page, :, off].double().cpu(), v[m], **tol)
    keep = ~touched.to(DEV)
    assert torch.equal(k_pool.permute(0, 2, 1, 3)[keep], k_before.permute(0, 2, 1, 3)[keep])
    assert torch.equal(v_pool.permute(0, 2, 1, 3)[keep], v_before.permute(0, 2, 1, 3)[keep])


def _llama3_inv_freq(hd, factor):
    return P.rope_inv_freq(500000.0, hd, {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0,
                                          "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}).to(DEV)


FAR_POSITIONS = [0, 4095, 4096, 4223, 4224, 8191, 8192, 8703]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,factor,interleaved", [(8, 2, 128, 8.0, False), (8, 2, 64, 32.0, False), (3, 1, 128, 8.0, True)])
def test_rope_kv_write_at_positions_in_the_thousands(dtype, H, G, hd, factor, interleaved):
    """Positions up to 8,703 with the real models' rope constants: the angle is the float product
    pos * inv_freq, whose sine needs an accurate range reduction there, and the slot's page table
    is 137 entries long."""
    k = K()
    M = len(FAR_POSITIONS)
    qkv = _rand(M, (H + 2 * G) * hd, dtype=dtype, seed=21)
    positions = torch.tensor(FAR_POSITIONS, dtype=torch.int32, device=DEV)
    slot_of_token = torch.full((M,), 1, dtype=torch.int32, device=DEV)
    g = torch.Generator().manual_seed(5)
    page_table = torch.stack([torch.zeros(137, dtype=torch.int64), torch.randperm(140, generator=g)[:137]]).to(torch.int32).to(DEV)
    inv = _llama3_inv_freq(hd, factor)
    k_pool, v_pool = _paged(G, hd, 140, dtype)
    src = qkv.clone()
    k.rope_kv_write(qkv, positions, slot_of_token, page_table, inv, H, G, hd, hd, interleaved, k_pool, v_pool)
    x = src.double().cpu()
    q, kk, v = x[:, :H * hd].view(M, H, hd), x[:, H * hd:(H + G) * hd].view(M, G, hd), x[:, (H + G) * hd:].view(M, G, hd)
    sin, cos = P.rope_angles(positions.cpu(), inv.cpu())
    f = P.apply_rope_interleaved if interleaved else P.apply_rope_half
    q, kk = f(q, sin, cos), f(kk, sin, cos)
    tol = _tol(dtype)
    torch.testing.assert_close(qkv[:, :H * hd].double().cpu().view(M, H, hd), q, **tol)
    for m, p in enumerate(FAR_POSITIONS):
        page = int(page_table[1, p // PAGE]); off = p % PAGE
        torch.testing.assert_close(k_pool[page, :, off].double().cpu(), kk[m], **tol)
        assert torch.equal(v_pool[page, :, off].double().cpu(), v[m])


@pytest.mark.parametrize("interleaved", [False, True])
def test_gemm_tc_qkv_rope_at_positions_in_the_thousands(interleaved):
    k = K()
    H, G, hd, K_ = 4, 2, 128, 1024
    M = len(FAR_POSITIONS)
    N = (H + 2 * G) * hd
    a = _rand(M, K_, dtype=torch.bfloat16, seed=61, scale=1.0)
    w = _rand(N, K_, dtype=torch.bfloat16, seed=62, scale=0.05)
    assert k.gemm_tc_qkv_rope_supported(a, w, H, G, hd, hd)
    positions = torch.tensor(FAR_POSITIONS, dtype=torch.int32, device=DEV)
    slot_of_token = torch.full((M,), 1, dtype=torch.int32, device=DEV)
    g = torch.Generator().manual_seed(6)
    page_table = torch.stack([torch.zeros(137, dtype=torch.int64), torch.randperm(140, generator=g)[:137]]).to(torch.int32).to(DEV)
    inv = _llama3_inv_freq(hd, 8.0)
    k_pool, v_pool = _paged(G, hd, 140, torch.bfloat16)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gemm_tc_qkv_rope(a, w, out, None, positions, slot_of_token, page_table, inv, interleaved, H, G, k_pool, v_pool)
    k.check_device_errors()
    y = a.double().cpu() @ w.double().cpu().T
    q, kk, v = y[:, :H * hd].view(M, H, hd), y[:, H * hd:(H + G) * hd].view(M, G, hd), y[:, (H + G) * hd:].view(M, G, hd)
    sin, cos = P.rope_angles(positions.cpu(), inv.cpu())
    f = P.apply_rope_interleaved if interleaved else P.apply_rope_half
    q, kk = f(q, sin, cos), f(kk, sin, cos)
    tol = dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out[:, :H * hd].double().cpu().view(M, H, hd), q, **tol)
    for m, p in enumerate(FAR_POSITIONS):
        page = int(page_table[1, p // PAGE]); off = p % PAGE
        torch.testing.assert_close(k_pool[page, :, off].double().cpu(), kk[m], **tol)
        torch.testing.assert_close(v_pool[page, :, off].double().cpu(), v[m], **tol)


# ----------------------------------------------------------------------------- attention
def _attention_case(dtype, H, G, hd, lens_q, lens_kv, window=0, seed=0, craft=None):
    """Builds a paged cache with scrambled pages for sequences of lens_kv tokens; the
    last lens_q[b] tokens of each are the step's queries.  Returns inputs and the
    plain float64 result."""
    B = len(lens_kv)
    g = torch.Generator().manual_seed(seed)
    n_pages_each = [-(-n // PAGE) for n in lens_kv]
    total_pages = sum(n_pages_each) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    max_pages = max(n_pages_each) + 1
    page_table = torch.full((B + 1, max_pages), 0, dtype=torch.int32)
    k_pool = (torch.randn(total_pages, G, PAGE, hd, generator=g) * 3).to(dtype)   # stale values, large
    v_pool = (torch.randn(total_pages, G, PAGE, hd, generator=g) * 3).to(dtype)
    slots = list(range(B, 0, -1))      # slots in reverse order
    ks, vs, qs = [], [], []
    pi = 0
    for b in range(B):
        n = lens_kv[b]
        kb = torch.randn(n, G, hd, generator=g).to(dtype)
        vb = torch.randn(n, G, hd, generator=g).to(dtype)
        qb = torch.randn(lens_q[b], H, hd, generator=g).to(dtype)
        if craft is not None:
            craft(b, qb, kb, vb)
        for p in range(n_pages_each[b]):
            page = perm[pi]; pi += 1
            page_table[slots[b], p] = page
            lo, hi = p * PAGE, min(n, (p + 1) * PAGE)
            k_pool[page, :, :hi - lo] = kb[lo:hi].transpose(0, 1)
            v_pool[page, :, :hi - lo] = vb[lo:hi].transpose(0, 1)
        ks.append(kb); vs.append(vb); qs.append(qb)
    positions, slot_of_token, refs = [], [], []
    for b in range(B):
        n, nq = lens_kv[b], lens_q[b]
        full_q = torch.zeros(n, H, hd, dtype=torch.float64)
        full_q[n - nq:] = qs[b].double()
        out = P.causal_attention(full_q, ks[b].double(), vs[b].double(), window=window or None)
        refs.append(out[n - nq:].reshape(nq, H * hd))
        positions += list(range(n - nq, n))
        slot_of_token += [slots[b]] * nq
    q = torch.cat([x.reshape(x.shape[0], H * hd) for x in qs]).to(DEV)
    return (q, k_pool.to(DEV), v_pool.to(DEV), page_table.to(DEV),
            torch.tensor(slot_of_token, dtype=torch.int32, device=DEV),
            torch.tensor(positions, dtype=torch.int32, device=DEV), torch.cat(refs))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd", [(4, 2, 16), (3, 1, 32), (5, 5, 48), (8, 2, 64), (6, 2, 80), (8, 1, 128), (2, 2, 256), (7, 7, 112)])
def test_attention_simt_prefill_and_decode_shapes(dtype, H, G, hd):
    k = K()
    for lens_q, lens_kv in (([1, 1, 1], [1, 64, 200]), ([5, 70, 1, 33], [5, 70, 129, 97]), ([130], [130])):
        q, kp, vp, pt, sot, pos, ref = _attention_case(dtype, H, G, hd, lens_q, lens_kv, seed=hd + len(lens_q))
        out = torch.empty(q.shape[0], H * hd, dtype=dtype, device=DEV)
        k.attention_simt(q, kp, vp, pt, sot, pos, out, H, G, hd, 1.0 / math.sqrt(hd))
        torch.testing.assert_close(out.double().cpu(), ref, **(_tol(dtype) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_simt_window(dtype):
    k = K()
    H, G, hd, W = 4, 2, 32, 70
    q, kp, vp, pt, sot, pos, ref = _attention_case(dtype, H, G, hd, [40, 1, 150], [40, 300, 150], window=W, seed=3)
    out = torch.empty(q.shape[0], H * hd, dtype=dtype, device=DEV)
    k.attention_simt(q, kp, vp, pt, sot, pos, out, H, G, hd, 1.0 / math.sqrt(hd), W)
    torch.testing.assert_close(out.double().cpu(), ref, **(_tol(dtype) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far", [0, 63, 64, 449, 450])
def test_attention_finds_one_far_key_among_hundreds(dtype, far):
    """One key is made to stand out (query and key scaled so that its score dominates):
    the output must be that key's value, wherever in the pages it lies."""
    H, G, hd, n = 4, 2, 64, 451

    def craft(b, qb, kb, vb):
        direction = torch.ones(hd) / math.sqrt(hd)
        qb[:] = (direction * 12.0).to(qb.dtype)          # every head asks for the same direction
        kb[:] = (kb.float() * 0.05).to(kb.dtype)
        kb[far] = (direction * 12.0).to(kb.dtype)        # score 144/8 = 18 against ~0 elsewhere
    q, kp, vp, pt, sot, pos, ref = _attention_case(dtype, H, G, hd, [1], [n], seed=5, craft=craft)
    out = torch.empty(1, H * hd, dtype=dtype, device=DEV)
    K().attention_simt(q, kp, vp, pt, sot, pos, out, H, G, hd, 1.0 / math.sqrt(hd))
    torch.testing.assert_close(out.double().cpu(), ref, **(_tol(dtype) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)))
    # and the plain result is, to 1e-4, the far key's value: the test would notice a missed key
    page = int(pt[1, far // PAGE]); v_far = vp[page, :, far % PAGE].double().cpu()   # [G, hd]
    want = v_far.repeat_interleave(H // G, dim=0).reshape(1, H * hd)
    assert (ref - want).abs().max() < 1e-3


# ----------------------------------------------------------------------------- decode attention (tensor cores)
def _decode_inputs(case):
    q, kp, vp, pt, sot, pos, ref = case
    return q, kp, vp, pt, sot.clone(), (pos + 1).to(torch.int32), ref


@pytest.mark.parametrize("H,G,hd", [(32, 8, 128), (8, 8, 128), (6, 2, 64), (16, 1, 64), (5, 5, 128), (24, 8, 64)])
@pytest.mark.parametrize("splits", [1, 2, 7, 32])
@pytest.mark.parametrize("planned", [False, True])
def test_attention_decode_matches_plain(H, G, hd, splits, planned):
    """``planned``: the chunks are dealt to the sequences by length (as the engine does
    for a batch); otherwise every sequence is cut into ``splits`` equal chunks."""
    k = K()
    assert k.attention_decode_supported(torch.bfloat16, H, G, hd)
    lens = [1, 15, 16, 17, 64, 65, 200, 513]
    case = _attention_case(torch.bfloat16, H, G, hd, [1] * len(lens), lens, seed=hd + H + splits)
    q, kp, vp, pt, slots, kv_lens, ref = _decode_inputs(case)
    out = torch.empty(len(lens), H * hd, dtype=torch.bfloat16, device=DEV)
    plan = k.decode_plan(slots, kv_lens, 0, splits) if planned else None
    assert (plan is not None) == (planned and splits > 1)
    k.attention_decode(q, kp, vp, pt, slots, kv_lens, out, H, G, hd, 1.0 / math.sqrt(hd), num_splits=splits, plan=plan)
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))
    # and the any-shape kernel gives the same to bf16 rounding
    simt = torch.empty_like(out)
    k.attention_simt(q, kp, vp, pt, slots, (kv_lens - 1).to(torch.int32), simt, H, G, hd, 1.0 / math.sqrt(hd))
    torch.testing.assert_close(out.float(), simt.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("H,G,hd", [(32, 8, 128), (6, 2, 64), (16, 1, 128)])
@pytest.mark.parametrize("splits", [2, 4, 8])
def test_attention_decode_chunks_of_a_sequence_as_a_cluster(H, G, hd, splits):
    """No scratch, one kernel: the chunks' CTAs combine through distributed shared memory."""
    k = K()
    lens = [1, 15, 64, 65, 200, 513, 1100]
    for window in (0, 90):
        case = _attention_case(torch.bfloat16, H, G, hd, [1] * len(lens), lens, window=window, seed=hd + splits)
        q, kp, vp, pt, slots, kv_lens, ref = _decode_inputs(case)
        out = torch.full((len(lens), H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        before = k.launch_count
        k.attention_decode(q, kp, vp, pt, slots, kv_lens, out, H, G, hd, 1.0 / math.sqrt(hd), window, num_splits=splits, cluster=True)
        assert k.launch_count - before == 1
        torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))


@pytest.mark.parametrize("H,G,hd", [(32, 8, 128), (6, 2, 64)])
def test_attention_decode_whole_sequences_longest_first(H, G, hd):
    """Every sequence whole in one CTA a KV head, started in the order of their lengths (inside the
    window): the order plan lists the sequences longest first, ties in the order of the batch, and
    the answers are those of the batch's own order."""
    k = K()
    lens = [1 + (i * 131) % 700 for i in range(70)] + [1500, 64, 64, 1]
    for window in (0, 90):
        case = _attention_case(torch.bfloat16, H, G, hd, [1] * len(lens), lens, window=window, seed=hd + window)
        q, kp, vp, pt, slots, kv_lens, ref = _decode_inputs(case)
        order = k.decode_order(slots, kv_lens, window)
        n = len(lens)
        entries = order[:4 * n].view(n, 4).cpu().tolist()
        inside = [min(v, window) if window else v for v in lens]
        assert [e[0] for e in entries] == sorted(range(n), key=lambda b: (-inside[b], b))
        assert all(e[1] == 1 << 16 and e[2] == lens[e[0]] and e[3] == int(slots[e[0]]) for e in entries)
        out = torch.full((n, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        before = k.launch_count
        k.attention_decode(q, kp, vp, pt, slots, kv_lens, out, H, G, hd, 1.0 / math.sqrt(hd), window, num_splits=1, plan=order)
        assert k.launch_count - before == 1
        torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))
        plain = torch.empty_like(out)
        k.attention_decode(q, kp, vp, pt, slots, kv_lens, plain, H, G, hd, 1.0 / math.sqrt(hd), window, num_splits=1)
        assert torch.equal(out, plain)


@pytest.mark.parametrize("splits,window", [(2, 0), (7, 0), (3, 100)])
def test_attention_decode_deals_chunks_by_length(splits, window):
    """More sequences than a warp has lanes, one of them far longer than the rest: the
    long one gets most of the chunks, and every sequence is still answered whole."""
    k = K()
    H, G, hd = 4, 2, 64
    lens = [1] * 14 + [1500] + [64, 65, 129] * 6 + [700, 3]
    assert len(lens) > 32
    case = _attention_case(torch.bfloat16, H, G, hd, [1] * len(lens), lens, window=window, seed=splits)
    q, kp, vp, pt, slots, kv_lens, ref = _decode_inputs(case)
    out = torch.full((len(lens), H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    plan = k.decode_plan(slots, kv_lens, window, splits)
    # the plan itself: every sequence has at least one chunk, together no more than the grid,
    # neighbours in the grid, and the longer a sequence the more it gets
    B = len(lens)
    entries = plan[:4 * B * splits].view(-1, 4).cpu()
    seqs = plan[4 * B * splits:].view(-1, 2).cpu()
    assert int(seqs[:, 1].min()) >= 1 and int(seqs[:, 1].sum()) <= B * splits
    assert seqs[:, 0].tolist() == [int(x) for x in (torch.cumsum(seqs[:, 1], 0) - seqs[:, 1])]
    assert int(seqs[14, 1]) == int(seqs[:, 1].max()) and int(seqs[0, 1]) == 1
    if window == 0:
        assert int(seqs[14, 1]) > int(seqs[33, 1]) > int(seqs[34, 1])      # 1500, 700 and 3 keys
    for b in range(B):
        for j in range(int(seqs[b, 1])):
            e = entries[int(seqs[b, 0]) + j].tolist()
            assert e == [b, j | (int(seqs[b, 1]) << 16), lens[b], int(slots[b])]
    assert (entries[int(seqs[:, 1].sum()):, 0] == -1).all()
    k.attention_decode(q, kp, vp, pt, slots, kv_lens, out, H, G, hd, 1.0 / math.sqrt(hd), window, num_splits=splits, plan=plan)
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))


def test_attention_decode_window_and_strided_queries():
    k = K()
    H, G, hd, W = 8, 2, 128, 70
    lens = [10, 70, 71, 300]
    case = _attention_case(torch.bfloat16, H, G, hd, [1] * 4, lens, window=W, seed=9)
    q, kp, vp, pt, slots, kv_lens, ref = _decode_inputs(case)
    wide = torch.zeros(4, (H + 2 * G) * hd, dtype=torch.bfloat16, device=DEV)     # q as a view into a qkv buffer
    wide[:, :H * hd] = q
    out = torch.empty(4, H * hd, dtype=torch.bfloat16, device=DEV)
    k.attention_decode(wide[:, :H * hd], kp, vp, pt, slots, kv_lens, out, H, G, hd, 1.0 / math.sqrt(hd), W, num_splits=3)
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 449, 450])
@pytest.mark.parametrize("splits", [1, 5])
def test_attention_decode_finds_one_far_key_among_hundreds(far, splits):
    H, G, hd, n = 8, 2, 128, 451

    def craft(b, qb, kb, vb):
        direction = torch.ones(hd) / math.sqrt(hd)
        qb[:] = (direction * 14.0).to(qb.dtype)
        kb[:] = (kb.float() * 0.05).to(kb.dtype)
        kb[far] = (direction * 14.0).to(kb.dtype)
    case = _attention_case(torch.bfloat16, H, G, hd, [1], [n], seed=5, craft=craft)
    q, kp, vp, pt, slots, kv_lens, ref = _decode_inputs(case)
    out = torch.empty(1, H * hd, dtype=torch.bfloat16, device=DEV)
    K().attention_decode(q, kp, vp, pt, slots, kv_lens, out, H, G, hd, 1.0 / math.sqrt(hd), num_splits=splits)
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))
    page = int(pt[1, far // PAGE]); v_far = vp[page, :, far % PAGE].double().cpu()
    assert (ref - v_far.repeat_interleave(H // G, dim=0).reshape(1, H * hd)).abs().max() < 1e-3


def test_attention_decode_ignores_garbage_beyond_the_sequence():
    """Rows of a page beyond the sequence's length may hold anything, NaN included."""
    k = K()
    H, G, hd = 4, 1, 64
    case = _attention_case(torch.bfloat16, H, G, hd, [1, 1], [5, 70], seed=2)
    q, kp, vp, pt, slots, kv_lens, ref = _decode_inputs(case)
    for b, n in enumerate([5, 70]):
        page = int(pt[int(slots[b]), (n - 1) // PAGE])
        kp[page, :, n % PAGE:] = float("nan"); vp[page, :, n % PAGE:] = float("nan")
    out = torch.empty(2, H * hd, dtype=torch.bfloat16, device=DEV)
    k.attention_decode(q, kp, vp, pt, slots, kv_lens, out, H, G, hd, 1.0 / math.sqrt(hd), num_splits=2)
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))


# ----------------------------------------------------------------------------- prefill attention (tensor cores)
def _prefill_inputs(case, lens_q, lens_kv):
    q, kp, vp, pt, sot, pos, ref = case
    B = len(lens_q)
    cu = [0]
    for n in lens_q:
        cu.append(cu[-1] + n)
    slots = list(range(B, 0, -1))        # as _attention_case assigns them
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return q, kp, vp, pt, i32(cu), i32(slots), i32(lens_kv), ref


@pytest.mark.parametrize("H,G,hd", [(32, 8, 128), (4, 4, 128), (6, 2, 64), (3, 1, 64)])
@pytest.mark.parametrize("lens_q,lens_kv", [([1, 5, 64, 65, 200], [1, 5, 64, 65, 200]),      # whole prompts
                                            ([130, 1, 33, 64], [130, 300, 97, 128]),            # chunks after a cached prefix
                                            ([700], [700])])
def test_attention_prefill_matches_plain(H, G, hd, lens_q, lens_kv):
    k = K()
    assert k.attention_prefill_supported(torch.bfloat16, H, G, hd)
    case = _attention_case(torch.bfloat16, H, G, hd, lens_q, lens_kv, seed=hd + H + len(lens_q))
    q, kp, vp, pt, cu, slots, kv_lens, ref = _prefill_inputs(case, lens_q, lens_kv)
    out = torch.full((q.shape[0], H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.attention_prefill(q, kp, vp, pt, cu, slots, kv_lens, lens_q, out, H, G, hd, 1.0 / math.sqrt(hd))
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))
    simt = torch.empty_like(out)
    k.attention_simt(q, kp, vp, pt, case[4], case[5], simt, H, G, hd, 1.0 / math.sqrt(hd))
    torch.testing.assert_close(out.float(), simt.float(), rtol=2e-2, atol=2e-2)


def test_attention_prefill_window_and_garbage_beyond_the_sequence():
    k = K()
    H, G, hd, W = 4, 2, 64, 70
    lens_q, lens_kv = [40, 150, 3], [40, 300, 200]
    case = _attention_case(torch.bfloat16, H, G, hd, lens_q, lens_kv, window=W, seed=4)
    q, kp, vp, pt, cu, slots, kv_lens, ref = _prefill_inputs(case, lens_q, lens_kv)
    for b, n in enumerate(lens_kv):       # rows of the last page beyond the sequence: NaN
        if n % PAGE:
            page = int(pt[int(slots[b]), (n - 1) // PAGE])
            kp[page, :, n % PAGE:] = float("nan"); vp[page, :, n % PAGE:] = float("nan")
    out = torch.empty(q.shape[0], H * hd, dtype=torch.bfloat16, device=DEV)
    k.attention_prefill(q, kp, vp, pt, cu, slots, kv_lens, lens_q, out, H, G, hd, 1.0 / math.sqrt(hd), W)
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))


@pytest.mark.parametrize("far", [0, 63, 64, 300])
def test_attention_prefill_finds_one_far_key(far):
    """Every query from position `far` on must return the value of key `far` (its score dominates)."""
    H, G, hd, n = 4, 2, 128, 451

    def craft(b, qb, kb, vb):
        direction = torch.ones(hd) / math.sqrt(hd)
        qb[:] = (direction * 14.0).to(qb.dtype)
        kb[:] = (kb.float() * 0.05).to(kb.dtype)
        kb[far] = (direction * 14.0).to(kb.dtype)
    case = _attention_case(torch.bfloat16, H, G, hd, [n], [n], seed=6, craft=craft)
    q, kp, vp, pt, cu, slots, kv_lens, ref = _prefill_inputs(case, [n], [n])
    out = torch.empty(n, H * hd, dtype=torch.bfloat16, device=DEV)
    K().attention_prefill(q, kp, vp, pt, cu, slots, kv_lens, [n], out, H, G, hd, 1.0 / math.sqrt(hd))
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))
    page = int(pt[1, far // PAGE]); v_far = vp[page, :, far % PAGE].double().cpu()
    want = v_far.repeat_interleave(H // G, dim=0).reshape(1, H * hd)
    assert (ref[far + 1:] - want).abs().max() < 1e-3


# ----------------------------------------------------------------------------- prefill attention (tcgen05)
@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("H,G", [(32, 8), (4, 4), (3, 1)])
@pytest.mark.parametrize("lens_q,lens_kv", [([1, 5, 64, 65, 200], [1, 5, 64, 65, 200]),
                                            ([130, 1, 33, 64], [130, 300, 97, 128]),
                                            ([129], [129]), ([128, 256], [128, 256]), ([700], [700]), ([40], [1000]),
                                            # 18 key tiles, the query tiles not aligned with them: both of a query tile's
                                            # last two key tiles are masked in part, and every ring and barrier wraps
                                            ([1700], [2304])])
def test_attention_prefill_tc_matches_plain(H, G, lens_q, lens_kv, hd):
    k = K()
    assert k.attention_prefill_tc_supported(torch.bfloat16, H, G, hd)
    case = _attention_case(torch.bfloat16, H, G, hd, lens_q, lens_kv, seed=H + len(lens_q) + lens_kv[0])
    q, kp, vp, pt, cu, slots, kv_lens, ref = _prefill_inputs(case, lens_q, lens_kv)
    out = torch.full((q.shape[0], H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.attention_prefill_tc(q, kp, vp, pt, cu, slots, kv_lens, lens_q, out, H, G, hd, 1.0 / math.sqrt(hd))
    k.check_device_errors()
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))


@pytest.mark.parametrize("hd", [64, 128])
def test_attention_prefill_tc_window_and_strided_queries(hd):
    k = K()
    H, G, W = 4, 2, 200
    lens_q, lens_kv = [40, 350, 3], [40, 500, 300]
    case = _attention_case(torch.bfloat16, H, G, hd, lens_q, lens_kv, window=W, seed=4)
    q, kp, vp, pt, cu, slots, kv_lens, ref = _prefill_inputs(case, lens_q, lens_kv)
    wide = torch.zeros(q.shape[0], (H + 2 * G) * hd, dtype=torch.bfloat16, device=DEV)
    wide[:, :H * hd] = q
    out = torch.empty(q.shape[0], H * hd, dtype=torch.bfloat16, device=DEV)
    k.attention_prefill_tc(wide[:, :H * hd], kp, vp, pt, cu, slots, kv_lens, lens_q, out, H, G, hd, 1.0 / math.sqrt(hd), W)
    k.check_device_errors()
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("far", [0, 63, 64, 127, 128, 300])
def test_attention_prefill_tc_finds_one_far_key_and_rescales(far, hd):
    """Every query from position `far` on must return the value of key `far`: its score is far
    above the running maximum of the tiles before it, so the lazily kept maximum has to move
    and the accumulator has to be rescaled."""
    H, G, n = 4, 2, 451

    def craft(b, qb, kb, vb):
        direction = torch.ones(hd) / math.sqrt(hd)
        qb[:] = (direction * 14.0).to(qb.dtype)
        kb[:] = (kb.float() * 0.05).to(kb.dtype)
        kb[far] = (direction * 14.0).to(kb.dtype)
    case = _attention_case(torch.bfloat16, H, G, hd, [n], [n], seed=6, craft=craft)
    q, kp, vp, pt, cu, slots, kv_lens, ref = _prefill_inputs(case, [n], [n])
    out = torch.empty(n, H * hd, dtype=torch.bfloat16, device=DEV)
    K().attention_prefill_tc(q, kp, vp, pt, cu, slots, kv_lens, [n], out, H, G, hd, 1.0 / math.sqrt(hd))
    K().check_device_errors()
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))
    page = int(pt[1, far // PAGE]); v_far = vp[page, :, far % PAGE].double().cpu()
    want = v_far.repeat_interleave(H // G, dim=0).reshape(1, H * hd)
    assert (ref[far + 1:] - want).abs().max() < 1e-3


# ----------------------------------------------------------------------------- attention over thousands of keys
def _far_key_craft(far, hd, gain=16.0):
    def craft(b, qb, kb, vb):
        direction = torch.ones(hd) / math.sqrt(hd)
        qb[:] = (direction * gain).to(qb.dtype)
        kb[:] = (kb.float() * 0.05).to(kb.dtype)
        kb[far] = (direction * gain).to(kb.dtype)      # its score stands far above the thousands of others
    return craft


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("n,far", [(4096, 0), (4096, 4095), (8704, 77), (8704, 8640)])
def test_attention_decode_over_thousands_of_keys(n, far, hd):
    """The contexts the benchmarks decode at: one key among 4,096 or 8,704 made to stand out, a
    short sequence beside it; every way the engine runs it (one chunk, dealt chunks, a cluster)."""
    k = K()
    H, G = 8, 2
    lens = [n, 33]
    craft = _far_key_craft(far, hd)
    case = _attention_case(torch.bfloat16, H, G, hd, [1, 1], lens, seed=n + far,
                           craft=lambda b, qb, kb, vb: craft(b, qb, kb, vb) if b == 0 else None)
    q, kp, vp, pt, slots, kv_lens, ref = _decode_inputs(case)
    page = int(pt[int(slots[0]), far // PAGE]); v_far = vp[page, :, far % PAGE].double().cpu()
    assert (ref[0:1] - v_far.repeat_interleave(H // G, dim=0).reshape(1, H * hd)).abs().max() < 2e-3
    for splits, planned, cluster in ((1, False, False), (8, False, False), (8, True, False), (8, False, True)):
        out = torch.full((2, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        plan = k.decode_plan(slots, kv_lens, 0, splits) if planned else None
        k.attention_decode(q, kp, vp, pt, slots, kv_lens, out, H, G, hd, 1.0 / math.sqrt(hd), num_splits=splits,
                           plan=plan, cluster=cluster)
        torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))
    simt = torch.empty(2, H * hd, dtype=torch.bfloat16, device=DEV)
    k.attention_simt(q, kp, vp, pt, slots, (kv_lens - 1).to(torch.int32), simt, H, G, hd, 1.0 / math.sqrt(hd))
    torch.testing.assert_close(simt.double().cpu(), ref, **_tol(torch.bfloat16))


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("lens_q,lens_kv,far", [([4096], [4096], 1), ([4096], [4096], 3900), ([600, 70], [8704, 70], 8100),
                                                ([600, 70], [8704, 70], 5)])
def test_attention_prefill_tc_over_thousands_of_keys(lens_q, lens_kv, far, hd):
    """A whole prompt of 4,096 tokens, and a 600-token portion behind 8,104 cached positions."""
    k = K()
    H, G = 4, 2
    craft = _far_key_craft(far, hd)
    case = _attention_case(torch.bfloat16, H, G, hd, lens_q, lens_kv, seed=far + lens_kv[0],
                           craft=lambda b, qb, kb, vb: craft(b, qb, kb, vb) if b == 0 else None)
    q, kp, vp, pt, cu, slots, kv_lens, ref = _prefill_inputs(case, lens_q, lens_kv)
    out = torch.full((q.shape[0], H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.attention_prefill_tc(q, kp, vp, pt, cu, slots, kv_lens, lens_q, out, H, G, hd, 1.0 / math.sqrt(hd))
    k.check_device_errors()
    torch.testing.assert_close(out.double().cpu(), ref, **_tol(torch.bfloat16))
    # queries behind the far key return its value
    first_q = lens_kv[0] - lens_q[0]
    page = int(pt[int(slots[0]), far // PAGE]); v_far = vp[page, :, far % PAGE].double().cpu()
    want = v_far.repeat_interleave(H // G, dim=0).reshape(1, H * hd)
    lo = max(far + 1 - first_q, 0)
    assert (ref[lo:lens_q[0]] - want).abs().max() < 2e-3
    other = torch.empty_like(out)
    k.attention_prefill(q, kp, vp, pt, cu, slots, kv_lens, lens_q, other, H, G, hd, 1.0 / math.sqrt(hd))
    torch.testing.assert_close(other.double().cpu(), ref, **_tol(torch.bfloat16))


# ----------------------------------------------------------------------------- sampling
def test_argmax_first_maximum_wins_and_non_finite_is_skipped():
    k = K()
    V = 5000
    logits = _rand(6, V, seed=12)
    logits[0, 4000] = 50.0; logits[0, 17] = 50.0             # tie: the first wins
    logits[1, :] = float("-inf"); logits[1, 4999] = -3.0
    logits[2, 100] = float("nan"); logits[2, 7] = 99.0
    logits[3, :] = float("nan")                              # nothing finite: token 0
    logits[4, 0] = float("inf"); logits[4, 9] = 60.0         # +inf is not finite either
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    k.argmax(logits, out)
    want = [P.argmax_finite(logits[i].cpu().numpy()) for i in range(6)]
    assert out.tolist() == want and want[:5] == [17, 4999, 7, 0, 9]


@pytest.mark.parametrize("V", [7, 384, 5000, 128256])
def test_temperature_sampling_follows_the_plain_sampler(V):
    k = K()
    rows = 24
    logits = _rand(rows, V, seed=13, scale=2.0)
    logits[3, 5 % V] = float("-inf"); logits[4, 2 % V] = float("nan")
    temps = torch.tensor([0.8, 1.0, 0.3, 1.5] * 6)
    rngs = [P.Rng(100 + i) for i in range(rows)]
    for trial in range(6):
        u = torch.tensor([r.next_f32() for r in rngs])
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        k.sample_temperature(logits, temps.to(DEV), u.to(DEV), out)
        for i in range(rows):
            class Fixed:                      # hands the plain sampler the same uniform
                def next_f32(self, v=float(u[i])): return v
            want = P.sample(logits[i].cpu().numpy(), float(temps[i]), Fixed())
            got = out[i].item()
            if got == want:
                continue
            # The plain sampler sums V weights one after another in float32 (as the
            # reference does); its running sum carries a relative error of up to
            # ~V * 2^-24.  A different answer is right if the exact (float64) running
            # sum around it brackets u * total within that uncertainty.
            l = np.where(np.isfinite(logits[i].cpu().numpy()), logits[i].cpu().numpy(), -np.inf).astype(np.float64)
            w = np.exp((l - l.max()) / float(temps[i]))
            pre = np.cumsum(w) / w.sum()
            slack = max(V * 2.0 ** -24, 1e-6)
            lo = pre[got - 1] if got > 0 else 0.0
            assert lo <= float(u[i]) + slack and pre[got] >= float(u[i]) - slack and w[got] > 0, \
                f"row {i} trial {trial}: {got} vs {want}"
            assert abs(got - want) < 64


def _kept_candidates(logits, temperature, top_k, top_p, min_p):
    """The reference's candidate set in float64: tokens by descending logit (ties: lower index),
    the top-k head of it, min-p's head of that, top-p's head of that; with their weights."""
    n = logits.shape[0]
    v = np.where(np.isfinite(logits), logits, -np.inf).astype(np.float64)
    order = np.lexsort((np.arange(n), -v))
    if 0 < top_k < n:
        order = order[:top_k]
    w = np.exp((v[order] - v[order[0]]) / temperature)
    total, limit = w.sum(), len(order)
    if min_p > 0:
        below = np.nonzero(w < min_p * w[0])[0]
        limit = max(int(below[0]) if below.size else len(order), 1)
    cutoff = limit
    if top_p < 1.0:
        over = np.nonzero(np.cumsum(w[:limit]) > top_p * total)[0]
        cutoff = int(over[0]) + 1 if over.size else limit
    return order[:cutoff], w[:cutoff]


@pytest.mark.parametrize("V", [5000, 128256])
def test_candidate_sampling_at_real_vocabularies_follows_the_plain_sampler(V):
    """Top-k, top-p and min-p in every combination the options allow, at vocabularies far larger
    than a thread block: the same generator seeds as the plain sampler, the same tokens.  Where
    they differ, the uniform number must lie within float rounding of the boundary between the
    two tokens' shares (the kernels add in another order than the reference's float32 loop)."""
    from rustyllm_b200.sampling.config import SamplerConfig
    from rustyllm_b200.sampling.sampler import Sampler, SequenceSamplingState
    options = [dict(top_k=2), dict(top_k=40), dict(top_k=1024), dict(top_k=40, top_p=0.9), dict(top_k=40, min_p=0.05),
               dict(top_k=1024, top_p=0.95, min_p=0.001), dict(top_p=0.9), dict(top_p=0.5, min_p=0.02), dict(top_p=0.99),
               dict(top_p=0.9, top_k=40, repeat_penalty=1.1), dict(top_p=0.3), dict(top_p=0.999, min_p=0.0001)]
    temps = [0.8, 1.3, 0.7]
    rows = len(options)
    g = torch.Generator().manual_seed(V)
    base = torch.randn(rows, V, generator=g) * 3.0
    base[1, 7] = float("-inf"); base[6, 11] = float("nan"); base[2, 100] = base[2, 200] = base[2].max() + 1.0   # a tie at the top
    recent = torch.randint(0, V, (30,), generator=g).tolist()
    configs = [SamplerConfig(temperature=temps[i % 3], **o) for i, o in enumerate(options)]
    sampler = Sampler(torch.device(DEV))
    states = [SequenceSamplingState(c, 500 + i, recent) for i, c in enumerate(configs)]
    twins = [P.Rng(500 + i) for i in range(rows)]
    differed = 0
    for trial in range(8):
        got = sampler.sample(base.clone().to(DEV), states)
        for i, c in enumerate(configs):
            u = twins[i].next_f32()

            class Fixed:
                def next_f32(self, v=u): return v
            lg = base[i].numpy().copy()
            want = P.sample(lg, c.temperature, Fixed(), c.top_k, c.top_p, c.min_p, c.repeat_penalty, recent=recent[-64:])
            if got[i] == want:
                continue
            differed += 1
            P.apply_repeat_penalty(lg, recent[-64:], c.repeat_penalty)
            kept, w = _kept_candidates(lg, c.temperature, c.top_k, c.top_p, c.min_p)
            where = np.nonzero(kept == got[i])[0]
            assert where.size == 1, f"options {options[i]} trial {trial}: token {got[i]} is not among the {len(kept)} kept (plain: {want})"
            j = int(where[0])
            pre = np.cumsum(w) / w.sum()
            slack = max(len(kept) * 2.0 ** -24, 1e-6)
            assert (pre[j - 1] if j else 0.0) <= u + slack and pre[j] >= u - slack, \
                f"options {options[i]} trial {trial}: {got[i]} (place {j}) vs {want}, u = {u}"
    assert differed <= 4, f"{differed} of {8 * rows} draws differ from the plain sampler"



@pytest.mark.parametrize("V", [5000, 128256])
def test_candidate_sampling_with_thousands_of_equal_logits(V):
    """Rows whose boundary classes are large: all logits equal, logits rounded to halves (classes of
    thousands of identical keys), two values in turn, a few thousand equal finite logits among
    -inf.  The selection then refines a class down to all 32 bits and tells its tokens apart by
    index; the answers follow the plain sampler as in the test above."""
    from rustyllm_b200.sampling.config import SamplerConfig
    from rustyllm_b200.sampling.sampler import Sampler, SequenceSamplingState
    g = torch.Generator().manual_seed(V + 1)
    flat = torch.zeros(V)
    halves = (torch.randn(V, generator=g) * 3.0 * 2).round() / 2
    two = torch.where(torch.arange(V) % 2 == 0, torch.tensor(1.0), torch.tensor(0.5))
    few = torch.full((V,), float("-inf")); few[torch.randperm(V, generator=g)[:3000]] = 2.0
    dists = [flat, halves, two, few]
    options = [dict(top_k=40), dict(top_k=1024, top_p=0.9), dict(top_p=0.9), dict(top_p=0.5, min_p=0.5), dict(top_k=2)]
    rows = [(d, o) for d in dists for o in options]
    base = torch.stack([d for d, _ in rows])
    configs = [SamplerConfig(temperature=0.9, **o) for _, o in rows]
    sampler = Sampler(torch.device(DEV))
    states = [SequenceSamplingState(c, 900 + i, []) for i, c in enumerate(configs)]
    twins = [P.Rng(900 + i) for i in range(len(rows))]
    for trial in range(6):
        got = sampler.sample(base.clone().to(DEV), states)
        for i, c in enumerate(configs):
            u = twins[i].next_f32()

            class Fixed:
                def next_f32(self, v=u): return v
            lg = base[i].numpy().copy()
            want = P.sample(lg, c.temperature, Fixed(), c.top_k, c.top_p, c.min_p, c.repeat_penalty, recent=[])
            if got[i] == want:
                continue
            kept, w = _kept_candidates(lg, c.temperature, c.top_k, c.top_p, c.min_p)
            where = np.nonzero(kept == got[i])[0]
            assert where.size == 1, f"row {i} {rows[i][1]} trial {trial}: token {got[i]} is not among the {len(kept)} kept (plain: {want})"
            j = int(where[0])
            pre = np.cumsum(w) / w.sum()
            slack = max(len(kept) * 2.0 ** -24, 1e-6)
            assert (pre[j - 1] if j else 0.0) <= u + slack and pre[j] >= u - slack, \
                f"row {i} {rows[i][1]} trial {trial}: {got[i]} (place {j}) vs {want}, u = {u}"


@pytest.mark.parametrize("rows", [5, 30, 60, 90])
def test_top_k_rows_in_clusters_of_every_size(rows):
    """The top-k kernel gives a row of a large vocabulary to a cluster of 8, 4 or 2 CTAs or to one
    CTA, by the number of rows of the call; the temperature and argmax kernels likewise.  Every
    row of every such call against the plain sampler."""
    from rustyllm_b200.sampling.config import SamplerConfig
    from rustyllm_b200.sampling.sampler import Sampler, SequenceSamplingState
    V = 20000
    g = torch.Generator().manual_seed(rows)
    base = torch.randn(rows, V, generator=g) * 3.0
    kinds = [dict(top_k=40, top_p=0.9), dict(), dict(temperature=0.0), dict(top_k=7, min_p=0.05)]
    configs = [SamplerConfig(**{"temperature": 0.8, **kinds[i % 4]}) for i in range(rows)]
    sampler = Sampler(torch.device(DEV))
    states = [SequenceSamplingState(c, 70 + i, []) for i, c in enumerate(configs)]
    twins = [P.Rng(70 + i) for i in range(rows)]
    differed = 0
    for trial in range(2):
        got = sampler.sample(base.clone().to(DEV), states)
        for i, c in enumerate(configs):
            if c.is_greedy:
                assert got[i] == int(base[i].argmax())
                continue
            u = twins[i].next_f32()

            class Fixed:
                def next_f32(self, v=u): return v
            lg = base[i].numpy().copy()
            want = P.sample(lg, c.temperature, Fixed(), c.top_k, c.top_p, c.min_p, c.repeat_penalty, recent=[])
            if got[i] == want:
                continue
            differed += 1
            if c.top_k > 0:
                kept, w = _kept_candidates(lg, c.temperature, c.top_k, c.top_p, c.min_p)
            else:                     # the whole vocabulary in index order, as the reference walks it
                kept = np.arange(V)
                w = np.exp((lg.astype(np.float64) - lg.max()) / c.temperature)
            where = np.nonzero(kept == got[i])[0]
            assert where.size == 1, f"row {i} {kinds[i % 4]}: token {got[i]} is not among the {len(kept)} kept (plain: {want})"
            j = int(where[0])
            pre = np.cumsum(w) / w.sum()
            slack = max(len(kept) * 2.0 ** -24, 1e-6)
            assert (pre[j - 1] if j else 0.0) <= u + slack and pre[j] >= u - slack, f"row {i}: {got[i]} vs {want}, u = {u}"
    assert differed <= max(2, rows // 10)


def test_a_rows_draw_does_not_depend_on_how_many_rows_the_call_has():
    """The temperature kernel gives a row 8, 4, 2 or 1 CTAs by the number of rows of the call and
    sums the row in the same eight parts either way: the same logits and the same uniform number
    give the same token in calls of 1, 12, 40 and 80 rows, bit for bit the same sums."""
    k = K()
    V = 128256
    g = torch.Generator().manual_seed(11)
    row = (torch.randn(V, generator=g) * 3.0).to(DEV)
    answers = []
    for u in (0.013, 0.37, 0.5, 0.93, 0.999999):
        per_call = []
        for rows in (1, 12, 40, 80):
            logits = row.repeat(rows, 1).contiguous()
            out = torch.empty(rows, dtype=torch.int32, device=DEV)
            k.sample_temperature(logits, torch.full((rows,), 0.8, device=DEV), torch.full((rows,), u, device=DEV), out)
            assert (out == out[0]).all()
            per_call.append(int(out[0]))
        assert len(set(per_call)) == 1, f"u = {u}: {per_call}"
        answers.append(per_call[0])
    assert len(set(answers)) > 2


def test_temperature_zero_rows_are_greedy_and_min_p_cuts():
    k = K()
    logits = torch.tensor([[1.0, 5.0, 2.0, 4.9], [10.0, 9.5, 3.0, 1.0]], device=DEV)
    out = torch.empty(2, dtype=torch.int32, device=DEV)
    for u in (0.0, 0.5, 0.999):
        k.sample_temperature(logits, torch.tensor([0.0, 1.0], device=DEV), torch.tensor([u, u], device=DEV), out,
                             torch.tensor([0.0, 0.3], device=DEV))
        assert out[0].item() == 1 and out[1].item() in (0, 1)
    k.sample_temperature(logits, torch.tensor([1.0, 1.0], device=DEV), torch.tensor([0.999999, 0.999999], device=DEV), out,
                         torch.tensor([0.0, 0.3], device=DEV))
    assert out[1].item() == 1      # the tail (tokens 2, 3) is cut: the last kept candidate


def test_repeat_penalty_kernel():
    k = K()
    logits = torch.tensor([[4.0, -4.0, 2.0, float("nan")], [1.0, 2.0, 3.0, 4.0]], device=DEV)
    recent = torch.zeros(2, 64, dtype=torch.int32, device=DEV)
    recent[0, :4] = torch.tensor([0, 1, 3, 99]); recent[1, :3] = torch.tensor([2, 2, 0])
    k.repeat_penalty(logits, recent, torch.tensor([4, 3], dtype=torch.int32, device=DEV), 2.0)
    assert logits[0, :3].tolist() == [2.0, -8.0, 2.0] and logits[0, 3].item() == float("-inf")
    assert logits[1].tolist() == [0.5, 2.0, 0.75, 4.0]      # token 2 twice: divided twice


def test_sampler_object_runs_the_reference_cases():
    from rustyllm_b200.sampling.config import SamplerConfig
    from rustyllm_b200.sampling.sampler import Sampler, SequenceSamplingState
    s = Sampler(torch.device(DEV))
    for name, opt, seed, draws, logits, recent, allowed, must in CASES:
        st = SequenceSamplingState(SamplerConfig(**opt), seed, recent)
        seen = set()
        for _ in range(draws):
            t = s.sample(torch.tensor([logits], device=DEV), [st])[0]
            assert t in allowed, name
            seen.add(t)
        assert must <= seen, name


def test_kernels_refuse_what_they_cannot_do():
    k = K()
    with pytest.raises(k.KernelError, match="CUDA tensors only"):
        k.swiglu(torch.zeros(2, 4), torch.zeros(2, 2))
    q = torch.zeros(1, 2 * 300, device=DEV)
    with pytest.raises(k.KernelError, match="head_dim"):
        k.attention_simt(q, torch.zeros(1, 2, PAGE, 300, device=DEV), torch.zeros(1, 2, PAGE, 300, device=DEV),
                         torch.zeros(1, 1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                         torch.zeros(1, dtype=torch.int32, device=DEV), torch.zeros(1, 600, device=DEV), 2, 2, 300, 1.0)
    with pytest.raises(k.KernelError, match="not handled"):
        k.swiglu(torch.zeros(2, 4, dtype=torch.float16, device=DEV), torch.zeros(2, 2, dtype=torch.float16, device=DEV))
