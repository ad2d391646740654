"""Each kernel alone against a plain float64 PyTorch reference of the same operation, at sizes other
than the engine's tiny configurations (sizes that are no power of two, odd head counts and groups,
page edges, windows), in 32-bit and in bfloat16."""

import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def rand(shape, dtype, device, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(device)


@pytest.fixture(scope="module")
def ops(cuda_device):
    from zephyr_b200.kernels import ops as module

    module.library()
    return module


def ref_rmsnorm(x, w, eps):
    x = x.double()
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()


# ------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,V", [(100, 77), (1000, 311), (4096, 1000), (8, 3)])
def test_embedding(ops, cuda_device, dtype, H, V):
    table = rand((V, H), dtype, cuda_device, 1)
    ids = torch.randint(0, V, (37,), generator=torch.Generator().manual_seed(2)).int().to(cuda_device)
    status = ops.new_status(cuda_device)
    out = ops.embedding(table, ids, status)
    assert torch.equal(out, table[ids.long()])
    ops.check_status(status)


def test_embedding_reports_bad_token(ops, cuda_device):
    table = rand((10, 16), torch.float32, cuda_device, 1)
    ids = torch.tensor([1, 10, 3], dtype=torch.int32, device=cuda_device)
    status = ops.new_status(cuda_device)
    ops.embedding(table, ids, status)
    with pytest.raises(ops.KernelError, match="token id"):
        ops.check_status(status)
    ops.check_status(status)        # the word was cleared


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("rows,H", [(5, 100), (3, 1000), (2, 4096), (7, 24), (1, 5120),
                                    # many rows: bfloat16 rows of up to 2048 go a warp a row
                                    (200, 1024), (70, 1000), (64, 2048), (100, 136), (65, 2056), (333, 8)])
def test_rmsnorm_and_fused_add(ops, cuda_device, dtype, wdtype, rows, H):
    x = rand((rows, H), dtype, cuda_device, 3, 2.0)
    d = rand((rows, H), dtype, cuda_device, 4)
    w = (1 + rand((H,), torch.float32, cuda_device, 5, 0.1)).to(wdtype)
    eps = 1e-5
    got = ops.rmsnorm(x, w, eps)
    assert (got.double() - ref_rmsnorm(x, w, eps)).abs().max() <= tol(dtype, 4.0)
    residual = x.clone()
    got = ops.add_rmsnorm(residual, d, w, eps)
    summed = (x.double() + d.double()).to(dtype)           # one rounding of the float sum
    assert torch.equal(residual, summed)
    assert (got.double() - ref_rmsnorm(summed, w, eps)).abs().max() <= tol(dtype, 4.0)
    # fused and separate give the same bits
    assert torch.equal(got, ops.rmsnorm(summed, w, eps))


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_over_heads(ops, cuda_device, dtype):
    for tokens in (9, 40):
        x = rand((tokens, 5, 48), dtype, cuda_device, 6)
        w = (1 + rand((48,), torch.float32, cuda_device, 7, 0.1)).to(dtype)
        got = ops.rmsnorm(x, w, 1e-6)
        assert (got.double() - ref_rmsnorm(x, w, 1e-6)).abs().max() <= tol(dtype, 4.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(5, 200), (3, 3072), (2, 37), (130, 144)])
def test_silu_mul(ops, cuda_device, dtype, T, I):
    gu = rand((T, 2 * I), dtype, cuda_device, 8, 3.0)
    got = ops.silu_mul(gu)
    g, u = gu[:, :I].double(), gu[:, I:].double()
    assert (got.double() - g / (1 + torch.exp(-g)) * u).abs().max() <= tol(dtype, 8.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gather_rows(ops, cuda_device, dtype):
    x = rand((50, 96), dtype, cuda_device, 9)
    rows = torch.tensor([49, 0, 7, 7, 13], dtype=torch.int32, device=cuda_device)
    status = ops.new_status(cuda_device)
    assert torch.equal(ops.gather_rows(x, rows, status), x[rows.long()])
    ops.check_status(status)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(5, 200), (3, 3072), (130, 144), (1, 8), (64, 3072), (100, 8), (77, 4104), (300, 264)])
def test_silu_mul_blocked_layout(ops, cuda_device, dtype, T, I):
    g = rand((T, I), dtype, cuda_device, 8, 3.0)
    u = rand((T, I), dtype, cuda_device, 9, 3.0)
    gu = torch.stack([g.view(T, I // 8, 8), u.view(T, I // 8, 8)], dim=2).reshape(T, 2 * I).contiguous()
    got = ops.silu_mul(gu, blocked=True)
    assert torch.equal(got, ops.silu_mul(torch.cat([g, u], dim=1).contiguous()))


# ------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,N,K", [(1, 311, 100), (7, 64, 64), (130, 200, 96), (65, 1000, 1030), (3, 5, 1)])
def test_gemm_simt_float32_is_exact_float32(ops, cuda_device, M, N, K):
    x = rand((M, K), torch.float32, cuda_device, 10)
    w = rand((N, K), torch.float32, cuda_device, 11)
    got = ops.gemm_nt_simt(x, w)
    expected = x.double() @ w.double().T
    # float32 accumulation of K products of magnitude ~1: error ~ sqrt(K) * 2^-24 * |terms|.
    assert (got.double() - expected).abs().max() <= 3e-6 * math.sqrt(K) * 4
    # TF32 would be wrong in the 4th digit: this bound is 1000x tighter than that.


def test_gemm_simt_rows_do_not_depend_on_batch(ops, cuda_device):
    x = rand((70, 200), torch.float32, cuda_device, 12)
    w = rand((311, 200), torch.float32, cuda_device, 13)
    whole = ops.gemm_nt_simt(x, w)
    assert torch.equal(ops.gemm_nt_simt(x[5:6].contiguous(), w), whole[5:6])
    assert torch.equal(ops.gemm_nt_simt(x[60:].contiguous(), w), whole[60:])


def test_gemm_simt_bfloat16_inputs(ops, cuda_device):
    x = rand((33, 136), torch.bfloat16, cuda_device, 14)
    w = rand((77, 136), torch.bfloat16, cuda_device, 15)
    got = ops.gemm_nt_simt(x, w, out_dtype=torch.float32)
    assert (got.double() - x.double() @ w.double().T).abs().max() <= 1e-4
    assert ops.linear(x, w, out_dtype=torch.float32).dtype == torch.float32
    assert (ops.linear(x, w, out_dtype=torch.float32).double() - x.double() @ w.double().T).abs().max() <= 1e-3


SMALL_GEMM_CASES = [(1, 311, 96), (8, 4096, 1024), (8, 1024, 3072), (3, 200, 200), (16, 1024, 2048), (33, 96, 136),
                    (64, 6144, 1024), (7, 50, 8), (8, 151936, 1024)]


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", SMALL_GEMM_CASES)
def test_gemm_small_weight_streamer(ops, cuda_device, M, N, K, out_dtype):
    x = rand((M, K), torch.bfloat16, cuda_device, 40)
    w = rand((N, K), torch.bfloat16, cuda_device, 41, 0.1)
    assert ops.gemm_small_supported(x, w)
    got = ops.gemm_small(x, w, out_dtype=out_dtype)
    expected = x.double() @ w.double().T
    bound = 1e-3 * math.sqrt(K) if out_dtype == torch.float32 else 4e-3 * max(1.0, float(expected.abs().max()))
    assert got.dtype == out_dtype and (got.double() - expected).abs().max() <= bound
    # rows do not depend on the rows beside them
    if M > 1:
        alone = ops.gemm_small(x[M - 1:].contiguous(), w, out_dtype=out_dtype)
        assert torch.equal(alone, got[M - 1:])
    # strided activations (a slice of a wider buffer)
    wide = torch.zeros((M, K + 16), dtype=torch.bfloat16, device=cuda_device)
    wide[:, :K] = x
    assert torch.equal(ops.gemm_small(wide[:, :K], w, out_dtype=out_dtype), got)


@pytest.mark.parametrize("M,I,K", [(1, 128, 64), (8, 3072, 1024), (20, 200, 96), (64, 144, 80)])
def test_gemm_small_fused_swiglu(ops, cuda_device, M, I, K):
    x = rand((M, K), torch.bfloat16, cuda_device, 42)
    gate = rand((I, K), torch.bfloat16, cuda_device, 43, 0.2)
    up = rand((I, K), torch.bfloat16, cuda_device, 44, 0.2)
    w = torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    got = ops.gemm_small(x, w, swiglu=True)
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    expected = g / (1 + torch.exp(-g)) * u
    assert got.shape == (M, I) and (got.double() - expected).abs().max() <= 8e-3 * max(1.0, float(expected.abs().max()))


def test_gemm_small_refuses(ops, cuda_device):
    x = rand((65, 64), torch.bfloat16, cuda_device, 45)
    w = rand((32, 64), torch.bfloat16, cuda_device, 46)
    assert not ops.gemm_small_supported(x, w)
    assert not ops.gemm_small_supported(x[:4, :60], w[:, :60])          # K no multiple of 8
    assert not ops.gemm_small_supported(x[:4].float(), w.float())
    assert ops.linear(x, w).shape == (65, 32)                            # the library product takes over


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,N", [(1, 7), (13, 96), (300, 1000)])
def test_add_bias(ops, cuda_device, dtype, T, N):
    y = rand((T, N + 8), dtype, cuda_device, 160)
    bias = rand((N,), torch.float32, cuda_device, 161)
    expected = (y[:, :N].float() + bias[None, :]).to(dtype)
    untouched = y[:, N:].clone()
    ops.add_bias(y[:, :N], bias)                       # a slice of a wider buffer
    assert torch.equal(y[:, :N], expected) and torch.equal(y[:, N:], untouched)
    x, w = rand((T, 64), dtype, cuda_device, 162), rand((N, 64), dtype, cuda_device, 163, 0.1)
    assert torch.equal(ops.linear(x, w, bias=bias.to(dtype)), ops.add_bias(ops.linear(x, w), bias.to(dtype)))


# ------------------------------------------------------- seeded fill
def philox_4x32_10(counter: int, key: int) -> list[int]:
    """The published Philox 4x32 generator with ten rounds (Salmon et al. 2011), counter in the two low words."""
    m0, m1, w0, w1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    c = [counter & mask, (counter >> 32) & mask, 0, 0]
    k = [key & mask, (key >> 32) & mask]
    for _ in range(10):
        p0, p1 = m0 * c[0], m1 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k[0], p1 & mask, (p0 >> 32) ^ c[3] ^ k[1], p0 & mask]
        k = [(k[0] + w0) & mask, (k[1] + w1) & mask]
    return c


def ref_normals(n: int, key: int) -> torch.Tensor:
    out = []
    for i in range((n + 3) // 4):
        w = philox_4x32_10(i, key)
        for a, b in ((w[0], w[1]), (w[2], w[3])):
            u1, u2 = ((a >> 8) + 1) / 16777216.0, (b >> 8) / 16777216.0
            radius = math.sqrt(-2.0 * math.log(u1))
            out += [radius * math.cos(2 * math.pi * u2), radius * math.sin(2 * math.pi * u2)]
    return torch.tensor(out[:n], dtype=torch.float64)


@pytest.mark.parametrize("n", [1, 7, 4096, 100003])
def test_fill_normal(ops, cuda_device, n):
    key = 0x9E3779B97F4A7C15 ^ n
    got = ops.fill_normal(torch.empty(n, dtype=torch.float32, device=cuda_device), key, 0.0, 1.0)
    head = min(n, 2000)
    assert (got[:head].double().cpu() - ref_normals(head, key)).abs().max() <= 2e-5      # float32 log, sqrt, sin and cos
    # the same values scaled and shifted, rounded once to bfloat16; every element written, none beyond
    wide = torch.full((n + 8,), 7.0, dtype=torch.bfloat16, device=cuda_device)
    ops.fill_normal(wide[:n], key, 1.0, 0.02)
    assert torch.equal(wide[:n], (got * 0.02 + 1.0).to(torch.bfloat16)) and bool((wide[n:] == 7.0).all())
    # another key, other values; the same key, the same values
    assert not torch.equal(ops.fill_normal(torch.empty_like(got), key + 1, 0.0, 1.0), got)
    assert torch.equal(ops.fill_normal(torch.empty_like(got), key, 0.0, 1.0), got)
    if n >= 4096:
        assert abs(float(got.mean())) < 5.0 / math.sqrt(n) and abs(float(got.std()) - 1.0) < 5.0 / math.sqrt(n)


def test_random_weights_on_the_device(cuda_device):
    from zephyr_b200.weights.loader import ROLE_NORM, RandomWeights, WeightDecl
    decls = {"a.weight": WeightDecl((40, 24)), "b.weight": WeightDecl((24,), ROLE_NORM), "c.weight": WeightDecl((40, 24))}
    store = RandomWeights(decls, 3, torch.bfloat16, device=cuda_device)
    a, b, c = (store.read(name) for name in decls)
    assert a.shape == (40, 24) and a.dtype == torch.bfloat16 and a.is_cuda
    assert not torch.equal(a, c) and abs(float(b.float().mean()) - 1.0) < 0.02 and float(a.float().std()) < 0.03
    other_order = RandomWeights(dict(reversed(list(decls.items()))), 3, torch.bfloat16, device=cuda_device)
    assert torch.equal(other_order.read("a.weight"), a)
    assert not torch.equal(RandomWeights(decls, 4, torch.bfloat16, device=cuda_device).read("a.weight"), a)


# ------------------------------------------------------- the tcgen05 product for many rows
TC_GEMM_CASES = [(128, 256, 64, 0), (200, 264, 136, 0), (2048, 1024, 3072, 0), (333, 250, 1000, 128), (333, 250, 1000, 256),
                 (17, 1024, 2048, 128), (1000, 4096, 1024, 256), (129, 8, 8, 0), (2500, 1544, 520, 0),
                 (256, 256, 64, 2), (300, 520, 200, 2), (2500, 1544, 520, 2), (5000, 6144, 1024, 2)]


@pytest.mark.parametrize("M,N,K,block_n", TC_GEMM_CASES)
def test_gemm_tc_product(ops, cuda_device, M, N, K, block_n):
    """Rows, columns and depths that end inside a tile, a stage and a swizzled row; more tiles than SMs
    (a CTA takes several, through both accumulators) and fewer."""
    x = rand((M, K), torch.bfloat16, cuda_device, 140)
    w = rand((N, K), torch.bfloat16, cuda_device, 141, 0.1)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    assert ops.gemm_tc_supported(x, w)
    got = ops.gemm_tc(x, w, block_n=block_n, status=status)
    expected = x.double() @ w.double().T
    assert status.tolist()[0] == 0, status.tolist()
    assert got.shape == (M, N)
    assert (got.double() - expected).abs().max() <= 4e-3 * max(1.0, float(expected.abs().max()))
    # rows do not depend on the rows beside them, nor on the tile width
    other = ops.gemm_tc(x[M // 2:], w, block_n=128 if block_n != 128 else 256, status=status)
    assert torch.equal(other, got[M // 2:])
    # strided activations (a slice of a wider buffer)
    wide = torch.zeros((M, K + 16), dtype=torch.bfloat16, device=cuda_device)
    wide[:, :K] = x
    assert torch.equal(ops.gemm_tc(wide[:, :K], w, block_n=block_n, status=status), got)
    assert status.tolist()[0] == 0


@pytest.mark.parametrize("M,I,K,block_n", [(128, 128, 64, 0), (2048, 3072, 1024, 0), (300, 200, 96, 128), (300, 200, 96, 256),
                                           (1111, 520, 264, 0), (300, 200, 96, 2), (2048, 3072, 1024, 2), (1111, 520, 264, 2)])
def test_gemm_tc_fused_swiglu(ops, cuda_device, M, I, K, block_n):
    x = rand((M, K), torch.bfloat16, cuda_device, 142)
    gate = rand((I, K), torch.bfloat16, cuda_device, 143, 0.2)
    up = rand((I, K), torch.bfloat16, cuda_device, 144, 0.2)
    w = torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    got = ops.gemm_tc(x, w, swiglu=True, block_n=block_n, status=status)
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    expected = g / (1 + torch.exp(-g)) * u
    assert status.tolist()[0] == 0, status.tolist()
    assert got.shape == (M, I) and (got.double() - expected).abs().max() <= 8e-3 * max(1.0, float(expected.abs().max()))
    # the same sums, activation and rounding as the kernel for few rows
    few = ops.gemm_small(x[:8].contiguous(), w, swiglu=True)
    assert (few.double() - got[:8].double()).abs().max() <= 2.0 ** -7 * max(1.0, float(expected[:8].abs().max()))


@pytest.mark.parametrize("M,N,K,block_n", [(128, 256, 64, 0), (200, 250, 136, 0), (333, 151, 1000, 2), (40, 1001, 96, 0),
                                          (1000, 4096, 1024, 2), (17, 517, 264, 128)])
def test_gemm_tc_float_out(ops, cuda_device, M, N, K, block_n):
    """The sums as they are (logits): float32 out, any width."""
    x = rand((M, K), torch.bfloat16, cuda_device, 147)
    w = rand((N, K), torch.bfloat16, cuda_device, 148, 0.1)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    got = ops.gemm_tc(x, w, block_n=block_n, status=status, out_dtype=torch.float32)
    expected = x.double() @ w.double().T
    assert status.tolist()[0] == 0 and got.dtype == torch.float32 and got.shape == (M, N) and got.is_contiguous()
    assert (got.double() - expected).abs().max() <= 1e-3 * math.sqrt(K)
    assert torch.equal(got.to(torch.bfloat16), ops.gemm_tc(x, w, block_n=block_n, status=status))       # the same sums, rounded


def test_gemm_tc_refuses(ops, cuda_device):
    x = rand((200, 64), torch.bfloat16, cuda_device, 145)
    w = rand((32, 64), torch.bfloat16, cuda_device, 146)
    assert not ops.gemm_tc_supported(x[:, :60], w[:, :60].contiguous())          # K no multiple of 8
    assert not ops.gemm_tc_supported(x.float(), w.float())
    assert not ops.gemm_tc_supported(x, w[:24], swiglu=True)                      # gate/up blocks need N % 16 == 0
    from zephyr_b200.config import InvalidArgumentError
    with pytest.raises(InvalidArgumentError):
        ops.gemm_tc(x[:, :60], w[:, :60].contiguous())


# ------------------------------------------------------- norm + rotation + cache
def ref_rope(x, positions, theta):
    """x [T, heads, hd] double; float32 angles as the reference computes them."""
    hd = x.shape[-1]
    i = torch.arange(hd // 2, dtype=torch.float32)
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2.0 * i / hd)
    ang = (positions.float()[:, None] * inv[None, :]).double()
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., : hd // 2], x[..., hd // 2:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def make_tables(ctx_lens, page_size, num_pages, seed):
    """Random distinct pages for each row's context; returns (block_table tensor rows, list of lists)."""
    rng = random.Random(seed)
    pages = list(range(1, num_pages))
    rng.shuffle(pages)
    tables, cursor = [], 0
    for n in ctx_lens:
        need = -(-n // page_size)
        tables.append(pages[cursor:cursor + need])
        cursor += need
    assert cursor <= len(pages)
    width = max(1, max(len(t) for t in tables))
    table = torch.zeros((len(tables), width), dtype=torch.int32)
    for r, t in enumerate(tables):
        table[r, :len(t)] = torch.tensor(t, dtype=torch.int32)
    return table, tables


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,page", [(4, 2, 16, 4), (6, 3, 48, 8), (16, 8, 128, 16), (5, 5, 256, 32), (8, 1, 80, 64),
                                            (7, 2, 64, 16), (3, 1, 128, 8)])
def test_qk_norm_rope_cache(ops, cuda_device, dtype, nh, nkv, hd, page):
    from zephyr_b200.parts import rope_tables

    q_lens, ctx = [3, 1, 9], [5, 31, 0]
    T, R = sum(q_lens), len(q_lens)
    theta, eps = 50000.0, 1e-5
    qkv = rand((T, (nh + 2 * nkv) * hd), dtype, cuda_device, 20)
    wq = (1 + rand((hd,), torch.float32, cuda_device, 21, 0.1)).to(dtype)
    wk = (1 + rand((hd,), torch.float32, cuda_device, 22, 0.1)).to(dtype)
    cos, sin = (t.to(cuda_device) for t in rope_tables(hd, 64, theta))
    positions = torch.cat([torch.arange(c, c + n) for c, n in zip(ctx, q_lens)]).int().to(cuda_device)
    token_row = torch.repeat_interleave(torch.arange(R), torch.tensor(q_lens)).int().to(cuda_device)
    num_pages = 40
    table, tables = make_tables([c + n for c, n in zip(ctx, q_lens)], page, num_pages, 23)
    cache = torch.full((num_pages, 2, nkv, page, hd), float("nan"), dtype=dtype, device=cuda_device)
    status = ops.new_status(cuda_device)
    q = ops.qk_norm_rope_cache(qkv, nh, nkv, hd, wq, wk, eps, cos, sin, positions, token_row, cache,
                               table.to(cuda_device), status)
    ops.check_status(status)
    x = qkv.double().cpu()
    pos = positions.cpu()
    q_ref = ref_rope(ref_rmsnorm(x[:, : nh * hd].view(T, nh, hd), wq.cpu(), eps), pos, theta)
    k_ref = ref_rope(ref_rmsnorm(x[:, nh * hd: (nh + nkv) * hd].view(T, nkv, hd), wk.cpu(), eps), pos, theta)
    v_ref = x[:, (nh + nkv) * hd:].view(T, nkv, hd)
    assert (q.double().cpu().view(T, nh, hd) - q_ref).abs().max() <= tol(dtype, 8.0)
    cache_cpu = cache.double().cpu()
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for t in range(T):
        r, p = int(token_row[t]), int(pos[t])
        pg, off = tables[r][p // page], p % page
        written[pg, off] = True
        perm = ops.kv_row_permutation(p, hd, dtype)            # rows are stored with permuted 16-byte chunks
        assert (cache_cpu[pg, 0, :, off][:, perm] - k_ref[t]).abs().max() <= tol(dtype, 8.0)
        assert torch.equal(cache_cpu[pg, 1, :, off][:, perm], v_ref[t])
    # nothing else was touched
    untouched = cache_cpu[:, 0, 0, :, 0][~written]
    assert torch.isnan(untouched).all()

    # The separate kernels give the same q (float32: the same bits up to the norm's rounding).
    q2 = ops.rmsnorm(qkv[:, : nh * hd].contiguous().view(T, nh, hd), wq, eps).view(T, nh * hd)
    q2 = ops.rope(q2, nh, hd, cos, sin, positions, status)
    assert (q2.double() - q.double()).abs().max() <= tol(dtype, 8.0)
    k2 = ops.rmsnorm(qkv[:, nh * hd: (nh + nkv) * hd].contiguous().view(T, nkv, hd), wk, eps).view(T, nkv * hd)
    k2 = ops.rope(k2, nkv, hd, cos, sin, positions, status)
    cache2 = torch.zeros_like(cache)
    ops.kv_write(k2, qkv[:, (nh + nkv) * hd:], nkv, hd, positions, token_row, cache2, table.to(cuda_device), status)
    ops.check_status(status)
    mask = written[:, None, None, :, None].expand_as(cache_cpu)
    assert (cache2.double().cpu()[mask] - cache_cpu[mask]).abs().max() <= tol(dtype, 8.0)


def test_cache_write_reports_bad_page_and_position(ops, cuda_device):
    from zephyr_b200.parts import rope_tables

    nh, nkv, hd, page = 2, 1, 16, 4
    qkv = rand((2, (nh + 2 * nkv) * hd), torch.float32, cuda_device, 30)
    cos, sin = (t.to(cuda_device) for t in rope_tables(hd, 8, 10000.0))
    cache = torch.zeros((6, 2, nkv, page, hd), device=cuda_device)
    token_row = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    status = ops.new_status(cuda_device)
    table = torch.tensor([[9]], dtype=torch.int32, device=cuda_device)       # page 9 of 6
    ops.qk_norm_rope_cache(qkv, nh, nkv, hd, None, None, 0.0, cos, sin,
                           torch.tensor([0, 1], dtype=torch.int32, device=cuda_device), token_row, cache, table, status)
    with pytest.raises(ops.KernelError, match="page id"):
        ops.check_status(status)
    table = torch.tensor([[1, 2, 3]], dtype=torch.int32, device=cuda_device)
    ops.qk_norm_rope_cache(qkv, nh, nkv, hd, None, None, 0.0, cos, sin,
                           torch.tensor([7, 8], dtype=torch.int32, device=cuda_device), token_row, cache, table, status)
    with pytest.raises(ops.KernelError, match="position"):
        ops.check_status(status)


# --------------------------------------------------------------------- attention
def ref_attention_row(q, K, V, ctx, q_len, window, nh, nkv, slopes=None):
    """q [q_len, nh, hd]; K, V [ctx + q_len, nkv, hd] doubles; the new tokens sit at ctx..ctx+q_len-1.
    ``slopes`` [nh]: head h adds slopes[h] * (key position - query position) to its scores."""
    hd = q.shape[-1]
    g = nh // nkv
    out = torch.zeros_like(q)
    for i in range(q_len):
        p = ctx + i
        lo = max(0, p - window + 1) if window > 0 else 0
        for h in range(nh):
            s = (K[lo:p + 1, h // g] @ q[i, h]) / math.sqrt(hd)
            if slopes is not None:
                s = s + float(slopes[h]) * (torch.arange(lo, p + 1, dtype=torch.float64) - p)
            out[i, h] = torch.softmax(s, 0) @ V[lo:p + 1, h // g]
    return out


def build_paged_case(device, dtype, nh, nkv, hd, page, q_lens, ctx, seed, spike=None):
    """Dense random K/V per row placed into shuffled pages of a NaN-filled cache.
    ``spike=(row, key_position)`` scales that key and the row's last query so that this one key,
    however far away, must dominate the softmax."""
    R = len(q_lens)
    totals = [c + n for c, n in zip(ctx, q_lens)]
    num_pages = sum(-(-n // page) for n in totals) + 3
    table, tables = make_tables(totals, page, num_pages, seed)
    cache = torch.full((num_pages, 2, nkv, page, hd), float("nan"), dtype=dtype, device=device)
    Ks, Vs, qs = [], [], []
    for r in range(R):
        K = rand((totals[r], nkv, hd), dtype, "cpu", seed + 10 * r + 1)
        V = rand((totals[r], nkv, hd), dtype, "cpu", seed + 10 * r + 2)
        q = rand((q_lens[r], nh, hd), dtype, "cpu", seed + 10 * r + 3)
        if spike is not None and spike[0] == r:
            direction = torch.ones(hd) / math.sqrt(hd)
            K[spike[1]] = (direction * 6.0).to(dtype)
            q[-1] = (direction * 6.0 * math.sqrt(hd) / 2).to(dtype)
        Ks.append(K), Vs.append(V), qs.append(q)
        from zephyr_b200.kernels.ops import kv_row_permutation

        for p in range(totals[r]):
            pg, off = tables[r][p // page], p % page
            inverse = torch.argsort(kv_row_permutation(p, hd, dtype))     # stored[j] = logical[inverse[j]]
            cache[pg, 0, :, off] = K[p][:, inverse].to(device)
            cache[pg, 1, :, off] = V[p][:, inverse].to(device)
    q_all = torch.cat(qs).reshape(-1, nh * hd).to(device)
    meta = dict(
        table=table.to(device),
        row_q_start=torch.tensor([sum(q_lens[:r]) for r in range(R)], dtype=torch.int32, device=device),
        row_q_len=torch.tensor(q_lens, dtype=torch.int32, device=device),
        row_ctx=torch.tensor(ctx, dtype=torch.int32, device=device))
    return q_all, cache, meta, Ks, Vs, qs


def tiles_for(q_lens, tile_tokens, device, only_multi=False):
    rows, q0s = [], []
    for r, n in enumerate(q_lens):
        if only_multi and n == 1:
            continue
        for q0 in range(0, n, tile_tokens):
            rows.append(r), q0s.append(q0)
    return (torch.tensor(rows, dtype=torch.int32, device=device), torch.tensor(q0s, dtype=torch.int32, device=device))


SIMT_CASES = [
    # nh, nkv, hd, page, window
    (4, 2, 16, 4, 0), (6, 3, 32, 8, 0), (8, 2, 48, 16, 24), (16, 8, 128, 16, 0), (3, 3, 80, 4, 7),
    (20, 1, 64, 32, 0), (5, 1, 256, 64, 100), (9, 3, 112, 16, 0),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,page,window", SIMT_CASES)
def test_paged_attention_general(ops, cuda_device, dtype, nh, nkv, hd, page, window):
    q_lens, ctx = [1, 37, 2, 1, 70], [130, 0, 63, 0, 41]
    q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, dtype, nh, nkv, hd, page, q_lens, ctx, 100)
    tile_tokens = ops.attention_tile_tokens(nh // nkv)
    tile_row, tile_q0 = tiles_for(q_lens, tile_tokens, cuda_device)
    status = ops.new_status(cuda_device)
    out = ops.paged_attention(q, cache, meta["table"], tile_row, tile_q0, tile_tokens, meta["row_q_start"],
                              meta["row_q_len"], meta["row_ctx"], nh, nkv, hd, window, 1 / math.sqrt(hd), status)
    ops.check_status(status)
    got = out.double().cpu().view(-1, nh, hd)
    cursor = 0
    for r, n in enumerate(q_lens):
        expected = ref_attention_row(qs[r].double(), Ks[r].double(), Vs[r].double(), ctx[r], n, window, nh, nkv)
        error = (got[cursor:cursor + n] - expected).abs().max()
        assert torch.isfinite(got[cursor:cursor + n]).all()
        assert error <= tol(dtype, 2.0), f"row {r}: {error}"
        cursor += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,page,window", [(4, 2, 16, 4, 0), (6, 3, 32, 8, 20), (16, 8, 128, 16, 0)])
def test_paged_attention_with_a_bias_on_the_scores(ops, cuda_device, dtype, nh, nkv, hd, page, window):
    """A slope per query head times the distance between key and query, added to the scores: steep
    for some heads (they see little but the nearest keys), zero for one."""
    q_lens, ctx = [1, 37, 2, 70], [130, 0, 63, 41]
    q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, dtype, nh, nkv, hd, page, q_lens, ctx, 101)
    slopes = torch.tensor([0.0 if h == 1 else 2.0 ** -(h % 5) for h in range(nh)], dtype=torch.float32)
    tile_tokens = ops.attention_tile_tokens(nh // nkv)
    tile_row, tile_q0 = tiles_for(q_lens, tile_tokens, cuda_device)
    status = ops.new_status(cuda_device)
    out = ops.paged_attention(q, cache, meta["table"], tile_row, tile_q0, tile_tokens, meta["row_q_start"],
                              meta["row_q_len"], meta["row_ctx"], nh, nkv, hd, window, 1 / math.sqrt(hd), status,
                              head_slopes=slopes.to(cuda_device))
    ops.check_status(status)
    got = out.double().cpu().view(-1, nh, hd)
    plain = ops.paged_attention(q, cache, meta["table"], tile_row, tile_q0, tile_tokens, meta["row_q_start"],
                                meta["row_q_len"], meta["row_ctx"], nh, nkv, hd, window, 1 / math.sqrt(hd), status)
    assert torch.equal(out.view(-1, nh, hd)[:, 1], plain.view(-1, nh, hd)[:, 1])          # the head without a slope
    cursor = 0
    for r, n in enumerate(q_lens):
        expected = ref_attention_row(qs[r].double(), Ks[r].double(), Vs[r].double(), ctx[r], n, window, nh, nkv, slopes)
        assert (got[cursor:cursor + n] - expected).abs().max() <= tol(dtype, 2.0), f"row {r}"
        cursor += n
    assert (out.float() - plain.float()).abs().max() > 0.05                                 # and the slopes do matter


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_far_key_and_window_edge(ops, cuda_device, dtype):
    """One key among hundreds carries the softmax: at position 3 (far), and exactly at / just outside a window's edge."""
    nh, nkv, hd, page = 4, 2, 64, 16
    for window, key, visible in ((0, 3, True), (50, 700 - 50 + 1, True), (50, 700 - 50, False)):
        q_lens, ctx = [1, 5], [700, 696]
        for row in (0, 1):
            q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, dtype, nh, nkv, hd, page, q_lens, ctx, 200,
                                                          spike=(row, key))
            tile_tokens = ops.attention_tile_tokens(nh // nkv)
            tile_row, tile_q0 = tiles_for(q_lens, tile_tokens, cuda_device)
            status = ops.new_status(cuda_device)
            out = ops.paged_attention(q, cache, meta["table"], tile_row, tile_q0, tile_tokens, meta["row_q_start"],
                                      meta["row_q_len"], meta["row_ctx"], nh, nkv, hd, window, 1 / math.sqrt(hd),
                                      status)
            ops.check_status(status)
            got = out.double().cpu().view(-1, nh, hd)
            last = sum(q_lens[:row + 1]) - 1
            expected = ref_attention_row(qs[row].double(), Ks[row].double(), Vs[row].double(), ctx[row], q_lens[row],
                                         window, nh, nkv)[-1]
            assert (got[last] - expected).abs().max() <= tol(dtype, 2.0)
            spike_value = Vs[row][key].double()                        # what the output is if that key dominates
            dominated = (got[last, 0] - spike_value[0]).abs().max() <= 0.05
            assert dominated == visible


PREFILL_CASES = [(4, 2, 32, 8, 0), (16, 8, 128, 16, 0), (6, 6, 64, 4, 0), (32, 2, 128, 16, 0), (12, 3, 96, 32, 0),
                 (16, 8, 128, 16, 100), (6, 2, 64, 64, 17), (40, 1, 128, 16, 0)]


@pytest.mark.parametrize("nh,nkv,hd,page,window", PREFILL_CASES)
def test_paged_prefill_tensor_core(ops, cuda_device, nh, nkv, hd, page, window):
    """The tensor-core prompt kernel: portions of 2 to 300 tokens, with and without cached context
    before them (lower-right causal alignment), tile edges at 64 and 128, next to single-token rows
    that it must leave alone."""
    dtype = torch.bfloat16
    assert ops.paged_prefill_supported(nh, nkv, hd, dtype)
    q_lens = [2, 1, 129, 64, 300, 1, 17]
    ctx = [0, 50, 0, 63, 200, 7, 500]
    q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, dtype, nh, nkv, hd, page, q_lens, ctx, 500)
    tile_row, tile_q0 = tiles_for(q_lens, ops.paged_prefill_tile_tokens(), cuda_device, only_multi=True)
    status = ops.new_status(cuda_device)
    out = torch.full_like(q, float("nan"))
    ops.paged_prefill(q, cache, meta["table"], tile_row, tile_q0, meta["row_q_start"], meta["row_q_len"],
                      meta["row_ctx"], nh, nkv, hd, window, 1 / math.sqrt(hd), status, out=out)
    ops.check_status(status)
    got = out.double().cpu().view(-1, nh, hd)
    cursor = 0
    for r, n in enumerate(q_lens):
        if n == 1:
            assert torch.isnan(got[cursor]).all()              # a single-token row: untouched
        else:
            expected = ref_attention_row(qs[r].double(), Ks[r].double(), Vs[r].double(), ctx[r], n, window, nh, nkv)
            assert torch.isfinite(got[cursor:cursor + n]).all(), f"row {r}"
            error = (got[cursor:cursor + n] - expected).abs().max()
            assert error <= tol(dtype, 2.0), f"row {r} (context {ctx[r]}, {n} new): {error}"
        cursor += n


@pytest.mark.parametrize("page,window", [(8, 0), (16, 0), (32, 300), (64, 0), (128, 129), (256, 0)])
def test_paged_prefill_tensor_memory(ops, cuda_device, page, window):
    """The tcgen05 kernel (head size 128) at every page size it takes: portions that start and end
    inside tiles of 128 keys, contexts of several tiles (interior tiles arrive by TMA, edge tiles
    by 16-byte copies with zero fill; freed and unused cache rows hold NaN), a window that ends
    inside a tile, and the same inputs through the mma.sync kernel."""
    nh, nkv, hd, dtype = 6, 2, 128, torch.bfloat16
    q_lens = [130, 2, 257, 128, 1, 40]
    ctx = [0, 700, 383, 1, 9, 1000]
    q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, dtype, nh, nkv, hd, page, q_lens, ctx, 900 + page)
    tile_row, tile_q0 = tiles_for(q_lens, ops.paged_prefill_tile_tokens(), cuda_device, only_multi=True)
    outs = []
    for tensor_memory in (True, False):
        ops.USE_TCGEN05_PREFILL = tensor_memory
        try:
            status = ops.new_status(cuda_device)
            out = torch.full_like(q, float("nan"))
            ops.paged_prefill(q, cache, meta["table"], tile_row, tile_q0, meta["row_q_start"], meta["row_q_len"],
                              meta["row_ctx"], nh, nkv, hd, window, 1 / math.sqrt(hd), status, out=out)
            ops.check_status(status)
        finally:
            ops.USE_TCGEN05_PREFILL = True
        outs.append(out.double().cpu().view(-1, nh, hd))
    cursor = 0
    for r, n in enumerate(q_lens):
        if n > 1:
            expected = ref_attention_row(qs[r].double(), Ks[r].double(), Vs[r].double(), ctx[r], n, window, nh, nkv)
            for got, name in zip(outs, ("tcgen05", "mma.sync")):
                assert torch.isfinite(got[cursor:cursor + n]).all(), f"{name} row {r}"
                error = (got[cursor:cursor + n] - expected).abs().max()
                assert error <= tol(dtype, 2.0), f"{name} row {r} (context {ctx[r]}, {n} new): {error}"
        cursor += n


def test_paged_prefill_tensor_memory_growing_scores(ops, cuda_device):
    """Scores that grow along the context by far more than 2^8 from tile to tile: every tile moves
    the rows' shift and rescales the output kept in tensor memory."""
    nh, nkv, hd, page, dtype = 2, 1, 128, 16, torch.bfloat16
    n = 640
    q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, dtype, nh, nkv, hd, page, [n], [0], 77)
    direction = torch.ones(hd) / math.sqrt(hd)
    K = Ks[0].clone()
    for p in range(n):
        K[p, 0] = (direction * (0.05 * p)).to(dtype)                  # key p scores 0.05 p * |q|: about 12 per 128 keys in base 2
    Ks[0] = K
    qs[0][:] = (direction * 4.0 * math.sqrt(hd)).to(dtype)
    # rebuild the cache and the queries with the edited tensors
    from zephyr_b200.kernels.ops import kv_row_permutation
    table = meta["table"].cpu()
    for p in range(n):
        inverse = torch.argsort(kv_row_permutation(p, hd, dtype))
        cache[int(table[0, p // page]), 0, :, p % page] = K[p][:, inverse].to(cuda_device)
    q = qs[0].reshape(-1, nh * hd).to(cuda_device)
    tile_row, tile_q0 = tiles_for([n], ops.paged_prefill_tile_tokens(), cuda_device, only_multi=True)
    status = ops.new_status(cuda_device)
    out = torch.full_like(q, float("nan"))
    ops.paged_prefill(q, cache, meta["table"], tile_row, tile_q0, meta["row_q_start"], meta["row_q_len"], meta["row_ctx"],
                      nh, nkv, hd, 0, 1 / math.sqrt(hd), status, out=out)
    ops.check_status(status)
    expected = ref_attention_row(qs[0].double(), Ks[0].double(), Vs[0].double(), 0, n, 0, nh, nkv)
    got = out.double().cpu().view(-1, nh, hd)
    assert torch.isfinite(got).all()
    assert (got - expected).abs().max() <= tol(dtype, 2.0)


def test_paged_prefill_far_key_and_window_edge(ops, cuda_device):
    nh, nkv, hd, page = 4, 2, 64, 16
    for window, key, visible in ((0, 3, True), (50, 700 - 50 + 1, True), (50, 700 - 50, False)):
        q_lens, ctx = [150, 5], [551, 696]                         # both rows end at position 700
        for row in (0, 1):
            q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, torch.bfloat16, nh, nkv, hd, page, q_lens, ctx,
                                                          600, spike=(row, key))
            tile_row, tile_q0 = tiles_for(q_lens, ops.paged_prefill_tile_tokens(), cuda_device, only_multi=True)
            status = ops.new_status(cuda_device)
            out = torch.zeros_like(q)
            ops.paged_prefill(q, cache, meta["table"], tile_row, tile_q0, meta["row_q_start"], meta["row_q_len"],
                              meta["row_ctx"], nh, nkv, hd, window, 1 / math.sqrt(hd), status, out=out)
            ops.check_status(status)
            got = out.double().cpu().view(-1, nh, hd)
            last = sum(q_lens[:row + 1]) - 1
            expected = ref_attention_row(qs[row].double(), Ks[row].double(), Vs[row].double(), ctx[row], q_lens[row],
                                         window, nh, nkv)[-1]
            assert (got[last] - expected).abs().max() <= tol(torch.bfloat16, 2.0)
            dominated = (got[last, 0] - Vs[row][key].double()[0]).abs().max() <= 0.05
            assert dominated == visible


DECODE_CASES = [(4, 2, 32, 8, 0), (16, 8, 128, 16, 0), (8, 8, 64, 4, 0), (32, 2, 128, 16, 0), (12, 3, 96, 32, 0),
                (16, 8, 128, 16, 300), (6, 2, 64, 64, 0)]


@pytest.mark.parametrize("split_size", [None, 0, 32, 64, 256])       # 0: balanced items whatever the batch
@pytest.mark.parametrize("nh,nkv,hd,page,window", DECODE_CASES)
def test_paged_decode_split(ops, cuda_device, nh, nkv, hd, page, window, split_size):
    """The split-context decode kernel at context lengths around tile and split edges, mixed with
    multi-token rows that it must leave alone."""
    dtype = torch.bfloat16
    assert ops.paged_decode_supported(nh, nkv, hd, dtype)
    q_lens = [1, 1, 4, 1, 1, 1, 1, 1]
    ctx = [0, 15, 20, 63, 255, 256, 600, 1029]
    q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, dtype, nh, nkv, hd, page, q_lens, ctx, 300)
    rows = torch.tensor([r for r, n in enumerate(q_lens) if n == 1], dtype=torch.int32, device=cuda_device)
    status = ops.new_status(cuda_device)
    out = torch.full_like(q, float("nan"))
    for _ in range(2):          # twice: the second call finds the counters as the first one left them
        out.fill_(float("nan"))
        ops.paged_decode(q, cache, meta["table"], rows, meta["row_q_start"], meta["row_ctx"], max(ctx) + 1, nh, nkv,
                         hd, window, 1 / math.sqrt(hd), status, out=out, split_size=split_size)
    ops.check_status(status)
    got = out.double().cpu().view(-1, nh, hd)
    cursor = 0
    for r, n in enumerate(q_lens):
        if n == 1:
            expected = ref_attention_row(qs[r].double(), Ks[r].double(), Vs[r].double(), ctx[r], 1, window, nh, nkv)
            error = (got[cursor:cursor + 1] - expected).abs().max()
            assert error <= tol(dtype, 2.0), f"row {r} (context {ctx[r]}): {error}"
        else:
            assert torch.isnan(got[cursor:cursor + n]).all()      # not a decode row: untouched
        cursor += n


@pytest.mark.parametrize("split_size", [None, 0, 64])
@pytest.mark.parametrize("nh,nkv,hd,page,window,norms,rotate", [
    (16, 8, 128, 16, 0, True, True), (4, 2, 32, 8, 0, True, True), (12, 3, 96, 32, 0, False, True),
    (8, 8, 64, 4, 0, True, False), (16, 8, 128, 16, 300, True, True), (6, 2, 64, 64, 0, False, False)])
def test_paged_decode_with_the_position_encoding_inside(ops, cuda_device, nh, nkv, hd, page, window, norms, rotate, split_size):
    """Norms, rotation, the cache write of the new key and value and the attention in one kernel give
    what the two kernels give one after the other, bit for bit: the attention's result and the
    cache.  Contexts around tile, page and split edges; the new position is a page's first, a
    page's last, a tile's first and so on."""
    dtype = torch.bfloat16
    ctx = [0, 15, 16, 31, 32, 63, 255, 256, 600, 1029]
    R = len(ctx)
    _, cache, meta, _, _, _ = build_paged_case(cuda_device, dtype, nh, nkv, hd, page, [1] * R, ctx, 700)
    cache = torch.nan_to_num(cache, nan=0.0)          # rows nobody wrote compare equal
    width = (nh + 2 * nkv) * hd
    qkv = rand((R, width + 16), dtype, cuda_device, 701, 2.0)[:, :width]        # rows further apart than they are long
    q_norm = (1 + rand((hd,), torch.float32, cuda_device, 702, 0.1)).to(dtype) if norms else None
    k_norm = (1 + rand((hd,), torch.float32, cuda_device, 703, 0.1)).to(dtype) if norms else None
    positions = torch.arange(1100, dtype=torch.float32, device=cuda_device)[:, None]
    freq = 1.0 / (10000.0 ** (torch.arange(hd // 2, dtype=torch.float32, device=cuda_device) / (hd // 2)))
    cos, sin = (torch.cos(positions * freq).contiguous(), torch.sin(positions * freq).contiguous()) if rotate else (None, None)
    rows = torch.arange(R, dtype=torch.int32, device=cuda_device)
    scale, eps = 1 / math.sqrt(hd), 1e-6
    status = ops.new_status(cuda_device)

    two_cache = cache.clone()
    q = ops.qk_norm_rope_cache(qkv, nh, nkv, hd, q_norm, k_norm, eps, cos, sin, meta["row_ctx"], rows, two_cache,
                               meta["table"], status)
    two = torch.empty_like(q)
    ops.paged_decode(q, two_cache, meta["table"], rows, meta["row_q_start"], meta["row_ctx"], max(ctx) + 1, nh, nkv, hd,
                     window, scale, status, out=two, split_size=split_size)
    one_cache = cache.clone()
    one = torch.full_like(q, float("nan"))
    for _ in range(2):          # the second call finds the counters as the first left them, and the cache written
        ops.paged_decode_fused(qkv, one_cache, meta["table"], rows, meta["row_q_start"], meta["row_ctx"], max(ctx) + 1,
                               nh, nkv, hd, window, scale, q_norm, k_norm, eps, cos, sin, status, one, split_size=split_size)
    ops.check_status(status)
    assert torch.equal(one_cache, two_cache)
    assert torch.equal(one, two)


def test_paged_decode_far_key(ops, cuda_device):
    nh, nkv, hd, page = 16, 8, 128, 16
    for key in (2, 255, 256, 511, 900):
        q_lens, ctx = [1, 1], [1000, 1000]
        q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, torch.bfloat16, nh, nkv, hd, page, q_lens, ctx, 400,
                                                      spike=(1, key))
        rows = torch.tensor([0, 1], dtype=torch.int32, device=cuda_device)
        status = ops.new_status(cuda_device)
        out = torch.zeros_like(q)
        ops.paged_decode(q, cache, meta["table"], rows, meta["row_q_start"], meta["row_ctx"], 1001, nh, nkv, hd, 0,
                         1 / math.sqrt(hd), status, out=out)
        ops.check_status(status)
        got = out.double().cpu().view(-1, nh, hd)
        assert (got[1, 0] - Vs[1][key].double()[0]).abs().max() <= 0.05
        expected = ref_attention_row(qs[1].double(), Ks[1].double(), Vs[1].double(), 1000, 1, 0, nh, nkv)
        assert (got[1:2] - expected).abs().max() <= tol(torch.bfloat16, 2.0)


@pytest.mark.parametrize("split_size", [None, 0, 64])
@pytest.mark.parametrize("hd,page,window", [(128, 16, 300), (64, 8, 24), (32, 8, 129)])
def test_paged_decode_window_edge(ops, cuda_device, hd, page, window, split_size):
    """The window's edge on the fast decode path: the new token at position 1000 sees the positions
    above 1000 - window.  A key made to dominate the softmax just inside the window (1001 - window)
    decides the output; the same key one position further back (1000 - window) must not count at all.
    The pages that lie wholly before the window are given back by the cache manager: the table holds
    the null page there, whose contents are NaN here, so a kernel that reads them shows up."""
    nh, nkv = 8, 4
    for key, visible in ((1001 - window, True), (1000 - window, False)):
        q, cache, meta, Ks, Vs, qs = build_paged_case(cuda_device, torch.bfloat16, nh, nkv, hd, page, [1, 1], [1000, 1000],
                                                      410, spike=(1, key))
        table = meta["table"].clone()
        table[:, : (1001 - window) // page] = 0           # released blocks: the null page, all NaN
        assert torch.isnan(cache[0]).all()
        rows = torch.tensor([0, 1], dtype=torch.int32, device=cuda_device)
        status = ops.new_status(cuda_device)
        out = torch.zeros_like(q)
        ops.paged_decode(q, cache, table, rows, meta["row_q_start"], meta["row_ctx"], 1001, nh, nkv, hd, window,
                         1 / math.sqrt(hd), status, out=out, split_size=split_size)
        ops.check_status(status)
        got = out.double().cpu().view(-1, nh, hd)
        assert torch.isfinite(got).all()
        expected = ref_attention_row(qs[1].double(), Ks[1].double(), Vs[1].double(), 1000, 1, window, nh, nkv)
        assert (got[1:2] - expected).abs().max() <= tol(torch.bfloat16, 2.0)
        near = (got[1, 0] - Vs[1][key].double()[0]).abs().max()
        assert (near <= 0.05) == visible, (key, float(near))


def test_kernels_refuse_what_they_do_not_take(ops, cuda_device):
    assert not ops.paged_decode_supported(16, 8, 128, torch.float32)
    assert not ops.paged_decode_supported(34, 2, 128, torch.bfloat16)     # 17 heads per group
    assert not ops.paged_decode_supported(4, 2, 48, torch.bfloat16)
    q = torch.zeros((1, 2 * 24), device=cuda_device)
    cache = torch.zeros((3, 2, 2, 4, 24), device=cuda_device)
    z = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    with pytest.raises(ops.KernelError, match="does not support"):
        ops.paged_attention(q, cache, z.view(1, 1), z, z, 1, z, z, z, 2, 2, 24, 0, 1.0, ops.new_status(cuda_device))
    with pytest.raises(ops.KernelError):
        ops.rmsnorm(torch.zeros(4, 4), torch.ones(4), 1e-6)               # CPU tensors: no CPU path


# ------------------------------------------------------------------ chains of small products
def _plain_rmsnorm(x, w, eps):
    x = x.float()
    return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float())


@pytest.mark.parametrize("M,d,q,ffn,qkv", [(1, 1024, 2048, 3072, 4096), (8, 1024, 2048, 3072, 4096), (16, 320, 256, 880, 384),
                                           (5, 2056, 1032, 4112, 136), (13, 64, 2304, 48, 8),
                                           # long rows: normalised once, by the CTA of the row's number
                                           (8, 4096, 512, 264, 136), (3, 4608, 128, 136, 72)])
def test_fused_chain_matches_plain(ops, cuda_device, M, d, q, ffn, qkv):
    """A layer's tail as one chain: output projection; residual add, norm, gate/up with silu * up;
    down projection; residual add, norm, the next projection.  Against float64 products of the same
    bfloat16 inputs, with the roundings the chain makes (every stored tensor is bfloat16)."""
    g = torch.Generator().manual_seed(M * 1000 + d)
    rnd = lambda *shape, scale=1.0: (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(cuda_device)
    attn, residual = rnd(M, q), rnd(M, d)
    w_o, w_gu, w_down, w_qkv = rnd(d, q, scale=q ** -0.5), rnd(2 * ffn, d, scale=d ** -0.5), rnd(d, ffn, scale=ffn ** -0.5), rnd(qkv, d, scale=d ** -0.5)
    norm1 = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16).to(cuda_device)
    norm2 = (1 + 0.1 * torch.randn(d, generator=g)).to(cuda_device)          # a float32 scale
    eps1, eps2 = 1e-6, 3e-5
    empty = lambda *shape: torch.full(shape, float("nan"), dtype=torch.bfloat16, device=cuda_device)
    o, act, down, out = empty(M, d), empty(M, ffn), empty(M, d), empty(M, qkv)
    residual1, residual2 = empty(M, d), empty(M, d)
    stages = [ops.ChainStage(w=w_o, y=o, x=attn),
              ops.ChainStage(w=w_gu, y=act, residual_in=residual, residual_out=residual1, delta=o, norm_w=norm1, eps=eps1, swiglu=True),
              ops.ChainStage(w=w_down, y=down, x=act),
              ops.ChainStage(w=w_qkv, y=out, residual_in=residual1, residual_out=residual2, delta=down, norm_w=norm2, eps=eps2)]
    for stage, normed in zip(stages, (False, True, False, True)):
        assert ops.fused_chain_stage_supported(M, stage.w, normed, stage.swiglu)
    status = ops.new_status(cuda_device)
    for _ in range(3):                                   # the barrier's counters are left at zero each time
        ops.fused_chain(stages, M, status)
    ops.check_status(status)

    bf = lambda t: t.to(torch.bfloat16)
    mm = lambda x, w: (x.double() @ w.double().t()).float()
    want_o = bf(mm(attn, w_o))
    want_r1 = bf(residual.float() + want_o.float())
    x1 = bf(_plain_rmsnorm(want_r1, norm1, eps1))
    gu = mm(x1, w_gu).view(M, ffn // 8, 2, 8)
    want_act = bf((torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(M, ffn))
    want_down = bf(mm(want_act, w_down))
    want_r2 = bf(want_r1.float() + want_down.float())
    x2 = bf(_plain_rmsnorm(want_r2, norm2, eps2))
    want_out = bf(mm(x2, w_qkv))
    # bfloat16 stores: one unit in the last place of a value, and a little more where an input
    # rounded the other way upstream.
    for got, want, name in ((o, want_o, "o"), (residual1, want_r1, "residual1"), (act, want_act, "act"),
                            (down, want_down, "down"), (residual2, want_r2, "residual2"), (out, want_out, "out")):
        assert torch.isfinite(got.float()).all(), name
        scale = float(want.float().abs().max())
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2 * scale, msg=lambda m: f"{name}: {m}")


def test_fused_chain_refuses_what_it_cannot_run(ops, cuda_device):
    w = torch.zeros((24, 64), dtype=torch.bfloat16, device=cuda_device)
    assert ops.fused_chain_stage_supported(4, w, False, False)
    assert not ops.fused_chain_stage_supported(4, w, False, True)          # 24 rows are no whole gate/up blocks
    assert not ops.fused_chain_stage_supported(17, w, False, False)
    assert not ops.fused_chain_stage_supported(4, w[:, :60], False, False)
    big = torch.zeros((8, 65536), dtype=torch.bfloat16, device=cuda_device)
    assert not ops.fused_chain_stage_supported(16, big, True, False)       # the normalised rows would not fit
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device=cuda_device)
    y = torch.zeros((4, 20), dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ops.KernelError):
        ops.fused_chain([ops.ChainStage(w=w[:20], y=y, x=x)], 4, ops.new_status(cuda_device))


# ---------------------------------------------------------------------- sampling
def test_argmax_lowest_index_on_ties(ops, cuda_device):
    logits = torch.full((3, 151936), -1.0, device=cuda_device)
    logits[0, [77, 5000, 151935]] = 3.0
    logits[1, 151935] = 0.5
    logits[2, 0] = 0.0
    status = ops.new_status(cuda_device)
    assert ops.sample(logits, status).tolist() == [77, 151935, 0]
    assert ops.sample(logits, status).tolist() == [77, 151935, 0]       # the arrival counters were left at zero
    ops.check_status(status)


def test_temperature_sampling_follows_the_prefix_sums(ops, cuda_device):
    from plain_qwen3 import plain_sample

    for V in (311, 5000, 151936):
        g = torch.Generator().manual_seed(V)
        logits = (torch.randn((16, V), generator=g) * 2).to(cuda_device)
        temperature = [0.7, 1.0, 0.3, 1.5] * 4
        temperature[5] = 0.0            # a greedy row among sampled ones
        uniform = torch.rand(16, generator=g).tolist()
        status = ops.new_status(cuda_device)
        rows = [ops.SampleRow(temperature=t, uniform=u) for t, u in zip(temperature, uniform)]
        got = ops.sample_rows(logits, rows, status).ids.tolist()
        ops.check_status(status)
        for r in range(16):
            if r == 5:
                assert got[r] == int(logits[r].argmax())
                continue
            index, margin = plain_sample(logits[r].cpu(), temperature[r], uniform[r])
            if margin > 1e-4:
                assert got[r] == index, (V, r, got[r], index, margin)
            # Always: u * total lies in the chosen token's interval of the exact prefix sums, give or
            # take what float32 prefix sums over V terms can differ by.
            z = (logits[r].double().cpu() - logits[r].double().max().cpu()) / temperature[r]
            cdf = torch.cumsum(torch.exp(z), 0)
            target, slack = uniform[r] * float(cdf[-1]), 1e-4 * float(cdf[-1])
            assert float(cdf[got[r]]) >= target - slack
            assert (float(cdf[got[r] - 1]) if got[r] > 0 else 0.0) <= target + slack


FILTERS = [dict(top_k=1), dict(top_k=7), dict(top_k=300), dict(top_p=0.9), dict(top_p=0.3), dict(top_k=40, top_p=0.8),
           dict(min_p=0.05), dict(top_k=50, min_p=0.1), dict(top_p=0.95, min_p=0.02), dict(top_k=20, top_p=0.5, min_p=0.2),
           dict(top_k=10 ** 9), dict(top_p=0.999), dict(top_k=6000), dict(top_k=5000, top_p=0.7), dict(top_k=4096, top_p=0.99)]


def test_filtered_sampling_matches_the_plain_sampler(ops, cuda_device):
    """top-k, top-p and min-p, alone and together, at three vocabulary sizes.  A row is compared
    token for token unless the plain sampler says that one of its decisions was a near tie."""
    import plain_sampler

    compared = 0
    decided_in_head, decided_by_whole_order = 0, 0
    for V, spread, peaks in ((311, 2.0, 0), (5000, 3.0, 0), (151936, 4.0, 0), (151936, 1.0, 0), (151936, 1.5, 40)):
        g = torch.Generator().manual_seed(V + 1)
        logits = (torch.randn((len(FILTERS) * 2, V), generator=g) * spread)
        if peaks:       # a few tokens far above a broad bulk, as a trained model's logits are
            for r in range(logits.shape[0]):
                at = torch.randperm(V, generator=g)[:peaks]
                logits[r, at] += 8.0 + 6.0 * torch.rand(peaks, generator=g)
        uniform = torch.rand(logits.shape[0], generator=g).tolist()
        rows = []
        for r in range(logits.shape[0]):
            f = FILTERS[r % len(FILTERS)]
            rows.append(ops.SampleRow(temperature=0.6 + 0.1 * (r % 7), uniform=uniform[r],
                                      top_k=min(f.get("top_k", 0), V), top_p=f.get("top_p", 0.0),
                                      min_p=f.get("min_p", 0.0)))
        status = ops.new_status(cuda_device)
        got = ops.sample_rows(logits.to(cuda_device), rows, status).ids.tolist()
        ops.check_status(status)
        state = ops.last_sample_job_state()
        assert len(state) == sum(1 for row in rows if row.ranked)
        for sorted_ranks, head_was_enough in state:
            assert sorted_ranks == V or (head_was_enough and 0 < sorted_ranks <= 4096)
            decided_in_head += head_was_enough
            decided_by_whole_order += not head_was_enough
        for r, row in enumerate(rows):
            want, margin = plain_sampler.sample(logits[r], row.temperature, row.uniform, row.top_k, row.top_p or 1.0,
                                                row.min_p)
            if margin > 1e-5:
                assert got[r] == want, (V, r, FILTERS[r % len(FILTERS)], got[r], want, margin)
                compared += 1
            # Always: the token lies inside what the filters keep, give or take a near tie at the edge.
            p = torch.softmax(plain_sampler.scale(logits[r], row.temperature), 0)
            order = plain_sampler.rank(p).tolist()
            if row.top_k:
                assert order.index(got[r]) < row.top_k
            if row.min_p:
                assert float(p[got[r]]) > row.min_p * float(p.max()) * (1 - 1e-5)
    assert compared >= 0.75 * 5 * 2 * len(FILTERS)        # most rows were decided clearly and compared exactly
    # Both ways of ranking were at work: the head of the order alone, and the whole vocabulary.
    assert decided_in_head >= 20 and decided_by_whole_order >= 20, (decided_in_head, decided_by_whole_order)


def test_ranked_draw_takes_equal_weights_in_index_order(ops, cuda_device):
    """Five tokens share the largest logit.  With top_k = 5 each holds a fifth of the mass, and the
    draw walks them by ascending index whatever their place in the vocabulary."""
    V = 70000
    tied = [69999, 3, 40000, 512, 4097]
    logits = torch.full((5, V), -20.0)
    logits[:, tied] = 1.5
    rows = [ops.SampleRow(temperature=1.0, uniform=0.1 + 0.2 * r, top_k=5) for r in range(5)]
    status = ops.new_status(cuda_device)
    got = ops.sample_rows(logits.to(cuda_device), rows, status).ids.tolist()
    ops.check_status(status)
    assert got == sorted(tied)


def test_ranking_is_a_stable_sort_of_the_whole_vocabulary(ops, cuda_device):
    """A report of as many tokens as the vocabulary has shows the whole ranking: by value,
    descending, equal values by index; values that underflow as probabilities still rank by z."""
    import plain_sampler

    for V in (33, 1000, 4097, 50001):
        g = torch.Generator().manual_seed(V)
        logits = torch.randn((2, V), generator=g) * 3
        logits[0] = torch.round(logits[0] * 2) / 2            # many equal values
        logits[1, ::3] -= 200.0                               # exp underflows to zero for a third of the row
        rows = [ops.SampleRow(temperature=0.0, num_logprobs=V), ops.SampleRow(temperature=0.5, uniform=0.3, num_logprobs=V)]
        status = ops.new_status(cuda_device)
        out = ops.sample_rows(logits.to(cuda_device), rows, status)
        ops.check_status(status)
        ids, values = out.ids.tolist(), out.logprobs.tolist()
        for r, row in enumerate(rows):
            at = out.offsets[r]
            chosen, best = plain_sampler.report(logits[r], row.temperature, ids[at], V)
            assert ids[at + 1:at + 1 + V] == [token for token, _ in best], (V, r)
            assert abs(values[at] - chosen) <= 1e-4 * max(1.0, abs(chosen))
            for got, (_, want) in zip(values[at + 1:at + 1 + V], best):
                assert abs(got - want) <= 1e-4 * max(1.0, abs(want))
        assert out.offsets == [0, V + 1]


def test_penalties_and_biases(ops, cuda_device):
    """Adjustments change the logits in place, once per token, before anything else looks at them."""
    import plain_sampler

    V = 5000
    g = torch.Generator().manual_seed(9)
    logits = torch.randn((3, V), generator=g) * 2
    histories = [torch.randint(0, V, (60,), generator=g).tolist() for _ in range(3)]
    histories[1] += histories[1][-5:] * 3                      # tokens generated several times
    prompt_lengths = [20, 10, 60]
    settings = [dict(frequency_penalty=0.4, presence_penalty=0.3), dict(repetition_penalty=1.7, frequency_penalty=0.2),
                dict(repetition_penalty=0.8)]
    biases = [{7: 50.0, histories[0][30]: -3.0}, {}, {11: float("-inf"), 12: 2.5}]
    want = [plain_sampler.adjust(logits[r], histories[r], prompt_lengths[r], bias=biases[r], **settings[r]) for r in range(3)]
    adjustments = []
    for r in range(3):
        merged = {}
        for position, token in enumerate(histories[r]):
            entry = merged.setdefault(token, [0, True, 0.0])
            entry[0] += position >= prompt_lengths[r]
        for token, bias in biases[r].items():
            merged.setdefault(token, [0, False, 0.0])[2] = bias
        adjustments += [ops.TokenAdjustment(r, t, c, s, b) for t, (c, s, b) in merged.items()]
    rows = [ops.SampleRow(temperature=0.0, num_logprobs=3, **settings[r]) for r in range(3)]
    device_logits = logits.to(cuda_device)
    status = ops.new_status(cuda_device)
    out = ops.sample_rows(device_logits, rows, status, adjustments)
    ops.check_status(status)
    torch.testing.assert_close(device_logits.cpu(), torch.stack(want), rtol=1e-6, atol=1e-6)
    ids, values = out.ids.tolist(), out.logprobs.tolist()
    for r in range(3):
        at = out.offsets[r]
        assert ids[at] == int(plain_sampler.rank(want[r].double())[0])
        chosen, best = plain_sampler.report(want[r], 0.0, ids[at], 3)
        assert ids[at + 1:at + 4] == [t for t, _ in best]
        assert abs(values[at] - chosen) <= 1e-4
    assert ids[out.offsets[0]] == 7                            # the bias of +50 wins its row


def test_sampling_reports_nan(ops, cuda_device):
    logits = torch.zeros((2, 100), device=cuda_device)
    logits[1, 7] = float("nan")
    status = ops.new_status(cuda_device)
    ops.sample(logits, status)
    with pytest.raises(ops.KernelError, match="NaN"):
        ops.check_status(status)
    # A row that a bias of -inf everywhere leaves without a finite maximum is reported too, and the
    # kernels that follow leave it alone instead of dividing by an empty mass.
    logits = torch.full((1, 64), float("-inf"), device=cuda_device)
    status = ops.new_status(cuda_device)
    ops.sample_rows(logits, [ops.SampleRow(temperature=0.8, uniform=0.5, top_k=5, num_logprobs=2)], status)
    with pytest.raises(ops.KernelError):
        ops.check_status(status)
