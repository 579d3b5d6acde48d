"""Each kernel alone against a plain float32 reference of the same operation, at sizes other
than the engine's: tails, odd widths, sizes that are no power of two."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def rand(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embed(status, table_dtype):
    from sprout_lm_b200 import kernels
    table = rand(101, 72, dtype=table_dtype)
    tokens = torch.tensor([0, 100, 5, 5, 37], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, dtype=torch.float32, device=DEV)
    kernels.embed(table, tokens, out, status)
    assert torch.equal(out, table[tokens.long()].float())
    assert int(status.item()) == 0
    bad = torch.tensor([3, 101], dtype=torch.int32, device=DEV)
    kernels.embed(table, bad, out[:2], status)                    # flagged, not faulted
    assert int(status.item()) & 2
    status.zero_()


@pytest.mark.parametrize("hidden,eps", [(72, 1e-6), (896, 1e-5), (1000, 1e-6), (4100, 1e-5)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(hidden, eps, out_dtype):
    from sprout_lm_b200 import kernels
    x = rand(7, hidden, scale=3.0)
    gain = 1 + rand(hidden, scale=0.1, seed=1)
    out = torch.empty(7, hidden, dtype=out_dtype, device=DEV)
    kernels.rmsnorm(x, gain, out, eps)
    x64 = x.double()
    want = (x64 / torch.sqrt((x64 * x64).mean(-1, keepdim=True) + eps)).float().double() * gain.double()
    tol = 2e-6 if out_dtype == torch.float32 else 8e-3
    assert (out.double() - want).abs().max().item() <= tol * want.abs().max().item()
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    picked = torch.empty(3, hidden, dtype=out_dtype, device=DEV)
    kernels.rmsnorm(x, gain, picked, eps, rows)
    assert torch.equal(picked, out[rows.long()])


@pytest.mark.parametrize("hidden", [72, 896, 1000, 2048])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_many_rows(hidden, out_dtype):
    """A prefill's worth of rows takes the warp-per-row kernel: the same numbers as the
    block-per-row kernel gives for a few rows, to the last bit of the output's rounding."""
    from sprout_lm_b200 import kernels
    rows, eps = 203, 1e-6
    x = rand(rows, hidden, scale=3.0, seed=4)
    gain = 1 + rand(hidden, scale=0.1, seed=1)
    out = torch.empty(rows, hidden, dtype=out_dtype, device=DEV)
    kernels.rmsnorm(x, gain, out, eps)
    x64 = x.double()
    want = (x64 / torch.sqrt((x64 * x64).mean(-1, keepdim=True) + eps)).float().double() * gain.double()
    tol = 2e-6 if out_dtype == torch.float32 else 8e-3
    assert (out.double() - want).abs().max().item() <= tol * want.abs().max().item()
    few = torch.empty(5, hidden, dtype=out_dtype, device=DEV)
    kernels.rmsnorm(x[100:105].contiguous(), gain, few, eps)
    assert (few.double() - out[100:105].double()).abs().max().item() <= tol * want.abs().max().item()


@pytest.mark.parametrize("heads,kv_heads,head_dim,page,theta", [(14, 2, 64, 16, 1e6), (8, 2, 128, 32, 1e4), (4, 2, 16, 8, 1e4), (3, 1, 48, 16, 1e5)])
@pytest.mark.parametrize("rotate", [True, False])
def test_rope_append_many_tokens(status, heads, kv_heads, head_dim, page, theta, rotate):
    """A prefill's worth of tokens takes the vectorised kernel (bfloat16): checked against the
    float64 rotation and against the cache slots that the block tables name."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.rope import HalfSplitRotary
    dtype = torch.bfloat16
    lengths = [97, 3, 130]                                   # tokens of three requests, from position 5, 0 and 40
    starts = [5, 0, 40]
    pages_each = [-(-(s0 + n) // page) for s0, n in zip(starts, lengths)]
    pool = sum(pages_each) + 2
    perm = torch.randperm(pool, generator=torch.Generator().manual_seed(3)).to(torch.int32)
    table = torch.full((3, max(pages_each)), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(pages_each):
        table[r, :n] = perm[at:at + n]
        at += n
    positions = torch.cat([torch.arange(s0, s0 + n, dtype=torch.int32) for s0, n in zip(starts, lengths)])
    seq_of_token = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(lengths)])
    T = positions.numel()

    class RT:
        device = torch.device(DEV)
    cos, sin = HalfSplitRotary("", head_dim, theta, 512).rotary_tables(RT) if rotate else (None, None)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = rand(T, width, dtype=dtype, seed=8)
    original = qkv.clone()
    k_cache = torch.zeros(pool, kv_heads, page, head_dim, dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    kernels.rope_append(qkv, positions.to(DEV), seq_of_token.to(DEV), table.to(DEV), cos, sin, k_cache, v_cache,
                        heads, kv_heads, head_dim, page, True, status)
    assert int(status.item()) == 0
    q0, k0 = original[:, :heads * head_dim], original[:, heads * head_dim:(heads + kv_heads) * head_dim]
    q_want = rope_reference(q0, positions, head_dim, theta) if rotate else q0.double().cpu()
    k_want = rope_reference(k0, positions, head_dim, theta) if rotate else k0.double().cpu()
    assert (qkv[:, :heads * head_dim].double().cpu() - q_want).abs().max().item() <= 6.4e-2
    assert torch.equal(qkv[:, heads * head_dim:], original[:, heads * head_dim:])       # k and v stay in qkv as projected
    pg = table[seq_of_token.long(), (positions // page).long()].long()
    slot = (positions % page).long()
    got_k = k_cache[pg.to(DEV), :, slot.to(DEV), :].reshape(T, -1).double().cpu()
    assert (got_k - k_want).abs().max().item() <= 6.4e-2
    assert torch.equal(v_cache[pg.to(DEV), :, slot.to(DEV), :].reshape(T, -1), original[:, (heads + kv_heads) * head_dim:])
    assert int((k_cache != 0).any(-1).any(1).sum().item()) == T                      # no other slot was touched
    # the few-token kernel gives the same bits
    few_q = original[:6].clone()
    k2, v2 = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    kernels.rope_append(few_q, positions[:6].to(DEV), seq_of_token[:6].to(DEV), table.to(DEV), cos, sin, k2, v2,
                        heads, kv_heads, head_dim, page, True, status)
    assert torch.equal(few_q, qkv[:6])
    assert torch.equal(k2[pg[:6].to(DEV), :, slot[:6].to(DEV), :], k_cache[pg[:6].to(DEV), :, slot[:6].to(DEV), :])
    # the same from float32 sums plus a bias (what a split-K product leaves): the rotated q lands in
    # qkv, k and v in the cache, the sums are cleared
    bias = rand(width, seed=9)
    acc = torch.zeros(T + 2, width, device=DEV)
    acc[:T] = original.float() - bias
    out_q = torch.zeros_like(original)
    k4, v4 = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    kernels.rope_append(out_q, positions.to(DEV), seq_of_token.to(DEV), table.to(DEV), cos, sin, k4, v4,
                        heads, kv_heads, head_dim, page, True, status, acc=acc[:T], bias=bias)
    assert (out_q[:, :heads * head_dim].float() - qkv[:, :heads * head_dim].float()).abs().max().item() <= 2e-2
    assert (k4.float() - k_cache.float()).abs().max().item() <= 2e-2
    assert (v4.float() - v_cache.float()).abs().max().item() <= 2e-2
    assert float(acc.abs().max()) == 0.0
    assert int((k4 != 0).any(-1).any(1).sum().item()) == T
    # without the cache write only q changes
    k3 = torch.zeros_like(k_cache)
    only_q = original.clone()
    kernels.rope_append(only_q, positions.to(DEV), seq_of_token.to(DEV), table.to(DEV), cos, sin, k3, v2.zero_(),
                        heads, kv_heads, head_dim, page, False, status)
    assert torch.equal(only_q, qkv) and float(k3.abs().max()) == 0.0 and float(v2.abs().max()) == 0.0
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [8, 320, 4864])
def test_swiglu_interleaved(dtype, inter):
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.mlp import interleave_gate_up
    gate, up = rand(5, inter, dtype=dtype, scale=2.0), rand(5, inter, dtype=dtype, scale=2.0, seed=3)
    fused = interleave_gate_up(gate.T.contiguous(), up.T.contiguous()).T.contiguous()   # columns interleaved like weight rows
    out = torch.empty(5, inter, dtype=dtype, device=DEV)
    kernels.swiglu(fused, out)
    g = gate.double()
    want = (g / (1 + torch.exp(-g))).float().double() * up.double()
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    assert (out.double() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
    with pytest.raises(kernels.KernelError, match="multiple of 8"):
        kernels.swiglu(torch.empty(2, 24, dtype=dtype, device=DEV), torch.empty(2, 12, dtype=dtype, device=DEV))


def rope_reference(x, positions, head_dim, theta):
    tokens = x.shape[0]
    heads = x.shape[1] // head_dim
    half = head_dim // 2
    d = torch.arange(half, dtype=torch.float64)
    angle = positions.double()[:, None, None] / theta ** (2 * d / head_dim)[None, None, :]
    xs = x.double().cpu().reshape(tokens, heads, head_dim)
    a, b = xs[..., :half], xs[..., half:]
    return torch.cat([a * angle.cos() - b * angle.sin(), b * angle.cos() + a * angle.sin()], -1).reshape(tokens, -1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page,theta", [(4, 2, 16, 16, 1e4), (3, 1, 32, 8, 1e6), (5, 5, 48, 4, 5e5), (14, 2, 64, 16, 1e6)])
def test_rope_append(status, dtype, heads, kv_heads, head_dim, page, theta):
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.rope import HalfSplitRotary
    max_pos, pages = 4096, 40
    rotary = HalfSplitRotary("", head_dim, theta, max_pos)

    class RT:
        device = torch.device(DEV)
    cos, sin = rotary.rotary_tables(RT)
    positions = torch.tensor([0, 1, page - 1, page, 3 * page + 1, 4095 % (pages * page // 2)], dtype=torch.int32)
    T = positions.numel()
    # two requests with scattered pages
    seq_of_token = torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.int32)
    max_pages = pages // 2
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    table = perm.reshape(2, max_pages).contiguous()
    width = (heads + 2 * kv_heads) * head_dim
    qkv = rand(T, width, dtype=dtype)
    original = qkv.clone()
    k_cache = torch.zeros(pages, kv_heads, page, head_dim, dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    kernels.rope_append(qkv, positions.to(DEV), seq_of_token.to(DEV), table.to(DEV), cos, sin, k_cache, v_cache,
                        heads, kv_heads, head_dim, page, True, status)
    assert int(status.item()) == 0
    q_want = rope_reference(original[:, :heads * head_dim], positions, head_dim, theta)
    k_want = rope_reference(original[:, heads * head_dim:(heads + kv_heads) * head_dim], positions, head_dim, theta)
    tol = 2e-6 if dtype == torch.float32 else 1.6e-2
    assert (qkv[:, :heads * head_dim].double().cpu() - q_want).abs().max().item() <= tol * 4
    for t in range(T):
        pos = int(positions[t])
        pg, slot = int(table[seq_of_token[t], pos // page]), pos % page
        got_k = k_cache[pg, :, slot, :].reshape(-1).double().cpu()
        assert (got_k - k_want[t]).abs().max().item() <= tol * 4
        got_v = v_cache[pg, :, slot, :].reshape(-1)
        assert torch.equal(got_v, original[t, (heads + kv_heads) * head_dim:])
    # nothing else was touched
    assert int((k_cache != 0).any(-1).any(1).sum().item()) == T
    # the same from float32 sums plus a bias (what a split-K product leaves): same rotation, the
    # rotated q lands in qkv, the sums are cleared
    bias = rand(width, seed=9)
    acc = torch.zeros(T + 2, width, device=DEV)
    acc[:T] = original.float() - bias
    out_q = torch.zeros_like(original)
    k2, v2 = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    kernels.rope_append(out_q, positions.to(DEV), seq_of_token.to(DEV), table.to(DEV), cos, sin, k2, v2,
                        heads, kv_heads, head_dim, page, True, status, acc=acc[:T], bias=bias)
    slack = 1e-5 if dtype == torch.float32 else 2e-2
    assert (out_q[:, :heads * head_dim].float() - qkv[:, :heads * head_dim].float()).abs().max().item() <= slack
    assert (k2.float() - k_cache.float()).abs().max().item() <= slack
    assert (v2.float() - v_cache.float()).abs().max().item() <= slack
    assert float(acc.abs().max()) == 0.0
    # a page id outside the pool is flagged and skipped
    bad = table.clone()
    bad[0, 0] = pages + 3
    kernels.rope_append(original.clone(), positions.to(DEV), seq_of_token.to(DEV), bad.to(DEV), cos, sin, k_cache,
                        v_cache, heads, kv_heads, head_dim, page, True, status)
    assert int(status.item()) & 1
    status.zero_()


# ------------------------------------------------------------------------------- matrix products
SHAPES = [(1, 1, 8), (1, 896, 896), (3, 130, 72), (8, 1152, 896), (17, 509, 96), (64, 256, 4864), (100, 77, 200),
          (128, 896, 896), (129, 300, 136), (257, 1000, 328), (600, 1152, 896), (2048, 896, 4864), (300, 512, 200),
          (1100, 1024, 896)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_simple_float32(M, N, K):
    from sprout_lm_b200 import kernels
    a, w, bias = rand(M, K), rand(N, K, seed=1), rand(N, seed=2)
    out = torch.empty(M, N, device=DEV)
    kernels.gemm_simple(a, w, out, bias=bias)
    want = a.double() @ w.double().T + bias.double()
    # sequential float32 accumulation: error grows like eps * sqrt(K) times the magnitude of the sums
    tol = 4 * 6e-8 * math.sqrt(K) * want.abs().max().item() + 1e-6
    assert (out.double() - want).abs().max().item() <= tol
    # a row's result does not depend on the rows around it
    if M > 2:
        alone = torch.empty(1, N, device=DEV)
        kernels.gemm_simple(a[M // 2:M // 2 + 1], w, alone, bias=bias)
        assert torch.equal(alone[0], out[M // 2])
    x = rand(M, N, seed=5)
    want = x.double() + a.double() @ w.double().T
    kernels.gemm_simple(a, w, x, residual=x)
    assert (x.double() - want).abs().max().item() <= tol


@pytest.mark.parametrize("orientation", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_bf16_tensor_cores(status, M, N, K, orientation):
    """orientation 0: the kernel's own choice; 1: tokens on the MMA's M axis; 2: weight rows on M;
    3: tokens on M with single CTAs; 4: with CTA pairs (tcgen05.mma.cta_group::2)."""
    from sprout_lm_b200 import kernels
    a, w, bias = rand(M, K, dtype=torch.bfloat16), rand(N, K, dtype=torch.bfloat16, seed=1), rand(N, seed=2)
    want = a.double() @ w.double().T + bias.double()
    scale = want.abs().max().item()
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemm_bf16(a, w, out, status, bias=bias, orientation=orientation)
    assert (out.double() - want).abs().max().item() <= 1e-5 * scale + 1e-6       # float32 accumulation of exact products
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_bf16(a, w, out16, status, bias=bias, orientation=orientation)
    assert (out16.double() - want).abs().max().item() <= 8e-3 * scale
    x = rand(M, N, seed=5)
    want_res = x.double() + a.double() @ w.double().T
    kernels.gemm_bf16(a, w, x, status, residual=x, orientation=orientation)
    assert (x.double() - want_res).abs().max().item() <= 1e-5 * scale + 1e-6
    assert int(status.item()) == 0


@pytest.mark.parametrize("orientation", [0, 2, 3, 4])
@pytest.mark.parametrize("M,inter,K", [(5, 200, 72), (300, 256, 136), (2048, 384, 896), (513, 4864, 96),
                                       (64, 640, 200), (65, 640, 200), (100, 4864, 896), (128, 256, 136), (129, 768, 72), (200, 4864, 96)])
def test_gemm_bf16_swiglu_epilogue(status, M, inter, K, orientation):
    """gate and up rows interleaved in blocks of 8; the epilogue writes silu(gate) * up.  The sizes
    lie on both sides of the token counts at which the arrangement changes (64, 128, 256)."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.mlp import interleave_gate_up
    if orientation == 2 and M > 256:
        pytest.skip("weights on M takes up to 256 tokens")
    a = rand(M, K, dtype=torch.bfloat16)
    gate, up = rand(inter, K, dtype=torch.bfloat16, seed=1), rand(inter, K, dtype=torch.bfloat16, seed=2)
    w = interleave_gate_up(gate, up)
    out = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_bf16(a, w, out, status, swiglu=True, orientation=orientation)
    g, u = a.double() @ gate.double().T, a.double() @ up.double().T
    want = g / (1 + torch.exp(-g)) * u
    assert (out.double() - want).abs().max().item() <= 8e-3 * max(1.0, want.abs().max().item())
    assert int(status.item()) == 0


@pytest.mark.parametrize("M,N,K,split", [(1, 896, 4864, 16), (8, 896, 896, 14), (64, 130, 1000, 5), (128, 256, 264, 9)])
def test_gemm_bf16_split_k(status, M, N, K, split):
    from sprout_lm_b200 import kernels
    a, w = rand(M, K, dtype=torch.bfloat16), rand(N, K, dtype=torch.bfloat16, seed=1)
    x = rand(M, N, seed=5)
    want = x.double() + a.double() @ w.double().T
    kernels.gemm_bf16(a, w, x, status, residual=x, orientation=2, split_k=split)
    assert (x.double() - want).abs().max().item() <= 2e-5 * want.abs().max().item() + 1e-6
    assert int(status.item()) == 0


@pytest.mark.parametrize("tokens,hidden,inter,eps", [(1, 64, 128, 1e-6), (5, 96, 320, 1e-5), (8, 896, 4864, 1e-6),
                                                     (3, 1024, 2816, 1e-5), (8, 1536, 2048, 1e-6), (2, 48, 16, 1e-6),
                                                     (9, 896, 4864, 1e-6), (16, 896, 4864, 1e-6), (13, 96, 320, 1e-5),
                                                     (11, 1024, 2816, 1e-5), (16, 48, 16, 1e-6)])
def test_ffn_decode_one_kernel(status, tokens, hidden, inter, eps):
    """RMSNorm, gate/up, SwiGLU, down and the residual sum in one launch, against the same
    arithmetic in float64 with the kernel's two roundings to bfloat16 (the normalised rows, the
    activation).  Three launches in a row, and one channel of the input is made large so that a
    wrong row or column of any operand shows."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.mlp import interleave_gate_up
    assert kernels.ffn_decode_supported(tokens, hidden, inter)
    gate, up = rand(inter, hidden, dtype=torch.bfloat16, scale=0.05, seed=1), rand(inter, hidden, dtype=torch.bfloat16, scale=0.05, seed=2)
    down = rand(hidden, inter, dtype=torch.bfloat16, scale=0.05, seed=3)
    gain = 1 + rand(hidden, scale=0.1, seed=4)
    w = interleave_gate_up(gate, up)
    for round_ in range(3):
        x = rand(tokens, hidden, seed=10 + round_)
        x[:, (7 * round_ + 3) % hidden] *= 6.0
        h = x.double() / torch.sqrt((x.double() ** 2).mean(dim=1, keepdim=True) + eps) * gain.double()
        h = h.float().to(torch.bfloat16).double()
        g, u = h @ gate.double().T, h @ up.double().T
        t = (g / (1 + torch.exp(-g)) * u).float().to(torch.bfloat16).double()
        delta = t @ down.double().T
        want = x.double() + delta
        kernels.ffn_decode(x, gain, eps, w, down, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert (x.double() - want).abs().max().item() <= 4e-3 * max(1e-3, delta.abs().max().item())


def test_ffn_decode_refuses_what_does_not_fit(status):
    from sprout_lm_b200 import kernels
    assert not kernels.ffn_decode_supported(17, 896, 4864)         # more tokens than two tiles have columns
    assert not kernels.ffn_decode_supported(8, 904, 4864)          # sizes that are no multiple of 16
    assert not kernels.ffn_decode_supported(8, 3584, 18944)        # a CTA's share exceeds shared memory
    x = rand(8, 3584)
    with pytest.raises(kernels.KernelError, match="ffn_decode"):
        kernels.ffn_decode(x, rand(3584), 1e-6, rand(2 * 18944, 3584, dtype=torch.bfloat16), rand(3584, 18944, dtype=torch.bfloat16), status)


@pytest.mark.parametrize("normed", [False, True])
@pytest.mark.parametrize("tokens,N,K", [(1, 128, 64), (8, 1152, 896), (5, 160, 96), (8, 896, 896), (3, 48, 16), (7, 2048, 1536),
                                        (9, 1152, 896), (16, 896, 896), (12, 160, 96), (16, 48, 16), (10, 2048, 1536)])
def test_linear_decode_small_batch(status, tokens, N, K, normed):
    """out += input W^T for a few tokens with light CTAs; the input is bfloat16 rows or the RMSNorm
    of float32 rows computed inside the kernel.  The sums land on what the output held before."""
    from sprout_lm_b200 import kernels
    assert kernels.linear_decode_supported(tokens, N, K)
    w = rand(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    before = rand(tokens, N, seed=2)
    for round_ in range(2):
        out = before.clone()
        if normed:
            x, gain, eps = rand(tokens, K, seed=3 + round_), 1 + rand(K, scale=0.1, seed=4), 1e-5
            x[:, (5 * round_ + 2) % K] *= 6.0
            h = x.double() / torch.sqrt((x.double() ** 2).mean(dim=1, keepdim=True) + eps) * gain.double()
            h = h.float().to(torch.bfloat16).double()
            kernels.linear_decode(w, out, status, norm=(x, gain, eps))
        else:
            a = rand(tokens, K, dtype=torch.bfloat16, seed=3 + round_)
            h = a.double()
            kernels.linear_decode(w, out, status, a=a)
        delta = h @ w.double().T
        # a normalised value may round to the neighbouring bfloat16 where the row's sum differs in order
        bound = (4e-3 if normed else 2e-5) * max(1e-3, delta.abs().max().item()) + 1e-6
        assert (out.double() - (before.double() + delta)).abs().max().item() <= bound
    assert int(status.item()) == 0


def test_linear_decode_refuses_what_does_not_fit(status):
    from sprout_lm_b200 import kernels
    assert not kernels.linear_decode_supported(17, 896, 896)
    assert not kernels.linear_decode_supported(8, 900, 896)
    assert not kernels.linear_decode_supported(8, 3584, 3584)       # pieces too large for light CTAs
    with pytest.raises(kernels.KernelError, match="linear_decode"):
        kernels.linear_decode(rand(3584, 3584, dtype=torch.bfloat16), rand(8, 3584), status, a=rand(8, 3584, dtype=torch.bfloat16))


@pytest.mark.parametrize("tokens,N,K,split", [(17, 1152, 896, 14), (64, 1152, 896, 14), (33, 256, 136, 3), (200, 384, 520, 9), (64, 1152, 896, 1),
                                              (64, 4608, 3584, 4), (40, 256, 2000, 1), (130, 300, 3000, 2), (8, 20000, 64, 1)])
def test_gemm_bf16_unscaled_is_the_normed_product_without_its_scale(status, tokens, N, K, split):
    """out += bfloat16(x * gain) W^T with the tokens' tiles made inside the kernel: against float64
    with that one rounding, on top of what the output held; and scaled by 1 / rms(x) it is the
    product of the RMSNorm's output, to bfloat16's precision.  K ranges of 14, 32 and 24 k-blocks per
    CTA go round the ring of stages more than once."""
    from sprout_lm_b200 import kernels
    if not kernels.gemm_bf16_unscaled_supported(tokens, N, K, split):
        assert N == 20000                                  # more work items than SMs (K ranges longer than the ring are taken)
        with pytest.raises(kernels.KernelError, match="gemm_bf16_unscaled"):
            kernels.gemm_bf16_unscaled(rand(tokens, K), rand(K), rand(N, K, dtype=torch.bfloat16), rand(tokens, N), status, split_k=split)
        return
    x = rand(tokens, K, seed=1)
    x[:, 5 % K] *= 6.0
    gain = 1 + rand(K, scale=0.1, seed=2)
    w = rand(N, K, dtype=torch.bfloat16, scale=0.05, seed=3)
    before = rand(tokens, N, seed=4)
    out = before.clone()
    for _ in range(2):                                     # twice: the sums add up
        kernels.gemm_bf16_unscaled(x, gain, w, out, status, split_k=split)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    h = (x.double() * gain.double()).float().to(torch.bfloat16).double()
    want = before.double() + 2 * (h @ w.double().T)
    assert (out.double() - want).abs().max().item() <= 2e-5 * max(1.0, want.abs().max().item())
    eps = 1e-5
    inv = 1.0 / torch.sqrt((x.double() ** 2).mean(dim=1, keepdim=True) + eps)
    normed = (x.double() * inv * gain.double()).float().to(torch.bfloat16).double() @ w.double().T
    scaled = (out.double() - before.double()) / 2 * inv
    assert (scaled - normed).abs().max().item() <= 8e-3 * max(1e-3, normed.abs().max().item())


def test_gemm_bf16_refuses_unaligned_rows(status):
    from sprout_lm_b200 import kernels
    a, w = rand(4, 20, dtype=torch.bfloat16), rand(8, 20, dtype=torch.bfloat16)
    with pytest.raises(kernels.KernelError, match="multiples of 8"):
        kernels.gemm_bf16(a, w, torch.empty(4, 8, device=DEV), status)


# ------------------------------------------------------------------------------- attention
def attention_reference(q, keys, values, heads, kv_heads, head_dim):
    """q [heads*hd]; keys, values [n, kv_heads*hd] (float64) -> [heads*hd]."""
    out = torch.zeros(heads * head_dim, dtype=torch.float64)
    group = heads // kv_heads
    for h in range(heads):
        g = h // group
        s = keys[:, g * head_dim:(g + 1) * head_dim] @ q[h * head_dim:(h + 1) * head_dim] / math.sqrt(head_dim)
        out[h * head_dim:(h + 1) * head_dim] = torch.softmax(s, 0) @ values[:, g * head_dim:(g + 1) * head_dim]
    return out


def build_paged_case(dtype, heads, kv_heads, head_dim, page, lengths, q_counts, seed=0, spike=None, poison=False,
                     layout="scattered"):
    """Requests with ``lengths`` cached positions each (the last ``q_counts`` of them are this
    step's queries), in pages scattered over the pool (``layout`` "runs": in runs of 1 to 11 pages
    that follow one another in the pool, the runs scattered; "in order": as a fresh pool hands
    them out).  ``poison``: every slot that holds no key of a request (the rest of a last page,
    pages nobody owns) is NaN instead of zero."""
    g = torch.Generator().manual_seed(seed)
    R = len(lengths)
    pages_each = [-(-n // page) for n in lengths]
    pool = sum(pages_each) + 3
    if layout == "scattered":
        order = torch.randperm(pool, generator=g)
    elif layout == "in order":
        order = torch.arange(pool)
    else:
        runs, at = [], 0
        while at < pool:
            n = min(pool - at, int(torch.randint(1, 12, (1,), generator=g)))
            runs.append(torch.arange(at, at + n))
            at += n
        order = torch.cat([runs[i] for i in torch.randperm(len(runs), generator=g)])
    table = torch.full((R, max(pages_each)), -1, dtype=torch.int32)
    k_cache = torch.full((pool, kv_heads, page, head_dim), float("nan") if poison else 0.0)
    v_cache = torch.full((pool, kv_heads, page, head_dim), float("nan") if poison else 0.0)
    keys, values, at = [], [], 0
    for r, n in enumerate(lengths):
        k = torch.randn(n, kv_heads * head_dim, generator=g)
        v = torch.randn(n, kv_heads * head_dim, generator=g)
        if spike is not None and r == spike[0]:
            k[spike[1]] *= 6.0                       # one far key whose score stands out
        k, v = k.to(dtype).float(), v.to(dtype).float()
        keys.append(k.double())
        values.append(v.double())
        for i in range(pages_each[r]):
            pg = int(order[at]); at += 1
            table[r, i] = pg
            rows = slice(i * page, min(n, (i + 1) * page))
            count = rows.stop - rows.start
            k_cache[pg, :, :count] = k[rows].reshape(count, kv_heads, head_dim).transpose(0, 1)
            v_cache[pg, :, :count] = v[rows].reshape(count, kv_heads, head_dim).transpose(0, 1)
    positions, seq_of_token = [], []
    for r, (n, c) in enumerate(zip(lengths, q_counts)):
        positions += list(range(n - c, n))
        seq_of_token += [r] * c
    T = len(positions)
    q = torch.randn(T, heads * head_dim, generator=g)
    if spike is not None:
        # queries of the spiked request look at the spiked key
        for t in range(T):
            if seq_of_token[t] == spike[0]:
                group = heads // kv_heads
                for h in range(heads):
                    gk = h // group
                    q[t, h * head_dim:(h + 1) * head_dim] = keys[spike[0]][spike[1], gk * head_dim:(gk + 1) * head_dim].float()
    q = q.to(dtype)
    want = torch.stack([attention_reference(q[t].double(), keys[seq_of_token[t]][:positions[t] + 1],
                                            values[seq_of_token[t]][:positions[t] + 1], heads, kv_heads, head_dim)
                        for t in range(T)])
    dev = lambda x, dt=None: x.to(dt or x.dtype).to(DEV)
    return dict(q=dev(q), k_cache=dev(k_cache, dtype), v_cache=dev(v_cache, dtype), table=dev(table),
                positions=dev(torch.tensor(positions, dtype=torch.int32)),
                seq_of_token=dev(torch.tensor(seq_of_token, dtype=torch.int32)), want=want, T=T,
                q_start=dev(torch.tensor(np.cumsum([0] + list(q_counts)), dtype=torch.int32)),
                context_lens=dev(torch.tensor(lengths, dtype=torch.int32)), lengths=lengths, q_counts=q_counts)


ATTN_CASES = [
    # heads, kv_heads, head_dim, page, cached lengths, queries of this step
    (4, 2, 16, 16, [5, 17, 33], [5, 1, 33]),
    (3, 1, 32, 8, [61, 1, 130], [7, 1, 1]),
    (14, 2, 64, 16, [300, 129, 16], [1, 1, 16]),
    (5, 5, 48, 4, [40, 9], [2, 9]),
    (8, 2, 128, 16, [257, 64], [3, 64]),
    (6, 3, 80, 32, [100], [100]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page,lengths,q_counts", ATTN_CASES)
def test_attention_simple(status, dtype, heads, kv_heads, head_dim, page, lengths, q_counts):
    from sprout_lm_b200 import kernels
    case = build_paged_case(dtype, heads, kv_heads, head_dim, page, lengths, q_counts)
    out = torch.empty(case["T"], heads * head_dim, dtype=dtype, device=DEV)
    kernels.attention_simple(case["q"], case["k_cache"], case["v_cache"], case["table"], case["seq_of_token"],
                             case["positions"], out, heads, kv_heads, head_dim, status)
    tol = 3e-6 if dtype == torch.float32 else 1.2e-2
    assert (out.double().cpu() - case["want"]).abs().max().item() <= tol
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("where", [0, 15, 16, 255, 256, 383, 500])
def test_attention_finds_one_far_key_among_hundreds(status, dtype, where):
    """The query equals one key scaled up: nearly all the weight lies on that key, at a page's
    first or last slot or far back; an attention that skips it returns something else."""
    from sprout_lm_b200 import kernels
    heads, kv_heads, head_dim, page = 4, 2, 32, 16
    case = build_paged_case(dtype, heads, kv_heads, head_dim, page, [40, 501], [1, 1], seed=where, spike=(1, where))
    out = torch.empty(case["T"], heads * head_dim, dtype=dtype, device=DEV)
    kernels.attention_simple(case["q"], case["k_cache"], case["v_cache"], case["table"], case["seq_of_token"],
                             case["positions"], out, heads, kv_heads, head_dim, status)
    tol = 3e-6 if dtype == torch.float32 else 1.5e-2
    assert (out.double().cpu() - case["want"]).abs().max().item() <= tol


DECODE_CASES = [
    (4, 2, 16, 16, [5, 17, 33, 1]), (3, 1, 32, 8, [61, 1, 130]), (14, 2, 64, 16, [300, 129, 16, 640, 513]),
    (5, 5, 48, 4, [40, 9]), (8, 2, 128, 16, [257, 64, 1000]), (6, 3, 80, 32, [100]), (16, 1, 256, 16, [70, 200]),
    (8, 2, 128, 16, [3000, 1200, 17]),                         # head size 128 through memory: swizzled rows, three CTAs per SM
    (6, 2, 96, 32, [2100, 5]),                                 # padded rows through memory
]


@pytest.mark.parametrize("split_keys", [None, 128, 256])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page,lengths", DECODE_CASES)
def test_attention_decode_split_keys(status, heads, kv_heads, head_dim, page, lengths, split_keys):
    from sprout_lm_b200 import kernels
    case = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lengths, [1] * len(lengths))
    out = torch.full((case["T"], heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.attention_decode(case["q"], case["k_cache"], case["v_cache"], case["table"], case["context_lens"], out,
                             heads, kv_heads, head_dim, status, split_keys=split_keys)
    assert (out.double().cpu() - case["want"]).abs().max().item() <= 1.2e-2
    # a wider block table (as under a captured graph) changes the split count, not the result
    wide = torch.full((len(lengths), case["table"].shape[1] + 19), -1, dtype=torch.int32, device=DEV)
    wide[:, :case["table"].shape[1]] = case["table"]
    again = torch.empty_like(out)
    kernels.attention_decode(case["q"], case["k_cache"], case["v_cache"], wide, case["context_lens"], again,
                             heads, kv_heads, head_dim, status, split_keys=split_keys)
    assert (again.double().cpu() - case["want"]).abs().max().item() <= 1.2e-2
    assert int(status.item()) == 0


@pytest.mark.parametrize("rotate", [False, True])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page,lengths", DECODE_CASES[:6] + [
    (14, 2, 64, 16, [37 + 13 * i for i in range(70)]),        # a large batch: longer splits, few per request
    (4, 2, 64, 16, [6000, 1500]),                              # more than 8 splits: through memory too
    (4, 2, 64, 16, [2900 + 2 * i for i in range(80)]),         # more CTAs than four per SM: the variant held to five per SM's registers
    (6, 2, 32, 16, [5000 + 2 * i for i in range(60)]),
    (8, 2, 128, 16, [2500, 700, 90]),                          # head size 128 through memory
    (8, 4, 128, 32, [1300 + 7 * i for i in range(40)]),        # and with more CTAs than places
])
def test_attention_decode_fused_projection_tail(status, heads, kv_heads, head_dim, page, lengths, rotate):
    """The decode kernel that also finishes the projection: the new token's q, k, v arrive as
    float32 sums plus a bias; the kernel rotates, appends to the cache, attends and clears the sums.
    Compared with the separate rotary kernel followed by the decode kernel."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.rope import HalfSplitRotary
    R = len(lengths)
    case = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lengths, [1] * R, seed=3)
    width = (heads + 2 * kv_heads) * head_dim
    g = torch.Generator().manual_seed(11)
    sums = torch.randn(R, width, generator=g).to(DEV)
    bias = (torch.randn(width, generator=g) * 0.3).to(DEV)

    from sprout_lm_b200.parts import Runtime
    cos, sin = HalfSplitRotary("", head_dim, 1e4, max(1024, max(lengths))).rotary_tables(Runtime(DEV, torch.bfloat16)) if rotate else (None, None)
    positions = (case["context_lens"] - 1).to(torch.int32)
    seq_of_token = torch.arange(R, dtype=torch.int32, device=DEV)
    # the separate path
    k1, v1 = case["k_cache"].clone(), case["v_cache"].clone()
    acc1 = torch.zeros(R + 1, width, device=DEV)
    acc1[:R] = sums
    qkv = torch.zeros(R, width, dtype=torch.bfloat16, device=DEV)
    kernels.rope_append(qkv, positions, seq_of_token, case["table"], cos, sin, k1, v1, heads, kv_heads, head_dim, page,
                        True, status, acc=acc1[:R], bias=bias)
    want = torch.empty(R, heads * head_dim, dtype=torch.bfloat16, device=DEV)
    kernels.attention_decode(qkv[:, :heads * head_dim], k1, v1, case["table"], case["context_lens"], want, heads,
                             kv_heads, head_dim, status)
    # the fused kernel
    k2, v2 = case["k_cache"].clone(), case["v_cache"].clone()
    acc2 = sums.clone()
    got = torch.full_like(want, float("nan"))
    assert kernels.decode_fusable(R, heads, kv_heads, head_dim, case["table"].shape[1] * page)
    if max(lengths) > 5000:
        assert kernels.decode_split_plan(R, kv_heads, case["table"].shape[1] * page, head_dim)[2]      # this case goes through memory
    if R >= 60 and max(lengths) > 2000:
        _, splits, through_memory = kernels.decode_split_plan(R, kv_heads, case["table"].shape[1] * page, head_dim)
        assert through_memory and splits * kv_heads * R > 4 * kernels.sm_count()
    kernels.attention_decode_fused(acc2, bias, cos, sin, k2, v2, case["table"], case["context_lens"], got, heads,
                                   kv_heads, head_dim, status)
    assert torch.equal(k2, k1) and torch.equal(v2, v1)                 # the same append, bit for bit
    assert float(acc2.abs().max()) == 0.0                               # the sums are cleared
    assert (got.float() - want.float()).abs().max().item() <= 1.2e-2
    assert int(status.item()) == 0


RESIDENT_CASES = [
    (14, 2, 64, 16, [300, 129, 16, 640, 513, 1, 768, 32, 33]), (8, 2, 128, 16, [257, 64, 384, 1, 100]), (4, 4, 64, 8, [61, 1, 130, 8, 9]),
    (16, 1, 64, 128, [500, 128, 129]), (7, 1, 128, 32, [100, 31]), (3, 3, 64, 64, [64, 65, 700]),
]


@pytest.mark.parametrize("layout", ["scattered", "runs", "in order"])
@pytest.mark.parametrize("rotate", [False, True])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page,lengths", RESIDENT_CASES)
def test_attention_decode_resident(status, heads, kv_heads, head_dim, page, lengths, fused, rotate, layout):
    """Decode attention with each request's whole context in one CTA's shared memory (pages by
    TMA; pages scattered, in runs, or in the pool's order): against the float64
    reference; in the fused form (sums in, rotation, cache append) also against the separate
    rotary kernel.  Every cache slot outside the requests is NaN."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts import Runtime
    from sprout_lm_b200.parts.rope import HalfSplitRotary
    if rotate and not fused:
        pytest.skip("the rotation belongs to the fused form")
    R = len(lengths)
    room = kernels.decode_attention_plan(kernels.sm_count() // kv_heads, heads, kv_heads, head_dim, page, -(-max(lengths) // page) * page, max(lengths))
    assert room[0] == "resident"
    case = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lengths, [1] * R, seed=7, poison=True, layout=layout)
    out = torch.full((R, heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    if not fused:
        kernels.attention_decode_resident(case["k_cache"], case["v_cache"], case["table"], case["context_lens"], out, heads,
                                          kv_heads, head_dim, status, room[1], q=case["q"])
        assert (out.double().cpu() - case["want"]).abs().max().item() <= 1.2e-2
        assert int(status.item()) == 0
        return
    width = (heads + 2 * kv_heads) * head_dim
    g = torch.Generator().manual_seed(11)
    sums = torch.randn(R, width, generator=g).to(DEV)
    bias = (torch.randn(width, generator=g) * 0.3).to(DEV)
    cos, sin = HalfSplitRotary("", head_dim, 1e4, 1024).rotary_tables(Runtime(DEV, torch.bfloat16)) if rotate else (None, None)
    positions = (case["context_lens"] - 1).to(torch.int32)
    seq_of_token = torch.arange(R, dtype=torch.int32, device=DEV)
    # the separate path on a cache without the poison beyond the requests (its kernels are tested for that elsewhere)
    clean = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lengths, [1] * R, seed=7, layout=layout)
    k1, v1 = clean["k_cache"].clone(), clean["v_cache"].clone()
    acc1 = sums.clone()
    qkv = torch.zeros(R, width, dtype=torch.bfloat16, device=DEV)
    kernels.rope_append(qkv, positions, seq_of_token, case["table"], cos, sin, k1, v1, heads, kv_heads, head_dim, page,
                        True, status, acc=acc1, bias=bias)
    want = torch.empty(R, heads * head_dim, dtype=torch.bfloat16, device=DEV)
    kernels.attention_decode(qkv[:, :heads * head_dim], k1, v1, case["table"], case["context_lens"], want, heads,
                             kv_heads, head_dim, status, split_keys=128)
    k2, v2 = case["k_cache"].clone(), case["v_cache"].clone()
    acc2 = sums.clone()
    kernels.attention_decode_resident(k2, v2, case["table"], case["context_lens"], out, heads, kv_heads, head_dim, status,
                                      room[1], acc=acc2, bias=bias, cos_table=cos, sin_table=sin)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for r, n in enumerate(lengths):                         # the same append, bit for bit, and nothing else touched
        pg, slot = int(case["table"][r, (n - 1) // page]), (n - 1) % page
        assert torch.equal(k2[pg, :, slot], k1[pg, :, slot]) and torch.equal(v2[pg, :, slot], v1[pg, :, slot])
        k2[pg, :, slot] = case["k_cache"][pg, :, slot]
        v2[pg, :, slot] = case["v_cache"][pg, :, slot]
    same = lambda a, b: torch.equal(torch.nan_to_num(a.float(), nan=7.0), torch.nan_to_num(b.float(), nan=7.0))
    assert same(k2, case["k_cache"]) and same(v2, case["v_cache"])
    assert float(acc2.abs().max()) == 0.0                   # the sums are cleared
    assert (out.float() - want.float()).abs().max().item() <= 1.2e-2


@pytest.mark.parametrize("kernel", ["split", "resident"])
def test_decode_attention_applies_the_norms_scale_to_the_sums(status, kernel):
    """The fused decode kernels with ``norm_x``: the float32 sums are those of a product whose
    normalised input went without its scale; multiplied by 1 / rms of the request's row they must
    give what the same kernel gives for sums that were scaled beforehand."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts import Runtime
    from sprout_lm_b200.parts.rope import HalfSplitRotary
    heads, kv_heads, head_dim, page = 14, 2, 64, 16
    lengths = [300, 129, 16, 640, 513, 1, 77, 33]
    R = len(lengths)
    case = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lengths, [1] * R, seed=9)
    width = (heads + 2 * kv_heads) * head_dim
    g = torch.Generator().manual_seed(13)
    sums = torch.randn(R, width, generator=g).to(DEV) * 3.0
    bias = (torch.randn(width, generator=g) * 0.3).to(DEV)
    x = (torch.randn(R, 200, generator=g) * torch.linspace(0.2, 4.0, R)[:, None]).to(DEV)     # rows of very different size
    eps = 1e-5
    inv = 1.0 / torch.sqrt((x.double() ** 2).mean(dim=1, keepdim=True) + eps)
    cos, sin = HalfSplitRotary("", head_dim, 1e4, 1024).rotary_tables(Runtime(DEV, torch.bfloat16))
    outs, caches = [], []
    for scaled_before in (True, False):
        acc = (sums.double() * inv).float() if scaled_before else sums.clone()
        k, v = case["k_cache"].clone(), case["v_cache"].clone()
        out = torch.empty(R, heads * head_dim, dtype=torch.bfloat16, device=DEV)
        norm_x = None if scaled_before else (x, eps)
        if kernel == "resident":
            kernels.attention_decode_resident(k, v, case["table"], case["context_lens"], out, heads, kv_heads, head_dim, status, 640,
                                              acc=acc, bias=bias, cos_table=cos, sin_table=sin, norm_x=norm_x)
        else:
            kernels.attention_decode_fused(acc, bias, cos, sin, k, v, case["table"], case["context_lens"], out, heads, kv_heads,
                                           head_dim, status, norm_x=norm_x)
        torch.cuda.synchronize()
        assert float(acc.abs().max()) == 0.0
        outs.append(out.float())
        caches.append((k.float(), v.float()))
    assert int(status.item()) == 0
    assert (outs[0] - outs[1]).abs().max().item() <= 2e-2                     # the scale in float32, before or inside: a bfloat16 step apart at most
    assert (caches[0][0] - caches[1][0]).abs().max().item() <= 4e-2 and (caches[0][1] - caches[1][1]).abs().max().item() <= 4e-2
    assert (outs[0].abs().max().item()) > 0.1


def test_attention_decode_resident_refuses_a_context_beyond_its_room(status):
    """A request longer than the launch has room for is flagged in the status word and gets no
    output; nothing is read or written out of bounds."""
    from sprout_lm_b200 import kernels
    case = build_paged_case(torch.bfloat16, 4, 2, 64, 16, [300, 40], [1, 1])
    out = torch.zeros(2, 4 * 64, dtype=torch.bfloat16, device=DEV)
    kernels.attention_decode_resident(case["k_cache"], case["v_cache"], case["table"], case["context_lens"], out, 4, 2, 64,
                                      status, 256, q=case["q"])
    torch.cuda.synchronize()
    assert int(status.item()) == 32
    status.zero_()
    assert float(out[0].float().abs().max()) == 0.0
    assert (out[1].double().cpu() - case["want"][1]).abs().max().item() <= 1.2e-2
    with pytest.raises(kernels.KernelError, match="cap_keys"):
        kernels.attention_decode_resident(case["k_cache"], case["v_cache"], case["table"], case["context_lens"], out, 4, 2, 64,
                                          status, 1024, q=case["q"])


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page,lengths", [(14, 2, 64, 16, [300, 129, 16, 640, 513, 1]),
                                                                   (3, 1, 48, 8, [61, 1, 130]), (4, 2, 64, 16, [3000, 70])])
def test_attention_decode_ignores_what_lies_beyond_a_request(status, heads, kv_heads, head_dim, page, lengths, fused):
    """Every cache slot that holds no key of a request is NaN: the rest of a last page (which the
    kernel's first pass loads before it knows the request's length), and pages nobody owns.  A
    page that another request used before holds whatever that request left; none of it may reach
    the result."""
    from sprout_lm_b200 import kernels
    R = len(lengths)
    case = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lengths, [1] * R, seed=5, poison=True)
    out = torch.full((R, heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    if not fused:
        kernels.attention_decode(case["q"], case["k_cache"], case["v_cache"], case["table"], case["context_lens"], out,
                                 heads, kv_heads, head_dim, status)
        assert (out.double().cpu() - case["want"]).abs().max().item() <= 1.2e-2
    else:
        # the new token's q, k, v as sums: q is the case's query, k and v the case's last key and value
        width = (heads + 2 * kv_heads) * head_dim
        sums = torch.zeros(R, width, device=DEV)
        sums[:, :heads * head_dim] = case["q"].float()
        k, v = case["k_cache"].clone(), case["v_cache"].clone()
        for r, n in enumerate(lengths):
            pg, slot = int(case["table"][r, (n - 1) // page]), (n - 1) % page
            sums[r, heads * head_dim:(heads + kv_heads) * head_dim] = k[pg, :, slot].float().reshape(-1)
            sums[r, (heads + kv_heads) * head_dim:] = v[pg, :, slot].float().reshape(-1)
            k[pg, :, slot] = float("nan")                  # the kernel writes the new token's slot itself
            v[pg, :, slot] = float("nan")
        kernels.attention_decode_fused(sums, None, None, None, k, v, case["table"], case["context_lens"], out, heads,
                                       kv_heads, head_dim, status)
        assert (out.double().cpu() - case["want"]).abs().max().item() <= 1.2e-2
        assert float(sums.abs().max()) == 0.0
    assert int(status.item()) == 0


@pytest.mark.parametrize("tokens,head_dim", [(3, 32), (20, 64)])
def test_rope_append_clears_the_sums_of_a_refused_position(status, tokens, head_dim):
    """A position beyond the rotary table is flagged and skipped; the float32 sums of that token
    must still be emptied, or the next product into the workspace would add to them."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts import Runtime
    from sprout_lm_b200.parts.rope import HalfSplitRotary
    heads, kv_heads, page = 4, 2, 16
    width = (heads + 2 * kv_heads) * head_dim
    cos, sin = HalfSplitRotary("", head_dim, 1e4, 64).rotary_tables(Runtime(DEV, torch.bfloat16))
    acc = rand(tokens, width, seed=2) + 3.0
    bias = rand(width, seed=3)
    positions = torch.arange(tokens, dtype=torch.int32, device=DEV)
    positions[1] = 64                                    # one past the table
    table = torch.arange(4, dtype=torch.int32, device=DEV).reshape(1, 4)
    k_cache = torch.zeros(4, kv_heads, page, head_dim, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    qkv = torch.zeros(tokens, width, dtype=torch.bfloat16, device=DEV)
    kernels.rope_append(qkv, positions, torch.zeros(tokens, dtype=torch.int32, device=DEV), table, cos, sin, k_cache,
                        v_cache, heads, kv_heads, head_dim, page, True, status, acc=acc, bias=bias)
    torch.cuda.synchronize()
    assert int(status.item()) == 16
    status.zero_()
    assert float(acc.abs().max()) == 0.0
    assert float(qkv[0].float().abs().max()) > 0 and float(qkv[1].float().abs().max()) == 0.0


def test_a_bounded_wait_runs_out_and_the_kernel_returns(status):
    """Every wait of the kernels on an mbarrier (a copy's arrival, a product's completion) is
    bounded in time.  A one-warp kernel waits, with that same helper, on a barrier on which nothing
    ever arrives: after the bound (about a second and a half) it gives up, sets the status word's
    wait bit and returns: no fault, no hang, and the device goes on working."""
    import time
    from sprout_lm_b200 import kernels
    torch.cuda.synchronize()
    begin = time.perf_counter()
    kernels.wait_probe(status)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - begin
    assert int(status.item()) == 8 and kernels.describe_status(8) == "a bounded device-side wait ran out"
    assert 0.5 <= seconds <= 10.0, seconds
    status.zero_()
    out = torch.empty(2, 64, device=DEV)
    kernels.rmsnorm(torch.ones(2, 64, device=DEV), torch.ones(64, device=DEV), out, 1e-6)
    torch.cuda.synchronize()
    assert abs(float(out[0, 0]) - 1.0) < 1e-5 and int(status.item()) == 0


def test_sampling_never_draws_a_token_of_probability_zero(status):
    """A peaked row whose tail is far below: with the uniform number just under 1 the draw falls
    where rounding decides (the two kernels add the same exponentials in different orders); it must
    land on a token that has weight, not on the tail."""
    from sprout_lm_b200 import kernels
    vocab = 4099
    for heavy in (1, 5, 40):
        logits = torch.full((3, vocab), -1e30, device=DEV)
        logits[:, :heavy] = rand(3, heavy, scale=1.0, seed=heavy)
        logits[2, vocab - 1] = -80.0                              # a weight that underflows against the maximum
        out = torch.empty(3, dtype=torch.int32, device=DEV)
        temperature = torch.tensor([1.0, 0.7, 1.3], device=DEV)
        for u in (1.0 - 2.0 ** -24, 0.999, 0.5, 0.0):
            kernels.sample(logits, out, status, temperature, torch.full((3,), u, device=DEV))
            assert all(0 <= t < heavy for t in out.tolist()), (heavy, u, out.tolist())
    assert int(status.item()) == 0


@pytest.mark.parametrize("heads,kv_heads,head_dim,page,lengths,q_counts", ATTN_CASES + [
    (14, 2, 64, 16, [700, 650, 2, 90], [700, 1, 2, 9]), (2, 1, 112, 8, [75], [75]), (7, 7, 96, 16, [33, 64], [2, 64])])
def test_attention_prefill_tensor_cores(status, heads, kv_heads, head_dim, page, lengths, q_counts):
    from sprout_lm_b200 import kernels
    case = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lengths, q_counts)
    out = torch.full((case["T"], heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.attention_prefill(case["q"], case["k_cache"], case["v_cache"], case["table"], case["q_start"],
                              case["positions"], out, heads, kv_heads, head_dim, status)
    assert (out.double().cpu() - case["want"]).abs().max().item() <= 1.5e-2
    assert int(status.item()) == 0


TC_PREFILL_CASES = [
    # heads, kv_heads, head_dim, page, cached lengths, queries of this step
    (14, 2, 64, 16, [700, 650, 2, 90], [700, 1, 2, 9]),       # several key tiles, rows of several requests
    (4, 2, 64, 8, [129, 128, 127], [129, 128, 1]),            # the edges of a key tile
    (8, 2, 128, 16, [300, 64], [37, 64]),                     # head_dim 128: two 64-element blocks, one P buffer
    (3, 1, 64, 32, [513], [200]),                             # a portion in the middle of a long request
    (2, 2, 128, 64, [260, 5], [260, 5]),
    (5, 1, 64, 128, [400], [400]),                            # a page as long as a key tile
    (2, 1, 64, 256, [600, 100], [90, 100]),                   # pages longer than a key tile
    (16, 1, 64, 16, [45], [45]),                              # many heads per key head: a tile holds few tokens
    (4, 1, 128, 128, [300, 129], [300, 70]),                  # head_dim 128 with pages of two key tiles
    (14, 2, 64, 16, [1500], [1500]),                          # Q tile 0 of a piece ends a key tile before Q tile 1
    (2, 2, 64, 16, [40, 128, 200], [40, 128, 129]),           # pieces with one Q tile and with two
]


@pytest.mark.parametrize("heads,kv_heads,head_dim,page,lengths,q_counts", TC_PREFILL_CASES)
def test_attention_prefill_tcgen05(status, heads, kv_heads, head_dim, page, lengths, q_counts):
    """The tcgen05 prefill kernel against the float64 reference, with NaN in every cache slot
    that holds no key: a kernel that lets one of them into a product shows it."""
    from sprout_lm_b200 import kernels
    case = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lengths, q_counts, seed=5, poison=True)
    out = torch.full((case["T"], heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.attention_prefill(case["q"], case["k_cache"], case["v_cache"], case["table"], case["q_start"],
                              case["positions"], out, heads, kv_heads, head_dim, status, variant="tcgen05")
    assert int(status.item()) == 0
    err = (out.double().cpu() - case["want"]).abs().max(dim=1).values
    assert float(err.max()) <= 1.5e-2, f"token {int(err.argmax())} of {case['T']} differs by {float(err.max()):.3e}"
    # the other kernel on the same case (it must not read the poisoned slots either)
    again = torch.full_like(out, float("nan"))
    kernels.attention_prefill(case["q"], case["k_cache"], case["v_cache"], case["table"], case["q_start"],
                              case["positions"], again, heads, kv_heads, head_dim, status, variant="mma_sync")
    assert float((again.double().cpu() - case["want"]).abs().max()) <= 1.5e-2


def test_attention_prefill_tcgen05_refuses_other_sizes(status):
    from sprout_lm_b200 import kernels
    case = build_paged_case(torch.bfloat16, 4, 2, 48, 16, [40], [40])
    out = torch.empty(case["T"], 4 * 48, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(kernels.KernelError, match="head_dim 64 or 128"):
        kernels.attention_prefill(case["q"], case["k_cache"], case["v_cache"], case["table"], case["q_start"],
                                  case["positions"], out, 4, 2, 48, status, variant="tcgen05")


@pytest.mark.parametrize("where", [0, 127, 128, 255, 256, 700, 1023])
def test_tcgen05_prefill_finds_one_far_key(status, where):
    """One key among 1,024 whose score stands out, at the edges of the 128-key tiles."""
    from sprout_lm_b200 import kernels
    heads, kv_heads, head_dim, page = 4, 2, 64, 16
    case = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, [1024], [40], seed=where, spike=(0, where))
    out = torch.empty(case["T"], heads * head_dim, dtype=torch.bfloat16, device=DEV)
    kernels.attention_prefill(case["q"], case["k_cache"], case["v_cache"], case["table"], case["q_start"],
                              case["positions"], out, heads, kv_heads, head_dim, status, variant="tcgen05")
    assert (out.double().cpu() - case["want"]).abs().max().item() <= 1.5e-2


@pytest.mark.parametrize("where", [0, 15, 16, 63, 64, 255, 256, 383, 500])
def test_fast_attention_finds_one_far_key(status, where):
    from sprout_lm_b200 import kernels
    heads, kv_heads, head_dim, page = 4, 2, 32, 16
    case = build_paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, [40, 501], [1, 1], seed=where, spike=(1, where))
    for name in ("decode", "prefill"):
        out = torch.empty(case["T"], heads * head_dim, dtype=torch.bfloat16, device=DEV)
        if name == "decode":
            kernels.attention_decode(case["q"], case["k_cache"], case["v_cache"], case["table"], case["context_lens"],
                                     out, heads, kv_heads, head_dim, status)
        else:
            kernels.attention_prefill(case["q"], case["k_cache"], case["v_cache"], case["table"], case["q_start"],
                                      case["positions"], out, heads, kv_heads, head_dim, status)
        assert (out.double().cpu() - case["want"]).abs().max().item() <= 1.5e-2, name


# ------------------------------------------------------------------------------- sampling
@pytest.mark.parametrize("vocab", [7, 256, 509, 4099, 151936])
def test_sampling(status, vocab):
    from sprout_lm_b200 import kernels
    logits = rand(6, vocab, scale=2.0)
    logits[1, 3] = logits[1].max() + 1
    logits[1, vocab - 1] = logits[1, 3]                           # a tie: the lowest index wins
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    kernels.sample(logits, out, status)
    assert out.tolist() == logits.argmax(-1).tolist() or out[1].item() == 3
    assert out[1].item() == 3
    temperature = torch.tensor([0.0, 0.8, 0.8, 1.5, 0.3, 0.8], device=DEV)
    for u in (0.0, 0.25, 0.5, 0.999999):
        uniform = torch.full((6,), u, device=DEV)
        kernels.sample(logits, out, status, temperature, uniform)
        assert out[0].item() == int(logits[0].argmax())
        for r in range(1, 6):
            p = torch.softmax(logits[r].double() / temperature[r].double(), 0)
            c = torch.cumsum(p, 0)
            pick = out[r].item()
            low = c[pick - 1].item() if pick else 0.0
            assert low - 1e-4 <= u <= c[pick].item() + 1e-4, (r, u, pick)
    assert int(status.item()) == 0
    logits[2, 1] = float("nan")
    kernels.sample(logits, out, status)
    assert out[2].item() == -1 and int(status.item()) & 4
    status.zero_()
