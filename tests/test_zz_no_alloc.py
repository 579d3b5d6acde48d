"""The allocation-free decode attention, called through its exported C symbol.

Some hosts of this library cannot allocate device memory while serving (all of it belongs to
their own arena, or they are plain C programs without an allocator to ask); for them the
library carries a fixed scratch array of its own.  This test calls that entry point by its C
name, twice in a row on different inputs (the array keeps the first call's contents), and
compares each result with the ordinary entry point that takes scratch from the caller and with
a plain float64 attention over the same pages.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _case(seed, requests, heads, kv_heads, head_dim, page, lengths):
    g = torch.Generator().manual_seed(seed)
    pages_each = [-(-n // page) for n in lengths]
    pool = sum(pages_each) + 2
    order = torch.randperm(pool, generator=g)
    table = torch.full((requests, max(pages_each)), -1, dtype=torch.int32)
    at = 0
    for r, count in enumerate(pages_each):
        table[r, :count] = order[at:at + count].to(torch.int32)
        at += count
    k = torch.randn(pool, kv_heads, page, head_dim, generator=g).to(torch.bfloat16)
    v = torch.randn(pool, kv_heads, page, head_dim, generator=g).to(torch.bfloat16)
    q = torch.randn(requests, heads * head_dim, generator=g).to(torch.bfloat16)
    return (q.to(DEV), k.to(DEV), v.to(DEV), table.to(DEV), torch.tensor(lengths, dtype=torch.int32, device=DEV))


def _plain(q, k, v, table, lengths, heads, kv_heads, head_dim, page):
    """softmax(q k^T / sqrt(d)) v per request and head in float64, from the pages the table names."""
    out = torch.zeros(q.shape, dtype=torch.float64)
    group = heads // kv_heads
    q, k, v, table = q.double().cpu(), k.double().cpu(), v.double().cpu(), table.cpu()
    for r, n in enumerate(lengths):
        keys = torch.cat([k[int(p)] for p in table[r, :-(-n // page)]], dim=1)[:, :n]        # [kv_heads, n, hd]
        values = torch.cat([v[int(p)] for p in table[r, :-(-n // page)]], dim=1)[:, :n]
        for h in range(heads):
            qh = q[r, h * head_dim:(h + 1) * head_dim]
            weights = torch.softmax(keys[h // group] @ qh / head_dim ** 0.5, dim=0)
            out[r, h * head_dim:(h + 1) * head_dim] = weights @ values[h // group]
    return out


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from sprout_lm_b200 import kernels
    lib = kernels.load_library()
    static = lib.sprout_attention_decode_static
    static.restype = ctypes.c_int
    P, I = ctypes.c_void_p, ctypes.c_int
    static.argtypes = [P, I, P, P, P, I, P, P, I, I, I, I, I, I, I, I, I, P, P]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    heads, kv_heads, head_dim, page, split_keys = 14, 2, 64, 16, 128
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lengths in ((1, [300, 129, 16, 640]), (2, [513, 77, 640, 5])):      # two calls in a row
        q, k, v, table, lens = _case(seed, len(lengths), heads, kv_heads, head_dim, page, lengths)
        splits = -(-table.shape[1] * page // split_keys)
        assert splits > 1
        want = torch.empty_like(q)
        kernels.attention_decode(q, k, v, table, lens, want, heads, kv_heads, head_dim, status, split_keys=split_keys)
        got = torch.full_like(q, float("nan"))
        code = static(q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.stride(0),
                      lens.data_ptr(), got.data_ptr(), got.stride(0), len(lengths), heads, kv_heads, head_dim, page,
                      k.shape[0], split_keys, splits, status.data_ptr(), stream)
        assert code == 0, lib.sprout_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert (got.float() - want.float()).abs().max().item() <= 1.2e-2
        plain = _plain(q, k, v, table, lengths, heads, kv_heads, head_dim, page)
        assert (got.double().cpu() - plain).abs().max().item() <= 1.2e-2
    assert int(status.item()) == 0
    # a request that would not fit the built-in array is refused with an explanation, nothing runs
    code = static(q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.stride(0),
                  lens.data_ptr(), got.data_ptr(), got.stride(0), 4, heads, kv_heads, head_dim, page, k.shape[0],
                  split_keys, 20000, status.data_ptr(), stream)
    assert code != 0 and b"built-in array" in lib.sprout_last_error()
