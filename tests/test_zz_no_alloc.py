"""The allocation-free attention entry point, called through the C ABI.

Some users of this library cannot allocate device memory at the moment they need a
decode-attention launch: code written against the reference's launcher signature (which
has no workspace argument), plug-ins inside a server that already gave all of HBM to its
arenas, hosts under a fixed memory budget. For them
`cacheir_b200_paged_attention_decode_batch_noalloc` keeps the split-K scratch in an array
inside the library. This test checks that it returns what the workspace entry point
returns, twice in a row on different inputs (the second call finds the first call's
partials still in the shared array and must not be affected by them), and that sizes
beyond the array are refused. The file name makes pytest collect it last.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed: int, batch: int, heads: int, kv_heads: int, head_dim: int, lens):
    rng = np.random.default_rng(seed)
    page = 16
    pages = [(int(n) + page - 1) // page for n in lens]
    table = np.zeros((batch, max(pages)), dtype=np.int32)
    perm = rng.permutation(sum(pages) + 1).astype(np.int32)
    cur = 0
    for b, n in enumerate(pages):
        table[b, :n] = perm[cur:cur + n]
        cur += n
    q = torch.from_numpy(rng.standard_normal((batch, heads, head_dim)).astype(np.float32)).half().cuda()
    k = torch.from_numpy(rng.standard_normal((sum(pages) + 1, kv_heads, page, head_dim)).astype(np.float32)).half().cuda()
    v = torch.from_numpy(rng.standard_normal((sum(pages) + 1, kv_heads, page, head_dim)).astype(np.float32)).half().cuda()
    return q, k, v, torch.from_numpy(table).cuda(), torch.tensor(list(lens), dtype=torch.int32, device="cuda")


def _call_noalloc(lib, q, k, v, table, lens, splits, out=None):
    out = torch.empty_like(q) if out is None else out
    batch, heads, head_dim = q.shape
    rc = lib.cacheir_b200_paged_attention_decode_batch_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), lens.data_ptr(), out.data_ptr(),
        batch, heads, k.shape[1], table.shape[1], k.shape[2], head_dim, 1, 0, 0, 0.0, splits,
        torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_noalloc_entry_matches_workspace_entry_twice_in_a_row():
    from cacheir_b200 import _lib, ops

    lib = _lib.load()
    assert lib.cacheir_b200_paged_attention_noalloc_max_workspace_bytes() == 16 * 1024 * 1024
    cases = [(1, 4, 8, 2, 128, [700, 33, 1, 450], 4), (2, 3, 16, 4, 64, [90, 1200, 310], 3)]
    for seed, batch, heads, kv_heads, head_dim, lens, splits in cases:
        q, k, v, table, seq = _inputs(seed, batch, heads, kv_heads, head_dim, lens)
        want = ops.paged_attention_decode_batch(q, k, v, table, seq, num_splits=splits)
        got = torch.empty_like(q)
        before = torch.cuda.memory_allocated()
        rc, got = _call_noalloc(lib, q, k, v, table, seq, splits, out=got)
        assert rc == 0, lib.cacheir_b200_error_string(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before      # the call took nothing from torch's allocator
        # same kernels, same partial layout: identical bits; the suite's fp16 gate is rel-L2 <= 2e-3
        err = float((got.float() - want.float()).norm() / want.float().norm())
        assert err <= 2e-3
        assert torch.equal(got, want)


def test_noalloc_entry_refuses_sizes_beyond_its_array():
    from cacheir_b200 import _lib

    lib = _lib.load()
    # 64 sequences x 64 heads x 11 splits (520 tokens in 48-token chunks) x (128+2) floats = 23 MB > 16 MiB
    q, k, v, table, seq = _inputs(3, 64, 64, 8, 128, [520] * 64)
    rc, _ = _call_noalloc(lib, q, k, v, table, seq, 16)
    assert rc == -5
    assert b"maximum" in lib.cacheir_b200_error_string(rc)
    rc, out = _call_noalloc(lib, q, k, v, table, seq, 1)    # one split needs no scratch
    assert rc == 0 and torch.isfinite(out).all()
    # fewer query heads than KV heads is an argument error (checked on the host, before the split count is worked out)
    rc = lib.cacheir_b200_paged_attention_decode_batch_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), seq.data_ptr(), out.data_ptr(),
        64, 4, 8, table.shape[1], 16, 128, 1, 0, 0, 0.0, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    assert lib.cacheir_b200_paged_attention_auto_splits(64, 4, 8, int(table.shape[1]), 16, 128) == 1
