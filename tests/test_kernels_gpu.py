"""Parity of every CUDA kernel, called through the C ABI, against the CPU oracle.

Bars: integer/byte/index results bit-exact; floating point rel-L2 <= 2e-3 in
fp16/bf16 (the tolerance of the decode path's acceptance gate) and <= 2e-5 in fp32.
"""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

# bf16 keeps 8 significant bits: rounding the OUTPUT alone costs up to 2^-8 = 3.9e-3 relative
# (about 1.6e-3 rms), so 2e-3 is not reachable on small outputs whatever the kernel does.
TOL = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 4e-3}
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _ops():
    from cacheir_b200 import ops
    return ops


def _rel(got: torch.Tensor, want: np.ndarray) -> float:
    return oracle.rel_l2(got.detach().float().cpu().numpy(), want)


def _make_paged(rng, batch, heads, kv_heads, head_dim, page, lens, dtype, extra_slots=3, shared_prefix_pages=0):
    """Random q / pools / permuted page table. Inputs are rounded to `dtype` first so the
    oracle sees exactly what the kernel sees."""
    pages_per_seq = [(n + page - 1) // page for n in lens]
    max_pages = max(1, max(pages_per_seq))
    total = sum(pages_per_seq) + extra_slots
    perm = rng.permutation(total).astype(np.int32)
    table = np.zeros((batch, max_pages), dtype=np.int32)   # padding aliases slot 0, as in the reference test
    cursor = 0
    for b, n in enumerate(pages_per_seq):
        table[b, :n] = perm[cursor:cursor + n]
        cursor += n
    if shared_prefix_pages:
        for b in range(1, batch):
            k = min(shared_prefix_pages, pages_per_seq[b], pages_per_seq[0])
            table[b, :k] = table[0, :k]
    q = torch.from_numpy(rng.standard_normal((batch, heads, head_dim)).astype(np.float32)).to(dtype)
    k_pool = torch.from_numpy(rng.standard_normal((total, kv_heads, page, head_dim)).astype(np.float32)).to(dtype)
    v_pool = torch.from_numpy(rng.standard_normal((total, kv_heads, page, head_dim)).astype(np.float32)).to(dtype)
    return q, k_pool, v_pool, table, np.asarray(lens, dtype=np.int32)


def _run_attention(q, k_pool, v_pool, table, lens, **kw):
    ops = _ops()
    out = ops.paged_attention_decode_batch(q.cuda(), k_pool.cuda(), v_pool.cuda(), torch.from_numpy(table).cuda(),
                                           torch.from_numpy(lens).cuda(), **kw)
    want = oracle.paged_attention_decode(q.float().numpy(), k_pool.float().numpy(), v_pool.float().numpy(), table, lens)
    return out, want


def test_attention_reference_test_shape():
    # B=2, H=4, KVH=2, page=2, max_pages=3, D=8 fp32, page table [[0,1,2],[3,4,0]], seq_lens [5,3]:
    # the case of the reference's tests/test_advanced_experiments.py:519-558 (atol 1e-4 there)
    rng = np.random.default_rng(0)
    q = torch.from_numpy(rng.standard_normal((2, 4, 8)).astype(np.float32))
    k_pool = torch.from_numpy(rng.standard_normal((5, 2, 2, 8)).astype(np.float32))
    v_pool = torch.from_numpy(rng.standard_normal((5, 2, 2, 8)).astype(np.float32))
    table = np.asarray([[0, 1, 2], [3, 4, 0]], dtype=np.int32)
    lens = np.asarray([5, 3], dtype=np.int32)
    for splits in (0, 1, 2, 3):
        out, want = _run_attention(q, k_pool, v_pool, table, lens, num_splits=splits)
        np.testing.assert_allclose(out.cpu().numpy(), want, atol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [
    (4, 2, 64, 16), (32, 8, 128, 16), (8, 1, 128, 16), (4, 4, 16, 4), (6, 2, 40, 8), (16, 2, 256, 16), (7, 7, 4, 1),
])
def test_attention_matches_oracle(dtype, heads, kv_heads, head_dim, page):
    rng = np.random.default_rng(heads * 1000 + head_dim)
    lens = [1, page, page + 1, 5 * page - 1, 333, 64]
    q, k_pool, v_pool, table, lens = _make_paged(rng, len(lens), heads, kv_heads, head_dim, page, lens, dtype)
    for splits in (0, 1, 4):
        out, want = _run_attention(q, k_pool, v_pool, table, lens, num_splits=splits)
        assert _rel(out, want) <= TOL[dtype], (dtype, splits)


def test_attention_empty_and_ragged_sequences():
    rng = np.random.default_rng(7)
    lens = [0, 1, 17, 0, 200]
    q, k_pool, v_pool, table, lens = _make_paged(rng, 5, 8, 2, 64, 16, lens, torch.float16)
    out, want = _run_attention(q, k_pool, v_pool, table, lens, num_splits=3)
    assert torch.isfinite(out).all()
    assert float(out[0].abs().max()) == 0.0 and float(out[3].abs().max()) == 0.0
    assert _rel(out, want) <= TOL[torch.float16]


def test_attention_prefix_shared_pages_and_strided_q():
    rng = np.random.default_rng(9)
    lens = [96, 80, 130, 64]
    q, k_pool, v_pool, table, lens = _make_paged(rng, 4, 8, 2, 128, 16, lens, torch.float16, shared_prefix_pages=4)
    assert (table[1:, :4] == table[0, :4]).all()
    out, want = _run_attention(q, k_pool, v_pool, table, lens)
    assert _rel(out, want) <= TOL[torch.float16]
    # q as a strided view of a wider [B, (H+2KVH)*D] projection buffer
    wide = torch.zeros((4, (8 + 4) * 128), dtype=torch.float16, device="cuda")
    wide[:, : 8 * 128] = q.cuda().reshape(4, -1)
    q_view = wide.as_strided((4, 8, 128), (wide.stride(0), 128, 1))
    ops = _ops()
    out2 = ops.paged_attention_decode_batch(q_view, k_pool.cuda(), v_pool.cuda(), torch.from_numpy(table).cuda(),
                                            torch.from_numpy(lens).cuda())
    assert torch.equal(out2, out)


def test_attention_split_combine_is_deterministic():
    rng = np.random.default_rng(3)
    lens = list(rng.integers(100, 3000, 6))
    q, k_pool, v_pool, table, lens = _make_paged(rng, 6, 32, 8, 128, 16, lens, torch.float16)
    a, want = _run_attention(q, k_pool, v_pool, table, lens, num_splits=0)
    b, _ = _run_attention(q, k_pool, v_pool, table, lens, num_splits=0)
    assert torch.equal(a, b)
    assert _rel(a, want) <= TOL[torch.float16]


def test_attention_workspace_contract():
    from cacheir_b200._lib import CacheIRB200Error
    ops = _ops()
    rng = np.random.default_rng(4)
    q, k_pool, v_pool, table, lens = _make_paged(rng, 2, 4, 2, 64, 16, [40, 50], torch.float16)
    tiny_ws = torch.empty(4, dtype=torch.float32, device="cuda")
    with pytest.raises(CacheIRB200Error):
        ops.paged_attention_decode_batch(q.cuda(), k_pool.cuda(), v_pool.cuda(), torch.from_numpy(table).cuda(),
                                         torch.from_numpy(lens).cuda(), num_splits=2, workspace=tiny_ws)
    with pytest.raises((ValueError, TypeError)):
        ops.paged_attention_decode_batch(q.cuda(), k_pool.cuda(), v_pool.cuda(), torch.from_numpy(table).long().cuda(),
                                         torch.from_numpy(lens).cuda())


# ---- dequant GEMV -------------------------------------------------------------------
@pytest.mark.parametrize("batch,heads,kv_heads,lens", [
    (32, 32, 8, None), (5, 16, 4, [1, 16, 17, 300, 0]), (16, 8, 8, None), (17, 20, 4, None), (3, 4, 1, [40, 2, 129])])
def test_attention_with_fused_activation_prepass(batch, heads, kv_heads, lens):
    """The single-split fast kernel run as clusters over the kv heads: the same output bits as the plain launch, and a
    GEMM workspace that is bit for bit what the stand-alone pre-pass makes of that output (padding rows zeroed)."""
    ops = _ops()
    rng = np.random.default_rng(batch * 100 + heads)
    D, page = 128, 16
    if lens is None:
        lens = [int(v) for v in rng.integers(1, 700, batch)]
    assert ops.attention_quantize_supported(batch, heads, kv_heads, (max(lens) + page - 1) // page, page, D, torch.float16)
    q, k_pool, v_pool, table, lens_np = _make_paged(rng, batch, heads, kv_heads, D, page, lens, torch.float16)
    q = (q.float() * torch.from_numpy(rng.uniform(0.05, 8.0, (batch, 1, 1)).astype(np.float32))).half()
    args = (q.cuda(), k_pool.cuda(), v_pool.cuda(), torch.from_numpy(table).cuda(), torch.from_numpy(lens_np).cuda())
    plain = ops.paged_attention_decode_batch(*args, num_splits=1)
    k_total = heads * D
    nbytes = ops.qgemv_workspace_bytes(batch, k_total)
    ws_ref = torch.full((nbytes,), 0xAB, dtype=torch.uint8, device="cuda")
    ops.quantize_activations(plain.view(batch, k_total), ws_ref)
    ws = torch.full((nbytes,), 0xCD, dtype=torch.uint8, device="cuda")          # stale bytes must all be overwritten
    out = torch.empty_like(plain)
    ops.paged_attention_decode_batch_quantize(*args, out=out, gemm_workspace=ws)
    _device_status_ok()
    assert torch.equal(out, plain)
    mp = 16 if batch <= 16 else (32 if batch <= 32 else 64)
    planes = 2 * mp * k_total
    assert torch.equal(ws[:planes], ws_ref[:planes])
    sx, sx_ref = ws[planes:planes + 256].view(torch.float32), ws_ref[planes:planes + 256].view(torch.float32)
    qs, qs_ref = ws[planes + 256:planes + 512].view(torch.int32), ws_ref[planes + 256:planes + 512].view(torch.int32)
    assert torch.equal(sx[:mp], sx_ref[:mp]) and torch.equal(qs[:mp], qs_ref[:mp])
    want = oracle.paged_attention_decode(q.float().numpy(), k_pool.float().numpy(), v_pool.float().numpy(), table, lens_np)
    assert _rel(out, want) <= TOL[torch.float16]
    # the projection behind it takes the planes as they are
    n = 256
    x, packed = _qgemv_case(rng, batch, n, k_total, 8, torch.float16)
    dev = _device_pack(packed)
    kw = dict(bits=8, n=n, k=k_total)
    y_fused = ops.qgemv(out.view(batch, k_total), dev.packed_values, dev.scales, dev.zero_points, workspace=ws, prequantized=True, **kw)
    y_two = ops.qgemv(plain.view(batch, k_total), dev.packed_values, dev.scales, dev.zero_points, workspace=ws_ref, **kw)
    assert torch.equal(y_fused, y_two)
    _device_status_ok()


def test_attention_fused_prepass_support_limits():
    ops = _ops()
    ok = lambda **kw: ops.attention_quantize_supported(**{**dict(batch=8, heads=32, kv_heads=8, max_pages=64, page_size=16,
                                                                  head_dim=128, dtype=torch.float16), **kw})
    assert ok()
    assert not ok(head_dim=64) and not ok(dtype=torch.bfloat16) and not ok(page_size=32)
    assert not ok(kv_heads=16, heads=32)            # more kv heads than a portable cluster holds
    assert not ok(heads=64, kv_heads=8)             # more query heads per kv head than one item per thread covers
    assert not ok(batch=65)


def _qgemv_case(rng, m, n, k, bits, dtype, group=0, reference_pack=True):
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype)
    if group:
        codes = rng.integers(0, 1 << bits, (n, k)).astype(np.uint8)
        scales = rng.uniform(0.005, 0.02, (n, k // group)).astype(np.float16)
        packed = oracle.symmetric_group_pack_from_codes(codes, scales, bits, group)
    elif reference_pack:
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        packed = oracle.asymmetric_pack(w, bits)
    else:   # codes uniform, fp16 per-channel scale, zero point at the midpoint
        codes = rng.integers(0, 1 << bits, (n, k)).astype(np.uint8)
        packed = oracle.PackedQuantizedTensor(oracle.pack_int4(codes) if bits == 4 else codes,
                                              rng.uniform(0.005, 0.02, n).astype(np.float16),
                                              np.full(n, 1 << (bits - 1), dtype=np.int32), bits, (n, k))
    return x, packed


def _device_pack(packed):
    from cacheir_b200.quantization import upload_reference_pack
    return upload_reference_pack(packed, "cuda")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,n,k", [(1, 64, 256), (3, 96, 688), (8, 40, 1024), (32, 128, 512), (64, 24, 96), (2, 17, 53)])
def test_qgemv_per_row_affine_matches_oracle(dtype, bits, m, n, k):
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(m * 7 + n + k + bits)
    x, packed = _qgemv_case(rng, m, n, k, bits, dtype)
    y = quantized_matmul(x.cuda(), _device_pack(packed))
    want = oracle.quantized_matmul(x.float().numpy(), packed)
    assert y.shape == (m, n)
    assert _rel(y, want) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m", [1, 8, 32])
def test_qgemv_group128_int4_matches_oracle(dtype, m):
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(100 + m)
    x, packed = _qgemv_case(rng, m, 192, 1024, 4, dtype, group=128)
    y = quantized_matmul(x.cuda(), _device_pack(packed))
    want = oracle.quantized_matmul(x.float().numpy(), packed)
    assert _rel(y, want) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_qgemv_fp16_scales_and_epilogues(dtype):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(21)
    m, n, k = 4, 128, 512
    x, packed = _qgemv_case(rng, m, n, k, 8, dtype, reference_pack=False)
    dev = _device_pack(packed)
    dev.scales = torch.from_numpy(packed.scales).cuda()         # keep the fp16 per-channel scales
    base = oracle.quantized_matmul(x.float().numpy(), packed)
    assert _rel(quantized_matmul(x.cuda(), dev), base) <= TOL[dtype]
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(dtype)
    y = quantized_matmul(x.cuda(), dev, epilogue=ops.EPI_RESIDUAL, residual=res.cuda())
    assert _rel(y, base + res.float().numpy()) <= TOL[dtype]
    y = quantized_matmul(x.cuda(), dev, epilogue=ops.EPI_SWIGLU)
    assert y.shape == (m, n // 2)
    assert _rel(y, oracle.silu_mul(base[:, : n // 2], base[:, n // 2:])) <= TOL[dtype] * 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_gemv_matches_oracle(dtype):
    ops = _ops()
    rng = np.random.default_rng(5)
    for m, n, k in [(1, 64, 256), (5, 33, 100), (16, 1024, 256)]:
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype)
        w = torch.from_numpy((rng.standard_normal((n, k)) * 0.05).astype(np.float32)).to(dtype)
        y = ops.qgemv(x.cuda(), w.cuda(), None, None, bits=0, n=n, k=k)
        assert _rel(y, oracle.matmul(x.float().numpy(), w.float().numpy())) <= TOL[dtype]


# ---- quantization loader: bit-exact -------------------------------------------------
def test_pack_rows_is_bit_exact_with_reference_golden(golden_dir):
    ops = _ops()
    g = np.load(golden_dir / "pack.npz")
    for prefix in ("lin", "rnd", "even"):
        w = torch.from_numpy(g[f"{prefix}_w"]).cuda()
        for bits, tag in ((4, "q4"), (8, "q8")):
            packed, scales, zp_i, zp_f = ops.pack_rows(w, bits)
            np.testing.assert_array_equal(packed.cpu().numpy(), g[f"{prefix}_{tag}_packed"])
            np.testing.assert_array_equal(zp_i.cpu().numpy(), g[f"{prefix}_{tag}_zero_points"])
            np.testing.assert_array_equal(scales.cpu().numpy(), g[f"{prefix}_{tag}_scales"])
            np.testing.assert_array_equal(zp_f.cpu().numpy(), g[f"{prefix}_{tag}_zero_points"].astype(np.float32))
            deq = ops.dequantize_rows(packed, scales, zp_f, bits=bits, k=w.shape[1], dtype=torch.float32)
            np.testing.assert_array_equal(deq.cpu().numpy(), g[f"{prefix}_{tag}_dequant"])


def test_pack_rows_matches_oracle_on_model_sized_rows():
    ops = _ops()
    rng = np.random.default_rng(12)
    w = (rng.standard_normal((64, 4096)) * 0.02).astype(np.float32)
    for bits in (4, 8):
        want = oracle.asymmetric_pack(w, bits)
        packed, scales, zp_i, _ = ops.pack_rows(torch.from_numpy(w).cuda(), bits)
        np.testing.assert_array_equal(packed.cpu().numpy(), want.packed_values)
        np.testing.assert_array_equal(scales.cpu().numpy(), want.scales)
        np.testing.assert_array_equal(zp_i.cpu().numpy(), want.zero_points)


# ---- glue ops -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [48, 256, 4096, 8192, 1000])
def test_rms_norm_and_fused_residual(dtype, hidden):
    ops = _ops()
    rng = np.random.default_rng(hidden)
    x = torch.from_numpy(rng.standard_normal((5, hidden)).astype(np.float32)).to(dtype)
    r = torch.from_numpy(rng.standard_normal((5, hidden)).astype(np.float32)).to(dtype)
    w = torch.from_numpy(rng.standard_normal((hidden,)).astype(np.float32)).to(dtype)
    out = ops.rms_norm(x.cuda(), w.cuda(), 1e-5)
    assert _rel(out, oracle.rms_norm(x.float().numpy(), w.float().numpy(), 1e-5)) <= TOL[dtype]
    summed = torch.empty_like(x, device="cuda")
    out = ops.rms_norm(x.cuda(), w.cuda(), 1e-5, residual=r.cuda(), sum_out=summed)
    want_sum = (x.float() + r.float()).to(dtype)
    assert torch.equal(summed.cpu(), want_sum)          # the residual stream is the rounded sum, exactly
    assert _rel(out, oracle.rms_norm(want_sum.float().numpy(), w.float().numpy(), 1e-5)) <= TOL[dtype]


def test_rope_matches_reference_golden(golden_dir):
    ops = _ops()
    g = np.load(golden_dir / "numerics.npz")
    x = g["rope_x"]                                      # [2, 3, 4*16]; every (batch, seq) row gets its own position
    for off, key in ((7, "rope_out_off7"), (0, "rope_out_off0")):
        rows = torch.from_numpy(x.reshape(6, 64).copy()).cuda()
        pos = torch.tensor([off, off + 1, off + 2] * 2, dtype=torch.int32, device="cuda")
        ops.rope_inplace(rows, pos, num_heads=4, head_dim=16, theta=10000.0)
        np.testing.assert_allclose(rows.cpu().numpy().reshape(2, 3, 64), g[key], rtol=2e-5, atol=2e-5)


def test_kv_append_writes_the_right_page_rows():
    ops = _ops()
    rng = np.random.default_rng(2)
    batch, kvh, d, page = 3, 2, 8, 4
    k_pool = torch.zeros((10, kvh, page, d), device="cuda")
    v_pool = torch.zeros_like(k_pool)
    table = torch.tensor([[5, 1, 0], [2, 7, 9], [3, 0, 0]], dtype=torch.int32, device="cuda")
    pos = torch.tensor([6, 11, 0], dtype=torch.int32, device="cuda")
    wide = torch.from_numpy(rng.standard_normal((batch, 3 * kvh * d)).astype(np.float32)).cuda()
    k, v = wide[:, kvh * d: 2 * kvh * d], wide[:, 2 * kvh * d:]
    ops.kv_append(k, v, k_pool, v_pool, table, pos)
    want_k = np.zeros((10, kvh, page, d), dtype=np.float32)
    want_v = np.zeros_like(want_k)
    for b, (slot, off) in enumerate([(1, 2), (9, 3), (3, 0)]):
        want_k[slot, :, off] = k[b].cpu().numpy().reshape(kvh, d)
        want_v[slot, :, off] = v[b].cpu().numpy().reshape(kvh, d)
    np.testing.assert_array_equal(k_pool.cpu().numpy(), want_k)
    np.testing.assert_array_equal(v_pool.cpu().numpy(), want_v)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rope_append_equals_rope_then_append(dtype):
    """One launch for RoPE on q|k and the append of the new k / v rows: the bits of the two separate launches,
    on a row-strided fused buffer, with a position past the reserved pages (dropped) and q wider than k (GQA)."""
    ops = _ops()
    rng = np.random.default_rng(11)
    batch, heads, kvh, d, page = 5, 6, 2, 16, 4
    q_dim, k_dim = heads * d, kvh * d
    pool_shape = (12, kvh, page, d)
    table = torch.tensor([[5, 1, 0], [2, 7, 9], [3, 0, 0], [4, 6, 8], [10, 11, 0]], dtype=torch.int32, device="cuda")
    pos = torch.tensor([6, 11, 0, 13, 5], dtype=torch.int32, device="cuda")     # row 3: page index 3 is not in the table
    wide = torch.from_numpy(rng.standard_normal((batch, q_dim + 2 * k_dim + 8)).astype(np.float32)).to(dtype).cuda()
    a, b = wide.clone(), wide.clone()
    qkv_a, qkv_b = a[:, 4:4 + q_dim + 2 * k_dim], b[:, 4:4 + q_dim + 2 * k_dim]
    ka, va = torch.zeros(pool_shape, device="cuda", dtype=dtype), torch.zeros(pool_shape, device="cuda", dtype=dtype)
    kb, vb = torch.zeros_like(ka), torch.zeros_like(va)
    ops.rope_inplace(qkv_a[:, : q_dim + k_dim], pos, num_heads=heads + kvh, head_dim=d, theta=10000.0)
    ops.kv_append(qkv_a[:, q_dim:q_dim + k_dim], qkv_a[:, q_dim + k_dim:], ka, va, table[:, :3].contiguous(), pos)
    ops.rope_append(qkv_b, pos, table[:, :3].contiguous(), kb, vb, q_dim=q_dim, k_dim=k_dim, head_dim=d, theta=10000.0)
    assert torch.equal(a, b) and torch.equal(ka, kb) and torch.equal(va, vb)
    assert ka.abs().sum() > 0 and not ka[0].any()                                 # rows were written; slot 0 was not touched


@pytest.mark.parametrize("dtype", DTYPES)
def test_elementwise_embedding_argmax(dtype):
    ops = _ops()
    rng = np.random.default_rng(8)
    a = torch.from_numpy(rng.standard_normal((3, 1000)).astype(np.float32)).to(dtype)
    b = torch.from_numpy(rng.standard_normal((3, 1000)).astype(np.float32)).to(dtype)
    assert torch.equal(ops.add(a.cuda(), b.cuda()).cpu(), (a.float() + b.float()).to(dtype))
    assert _rel(ops.silu_mul(a.cuda(), b.cuda()), oracle.silu_mul(a.float().numpy(), b.float().numpy())) <= TOL[dtype]
    table = torch.from_numpy(rng.standard_normal((50, 24)).astype(np.float32)).to(dtype)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int64)
    assert torch.equal(ops.embedding_gather(table.cuda(), ids.cuda()).cpu(), table[ids])
    logits = torch.from_numpy(rng.standard_normal((4, 5000)).astype(np.float32)).to(dtype)
    logits[1, 77] = 100.0
    logits[2, 10] = logits[2, 4000] = 50.0             # tie -> lowest index
    got = ops.argmax_rows(logits.cuda()).cpu()
    assert torch.equal(got, logits.float().argmax(dim=-1))
    assert got[1] == 77 and got[2] == 10


def test_advance_positions():
    ops = _ops()
    lens = torch.tensor([0, 5, 31], dtype=torch.int32, device="cuda")
    pos = torch.zeros_like(lens)
    ops.advance_positions(pos, lens)
    assert pos.tolist() == [0, 5, 31] and lens.tolist() == [1, 6, 32]


# ---- tensor-core (tcgen05) small-M dequant-GEMM: fp16 activations, K % 128 == 0 -----------
def _device_status_ok():
    from cacheir_b200 import _lib
    status = _lib.load().cacheir_b200_device_status(1)
    assert status == 0, f"a bounded device wait gave up: status {status:#x}"


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m", [1, 8, 16, 17, 32, 64])
@pytest.mark.parametrize("n,k", [(512, 1024), (200, 256), (128, 4096)])
def test_qgemm_tensor_core_per_row_affine(bits, m, n, k):
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(bits * 1000 + m * 10 + n + k)
    x, packed = _qgemv_case(rng, m, n, k, bits, torch.float16)
    y = quantized_matmul(x.cuda(), _device_pack(packed))
    torch.cuda.synchronize()
    _device_status_ok()
    want = oracle.quantized_matmul(x.float().numpy(), packed)
    assert _rel(y, want) <= TOL[torch.float16]


@pytest.mark.parametrize("m", [1, 32, 64])
def test_qgemm_tensor_core_group128_int4_and_midpoint_int8(m):
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(300 + m)
    x, packed = _qgemv_case(rng, m, 384, 2048, 4, torch.float16, group=128)
    y = quantized_matmul(x.cuda(), _device_pack(packed))
    assert _rel(y, oracle.quantized_matmul(x.float().numpy(), packed)) <= TOL[torch.float16]
    x, packed = _qgemv_case(rng, m, 256, 1024, 8, torch.float16, reference_pack=False)   # fp16 scales, zero = 128
    dev = _device_pack(packed)
    dev.scales = torch.from_numpy(packed.scales).cuda()
    y = quantized_matmul(x.cuda(), dev)
    torch.cuda.synchronize()
    _device_status_ok()
    assert _rel(y, oracle.quantized_matmul(x.float().numpy(), packed)) <= TOL[torch.float16]


def test_qgemm_tensor_core_epilogues_and_odd_zero_points():
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(77)
    m, n, k = 32, 512, 1024
    x, packed = _qgemv_case(rng, m, n, k, 8, torch.float16)
    # rows the fast in-register path cannot take: huge and fractional zero points
    packed.zero_points = packed.zero_points.astype(np.float64)
    dev = _device_pack(packed)
    zp = dev.zero_points.clone()
    zp[3] = 25000.0
    zp[5] = 100.5
    dev.zero_points = zp
    host = oracle.PackedQuantizedTensor(packed.packed_values, packed.scales, zp.cpu().numpy(), 8, (n, k))
    base = oracle.quantized_matmul(x.float().numpy(), host)
    keep = [i for i in range(n) if i != 3]      # row 3 saturates fp16 by construction; compare the rest
    y = quantized_matmul(x.cuda(), dev)
    assert _rel(y[:, keep], base[:, keep]) <= TOL[torch.float16]
    x, packed = _qgemv_case(rng, m, n, k, 8, torch.float16)
    dev = _device_pack(packed)
    base = oracle.quantized_matmul(x.float().numpy(), packed)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).half()
    y = quantized_matmul(x.cuda(), dev, epilogue=ops.EPI_RESIDUAL, residual=res.cuda())
    assert _rel(y, base + res.float().numpy()) <= TOL[torch.float16]
    y = quantized_matmul(x.cuda(), dev, epilogue=ops.EPI_SWIGLU)
    assert y.shape == (m, n // 2)
    assert _rel(y, oracle.silu_mul(base[:, : n // 2], base[:, n // 2:])) <= TOL[torch.float16] * 2
    # x as a strided view of a wider buffer
    wide = torch.zeros((m, k + 256), dtype=torch.float16, device="cuda")
    wide[:, :k] = x.cuda()
    y2 = quantized_matmul(wide[:, :k], dev)
    assert _rel(y2, base) <= TOL[torch.float16]
    torch.cuda.synchronize()
    _device_status_ok()


# ---- integer tensor-core path: int8 codes straight into tcgen05.mma kind::i8 -------------
@pytest.mark.parametrize("bits", [8, 4])       # int4 per-row codes are unpacked to bytes inside the same kernel
@pytest.mark.parametrize("m", [1, 8, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k", [(512, 1024), (200, 256), (128, 4096), (4096, 2048)])
def test_qgemm_int8_tensor_core_with_workspace(m, n, k, bits):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(m * 31 + n + k)
    x, packed = _qgemv_case(rng, m, n, k, bits, torch.float16)
    ws = torch.zeros(ops.qgemv_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")
    y = quantized_matmul(x.cuda(), _device_pack(packed), workspace=ws)
    torch.cuda.synchronize()
    _device_status_ok()
    want = oracle.quantized_matmul(x.float().numpy(), packed)
    assert _rel(y, want) <= TOL[torch.float16]
    # and it agrees with the fp16 tensor-core path to well inside the gate
    y2 = quantized_matmul(x.cuda(), _device_pack(packed))
    assert _rel(y, y2.float().cpu().numpy()) <= TOL[torch.float16]


def test_qgemm_int8_tensor_core_epilogues_offsets_and_determinism():
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(91)
    m, n, k = 32, 512, 2048
    x, packed = _qgemv_case(rng, m, n, k, 8, torch.float16)
    x = (x.float() * 3.0 + 2.5).half()          # activations with a large mean: the zero-point term must cancel exactly
    x[5] = 0                                    # an all-zero row
    x[7, 3] = 60000.0                           # a row dominated by one huge value
    dev = _device_pack(packed)
    dev.zero_points[3] = 2500.0                 # an unclipped zero point of the reference packer
    dev.zero_points[9] = 100.5
    host = oracle.PackedQuantizedTensor(packed.packed_values, packed.scales, dev.zero_points.cpu().numpy(), 8, (n, k))
    base = oracle.quantized_matmul(x.float().numpy(), host)
    ws = torch.zeros(ops.qgemv_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")
    y = quantized_matmul(x.cuda(), dev, workspace=ws)
    rows = [i for i in range(m) if i != 7]      # row 7 overflows fp16 in the oracle too
    assert _rel(y[rows], base[rows]) <= TOL[torch.float16]
    assert float(y[5].abs().max()) == 0.0
    y_again = quantized_matmul(x.cuda(), dev, workspace=ws)
    assert torch.equal(y, y_again)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).half()
    y = quantized_matmul(x.cuda(), dev, epilogue=ops.EPI_RESIDUAL, residual=res.cuda(), workspace=ws)
    assert _rel(y[rows], (base + res.float().numpy())[rows]) <= TOL[torch.float16]
    x2, packed2 = _qgemv_case(rng, m, n, k, 8, torch.float16)
    base2 = oracle.quantized_matmul(x2.float().numpy(), packed2)
    y = quantized_matmul(x2.cuda(), _device_pack(packed2), epilogue=ops.EPI_SWIGLU, workspace=ws)
    assert y.shape == (m, n // 2)
    assert _rel(y, oracle.silu_mul(base2[:, : n // 2], base2[:, n // 2:])) <= TOL[torch.float16] * 2
    torch.cuda.synchronize()
    _device_status_ok()


# ---- the GEMM's own pre-pass == the stand-alone pre-pass entry point; strided activations; RMSNorm in front ----
@pytest.mark.parametrize("m", [1, 7, 17, 32, 64])
@pytest.mark.parametrize("n,k,tiled", [(512, 1024, True), (200, 256, False), (2304, 2048, True)])
def test_qgemm_int8_prepass_forms_agree(m, n, k, tiled):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import to_tiled
    rng = np.random.default_rng(m * 13 + n + k)
    x, packed = _qgemv_case(rng, m, n, k, 8, torch.float16)
    x = (x.float() * torch.from_numpy(rng.uniform(0.01, 30.0, (m, 1)).astype(np.float32))).half()   # rows of very different size
    dev = to_tiled(_device_pack(packed)) if tiled else _device_pack(packed)
    ws = torch.zeros(ops.qgemv_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")
    kw = dict(bits=8, n=n, k=k, workspace=ws, tiled=tiled)
    xd = x.cuda()
    assert ops.qgemv_plan(m, n, k, bits=8, tiled=tiled)["family"] == "i8"
    direct = ops.qgemv(xd, dev.packed_values, dev.scales, dev.zero_points, **kw)
    ops.quantize_activations(xd, ws)
    prequantized = ops.qgemv(xd, dev.packed_values, dev.scales, dev.zero_points, prequantized=True, **kw)
    _device_status_ok()
    assert torch.equal(direct, prequantized)                  # the same fixed-point integers, so the same bits
    assert _rel(direct, oracle.quantized_matmul(x.float().numpy(), packed)) <= TOL[torch.float16]
    # a strided view of a wider buffer (what the runtime passes for q / k / v slices)
    wide = torch.zeros((m, k + 64), dtype=torch.float16, device="cuda")
    wide[:, 8:8 + k] = xd
    strided = ops.qgemv(wide[:, 8:8 + k], dev.packed_values, dev.scales, dev.zero_points, **kw)
    assert torch.equal(strided, direct)
    _device_status_ok()


@pytest.mark.parametrize("m", [1, 8, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k,tiled", [(512, 1024, True), (200, 256, False), (128, 4096, True), (2304, 2048, False)])
def test_rmsnorm_in_front_of_the_integer_gemm(m, n, k, tiled):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul, to_tiled
    rng = np.random.default_rng(m * 17 + n + k)
    x, packed = _qgemv_case(rng, m, n, k, 8, torch.float16)
    x = (x.float() * torch.from_numpy(rng.uniform(0.05, 20.0, (m, 1)).astype(np.float32))).half()
    w = torch.from_numpy((1.0 + 0.3 * rng.standard_normal(k)).astype(np.float32)).half()
    dev = to_tiled(_device_pack(packed)) if tiled else _device_pack(packed)
    ws = torch.zeros(ops.qgemv_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")
    fused = ops.qgemv(x.cuda(), dev.packed_values, dev.scales, dev.zero_points, bits=8, n=n, k=k, workspace=ws, tiled=tiled,
                      norm_weight=w.cuda(), norm_eps=1e-5)
    _device_status_ok()
    # the same as its two launches called one by one, bit for bit
    ops.rms_norm_quantize(x.cuda(), w.cuda(), 1e-5, ws)
    two_calls = ops.qgemv(x.cuda(), dev.packed_values, dev.scales, dev.zero_points, bits=8, n=n, k=k, workspace=ws, tiled=tiled,
                          prequantized=True)
    assert torch.equal(fused, two_calls)
    # and close to RMSNorm stored as fp16 followed by the GEMM with its own pre-pass, and to the oracle
    normed = ops.rms_norm(x.cuda(), w.cuda(), 1e-5)
    two_step = quantized_matmul(normed, dev, workspace=ws)
    want = oracle.quantized_matmul(oracle.rms_norm(x.float().numpy(), w.float().numpy(), 1e-5), packed)
    assert _rel(fused, want) <= TOL[torch.float16]
    assert _rel(fused, two_step.float().cpu().numpy()) <= 1e-3
    # an all-zero row stays zero (rms -> eps)
    x0 = x.clone()
    x0[0] = 0
    out0 = ops.qgemv(x0.cuda(), dev.packed_values, dev.scales, dev.zero_points, bits=8, n=n, k=k, workspace=ws, tiled=tiled,
                     norm_weight=w.cuda(), norm_eps=1e-5)
    assert float(out0[0].abs().max()) == 0.0 and torch.equal(out0[1:], fused[1:])
    _device_status_ok()


def test_rmsnorm_qkv_rope_append_equals_its_two_launches():
    from cacheir_b200 import ops
    from cacheir_b200.quantization import to_tiled
    rng = np.random.default_rng(77)
    m, k, head_dim, heads, kv_heads, page, max_pages, theta = 19, 1024, 128, 4, 2, 16, 6, 10000.0
    q_dim, k_dim = heads * head_dim, kv_heads * head_dim
    n = q_dim + 2 * k_dim
    x, packed = _qgemv_case(rng, m, n, k, 8, torch.float16)
    weight = to_tiled(_device_pack(packed))
    w = torch.from_numpy((1.0 + 0.3 * rng.standard_normal(k)).astype(np.float32)).half().cuda()
    slots = m * max_pages + 3
    table_np = rng.permutation(slots)[: m * max_pages].astype(np.int32).reshape(m, max_pages)
    pos_np = rng.integers(0, page * max_pages, m).astype(np.int32)
    positions, page_table = torch.from_numpy(pos_np).cuda(), torch.from_numpy(table_np).cuda()
    pool = lambda: torch.zeros((slots, kv_heads, page, head_dim), dtype=torch.float16, device="cuda")
    k_a, v_a, k_b, v_b = pool(), pool(), pool(), pool()
    ws = torch.zeros(ops.qgemv_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")
    rope = ops.rope_table(page * max_pages, head_dim, theta, "cuda")
    common = dict(n=n, k=k, q_dim=q_dim, k_dim=k_dim, head_dim=head_dim, theta=theta, table=rope, positions=positions,
                  page_table=page_table, workspace=ws, tiled=True)
    xd = x.cuda()
    fused = torch.empty((m, n), dtype=torch.float16, device="cuda")
    ops.qkv_rope_append(xd, weight.packed_values, weight.scales, weight.zero_points, fused, k_cache=k_a, v_cache=v_a,
                        norm_weight=w, norm_eps=1e-5, **common)
    ops.rms_norm_quantize(xd, w, 1e-5, ws)
    ref = torch.empty_like(fused)
    ops.qkv_rope_append(None, weight.packed_values, weight.scales, weight.zero_points, ref, k_cache=k_b, v_cache=v_b,
                        prequantized=True, **common)
    _device_status_ok()
    assert torch.equal(fused, ref) and torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
    for b in range(m):     # the appended rows are bit copies of the k / v columns of the same launch
        slot, off = int(table_np[b, pos_np[b] // page]), int(pos_np[b] % page)
        assert torch.equal(k_a[slot, :, off].reshape(-1), fused[b, q_dim:q_dim + k_dim])
        assert torch.equal(v_a[slot, :, off].reshape(-1), fused[b, q_dim + k_dim:])


# ---- streaming int4 GEMV (up to 8 batch rows, row-major codes): group-wise and the reference's per-row form ----
@pytest.mark.parametrize("m", [1, 2, 5, 8])
@pytest.mark.parametrize("n,k,group", [(200, 256, 128), (48, 1024, 128), (512, 4096, 128), (96, 8192, 256), (64, 14336, 128),
                                       (200, 512, 0), (1024, 4096, 0), (33, 9216, 0)])
def test_streaming_int4_gemv_small_batches(m, n, k, group):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(m * 1000 + n + k + group)
    x, packed = _qgemv_case(rng, m, n, k, 4, torch.float16, group=group)
    dev = _device_pack(packed)
    assert ops.qgemv_plan(m, n, k, bits=4, group_size=group, workspace=False)["family"] == "stream_int4"
    want = oracle.quantized_matmul(x.float().numpy(), packed)
    y = quantized_matmul(x.cuda(), dev)
    assert y.shape == (m, n)
    assert _rel(y, want) <= TOL[torch.float16]
    assert torch.equal(y, quantized_matmul(x.cuda(), dev))          # fixed order of additions: the same bits every time
    # a row-strided view of a wider buffer, and the residual epilogue
    wide = torch.zeros((m, k + 32), dtype=torch.float16, device="cuda")
    wide[:, 16:16 + k] = x.cuda()
    assert torch.equal(quantized_matmul(wide[:, 16:16 + k], dev), y)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).half()
    yr = quantized_matmul(x.cuda(), dev, epilogue=ops.EPI_RESIDUAL, residual=res.cuda())
    assert _rel(yr, want + res.float().numpy()) <= TOL[torch.float16]


def test_streaming_int4_gemv_swiglu_and_unclipped_zero_points():
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(4242)
    m, n, k = 3, 256, 1024
    for group in (128, 0):
        x, packed = _qgemv_case(rng, m, n, k, 4, torch.float16, group=group)
        dev = _device_pack(packed)
        if group == 0:
            dev.zero_points[5] = 100.0          # the reference packer does not clip zero points
            dev.zero_points[9] = 7.5
            packed = oracle.PackedQuantizedTensor(packed.packed_values, packed.scales, dev.zero_points.cpu().numpy(), 4, (n, k))
        base = oracle.quantized_matmul(x.float().numpy(), packed)
        y = quantized_matmul(x.cuda(), dev, epilogue=ops.EPI_SWIGLU)
        assert y.shape == (m, n // 2)
        assert _rel(y, oracle.silu_mul(base[:, : n // 2], base[:, n // 2:])) <= 2 * TOL[torch.float16]
        assert _rel(quantized_matmul(x.cuda(), dev), base) <= TOL[torch.float16]


@pytest.mark.parametrize("m,n,k,group,swiglu", [(2, 40000, 256, 128, False), (3, 40960, 256, 128, True), (8, 40000, 512, 0, False),
                                                (7, 2400, 14336, 128, False)])
def test_streaming_int4_gemv_many_tiles_per_sm(m, n, k, group, swiglu):
    """More than 16 weight tiles per SM (several rounds) and several chunks of x with full rounds."""
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(n + k + m)
    x, packed = _qgemv_case(rng, m, n, k, 4, torch.float16, group=group)
    dev = _device_pack(packed)
    assert ops.qgemv_plan(m, n, k, bits=4, group_size=group, workspace=False,
                          epilogue=ops.EPI_SWIGLU if swiglu else ops.EPI_NONE)["family"] == "stream_int4"
    base = oracle.quantized_matmul(x.float().numpy(), packed)
    if swiglu:
        y = quantized_matmul(x.cuda(), dev, epilogue=ops.EPI_SWIGLU)
        assert _rel(y, oracle.silu_mul(base[:, : n // 2], base[:, n // 2:])) <= 2 * TOL[torch.float16]
    else:
        y = quantized_matmul(x.cuda(), dev)
        assert _rel(y, base) <= TOL[torch.float16]
    _device_status_ok()


# ---- device pack layout: tile order is an exact permutation and changes no result ---------
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("n,k", [(512, 1024), (200, 256), (128, 4096)])
def test_pack_relayout_roundtrip_and_gemm_equivalence(bits, n, k):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul, to_rows, to_tiled
    rng = np.random.default_rng(bits + n + k)
    x, packed = _qgemv_case(rng, 32, n, k, bits, torch.float16)
    rows = _device_pack(packed)
    tiled = to_tiled(rows)
    assert tiled.tiled and tiled.packed_values.numel() == ops.pack_tiled_bytes(n, k, bits)
    back = to_rows(tiled)
    assert torch.equal(back.packed_values, rows.packed_values)            # bit-exact inverse
    # spot-check the permutation itself: tile (band, kb) holds rows band*128.. and bytes kb*TB..
    tb = 128 if bits == 8 else 64
    kblocks = (k if bits == 8 else k // 2) // tb
    t = tiled.packed_values.cpu().numpy().reshape(-1, kblocks, 128, tb)
    ref = packed.packed_values
    band, kb, r = (n - 1) // 128, kblocks - 1, (n - 1) % 128
    # inside a tile row the 16-byte chunks sit in the shared-memory swizzle order (chunk c at c ^ key(r))
    key = (r & 7) if bits == 8 else ((r >> 1) & 3)
    chunks = t[band, kb, r].reshape(tb // 16, 16)
    unswizzled = np.stack([chunks[c ^ key] for c in range(tb // 16)]).reshape(-1)
    np.testing.assert_array_equal(unswizzled, ref[n - 1, kb * tb:(kb + 1) * tb])
    assert not t[band, :, r + 1:].any()                                  # rows past N are zero padding
    y_rows = quantized_matmul(x.cuda(), rows)
    y_tiled = quantized_matmul(x.cuda(), tiled)
    assert torch.equal(y_rows, y_tiled)
    ws = torch.zeros(ops.qgemv_workspace_bytes(32, k), dtype=torch.uint8, device="cuda")
    assert torch.equal(quantized_matmul(x.cuda(), rows, workspace=ws), quantized_matmul(x.cuda(), tiled, workspace=ws))
    if n % 256 == 0:
        a = quantized_matmul(x.cuda(), rows, epilogue=ops.EPI_SWIGLU)
        b = quantized_matmul(x.cuda(), tiled, epilogue=ops.EPI_SWIGLU)
        assert torch.equal(a, b)
    if n % 128 == 0:
        # [gate; up] pairing: tile t = gate rows 64t.. followed by up rows n/2+64t..; exact inverse, same SwiGLU result
        paired = to_tiled(rows, paired=True)
        assert paired.paired and torch.equal(to_rows(paired).packed_values, rows.packed_values)
        tp = paired.packed_values.cpu().numpy().reshape(-1, kblocks, 128, tb)
        for r, src in ((5, 64 + 5), (64 + 9, n // 2 + 64 + 9)):            # tile 1: a gate row and an up row
            if n >= 256:
                key = (r & 7) if bits == 8 else ((r >> 1) & 3)
                chunks = tp[1, 0, r].reshape(tb // 16, 16)
                np.testing.assert_array_equal(np.stack([chunks[c ^ key] for c in range(tb // 16)]).reshape(-1), ref[src, :tb])
        ws = torch.zeros(ops.qgemv_workspace_bytes(32, k), dtype=torch.uint8, device="cuda")
        a = quantized_matmul(x.cuda(), rows, epilogue=ops.EPI_SWIGLU, workspace=ws)
        b = quantized_matmul(x.cuda(), paired, epilogue=ops.EPI_SWIGLU, workspace=ws)
        assert torch.equal(a, b)
        base = oracle.quantized_matmul(x.float().numpy(), packed)
        assert _rel(a, oracle.silu_mul(base[:, : n // 2], base[:, n // 2:])) <= TOL[torch.float16] * 2
        with pytest.raises(Exception):                                      # only the integer kernel reads paired tiles
            quantized_matmul(x.cuda(), paired, epilogue=ops.EPI_SWIGLU)
    torch.cuda.synchronize()
    _device_status_ok()


def test_rms_norm_quantize_and_prequantized_gemm_match_the_two_step_path():
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(123)
    for m, n, k in [(32, 512, 4096), (5, 256, 1024), (64, 384, 8192)]:
        x, packed = _qgemv_case(rng, m, n, k, 8, torch.float16)
        res = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).half().cuda()
        w = torch.from_numpy(rng.standard_normal((k,)).astype(np.float32)).half().cuda()
        dev = _device_pack(packed)
        ws = torch.zeros(ops.qgemv_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")
        # two-step: rms_norm (+residual) to fp16, then the GEMM with its own pre-pass
        summed = torch.empty_like(res)
        normed = ops.rms_norm(x.cuda(), w, 1e-5, residual=res, sum_out=summed)
        want = quantized_matmul(normed, dev, workspace=ws)
        # fused: one kernel normalises and quantises, the GEMM consumes the workspace
        summed2 = torch.empty_like(res)
        out2 = torch.empty_like(res)
        ops.rms_norm_quantize(x.cuda(), w, 1e-5, ws, residual=res, sum_out=summed2, out=out2)
        got = ops.qgemv(x.cuda(), dev.packed_values, dev.scales, dev.zero_points, bits=8, n=n, k=k, workspace=ws, prequantized=True)
        assert torch.equal(summed, summed2)
        # the two kernels reduce the sum of squares with different block shapes: the fp16 rows may differ by one ulp
        assert _rel(out2, normed.float().cpu().numpy()) <= 5e-4
        assert _rel(got, want.float().cpu().numpy()) <= TOL[torch.float16]
        # stand-alone pre-pass entry point
        ops.quantize_activations(normed, ws)
        got2 = ops.qgemv(x.cuda(), dev.packed_values, dev.scales, dev.zero_points, bits=8, n=n, k=k, workspace=ws, prequantized=True)
        assert torch.equal(got2, want)          # same pre-pass arithmetic, same integers
        base = oracle.quantized_matmul(normed.float().cpu().numpy(), packed)
        assert _rel(got, base) <= TOL[torch.float16]
    torch.cuda.synchronize()
    _device_status_ok()


# ---- fused QKV projection + RoPE + cache append == the three separate kernels, bit for bit ----
@pytest.mark.parametrize("k,tiled", [(1024, True), (1024, False), (256, True)])   # K=1024: cluster split-K; K=256: one CTA per tile
def test_qkv_rope_append_equals_separate_kernels(k, tiled):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul, to_tiled
    rng = np.random.default_rng(k + int(tiled))
    m, head_dim, heads, kv_heads, page, max_pages, theta = 13, 128, 4, 2, 16, 6, 10000.0
    q_dim, k_dim = heads * head_dim, kv_heads * head_dim
    n = q_dim + 2 * k_dim
    x, packed = _qgemv_case(rng, m, n, k, 8, torch.float16)
    rows = _device_pack(packed)
    weight = to_tiled(rows) if tiled else rows
    slots = m * max_pages + 3
    table_np = rng.permutation(slots)[: m * max_pages].astype(np.int32).reshape(m, max_pages)
    # positions inside the table of cos/sin, one of them without a reserved page
    pos_np = rng.integers(0, 60, m).astype(np.int32)
    pos_np[5] = page * max_pages + 2
    positions = torch.from_numpy(pos_np).cuda()
    page_table = torch.from_numpy(table_np).cuda()
    pools = [torch.from_numpy(rng.standard_normal((slots, kv_heads, page, head_dim)).astype(np.float32)).half().cuda() for _ in range(4)]
    k_ref, v_ref, k_fused, v_fused = pools[0], pools[1], pools[0].clone(), pools[1].clone()
    ws = torch.zeros(ops.qgemv_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")
    xd = x.cuda()
    # separate kernels
    qkv_ref = quantized_matmul(xd, weight, workspace=ws)
    ops.rope_inplace(qkv_ref[:, : q_dim + k_dim], positions, num_heads=heads + kv_heads, head_dim=head_dim, theta=theta)
    ops.kv_append(qkv_ref[:, q_dim:q_dim + k_dim], qkv_ref[:, q_dim + k_dim:], k_ref, v_ref, page_table, positions)
    # fused kernel
    rope = ops.rope_table(page * max_pages + 3, head_dim, theta, xd.device)
    qkv = torch.empty_like(qkv_ref)
    ops.qkv_rope_append(xd, weight.packed_values, weight.scales, weight.zero_points, qkv, n=n, k=k, q_dim=q_dim, k_dim=k_dim,
                        head_dim=head_dim, theta=theta, table=rope, positions=positions, page_table=page_table,
                        k_cache=k_fused, v_cache=v_fused, workspace=ws, tiled=weight.tiled)
    torch.cuda.synchronize()
    assert torch.equal(qkv, qkv_ref)
    assert torch.equal(k_fused, k_ref) and torch.equal(v_fused, v_ref)
    # the append really happened for a row with a page, and not for the row without one
    b = 0
    slot, off = int(table_np[b, pos_np[b] // page]), int(pos_np[b] % page)
    assert torch.equal(k_fused[slot, :, off].reshape(-1), qkv[b, q_dim:q_dim + k_dim])
    assert torch.equal(v_fused[slot, :, off].reshape(-1), qkv[b, q_dim + k_dim:])
    # pre-quantized activations give the same result without reading x
    ops.quantize_activations(xd, ws)
    qkv2 = torch.empty_like(qkv)
    ops.qkv_rope_append(None, weight.packed_values, weight.scales, weight.zero_points, qkv2, n=n, k=k, q_dim=q_dim, k_dim=k_dim,
                        head_dim=head_dim, theta=theta, table=rope, positions=positions, page_table=page_table,
                        k_cache=k_fused, v_cache=v_fused, workspace=ws, tiled=weight.tiled, prequantized=True)
    assert torch.equal(qkv2, qkv_ref)
    _device_status_ok()
    # a position outside the table is reported through the device status word, not computed silently
    ops.qkv_rope_append(None, weight.packed_values, weight.scales, weight.zero_points, qkv2, n=n, k=k, q_dim=q_dim, k_dim=k_dim,
                        head_dim=head_dim, theta=theta, table=rope[:8].contiguous(), positions=positions, page_table=page_table,
                        k_cache=k_fused, v_cache=v_fused, workspace=ws, tiled=weight.tiled, prequantized=True)
    torch.cuda.synchronize()
    from cacheir_b200 import _lib
    assert _lib.load().cacheir_b200_device_status(1) != 0
    assert _lib.load().cacheir_b200_device_status(1) == 0        # cleared by the read above
    # the cos/sin table holds what rope_inplace evaluates
    want = oracle.rope_one(np.ones((1, 1, head_dim), dtype=np.float32), head_dim, theta, np.array([37]))
    got = rope[37].cpu().numpy()
    np.testing.assert_allclose(got[:, 0] - got[:, 1], want.reshape(-1)[0::2], rtol=0, atol=1e-5)
    _device_status_ok()


# ---- batches taller than one tensor-core launch run as chunks (64 rows integer kernel, 128 rows fp16 kernel) --------------------------
@pytest.mark.parametrize("bits,group,tiled", [(8, 0, True), (8, 0, False), (4, 128, True), (4, 0, False)])
def test_qgemv_tall_batch_runs_in_chunks(bits, group, tiled):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul, to_tiled
    rng = np.random.default_rng(7 + bits + group)
    m, n, k = 150, 384, 512
    x, packed = _qgemv_case(rng, m, n, k, bits, torch.float16, group=group, reference_pack=not group)
    dev = _device_pack(packed)
    if group:
        dev.scales = torch.from_numpy(packed.scales).cuda()
    weight = to_tiled(dev) if tiled else dev
    ws = torch.zeros(ops.qgemv_workspace_bytes(m, k), dtype=torch.uint8, device="cuda") if bits == 8 else None
    base = oracle.quantized_matmul(x.float().numpy(), packed)
    y = quantized_matmul(x.cuda(), weight, workspace=ws)
    assert y.shape == (m, n)
    assert _rel(y, base) <= TOL[torch.float16]
    # each chunk equals the same rows computed on their own
    y_tail = quantized_matmul(x[128:].cuda().contiguous(), weight, workspace=ws)
    assert torch.equal(y[128:], y_tail)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).half()
    y = quantized_matmul(x.cuda(), weight, epilogue=ops.EPI_RESIDUAL, residual=res.cuda(), workspace=ws)
    assert _rel(y, base + res.float().numpy()) <= TOL[torch.float16]
    torch.cuda.synchronize()
    _device_status_ok()


# ---- 65..128 batch rows: one launch of the fp16 tensor-core kernel with the operand roles exchanged ----
@pytest.mark.parametrize("m", [65, 100, 128])
@pytest.mark.parametrize("bits,group,tiled", [(4, 128, True), (4, 128, False), (8, 128, True), (4, 0, False), (8, 0, True)])
def test_qgemv_wide_batch_single_launch(m, bits, group, tiled):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul, to_tiled
    rng = np.random.default_rng(1000 * bits + group + m)
    # (n, k): many tiles without split-K; few tiles so that four CTAs share the k range; rows that do not fill
    # the last tile; one tile split over eight CTAs
    for n, k in ((1024, 512), (256, 2048), (200, 1024), (128, 4096)):
        x, packed = _qgemv_case(rng, m, n, k, bits, torch.float16, group=group, reference_pack=not group)
        dev = _device_pack(packed)
        if group:
            dev.scales = torch.from_numpy(packed.scales).cuda()
        weight = to_tiled(dev) if tiled else dev
        base = oracle.quantized_matmul(x.float().numpy(), packed)
        y = quantized_matmul(x.cuda(), weight)            # no workspace: the fp16 kernel, not the integer one
        assert y.shape == (m, n)
        assert _rel(y, base) <= TOL[torch.float16], (n, k)
        # a row's result does not depend on the batch it sits in: the 16-row kernel gives the same sums up to fp32 order
        y_small = quantized_matmul(x[:16].cuda().contiguous(), weight)
        assert _rel(y[:16], y_small.float().cpu().numpy()) <= 2e-3
        res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).half()
        y = quantized_matmul(x.cuda(), weight, epilogue=ops.EPI_RESIDUAL, residual=res.cuda())
        assert _rel(y, base + res.float().numpy()) <= TOL[torch.float16], (n, k)
        if n % 256 == 0:
            y = quantized_matmul(x.cuda(), weight, epilogue=ops.EPI_SWIGLU)
            gate, up = base[:, :n // 2], base[:, n // 2:]
            assert _rel(y, gate / (1.0 + np.exp(-gate)) * up) <= 2 * TOL[torch.float16], (n, k)
    torch.cuda.synchronize()
    _device_status_ok()


# ---- llama.cpp block formats streamed as group-32 packs (no fp32 dequantisation at load) ---------
@pytest.mark.parametrize("fmt", ["q4_0", "q8_0"])
def test_gguf_block_weights_run_in_place(fmt):
    from cacheir_b200.gguf_blocks import q4_0_to_packed, q8_0_to_packed
    from cacheir_b200.quantization import quantized_matmul
    rng = np.random.default_rng(11)
    m, n, k = 5, 96, 256
    blocks = n * k // 32
    if fmt == "q4_0":
        raw = b"".join(np.float16(rng.uniform(0.005, 0.02)).tobytes() + rng.integers(0, 256, 16, dtype=np.uint8).tobytes()
                       for _ in range(blocks))
        dense = oracle.decode_q4_0_blocks(raw, n * k).reshape(n, k)
        packed = q4_0_to_packed(raw, n, k, "cuda")
    else:
        raw = b"".join(np.float16(rng.uniform(0.0005, 0.002)).tobytes() + rng.integers(-128, 128, 32).astype(np.int8).tobytes()
                       for _ in range(blocks))
        dense = oracle.decode_q8_0_blocks(raw, n * k).reshape(n, k)
        packed = q8_0_to_packed(raw, n, k, "cuda")
    for dtype in (torch.float32, torch.float16):
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype)
        want = x.float().numpy() @ dense.T                       # the reference: dequantise the blocks, then matmul
        assert _rel(quantized_matmul(x.cuda(), packed), want) <= TOL[dtype]
