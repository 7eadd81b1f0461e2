"""Parity at the shapes the benchmark times, against the CPU oracle.

The other GPU tests cover every kernel on small shapes. These run the kernel
instances that `bench.py` measures, through the same entry points and flags the
runtime uses, at their real sizes:

  * the paged decode attention microbench: batch 64, 32 query / 8 KV heads,
    head_dim 128, contexts `rng(0).integers(512, 8193, 64)`, one permuted pool,
    two context splits + the combine kernel;
  * the dequant-GEMV microbench: N 14336, K 4096, M in {1, 8, 32, 64}, for the
    group-128 symmetric int4 format, int8 per channel with fp16 scales, and the
    reference packer's own int8 / int4 output for N(0, 0.02) weights;
  * the projections of one decoder layer of the 8B-shaped model at batch 32 --
    fused QKV + RoPE + cache append (N 6144), o (4096 x 4096, residual), paired
    gate|up + SwiGLU (N 28672), down (K 14336, residual) and the lm_head
    (N 128256) -- in the tile order, after the fused RMSNorm / activation
    pre-pass, and the attention call of that step (batch 32, context 2100).

Bars: rel-L2 <= 2e-3 against the oracle (fp16), the device status word stays 0,
and the launcher picks the split-K factor that the committed profiles describe.
"""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _ops():
    from cacheir_b200 import ops
    return ops


def _rel(got: torch.Tensor, want: np.ndarray) -> float:
    return oracle.rel_l2(got.detach().float().cpu().numpy(), want)


def _status_ok():
    from cacheir_b200 import _lib
    torch.cuda.synchronize()
    status = _lib.load().cacheir_b200_device_status(1)
    assert status == 0, f"a bounded device wait gave up: status {status:#x}"


def _oracle_qmatmul(x: np.ndarray, packed, rows_per_chunk: int = 16384) -> np.ndarray:
    """oracle.quantized_matmul evaluated over slices of the weight's rows, so that a 128256-row
    weight never needs its 2 GB dense fp32 form at once. Same arithmetic per output column."""
    n = int(packed.shape[0])
    outs = []
    for r0 in range(0, n, rows_per_chunk):
        r1 = min(n, r0 + rows_per_chunk)
        part = oracle.PackedQuantizedTensor(packed.packed_values[r0:r1], packed.scales[r0:r1],
                                            None if packed.zero_points is None else packed.zero_points[r0:r1],
                                            packed.bits, (r1 - r0, int(packed.shape[1])),
                                            group_size=getattr(packed, "group_size", None))
        outs.append(oracle.quantized_matmul(x, part))
    return np.concatenate(outs, axis=-1)


def _device_pack_to_oracle(weight: torch.Tensor, bits: int):
    """Pack fp32 weights on the device (bit-exact with the reference packer, see test_kernels_gpu) and
    hand the same codes to the oracle."""
    from cacheir_b200.quantization import pack_weight_device
    dev = pack_weight_device(weight, "int8" if bits == 8 else "int4")
    host = oracle.PackedQuantizedTensor(dev.packed_values.cpu().numpy(), dev.scales.cpu().numpy(),
                                        dev.zero_points_i32.cpu().numpy(), bits, tuple(dev.shape))
    return dev, host


# ---- attention microbench (batch 64, contexts U[512, 8192], permuted shared pool) -------------------
def test_attention_microbench_shape_two_splits():
    ops = _ops()
    batch, heads, kv_heads, hd, page = 64, 32, 8, 128, 16
    lens = np.random.default_rng(0).integers(512, 8193, batch).astype(np.int32)
    pages = (lens + page - 1) // page
    total = int(pages.sum())
    assert int(lens.sum()) == 283360 and total == 17742          # the figures quoted for this workload
    table = np.zeros((batch, int(pages.max())), dtype=np.int32)
    perm = np.random.default_rng(1).permutation(total).astype(np.int32)
    cur = 0
    for b in range(batch):
        table[b, : pages[b]] = perm[cur:cur + pages[b]]
        cur += int(pages[b])
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    k_pool = torch.randn((total, kv_heads, page, hd), device="cuda", dtype=torch.float16, generator=gen)
    v_pool = torch.randn((total, kv_heads, page, hd), device="cuda", dtype=torch.float16, generator=gen)
    q = torch.randn((batch, heads, hd), device="cuda", dtype=torch.float16, generator=gen)
    d_table, d_lens = torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda()
    auto = ops.attention_auto_splits(batch, heads, kv_heads, table.shape[1], page, hd)
    assert auto == 2                                              # what `bench.py --micro attention` runs and the profile describes
    out = ops.paged_attention_decode_batch(q, k_pool, v_pool, d_table, d_lens, num_splits=0)
    again = ops.paged_attention_decode_batch(q, k_pool, v_pool, d_table, d_lens, num_splits=2)
    one = ops.paged_attention_decode_batch(q, k_pool, v_pool, d_table, d_lens, num_splits=1)
    _status_ok()
    want = oracle.paged_attention_decode(q.cpu().numpy(), k_pool.cpu().numpy(), v_pool.cpu().numpy(), table, lens)
    assert torch.equal(out, again)                                # deterministic combine
    assert _rel(out, want) <= TOL
    assert _rel(one, want) <= TOL


def test_attention_decode_step_shape_one_split():
    # the call of the 8B-shaped step: batch 32, every sequence at 2100 tokens, one split
    ops = _ops()
    batch, heads, kv_heads, hd, page, ctx = 32, 32, 8, 128, 16, 2100
    pages = (ctx + page - 1) // page
    width = 140                                                   # page-table width of the plan (2048 + headroom)
    total = batch * pages
    table = np.zeros((batch, width), dtype=np.int32)
    table[:, :pages] = np.random.default_rng(2).permutation(total).astype(np.int32).reshape(batch, pages)
    lens = np.full(batch, ctx, dtype=np.int32)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    k_pool = torch.randn((total + 8, kv_heads, page, hd), device="cuda", dtype=torch.float16, generator=gen)
    v_pool = torch.randn((total + 8, kv_heads, page, hd), device="cuda", dtype=torch.float16, generator=gen)
    q = torch.randn((batch, heads, hd), device="cuda", dtype=torch.float16, generator=gen)
    assert ops.attention_auto_splits(batch, heads, kv_heads, width, page, hd) == 1
    out = ops.paged_attention_decode_batch(q, k_pool, v_pool, torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda())
    _status_ok()
    want = oracle.paged_attention_decode(q.cpu().numpy(), k_pool.cpu().numpy(), v_pool.cpu().numpy(), table, lens)
    assert _rel(out, want) <= TOL


# ---- dequant-GEMV microbench: N 14336 x K 4096 -----------------------------------------------------
N3, K3 = 14336, 4096


@pytest.fixture(scope="module")
def gemv_weights():
    """The four weight formats of the GEMV microbench, built once: oracle-side pack + device upload."""
    from cacheir_b200.quantization import upload_reference_pack
    rng = np.random.default_rng(33)
    out = {}
    codes = rng.integers(0, 16, (N3, K3)).astype(np.uint8)
    scales = rng.uniform(0.005, 0.02, (N3, K3 // 128)).astype(np.float16)
    out["int4_g128"] = oracle.symmetric_group_pack_from_codes(codes, scales, 4, 128)
    codes8 = rng.integers(0, 256, (N3, K3)).astype(np.uint8)
    out["int8_channel_f16"] = oracle.PackedQuantizedTensor(codes8, rng.uniform(0.005, 0.02, N3).astype(np.float16),
                                                           np.full(N3, 128, dtype=np.int32), 8, (N3, K3))
    w = (rng.standard_normal((N3, K3)) * 0.02).astype(np.float32)
    out["int8_reference_pack"] = oracle.asymmetric_pack(w, 8)
    out["int4_reference_pack"] = oracle.asymmetric_pack(w, 4)
    dev = {}
    for name, packed in out.items():
        d = upload_reference_pack(packed, "cuda")
        if name == "int8_channel_f16":
            d.scales = torch.from_numpy(packed.scales).cuda()     # keep the fp16 per-channel scales as fp16
        dev[name] = d
    dense = {name: oracle.dequantize_packed_weight(p).astype(np.float32) for name, p in out.items()}
    return out, dev, dense


@pytest.mark.parametrize("m", [1, 8, 32, 64])
@pytest.mark.parametrize("fmt", ["int4_g128", "int8_channel_f16", "int8_reference_pack", "int4_reference_pack"])
def test_gemv_microbench_shapes(gemv_weights, fmt, m):
    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul, to_tiled
    host, dev, dense = gemv_weights
    rng = np.random.default_rng(1000 + m)
    x = torch.from_numpy(rng.standard_normal((m, K3)).astype(np.float32)).half()
    want = oracle.matmul(x.float().numpy(), dense[fmt])           # the oracle's dequantize-then-matmul, dense form cached
    xd = x.cuda()
    # reference row order, no scratch (what `bench.py --micro qgemv` runs by default)
    assert _rel(quantized_matmul(xd, dev[fmt]), want) <= TOL
    # tile order + scratch: the layout and path of the runtime
    tiled = to_tiled(dev[fmt])
    ws = torch.zeros(ops.qgemv_workspace_bytes(m, K3), dtype=torch.uint8, device="cuda")
    assert _rel(quantized_matmul(xd, tiled, workspace=ws), want) <= TOL
    _status_ok()


# ---- one decoder layer of the 8B-shaped int8 model at batch 32, as the runtime launches it ---------------
H, KVD, FFN, VOCAB, B4 = 4096, 1024, 14336, 128256, 32


def _randn(shape, seed, scale=1.0):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    return torch.randn(shape, device="cuda", dtype=torch.float32, generator=gen) * scale


def test_layer_projection_qkv_rope_append():
    from cacheir_b200 import _lib, ops
    from cacheir_b200.quantization import to_tiled
    n, k, hd, heads, kv_heads, page, theta = H + 2 * KVD, H, 128, 32, 8, 16, 500000.0
    dev, host = _device_pack_to_oracle(_randn((n, k), 11, 0.02), 8)
    weight = to_tiled(dev)
    x = _randn((B4, k), 12).half()
    norm_w = (1.0 + 0.1 * _randn((k,), 13)).half()
    max_pages, ctx = 140, 2100
    rng = np.random.default_rng(14)
    pos_np = rng.integers(ctx - 40, ctx, B4).astype(np.int32)
    table_np = rng.permutation(B4 * max_pages).astype(np.int32).reshape(B4, max_pages)
    positions, page_table = torch.from_numpy(pos_np).cuda(), torch.from_numpy(table_np).cuda()
    slots = B4 * max_pages
    k_pool = torch.zeros((slots, kv_heads, page, hd), device="cuda", dtype=torch.float16)
    v_pool = torch.zeros_like(k_pool)
    ws = torch.zeros(ops.qgemv_workspace_bytes(B4, k), dtype=torch.uint8, device="cuda")
    normed = torch.empty_like(x)
    ops.rms_norm_quantize(x, norm_w, 1e-5, ws, out=normed)
    rope = ops.rope_table(ctx + 8, hd, theta, x.device)
    qkv = torch.empty((B4, n), device="cuda", dtype=torch.float16)
    ops.qkv_rope_append(None, weight.packed_values, weight.scales, weight.zero_points, qkv, n=n, k=k, q_dim=H, k_dim=KVD,
                        head_dim=hd, theta=theta, table=rope, positions=positions, page_table=page_table, k_cache=k_pool,
                        v_cache=v_pool, workspace=ws, tiled=True, prequantized=True)
    _status_ok()
    plan = _lib.load().cacheir_b200_qgemv_plan(B4, n, k, 8, 0, 3, 1 | 2, 1)
    assert plan == (1 << 8) | 4                                    # integer kernel, split-K 4: the profiled instance
    # oracle: RMSNorm -> dequantize-then-matmul -> interleaved RoPE on q and k
    xn = oracle.rms_norm(x.float().cpu().numpy(), norm_w.float().cpu().numpy(), 1e-5)
    assert _rel(normed, xn) <= 1e-3
    base = _oracle_qmatmul(normed.float().cpu().numpy(), host)     # from the fp16 activations the GEMM consumed
    q_ref = oracle.rope_one(base[:, None, :H], hd, theta, pos_np)[:, 0]
    k_ref = oracle.rope_one(base[:, None, H:H + KVD], hd, theta, pos_np)[:, 0]
    v_ref = base[:, H + KVD:]
    assert _rel(qkv[:, :H], q_ref) <= TOL
    assert _rel(qkv[:, H:H + KVD], k_ref) <= TOL
    assert _rel(qkv[:, H + KVD:], v_ref) <= TOL
    # the appended rows are the k / v values just produced, at (page_table[b, pos/16], pos%16): bit-exact copies
    for b in range(B4):
        slot, off = int(table_np[b, pos_np[b] // page]), int(pos_np[b] % page)
        assert torch.equal(k_pool[slot, :, off].reshape(-1), qkv[b, H:H + KVD])
        assert torch.equal(v_pool[slot, :, off].reshape(-1), qkv[b, H + KVD:])
    assert int((k_pool != 0).any(dim=3).sum().item()) <= B4 * kv_heads      # nothing else was written
    # the one-call form (RMSNorm + pre-pass kernel, then the fused QKV kernel)
    qkv1 = torch.empty_like(qkv)
    k1, v1 = torch.zeros_like(k_pool), torch.zeros_like(v_pool)
    ops.qkv_rope_append(x, weight.packed_values, weight.scales, weight.zero_points, qkv1, n=n, k=k, q_dim=H, k_dim=KVD,
                        head_dim=hd, theta=theta, table=rope, positions=positions, page_table=page_table, k_cache=k1,
                        v_cache=v1, workspace=ws, tiled=True, norm_weight=norm_w, norm_eps=1e-5)
    _status_ok()
    assert torch.equal(qkv1, qkv)
    base1 = _oracle_qmatmul(xn, host)
    assert _rel(qkv1[:, :H], oracle.rope_one(base1[:, None, :H], hd, theta, pos_np)[:, 0]) <= TOL
    assert _rel(qkv1[:, H:H + KVD], oracle.rope_one(base1[:, None, H:H + KVD], hd, theta, pos_np)[:, 0]) <= TOL
    assert _rel(qkv1[:, H + KVD:], base1[:, H + KVD:]) <= TOL
    for b in range(B4):
        slot, off = int(table_np[b, pos_np[b] // page]), int(pos_np[b] % page)
        assert torch.equal(k1[slot, :, off].reshape(-1), qkv1[b, H:H + KVD])


@pytest.mark.parametrize("name,n,k,seed", [("o", H, H, 21), ("down", H, FFN, 22)])
def test_layer_projection_residual_split_k8(name, n, k, seed):
    from cacheir_b200 import _lib, ops
    from cacheir_b200.quantization import to_tiled
    dev, host = _device_pack_to_oracle(_randn((n, k), seed, 0.02), 8)
    weight = to_tiled(dev)
    x = _randn((B4, k), seed + 100).half()
    res = _randn((B4, n), seed + 200).half()
    ws = torch.zeros(ops.qgemv_workspace_bytes(B4, k), dtype=torch.uint8, device="cuda")
    ops.quantize_activations(x, ws)
    y = ops.qgemv(x, weight.packed_values, weight.scales, weight.zero_points, bits=8, n=n, k=k, epilogue=ops.EPI_RESIDUAL,
                  residual=res, workspace=ws, tiled=True, prequantized=True)
    _status_ok()
    assert _lib.load().cacheir_b200_qgemv_plan(B4, n, k, 8, 0, ops.EPI_RESIDUAL, 1 | 2, 1) == (1 << 8) | 8
    want = _oracle_qmatmul(x.float().cpu().numpy(), host) + res.float().cpu().numpy()
    assert _rel(y, want) <= TOL
    # the GEMM's own pre-pass gives the same integers
    assert _lib.load().cacheir_b200_qgemv_plan(B4, n, k, 8, 0, ops.EPI_RESIDUAL, 1, 1) == (1 << 8) | 8
    y1 = ops.qgemv(x, weight.packed_values, weight.scales, weight.zero_points, bits=8, n=n, k=k, epilogue=ops.EPI_RESIDUAL,
                   residual=res, workspace=ws, tiled=True)
    assert torch.equal(y1, y)
    # without the residual the projection itself meets the bar too (the residual would otherwise dominate the norm)
    y0 = ops.qgemv(x, weight.packed_values, weight.scales, weight.zero_points, bits=8, n=n, k=k, workspace=ws, tiled=True,
                   prequantized=True)
    assert _rel(y0, want - res.float().cpu().numpy()) <= TOL
    _status_ok()


def test_layer_projection_gate_up_swiglu_paired():
    from cacheir_b200 import _lib, ops
    from cacheir_b200.quantization import to_tiled
    n, k = 2 * FFN, H
    dev, host = _device_pack_to_oracle(_randn((n, k), 31, 0.02), 8)
    weight = to_tiled(dev, paired=True)
    x = _randn((B4, k), 32).half()
    norm_w = (1.0 + 0.1 * _randn((k,), 33)).half()
    ws = torch.zeros(ops.qgemv_workspace_bytes(B4, k), dtype=torch.uint8, device="cuda")
    normed = torch.empty_like(x)
    ops.rms_norm_quantize(x, norm_w, 1e-5, ws, out=normed)
    y = ops.qgemv(x, weight.packed_values, weight.scales, weight.zero_points, bits=8, n=n, k=k, epilogue=ops.EPI_SWIGLU,
                  workspace=ws, tiled=True, prequantized=True, paired=True)
    _status_ok()
    assert _lib.load().cacheir_b200_qgemv_plan(B4, n, k, 8, 0, ops.EPI_SWIGLU, 1 | 2 | 4, 1) == (1 << 8) | 1
    base = _oracle_qmatmul(normed.float().cpu().numpy(), host)
    want = oracle.silu_mul(base[:, :FFN], base[:, FFN:])
    assert y.shape == (B4, FFN)
    assert _rel(y, want) <= 2 * TOL                               # a product of two projections: each factor is within the bar
    # the one-call form (RMSNorm + pre-pass kernel, then the GEMM)
    y1 = ops.qgemv(x, weight.packed_values, weight.scales, weight.zero_points, bits=8, n=n, k=k, epilogue=ops.EPI_SWIGLU,
                   workspace=ws, tiled=True, paired=True, norm_weight=norm_w, norm_eps=1e-5)
    _status_ok()
    want1 = _oracle_qmatmul(oracle.rms_norm(x.float().cpu().numpy(), norm_w.float().cpu().numpy(), 1e-5), host)
    assert _rel(y1, oracle.silu_mul(want1[:, :FFN], want1[:, FFN:])) <= 2 * TOL


def test_lm_head_projection():
    from cacheir_b200 import ops
    from cacheir_b200.quantization import to_tiled
    n, k = VOCAB, H
    dev, host = _device_pack_to_oracle(_randn((n, k), 41, 0.02), 8)
    weight = to_tiled(dev)
    x = _randn((B4, k), 42).half()
    norm_w = torch.ones((k,), device="cuda", dtype=torch.float16)
    ws = torch.zeros(ops.qgemv_workspace_bytes(B4, k), dtype=torch.uint8, device="cuda")
    normed = torch.empty_like(x)
    ops.rms_norm_quantize(x, norm_w, 1e-5, ws, out=normed)
    logits = ops.qgemv(x, weight.packed_values, weight.scales, weight.zero_points, bits=8, n=n, k=k, workspace=ws, tiled=True,
                       prequantized=True)
    _status_ok()
    want = _oracle_qmatmul(normed.float().cpu().numpy(), host)
    assert _rel(logits, want) <= TOL
    fused = ops.qgemv(x, weight.packed_values, weight.scales, weight.zero_points, bits=8, n=n, k=k, workspace=ws, tiled=True,
                      norm_weight=norm_w, norm_eps=1e-5)                 # the one-call form
    _status_ok()
    assert _rel(fused, _oracle_qmatmul(oracle.rms_norm(x.float().cpu().numpy(), norm_w.float().cpu().numpy(), 1e-5), host)) <= TOL
    # greedy sampling: the device argmax picks the oracle's token wherever the oracle's top-2 margin exceeds the tolerance
    ids = ops.argmax_rows(logits).cpu().numpy()
    top2 = np.sort(want, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 4 * TOL * np.abs(top2[:, 1])
    assert np.array_equal(ids[clear], want.argmax(axis=1)[clear]) and clear.sum() >= B4 // 2
