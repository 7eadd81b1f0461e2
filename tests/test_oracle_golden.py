"""Pin the CPU oracle against fixtures produced by the reference itself
(tests/golden/make_golden.py). No GPU needed."""
import hashlib
import json

import numpy as np
import pytest

from oracle import oracle


def test_pack_matches_reference_bit_exact(golden_dir):
    g = np.load(golden_dir / "pack.npz")
    for prefix in ("lin", "rnd", "even"):
        w = g[f"{prefix}_w"]
        for quant, tag in (("int4_awq", "q4"), ("int8", "q8")):
            packed = oracle.pack_quantized_weight(w, quant)
            assert packed.packed_values.dtype == np.uint8
            np.testing.assert_array_equal(packed.packed_values, g[f"{prefix}_{tag}_packed"])
            np.testing.assert_array_equal(packed.zero_points, g[f"{prefix}_{tag}_zero_points"])
            np.testing.assert_array_equal(packed.scales, g[f"{prefix}_{tag}_scales"])
            np.testing.assert_array_equal(oracle.dequantize_packed_weight(packed), g[f"{prefix}_{tag}_dequant"])


def test_pack_shapes_of_reference_test(golden_dir):
    # shapes asserted by the reference's tests/test_project_surfaces.py:73-82
    w = np.linspace(-1.5, 2.0, num=30, dtype=np.float32).reshape(3, 10)
    q4 = oracle.pack_quantized_weight(w, "int4_awq")
    q8 = oracle.pack_quantized_weight(w, "int8")
    assert q4.packed_values.shape == (3, 5) and q8.packed_values.shape == (3, 10)
    assert q4.zero_points.shape == (3,)
    np.testing.assert_allclose(oracle.dequantize_packed_weight(q8), w, rtol=0.02, atol=0.02)


def test_int4_nibble_order_roundtrip():
    rng = np.random.default_rng(3)
    codes = rng.integers(0, 16, (5, 11)).astype(np.uint8)
    packed = oracle.pack_int4(codes)
    assert packed.shape == (5, 6)
    assert packed[0, 0] == (codes[0, 0] | (codes[0, 1] << 4))
    assert (packed[:, -1] >> 4 == 0).all()  # odd K: padding nibble is zero
    np.testing.assert_array_equal(oracle.unpack_int4(packed, 11).astype(np.uint8), codes)


def test_page_metadata_matches_reference(golden_dir):
    cases = json.loads((golden_dir / "pages.json").read_text())
    for case in cases:
        pages = {0: [], 1: []}
        lengths = {0: 0, 1: 0}
        next_id = 0
        for step in case["history"]:
            layer, n = step["layer"], step["append"]
            next_id = oracle.extend_pages(pages[layer], next_id, case["page_size"], lengths[layer], n)
            lengths[layer] += n
            assert [p.to_dict() for p in pages[layer]] == step["pages"]
        assert sum(len(v) for v in pages.values()) == case["total_pages"]


def test_numerics_match_reference(golden_dir):
    g = np.load(golden_dir / "numerics.npz")
    for tag in "abc":
        heads, kv_heads, hd, t = (int(v) for v in g[f"attn_{tag}_dims"])
        keys = g[f"attn_{tag}_k"].reshape(1, t, kv_heads, hd)
        vals = g[f"attn_{tag}_v"].reshape(1, t, kv_heads, hd)
        out = oracle.attention_contiguous(g[f"attn_{tag}_q"], keys, vals, heads, kv_heads, hd)
        np.testing.assert_allclose(out, g[f"attn_{tag}_out"], rtol=1e-6, atol=1e-6)
        # the paged form over a shuffled pool must agree with the contiguous form
        page = 4
        n_pages = (t + page - 1) // page
        rng = np.random.default_rng(t)
        table = rng.permutation(n_pages + 3)[:n_pages].astype(np.int32)
        k_pool = rng.standard_normal((n_pages + 3, kv_heads, page, hd)).astype(np.float32)
        v_pool = rng.standard_normal((n_pages + 3, kv_heads, page, hd)).astype(np.float32)
        for pos in range(t):
            k_pool[table[pos // page], :, pos % page] = keys[0, pos]
            v_pool[table[pos // page], :, pos % page] = vals[0, pos]
        paged = oracle.paged_attention_decode(g[f"attn_{tag}_q"].reshape(1, heads, hd), k_pool, v_pool,
                                              table[None, :], np.asarray([t]))
        np.testing.assert_allclose(paged.reshape(1, 1, -1), g[f"attn_{tag}_out"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(oracle.rope_one(g["rope_x"], 16, 10000.0, [7]), g["rope_out_off7"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(oracle.rope_one(g["rope_x"], 16, 10000.0, [0]), g["rope_out_off0"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(oracle.rms_norm(g["rms_x"], g["rms_w"], 1e-5), g["rms_out"], rtol=1e-6, atol=1e-6)


def test_reference_paged_attention_test_shape():
    # shape and page table of the reference's tests/test_advanced_experiments.py:519-558,
    # including the padding entry that aliases slot 0; expected = its gather + softmax loop
    rng = np.random.default_rng(0)
    batch, heads, kv_heads, page, max_pages, hd = 2, 4, 2, 2, 3, 8
    q = rng.standard_normal((batch, heads, hd)).astype(np.float32)
    k_pool = rng.standard_normal((5, kv_heads, page, hd)).astype(np.float32)
    v_pool = rng.standard_normal((5, kv_heads, page, hd)).astype(np.float32)
    table = np.asarray([[0, 1, 2], [3, 4, 0]], dtype=np.int32)
    lens = np.asarray([5, 3], dtype=np.int32)
    got = oracle.paged_attention_decode(q, k_pool, v_pool, table, lens)
    for b in range(batch):
        for h in range(heads):
            kvh = h // (heads // kv_heads)
            ks = np.stack([k_pool[table[b, t // page], kvh, t % page] for t in range(lens[b])])
            vs = np.stack([v_pool[table[b, t // page], kvh, t % page] for t in range(lens[b])])
            s = (q[b, h][None, :] * ks).sum(-1) / np.sqrt(hd)
            p = np.exp(s - s.max())
            p /= p.sum()
            np.testing.assert_allclose(got[b, h], (p[:, None] * vs).sum(0), atol=1e-5)


def test_tiny_model_greedy_tokens_match_reference(golden_dir):
    from cacheir_b200.tiny import tiny_model_tensors

    meta = json.loads((golden_dir / "tiny_c1_meta.json").read_text())
    g = np.load(golden_dir / "tiny_c1.npz")
    artifacts = json.loads((golden_dir / "tiny_artifacts.json").read_text())
    tensors = tiny_model_tensors(seed=meta["seed"], **meta["shape"])
    for key, digest in meta["weight_sha256"].items():
        assert hashlib.sha256(np.ascontiguousarray(tensors[key]).tobytes()).hexdigest() == digest, key
    for tag in ("fp32", "int8", "int4"):
        art = artifacts[tag]
        rt = oracle.OracleRuntime(art["graphs"], tensors, art["quant"])
        tokens, logits = oracle.greedy_decode(rt, g["prompt"].tolist(), meta["steps"], meta["shape"]["vocab_size"])
        np.testing.assert_array_equal(np.asarray(tokens), g[f"{tag}_tokens"])
        np.testing.assert_allclose(logits[0], g[f"{tag}_prefill_logits_last"], rtol=1e-4, atol=1e-5)
        np.testing.assert_array_equal(
            np.asarray([[p.page_id, p.start, p.length] for p in rt.pages[0]]), g[f"{tag}_pages_layer0"])


def test_oracle_agrees_with_reference_native_kernels():
    # the reference's own native-vs-NumPy check (tests/test_advanced_experiments.py:440-452,
    # tests/test_runtime.py:34-41), run against its C++ kernels compiled from its sources
    import pytest
    from oracle import ref_native

    if not ref_native.available():
        pytest.skip("oracle/_ref not built (needs the reference checkout: make -C oracle)")
    assert ref_native.simd_backend() in {"avx512", "avx2", "scalar"}
    x = (np.arange(24, dtype=np.float32).reshape(1, 3, 8) / 10.0).astype(np.float32)
    w = np.ones(8, dtype=np.float32)
    np.testing.assert_allclose(ref_native.rms_norm(x, w, 1e-6), oracle.rms_norm(x, w, 1e-6), rtol=1e-5, atol=1e-6)
    weight = (np.arange(32, dtype=np.float32).reshape(4, 8) / 100.0).astype(np.float32)
    np.testing.assert_allclose(ref_native.matmul_out_in(x, weight), oracle.matmul(x, weight), rtol=1e-5, atol=1e-6)
    gate = np.linspace(-3.0, 3.0, num=24, dtype=np.float32).reshape(2, 3, 4)
    up = np.linspace(0.5, 2.0, num=24, dtype=np.float32).reshape(2, 3, 4)
    np.testing.assert_allclose(ref_native.silu_mul(gate, up), oracle.silu_mul(gate, up), rtol=1e-6, atol=1e-6)
    rng = np.random.default_rng(0)
    xb = rng.standard_normal((2, 5, 300)).astype(np.float32)
    wb = rng.standard_normal((77, 300)).astype(np.float32)
    np.testing.assert_allclose(ref_native.matmul_out_in(xb, wb), oracle.matmul(xb, wb), rtol=1e-4, atol=1e-4)


def test_gguf_block_formats_known_answers_and_native_repack():
    """Q4_0 / Q8_0 (cacheir/importers/gguf.py:273-310). Known-answer blocks of the shape the reference's
    reader test builds (tests/test_advanced_experiments.py:59-128): ascending / descending nibbles with
    d = 0.25, and the signed ramp -16..15 with d = 0.5. The native repack is a pure permutation of the
    codes: dequantising the repacked weight with the group-wise formula gives the block decode exactly."""
    import torch

    from cacheir_b200.gguf_blocks import q4_0_to_packed, q8_0_to_packed

    low = np.arange(16, dtype=np.uint8)
    high = (15 - np.arange(16, dtype=np.uint8)).astype(np.uint8)
    q4_block = np.float16(0.25).tobytes() + (low | (high << 4)).astype(np.uint8).tobytes()
    want4 = np.concatenate([(low.astype(np.float32) - 8) * 0.25, (high.astype(np.float32) - 8) * 0.25])
    np.testing.assert_array_equal(oracle.decode_q4_0_blocks(q4_block, 32), want4)
    q8_values = np.arange(-16, 16, dtype=np.int8)
    q8_block = np.float16(0.5).tobytes() + q8_values.tobytes()
    np.testing.assert_array_equal(oracle.decode_q8_0_blocks(q8_block, 32), q8_values.astype(np.float32) * 0.5)

    rng = np.random.default_rng(5)
    n, k = 6, 96
    raw4 = b"".join(np.float16(rng.uniform(0.01, 0.5)).tobytes() + rng.integers(0, 256, 16, dtype=np.uint8).tobytes()
                    for _ in range(n * k // 32))
    raw8 = b"".join(np.float16(rng.uniform(0.01, 0.5)).tobytes() + rng.integers(-128, 128, 32).astype(np.int8).tobytes()
                    for _ in range(n * k // 32))
    for raw, decode, repack, bits in ((raw4, oracle.decode_q4_0_blocks, q4_0_to_packed, 4),
                                      (raw8, oracle.decode_q8_0_blocks, q8_0_to_packed, 8)):
        packed = repack(raw, n, k)
        assert packed.bits == bits and packed.group_size == 32 and packed.scales.dtype == torch.float16
        ref = oracle.PackedQuantizedTensor(packed.packed_values.numpy(), packed.scales.numpy(), None, bits, (n, k), group_size=32)
        np.testing.assert_array_equal(oracle.dequantize_packed_weight(ref), decode(raw, n * k).reshape(n, k))
    with pytest.raises(ValueError):
        q4_0_to_packed(raw4[:-1], n, k)
