"""8-bit KV pages: unsigned bytes with one fp16 scale per cached row.

The reference keeps KV pages in the activation type and only models what a smaller cache would cost
(cacheir/runtime/kv_cache.py:138-259), so the format is this package's extension; the oracle states it
(`oracle.quantize_kv_rows`, `oracle.dequantize_kv_pool`). Two bars:
  * against the oracle's attention over the SAME bytes (dequantised in fp32): the usual rel-L2 <= 2e-3,
    and the appended bytes and scales bit-exact;
  * against attention over the unquantised fp16 values: what the 8-bit cache itself costs, rel-L2 <= 2e-2
    on N(0,1) data (measured about 6e-3).
"""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _status_ok():
    from cacheir_b200 import _lib
    torch.cuda.synchronize()
    assert _lib.load().cacheir_b200_device_status(1) == 0


def _pools(rng, slots, kv_heads, page, hd):
    k = rng.standard_normal((slots, kv_heads, page, hd)).astype(np.float32)
    v = rng.standard_normal((slots, kv_heads, page, hd)).astype(np.float32)
    k8, ks = oracle.quantize_kv_rows(k)
    v8, vs = oracle.quantize_kv_rows(v)
    scales = np.stack([ks, vs], axis=2)                      # [slots, kv_heads, 2, page]
    return k, v, k8, v8, scales


def _table(rng, lens, page, slots, width=None):
    pages = [(int(n) + page - 1) // page for n in lens]
    width = width or max(1, max(pages))
    table = np.zeros((len(lens), width), dtype=np.int32)
    perm = rng.permutation(slots).astype(np.int32)
    cur = 0
    for b, n in enumerate(pages):
        table[b, :n] = perm[cur:cur + n]
        cur += n
    return table


@pytest.mark.parametrize("dtype,heads,kv_heads,hd,page,lens,splits", [
    (torch.float16, 32, 8, 128, 16, [2100] * 4 + [1, 17, 333, 2048], 1),      # fast kernel, the decode step's shape per sequence
    (torch.float16, 8, 2, 128, 16, [700, 33, 4500, 450], 3),                  # fast kernel, context splits + combine
    (torch.float16, 16, 1, 128, 16, [129, 64], 1),                            # a GQA group of 16
    (torch.float16, 4, 2, 64, 16, [300, 17, 1], 2),                           # head_dim 64: general kernel
    (torch.float32, 4, 2, 64, 8, [50, 9], 1),                                 # fp32 queries, page 8
    (torch.bfloat16, 8, 4, 128, 16, [200, 31], 1),
])
def test_attention_over_8bit_pages(dtype, heads, kv_heads, hd, page, lens, splits):
    from cacheir_b200 import ops
    rng = np.random.default_rng(heads * 7 + hd + len(lens))
    pages = sum((n + page - 1) // page for n in lens)
    slots = pages + 3
    k, v, k8, v8, scales = _pools(rng, slots, kv_heads, page, hd)
    table = _table(rng, lens, page, slots)
    lens_np = np.asarray(lens, dtype=np.int32)
    q = torch.from_numpy(rng.standard_normal((len(lens), heads, hd)).astype(np.float32)).to(dtype)
    out = ops.paged_attention_decode_batch(q.cuda(), torch.from_numpy(k8).cuda(), torch.from_numpy(v8).cuda(),
                                           torch.from_numpy(table).cuda(), torch.from_numpy(lens_np).cuda(), num_splits=splits,
                                           kv_scales=torch.from_numpy(scales).cuda())
    _status_ok()
    qf = q.float().numpy()
    same_bytes = oracle.paged_attention_decode(qf, oracle.dequantize_kv_pool(k8, scales, 0), oracle.dequantize_kv_pool(v8, scales, 1),
                                               table, lens_np)
    tol = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 4e-3}[dtype]
    assert oracle.rel_l2(out.float().cpu().numpy(), same_bytes) <= tol
    unquantised = oracle.paged_attention_decode(qf, k, v, table, lens_np)
    assert oracle.rel_l2(out.float().cpu().numpy(), unquantised) <= 2e-2


def test_attention_8bit_microbench_shape():
    # the attention microbench (batch 64, contexts U[512, 8192], permuted pool, two splits) on 8-bit pages
    from cacheir_b200 import ops
    batch, heads, kv_heads, hd, page = 64, 32, 8, 128, 16
    lens = np.random.default_rng(0).integers(512, 8193, batch).astype(np.int32)
    pages = (lens + page - 1) // page
    total = int(pages.sum())
    table = np.zeros((batch, int(pages.max())), dtype=np.int32)
    perm = np.random.default_rng(1).permutation(total).astype(np.int32)
    cur = 0
    for b in range(batch):
        table[b, : pages[b]] = perm[cur:cur + pages[b]]
        cur += int(pages[b])
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    k8 = torch.randint(0, 256, (total, kv_heads, page, hd), device="cuda", dtype=torch.uint8, generator=gen)
    v8 = torch.randint(0, 256, (total, kv_heads, page, hd), device="cuda", dtype=torch.uint8, generator=gen)
    scales = (torch.rand((total, kv_heads, 2, page), device="cuda", generator=gen) * 0.02 + 0.01).half()
    q = torch.randn((batch, heads, hd), device="cuda", dtype=torch.float16, generator=gen)
    out = ops.paged_attention_decode_batch(q, k8, v8, torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda(), kv_scales=scales)
    again = ops.paged_attention_decode_batch(q, k8, v8, torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda(), kv_scales=scales)
    _status_ok()
    assert torch.equal(out, again)
    sc = scales.cpu().numpy()
    want = oracle.paged_attention_decode(q.cpu().numpy(), oracle.dequantize_kv_pool(k8.cpu().numpy(), sc, 0),
                                         oracle.dequantize_kv_pool(v8.cpu().numpy(), sc, 1), table, lens)
    assert oracle.rel_l2(out.float().cpu().numpy(), want) <= 2e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_kv_append_q8_bytes_and_scales_are_bit_exact(dtype):
    from cacheir_b200 import ops
    rng = np.random.default_rng(9)
    batch, kv_heads, hd, page, max_pages = 7, 2, 128, 16, 4
    slots = batch * max_pages + 2
    k = torch.from_numpy(rng.standard_normal((batch, kv_heads * hd)).astype(np.float32) * 3.0).to(dtype)
    v = torch.from_numpy(rng.standard_normal((batch, kv_heads * hd)).astype(np.float32) * 0.01).to(dtype)
    k[2] = 0                                                   # an all-zero row keeps scale 1
    pos = rng.integers(0, page * max_pages, batch).astype(np.int32)
    pos[5] = page * max_pages + 3                              # no page reserved: dropped
    table = rng.permutation(slots)[: batch * max_pages].astype(np.int32).reshape(batch, max_pages)
    k8 = torch.zeros((slots, kv_heads, page, hd), dtype=torch.uint8, device="cuda")
    v8 = torch.zeros_like(k8)
    scales = torch.zeros((slots, kv_heads, 2, page), dtype=torch.float16, device="cuda")
    ops.kv_append_q8(k.cuda(), v.cuda(), k8, v8, scales, torch.from_numpy(table).cuda(), torch.from_numpy(pos).cuda())
    torch.cuda.synchronize()
    want_k, want_ks = oracle.quantize_kv_rows(k.float().numpy().reshape(batch, kv_heads, hd))
    want_v, want_vs = oracle.quantize_kv_rows(v.float().numpy().reshape(batch, kv_heads, hd))
    written = 0
    for b in range(batch):
        if pos[b] >= page * max_pages:
            continue
        slot, off = int(table[b, pos[b] // page]), int(pos[b] % page)
        assert np.array_equal(k8[slot, :, off].cpu().numpy(), want_k[b])
        assert np.array_equal(v8[slot, :, off].cpu().numpy(), want_v[b])
        assert np.array_equal(scales[slot, :, 0, off].cpu().numpy(), want_ks[b])
        assert np.array_equal(scales[slot, :, 1, off].cpu().numpy(), want_vs[b])
        written += 1
    assert written == batch - 1
    assert int((scales != 0).sum().item()) == 2 * kv_heads * written            # nothing else was touched
    assert float(scales[int(table[2, pos[2] // page]), 0, 0, int(pos[2] % page)]) == 1.0


def test_runtime_with_8bit_kv_pages_tracks_the_fp16_cache(golden_dir, tmp_path):
    import json

    from cacheir_b200 import B200DecodeRuntime, CompileArtifact
    from cacheir_b200.tiny import create_tiny_model

    meta = json.loads((golden_dir / "tiny_c1_meta.json").read_text())
    arts = json.loads((golden_dir / "tiny_artifacts.json").read_text())
    model = create_tiny_model(tmp_path / "tiny", seed=meta["seed"], **meta["shape"])
    art = CompileArtifact.from_dict({**arts["int8"], "model_path": str(model)})
    g = np.load(golden_dir / "tiny_c1.npz")
    prompt = g["prompt"].tolist()
    runs = {}
    for kv in ("same", "int8"):
        rt = B200DecodeRuntime(art, dtype="float16", kv_dtype=kv, max_seq_len=128)
        s = rt.fork()
        logits, _ = s.prefill_tokens(prompt)
        trace = [logits[0, -1].float().cpu().numpy()]
        for tok in g["int8_tokens"].tolist()[:12]:                       # teacher-forced with the reference's tokens
            trace.append(rt.run_decode_batch([s], [tok])[0, -1].float().cpu().numpy())
        runs[kv] = np.stack(trace)
        if kv == "int8":
            pool = rt.kv_allocator.pool_for_layer(0)
            assert pool["keys"].dtype == torch.uint8 and pool["scales"].dtype == torch.float16
            assert rt.cache_stats()["kernel_counts"]["b200.kv_append_q8"] > 0
    assert oracle.rel_l2(runs["int8"], runs["same"]) <= 2e-2
    assert np.mean(runs["int8"].argmax(-1) == runs["same"].argmax(-1)) >= 0.9
    _status_ok()
