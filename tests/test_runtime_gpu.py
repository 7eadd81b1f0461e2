"""End-to-end parity of the B200 decode runtime on the reference's tiny model
(2 layers, hidden 256, 4 query / 2 KV heads, head_dim 64, FFN 688, vocab 1024,
fp32 weights from seed 0; prompt of 32 seeded ids, 32 greedy steps, page 16)."""
import json

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _tiny(golden_dir, tag, tmp_path, **kwargs):
    from cacheir_b200 import B200DecodeRuntime, CompileArtifact
    from cacheir_b200.tiny import create_tiny_model

    meta = json.loads((golden_dir / "tiny_c1_meta.json").read_text())
    arts = json.loads((golden_dir / "tiny_artifacts.json").read_text())
    model = create_tiny_model(tmp_path / "tiny", seed=meta["seed"], **meta["shape"])
    art = CompileArtifact.from_dict({**arts[tag], "model_path": str(model)})
    return B200DecodeRuntime(art, **kwargs), meta, np.load(golden_dir / "tiny_c1.npz")


def _greedy(rt, prompt, steps, vocab):
    logits = rt.run([list(prompt)], mode="prefill")
    tokens, first = [], logits[0, -1].float().cpu().numpy()
    for _ in range(steps):
        nxt = int(torch.argmax(logits[0, -1]).item()) % vocab
        tokens.append(nxt)
        logits = rt.run([[nxt]], mode="decode")
    return tokens, first, logits[0, -1].float().cpu().numpy()


@pytest.mark.parametrize("tag", ["fp32", "int8", "int4"])
def test_tiny_model_greedy_tokens_identical_to_reference(golden_dir, tmp_path, tag):
    rt, meta, g = _tiny(golden_dir, tag, tmp_path, dtype="float32")
    tokens, first, last = _greedy(rt, g["prompt"].tolist(), meta["steps"], meta["shape"]["vocab_size"])
    assert tokens == g[f"{tag}_tokens"].tolist()
    # reference CPU<->CUDA logits tolerance (tests/test_runtime.py:51-69): 1e-4
    np.testing.assert_allclose(first, g[f"{tag}_prefill_logits_last"], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(last, g[f"{tag}_decode_logits"][2], rtol=1e-4, atol=1e-4)
    pages = [[p.page_id, p.start, p.length] for p in rt.kv_cache.pages]
    want = g[f"{tag}_pages_layer0"]
    assert [p[1:] for p in pages] == [list(r[1:]) for r in want.tolist()]   # page boundaries bit-exact
    stats = rt.cache_stats()
    assert stats["kernel_counts"]["b200.paged_attention_decode_batch.persistent_shared"] >= 1
    assert stats["allocator"]["persistent_pools"]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_tiny_model_half_precision_logits_within_gate(golden_dir, tmp_path, dtype):
    rt, meta, g = _tiny(golden_dir, "int8", tmp_path, dtype=dtype)
    tokens, first, _ = _greedy(rt, g["prompt"].tolist(), meta["steps"], meta["shape"]["vocab_size"])
    tol = 4e-3 if dtype == "float16" else 3e-2   # whole-model error: a dozen roundings per layer, not the per-op gate
    assert oracle.rel_l2(first, g["int8_prefill_logits_last"]) <= tol
    if dtype == "float16":   # min top-1/top-2 margin of the fp32 run is 10x the fp16 error: same tokens
        assert tokens == g["int8_tokens"].tolist()


def test_batched_decode_equals_sequential_and_graph_equals_eager(golden_dir, tmp_path):
    rt, meta, g = _tiny(golden_dir, "int8", tmp_path, dtype="float32")
    eager, _, _ = _tiny(golden_dir, "int8", tmp_path / "e", dtype="float32", use_cuda_graph=False)
    prompts = [g["prompt"][:5].tolist(), g["prompt"][5:22].tolist(), g["prompt"][3:4].tolist()]
    vocab = meta["shape"]["vocab_size"]

    def batched(template):
        sessions = [template.fork() for _ in prompts]
        nxt = []
        for s, p in zip(sessions, prompts):
            logits, _ = s.prefill_tokens(p)
            nxt.append(int(logits[0, -1].argmax().item()) % vocab)
        out = [[] for _ in prompts]
        for _ in range(20):
            logits = template.run_decode_batch(sessions, nxt)
            assert tuple(logits.shape) == (len(prompts), 1, vocab)
            for i, t in enumerate(nxt):
                out[i].append(t)
            nxt = [int(v) % vocab for v in logits[:, -1].argmax(dim=-1).tolist()]
        return out

    def sequential(template):
        out = []
        for p in prompts:
            s = template.fork()
            toks, _, _ = _greedy(s, p, 20, vocab)
            out.append(toks)
        return out

    a, b, c = batched(rt), sequential(rt), batched(eager)
    assert a == b == c


def test_device_feedback_loop_matches_host_loop(golden_dir, tmp_path):
    rt, meta, g = _tiny(golden_dir, "fp32", tmp_path, dtype="float32")
    vocab = meta["shape"]["vocab_size"]
    s = rt.fork()
    logits, _ = s.prefill_tokens(g["prompt"].tolist())
    first = int(logits[0, -1].argmax().item()) % vocab
    toks = rt.decode_greedy_batch([s], [first], meta["steps"] - 1).cpu().numpy()[:, 0].tolist()
    assert [first] + toks == g["fp32_tokens"].tolist()
    assert s.kv_cache.tokens == 32 + meta["steps"] - 1


def test_prefix_sharing_gives_same_tokens_and_aliases_pages(golden_dir, tmp_path):
    rt, meta, g = _tiny(golden_dir, "int8", tmp_path, dtype="float32")
    vocab = meta["shape"]["vocab_size"]
    prompt = g["prompt"].tolist()
    a = rt.fork()
    logits_a, reused = a.prefill_tokens(prompt, use_prefix_cache=True, remember_prefix=True)
    assert reused == ()
    b = rt.fork()
    logits_b, reused = b.prefill_tokens(prompt[:32] + [1, 2, 3], use_prefix_cache=True)
    assert len(reused) == 32 and b.kv_cache.page_ids()[:2] == a.kv_cache.page_ids()[:2]
    c = rt.fork()
    logits_c, _ = c.prefill_tokens(prompt[:32] + [1, 2, 3])
    np.testing.assert_allclose(logits_b[0, -1].cpu().numpy(), logits_c[0, -1].cpu().numpy(), rtol=1e-5, atol=1e-6)
    assert rt.kv_allocator.stats()["shared_page_refs"] >= 2


def test_runtime_errors_mirror_reference(golden_dir, tmp_path):
    rt, _, _ = _tiny(golden_dir, "fp32", tmp_path, dtype="float32")
    with pytest.raises(ValueError):
        rt.run_decode_batch([], [])
    with pytest.raises(ValueError):
        rt.run_decode_batch([rt], [1, 2])
    with pytest.raises(TypeError):
        rt.run_decode_batch([object()], [1])
    other, _, _ = _tiny(golden_dir, "fp32", tmp_path / "o", dtype="float32")
    with pytest.raises(ValueError):
        rt.run_decode_batch([rt, other], [1, 2])


def test_chunked_prefill_equals_token_by_token(golden_dir, tmp_path):
    """Prefill that pushes 64 prompt tokens per pass through the decode graph (rows = tokens of one
    sequence, causal through per-row lengths over the shared page table) against one token per step:
    same logits at every position, same K/V rows in the pool, same page boundaries."""
    rng = np.random.default_rng(3)
    rt, meta, _ = _tiny(golden_dir, "fp32", tmp_path, dtype="float32", max_seq_len=256)
    vocab = meta["shape"]["vocab_size"]
    prompt = [int(t) for t in rng.integers(0, vocab, 150)]          # 64 + 64 + 22 tokens, 10 pages
    chunked, stepped = rt.fork(), rt.fork()
    a = chunked.run([prompt], mode="prefill")
    assert rt.cache_stats()["kernel_counts"]["cacheir.b200_prefill_chunk"] == 3
    rt._engine.prefill_chunk = 0
    b = stepped.run([prompt], mode="prefill")
    rt._engine.prefill_chunk = 64
    assert a.shape == b.shape == (1, 150, vocab)
    np.testing.assert_allclose(a.float().cpu().numpy(), b.float().cpu().numpy(), rtol=2e-4, atol=2e-4)
    assert [(p.start, p.length) for p in chunked.kv_cache.pages] == [(p.start, p.length) for p in stepped.kv_cache.pages]
    for layer in range(2):
        pool = rt.kv_allocator.pool_for_layer(layer)
        for pa, pb in zip(chunked.kv_cache.pages, stepped.kv_cache.pages):
            for name in ("keys", "values"):
                ka = pool[name][pa.page_id][:, : pa.length]
                kb = pool[name][pb.page_id][:, : pb.length]
                np.testing.assert_allclose(ka.float().cpu().numpy(), kb.float().cpu().numpy(), rtol=2e-4, atol=2e-4)
    # decoding continues identically from either cache
    ta = chunked.run([[7]], mode="decode")
    tb = stepped.run([[7]], mode="decode")
    np.testing.assert_allclose(ta.float().cpu().numpy(), tb.float().cpu().numpy(), rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("batch", [40, 70])
def test_wide_batches_match_single_sequence_decoding(batch):
    """Batches above 32 rows (64-row tiles) and above 64 rows (chunked tensor-core launches, unfused
    RMSNorm / RoPE / append) give each sequence the logits it gets when decoded alone."""
    import zlib

    from cacheir_b200 import B200DecodeRuntime
    from cacheir_b200.artifact import ModelConfig, build_decoder_artifact

    cfg = ModelConfig(architecture="LlamaForCausalLM", hidden_size=512, intermediate_size=1024, num_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, vocab_size=512, max_position_embeddings=128,
                      rope_theta=10000.0, rms_norm_eps=1e-5, dtype="float16")
    art = build_decoder_artifact(cfg, quant="int8")

    def source(key, shape):
        g = torch.Generator(device="cpu")
        g.manual_seed(zlib.crc32(key.encode()))
        return torch.ones(shape) if len(shape) == 1 else torch.randn(shape, generator=g) * 0.05

    rt = B200DecodeRuntime(art, dtype="float16", tensor_source=source, max_seq_len=128)
    rng = np.random.default_rng(batch)
    prompts = [[int(t) for t in rng.integers(0, 512, int(rng.integers(3, 9)))] for _ in range(batch)]
    sessions = [rt.fork() for _ in prompts]
    for s, p in zip(sessions, prompts):
        s.run([p], mode="prefill")
    tokens = [int(t) for t in rng.integers(0, 512, batch)]
    wide = rt.run_decode_batch(sessions, tokens)[:, 0].float().cpu().numpy()
    wide2 = rt.run_decode_batch(sessions, tokens)[:, 0].float().cpu().numpy()        # second step: the captured graph
    for i in (0, batch // 2, batch - 1):
        alone = rt.fork()
        alone.run([prompts[i]], mode="prefill")
        a1 = alone.run_decode_batch([alone], [tokens[i]])[0, 0].float().cpu().numpy()
        a2 = alone.run_decode_batch([alone], [tokens[i]])[0, 0].float().cpu().numpy()
        assert oracle.rel_l2(wide[i], a1) <= 4e-3
        assert oracle.rel_l2(wide2[i], a2) <= 4e-3
    from cacheir_b200 import _lib
    assert _lib.load().cacheir_b200_device_status(1) == 0
