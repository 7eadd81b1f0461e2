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


# ---- the batched-decode launcher on the real runtime: changing batch composition, row slots, limits ----
def test_launcher_on_the_b200_runtime_batched_equals_one_at_a_time(golden_dir, tmp_path):
    """What the reference checks for its scheduler (tests/test_scheduler.py:146-183): requests decoded together give
    the ids they get one at a time, and the counters add up -- here on the CUDA runtime, with token budgets that
    make requests retire at different rounds, so the batch shrinks and refills while it runs."""
    from cacheir_b200.scheduler import BatchedDecodeLauncher

    rt, meta, g = _tiny(golden_dir, "int8", tmp_path, dtype="float16", max_seq_len=128)
    prompt = g["prompt"].tolist()
    requests = [(prompt[:7], 5), (prompt[3:30], 12), (prompt[10:11], 3), (prompt[:32], 9), (prompt[5:9], 12), (prompt[20:28], 1)]

    def run(max_batch):
        launcher = BatchedDecodeLauncher(rt, max_batch_size=max_batch)
        ids = [launcher.submit(p, max_new_tokens=n) for p, n in requests]
        results = launcher.run_until_complete()
        return [results[i] for i in ids], launcher.metrics

    lowered_before = rt.cache_stats()["plans_lowered"]
    batched, metrics = run(4)
    single, single_metrics = run(1)
    assert batched == single
    assert [len(t) for t in batched] == [n for _, n in requests]
    assert metrics.completed_requests == len(requests) and metrics.generated_tokens == sum(n for _, n in requests)
    assert metrics.batched_decode_tokens == metrics.generated_tokens
    assert metrics.batched_decode_rounds < single_metrics.batched_decode_rounds
    # plans are keyed by batch size: four sizes were seen (4, 3, 2, 1), however often the occupants changed
    stats = rt.cache_stats()
    assert stats["plans_lowered"] - lowered_before <= 4 + 1          # + the prefill plan
    assert stats["graph_captures"] <= stats["plans_lowered"] + 4
    rt.synchronize()
    from cacheir_b200 import _lib
    assert _lib.load().cacheir_b200_device_status(1) == 0


def test_reference_scheduler_drives_the_b200_runtime(golden_dir, tmp_path):
    """The reference's own ContinuousBatchScheduler (cacheir/runtime/scheduler.py:109, 456-478, 508-509) accepts any
    object with the runtime duck type. Runs where the reference package is importable."""
    cacheir_scheduler = pytest.importorskip("cacheir.runtime.scheduler")
    rt, meta, g = _tiny(golden_dir, "int8", tmp_path, dtype="float16", max_seq_len=256)
    prompts = ["paged attention", "decode", "a longer prompt that spans more than one page of sixteen tokens", "kv"]
    budgets = [6, 11, 4, 9]

    def run(max_batch):
        sched = cacheir_scheduler.ContinuousBatchScheduler(rt, max_batch_size=max_batch, use_prefix_cache=False)
        for p, n in zip(prompts, budgets):
            sched.submit(p, max_new_tokens=n)
        results = sched.run_until_complete()
        return {r.request_id: list(r.generated_ids) for r in results}, sched.metrics

    batched, metrics = run(4)
    single, _ = run(1)
    assert batched == single
    assert metrics.batched_decode_rounds > 0 and metrics.completed_requests == len(prompts)


def test_pool_exhaustion_and_position_limit_are_reported_like_the_reference(golden_dir, tmp_path):
    from cacheir_b200 import B200KVPageAllocator
    rt, meta, g = _tiny(golden_dir, "fp32", tmp_path, dtype="float32", max_seq_len=64,
                        kv_allocator=B200KVPageAllocator(page_size=16, initial_slots=3, max_slots=3))
    prompt = g["prompt"].tolist()
    s = rt.fork()
    s.run([prompt[:30]], mode="prefill")                 # two pages
    t = rt.fork()
    t.run([prompt[:10]], mode="prefill")                 # the third and last page
    # the next page cannot be allocated: wrapped like the reference's out-of-memory path (cuda.py:577-579), the caller's
    # session is cleared and counted
    with pytest.raises(RuntimeError, match="out-of-memory"):
        for tok in range(10):
            s.run_decode_batch([s], [tok])
    assert s.oom_recoveries == 1 and s.kv_cache.tokens == 0
    assert s.cache_stats()["oom_recoveries"] == 1
    # the freed pages serve a new request
    u = rt.fork()
    u.run([prompt[:20]], mode="prefill")
    assert u.kv_cache.tokens == 20
    # a sequence may not grow past the cos/sin table
    rt2, _, _ = _tiny(golden_dir, "fp32", tmp_path / "b", dtype="float32", max_seq_len=40)
    v = rt2.fork()
    v.run([prompt[:32]], mode="prefill")
    with pytest.raises(ValueError, match="max_seq_len"):
        for tok in range(12):
            v.run_decode_batch([v], [tok])


def test_packed_prefill_of_several_sequences_equals_one_by_one(golden_dir, tmp_path):
    """`run_prefill_batch` lays the prompt tokens of all sequences out as the rows of shared 64-row passes (short
    prompts share a pass, a long one spans several): same logits, same K/V rows and page boundaries as prefilling
    each sequence on its own, and decoding continues identically."""
    rng = np.random.default_rng(11)
    rt, meta, _ = _tiny(golden_dir, "fp32", tmp_path, dtype="float32", max_seq_len=256)
    vocab = meta["shape"]["vocab_size"]
    lens = [5, 70, 1, 33, 64]                                            # 173 tokens: three passes
    prompts = [[int(t) for t in rng.integers(0, vocab, n)] for n in lens]
    packed = [rt.fork() for _ in prompts]
    before = rt.cache_stats()["kernel_counts"].get("cacheir.b200_prefill_chunk", 0)
    out = rt.run_prefill_batch(packed, prompts)
    assert rt.cache_stats()["kernel_counts"]["cacheir.b200_prefill_chunk"] - before == 3
    assert tuple(out.shape) == (len(prompts), max(lens), vocab)
    pools = [rt.kv_allocator.pool_for_layer(layer) for layer in range(2)]
    for i, (p, n) in enumerate(zip(prompts, lens)):
        alone = rt.fork()
        rt._engine.prefill_chunk = 0                                      # one token per step
        want = alone.run([p], mode="prefill")
        rt._engine.prefill_chunk = 64
        np.testing.assert_allclose(out[i, :n].float().cpu().numpy(), want[0].float().cpu().numpy(), rtol=2e-4, atol=2e-4)
        assert float(out[i, n:].abs().max()) == 0.0 if n < max(lens) else True
        assert [(pg.start, pg.length) for pg in packed[i].kv_cache.pages] == [(pg.start, pg.length) for pg in alone.kv_cache.pages]
        for pool in pools:
            for pa, pb in zip(packed[i].kv_cache.pages, alone.kv_cache.pages):
                for name in ("keys", "values"):
                    np.testing.assert_allclose(pool[name][pa.page_id][:, : pa.length].float().cpu().numpy(),
                                               pool[name][pb.page_id][:, : pb.length].float().cpu().numpy(), rtol=2e-4, atol=2e-4)
        a = packed[i].run([[7]], mode="decode")
        b = alone.run([[7]], mode="decode")
        np.testing.assert_allclose(a.float().cpu().numpy(), b.float().cpu().numpy(), rtol=2e-4, atol=2e-4)


def test_attention_prepass_fusion_changes_no_bit(tmp_path):
    """A 2-layer int8 model with head_dim 128 (the shape class the fused launch takes): with and without the attention
    kernel writing the o-projection's activation planes, batched greedy decoding yields the same logits bits."""
    import zlib

    from cacheir_b200 import B200DecodeRuntime, B200KVPageAllocator, ModelConfig, build_decoder_artifact

    mc = ModelConfig(architecture="LlamaForCausalLM", hidden_size=1024, intermediate_size=2048, num_layers=2,
                     num_attention_heads=8, num_key_value_heads=2, vocab_size=512, max_position_embeddings=256,
                     rope_theta=10000.0, rms_norm_eps=1e-5, dtype="float16")
    art = build_decoder_artifact(mc, target="cuda", quant="int8", modes=("decode",))
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev)

    def synth(key, shape):
        if len(shape) == 1:
            return torch.ones(shape, device=dev, dtype=torch.float32)
        gen.manual_seed(zlib.crc32(key.encode()))
        return torch.randn(shape, device=dev, dtype=torch.float32, generator=gen) * 0.05

    rng = np.random.default_rng(5)
    prompts = [[int(t) for t in rng.integers(0, 512, n)] for n in (5, 40, 17, 3, 64, 9)]
    results = []
    for fuse in (True, False):
        rt = B200DecodeRuntime(art, dtype="float16", tensor_source=synth, kv_allocator=B200KVPageAllocator(page_size=16),
                               max_seq_len=256, fuse_attention_prepass=fuse)
        sessions = [rt.fork() for _ in prompts]
        prefill = rt.run_prefill_batch(sessions, prompts)
        tokens = [int(torch.argmax(prefill[i, len(p) - 1]).item()) for i, p in enumerate(prompts)]
        steps = [prefill.clone()]
        for _ in range(6):
            logits = rt.run_decode_batch(sessions, tokens)
            steps.append(logits[:, 0].clone())
            tokens = [int(torch.argmax(row).item()) for row in logits[:, 0]]
        counts = rt.cache_stats()["kernel_counts"]
        assert (counts.get("b200.attention_prepass_fused", 0) > 0) == fuse
        rt.check_device_status()
        results.append(steps)
    for a, b in zip(*results):
        assert torch.equal(a, b)
