"""CPU-side checks: the C-ABI library loads and exports every declared symbol,
and the host logic (page allocator, artifact builder, registry, launcher)
behaves like the reference's. No GPU and no compute calls."""
import ctypes
import json
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols() -> list[str]:
    text = (ROOT / "include" / "cacheir_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cacheir_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from cacheir_b200 import _lib, build

    build.build()
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    declared = _declared_symbols()
    assert len(declared) >= 17
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/cacheir_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == declared, "ctypes table and header disagree"
    loaded = _lib.load()
    assert loaded.cacheir_b200_version() >= 100
    assert b"invalid argument" in loaded.cacheir_b200_error_string(-1)
    # pure host helpers may be called without a GPU
    assert loaded.cacheir_b200_paged_attention_workspace_bytes(2, 4, 8, 1) == 0
    assert loaded.cacheir_b200_paged_attention_workspace_bytes(2, 4, 8, 3) == 2 * 4 * 3 * 10 * 4
    s = loaded.cacheir_b200_paged_attention_auto_splits(64, 32, 8, 511, 16, 128)
    assert 1 <= s <= 64


def test_ops_refuse_cpu_tensors():
    import torch
    from cacheir_b200 import ops
    from cacheir_b200._lib import CacheIRB200Error

    x = torch.zeros(2, 8)
    with pytest.raises(CacheIRB200Error):
        ops.add(x, x)
    with pytest.raises(CacheIRB200Error):
        ops.rms_norm(x, torch.ones(8), 1e-5)


def test_page_allocator_follows_reference_page_boundaries(golden_dir):
    from cacheir_b200.kv_cache import B200KVPageAllocator, B200PagedKVCache

    cases = json.loads((golden_dir / "pages.json").read_text())
    for case in cases:
        alloc = B200KVPageAllocator(page_size=case["page_size"])
        cache = B200PagedKVCache(alloc, num_layers=2)
        layer0 = [h for h in case["history"] if h["layer"] == 0]
        for step in layer0:
            cache.extend(step["append"])
            got = [(p.start, p.length) for p in cache.pages]
            want = [(p["start"], p["length"]) for p in step["pages"]]
            assert got == want
        assert cache.tokens == sum(case["appends"])
        assert len(set(cache.page_ids())) == len(cache.pages)


def test_page_allocator_reuse_and_prefix_sharing():
    from cacheir_b200.kv_cache import B200KVPageAllocator, B200PagedKVCache

    alloc = B200KVPageAllocator(page_size=4, initial_slots=2)
    a = B200PagedKVCache(alloc, 1)
    a.extend(10)                       # pages [0,4) [4,8) [8,10)
    assert a.page_ids() == [0, 1, 2] and alloc.capacity >= 3
    b = B200PagedKVCache(alloc, 1)
    assert b.share_prefix(a, 9) == 8   # whole pages only
    assert b.page_ids() == [0, 1] and alloc.refcount(0) == 2
    b.extend(3)                        # diverges into its own page
    assert b.page_ids()[:2] == [0, 1] and b.page_ids()[2] not in a.page_ids()
    assert b.tokens == 11
    row = b.page_table_row(6)
    assert row.dtype == np.int32 and list(row[:3]) == b.page_ids() and list(row[3:]) == [0, 0, 0]
    a.clear()
    assert alloc.refcount(0) == 1 and alloc.refcount(2) == 0     # shared pages survive their first owner
    c = B200PagedKVCache(alloc, 1)
    c.extend(1)
    assert c.page_ids() == [2]                                   # released slot is reused
    stats = alloc.stats()
    assert stats["released_pages"] == 1 and stats["shared_page_refs"] == 2


def test_decoder_graph_builder_matches_reference_artifacts(golden_dir):
    from cacheir_b200.artifact import CompileArtifact, ModelConfig, build_decoder_graph

    arts = json.loads((golden_dir / "tiny_artifacts.json").read_text())
    for tag, art in arts.items():
        cfg = ModelConfig.from_dict(art["config"])
        loaded = CompileArtifact.from_dict({**art, "model_path": ""})
        for mode in ("decode", "prefill"):
            built = build_decoder_graph(cfg, mode=mode, target="cuda", quant=art["quant"])
            ref = art["graphs"][mode]
            assert [n.op for n in built.nodes] == [n["op"] for n in ref["nodes"]]
            for node, want in zip(built.nodes, ref["nodes"]):
                assert node.inputs == want["inputs"] and node.outputs == want["outputs"]
                assert node.attrs == want["attrs"], (tag, mode, node.op)
            assert [n.op for n in loaded.graph(mode).nodes] == [n.op for n in built.nodes]
            assert built.attrs["execution_hints"] == ref["attrs"]["execution_hints"]
    ops_int8 = [n["op"] for n in arts["int8"]["graphs"]["decode"]["nodes"]]
    # op names the reference's own test pins (tests/test_project_surfaces.py:56-70)
    assert "quantized_fused_rmsnorm_qkv_rope" in ops_int8 and "quantized_matmul" in ops_int8
    assert "paged_attention_decode" in ops_int8 and "quantized_fused_swiglu" in ops_int8


def test_registry_lists_b200_backend():
    from cacheir_b200.registry import KERNEL_FOR_OP, default_registry
    from cacheir_b200 import _lib

    reg = default_registry()
    assert reg.names() == ["cuda-b200"]
    backend = reg.get("cuda-b200")
    assert backend.devices == ("sm100a",) and "paged_attention_decode" in backend.kernels
    for _, entry_points in KERNEL_FOR_OP.values():
        for name in entry_points:
            assert name in _lib.SIGNATURES


def test_tiny_model_generator_is_deterministic(tmp_path):
    from cacheir_b200.tiny import create_tiny_model

    a = create_tiny_model(tmp_path / "a", seed=3, vocab_size=32, hidden_size=16, intermediate_size=32, num_layers=1)
    b = create_tiny_model(tmp_path / "b", seed=3, vocab_size=32, hidden_size=16, intermediate_size=32, num_layers=1)
    wa, wb = np.load(a / "weights.npz"), np.load(b / "weights.npz")
    assert sorted(wa.files) == sorted(wb.files)
    for k in wa.files:
        np.testing.assert_array_equal(wa[k], wb[k])
    assert json.loads((a / "config.json").read_text())["rms_norm_eps"] == 1e-5


class _FakeRuntime:
    """Deterministic stand-in exposing the runtime duck type, for the launcher logic."""

    class _KV:
        def clear(self):
            pass

    class _Cfg:
        vocab_size = 11

    class _Art:
        pass

    def __init__(self):
        self.artifact = self._Art()
        self.artifact.config = self._Cfg()
        self.kv_cache = self._KV()
        self.tokens: list[int] = []

    def fork(self):
        return _FakeRuntime()

    def synchronize(self):
        pass

    def _logits(self, history):
        import torch
        out = torch.zeros(1, 1, 11)
        out[0, 0, (sum(history) * 7 + len(history)) % 11] = 1.0
        return out

    def prefill_tokens(self, ids, **_):
        self.tokens = list(ids)
        return self._logits(self.tokens), ()

    def run_decode_batch(self, sessions, token_ids):
        import torch
        rows = []
        for s, t in zip(sessions, token_ids):
            s.tokens.append(int(t))
            rows.append(s._logits(s.tokens))
        return torch.cat(rows, dim=0)


def test_batched_launcher_equals_sequential():
    # counters and equality mirrored from the reference's tests/test_scheduler.py:146-183
    from cacheir_b200.scheduler import BatchedDecodeLauncher

    prompts = [[1, 2, 3], [4, 5]]
    batched = BatchedDecodeLauncher(_FakeRuntime(), max_batch_size=2)
    ids = [batched.submit(p, max_new_tokens=3) for p in prompts]
    got = batched.run_until_complete()
    seq = BatchedDecodeLauncher(_FakeRuntime(), max_batch_size=1)
    ids2 = [seq.submit(p, max_new_tokens=3) for p in prompts]
    want = seq.run_until_complete()
    assert [got[i] for i in ids] == [want[i] for i in ids2]
    assert batched.metrics.batched_decode_rounds == 3
    assert batched.metrics.batched_decode_tokens == 6
    assert batched.metrics.completed_requests == 2


def test_group_int4_packer_matches_oracle_dequantisation():
    """Group-wise symmetric int4 (the extension the 70B-shaped configuration uses): codes and fp16 scales
    made by the host-side packer dequantise, through the oracle's formula, to within half a step of the weight."""
    import numpy as np
    import torch

    from cacheir_b200.quantization import pack_group_int4, quant_bits, quant_group_size
    from oracle import oracle

    assert quant_group_size("int4_g128") == 128 and quant_bits("int4_g128") == 4 and quant_group_size("int8") == 0
    rng = np.random.default_rng(0)
    w = rng.standard_normal((6, 384)).astype(np.float32) * 0.02
    w[2, :128] = 0.0                                             # an all-zero group keeps a tiny positive scale
    p = pack_group_int4(torch.from_numpy(w), 128)
    assert p.packed_values.shape == (6, 192) and p.scales.shape == (6, 3) and p.scales.dtype == torch.float16
    codes = p.packed_values.numpy()
    q = np.empty((6, 384), dtype=np.uint8)
    q[:, 0::2] = codes & 15                                      # even column in the low nibble
    q[:, 1::2] = codes >> 4
    deq = oracle.dequantize_packed_weight(oracle.symmetric_group_pack_from_codes(q, p.scales.numpy(), 4, 128))
    step = np.repeat(p.scales.numpy().astype(np.float32), 128, axis=1)
    assert np.all(np.abs(deq - w) <= step / 2 * 1.01 + 1e-7)
    assert np.all(deq[2, :128] == 0.0)
    with pytest.raises(ValueError):
        pack_group_int4(torch.zeros(4, 100), 128)
