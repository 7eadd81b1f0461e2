"""Generate the golden fixtures in this directory by running the reference.

Run where the reference checkout is importable:

    PYTHONPATH=/path/to/CacheIR python tests/golden/make_golden.py

It imports the reference package (`cacheir`) unmodified, feeds it seeded
inputs and stores inputs + outputs as small .npz/.json files. The fixtures pin
the CPU oracle (oracle/oracle.py) and, through it, the CUDA path. The GPU
machine never needs the reference: only the committed fixtures travel.
"""
from __future__ import annotations

import hashlib
import json
import tempfile
from pathlib import Path

import numpy as np

from cacheir.compiler import compile_model
from cacheir.importers.tiny import create_tiny_model
from cacheir.quantization import dequantize_packed_weight, pack_quantized_weight
from cacheir.runtime.cpu import Runtime
from cacheir.runtime.kv_cache import PagedKVCache

HERE = Path(__file__).resolve().parent


def _pack_case(weight: np.ndarray, prefix: str, out: dict[str, np.ndarray]) -> None:
    out[f"{prefix}_w"] = weight
    for quant, tag in (("int4_awq", "q4"), ("int8", "q8")):
        packed = pack_quantized_weight(weight, quant)
        out[f"{prefix}_{tag}_packed"] = packed.packed_values
        out[f"{prefix}_{tag}_scales"] = packed.scales
        out[f"{prefix}_{tag}_zero_points"] = packed.zero_points
        out[f"{prefix}_{tag}_dequant"] = dequantize_packed_weight(packed)


def make_pack() -> None:
    out: dict[str, np.ndarray] = {}
    # the reference's own test input (tests/test_project_surfaces.py:73-82)
    _pack_case(np.linspace(-1.5, 2.0, num=30, dtype=np.float32).reshape(3, 10), "lin", out)
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((37, 53)) * 0.02).astype(np.float32)   # odd K: padded nibble
    w[3] = 0.25                                  # constant row: scale floor 1e-8, huge zero point
    w[5] = np.abs(w[5]) + 0.5                    # all positive: negative, unclipped zero point
    w[7] = -np.abs(w[7]) - 0.5                   # all negative
    w[9, :] = np.linspace(-1.0, 1.0, 53)         # many exact .5 ties after scaling
    _pack_case(w, "rnd", out)
    w2 = (rng.standard_normal((16, 256)) * 0.02).astype(np.float32)
    _pack_case(w2, "even", out)
    np.savez_compressed(HERE / "pack.npz", **out)


def make_pages() -> None:
    cases = []
    for page_size, appends in ((16, [32] + [1] * 33), (2, [5, 1, 1, 3]), (16, [1] * 17), (4, [9, 7, 1]), (1, [3, 2])):
        cache = PagedKVCache(page_size=page_size)
        history = []
        for layer in (0, 1):
            for n in appends:
                keys = np.zeros((1, n, 1, 8), dtype=np.float32)
                cache.append(layer, keys, keys)
                history.append({"layer": layer, "append": n,
                                "pages": [p.to_dict() for p in cache.layers[layer].pages]})
        cases.append({"page_size": page_size, "appends": appends, "history": history,
                      "page_bytes": cache.page_bytes, "total_pages": cache.total_pages()})
    (HERE / "pages.json").write_text(json.dumps(cases, indent=1), encoding="utf-8")


def _strip_graph(graph) -> dict:
    data = graph.to_dict()
    attrs = data.get("attrs", {})
    for noisy in ("hardware_profile", "execution_schedule", "memory_plan"):
        attrs.pop(noisy, None)
    return data


def make_tiny() -> None:
    shape = dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_layers=2,
                 num_attention_heads=4, num_key_value_heads=2)
    prompt = np.random.default_rng(0).integers(0, 1024, 32)
    result: dict[str, np.ndarray] = {"prompt": prompt.astype(np.int64)}
    meta: dict[str, object] = {"shape": shape, "seed": 0, "steps": 32}
    with tempfile.TemporaryDirectory() as tmp:
        model = create_tiny_model(Path(tmp) / "tiny", seed=0, **shape)
        with np.load(model / "weights.npz") as data:
            meta["weight_sha256"] = {k: hashlib.sha256(np.ascontiguousarray(data[k]).tobytes()).hexdigest() for k in data.files}
        artifacts = {}
        for tag, quant in (("fp32", None), ("int8", "int8"), ("int4", "int4_awq")):
            art = compile_model(model, target="cuda", quant=quant, mode=["prefill", "decode"], max_seq=128)
            artifacts[tag] = {"target": art.target, "quant": art.quant, "config": art.config.to_dict(),
                              "graphs": {m: _strip_graph(g) for m, g in art.graphs.items()}}
            rt = Runtime(art)
            logits = rt.run([prompt.tolist()], mode="prefill")
            result[f"{tag}_prefill_logits_last"] = np.asarray(logits[0, -1], dtype=np.float32)
            tokens, step_logits = [], []
            for _ in range(32):
                nxt = int(np.argmax(logits[0, -1])) % 1024
                tokens.append(nxt)
                logits = rt.run([[nxt]], mode="decode")
                step_logits.append(np.asarray(logits[0, -1], dtype=np.float32))
            result[f"{tag}_tokens"] = np.asarray(tokens, dtype=np.int64)
            result[f"{tag}_decode_logits"] = np.stack(step_logits)[[0, 15, 31]]
            result[f"{tag}_pages_layer0"] = np.asarray(
                [[p.page_id, p.start, p.length] for p in rt.kv_cache.layers[0].pages], dtype=np.int64)
            top2 = np.sort(np.stack(step_logits), axis=-1)[:, -2:]
            meta[f"{tag}_min_top1_top2_margin"] = float(np.min(top2[:, 1] - top2[:, 0]))
        (HERE / "tiny_artifacts.json").write_text(json.dumps(artifacts), encoding="utf-8")
    np.savez_compressed(HERE / "tiny_c1.npz", **result)
    (HERE / "tiny_c1_meta.json").write_text(json.dumps(meta, indent=1), encoding="utf-8")


def make_numerics() -> None:
    """Attention, RoPE and RMSNorm of the reference CPU runtime on seeded inputs."""
    rng = np.random.default_rng(5)
    out: dict[str, np.ndarray] = {}
    with tempfile.TemporaryDirectory() as tmp:
        model = create_tiny_model(Path(tmp) / "tiny", seed=1)
        rt = Runtime(compile_model(model, target="cpu", mode=["decode"], max_seq=8))
        for tag, (heads, kv_heads, hd, t) in {"a": (4, 2, 8, 5), "b": (8, 2, 64, 37), "c": (4, 4, 16, 3)}.items():
            q = rng.standard_normal((1, 1, heads * hd)).astype(np.float32)
            k = rng.standard_normal((1, t, kv_heads * hd)).astype(np.float32)
            v = rng.standard_normal((1, t, kv_heads * hd)).astype(np.float32)
            attrs = {"layer": 100 + ord(tag), "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": hd}
            out[f"attn_{tag}_q"], out[f"attn_{tag}_k"], out[f"attn_{tag}_v"] = q, k, v
            out[f"attn_{tag}_out"] = rt._attention(q, k, v, attrs, "decode")
            out[f"attn_{tag}_dims"] = np.asarray([heads, kv_heads, hd, t])
        x = rng.standard_normal((2, 3, 4 * 16)).astype(np.float32)
        out["rope_x"] = x
        out["rope_out_off7"] = Runtime._rope_one(x, 16, 10000.0, 7)
        out["rope_out_off0"] = Runtime._rope_one(x, 16, 10000.0, 0)
        h = rng.standard_normal((2, 1, 48)).astype(np.float32)
        w = rng.standard_normal((48,)).astype(np.float32)
        out["rms_x"], out["rms_w"] = h, w
        out["rms_out"] = Runtime._rms_norm(h, w, 1e-5)
    np.savez_compressed(HERE / "numerics.npz", **out)


if __name__ == "__main__":
    make_pack()
    make_pages()
    make_tiny()
    make_numerics()
    for f in sorted(HERE.iterdir()):
        print(f.name, f.stat().st_size)
