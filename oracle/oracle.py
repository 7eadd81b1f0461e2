"""CPU oracle for the CacheIR decode hot path -- TEST INFRASTRUCTURE ONLY.

A NumPy restatement of the reference project's (AhanBhatt/CacheIR) CPU
algorithms for the batched decode step. Only the test-suite, the smoke check
and the CPU-baseline leg of the benchmark may import this module; the product
package never does. Every function cites the reference file:line it follows
(paths relative to the reference's root). Parity of this restatement is pinned
by the fixtures under tests/golden/, which were produced by importing the
reference itself (see tests/golden/make_golden.py).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


# --------------------------------------------------------------------------
# Quantization pack format (cacheir/quantization.py)
# --------------------------------------------------------------------------
@dataclass
class PackedQuantizedTensor:
    """cacheir/quantization.py:17-35."""

    packed_values: np.ndarray
    scales: np.ndarray
    zero_points: np.ndarray
    bits: int
    shape: tuple[int, int]
    axis: int = 1
    group_size: int | None = None


def quant_bits(quant: str | None) -> int | None:
    """Bit width chosen from the quant name, cacheir/quantization.py:63-71."""
    if not quant:
        return None
    name = quant.lower()
    if "int4" in name or "awq" in name or "gptq" in name:
        return 4
    if "int8" in name or "8bit" in name:
        return 8
    return None


def pack_int4(qvalues: np.ndarray) -> np.ndarray:
    """Two codes per byte, even column in the low nibble; cacheir/quantization.py:123-130."""
    rows, cols = qvalues.shape
    padded = np.zeros((rows, cols + (cols % 2)), dtype=np.uint8)
    padded[:, :cols] = qvalues & 0x0F
    return (padded[:, 0::2] | (padded[:, 1::2] << 4)).astype(np.uint8)


def unpack_int4(packed: np.ndarray, cols: int) -> np.ndarray:
    """cacheir/quantization.py:133-139 (codes returned as float32)."""
    rows = packed.shape[0]
    out = np.empty((rows, packed.shape[1] * 2), dtype=np.float32)
    out[:, 0::2] = (packed & 0x0F).astype(np.float32)
    out[:, 1::2] = ((packed >> 4) & 0x0F).astype(np.float32)
    return out[:, :cols]


def asymmetric_pack(weight: np.ndarray, bits: int) -> PackedQuantizedTensor:
    """Per-row affine quantization, cacheir/quantization.py:96-120.

    Kept operation for operation: the float32/float64 mix of the NumPy
    expression (`array / scales` is float32, adding the int32 zero points
    promotes to float64) decides ties, so it is part of the format.
    """
    array = np.asarray(weight, dtype=np.float32)
    if array.ndim != 2:
        raise ValueError("packed quantization expects a 2D out_features x in_features weight")
    if bits not in (4, 8):
        raise ValueError(f"unsupported packed bit width {bits}")
    qmin, qmax = 0, (1 << bits) - 1
    mins = np.min(array, axis=1)
    maxs = np.max(array, axis=1)
    scales = np.maximum((maxs - mins) / float(qmax - qmin), 1.0e-8).astype(np.float32)
    zero_points = np.round(qmin - mins / scales).astype(np.int32)
    qvalues = np.round(array / scales[:, None] + zero_points[:, None]).clip(qmin, qmax).astype(np.uint8)
    packed = pack_int4(qvalues) if bits == 4 else qvalues
    return PackedQuantizedTensor(
        packed_values=np.ascontiguousarray(packed),
        scales=np.ascontiguousarray(scales),
        zero_points=np.ascontiguousarray(zero_points),
        bits=bits,
        shape=(int(array.shape[0]), int(array.shape[1])),
    )


def pack_quantized_weight(weight: np.ndarray, quant: str | None) -> PackedQuantizedTensor | None:
    """cacheir/quantization.py:63-71."""
    bits = quant_bits(quant)
    return None if bits is None else asymmetric_pack(weight, bits)


def dequantize_packed_weight(q: PackedQuantizedTensor) -> np.ndarray:
    """(code - zero) * scale in float32; cacheir/quantization.py:74-84.

    group_size > 0 is the group-wise symmetric extension: scales[n, k // group],
    zero point 2**(bits-1) (nearest relative in the reference: the Q4_0 block
    decode `(nibble - 8) * d`, cacheir/importers/gguf.py:297-310).
    """
    rows, cols = q.shape
    if q.bits == 4:
        codes = unpack_int4(q.packed_values, cols)
    elif q.bits == 8:
        codes = q.packed_values.astype(np.float32)
    else:
        raise ValueError(f"unsupported packed bit width {q.bits}")
    codes = codes[:rows, :cols].astype(np.float32)
    if q.group_size:
        scale = np.repeat(q.scales.astype(np.float32), q.group_size, axis=1)[:, :cols]
        return (codes - np.float32(1 << (q.bits - 1))) * scale
    scale = q.scales.astype(np.float32)[:, None]
    zero = q.zero_points.astype(np.float32)[:, None]
    return (codes - zero) * scale


def decode_q4_0_blocks(raw: bytes, count: int) -> np.ndarray:
    """llama.cpp Q4_0: per 32 elements an fp16 scale d and 16 bytes; low nibbles are elements
    0..15, high nibbles 16..31; value = (nibble - 8) * d. cacheir/importers/gguf.py:297-310."""
    data = np.frombuffer(raw, dtype=np.uint8).reshape(count // 32, 18)
    d = data[:, :2].copy().view(np.float16).astype(np.float32)            # [blocks, 1]
    out = np.empty((count // 32, 32), dtype=np.float32)
    out[:, :16] = (data[:, 2:] & 0x0F).astype(np.float32) - 8.0
    out[:, 16:] = (data[:, 2:] >> 4).astype(np.float32) - 8.0
    return (out * d).reshape(-1)


def decode_q8_0_blocks(raw: bytes, count: int) -> np.ndarray:
    """llama.cpp Q8_0: per 32 elements an fp16 scale d and 32 signed bytes; value = int8 * d.
    cacheir/importers/gguf.py:273-283."""
    data = np.frombuffer(raw, dtype=np.uint8).reshape(count // 32, 34)
    d = data[:, :2].copy().view(np.float16).astype(np.float32)
    return (data[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1)


def quantize_dequantize(weight: np.ndarray, quant: str | None) -> np.ndarray:
    """cacheir/quantization.py:52-60 (packed branch): what a non-matmul 2-D weight becomes under quant."""
    packed = pack_quantized_weight(weight, quant)
    if packed is None:
        return np.asarray(weight, dtype=np.float32)
    return dequantize_packed_weight(packed)


def symmetric_group_pack_from_codes(codes: np.ndarray, scales: np.ndarray, bits: int, group_size: int) -> PackedQuantizedTensor:
    """Wrap given codes/scales in the group-wise symmetric layout (synthetic benchmark weights)."""
    n, k = codes.shape
    packed = pack_int4(codes.astype(np.uint8)) if bits == 4 else codes.astype(np.uint8)
    return PackedQuantizedTensor(
        packed_values=np.ascontiguousarray(packed),
        scales=np.ascontiguousarray(scales),
        zero_points=np.full((n,), 1 << (bits - 1), dtype=np.int32),
        bits=bits,
        shape=(n, k),
        group_size=group_size,
    )


# --------------------------------------------------------------------------
# Page metadata (cacheir/runtime/kv_cache.py)
# --------------------------------------------------------------------------
@dataclass
class KVPage:
    """cacheir/runtime/kv_cache.py:9-16."""

    page_id: int
    start: int
    length: int

    def to_dict(self) -> dict[str, int]:
        return {"page_id": self.page_id, "start": self.start, "length": self.length}


@dataclass
class PageList:
    """Page bookkeeping of one layer of `PagedKVCache` (kv_cache.py:31-46)."""

    page_size: int = 16
    pages: list[KVPage] = field(default_factory=list)
    length: int = 0


def extend_pages(pages: list[KVPage], next_page_id: int, page_size: int, start: int, length: int) -> int:
    """`PagedKVCache._extend_pages`, cacheir/runtime/kv_cache.py:111-123. Returns the new next_page_id."""
    remaining = length
    cursor = start
    while remaining > 0:
        page_offset = cursor % page_size
        take = min(remaining, page_size - page_offset)
        if page_offset == 0:
            pages.append(KVPage(page_id=next_page_id, start=cursor, length=take))
            next_page_id += 1
        else:
            pages[-1].length += take
        cursor += take
        remaining -= take
    return next_page_id


# --------------------------------------------------------------------------
# Numerics of the decode graph (cacheir/runtime/cpu.py)
# --------------------------------------------------------------------------
def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """cacheir/runtime/cpu.py:285-289."""
    scale = 1.0 / np.sqrt(np.mean(np.square(x), axis=-1, keepdims=True) + eps)
    return (x * scale) * weight


def matmul(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    """`Runtime._matmul`, cacheir/runtime/cpu.py:292-304: x[..., i] . weight[o, i]."""
    return np.einsum("...i,oi->...o", x, weight, optimize=True)


def quantized_matmul(x: np.ndarray, weight: PackedQuantizedTensor | np.ndarray) -> np.ndarray:
    """Dequantize the whole weight, then matmul; cacheir/runtime/cpu.py:306-312."""
    dense = dequantize_packed_weight(weight) if isinstance(weight, PackedQuantizedTensor) else weight
    return matmul(x, dense.astype(np.float32, copy=False))


def rope_one(x: np.ndarray, head_dim: int, theta: float, offsets) -> np.ndarray:
    """Interleaved-pair RoPE, cacheir/runtime/cpu.py:324-340; `offsets` is one
    position offset per batch row (the batched form, cacheir/runtime/cuda.py:1084-1102)."""
    batch, seq, flat = x.shape
    heads = flat // head_dim
    view = x.reshape(batch, seq, heads, head_dim)
    half = head_dim // 2
    freq = 1.0 / (theta ** (np.arange(0, half, dtype=np.float32) * 2.0 / head_dim))
    base = np.asarray(offsets, dtype=np.float32).reshape(-1)
    if base.size == 1:
        base = np.repeat(base, batch)
    pos = base[:, None] + np.arange(seq, dtype=np.float32)[None, :]
    angles = pos[:, :, None] * freq[None, None, :]
    cos = np.cos(angles)[:, :, None, :]
    sin = np.sin(angles)[:, :, None, :]
    even = view[..., 0::2]
    odd = view[..., 1::2]
    rotated = np.empty_like(view)
    rotated[..., 0::2] = even * cos - odd * sin
    rotated[..., 1::2] = even * sin + odd * cos
    return rotated.reshape(batch, seq, flat)


def softmax(x: np.ndarray, axis: int = -1) -> np.ndarray:
    """cacheir/runtime/cpu.py:373-377."""
    shifted = x - np.max(x, axis=axis, keepdims=True)
    e = np.exp(shifted)
    return e / np.sum(e, axis=axis, keepdims=True)


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """cacheir/runtime/cpu.py:272 (and cpp/src/cacheir_backend.cpp:129-144)."""
    return (gate / (1.0 + np.exp(-gate))) * up


def attention_contiguous(q: np.ndarray, keys: np.ndarray, values: np.ndarray, heads: int, kv_heads: int,
                         head_dim: int, causal: bool = False) -> np.ndarray:
    """`Runtime._attention` after the cache append, cacheir/runtime/cpu.py:355-371.

    q: [B, Q, heads*D]; keys/values: [B, T, kv_heads, D] (the full cache)."""
    batch, q_len, _ = q.shape
    qh = q.reshape(batch, q_len, heads, head_dim)
    repeat = heads // kv_heads
    kh = np.repeat(keys, repeat, axis=2) if repeat > 1 else keys
    vh = np.repeat(values, repeat, axis=2) if repeat > 1 else values
    scores = np.einsum("bqhd,bkhd->bhqk", qh, kh, optimize=True) / float(np.sqrt(float(head_dim)))
    if causal:
        k_len = kh.shape[1]
        past = max(0, k_len - q_len)
        qpos = past + np.arange(q_len, dtype=np.int64)[:, None]
        kpos = np.arange(k_len, dtype=np.int64)[None, :]
        scores = np.where((kpos > qpos)[None, None, :, :], -1.0e30, scores)
    probs = softmax(scores, axis=-1)
    ctx = np.einsum("bhqk,bkhd->bqhd", probs, vh, optimize=True)
    return ctx.reshape(batch, q_len, heads * head_dim)


def gather_pages(pool: np.ndarray, page_table_row: np.ndarray, seq_len: int) -> np.ndarray:
    """Rows 0..seq_len-1 of one sequence out of a [slots, kv_heads, page, D] pool ->
    [seq_len, kv_heads, D]. Row t lives in page_table[t // page] at slot t % page
    (cacheir/backends/triton_kernels.py:199-206; pinned by the gather loop of
    tests/test_advanced_experiments.py:546-557)."""
    page_size = pool.shape[2]
    n_pages = (seq_len + page_size - 1) // page_size
    pages = pool[np.asarray(page_table_row[:n_pages], dtype=np.int64)]  # [n, kvh, page, D]
    rows = pages.transpose(0, 2, 1, 3).reshape(n_pages * page_size, pool.shape[1], pool.shape[3])
    return rows[:seq_len]


def paged_attention_decode(q: np.ndarray, k_pool: np.ndarray, v_pool: np.ndarray, page_table: np.ndarray,
                           seq_lens: np.ndarray, scale: float | None = None) -> np.ndarray:
    """Batched paged decode attention: the page gather of the Triton kernel
    (cacheir/backends/triton_kernels.py:174-217) followed by the CPU attention
    math (cacheir/runtime/cpu.py:355-371). q: [B, H, D] -> out [B, H, D], float32 math."""
    batch, heads, head_dim = q.shape
    kv_heads = k_pool.shape[1]
    repeat = heads // kv_heads
    out = np.zeros((batch, heads, head_dim), dtype=np.float32)
    s = float(scale) if scale else 1.0 / float(np.sqrt(float(head_dim)))
    for b in range(batch):
        n = int(seq_lens[b])
        if n <= 0:
            continue
        keys = gather_pages(k_pool, page_table[b], n).astype(np.float32)    # [n, kvh, D]
        vals = gather_pages(v_pool, page_table[b], n).astype(np.float32)
        qb = q[b].astype(np.float32).reshape(kv_heads, repeat, head_dim)
        scores = np.einsum("grd,ngd->grn", qb, keys, optimize=True) * s
        probs = softmax(scores, axis=-1)
        out[b] = np.einsum("grn,ngd->grd", probs, vals, optimize=True).reshape(heads, head_dim)
    return out


def quantize_kv_rows(rows: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """8-bit KV pages (an extension: the reference only models the byte cost of a smaller cache,
    cacheir/runtime/kv_cache.py:138-259). Each cached row [..., D] gets its own scale:
    scale = fp16(max|row| / 127) (1 for an all-zero row), byte = clip(rint(row / scale), -127, 127) + 128.
    Returns (uint8 bytes, fp16 scales [...])."""
    rows = np.asarray(rows, dtype=np.float32)
    amax = np.max(np.abs(rows), axis=-1)
    scale = (amax / np.float32(127.0)).astype(np.float16)
    scale = np.where(scale.astype(np.float32) == 0.0, np.float16(1.0), scale).astype(np.float16)
    q = np.clip(np.rint(rows / scale.astype(np.float32)[..., None]), -127, 127)
    return (q + 128).astype(np.uint8), scale


def dequantize_kv_pool(pool_u8: np.ndarray, scales: np.ndarray, which: int) -> np.ndarray:
    """[slots, kv_heads, page, D] bytes and scales [slots, kv_heads, 2, page] -> float32 values; which: 0 = K, 1 = V."""
    return (pool_u8.astype(np.float32) - np.float32(128.0)) * scales[:, :, which, :].astype(np.float32)[..., None]


# --------------------------------------------------------------------------
# Decode-graph executor (cacheir/runtime/cpu.py:82-381), one session per object
# --------------------------------------------------------------------------
def quantized_weight_inputs(nodes) -> set[str]:
    """cacheir/runtime/cpu.py:399-409."""
    names: set[str] = set()
    for node in nodes:
        if node["op"] == "quantized_matmul" and len(node["inputs"]) >= 2:
            names.add(node["inputs"][1])
        elif node["op"] == "quantized_fused_rmsnorm_qkv_rope" and len(node["inputs"]) >= 5:
            names.update(node["inputs"][2:5])
        elif node["op"] == "quantized_fused_swiglu" and len(node["inputs"]) >= 3:
            names.update(node["inputs"][1:3])
    return names


class OracleRuntime:
    """NumPy walk of a lowered decode/prefill graph, following `Runtime.run`
    and `Runtime._execute_node` (cacheir/runtime/cpu.py:111-140, 221-282).

    `graphs` maps mode -> {"nodes": [...], "weights": {value: {"key": ...}},
    "outputs": [...]} in the artifact's JSON form; `tensors` maps weight key ->
    float array. The KV cache is contiguous per layer, with page metadata kept
    alongside exactly as `PagedKVCache.append` does (kv_cache.py:66-79)."""

    def __init__(self, graphs: dict, tensors: dict[str, np.ndarray], quant: str | None, page_size: int = 16):
        self.graphs = graphs
        self.tensors = tensors
        self.quant = quant
        self.page_size = page_size
        self._cache: dict[str, np.ndarray] = {}
        self._qcache: dict[str, PackedQuantizedTensor] = {}
        self.keys: dict[int, np.ndarray] = {}
        self.values: dict[int, np.ndarray] = {}
        self.pages: dict[int, list[KVPage]] = {}
        self._next_page_id = 0

    def fork(self) -> "OracleRuntime":
        other = OracleRuntime(self.graphs, self.tensors, self.quant, self.page_size)
        other._cache, other._qcache = self._cache, self._qcache
        return other

    # WeightStore.get / get_quantized, cacheir/runtime/cpu.py:28-58
    def _get(self, graph: dict, name: str) -> np.ndarray:
        if name not in self._cache:
            tensor = np.asarray(self.tensors[graph["weights"][name]["key"]]).astype(np.float32, copy=False)
            if self.quant and tensor.ndim == 2:
                tensor = dequantize_packed_weight(self._get_quantized(graph, name))
            self._cache[name] = tensor
        return self._cache[name]

    def _get_quantized(self, graph: dict, name: str) -> PackedQuantizedTensor:
        if name not in self._qcache:
            tensor = np.asarray(self.tensors[graph["weights"][name]["key"]]).astype(np.float32, copy=False)
            packed = pack_quantized_weight(tensor, self.quant)
            if packed is None:  # cpu.py:52-56: unknown quant names fall back to an int8 pack
                packed = pack_quantized_weight(quantize_dequantize(tensor, self.quant), "int8")
            self._qcache[name] = packed
        return self._qcache[name]

    def length(self, layer: int = 0) -> int:
        return 0 if layer not in self.keys else int(self.keys[layer].shape[1])

    def clear(self) -> None:
        self.keys.clear()
        self.values.clear()
        self.pages.clear()
        self._next_page_id = 0

    def run(self, input_ids, mode: str = "prefill", reset_kv: bool | None = None) -> np.ndarray:
        graph = self.graphs[mode]
        if reset_kv is None:
            reset_kv = mode == "prefill"
        if mode == "prefill" and reset_kv:
            self.clear()
        ids = np.asarray(input_ids, dtype=np.int64)
        if ids.ndim == 1:
            ids = ids[None, :]
        env: dict[str, object] = {"input_ids": ids}
        qnames = quantized_weight_inputs(graph["nodes"])
        for name in graph["weights"]:
            env[name] = self._get_quantized(graph, name) if name in qnames else self._get(graph, name)
        for node in graph["nodes"]:
            outs = self._execute(node, env, mode)
            for name, value in zip(node["outputs"], outs):
                env[name] = value
        return env[graph["outputs"][0]]

    def _execute(self, node: dict, env: dict, mode: str) -> list[np.ndarray]:
        op, ins, attrs = node["op"], node["inputs"], node.get("attrs", {})
        if op == "token_embedding":
            return [env[ins[1]][env[ins[0]]]]
        if op == "rms_norm":
            return [rms_norm(env[ins[0]], env[ins[1]], float(attrs.get("eps", 1e-6)))]
        if op in ("matmul", "quantized_matmul"):
            return [quantized_matmul(env[ins[0]], env[ins[1]])]
        if op in ("fused_rmsnorm_qkv_rope", "quantized_fused_rmsnorm_qkv_rope"):
            x = rms_norm(env[ins[0]], env[ins[1]], float(attrs.get("eps", 1e-6)))
            q = quantized_matmul(x, env[ins[2]])
            k = quantized_matmul(x, env[ins[3]])
            v = quantized_matmul(x, env[ins[4]])
            offset = self.length(int(attrs.get("layer", 0)))
            hd, theta = int(attrs["head_dim"]), float(attrs.get("rope_theta", 10000.0))
            return [rope_one(q, hd, theta, [offset]), rope_one(k, hd, theta, [offset]), v]
        if op == "rope":
            offset = self.length(int(attrs.get("layer", 0)))
            hd, theta = int(attrs["head_dim"]), float(attrs.get("rope_theta", 10000.0))
            return [rope_one(env[ins[0]], hd, theta, [offset]), rope_one(env[ins[1]], hd, theta, [offset])]
        if op in ("paged_attention_prefill", "paged_attention_decode", "grouped_query_attention"):
            return [self._attention(env[ins[0]], env[ins[1]], env[ins[2]], attrs, mode)]
        if op == "add":
            return [env[ins[0]] + env[ins[1]]]
        if op == "silu":
            x = env[ins[0]]
            return [x / (1.0 + np.exp(-x))]
        if op == "elementwise_mul":
            return [env[ins[0]] * env[ins[1]]]
        if op in ("fused_swiglu", "quantized_fused_swiglu"):
            x = env[ins[0]]
            return [silu_mul(quantized_matmul(x, env[ins[1]]), quantized_matmul(x, env[ins[2]]))]
        raise NotImplementedError(f"oracle does not implement op {op}")

    def _attention(self, q, k, v, attrs, mode) -> np.ndarray:
        layer = int(attrs.get("layer", 0))
        heads, kv_heads, hd = int(attrs["num_heads"]), int(attrs["num_kv_heads"]), int(attrs["head_dim"])
        batch = q.shape[0]
        k_new = k.reshape(batch, k.shape[1], kv_heads, hd)
        v_new = v.reshape(batch, v.shape[1], kv_heads, hd)
        start = self.length(layer)
        if layer not in self.keys:
            self.keys[layer], self.values[layer] = k_new.copy(), v_new.copy()
        else:
            self.keys[layer] = np.concatenate([self.keys[layer], k_new], axis=1)
            self.values[layer] = np.concatenate([self.values[layer], v_new], axis=1)
        self._next_page_id = extend_pages(self.pages.setdefault(layer, []), self._next_page_id,
                                          self.page_size, start, int(k_new.shape[1]))
        return attention_contiguous(q, self.keys[layer], self.values[layer], heads, kv_heads, hd,
                                    causal=(mode == "prefill"))


def greedy_decode(runtime: OracleRuntime, prompt_ids, steps: int, vocab_size: int) -> tuple[list[int], list[np.ndarray]]:
    """Prefill + greedy loop of `Runtime.generate`, cacheir/runtime/cpu.py:162-181."""
    logits = runtime.run([list(prompt_ids)], mode="prefill")
    tokens: list[int] = []
    all_logits: list[np.ndarray] = []
    for _ in range(steps):
        all_logits.append(np.array(logits[0, -1], copy=True))
        nxt = int(np.argmax(logits[0, -1])) % vocab_size
        tokens.append(nxt)
        logits = runtime.run([[nxt]], mode="decode")
    return tokens, all_logits


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    """||a-b|| / ||b|| in float64 (b is the oracle)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = float(np.linalg.norm(b))
    return float(np.linalg.norm(a - b)) / (denom if denom > 0 else 1.0)
