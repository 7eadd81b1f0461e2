"""B200 decode runtime: drop-in for the reference's `CudaRuntime` on the batched
decode path.

`B200DecodeRuntime` exposes the duck type the reference's dispatcher,
scheduler, benchmark and server use (cacheir/runtime/cuda.py:430-714,
cacheir/runtime/scheduler.py:508-577): `run`, `fork`, `run_decode_batch`,
`run_prefill_batch`, `prefill_tokens`, `generate`, `cache_stats`,
`synchronize`, `tokenizer`, `artifact`, `kv_cache`, `prefix_cache`,
`kernel_counts`. It walks the same lowered graph and dispatches on the same
`node.op` strings (cuda.py:779-874), but:

  * every op is a hand-written sm_100a kernel called through the C ABI; there
    is no torch math, no Triton and no CPU fallback on the path;
  * the graph walk happens once per batch composition: it is lowered to a flat
    launch list over static buffers ("plan") and, after the first step,
    captured in a CUDA graph that later steps replay;
  * request state lives on the device (token ids, positions, sequence lengths,
    page table); the host only mirrors lengths and pushes page-table rows when
    a sequence crosses a page boundary;
  * K/V rows are written straight into the shared page pool, and sessions can
    alias the pages of a common prefix.
"""
from __future__ import annotations

import os

from collections import OrderedDict
from pathlib import Path
from typing import Any, Callable, Iterable

import numpy as np
import torch

from . import ops
from .artifact import CompileArtifact
from .kv_cache import B200KVPageAllocator, B200PagedKVCache, KVPoolExhausted
from .quantization import B200PackedWeight, concat_rows, quant_bits, to_tiled
from .tensor_parallel import PeerCollectives, TensorParallel, shard_columns, shard_rows
from .weights import B200WeightStore, TensorSource


def b200_runtime_available() -> bool:
    return bool(torch.cuda.is_available())


def _dtype_from_name(name: str | None) -> torch.dtype | None:
    if name in {None, "auto"}:
        return None
    table = {"float16": torch.float16, "fp16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
             "float32": torch.float32, "fp32": torch.float32}
    try:
        return table[str(name).lower()]
    except KeyError as exc:
        raise ValueError(f"Unsupported CUDA runtime dtype {name!r}") from exc


class ByteTokenizer:
    """Byte-mod tokenizer of the reference's tiny models (cacheir/runtime/tokenizer.py:7-24)."""

    def __init__(self, vocab_size: int):
        self.vocab_size = max(1, int(vocab_size))

    def encode(self, text: str) -> list[int]:
        if not isinstance(text, str):
            raise TypeError("tokenizer.encode expects a string prompt")
        data = text.encode("utf-8") or b"\x00"
        return [int(byte) % self.vocab_size for byte in data]

    def decode(self, token_ids: list[int]) -> str:
        out = []
        for token_id in token_ids:
            value = int(token_id) % self.vocab_size
            out.append(chr(value) if 32 <= value <= 126 else f"<{value}>")
        return "".join(out)


class B200PrefixCache:
    """LRU of reusable prompt prefixes, keyed by token tuple like the reference's
    `PrefixCache` (cacheir/runtime/kv_cache.py:262-307), but an entry holds
    references to the prefix's full KV pages instead of a copy of the tensors."""

    def __init__(self, allocator: B200KVPageAllocator, num_layers: int, capacity: int = 8):
        self.capacity = max(1, int(capacity))
        self.allocator = allocator
        self.num_layers = num_layers
        self._entries: OrderedDict[tuple[int, ...], B200PagedKVCache] = OrderedDict()
        self.hits = self.misses = self.evictions = 0

    def put(self, token_ids, cache: B200PagedKVCache) -> None:
        page = cache.page_size
        key = tuple(int(t) for t in token_ids)[: (min(len(token_ids), cache.tokens) // page) * page]
        if not key:
            return
        if key in self._entries:
            self._entries.pop(key).clear()
        holder = B200PagedKVCache(self.allocator, self.num_layers)
        holder.share_prefix(cache, len(key))
        self._entries[key] = holder
        while len(self._entries) > self.capacity:
            _, old = self._entries.popitem(last=False)
            old.clear()
            self.evictions += 1

    def longest_prefix(self, token_ids) -> tuple[tuple[int, ...], B200PagedKVCache | None]:
        query = tuple(int(t) for t in token_ids)
        best_key: tuple[int, ...] = ()
        best = None
        for key, value in self._entries.items():
            if len(key) > len(best_key) and query[: len(key)] == key:
                best_key, best = key, value
        if best is not None:
            self._entries.move_to_end(best_key)
            self.hits += 1
        else:
            self.misses += 1
        return best_key, best

    def stats(self) -> dict[str, int]:
        return {"capacity": self.capacity, "entries": len(self._entries), "hits": self.hits,
                "misses": self.misses, "evictions": self.evictions}


class _Engine:
    """State shared by every fork of a runtime: weights, page pools, plans."""

    def __init__(self, artifact: Any, *, device: torch.device, dtype: torch.dtype, weights: B200WeightStore | None,
                 tensor_source: Any, kv_allocator: B200KVPageAllocator | None, max_seq_len: int | None,
                 use_cuda_graph: bool, attention_splits: int, max_plans: int, tensor_parallel: TensorParallel | None = None,
                 kv_dtype: str = "same", fuse_attention_prepass: bool = True):
        self.artifact = artifact
        self.fuse_attention_prepass = bool(fuse_attention_prepass)   # attention writes the next projection's activation planes
        self.tp = tensor_parallel or TensorParallel(0, 1)
        self.device = device
        self.dtype = dtype
        self.graph = artifact.graph("decode")
        self.config = artifact.config
        self.quant = artifact.quant
        if self.quant and quant_bits(self.quant) is None:
            raise ValueError(f"Unsupported quantization mode {self.quant!r}")
        source = tensor_source if tensor_source is not None else artifact.model_path
        self.weights = weights or B200WeightStore(TensorSource(source), self.graph.weights, self.quant,
                                                  device=device, dtype=dtype)
        hints = self.graph.attrs.get("execution_hints", {}) if isinstance(self.graph.attrs, dict) else {}
        self.page_size = int(hints.get("page_size", 16))
        self.allocator = kv_allocator or B200KVPageAllocator(page_size=self.page_size)
        if self.allocator.page_size != self.page_size:
            raise ValueError("kv_allocator page_size differs from the artifact's decode page size")
        self.tp.check_model(heads=int(self.config.num_attention_heads), kv_heads=int(self.config.num_key_value_heads),
                            intermediate=int(self.config.intermediate_size), vocab=int(self.config.vocab_size))
        # under tensor parallelism a rank's pool holds only its own KV heads
        self.allocator.configure(torch=torch, device=device, dtype=dtype, num_layers=int(self.config.num_layers),
                                 kv_heads=int(self.config.num_key_value_heads) // self.tp.world,
                                 head_dim=int(self.config.head_dim), kv_dtype=kv_dtype)
        self.max_seq_len = int(max_seq_len or self.config.max_position_embeddings)
        # Tensor-parallel collectives: this package's own kernels over peer memory (graph-capturable), or the
        # process group's library collectives launched eagerly (CB200_TP_COLLECTIVES=nccl; never captured).
        self.peer_mode = self.tp.enabled and os.environ.get("CB200_TP_COLLECTIVES", "peer") != "nccl"
        self.peer: PeerCollectives | None = None
        self.use_cuda_graph = use_cuda_graph and (not self.tp.enabled or self.peer_mode)
        self.tile_weights = True
        self.validated_batch: tuple[int, ...] | None = None      # identity of the last decode batch that passed the checks
        self.validated_sessions: list[Any] = []
        self.prefill_chunk = 64        # prompt tokens per pass of the chunked prefill (0: one token per step)
        self._rope_tables: dict[tuple[int, float], torch.Tensor] = {}
        self.attention_splits = int(attention_splits)
        self.max_plans = max(1, int(max_plans))
        self.plans: OrderedDict[tuple, "_DecodePlan"] = OrderedDict()
        self.plans_lowered = 0          # decode graphs lowered to launch lists so far
        self.graph_captures = 0         # CUDA graphs captured so far
        self.kernel_counts: OrderedDict[str, int] = OrderedDict()
        self.gemm_plans: OrderedDict[str, str] = OrderedDict()
        self.fused_weights: dict[tuple[str, ...], B200PackedWeight | torch.Tensor] = {}
        self.prefix_cache = B200PrefixCache(self.allocator, int(self.config.num_layers))
        self.tokenizer = ByteTokenizer(int(self.config.vocab_size))

    def count(self, name: str, n: int = 1) -> None:
        self.kernel_counts[name] = self.kernel_counts.get(name, 0) + n

    # -- weights as the kernels want them -------------------------------------------
    def matmul_weight(self, names: tuple[str, ...], quantized: bool, batch: int = 1,
                      role: str = "column") -> B200PackedWeight | torch.Tensor:
        """One (row-concatenated) weight for a matmul-family node: packed when the
        node is a quantized op, dense [N, K] otherwise (cuda.py:1017-1023 caches the
        same concatenation for its unquantized fused ops). (Batches beyond the tensor-core
        kernels' 64 rows are run by the library as 64-row chunks, so the tile order serves them too.)
        `role` says how tensor parallelism slices it: "column" (output rows, each fused
        part separately so a rank keeps whole heads / matching gate and up rows), "row"
        (the input dimension) or "replicated"."""
        if names in self.fused_weights:
            return self.fused_weights[names]

        def shard(w):
            if not self.tp.enabled or role == "replicated":
                return w
            return shard_rows(w, self.tp) if role == "column" else shard_columns(w, self.tp)

        if quantized:
            parts = [shard(self.weights.get_quantized(n)) for n in names]
            fused = parts[0] if len(parts) == 1 else concat_rows(parts)
            if len(parts) > 1 or self.tp.enabled:   # the concatenation / shard replaces the parts: keep one copy of the codes in HBM
                for n in names:
                    self.weights.release(n)
            # device pack layout: tile order for the tensor-core kernels (fp16 activations, K a multiple of 128).
            # A gate|up pair of per-row int8 weights takes the paired form (64 gate + 64 up rows per tile) that the
            # integer kernel's SwiGLU epilogue reads; any other pair needs each half to be whole 128-row bands.
            pair = len(names) == 2
            half = fused.shape[0] // 2
            paired = pair and fused.bits in (4, 8) and not fused.group_size and half % 64 == 0
            halves_ok = not pair or paired or half % 128 == 0
            if self.dtype == torch.float16 and fused.shape[1] % 128 == 0 and halves_ok and self.tile_weights:
                tiled = to_tiled(fused, paired=paired)
                if len(parts) == 1:
                    self.weights.release(names[0])
                fused = tiled
        else:
            dense = [shard(self.weights.get(n)) for n in names]
            fused = dense[0] if len(dense) == 1 else torch.cat(dense, dim=0).contiguous()
            if len(dense) > 1:
                for n in names:
                    self.weights.release(n)
        self.fused_weights[names] = fused
        return fused

    def peer_collectives(self, rows: int) -> PeerCollectives:
        """The peer-memory buffers, sized on first use for up to max(rows, 256) batch rows."""
        if self.peer is None:
            widest = max(int(self.config.hidden_size), int(self.config.vocab_size) // self.tp.world)
            elem = torch.empty((), dtype=self.dtype).element_size()
            self.peer = PeerCollectives(self.tp, self.device, max(rows, 256) * widest * elem)
        return self.peer

    def rope_table(self, head_dim: int, theta: float) -> torch.Tensor:
        """(cos, sin) for every position up to max_seq_len, shared by all plans and layers."""
        key = (int(head_dim), float(theta))
        if key not in self._rope_tables:
            self._rope_tables[key] = ops.rope_table(self.max_seq_len, head_dim, theta, self.device)
        return self._rope_tables[key]

    def prefill_plan(self, rows: int, needed_pages: int) -> "_DecodePlan":
        """The plan that pushes `rows` prompt tokens through the decode graph at once: row i is one (sequence,
        position) pair, reads that sequence's page table and attends to position+1 tokens."""
        key = ("prefill", rows)
        plan = self.plans.get(key)
        if plan is not None and (plan.pool_generation != self.allocator.generation or plan.width < needed_pages):
            self.plans.pop(key)
            plan = None
        if plan is None:
            width = max(needed_pages, (self.max_seq_len + self.page_size - 1) // self.page_size)
            plan = _DecodePlan(self, rows, width)
            self.plans_lowered += 1
            self.plans[key] = plan
            while len(self.plans) > self.max_plans:
                self.plans.popitem(last=False)
        else:
            self.plans.move_to_end(key)
        return plan

    def plan_for(self, sessions: list["B200DecodeRuntime"]) -> "_DecodePlan":
        """The plan for a decode batch of this size. Plans are keyed by batch size, not by who is in the batch:
        a session is bound to a row for one step only, and `sync_sessions` rewrites the rows whose occupant,
        length or page list changed. Admitting or retiring a request therefore costs a few small copies, not
        a new lowering and a new CUDA-graph capture."""
        key = ("decode", len(sessions))
        plan = self.plans.get(key)
        needed_pages = max((s.kv_cache.tokens + 1 + self.page_size - 1) // self.page_size for s in sessions)
        if plan is not None and (plan.pool_generation != self.allocator.generation or plan.width < needed_pages):
            self.plans.pop(key)
            plan = None
        if plan is None:
            width = max(needed_pages, (self.max_seq_len + self.page_size - 1) // self.page_size)
            plan = _DecodePlan(self, len(sessions), width)
            self.plans_lowered += 1
            self.plans[key] = plan
            while len(self.plans) > self.max_plans:
                self.plans.popitem(last=False)
        else:
            self.plans.move_to_end(key)
        return plan


class _DecodePlan:
    """Static device buffers and the flat launch list of one decode step for a
    fixed batch size; optionally a CUDA graph of that list."""

    def __init__(self, engine: _Engine, batch: int, width: int):
        self.engine = engine
        self.batch = batch
        self.width = width
        self.pool_generation = engine.allocator.generation
        dev = engine.device
        self.ids = torch.zeros((batch,), device=dev, dtype=torch.int64)
        self.positions = torch.zeros((batch,), device=dev, dtype=torch.int32)
        self.seq_lens = torch.zeros((batch,), device=dev, dtype=torch.int32)
        self.page_table = torch.zeros((batch, width), device=dev, dtype=torch.int32)
        self.host_ids = torch.zeros((batch,), dtype=torch.int64).pin_memory()
        self.host_lens = torch.zeros((batch,), dtype=torch.int32).pin_memory()
        self.host_table = torch.zeros((batch, width), dtype=torch.int32).pin_memory()
        self.synced_owner_state: list[tuple[str, int, int, int]] | None = None
        self.repeat_key: tuple | None = None     # the session list whose next steps need only new token ids (see _repeat_step)
        self.repeat_tokens: list[int] = []
        self.repeat_left = 0
        self.repeat_version = -1
        self.program: list[Callable[[], None]] = []
        self.launches_per_step = 0
        self.cuda_graph: torch.cuda.CUDAGraph | None = None
        self.feedback_graph: torch.cuda.CUDAGraph | None = None
        self.h2d_done = torch.cuda.Event()
        self.steps_run = 0
        self.logits: torch.Tensor | None = None
        self._lower()

    # -- graph lowering --------------------------------------------------------------
    def _emit(self, fn: Callable[[], None], count_key: str, launches: int = 1) -> None:
        self.program.append(fn)
        self.launches_per_step += launches
        self._count_keys.append((count_key, 1))

    def _buf(self, cols: int) -> torch.Tensor:
        return torch.empty((self.batch, cols), device=self.engine.device, dtype=self.engine.dtype)

    def _lower(self) -> None:
        eng = self.engine
        nodes = list(eng.graph.nodes)
        env: dict[str, Any] = {}
        self._count_keys: list[tuple[str, int]] = []
        self._count_totals: dict[str, int] | None = None
        self._prequantized: set[str] = set()
        self._kv_appended: set[str] = set()
        self._peer_calls = 0
        self._peer_gathers = 0
        uses: dict[str, int] = {}
        for node in nodes:
            for name in node.inputs:
                uses[name] = uses.get(name, 0) + 1
        for name in eng.graph.outputs:
            uses[name] = uses.get(name, 0) + 1

        if eng.dtype == torch.float16 and eng.quant:
            widest = max(int(eng.config.hidden_size), int(eng.config.intermediate_size))
            self._gemm_ws = torch.zeros((ops.qgemv_workspace_bytes(self.batch, widest),), device=eng.device, dtype=torch.uint8)
        self._emit(lambda: ops.advance_positions(self.positions, self.seq_lens), "b200.advance_positions")
        skip: set[int] = set()
        for idx, node in enumerate(nodes):
            if idx in skip:
                continue
            op = node.op
            attrs = node.attrs
            if op == "token_embedding":
                table = eng.weights.get(node.inputs[1])
                out = self._buf(int(table.shape[1]))
                self._emit(lambda table=table, out=out: ops.embedding_gather(table, self.ids, out), "b200.embedding_gather")
                env[node.outputs[0]] = out
            elif op == "rms_norm":
                x, w = env[node.inputs[0]], eng.weights.get(node.inputs[1])
                eps = float(attrs.get("eps", 1e-6))
                nxt = nodes[idx + 1] if idx + 1 < len(nodes) else None
                fused = False
                if (nxt is not None and nxt.op in {"quantized_matmul", "quantized_fused_swiglu"}
                        and nxt.inputs[0] == node.outputs[0] and uses.get(node.outputs[0], 0) == 1):
                    names = (nxt.inputs[1],) if nxt.op == "quantized_matmul" else tuple(nxt.inputs[1:3])
                    if self._i8_eligible(eng.matmul_weight(names, True, self.batch), int(x.shape[1]), swiglu=len(names) == 2):
                        ws = self._gemm_workspace(int(x.shape[1]))
                        self._emit(lambda x=x, w=w, eps=eps, ws=ws: ops.rms_norm_quantize(x, w, eps, ws), "b200.rms_norm_quantize")
                        env[node.outputs[0]] = x            # placeholder: the consumer reads the workspace, not this tensor
                        self._prequantized.add(node.outputs[0])
                        fused = True
                if not fused:
                    out = self._buf(int(x.shape[1]))
                    self._emit(lambda x=x, w=w, out=out, eps=eps: ops.rms_norm(x, w, eps, out=out), "b200.rms_norm")
                    env[node.outputs[0]] = out
            elif op in {"matmul", "quantized_matmul"}:
                x = env[node.inputs[0]]
                tp = eng.tp
                projection = attrs.get("projection")
                role = "replicated"
                if tp.enabled:   # o / down consume a rank-local activation slice; lm_head produces a vocabulary slice
                    role = {"o": "row", "down": "row", "lm_head": "column"}.get(projection, "replicated")
                    if role == "replicated":
                        # a stand-alone q / k / v / gate / up projection would stay full width while attention, the cache
                        # append and the row-parallel projections work on this rank's heads and columns only
                        raise NotImplementedError(
                            f"tensor parallelism needs the fused graph (fused QKV and SwiGLU ops): found a separate matmul "
                            f"{node.name or node.outputs[0]!r} with projection {projection!r}")
                weight = eng.matmul_weight((node.inputs[1],), op == "quantized_matmul", self.batch, role)
                out_name = node.outputs[0]
                nxt = nodes[idx + 1] if idx + 1 < len(nodes) else None
                residual = None
                if (nxt is not None and nxt.op == "add" and out_name in nxt.inputs and uses.get(out_name, 0) == 1
                        and nxt.inputs[0] != nxt.inputs[1]):
                    other = nxt.inputs[0] if nxt.inputs[1] == out_name else nxt.inputs[1]
                    # a row-parallel projection yields partial sums: the residual joins on rank 0 only
                    residual = env[other] if (role != "row" or tp.rank == 0) else None
                    skip.add(idx + 1)
                    out_name = nxt.outputs[0]
                peer = eng.peer_collectives(self.batch) if (role != "replicated" and eng.peer_mode) else None
                n_local = int(weight.shape[0])
                if peer is not None and role == "row":
                    # partial sums go straight into a peer-visible buffer (A and B alternate), one kernel sums all ranks
                    which = self._peer_calls % 2
                    self._peer_calls += 1
                    partial = peer.buffer(which, self.batch, n_local, eng.dtype)
                    self._matmul(x, weight, residual=residual, prequantized=node.inputs[0] in self._prequantized, out=partial)
                    out = self._buf(n_local)
                    self._emit(lambda out=out, which=which: peer.all_reduce(which, out), "b200.peer_all_reduce")
                elif peer is not None and role == "column":
                    local = peer.buffer(2, self.batch, n_local, eng.dtype)
                    self._matmul(x, weight, residual=residual, prequantized=node.inputs[0] in self._prequantized, out=local)
                    out = self._buf(n_local * tp.world)
                    self._emit(lambda out=out: peer.all_gather_columns(2, out), "b200.peer_all_gather")
                    self._peer_gathers += 1
                else:
                    out = self._matmul(x, weight, residual=residual, prequantized=node.inputs[0] in self._prequantized)
                    if role == "row":
                        self._emit(lambda out=out: tp.all_reduce_sum(out), "b200.tp.all_reduce", launches=0)
                    elif role == "column":
                        local = out
                        out = self._buf(n_local * tp.world)
                        gathered = torch.empty((tp.world * self.batch, n_local), device=eng.device, dtype=eng.dtype)
                        self._emit(lambda local=local, gathered=gathered, out=out: tp.all_gather_columns(local, gathered, out),
                                   "b200.tp.all_gather", launches=0)
                env[out_name] = out
            elif op in {"fused_rmsnorm_qkv_rope", "quantized_fused_rmsnorm_qkv_rope"}:
                x, norm_w = env[node.inputs[0]], eng.weights.get(node.inputs[1])
                weight = eng.matmul_weight(tuple(node.inputs[2:5]), op.startswith("quantized_"), self.batch)
                eps = float(attrs.get("eps", 1e-6))
                q_dim = self._rows_of(node.inputs[2]) // eng.tp.world      # whole heads per rank
                k_dim = self._rows_of(node.inputs[3]) // eng.tp.world
                head_dim = int(attrs["head_dim"])
                theta = float(attrs.get("rope_theta", 10000.0))
                consumer = self._attention_consumer(nodes, idx, node)
                if self._i8_eligible(weight, int(x.shape[1])):
                    ws = self._gemm_workspace(int(x.shape[1]))
                    self._emit(lambda x=x, w=norm_w, eps=eps, ws=ws: ops.rms_norm_quantize(x, w, eps, ws), "b200.rms_norm_quantize")
                    pool = eng.allocator.pool_for_layer(int(consumer.attrs.get("layer", 0))) if consumer is not None else None
                    if (pool is not None and weight.bits == 8 and self._rows_of(node.inputs[4]) // eng.tp.world == k_dim and pool["keys"].dtype == torch.float16
                            and int(pool["keys"].shape[3]) == head_dim and int(pool["keys"].shape[1]) * head_dim == k_dim):
                        # projection + RoPE + append of the new k/v rows in one kernel
                        n, k = weight.shape
                        qkv = self._buf(n)
                        table = eng.rope_table(head_dim, theta)
                        k_pool, v_pool = pool["keys"], pool["values"]
                        self._emit(lambda qkv=qkv, weight=weight, n=n, k=k, ws=ws, table=table, k_pool=k_pool, v_pool=v_pool:
                                   ops.qkv_rope_append(None, weight.packed_values, weight.scales, weight.zero_points, qkv, n=n, k=k,
                                                       q_dim=q_dim, k_dim=k_dim, head_dim=head_dim, theta=theta, table=table,
                                                       positions=self.positions, page_table=self.page_table, k_cache=k_pool,
                                                       v_cache=v_pool, workspace=ws, tiled=weight.tiled, prequantized=True),
                                   "b200.qkv_rope_append")
                        eng.gemm_plans[f"q8:{(self.batch, 1, k)}x{weight.shape}"] = "b200.qkv_rope_append"
                        self._kv_appended.add(node.outputs[1])
                        env[node.outputs[0]] = qkv[:, :q_dim]
                        env[node.outputs[1]] = qkv[:, q_dim:q_dim + k_dim]
                        env[node.outputs[2]] = qkv[:, q_dim + k_dim:]
                        continue
                    qkv = self._matmul(x, weight, prequantized=True)
                else:
                    normed = self._buf(int(x.shape[1]))
                    self._emit(lambda x=x, w=norm_w, out=normed, eps=eps: ops.rms_norm(x, w, eps, out=out), "b200.rms_norm")
                    qkv = self._matmul(normed, weight)
                pool = eng.allocator.pool_for_layer(int(consumer.attrs.get("layer", 0))) if consumer is not None else None
                if (pool is not None and "scales" not in pool and pool["keys"].dtype == qkv.dtype and int(pool["keys"].shape[3]) == head_dim
                        and int(pool["keys"].shape[1]) * head_dim == k_dim and int(qkv.shape[1]) == q_dim + 2 * k_dim):
                    # RoPE on q|k and the append of the new k / v rows in one launch
                    k_pool, v_pool = pool["keys"], pool["values"]
                    self._emit(lambda qkv=qkv, k_pool=k_pool, v_pool=v_pool, hd=head_dim, theta=theta:
                               ops.rope_append(qkv, self.positions, self.page_table, k_pool, v_pool, q_dim=q_dim, k_dim=k_dim,
                                               head_dim=hd, theta=theta), "b200.rope_append")
                    self._kv_appended.add(node.outputs[1])
                else:
                    qk = qkv[:, : q_dim + k_dim]   # q and k heads are adjacent: one RoPE launch covers both
                    self._emit(lambda qk=qk, hd=head_dim, theta=theta, nh=(q_dim + k_dim) // head_dim:
                               ops.rope_inplace(qk, self.positions, num_heads=nh, head_dim=hd, theta=theta), "b200.rope")
                env[node.outputs[0]] = qkv[:, :q_dim]
                env[node.outputs[1]] = qkv[:, q_dim:q_dim + k_dim]
                env[node.outputs[2]] = qkv[:, q_dim + k_dim:]
            elif op == "qkv_projection":
                if eng.tp.enabled:
                    raise NotImplementedError("tensor parallelism needs the fused graph: qkv_projection is not sharded")
                x = env[node.inputs[0]]
                for w_name, out_name in zip(node.inputs[1:4], node.outputs[:3]):
                    env[out_name] = self._matmul(x, eng.matmul_weight((w_name,), False))
            elif op == "rope":
                head_dim = int(attrs["head_dim"])
                theta = float(attrs.get("rope_theta", 10000.0))
                for in_name, out_name in zip(node.inputs[:2], node.outputs[:2]):
                    t = env[in_name]
                    self._emit(lambda t=t, hd=head_dim, theta=theta:
                               ops.rope_inplace(t, self.positions, num_heads=int(t.shape[1]) // hd, head_dim=hd, theta=theta),
                               "b200.rope")
                    env[out_name] = t
            elif op in {"paged_attention_decode", "grouped_query_attention"}:
                # The projection behind the attention: when it runs on the integer tensor cores, the attention kernel
                # itself can leave the activation planes it needs (no pre-pass launch in between).
                nxt = nodes[idx + 1] if idx + 1 < len(nodes) else None
                quant_ws = None
                if (nxt is not None and nxt.op == "quantized_matmul" and nxt.inputs[0] == node.outputs[0]
                        and uses.get(node.outputs[0], 0) == 1 and eng.fuse_attention_prepass and not eng.tp.enabled):
                    # (single GPU only: under tensor parallelism the o projection keeps its own pre-pass)
                    k_total = int(attrs["num_heads"]) * int(attrs["head_dim"])
                    if (self._i8_eligible(eng.matmul_weight((nxt.inputs[1],), True, self.batch, "replicated"), k_total)
                            and ops.qgemv_workspace_bytes(self.batch, k_total) <= self._gemm_ws.numel()):   # (never grows it here)
                        quant_ws = self._gemm_workspace(k_total)
                out, fused = self._attention(env[node.inputs[0]], env[node.inputs[1]], env[node.inputs[2]], attrs,
                                             appended=node.inputs[1] in self._kv_appended, quant_ws=quant_ws)
                env[node.outputs[0]] = out
                if fused:
                    self._prequantized.add(node.outputs[0])
            elif op == "add":
                a, b = env[node.inputs[0]], env[node.inputs[1]]
                out = self._buf(int(a.shape[1]))
                self._emit(lambda a=a, b=b, out=out: ops.add(a, b, out), "b200.add")
                env[node.outputs[0]] = out
            elif op in {"fused_swiglu", "quantized_fused_swiglu"}:
                x = env[node.inputs[0]]
                weight = eng.matmul_weight(tuple(node.inputs[1:3]), op.startswith("quantized_"), self.batch)
                env[node.outputs[0]] = self._matmul(x, weight, epilogue=ops.EPI_SWIGLU,
                                                    prequantized=node.inputs[0] in self._prequantized)
            elif op == "elementwise_mul" and idx > 0 and nodes[idx - 1].op == "silu" and nodes[idx - 1].outputs[0] in node.inputs:
                gate = env["__silu_in__" + nodes[idx - 1].outputs[0]]
                up = env[node.inputs[1] if node.inputs[0] == nodes[idx - 1].outputs[0] else node.inputs[0]]
                out = self._buf(int(gate.shape[1]))
                self._emit(lambda g=gate, u=up, out=out: ops.silu_mul(g, u, out), "b200.silu_mul")
                env[node.outputs[0]] = out
            elif op == "silu" and idx + 1 < len(nodes) and nodes[idx + 1].op == "elementwise_mul":
                env["__silu_in__" + node.outputs[0]] = env[node.inputs[0]]
            elif op == "paged_attention_prefill":
                raise NotImplementedError("the B200 runtime executes the decode graph; prefill runs as decode steps")
            else:
                raise NotImplementedError(f"B200 decode runtime does not implement op {op}")
        if self._peer_calls % 2 == 1 and self._peer_gathers == 0:
            # consecutive steps would refill the same peer buffer with no other call in between
            raise NotImplementedError("an odd number of row-parallel projections per step needs a gather (or a third buffer) between steps")
        logits = env[eng.graph.outputs[0]]
        self.logits = logits
        # Greedy feedback variant: the row argmax overwrites `ids` (already consumed by the
        # embedding gather of this step), so the next replay needs nothing from the host.
        self.feedback_tail = lambda: ops.argmax_rows(logits, self.ids)

    def _rows_of(self, weight_name: str) -> int:
        spec = self.engine.graph.weights[weight_name]
        shape = getattr(spec, "shape", None) or spec.tensor_type.shape
        return int(shape[0])

    def _i8_eligible(self, weight: Any, k: int, swiglu: bool = False) -> bool:
        """Will this projection run on the integer tensor cores (and so accept pre-quantized activations)?"""
        if swiglu and isinstance(weight, B200PackedWeight) and ((weight.shape[0] // 2) % 64 != 0 or (weight.tiled and not weight.paired)):
            return False
        return (isinstance(weight, B200PackedWeight) and weight.bits in (4, 8) and not weight.group_size
                and self.engine.dtype == torch.float16 and self.batch <= 64 and k % 128 == 0 and k <= 8192
                and hasattr(self, "_gemm_ws"))

    def _matmul(self, x: torch.Tensor, weight: B200PackedWeight | torch.Tensor, *, epilogue: int = ops.EPI_NONE,
                residual: torch.Tensor | None = None, prequantized: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
        eng = self.engine
        if residual is not None:
            epilogue = ops.EPI_RESIDUAL
        if isinstance(weight, B200PackedWeight):
            n, k, bits = weight.shape[0], weight.shape[1], weight.bits
            out = out if out is not None else self._buf(n // 2 if epilogue == ops.EPI_SWIGLU else n)
            ws = self._gemm_workspace(k) if (bits in (4, 8) and not weight.group_size and eng.dtype == torch.float16) else None
            fn = lambda: ops.qgemv(x, weight.packed_values, weight.scales, weight.zero_points, bits=bits, n=n, k=k,
                                   group_size=weight.group_size or 0, epilogue=epilogue, residual=residual, out=out,
                                   workspace=ws, tiled=weight.tiled, prequantized=prequantized, paired=weight.paired)
            key = f"b200.qgemv.int{bits}" + (".swiglu" if epilogue == ops.EPI_SWIGLU else ".residual" if residual is not None else "")
            eng.gemm_plans[f"q{bits}:{(self.batch, 1, k)}x{weight.shape}"] = key
            if ws is not None and k % 128 == 0 and k <= 32768 and not prequantized:   # activation pre-pass + integer GEMM per 64-row chunk
                self._emit(fn, key, launches=2 * ((self.batch + 63) // 64))
                return out
        else:
            n, k = int(weight.shape[0]), int(weight.shape[1])
            out = out if out is not None else self._buf(n // 2 if epilogue == ops.EPI_SWIGLU else n)
            fn = lambda: ops.qgemv(x, weight, None, None, bits=0, n=n, k=k, epilogue=epilogue, residual=residual, out=out)
            key = "b200.gemv.dense" + (".swiglu" if epilogue == ops.EPI_SWIGLU else ".residual" if residual is not None else "")
            eng.gemm_plans[f"{(self.batch, 1, k)}x{(n, k)}"] = key
        self._emit(fn, key)
        return out

    def _gemm_workspace(self, k: int) -> torch.Tensor:
        """Scratch for the integer tensor-core GEMM (activation bytes); one buffer per plan, sized for
        the widest input, reused by every projection of the step (they run back to back on one stream)."""
        need = ops.qgemv_workspace_bytes(self.batch, k)
        ws = getattr(self, "_gemm_ws", None)
        if ws is None or ws.numel() < need:
            if ws is not None and self.program:
                raise RuntimeError("GEMM workspace must be sized before the first projection is lowered")
            self._gemm_ws = ws = torch.zeros((need,), device=self.engine.device, dtype=torch.uint8)
        return ws

    @staticmethod
    def _attention_consumer(nodes: list[Any], idx: int, node: Any) -> Any | None:
        """The decode-attention node that takes this node's q, k, v outputs (and so owns the cache append)."""
        for later in nodes[idx + 1:]:
            if later.op in {"paged_attention_decode", "grouped_query_attention"} and list(later.inputs[:3]) == list(node.outputs[:3]):
                return later
        return None

    def _attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, attrs: dict[str, Any], *,
                   appended: bool = False, quant_ws: torch.Tensor | None = None) -> tuple[torch.Tensor, bool]:
        """Emits the cache append (unless the QKV kernel did it) and the attention launch; returns the output and
        whether the launch also left it in `quant_ws` as the next projection's activation planes."""
        eng = self.engine
        layer = int(attrs.get("layer", 0))
        heads, kv_heads, head_dim = int(attrs["num_heads"]), int(attrs["num_kv_heads"]), int(attrs["head_dim"])
        heads, kv_heads = heads // eng.tp.world, kv_heads // eng.tp.world      # this rank's heads
        pool = eng.allocator.pool_for_layer(layer)
        if pool is None:
            raise RuntimeError(f"no KV page pool for layer {layer}")
        k_pool, v_pool, kv_scales = pool["keys"], pool["values"], pool.get("scales")
        out = self._buf(heads * head_dim)
        q3 = q.as_strided((self.batch, heads, head_dim), (q.stride(0), head_dim, 1), q.storage_offset())
        out3 = out.view(self.batch, heads, head_dim)
        splits = eng.attention_splits or ops.attention_auto_splits(self.batch, heads, kv_heads, self.width,
                                                                  eng.page_size, head_dim)
        ws_bytes = ops.attention_workspace_bytes(self.batch, heads, head_dim, splits)
        if not hasattr(self, "_attn_ws") or self._attn_ws.numel() * 4 < ws_bytes:
            self._attn_ws = torch.empty((max(1, (ws_bytes + 3) // 4),), device=eng.device, dtype=torch.float32)
        ws = self._attn_ws if ws_bytes else None
        if not appended:   # (the fused QKV kernel has already written the new rows)
            if kv_scales is not None:
                self._emit(lambda: ops.kv_append_q8(k, v, k_pool, v_pool, kv_scales, self.page_table, self.positions), "b200.kv_append_q8")
            else:
                self._emit(lambda: ops.kv_append(k, v, k_pool, v_pool, self.page_table, self.positions), "b200.kv_append")
        if (quant_ws is not None and splits == 1 and kv_scales is None
                and ops.attention_quantize_supported(self.batch, heads, kv_heads, self.width, eng.page_size, head_dim, out.dtype)):
            self._emit(lambda: ops.paged_attention_decode_batch_quantize(q3, k_pool, v_pool, self.page_table, self.seq_lens,
                                                                         out=out3, gemm_workspace=quant_ws),
                       "b200.paged_attention_decode_batch.persistent_shared")
            eng.count("b200.attention_prepass_fused")         # attention launches lowered in the fused form
            return out, True
        self._emit(lambda: ops.paged_attention_decode_batch(q3, k_pool, v_pool, self.page_table, self.seq_lens, out=out3,
                                                            num_splits=splits, workspace=ws, kv_scales=kv_scales),
                   "b200.paged_attention_decode_batch.persistent_shared", launches=2 if splits > 1 else 1)
        return out, False

    # -- stepping --------------------------------------------------------------------
    def sync_sessions(self, sessions: list["B200DecodeRuntime"]) -> None:
        """Make the device copy of lengths and page tables match the host bookkeeping
        (which already accounts for the token about to be decoded)."""
        state = [(s.kv_cache.owner_id, s.kv_cache.tokens, len(s.kv_cache.pages), s.kv_cache.epoch) for s in sessions]
        previous = self.synced_owner_state
        lens_ok = previous is not None and all(p[0] == c[0] and p[3] == c[3] and p[1] + 1 == c[1] for p, c in zip(previous, state))
        pages_ok = previous is not None and all(p[0] == c[0] and p[3] == c[3] and p[2] == c[2] for p, c in zip(previous, state))
        self.h2d_done.synchronize()   # the pinned staging buffers must not change under a pending copy
        if not pages_ok:
            table = self.host_table.numpy()
            for row, s in enumerate(sessions):
                table[row] = s.kv_cache.page_table_row(self.width)
            self.page_table.copy_(self.host_table, non_blocking=True)
        if not lens_ok:
            lens = self.host_lens.numpy()
            for row, s in enumerate(sessions):
                lens[row] = s.kv_cache.tokens - 1   # the step itself advances the device copy by one
            self.seq_lens.copy_(self.host_lens, non_blocking=True)
        self.synced_owner_state = state

    def sync_prefill_rows(self, rows: list[tuple[B200PagedKVCache, int, int]]) -> None:
        """Row r of the pass is the prompt token `rows[r] = (cache, position, token id)`: it reads that sequence's
        page table, appends its K/V row at `position` and attends to `position + 1` tokens. Rows may belong to
        different sequences; rows of one sequence see each other's K/V through the pool (all rows append before
        any row attends). Rows beyond the list repeat the last entry (same position, same values: harmless
        duplicates). The pages of every position must already be reserved."""
        n = len(rows)
        self.h2d_done.synchronize()
        ids = self.host_ids.numpy()
        lens = self.host_lens.numpy()
        table = self.host_table.numpy()
        cached_rows: dict[int, np.ndarray] = {}
        for row in range(self.batch):
            cache, position, token = rows[min(row, n - 1)]
            ids[row] = int(token)
            lens[row] = int(position)            # the step turns this into position and length position + 1
            key = id(cache)
            if key not in cached_rows:
                cached_rows[key] = cache.page_table_row(self.width)
            table[row] = cached_rows[key]
        self.ids.copy_(self.host_ids, non_blocking=True)
        self.seq_lens.copy_(self.host_lens, non_blocking=True)
        self.page_table.copy_(self.host_table, non_blocking=True)
        self.h2d_done.record()
        self.synced_owner_state = None
        self.repeat_left = 0            # the device rows now belong to this pass

    def sync_prefill_chunk(self, cache: B200PagedKVCache, start: int, token_ids: list[int]) -> None:
        """Rows 0..n-1 are the tokens at positions start..start+n-1 of one sequence."""
        self.sync_prefill_rows([(cache, start + i, int(t)) for i, t in enumerate(token_ids)])

    def run_program(self, *, feedback: bool = False) -> None:
        """One decode step: eager launches on the first step, CUDA-graph replay afterwards."""
        eng = self.engine
        if eng.use_cuda_graph and self.steps_run >= 1:
            attr = "feedback_graph" if feedback else "cuda_graph"
            graph = getattr(self, attr)
            if graph is None:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for fn in self.program:
                        fn()
                    if feedback:
                        self.feedback_tail()
                setattr(self, attr, graph)
                eng.graph_captures += 1
            graph.replay()
        else:
            for fn in self.program:
                fn()
            if feedback:
                self.feedback_tail()
        self.steps_run += 1
        if self._count_totals is None:      # launches per kernel name of one step, summed once
            totals: dict[str, int] = {}
            for key, n in self._count_keys:
                totals[key] = totals.get(key, 0) + n
            self._count_totals = totals
        for key, n in self._count_totals.items():
            eng.count(key, n)
        if feedback:
            eng.count("b200.argmax_rows")

    def run_feedback_steps(self, steps: int) -> torch.Tensor:
        """`steps` greedy decode steps with the argmax fed back on the device (no host
        round trip between steps). Returns the generated tokens [steps, B]."""
        out = torch.empty((steps, self.batch), device=self.engine.device, dtype=torch.int64)
        for i in range(steps):
            self.run_program(feedback=True)
            out[i].copy_(self.ids, non_blocking=True)
        return out


class B200DecodeRuntime:
    """Execute compiled CacheIR decode graphs on a B200 (see module docstring)."""

    supports_variable_prefill_batch = True

    def __init__(
        self,
        artifact: CompileArtifact | Any | str | Path,
        *,
        device: str = "cuda",
        dtype: str | None = "auto",
        weights: B200WeightStore | None = None,
        tensor_source: Any = None,
        kv_allocator: B200KVPageAllocator | None = None,
        max_seq_len: int | None = None,
        use_cuda_graph: bool = True,
        attention_splits: int = 0,
        max_plans: int = 8,
        clone_outputs: bool = True,
        tensor_parallel: TensorParallel | None = None,
        memory_limit_mb: float | None = None,
        kv_dtype: str = "same",
        fuse_attention_prepass: bool = True,
        _engine: _Engine | None = None,
    ):
        if isinstance(artifact, (str, Path)):
            artifact = CompileArtifact.load(artifact)
        if _engine is None:
            if not torch.cuda.is_available():
                raise RuntimeError("B200DecodeRuntime needs a CUDA device; cacheir_b200 has no CPU fallback")
            dev = torch.device(device)
            if dev.type != "cuda":
                raise RuntimeError("B200DecodeRuntime runs on CUDA devices only")
            if dev.index is None:
                dev = torch.device("cuda", torch.cuda.current_device())
            selected = _dtype_from_name(dtype)
            if selected is None:
                selected = torch.float16 if str(artifact.config.dtype).lower() in {"float16", "fp16", "bfloat16", "bf16"} else torch.float32
            with torch.cuda.device(dev):
                _engine = _Engine(artifact, device=dev, dtype=selected, weights=weights, tensor_source=tensor_source,
                                  kv_allocator=kv_allocator, max_seq_len=max_seq_len, use_cuda_graph=use_cuda_graph,
                                  attention_splits=attention_splits, max_plans=max_plans, tensor_parallel=tensor_parallel,
                                  kv_dtype=kv_dtype, fuse_attention_prepass=fuse_attention_prepass)
        self._engine = _engine
        self.artifact = _engine.artifact
        self.device = _engine.device
        self.dtype = _engine.dtype
        self.weights = _engine.weights
        self.tokenizer = _engine.tokenizer
        self.kv_allocator = _engine.allocator
        self.prefix_cache = _engine.prefix_cache
        self.kernel_counts = _engine.kernel_counts
        self.gemm_plans = _engine.gemm_plans
        self.kv_cache = B200PagedKVCache(_engine.allocator, int(_engine.config.num_layers))
        self.clone_outputs = clone_outputs
        self.oom_recoveries = 0
        self.memory_limit_mb = memory_limit_mb

    @classmethod
    def available(cls) -> bool:
        return b200_runtime_available()

    def fork(self) -> "B200DecodeRuntime":
        """Independent KV session sharing weights, page pools, plans and prefix cache (cuda.py:491-506)."""
        return B200DecodeRuntime(self.artifact, clone_outputs=self.clone_outputs, memory_limit_mb=self.memory_limit_mb,
                                 _engine=self._engine)

    # -- decode ----------------------------------------------------------------------
    def run_decode_batch(self, sessions: list["B200DecodeRuntime"], token_ids: list[int] | tuple[int, ...]) -> torch.Tensor:
        """Advance one decode token for several sessions; returns logits [N, 1, vocab] (cuda.py:541-582)."""
        self._enforce_memory_limit()
        try:
            plan = self._repeat_step(sessions, token_ids)
            if plan is None:
                plan = self._prepare_batch(sessions, token_ids)
                with torch.cuda.device(self.device):
                    plan.run_program()
                self._arm_repeat(plan, sessions)
        except (torch.cuda.OutOfMemoryError, KVPoolExhausted) as exc:
            self._recover_from_oom()
            raise RuntimeError("CacheIR CUDA batch decode recovered from an out-of-memory condition; "
                               "retry with fewer active requests") from exc
        self._engine.count("cacheir.b200_decode_batch_graph")
        logits = plan.logits.view(len(sessions), 1, -1)
        return logits.clone() if self.clone_outputs else logits

    # -- memory pressure (cuda.py:696-714) ----------------------------------------------
    def _enforce_memory_limit(self) -> None:
        """`memory_limit_mb` is a soft cap on this device's allocated memory: above it the session drops its
        own KV pages and cached blocks first and raises only if that was not enough."""
        if self.memory_limit_mb is None:
            return
        limit = float(self.memory_limit_mb)
        if float(torch.cuda.memory_allocated(self.device)) / (1024.0 * 1024.0) <= limit:
            return
        self._recover_from_oom()
        after = float(torch.cuda.memory_allocated(self.device)) / (1024.0 * 1024.0)
        if after > limit:
            raise RuntimeError(f"CacheIR CUDA memory limit exceeded: {after:.1f} MB allocated after recovery, "
                               f"limit is {limit:.1f} MB")

    def _recover_from_oom(self) -> None:
        """What the reference does after an allocation failure: count it, give this session's pages back to the
        pool, return cached blocks to the driver. The step that failed is not retried here."""
        self.oom_recoveries += 1
        self.kv_cache.clear()
        self._engine.validated_batch = None
        torch.cuda.empty_cache()

    def _check_positions(self, sessions) -> None:
        """The cos/sin table and the page-table width cover `max_seq_len` positions; a longer sequence would read
        RoPE angles outside the table (left unrotated, flagged only in the device status word)."""
        limit = self._engine.max_seq_len
        for session in sessions:
            if session.kv_cache.tokens > limit:
                raise ValueError(f"sequence of {session.kv_cache.tokens} tokens exceeds max_seq_len={limit}; "
                                 "construct the runtime with a larger max_seq_len")

    # -- the steady state of a decode loop ---------------------------------------------------
    # While the same sessions step together and none of them opens a page, the device already holds everything a
    # step needs except the token ids (lengths advance on the device, the page table is unchanged). Such a step is
    # launched first and the host bookkeeping (one more token per session) runs while the GPU works.
    def _arm_repeat(self, plan: "_DecodePlan", sessions) -> None:
        eng = self._engine
        page, limit = eng.page_size, eng.max_seq_len
        caches = [s.kv_cache for s in sessions]
        plan.repeat_key = eng.validated_batch
        plan.repeat_tokens = [c.tokens for c in caches]
        plan.repeat_left = min(min(page * len(c.pages) - c.tokens, limit - c.tokens) for c in caches)
        plan.repeat_version = eng.allocator.version

    def _repeat_step(self, sessions, token_ids) -> "_DecodePlan | None":
        eng = self._engine
        n = len(sessions)
        if n == 0 or n != len(token_ids):
            return None
        plan = eng.plans.get(("decode", n))
        if (plan is None or plan.repeat_left <= 0 or plan.repeat_key != tuple(map(id, sessions)) or plan.repeat_key != eng.validated_batch
                or plan.repeat_version != eng.allocator.version or plan.pool_generation != eng.allocator.generation):
            return None
        caches = [s.kv_cache for s in sessions]
        if [c.tokens for c in caches] != plan.repeat_tokens:      # someone moved a cache between the steps
            plan.repeat_left = 0
            return None
        with torch.cuda.device(self.device):
            plan.h2d_done.synchronize()   # the pinned staging buffer must not change under a pending copy
            plan.host_ids.numpy()[:] = [int(t) for t in token_ids]
            plan.ids.copy_(plan.host_ids, non_blocking=True)
            plan.h2d_done.record()
            plan.run_program()
        # bookkeeping of the step just launched (no page opens: `repeat_left` counted the room in the open pages)
        for c in caches:
            c.extend(1)
        plan.repeat_tokens = [t + 1 for t in plan.repeat_tokens]
        plan.repeat_left -= 1
        plan.synced_owner_state = [(c.owner_id, c.tokens, len(c.pages), c.epoch) for c in caches]
        eng.plans.move_to_end(("decode", n))
        return plan

    def _prepare_batch(self, sessions, token_ids) -> _DecodePlan:
        if not sessions:
            raise ValueError("run_decode_batch requires at least one session")
        if len(sessions) != len(token_ids):
            raise ValueError("sessions and token_ids must have the same length")
        batch_key = tuple(map(id, sessions))
        if batch_key != self._engine.validated_batch:      # the same sessions as last step were checked then
            for session in sessions:
                if not isinstance(session, B200DecodeRuntime):
                    raise TypeError("run_decode_batch only accepts B200DecodeRuntime sessions")
                if session._engine is not self._engine:
                    raise ValueError("all sessions must be forks of the same runtime (same artifact, weights and device)")
            if len({s.kv_cache.owner_id for s in sessions}) != len(sessions):
                raise ValueError("a session may appear only once in a decode batch")
            self._engine.validated_batch = batch_key
            self._engine.validated_sessions = list(sessions)      # keeps the ids above from being recycled
        with torch.cuda.device(self.device):
            for session in sessions:
                session.kv_cache.extend(1)      # opens a page when the new token starts one
            self._check_positions(sessions)
            plan = self._engine.plan_for(list(sessions))
            plan.sync_sessions(list(sessions))
            ids = plan.host_ids.numpy()
            ids[:] = [int(t) for t in token_ids]
            plan.ids.copy_(plan.host_ids, non_blocking=True)
            plan.h2d_done.record()
        return plan

    def decode_greedy_batch(self, sessions: list["B200DecodeRuntime"], token_ids, steps: int) -> torch.Tensor:
        """`steps` greedy tokens per session with on-device argmax feedback
        (no per-step host round trip). Returns int64 tokens [steps, N] on the device."""
        steps = int(steps)
        if steps <= 0:
            raise ValueError("steps must be positive")
        plan = self._prepare_batch(sessions, token_ids)
        with torch.cuda.device(self.device):
            for session in sessions:          # reserve the pages of the remaining steps up front
                session.kv_cache.extend(steps - 1)
            self._check_positions(sessions)
            if any(len(s.kv_cache.pages) > plan.width for s in sessions):
                raise RuntimeError("decode_greedy_batch would outgrow the plan's page table; raise max_seq_len")
            if plan.pool_generation != self._engine.allocator.generation:
                raise RuntimeError("the KV page pool grew while reserving pages; pre-size it with reserve_slots()")
            plan.h2d_done.synchronize()
            table = plan.host_table.numpy()
            for row, s in enumerate(sessions):
                table[row] = s.kv_cache.page_table_row(plan.width)
            plan.page_table.copy_(plan.host_table, non_blocking=True)
            plan.h2d_done.record()
            plan.repeat_left = 0
            tokens = plan.run_feedback_steps(steps)
            plan.synced_owner_state = [(s.kv_cache.owner_id, s.kv_cache.tokens, len(s.kv_cache.pages), s.kv_cache.epoch)
                                       for s in sessions]
        self._engine.count("cacheir.b200_decode_batch_graph", steps)
        return tokens

    def run(self, input_ids: Iterable[Iterable[int]] | np.ndarray, *, mode: str = "prefill",
            reset_kv: bool | None = None) -> torch.Tensor:
        """`CudaRuntime.run` (cuda.py:508-539). Prefill is executed as decode steps
        over the prompt (identical results: causal attention over an append-only cache)."""
        if reset_kv is None:
            reset_kv = mode == "prefill"
        if mode == "prefill" and reset_kv:
            self.kv_cache.clear()
        ids = np.asarray(input_ids, dtype=np.int64)
        if ids.ndim == 1:
            ids = ids[None, :]
        if ids.shape[0] != 1:
            raise ValueError("B200DecodeRuntime.run handles one sequence; use run_decode_batch / run_prefill_batch for batches")
        if ids.shape[1] == 0:
            raise ValueError("run needs at least one token")
        tokens = [int(t) for t in ids[0]]
        chunk = self._engine.prefill_chunk
        if mode == "prefill" and chunk > 1 and len(tokens) > chunk // 4:
            self._enforce_memory_limit()
            try:
                return self._prefill_chunked(tokens, chunk)
            except (torch.cuda.OutOfMemoryError, KVPoolExhausted) as exc:
                self._recover_from_oom()
                raise RuntimeError("CacheIR CUDA runtime recovered from an out-of-memory condition; "
                                   "retry with a smaller batch/context") from exc
        steps = []
        keep = self.clone_outputs
        self.clone_outputs = True
        try:
            for token in tokens:
                steps.append(self.run_decode_batch([self], [token]))
        finally:
            self.clone_outputs = keep
        return torch.cat(steps, dim=1) if len(steps) > 1 else steps[0]

    def _prefill_chunked(self, tokens: list[int], chunk: int) -> torch.Tensor:
        """Prefill that fills the page pool directly, `chunk` prompt tokens per pass through the decode
        graph (cuda.py:584-629 computes the same thing with a causal mask over contiguous copies): the
        tokens of a chunk are the rows of one batched step -- the projections see a [chunk, hidden] matrix,
        every row appends its K/V at its own position and attends, through the sequence's own page table,
        to exactly the tokens up to itself. Returns logits [1, T, vocab]."""
        eng = self._engine
        cache = self.kv_cache
        vocab = int(eng.config.vocab_size)
        out = torch.empty((1, len(tokens), vocab), device=self.device, dtype=self.dtype)
        with torch.cuda.device(self.device):
            for c0 in range(0, len(tokens), chunk):
                part = tokens[c0:c0 + chunk]
                start = cache.tokens
                cache.extend(len(part))
                self._check_positions([self])
                needed = (cache.tokens + eng.page_size - 1) // eng.page_size
                plan = eng.prefill_plan(chunk, needed)
                plan.sync_prefill_chunk(cache, start, part)
                plan.run_program()
                out[0, c0:c0 + len(part)] = plan.logits[: len(part)]
        eng.count("cacheir.b200_prefill_chunk", (len(tokens) + chunk - 1) // chunk)
        return out

    def _prefill_packed(self, sessions: list["B200DecodeRuntime"], token_id_batches: list[list[int]], out: torch.Tensor) -> None:
        """Prefill of several sequences through shared passes (cuda.py:584-629 pads every prompt to the longest and
        masks; here nothing is padded): the (sequence, position) pairs are laid out in order and cut into passes of
        `prefill_chunk` rows; a pass appends all its K/V rows, then every row attends to the tokens up to itself
        through its own sequence's page table. `out[i, t]` receives the logits of token t of sequence i."""
        eng = self._engine
        chunk = eng.prefill_chunk
        work: list[tuple[int, int]] = []                       # (sequence index, position)
        for i, (session, ids) in enumerate(zip(sessions, token_id_batches)):
            start = session.kv_cache.tokens
            session.kv_cache.extend(len(ids))                  # reserves the pages of the whole prompt
            work.extend((i, start + t) for t in range(len(ids)))
        self._check_positions(sessions)
        needed = max((s.kv_cache.tokens + eng.page_size - 1) // eng.page_size for s in sessions)
        starts = [s.kv_cache.tokens - len(ids) for s, ids in zip(sessions, token_id_batches)]
        passes = 0
        with torch.cuda.device(self.device):
            for w0 in range(0, len(work), chunk):
                part = work[w0:w0 + chunk]
                plan = eng.prefill_plan(chunk, needed)
                plan.sync_prefill_rows([(sessions[i].kv_cache, pos, int(token_id_batches[i][pos - starts[i]])) for i, pos in part])
                plan.run_program()
                seq = torch.tensor([i for i, _ in part], device=self.device, dtype=torch.long)
                tok = torch.tensor([pos - starts[i] for i, pos in part], device=self.device, dtype=torch.long)
                out[seq, tok] = plan.logits[: len(part)]
                passes += 1
        eng.count("cacheir.b200_prefill_chunk", passes)

    def run_prefill_batch(self, sessions: list["B200DecodeRuntime"], token_id_batches: list[list[int]]) -> torch.Tensor:
        """Variable-length batched prefill (cuda.py:584-629): returns zero-padded logits [N, max_len, vocab]."""
        if not sessions:
            raise ValueError("run_prefill_batch requires at least one session")
        if len(sessions) != len(token_id_batches):
            raise ValueError("sessions and token_id_batches must have the same length")
        lens = [len(t) for t in token_id_batches]
        if any(n <= 0 for n in lens):
            raise ValueError("run_prefill_batch requires non-empty token batches")
        for session in sessions:
            session.kv_cache.clear()
        vocab = int(self._engine.config.vocab_size)
        out = torch.zeros((len(sessions), max(lens), vocab), device=self.device, dtype=self.dtype)
        chunk = self._engine.prefill_chunk
        if chunk > 1 and sum(lens) > chunk // 4:
            # Packed prefill: the prompt tokens of all sequences are the rows of 64-row passes through the decode
            # graph, sequence after sequence, so short prompts share a pass and a long prompt spans several.
            self._enforce_memory_limit()
            try:
                self._prefill_packed(sessions, token_id_batches, out)
            except (torch.cuda.OutOfMemoryError, KVPoolExhausted) as exc:
                self._recover_from_oom()
                raise RuntimeError("CacheIR CUDA runtime recovered from an out-of-memory condition; "
                                   "retry with a smaller batch/context") from exc
        else:
            for pos in range(max(lens)):
                rows = [i for i, n in enumerate(lens) if pos < n]
                logits = self.run_decode_batch([sessions[i] for i in rows], [token_id_batches[i][pos] for i in rows])
                out[rows, pos] = logits[:, 0]
        self._engine.count("cacheir.b200_prefill_batch_graph")
        return out

    def prefill_tokens(self, token_ids, *, use_prefix_cache: bool = False, remember_prefix: bool = False):
        """cuda.py:631-653. A reused prefix aliases the stored pages instead of copying a snapshot."""
        ids = [int(t) for t in token_ids]
        reused: tuple[int, ...] = ()
        if use_prefix_cache and ids:
            prefix, holder = self.prefix_cache.longest_prefix(ids)
            if holder is not None and 0 < len(prefix) < len(ids):
                self.kv_cache.clear()
                self.kv_cache.share_prefix(holder, len(prefix))
                reused = prefix
                logits = self.run([ids[len(prefix):]], mode="prefill", reset_kv=False)
            else:
                logits = self.run([ids], mode="prefill", reset_kv=True)
        else:
            logits = self.run([ids], mode="prefill", reset_kv=True)
        if remember_prefix and ids:
            self.remember_prefix(ids)
        return logits, reused

    def generate(self, prompt: str, *, max_new_tokens: int = 16, use_prefix_cache: bool = False,
                 remember_prefix: bool = True) -> Iterable[str]:
        token_ids = self.tokenizer.encode(prompt)
        logits, _ = self.prefill_tokens(token_ids, use_prefix_cache=use_prefix_cache,
                                        remember_prefix=remember_prefix and use_prefix_cache)
        vocab = int(self._engine.config.vocab_size)
        for _ in range(max_new_tokens):
            next_id = int(torch.argmax(logits[0, -1]).item()) % vocab
            yield self.tokenizer.decode([next_id])
            logits = self.run([[next_id]], mode="decode")

    def remember_prefix(self, token_ids) -> None:
        self.prefix_cache.put(token_ids, self.kv_cache)

    def load_longest_prefix(self, token_ids) -> tuple[int, ...]:
        prefix, holder = self.prefix_cache.longest_prefix(token_ids)
        if holder is not None:
            self.kv_cache.clear()
            self.kv_cache.share_prefix(holder, len(prefix))
        return prefix

    def _position_offset(self, layer: int) -> int:
        return self.kv_cache.length(layer)

    def cache_stats(self) -> dict[str, object]:
        stats = self.kv_cache.stats()
        stats["device"] = str(self.device)
        stats["prefix_cache"] = self.prefix_cache.stats()
        stats["kernel_counts"] = dict(self.kernel_counts)
        stats["gemm_plans"] = dict(self.gemm_plans)
        stats["plans_lowered"] = self._engine.plans_lowered
        stats["graph_captures"] = self._engine.graph_captures
        stats["oom_recoveries"] = self.oom_recoveries
        stats["memory_limit_mb"] = self.memory_limit_mb
        return stats

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.device)
        if self._engine.tp.enabled and self._engine.peer_mode:
            self.check_device_status()

    def check_device_status(self) -> None:
        """Raise if a bounded device wait gave up since the last check (a tensor-parallel peer that never answered,
        a pipeline barrier that never completed): the outputs of that step are undefined. Synchronises the device
        and clears the word."""
        from . import _lib
        with torch.cuda.device(self.device):
            status = int(_lib.load().cacheir_b200_device_status(1))
        if status != 0:
            raise RuntimeError(f"cacheir_b200 device status {status:#x}: a bounded wait on the GPU gave up "
                               f"(kernel class {status >> 8}, wait {status & 0xFF}); the last results are undefined")


def create_runtime(artifact: Any, *, backend: str = "auto", **kwargs) -> B200DecodeRuntime:
    """The `cuda` branch of the reference dispatcher (cacheir/runtime/__init__.py:10-24).
    `auto` and `cuda` select the B200 runtime; there is no CPU backend in this package."""
    if backend not in {"auto", "cuda", "cuda-b200"}:
        raise ValueError(f"Unknown CacheIR runtime backend {backend!r} (cacheir_b200 provides the CUDA backend only)")
    return B200DecodeRuntime(artifact, **kwargs)
