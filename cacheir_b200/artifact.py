"""Read-only view of CacheIR compile artifacts, plus a builder for the lowered
decode graph of Llama-style decoders.

The runtime dispatches purely on `node.op`, `node.inputs/outputs` and
`node.attrs`, exactly like the reference runtimes
(cacheir/runtime/cuda.py:779-874), so anything that quacks like the reference's
`CompileArtifact` (cacheir/runtime/artifact.py:14-57) works: an object of the
reference package itself, or the classes below loaded from the same
`artifact.json`. `build_decoder_artifact` emits, for a given model config, the
graph the reference compiler produces for mode "decode"/"prefill" after its
fusion, quantization-lowering, specialization and kernel-selection passes
(cacheir/importers/hf.py:171-268 + cacheir/passes/transformer.py:284-424), so
large synthetic shapes do not need the reference compiler at run time.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any


@dataclass
class ModelConfig:
    """Mirror of cacheir/importers/hf.py:12-56."""

    architecture: str
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    dtype: str = "float32"
    tie_word_embeddings: bool = False
    quantization: str | None = None

    @property
    def head_dim(self) -> int:
        if self.hidden_size % self.num_attention_heads != 0:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "ModelConfig":
        return cls(
            architecture=data.get("architecture") or (data.get("architectures") or ["Unknown"])[0],
            hidden_size=int(data["hidden_size"]),
            intermediate_size=int(data.get("intermediate_size", data.get("ffn_hidden_size", data["hidden_size"] * 4))),
            num_layers=int(data.get("num_layers", data.get("num_hidden_layers", data.get("n_layer", 0)))),
            num_attention_heads=int(data.get("num_attention_heads", data.get("n_head", 0))),
            num_key_value_heads=int(data.get("num_key_value_heads", data.get("num_attention_heads", data.get("n_head", 0)))),
            vocab_size=int(data["vocab_size"]),
            max_position_embeddings=int(data.get("max_position_embeddings", data.get("seq_length", 2048))),
            rope_theta=float(data.get("rope_theta", data.get("rope_freq_base", 10000.0))),
            rms_norm_eps=float(data.get("rms_norm_eps", data.get("layer_norm_epsilon", 1e-6))),
            dtype=str(data.get("torch_dtype", data.get("dtype", "float32"))).replace("torch.", ""),
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            quantization=data.get("quantization") if isinstance(data.get("quantization"), str) else None,
        )


@dataclass
class WeightSpec:
    """cacheir/ir.py:70-95 (tensor type kept as a plain dict)."""

    key: str
    shape: tuple[int, ...]
    dtype: str = "float32"
    quant: str | None = None
    file: str | None = None

    def to_dict(self) -> dict[str, Any]:
        return {
            "key": self.key,
            "tensor_type": {"shape": list(self.shape), "dtype": self.dtype, "layout": "row_major"},
            "quant": self.quant,
            "file": self.file,
        }

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "WeightSpec":
        tt = data.get("tensor_type", {})
        return cls(key=data["key"], shape=tuple(tt.get("shape", ())), dtype=tt.get("dtype", "float32"),
                   quant=data.get("quant"), file=data.get("file"))


@dataclass
class Node:
    """cacheir/ir.py:98-133."""

    op: str
    inputs: list[str]
    outputs: list[str]
    attrs: dict[str, Any] = field(default_factory=dict)
    name: str | None = None

    def to_dict(self) -> dict[str, Any]:
        return {"op": self.op, "inputs": list(self.inputs), "outputs": list(self.outputs),
                "attrs": dict(self.attrs), "name": self.name, "side_effect": False}

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "Node":
        return cls(op=data["op"], inputs=list(data.get("inputs", [])), outputs=list(data.get("outputs", [])),
                   attrs=dict(data.get("attrs", {})), name=data.get("name"))


@dataclass
class Graph:
    """The fields of cacheir/ir.py `Graph` that a runtime reads."""

    name: str
    mode: str
    target: str
    nodes: list[Node] = field(default_factory=list)
    weights: dict[str, WeightSpec] = field(default_factory=dict)
    constants: dict[str, Any] = field(default_factory=dict)
    outputs: list[str] = field(default_factory=list)
    attrs: dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return {
            "name": self.name, "mode": self.mode, "target": self.target,
            "inputs": {"input_ids": {"shape": ["batch", "seq"], "dtype": "int64", "layout": "row_major"}},
            "outputs": list(self.outputs),
            "weights": {name: spec.to_dict() for name, spec in self.weights.items()},
            "constants": dict(self.constants),
            "nodes": [node.to_dict() for node in self.nodes],
            "attrs": dict(self.attrs),
        }

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "Graph":
        return cls(
            name=data.get("name", "graph"), mode=data.get("mode", "decode"), target=data.get("target", "cuda"),
            nodes=[Node.from_dict(n) for n in data.get("nodes", [])],
            weights={name: WeightSpec.from_dict(spec) for name, spec in data.get("weights", {}).items()},
            constants=dict(data.get("constants", {})),
            outputs=list(data.get("outputs", [])),
            attrs=dict(data.get("attrs", {})),
        )


@dataclass
class CompileArtifact:
    """cacheir/runtime/artifact.py:14-57, 107-114 (load side)."""

    target: str
    quant: str | None
    model_path: str
    config: ModelConfig
    graphs: dict[str, Graph]
    version: str = "0.1"
    metadata: dict[str, Any] = field(default_factory=dict)

    def graph(self, mode: str = "decode") -> Graph:
        if mode in self.graphs:
            return self.graphs[mode]
        if self.graphs:
            return next(iter(self.graphs.values()))
        raise KeyError("artifact has no graphs")

    def to_dict(self) -> dict[str, Any]:
        return {
            "version": self.version, "target": self.target, "quant": self.quant,
            "model_path": self.model_path, "config": self.config.to_dict(),
            "graphs": {mode: graph.to_dict() for mode, graph in self.graphs.items()},
            "pass_traces": {}, "metadata": dict(self.metadata),
        }

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "CompileArtifact":
        return cls(
            version=data.get("version", "0.1"), target=data.get("target", "cuda"), quant=data.get("quant"),
            model_path=data.get("model_path", ""), config=ModelConfig.from_dict(data["config"]),
            graphs={mode: Graph.from_dict(g) for mode, g in data.get("graphs", {}).items()},
            metadata=dict(data.get("metadata", {})),
        )

    def save(self, path: str | Path) -> Path:
        out = Path(path)
        out.parent.mkdir(parents=True, exist_ok=True)
        out.write_text(json.dumps(self.to_dict(), indent=2), encoding="utf-8")
        return out

    @classmethod
    def load(cls, path: str | Path) -> "CompileArtifact":
        p = Path(path)
        if p.is_dir():
            p = p / "artifact.json"
        return cls.from_dict(json.loads(p.read_text(encoding="utf-8")))


def _kernel_name(op: str, target: str) -> str:
    """`KernelSelection._kernel_for`, cacheir/passes/transformer.py:370-388."""
    prefix = "triton" if target in {"cuda", "triton"} else "cpu"
    table = {
        "token_embedding": "embedding_gather",
        "rms_norm": "rms_norm",
        "matmul": "matmul_avx" if prefix == "cpu" else "matmul_tensorcore",
        "quantized_matmul": "qmatmul_dequant" if prefix == "cpu" else "awq_int4_tensorcore",
        "fused_rmsnorm_qkv_rope": "fused_rmsnorm_qkv_rope",
        "quantized_fused_rmsnorm_qkv_rope": "awq_fused_rmsnorm_qkv_rope",
        "paged_attention_prefill": "paged_attention_prefill",
        "paged_attention_decode": "paged_attention_decode",
        "fused_swiglu": "fused_swiglu",
        "quantized_fused_swiglu": "awq_fused_swiglu",
        "add": "vector_add",
    }
    return f"{prefix}.{table.get(op, op)}"


def build_decoder_graph(config: ModelConfig, *, mode: str = "decode", target: str = "cuda",
                        quant: str | None = None, weight_file: str | None = "weights.npz") -> Graph:
    """The lowered graph for one mode: token_embedding, then per layer
    [(quantized_)fused_rmsnorm_qkv_rope, paged_attention_<mode>, matmul(o), add,
    rms_norm, (quantized_)fused_swiglu, matmul(down), add], final rms_norm and
    lm_head matmul -- value names, weight keys and attrs as the reference emits
    them (cacheir/importers/hf.py:171-268 after cacheir/compiler.py:114-132)."""
    q = "quantized_" if quant else ""
    h, inter, kv = config.hidden_size, config.intermediate_size, config.kv_dim
    dtype = config.dtype
    # The runtimes read the page size from the decode graph, where the reference
    # caps it at 16 (cacheir/passes/transformer.py:398-400, cacheir/runtime/cuda.py:474).
    graph = Graph(name=config.architecture, mode=mode, target=target)
    graph.attrs = {
        "model_config": config.to_dict(),
        "execution_mode": mode,
        "kv_cache": {"policy": "paged", "compiled_with_graph": True, "decode_token_granularity": mode == "decode"},
        "execution_hints": {"target": target, "mode": mode, "page_size": 16,
                            "prefer_fused_decode_attention": mode == "decode", "low_vram_mode": False},
        "kernel_target": target,
    }
    layout = "row_major_out_in" if target == "cpu" else "tensorcore_interleaved"

    def weight(name: str, key: str, shape: tuple[int, ...]) -> None:
        graph.weights[name] = WeightSpec(key=key, shape=shape, dtype=dtype, file=weight_file)

    def node(op: str, inputs: list[str], outputs: list[str], attrs: dict[str, Any], name: str) -> None:
        full = dict(attrs)
        if op in {"matmul", "quantized_matmul", "fused_rmsnorm_qkv_rope", "quantized_fused_rmsnorm_qkv_rope",
                  "fused_swiglu", "quantized_fused_swiglu"}:
            full["weight_layout"] = layout
            full["activation_layout"] = "bsh"
            if quant:
                full["quant"] = quant
        if op in {"matmul", "quantized_matmul"}:
            full["cost_class"] = "compute_bound"
        elif op == "paged_attention_decode":
            full["cost_class"] = "kv_bandwidth_bound"
        elif op == "paged_attention_prefill":
            full["cost_class"] = "mixed_attention"
        else:
            full["cost_class"] = "elementwise_or_fused"
        full["kernel"] = _kernel_name(op, target)
        full["schedule_index"] = len(graph.nodes)
        graph.nodes.append(Node(op=op, inputs=inputs, outputs=outputs, attrs=full, name=name))

    weight("tok_embeddings", "model.embed_tokens.weight", (config.vocab_size, h))
    weight("final_norm_w", "model.norm.weight", (h,))
    weight("lm_head_w", "model.embed_tokens.weight" if config.tie_word_embeddings else "lm_head.weight",
           (config.vocab_size, h))
    node("token_embedding", ["input_ids", "tok_embeddings"], ["hidden_0"], {}, "embed")
    hidden = "hidden_0"
    attn_op = "paged_attention_decode" if mode == "decode" else "paged_attention_prefill"
    for layer in range(config.num_layers):
        p, ln = f"model.layers.{layer}", f"layer{layer}"
        weight(f"{ln}_attn_norm_w", f"{p}.input_layernorm.weight", (h,))
        weight(f"{ln}_q_w", f"{p}.self_attn.q_proj.weight", (h, h))
        weight(f"{ln}_k_w", f"{p}.self_attn.k_proj.weight", (kv, h))
        weight(f"{ln}_v_w", f"{p}.self_attn.v_proj.weight", (kv, h))
        weight(f"{ln}_o_w", f"{p}.self_attn.o_proj.weight", (h, h))
        weight(f"{ln}_mlp_norm_w", f"{p}.post_attention_layernorm.weight", (h,))
        weight(f"{ln}_gate_w", f"{p}.mlp.gate_proj.weight", (inter, h))
        weight(f"{ln}_up_w", f"{p}.mlp.up_proj.weight", (inter, h))
        weight(f"{ln}_down_w", f"{p}.mlp.down_proj.weight", (h, inter))
        node(f"{q}fused_rmsnorm_qkv_rope",
             [hidden, f"{ln}_attn_norm_w", f"{ln}_q_w", f"{ln}_k_w", f"{ln}_v_w"],
             [f"{ln}_q_rope", f"{ln}_k_rope", f"{ln}_v"],
             {"layer": layer, "eps": config.rms_norm_eps, "head_dim": config.head_dim, "rope_theta": config.rope_theta},
             f"{ln}.fused_rmsnorm_qkv_rope")
        node(attn_op, [f"{ln}_q_rope", f"{ln}_k_rope", f"{ln}_v"], [f"{ln}_attn"],
             {"layer": layer, "num_heads": config.num_attention_heads, "num_kv_heads": config.num_key_value_heads,
              "head_dim": config.head_dim, "kv_cache": "paged", "mode": mode,
              "kv_cache_policy": "append_only_pages", "page_size": 16, "low_vram_mode": False},
             f"{ln}.attention")
        node(f"{q}matmul", [f"{ln}_attn", f"{ln}_o_w"], [f"{ln}_attn_out"], {"layer": layer, "projection": "o"}, f"{ln}.o_proj")
        node("add", [hidden, f"{ln}_attn_out"], [f"{ln}_post_attn"], {"layer": layer, "kind": "residual"}, f"{ln}.attn_residual")
        node("rms_norm", [f"{ln}_post_attn", f"{ln}_mlp_norm_w"], [f"{ln}_mlp_norm"], {"eps": config.rms_norm_eps, "layer": layer}, f"{ln}.mlp_norm")
        node(f"{q}fused_swiglu", [f"{ln}_mlp_norm", f"{ln}_gate_w", f"{ln}_up_w"], [f"{ln}_gated"], {"layer": layer}, f"{ln}.fused_swiglu")
        node(f"{q}matmul", [f"{ln}_gated", f"{ln}_down_w"], [f"{ln}_down"], {"layer": layer, "projection": "down"}, f"{ln}.down_proj")
        node("add", [f"{ln}_post_attn", f"{ln}_down"], [f"{ln}_post_mlp"], {"layer": layer, "kind": "residual"}, f"{ln}.mlp_residual")
        hidden = f"{ln}_post_mlp"
    node("rms_norm", [hidden, "final_norm_w"], ["final_hidden"], {"eps": config.rms_norm_eps}, "final_norm")
    node(f"{q}matmul", ["final_hidden", "lm_head_w"], ["logits"], {"projection": "lm_head"}, "lm_head")
    graph.outputs = ["logits"]
    return graph


def build_decoder_artifact(config: ModelConfig, *, model_path: str = "", target: str = "cuda",
                           quant: str | None = None, modes: tuple[str, ...] = ("prefill", "decode")) -> CompileArtifact:
    return CompileArtifact(
        target=target, quant=quant, model_path=str(model_path), config=config,
        graphs={mode: build_decoder_graph(config, mode=mode, target=target, quant=quant) for mode in modes},
    )
