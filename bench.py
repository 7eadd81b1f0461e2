#!/usr/bin/env python
"""Decode-throughput benchmark of the CacheIR batched decode step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (default): the Llama-3-8B-shaped random-init decoder of the reference's
headline configuration -- 32 layers, hidden 4096, 32 query / 8 KV heads,
head_dim 128, FFN 14336, vocab 128256, int8 per-channel weights (fp32 scale +
zero point per row, the reference's pack format), fp16 activations and KV pages
of 16 tokens; batch 32 requests, each with 2048 cached context tokens; greedy
decode. Weights are N(0, 0.02) generated and packed on the device, the KV cache
is pre-filled with N(0,1): synthetic data of the benchmark's shapes.

One "step" is one decode step of the whole batch. Reported on one JSON line:
  value         tokens/s with all state resident in HBM (CUDA-graph replay with
                on-device argmax feedback), timed with CUDA events, max over ranks
  e2e           tokens/s through `run_decode_batch(sessions, token_ids)` with host
                token lists in and host argmax ids out every step (H2D/D2H inside)
  roofline      achieved HBM GB/s of the dominant kernel (paged decode attention),
                timed alone with CUDA events over all layers' page pools, against
                the measured copy bandwidth in MEASURED_PEAKS.json
  cpu_baseline  the reference's CPU algorithm (NumPy dequantize-then-matmul +
                gather attention) timed on this host on a bounded sample
With --gpus N (launched under torchrun) every rank runs its own batch of 32
requests on its own weight replica: data parallel by sequence, no collective in
the step ("scaling": "weak").
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

if "reference" in sys.argv and "TORCHELASTIC_RUN_ID" in os.environ and os.environ.get("OMP_NUM_THREADS") == "1":
    # torchrun defaults every rank to one OpenMP thread; the CPU arm runs on rank 0 alone with all host cores
    del os.environ["OMP_NUM_THREADS"]

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"

WORKLOADS = {
    # name: layers hidden heads kv_heads ffn vocab batch ctx
    "llama3-8b-int8-b32-ctx2048": dict(layers=32, hidden=4096, heads=32, kv_heads=8, ffn=14336, vocab=128256,
                                       batch=32, ctx=2048, quant="int8"),
    "small": dict(layers=2, hidden=1024, heads=8, kv_heads=2, ffn=2816, vocab=4096, batch=8, ctx=256, quant="int8"),
    # the 70B-shaped tensor-parallel configuration: group-128 int4 weights, 128 sequences with log-uniform
    # contexts, 8 groups of 16 requests sharing a 512-token prefix (run with --tp on 8 GPUs)
    "llama3-70b-int4g128-b128-tp8": dict(layers=80, hidden=8192, heads=64, kv_heads=8, ffn=28672, vocab=128256,
                                         batch=128, ctx_range=(1024, 32768), shared_prefix=(16, 512), quant="int4_g128"),
    # the same code path at a size two GPUs handle in seconds
    "small-tp": dict(layers=4, hidden=1024, heads=8, kv_heads=8, ffn=3072, vocab=4096, batch=72,
                     ctx_range=(64, 1024), shared_prefix=(8, 32), quant="int4_g128"),
}


ATTENTION_TRAFFIC_RATIO = 1.024     # ncu: DRAM bytes / algorithmic bytes of the paged decode attention kernel


def workload_config(cfg: dict, workload: str, world: int, tp: bool) -> dict:
    """The `config` object of a result line; both arms (B200 and the CPU reference arm) print the same keys."""
    return {"workload": workload, "batch_per_gpu": cfg["batch"],
            "context": (f"log-uniform {cfg['ctx_range'][0]}..{cfg['ctx_range'][1]} (mean {cfg['ctx_mean']}), "
                        f"{cfg['shared_prefix'][0]}-way shared {cfg['shared_prefix'][1]}-token prefixes"
                        if "ctx_range" in cfg else cfg["ctx"]),
            "layers": cfg["layers"],
            "weights": ("int4 group-128 symmetric (fp16 scales)" if "g128" in cfg["quant"]
                        else "int8 per-row affine (fp32 scale+zero)"),
            "kv": "int8 pages of 16 (fp16 scale per cached row)" if cfg.get("kv_dtype") == "int8" else "fp16 pages of 16",
            "parallelism": (f"tp{world}: heads and FFN split, own all-reduce kernels over NVLink peer memory" if tp
                            else f"dp{world} by sequence, no collective"), "l2_policy": "inputs larger than L2 (16 GB/step)"}


def context_lengths(cfg: dict) -> list[int]:
    """Per-sequence context: the fixed `ctx`, or log-uniform in `ctx_range` (seed 0) for the ragged workloads."""
    if "ctx_range" not in cfg:
        return [int(cfg["ctx"])] * cfg["batch"]
    lo, hi = cfg["ctx_range"]
    u = np.random.default_rng(0).uniform(np.log(lo), np.log(hi), cfg["batch"])
    lens = np.exp(u).astype(np.int64)
    group, shared = cfg.get("shared_prefix", (1, 0))
    return [int(max(v, shared + 1 if group > 1 else 1)) for v in lens]


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# --------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows: list[list[str]] = []
        self.proc: subprocess.Popen | None = None
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump() -> None:
            assert self.proc is not None and self.proc.stdout is not None
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            if len(row) < 9:
                continue
            try:
                sm.append(float(row[1]))
                sm_max.append(float(row[2]))
            except ValueError:
                continue
            for name, cell in zip(names, row[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------
def build_runtime(cfg: dict, device_index: int, extra_tokens: int, tensor_parallel=None, kv_dtype: str = "same",
                  fuse_attention_prepass: bool = True):
    import zlib

    import torch

    from cacheir_b200 import B200DecodeRuntime, B200KVPageAllocator, ModelConfig, build_decoder_artifact

    head_dim = cfg["hidden"] // cfg["heads"]
    mc = ModelConfig(architecture="LlamaForCausalLM", hidden_size=cfg["hidden"], intermediate_size=cfg["ffn"],
                     num_layers=cfg["layers"], num_attention_heads=cfg["heads"], num_key_value_heads=cfg["kv_heads"],
                     vocab_size=cfg["vocab"], max_position_embeddings=cfg["ctx"] + extra_tokens, rope_theta=500000.0,
                     rms_norm_eps=1e-5, dtype="float16")
    art = build_decoder_artifact(mc, target="cuda", quant=cfg["quant"], modes=("decode",))
    dev = torch.device("cuda", device_index)
    gen = torch.Generator(device=dev)

    def synth(key: str, shape: tuple[int, ...]) -> "torch.Tensor":
        # random-init weights of the reference's tiny-model recipe at full shape: N(0, 0.02), norms = 1
        if len(shape) == 1:
            return torch.ones(shape, device=dev, dtype=torch.float32)
        gen.manual_seed(zlib.crc32(key.encode()))          # the same weights in every process
        return torch.randn(shape, device=dev, dtype=torch.float32, generator=gen) * 0.02

    page = 16
    total_pages = sum((c + extra_tokens + page - 1) // page + 1 for c in context_lengths(cfg))
    alloc = B200KVPageAllocator(page_size=page, initial_slots=total_pages + 8)
    rt = B200DecodeRuntime(art, device=f"cuda:{device_index}", dtype="float16", tensor_source=synth,
                           kv_allocator=alloc, max_seq_len=cfg["ctx"] + extra_tokens, clone_outputs=False,
                           tensor_parallel=tensor_parallel, kv_dtype=kv_dtype, fuse_attention_prepass=fuse_attention_prepass)
    del head_dim
    return rt, art


def prefill_synthetic_context(rt, cfg: dict):
    """`batch` sessions with `ctx` cached tokens each: pages are allocated through the
    allocator, their contents are N(0,1) (stand-in for a real prompt's K/V)."""
    import torch

    sessions = [rt.fork() for _ in range(cfg["batch"])]
    group, shared = cfg.get("shared_prefix", (1, 0))
    for i, (s, ctx) in enumerate(zip(sessions, context_lengths(cfg))):
        if group > 1 and i % group != 0:                  # alias the full pages of the group leader's prefix
            s.kv_cache.share_prefix(sessions[i - i % group].kv_cache, shared)
        s.kv_cache.extend(ctx - s.kv_cache.tokens)
    gen = torch.Generator(device=rt.device)
    gen.manual_seed(1234)
    for layer in range(cfg["layers"]):
        pool = rt.kv_allocator.pool_for_layer(layer)
        if "scales" in pool:                              # 8-bit pages: uniform bytes, scales of N(0,1) rows (max|row| / 127 ~ 0.02 .. 0.03)
            pool["keys"].random_(0, 256, generator=gen)
            pool["values"].random_(0, 256, generator=gen)
            pool["scales"].copy_(torch.rand(pool["scales"].shape, device=rt.device, generator=gen) * 0.01 + 0.02)
        else:
            pool["keys"].normal_(generator=gen)
            pool["values"].normal_(generator=gen)
    return sessions


def unique_kv_tokens(cfg: dict, generated: int) -> int:
    """Cached tokens that occupy distinct physical pages: pages of a shared prefix count once."""
    lens = context_lengths(cfg)
    group, shared = cfg.get("shared_prefix", (1, 0))
    aliased = (shared // 16) * 16 * (cfg["batch"] - (cfg["batch"] + group - 1) // group) if group > 1 else 0
    return sum(lens) - aliased + cfg["batch"] * generated


def kv_row_bytes(cfg: dict) -> int:
    """Bytes of one cached token of one layer: K and V rows of every KV head (8-bit pages: plus an fp16 scale per row)."""
    hd = cfg["hidden"] // cfg["heads"]
    if cfg.get("kv_dtype", "same") == "int8":
        return cfg["kv_heads"] * 2 * (hd + 2)
    return cfg["kv_heads"] * 2 * hd * 2


def step_bytes(cfg: dict, kv_tokens: int) -> dict:
    """Algorithmic HBM bytes of one decode step: every weight byte once, every cached K/V row once
    (`kv_tokens` = unique cached tokens over the whole batch)."""
    h, f, v, L = cfg["hidden"], cfg["ffn"], cfg["vocab"], cfg["layers"]
    hd = h // cfg["heads"]
    kvd = cfg["kv_heads"] * hd
    bits = 8 if cfg["quant"] == "int8" else 4
    rows = (h + 2 * kvd) + h + 2 * f + h          # q,k,v | o | gate,up | down
    elems = (h + 2 * kvd) * h + h * h + 2 * f * h + h * f
    group = 128 if "g128" in cfg["quant"] else 0
    meta = elems // group * 2 if group else rows * 8            # fp16 group scales | fp32 scale + zero per row
    layer_w = elems * bits // 8 + meta
    weights = L * layer_w + v * h * bits // 8 + (v * h // group * 2 if group else v * 8)
    del kvd
    kv = L * kv_tokens * kv_row_bytes(cfg)
    return {"weights": weights, "kv": kv, "total": weights + kv}


def time_graph(fn, iters: int) -> float:
    """Seconds per call of `fn`, timed with CUDA events around the replay of a CUDA graph that
    holds `iters` calls (host launch cost would otherwise dominate kernels of a few microseconds)."""
    import torch

    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1e-3 / iters


def time_attention_kernel(rt, sessions, cfg: dict, iters: int = 3) -> dict:
    """The dominant kernel alone: one launch per layer over that layer's page pool (each
    pool is larger than L2, so every launch streams from HBM), CUDA events on the launch stream."""
    import torch

    from cacheir_b200 import ops

    hd = cfg["hidden"] // cfg["heads"]
    tp_world = rt._engine.tp.world                      # tensor parallel: this rank's heads only
    B, H, KVH = cfg["batch"], cfg["heads"] // tp_world, cfg["kv_heads"] // tp_world
    plan = rt._engine.plan_for(sessions)
    lens = torch.tensor([s.kv_cache.tokens for s in sessions], dtype=torch.int32, device=rt.device)
    q = torch.randn((B, H, hd), device=rt.device, dtype=torch.float16)
    out = torch.empty_like(q)
    splits = ops.attention_auto_splits(B, H, KVH, plan.width, 16, hd)
    ws = torch.empty(max(1, ops.attention_workspace_bytes(B, H, hd, splits) // 4), device=rt.device, dtype=torch.float32)
    pools = [rt.kv_allocator.pool_for_layer(l) for l in range(cfg["layers"])]

    def sweep() -> None:
        for pool in pools:
            ops.paged_attention_decode_batch(q, pool["keys"], pool["values"], plan.page_table, lens, out=out,
                                             num_splits=splits, workspace=ws, kv_scales=pool.get("scales"))

    per_launch_s = time_graph(sweep, iters) / len(pools)
    group, shared = cfg.get("shared_prefix", (1, 0))      # physical pages of a shared prefix are read (and count) once
    aliased = (shared // 16) * 16 * (B - (B + group - 1) // group) if group > 1 else 0
    total_ctx = int(lens.sum().item()) - aliased
    algo = total_ctx * kv_row_bytes(cfg) // tp_world + 2 * B * H * hd * 2 + B * plan.width * 4 + B * 4
    return {"kernel": "paged_attention_decode_batch", "seconds": per_launch_s, "bytes": algo, "splits": splits}


def time_gemv_kernels(rt, cfg: dict, iters: int = 3) -> list[dict]:
    """Each projection shape alone, cycling over the layers' weights (cold in L2)."""
    import torch

    from cacheir_b200 import ops
    from cacheir_b200.quantization import quantized_matmul

    eng = rt._engine
    B = cfg["batch"]
    groups: dict[str, list] = {"qkv": [], "o": [], "gate_up": [], "down": []}
    for names, w in eng.fused_weights.items():
        n0 = names[0]
        if n0.endswith("_q_w"):
            groups["qkv"].append(w)
        elif n0.endswith("_o_w"):
            groups["o"].append(w)
        elif n0.endswith("_gate_w"):
            groups["gate_up"].append(w)
        elif n0.endswith("_down_w"):
            groups["down"].append(w)
    results = []
    for name, ws in groups.items():
        if not ws:
            continue
        n, k = ws[0].shape
        epi = ops.EPI_SWIGLU if name == "gate_up" else ops.EPI_NONE
        x = torch.randn((B, k), device=rt.device, dtype=torch.float16)
        out = torch.empty((B, n // 2 if epi == ops.EPI_SWIGLU else n), device=rt.device, dtype=torch.float16)
        scratch = torch.zeros(ops.qgemv_workspace_bytes(B, k), device=rt.device, dtype=torch.uint8)

        def sweep(ws=ws, x=x, out=out, epi=epi, scratch=scratch) -> None:
            for w in ws:
                quantized_matmul(x, w, epilogue=epi, out=out, workspace=scratch)

        sec = time_graph(sweep, iters) / len(ws)
        algo = ws[0].nbytes + B * k * 2 + out.numel() * 2
        results.append({"kernel": f"qgemv_int{ws[0].bits}_{name}", "shape": [B, n, k], "seconds": sec, "bytes": algo})
    return results


# --------------------------------------------------------------------------------------
def cpu_reference_layer_step(cfg: dict, rng: np.random.Generator, weights: dict, kv: dict, x: np.ndarray,
                             rows_fraction: float = 1.0) -> np.ndarray:
    """One decoder layer of one decode step with the reference's CPU algorithm (dequantize the
    whole weight, then matmul; gather K/V, attention), batch `x.shape[0]`."""
    from oracle import oracle, ref_native

    h = cfg["hidden"]
    heads, kv_heads = cfg["heads"], cfg["kv_heads"]
    hd = h // heads
    use_native = ref_native.available()
    norm = (lambda a, w: ref_native.rms_norm(a, w, 1e-5)) if use_native else (lambda a, w: oracle.rms_norm(a, w, 1e-5))
    xn = norm(x, weights["norm"])
    q = oracle.quantized_matmul(xn, weights["q"])
    k = oracle.quantized_matmul(xn, weights["k"])
    v = oracle.quantized_matmul(xn, weights["v"])
    offsets = kv["lens"]
    q = oracle.rope_one(q, hd, 500000.0, offsets)
    k = oracle.rope_one(k, hd, 500000.0, offsets)
    del v
    attn = oracle.paged_attention_decode(q.reshape(-1, heads, hd), kv["k_pool"], kv["v_pool"], kv["table"], kv["lens"])
    attn = attn.reshape(x.shape[0], 1, heads * hd)
    hidden = x + oracle.quantized_matmul(attn, weights["o"])
    hn = norm(hidden, weights["norm"])
    gate = oracle.quantized_matmul(hn, weights["gate"])
    up = oracle.quantized_matmul(hn, weights["up"])
    gated = ref_native.silu_mul(gate, up) if use_native else oracle.silu_mul(gate, up)
    return hidden + oracle.quantized_matmul(gated, weights["down"])


def make_cpu_sample(cfg: dict, batch: int, ctx: int, seed: int = 0):
    from oracle import oracle

    rng = np.random.default_rng(seed)
    h, f = cfg["hidden"], cfg["ffn"]
    hd = h // cfg["heads"]
    kvd = cfg["kv_heads"] * hd
    bits = 8 if cfg["quant"] == "int8" else 4

    def packed(n: int, k: int):
        codes = rng.integers(0, 1 << bits, (n, k), dtype=np.uint8)
        return oracle.PackedQuantizedTensor(oracle.pack_int4(codes) if bits == 4 else codes,
                                            rng.uniform(1e-4, 2e-4, n).astype(np.float32),
                                            np.full(n, 1 << (bits - 1), dtype=np.int32), bits, (n, k))

    weights = {"norm": np.ones(h, dtype=np.float32), "q": packed(h, h), "k": packed(kvd, h), "v": packed(kvd, h),
               "o": packed(h, h), "gate": packed(f, h), "up": packed(f, h), "down": packed(h, f)}
    pages = (ctx + 15) // 16
    kv = {"k_pool": rng.standard_normal((batch * pages, cfg["kv_heads"], 16, hd), dtype=np.float32),
          "v_pool": rng.standard_normal((batch * pages, cfg["kv_heads"], 16, hd), dtype=np.float32),
          "table": rng.permutation(batch * pages).astype(np.int32).reshape(batch, pages),
          "lens": np.full(batch, ctx, dtype=np.int32)}
    x = rng.standard_normal((batch, 1, h), dtype=np.float32)
    return rng, weights, kv, x


def cpu_lm_head_seconds(cfg: dict, batch: int) -> float:
    """The lm_head of one decode step with the reference's CPU algorithm (dequantize, then matmul), timed once over
    the whole vocabulary in slices of 16384 rows (the dense fp32 form of the full weight would be 2 GB)."""
    from oracle import oracle

    rng = np.random.default_rng(7)
    h, v = cfg["hidden"], cfg["vocab"]
    bits = 8 if cfg["quant"] == "int8" else 4
    x = rng.standard_normal((batch, 1, h), dtype=np.float32)
    rows = 16384
    codes = rng.integers(0, 1 << bits, (rows, h), dtype=np.uint8)
    part = oracle.PackedQuantizedTensor(oracle.pack_int4(codes) if bits == 4 else codes, rng.uniform(1e-4, 2e-4, rows).astype(np.float32),
                                        np.full(rows, 1 << (bits - 1), dtype=np.int32), bits, (rows, h))
    oracle.quantized_matmul(x, part)       # warm
    t0 = time.perf_counter()
    done = 0
    while done < v:
        oracle.quantized_matmul(x, part)   # every slice costs the same: the codes' values do not matter for the time
        done += rows
    return (time.perf_counter() - t0) * min(1.0, v / done)


def cpu_threads() -> int:
    try:
        from threadpoolctl import threadpool_info
        counts = [int(p.get("num_threads", 1)) for p in threadpool_info()]
        if counts:
            return max(counts)
    except Exception:
        pass
    return os.cpu_count() or 1


def run_cpu_baseline(cfg: dict, budget_s: float = 20.0) -> dict:
    """Tokens/s of the reference's CPU algorithm, from a bounded sample: repeated single-layer
    decode steps at full batch and context, extrapolated linearly to all layers (the lm_head is
    charged as vocab/ffn-proportional extra matmul rows)."""
    from oracle import ref_native

    rng, weights, kv, x = make_cpu_sample(cfg, cfg["batch"], cfg["ctx"])
    cpu_reference_layer_step(cfg, rng, weights, kv, x)   # warm
    times = []
    t_end = time.perf_counter() + budget_s
    while time.perf_counter() < t_end and len(times) < 8:
        t0 = time.perf_counter()
        cpu_reference_layer_step(cfg, rng, weights, kv, x)
        times.append(time.perf_counter() - t0)
    layer_s = float(np.median(times))
    lm_head_s = cpu_lm_head_seconds(cfg, cfg["batch"])
    step_s = layer_s * cfg["layers"] + lm_head_s
    return {"value": cfg["batch"] / step_s, "unit": UNIT, "cores": cpu_threads(), "kind": "port",
            "sample": (f"{len(times)} x one decoder layer of one decode step (batch {cfg['batch']}, ctx {cfg['ctx']}; "
                       f"NumPy dequantize-then-matmul + gather attention"
                       f"{', reference C++/OpenMP rms_norm+silu_mul' if ref_native.available() else ''}), "
                       f"median {layer_s:.3f} s/layer, extrapolated to {cfg['layers']} layers + the lm_head timed once ({lm_head_s:.2f} s)")}


def run_reference_arm(args, cfg: dict, workload: str) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref_native

    total_steps = args.steps + args.warmup
    budget = 150.0
    rng, weights, kv, x = make_cpu_sample(cfg, cfg["batch"], cfg["ctx"])
    t0 = time.perf_counter()
    cpu_reference_layer_step(cfg, rng, weights, kv, x)
    first = time.perf_counter() - t0
    # A step of this arm is one decoder layer of one decode step at full batch/context; if even that
    # would overrun the time budget for K+W steps, shrink the batch of the sample (time is ~linear in it
    # for the attention part and constant for the dequantisation, so the extrapolation is conservative).
    sample_batch = cfg["batch"]
    while first * total_steps > budget and sample_batch > 1:
        sample_batch //= 2
        rng, weights, kv, x = make_cpu_sample(cfg, sample_batch, cfg["ctx"])
        t0 = time.perf_counter()
        cpu_reference_layer_step(cfg, rng, weights, kv, x)
        first = time.perf_counter() - t0
    for _ in range(args.warmup):
        cpu_reference_layer_step(cfg, rng, weights, kv, x)
    t0 = time.perf_counter()
    done = 0
    for _ in range(args.steps):
        cpu_reference_layer_step(cfg, rng, weights, kv, x)
        done += 1
    elapsed = time.perf_counter() - t0
    layer_s = elapsed / max(1, done)
    lm_head_s = cpu_lm_head_seconds(cfg, sample_batch)
    step_s = layer_s * cfg["layers"] + lm_head_s
    value = sample_batch / step_s
    sample = (f"each step = one decoder layer of one decode step (batch {sample_batch} of {cfg['batch']}, ctx {cfg['ctx']}) with "
              f"the reference CPU algorithm (NumPy dequantize-then-matmul, gather attention"
              f"{', reference C++/OpenMP rms_norm+silu_mul' if ref_native.available() else ''}); "
              f"tokens/s extrapolated to {cfg['layers']} layers + the lm_head timed once ({lm_head_s:.2f} s)")
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "ms_per_timed_step": layer_s * 1e3,
            "timed_step": "one decoder layer of one decode step", "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(cfg, workload, world, False),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cpu_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)



# --------------------------------------------------------------------------------------
def parity_self_check(rt, sessions, cfg: dict) -> dict:
    """Outside the timed region: the kernels of the first decoder layer, on this run's own device-generated
    weights and page pool, against the CPU oracle (dequantize-then-matmul, gather attention). One fp16 batch of
    activations goes through the entry points the step uses (RMSNorm + pre-pass, the tiled integer GEMMs with
    their epilogues, paged decode attention); the worst rel-L2 is reported next to the 2e-3 gate."""
    import torch

    from cacheir_b200 import ops
    from cacheir_b200.quantization import to_rows
    from oracle import oracle

    eng = rt._engine
    dev = rt.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)
    B = min(cfg["batch"], 32)
    worst: dict[str, float] = {}

    def host_pack(w):
        rows = to_rows(w)
        return oracle.PackedQuantizedTensor(rows.packed_values.cpu().numpy(), rows.scales.float().cpu().numpy() if not w.group_size else rows.scales.cpu().numpy(),
                                            None if w.zero_points is None else w.zero_points.cpu().numpy(), w.bits, tuple(w.shape),
                                            group_size=w.group_size or None)

    def oracle_mm(x, packed):
        out = []
        for r0 in range(0, packed.shape[0], 8192):
            r1 = min(packed.shape[0], r0 + 8192)
            part = oracle.PackedQuantizedTensor(packed.packed_values[r0:r1], packed.scales[r0:r1],
                                                None if packed.zero_points is None else packed.zero_points[r0:r1],
                                                packed.bits, (r1 - r0, packed.shape[1]), group_size=packed.group_size)
            out.append(oracle.quantized_matmul(x, part))
        return np.concatenate(out, axis=-1)

    for names, w in eng.fused_weights.items():
        n0 = names[0]
        if not n0.startswith("layer0_"):
            continue
        if not hasattr(w, "bits"):
            continue
        role = "qkv" if n0.endswith("_q_w") else "o" if n0.endswith("_o_w") else "gate_up" if n0.endswith("_gate_w") else "down" if n0.endswith("_down_w") else None
        if role is None or role in worst:
            continue
        n, k = w.shape
        x = torch.randn((B, k), device=dev, dtype=torch.float16, generator=gen)
        ws = torch.zeros(ops.qgemv_workspace_bytes(B, k), device=dev, dtype=torch.uint8) if not w.group_size else None
        epi = ops.EPI_SWIGLU if role == "gate_up" else ops.EPI_NONE
        y = ops.qgemv(x, w.packed_values, w.scales, w.zero_points, bits=w.bits, n=n, k=k, group_size=w.group_size or 0,
                      epilogue=epi, workspace=ws, tiled=w.tiled, paired=w.paired)
        want = oracle_mm(x.float().cpu().numpy(), host_pack(w))
        if role == "gate_up":
            want = oracle.silu_mul(want[:, : n // 2], want[:, n // 2:])
        worst[role] = oracle.rel_l2(y.float().cpu().numpy(), want) / (2.0 if role == "gate_up" else 1.0)   # a product of two projections
    # attention over the real pool of layer 0 (its rows were written by the timed steps), first 4 sequences
    hd = cfg["hidden"] // cfg["heads"]
    tpw = eng.tp.world
    H, KVH = cfg["heads"] // tpw, cfg["kv_heads"] // tpw
    pool = rt.kv_allocator.pool_for_layer(0)
    sub = sessions[:4]
    width = max(len(s.kv_cache.pages) for s in sub)
    table = np.stack([s.kv_cache.page_table_row(width) for s in sub]).astype(np.int32)
    lens = np.array([min(s.kv_cache.tokens, 4096) for s in sub], dtype=np.int32)
    q = torch.randn((len(sub), H, hd), device=dev, dtype=torch.float16, generator=gen)
    out = ops.paged_attention_decode_batch(q, pool["keys"], pool["values"], torch.from_numpy(table).to(dev), torch.from_numpy(lens).to(dev),
                                           kv_scales=pool.get("scales"))
    used = np.unique(table)
    remap = np.zeros(int(table.max()) + 1, dtype=np.int32)
    remap[used] = np.arange(len(used), dtype=np.int32)
    idx = torch.from_numpy(used.astype(np.int64)).to(dev)
    keys, values = pool["keys"][idx].cpu().numpy(), pool["values"][idx].cpu().numpy()
    if "scales" in pool:                                  # 8-bit pages: the oracle sees the same bytes, dequantised in fp32
        sc = pool["scales"][idx].cpu().numpy()
        keys, values = oracle.dequantize_kv_pool(keys, sc, 0), oracle.dequantize_kv_pool(values, sc, 1)
    want = oracle.paged_attention_decode(q.cpu().numpy(), keys, values, remap[table], lens)
    worst["attention"] = oracle.rel_l2(out.float().cpu().numpy(), want)
    torch.cuda.synchronize()
    return {"rel_l2": round(max(worst.values()), 6), "gate": 2e-3, "per_kernel": {k: round(v, 6) for k, v in worst.items()},
            "against": "CPU oracle on this run's layer-0 weights and page pool"}


def tensor_parallel_parity(rank: int, world: int, local_rank: int) -> dict | None:
    """A two-layer int8 model decoded tensor parallel on all ranks and on rank 0 alone, teacher-forced with the same
    tokens: logits rel-L2 and whether the greedy tokens agree wherever the single-GPU top-1 / top-2 margin is clear."""
    import zlib

    import torch
    import torch.distributed as dist

    from cacheir_b200 import B200DecodeRuntime
    from cacheir_b200.artifact import ModelConfig, build_decoder_artifact
    from cacheir_b200.tensor_parallel import TensorParallel
    from oracle import oracle

    heads = max(4, world)
    cfg = ModelConfig(architecture="LlamaForCausalLM", hidden_size=128 * heads, intermediate_size=256 * world * 2, num_layers=2,
                      num_attention_heads=heads, num_key_value_heads=world, vocab_size=512 * world, max_position_embeddings=256,
                      rope_theta=10000.0, rms_norm_eps=1e-5, dtype="float16")
    artifact = build_decoder_artifact(cfg, quant="int8")

    def source(key, shape):
        g = torch.Generator(device="cpu")
        g.manual_seed(zlib.crc32(key.encode()))
        return torch.ones(shape) if len(shape) == 1 else torch.randn(shape, generator=g) * 0.05

    rng = np.random.default_rng(5)
    prompts = [[int(t) for t in rng.integers(0, cfg.vocab_size, 9)] for _ in range(4)]
    forced = [[int(t) for t in rng.integers(0, cfg.vocab_size, 4)] for _ in range(6)]
    traces = {}
    for name, tp in (("tp", TensorParallel(rank, world)), ("single", None)):
        if name == "single" and rank != 0:
            continue
        rt = B200DecodeRuntime(artifact, device=f"cuda:{local_rank}", dtype="float16", tensor_source=source, max_seq_len=256,
                               tensor_parallel=tp)
        sessions = [rt.fork() for _ in prompts]
        logits = rt.run_prefill_batch(sessions, prompts)
        trace = [logits[:, -1].float().cpu().numpy()]
        for tokens in forced:
            trace.append(rt.run_decode_batch(sessions, tokens)[:, -1].float().cpu().numpy())
        traces[name] = np.stack(trace)
        if name == "tp":
            rt.synchronize()
            dist.barrier()
    if rank != 0:
        return None
    tp_l, one_l = traces["tp"], traces["single"]
    rel = oracle.rel_l2(tp_l, one_l)
    top2 = np.sort(one_l, axis=-1)[..., -2:]
    clear = (top2[..., 1] - top2[..., 0]) > 8e-3 * np.abs(one_l).max(axis=-1)
    equal = bool(np.array_equal(tp_l.argmax(-1)[clear], one_l.argmax(-1)[clear]))
    return {"parity_rel_l2": round(float(rel), 6), "tokens_equal": equal, "tokens_compared": int(clear.sum()), "gate": 4e-3}


# --------------------------------------------------------------------------------------
def run_micro(args) -> None:
    """Single-kernel runs for profiling (`ncu ... python bench.py --micro qgemv ...`): prints one JSON
    line with the CUDA-event time per launch; inputs rotate over `--copies` buffers so that every launch
    streams from HBM."""
    import torch

    from cacheir_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    peak, kind = measured_peaks()
    if args.micro == "layer":
        run_micro_layer(args, dev, gen, peak, kind)
        return
    if args.micro == "qgemv":
        m, n, k, bits = args.m, args.n, args.k, args.bits
        row_bytes = k if bits == 8 else k // 2
        copies = max(1, args.copies)
        packed = [torch.randint(0, 256, (n, row_bytes), device=dev, dtype=torch.uint8, generator=gen) for _ in range(copies)]
        if args.group:
            scales = torch.rand((n, k // args.group), device=dev, generator=gen).mul_(0.015).add_(0.005).half()
            zeros = None
        else:
            scales = torch.rand((n,), device=dev, generator=gen).mul_(0.015).add_(0.005)
            zeros = torch.full((n,), float(1 << (bits - 1)), device=dev)
        x = torch.randn((m, k), device=dev, dtype=torch.float16, generator=gen)
        epi = {"none": ops.EPI_NONE, "swiglu": ops.EPI_SWIGLU}[args.epilogue]
        out = torch.empty((m, n // 2 if epi == ops.EPI_SWIGLU else n), device=dev, dtype=torch.float16)

        paired = args.tiled and epi == ops.EPI_SWIGLU and bits == 8 and not args.group
        if args.tiled:
            packed = [ops.pack_relayout(w, n=n, k=k, bits=bits, paired=paired) for w in packed]
        ws = None
        if args.workspace:
            ws = torch.zeros(ops.qgemv_workspace_bytes(m, k), device=dev, dtype=torch.uint8)

        def launch(i: int) -> None:
            ops.qgemv(x, packed[i % copies], scales, zeros, bits=bits, n=n, k=k, group_size=args.group, epilogue=epi,
                      out=out, workspace=ws, tiled=args.tiled, paired=paired)

        algo = n * row_bytes + scales.numel() * scales.element_size() + (n * 4 if zeros is not None else 0) + m * k * 2 + out.numel() * 2
        name = f"qgemv_int{bits}" + (f"_g{args.group}" if args.group else "")
        shape = {"M": m, "N": n, "K": k}
    else:
        batch, heads, kv_heads, hd, page = args.batch, args.heads, args.kv_heads, 128, 16
        rng = np.random.default_rng(0)
        if args.ctx_log:      # log-uniform lengths (many short sequences, a few long ones)
            lens_np = np.exp(rng.uniform(np.log(args.ctx_min), np.log(args.ctx_max), batch)).astype(np.int32)
        else:
            lens_np = rng.integers(args.ctx_min, args.ctx_max + 1, batch).astype(np.int32)
        pages = (lens_np + page - 1) // page
        total = int(pages.sum())
        table_np = np.zeros((batch, int(pages.max())), dtype=np.int32)
        perm = np.random.default_rng(1).permutation(total).astype(np.int32)
        cur = 0
        for b in range(batch):
            table_np[b, : pages[b]] = perm[cur:cur + pages[b]]
            cur += int(pages[b])
        kv8 = args.kv == "int8"
        scales = None
        if kv8:      # 8-bit pages: uniform bytes and per-row scales of N(0,1) data
            k_pool = torch.randint(0, 256, (total, kv_heads, page, hd), device=dev, dtype=torch.uint8, generator=gen)
            v_pool = torch.randint(0, 256, (total, kv_heads, page, hd), device=dev, dtype=torch.uint8, generator=gen)
            scales = (torch.rand((total, kv_heads, 2, page), device=dev, generator=gen) * 0.01 + 0.02).half()
        else:
            k_pool = torch.randn((total, kv_heads, page, hd), device=dev, dtype=torch.float16, generator=gen)
            v_pool = torch.randn((total, kv_heads, page, hd), device=dev, dtype=torch.float16, generator=gen)
        q = torch.randn((batch, heads, hd), device=dev, dtype=torch.float16, generator=gen)
        table = torch.from_numpy(table_np).to(dev)
        lens = torch.from_numpy(lens_np).to(dev)
        out = torch.empty_like(q)
        splits = args.splits or ops.attention_auto_splits(batch, heads, kv_heads, table.shape[1], page, hd)
        ws = torch.empty(max(1, ops.attention_workspace_bytes(batch, heads, hd, splits) // 4), device=dev, dtype=torch.float32)

        def launch(i: int) -> None:
            ops.paged_attention_decode_batch(q, k_pool, v_pool, table, lens, out=out, num_splits=splits, workspace=ws, kv_scales=scales)

        row_bytes = kv_heads * 2 * (hd + 2) if kv8 else kv_heads * hd * 2 * 2
        algo = int(lens_np.sum()) * row_bytes + 2 * batch * heads * hd * 2 + table.numel() * 4 + batch * 4
        name = "paged_attention_decode_batch" + ("_int8_pages" if kv8 else "")
        shape = {"batch": batch, "heads": heads, "kv_heads": kv_heads, "head_dim": hd, "total_ctx": int(lens_np.sum()), "splits": splits}
    for i in range(max(1, args.warmup)):
        launch(i)
    torch.cuda.synchronize()
    # The launches are captured in a CUDA graph so that the host's launch cost (tens of
    # microseconds from Python) does not hide kernels that take a few microseconds.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            launch(i)
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    sec = start.elapsed_time(end) * 1e-3 / args.steps
    from cacheir_b200 import _lib
    emit({"micro": name, **shape, "us_per_launch": round(sec * 1e6, 2), "algorithmic_bytes": int(algo),
          "achieved_gbs": round(algo / sec / 1e9, 1), "frac": round(algo / sec / 1e9 / peak, 4),
          "peak": peak, "peak_source": f"of {kind}", "device_status": _lib.load().cacheir_b200_device_status(0)})


def run_micro_layer(args, dev, gen, peak: float, kind: str) -> None:
    """The eight launches of one decoder layer of the 8B-shaped decode step, with the entry points and flags the runtime
    uses (RMSNorm + pre-pass, fused QKV + RoPE + cache append, paged decode attention that also writes the pre-pass of
    o, o with residual, RMSNorm + pre-pass, paired gate|up with SwiGLU, pre-pass, down with residual; with `--splits`
    above 1 the attention is split and o runs its own pre-pass: nine and a combine), batch `--m`, context `--ctx-max`;
    the weights alternate between two copies. A profiling aid: small enough to capture whole under ncu."""
    import torch

    from cacheir_b200 import ops
    from cacheir_b200.quantization import pack_weight_device, to_tiled

    B, H, KVD, FFN, hd, kvh, page, theta = args.m, 4096, 1024, 14336, 128, 8, 16, 500000.0
    ctx = args.ctx_max
    copies = 2

    def weight(n, k, paired=False):
        return [to_tiled(pack_weight_device(torch.randn((n, k), device=dev, generator=gen) * 0.02, "int8"), paired=paired) for _ in range(copies)]

    w_qkv, w_o, w_gu, w_down = weight(H + 2 * KVD, H), weight(H, H), weight(2 * FFN, H, True), weight(H, FFN)
    norm = torch.ones((H,), device=dev, dtype=torch.float16)
    pages = (ctx + 64 + page - 1) // page
    slots = B * pages
    k_pool = torch.randn((slots, kvh, page, hd), device=dev, dtype=torch.float16, generator=gen)
    v_pool = torch.randn((slots, kvh, page, hd), device=dev, dtype=torch.float16, generator=gen)
    table = torch.from_numpy(np.random.default_rng(1).permutation(slots).astype(np.int32).reshape(B, pages)).to(dev)
    positions = torch.full((B,), ctx, device=dev, dtype=torch.int32)
    lens = positions + 1
    rope = ops.rope_table(ctx + 64, hd, theta, dev)
    h0 = torch.randn((B, H), device=dev, dtype=torch.float16, generator=gen)
    qkv = torch.empty((B, H + 2 * KVD), device=dev, dtype=torch.float16)
    attn = torch.empty((B, H), device=dev, dtype=torch.float16)
    h1, h2 = torch.empty_like(h0), torch.empty_like(h0)
    act = torch.empty((B, FFN), device=dev, dtype=torch.float16)
    ws = torch.zeros(ops.qgemv_workspace_bytes(B, FFN), device=dev, dtype=torch.uint8)

    fused_prepass = (args.splits or 1) == 1 and ops.attention_quantize_supported(B, 32, kvh, pages, page, hd, torch.float16)

    def launch(i: int) -> None:
        c = i % copies
        ops.rms_norm_quantize(h0, norm, 1e-5, ws)
        w = w_qkv[c]
        ops.qkv_rope_append(None, w.packed_values, w.scales, w.zero_points, qkv, n=H + 2 * KVD, k=H, q_dim=H, k_dim=KVD, head_dim=hd,
                            theta=theta, table=rope, positions=positions, page_table=table, k_cache=k_pool, v_cache=v_pool,
                            workspace=ws, tiled=True, prequantized=True)
        q3 = qkv[:, :H].as_strided((B, 32, hd), (qkv.stride(0), hd, 1))
        w = w_o[c]
        if fused_prepass:
            ops.paged_attention_decode_batch_quantize(q3, k_pool, v_pool, table, lens, out=attn.view(B, 32, hd), gemm_workspace=ws)
        else:
            ops.paged_attention_decode_batch(q3, k_pool, v_pool, table, lens, out=attn.view(B, 32, hd), num_splits=args.splits or 1)
        ops.qgemv(attn, w.packed_values, w.scales, w.zero_points, bits=8, n=H, k=H, epilogue=ops.EPI_RESIDUAL, residual=h0, out=h1,
                  workspace=ws, tiled=True, prequantized=fused_prepass)
        ops.rms_norm_quantize(h1, norm, 1e-5, ws)
        w = w_gu[c]
        ops.qgemv(h1, w.packed_values, w.scales, w.zero_points, bits=8, n=2 * FFN, k=H, epilogue=ops.EPI_SWIGLU, out=act, workspace=ws,
                  tiled=True, paired=True, prequantized=True)
        w = w_down[c]
        ops.qgemv(act, w.packed_values, w.scales, w.zero_points, bits=8, n=H, k=FFN, epilogue=ops.EPI_RESIDUAL, residual=h1, out=h2,
                  workspace=ws, tiled=True)

    for i in range(max(1, args.warmup)):
        launch(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        launch(i)
    end.record()
    torch.cuda.synchronize()
    from cacheir_b200 import _lib
    emit({"micro": "decoder_layer", "batch": B, "context": ctx, "launches_per_step": 8 if fused_prepass else 9, "steps": args.steps,
          "us_per_step_eager": round(start.elapsed_time(end) * 1e3 / args.steps, 2), "peak": peak, "peak_source": f"of {kind}",
          "device_status": _lib.load().cacheir_b200_device_status(0)})


_RESULT_STREAM = None


def claim_stdout() -> None:
    """Keep the caller's stdout for the one JSON line: everything else that writes to file
    descriptor 1 from here on (library banners from native code included) goes to stderr."""
    global _RESULT_STREAM
    if _RESULT_STREAM is None:
        sys.stdout.flush()
        _RESULT_STREAM = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict) -> None:
    stream = _RESULT_STREAM if _RESULT_STREAM is not None else sys.stdout
    stream.write(json.dumps(line) + "\n")
    stream.flush()


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="llama3-8b-int8-b32-ctx2048", choices=sorted(WORKLOADS))
    parser.add_argument("--e2e-steps", type=int, default=32)
    parser.add_argument("--tp", action="store_true",
                        help="all ranks form one tensor-parallel group decoding one batch (default: data parallel by sequence)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--kv", default="fp16", choices=["fp16", "int8"],
                        help="KV page format: fp16 (the benchmark's configuration) or 8-bit pages with a scale per cached row (an extra)")
    parser.add_argument("--separate-attention-prepass", action="store_true",
                        help="diagnostic: run the o projection's activation pre-pass as its own launch instead of inside the attention kernel")
    parser.add_argument("--no-tp-leg", action="store_true", help="with --gpus N > 1: skip the tensor-parallel leg attached to the line")
    parser.add_argument("--micro", choices=["qgemv", "attention", "layer"],
                        help="time one kernel alone, or the kernels of one decoder layer of the 8B-shaped step (profiling aid)")
    parser.add_argument("--m", type=int, default=32)
    parser.add_argument("--n", type=int, default=14336)
    parser.add_argument("--k", type=int, default=4096)
    parser.add_argument("--bits", type=int, default=8)
    parser.add_argument("--group", type=int, default=0)
    parser.add_argument("--epilogue", default="none", choices=["none", "swiglu"])
    parser.add_argument("--copies", type=int, default=4)
    parser.add_argument("--workspace", action="store_true", help="give qgemv its scratch (integer tensor-core path)")
    parser.add_argument("--tiled", action="store_true", help="weights in the tile order of pack_relayout")
    parser.add_argument("--batch", type=int, default=64)
    parser.add_argument("--ctx-min", type=int, default=512)
    parser.add_argument("--ctx-max", type=int, default=8192)
    parser.add_argument("--splits", type=int, default=0)
    parser.add_argument("--ctx-log", action="store_true", help="--micro attention: log-uniform context lengths")
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv-heads", type=int, default=8)
    args = parser.parse_args()
    claim_stdout()
    if args.micro:
        run_micro(args)
        return
    cfg = dict(WORKLOADS[args.workload])
    if args.kv == "int8":
        cfg["kv_dtype"] = "int8"
    if "ctx_range" in cfg:
        lens_all = context_lengths(cfg)
        cfg["ctx"] = max(lens_all)                      # sizing (positions, page-table width)
        cfg["ctx_mean"] = int(np.mean(lens_all))
    warmup = max(3, args.warmup)

    if args.impl == "reference":
        run_reference_arm(args, dict(cfg, ctx=cfg.get("ctx_mean", cfg["ctx"])), args.workload)   # ragged: the mean context
        return

    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: cacheir_b200 has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist  # type: ignore[no-redef]
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank))

    line = measure(args, cfg, args.workload, bool(args.tp and world > 1), world, rank, local_rank, dist,
                   steps=args.steps, warmup=warmup, e2e_steps=max(4, args.e2e_steps), full=True)
    if world > 1 and not args.tp and not args.no_tp_leg:
        # A tensor-parallel leg in the same process group, attached to the data-parallel line: the 70B-shaped
        # configuration on 8 GPUs, the same code path at a small size on 2 and 4.
        tp_workload = "llama3-70b-int4g128-b128-tp8" if world == 8 else "small-tp"
        tp_cfg = dict(WORKLOADS[tp_workload])
        lens_all = context_lengths(tp_cfg)
        tp_cfg["ctx"] = max(lens_all)
        tp_cfg["ctx_mean"] = int(np.mean(lens_all))
        tp_line = measure(args, tp_cfg, tp_workload, True, world, rank, local_rank, dist,
                          steps=min(args.steps, 16), warmup=3, e2e_steps=4, full=False)
        parity = tensor_parallel_parity(rank, world, local_rank)
        if rank == 0 and line is not None and tp_line is not None:
            ar = [k for k in tp_line["kernels"] if k["kernel"].startswith("peer_all_reduce")]
            line["tp"] = {"workload": tp_workload, "tokens_per_s": tp_line["value"], "ms_per_step": tp_line["ms_per_step"],
                          "e2e_tokens_per_s": tp_line["e2e"]["value"], "steps": tp_line["steps"],
                          "frac_of_hbm_roofline": tp_line["step"]["frac_of_hbm_roofline"],
                          "all_reduce_us": ar[0]["us"] if ar else None, "device_status": tp_line["device_status"],
                          "kernels": tp_line["kernels"], "parallelism": tp_line["config"]["parallelism"], **(parity or {})}
    if rank == 0 and line is not None:
        emit(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def measure(args, cfg: dict, workload: str, use_tp: bool, world: int, rank: int, local_rank: int, dist, *, steps: int,
            warmup: int, e2e_steps: int, full: bool) -> dict | None:
    """One measurement of `workload`: data parallel by sequence (every rank its own batch), or, with `use_tp`, all
    ranks as one tensor-parallel group on one batch. Returns the result line on rank 0. `full` adds the CPU
    baseline and the parity self-check."""
    import torch

    from cacheir_b200.sharding import max_over_ranks

    extra = warmup + steps + e2e_steps + 3 + 48
    tp = None
    if use_tp:
        from cacheir_b200.tensor_parallel import TensorParallel
        tp = TensorParallel(rank, world)
    rt, _ = build_runtime(cfg, local_rank, extra, tp, cfg.get("kv_dtype", "same"), not args.separate_attention_prepass)
    sessions = prefill_synthetic_context(rt, cfg)
    first_tokens = [int(t) for t in np.random.default_rng(0 if tp else rank).integers(0, cfg["vocab"], cfg["batch"])]
    replicas = 1 if tp else world                          # independent batches in flight

    def barrier() -> None:
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident loop: `value` ------------------------------------------------
    toks = rt.decode_greedy_batch(sessions, first_tokens, warmup)     # eager step, graph capture, replays
    last = [int(t) for t in toks[-1].tolist()]
    plan = rt._engine.plan_for(sessions)
    launches_per_step = plan.launches_per_step + 1                    # + the feedback argmax
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    toks = rt.decode_greedy_batch(sessions, last, steps)
    end.record()
    barrier()
    elapsed_s = start.elapsed_time(end) * 1e-3
    clocks = sampler.stop()
    last = [int(t) for t in toks[-1].tolist()]
    kv_tokens_mid = unique_kv_tokens(cfg, warmup + steps // 2)
    elapsed_s = max_over_ranks(elapsed_s, torch.device("cuda", local_rank))
    tokens_total = replicas * cfg["batch"] * steps
    value = tokens_total / elapsed_s

    # ---- host-facing loop: `e2e` ------------------------------------------------------
    from cacheir_b200.scheduler import argmax_tokens

    token_ids = last
    for _ in range(2):
        token_ids = argmax_tokens(rt.run_decode_batch(sessions, token_ids))
    barrier()
    h2d = d2h = 0
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        pages_before = sum(len(s.kv_cache.pages) for s in sessions)
        logits = rt.run_decode_batch(sessions, token_ids)             # host ids in (pinned staging + H2D)
        token_ids = argmax_tokens(logits)                             # argmax ids out (D2H)
        h2d += cfg["batch"] * 8
        if sum(len(s.kv_cache.pages) for s in sessions) != pages_before:
            h2d += plan.page_table.numel() * 4
        d2h += cfg["batch"] * 8
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_s = max_over_ranks(e2e_s, torch.device("cuda", local_rank))
    e2e_value = replicas * cfg["batch"] * e2e_steps / e2e_s

    # ---- per-kernel roofline (rank 0 reports) -------------------------------------------
    peak, peak_kind = measured_peaks()
    attn = time_attention_kernel(rt, sessions, cfg)
    gemvs = time_gemv_kernels(rt, cfg)
    kernels = []
    for k in [attn] + gemvs:
        gbs = k["bytes"] / k["seconds"] / 1e9
        kernels.append({"kernel": k["kernel"], "us": round(k["seconds"] * 1e6, 2), "algorithmic_bytes": int(k["bytes"]),
                        "achieved_gbs": round(gbs, 1), "frac": round(gbs / peak, 4), **({"shape": k["shape"]} if "shape" in k else {})})
    if tp and rt._engine.peer_mode:
        # the all-reduce that follows the o- and down-projection: [batch, hidden] over all ranks (every rank runs the
        # same sequence of calls; NVLink bytes per rank: what it reads from and pushes to its peers)
        peer = rt._engine.peer_collectives(cfg["batch"])
        ar_out = torch.empty((cfg["batch"], cfg["hidden"]), device=rt.device, dtype=torch.float16)
        calls = [0]

        def one_all_reduce() -> None:
            peer.all_reduce(calls[0] % 2, ar_out)
            calls[0] += 1

        dist.barrier()
        ar_s = max_over_ranks(time_graph(one_all_reduce, 16), torch.device("cuda", local_rank))
        msg = ar_out.numel() * 2
        two_step = world >= peer.two_step_ranks and msg >= peer.two_step_bytes
        link = msg * (2 * (world - 1) / world if two_step else (world - 1))
        kernels.append({"kernel": "peer_all_reduce" + ("_two_step" if two_step else ""), "us": round(ar_s * 1e6, 2),
                        "algorithmic_bytes": int(link), "achieved_gbs": round(link / ar_s / 1e9, 1), "bound": "nvlink",
                        "shape": [cfg["batch"], cfg["hidden"]]})
    sb = step_bytes(cfg, kv_tokens_mid)
    shards = world if tp else 1                              # tensor parallel: each rank streams its share of the step
    step_gbs = sb["total"] / shards / (elapsed_s / steps) / 1e9
    parity = parity_self_check(rt, sessions, cfg) if (full and rank == 0) else None
    torch.cuda.synchronize()
    from cacheir_b200 import _lib
    status = int(_lib.load().cacheir_b200_device_status(0))   # 0: no bounded device wait ever gave up

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": elapsed_s / steps * 1e3, "higher_is_better": True, "scaling": "strong" if tp else "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(cfg, workload, world, bool(tp)),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d // e2e_steps, "d2h_bytes_per_step": d2h // e2e_steps,
                    "steps": e2e_steps, "api": "B200DecodeRuntime.run_decode_batch + argmax_tokens"},
            "gpu_launches": launches_per_step * steps,
            "device_status": status,
            "clocks": clocks,
            # DRAM traffic of the attention kernel: ncu measured dram__bytes_read + dram__bytes_write = 1.024 x the
            # algorithmic bytes on a small case (K/V bytes dominate both, so the ratio carries over to this workload)
            "roofline": {"bound": "hbm", "kernel": attn["kernel"], "achieved": kernels[0]["achieved_gbs"], "peak": peak,
                         "unit": "GB/s", "frac": kernels[0]["frac"], "traffic": int(ATTENTION_TRAFFIC_RATIO * attn["bytes"]),
                         "traffic_source": f"{ATTENTION_TRAFFIC_RATIO} x algorithmic bytes (ncu, profiles/paged_decode_mma_b16_ctx2048-4096.md)",
                         "peak_source": f"of {peak_kind}",
                         "algorithmic_bytes_per_launch": int(attn["bytes"]), "us_per_launch": kernels[0]["us"]},
            "kernels": kernels,
            "step": {"algorithmic_bytes": int(sb["total"]), "weight_bytes": int(sb["weights"]), "kv_bytes": int(sb["kv"]),
                     "achieved_gbs": round(step_gbs, 1), "frac_of_hbm_roofline": round(step_gbs / peak, 4),
                     "roofline_tokens_per_s": round(cfg["batch"] * peak * 1e9 * shards / sb["total"], 1),
                     "launches_per_step": launches_per_step},
        }
        if parity is not None:
            line["parity"] = parity
        if full and world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = run_cpu_baseline(dict(cfg, ctx=cfg.get("ctx_mean", cfg["ctx"])))
    # give the memory back before another measurement in the same process
    if rt._engine.peer is not None:
        if dist is not None:
            dist.barrier()
        rt._engine.peer.close()
    del plan, sessions, rt, attn, gemvs
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return line


if __name__ == "__main__":
    main()
