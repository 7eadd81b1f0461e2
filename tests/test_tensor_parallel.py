"""Tensor-parallel sharding of packed weights.

CPU part (gloo, two ranks): the shards are slices of the same integer codes, so the partial
products of a row-parallel projection all-reduce to the full product and the column-parallel
shards concatenate to it -- checked with the oracle's dequantisation on the host.
GPU part (two B200s, skipped with fewer): a two-layer int8 model decoded with TP=2 produces the
logits and greedy tokens of the single-GPU runtime.
"""
from __future__ import annotations

import os
import socket
import zlib

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle
from cacheir_b200.quantization import B200PackedWeight
from cacheir_b200.tensor_parallel import TensorParallel, shard_columns, shard_rows


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _host_packed(rng, n, k, bits, group=0):
    """A packed weight on the host in the runtime's container type."""
    w = rng.standard_normal((n, k)).astype(np.float32) * 0.05
    if group:
        codes = rng.integers(0, 16, (n, k)).astype(np.uint8)
        packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
        scales = rng.uniform(0.005, 0.02, (n, k // group)).astype(np.float16)
        return B200PackedWeight(torch.from_numpy(packed), torch.from_numpy(scales), None, 4, (n, k), group_size=group)
    ref = oracle.pack_quantized_weight(w, f"int{bits}")
    return B200PackedWeight(torch.from_numpy(ref.packed_values), torch.from_numpy(ref.scales.astype(np.float32)),
                            torch.from_numpy(ref.zero_points.astype(np.float32)), bits, (n, k),
                            zero_points_i32=torch.from_numpy(ref.zero_points.astype(np.int32)))


def _dequant(w: B200PackedWeight) -> np.ndarray:
    n, k = w.shape
    codes = w.packed_values.numpy()
    if w.bits == 4:
        q = np.empty((n, codes.shape[1] * 2), dtype=np.float32)
        q[:, 0::2] = codes & 0xF
        q[:, 1::2] = codes >> 4
        q = q[:, :k]
    else:
        q = codes.astype(np.float32)
    if w.group_size:
        s = np.repeat(w.scales.numpy().astype(np.float32).reshape(n, -1), w.group_size, axis=1)
        return (q - 8.0) * s
    return (q - w.zero_points.numpy()[:, None]) * w.scales.numpy()[:, None]


def test_shards_partition_the_codes():
    rng = np.random.default_rng(0)
    for bits, group in ((8, 0), (4, 0), (4, 128)):
        w = _host_packed(rng, 64, 512, bits, group)
        full = _dequant(w)
        for world in (2, 4):
            rows = [_dequant(shard_rows(w, TensorParallel(r, world))) for r in range(world)]
            cols = [_dequant(shard_columns(w, TensorParallel(r, world))) for r in range(world)]
            np.testing.assert_array_equal(np.concatenate(rows, axis=0), full)
            np.testing.assert_array_equal(np.concatenate(cols, axis=1), full)
    with pytest.raises(ValueError):
        shard_rows(_host_packed(rng, 10, 128, 8), TensorParallel(0, 4))
    with pytest.raises(ValueError):
        shard_columns(_host_packed(rng, 8, 384, 4, 128), TensorParallel(0, 2))      # 192 columns: not whole groups
    with pytest.raises(ValueError):
        TensorParallel(2, 2)
    with pytest.raises(ValueError):
        TensorParallel(0, 4).check_model(heads=8, kv_heads=2, intermediate=64, vocab=64)


def _cpu_worker(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp = TensorParallel(rank, world)
        rng = np.random.default_rng(3)                     # same weights and activations on every rank
        x = rng.standard_normal((5, 256)).astype(np.float32)
        w_row = _host_packed(rng, 48, 256, 8)              # row-parallel (o / down): slice K
        w_col = _host_packed(rng, 64, 256, 4, 128)         # column-parallel (lm_head): slice N
        k0, k1 = rank * 128, (rank + 1) * 128
        partial = torch.from_numpy(x[:, k0:k1] @ _dequant(shard_columns(w_row, tp)).T)
        tp.all_reduce_sum(partial)
        local = torch.from_numpy(x @ _dequant(shard_rows(w_col, tp)).T)
        gathered = torch.empty((world * local.shape[0], local.shape[1]))
        out = torch.empty((5, 64))
        tp.all_gather_columns(local, gathered, out)
        results[rank] = {"row": partial.numpy(), "col": out.numpy(),
                         "row_full": x @ _dequant(w_row).T, "col_full": x @ _dequant(w_col).T}
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_ranks_reduce_and_gather_to_the_unsharded_product():
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_cpu_worker, args=(r, 2, port, results), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.kill()
    assert not stuck and all(p.exitcode == 0 for p in procs)
    for r in range(2):
        np.testing.assert_allclose(results[r]["row"], results[r]["row_full"], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(results[r]["col"], results[r]["col_full"], rtol=1e-5, atol=1e-5)
    np.testing.assert_array_equal(results[0]["row"], results[1]["row"])      # every rank ends with the same sum


# ---- GPU: TP=2 against the single-GPU runtime ------------------------------------------------
def _peer_collectives_check(rank: int, world: int) -> dict:
    """The library's own all-reduce / all-gather: eager calls alternating buffers, then a captured graph replayed."""
    from cacheir_b200.tensor_parallel import PeerCollectives

    dev = torch.device("cuda", rank)
    peer = PeerCollectives(TensorParallel(rank, world), dev, 512 * 1024)
    peer.two_step_ranks = 2                                  # exercise the two-step kernel on two ranks as well
    gens = [torch.Generator(device="cpu") for _ in range(world)]
    report = {"reduce_ok": True, "gather_ok": True, "graph_ok": True}
    # a small message (one step: every rank reads every buffer) and one past the two-step threshold
    # (reduce-scatter + all-gather inside one launch), each first with the flag inside every word (the default for
    # messages of this size), then with the flag rounds
    for rows, cols, flagged in ((8, 512, True), (128, 2048, True), (8, 512, False), (128, 2048, False)):
        assert (rows * cols * 2 >= PeerCollectives.two_step_bytes) == (rows == 128)
        peer.flagged_word_bytes = PeerCollectives.flagged_word_bytes if flagged else 0
        assert rows * cols * 2 <= PeerCollectives.flagged_word_bytes
        out = torch.empty((rows, cols), device=dev, dtype=torch.float16)
        for call in range(6):                                   # every rank can regenerate every rank's data
            parts = []
            for r in range(world):
                gens[r].manual_seed(1000 * call + r + rows)
                parts.append(torch.randn((rows, cols), generator=gens[r]).half())
            which = call % 2
            peer.buffer(which, rows, cols, torch.float16).copy_(parts[rank].to(dev))
            peer.all_reduce(which, out)
            want = sum(p.float() for p in parts).half()          # rank order, fp32 accumulation, one rounding
            report["reduce_ok"] &= bool(torch.equal(out.cpu(), want))
        if rows == 8:
            wide = torch.empty((rows, cols * world), device=dev, dtype=torch.float16)
            peer.buffer(2, rows, cols, torch.float16).copy_(parts[rank].to(dev))
            peer.all_gather_columns(2, wide)
            report["gather_ok"] = bool(torch.equal(wide.cpu(), torch.cat(parts, dim=1)))
        # captured: the producer copy and the collective replay together; the call counter lives on the device
        src = parts[rank].to(dev)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for which in (0, 1):
                peer.buffer(which, rows, cols, torch.float16).copy_(src)
                peer.all_reduce(which, out)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        report["graph_ok"] &= bool(torch.equal(out.cpu(), want))
    from cacheir_b200 import _lib
    report["status"] = int(_lib.load().cacheir_b200_device_status(1))
    dist.barrier()
    peer.close()
    return report


def _gpu_worker(rank: int, world: int, port: int, results, collectives: str = "peer"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["CB200_TP_COLLECTIVES"] = collectives
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))     # a lost rank ends the others' collectives quickly
    try:
        from cacheir_b200 import B200DecodeRuntime
        from cacheir_b200.artifact import ModelConfig, build_decoder_artifact

        cfg = ModelConfig(architecture="LlamaForCausalLM", hidden_size=512, intermediate_size=1024, num_layers=2,
                          num_attention_heads=4, num_key_value_heads=2, vocab_size=512, max_position_embeddings=256,
                          rope_theta=10000.0, rms_norm_eps=1e-5, dtype="float16")
        artifact = build_decoder_artifact(cfg, quant="int8")

        def source(key, shape):                           # identical synthetic weights on every rank
            g = torch.Generator(device="cpu")
            g.manual_seed(zlib.crc32(key.encode()))
            if len(shape) == 1:
                return torch.ones(shape)
            return torch.randn(shape, generator=g) * 0.05

        prompts = [[3, 17, 200, 45, 9, 310, 77, 5], [8, 1, 499, 23, 64, 2, 11, 90]]
        outs = {}
        if collectives == "peer":
            outs["collectives"] = _peer_collectives_check(rank, world)
        for name, tp in (("tp", TensorParallel(rank, world)), ("single", None)):
            if name == "single" and rank != 0:
                continue
            rt = B200DecodeRuntime(artifact, device=f"cuda:{rank}", dtype="float16", tensor_source=source,
                                   max_seq_len=256, tensor_parallel=tp)
            sessions = [rt.fork() for _ in prompts]
            logits = rt.run_prefill_batch(sessions, prompts)
            trace = [logits[:, -1].float().cpu().numpy()]
            generated = [[int(t) for t in logits[:, -1].argmax(dim=-1).tolist()]]
            forced = [[41, 7], [300, 12], [5, 5], [128, 64], [2, 509], [77, 30]]      # the same next tokens for both runs
            for tokens in forced:
                logits = rt.run_decode_batch(sessions, tokens)
                generated.append([int(t) for t in logits[:, -1].argmax(dim=-1).tolist()])
                trace.append(logits[:, -1].float().cpu().numpy())
            outs[name] = {"tokens": generated, "logits": np.stack(trace)}
            if name == "tp":
                dist.barrier()
        results[rank] = outs
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.timeout(400)
@pytest.mark.parametrize("collectives", ["peer", "nccl"])
def test_tp2_matches_single_gpu(collectives):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_worker, args=(r, 2, port, results, collectives), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:                       # never leave a rank behind: a stuck collective would outlive the test
        p.kill()
    assert not stuck, "a tensor-parallel rank did not finish in time"
    assert all(p.exitcode == 0 for p in procs)
    if collectives == "peer":
        for r in range(2):
            assert results[r]["collectives"] == {"reduce_ok": True, "gather_ok": True, "graph_ok": True, "status": 0}
    single, tp0, tp1 = results[0]["single"], results[0]["tp"], results[1]["tp"]
    np.testing.assert_array_equal(tp0["logits"], tp1["logits"])          # both ranks hold the same gathered logits
    # fp16 partial sums and per-rank activation scales across two layers: twice the single-kernel gate
    assert oracle.rel_l2(tp0["logits"], single["logits"]) <= 4e-3
    assert tp0["tokens"] == tp1["tokens"]
    # identical greedy tokens wherever the single-GPU top-1 / top-2 margin is clear of that tolerance
    one = single["logits"]
    top2 = np.sort(one, axis=-1)[..., -2:]
    clear = (top2[..., 1] - top2[..., 0]) > 8e-3 * np.abs(one).max(axis=-1)
    assert clear.sum() >= clear.size // 2
    np.testing.assert_array_equal(tp0["logits"].argmax(-1)[clear], one.argmax(-1)[clear])


def _lost_peer_worker():
    """One GPU, world = 2: the second rank's buffers are local stand-ins whose flag never advances."""
    import ctypes

    from cacheir_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    n = 4096
    data0 = torch.ones((n,), device=dev, dtype=torch.float16)
    data1 = torch.full((n,), 2.0, device=dev, dtype=torch.float16)
    flags0 = torch.zeros((64,), device=dev, dtype=torch.int32)
    flags1 = torch.zeros((64,), device=dev, dtype=torch.int32)      # the "peer" never announces into flags0
    out = torch.zeros((n,), device=dev, dtype=torch.float16)
    state = torch.zeros((4,), device=dev, dtype=torch.int32)
    state[3] = 2000                                                 # polls before a wait gives up: a few milliseconds
    data = (ctypes.c_void_p * 2)(data0.data_ptr(), data1.data_ptr())
    flags = (ctypes.c_void_p * 2)(flags0.data_ptr(), flags1.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        return lib.cacheir_b200_peer_all_reduce(data, flags, out.data_ptr(), n, 1, 0, 2, state.data_ptr(), stream)

    import time
    assert lib.cacheir_b200_device_status(1) == 0
    t0 = time.perf_counter()
    assert call() == 0
    torch.cuda.synchronize()
    first = time.perf_counter() - t0
    assert lib.cacheir_b200_device_status(0) == (4 << 8) | 1        # the wait for rank 1 ran out; the kernel returned
    t0 = time.perf_counter()
    for _ in range(50):                                             # later calls do not wait again
        assert call() == 0
    torch.cuda.synchronize()
    later = (time.perf_counter() - t0) / 50
    assert later < max(first / 4, 2e-3), (first, later)
    assert lib.cacheir_b200_device_status(1) == (4 << 8) | 1        # read and cleared
    assert lib.cacheir_b200_device_status(0) == 0
    # a healthy call: the stand-in peer has "announced" every epoch to come
    flags0[1] = 1 << 30
    assert call() == 0
    torch.cuda.synchronize()
    assert lib.cacheir_b200_device_status(1) == 0
    assert torch.equal(out, torch.full_like(out, 3.0))              # 1 + 2, in rank order


def _lost_peer_flagged_word_worker():
    """The all-reduce with the flag inside every word, one GPU, world = 2: rank 1's words never arrive, then a call whose
    words the host has put in place (epoch in the upper half of every 64-bit word)."""
    import ctypes

    from cacheir_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    n, world = 4096, 2
    words = n // 2                  # 32-bit words of an fp16 message
    wps = words // world
    mine = torch.ones((n,), device=dev, dtype=torch.float16)
    areas = [torch.zeros((2 * world * wps,), device=dev, dtype=torch.int64) for _ in range(4)]   # rs0, rs1, ag0, ag1
    out = torch.zeros((n,), device=dev, dtype=torch.float16)
    state = torch.zeros((4,), device=dev, dtype=torch.int32)
    state[3] = 2000
    rs = (ctypes.c_void_p * 2)(areas[0].data_ptr(), areas[1].data_ptr())
    ag = (ctypes.c_void_p * 2)(areas[2].data_ptr(), areas[3].data_ptr())
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        return lib.cacheir_b200_peer_all_reduce_ll(mine.data_ptr(), rs, ag, out.data_ptr(), n, 1, 0, world, state.data_ptr(), stream)

    assert lib.cacheir_b200_device_status(1) == 0
    assert call() == 0
    torch.cuda.synchronize()
    assert lib.cacheir_b200_device_status(0) == (4 << 8) | 3        # a word of rank 1 never came; the kernel returned
    for _ in range(20):                                             # later calls return at once
        assert call() == 0
    torch.cuda.synchronize()
    assert lib.cacheir_b200_device_status(1) == (4 << 8) | 3
    # a healthy call: what rank 1 would have sent (2.0 everywhere) and its finished slice (1 + 2 = 3)
    epoch = int(state[0].item()) + 1
    half = lambda v: int(torch.tensor([v, v], dtype=torch.float16).view(torch.int32).item()) & 0xFFFFFFFF
    base = (epoch & 1) * world * wps
    areas[0][base + 1 * wps: base + 2 * wps] = (epoch << 32) | half(2.0)       # reduce-scatter area, sender 1
    areas[2][base + 1 * wps: base + 2 * wps] = (epoch << 32) | half(3.0)       # all-gather area, owner 1
    assert call() == 0
    torch.cuda.synchronize()
    assert lib.cacheir_b200_device_status(1) == 0
    assert torch.equal(out, torch.full_like(out, 3.0))
    # rank 0 pushed its contribution and its finished slice into "rank 1's" areas, flagged with the epoch
    sent = areas[1][base: base + wps]
    assert torch.equal(sent, torch.full_like(sent, (epoch << 32) | half(1.0)))
    done = areas[3][base: base + wps]
    assert torch.equal(done, torch.full_like(done, (epoch << 32) | half(3.0)))


@pytest.mark.gpu
def test_lost_peer_flagged_word_all_reduce():
    _lost_peer_flagged_word_worker()


@pytest.mark.gpu
def test_lost_peer_times_out_once_and_is_reported():
    """A rank that never shows up costs the others one short, bounded wait; the status word says so and later
    collectives return at once until the host has read it. Made on the host: nothing on the GPU faults or hangs."""
    _lost_peer_worker()
