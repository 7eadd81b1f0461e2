"""Tensor parallelism for the decode step (the 70B-shaped configuration on 8 GPUs).

Megatron-style split of one decoder layer over `world` ranks, applied to the
reference's packed weights after quantization, so every rank holds a slice of the
*same* integer codes the single-GPU model has:

* column-parallel (rows of W sliced): Q, K, V (whole heads per rank), gate, up, lm_head.
  Per-row scales and zero points are sliced with their rows.
* row-parallel (the K dimension sliced): O and down. A row keeps its scale and zero
  point; group-wise scales are sliced with their groups. Each rank produces a partial
  sum over its K slice; the residual is added on rank 0 only and one all-reduce (sum)
  completes the output on every rank.
* each rank owns `kv_heads / world` KV heads, so its page pool holds only those heads
  and attention needs no exchange; the page table is the same on every rank.
* lm_head logits are all-gathered so every rank sees `[B, vocab]` and picks the same
  greedy token.

The reference has no multi-device execution (its CUDA runtime is one process on one
device, cacheir/runtime/cuda.py:430-506); this module extends its per-layer graph
(cacheir/importers/hf.py:171-268) without changing op names or weight formats.
Collectives go through `torch.distributed` (NCCL on GPUs; gloo in the CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from .quantization import B200PackedWeight


@dataclass(frozen=True)
class TensorParallel:
    rank: int
    world: int
    group: Any = None          # a torch.distributed process group (None = the default group)

    def __post_init__(self) -> None:
        if self.world < 1 or not (0 <= self.rank < self.world):
            raise ValueError(f"bad tensor-parallel rank {self.rank} of {self.world}")

    @property
    def enabled(self) -> bool:
        return self.world > 1

    def check_model(self, *, heads: int, kv_heads: int, intermediate: int, vocab: int) -> None:
        for name, value in (("attention heads", heads), ("KV heads", kv_heads), ("intermediate size", intermediate),
                            ("vocabulary", vocab)):
            if value % self.world != 0:
                raise ValueError(f"{name} ({value}) is not divisible by the tensor-parallel size {self.world}")

    # -- collectives (enqueued on the current stream; NCCL captures into CUDA graphs) -------------
    def all_reduce_sum(self, t: torch.Tensor) -> None:
        if self.enabled:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)

    def all_gather_columns(self, local: torch.Tensor, gathered: torch.Tensor, out: torch.Tensor) -> None:
        """local [B, n] on every rank -> out [B, world*n] (rank r's columns at [r*n, (r+1)*n)).
        `gathered` is a [world*B, n] staging buffer (rank-major)."""
        if not self.enabled:
            out.copy_(local)
            return
        dist.all_gather_into_tensor(gathered, local, group=self.group)
        b, n = int(local.shape[0]), int(local.shape[1])
        out.view(b, self.world, n).copy_(gathered.view(self.world, b, n).permute(1, 0, 2))


def _rows(w: B200PackedWeight | torch.Tensor, start: int, stop: int) -> B200PackedWeight | torch.Tensor:
    if isinstance(w, torch.Tensor):
        return w[start:stop].contiguous()
    if w.tiled:
        raise ValueError("shard the reference row layout, then tile the shard")
    zp = None if w.zero_points is None else w.zero_points[start:stop].contiguous()
    zpi = None if w.zero_points_i32 is None else w.zero_points_i32[start:stop].contiguous()
    scales = w.scales[start:stop].contiguous()
    return B200PackedWeight(w.packed_values[start:stop].contiguous(), scales, zp, w.bits, (stop - start, w.shape[1]),
                            group_size=w.group_size, zero_points_i32=zpi)


def shard_rows(w: B200PackedWeight | torch.Tensor, tp: TensorParallel) -> B200PackedWeight | torch.Tensor:
    """Column-parallel shard: rank r keeps output rows [r*N/world, (r+1)*N/world)."""
    n = int(w.shape[0])
    if n % tp.world != 0:
        raise ValueError(f"{n} output rows do not split over {tp.world} ranks")
    per = n // tp.world
    return _rows(w, tp.rank * per, (tp.rank + 1) * per)


def shard_columns(w: B200PackedWeight | torch.Tensor, tp: TensorParallel) -> B200PackedWeight | torch.Tensor:
    """Row-parallel shard: rank r keeps input columns [r*K/world, (r+1)*K/world) of every row.
    Rows keep their scale and zero point; group-wise scales are sliced with their groups."""
    k = int(w.shape[1])
    if k % tp.world != 0:
        raise ValueError(f"{k} input columns do not split over {tp.world} ranks")
    per = k // tp.world
    lo, hi = tp.rank * per, (tp.rank + 1) * per
    if isinstance(w, torch.Tensor):
        return w[:, lo:hi].contiguous()
    if w.tiled:
        raise ValueError("shard the reference row layout, then tile the shard")
    if w.bits == 4:
        if per % 2 != 0:
            raise ValueError("an int4 K slice must start on a byte boundary")
        codes = w.packed_values[:, lo // 2:hi // 2].contiguous()
    else:
        codes = w.packed_values[:, lo:hi].contiguous()
    scales = w.scales
    if w.group_size:
        if per % w.group_size != 0:
            raise ValueError("a K slice must hold whole quantization groups")
        scales = w.scales.reshape(int(w.shape[0]), -1)[:, lo // w.group_size:hi // w.group_size].contiguous()
    return B200PackedWeight(codes, scales, w.zero_points, w.bits, (int(w.shape[0]), per), group_size=w.group_size,
                            zero_points_i32=w.zero_points_i32)


class _RawCudaBuffer:
    """Lets torch wrap device memory that this library allocated (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerCollectives:
    """The library's own all-reduce / all-gather over NVLink peer memory (include/cacheir_b200.h,
    `cacheir_b200_peer_*`): three data buffers per rank (A and B alternate between consecutive
    all-reduces, C carries the logits slice), one flag array, the gather buffer of the two-step
    all-reduce (messages of `two_step_bytes` and more on `two_step_ranks` ranks and more) and the two receive
    areas of the flagged-word all-reduce (messages up to `flagged_word_bytes`), all mapped into every peer through CUDA IPC. Unlike a library collective these are plain kernels of this package, so a whole
    tensor-parallel step can be captured into one CUDA graph. All ranks must construct it, and
    issue its calls, in the same order."""

    two_step_bytes = 256 * 1024       # the two-step all-reduce pays a second round of flags: worth it only when
    two_step_ranks = 4                # it saves much NVLink traffic, (world-1) against 2 (world-1)/world messages
    flagged_word_bytes = 1024 * 1024  # up to this size the all-reduce with the flag inside every word is the fastest
                                      # (8 GPUs: 14 / 15 / 23 us for 128 KB / 512 KB / 2 MB against 21 / 18 / 22 us with flag rounds)

    def __init__(self, tp: TensorParallel, device: torch.device, data_bytes: int):
        import ctypes

        from . import _lib
        from ._lib import check

        if not tp.enabled:
            raise ValueError("peer collectives need more than one rank")
        self.tp = tp
        self.device = device
        self.data_bytes = (int(data_bytes) + 255) // 256 * 256
        self._lib = _lib.load()
        self._ctypes = ctypes
        self._local: list[int] = []
        self._opened: list[int] = []
        handles: list[bytes] = []
        with torch.cuda.device(device):
            # A, B, C, flags, gather, and the two areas of the flagged-word all-reduce (2 parities x 2 x the message each)
            for nbytes in (self.data_bytes, self.data_bytes, self.data_bytes, 256, self.data_bytes, 4 * self.data_bytes, 4 * self.data_bytes):
                ptr = ctypes.c_void_p()
                handle = (ctypes.c_ubyte * 64)()
                check(self._lib.cacheir_b200_peer_alloc(nbytes, ctypes.byref(ptr), handle), "peer_alloc")
                self._local.append(int(ptr.value))
                handles.append(bytes(handle))
            everyone: list[Any] = [None] * tp.world
            dist.all_gather_object(everyone, handles, group=tp.group)
            # pointer tables [buffer][rank]
            self._ptrs: list[list[int]] = [[0] * tp.world for _ in range(7)]
            for r in range(tp.world):
                for b in range(7):
                    if r == tp.rank:
                        self._ptrs[b][r] = self._local[b]
                    else:
                        ptr = ctypes.c_void_p()
                        blob = (ctypes.c_ubyte * 64).from_buffer_copy(everyone[r][b])
                        check(self._lib.cacheir_b200_peer_open(blob, ctypes.byref(ptr)), "peer_open")
                        self._ptrs[b][r] = int(ptr.value)
                        self._opened.append(int(ptr.value))
            self._tables = [(ctypes.c_void_p * tp.world)(*self._ptrs[b]) for b in range(7)]
            self.state = torch.zeros((4,), device=device, dtype=torch.int32)
            self._views = [torch.as_tensor(_RawCudaBuffer(self._local[b], self.data_bytes), device=device) for b in range(3)]
        dist.barrier(group=tp.group)

    def buffer(self, index: int, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """A [rows, cols] view of local data buffer `index` (0 = A, 1 = B, 2 = C) for a producer kernel to fill."""
        nbytes = rows * cols * torch.empty((), dtype=dtype).element_size()
        if nbytes > self.data_bytes:
            raise ValueError(f"a peer buffer holds {self.data_bytes} bytes, {nbytes} requested")
        return self._views[index][:nbytes].view(dtype).view(rows, cols)

    def all_reduce(self, index: int, out: torch.Tensor) -> None:
        """out = sum over ranks of their buffer `index` (same shape and dtype as `out`), identical bits on every rank."""
        from . import ops
        from ._lib import check

        nbytes = out.numel() * out.element_size()
        if nbytes <= min(self.flagged_word_bytes, self.data_bytes) and nbytes % (4 * self.tp.world) == 0:
            check(self._lib.cacheir_b200_peer_all_reduce_ll(self._ptrs[index][self.tp.rank], self._tables[5], self._tables[6],
                                                            out.data_ptr(), out.numel(), ops.dtype_code(out.dtype),
                                                            self.tp.rank, self.tp.world, self.state.data_ptr(),
                                                            ops._stream()), "peer_all_reduce_ll")
            return
        if self.tp.world >= self.two_step_ranks and nbytes >= self.two_step_bytes and nbytes % (16 * self.tp.world) == 0:
            check(self._lib.cacheir_b200_peer_all_reduce_two_step(self._tables[index], self._tables[4], self._tables[3],
                                                                  out.data_ptr(), out.numel(), ops.dtype_code(out.dtype),
                                                                  self.tp.rank, self.tp.world, self.state.data_ptr(),
                                                                  ops._stream()), "peer_all_reduce_two_step")
            return
        check(self._lib.cacheir_b200_peer_all_reduce(self._tables[index], self._tables[3], out.data_ptr(), out.numel(),
                                                     ops.dtype_code(out.dtype), self.tp.rank, self.tp.world,
                                                     self.state.data_ptr(), ops._stream()), "peer_all_reduce")

    def all_gather_columns(self, index: int, out: torch.Tensor) -> None:
        """out [rows, world*cols] from every rank's [rows, cols] slice in its buffer `index`."""
        from . import ops
        from ._lib import check

        rows, cols = int(out.shape[0]), int(out.shape[1]) // self.tp.world
        check(self._lib.cacheir_b200_peer_all_gather(self._tables[index], self._tables[3], out.data_ptr(), rows, cols,
                                                     ops.dtype_code(out.dtype), self.tp.rank, self.tp.world,
                                                     self.state.data_ptr(), ops._stream()), "peer_all_gather")

    def set_poll_limit(self, polls: int) -> None:
        """How many times a collective polls for a peer before it gives up (0: the library default, about a
        second). A kernel that gives up records a code in the device status word and returns; until the host has
        read and cleared that word (`device_status`), later collectives return at once."""
        self.state[3] = int(polls)

    def device_status(self, reset: bool = True) -> int:
        """The library's device status word (0: every bounded wait so far was satisfied). Synchronises the device."""
        return int(self._lib.cacheir_b200_device_status(1 if reset else 0))

    def close(self) -> None:
        """Unmap the peers' buffers and free the local ones (call on every rank, after a barrier)."""
        torch.cuda.synchronize(self.device)
        for ptr in self._opened:
            self._lib.cacheir_b200_peer_close(self._ctypes.c_void_p(ptr))
        self._opened = []
        self._views = []
        for ptr in self._local:
            self._lib.cacheir_b200_peer_free(self._ctypes.c_void_p(ptr))
        self._local = []
