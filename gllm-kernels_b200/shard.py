"""N-wise (row) sharding of a quantized weight matrix over the ranks of a torch.distributed group.

Rows of W[n, k] are independent in y[t, r] = sum_k W[r, k] * x[t, k]: every rank keeps a contiguous band of
rows (cut at multiples of 16, the row tile of the device layouts), x is replicated, each rank computes its band
of y and ONE all-gather per product puts the bands side by side.  No other data-path collective exists.

The gather buffer is [world, m, band] with `band` the largest band (ragged bands are zero padded), so that
`all_gather_into_tensor` can be used on equal chunks; for m == 1 and equal bands the buffer IS y.
`ShardedLinear` takes the product as a callable, so the same plumbing runs on GPUs over NCCL (GpuKernels)
and in the CPU tests over gloo with a stand-in product.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import numpy as np

from .quant import MXFP4, QuantType

ROW_TILE = 16


def shard_rows(n: int, world: int, rank: int, multiple: int = ROW_TILE) -> Tuple[int, int]:
    """[r0, r1) of `rank`: bands differ by at most one tile; the last band also takes the rows past the last
    full tile."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside 0..{world - 1}")
    tiles = n // multiple
    t0, t1 = tiles * rank // world, tiles * (rank + 1) // world
    r0, r1 = multiple * t0, multiple * t1
    if rank == world - 1:
        r1 = n
    return r0, r1


def band_width(n: int, world: int, multiple: int = ROW_TILE) -> int:
    return max(r1 - r0 for r0, r1 in (shard_rows(n, world, r, multiple) for r in range(world)))


def slice_blocks(qt: QuantType, blocks, n: int, k: int, r0: int, r1: int, scales=None):
    """Rows [r0, r1) of a row-major block buffer (reference formats: rows x k/bs blocks x block bytes).
    MXFP4 in split form (separate scale bytes) returns (blocks, scales)."""
    bs, bb = qt.block_size(), qt.block_bytes()
    if k % bs:
        raise ValueError(f"k={k} is not a multiple of the block size {bs}")
    nb = k // bs
    flat = np.ascontiguousarray(blocks).reshape(-1)
    if qt.id == MXFP4 and scales is not None:
        per_row = nb * (bs // 2)
        if flat.size != n * per_row:
            raise ValueError("block buffer size does not match n x k")
        sc = np.ascontiguousarray(scales).reshape(-1)
        return flat[r0 * per_row:r1 * per_row], sc[r0 * nb:r1 * nb]
    per_row = nb * bb
    if flat.size != n * per_row:
        raise ValueError("block buffer size does not match n x k")
    return flat[r0 * per_row:r1 * per_row]


class ShardedLinear:
    """One row-sharded product.  `product(x, out)` must write this rank's band y[:, r0:r1] (shape [m, r1-r0])
    into `out` (a [m, band] view of the gather buffer, only the first r1-r0 columns are the band)."""

    def __init__(self, n: int, k: int, product: Callable, world: int, rank: int, group=None):
        self.n, self.k, self.world, self.rank, self.group = n, k, world, rank, group
        self.r0, self.r1 = shard_rows(n, world, rank)
        self.band = band_width(n, world)
        self.product = product
        self._buf = None

    def _buffer(self, m: int, like):
        import torch
        if self._buf is None or self._buf.shape[1] != m or self._buf.device != like.device:
            self._buf = torch.zeros((self.world, m, self.band), dtype=torch.float32, device=like.device)
        return self._buf

    def forward(self, x, assemble: bool = True):
        """x [m, k] replicated on every rank -> y [m, n] on every rank (or the raw gather buffer)."""
        import torch.distributed as dist
        m = x.shape[0]
        buf = self._buffer(m, x)
        mine = buf[self.rank]
        self.product(x, mine[:, : self.r1 - self.r0])
        if self.world > 1:
            src = mine.reshape(-1)
            if dist.get_backend(self.group) != "nccl":
                src = src.clone()  # only NCCL documents the in-place form (input = own chunk of the output)
            dist.all_gather_into_tensor(buf.view(-1), src, group=self.group)
        return self.assemble(buf) if assemble else buf

    def assemble(self, buf):
        """[world, m, band] -> [m, n]; free when m == 1 and the bands are equal."""
        import torch
        m = buf.shape[1]
        if self.band * self.world == self.n and m == 1:
            return buf.view(1, self.n)
        parts = []
        for r in range(self.world):
            r0, r1 = shard_rows(self.n, self.world, r)
            parts.append(buf[r, :, : r1 - r0])
        return torch.cat(parts, dim=1)


def gpu_sharded_linear(K, qt: QuantType, blocks, n: int, k: int, world: int, rank: int, scales=None,
                       global_scale: Optional[float] = None, group=None) -> ShardedLinear:
    """Uploads this rank's band of rows to its GPU and returns the sharded product (decode GEMV for m <= 16,
    prefill GEMM above).  `blocks` is the FULL matrix in the reference's block format (host numpy)."""
    r0, r1 = shard_rows(n, world, rank)
    part = slice_blocks(qt, blocks, n, k, r0, r1, scales)
    if isinstance(part, tuple):
        w = K.upload(qt, r1 - r0, k, part[0], part[1])
    elif global_scale is not None:
        w = K.upload(qt, r1 - r0, k, part, None, global_scale)
    else:
        w = K.upload(qt, r1 - r0, k, part)

    def product(x, out):
        # the band is a strided view of the gather buffer: both kernels take a leading dimension
        if x.shape[0] <= 16 and qt.id in (1, 2):
            K.gemv(w, x, y=out)
        else:
            K.gemm(w, x, y=out)

    lin = ShardedLinear(n, k, product, world, rank, group)
    lin.weight = w
    return lin


class PeerExchange:
    """Exchange buffers of the ranks of one node, mapped into each other (CUDA IPC through the C ABI), for the
    GEMV that stores its band of y into every rank's copy.  Layout of each rank's buffer: 256 bytes of barrier
    flags, then `slots` y copies of `slot_floats` f32 each.  The handles travel through the process group
    (all_gather_object: host plumbing, once at set-up)."""

    FLAG_BYTES = 256

    def __init__(self, K, world: int, rank: int, slots: int, slot_floats: int, group=None):
        import torch.distributed as dist
        self.K, self.world, self.rank, self.slots, self.slot_floats = K, world, rank, slots, slot_floats
        self.nbytes = self.FLAG_BYTES + slots * slot_floats * 4
        # Set-up failures (no device memory, IPC not permitted, ...) must not leave other ranks waiting in a
        # collective: every step's outcome is shared before the next one, and all ranks raise together.
        self.local, self.bases, handle, err = None, [], None, None
        try:
            self.local, handle = K.shared_alloc(self.nbytes)
        except Exception as e:
            err = f"rank {rank}: {e}"
        handles = [None] * world
        dist.all_gather_object(handles, (handle, err), group=group)
        errs = [e for (_, e) in handles if e]
        if not errs:
            try:
                self.bases = [self.local if r == rank else K.shared_open(handles[r][0]) for r in range(world)]
            except Exception as e:
                err = f"rank {rank}: {e}"
            opened = [None] * world
            dist.all_gather_object(opened, err, group=group)
            errs = [e for e in opened if e]
        if errs:
            self.close()
            raise RuntimeError("peer exchange set-up failed: " + "; ".join(errs))
        self.peers = [self.bases[r] for r in range(world) if r != rank]
        dist.barrier(group=group)  # every rank has mapped every buffer before anyone writes

    def slot_ptr(self, rank: int, slot: int, offset_floats: int = 0) -> int:
        return self.bases[rank] + self.FLAG_BYTES + (slot * self.slot_floats + offset_floats) * 4

    def local_tensor(self, slot: int, shape):
        """This rank's copy of y in `slot` as a torch tensor (no copy)."""
        import torch
        n = int(np.prod(shape))
        assert n <= self.slot_floats

        class _Raw:  # minimal __cuda_array_interface__ carrier
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (self.slot_ptr(self.rank, slot), False),
                                        "version": 2}
        return torch.as_tensor(raw, device=f"cuda:{self.K.device}").view(*shape)

    def gemv(self, w, x, slot: int, r0: int, n_total: int, stream=None) -> None:
        """y[:, r0:r0 + w.n] of every rank's `slot` (laid out [m, n_total]) = this rank's band."""
        m = x.shape[0]
        dst = [self.slot_ptr(r, slot, r0) for r in range(self.world)]
        mine = dst[self.rank]
        others = [d for r, d in enumerate(dst) if r != self.rank]
        self.K.gemv_allgather(w, x, mine, others, n_total, m, stream)

    def ffn_decode_sharded(self, w_gate_up, w_down, x, slot_h: int, slot_y: int, r0_h: int, r0_y: int, stream=None):
        """The gated feed-forward block with row-sharded weights, two chained exchange products: this rank's band of
        [gate | up] = W_gate_up x is stored into every rank's h [m, 2f] (slot_h), then y = W_down (silu(gate) * up) reads the
        gathered h with SwiGLU applied while staging, and its band goes into every rank's y [m, d] (slot_y).  `w_gate_up` /
        `w_down` are this rank's row bands, r0_h / r0_y their first rows.  Returns (h, y) views of this rank's copies;
        y is complete after `wait()` (or inside the next chained product)."""
        m = x.shape[0]
        two_f, d = 2 * w_down.k, w_gate_up.k
        self.gemv_chained(w_gate_up, x, slot_h, r0_h, two_f, stream)
        h = self.local_tensor(slot_h, (m, two_f))
        dst = [self.slot_ptr(r, slot_y, r0_y) for r in range(self.world)]
        others = [p for r, p in enumerate(dst) if r != self.rank]
        self.K.gemv_exchange(w_down, h, dst[self.rank], others, d, m, self.bases[self.rank], self.peers, self.rank, stream,
                             x_up=h[:, two_f // 2:])
        return h, self.local_tensor(slot_y, (m, d))

    def gemv_chained(self, w, x, slot: int, r0: int, n_total: int, stream=None) -> None:
        """The same product as `gemv` for chains of sharded products: it first waits until every rank has completed
        the previous chained product (so an x that is a gathered y is complete) and signals its own completion from
        the GEMV's last block — no barrier launch in between.  Finish a chain with `wait`."""
        m = x.shape[0]
        dst = [self.slot_ptr(r, slot, r0) for r in range(self.world)]
        others = [d for r, d in enumerate(dst) if r != self.rank]
        self.K.gemv_exchange(w, x, dst[self.rank], others, n_total, m, self.bases[self.rank], self.peers, self.rank, stream)

    def wait(self, stream=None) -> None:
        """After the last `gemv_chained` of a chain: returns (on the stream) when its bands have landed here."""
        self.K.exchange_wait(self.bases[self.rank], self.world - 1, self.rank, stream)

    def barrier(self, stream=None) -> None:
        """After this rank's products: returns (on the stream) when every rank's bands have landed here."""
        # sequence number 0 = the counter in the flag area: the launch can be captured in a graph and replayed
        self.K.peer_barrier(self.bases[self.rank], self.peers, self.rank, 0, stream)

    def close(self) -> None:
        for r, b in enumerate(self.bases):
            if r != self.rank and b:
                self.K.shared_close(b)
        if self.local:
            self.K.shared_free(self.local)
        self.bases, self.local = [], None
