"""Row sharding over a process group: two gloo ranks on CPU.  The product on each rank is the CPU oracle on
that rank's band of blocks (a stand-in for the GPU kernel), so what is tested is the sharding plumbing: band
limits, slicing of the block bytes, the gather buffer and the assembly of y."""
import importlib
import os
import socket

import numpy as np
import pytest


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, cases, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    gk = importlib.import_module("gllm-kernels_b200")
    from oracle import oracle as O
    try:
        for fmt, n, k, m in cases:
            rng = np.random.default_rng(n + k + m)  # same data on every rank
            W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
            x = rng.standard_normal((m, k)).astype(np.float32)
            if fmt == "q4k":
                qt, oid, blocks, scales = gk.QuantType.q4k(), O.Q4K, O.quantize_q4_k(W), None
            elif fmt == "q8_0":
                qt, oid, blocks, scales = gk.QuantType.q8_0(), O.Q8_0, O.quantize_q8_0(W), None
            else:
                qt, oid = gk.QuantType.mxfp4(32), O.MXFP4
                blocks, scales = O.quantize_mxfp4(W)
            r0, r1 = gk.shard_rows(n, world, rank)
            part = gk.slice_blocks(qt, blocks, n, k, r0, r1, scales)

            def product(xt, out, part=part, r0=r0, r1=r1):
                xn = xt.numpy()
                if isinstance(part, tuple):
                    wd = O.dequant_matrix(oid, part[0], r1 - r0, k, scales=part[1])
                    y = O.gemm_f32_nt(xn, wd)
                else:
                    y = O.quant_matmul(part, np.ascontiguousarray(xn.T), oid, r1 - r0, xn.shape[0], k).T
                out.copy_(torch.from_numpy(np.ascontiguousarray(y)))

            lin = gk.ShardedLinear(n, k, product, world, rank)
            y = lin.forward(torch.from_numpy(x)).numpy()
            if scales is None:
                ref = O.quant_matmul(blocks, np.ascontiguousarray(x.T), oid, n, m, k).T
            else:
                ref = O.gemm_f32_nt(x, O.dequant_matrix(oid, blocks, n, k, scales=scales))
            assert y.shape == (m, n), (y.shape, m, n)
            assert np.array_equal(y, ref), f"rank {rank} {fmt} n={n} k={k} m={m}: max diff {np.abs(y - ref).max()}"
        q.put((rank, "ok"))
    except Exception as e:  # reported to the parent, which fails the test
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_sharded_linear_two_ranks_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    # equal bands with m = 1 (the buffer is y), ragged bands (n = 200: 96 + 104 rows), batch > 1, split-scale MXFP4
    cases = [("q4k", 64, 512, 1), ("q4k", 200, 256, 3), ("q8_0", 176, 96, 2), ("mxfp4", 48, 128, 2)]
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, cases, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=150) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert res == {0: "ok", 1: "ok"}, res


def test_shard_rows_cover_and_align():
    gk = importlib.import_module("gllm-kernels_b200")
    for n in (16, 200, 4096, 28672, 8192, 11008):
        for world in (1, 2, 4, 8):
            bands = [gk.shard_rows(n, world, r) for r in range(world)]
            assert bands[0][0] == 0 and bands[-1][1] == n
            for (a0, a1), (b0, b1) in zip(bands, bands[1:]):
                assert a1 == b0 and a1 % 16 == 0
            widths = [b - a for a, b in bands]
            assert max(widths) - min(widths) <= 16 + n % 16
    with pytest.raises(ValueError):
        gk.shard_rows(64, 2, 2)


def test_slice_blocks_rejects_wrong_sizes():
    gk = importlib.import_module("gllm-kernels_b200")
    qt = gk.QuantType.q8_0()
    with pytest.raises(ValueError):
        gk.slice_blocks(qt, np.zeros(10, np.uint8), 4, 64, 0, 2)
    with pytest.raises(ValueError):
        gk.slice_blocks(qt, np.zeros(4 * 2 * 34, np.uint8), 4, 65, 0, 2)
    part = gk.slice_blocks(qt, np.arange(4 * 2 * 34, dtype=np.uint8) % 251, 4, 64, 1, 3)
    assert part.size == 2 * 2 * 34 and part[0] == (2 * 34) % 251


class _FakeK:
    """Stands in for GpuKernels in the set-up protocol of PeerExchange: no GPU, failures injected on the host."""

    def __init__(self, rank, fail_alloc_on=None, fail_open_on=None):
        self.rank, self.fail_alloc_on, self.fail_open_on, self.device = rank, fail_alloc_on, fail_open_on, 0
        self.freed, self.closed = [], []

    def shared_alloc(self, nbytes):
        if self.rank == self.fail_alloc_on:
            raise RuntimeError("injected: out of device memory")
        return 0x1000 * (self.rank + 1), bytes([self.rank]) * 64

    def shared_open(self, handle):
        if self.rank == self.fail_open_on:
            raise RuntimeError("injected: IPC not permitted")
        return 0x100000 + handle[0]

    def shared_close(self, ptr):
        self.closed.append(ptr)

    def shared_free(self, ptr):
        self.freed.append(ptr)


def _setup_worker(rank, world, port, mode, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    gk = importlib.import_module("gllm-kernels_b200")
    try:
        K = _FakeK(rank, fail_alloc_on=1 if mode == "alloc" else None, fail_open_on=0 if mode == "open" else None)
        try:
            ex = gk.PeerExchange(K, world, rank, slots=2, slot_floats=64)
            q.put((rank, "up", sorted(ex.bases), len(ex.peers)))
        except RuntimeError as e:
            # every rank raises together and has released what it had
            released = (K.freed == [0x1000 * (rank + 1)]) if not (mode == "alloc" and rank == 1) else (K.freed == [])
            q.put((rank, "raised", "injected" in str(e), released))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
@pytest.mark.parametrize("mode", ["ok", "alloc", "open"])
def test_peer_exchange_setup_failures_reach_every_rank(mode):
    """A rank whose allocation or mapping fails must not leave the others in a collective: all ranks raise."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_setup_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=100) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    if mode == "ok":
        assert [r[1] for r in res] == ["up", "up"] and all(r[3] == 1 for r in res)
    else:
        assert [r[1:] for r in res] == [("raised", True, True)] * 2, res
