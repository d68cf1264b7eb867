"""Row-sharded decode on 2 GPUs: the GEMV stores its band of y into both ranks' copies over peer pointers and
a flag barrier says when they are complete.  One child process per GPU; skipped on a single-GPU box."""
import importlib
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        gk = importlib.import_module("gllm-kernels_b200")
        from oracle import oracle as O
        K = gk.GpuKernels(rank)
        cases = [("q4k", 256, 512, 1), ("q4k", 200, 256, 3), ("q8_0", 176, 96, 16)]
        ex = gk.PeerExchange(K, world, rank, slots=len(cases), slot_floats=16 * 512)
        for rep in range(3):  # the same slots are rewritten: sequence numbers and flag reuse
            for slot, (fmt, n, k, m) in enumerate(cases):
                rng = np.random.default_rng(n + k + m + rep)
                W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
                x = rng.standard_normal((m, k)).astype(np.float32)
                qt, oid, blocks = ((gk.QuantType.q4k(), O.Q4K, O.quantize_q4_k(W)) if fmt == "q4k" else
                                   (gk.QuantType.q8_0(), O.Q8_0, O.quantize_q8_0(W)))
                r0, r1 = gk.shard_rows(n, world, rank)
                w = K.upload(qt, r1 - r0, k, gk.slice_blocks(qt, blocks, n, k, r0, r1))
                ex.gemv(w, torch.from_numpy(x).cuda(), slot, r0, n)
                ex.barrier()
                torch.cuda.synchronize()
                assert K.status() == 0
                y = ex.local_tensor(slot, (m, n)).cpu().numpy()
                ref = O.quant_matmul(blocks, np.ascontiguousarray(x.T), oid, n, m, k).T
                err = O.rel_err(y, ref)
                assert err <= 2e-3, f"rank {rank} {fmt} n={n} m={m} rep={rep}: {err}"
                w.free()
                dist.barrier()  # nobody rewrites a slot another rank is still reading back to the host
        # chained products without a barrier launch: y1 = W1 x is gathered into slot 0 of every rank, y2 = W2 y1
        # reads it there (its staging kernel waits for every rank's bands of y1), and the chain ends with wait().
        # Eager launches first, then the same chain captured once and replayed (the epochs live in device memory).
        n1, k1, n2, m = 512, 256, 208, 2
        rng = np.random.default_rng(99)
        W1 = (rng.standard_normal((n1, k1)) * 0.05).astype(np.float32)
        W2 = (rng.standard_normal((n2, n1)) * 0.05).astype(np.float32)
        b1, b2 = O.quantize_q4_k(W1), O.quantize_q4_k(W2)
        qt = gk.QuantType.q4k()
        ra, rb = gk.shard_rows(n1, world, rank), gk.shard_rows(n2, world, rank)
        w1 = K.upload(qt, ra[1] - ra[0], k1, gk.slice_blocks(qt, b1, n1, k1, *ra))
        w2 = K.upload(qt, rb[1] - rb[0], n1, gk.slice_blocks(qt, b2, n2, n1, *rb))
        y1_t, y2_t = ex.local_tensor(0, (m, n1)), ex.local_tensor(1, (m, n2))
        xs = torch.empty((m, k1), device="cuda")

        def chain():
            ex.gemv_chained(w1, xs, 0, ra[0], n1)
            ex.gemv_chained(w2, y1_t, 1, rb[0], n2)
            ex.wait()

        def check(tag):
            torch.cuda.synchronize()
            assert K.status() == 0
            x = xs.cpu().numpy()
            y1 = O.quant_matmul(b1, np.ascontiguousarray(x.T), O.Q4K, n1, m, k1).T
            y2 = O.quant_matmul(b2, np.ascontiguousarray(y1.T), O.Q4K, n2, m, n1).T
            e1, e2 = O.rel_err(y1_t.cpu().numpy(), y1), O.rel_err(y2_t.cpu().numpy(), y2)
            assert e1 <= 2e-3 and e2 <= 4e-3, f"rank {rank} {tag}: {e1} {e2}"
            dist.barrier()

        for rep in range(3):
            xs.copy_(torch.from_numpy(np.random.default_rng(200 + rep).standard_normal((m, k1)).astype(np.float32)))
            chain()
            check(f"eager {rep}")
        for fuse in (1, 0):  # the exchange products staging their own activations inside the GEMV, then the default again
            K.set("gemv_fuse", fuse)
            xs.copy_(torch.from_numpy(np.random.default_rng(250 + fuse).standard_normal((m, k1)).astype(np.float32)))
            chain()
            check(f"gemv_fuse {fuse}")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            chain()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            chain()
        for rep in range(4):
            xs.copy_(torch.from_numpy(np.random.default_rng(300 + rep).standard_normal((m, k1)).astype(np.float32)))
            graph.replay()
            if rep % 2:
                graph.replay()  # back-to-back replays: slot reuse one chain later
            check(f"graph {rep}")
        w1.free()
        w2.free()
        # the gated feed-forward block with row-sharded weights: gate || up gathered into h, the down product reads it with
        # SwiGLU applied while staging (two chained exchange products), against the oracle's chain
        d_model, f, m = 256, 256, 2
        b_gu = O.quantize_q4_k((np.random.default_rng(401).standard_normal((2 * f, d_model)) * 0.05).astype(np.float32))
        b_dn = O.quantize_q4_k((np.random.default_rng(402).standard_normal((d_model, f)) * 0.05).astype(np.float32))
        rg, rd = gk.shard_rows(2 * f, world, rank), gk.shard_rows(d_model, world, rank)
        w_gu = K.upload(qt, rg[1] - rg[0], d_model, gk.slice_blocks(qt, b_gu, 2 * f, d_model, *rg))
        w_dn = K.upload(qt, rd[1] - rd[0], f, gk.slice_blocks(qt, b_dn, d_model, f, *rd))
        for rep in range(2):
            xf = (np.random.default_rng(410 + rep).standard_normal((m, d_model)) * 4.0).astype(np.float32)
            h_t, y_t = ex.ffn_decode_sharded(w_gu, w_dn, torch.from_numpy(xf).cuda(), 0, 1, rg[0], rd[0])
            ex.wait()
            torch.cuda.synchronize()
            assert K.status() == 0
            h_ref = O.quant_matmul(b_gu, np.ascontiguousarray(xf.T), O.Q4K, 2 * f, m, d_model).T
            act = ((h_ref[:, :f] / (np.float32(1.0) + np.exp(-h_ref[:, :f], dtype=np.float32))) * h_ref[:, f:]).astype(np.float32)
            y_ref = O.quant_matmul(b_dn, np.ascontiguousarray(act.T), O.Q4K, d_model, m, f).T
            e1, e2 = O.rel_err(h_t.cpu().numpy(), h_ref), O.rel_err(y_t.cpu().numpy(), y_ref)
            assert e1 <= 2e-3 and e2 <= 4e-3, f"rank {rank} sharded ffn {rep}: {e1} {e2}"
            dist.barrier()
        w_gu.free()
        w_dn.free()
        ex.close()
        K.close()
        q.put((rank, "ok"))
    except Exception as e:
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_gemv_allgather_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert res == {0: "ok", 1: "ok"}, res


def test_two_devices_in_one_process():
    """Contexts on two GPUs of one process: kernels' per-device attributes, buffers and the static scratch are set up
    for each device separately."""
    import importlib
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    gk = importlib.import_module("gllm-kernels_b200")
    from oracle import oracle as O
    rng = np.random.default_rng(3)
    n, k = 256, 512
    W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    blocks = O.quantize_q4_k(W)
    wd = O.dequant_matrix(O.Q4K, blocks, n, k)
    x1 = rng.standard_normal((1, k)).astype(np.float32)
    xm = rng.standard_normal((96, k)).astype(np.float32)
    for dev in (1, 0, 1):
        K = gk.GpuKernels(dev)
        w = K.upload(gk.QuantType.q4k(), n, k, blocks)
        with torch.cuda.device(dev):
            y1 = K.gemv(w, torch.from_numpy(x1).to(f"cuda:{dev}")).cpu().numpy()
            ym = K.gemm(w, torch.from_numpy(xm).to(f"cuda:{dev}").to(torch.bfloat16)).cpu().numpy()
            ys = torch.full((1, n), float("nan"), device=f"cuda:{dev}")
            K.gemv_static(w, torch.from_numpy(x1).to(f"cuda:{dev}"), ys)  # its scratch array exists once per device
            torch.cuda.synchronize(dev)
            assert np.array_equal(ys.cpu().numpy(), y1)
        assert O.rel_err(y1, O.quant_matmul(blocks, np.ascontiguousarray(x1.T), O.Q4K, n, 1, k).T) <= 2e-3
        xb = torch.from_numpy(xm).to(torch.bfloat16).to(torch.float32).numpy()
        assert O.rel_err(ym, O.gemm_f32_nt(xb, wd)) <= 1e-2
        assert K.status() == 0
        w.free()
        K.close()
