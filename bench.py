#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200.

Headline workload ("step"): one decode pass (M = 1 token) over a stack of 70B-shaped Q4_K FFN
layers — gate W[28672, 8192], up W[28672, 8192], down W[8192, 28672] per layer — i.e. BASELINE
config 5 at M = 1.  Metric: quant GEMV weight-GB/s (reference-format weight bytes / time), reported
with its fraction of the measured HBM copy bandwidth.  A stack of several layers keeps the per-GPU
weight set larger than the 126 MB L2 at every GPU count, so no L2 flush is needed between steps.

  python bench.py --gpus 1 --steps 50 --warmup 5             # this implementation
  python bench.py --impl reference ...                       # the reference's CPU algorithm, host cores
  torchrun ... bench.py --gpus N ...                         # N-wise sharded, one NCCL all-gather per GEMV

One JSON line on stdout (rank 0).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_FF, D_MODEL = 28672, 8192
Q4K_BLOCK_BYTES, Q4K_BLOCK = 144, 256
METRIC = "quant GEMV weight-GB/s (Q4_K decode, 70B-shaped FFN)"
# what the decode kernel computes in: packed u4 weights as they are x activations re-expressed per 256-block as two
# s8 digits with one f32 scale (x = amax/127 * (d1 + d2/254)), exact s32 dot products (mma.sync u8 x s8), sub-block
# scales applied as integers, one f32 multiply-add per block for d, dmin and the activation scale, f32 sums over blocks
DTYPE = "u4 x (2 x s8 digit-split f32 activations), s32 dot products then f32 accumulate"
DTYPE_REF = "u4 decoded to f32 x f32 activations, sequential f32 accumulate (CPU port of the reference)"
GEMV_DRAM_TRAFFIC_PER_LAUNCH = 276.03e6


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if not self.nv:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop_evt.wait(0.002)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def shard_rows(n: int, world: int, rank: int):
    """N-wise split in multiples of 16 rows (the row tile of the device layout); the package's rule."""
    return importlib.import_module("gllm-kernels_b200").shard_rows(n, world, rank)


# ------------------------------------------------------------------------------------------------
# Parity of a full-size product on a SAMPLE of its weight rows (the oracle is scalar C: whole matrices of the
# benchmark shapes would take minutes, 256 rows x every token take seconds).  Used by the bench's `parity` records
# and by tests/test_gpu_shapes.py, so both check the same thing.
PARITY_METRIC = "max_i |y_i - ref_i| / max(|ref_i|, rms(ref))"


def sample_rows(n: int, count: int = 256, seed: int = 0):
    """`count` weight rows: the first and the last 32 (edge tiles) and a random draw of the rest, sorted."""
    import numpy as np
    if n <= count:
        return np.arange(n)
    rng = np.random.default_rng(seed)
    mid = rng.choice(np.arange(32, n - 32), size=count - 64, replace=False)
    return np.sort(np.concatenate([np.arange(32), mid, np.arange(n - 32, n)]))


def sampled_parity(O, oid, blocks, n, k, rows, x_host, y, bar, scales=None, global_scale=1.0, sequential=False, threads=8):
    """Compares columns `rows` of y [m, n] (torch, any float dtype) with the oracle's product of x_host [m, k] and
    the sampled rows of the quantized weight.  blocks / scales: the whole matrix in the reference's block format
    (torch uint8 on the device, or numpy).  sequential=True: the reference's own quantized matmul (block-ordered
    f32 sum, Q4_K / Q8_0 / GGUF formats); False: its decode followed by its f32 GEMM loop (scalar_gemm order)."""
    import numpy as np
    import torch

    def take(buf, per_row):
        if isinstance(buf, np.ndarray):
            return np.ascontiguousarray(buf.reshape(n, per_row)[rows]).reshape(-1)
        idx = torch.from_numpy(np.asarray(rows)).to(buf.device)
        return buf.reshape(n, per_row)[idx].cpu().numpy().reshape(-1)
    m = x_host.shape[0]
    hb = take(blocks, blocks.numel() // n if hasattr(blocks, "numel") else blocks.size // n)
    hs = None if scales is None else take(scales, scales.numel() // n if hasattr(scales, "numel") else scales.size // n)
    if sequential:
        ref = O.quant_matmul(hb, np.ascontiguousarray(x_host.T), oid, len(rows), m, k, threads=threads).T
    else:
        ref = O.gemm_f32_nt(x_host, O.dequant_matrix(oid, hb, len(rows), k, scales=hs, global_scale=global_scale))
    got = y[:, torch.from_numpy(np.asarray(rows)).to(y.device)].to(torch.float32).cpu().numpy()
    err = O.rel_err(got, ref)
    return {"metric": PARITY_METRIC, "rows_sampled": int(len(rows)), "tokens": int(m), "rel_err": err, "bar": bar,
            "ok": bool(err <= bar), "non_finite": {"y": int((~np.isfinite(got)).sum()), "oracle": int((~np.isfinite(ref)).sum())},
            "oracle": "reference quantized matmul (sequential f32)" if sequential else "reference decode + f32 GEMM loop order"}


def workload_config(L, M, fused):
    """The workload, named identically by both arms (the GPU arm adds how it ran under `run`)."""
    return {"workload": f"70B-shaped FFN decode (W gate/up [28672, 8192], W down [8192, 28672], Q4_K), {L} layers, M={M}; " +
                        ("gate and up stored as one 57344-row weight (2 products per layer)" if fused
                         else "one product per matrix (3 per layer)"),
            "layers": L, "M": M, "N_ff": N_FF, "d_model": D_MODEL,
            "weight_bytes_per_step": L * 3 * N_FF * (D_MODEL // Q4K_BLOCK) * Q4K_BLOCK_BYTES}


# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    gk = importlib.import_module("gllm-kernels_b200")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    K = gk.GpuKernels(local)
    if args.gemv_ctas_per_sm:
        K.set("gemv_ctas_per_sm", args.gemv_ctas_per_sm)
    if args.gemv_fuse >= 0:
        K.set("gemv_fuse", args.gemv_fuse)
    qt = gk.QuantType.q4k()
    M, L = args.m, args.layers

    # ---- synthetic weights: N(0, 0.02) f32 from the seed, quantized on the device, row-sharded ----
    # gate and up read the same x: by default they are stored as ONE weight of 2*N_ff rows (a load-time layout
    # choice like the repack itself: same bytes, same arithmetic, y = gate || up), so a layer is two products
    fused = not args.separate_gate_up
    shapes = ([("gate_up", 2 * N_FF, D_MODEL), ("down", D_MODEL, N_FF)] if fused else
              [("gate", N_FF, D_MODEL), ("up", N_FF, D_MODEL), ("down", D_MODEL, N_FF)])
    weights, host_blocks = [], []
    gen = torch.Generator(device=dev).manual_seed(20244)
    keep_host = rank == 0 and world == 1 and not args.no_cpu_baseline
    for layer in range(L):
        for name, n, k in shapes:
            W = torch.randn((n, k), generator=gen, device=dev) * 0.02  # same stream on every rank
            r0, r1 = shard_rows(n, world, rank)
            blocks = K.quantize(qt, W[r0:r1].contiguous())
            del W
            weights.append((name, K.upload(qt, r1 - r0, k, blocks), n, k, r0, r1))
            if keep_host and layer == 0:
                host_blocks.append((name, n, k, blocks.cpu().numpy()))
            del blocks
    torch.cuda.empty_cache()
    x_model = torch.randn((M, D_MODEL), generator=gen, device=dev)
    x_ff = torch.randn((M, N_FF), generator=gen, device=dev)
    ys = [torch.empty((M, n), dtype=torch.float32, device=dev) for (_, _, n, _, _, _) in weights]
    # sharded, default: every rank's GEMV stores its band of y into all ranks' copies of y over NVLink peer
    # pointers and a flag barrier follows (no library collective on the data path).
    # --exchange nccl: each rank's GEMV writes its slice of a [world, M, n/world] buffer, then one all-gather.
    gbufs, ex = [], None
    if world > 1 and args.exchange == "peer":
        # every rank must take the same path: agree on whether the peer mapping came up everywhere
        try:
            ex = gk.PeerExchange(K, world, rank, slots=len(weights), slot_floats=M * 2 * N_FF)
            ok = torch.ones(1, device=dev)
        except Exception as e:  # e.g. CUDA IPC not permitted in this container
            print(f"rank {rank}: peer exchange unavailable ({e}); falling back to NCCL all-gather", file=sys.stderr)
            ex, ok = None, torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0 and ex is not None:
            ex = None
    if world > 1 and ex is None:
        gbufs = [torch.empty((world, M, (r1 - r0)), dtype=torch.float32, device=dev) for (_, _, n, _, r0, r1) in weights]

    weight_bytes_local = sum(w.ref_bytes for (_, w, *_r) in weights)
    weight_bytes_total = L * sum(n * (k // Q4K_BLOCK) * Q4K_BLOCK_BYTES for _, n, k in shapes)
    algo_bytes_step = weight_bytes_total + L * sum(M * (k + n) * 4 for _, n, k in shapes)

    def step():
        for i, (name, w, n, k, r0, r1) in enumerate(weights):
            x = x_ff if name == "down" else x_model
            if world == 1:
                K.gemv(w, x, y=ys[i])
            elif ex is not None:
                # every product waits (in its staging kernel) for all ranks' bands of the product before it, as a
                # real decode step must, and signals its own completion from the GEMV's last block
                ex.gemv_chained(w, x, i, r0, n)
            else:
                K.gemv(w, x, y=gbufs[i][rank])
                dist.all_gather_into_tensor(gbufs[i].view(-1), gbufs[i][rank].view(-1))

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    graphed = False
    if not args.no_graph and (world == 1 or ex is not None):
        # one decode step = 12 x (staging, GEMV[, barrier]) launches of ~10-30 us each: replayed as a CUDA graph so
        # that the host's launch cost does not bound the step (all context buffers exist after the warm-up)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        eager_step, step = step, graph.replay
        graphed = True
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(args.steps):
        step()
    if ex is not None:
        ex.wait()  # the last product's bands have landed on this rank
    ev1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    ms_step = ms / args.steps
    value = weight_bytes_total / (ms_step * 1e-3) / 1e9

    # Sharded runs: where does the step go?  The same shards multiplied WITHOUT the exchange (no peer stores, no waits
    # for other ranks; y stays local), replayed as a graph like the step itself: the difference is what the exchange
    # costs; the remainder, against the HBM time of a rank's bytes, is the per-product launch / ramp / tail cost.
    breakdown = None
    if world > 1 and ex is not None and graphed:
        def local_step():
            for i, (name, w, n, k, r0, r1) in enumerate(weights):
                K.gemv(w, x_ff if name == "down" else x_model, y=ys[i][:, r0:r1])
        for _ in range(3):
            local_step()
        torch.cuda.synchronize()
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2):
            local_step()
        for _ in range(3):
            g2.replay()
        torch.cuda.synchronize()
        dist.barrier()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record()
        for _ in range(args.steps):
            g2.replay()
        l1.record()
        torch.cuda.synchronize()
        tl = torch.tensor([l0.elapsed_time(l1) / args.steps], device=dev)
        dist.all_reduce(tl, op=dist.ReduceOp.MAX)
        peak_gbs = measured_peaks()[0]
        hbm_us = weight_bytes_local / peak_gbs / 1e3
        breakdown = {"step_us": ms_step * 1e3, "same_shards_without_exchange_us": tl.item() * 1e3,
                     "exchange_us": ms_step * 1e3 - tl.item() * 1e3, "hbm_time_of_a_rank_s_bytes_us": hbm_us,
                     "products_per_step": len(weights),
                     "fixed_cost_per_product_us": (tl.item() * 1e3 - hbm_us) / len(weights),
                     "exchange_per_product_us": (ms_step * 1e3 - tl.item() * 1e3) / len(weights)}

    # ---- end to end through the host-pointer call: pinned x -> device, GEMVs, y -> host, every step ----
    # host activations and outputs live in page-locked memory, as a serving loop keeps them
    xh_model = torch.empty(x_model.shape, dtype=torch.float32, pin_memory=True).copy_(x_model).numpy()
    xh_ff = torch.empty(x_ff.shape, dtype=torch.float32, pin_memory=True).copy_(x_ff).numpy()
    yh = {n: torch.empty((M, n), dtype=torch.float32, pin_memory=True).numpy() for n in {n for (_, _, n, _, _, _) in weights}}
    e2e = None
    if world == 1:
        # one output buffer per product (a step's products do not share results), all enqueued by one call that waits
        # once: gllmk_matmul_host_batch
        yh_all = [torch.empty((M, n), dtype=torch.float32, pin_memory=True).numpy() for (_, _, n, _, _, _) in weights]
        ws_all = [w for (_, w, *_r) in weights]
        xs_all = [xh_ff if name == "down" else xh_model for (name, *_r) in weights]

        plan = K.host_batch(ws_all, xs_all, yh_all)  # the argument arrays of the step, built once

        def step_host():
            return plan.run()
        def step_host_each():
            for (name, w, n, k, r0, r1), y in zip(weights, yh_all):
                K.matmul_host(w, xh_ff if name == "down" else xh_model, out=y)
        for _ in range(3):
            step_host_each()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_host_each()
        e2e_per_product = weight_bytes_total / ((time.perf_counter() - t0) / args.steps) / 1e9
        for _ in range(3):
            step_host()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_host()
        dt = (time.perf_counter() - t0) / args.steps
        e2e = {"value": weight_bytes_total / dt / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": L * sum(M * k * 4 for _, n, k in shapes),
               "d2h_bytes_per_step": L * sum(M * n * 4 for _, n, k in shapes),
               "note": "weights resident (uploaded once, like the reference's weights handle); activations and "
                       "outputs are page-locked host buffers, transferred inside the timed region (every product's x uploaded "
                       "and its y downloaded on a copy stream beside the products); the step's products go through ONE "
                       "gllmk_matmul_host_batch call, which replays the step as a captured CUDA graph and waits once at the end",
               "one_synchronous_call_per_product": e2e_per_product}

    elif ex is not None:
        # sharded: every rank copies the step's activations from page-locked host memory, runs its band of every
        # product (bands exchanged over NVLink as above) and reads the last product's gathered y back to the host
        xd = {"model": torch.empty_like(x_model), "ff": torch.empty_like(x_ff)}
        xp = {"model": torch.from_numpy(xh_model), "ff": torch.from_numpy(xh_ff)}
        last = len(weights) - 1
        y_last = ex.local_tensor(last, (M, weights[last][2]))
        y_host = torch.empty((M, weights[last][2]), dtype=torch.float32, pin_memory=True)

        # every product's activations have their own device buffer; all uploads are issued up front on a copy stream and
        # product i only waits for the upload of product i + 1 (so nothing sits between a GEMV and the next staging kernel)
        xdev = [torch.empty_like(x_ff if name == "down" else x_model) for (name, *_r) in weights]
        copy_stream = torch.cuda.Stream()
        up_events = [torch.cuda.Event() for _ in weights]

        def enqueue_host_step():
            main = torch.cuda.current_stream()
            copy_stream.wait_stream(main)
            with torch.cuda.stream(copy_stream):
                for i, (name, *_r) in enumerate(weights):
                    xdev[i].copy_(xp["ff" if name == "down" else "model"], non_blocking=True)
                    up_events[i].record(copy_stream)
            main.wait_event(up_events[0])
            for i, (name, w, n, k, r0, r1) in enumerate(weights):
                if i + 1 < len(weights):
                    main.wait_event(up_events[i + 1])
                ex.gemv_chained(w, xdev[i], i, r0, n)
            ex.wait()
            y_host.copy_(y_last, non_blocking=True)

        def step_host():
            enqueue_host_step()
            torch.cuda.synchronize()
        for _ in range(3):
            step_host()
        dist.barrier()
        e2e_graphed = False
        if not args.no_graph:
            # the same step (uploads, chained products, download) captured once and replayed; the host still waits for
            # the downloaded result every step
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                enqueue_host_step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            dist.barrier()
            ge = torch.cuda.CUDAGraph()
            with torch.cuda.graph(ge):
                enqueue_host_step()

            def step_host():
                ge.replay()
                torch.cuda.synchronize()
            e2e_graphed = True
            for _ in range(3):
                step_host()
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_host()
        dt_t = torch.tensor([(time.perf_counter() - t0) / args.steps], device=dev)
        dist.all_reduce(dt_t, op=dist.ReduceOp.MAX)
        e2e = {"value": weight_bytes_total / dt_t.item() / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": world * L * sum(M * k * 4 for _, n, k in shapes),
               "d2h_bytes_per_step": world * M * weights[last][2] * 4,
               "note": "per step every rank copies each product's activations from page-locked host memory, the bands "
                       "are exchanged over NVLink, and every rank reads the last product's gathered y back and waits for it; "
                       + ("the step is a replayed CUDA graph" if e2e_graphed else "host launches (no graph)") + "; wall clock, max over ranks"}

    parity_multi = None
    if world > 1:
        parity_multi = multi_gpu_parity(args, K, gk, torch, dev, weights, ex, gbufs, x_model, M, world, rank)

    peak, peak_kind = measured_peaks()
    out = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": workload_config(L, M, fused),
        "run": {"l2": "per-GPU weight set larger than L2, no flush", "cuda_graph": graphed,
                "parallelism": "single GPU" if world == 1 else (
                    f"N-wise row shards x{world}, GEMV stores its band into every rank's y over NVLink peer pointers, "
                    f"flags signalled by the GEMV's last block and awaited by the next product's staging kernel"
                    if ex is not None else f"N-wise row shards x{world} + NCCL all-gather")},
        "roofline": {"bound": "hbm", "achieved": algo_bytes_step / (ms_step * 1e-3) / 1e9 / world, "peak": peak,
                     "unit": "GB/s", "frac": algo_bytes_step / (ms_step * 1e-3) / 1e9 / world / peak,
                     # dram__bytes_read + dram__bytes_write of one gemv_kernel launch on the 264.2 MB gate||up weight,
                     # from the ncu capture summarised in profiles/gemv_kernel_q4k_m1_decode_cfg5.md
                     "traffic": GEMV_DRAM_TRAFFIC_PER_LAUNCH if (M == 1 and world == 1 and fused) else None,
                     "traffic_note": "bytes per gemv_kernel launch on the 57344x8192 gate||up weight (algorithmic 264.50e6), ncu",
                     "peak_kind": peak_kind,
                     "kernel": "gemv_kernel<Q4_K, 1 n-tile> (+ stage_x_kernel), per-GPU average"},
        "gpu_launches": args.steps * len(weights) * 2 + (1 if ex is not None else 0),
        "device_status": K.status(),
        "clocks": clocks,
        "e2e": e2e,
    }
    if world == 1 and rank == 0 and not args.no_extra:
        out["extra"] = extra_configs(K, gk, torch, dev, peak)
    if world > 1 and not args.no_extra:
        sharded = sharded_prefill_extra(K, gk, torch, dist, dev, world, rank)
        if rank == 0:
            out["extra"] = sharded
    if parity_multi is not None:
        out["parity"] = parity_multi
    if breakdown is not None:
        out["breakdown"] = breakdown
    if keep_host:
        out["cpu_baseline"] = cpu_baseline(host_blocks, xh_model, xh_ff, M, threads=1)
        out["parity"] = parity_record(K, weights[0][1], host_blocks[0], x_model, xh_model, M)
        out["cpu_bench_quant_path"] = bench_quant_cpu()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        if ex is not None:
            ex.close()
        dist.destroy_process_group()


def multi_gpu_parity(args, K, gk, torch, dev, weights, ex, gbufs, x_model, M, world, rank):
    """Sharded run: the gathered y of the step's first product, as it sits in rank 0's buffer after the timed
    region, against the CPU oracle on sampled rows of EVERY rank's band.  Rank 0 regenerates the first matrix from
    the seed (every rank drew the same stream and kept its band) and quantizes the sampled rows again: the
    quantizer works row by row, so these are the bytes the owning rank uploaded."""
    import numpy as np
    name, w, n, k, r0, r1 = weights[0]
    torch.cuda.synchronize()
    if rank != 0:
        return None
    from oracle import oracle as O
    gen = torch.Generator(device=dev).manual_seed(20244)
    W = torch.randn((n, k), generator=gen, device=dev) * 0.02
    rows = []
    for r in range(world):
        b0, b1 = shard_rows(n, world, r)
        rows.append(b0 + sample_rows(b1 - b0, max(64, 256 // world), seed=r))
    rows = np.concatenate(rows)
    sub = W[torch.from_numpy(rows).to(dev)].contiguous()
    del W
    blocks = K.quantize(gk.QuantType.q4k(), sub)
    if ex is not None:
        y = ex.local_tensor(0, (M, n))
    else:
        parts = [gbufs[0][r, :, : shard_rows(n, world, r)[1] - shard_rows(n, world, r)[0]] for r in range(world)]
        y = torch.cat(parts, dim=1)
    rec = sampled_parity(O, O.Q4K, blocks, len(rows), k, np.arange(len(rows)), x_model.cpu().numpy(),
                         y[:, torch.from_numpy(rows).to(dev)], bar=2e-3, sequential=True)
    rec["matrix"] = f"{name} [{n}, {k}]: rows sampled from each of the {world} ranks' bands, read from rank 0's gathered y"
    return rec


def sharded_prefill_extra(K, gk, torch, dist, dev, world, rank):
    """The sharded gate matrix W[28672, 8192] (Q4_K) at M = 32 and M = 512: every rank multiplies its band of rows
    (the tensor-core kernel, bf16 output) and ONE NCCL all-gather puts the
    bands side by side.  Device time (CUDA events), max over ranks; parity on rank 0 against the oracle on rows sampled
    from every rank's band of the gathered result."""
    import numpy as np
    qt = gk.QuantType.q4k()
    n, k = N_FF, D_MODEL
    gen = torch.Generator(device=dev).manual_seed(20246)
    W = torch.randn((n, k), generator=gen, device=dev) * 0.02
    r0, r1 = shard_rows(n, world, rank)
    band = r1 - r0
    w = K.upload(qt, band, k, K.quantize(qt, W[r0:r1].contiguous()))
    rows = np.concatenate([shard_rows(n, world, r)[0] + sample_rows(shard_rows(n, world, r)[1] - shard_rows(n, world, r)[0],
                                                                     max(64, 256 // world), seed=r) for r in range(world)])
    sub_blocks = K.quantize(qt, W[torch.from_numpy(rows).to(dev)].contiguous()) if rank == 0 else None
    del W
    res = {}
    for m in (32, 512):
        x = torch.randn((m, k), generator=gen, device=dev)
        dt = torch.float32 if m <= K.GEMM_GEMV_MAX_M else torch.bfloat16
        buf = torch.empty((world, m, band), dtype=dt, device=dev)
        mine = torch.empty((m, band), dtype=dt, device=dev)

        def step():
            K.gemm(w, x, y=mine)
            dist.all_gather_into_tensor(buf.view(-1), mine.view(-1))
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = t.item() * 1e3
        entry = {"us": us, "tflops": 2.0 * m * n * k / us / 1e6, "weight_GBps": n * (k // Q4K_BLOCK) * Q4K_BLOCK_BYTES / us / 1e3,
                 "gather": f"one NCCL all_gather_into_tensor of [{m}, {band}] {str(dt).split('.')[-1]} bands",
                 "all_gather_bytes_per_rank": m * band * (4 if dt == torch.float32 else 2)}
        if rank == 0:
            from oracle import oracle as O
            y = torch.cat([buf[r] for r in range(world)], dim=1)
            tc = m > K.GEMM_GEMV_MAX_M
            entry["parity"] = sampled_parity(O, O.Q4K, sub_blocks, len(rows), k, np.arange(len(rows)), x.cpu().numpy(),
                                             y[:, torch.from_numpy(rows).to(dev)], bar=1e-2 if tc else 2e-3, sequential=not tc)
            entry["parity"]["non_finite"]["y_per_band"] = [int((~torch.isfinite(buf[r].float())).sum().item()) for r in range(world)]
        res[f"sharded_q4k_{n}x{k}_M{m}"] = entry
    w.free()
    return res


def extra_configs(K, gk, torch, dev, peak):
    """Configs 1 and 2 (small matrices): rotate over distinct weight copies totalling > 2x L2."""
    res = {}
    gen = torch.Generator(device=dev).manual_seed(20240)
    torch.cuda.empty_cache()

    def random_gguf_blocks(qt, n, k):
        """Formats without a device quantizer: random payload bytes, f16 (Q8_K: f32) scale fields of +-0.02."""
        bs, bb = qt.block_size(), qt.block_bytes()
        nblk = n * (k // bs)
        b = torch.randint(0, 256, (nblk, bb), generator=gen, device=dev, dtype=torch.uint8)
        d = (torch.rand((nblk, 2), generator=gen, device=dev) - 0.5) * 0.04
        if qt.id == 10:
            b[:, 0:4] = d[:, :1].contiguous().view(torch.uint8)
        else:
            h = d.to(torch.float16).view(torch.uint8)  # [nblk, 4]: two f16
            if qt.id == 6:
                b[:, 208:210] = h[:, 0:2]
            else:
                b[:, 0:2] = h[:, 0:2]
            if qt.id == 7:
                b[:, 2:4] = h[:, 2:4]
        return b.reshape(-1)

    from oracle import oracle as O  # checker and CPU-baseline legs only, outside every timed region

    def run(qt, n, k, ms, copies, name):
        bs, bb = qt.block_size(), qt.block_bytes()
        ws, first = [], None
        for _ in range(copies):
            if qt.id >= 6:
                q = random_gguf_blocks(qt, n, k)
                ws.append(K.upload(qt, n, k, q))
                first = first or (q, None, 1.0)
                del q
                continue
            W = torch.randn((n, k), generator=gen, device=dev) * 0.02
            q = K.quantize(qt, W)
            ws.append(K.upload(qt, n, k, q[0], q[1]) if qt.id == 3 else (K.upload(qt, n, k, q[0], None, q[1]) if qt.id == 4
                                                                           else K.upload(qt, n, k, q)))
            first = first or ((q[0], q[1], 1.0) if qt.id == 3 else ((q[0], None, q[1]) if qt.id == 4 else (q, None, 1.0)))
            del W, q
        wbytes = n * (k // bs) * bb
        rows = sample_rows(n, 256, seed=n)
        for m in ms:
            x = torch.randn((m, k), generator=gen, device=dev)
            y = torch.empty((m, n), dtype=torch.float32, device=dev)
            reps = 20
            K.gemv(ws[0], x, y=y)
            par = sampled_parity(O, qt.id, first[0], n, k, rows, x.cpu().numpy(), y, bar=2e-3, scales=first[1], global_scale=first[2],
                                 sequential=qt.id not in (3, 4))

            def sweep():
                for w in ws:
                    K.gemv(w, x, y=y)
            sweep()
            torch.cuda.synchronize()
            # one pass over the rotating copies as a CUDA graph: these products take 10-20 us each, less than the
            # host needs to launch their two kernels
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                sweep()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                sweep()
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
            res[f"{name}_M{m}"] = {"us_per_gemv": us, "weight_GBps": wbytes / us / 1e3, "frac_hbm": wbytes / us / 1e3 / peak,
                                   "tflops": 2.0 * m * n * k / us / 1e6, "copies_rotated": copies, "parity": par}
            if name.startswith("cfg"):
                res[f"{name}_M{m}"]["cpu_baseline"] = cpu_baseline_rows(O, qt.id, first, n, k, rows, x.cpu().numpy(), wbytes)
        for w in ws:
            w.free()

    res["cfg5_decode_separate_gate_up"] = decode_layers(K, gk, torch, dev, gen, peak, fused=False)
    res["cfg5_ffn_decode_swiglu"] = decode_layers(K, gk, torch, dev, gen, peak, fused=True, ffn=True)
    run(gk.QuantType.q4k(), 4096, 4096, [1], 32, "cfg1_q4k_4096x4096")
    run(gk.QuantType.q8_0(), 11008, 4096, [1, 4, 8, 16], 6, "cfg2_q8_0_11008x4096")
    run(gk.QuantType.mxfp4(32), 14336, 4096, [1], 10, "cfg3_mxfp4_expert_decode_14336x4096")
    run(gk.QuantType.nvfp4(), 14336, 4096, [1], 10, "cfg4_nvfp4_decode_14336x4096")
    run(gk.QuantType.q4k(), N_FF, D_MODEL, [16], 3, "cfg5_q4k_28672x8192")
    # the other GGUF formats (streaming CUDA-core GEMV over reference-layout blocks), down-projection shape of config 5
    run(gk.QuantType.q6k(), D_MODEL, N_FF, [1, 8], 2, "gguf_q6k_8192x28672")
    run(gk.QuantType.q5k(), D_MODEL, N_FF, [1], 2, "gguf_q5k_8192x28672")
    run(gk.QuantType.q8k(), D_MODEL, N_FF, [1], 2, "gguf_q8k_8192x28672")
    run(gk.QuantType.q4_0(), D_MODEL, N_FF, [1], 3, "gguf_q4_0_8192x28672")
    run(gk.QuantType.q5_0(), D_MODEL, N_FF, [1], 3, "gguf_q5_0_8192x28672")
    # Q6_K prefill on the fused-dequant tensor-core GEMM, same shape at M = 512
    q = random_gguf_blocks(gk.QuantType.q6k(), D_MODEL, N_FF)
    w6 = K.upload(gk.QuantType.q6k(), D_MODEL, N_FF, q)
    x6 = torch.randn((512, N_FF), generator=gen, device=dev)
    y6 = torch.empty((512, D_MODEL), dtype=torch.float32, device=dev)
    for _ in range(3):
        K.gemm(w6, x6, y=y6)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        K.gemm(w6, x6, y=y6)
    e1.record()
    torch.cuda.synchronize()
    us6 = e0.elapsed_time(e1) * 1e3 / 5
    res["gguf_q6k_8192x28672_M512"] = {"us": us6, "tflops": 2.0 * 512 * D_MODEL * N_FF / us6 / 1e6, "staging": "fp16 x fp16 -> f32 (kind::f16)",
                                       "parity": sampled_parity(O, gk.QuantType.q6k().id, q, D_MODEL, N_FF, sample_rows(D_MODEL, 256, seed=6), x6.cpu().numpy(),
                                                                y6, bar=1e-2, sequential=False)}
    w6.free()
    del q, x6, y6
    res.update(extra_gemm(K, gk, torch, dev, gen))
    res["cpu_bench_quant_kernels"] = bench_quant_cpu_all()
    return res


def cpu_baseline_rows(O, oid, packed, n, k, rows, x_host, wbytes, flops=None):
    """The CPU port of the reference on a row subset of one configuration, scaled to the whole matrix (its cost is
    proportional to the rows): 1 thread (as the reference runs it) and all host threads (rows in parallel).
    Q4_K / Q8_0 / GGUF formats: the reference's quantized matmul.  MXFP4 / NVFP4: the reference has no matmul for
    them; its decode followed by its scalar f32 GEMM is timed, 1 thread."""
    import numpy as np
    blocks, scales, g = packed
    idx = None

    def take(buf):
        nonlocal idx
        if isinstance(buf, np.ndarray):
            return np.ascontiguousarray(buf.reshape(n, -1)[rows]).reshape(-1)
        import torch
        idx = torch.from_numpy(np.asarray(rows)).to(buf.device) if idx is None else idx
        return buf.reshape(n, -1)[idx].cpu().numpy().reshape(-1)
    hb = take(blocks)
    hs = None if scales is None else take(scales)
    m = x_host.shape[0]
    xt = np.ascontiguousarray(x_host.T)
    out = {"rows_timed": int(len(rows)), "of_rows": int(n), "kind": "port", "scaled": "time x n / rows_timed"}
    threads = os.cpu_count() or 1
    for label, th in (("1_thread", 1), ("all_threads", threads)):
        if oid in (3, 4) and th > 1:
            continue
        t0 = time.perf_counter()
        if oid in (3, 4):
            O.gemm_f32_nt(x_host, O.dequant_matrix(oid, hb, len(rows), k, scales=hs, global_scale=g))
        else:
            O.quant_matmul(hb, xt, oid, len(rows), m, k, threads=th)
        dt = (time.perf_counter() - t0) * n / len(rows)
        out[label] = {"cores": th, "ms": dt * 1e3, "weight_GBps": wbytes / dt / 1e9, "gflops": 2.0 * m * n * k / dt / 1e9}
    return out


def bench_quant_cpu_all():
    """Every group of the reference's benches/bench_quant.rs (:21-25, :67, :150, :191, :272-279) on this box's host:
    the five scalar-ops kernels restated in C and built -O1 -fno-tree-vectorize like the reference's bench
    profile, one thread, at bench_quant's own shapes.  GEMM groups time 8 of the M rows and scale."""
    from oracle import oracle as O
    res = {}
    groups = [("gemv_q8", [(1, 4096, 4096), (1, 11008, 4096), (1, 16384, 4096)]),
              ("gemv_q4", [(1, 4096, 4096), (1, 11008, 4096)]),
              ("gemm_q8", [(32, 4096, 4096), (64, 4096, 4096), (128, 4096, 4096)]),
              ("gemm_q4", [(32, 4096, 4096), (64, 4096, 4096), (128, 4096, 4096)]),
              ("kquant_matmul", [(1, 4096, 4096), (32, 4096, 4096)])]
    for kind, shapes in groups:
        for m, n, k in shapes:
            dt, mi = O.bench_quant_kernel(kind, m, n, k)
            dt_full = dt * m / mi
            res[f"{kind}_{m}x{n}x{k}"] = {"ms": dt_full * 1e3, "gflops": 2.0 * m * n * k / dt_full / 1e9, "rows_of_x_timed": mi,
                                         "cores": 1, "build": "-O1 -fno-tree-vectorize"}
    return res


def decode_layers(K, gk, torch, dev, gen, peak, fused, layers=4, ffn=False):
    """The headline workload with gate and up as two weights (fused=False: 3 products per layer) or as one weight
    of 57344 rows (fused=True), graph replay.  ffn=True: the layers as real gated feed-forward blocks
    (gllmk_ffn_decode: the down product reads silu(gate) * up, each layer's output feeds the next)."""
    qt = gk.QuantType.q4k()
    ws = []
    for _ in range(layers):
        for n, k in (((2 * N_FF, D_MODEL), (D_MODEL, N_FF)) if fused else ((N_FF, D_MODEL), (N_FF, D_MODEL), (D_MODEL, N_FF))):
            W = torch.randn((n, k), generator=gen, device=dev) * 0.02
            ws.append(K.upload(qt, n, k, K.quantize(qt, W)))
            del W
    torch.cuda.empty_cache()
    xs = {D_MODEL: torch.randn((1, D_MODEL), generator=gen, device=dev), N_FF: torch.randn((1, N_FF), generator=gen, device=dev)}
    ys = [torch.empty((1, w.n), dtype=torch.float32, device=dev) for w in ws]

    hs = [torch.empty((1, 2 * N_FF), dtype=torch.float32, device=dev) for _ in range(layers)] if ffn else []

    def step():
        if ffn:
            x = xs[D_MODEL]
            for layer in range(layers):
                x = K.ffn_decode(ws[2 * layer], ws[2 * layer + 1], x, h=hs[layer], y=ys[2 * layer + 1])
            return
        for w, y in zip(ws, ys):
            K.gemv(w, xs[w.k], y=y)
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 30
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    wbytes = sum(w.ref_bytes for w in ws)
    for w in ws:
        w.free()
    return {"ms_per_step": ms, "weight_GBps": wbytes / ms / 1e6, "frac_hbm": wbytes / ms / 1e6 / peak, "products_per_step": len(ws)}


def extra_gemm(K, gk, torch, dev, gen):
    """Prefill configs: 3 (MXFP4 MoE experts, bf16 activations), 4 (NVFP4 x NVFP4), 5 at M = 32 / 512 (Q4_K)."""
    import numpy as np
    res = {}
    QT = gk.QuantType

    from oracle import oracle as O  # checker and CPU-baseline legs only, outside every timed region

    def upload(qt, n, k):
        """-> (weight handle, (blocks, scales, global scale) as the reference stores them, on the device)"""
        W = torch.randn((n, k), generator=gen, device=dev) * 0.02
        q = K.quantize(qt, W)
        del W
        if qt.id == 3:
            return K.upload(qt, n, k, q[0], q[1]), (q[0], q[1], 1.0)
        if qt.id == 4:
            return K.upload(qt, n, k, q[0], None, q[1]), (q[0], None, q[1])
        return K.upload(qt, n, k, q), (q, None, 1.0)

    def timeit(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    # config 5 prefill: gate/up-shaped and down-shaped Q4_K, f32 activations
    for n, k in ((28672, 8192), (8192, 28672)):
        w, packed = upload(QT.q4k(), n, k)
        rows = sample_rows(n, 256, seed=k)
        for m in (32, 512):
            a = torch.randn((m, k), generator=gen, device=dev)
            y = torch.empty((m, n), dtype=torch.float32, device=dev)
            us = timeit(lambda: K.gemm(w, a, y=y), 5)
            tc = m > K.GEMM_GEMV_MAX_M
            res[f"cfg5_q4k_{n}x{k}_M{m}"] = {"us": us, "tflops": 2.0 * m * n * k / us / 1e6, "weight_GBps": w.ref_bytes / us / 1e3,
                                            "staging": "fp16 x fp16 -> f32 (kind::f16)" if tc else "a pass of the decode kernel",
                                            "parity": sampled_parity(O, O.Q4K, packed[0], n, k, rows, a.cpu().numpy(), y,
                                                                     bar=1e-2 if tc else 2e-3, sequential=not tc)}
            if k == 8192:
                res[f"cfg5_q4k_{n}x{k}_M{m}"]["cpu_baseline"] = cpu_baseline_rows(O, O.Q4K, packed, n, k, rows[:64 if m > 32 else 256],
                                                                                   a.cpu().numpy(), w.ref_bytes)
        w.free()
        del packed
    # config 3: 8 experts MXFP4 [14336, 4096], 512 tokens, top-2 routing by the reference's conventions (scalar_topk: the
    # two largest of 8 uniform draws = two distinct experts, uniform), rows grouped per expert, bf16 activations
    ups = [upload(QT.mxfp4(32), 14336, 4096) for _ in range(8)]
    experts = [u[0] for u in ups]
    x_tok = torch.randn((512, 4096), generator=gen, device=dev).to(torch.bfloat16)
    probs = torch.rand((512, 8), generator=gen, device=dev)
    probs = probs / probs.sum(dim=1, keepdim=True)
    routing = K.moe_topk(probs, 2)
    offs, perm, inv = K.moe_route(routing, 512, 8, 2)
    counts = [offs[e + 1] - offs[e] for e in range(8)]
    a = K.moe_gather(x_tok, perm, 2)
    y = torch.empty((1024, 14336), dtype=torch.bfloat16, device=dev)

    def moe_loop():
        for e, w in enumerate(experts):
            if counts[e]:
                K.gemm(w, a[offs[e]:offs[e + 1]], y=y[offs[e]:offs[e + 1]])
    us_loop = timeit(moe_loop, 5)
    us = timeit(lambda: K.gemm_grouped(experts, a, offs, y=y), 10)
    res["cfg3_mxfp4_moe_8x14336x4096_M512_top2"] = {"us": us, "tflops": 2.0 * 1024 * 14336 * 4096 / us / 1e6,
                                                     "weight_GBps": sum(w.ref_bytes for w in experts) / us / 1e3,
                                                     "rows_per_expert": counts, "staging": "fp16 x fp16 -> f32 (kind::f16)",
                                                     "launch": "one grouped launch over the 8 experts",
                                                     "us_one_call_per_expert": us_loop}
    a_host, worst = a.to(torch.float32).cpu().numpy(), None
    for e in range(8):
        rec = sampled_parity(O, O.MXFP4, ups[e][1][0], 14336, 4096, sample_rows(14336, 256, seed=e), a_host[offs[e]:offs[e + 1]],
                             y[offs[e]:offs[e + 1]], bar=1e-2, scales=ups[e][1][1])
        worst = rec if worst is None or rec["rel_err"] > worst["rel_err"] else worst
    worst["note"] = "worst of the 8 experts; 256 sampled rows x the expert's tokens each; bf16 output"
    res["cfg3_mxfp4_moe_8x14336x4096_M512_top2"]["parity"] = worst
    res["cfg3_mxfp4_moe_8x14336x4096_M512_top2"]["cpu_baseline"] = cpu_baseline_rows(
        O, O.MXFP4, ups[0][1], 14336, 4096, sample_rows(14336, 64, seed=0), a_host[offs[0]:offs[1]],
        ups[0][0].ref_bytes, None)
    for w in experts:
        w.free()
    del ups
    # W8A8: s8 weights x u8 activations -> s32 (exact), tcgen05 kind::i8, at config 2's matrix and a 70B-shaped one
    for n, k, m in ((11008, 4096, 2048), (28672, 8192, 2048)):
        b = torch.randint(-128, 128, (n, k), generator=gen, device=dev, dtype=torch.int8)
        w = K.upload_int8(b, layout_kn=False)
        rows = sample_rows(n, 256, seed=n)
        b_rows = b[torch.from_numpy(rows).to(dev)].cpu().numpy().astype(np.float64)
        del b
        a8 = torch.randint(0, 256, (m, k), generator=gen, device=dev, dtype=torch.uint8)
        c32 = torch.empty((m, n), dtype=torch.int32, device=dev)
        us = timeit(lambda: K.gemm_int8(w, a8, c=c32), 10)
        # exact integer reference on 256 sampled weight rows x every token (f64 products and sums of 8-bit integers are exact)
        ref = a8.cpu().numpy().astype(np.float64) @ b_rows.T
        got = c32[:, torch.from_numpy(rows).to(dev)].cpu().numpy().astype(np.float64)
        res[f"w8a8_int8_{n}x{k}_M{m}"] = {"us": us, "tops": 2.0 * m * n * k / us / 1e6, "frac_of_nominal_int8_4500": 2.0 * m * n * k / us / 1e6 / 4500.0,
                                          "mma": "tcgen05 kind::i8 on CTA pairs, s32 accumulate (bit-exact)",
                                          "parity": {"metric": "s32 results equal to the exact integer product", "rows_sampled": int(len(rows)),
                                                     "tokens": m, "mismatches": int((ref != got).sum()), "ok": bool((ref == got).all())}}
        w.free()
        del a8, c32
    # config 4: NVFP4 weights x NVFP4 activations, bf16 out, native block-scaled MMA
    n, k, m = 14336, 4096, 2048
    w, packed = upload(QT.nvfp4(), n, k)
    X = torch.randn((m, k), generator=gen, device=dev)
    xb, gx = K.quantize(QT.nvfp4(), X)
    x = K.upload(QT.nvfp4(), m, k, xb, None, gx)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    us = timeit(lambda: K.gemm_fp4(w, x, y=y), 20)
    a_host = O.dequant_matrix(O.NVFP4, xb.cpu().numpy(), m, k, global_scale=gx)
    rows = sample_rows(n, 256, seed=4)
    ceil_tf = K.probe_fp4_mma(True, 2)
    res["cfg4_nvfp4_14336x4096_M2048"] = {"us": us, "tflops": 2.0 * m * n * k / us / 1e6, "frac_of_nominal_fp4_9000": 2.0 * m * n * k / us / 1e6 / 9000.0,
                                          "measured_mma_ceiling_tflops": ceil_tf, "frac_of_measured_mma_ceiling": 2.0 * m * n * k / us / 1e6 / ceil_tf,
                                          "mma": "tcgen05 kind::mxf4nvf4 block_scale, cta_group::2",
                                          "parity": sampled_parity(O, O.NVFP4, packed[0], n, k, rows, a_host, y, bar=2e-3 + 2.0 ** -8,
                                                                   global_scale=packed[2]),
                                          "cpu_baseline": cpu_baseline_rows(O, O.NVFP4, packed, n, k, rows[:32], a_host, w.ref_bytes)}
    w.free()
    x.free()
    return res


def cpu_baseline(host_blocks, xh_model, xh_ff, M, threads, reps=None):
    """The oracle (a port of the reference's scalar path) on this box's host cores: one layer's gate, up and
    down GEMVs — the same work as 1/L of a step."""
    import numpy as np
    from oracle import oracle as O
    import numpy as _np
    xt_model = _np.ascontiguousarray(xh_model.T)
    xt_ff = _np.ascontiguousarray(xh_ff.T)
    wbytes = sum(b.size for (_, _, _, b) in host_blocks)

    def once():
        for name, n, k, b in host_blocks:
            O.quant_matmul(b, xt_ff if name == "down" else xt_model, O.Q4K, n, M, k, threads=threads)
    once()
    t0 = time.perf_counter()
    once()
    one = time.perf_counter() - t0
    reps = reps or max(2, min(40, int(12.0 / max(one, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        once()
    dt = (time.perf_counter() - t0) / reps
    return {"value": wbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{reps} passes over one layer (gate, up, down = {wbytes} weight bytes) of the same workload",
            "cpu_count": os.cpu_count()}


def bench_quant_cpu():
    """The reference's own micro-benchmark loop for a 4-bit GEMV (benches/bench_quant.rs, quant/gemv_q4 at
    K = N = 4096: simplified nibble format, one scalar call per row), restated in C and built -O1 like the
    reference's bench profile, one thread.  Reported beside config 1, which has the same shape."""
    import numpy as np
    from oracle import oracle as O
    k = n = 4096
    rng = np.random.default_rng(20241)
    w = rng.integers(0, 256, size=n * k // 2, dtype=np.uint8)
    x = rng.standard_normal(k, dtype=np.float32)
    sc = rng.random(n, dtype=np.float32)
    O.bench_gemv_q4_rows(w, x, sc, n, k)
    reps, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < 2.0:
        O.bench_gemv_q4_rows(w, x, sc, n, k)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"kernel": "scalar_gemv_q4 row loop, 1x4096x4096, -O1, 1 thread", "us": dt * 1e6, "gflops": 2.0 * n * k / dt / 1e9,
            "weight_GBps": n * k / 2 / dt / 1e9, "reps": reps}


def parity_record(K, w, host, x_dev, x_host, M, rows=2048):
    """The first product of the step on its first `rows` weight rows: this implementation and the CPU port of the
    reference, each against the other and against an f64-accumulated evaluation of the decoded weights."""
    import numpy as np
    from oracle import oracle as O
    name, n, k, blocks = host
    sub = np.ascontiguousarray(blocks.reshape(n, -1)[:rows]).reshape(-1)
    y_gpu = K.gemv(w, x_dev).cpu().numpy()[:, :rows]
    y_cpu = O.quant_matmul(sub, np.ascontiguousarray(x_host.T), O.Q4K, rows, M, k).T
    y_f64 = x_host.astype(np.float64) @ O.dequant_matrix(O.Q4K, sub, rows, k).astype(np.float64).T
    return {"metric": "max_i |y_i - ref_i| / max(|ref_i|, rms(ref))", "rows": rows, "matrix": name,
            "gpu_vs_cpu_port": O.rel_err(y_gpu, y_cpu), "gpu_vs_f64": O.rel_err(y_gpu, y_f64),
            "cpu_port_vs_f64": O.rel_err(y_cpu, y_f64), "bar": 2e-3}


# ------------------------------------------------------------------------------------------------
def run_reference(args):
    """The reference's CPU algorithm for the same workload on the host cores (all threads, row-parallel).
    The reference is Rust and cannot be built in this image, so this runs the C port in oracle/."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as O
    threads = os.cpu_count() or 1
    M, L = args.m, args.layers
    # gate and up read the same x: by default they are stored as ONE weight of 2*N_ff rows (a load-time layout
    # choice like the repack itself: same bytes, same arithmetic, y = gate || up), so a layer is two products
    fused = not args.separate_gate_up
    shapes = ([("gate_up", 2 * N_FF, D_MODEL), ("down", D_MODEL, N_FF)] if fused else
              [("gate", N_FF, D_MODEL), ("up", N_FF, D_MODEL), ("down", D_MODEL, N_FF)])
    rng = np.random.default_rng(20244)
    # one layer of distinct weights, reused for every layer of the step (CPU caches are far smaller than a matrix)
    host_blocks = []
    for name, n, k in shapes:
        W = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
        host_blocks.append((name, n, k, O.quantize_q4_k(W)))
        del W
    x_model = rng.standard_normal((M, D_MODEL), dtype=np.float32)
    x_ff = rng.standard_normal((M, N_FF), dtype=np.float32)
    xt_model, xt_ff = np.ascontiguousarray(x_model.T), np.ascontiguousarray(x_ff.T)
    layer_bytes = sum(b.size for (_, _, _, b) in host_blocks)

    def step():  # bounded sample: one layer per step, scaled to the L-layer step below
        for name, n, k, b in host_blocks:
            O.quant_matmul(b, xt_ff if name == "down" else xt_model, O.Q4K, n, M, k, threads=threads)
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = layer_bytes / dt / 1e9
    out = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 1), "ms_per_step": dt * 1e3 * L, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE_REF, "data": "synthetic",
        "config": workload_config(L, M, fused),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"each step = one layer (gate, up, down, {layer_bytes} weight bytes) of the "
                                   f"{L}-layer step; ms_per_step is scaled x{L}"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


def run_prefill_case(args):
    """One prefill kernel on its own: `prefill_q4k` = config 5 gate matrix at M = 512 (tcgen05 kind::f16 with fused
    Q4_K dequant), `prefill_nvfp4` = config 4 (NVFP4 x NVFP4, block-scaled tcgen05).  One JSON line."""
    import torch
    gk = importlib.import_module("gllm-kernels_b200")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    K = gk.GpuKernels(0)
    gen = torch.Generator(device=dev).manual_seed(20245)
    QT = gk.QuantType
    if args.case == "decode_q6k":
        return run_gguf_case(args, K, gk, torch, dev, gen)
    if args.case == "decode_nvfp4":
        return run_fp4_decode_case(args, K, gk, torch, dev, gen)
    if args.case == "prefill_w8a8":
        return run_w8a8_case(args, K, gk, torch, dev, gen)
    if args.case == "prefill_q6k":
        # Q6_K down projection of the same model, reference-layout blocks with random payloads and small scales
        n, k, m = D_MODEL, N_FF, 512
        nblk = n * (k // 256)
        b = torch.randint(0, 256, (nblk, 210), generator=gen, device=dev, dtype=torch.uint8)
        b[:, 208:210] = ((torch.rand((nblk, 1), generator=gen, device=dev) - 0.5) * 0.04).to(torch.float16).view(torch.uint8)
        w = K.upload(QT.q6k(), n, k, b.reshape(-1))
        del b
        a = torch.randn((m, k), generator=gen, device=dev)
        y = torch.empty((m, n), dtype=torch.float32, device=dev)
        fn = lambda: K.gemm(w, a, y=y)
        kernel, peak_key, launches = "gemm_wq_kernel<Q6_K, 2 row tiles> (+ stage_act_kernel)", "bf16_tflops", 2
    elif args.case == "prefill_q4k":
        n, k, m = N_FF, D_MODEL, 512
        W = torch.randn((n, k), generator=gen, device=dev) * 0.02
        w = K.upload(QT.q4k(), n, k, K.quantize(QT.q4k(), W))
        del W
        a = torch.randn((m, k), generator=gen, device=dev)
        y = torch.empty((m, n), dtype=torch.float32, device=dev)
        fn = lambda: K.gemm(w, a, y=y)
        kernel, peak_key, launches = "gemm_wq_kernel<Q4_K, 2 row tiles> (+ stage_act_kernel)", "bf16_tflops", 2
    else:
        n, k, m = 14336, 4096, 2048
        W = torch.randn((n, k), generator=gen, device=dev) * 0.02
        X = torch.randn((m, k), generator=gen, device=dev)
        wb, gw = K.quantize(QT.nvfp4(), W)
        xb, gx = K.quantize(QT.nvfp4(), X)
        w, x = K.upload(QT.nvfp4(), n, k, wb, None, gw), K.upload(QT.nvfp4(), m, k, xb, None, gx)
        y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        fn = lambda: K.gemm_fp4(w, x, y=y)
        kernel, peak_key, launches = "gemm_fp4_pair_kernel", None, 1
    for _ in range(max(args.warmup, 3)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    tflops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    peak, kind = 9000.0, "nominal dense FP4"
    ceiling = None
    variants = None
    if not peak_key:
        # the same product on the other FP4 x FP4 kernels the "gemm_fp4_pair" knob selects (the headline is the default, 1)
        variants = {}
        for v, name in ((0, "one_cta_128x128"), (1, "cta_pair_256x256_one_accumulator"), (2, "cta_pair_256x192_two_accumulators"),
                        (3, "cta_pair_256x128_two_accumulators")):
            K.set("gemm_fp4_pair", v)
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            variants[name] = {"us": e0.elapsed_time(e1) / args.steps * 1e3, "status": K.status()}
        K.set("gemm_fp4_pair", 1)
        # what the same MMA reaches on operands parked in shared memory (no copies, no epilogue), with and without the
        # per-k-step scale-factor copies: the practical ceiling of this kernel on this device
        ceiling = {"mma_and_scale_warps_cta_pair": K.probe_fp4_mma(True, 2), "mma_and_scale_copies_cta_pair": K.probe_fp4_mma(True, 1),
                   "mma_only_cta_pair": K.probe_fp4_mma(True, 0), "mma_and_scale_warps_one_cta": K.probe_fp4_mma(False, 2),
                   "mma_and_scale_copies_one_cta": K.probe_fp4_mma(False, 1), "mma_only_one_cta": K.probe_fp4_mma(False, 0),
                   "unit": "TFLOP/s", "how": "gllmk_probe_fp4_mma: 4096 k-steps of 4 block-scaled MMAs per CTA, best of 3 launches"}
    if peak_key:
        pth = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(pth):
            with open(pth) as f:
                peak, kind = float(json.load(f)[peak_key]), "measured (cuBLAS bf16, burst)"
        else:
            peak, kind = 1590.0, "fallback"
    print(json.dumps({"metric": f"prefill GEMM TFLOP/s ({args.case})", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
                      "data": "synthetic", "config": {"workload": args.case, "n": n, "k": k, "m": m},
                      "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                                   "traffic": None, "peak_kind": kind, "kernel": kernel, "measured_mma_ceiling": ceiling, "kernel_variants": variants,
                                   "frac_of_measured_ceiling": (tflops / ceiling["mma_and_scale_warps_cta_pair"]) if ceiling else None},
                      "gpu_launches": args.steps * launches, "status": K.status()}), flush=True)


def run_fp4_decode_case(args, K, gk, torch, dev, gen):
    """NVFP4 decode product on its own: W[28672, 8192] (the gate matrix of config 5), M = 1, on the block-scaled
    tensor core; two weight copies in rotation (2 x 132 MB > L2)."""
    qt = gk.QuantType.nvfp4()
    n, k = N_FF, D_MODEL
    ws = []
    for _ in range(2):
        W = torch.randn((n, k), generator=gen, device=dev) * 0.02
        wb, gw = K.quantize(qt, W)
        ws.append(K.upload(qt, n, k, wb, None, gw))
        del W, wb
    x = torch.randn((1, k), generator=gen, device=dev)
    y = torch.empty((1, n), dtype=torch.float32, device=dev)
    for i in range(max(args.warmup, 3)):
        K.gemv(ws[i % 2], x, y=y)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        K.gemv(ws[i % 2], x, y=y)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    wbytes = n * k // 2 + n * k // 16
    gbs = wbytes / (ms * 1e-3) / 1e9
    peak, kind = measured_peaks()
    print(json.dumps({"metric": "NVFP4 decode weight GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
                      "config": {"workload": args.case, "n": n, "k": k, "m": 1, "l2": "two weight copies in rotation"},
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                   "traffic": None, "peak_kind": kind, "kernel": "gemv_fp4_tc_kernel (+ fd_stage_kernel)"},
                      "gpu_launches": args.steps * 2, "status": K.status()}), flush=True)


def run_w8a8_case(args, K, gk, torch, dev, gen):
    """W8A8 prefill product on its own: u8 activations [2048, 4096] x s8 W[11008, 4096] -> s32, exact (tcgen05 kind::i8
    on CTA pairs)."""
    n, k, m = 11008, 4096, 2048
    b = torch.randint(-128, 128, (n, k), generator=gen, device=dev, dtype=torch.int8)
    w = K.upload_int8(b, layout_kn=False)
    a8 = torch.randint(0, 256, (m, k), generator=gen, device=dev, dtype=torch.uint8)
    c32 = torch.empty((m, n), dtype=torch.int32, device=dev)
    fn = lambda: K.gemm_int8(w, a8, c=c32)
    for _ in range(max(args.warmup, 3)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    tops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    rows = torch.arange(0, m, 64, device=dev)
    exact = bool(torch.equal(c32[rows].to(torch.float64), a8[rows].to(torch.float64) @ b.to(torch.float64).t()))
    print(json.dumps({"metric": "W8A8 prefill GEMM TOP/s", "value": tops, "unit": "TOP/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
                      "config": {"workload": args.case, "n": n, "k": k, "m": m},
                      "roofline": {"bound": "tensor", "achieved": tops, "peak": 4500.0, "unit": "TOP/s", "frac": tops / 4500.0,
                                   "traffic": None, "peak_kind": "nominal dense int8", "kernel": "gemm_i8_pair_kernel (+ stage_act_u8_kernel)"},
                      "parity": {"exact_on_sampled_rows": exact, "rows": int(rows.numel())},
                      "gpu_launches": args.steps * 2, "status": K.status()}), flush=True)


def run_gguf_case(args, K, gk, torch, dev, gen):
    """Q6_K decode product on its own: W[8192, 28672] (the down projection of config 5), M = --m tokens (1: the dp2a kernel,
    2 .. 16: the mma.sync kernel), two weight copies in rotation (2 x 193 MB > L2)."""
    qt = gk.QuantType.q6k()
    n, k = D_MODEL, N_FF
    nblk = n * (k // 256)
    ws = []
    for _ in range(2):
        b = torch.randint(0, 256, (nblk, 210), generator=gen, device=dev, dtype=torch.uint8)
        d = ((torch.rand((nblk, 1), generator=gen, device=dev) - 0.5) * 0.04).to(torch.float16)
        b[:, 208:210] = d.view(torch.uint8)
        ws.append(K.upload(qt, n, k, b.reshape(-1)))
        del b, d
    m = max(1, min(int(args.m), 16))
    x = torch.randn((m, k), generator=gen, device=dev)
    y = torch.empty((m, n), dtype=torch.float32, device=dev)
    for i in range(max(args.warmup, 3)):
        K.gemv(ws[i % 2], x, y=y)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        K.gemv(ws[i % 2], x, y=y)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    wbytes = nblk * 210
    gbs = wbytes / (ms * 1e-3) / 1e9
    peak, kind = measured_peaks()
    print(json.dumps({"metric": "Q6_K decode weight GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
                      "config": {"workload": args.case, "n": n, "k": k, "m": m, "l2": "two weight copies in rotation"},
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                   "traffic": None, "peak_kind": kind, "kernel": ("raw_gemv_kernel<Q6_K, 1>" if m == 1 else "q6k_gemv_mma_kernel") + " (+ act_quant_kernel)"},
                      "gpu_launches": args.steps * 2, "status": K.status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--separate-gate-up", action="store_true", help="keep gate and up as two weights (3 products per layer)")
    ap.add_argument("--gemv-ctas-per-sm", type=int, default=0, help="tuning knob: resident GEMV CTAs per SM (0 = occupancy limit)")
    ap.add_argument("--gemv-fuse", type=int, default=-1,
                    help="tuning knob: decode GEMV converting its own activation slices (0 never, 1 exchange products, 2 always; -1 = library default)")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the bands of y reach every rank (peer stores fused into the GEMV, or NCCL all-gather)")
    ap.add_argument("--case", default="decode", choices=["decode", "prefill_q4k", "prefill_q6k", "prefill_nvfp4", "prefill_w8a8", "decode_q6k", "decode_nvfp4"],
                    help="decode = the headline workload; prefill_* / decode_* = one kernel on its own (1 GPU)")
    args = ap.parse_args()
    if args.case != "decode":
        run_prefill_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
