"""Parity at the benchmark's own shapes (the five configurations the throughput numbers are quoted on).

The weights are drawn and quantized on the device (the device quantizers are byte-identical to the oracle's,
tests/test_gpu_parity.py), the product runs at full size through the C ABI, and 256 sampled weight rows x every
token are compared with the CPU oracle (bench.sampled_parity: the reference's quantized matmul for the f32
decode path, its decode followed by its f32 GEMM loop order where operands are staged in 16 bits or the
reference has no matmul at all).  Bars: 2e-3 for f32-accumulated exact-operand paths, 1e-2 where operands are
staged in fp16 / bf16.
"""
import numpy as np
import pytest

import bench

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K(gk):
    k = gk.GpuKernels(0)
    yield k
    k.close()


def device_weight(gk, K, torch, qt, n, k, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    W = torch.randn((n, k), generator=g, device="cuda") * 0.02
    q = K.quantize(qt, W)
    del W
    if qt.id == 3:
        return K.upload(qt, n, k, q[0], q[1]), q[0], q[1], 1.0, g
    if qt.id == 4:
        return K.upload(qt, n, k, q[0], None, q[1]), q[0], None, q[1], g
    return K.upload(qt, n, k, q), q, None, 1.0, g


@pytest.mark.parametrize("n,k", [(28672, 8192), (8192, 28672)])
@pytest.mark.parametrize("m", [1, 16, 32, 512])
def test_q4k_70b_ffn_matrices_at_every_batch(gk, K, oracle, n, k, m):
    """W[28672, 8192] (gate / up) and W[8192, 28672] (down), Q4_K, x[M, K] f32 ~ N(0, 1), M in {1, 16, 32, 512}."""
    import torch
    w, blocks, _, _, g = device_weight(gk, K, torch, gk.QuantType.q4k(), n, k, 20244)
    x = torch.randn((m, k), generator=g, device="cuda")
    y = K.gemm(w, x) if m > 16 else K.gemv(w, x)
    torch.cuda.synchronize()
    assert K.status() == 0
    tensor_core = m > gk.GpuKernels.GEMM_GEMV_MAX_M
    rec = bench.sampled_parity(oracle, oracle.Q4K, blocks, n, k, bench.sample_rows(n, 256, seed=m), x.cpu().numpy(), y,
                               bar=1e-2 if tensor_core else 2e-3, sequential=not tensor_core)
    assert rec["ok"], rec
    w.free()


def test_nvfp4_prefill_14336x4096_m2048(gk, K, oracle):
    """W[14336, 4096] NVFP4 x A[2048, 4096] NVFP4 (quantized the same way from N(0, 1)), bf16 out, block-scaled MMA.
    Codes and scales are consumed exactly: the f32 bar applies, plus the bf16 rounding of the output (half an ulp of an
    8-bit significand: up to 2^-8 of the value)."""
    import torch
    n, k, m = 14336, 4096, 2048
    qt = gk.QuantType.nvfp4()
    w, wb, _, gw, g = device_weight(gk, K, torch, qt, n, k, 20243)
    X = torch.randn((m, k), generator=g, device="cuda")
    xb, gx = K.quantize(qt, X)
    x = K.upload(qt, m, k, xb, None, gx)
    a_host = oracle.dequant_matrix(oracle.NVFP4, xb.cpu().numpy(), m, k, global_scale=gx)
    for dtype, bar in ((torch.float32, 2e-3), (torch.bfloat16, 2e-3 + 2.0 ** -8)):
        y = K.gemm_fp4(w, x, out_dtype=dtype)
        torch.cuda.synchronize()
        assert K.status() == 0
        rec = bench.sampled_parity(oracle, oracle.NVFP4, wb, n, k, bench.sample_rows(n, 256, seed=4), a_host, y, bar=bar,
                                   global_scale=gw)
        assert rec["ok"], (dtype, rec)
    w.free()
    x.free()


def test_mxfp4_moe_8_experts_512_tokens_top2(gk, K, oracle):
    """8 experts W[14336, 4096] MXFP4, 512 bf16 tokens, top-2 routing with the reference's conventions
    (scalar_topk: indices as f32 bit patterns, renormalised weights), rows grouped per expert, one grouped launch,
    expert outputs recombined with scalar_weighted_sum's rule.  256 sampled weight rows per expert x that expert's
    tokens against the oracle, and the recombined output on the same rows."""
    import torch
    E, n, k, T, top_k = 8, 14336, 4096, 512, 2
    qt = gk.QuantType.mxfp4(32)
    ws, blk, scl = [], [], []
    for e in range(E):
        w, b, s, _, g = device_weight(gk, K, torch, qt, n, k, 20242 + 100 * e)
        ws.append(w), blk.append(b), scl.append(s)
    x = torch.randn((T, k), generator=g, device="cuda").to(torch.bfloat16)
    # expert ids uniform from the seed (distinct per token): probabilities whose two largest entries are those experts
    probs = torch.rand((T, E), generator=g, device="cuda")
    probs = probs / probs.sum(dim=1, keepdim=True)
    routing = K.moe_topk(probs, top_k)                    # [2, T * top_k]: index bit patterns | weights
    offs, perm, inv = K.moe_route(routing, T, E, top_k)   # rows grouped per expert
    a = K.moe_gather(x, perm, top_k)                      # [T * top_k, k] bf16
    y = K.gemm_grouped(ws, a, offs, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert K.status() == 0
    # conventions against the oracle's restatement of scalar_topk
    ref_routing = oracle.scalar_topk(probs.cpu().numpy(), top_k)
    assert np.array_equal(routing.cpu().numpy().view(np.uint32), ref_routing.view(np.uint32))
    idx = ref_routing[0].view(np.uint32).reshape(T, top_k)
    assert (idx[:, 0] != idx[:, 1]).all()
    counts = np.bincount(idx.reshape(-1), minlength=E)
    assert offs == [0] + np.cumsum(counts).tolist()
    a_host = a.to(torch.float32).cpu().numpy()
    worst = 0.0
    for e in range(E):
        r0, r1 = offs[e], offs[e + 1]
        rec = bench.sampled_parity(oracle, oracle.MXFP4, blk[e], n, k, bench.sample_rows(n, 256, seed=e), a_host[r0:r1],
                                   y[r0:r1], bar=1e-2, scales=scl[e])
        assert rec["ok"], (e, rec)
        worst = max(worst, rec["rel_err"])
    # recombination: out[t] = sum_ki weight[t, ki] * y[row of (t, ki)], ki ascending, bit-exact with the oracle's rule
    out = K.moe_weighted_sum(y, routing, inv, T, top_k)
    inv_host = np.empty(T * top_k, np.int64)
    inv_host[perm.cpu().numpy()] = np.arange(T * top_k)
    assert np.array_equal(inv.cpu().numpy(), inv_host)
    ref = oracle.scalar_weighted_sum_grouped(y.cpu().numpy(), ref_routing, inv_host, T, top_k)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    for w in ws:
        w.free()


@pytest.mark.parametrize("m", [1, 4, 8, 16])
def test_q8_0_11008x4096_sampled_rows_device_weights(gk, K, oracle, m):
    """W[11008, 4096] Q8_0 at M in {1, 4, 8, 16} with device-quantized weights (the whole-matrix oracle comparison of
    the same shape is in tests/test_gpu_parity.py)."""
    import torch
    n, k = 11008, 4096
    w, blocks, _, _, g = device_weight(gk, K, torch, gk.QuantType.q8_0(), n, k, 20241)
    x = torch.randn((m, k), generator=g, device="cuda")
    y = K.gemv(w, x)
    rec = bench.sampled_parity(oracle, oracle.Q8_0, blocks, n, k, bench.sample_rows(n, 256, seed=m), x.cpu().numpy(), y, bar=2e-3,
                               sequential=True)
    assert rec["ok"], rec
    w.free()
