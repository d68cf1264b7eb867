"""gllmk_gemv_static — the decode GEMV for hosts that may not allocate device memory while they run
(an inference loop whose allocator already owns all of HBM, or a section where cudaMalloc's implicit
synchronisation is not tolerable).  Its scratch is a fixed array inside the library, so the test checks,
through the C ABI, that it gives what gllmk_gemv gives — on two calls in a row, because the second call
starts from whatever the first one left in that array — and that oversized shapes are refused.

This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K(gk):
    k = gk.GpuKernels(0)
    yield k
    k.close()


@pytest.mark.parametrize("fmt,n,k,m", [("q4k", 4096, 4096, 1), ("q4k", 1000, 2048, 5), ("q8_0", 2000, 1056, 16)])
def test_static_scratch_gemv_matches_gemv_twice(gk, K, oracle, fmt, n, k, m):
    import torch
    rng = np.random.default_rng(123)
    W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    if fmt == "q4k":
        qt, blocks, oid = gk.QuantType.q4k(), oracle.quantize_q4_k(W), oracle.Q4K
    else:
        qt, blocks, oid = gk.QuantType.q8_0(), oracle.quantize_q8_0(W), oracle.Q8_0
    w = K.upload(qt, n, k, blocks)
    for call in range(2):  # second call: different activations, same scratch
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
        want = K.gemv(w, x)
        got = torch.full((m, n), float("nan"), device="cuda")
        K.gemv_static(w, x, got)
        torch.cuda.synchronize()
        assert K.status() == 0
        # the same kernels run with the same partition: identical results, and both within the parity bar
        assert torch.equal(got, want), f"call {call}"
        ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.cpu().numpy().T), oid, n, m, k, threads=8).T
        assert oracle.rel_err(got.cpu().numpy(), ref) <= 2e-3
    w.free()


def test_static_scratch_rejects_shapes_beyond_its_area(gk, K):
    import torch
    n, k, m = 131200, 32, 1  # 8200 row tiles: more arrival counters than the built-in area has
    qt = gk.QuantType.q8_0()
    blocks = torch.zeros(n * (k // 32) * 34, dtype=torch.uint8, device="cuda")
    w = K.upload(qt, n, k, blocks)
    x = torch.zeros((m, k), device="cuda")
    y = torch.zeros((m, n), device="cuda")
    with pytest.raises(gk.GllmkError) as e:
        K.gemv_static(w, x, y)
    assert e.value.status == gk.Status.INVALID_ARG and "8388608" in str(e.value)
    K.gemv(w, x, y=y)  # the allocating entry point still serves it
    torch.cuda.synchronize()
    w.free()
