"""Mixture-of-experts conventions on the device against the oracle's restatement of scalar-ops/src/moe.rs:
scalar_topk (indices as u32 bit patterns in f32 slots, renormalised weights), the per-expert grouping that feeds
gllmk_gemm_grouped, and scalar_weighted_sum.  All bit-exact."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_known_answers.json")) as f:
    KA = json.load(f)


@pytest.fixture(scope="module")
def K(gk):
    k = gk.GpuKernels(0)
    yield k
    k.close()


def test_reference_known_answers(gk, K):
    import torch
    c = KA["moe_topk"]
    probs = torch.tensor(c["probs"], device="cuda").reshape(c["seq_len"], c["num_experts"])
    out = K.moe_topk(probs, c["top_k"]).cpu().numpy()
    assert out[0].view(np.uint32).tolist() == c["expect_indices"]
    assert abs(out[1].sum() - c["weights_sum"]) < c["weights_sum_tol"]
    c = KA["moe_weighted_sum"]
    routing = torch.from_numpy(np.stack([np.array(c["indices"], np.uint32).view(np.float32), np.array(c["weights"], np.float32)])).cuda()
    eo = torch.tensor(c["expert_outputs"], device="cuda").reshape(1, c["seq_len"], c["hidden"])
    got = K.moe_weighted_sum(eo, routing, None, c["seq_len"], c["top_k"])
    assert got.cpu().numpy().reshape(-1).tolist() == c["expect"]


@pytest.mark.parametrize("T,E,top_k", [(1, 4, 2), (37, 8, 2), (512, 8, 2), (100, 64, 6), (33, 5, 5), (1000, 128, 1)])
def test_topk_route_gather_weighted_sum_bit_exact(gk, K, oracle, T, E, top_k):
    import torch
    rng = np.random.default_rng(T + E)
    probs = rng.random((T, E), dtype=np.float32)
    probs[0, :] = 0.25                      # ties: the earlier expert wins
    if T > 3:
        probs[1, 0] = np.nan                # never selected
        probs[2, :] = 0.0                   # zero sum -> zero weights
    probs_d = torch.from_numpy(probs).cuda()
    routing = K.moe_topk(probs_d, top_k)
    ref = oracle.scalar_topk(probs, top_k)
    got = routing.cpu().numpy()
    # (a row with fewer selectable experts than top_k has -inf entries left: its weights are NaN on both sides, whose
    # bit patterns differ between the CPU and the GPU)
    same = (got.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(got) & np.isnan(ref))
    assert same.all()
    offs, perm, inv = K.moe_route(routing, T, E, top_k)
    idx = ref[0].view(np.uint32)
    counts = np.bincount(idx, minlength=E)
    assert offs == [0] + np.cumsum(counts).tolist()
    want_perm = np.argsort(idx, kind="stable")  # grouped per expert, slot order kept inside an expert
    assert np.array_equal(perm.cpu().numpy(), want_perm)
    inv_h = np.empty(T * top_k, np.int64)
    inv_h[want_perm] = np.arange(T * top_k)
    assert np.array_equal(inv.cpu().numpy(), inv_h)
    k, H = 96, 40
    for dt in (torch.float32, torch.bfloat16):
        x = torch.randn((T, k), device="cuda").to(dt)
        a = K.moe_gather(x, perm, top_k)
        assert torch.equal(a, x[torch.from_numpy(want_perm // top_k).cuda()])
    rows = torch.randn((T * top_k, H), device="cuda")
    out = K.moe_weighted_sum(rows, routing, inv, T, top_k)
    want = oracle.scalar_weighted_sum_grouped(rows.cpu().numpy(), ref, inv_h, T, top_k)
    a_, b_ = out.cpu().numpy(), want
    assert np.array_equal(a_.view(np.uint32)[~np.isnan(b_)], b_.view(np.uint32)[~np.isnan(b_)]) and np.array_equal(np.isnan(a_), np.isnan(b_))
    # the reference's own buffer layout [expert][seq][hidden]
    eo = torch.randn((E, T, H), device="cuda")
    out = K.moe_weighted_sum(eo, routing, None, T, top_k).cpu().numpy()
    want = oracle.scalar_weighted_sum(eo.cpu().numpy(), ref, T, top_k)
    assert np.array_equal(out.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])


def test_route_skips_indices_no_expert_serves(gk, K):
    """scalar_moe_dispatch_packed skips an index >= num_experts (scalar-ops/src/moe_dispatch_packed.rs:113-116)."""
    import torch
    T, E, top_k = 4, 3, 2
    idx = np.array([0, 7, 2, 2, 1, 0, 9, 1], np.uint32)
    routing = torch.from_numpy(np.stack([idx.view(np.float32), np.full(8, 0.5, np.float32)])).cuda()
    offs, perm, inv = K.moe_route(routing, T, E, top_k)
    assert offs == [0, 2, 4, 6]
    assert perm.cpu().numpy()[:6].tolist() == [0, 5, 4, 7, 2, 3]
    assert inv.cpu().numpy().tolist() == [0, -1, 4, 5, 2, 1, -1, 3]
    rows = torch.arange(6, dtype=torch.float32, device="cuda").reshape(6, 1) + 1.0
    out = K.moe_weighted_sum(rows, routing, inv, T, top_k).cpu().numpy().reshape(-1)
    assert out.tolist() == [0.5 * 1, 0.5 * 5 + 0.5 * 6, 0.5 * 3 + 0.5 * 2, 0.5 * 4]


def test_moe_argument_checks(gk, K):
    import torch
    p = torch.rand((4, 8), device="cuda")
    with pytest.raises(gk.GllmkError) as e:
        K.moe_topk(p, 17)
    assert e.value.status == gk.Status.UNSUPPORTED
    r = K.moe_topk(p, 2)
    with pytest.raises(gk.GllmkError) as e:
        K.moe_route(r, 4, 2000, 2)
    assert e.value.status == gk.Status.UNSUPPORTED
