"""GGUF container reader / writer (host logic, no GPU) and loading tensors into HBM (GPU)."""
import os
import struct

import numpy as np
import pytest


def _blocks(qt, n, k, seed):
    rng = np.random.default_rng(seed)
    b = rng.integers(0, 256, size=(n * (k // qt.block_size()), qt.block_bytes()), dtype=np.uint8)
    half = np.frombuffer(rng.uniform(-0.02, 0.02, b.shape[0]).astype(np.float16).tobytes(), np.uint8).reshape(-1, 2)
    if qt.name == "Q6K":
        b[:, 208:210] = half
    elif qt.name == "Q8K":
        b[:, 0:4] = np.frombuffer(rng.uniform(-0.02, 0.02, b.shape[0]).astype(np.float32).tobytes(), np.uint8).reshape(-1, 4)
    else:
        b[:, 0:2] = half
        if qt.name in ("Q4K", "Q5K"):
            b[:, 2:4] = half
    return b.reshape(-1)


def _make(gk, path):
    Q = gk.QuantType
    spec = {"blk.0.ffn_down.weight": (Q.q6k(), 24, 512), "blk.0.ffn_gate.weight": (Q.q4k(), 40, 256),
            "blk.0.attn_q.weight": (Q.q8_0(), 16, 96), "blk.0.attn_k.weight": (Q.q5_0(), 8, 64),
            "blk.0.attn_v.weight": (Q.q4_0(), 8, 64), "blk.0.ffn_up.weight": (Q.q5k(), 8, 256),
            "act.weight": (Q.q8k(), 4, 256)}
    tensors = {name: (qt, n, k, _blocks(qt, n, k, i)) for i, (name, (qt, n, k)) in enumerate(spec.items())}
    tensors["output_norm.weight"] = np.arange(64, dtype=np.float32).reshape(1, 64)
    tensors["half.weight"] = np.linspace(-1, 1, 32, dtype=np.float16).reshape(2, 16)
    gk.write_gguf(path, tensors, {"general.architecture": "llama", "llama.block_count": 1, "llama.rope.scale": 0.5,
                                  "big": 1 << 40, "flag": True})
    return tensors


def test_round_trip_of_the_container(gk, tmp_path):
    path = str(tmp_path / "m.gguf")
    tensors = _make(gk, path)
    with gk.GgufFile(path) as g:
        assert g.version == 3 and g.alignment == 32
        assert g.metadata["general.architecture"] == "llama" and g.metadata["llama.block_count"] == 1
        assert g.metadata["big"] == 1 << 40 and g.metadata["flag"] is True and g.metadata["llama.rope.scale"] == 0.5
        info = g.tensors()
        assert set(info) == set(tensors)
        assert g.data_start % 32 == 0
        for name, t in tensors.items():
            i = info[name]
            assert i.offset % 32 == 0
            if isinstance(t, tuple):
                qt, n, k, blocks = t
                assert (i.n, i.k) == (n, k) and i.quant_type == qt and i.nbytes == blocks.size
                assert np.array_equal(g.raw(name), blocks)
            else:
                assert np.array_equal(g.load(None, name), t)


def test_rejects_bad_files(gk, tmp_path):
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 60)
    with pytest.raises(gk.GgufError):
        gk.GgufFile(str(bad))
    path = str(tmp_path / "m.gguf")
    _make(gk, path)
    data = open(path, "rb").read()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(data[: len(data) // 2])  # tensor data past the end
    with pytest.raises(gk.GgufError):
        gk.GgufFile(str(cut))
    v9 = tmp_path / "v9.gguf"
    v9.write_bytes(data[:4] + struct.pack("<I", 9) + data[8:])
    with pytest.raises(gk.GgufError):
        gk.GgufFile(str(v9))
    # a tensor type the kernels do not serve is listed, and refused on load
    unk = tmp_path / "unk.gguf"
    head = struct.pack("<IIQQ", gk.gguf.GGUF_MAGIC, 3, 1, 0)
    name = b"w"
    head += struct.pack("<Q", len(name)) + name + struct.pack("<IQQIQ", 2, 256, 2, 10, 0)  # Q2_K
    unk.write_bytes(head + b"\0" * (64 - len(head) % 64) + b"\0" * 256)
    with gk.GgufFile(str(unk)) as g:
        assert g.tensors()["w"].ggml_type == 10 and g.tensors()["w"].quant_type is None
        with pytest.raises(gk.GgufError):
            g.load(None, "w")
    with pytest.raises(gk.GgufError):  # row length not a multiple of the block size
        gk.write_gguf(str(tmp_path / "x.gguf"), {"w": (gk.QuantType.q4k(), 1, 128, np.zeros(72, np.uint8))})


@pytest.mark.gpu
def test_load_into_hbm_and_multiply(gk, oracle, tmp_path):
    import torch
    path = str(tmp_path / "m.gguf")
    tensors = _make(gk, path)
    K = gk.GpuKernels(0)
    try:
        with gk.GgufFile(path) as g:
            loaded = g.load_all(K)
        assert set(loaded) == set(tensors)
        for name, t in tensors.items():
            if not isinstance(t, tuple):
                assert np.array_equal(loaded[name], t)
                continue
            qt, n, k, blocks = t
            w = loaded[name]
            ref_w = oracle.dequant_matrix(qt.id, blocks, n, k)
            got = K.dequant(w).cpu().numpy()
            assert np.array_equal(got.view(np.uint32), ref_w.view(np.uint32)), name
            x = np.random.default_rng(3).standard_normal((2, k)).astype(np.float32)
            ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), qt.id, n, 2, k)
            y = K.gemv(w, torch.from_numpy(x).cuda()).cpu().numpy()
            assert oracle.rel_err(y.T, ref) <= 2e-3, name
            w.free()
    finally:
        K.close()
