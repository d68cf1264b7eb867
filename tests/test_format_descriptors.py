"""QuantFormatDescriptor::for_type / registry() of the library against the reference's own registry, transcribed
from its source by tests/golden/make_format_descriptors.py.  The table checked here is the one the repack kernels,
the decoders and the raw-block GEMV compile their byte offsets from (csrc/quant_format.cuh), so a wrong offset fails
here on the CPU and in the bit-exact decode tests on the GPU.  No device needed."""
import json
import os
import struct

import numpy as np
import pytest

with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_format_descriptors.json")) as f:
    REF = json.load(f)["formats"]


def variant(v):
    return "None" if v is None else (v["variant"] if isinstance(v, dict) else v)


def test_registry_lists_the_served_formats(gk):
    reg = gk.registry()
    assert sorted(reg) == sorted(REF)
    for name, d in reg.items():
        assert gk.QuantFormatDescriptor.for_type(d.quant_type) == d


@pytest.mark.parametrize("name", sorted(REF))
def test_descriptor_equals_the_reference(gk, name):
    r, d = REF[name], gk.registry()[name]
    assert (d.block_size, d.block_bytes, d.bits_per_element) == (r["block_size"], r["block_bytes"], r["bits_per_element"])
    assert d.block_size == d.quant_type.block_size() and d.block_bytes == d.quant_type.block_bytes() and d.bits_per_element == d.quant_type.bits()
    assert d.data_kind == r["data_kind"] and d.storage_layout == r["storage_layout"] and d.native_isa == r["native_isa"]
    sl, zl, dl = r["scale_layout"], r["zero_layout"], r["data_layout"]
    assert d.scale_kind == variant(sl) and d.zero_kind == variant(zl) and d.data_layout == variant(dl)
    if d.scale_kind == "BlockScalar":
        assert (d.scale_offset, d.scale_dtype) == (sl["offset_bytes"], sl["dtype"])
    elif d.scale_kind == "Hierarchical":
        assert (d.scale_offset, d.scale_min_offset, d.sub_scales_offset, d.sub_scales_bits, d.sub_scales_count, d.sub_block_elements) == \
            (sl["block_d_offset"], sl["block_dmin_offset"], sl["sub_scales_offset"], sl["sub_scales_bits"], sl["sub_scales_count"],
             sl["sub_block_elements"])
        assert sl["packed_layout"]["algorithm"] == "KQuant6Bit"
    elif d.scale_kind == "Q6KScales":
        assert (d.scale_offset, d.sub_scales_offset, d.sub_scales_count, d.sub_block_elements) == \
            (sl["block_d_offset"], sl["sub_scales_offset"], sl["sub_scales_count"], sl["sub_block_elements"])
    elif d.scale_kind == "SubBlockScalars":
        assert (d.scale_offset, d.sub_block_elements, d.scale_dtype) == (sl["offset_bytes"], sl["sub_block_size"], sl["dtype"])
    else:
        raise AssertionError(d.scale_kind)
    if d.zero_kind == "Hierarchical":
        assert (d.zero_offset, d.zero_sub_offset) == (zl["dmin_offset"], zl["sub_m_offset"])
    elif d.zero_kind == "StaticBias":
        assert d.static_bias == zl["value"]
    else:
        assert d.zero_kind == "None"
    if d.data_layout == "PackedNibbles":
        assert (d.data_offset, d.data_low_first) == (dl["offset"], dl["low_first"])
    elif d.data_layout == "NibbleWithHighBits":
        assert (d.data_offset, d.data_high_offset, d.data_high_bits) == (dl["low_offset"], dl["high_offset"], dl["high_bits_per_elem"])
    else:
        assert (d.data_offset, d.data_signed) == (dl["offset"], dl["signed"])


def test_unserved_type_is_an_error(gk):
    with pytest.raises(gk.GllmkError) as e:
        gk.QuantFormatDescriptor.for_type(gk.QuantType(99))
    assert e.value.status == gk.Status.UNSUPPORTED


def test_mxfp4_descriptor_follows_the_block_size(gk):
    for bs in (16, 32, 64):
        d = gk.QuantFormatDescriptor.for_type(gk.QuantType.mxfp4(bs))
        assert (d.block_size, d.block_bytes, d.data_offset) == (bs, 1 + bs // 2, 1)


@pytest.mark.parametrize("name", ["Q4_0", "Q5_0", "Q8_0", "Q4_K", "Q5_K", "Q6_K", "Q8_K"])
def test_oracle_decoders_read_the_fields_where_the_descriptor_says(gk, oracle, name):
    """A block built FROM the descriptor (scale = 1 at scale_offset, one data byte set at data_offset, everything else
    zero) decodes, by the oracle's restatement of the reference decoders, to what the descriptor's layout implies."""
    d = gk.registry()[name]
    oid = {"Q4_0": oracle.Q4_0, "Q5_0": oracle.Q5_0, "Q8_0": oracle.Q8_0, "Q4_K": oracle.Q4K, "Q5_K": oracle.Q5K, "Q6_K": oracle.Q6K,
           "Q8_K": oracle.Q8K}[name]
    b = np.zeros(d.block_bytes, np.uint8)
    one = struct.pack("<f", 1.0) if d.scale_dtype == "F32" else struct.pack("<e", 1.0)
    b[d.scale_offset:d.scale_offset + len(one)] = np.frombuffer(one, np.uint8)
    if d.scale_kind == "Hierarchical":
        b[d.sub_scales_offset] = 3                      # 6-bit scale of sub-block 0
    if d.scale_kind == "Q6KScales":
        b[d.sub_scales_offset] = 3                      # i8 scale of the first 16 elements
    b[d.data_offset] = 0x05                             # element 0 <- code 5 (low nibble first / first byte)
    out = oracle.dequant_matrix(oid, b, 1, d.block_size)[0]
    sub = 3.0 if d.scale_kind in ("Hierarchical", "Q6KScales") else 1.0
    assert out[0] == sub * (5 - d.static_bias)
