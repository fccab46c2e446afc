"""Pins the packing oracle to the known-answer tests of the reference
(ml_drift/common/task/weights_conversion_test.cc).  Values below are the ones
those tests state; line numbers refer to that file."""
import numpy as np
import pytest


def _packed_0_to(n):
    # "Fill weights with 0 to n-1 -- packed": byte i = ((2i+1) << 4) | 2i
    return np.array([((2 * i + 1) << 4) | (2 * i) for i in range(n // 2)], np.uint8)


def _pack_expected(nibbles):
    nib = np.array(nibbles, np.uint8)
    return ((nib[0::2] | (nib[1::2] << 4)) ^ 0x88).astype(np.uint8)


def test_uint4_packed_base(oracle):
    # weights_conversion_test.cc:50-91
    out, sums = oracle.rearrange_uint4_packed(_packed_0_to(16), (4, 1, 1, 4), group=1, pad=8)
    exp = _pack_expected([0, 4, 8, 12, 1, 5, 9, 13, 2, 6, 10, 14, 3, 7, 11, 15])
    assert out.tolist() == exp.tolist()
    assert sums.tolist() == [6, 22, -26, -10]


def test_uint4_packed_zeroes_sum(oracle):
    # :93-135 - a stale value in sum_i[0] is cleared
    out, sums = oracle.rearrange_uint4_packed(_packed_0_to(16), (4, 1, 1, 4), group=1, pad=8,
                                              sum_init=[1, 0, 0, 0])
    assert sums.tolist() == [6, 22, -26, -10]


def test_uint4_packed_vs_int8_source_4x4(oracle):
    # :183-219 - packed-source path == int8-source path, sums == accumulated input channels
    q = np.array([-8, -7, -6, -5, -4, -3, -2, -1, 0, 1, 2, 3, 4, 5, 6, 7], np.int8).reshape(4, 4)
    dense = oracle.pack_int4_dense(q)
    out, sums = oracle.rearrange_uint4_packed(dense, (4, 1, 1, 4), group=1, pad=8)
    ref = oracle.rearrange_int8_as_uint4(q, group=1, shift=8, pad=8)
    assert out.tolist() == ref.tolist()
    assert sums.tolist() == oracle.weights_sum_i(q).tolist()


def test_uint4_packed_pad_o(oracle):
    # :306-348 - O = 3 padded to 4, sum_i has AlignByN(O,4) entries
    out, sums = oracle.rearrange_uint4_packed(_packed_0_to(12), (3, 1, 1, 4), group=1, pad=8,
                                              sum_len=4)
    pad = 8 ^ 0x8
    exp = _pack_expected([0, 4, 8, pad, 1, 5, 9, pad, 2, 6, 10, pad, 3, 7, 11, pad])
    assert out.tolist() == exp.tolist()
    assert sums.tolist() == [6, 22, -26, 0]


def test_uint4_packed_double_pad_i(oracle):
    # :394-438 - I = 2 padded to 4 ("double_pad")
    out, sums = oracle.rearrange_uint4_packed(_packed_0_to(8), (4, 1, 1, 2), group=1, pad=8)
    pad = 8 ^ 0x8
    exp = _pack_expected([0, 2, 4, 6, 1, 3, 5, 7] + [pad] * 8)
    assert out.tolist() == exp.tolist()
    assert sums.tolist() == [1, 5, 9, 13]


def test_uint4_packed_swap_dims(oracle):
    # :440-489 - IHWO source: the transpose cancels, only the 0x88 flip remains
    out, sums = oracle.rearrange_uint4_packed(_packed_0_to(16), (4, 1, 1, 4), group=1, pad=8,
                                              swap_dims=True)
    exp = np.array([((2 * i) | ((2 * i + 1) << 4)) ^ 0x88 for i in range(8)], np.uint8)
    assert out.tolist() == exp.tolist()
    assert sums.tolist() == [-8, -4, 0, 4]


@pytest.mark.parametrize("O,I,group", [(16, 8, 2), (16, 8, 4), (534, 171, None), (7, 6, None), (3, 10, None),
                                        (64, 96, None), (12, 32, 1)])
def test_packed_source_equals_int8_source(oracle, O, I, group):
    # generalises :183-262 to ragged shapes: both entry points give the same bytes and sums
    rng = np.random.default_rng(O * 1000 + I)
    q = rng.integers(-8, 8, size=(O, I), dtype=np.int8)
    dense = oracle.pack_int4_dense(q)
    out, sums = oracle.rearrange_uint4_packed(dense, (O, 1, 1, I), group=group, pad=8)
    ref = oracle.rearrange_int8_as_uint4(q, group=group)
    assert np.array_equal(out, ref)
    assert np.array_equal(sums, oracle.weights_sum_i(q))


def test_int8_layout_is_i4o4(oracle):
    # element (o, i) lands at [i/4][o/4][i%4][o%4] with +128 bias; padding holds 128
    O, I = 6, 10
    q = (np.arange(O * I, dtype=np.int32).reshape(O, I) % 200 - 100).astype(np.int8)
    out = oracle.rearrange_int8_as_uint8(q)
    S, D = 3, 2
    blk = out.reshape(S, D, 4, 4)
    for o in range(8):
        for i in range(12):
            v = blk[i // 4, o // 4, i % 4, o % 4]
            assert v == ((int(q[o, i]) + 128) if (o < O and i < I) else 128)


def test_total_elements(oracle):
    # GetTotalElementsCountForLayout (weights_conversion.cc:1015-1027)
    assert oracle.total_elements(533, 1, 1, 171) == 536 * 172
    assert oracle.total_elements(16, 2, 1, 8, group=2) == 16 * 8 * 2


def test_scale_layout_block(oracle):
    # OHIToHOIO4 in buffer storage == [G][O4] (tensor_desc.cc:266-292, 1852-1860)
    O, G = 6, 3
    s = np.arange(O * G, dtype=np.float32).reshape(O, G) + 1
    lay = oracle.scale_layout(s, f16=False)
    assert lay.shape == (G, 8)
    for g in range(G):
        for o in range(8):
            assert lay[g, o] == (s[o, g] if o < O else 0.0)
    lay16 = oracle.scale_layout(s * 0.1, f16=True)
    assert np.array_equal(lay16.view(np.float16)[:, :O], (s * np.float32(0.1)).astype(np.float16).T)


def test_f16_conversion_matches_ieee(oracle):
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 20000),
        np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5,
                  0.1, 0.2, 0.3, 0.4], np.float32)]).astype(np.float32)
    with np.errstate(over="ignore"):
        ref = x.astype(np.float16).view(np.uint16)
    bits = oracle.f32_to_f16_bits(x)
    assert np.array_equal(bits, ref)
    # weights_conversion_test.cc:43-49 (ConvertF32F16 BaseTest)
    assert np.array_equal(oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(np.float32([0.1, 0.2, 0.3, 0.4]))),
                          np.float32([0.1, 0.2, 0.3, 0.4]).astype(np.float16).astype(np.float32))
