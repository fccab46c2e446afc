"""CUDA weight conversion vs the CPU oracle: byte-for-byte (the reference
compares its GPU converter with its CPU rearranger the same way,
ml_drift/common/kernels/tests/conv_weights_converter_test_util.cc:512-587)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mld():
    import __graft_entry__ as g
    return g.import_package()


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


SHAPES = [(4, 1, 1, 4), (3, 1, 1, 4), (4, 1, 1, 2), (533, 1, 1, 171), (534, 1, 1, 171), (7, 1, 1, 6),
          (256, 1, 1, 512), (16, 2, 1, 8), (130, 3, 1, 36), (2048, 1, 1, 2048),
          # input channels a multiple of 16: the register-transpose kernel; ragged outputs, several tiles, H > 1
          (48, 1, 1, 64), (37, 1, 1, 16), (130, 1, 1, 400), (18, 2, 1, 144), (300, 1, 1, 1024),
          # nibble sources with input channels a multiple of 32 and whole output slices: their own transpose kernel
          (20, 2, 1, 96), (132, 1, 1, 288), (16, 1, 1, 32), (516, 1, 1, 544)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("bits", [8, 4])
def test_pack_from_int8(mld, oracle, shape, bits):
    O, H, W, I = shape
    rng = np.random.default_rng(O * 7 + I)
    lo, hi = (-128, 128) if bits == 8 else (-8, 8)
    q = rng.integers(lo, hi, size=shape, dtype=np.int8)
    for group in (0, 1, 2):
        if group and (O // 4) % group:
            pass
        g = None if group == 0 else group
        ref = oracle.rearrange_int8_as_uint8(q, group=g) if bits == 8 else oracle.rearrange_int8_as_uint4(q, group=g)
        got, sums = mld.pack_weights(_dev(q), shape, bits, group=group, want_sum=True)
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy(), ref), f"group={group}"
        assert np.array_equal(sums.cpu().numpy(), oracle.weights_sum_i(q))


@pytest.mark.parametrize("shape", [s for s in SHAPES if (s[0] * s[1] * s[2] * s[3]) % 2 == 0])
@pytest.mark.parametrize("swap", [False, True])
def test_pack_from_packed_nibbles(mld, oracle, shape, swap):
    O, H, W, I = shape
    rng = np.random.default_rng(O * 11 + I)
    q = rng.integers(-8, 8, size=shape, dtype=np.int8)
    src_order = np.ascontiguousarray(q.transpose(3, 1, 2, 0)) if swap else q   # IHWO when swap_dims
    dense = oracle.pack_int4_dense(src_order)
    for sum_len in (O, ((O + 3) // 4) * 4):
        ref, ref_sum = oracle.rearrange_uint4_packed(dense, shape, pad=8, swap_dims=swap, sum_len=sum_len)
        got, sums = mld.pack_weights(_dev(dense), shape, 4, source=mld.SRC_UINT4_PACKED, swap_dims=swap,
                                     want_sum=True, sum_len=sum_len)
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy(), ref)
        assert np.array_equal(sums.cpu().numpy(), ref_sum)


def test_reference_known_answers(mld, oracle):
    # weights_conversion_test.cc:50-91 and :306-348 through the CUDA kernel
    src = np.array([((2 * i + 1) << 4) | (2 * i) for i in range(8)], np.uint8)
    got, sums = mld.pack_weights(_dev(src), (4, 1, 1, 4), 4, source=mld.SRC_UINT4_PACKED, group=1, want_sum=True,
                                 sum_init=[1, 0, 0, 0])
    nib = np.array([0, 4, 8, 12, 1, 5, 9, 13, 2, 6, 10, 14, 3, 7, 11, 15], np.uint8)
    exp = (nib[0::2] | (nib[1::2] << 4)) ^ 0x88
    assert got.cpu().numpy().tolist() == exp.tolist()
    assert sums.cpu().numpy().tolist() == [6, 22, -26, -10]
    got, sums = mld.pack_weights(_dev(src[:6]), (3, 1, 1, 4), 4, source=mld.SRC_UINT4_PACKED, group=1,
                                 want_sum=True, sum_len=4)
    nib = np.array([0, 4, 8, 0, 1, 5, 9, 0, 2, 6, 10, 0, 3, 7, 11, 0], np.uint8)
    exp = (nib[0::2] | (nib[1::2] << 4)) ^ 0x88
    assert got.cpu().numpy().tolist() == exp.tolist()
    assert sums.cpu().numpy().tolist() == [6, 22, -26, 0]


@pytest.mark.parametrize("O,G", [(6, 3), (533, 13), (16384, 64), (2048, 1)])
@pytest.mark.parametrize("f16", [True, False])
def test_pack_scales(mld, oracle, O, G, f16):
    rng = np.random.default_rng(O + G)
    s = (rng.standard_normal((O, G)) * 0.01).astype(np.float32)
    got = mld.pack_scales(_dev(s), f16).cpu().numpy()
    ref = oracle.scale_layout(s, f16)
    if f16:
        assert np.array_equal(got.view(np.uint16), ref)
    else:
        assert np.array_equal(got, ref)


@pytest.mark.parametrize("O,I", [(8, 64), (37, 96), (256, 2048), (5, 36), (9, 4096), (3, 10), (64, 1000)])
def test_quantiser_bit_exact(mld, oracle, O, I):
    rng = np.random.default_rng(O * I)
    w = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    w[1, :] = 0.0
    q, s = mld.quantize_weights(_dev(w), 8)
    qr, sr = oracle.quantize_int8_sym(w)
    assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy().reshape(-1), sr)
    for block in (32, 0, 8, 64, 128, 12):
        if block and I % block:
            continue
        q, s = mld.quantize_weights(_dev(w), 4, block)
        qr, sr = oracle.quantize_int4_sym(w, block)
        assert np.array_equal(q.cpu().numpy(), qr)
        assert np.array_equal(s.cpu().numpy(), sr)


def test_quantiser_matches_reference_vectors(mld):
    import os
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantiser_vectors.npz"))
    for name in ("a", "b", "c"):
        w = _dev(gold[f"{name}_w"])
        q, s = mld.quantize_weights(w, 4, 32)
        assert np.array_equal(q.cpu().numpy(), gold[f"{name}_q4b"])
        assert np.array_equal(s.cpu().numpy(), gold[f"{name}_s4b"])
        q, s = mld.quantize_weights(w, 8)
        assert np.array_equal(q.cpu().numpy(), gold[f"{name}_q8"])
    q, _ = mld.quantize_weights(_dev(gold["tie_w"]), 4, 32)
    assert np.array_equal(q.cpu().numpy(), gold["tie_q4b"])


def test_full_size_packing_roundtrip(mld):
    # the decode GEMV benchmark size: unpacking the packed bytes on the host recovers every weight
    O, I = 16384, 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randint(-8, 8, (O, I), dtype=torch.int8, device="cuda", generator=g)
    packed, sums = mld.pack_weights(q, (O, 1, 1, I), 4, want_sum=True)
    p = packed.view(I // 4, O // 4, 4, 2)                      # [ks][ds][i][byte]
    lo, hi = (p & 0xF).to(torch.int16) - 8, (p >> 4).to(torch.int16) - 8
    blocks = torch.stack([lo[..., 0], hi[..., 0], lo[..., 1], hi[..., 1]], dim=-1)   # [ks][ds][i][o]
    rec = blocks.permute(1, 3, 0, 2).reshape(O, I)
    assert torch.equal(rec.to(torch.int8), q)
    assert torch.equal(sums, q.to(torch.int32).sum(dim=1).to(torch.int32))
