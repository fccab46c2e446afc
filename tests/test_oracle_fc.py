"""Pins the forward oracle to the hand-computed answers of the reference's
kernel tests (ml_drift/common/kernels/tests/fully_connected_test_util.cc) and to
its plain CPU reference (common/task/testing_ref_ops.cc:961-988) on the ragged
shapes the reference uses."""
import numpy as np
import pytest

PRECISIONS = ["F32", "F16", "F32F16"]


def _prec(oracle, name):
    return getattr(oracle, name)


def _eps(precision, K):
    # testing_util.cc:328-331 with GetEpsilon (common/util.cc:192-203)
    e = 1.1920929e-07 if precision == "F32" else 9.7656e-4
    return e * (K + 1)


@pytest.mark.parametrize("precision", PRECISIONS)
def test_int8_scalar_scale_bias(oracle, precision):
    # fully_connected_test_util.cc:49-103 -> {20.5, 15.5}
    q = np.array([[2, 4, 6, 8], [10, 12, -14, 16]], np.int8)
    packed = oracle.rearrange_int8_as_uint8(q)
    y = oracle.fc_forward(_prec(oracle, precision), 8, np.float32([[0, 1, 2, 3]]), packed, N=2, K=4,
                          bias=np.float32([0.5, -0.5]), scale_mode=oracle.SCALE_SCALAR, scalar_scale=0.5)
    eps = 1e-6 if precision == "F32" else 1e-3
    assert np.allclose(y, [[20.5, 15.5]], atol=eps, rtol=0)


@pytest.mark.parametrize("precision", PRECISIONS)
def test_int8_blockwise(oracle, precision):
    # :105-175 -> {91.0, 26.8}
    q = np.array([[1, 1, 1, 1, 2, 2, 2, 2], [3, 3, 3, 3, 4, 4, 4, 4]], np.int8)
    scale = np.float32([[0.5, 2.0], [1.0, 0.1]])
    packed = oracle.rearrange_int8_as_uint8(q)
    y = oracle.fc_forward(_prec(oracle, precision), 8, np.arange(8, dtype=np.float32)[None], packed, N=2, K=8,
                          scale=scale, bias=np.float32([0, 0]), scale_mode=oracle.SCALE_BLOCK, G=2)
    eps = 1e-5 if precision == "F32" else 0.05
    assert np.allclose(y, [[91.0, 26.8]], atol=eps, rtol=0)


@pytest.mark.parametrize("precision", PRECISIONS)
def test_int8_blockwise_zero_points(oracle, precision):
    # :177-249 -> {509.0, -121.4}
    q = np.array([[1, 2, 3, 4, 5, 6, 7, 8], [-8, -7, -6, -5, -4, -3, -2, -1]], np.int8)
    scale = np.float32([[0.5, 2.0], [1.5, 0.1]])
    zp = np.float32([[2, -3], [1, 4]])
    packed = oracle.rearrange_int8_as_uint8(q)
    y = oracle.fc_forward(_prec(oracle, precision), 8, np.arange(1, 9, dtype=np.float32)[None], packed, N=2, K=8,
                          scale=scale, zp=zp, bias=np.float32([0, 0]), scale_mode=oracle.SCALE_BLOCK, G=2)
    eps = 1e-5 if precision == "F32" else 0.1
    assert np.allclose(y, [[509.0, -121.4]], atol=eps, rtol=0)


@pytest.mark.parametrize("precision", PRECISIONS)
def test_int4_blockwise_all_ones(oracle, precision):
    # :1541-1614 -> 8.0 on every output
    q = np.ones((4, 16), np.int8)
    packed = oracle.rearrange_int8_as_uint4(q)
    y = oracle.fc_forward(_prec(oracle, precision), 4, np.ones((1, 16), np.float32), packed, N=4, K=16,
                          scale=np.full((4, 2), 0.5, np.float32), bias=np.zeros(4, np.float32),
                          scale_mode=oracle.SCALE_BLOCK, G=2)
    eps = 1e-6 if precision == "F32" else 1e-2
    assert np.allclose(y, 8.0, atol=eps, rtol=0)


def _uniform(rng, shape):
    # MakeSyntheticTensor: uniform [-1, 1) (common/task/testing_util.cc:262-266)
    return rng.uniform(-1.0, 1.0, size=shape).astype(np.float32)


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("bits,K,N,G,M,use_zp", [
    (8, 171, 533, 1, 1, False),     # :935-967  FullyConnectedInt8BigTest
    (8, 171, 533, 1, 15, False),    # width-15 variant
    (8, 364, 533, 13, 1, False),    # :969-1001 13 groups, K = 7*13*4
    (4, 171, 533, 1, 1, False),     # :1616-1648 FullyConnectedInt4BigTest
    (4, 364, 533, 13, 1, False),    # :1756-1788
    (4, 364, 533, 7, 1, True),      # :1955-1987 7 groups + zero points
    (4, 171, 533, 1, 4, False),     # :1722-1754 width 4
])
def test_against_plain_reference(oracle, precision, bits, K, N, G, M, use_zp):
    rng = np.random.default_rng(bits * 7919 + K + N + G + M)
    wf = _uniform(rng, (N, K))
    if bits == 8:
        q = (np.clip(((wf + 1.0) * 256.0).astype(np.int32), 0, 255) - 128).astype(np.int8)
        scale = _uniform(rng, (N, G)) / 128.0
        packed = oracle.rearrange_int8_as_uint8(q)
    else:
        q = (np.clip(((wf + 1.0) * 16.0).astype(np.int32), 0, 15) - 8).astype(np.int8)
        scale = _uniform(rng, (N, G)) / 8.0
        packed = oracle.rearrange_int8_as_uint4(q)
    zp = rng.integers(-3, 4, size=(N, G)).astype(np.float32) if use_zp else None
    bias = _uniform(rng, (N,))
    x = _uniform(rng, (M, K))
    mode = oracle.SCALE_BLOCK if G > 1 else oracle.SCALE_CHANNEL
    y = oracle.fc_forward(_prec(oracle, precision), bits, x, packed, N=N, K=K, scale=scale, zp=zp,
                          bias=bias, scale_mode=mode, G=G)
    ref = oracle.fc_plain_reference(q, scale, x, zp=zp, bias=bias)
    assert np.max(np.abs(y - ref)) <= 2.0 * _eps(precision, K)


def test_int8_activation_path_is_exact(oracle):
    # Si8Wi8 / Si8Wi4 (:1416-1486, :1989-2059): sum(x*u) - shift*sum(x) == sum(x*q) in int32
    rng = np.random.default_rng(5)
    for bits, lo, hi in ((8, -128, 128), (4, -8, 8)):
        q = rng.integers(lo, hi, size=(152, 112), dtype=np.int8)
        xq = rng.integers(-127, 128, size=(3, 112), dtype=np.int8)
        packed = oracle.rearrange_int8_as_uint8(q) if bits == 8 else oracle.rearrange_int8_as_uint4(q)
        acc = oracle.fc_forward_i8(bits, xq, packed, N=152)
        assert np.array_equal(acc, oracle.gemm_s8s8_s32(xq, q))
        assert np.array_equal(acc, xq.astype(np.int32) @ q.astype(np.int32).T)


def test_activation_quantiser_symmetric(oracle):
    # quantize_and_dequantize.cc:355-378, 421-441: codes in [-127, 127], round half up, (inv_scale, 0, sum)
    rng = np.random.default_rng(9)
    x = rng.standard_normal((5, 64)).astype(np.float32)
    x[3] = 0.0
    q, params = oracle.quantize_act_sym(x, src_f16=False)
    for m in range(5):
        amax = np.abs(x[m]).max()
        if amax == 0:
            assert params[m].tolist() == [0.0, 0.0, 0.0] and not q[m].any()
            continue
        inv = np.float32(amax) / np.float32(127.0)
        assert params[m, 0] == inv and params[m, 1] == 0.0
        exp = np.clip(np.floor(x[m] * (np.float32(1.0) / inv) + np.float32(128.5)), 0, 255) - 128
        assert np.array_equal(q[m], exp.astype(np.int8))
        assert params[m, 2] == q[m].astype(np.int32).sum()
        assert q[m].min() >= -127 and q[m].max() <= 127


def test_w8a8_chain_close_to_float(oracle):
    rng = np.random.default_rng(11)
    M, K, N = 6, 256, 40
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    xh = oracle.f32_to_f16_bits(x)
    q, s = oracle.quantize_int8_sym(w)
    xq, params = oracle.quantize_act_sym(xh, src_f16=True)
    acc = oracle.gemm_s8s8_s32(xq, q)
    y = oracle.f16_bits_to_f32(oracle.dequant_epilogue(acc, params, s, oracle.weights_sum_i(q)))
    ref = oracle.f16_bits_to_f32(xh) @ w.T
    assert np.max(np.abs(y - ref)) / np.max(np.abs(ref)) < 2e-2


def test_prefill_gemm_matches_gemv_oracle(oracle):
    # the dequant-then-float-GEMM route and the FC kernel route agree within F32F16 tolerance
    rng = np.random.default_rng(13)
    M, K, N = 5, 128, 24
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    q, s = oracle.quantize_int4_sym(w, block=32)
    packed = oracle.rearrange_int8_as_uint4(q)
    x = rng.standard_normal((M, K)).astype(np.float32)
    xh = oracle.f32_to_f16_bits(x)
    y = oracle.f16_bits_to_f32(oracle.prefill_gemm_int4(xh, packed, oracle.scale_layout(s, True), N))
    y2 = oracle.fc_forward(oracle.F32F16, 4, oracle.f16_bits_to_f32(xh), packed, N=N, K=K, scale=s,
                           scale_mode=oracle.SCALE_BLOCK, G=K // 32)
    assert np.max(np.abs(y - y2)) / np.max(np.abs(y2)) < 2e-3


def test_fast_gemv_equals_f32_kernel(oracle):
    rng = np.random.default_rng(17)
    K, N = 256, 72
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((1, K)).astype(np.float32)
    for bits in (4, 8):
        if bits == 4:
            q, s = oracle.quantize_int4_sym(w, block=32)
            packed = oracle.rearrange_int8_as_uint4(q)
            mode, G = oracle.SCALE_BLOCK, K // 32
        else:
            q, s = oracle.quantize_int8_sym(w)
            packed = oracle.rearrange_int8_as_uint8(q)
            mode, G = oracle.SCALE_CHANNEL, 1
        y = oracle.fc_forward(oracle.F32, bits, x, packed, N=N, K=K, scale=s, scale_mode=mode, G=G)
        yf = oracle.gemv_f32_fast(bits, x, packed, N, oracle.scale_layout(s, False))
        assert np.allclose(y[0], yf, rtol=0, atol=1e-6)
