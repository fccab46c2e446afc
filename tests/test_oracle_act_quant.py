"""Pins the oracle's per-token activation quantisers to the CPU restatement the reference's own test
compares its kernel with (ml_drift/common/kernels/tests/quantize_and_dequantize_test_util.cc:150-260,
QuantizationInt8Test): offset = min + range / 2, scale = 255 / range, code = clamp((x - offset) * scale,
-128, 127) truncated; the kernel's codes may differ from it by at most 1, its scale and offset by 5e-5
(fp32 source) and its sum by at most the channel count."""
import numpy as np


def _reference_int8(x):
    mn, mx = x.min(), x.max()
    rng = np.float32(mx - mn)
    offset = np.float32(mn + rng / np.float32(2.0))
    scale = np.float32(255.0) / rng
    v = np.clip((x - offset) * scale, -128.0, 127.0)
    return v.astype(np.int8), np.float32(1.0) / scale, offset      # C cast: truncation toward zero


def test_asymmetric_int8_against_the_reference_tests_restatement(oracle):
    rng = np.random.default_rng(0)
    x = rng.uniform(-3.0, 5.0, size=(7, 533)).astype(np.float32)
    q, params = oracle.quantize_act_asym(x, src_f16=False)
    for m in range(x.shape[0]):
        ref_q, ref_inv, ref_off = _reference_int8(x[m])
        assert np.max(np.abs(q[m].astype(np.int32) - ref_q.astype(np.int32))) <= 1
        assert abs(params[m, 0] - ref_inv) <= 5e-5
        # the kernel's offset is min + range * 128 / 255 (the code 0 sits half a step above the middle)
        assert abs(params[m, 1] - ref_off) <= 5e-5 + (x[m].max() - x[m].min()) / 510.0 + 1e-6
        assert abs(params[m, 2] - q[m].astype(np.int64).sum()) == 0
        # x ~ q * inv_scale + offset to half a quantisation step
        back = q[m].astype(np.float32) * params[m, 0] + params[m, 1]
        assert np.max(np.abs(back - x[m])) <= 0.5 * params[m, 0] * 1.001 + 1e-6


def test_asymmetric_int8_constant_token(oracle):
    x = np.full((2, 16), 1.5, np.float32)
    q, params = oracle.quantize_act_asym(x, src_f16=False)
    assert np.all(q == -128) and np.all(params[:, 0] == 0.0) and np.all(params[:, 1] == 1.5)


def test_dequantisation_identity_with_weight_sums(oracle):
    # sum_k x_k w_k = w_scale * (inv_scale * sum q_k wq_k + offset * sum wq_k): the epilogue's two terms
    # (quantize_and_dequantize.cc:867-925) reproduce the float product to quantisation accuracy
    rng = np.random.default_rng(1)
    M, K, N = 5, 256, 12
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    wq, ws = oracle.quantize_int8_sym(w)
    x = (rng.standard_normal((M, K)) + 0.7).astype(np.float32)      # a shifted distribution: offset matters
    q, params = oracle.quantize_act_asym(x, src_f16=False)
    acc = oracle.gemm_s8s8_s32(q, wq)
    y = oracle.dequant_epilogue(acc, params, ws.reshape(-1), oracle.weights_sum_i(wq), dst_f16=False)
    ref = x @ (wq.astype(np.float32) * ws.reshape(-1, 1)).T
    assert np.max(np.abs(y - ref)) / np.max(np.abs(ref)) < 2e-2
    # without the weights_sum term the result is off by the offset's share
    y0 = oracle.dequant_epilogue(acc, params, ws.reshape(-1), None, dst_f16=False)
    assert np.max(np.abs(y0 - ref)) > 5 * np.max(np.abs(y - ref))
