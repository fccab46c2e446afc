"""Pins the CPU restatement of the decode step's glue (oracle/decode_ref.py) to the known answers
held by the reference's own kernel tests.  Values are re-encoded from the cited lines of
ml_drift/common/kernels/tests/."""
import numpy as np

from oracle import decode_ref


def test_rope_known_answers():
    # rope_test_util.cc:40-80 (RoPETest) and :84-120 (SplitRoPEConcatTest): four tokens at positions 1..4,
    # left / right halves of four channels each, default RoPEAttributes (min 1, max 10000, common/operations.h:512-517)
    src_l = np.float32([[0, 1, 2, 3], [4, 5, 6, 7], [-1, -2, -3, -4], [-5, -6, -7, -8]])
    src_r = src_l.copy()
    want_l = np.float32([[0.0, 0.895171, 1.979900, 2.996999], [-5.301777, 3.906986, 5.878808, 6.985986],
                         [1.131112, -1.319633, -2.908664, -3.987982], [-0.515794, -3.189856, -6.714476, -7.967936]])
    want_r = np.float32([[0.0, 1.094838, 2.019900, 3.002999], [1.972603, 5.893680, 6.118792, 7.013986],
                         [0.848872, -2.501714, -3.088637, -4.011982], [7.052231, -7.862876, -7.274326, -8.031936]])
    for token in range(4):
        v = np.concatenate([src_l[token], src_r[token]])
        out = decode_ref.rope(v, token + 1, min_ts=1.0, max_ts=10000.0)
        assert np.allclose(out[:4], want_l[token], atol=5e-6, rtol=0)      # the reference's fp32 epsilon
        assert np.allclose(out[4:], want_r[token], atol=5e-6, rtol=0)
    # batched over heads, as decode_step calls it
    both = decode_ref.rope(np.stack([np.concatenate([src_l[1], src_r[1]])] * 3), 2, 1.0, 10000.0)
    assert np.allclose(both[:, :4], want_l[1], atol=5e-6) and np.allclose(both[:, 4:], want_r[1], atol=5e-6)


def test_softmax_known_answers():
    # softmax_test_util.cc:272-290: rows {log 1, log 2}, {log 3, log 4}
    s = np.log(np.float32([[1, 2], [3, 4]]))
    assert np.allclose(decode_ref.softmax(s), [[1 / 3, 2 / 3], [3 / 7, 4 / 7]], atol=1e-6, rtol=0)
    # :497-515 (Softmax1x1Test): {log 1 .. log 4} -> {0.1, 0.2, 0.3, 0.4}
    assert np.allclose(decode_ref.softmax(np.log(np.float32([1, 2, 3, 4]))), [0.1, 0.2, 0.3, 0.4], atol=1e-6, rtol=0)
    # :360-395 and :540-575 (big-number tests): exp(100) overflows fp32, the result must still be the
    # double-precision quotient
    d = np.float64([1.0, 2.0, 3.0, 100.0])
    want_rows = np.concatenate([np.exp(d[:2]) / np.exp(d[:2]).sum(), np.exp(d[2:]) / np.exp(d[2:]).sum()])
    got = decode_ref.softmax(np.float32([[1.0, 2.0], [3.0, 100.0]])).reshape(-1)
    assert np.isfinite(got).all() and np.allclose(got, want_rows.astype(np.float32), atol=1e-6, rtol=0)
    want_one = (np.exp(d) / np.exp(d).sum()).astype(np.float32)
    assert np.allclose(decode_ref.softmax(np.float32(d)), want_one, atol=1e-6, rtol=0)
    # :318-330: 256 equal logits -> 1 / 256 each
    assert np.allclose(decode_ref.softmax(np.zeros(256, np.float32)), 1.0 / 256.0, atol=1e-6, rtol=0)


def test_rmsnorm_follows_the_reference_definition():
    # RMSNormalizationReference (common/task/testing_ref_ops.cc:2537-2544): x * rsqrt(mean(x^2) + eps), eps 1e-6,
    # checked by the reference on BHWC(1, 15, 13, 17) within GetEpsilon * channels
    # (mean_stddev_normalization_test_util.cc:389-420); a gamma vector multiplies the result
    # (samples/llm/qwen3_model_builder.cc:890-902)
    rng = np.random.default_rng(0)
    x = rng.uniform(-4, 4, size=(15 * 13, 17)).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, size=17).astype(np.float32)
    for row in x[:40]:
        sq = row.astype(np.float64) ** 2
        want = row * (1.0 / np.sqrt(sq.mean() + 1e-6))
        got1 = decode_ref.rmsnorm(row, np.ones(17, np.float32))
        assert np.allclose(got1, want, atol=9.765625e-4 * 17, rtol=0)          # the reference's fp16 bound
        assert np.allclose(got1, want.astype(np.float16).astype(np.float32), atol=2e-3 * np.abs(want).max())
        got2 = decode_ref.rmsnorm(row, gamma)
        assert np.allclose(got2, want * gamma, atol=2e-3 * np.abs(want * gamma).max() + 1e-3)


def test_silu_mul():
    g = np.float32([-3.0, 0.0, 2.0])
    u = np.float32([2.0, 5.0, -1.0])
    want = g / (1 + np.exp(-g.astype(np.float64))) * u
    assert np.allclose(decode_ref.silu_mul(g, u), want, rtol=1e-6)
