"""The quantiser oracle reproduces, bit for bit, vectors produced by the
reference's own Python quantiser (tests/golden/make_quantiser_vectors.py ran
ml_drift/samples/llm/extract_weights_hf.py:137-241 with optimize_scale=False)."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantiser_vectors.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_int8_per_channel(oracle, gold, name):
    q, s = oracle.quantize_int8_sym(gold[f"{name}_w"])
    assert np.array_equal(q, gold[f"{name}_q8"])
    assert np.array_equal(s.view(np.uint32), gold[f"{name}_s8"].view(np.uint32))


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_int4_per_channel(oracle, gold, name):
    q, s = oracle.quantize_int4_sym(gold[f"{name}_w"], block=0)
    assert np.array_equal(q, gold[f"{name}_q4c"])
    assert np.array_equal(s.reshape(-1).view(np.uint32), gold[f"{name}_s4c"].reshape(-1).view(np.uint32))


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_int4_block32_and_dense_pack(oracle, gold, name):
    q, s = oracle.quantize_int4_sym(gold[f"{name}_w"], block=32)
    assert np.array_equal(q, gold[f"{name}_q4b"])
    assert np.array_equal(s.view(np.uint32), gold[f"{name}_s4b"].view(np.uint32))
    assert np.array_equal(oracle.pack_int4_dense(q), gold[f"{name}_p4b"])


def test_round_half_to_even(oracle, gold):
    q, s = oracle.quantize_int4_sym(gold["tie_w"], block=32)
    assert np.array_equal(q, gold["tie_q4b"])
    assert q[0, :8].tolist() == [7, 0, 2, 2, 0, -2, -2, 4]


def test_block_size_must_divide(oracle):
    with pytest.raises(ValueError):
        oracle.quantize_int4_sym(np.zeros((2, 48), np.float32), block=32)
