"""The allocation-free decode attention (mld_attn_decode_static) against the regular entry point.

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  The entry point exists for hosts that cannot let a library allocate device memory (their own
pool owns the GPU, or their memory plan is frozen); it must give the same answer as mld_attn_decode
on back-to-back calls that reuse the one fixed scratch array with different shapes."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mld():
    import __graft_entry__ as g
    return g.import_package()


def _case(rng, heads, n_tokens):
    q = (rng.standard_normal((heads, 128)) / np.sqrt(128)).astype(np.float16)
    k = rng.standard_normal((n_tokens, heads, 128)).astype(np.float16)
    v = rng.standard_normal((n_tokens, heads, 128)).astype(np.float16)
    return [torch.from_numpy(a).cuda() for a in (q, k, v)]


def test_static_scratch_attention_matches_regular_entry_point(mld):
    rng = np.random.default_rng(42)
    # two calls in a row on one stream; the second has a different shape, so it reuses slots the
    # first one filled with other data
    for heads, n_tokens in ((32, 2049), (8, 300)):
        q, k, v = _case(rng, heads, n_tokens)
        ref = torch.empty((heads, 128), dtype=torch.float16, device="cuda")
        got = torch.full((heads, 128), float("nan"), dtype=torch.float16, device="cuda")
        mld.attn_decode(q, k, v, ref, heads, n_tokens)
        mld.attn_decode_static(q, k, v, got, heads, n_tokens)
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        err = (got.float() - ref.float()).abs().max().item()
        assert err <= 2e-3 * max(1.0, ref.float().abs().max().item())


def test_static_scratch_attention_refuses_oversize(mld):
    t = torch.zeros(128, dtype=torch.float16, device="cuda")
    with pytest.raises(mld.MldError) as e:
        mld.attn_decode_static(t, t, t, t, 5000, 1)
    assert e.value.status == mld.OUT_OF_RANGE
    assert "4096" in str(e.value)
