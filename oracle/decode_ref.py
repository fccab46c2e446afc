"""CPU restatement of one decode step of the Llama-style decoder used by the
benchmark (TEST INFRASTRUCTURE ONLY).  The projections go through the FC oracle
(`oracle.fc_forward`, kF32F16 arithmetic over the packed reference layout); the
glue follows ml_drift/samples/llm/qwen3_model_builder.cc:890-1038 (RMSNorm with
epsilon 1e-6, SiLU*mul FFN, attention with 1/sqrt(head_dim) scaling, residual
links) and ml_drift/common/kernels/rope.cc:70-89 (split-half rotary embedding,
timescale = min * (max/min)^(2i/d)).  fp16 tensors between nodes, fp32 inside.

Pinned by tests/test_oracle_decode.py against the known answers the reference's own kernel tests hold:
rope against common/kernels/tests/rope_test_util.cc:40-165, softmax against softmax_test_util.cc:272-290,
360-395, 497-515, 540-575, rmsnorm against RMSNormalizationReference (common/task/testing_ref_ops.cc:
2537-2544) on the shape of mean_stddev_normalization_test_util.cc:410-420."""
import numpy as np

from . import oracle as orc


def _h(x):
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def rmsnorm(x, gamma, eps=1e-6):
    inv = 1.0 / np.sqrt(np.mean(x.astype(np.float32) ** 2) + eps)
    return _h(x * np.float32(inv) * gamma)


def rope(v, pos, min_ts=1.0, max_ts=1.0e6):
    d = v.shape[-1]
    half = d // 2
    i = np.arange(half, dtype=np.float32)
    timescale = np.float32(min_ts) * np.power(np.float32(max_ts / min_ts), 2.0 * i / d).astype(np.float32)
    ang = np.float32(pos) / timescale
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    v0, v1 = v[..., :half], v[..., half:]
    return np.concatenate([v0 * c - v1 * s, v1 * c + v0 * s], axis=-1)


def softmax(s):
    """Softmax over the last axis the way the reference's Softmax kernels compute it
    (ml_drift/common/kernels/softmax1x1.cc / softmax.cc: subtract the row maximum, exp, divide by the
    sum), fp32."""
    s = np.asarray(s, np.float32)
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    return (p / p.sum(axis=-1, keepdims=True)).astype(np.float32)


def silu_mul(g, u):
    """SiLU(gate) * up of the FFN (samples/llm/qwen3_model_builder.cc:918-932)."""
    return g / (1.0 + np.exp(-g)) * u


def fc(x, layer, name, N, K, block):
    q = layer[name]
    y = orc.fc_forward(orc.F32F16, 4, _h(x)[None], q["packed"], N=N, K=K, scale=q["scale"],
                       scale_mode=orc.SCALE_BLOCK, G=K // block)
    return y[0]


def decode_step(x, layers, kcache, vcache, pos, heads, head_dim, ffn, block=32, eps=1e-6, interleaved_gate_up=False):
    """x: [d] fp16-representable float32.  layers[l]: dict with 'qkv','o','gu','down' (each
    {'packed','scale'} from the FC oracle's quantiser/packer) and 'norm1','norm2'.
    kcache/vcache: [L][T][heads*head_dim] float32 arrays (fp16-representable), updated in place.
    interleaved_gate_up: the rows of 'gu' alternate gate_i, up_i (the order the device matrix uses)
    instead of [all gates ; all ups]."""
    d = heads * head_dim
    x = _h(x)
    resid = None
    for l, layer in enumerate(layers):
        if resid is not None:
            x = _h(x + resid)
        xn = rmsnorm(x, layer["norm1"], eps)
        qkv = fc(xn, layer, "qkv", 3 * d, d, block)
        q = qkv[:d].reshape(heads, head_dim)
        k = qkv[d:2 * d].reshape(heads, head_dim)
        v = qkv[2 * d:]
        q = _h(rope(q, pos) * np.float32(1.0 / np.sqrt(head_dim)))
        kcache[l][pos] = _h(rope(k, pos)).reshape(-1)
        vcache[l][pos] = v
        T = pos + 1
        kc = kcache[l][:T].reshape(T, heads, head_dim)
        vc = vcache[l][:T].reshape(T, heads, head_dim)
        p = softmax(np.einsum("hd,thd->ht", q, kc).astype(np.float32))
        attn = _h(np.einsum("ht,thd->hd", p, vc).reshape(-1))
        o = fc(attn, layer, "o", d, d, block)
        h = _h(x + o)
        hn = rmsnorm(h, layer["norm2"], eps)
        gu = fc(hn, layer, "gu", 2 * ffn, d, block)
        g, u = (gu[0::2], gu[1::2]) if interleaved_gate_up else (gu[:ffn], gu[ffn:])
        act = _h(silu_mul(g, u))
        resid = fc(act, layer, "down", d, ffn, block)
        x = h
    return _h(x + resid)
