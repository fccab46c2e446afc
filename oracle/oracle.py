"""ctypes/numpy front end of the CPU oracle (``mld_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, by the smoke check and by the
CPU-baseline leg of the benchmark.  The shipped library never touches it.

Each wrapper takes and returns numpy arrays; the C function it calls cites the
ml-drift source lines it restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmld_oracle.so")

F32, F16, F32F16 = 0, 1, 2
SCALE_SCALAR, SCALE_CHANNEL, SCALE_BLOCK = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "mld_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libmld_oracle.so"])
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_total_elements_i4o4.restype = C.c_int64
        _lib.orc_scale_layout.restype = C.c_int64
    return _lib


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def div_up(a, b):
    return (a + b - 1) // b


# --------------------------------------------------------------------- fp16
def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_f16(_p(x), _p(out), C.c_int64(x.size))
    return out


def f16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().orc_f16_to_f32(_p(h), _p(out), C.c_int64(h.size))
    return out


# --------------------------------------------------------------- quantisers
def quantize_int8_sym(w: np.ndarray):
    w = _c(w, np.float32)
    O, I = w.shape
    q = np.empty((O, I), np.int8)
    s = np.empty((O,), np.float32)
    lib().orc_quantize_int8_sym(_p(w), O, I, _p(q), _p(s))
    return q, s


def quantize_int4_sym(w: np.ndarray, block: int = 0):
    w = _c(w, np.float32)
    O, I = w.shape
    G = I // block if block > 0 else 1
    q = np.empty((O, I), np.int8)
    s = np.empty((O, G), np.float32)
    rc = lib().orc_quantize_int4_sym(_p(w), O, I, block, _p(q), _p(s))
    if rc != 0:
        raise ValueError("input channels not divisible by block size")
    return q, s


def pack_int4_dense(q: np.ndarray) -> np.ndarray:
    q = _c(q, np.int8)
    out = np.empty((q.size // 2,), np.uint8)
    if lib().orc_pack_int4_dense(_p(q), C.c_int64(q.size), _p(out)) != 0:
        raise ValueError("odd element count")
    return out


# ------------------------------------------------------------------ packers
def total_elements(O, H, W, I, group=None) -> int:
    group = div_up(O, 4) if group is None else group
    return int(lib().orc_total_elements_i4o4(O, H, W, I, group))


def rearrange_int8_as_uint8(q: np.ndarray, group=None, shift=128, pad=128):
    q = _c(q, np.int8)
    if q.ndim == 2:
        q = q.reshape(q.shape[0], 1, 1, q.shape[1])
    O, H, W, I = q.shape
    group = div_up(O, 4) if group is None else group
    dst = np.empty((total_elements(O, H, W, I, group),), np.uint8)
    lib().orc_rearrange_int8_as_uint8(_p(q), O, H, W, I, group, shift, pad, _p(dst))
    return dst


def rearrange_int8_as_uint4(q: np.ndarray, group=None, shift=8, pad=8):
    q = _c(q, np.int8)
    if q.ndim == 2:
        q = q.reshape(q.shape[0], 1, 1, q.shape[1])
    O, H, W, I = q.shape
    group = div_up(O, 4) if group is None else group
    dst = np.empty((total_elements(O, H, W, I, group) // 2,), np.uint8)
    lib().orc_rearrange_int8_as_uint4(_p(q), O, H, W, I, group, shift, pad, _p(dst))
    return dst


def rearrange_uint4_packed(src: np.ndarray, shape, group=None, pad=8,
                           swap_dims=False, sum_len=None, sum_init=None):
    src = _c(src, np.uint8)
    O, H, W, I = shape
    group = div_up(O, 4) if group is None else group
    dst = np.empty((total_elements(O, H, W, I, group) // 2,), np.uint8)
    sum_len = O if sum_len is None else sum_len
    sums = np.zeros((sum_len,), np.int32) if sum_init is None else _c(sum_init, np.int32).copy()
    lib().orc_rearrange_uint4_packed(_p(src), O, H, W, I, group, _p(dst), _p(sums),
                                     sum_len, pad, int(swap_dims))
    return dst, sums


def weights_sum_i(q: np.ndarray) -> np.ndarray:
    q = _c(q, np.int8)
    if q.ndim == 2:
        q = q.reshape(q.shape[0], 1, 1, q.shape[1])
    O, H, W, I = q.shape
    out = np.empty((O,), np.int32)
    lib().orc_weights_sum_i(_p(q), O, H, W, I, _p(out))
    return out


def scale_layout(scale: np.ndarray, f16: bool) -> np.ndarray:
    """[O] or [O][G] float scales -> device layout ([O4] or [G][O4]); fp16 bits or fp32."""
    scale = _c(scale, np.float32)
    if scale.ndim == 1:
        scale = scale.reshape(-1, 1)
    O, G = scale.shape
    O4 = div_up(O, 4) * 4
    dst = np.empty((G, O4), np.uint16 if f16 else np.float32)
    lib().orc_scale_layout(_p(scale), O, G, int(f16), _p(dst))
    return dst


def to_sliced(x: np.ndarray) -> np.ndarray:
    """[M][C] float32 -> [ceil(C/4)][M][4] float32 (zero padded)."""
    x = _c(x, np.float32)
    M, Cc = x.shape
    out = np.empty((div_up(Cc, 4), M, 4), np.float32)
    lib().orc_rowmajor_to_sliced_f32(_p(x), M, Cc, _p(out))
    return out


def from_sliced(x: np.ndarray, Cc: int) -> np.ndarray:
    x = _c(x, np.float32)
    S, M, _ = x.shape
    out = np.empty((M, Cc), np.float32)
    lib().orc_sliced_to_rowmajor_f32(_p(x), M, Cc, _p(out))
    return out


# ------------------------------------------------------------------ forward
def fc_forward(precision, bits, x, packed, N, K, scale=None, zp=None, bias=None,
               scale_mode=SCALE_CHANNEL, G=1, scalar_scale=0.0, scalar_zp=None):
    """x: [M][K] float32 logical activations.  scale/zp/bias: logical float32
    ([N], [N][G], [N]).  Converts to the device layouts/types, runs the restated
    kernel, returns [M][N] float32 (the stored type converted back)."""
    x = _c(x, np.float32)
    M = x.shape[0]
    half = precision != F32
    xs = to_sliced(x)
    xs_dev = f32_to_f16_bits(xs) if half else xs
    sc = zpd = bd = None
    if scale_mode != SCALE_SCALAR:
        sc = scale_layout(scale, half)
        if zp is not None:
            zpd = scale_layout(zp, half)
    if bias is not None:
        bd = scale_layout(np.asarray(bias, np.float32).reshape(-1), half)
    S = div_up(N, 4)
    y = np.empty((S, M, 4), np.uint16 if half else np.float32)
    rc = lib().orc_fc_forward(precision, bits, M, K, N, _p(xs_dev), _p(_c(packed, np.uint8)),
                              scale_mode, G, _p(sc), _p(zpd), C.c_float(scalar_scale),
                              C.c_float(0.0 if scalar_zp is None else scalar_zp),
                              int(scalar_zp is not None), _p(bd), _p(y))
    assert rc == 0
    yf = f16_bits_to_f32(y) if half else y
    return from_sliced(yf, N)


def fc_plain_reference(q, scale, x, zp=None, bias=None):
    q = _c(q, np.int8)
    N, K = q.shape
    scale = _c(scale, np.float32).reshape(N, -1)
    G = scale.shape[1]
    x = _c(x, np.float32)
    M = x.shape[0]
    y = np.empty((M, N), np.float32)
    zp = None if zp is None else _c(zp, np.float32).reshape(N, G)
    bias = None if bias is None else _c(bias, np.float32)
    lib().orc_fc_plain_reference(_p(q), N, K, _p(scale), _p(zp), G, _p(bias), _p(x), M, _p(y))
    return y


def quantize_act_sym(x_bits_or_f32: np.ndarray, src_f16: bool):
    x = _c(x_bits_or_f32, np.uint16 if src_f16 else np.float32)
    M, K = x.shape
    q = np.empty((M, K), np.int8)
    params = np.empty((M, 3), np.float32)
    lib().orc_quantize_act_sym(_p(x), int(src_f16), M, K, _p(q), _p(params))
    return q, params


def quantize_act_asym(x_bits_or_f32: np.ndarray, src_f16: bool):
    x = _c(x_bits_or_f32, np.uint16 if src_f16 else np.float32)
    M, K = x.shape
    q = np.empty((M, K), np.int8)
    params = np.empty((M, 3), np.float32)
    lib().orc_quantize_act_asym(_p(x), int(src_f16), M, K, _p(q), _p(params))
    return q, params


def gemm_s8s8_s32(xq, wq):
    xq = _c(xq, np.int8)
    wq = _c(wq, np.int8)
    M, K = xq.shape
    N = wq.shape[0]
    acc = np.empty((M, N), np.int32)
    lib().orc_gemm_s8s8_s32(_p(xq), _p(wq), M, K, N, _p(acc))
    return acc


def fc_forward_i8(bits, xq, packed, N):
    xq = _c(xq, np.int8)
    M, K = xq.shape
    acc = np.zeros((M, N), np.int32)
    lib().orc_fc_forward_i8(bits, M, K, N, _p(xq), _p(_c(packed, np.uint8)), _p(acc))
    return acc


def dequant_epilogue(acc, params, w_scale, w_sum=None, bias_bits_or_f32=None, dst_f16=True):
    acc = _c(acc, np.int32)
    M, N = acc.shape
    y = np.empty((M, N), np.uint16 if dst_f16 else np.float32)
    b = None
    if bias_bits_or_f32 is not None:
        b = _c(bias_bits_or_f32, np.uint16 if dst_f16 else np.float32)
    ws = None if w_sum is None else _c(w_sum, np.int32)
    lib().orc_dequant_epilogue(_p(acc), M, N, _p(_c(params, np.float32)), _p(_c(w_scale, np.float32)),
                               _p(ws), _p(b), int(dst_f16), _p(y))
    return y


def prefill_gemm_int4(x_bits, packed, scale_gn_bits, N, bits=4):
    x_bits = _c(x_bits, np.uint16)
    M, K = x_bits.shape
    scale_gn_bits = _c(scale_gn_bits, np.uint16)
    G = scale_gn_bits.shape[0]
    y = np.empty((M, N), np.uint16)
    lib().orc_prefill_gemm_int4(_p(x_bits), M, K, N, _p(_c(packed, np.uint8)), bits,
                                _p(scale_gn_bits), G, _p(y))
    return y


def gemv_f32_fast(bits, x, packed, N, scale_gn, bias=None):
    x = _c(x, np.float32).reshape(-1)
    K = x.size
    scale_gn = _c(scale_gn, np.float32)
    if scale_gn.ndim == 1:
        scale_gn = scale_gn.reshape(1, -1)
    G = scale_gn.shape[0]
    y = np.empty((div_up(N, 4) * 4,), np.float32)
    lib().orc_gemv_f32_fast(bits, K, N, _p(x), _p(_c(packed, np.uint8)), G, _p(scale_gn),
                            _p(None if bias is None else _c(bias, np.float32)), _p(y))
    return y[:N]


def embedding_lookup(ids, packed, vocab, dim, bits, scale, zp=None):
    """The generated kernel of EmbeddingLookup (ml_drift/common/kernels/embedding_lookup.cc:44-196) over the
    FullyConnected weight layout (O = vocab, I = dim): for token id `index` (clamped to [0, vocab - 1]) and
    input slice S, column index % 4 of block (S, index / 4), dequantised in fp32 as
    value * scale + (-scale * (shift + zero_point)).  scale / zp: [vocab] or [vocab][G] float32 (already
    rounded to the storage type).  Returns float32 [tokens][dim]."""
    ids = np.clip(np.asarray(ids, np.int64), 0, vocab - 1)
    scale = np.asarray(scale, np.float32).reshape(vocab, -1)
    G = scale.shape[1]
    zpa = None if zp is None else np.asarray(zp, np.float32).reshape(vocab, -1)
    S = div_up(dim, 4)
    OS = div_up(vocab, 4)
    blk = 16 if bits == 8 else 8
    pk = np.asarray(packed, np.uint8).reshape(S, OS, blk)
    shift = np.float32(128.0 if bits == 8 else 8.0)
    group_slices = (dim // G) // 4
    out = np.zeros((len(ids), S * 4), np.float32)
    for t, index in enumerate(ids):
        b = pk[:, index // 4, :]                                   # [S][blk]
        sub = int(index % 4)
        if bits == 8:
            vals = b.reshape(S, 4, 4)[:, :, sub].astype(np.float32)   # byte (k % 4) * 4 + sub
        else:
            nib = np.stack([b & 15, b >> 4], axis=-1).reshape(S, 16)  # nibble e = 2 * byte + (high)
            vals = nib.reshape(S, 4, 4)[:, :, sub].astype(np.float32)
        g = np.minimum(np.arange(S) // max(group_slices, 1), G - 1)
        sc = scale[index, g].astype(np.float32)[:, None]
        z = np.float32(0.0) if zpa is None else zpa[index, g].astype(np.float32)[:, None]
        bias = (-sc) * (shift + z)
        out[t] = (vals * sc + bias).astype(np.float32).reshape(-1)
    return out[:, :dim]


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """Thread count of the OpenMP loops (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    lib().orc_set_num_threads(int(n))


def host_cores() -> int:
    """Cores this process may run on."""
    import os
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1
