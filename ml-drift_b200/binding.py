"""ctypes binding of libmldfc.so.  torch is used only for device memory and
streams; every computation goes through the C ABI."""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmldfc.so")

OK, INVALID_ARGUMENT, UNIMPLEMENTED, CUDA_ERROR, NCCL_ERROR, TIMEOUT, OUT_OF_RANGE = range(7)
F32, F16, F32F16 = 0, 1, 2
SCALE_SCALAR, SCALE_PER_CHANNEL, SCALE_BLOCK = 0, 1, 2
LAYOUT_SLICED, LAYOUT_ROW_MAJOR = 0, 1
SRC_INT8, SRC_UINT4_PACKED = 0, 1
PATH_AUTO, PATH_GEMV, PATH_GEMM = 0, 1, 2
(ROUTE_NONE, ROUTE_DECODE_STREAMING, ROUTE_DECODE_GENERAL, ROUTE_PREFILL_INLINE, ROUTE_PREFILL_CONVERTED,
 ROUTE_PREFILL_CACHED) = range(6)
DECODER_AUTO, DECODER_OP_CHAIN, DECODER_SINGLE_KERNEL = 0, 1, 2
HANDOVER_TAGGED, HANDOVER_BARRIERS = 0, 1
EPILOGUE_NONE, EPILOGUE_SWIGLU_PAIRS = 0, 1


class MldError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        msg = lib().mld_last_error().decode()
        super().__init__(f"{where}: {lib().mld_status_string(status).decode()} ({msg})")


class PackDesc(C.Structure):
    _fields_ = [("o", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("i", C.c_int32),
                ("bits", C.c_int32), ("out_group_size", C.c_int32), ("source", C.c_int32),
                ("swap_dims", C.c_int32), ("pad_value", C.c_uint32)]


class FcDesc(C.Structure):
    _fields_ = [("n", C.c_int32), ("k", C.c_int32), ("weight_bits", C.c_int32),
                ("scale_mode", C.c_int32), ("groups", C.c_int32), ("scalar_scale", C.c_float),
                ("scalar_zero_point", C.c_float), ("has_zero_point", C.c_int32),
                ("has_bias", C.c_int32), ("precision", C.c_int32), ("src_layout", C.c_int32),
                ("dst_layout", C.c_int32), ("max_tokens", C.c_int32), ("force_path", C.c_int32),
                ("device", C.c_int32), ("prefill_act_quant", C.c_int32), ("cache_prepared_weights", C.c_int32),
                ("epilogue", C.c_int32), ("prefill_route", C.c_int32), ("runtime_channel_bounds", C.c_int32),
                ("has_batch_ids", C.c_int32), ("exact_operands", C.c_int32), ("no_overlap", C.c_int32),
                ("smem_limit_kb", C.c_int32), ("independent_io", C.c_int32)]


class DecoderDesc(C.Structure):
    _fields_ = [("layers", C.c_int32), ("d_model", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
                ("ffn", C.c_int32), ("max_seq", C.c_int32), ("block", C.c_int32), ("rms_eps", C.c_float),
                ("rope_min_timescale", C.c_float), ("rope_max_timescale", C.c_float), ("rank", C.c_int32),
                ("world", C.c_int32), ("device", C.c_int32), ("shard_layout", C.c_int32), ("mode", C.c_int32),
                ("handover", C.c_int32), ("grid_limit", C.c_int32), ("ring_stages", C.c_int32),
                ("wait_limit_us", C.c_int32)]


class LayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wqkv", "sqkv", "wo", "so", "wgu", "sgu", "wdown", "sdown",
                                          "norm1", "norm2", "kcache", "vcache")]


_lib = None


def lib() -> C.CDLL:
    """Loads the CUDA library; there is no fallback when it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python ml-drift_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        L.mld_status_string.restype = C.c_char_p
        L.mld_last_error.restype = C.c_char_p
        L.mld_kernel_launch_count.restype = C.c_int64
        L.mld_packed_size_bytes.restype = C.c_size_t
        L.mld_fc_plan_workspace_bytes.restype = C.c_size_t
        L.mld_decoder_scratch_bytes.restype = C.c_size_t
        _lib = L
    return _lib


def _check(rc, where):
    if rc != OK:
        raise MldError(rc, where)


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream(stream=None):
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


def kernel_launch_count() -> int:
    return int(lib().mld_kernel_launch_count())


def div_up(a, b):
    return (a + b - 1) // b


# ------------------------------------------------------------ weight conversion
def packed_size_bytes(o, i, bits, h=1, w=1, group=0) -> int:
    d = PackDesc(o, h, w, i, bits, group, SRC_INT8, 0, 128 if bits == 8 else 8)
    return int(lib().mld_packed_size_bytes(C.byref(d)))


def pack_weights(src: torch.Tensor, shape, bits, source=SRC_INT8, group=0, swap_dims=False,
                 pad_value=None, want_sum=False, sum_len=None, sum_init=None, stream=None):
    """src: device int8 OHWI tensor (SRC_INT8) or dense nibble bytes (SRC_UINT4_PACKED).
    Returns (packed uint8 tensor, sum_i int32 tensor or None)."""
    o, h, w, i = shape
    if pad_value is None:
        pad_value = 128 if bits == 8 else 8
    d = PackDesc(o, h, w, i, bits, group, source, int(swap_dims), pad_value)
    nbytes = int(lib().mld_packed_size_bytes(C.byref(d)))
    dst = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=src.device)[:nbytes]
    sums = None
    n_sum = 0
    if want_sum:
        n_sum = o if sum_len is None else sum_len
        sums = torch.zeros(n_sum, dtype=torch.int32, device=src.device)
        if sum_init is not None:
            sums.copy_(torch.as_tensor(sum_init, dtype=torch.int32))
    _check(lib().mld_pack_weights(C.byref(d), _ptr(src), _ptr(dst), _ptr(sums), n_sum, _stream(stream)),
           "mld_pack_weights")
    return dst, sums


def weights_sum_i(q: torch.Tensor, stream=None):
    o = q.shape[0]
    hwi = q.numel() // max(o, 1)
    out = torch.empty(o, dtype=torch.int32, device=q.device)
    _check(lib().mld_weights_sum_i(_ptr(q), o, hwi, _ptr(out), _stream(stream)), "mld_weights_sum_i")
    return out


def pack_scales(scale: torch.Tensor, f16: bool, stream=None):
    """[O] or [O][G] fp32 device tensor -> [G][O4] in fp16 or fp32."""
    s = scale.reshape(scale.shape[0], -1).contiguous()
    o, g = s.shape
    o4 = div_up(o, 4) * 4
    dst = torch.empty((g, o4), dtype=torch.float16 if f16 else torch.float32, device=s.device)
    _check(lib().mld_pack_scales(_ptr(s), o, g, int(f16), _ptr(dst), _stream(stream)), "mld_pack_scales")
    return dst


def quantize_weights(w: torch.Tensor, bits: int, block: int = 0, optimize_scale: bool = False, stream=None):
    o, i = w.shape
    g = i // block if (bits == 4 and block > 0) else 1
    q = torch.empty((o, i), dtype=torch.int8, device=w.device)
    s = torch.empty((o, g), dtype=torch.float32, device=w.device)
    _check(lib().mld_quantize_weights(_ptr(w), o, i, bits, block, int(optimize_scale), _ptr(q), _ptr(s), _stream(stream)),
           "mld_quantize_weights")
    return q, s


# --------------------------------------------------------------------- operator
def is_gemv_recommended(precision, tokens) -> bool:
    return bool(lib().mld_fc_is_gemv_recommended(precision, tokens))


class FullyConnectedPlan:
    """Owns one mld_fc_plan (the operator object of the C ABI)."""

    def __init__(self, n, k, weight_bits, scale_mode=SCALE_PER_CHANNEL, groups=1, scalar_scale=0.0,
                 scalar_zero_point=0.0, has_zero_point=False, has_bias=False, precision=F32F16,
                 src_layout=LAYOUT_SLICED, dst_layout=LAYOUT_SLICED, max_tokens=1, force_path=PATH_AUTO,
                 device=-1, prefill_act_quant=0, cache_prepared_weights=False, epilogue=0, exact_operands=False,
                 no_overlap=False, smem_limit_kb=0, prefill_route=0, independent_io=False, runtime_channel_bounds=False,
                 has_batch_ids=False):
        self.desc = FcDesc(n, k, weight_bits, scale_mode, groups, scalar_scale, scalar_zero_point,
                           int(has_zero_point), int(has_bias), precision, src_layout, dst_layout,
                           max_tokens, force_path, device, prefill_act_quant, int(cache_prepared_weights), epilogue,
                           prefill_route, int(runtime_channel_bounds), int(has_batch_ids), int(exact_operands),
                           int(no_overlap), smem_limit_kb, int(independent_io))
        self._h = C.c_void_p()
        _check(lib().mld_fc_plan_create(C.byref(self.desc), C.byref(self._h)), "mld_fc_plan_create")

    def set_weights_sum(self, sum_i):
        """sum_i: device int32 tensor [n] (kept alive here)."""
        self._w_sum = sum_i
        _check(lib().mld_fc_plan_set_weights_sum(self._h, _ptr(sum_i)), "mld_fc_plan_set_weights_sum")

    def last_route(self) -> int:
        """ROUTE_* of the most recent run."""
        return int(lib().mld_fc_plan_last_route(self._h))

    def workspace_bytes(self) -> int:
        return int(lib().mld_fc_plan_workspace_bytes(self._h))

    def device_status(self) -> int:
        """0, or the code of a bounded device-side wait that gave up (then cleared)."""
        code = C.c_int32(0)
        rc = lib().mld_fc_plan_device_status(self._h, C.byref(code))
        if rc not in (OK, TIMEOUT):
            raise MldError(rc, "mld_fc_plan_device_status")
        return code.value

    def run(self, src, weights, scale, dst, tokens, zero_point=None, bias=None, stream=None):
        _check(lib().mld_fc_run(self._h, _ptr(src), _ptr(weights), _ptr(scale), _ptr(zero_point), _ptr(bias),
                                _ptr(dst), tokens, _stream(stream)), "mld_fc_run")

    def close(self):
        if self._h:
            lib().mld_fc_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class EmbedDesc(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("dim", C.c_int32), ("weight_bits", C.c_int32), ("scale_mode", C.c_int32),
                ("groups", C.c_int32), ("has_zero_point", C.c_int32), ("f16", C.c_int32), ("dst_layout", C.c_int32)]


def embedding_lookup(ids, weights, scale, dst, vocab, dim, bits, scale_mode=SCALE_PER_CHANNEL, groups=1,
                     zero_point=None, f16=True, dst_layout=LAYOUT_ROW_MAJOR, stream=None):
    """ids: int32 device tensor [tokens]; weights / scale: the packed table as for the FullyConnected operator."""
    d = EmbedDesc(vocab, dim, bits, scale_mode, groups, int(zero_point is not None), int(f16), dst_layout)
    _check(lib().mld_embedding_lookup(C.byref(d), _ptr(ids), _ptr(weights), _ptr(scale), _ptr(zero_point), _ptr(dst),
                                      ids.numel(), _stream(stream)), "mld_embedding_lookup")


# ------------------------------------------------------------------ weight files
NOT_FOUND = 7


class FileTensorLoader:
    """Owns one mld_loader: the LlmFileTensorLoader surface over a directory of converted weight files."""

    def __init__(self, weights_directory: str):
        self._h = C.c_void_p()
        _check(lib().mld_loader_open(weights_directory.encode(), C.byref(self._h)), "mld_loader_open")

    def has_tensor(self, name: str) -> bool:
        return bool(lib().mld_loader_has_tensor(self._h, name.encode()))

    def element_bits(self, name: str, count: int) -> int:
        return int(lib().mld_loader_element_bits(self._h, name.encode(), C.c_int64(count)))

    def group_size(self, weights_name: str, o: int, i: int) -> int:
        return int(lib().mld_loader_group_size(self._h, weights_name.encode(), o, i))

    def load_float32(self, name: str, count: int) -> torch.Tensor:
        out = torch.empty(count, dtype=torch.float32)
        _check(lib().mld_loader_load_float32(self._h, name.encode(), C.c_int64(count), C.c_void_p(out.data_ptr())),
               "mld_loader_load_float32")
        return out

    def load_weights(self, name: str, bits: int, o: int, i: int, swap_dims=False, device="cuda", stream=None):
        """Returns (packed uint8 device tensor, weights_sum_i int32 device tensor)."""
        d = PackDesc(o, 1, 1, i, bits, 0, SRC_UINT4_PACKED if bits == 4 else SRC_INT8, 0, 8 if bits == 4 else 128)
        nbytes = int(lib().mld_packed_size_bytes(C.byref(d)))
        dst = torch.empty(nbytes, dtype=torch.uint8, device=device)
        sums = torch.zeros(o, dtype=torch.int32, device=device)
        _check(lib().mld_loader_load_weights(self._h, name.encode(), bits, o, i, int(swap_dims), _ptr(dst), _ptr(sums), o,
                                             _stream(stream)), "mld_loader_load_weights")
        return dst, sums

    def load_scale(self, name: str, o: int, g: int, f16=True, device="cuda", stream=None) -> torch.Tensor:
        o4 = (o + 3) // 4 * 4
        dst = torch.empty(g * o4, dtype=torch.float16 if f16 else torch.float32, device=device)
        _check(lib().mld_loader_load_scale(self._h, name.encode(), o, g, int(f16), _ptr(dst), _stream(stream)),
               "mld_loader_load_scale")
        return dst

    def load_zero_point(self, zero_point_name: str, scale_name: str, o: int, g: int, f16=True, device="cuda",
                        stream=None) -> torch.Tensor:
        o4 = (o + 3) // 4 * 4
        dst = torch.empty(g * o4, dtype=torch.float16 if f16 else torch.float32, device=device)
        _check(lib().mld_loader_load_zero_point(self._h, zero_point_name.encode(), scale_name.encode(), o, g, int(f16),
                                                _ptr(dst), _stream(stream)), "mld_loader_load_zero_point")
        return dst

    def close(self):
        if self._h:
            lib().mld_loader_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


# ------------------------------------------------------- operator split over GPUs
GATHER_NCCL, GATHER_PEER_STORES = 0, 1


class ShardGroup:
    """Owns one mld_shard_group: this rank's copy of a gathered output tensor."""

    def __init__(self, rank, world, output_bytes, nccl_id=None, device=-1):
        self._h = C.c_void_p()
        idbuf = None if nccl_id is None else C.create_string_buffer(nccl_id, 128)
        _check(lib().mld_shard_group_create(rank, world, device, C.c_size_t(output_bytes), idbuf, C.byref(self._h)),
               "mld_shard_group_create")
        self.output_bytes = output_bytes

    def ipc_export(self) -> bytes:
        buf = C.create_string_buffer(64)
        _check(lib().mld_shard_group_ipc_export(self._h, buf), "mld_shard_group_ipc_export")
        return buf.raw

    def ipc_import(self, handles: bytes):
        _check(lib().mld_shard_group_ipc_import(self._h, C.create_string_buffer(handles, len(handles))),
               "mld_shard_group_ipc_import")

    def output(self, elems, device):
        """The gathered tensor as a flat fp16 torch tensor of `elems` elements (a view of library memory)."""
        lib().mld_shard_group_output.restype = C.c_void_p
        ptr = lib().mld_shard_group_output(self._h)
        assert elems * 2 <= self.output_bytes

        class _Mem:
            __cuda_array_interface__ = {"shape": (elems,), "typestr": "<f2", "data": (ptr, False), "version": 2}
        keep = self
        t = torch.as_tensor(_Mem(), device=device)
        t._mld_keep = keep
        return t

    def run(self, plan, src, weights, scale, tokens, gather, zero_point=None, bias=None, stream=None):
        _check(lib().mld_fc_run_sharded(plan._h, self._h, _ptr(src), _ptr(weights), _ptr(scale), _ptr(zero_point),
                                        _ptr(bias), tokens, gather, _stream(stream)), "mld_fc_run_sharded")

    def device_status(self) -> int:
        code = C.c_int32(0)
        rc = lib().mld_shard_group_device_status(self._h, C.byref(code))
        if rc not in (OK, TIMEOUT):
            raise MldError(rc, "mld_shard_group_device_status")
        return code.value

    def close(self):
        if self._h:
            lib().mld_shard_group_destroy(self._h)
            self._h = C.c_void_p()


# ---------------------------------------------------------------- decode step
def attn_decode_static(q, kcache, vcache, out, heads, n_tokens, head_dim=128, stream=None):
    """Decode attention without any device allocation (fixed scratch array inside the library)."""
    _check(lib().mld_attn_decode_static(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(out), heads, head_dim, n_tokens,
                                        _stream(stream)), "mld_attn_decode_static")


def attn_decode(q, kcache, vcache, out, heads, n_tokens, head_dim=128, stream=None):
    _check(lib().mld_attn_decode(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(out), heads, head_dim, n_tokens,
                                 _stream(stream)), "mld_attn_decode")


def comm_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    _check(lib().mld_comm_unique_id(buf), "mld_comm_unique_id")
    return buf.raw


class Decoder:
    """Owns one mld_decoder: a stack of decoder layers whose projections are INT4
    FullyConnected nodes.  Layer tensors are torch tensors kept alive here."""

    def __init__(self, layers, d_model, heads, ffn, max_seq, block=32, head_dim=128, rms_eps=1e-6,
                 rope_min_timescale=1.0, rope_max_timescale=1.0e6, rank=0, world=1, nccl_id=None, device=-1,
                 shard_layout=0, mode=DECODER_AUTO, handover=HANDOVER_TAGGED, grid_limit=0, ring_stages=0,
                 wait_limit_us=0):
        self.desc = DecoderDesc(layers, d_model, heads, head_dim, ffn, max_seq, block, rms_eps,
                                rope_min_timescale, rope_max_timescale, rank, world, device, shard_layout, mode,
                                handover, grid_limit, ring_stages, wait_limit_us)
        self._h = C.c_void_p()
        self._keep = []
        idbuf = None if nccl_id is None else C.create_string_buffer(nccl_id, 128)
        _check(lib().mld_decoder_create(C.byref(self.desc), idbuf, C.byref(self._h)), "mld_decoder_create")

    def set_layer(self, layer, **tensors):
        lw = LayerWeights(*[tensors[n].data_ptr() for n, _ in LayerWeights._fields_])
        self._keep.append(tensors)
        _check(lib().mld_decoder_set_layer(self._h, layer, C.byref(lw)), "mld_decoder_set_layer")

    @property
    def single_kernel(self) -> bool:
        return bool(lib().mld_decoder_is_single_kernel(self._h))

    def device_status(self) -> int:
        """0, or the code of the bounded device-side wait that gave up (then cleared)."""
        code = C.c_int32(0)
        rc = lib().mld_decoder_device_status(self._h, C.byref(code))
        if rc not in (OK, TIMEOUT):
            raise MldError(rc, "mld_decoder_device_status")
        return code.value

    def reset(self):
        _check(lib().mld_decoder_reset(self._h), "mld_decoder_reset")

    def set_wait_limit(self, wait_limit_us: int):
        _check(lib().mld_decoder_set_wait_limit(self._h, int(wait_limit_us)), "mld_decoder_set_wait_limit")

    def ipc_export(self) -> bytes:
        buf = C.create_string_buffer(64)
        _check(lib().mld_decoder_ipc_export(self._h, buf), "mld_decoder_ipc_export")
        return buf.raw

    def ipc_import(self, handles: bytes):
        """handles: the 64-byte exports of all ranks, concatenated in rank order."""
        _check(lib().mld_decoder_ipc_import(self._h, C.create_string_buffer(handles, len(handles))),
               "mld_decoder_ipc_import")

    def step(self, x_in, x_out, pos, stream=None):
        _check(lib().mld_decoder_step(self._h, _ptr(x_in), _ptr(x_out), pos, _stream(stream)), "mld_decoder_step")

    def step_host(self, x_host, y_host, pos, stream=None):
        """x_host / y_host: pinned CPU fp16 tensors; includes both copies and a stream sync."""
        _check(lib().mld_decoder_step_host(self._h, _ptr(x_host), _ptr(y_host), pos, _stream(stream)),
               "mld_decoder_step_host")

    def scratch_bytes(self):
        return int(lib().mld_decoder_scratch_bytes(self._h))

    def close(self):
        if self._h:
            lib().mld_decoder_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
