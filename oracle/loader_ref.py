"""Test infrastructure, not product code: a numpy restatement of how the reference reads its weight
files (ml_drift/samples/llm/llm_file_tensor_loader.cc), used only by tests/ as the checker of the
library's loader.

Each function names the lines it follows.  Paths are `directory + name`, as the reference concatenates
them (:145-148)."""
import os

import numpy as np


def file_size(path: str) -> int:
    """GetFileSize (:46-55): 0 when the file cannot be opened."""
    return os.path.getsize(path) if os.path.isfile(path) else 0


def element_bits(directory: str, name: str, count: int) -> int:
    """GetTensorElementSizeInBits (:511-522)."""
    if count <= 0:
        return 0
    return file_size(directory + name) * 8 // count


def group_size(directory: str, weights_name: str, o: int, i: int) -> int:
    """GetQuantizationIGroupSize (:399-452)."""
    base = weights_name[:weights_name.rfind(".")]
    path = directory + base + ".weight_quantized_scale"
    size = file_size(path)
    if size < 4:
        return i
    if size % 4 == 0:
        n = size // 4
        if n > 0 and n % o == 0:
            per_output = n // o
            if i % per_output == 0:
                return i // per_output
    group = int(np.fromfile(path, dtype=np.int32, count=1)[0])
    if 0 < group <= i and i % group == 0:
        n = o * (i // group)
        if size in (4 + n, 4 + 2 * n):
            return group
    return i


def is_grouped(path: str, count: int) -> bool:
    """IsGroupedQuantization (:104-126)."""
    size = file_size(path)
    if size < 4:
        return False
    group = int(np.fromfile(path, dtype=np.int32, count=1)[0])
    return 0 < group < 65536 and size - 4 in (count, 2 * count)


def scale_values(path: str, o: int, g: int) -> np.ndarray:
    """LoadScaleOrZeroPoint (:128-143) / ReadScaleOrZeroPointInt (:57-96): [o][g] float32."""
    count = o * g
    if is_grouped(path, count):
        each = (file_size(path) - 4) // count
        raw = np.fromfile(path, dtype=np.int8 if each == 1 else np.int16, offset=4, count=count)
        return (raw.astype(np.float32) / np.float32(1024.0)).reshape(o, g)
    return np.fromfile(path, dtype=np.float32, count=count).reshape(o, g)


def zero_point_values(zp_path: str, scale_path: str, o: int, g: int) -> np.ndarray:
    """LoadZeroPoint (:469-497): the stored value is zero_point * scale."""
    if not os.path.isfile(zp_path):
        return np.zeros((o, g), np.float32)
    zp, s = scale_values(zp_path, o, g), scale_values(scale_path, o, g)
    out = np.zeros_like(zp)
    np.divide(zp, s, out=out, where=s != 0.0)
    return out


def int4_file_as_int8(path: str, count: int) -> np.ndarray:
    """LoadInt4AsInt8 (:213-241): nibbles low first, two's complement."""
    b = np.fromfile(path, dtype=np.uint8, count=count // 2)
    nib = np.stack([b & 0xF, b >> 4], axis=1).reshape(-1).astype(np.int16)
    return (((nib + 8) & 15) - 8).astype(np.int8)
