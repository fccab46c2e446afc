"""Column sharding of the decoder's FullyConnected nodes over `world` ranks.

Output channels are independent, so rank r owns a block of rows of every weight matrix and
quantises / packs that sub-matrix on its own (per-row and per-block scales do not see the split);
concatenating the shard outputs in rank order reproduces the unsharded output.  The fused matrices
are split so that the concatenation of shard outputs is again a plain vector:
  q|k|v   : each rank takes the rows of its own heads from q, from k and from v;
  gate|up : each rank takes its slice of the hidden dimension, rows interleaved gate_i, up_i, so
            that the projection's fused SiLU*mul write sees both halves of a pair.
The reference has no counterpart (it is single-device); the rule follows from the FC definition
(ml_drift/common/task/testing_ref_ops.cc:961-988: every output channel is its own dot product).
"""
from __future__ import annotations

import numpy as np


def _block(n, rank, world):
    if n % world:
        raise ValueError(f"{n} rows do not divide over {world} ranks")
    per = n // world
    return np.arange(rank * per, (rank + 1) * per)


def column_shard_rows(n: int, rank: int, world: int) -> np.ndarray:
    """Rows of an [n][k] projection held by `rank` (o_proj, down_proj)."""
    return _block(n, rank, world)


def qkv_shard_rows(heads: int, head_dim: int, rank: int, world: int) -> np.ndarray:
    """Rows of the fused [3*heads*head_dim][k] q|k|v matrix held by `rank`: its heads of q, k and v."""
    d = heads * head_dim
    own = _block(heads, rank, world)
    rows = (own[:, None] * head_dim + np.arange(head_dim)[None, :]).reshape(-1)
    return np.concatenate([rows, d + rows, 2 * d + rows])


def gate_up_shard_rows(ffn: int, rank: int, world: int) -> np.ndarray:
    """Rows of the logical [gate ; up] matrix ([2*ffn][k]) held by `rank`, in the interleaved order
    gate_i, up_i, gate_i+1, up_i+1, ... the decoder's fused gate/up projection expects."""
    own = _block(ffn, rank, world)
    return np.stack([own, ffn + own], axis=1).reshape(-1)


def gathered_order(kind: str, rank_outputs):
    """Reassembles the unsharded output vector from per-rank outputs (list in rank order).
    kind: 'column' (plain concatenation), 'qkv' or 'gate_up' (fused matrices: per-part concatenation)."""
    if kind == "column":
        return np.concatenate(rank_outputs)
    if kind == "gate_up":      # per rank: gate_i, up_i interleaved -> [all gates | all ups]
        outs = [np.asarray(o) for o in rank_outputs]
        return np.concatenate([np.concatenate([o[0::2] for o in outs]), np.concatenate([o[1::2] for o in outs])])
    split = [np.split(np.asarray(o), 3) for o in rank_outputs]
    return np.concatenate([np.concatenate([s[p] for s in split]) for p in range(3)])


def input_shard_cols(k: int, rank: int, world: int) -> np.ndarray:
    """Input columns of a projection split by inputs (shard_layout 1: o takes the columns of the rank's
    heads, down the columns of the rank's FFN units): a contiguous K / world slice."""
    assert k % world == 0
    per = k // world
    return np.arange(rank * per, (rank + 1) * per, dtype=np.int64)
