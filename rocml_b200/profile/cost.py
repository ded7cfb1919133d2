"""Bytes and floating-point operations of each kind of kernel, from sizes alone.

Pure arithmetic, no device: every formula is a LOWER bound on what the operation has to move
and compute (each weight once, each activation in and out once, each key and value of the live
contexts once), so time divided into it says how far the kernel is from the device's limits, not
how its implementation happens to move data.  The reference keeps the same kind of table
(rocml/src/profile/cost.rs:17-75); its sizes are 32-bit activations and a single sequence, here
the element sizes and the batch are arguments.
"""
from __future__ import annotations

from typing import Iterable, Optional, Tuple

Cost = Tuple[int, int]          # (bytes, flops)


def linear(m: int, n: int, k: int, w_esz: int, x_esz: int, out_esz: int, splits: int = 1,
           reads_out: bool = False) -> Cost:
    """y[m, n] = x[m, k] . W[n, k]^T: the weight once, the rows in, the result out (``splits`` partial
    results when the sum over k is cut; read and written when the product adds into its output)."""
    out = m * n * out_esz * splits * (2 if reads_out else 1)
    return n * k * w_esz + m * k * x_esz + out, 2 * m * n * k


def gated_linear(m: int, n2: int, k: int, w_esz: int, x_esz: int, out_esz: int) -> Cost:
    """act(gate) * up from a stacked [n2, k] weight: n2 / 2 outputs a row."""
    return n2 * k * w_esz + m * k * x_esz + m * (n2 // 2) * out_esz, 2 * m * n2 * k + 4 * m * (n2 // 2)


def embedding(rows: int, hidden: int, table_esz: int) -> Cost:
    """A row of the table in, a 32-bit row out; no arithmetic (rocml/src/profile/cost.rs:45-47)."""
    return rows * hidden * (table_esz + 4), 0


def add_norm(rows: int, hidden: int, n_delta: int, out_esz: int, write_back: bool, w_esz: int = 4) -> Cost:
    """Residual rows in (and back, when deltas were added), ``n_delta`` 32-bit deltas in, normalised
    rows out; about 4 operations an element (rocml/src/profile/cost.rs:28-40) plus the additions."""
    per_row = hidden * (4 + (4 if write_back else 0) + 4 * n_delta + out_esz)
    return rows * per_row + hidden * w_esz, rows * hidden * (4 + n_delta)


def silu_mul(rows: int, inter: int, n_in: int, in_esz: int, out_esz: int) -> Cost:
    return rows * inter * (2 * in_esz * n_in + out_esz), rows * inter * (4 + 2 * n_in)


def qk_norm_rope(rows: int, nq: int, nkv: int, hd: int, n_in: int, in_esz: int, out_esz: int, writes_kv: bool) -> Cost:
    """Projections in, queries out, keys and values into their pages."""
    width = (nq + (2 * nkv if writes_kv else 0)) * hd
    out = nq * hd + (2 * nkv * hd if writes_kv else 0)
    return rows * (width * in_esz * n_in + out * out_esz), rows * (nq + nkv) * hd * 10


def rope_table(rows: int, half: int) -> Cost:
    return rows * (4 + half * 8) + half * 4, rows * half * 40


def attention(q_lens: Iterable[int], kv_lens: Iterable[int], nq: int, nkv: int, hd: int, esz: int,
              window: Optional[int] = None) -> Cost:
    """Softmax attention of each sequence's last ``q_len`` positions over its own keys: the keys and
    values a sequence's queries can see once (grouped heads share them: the traffic scales with the
    key/value heads, rocml/src/profile/cost.rs:58-68), queries in, outputs out; 4 operations per
    (query head, visible key, head dimension) (rocml/src/profile/cost.rs:75-77)."""
    nbytes = flops = 0
    for ql, kl in zip(q_lens, kv_lens):
        if ql <= 0 or kl <= 0:
            continue
        first = kl - ql                                          # position of the first query
        seen_from = max(0, first - window + 1) if window else 0  # the oldest key any query sees
        nbytes += 2 * nkv * (kl - seen_from) * hd * esz + 2 * ql * nq * hd * esz
        if window:
            ramp = max(0, min(ql, window - first - 1))           # queries that still see fewer than a window
            pairs = ramp * (first + 1) + ramp * (ramp - 1) // 2 + (ql - ramp) * window
        else:
            pairs = ql * (first + 1) + ql * (ql - 1) // 2
        flops += 4 * nq * hd * pairs
    return nbytes, flops


def sample(rows: int, vocab: int) -> Cost:
    """The rows of 32-bit logits once."""
    return rows * vocab * 4, rows * vocab * 2


def model_step(layer_weight_bytes: int, n_layers: int, head_bytes: int, kv_bytes_per_token: int,
               live_tokens: int) -> int:
    """Bytes one decode step has to read: every weight once and the live sequences' keys and values."""
    return layer_weight_bytes * n_layers + head_bytes + kv_bytes_per_token * live_tokens


def decoder_flops(tokens: int, hidden: int, q_dim: int, kv_dim: int, inter: int, n_layers: int,
                  vocab: int, logit_rows: int, attention_flops: int = 0) -> int:
    """Floating-point operations of a dense decoder's products for ``tokens`` rows (q, k, v, o, gate, up,
    down in every layer, the head on ``logit_rows`` rows) plus the attention's own."""
    per_layer = 2 * tokens * (hidden * (q_dim + 2 * kv_dim) + q_dim * hidden + 3 * hidden * inter)
    return n_layers * per_layer + 2 * logit_rows * hidden * vocab + attention_flops
