"""A plain, slow implementation of the dense Qwen3 decoder, for tests only.

It rests on the reference's FORMULAS, not on its outputs: the reference
(xmiksay/rocml, a Rust + HIP project) cannot be compiled or imported here
(no Rust toolchain, no ROCm, and its fixtures need a GGUF checkpoint), so every
function below restates the formula of the file and line it cites.  Whole
sequences, no cache, one function for each part, torch on the CPU, and no code
shared with ``rocml_b200`` (it even reads the model folder with the
``safetensors`` package rather than with the library's reader).

``dtype`` is float32 (the reference's own arithmetic) or float64 (used to tell
rounding from faults).
"""
from __future__ import annotations

import json
import math
import os

import torch


# ---- parts -------------------------------------------------------------------------

def embedding(table, ids):
    """x[t, :] = table[id_t, :], no scaling (rocml-kernels/kernels/embedding.hip:13-17)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rmsnorm(x, weight, eps):
    """x * rsqrt(mean(x^2) + eps) * w over the last axis; the weight multiplies directly,
    no (1 + w) (rocml-kernels/kernels/rmsnorm.hip:18-41)."""
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * torch.rsqrt(mean_sq + eps) * weight


def linear(x, weight, bias=None):
    """y = x W^T (+ b); W is [out, in] row-major (rocml-kernels/kernels/gemv_f16.hip:8-36,
    gemm_f16.hip:10-41).  The reference loads no bias; where a configuration has one it is
    added after the product, before any norm."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def rope_neox(x, positions, theta):
    """Rotate-half rotary embedding over the whole head: for i < hd/2,
    inv_freq = theta^(-2i/hd), a = pos * inv_freq,
    (x_i, x_{i+hd/2}) <- (x_i cos a - x_{i+hd/2} sin a, x_i sin a + x_{i+hd/2} cos a)
    (rocml-kernels/kernels/rope.hip:18-33).  x: [T, heads, hd]; positions: [T], absolute,
    0-based."""
    hd = x.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=x.dtype)
    inv_freq = torch.pow(torch.tensor(theta, dtype=x.dtype), -2.0 * i / hd)
    ang = torch.as_tensor(positions, dtype=x.dtype)[:, None] * inv_freq[None, :]  # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def attention(q, k, v, window=None, scale=None):
    """Causal grouped-query attention of one whole sequence.

    Query head h reads key/value head h // g with g = n_q / n_kv, groups contiguous
    (rocml-kernels/kernels/attn_decode.hip:108); s_j = (q . k_j) * scale with
    scale = 1/sqrt(hd) applied after the dot (attn_decode.hip:158, rocml/src/forward/
    attention.rs:160); the query at position p sees j in [0, p] (attn_prefill.hip:57-60,121);
    softmax with the maximum subtracted (attn_decode.hip:160-170); o = sum p_j v_j / l
    (attn_prefill.hip:201-203).  ``window`` n keeps only j > p - n (the reference has no
    window; this is the sliding_window key of Qwen3's config.json).
    q: [T, nq, hd]; k, v: [T, nkv, hd]; returns [T, nq, hd].
    """
    T, nq, hd = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    out = torch.empty_like(q)
    pos = torch.arange(T)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - window
    for h in range(nq):
        kh, vh = k[:, h // g, :], v[:, h // g, :]
        s = (q[:, h, :] @ kh.t()) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        out[:, h, :] = (p @ vh) / p.sum(dim=-1, keepdim=True)
    return out


def silu_mul(gate, up):
    """(g / (1 + exp(-g))) * u (rocml-kernels/kernels/silu_mul.hip:15-18)."""
    return gate / (1.0 + torch.exp(-gate)) * up


# ---- the model -----------------------------------------------------------------------

class PlainQwen3:
    def __init__(self, folder, dtype=torch.float32):
        from safetensors.torch import load_file

        with open(os.path.join(folder, "config.json")) as f:
            self.cfg = json.load(f)
        self.dtype = dtype
        self.w = {k: v.to(dtype) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
        c = self.cfg
        self.n_layers = c["num_hidden_layers"]
        self.nq = c["num_attention_heads"]
        self.nkv = c["num_key_value_heads"]
        self.hd = c.get("head_dim") or c["hidden_size"] // self.nq
        self.eps = c["rms_norm_eps"]
        self.theta = c["rope_theta"]
        self.bias = bool(c.get("attention_bias", False))
        types = c.get("layer_types")
        self.windows = [None] * self.n_layers
        if types is not None:
            self.windows = [c["sliding_window"] if t == "sliding_attention" else None for t in types]
        elif c.get("use_sliding_window", False):
            self.windows = [c["sliding_window"] if i >= c["max_window_layers"] else None
                            for i in range(self.n_layers)]

    def attention_block(self, x, i, positions):
        """norm -> q, k, v -> per-head q_norm / k_norm (not v) -> rope(q, k) -> attention ->
        o_proj (rocml/src/forward/attention.rs:56-244, attention_chunk.rs:75-325)."""
        w, p = self.w, f"model.layers.{i}.self_attn."
        T = x.shape[0]
        b = (lambda n: w[p + n + ".bias"]) if self.bias else (lambda n: None)
        q = linear(x, w[p + "q_proj.weight"], b("q_proj")).view(T, self.nq, self.hd)
        k = linear(x, w[p + "k_proj.weight"], b("k_proj")).view(T, self.nkv, self.hd)
        v = linear(x, w[p + "v_proj.weight"], b("v_proj")).view(T, self.nkv, self.hd)
        q = rmsnorm(q, w[p + "q_norm.weight"], self.eps)
        k = rmsnorm(k, w[p + "k_norm.weight"], self.eps)
        q = rope_neox(q, positions, self.theta)
        k = rope_neox(k, positions, self.theta)
        o = attention(q, k, v, window=self.windows[i]).reshape(T, self.nq * self.hd)
        return linear(o, w[p + "o_proj.weight"], b("o_proj"))

    def mlp_block(self, x, i):
        """gate, up -> silu(gate) * up -> down (rocml/src/forward/ffn.rs:57-107)."""
        w, p = self.w, f"model.layers.{i}.mlp."
        h = silu_mul(linear(x, w[p + "gate_proj.weight"]), linear(x, w[p + "up_proj.weight"]))
        return linear(h, w[p + "down_proj.weight"])

    def hidden_states(self, ids):
        """Residual stream after the last layer, [T, H] (rocml/src/forward/mod.rs:271-340)."""
        w = self.w
        T = len(ids)
        positions = torch.arange(T)
        x = embedding(w["model.embed_tokens.weight"], ids)
        for i in range(self.n_layers):
            p = f"model.layers.{i}."
            x = x + self.attention_block(rmsnorm(x, w[p + "input_layernorm.weight"], self.eps), i, positions)
            x = x + self.mlp_block(rmsnorm(x, w[p + "post_attention_layernorm.weight"], self.eps), i)
        return x

    def logits(self, ids):
        """Logits at every position, [T, V]: final norm, then the head; a tied head reads
        the embedding table (rocml/src/forward/mod.rs:349-378, weights/mod.rs:48-62)."""
        w = self.w
        x = rmsnorm(self.hidden_states(ids), w["model.norm.weight"], self.eps)
        head = w["model.embed_tokens.weight"] if self.cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
        return linear(x, head)

    def greedy(self, ids, n):
        """n greedy tokens after ``ids``; the first maximum wins (rocml/src/sample.rs:172-182)."""
        ids = list(ids)
        out = []
        for _ in range(n):
            nxt = int(torch.argmax(self.logits(ids)[-1]))
            out.append(nxt)
            ids.append(nxt)
        return out
