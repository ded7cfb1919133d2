"""Python face of the CUDA kernel library: one thin function per kernel.

Each function checks devices, element types and layouts, passes raw pointers and the
current CUDA stream to the C entry point, and turns a non-zero return into
``KernelError``.  Nothing here computes; there is no CPU fallback.
"""
from __future__ import annotations

import ctypes
import functools
import inspect
from typing import Optional

import torch

from .csrc.build import library
from .errors import KernelError
from .profile import cost as _cost
from .profile import profiler as _profiler

F32, BF16 = 0, 1
PAGE = 64  # tokens per cache page (RB_PAGE in csrc/common.cuh)

_CODES = {
    10001: "a size the kernel does not take",
    10002: "an element type combination that is not built",
    10003: "a pointer or stride that breaks an alignment rule",
    10004: "a bounded wait inside a kernel ran out",
    10005: "a CUDA driver entry point could not be found",
    10006: "a file could not be read",
}

_c = ctypes
_vp, _i, _ll, _f = _c.c_void_p, _c.c_int, _c.c_longlong, _c.c_float


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {dt} is not supported by the kernels (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernel arguments must live on a CUDA device; there is no CPU path")
    return _vp(t.data_ptr())


def _stream():
    # the raw handle of torch's current stream on the current device, without building a Stream object
    return _vp(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


launch_count = 0  # kernel launches issued through this module (graph replays are counted by the engine)


def _check(rc: int, what: str):
    global launch_count
    launch_count += 1
    if rc != 0:
        if rc in _CODES:
            raise KernelError(f"{what}: {_CODES[rc]} (code {rc})")
        raise KernelError(f"{what}: CUDA error {rc}")


# ---- profiling: each wrapper below can be timed with what it had to move and compute ------------------

def _profiled(cost_of):
    """While a profiler is active (rocml_b200.profile), bracket the wrapped launch with a pair of CUDA
    events and file its bytes and operations: ``cost_of(a)`` gets the call's arguments by name and
    returns (bytes, flops).  A wrapper that returns False launched nothing and files nothing."""
    def deco(fn):
        sig = inspect.signature(fn)

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            prof = _profiler.ACTIVE
            if prof is None:
                return fn(*args, **kwargs)
            start = prof.begin()
            result = fn(*args, **kwargs)
            if result is not False:
                bound = sig.bind(*args, **kwargs)
                bound.apply_defaults()
                nbytes, flops = cost_of(bound.arguments, prof.facts)
                prof.end(start, fn.__name__, nbytes, flops)
            return result
        return wrapper
    return deco


def _esz(t) -> int:
    return t.element_size()


def _n_in(x) -> int:
    return x.shape[0] if x.dim() == 3 else 1


def _rows(a, x="x") -> int:
    return a[x].shape[0] if a.get("m") is None else a["m"]


def _attention_cost(a, facts, q="q"):
    window = a.get("window") or None
    n = a["n_seqs"]
    q_lens, kv_lens = facts.q_lens[:n], facts.kv_lens[:n]
    return _cost.attention(q_lens, kv_lens, a["nq"], a["nkv"], a["hd"], _esz(a["k_cache"]), window)


def _i32(t: torch.Tensor, name: str):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return _ptr(t)


_sigs_done = False


def _lib():
    global _sigs_done
    lib = library()
    if not _sigs_done:
        lib.rb_embedding.argtypes = [_vp, _vp, _i, _vp, _i, _i, _i, _vp, _vp]
        lib.rb_add_rmsnorm.argtypes = [_vp, _vp, _i, _ll, _vp, _i, _vp, _i, _vp, _i, _i, _f, _i, _vp]
        lib.rb_silu_mul.argtypes = [_vp, _i, _i, _ll, _vp, _i, _i, _i, _i, _vp]
        lib.rb_cast.argtypes = [_vp, _i, _vp, _i, _ll, _vp]
        lib.rb_qk_norm_rope_cache.argtypes = [_vp, _i, _i, _ll, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _f,
                                              _vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp]
        lib.rb_rope_table.argtypes = [_vp, _vp, _i, _i, _vp, _vp]
        lib.rb_gemm_generic.argtypes = [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _i, _ll, _vp]
        lib.rb_attention_generic.argtypes = [_vp, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i,
                                             _i, _i, _i, _f, _i, _i, _i, _vp, _vp, _vp]
        lib.rb_attention_merge.argtypes = [_vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]
        lib.rb_argmax.argtypes = [_vp, _ll, _i, _i, _vp, _vp, _vp, _i, _vp]
        lib.rb_attention_prefill.argtypes = [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                                             _f, _i, _vp]
        lib.rb_attention_prefill_tc5.argtypes = [_vp, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i,
                                                 _i, _i, _i, _f, _i, _i, _vp, _vp]
        lib.rb_attention_decode.argtypes = [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i,
                                            _i, _vp, _vp, _vp, _vp, _i, _vp]
        lib.rb_attention_decode_fused.argtypes = [_vp, _i, _ll, _i, _vp, _vp, _i, _f, _vp, _i, _vp, _i, _ll, _f, _i,
                                                  _vp, _vp, _vp, _i, _vp, _vp,
                                                  _vp, _i, _i, _i, _i, _f, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp]
        lib.rb_sample.argtypes = [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp]
        lib.rb_gemm_tcgen05.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _i, _ll, _i, _i, _vp, _vp]
        lib.rb_gemm_tcgen05_add.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _i, _vp, _vp]
        lib.rb_gemm_tcgen05_gated_pair.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _vp, _i, _ll, _f, _i, _vp, _vp]
        lib.rb_gemm_tcgen05_qkv_rope.argtypes = [_vp, _vp, _vp, _i, _i, _i, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _i, _vp,
                                                 _vp, _i, _f, _vp, _i, _i, _i, _vp, _vp]
        lib.rb_gemm_tcgen05_residual.argtypes = [_vp, _vp, _vp, _i, _i, _i, _ll, _i, _vp, _ll, _vp, _i, _vp, _ll, _vp,
                                                 _ll, _i, _vp, _vp]
        lib.rb_hold.argtypes = [_ll, _vp]
        lib.rb_gemm_tcgen05_set_wait.argtypes = [_ll, _i]
        lib.rb_gemm_tcgen05_set_wait.restype = None
        _sigs_done = True
    return lib


# ---- embedding --------------------------------------------------------------------------------

@_profiled(lambda a, facts: _cost.embedding(a["out"].shape[0], a["out"].shape[1], _esz(a["table"])))
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None):
    """out[t, :] = float32(table[ids[t], :]); out is [T, H] float32."""
    T, H = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embedding: out must be contiguous float32, table contiguous")
    if table.shape[1] != H or ids.numel() < T:
        raise KernelError("embedding: shapes do not fit")
    rc = _lib().rb_embedding(_i32(ids, "ids"), _ptr(table), dtype_code(table.dtype), _ptr(out), T, H,
                             table.shape[0], _ptr(status), _stream())
    _check(rc, "embedding")


# ---- fused residual add + RMSNorm ---------------------------------------------------------------

@_profiled(lambda a, facts: _cost.add_norm(
    a["n_rows"] if a["n_rows"] is not None else (a["rows"].numel() if a["rows"] is not None else a["resid"].shape[0]),
    a["resid"].shape[1], a["delta"].shape[0] if a["delta"] is not None else 0, _esz(a["out"]),
    bool(a["write_back"]) and a["delta"] is not None, _esz(a["weight"])))
def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                write_back: bool = True):
    """resid [T, H] float32 (+= sum of delta [S, T, H] float32); out[i] = rmsnorm(row) * weight.

    With ``rows`` (int32 indices, -1 = skip) output row i comes from source row rows[i]."""
    T, H = resid.shape
    if resid.dtype != torch.float32 or not resid.is_contiguous() or not out.is_contiguous():
        raise KernelError("add_rmsnorm: resid must be contiguous float32, out contiguous")
    n_delta, stride = 0, 0
    if delta is not None:
        if delta.dtype != torch.float32 or not delta.is_contiguous() or delta.dim() != 3 or \
                delta.shape[1] < T or delta.shape[2] != H:
            raise KernelError("add_rmsnorm: delta must be contiguous float32 [S, >=T, H]")
        n_delta, stride = delta.shape[0], delta.stride(0)
    n = (rows.numel() if rows is not None else T) if n_rows is None else n_rows
    if out.shape[-1] != H or out.numel() < n * H or weight.numel() != H:
        raise KernelError("add_rmsnorm: shapes do not fit")
    rc = _lib().rb_add_rmsnorm(_ptr(resid), _ptr(delta), n_delta, stride, _ptr(weight), dtype_code(weight.dtype),
                               _ptr(out), dtype_code(out.dtype), None if rows is None else _i32(rows, "rows"),
                               n, H, float(eps), 1 if write_back else 0, _stream())
    _check(rc, "add_rmsnorm")


def _partials(x: torch.Tensor, what: str):
    """(n partial sums, stride between them, row stride) of [T, N] or [S, T, N]."""
    if x.dim() == 3:
        if x.stride(2) != 1:
            raise KernelError(f"{what}: inner stride must be 1")
        return x.shape[0], x.stride(0), x.stride(1)
    if x.stride(1) != 1:
        raise KernelError(f"{what}: inner stride must be 1")
    return 1, 0, x.stride(0)


@_profiled(lambda a, facts: _cost.silu_mul(a["out"].shape[0], a["out"].shape[1], _n_in(a["x"]), _esz(a["x"]), _esz(a["out"])))
def silu_mul(x: torch.Tensor, out: torch.Tensor, paired: bool = False):
    """x [T, 2I] = [gate | up], or [S, T, 2I] partial sums to be added first -> out [T, I] = silu(gate) * up.
    ``paired``: gates and ups alternate in blocks of 16 columns instead of lying in two halves."""
    n_in, in_stride, row_stride = _partials(x, "silu_mul")
    T, I2 = x.shape[-2], x.shape[-1]
    if I2 % 2 or tuple(out.shape) != (T, I2 // 2) or row_stride != I2 or not out.is_contiguous():
        raise KernelError("silu_mul: shapes do not fit")
    _check(_lib().rb_silu_mul(_ptr(x), dtype_code(x.dtype), n_in, in_stride, _ptr(out), dtype_code(out.dtype), T,
                              I2 // 2, 1 if paired else 0, _stream()), "silu_mul")


@_profiled(lambda a, facts: (a["x"].numel() * (_esz(a["x"]) + _esz(a["out"])), 0))
def cast(x: torch.Tensor, out: torch.Tensor):
    if x.numel() != out.numel() or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("cast: shapes do not fit")
    _check(_lib().rb_cast(_ptr(x), dtype_code(x.dtype), _ptr(out), dtype_code(out.dtype), x.numel(), _stream()), "cast")


# ---- q/k norm + rotary + cache write --------------------------------------------------------------

@_profiled(lambda a, facts: _cost.qk_norm_rope(a["n_tokens"], a["nq"], a["nkv"], a["hd"], _n_in(a["proj"]), _esz(a["proj"]),
                                                  _esz(a["q_out"]), bool(a["write_kv"])))
def qk_norm_rope_cache(proj: torch.Tensor, q_out: torch.Tensor, n_tokens: int, nq: int, nkv: int, hd: int,
                       q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                       inv_freq: Optional[torch.Tensor], rot_dim: int, positions: torch.Tensor,
                       slot_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], write_kv: bool = True,
                       cos_sin: Optional[torch.Tensor] = None):
    """``cos_sin`` (from rope_table, float32 [T, rot_dim / 2, 2]) replaces the kernel's own sincosf.
    proj [T, nq*hd (+ 2*nkv*hd)] (or [S, T, ...] partial sums): q normalised and rotated into q_out
    (rows of nq*hd, any row stride; it may be ``proj`` itself); k (normalised, rotated) and v written
    to their pages."""
    width = (nq + (2 * nkv if write_kv else 0)) * hd
    n_in, in_stride, row_stride = _partials(proj, "qk_norm_rope_cache")
    if proj.shape[-1] != width:
        raise KernelError(f"qk_norm_rope_cache: projections must be {width} wide")
    if q_out.stride(-1) != 1 or q_out.shape[-1] < nq * hd:
        raise KernelError("qk_norm_rope_cache: q_out rows must hold nq * hd elements with unit stride")
    if (q_norm_w is None) != (k_norm_w is None):
        raise KernelError("qk_norm_rope_cache: give both norm weights or neither")
    wd = dtype_code(q_norm_w.dtype) if q_norm_w is not None else F32
    if q_norm_w is not None and (k_norm_w.dtype != q_norm_w.dtype or q_norm_w.numel() != hd or k_norm_w.numel() != hd):
        raise KernelError("qk_norm_rope_cache: norm weights must share a type and be [head_dim]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("qk_norm_rope_cache: inv_freq must be float32 [rot_dim / 2]")
    if write_kv:
        if k_cache is None or v_cache is None or block_table is None:
            raise KernelError("qk_norm_rope_cache: cache tensors missing")
        if k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype or not k_cache.is_contiguous() or \
                tuple(k_cache.shape[1:]) != (nkv, PAGE, hd):
            raise KernelError("qk_norm_rope_cache: cache must be [pages, nkv, 64, hd] of the activations' type")
    max_pages = block_table.shape[1] if block_table is not None else 0
    rc = _lib().rb_qk_norm_rope_cache(
        _ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride, _ptr(q_out), dtype_code(q_out.dtype),
        q_out.stride(-2), n_tokens, nq, nkv, hd, _ptr(q_norm_w), _ptr(k_norm_w), wd, float(eps), _ptr(inv_freq),
        rot_dim, _i32(positions, "positions"), _i32(slot_of_token, "slot_of_token"),
        None if block_table is None else _i32(block_table, "block_table"), max_pages, _ptr(k_cache), _ptr(v_cache),
        1 if write_kv else 0, _ptr(cos_sin), _stream())
    _check(rc, "qk_norm_rope_cache")


@_profiled(lambda a, facts: _cost.rope_table(a["n_tokens"], a["inv_freq"].numel()))
def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, n_tokens: int) -> torch.Tensor:
    """float32 [T, half, 2]: (cos, sin) of positions[t] * inv_freq[i], full-precision sincosf."""
    half = inv_freq.numel()
    out = torch.empty((n_tokens, half, 2), dtype=torch.float32, device=inv_freq.device)
    _check(_lib().rb_rope_table(_i32(positions, "positions"), _ptr(inv_freq), n_tokens, half, _ptr(out), _stream()),
           "rope_table")
    return out


# ---- matrix products ---------------------------------------------------------------------------------

@_profiled(lambda a, facts: _cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], _esz(a["w"]), _esz(a["x"]), _esz(a["out"]),
                                         _n_in(a["out"])))
def gemm_generic(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 m: Optional[int] = None):
    """out[M, N] = x[M, K] . w[N, K]^T (+ bias float32 [N]) on the CUDA cores, 32-bit accumulation.
    ``out`` float32 [S, M, N] with S > 1 (32-bit x and w, at most 16 rows): S partial sums over parts of K,
    to be added in order by the consumer (bias in the first)."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    splits, split_stride = 1, 0
    if out.dim() == 3:
        splits, split_stride = out.shape[0], out.stride(0)
        if out.dtype != torch.float32 or out.stride(2) != 1 or out.shape[2] != N:
            raise KernelError("gemm_generic: partial output must be float32 [S, M, N]")
        ldo = out.stride(1)
    else:
        if out.shape[1] != N or out.stride(1) != 1:
            raise KernelError("gemm_generic: shapes or strides do not fit")
        ldo = out.stride(0)
    if x.shape[1] != K or x.stride(1) != 1 or not w.is_contiguous():
        raise KernelError("gemm_generic: shapes or strides do not fit")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_generic: bias must be float32 [N]")
    rc = _lib().rb_gemm_generic(_ptr(x), dtype_code(x.dtype), _ptr(w), dtype_code(w.dtype), _ptr(bias), _ptr(out),
                                dtype_code(out.dtype), M, N, K, x.stride(0), ldo, splits, split_stride, _stream())
    _check(rc, "gemm_generic")


# ---- attention ------------------------------------------------------------------------------------------

@_profiled(lambda a, facts: _attention_cost(a, facts))
def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                      n_seqs: int, max_q_len: int, nq: int, nkv: int, hd: int, scale: float, window: int = 0,
                      chunk: int = 0, n_chunks: int = 1, part_acc: Optional[torch.Tensor] = None,
                      part_ml: Optional[torch.Tensor] = None):
    """q rows [T, >= nq*hd] (row stride free) -> out rows [T, >= nq*hd]; keys and values from the pages."""
    if q.stride(-1) != 1 or out.stride(-1) != 1 or q.dtype != out.dtype or k_cache.dtype != q.dtype:
        raise KernelError("attention_generic: strides or types do not fit")
    if tuple(k_cache.shape[1:]) != (nkv, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_generic: cache must be [pages, nkv, 64, hd]")
    rc = _lib().rb_attention_generic(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), dtype_code(q.dtype), _ptr(k_cache), _ptr(v_cache),
        _i32(block_table, "block_table"), block_table.shape[1], _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"),
        _i32(kv_len, "kv_len"), n_seqs, max_q_len, nq, nkv, hd, float(scale), int(window), int(chunk),
        int(n_chunks), _ptr(part_acc), _ptr(part_ml), _stream())
    _check(rc, "attention_generic")


PREFILL_L2_BYTES = 96 << 20     # keys and values that stay in the 126 MB L2 cache beside everything else


def prefill_heads_first(n_seqs: int, nkv: int, hd: int, max_kv_len: int, window: int = 0) -> bool:
    """Whether a prompt step's attention starts the longest blocks of all heads first (best balance) or
    runs one head after another (the blocks that run together share keys and values): the first while
    the bfloat16 keys and values of the step's contexts fit the L2 cache (measured: 26 % faster at 2,048
    tokens, 6 % at 16,384, 6 % slower at 32,768, where 134 MB are read by every query tile)."""
    span = min(max_kv_len, window) if window and window > 0 else max_kv_len
    return n_seqs * nkv * span * hd * 4 <= PREFILL_L2_BYTES


@_profiled(lambda a, facts: _attention_cost(a, facts))
def attention_prefill_tc5(q: torch.Tensor, n_tokens: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                          n_seqs: int, max_q_len: int, nq: int, nkv: int, hd: int, scale: float, window: int = 0,
                          max_kv_len: Optional[int] = None) -> bool:
    """bfloat16 flash attention with tcgen05 (accumulators in tensor memory, TMA loads), head sizes 64, 128 and 256.
    ``max_kv_len`` (the longest context of the step; the longest query if not given) only decides the
    order in which blocks start: the longest blocks of all heads first while the keys and values that
    the step reads fit the L2 cache, one head after another beyond.  Returns False when the kernel
    does not take the head size or the alignment."""
    if hd not in (64, 128, 256) or q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or \
            q.stride(-1) != 1 or out.stride(-1) != 1 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        return False
    if tuple(k_cache.shape[1:]) != (nkv, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_prefill_tc5: cache must be [pages, nkv, 64, hd]")
    rc = _lib().rb_attention_prefill_tc5(
        _ptr(q), q.stride(0), n_tokens, _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0],
        _i32(block_table, "block_table"), block_table.shape[1], _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"),
        _i32(kv_len, "kv_len"), n_seqs, max_q_len, nq, nkv, hd, float(scale), int(window),
        1 if prefill_heads_first(n_seqs, nkv, hd, max_q_len if max_kv_len is None else max_kv_len, window) else 0,
        _ptr(status_word(q.device)), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "attention_prefill_tc5")
    return True


@_profiled(lambda a, facts: _attention_cost(a, facts))
def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                      n_seqs: int, max_q_len: int, nq: int, nkv: int, hd: int, scale: float, window: int = 0) -> bool:
    """bfloat16 flash attention on the tensor cores for any number of query tokens per sequence.
    Returns False when the kernel does not take the head size or the alignment."""
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or \
            q.stride(-1) != 1 or out.stride(-1) != 1:
        return False
    if tuple(k_cache.shape[1:]) != (nkv, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_prefill: cache must be [pages, nkv, 64, hd]")
    rc = _lib().rb_attention_prefill(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _i32(block_table, "block_table"),
        block_table.shape[1], _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"), _i32(kv_len, "kv_len"), n_seqs,
        max_q_len, nq, nkv, hd, float(scale), int(window), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "attention_prefill")
    return True


_sm_count = {}


def decode_split(n_seqs: int, n_kv_groups: int, n_pages: int, device=0):
    """(blocks per sequence, pages per block) for decode attention.  Three blocks of the kernel fit a
    multiprocessor; the split is the finest that still runs as ONE wave (blocks per sequence times
    sequences times key/value head groups within the resident slots), because a second, partly filled
    wave costs a whole block's latency.  A large batch therefore walks many pages per block (one
    partial result and one merge for all of them) and a single sequence spreads over the device.
    Contexts beyond 4,096 tokens in a batch of four or more, and batches too large for one block a
    (sequence, head group): see below.  Up to 16 blocks per sequence form a thread-block cluster and
    merge through shared memory, which is so much quicker than through global memory that a finer
    split is always cut back to 16."""
    key = torch.device(device).index or 0
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(key).multi_processor_count
    slots = 3 * _sm_count[key]
    pairs = n_seqs * n_kv_groups
    if (4 <= n_seqs <= 256 and n_pages > 64) or \
            (2 <= n_seqs <= 256 and n_pages >= 8 and slots < pairs <= slots + slots // 3):
        # several long contexts, which may differ a lot in length, or a few more (sequence, head group)
        # pairs than blocks run at once (the second, thinly filled wave would take nearly as long as the
        # first; with more pairs than that, waves of whole sequences measured faster): one wave of blocks
        # a head group, which share the pages of all sequences equally (pages per block 0 says so to the
        # kernel)
        return max(1, min(1024, slots // max(1, n_kv_groups))), 0
    blocks = max(1, min(n_pages, slots // max(1, pairs)))
    # more than 16 blocks would merge through global memory, which costs more than the longer blocks
    # of a cluster do (one sequence of 8,192 tokens: 15 us with 16 blocks of 8 pages, 26 us with 43 of 3;
    # at 32,000 tokens 38 against 41)
    blocks = min(blocks, DECODE_CLUSTER_MAX)
    ppb = -(-n_pages // blocks)
    return -(-n_pages // ppb), ppb


DECODE_CLUSTER_MAX = 16

_counters = {}
_COUNTER_INTS = 1 << 20


def decode_counters(device) -> torch.Tensor:
    """Zeroed int32 work space of the decode attention kernel (one counter per sequence and head
    group); the kernel leaves it zeroed, so one buffer per device serves every launch."""
    key = torch.device(device).index or 0
    if key not in _counters:
        _counters[key] = torch.zeros(_COUNTER_INTS, dtype=torch.int32, device=device)
    return _counters[key]


def _check_parts(part_acc, part_ml, n_chunks: int, what: str) -> None:
    """The kernel numbers a row's partial results up to n_chunks - 1 and strides by n_chunks."""
    if n_chunks > 1 and (part_acc is None or part_ml is None or part_acc.shape[2] < n_chunks
                         or part_ml.shape[2] < n_chunks or part_acc.shape[2] != part_ml.shape[2]):
        raise KernelError(f"{what}: work space for {n_chunks} partial results a row is needed")


@_profiled(lambda a, facts: _attention_cost(a, facts))
def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                     n_seqs: int, nq: int, nkv: int, hd: int, scale: float, window: int, n_chunks: int,
                     part_acc: Optional[torch.Tensor], part_ml: Optional[torch.Tensor],
                     pages_per_block: int = 1) -> bool:
    """bfloat16 decode attention, one query token per sequence; a block takes ``pages_per_block``
    pages of 64 keys, ``n_chunks`` blocks cover the longest sequence and are merged by the kernel
    itself; part_acc / part_ml [T, nq, >= n_chunks, ...] are its work space when n_chunks > 1.
    ``pages_per_block`` 0: ``n_chunks`` blocks a key/value head group share the pages of all sequences
    equally, whatever their lengths (see ``decode_split``).  Returns False when the kernel does not
    take the head size or the alignment (use attention_generic)."""
    if n_seqs * nq > _COUNTER_INTS:
        return False
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or q.stride(-1) != 1 or out.stride(-1) != 1:
        return False
    if tuple(k_cache.shape[1:]) != (nkv, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_decode: cache must be [pages, nkv, 64, hd]")
    _check_parts(part_acc, part_ml, n_chunks, "attention_decode")
    rc = _lib().rb_attention_decode(
        _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _i32(block_table, "block_table"), block_table.shape[1],
        _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"), _i32(kv_len, "kv_len"), n_seqs, nq, nkv, hd, float(scale),
        int(window), int(n_chunks), int(pages_per_block), _ptr(part_acc), _ptr(part_ml),
        _ptr(decode_counters(q.device)), _ptr(out),
        out.stride(0), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "attention_decode")
    return True


@_profiled(lambda a, facts: tuple(map(sum, zip(_attention_cost(a, facts), (a["proj"].numel() * 4, 0)))))
def attention_decode_fused(proj: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                           n_seqs: int, nq: int, nkv: int, hd: int, q_norm_w: Optional[torch.Tensor],
                           k_norm_w: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                           write_kv: bool, scale: float, window: int, n_chunks: int,
                           part_acc: Optional[torch.Tensor], part_ml: Optional[torch.Tensor],
                           pages_per_block: int = 1, rowscale=None, row_width: int = 0) -> bool:
    """attention_decode for head size 128 that takes the step's projections as the matrix product left
    them: ``proj`` float32 [S, T, (nq + 2 nkv) * 128] partial sums (or [T, ...]; only the nq query heads
    when ``write_kv`` is off).  The kernel adds them, applies the per-head norm and the rotation
    (``cos_sin`` float32 [T, 64, 2] from rope_table) to the queries, and writes the new token's key and
    value into its page before reading it: the work of qk_norm_rope_cache, without a kernel in between.
    ``rowscale`` = (sumsq float32 [G, >= T], eps) with ``row_width``: the rows the projection was made
    from were residual * norm weight; the sums are scaled by rsqrt(sum / row_width + eps) first.
    Returns False when the kernel does not take the sizes (use the two kernels)."""
    if hd != 128 or proj.dtype != torch.float32 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 \
            or out.stride(-1) != 1 or n_seqs * nq > _COUNTER_INTS:
        return False
    width = (nq + (2 * nkv if write_kv else 0)) * hd
    n_in, in_stride, row_stride = _partials(proj, "attention_decode_fused")
    if proj.shape[-1] != width:
        raise KernelError(f"attention_decode_fused: projections must be {width} wide")
    if tuple(k_cache.shape[1:]) != (nkv, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_decode_fused: cache must be [pages, nkv, 64, hd]")
    if (q_norm_w is None) != (k_norm_w is None):
        raise KernelError("attention_decode_fused: give both norm weights or neither")
    w_f32 = 0
    if q_norm_w is not None:
        if q_norm_w.dtype != k_norm_w.dtype or q_norm_w.numel() != hd or k_norm_w.numel() != hd:
            raise KernelError("attention_decode_fused: norm weights must share a type and be [head_dim]")
        w_f32 = 1 if q_norm_w.dtype == torch.float32 else 0
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or cos_sin.numel() < n_seqs * hd):
        raise KernelError("attention_decode_fused: cos_sin must be float32 [T, 64, 2]")
    _check_parts(part_acc, part_ml, n_chunks, "attention_decode_fused")
    rc = _lib().rb_attention_decode_fused(
        _ptr(proj), n_in, in_stride, row_stride, _ptr(q_norm_w), _ptr(k_norm_w), w_f32, float(eps), _ptr(cos_sin),
        1 if write_kv else 0, *_row_scale(rowscale, n_seqs, "attention_decode_fused"), int(row_width),
        _ptr(k_cache), _ptr(v_cache), _i32(block_table, "block_table"), block_table.shape[1],
        _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"), _i32(kv_len, "kv_len"), n_seqs, nq, nkv, hd, float(scale),
        int(window), int(n_chunks), int(pages_per_block), _ptr(part_acc), _ptr(part_ml),
        _ptr(decode_counters(out.device)), _ptr(out), out.stride(0), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "attention_decode_fused")
    return True


@_profiled(lambda a, facts: (a["part_acc"].numel() * 4 + a["part_ml"].numel() * 4 + a["n_tokens"] * a["nq"] * a["hd"] * _esz(a["out"]), 0))
def attention_merge(part_acc: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                    slot_of_token: torch.Tensor, n_tokens: int, nq: int, hd: int, chunk: int, n_chunks: int,
                    window: int = 0):
    rc = _lib().rb_attention_merge(_ptr(part_acc), _ptr(part_ml), _ptr(out), out.stride(0), dtype_code(out.dtype),
                                   _i32(positions, "positions"), _i32(slot_of_token, "slot_of_token"), n_tokens,
                                   nq, hd, chunk, n_chunks, int(window), _stream())
    _check(rc, "attention_merge")


# ---- sampling ---------------------------------------------------------------------------------------------

_ARGMAX_SLICES = 64


@_profiled(lambda a, facts: _cost.sample(a["logits"].shape[0] if a["rows"] is None else a["rows"], a["logits"].shape[1]))
def argmax(logits: torch.Tensor, out: torch.Tensor, rows: Optional[int] = None):
    """out[r] = index of the first largest value of logits[r, :]; logits float32 [R, V].  Wide rows
    are searched by 64 blocks each, through a small work space."""
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32:
        raise KernelError("argmax: logits float32 with unit inner stride, out int32")
    R = logits.shape[0] if rows is None else rows
    V = logits.shape[1]
    sv = si = None
    slices = 1
    if V > 8192:
        slices = _ARGMAX_SLICES
        sv = torch.empty((R, slices), dtype=torch.float32, device=logits.device)
        si = torch.empty((R, slices), dtype=torch.int32, device=logits.device)
    _check(_lib().rb_argmax(_ptr(logits), logits.stride(0), R, V, _ptr(out), _ptr(sv), _ptr(si), slices, _stream()),
           "argmax")


@_profiled(lambda a, facts: _cost.sample(a["n"], a["logits"].shape[1]))
def sample(logits: torch.Tensor, n: int, rows: torch.Tensor, history: Optional[torch.Tensor], out: torch.Tensor):
    """One token per row of float32 logits [>= n, V].  ``rows`` holds n records of 8 x 32 bits
    {temperature f32, top_k i32 (0 off), top_p f32 (< 0 off), u f32, penalty f32 (<= 0 off),
    hist_begin i32, hist_len i32, 0} (an int32 tensor with the floats bit-cast); ``history``
    int32 ids.  The repeat penalty edits the logits in place."""
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32 or rows.numel() < 8 * n:
        raise KernelError("sample: logits float32 with unit inner stride, out int32, 8 words per row")
    _check(_lib().rb_sample(_ptr(logits), logits.stride(0), n, logits.shape[1], _i32(rows, "rows"),
                            None if history is None else _i32(history, "history"), _ptr(out), _stream()), "sample")


# ---- tensor-core matrix product (tcgen05) ----------------------------------------------------------------

_status = {}


def status_word(device) -> torch.Tensor:
    """One int32 per device where kernels record a bounded wait that ran out (or a bad token id)."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def raise_for_status(value: int, device=None) -> None:
    """Raise if ``value``, a copy of a device's status word, records a failure; the word itself
    is cleared so that the next step starts clean."""
    if value != 0:
        key = torch.device(device).index or 0 if device is not None else None
        for k, word in _status.items():
            if key is None or k == key:
                word.zero_()
        raise KernelError(f"a kernel reported failure: {_CODES.get(value, 'code ' + str(value))} (code {value})")


def check_status(device) -> None:
    """Read the device's status word (this synchronises) and raise if a kernel recorded a failure."""
    key = torch.device(device).index or 0
    if key in _status:
        raise_for_status(int(_status[key].item()), device)


def hold(microseconds: float) -> None:
    """Keep the current stream busy for about that long (at most a second; not counted as a launch): what is
    enqueued behind it starts when it ends.  The profiler holds the GPU back with it while the host
    enqueues a step."""
    rc = _lib().rb_hold(int(microseconds), _stream())
    if rc != 0:
        raise KernelError(f"hold: CUDA error {rc}")


def set_wait_limit(cycles: int = 0, withhold_first_stage: bool = False) -> None:
    """How long (in clock cycles; 0 restores the default of about two seconds) a warp of the tensor-core
    products waits on a barrier before it gives up, records the failure in the status word and lets
    its block unwind.  ``withhold_first_stage`` is for tests of that path only: few-token products then
    never request their first K block, so the wait for it must run out (with a limit of microseconds
    this takes microseconds and leaves the device usable); they compute nothing useful while it is set."""
    _lib().rb_gemm_tcgen05_set_wait(int(cycles), 1 if withhold_first_stage else 0)


@_profiled(lambda a, facts: (_cost.gated_linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, _esz(a["out"])) if a["gated"] else
                         _cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, _esz(a["out"]), _n_in(a["out"]))))
def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 m: Optional[int] = None, stages: int = 0, gated: bool = False) -> bool:
    """out = x . w^T on the tensor cores; x, w bfloat16, out bfloat16 [M, N] or float32 [M, N] or
    float32 [S, M, N] (S partial sums over K, to be added by the consumer).  Returns False when the
    kernel refuses the layout (K or a row stride not a multiple of 8, a pointer off 16 bytes);
    the caller then uses the plain kernel.

    ``gated``: w's rows alternate in blocks of 16 between a gate and an up projection of the same
    16 outputs, and out is bfloat16 [M, N / 2] = silu(gate) * up, computed in the epilogue."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05: x and w must be bfloat16, K-major, with matching K")
    if out.dim() == 3:
        splits, split_stride, ldo = out.shape[0], out.stride(0), out.stride(1)
        if out.shape[2] != N or out.stride(2) != 1 or out.dtype != torch.float32:
            raise KernelError("gemm_tcgen05: partial output must be float32 [S, M, N]")
    else:
        splits, split_stride, ldo = 1, 0, out.stride(0)
        if out.shape[1] != (N // 2 if gated else N) or out.stride(1) != 1:
            raise KernelError("gemm_tcgen05: output must be [M, N] (or [M, N / 2] when gated) with unit inner stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05: bias must be float32 [N]")
    rc = _lib().rb_gemm_tcgen05(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0),
                                ldo, splits, split_stride, stages, 1 if gated else 0, _ptr(status_word(x.device)), _stream())
    if rc == 10003:
        return False
    _check(rc, "gemm_tcgen05")
    return True


def _row_scale(rowscale, m: int, what: str):
    """(pointer, groups, stride, eps) of a deferred 1/RMS: ``rowscale`` = (sumsq float32 [G, >= M], eps)."""
    if rowscale is None:
        return None, 0, 0, 0.0
    sumsq, eps = rowscale
    if sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.stride(1) != 1 or sumsq.shape[1] < m:
        raise KernelError(f"{what}: the rows' sums of squares must be float32 [groups, >= rows]")
    return _ptr(sumsq), sumsq.shape[0], sumsq.stride(0), float(eps)


@_profiled(lambda a, facts: _cost.gated_linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, 2))
def gemm_tcgen05_gated_pair(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, bias: Optional[torch.Tensor] = None,
                            m: Optional[int] = None, rowscale=None) -> bool:
    """h = silu(gate) * up for at most 32 rows, w's rows alternating in blocks of 16 between gate and
    up, with the sum over K done in two halves by two blocks that form a thread-block cluster: the
    second hands its half to the first through shared memory, so no partial sums go through global
    memory.  h is bfloat16 [M, N / 2].  ``rowscale`` = (sumsq float32 [G, >= M], eps): x's rows are
    residual * norm weight, not yet divided by their RMS; column m of sumsq sums to row m's sum of
    squares over K values, and the product is scaled by rsqrt(sum / K + eps) before the bias.
    Returns False when the kernel refuses the sizes or the layout."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05_gated_pair: x and w must be bfloat16, K-major, with matching K")
    if h.dtype != torch.bfloat16 or h.shape[1] != N // 2 or h.stride(1) != 1:
        raise KernelError("gemm_tcgen05_gated_pair: h must be bfloat16 [M, N / 2] with unit inner stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_gated_pair: bias must be float32 [N]")
    if M > 32 or N % 32 or K <= 64:
        return False
    rc = _lib().rb_gemm_tcgen05_gated_pair(_ptr(x), _ptr(w), _ptr(bias), _ptr(h), M, N, K, x.stride(0), h.stride(0),
                                           *_row_scale(rowscale, M, "gemm_tcgen05_gated_pair"), 0,
                                           _ptr(status_word(x.device)), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "gemm_tcgen05_gated_pair")
    return True


@_profiled(lambda a, facts: _cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, 4, 1, True))
def gemm_tcgen05_add(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     m: Optional[int] = None) -> bool:
    """resid += x . w^T (+ bias) for many rows (more than 256, N at least 256): the product is added into
    the float32 residual stream in its own epilogue, so no delta goes through memory.  Returns False
    when the kernel refuses the sizes or the layout (write a delta instead)."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05_add: x and w must be bfloat16, K-major, with matching K")
    if resid.dtype != torch.float32 or resid.shape[1] != N or resid.stride(1) != 1 or resid.shape[0] < M:
        raise KernelError("gemm_tcgen05_add: resid must be float32 [>= M, N] with unit inner stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_add: bias must be float32 [N]")
    if M <= 256 or N < 256:
        return False
    rc = _lib().rb_gemm_tcgen05_add(_ptr(x), _ptr(w), _ptr(bias), _ptr(resid), M, N, K, x.stride(0), resid.stride(0), 0,
                                    _ptr(status_word(x.device)), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "gemm_tcgen05_add")
    return True


@_profiled(lambda a, facts: tuple(map(sum, zip(_cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, 4, 1, True),
                                                       (_rows(a) * a["w"].shape[0] * 2 if a["xhat"] is not None else 0, 0)))))
def gemm_tcgen05_residual(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, splits: int,
                          bias: Optional[torch.Tensor] = None, next_w: Optional[torch.Tensor] = None,
                          xhat: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None,
                          m: Optional[int] = None) -> bool:
    """resid += x . w^T (+ bias) for at most 64 rows, the sum over K in ``splits`` (4, 8, 16) parts by
    the blocks of a thread-block cluster that exchange their parts through shared memory.  For the
    norm that follows: ``xhat`` bfloat16 [M, N] = resid * next_w (the row's 1/RMS is applied by the
    consumer) and ``sumsq`` float32 [ceil(N / 128) * splits, >= M], whose column m sums to the sum of
    squares of row m.  Returns False when the kernel refuses the sizes or the layout."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05_residual: x and w must be bfloat16, K-major, with matching K")
    if resid.dtype != torch.float32 or resid.shape[1] != N or resid.stride(1) != 1:
        raise KernelError("gemm_tcgen05_residual: resid must be float32 [M, N] with unit inner stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_residual: bias must be float32 [N]")
    if xhat is not None:
        if next_w is None or next_w.numel() != N or next_w.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("gemm_tcgen05_residual: xhat needs the norm's weight [N], float32 or bfloat16")
        if xhat.dtype != torch.bfloat16 or xhat.shape[1] != N or xhat.stride(1) != 1:
            raise KernelError("gemm_tcgen05_residual: xhat must be bfloat16 [M, N] with unit inner stride")
    if sumsq is not None and (sumsq.dtype != torch.float32 or sumsq.stride(1) != 1 or sumsq.shape[1] < M
                              or sumsq.shape[0] != ((N + 127) // 128) * splits):
        raise KernelError("gemm_tcgen05_residual: sumsq must be float32 [ceil(N / 128) * splits, >= M]")
    if M > 64 or splits not in (4, 8, 16) or (K + 63) // 64 < splits:
        return False
    rc = _lib().rb_gemm_tcgen05_residual(
        _ptr(x), _ptr(w), _ptr(bias), M, N, K, x.stride(0), splits, _ptr(resid), resid.stride(0), _ptr(next_w),
        1 if (next_w is not None and next_w.dtype == torch.float32) else 0, _ptr(xhat),
        xhat.stride(0) if xhat is not None else 0, _ptr(sumsq), sumsq.stride(0) if sumsq is not None else 0, 0,
        _ptr(status_word(x.device)), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "gemm_tcgen05_residual")
    return True


@_profiled(lambda a, facts: _cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, 2))
def gemm_tcgen05_qkv_rope(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, nq: int, nkv: int,
                          q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                          cos_sin: Optional[torch.Tensor], positions: torch.Tensor, slot_of_token: torch.Tensor,
                          block_table: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], bias: Optional[torch.Tensor] = None,
                          m: Optional[int] = None) -> bool:
    """A prompt's q | k | v projection (more than 256 rows, heads of 128) with the per-head norm, the
    rotation and the cache write done in the product's epilogue: q_out bfloat16 [M, nq * 128] receives the
    queries, the keys and values go into their pages.  w is [(nq + 2 nkv) * 128, K], or [nq * 128, K] for
    a layer that only reads a cache (then the cache arguments are unused).  ``cos_sin`` float32
    [M, 64, 2] from rope_table, or None for no rotation.  Returns False when the kernel does not take
    the sizes (run the product and qk_norm_rope_cache instead)."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05_qkv_rope: x and w must be bfloat16, K-major, with matching K")
    writes = N == (nq + 2 * nkv) * 128
    if M <= 256 or N % 256 or not (writes or N == nq * 128) or K % 8:
        return False
    if q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1 or q_out.shape[1] < nq * 128:
        raise KernelError("gemm_tcgen05_qkv_rope: q_out must be bfloat16 rows of nq * 128 with unit inner stride")
    if writes:
        if k_cache is None or v_cache is None or block_table is None:
            raise KernelError("gemm_tcgen05_qkv_rope: cache tensors missing")
        if k_cache.dtype != torch.bfloat16 or not k_cache.is_contiguous() or tuple(k_cache.shape[1:]) != (nkv, PAGE, 128) \
                or k_cache.shape != v_cache.shape or not v_cache.is_contiguous():
            raise KernelError("gemm_tcgen05_qkv_rope: cache must be bfloat16 [pages, nkv, 64, 128]")
    if (q_norm_w is None) != (k_norm_w is None):
        raise KernelError("gemm_tcgen05_qkv_rope: give both norm weights or neither")
    w_f32 = 0
    if q_norm_w is not None:
        if q_norm_w.dtype != k_norm_w.dtype or q_norm_w.numel() != 128 or k_norm_w.numel() != 128:
            raise KernelError("gemm_tcgen05_qkv_rope: norm weights must share a type and be [128]")
        w_f32 = 1 if q_norm_w.dtype == torch.float32 else 0
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or cos_sin.numel() < M * 128):
        raise KernelError("gemm_tcgen05_qkv_rope: cos_sin must be float32 [M, 64, 2]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_qkv_rope: bias must be float32 [N]")
    rc = _lib().rb_gemm_tcgen05_qkv_rope(
        _ptr(x), _ptr(w), _ptr(bias), M, N, K, x.stride(0), _ptr(q_out), q_out.stride(0), _ptr(k_cache), _ptr(v_cache),
        _i32(positions, "positions"), _i32(slot_of_token, "slot_of_token"),
        None if block_table is None else _i32(block_table, "block_table"),
        block_table.shape[1] if block_table is not None else 0, _ptr(q_norm_w), _ptr(k_norm_w), w_f32, float(eps),
        _ptr(cos_sin), nq, nkv, 0, _ptr(status_word(x.device)), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "gemm_tcgen05_qkv_rope")
    return True

