"""Tensor-level wrappers of the kernel library: argument checks, then one launch on the current stream.

Tensors must be contiguous CUDA tensors; nothing here computes on the CPU or through torch ops.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as L

_CODE = {torch.float32: L.F32, torch.bfloat16: L.BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODE[dtype]
    except KeyError:
        raise L.KernelError(f"dtype {dtype} is not supported by the kernels (float32 and bfloat16 are)") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(name: str, t: torch.Tensor, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise L.KernelError(f"{name} must be a CUDA tensor: the kernels have no CPU path")
    if not t.is_contiguous():
        raise L.KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise L.KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise L.KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)   # the current stream's handle without building a Stream object
_device_index: Optional[int] = None


def _stream() -> int:
    """The handle of torch's current stream on the engine's device (every kernel is launched on it)."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


_KV_MAPS: dict = {}   # (pool address, shape) -> (buffer that owns the bytes, aligned address of the 128-byte tensor map) or None


def kv_tensor_map(pool: torch.Tensor):
    """The TMA description of a bfloat16 cache pool, made once per pool; None when the geometry
    cannot be served by TMA (the attention kernels then copy with cp.async)."""
    key = (pool.data_ptr(), tuple(pool.shape), pool.dtype)
    if key not in _KV_MAPS:
        entries, pages, two, kv_heads, page_size, head_dim = pool.shape
        made = None
        if two == 2 and pool.dtype == torch.bfloat16 and head_dim % 64 == 0 and page_size % 8 == 0 and (64 % page_size == 0 or page_size % 64 == 0):
            buf = C.create_string_buffer(128 + 64)
            addr = (C.addressof(buf) + 63) & ~63
            lib = L.load()
            lib.ib_make_kv_map.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int]
            lib.ib_make_kv_map.restype = C.c_int
            if lib.ib_make_kv_map(addr, pool.data_ptr(), pages * entries * two * kv_heads * page_size, head_dim, page_size) == 0:
                made = (buf, addr)
        _KV_MAPS[key] = made
    return _KV_MAPS[key]


@dataclass
class KvLayerView:
    """One layer's keys and values inside a paged pool, plus the block table of the step."""
    pool: torch.Tensor          # [entries, pages, 2, kv_heads, page_size, head_dim]: one layer's pages lie together
    entry: int
    block_table: torch.Tensor   # int32 [segments, table_stride]

    def tma(self) -> tuple[Optional[int], int]:
        """(address of the pool's tensor map or None, pool row where this view's keys of page 0, head 0 start)."""
        m = kv_tensor_map(self.pool)
        _, pages, _, kv_heads, page_size, _ = self.pool.shape
        return (m[1] if m else None), self.entry * pages * 2 * kv_heads * page_size

    def c_view(self) -> L.KvView:
        cv = self.__dict__.get("_cv")   # made once per view: a layer asks for it several times a step
        if cv is None:
            cv = self.__dict__["_cv"] = self._make_c_view()
        return cv

    def _make_c_view(self) -> L.KvView:
        entries, pages, planes, kv_heads, page_size, head_dim = self.pool.shape
        if planes not in (1, 2):
            raise L.KernelError(f"a cache pool must be [entries, pages, 2 (keys, values) or 1 (rows), kv_heads, page_size, head_dim], got {tuple(self.pool.shape)}")
        _check("kv pool", self.pool)
        _check("block_table", self.block_table, torch.int32)
        per_kv = kv_heads * page_size * head_dim
        esz = self.pool.element_size()
        return L.KvView(
            base=self.pool.data_ptr() + self.entry * pages * planes * per_kv * esz,
            page_stride=planes * per_kv,
            v_offset=per_kv if planes == 2 else 0,
            block_table=self.block_table.data_ptr(),
            table_stride=self.block_table.shape[1],
            page_size=page_size,
            num_pages=pages,
            kv_heads=kv_heads,
            head_dim=head_dim,
            dtype=dtype_code(self.pool.dtype),
        )


def embed(table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor, status: torch.Tensor) -> None:
    """x[t] = float32(table[tokens[t]])."""
    V, H = table.shape
    T = tokens.shape[0]
    _check("table", table)
    _check("tokens", tokens, torch.int32)
    _check("x", x, torch.float32, (T, H))
    L.call("ib_embed", table.data_ptr(), dtype_code(table.dtype), tokens.data_ptr(), x.data_ptr(), T, H, V, status.data_ptr(), _stream())


L.register("ib_embed_pos", [L._p, L._i, L._p, L._p, L._p, L._f, L._p, L._i, L._i, L._i, L._i, L._p, L._p])
L.register("ib_post_norm", [L._p, L._p, L._i, L._ll, L._p, L._p, L._p, L._f, L._p, L._i, L._p, L._i, L._i, L._p])


def embed_pos(table: torch.Tensor, tokens: torch.Tensor, pos_table: torch.Tensor, positions: torch.Tensor, scale: float, x: torch.Tensor, status: torch.Tensor) -> None:
    """x[t] = float32(table[tokens[t]]) * scale + float32(pos_table[positions[t]]): a learned vector per position beside the token's."""
    V, H = table.shape
    T = tokens.shape[0]
    _check("table", table)
    _check("pos_table", pos_table, table.dtype)
    if pos_table.shape[1] != H:
        raise L.KernelError(f"embed_pos: the position table has {pos_table.shape[1]} columns, the token table {H}")
    _check("tokens", tokens, torch.int32)
    _check("positions", positions, torch.int32, (T,))
    _check("x", x, torch.float32, (T, H))
    L.call("ib_embed_pos", table.data_ptr(), dtype_code(table.dtype), tokens.data_ptr(), pos_table.data_ptr(), positions.data_ptr(), float(scale), x.data_ptr(), T, H, V,
           pos_table.shape[0], status.data_ptr(), _stream())


def post_norm(x: torch.Tensor, delta: Optional[torch.Tensor], bias: Optional[torch.Tensor], w_post: Optional[torch.Tensor], w_next: Optional[torch.Tensor],
              out: Optional[torch.Tensor], eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """x += w_post * rms_unit(sum_p delta[p] + bias) (in place, unless `rows` gathers), then out = w_next * rms_unit(x): a sublayer's
    output through its own norm into the stream, and the next sublayer's input norm, in one kernel. delta None: no contribution;
    out None: the add alone. With `rows` (int32 [n]) output row r comes from source row rows[r] and x is left as it is."""
    T, H = x.shape
    _check("x", x, torch.float32)
    n_rows = T if rows is None else rows.shape[0]
    P, stride = 0, 0
    if delta is not None:
        _check("delta", delta, torch.float32)
        if delta.dim() != 3 or tuple(delta.shape[1:]) != (T, H):
            raise L.KernelError(f"post_norm: delta must be [P, {T}, {H}], got {tuple(delta.shape)}")
        P, stride = delta.shape[0], T * H
        _check("w_post", w_post, torch.float32, (H,))
        if bias is not None:
            _check("bias", bias, torch.float32, (H,))
    if out is not None:
        _check("out", out, None, (n_rows, H))
        _check("w_next", w_next, torch.float32, (H,))
    if rows is not None:
        _check("rows", rows, torch.int32)
    L.call("ib_post_norm", x.data_ptr(), _ptr(delta), P, stride, _ptr(bias) if delta is not None else None, _ptr(w_post), _ptr(w_next), float(eps), _ptr(out),
           dtype_code(out.dtype) if out is not None else 0, _ptr(rows), n_rows, H, _stream())


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, out: torch.Tensor, eps: float,
                rows: Optional[torch.Tensor] = None) -> None:
    """x += sum_p delta[p] (in place, unless `rows` gathers); out = w * (x * rsqrt(mean(x^2) + eps)).

    delta is None or float32 [P, T, H]; with `rows` (int32 [n]) output row r comes from source row rows[r]."""
    T, H = x.shape
    _check("x", x, torch.float32)
    _check("w", w, torch.float32, (H,))
    n_rows = T if rows is None else rows.shape[0]
    _check("out", out, None, (n_rows, H))
    P, stride = 0, 0
    if delta is not None:
        _check("delta", delta, torch.float32)
        if delta.dim() != 3 or tuple(delta.shape[1:]) != (T, H):
            raise L.KernelError(f"delta must be [P, {T}, {H}], got {tuple(delta.shape)}")
        P, stride = delta.shape[0], T * H
    if rows is not None:
        _check("rows", rows, torch.int32)
    L.call("ib_add_rmsnorm", x.data_ptr(), _ptr(delta), P, stride, w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), _ptr(rows), n_rows, H,
           float(eps), 0 if rows is not None else 1, _stream())


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    T, half = positions.shape[0], inv_freq.shape[0]
    _check("positions", positions, torch.int32)
    _check("inv_freq", inv_freq, torch.float32)
    _check("cos", cos, torch.float32, (T, half))
    _check("sin", sin, torch.float32, (T, half))
    L.call("ib_rope_table", positions.data_ptr(), inv_freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, half, _stream())


def silu_mul(gate_up: torch.Tensor, act: torch.Tensor) -> None:
    """act = silu(gate) * up with gate_up float32 [P, T, 2I] = [gate | up], partials summed first."""
    _check("gate_up", gate_up, torch.float32)
    P, T, I2 = gate_up.shape
    _check("act", act, None, (T, I2 // 2))
    L.call("ib_silu_mul", gate_up.data_ptr(), P, T * I2, act.data_ptr(), dtype_code(act.dtype), T, I2 // 2, _stream())


def qk_norm_rope_kv(qkv: torch.Tensor, q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor, seg_of_token: torch.Tensor,
                    q_out: torch.Tensor, kv: KvLayerView, heads: int, status: torch.Tensor, write_kv: bool = True,
                    bias: Optional[torch.Tensor] = None, qk_dim: Optional[int] = None, v_dim: Optional[int] = None,
                    columns: Optional[tuple] = None, unit_norm_after: bool = False) -> None:
    """qkv float32 [P, T, (heads + kv_heads) * qk_dim + kv_heads * v_dim] -> q_out [T, heads * qk_dim] and the paged cache.
    qk_dim, v_dim: a query/key head's and a value head's size (default: the cache's row; neither may exceed it). bias: float32, one
    value per column of the projection, added to the summed partial products.
    columns = (q, k, v): the projection's row is wider and the three parts start at these columns; v None: the values are the keys as
    projected (bias added, no norm, no rotation). unit_norm_after: q and k are divided by their root mean square over the head after
    the rotation, without weights."""
    _check("qkv", qkv, torch.float32)
    P, T, R = qkv.shape
    view = kv.c_view()
    qk_dim, v_dim = qk_dim or view.head_dim, v_dim or view.head_dim
    if columns is None and R != (heads + view.kv_heads) * qk_dim + view.kv_heads * v_dim:
        raise L.KernelError(f"qkv has {R} columns, expected {(heads + view.kv_heads) * qk_dim + view.kv_heads * v_dim}")
    row, q_col, k_col, v_col = (0, 0, 0, 0) if columns is None else (R, int(columns[0]), int(columns[1]), -1 if columns[2] is None else int(columns[2]))
    _check("q_out", q_out, None, (T, heads * qk_dim))
    if bias is not None:
        _check("bias", bias, torch.float32, (R,))
    _check("positions", positions, torch.int32, (T,))
    _check("seg_of_token", seg_of_token, torch.int32, (T,))
    rot_half = 0
    if cos is not None:
        rot_half = cos.shape[1]
        _check("cos", cos, torch.float32, (T, rot_half))
        _check("sin", sin, torch.float32, (T, rot_half))
    for name, w in (("q_norm", q_norm_w), ("k_norm", k_norm_w)):
        if w is not None:
            _check(name, w, torch.float32, (view.head_dim,))
    L.call("ib_qk_norm_rope_kv", qkv.data_ptr(), P, T * R, _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(cos), _ptr(sin), rot_half,
           positions.data_ptr(), seg_of_token.data_ptr(), q_out.data_ptr(), dtype_code(q_out.dtype), C.byref(view), 1 if write_kv else 0, T,
           heads, status.data_ptr(), _ptr(bias), qk_dim, v_dim, row, q_col, k_col, v_col, 1 if unit_norm_after else 0, _stream())


def attention_generic(q: torch.Tensor, kv: KvLayerView, positions: torch.Tensor, seg_of_token: torch.Tensor, window: Optional[int],
                      scale: float, out: torch.Tensor, heads: int, status: torch.Tensor, qk_dim: Optional[int] = None, v_dim: Optional[int] = None,
                      softcap: float = 0.0, sink: bool = False, chunk: int = 0, sink_values: Optional[torch.Tensor] = None,
                      gate: Optional[tuple] = None, out_scale: float = 1.0) -> None:
    """softcap > 0: scores become softcap * tanh(score / softcap); sink: the softmax's denominator has one added (a key of score 0
    without a value; with sink_values, float32 [heads], a key of that score per head); qk_dim, v_dim: a query/key head's and a value
    head's size (default: the cache's row). chunk > 0: a position sees the earlier positions of its own block of `chunk` positions
    (counted from 0) instead of a window. gate = (float32 partial sums [P, T, row], column of the first head): head h's output is
    multiplied by the sigmoid of its column. out_scale multiplies the output. out may be wider than heads * v_dim (a row of a larger
    buffer whose first columns are written)."""
    view = kv.c_view()
    T = q.shape[0]
    qk_dim, v_dim = qk_dim or view.head_dim, v_dim or view.head_dim
    _check("q", q, None, (T, heads * qk_dim))
    _check("out", out, q.dtype)
    if out.dim() != 2 or out.shape[0] != T or out.shape[1] < heads * v_dim:
        raise L.KernelError(f"attention_generic: out must be [{T}, >= {heads * v_dim}], got {tuple(out.shape)}")
    if sink_values is not None:
        _check("sink_values", sink_values, torch.float32, (heads,))
    g_ptr, g_P, g_stride, g_row = None, 0, 0, 0
    if gate is not None:
        g, col = gate
        _check("gate", g, torch.float32)
        g_P, g_row = g.shape[0], g.shape[2]
        if g.shape[1] != T or col + heads > g_row:
            raise L.KernelError(f"attention_generic: the gate's partial sums {tuple(g.shape)} do not hold {heads} columns from {col} for {T} tokens")
        g_ptr, g_stride = g.data_ptr() + 4 * col, T * g_row
    _check("positions", positions, torch.int32, (T,))
    _check("seg_of_token", seg_of_token, torch.int32, (T,))
    L.call("ib_attention_generic", q.data_ptr(), dtype_code(q.dtype), C.byref(view), positions.data_ptr(), seg_of_token.data_ptr(),
           int(window or 0), float(scale), out.data_ptr(), T, heads, status.data_ptr(), qk_dim, v_dim, float(softcap or 0.0), 1 if sink else 0,
           int(chunk or 0), _ptr(sink_values), g_ptr, g_P, g_stride, g_row, float(out_scale), out.shape[1], _stream())


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, n] = sum_k x[t, k] w[n, k], float32 FMA."""
    T, K = x.shape
    N = w.shape[0]
    _check("x", x)
    _check("w", w, None, (N, K))
    _check("out", out, torch.float32, (T, N))
    L.call("ib_gemm_simt", x.data_ptr(), dtype_code(x.dtype), w.data_ptr(), dtype_code(w.dtype), out.data_ptr(), T, N, K, _stream())


def sample_chunks(vocab: int) -> int:
    return int(L.load().ib_sample_chunks(int(vocab)))


def sample_rows(logits: torch.Tensor, params: torch.Tensor, tokens: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """params int32 [rows, 6] = (inv_temp bits, seed, step, top_k, top_p bits, min_p bits). With `status` (the
    device status word) tokens has rows + 1 entries and the last one receives the word's value, so one
    transfer brings the host both the tokens and whether a kernel of the step reported a fault."""
    rows, V = logits.shape
    _check("logits", logits, torch.float32)
    _check("params", params, torch.int32, (rows, 6))
    _check("tokens", tokens, torch.int32, (rows + (1 if status is not None else 0),))
    scratch = torch.empty(rows * (1 + 2 * sample_chunks(V)), dtype=torch.float32, device=logits.device)
    L.call("ib_sample_rows", logits.data_ptr(), rows, V, params.data_ptr(), tokens.data_ptr(), scratch.data_ptr(), _ptr(status), _stream())


def advance_rows(sampled: torch.Tensor, token_in: torch.Tensor, positions: torch.Tensor, pos0: torch.Tensor, params: torch.Tensor,
                 history: torch.Tensor, count: torch.Tensor) -> None:
    """Feed sampled tokens back as the next inputs of a decode batch and log them: history[count, :] = sampled."""
    rows = sampled.shape[0]
    for name, t in (("sampled", sampled), ("token_in", token_in), ("positions", positions), ("pos0", pos0)):
        _check(name, t, torch.int32, (rows,))
    _check("params", params, torch.int32, (rows, 6))
    _check("history", history, torch.int32)
    _check("count", count, torch.int32, (1,))
    L.call("ib_advance_rows", sampled.data_ptr(), token_in.data_ptr(), positions.data_ptr(), pos0.data_ptr(), params.data_ptr(), history.data_ptr(),
           count.data_ptr(), rows, history.shape[0], _stream())


# ---------------------------------------------------------------- norm on a sublayer's output
L.register("ib_norm_residual", [L._p, L._p, L._i, L._ll, L._p, L._f, L._f, L._p, L._i, L._i, L._i, L._p])
L.register("ib_cast_rows", [L._p, L._p, L._i, L._ll, L._p])


def norm_residual(x: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, mult: float, eps: float, act: Optional[torch.Tensor]) -> None:
    """x += mult * w * (y * rsqrt(mean(y^2) + eps)) with y = sum_p delta[p] (float32 [P, T, H]); act (optional, [T, H]) = the new x
    in act's dtype."""
    T, H = x.shape
    _check("x", x, torch.float32)
    _check("w", w, torch.float32, (H,))
    _check("delta", delta, torch.float32)
    if delta.dim() != 3 or tuple(delta.shape[1:]) != (T, H):
        raise L.KernelError(f"delta must be [P, {T}, {H}], got {tuple(delta.shape)}")
    if act is not None:
        _check("act", act, None, (T, H))
    L.call("ib_norm_residual", x.data_ptr(), delta.data_ptr(), delta.shape[0], T * H, w.data_ptr(), float(mult), float(eps), _ptr(act),
           dtype_code(act.dtype) if act is not None else L.F32, T, H, _stream())


def cast_rows(x: torch.Tensor, act: torch.Tensor) -> None:
    """act = x (float32) in act's dtype."""
    _check("x", x, torch.float32)
    _check("act", act, None, tuple(x.shape))
    L.call("ib_cast_rows", x.data_ptr(), act.data_ptr(), dtype_code(act.dtype), x.numel(), _stream())


# ---------------------------------------------------------------- latent attention (csrc/latent_attention.cu)
L.register("ib_latent_prepare", [L._p, L._i, L._ll, L._i, L._p, L._f, L._p, L._p, L._i, L._p, L._p, L._p, L._i, L._p, C.POINTER(L.KvView), L._i, L._i, L._i, L._i,
                                 L._i, L._i, L._p, L._p])
L.register("ib_gemm_heads", [L._p, L._i, L._ll, L._ll, L._p, L._i, L._p, L._i, L._ll, L._ll, L._i, L._i, L._i, L._i, L._p, L._i, L._ll, L._i, L._p])
L.register("ib_latent_attention", [L._p, C.POINTER(L.KvView), L._p, L._p, L._f, L._p, L._i, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._p, L._i, L._p])
L.register("ib_latent_down", [L._p, L._i, L._ll, L._i, L._i, L._p, L._p, L._i, L._p, L._f, L._p, L._p, L._i, L._p, L._p, C.POINTER(L.KvView), L._i, L._i, L._i, L._p, L._p])
L.KERNELS_PER_CALL["ib_latent_attention"] = 1   # two with slices; counted by the caller


def latent_prepare(qd: torch.Tensor, c_norm_w: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                   positions: torch.Tensor, seg_of_token: torch.Tensor, q_nope: torch.Tensor, q_full: torch.Tensor, kv: KvLayerView, heads: int, dim: int,
                   rot: int, rank: int, write_kv: bool, status: torch.Tensor) -> None:
    """qd float32 [P, T, heads * (dim + rot) (+ rank + rot)]: partial sums of the fused [q | dkv] projection.
    -> q_nope [T, heads, dim] (activation dtype), q_full[..., rank:] float32 [T, heads, rank + rot] (rotated part), and with
    write_kv the token's cache row [normed latent | rotated key part]."""
    _check("qd", qd, torch.float32)
    P, T, R = qd.shape
    _check("q_nope", q_nope, None, (T, heads, dim))
    _check("q_full", q_full, torch.float32, (T, heads, rank + rot))
    _check("positions", positions, torch.int32, (T,))
    _check("seg_of_token", seg_of_token, torch.int32, (T,))
    rot_half = 0
    if cos is not None:
        rot_half = cos.shape[1]
        _check("cos", cos, torch.float32, (T, rot_half))
        _check("sin", sin, torch.float32, (T, rot_half))
    if c_norm_w is not None:
        _check("c_norm_w", c_norm_w, torch.float32, (rank,))
    view = kv.c_view()
    L.call("ib_latent_prepare", qd.data_ptr(), P, T * R, R, _ptr(c_norm_w), float(eps), _ptr(cos), _ptr(sin), rot_half, positions.data_ptr(),
           seg_of_token.data_ptr(), q_nope.data_ptr(), dtype_code(q_nope.dtype), q_full.data_ptr(), C.byref(view), 1 if write_kv else 0, T, heads, dim,
           rot, rank, status.data_ptr(), _stream())


L.register("ib_gemm_grouped_mma", [L._p, L._p, L._p, L._p, L._i, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._p])
L.register("ib_gemm_heads_mma", [L._p, L._ll, L._ll, L._p, L._p, L._i, L._ll, L._ll, L._i, L._i, L._i, L._i, L._p, L._i, L._ll, L._i, L._p])


def latent_down(qd: torch.Tensor, q_rank: int, q_norm_w: torch.Tensor, cq: torch.Tensor, c_norm_w: torch.Tensor, eps: float, cos: Optional[torch.Tensor],
                sin: Optional[torch.Tensor], positions: torch.Tensor, seg_of_token: torch.Tensor, kv: KvLayerView, rank: int, rot: int, status: torch.Tensor) -> None:
    """qd float32 [P, T, >= q_rank + rank + rot]: partial sums of a layer's first product [query latent | latent | key part | ...].
    -> cq [T, q_rank] (activation dtype): the normed query latent, and the token's cache row [normed latent | rotated key part]."""
    _check("qd", qd, torch.float32)
    P, T, R = qd.shape
    _check("cq", cq, None, (T, q_rank))
    _check("q_norm_w", q_norm_w, torch.float32, (q_rank,))
    _check("c_norm_w", c_norm_w, torch.float32, (rank,))
    _check("positions", positions, torch.int32, (T,))
    _check("seg_of_token", seg_of_token, torch.int32, (T,))
    rot_half = 0
    if cos is not None:
        rot_half = cos.shape[1]
        _check("cos", cos, torch.float32, (T, rot_half))
        _check("sin", sin, torch.float32, (T, rot_half))
    view = kv.c_view()
    L.call("ib_latent_down", qd.data_ptr(), P, T * R, R, int(q_rank), q_norm_w.data_ptr(), cq.data_ptr(), dtype_code(cq.dtype), c_norm_w.data_ptr(), float(eps),
           _ptr(cos), _ptr(sin), rot_half, positions.data_ptr(), seg_of_token.data_ptr(), C.byref(view), int(rank), int(rot), T, status.data_ptr(), _stream())


def rows_mma_fits(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core kernel for products on row groups takes these operands: bfloat16, an inner size that is a multiple of 8."""
    return x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def gemm_heads(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n: int, tensor_cores: bool = False, gate: Optional[tuple] = None) -> None:
    """out[t, b, :n] = w[b] x[t, b] for every head b: x [T, heads, K] (contiguous), w [heads, N, K], out [T, heads, >= n] whose
    first n columns of every head are written (the rest stay). tensor_cores: the m16n8k16 kernel (see `rows_mma_fits`).
    gate = (float32 partial sums [P, T, row], column of the first head): head b's output is multiplied by the sigmoid of its column."""
    T, heads, K = x.shape
    g_ptr, g_P, g_stride, g_row = None, 0, 0, 0
    if gate is not None:
        g, col = gate
        _check("gate", g, torch.float32)
        g_P, g_row = g.shape[0], g.shape[2]
        if g.dim() != 3 or g.shape[1] != T or col + heads > g_row:
            raise L.KernelError(f"gemm_heads: the gate's partial sums {tuple(g.shape)} do not hold {heads} columns from {col} for {T} tokens")
        g_ptr, g_stride = g.data_ptr() + 4 * col, T * g_row
    _check("x", x)
    _check("w", w, None, (heads, n, K))
    _check("out", out)
    if out.dim() != 3 or out.shape[0] != T or out.shape[1] != heads or out.shape[2] < n:
        raise L.KernelError(f"gemm_heads: out must be [{T}, {heads}, >= {n}], got {tuple(out.shape)}")
    if tensor_cores:
        if not rows_mma_fits(x, w):
            raise L.KernelError("gemm_heads: the tensor-core kernel needs bfloat16 operands with an inner size that is a multiple of 8")
        L.call("ib_gemm_heads_mma", x.data_ptr(), heads * K, K, w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), heads * out.shape[2], out.shape[2], T, heads, n, K,
               g_ptr, g_P, g_stride, g_row, _stream())
        return
    L.call("ib_gemm_heads", x.data_ptr(), dtype_code(x.dtype), heads * K, K, w.data_ptr(), dtype_code(w.dtype), out.data_ptr(), dtype_code(out.dtype),
           heads * out.shape[2], out.shape[2], T, heads, n, K, g_ptr, g_P, g_stride, g_row, _stream())


def latent_attention(q_full: torch.Tensor, kv: KvLayerView, positions: torch.Tensor, seg_of_token: torch.Tensor, scale: float, out: torch.Tensor, rank: int,
                     n_slices: int, slice_keys: int, scratch, status: torch.Tensor, window: Optional[int] = None) -> None:
    """q_full float32 [T, heads, row] against the cached rows [latent (rank) | key part]: out [T, heads, rank] = softmax-weighted sum of
    the latents of the keys a token sees (all up to its own position, or with `window` itself and the window - 1 before it; the slices
    then cut that range). scratch: (part_o, part_ml) float32 when n_slices > 1."""
    T, heads, D = q_full.shape
    _check("q_full", q_full, torch.float32)
    _check("out", out, None, (T, heads, rank))
    _check("positions", positions, torch.int32, (T,))
    _check("seg_of_token", seg_of_token, torch.int32, (T,))
    view = kv.c_view()
    if view.head_dim != D:
        raise L.KernelError(f"latent_attention: queries have {D} values, cache rows {view.head_dim}")
    part_o, part_ml = scratch if scratch is not None else (None, None)
    if n_slices > 1:
        _check("part_o", part_o, torch.float32)
        _check("part_ml", part_ml, torch.float32)
        if part_o.numel() < T * heads * n_slices * rank or part_ml.numel() < T * heads * n_slices * 2:
            raise L.KernelError("latent_attention: the scratch for the slices is too small")
        L.launches += 1
    L.call("ib_latent_attention", q_full.data_ptr(), C.byref(view), positions.data_ptr(), seg_of_token.data_ptr(), float(scale), out.data_ptr(),
           dtype_code(out.dtype), _ptr(part_o), _ptr(part_ml), T, heads, rank, n_slices, slice_keys, status.data_ptr(), int(window or 0), _stream())


L.register("ib_latent_attention_mma", [L._p, C.POINTER(L.KvView), L._p, L._p, L._p, L._i, L._i, L._f, L._p, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._p, L._i, L._p])


def latent_attention_mma_rows(rank: int, row: int, rows_wanted: int) -> int:
    """Query rows a CTA of the tensor-core kernel holds (16, 32 or 64) when `rows_wanted` rows of a step can share key tiles."""
    return int(L.load().ib_latent_attention_mma_rows(int(rank), int(row), int(rows_wanted)))


def latent_attention_mma_supports(rank: int, row: int) -> bool:
    return bool(L.load().ib_latent_attention_mma_supports(int(rank), int(row)))


def latent_attention_mma(q_full: torch.Tensor, kv: KvLayerView, positions: torch.Tensor, seg_of_token: torch.Tensor, units: Optional[torch.Tensor], scale: float,
                         out: torch.Tensor, rank: int, n_slices: int, slice_keys: int, scratch, status: torch.Tensor, rows: int = 16,
                         window: Optional[int] = None) -> None:
    """The same as `latent_attention` on the tensor cores (bfloat16 cache and output). rows: query rows a CTA holds (16, 32 or 64).
    units: None (a CTA per token) or int32 [n, 2] of (first token, tokens): runs of consecutive tokens of one request that share a
    CTA's rows (at most rows // heads tokens each)."""
    T, heads, D = q_full.shape
    _check("q_full", q_full, torch.float32)
    _check("out", out, torch.bfloat16, (T, heads, rank))
    _check("positions", positions, torch.int32, (T,))
    _check("seg_of_token", seg_of_token, torch.int32, (T,))
    view = kv.c_view()
    if view.head_dim != D:
        raise L.KernelError(f"latent_attention_mma: queries have {D} values, cache rows {view.head_dim}")
    n_units = T
    if units is not None:
        _check("units", units, torch.int32)
        n_units = units.shape[0]
    part_o, part_ml = scratch if scratch is not None else (None, None)
    if n_slices > 1:
        if part_o.numel() < T * heads * n_slices * rank or part_ml.numel() < T * heads * n_slices * 2:
            raise L.KernelError("latent_attention_mma: the scratch for the slices is too small")
        L.launches += 1
    L.call("ib_latent_attention_mma", q_full.data_ptr(), C.byref(view), positions.data_ptr(), seg_of_token.data_ptr(), _ptr(units), n_units, int(rows), float(scale),
           out.data_ptr(), _ptr(part_o), _ptr(part_ml), T, heads, rank, n_slices, slice_keys, status.data_ptr(), int(window or 0), _stream())


# ---------------------------------------------------------------- routed experts (csrc/moe.cu)
L.register("ib_moe_route", [L._p, L._i, L._ll, L._i, L._i, L._i, L._i, L._i, L._f, L._i, L._p, L._p, L._i, L._p, L._i, L._p])
L.register("ib_scatter_scaled_rows", [L._p, L._i, L._p, L._p, L._i, L._p, L._i, L._i, L._p])
L.register("ib_moe_sort", [L._p, L._i, L._i, L._i, L._i, L._p, L._p, L._p, L._p, L._p])
L.register("ib_gather_rows", [L._p, L._p, L._p, L._i, L._i, L._i, L._p])


def moe_tile_rows() -> int:
    """Rows of a tile of the FMA and m16n8k16 kernels for regrouped rows."""
    return int(L.load().ib_moe_tile_rows())


def gather_rows(x: torch.Tensor, src_row: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = x[src_row[r]] (rows of a multiple of 16 bytes)."""
    R, K = out.shape
    _check("x", x, out.dtype)
    _check("out", out)
    _check("src_row", src_row, torch.int32, (R,))
    if x.shape[1] != K:
        raise L.KernelError(f"gather_rows: x has {x.shape[1]} columns, out {K}")
    L.call("ib_gather_rows", x.data_ptr(), src_row.data_ptr(), out.data_ptr(), R, K, x.element_size(), _stream())
L.register("ib_gemm_grouped", [L._p, L._i, L._p, L._p, L._i, L._p, L._i, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._p])
L.register("ib_moe_combine", [L._p, L._p, L._p, L._i, L._p, L._i, L._ll, L._p, L._i, L._i, L._p])


def moe_route(logits: torch.Tensor, n_groups: int, keep: int, top: int, route_scale: float, renorm: bool, idx: torch.Tensor, wt: torch.Tensor,
              score: str = "softmax", correction: Optional[torch.Tensor] = None, group_top: int = 1) -> None:
    """logits float32 [P, T, E] (partial sums) -> idx int32 [T, top], wt float32 [T, top]. score: "softmax" over all experts, or
    "sigmoid" of every expert's logit on its own. correction: float32 [E] added to the scores where groups and experts are chosen (the
    weights are the scores without it). group_top: a group's score is the sum of its `group_top` largest choice scores (1: the largest)."""
    if score not in ("softmax", "sigmoid"):
        raise L.KernelError(f"moe_route: score {score!r} is not known (softmax, sigmoid)")
    _check("logits", logits, torch.float32)
    P, T, E = logits.shape
    _check("idx", idx, torch.int32, (T, top))
    _check("wt", wt, torch.float32, (T, top))
    if correction is not None:
        _check("correction", correction, torch.float32, (E,))
    L.call("ib_moe_route", logits.data_ptr(), P, T * E, T, E, n_groups, keep, top, float(route_scale), 1 if renorm else 0, idx.data_ptr(), wt.data_ptr(),
           1 if score == "sigmoid" else 0, _ptr(correction), int(group_top), _stream())


def moe_sort(idx: torch.Tensor, n_experts: int, offsets: torch.Tensor, tile_start: torch.Tensor, row_of_pair: torch.Tensor, token_of_row: torch.Tensor,
             tile_rows: Optional[int] = None) -> None:
    """Regroup the step's (token, choice) pairs by expert: offsets[e] .. offsets[e + 1] are expert e's rows, row_of_pair / token_of_row map
    between pairs and rows, tile_start[e] is expert e's first tile of `tile_rows` rows (default: the FMA and m16n8k16 kernels' 64)."""
    T, top = idx.shape
    tile_rows = tile_rows or moe_tile_rows()
    _check("idx", idx, torch.int32)
    _check("offsets", offsets, torch.int32, (n_experts + 1,))
    _check("tile_start", tile_start, torch.int32, (n_experts + 1,))
    _check("row_of_pair", row_of_pair, torch.int32, (T * top,))
    _check("token_of_row", token_of_row, torch.int32, (T * top,))
    L.call("ib_moe_sort", idx.data_ptr(), T * top, top, n_experts, int(tile_rows), offsets.data_ptr(), tile_start.data_ptr(), row_of_pair.data_ptr(), token_of_row.data_ptr(), _stream())


def gemm_grouped(x: torch.Tensor, src_row: Optional[torch.Tensor], w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor, tile_start: torch.Tensor,
                 gated: bool, tensor_cores: bool = False) -> None:
    """out[r] = w[e(r)] x[src_row[r] or r] for the regrouped rows r (expert e's rows are offsets[e]..offsets[e+1]); w [E, N or 2N, K]; with
    `gated`, w holds gate rows then up rows and out = silu(gate) * up."""
    R, N = out.shape
    E, rows_w, K = w.shape
    if rows_w != (2 * N if gated else N) or x.shape[1] != K:
        raise L.KernelError(f"gemm_grouped: w {tuple(w.shape)}, x {tuple(x.shape)}, out {tuple(out.shape)} do not fit (gated={gated})")
    _check("x", x)
    _check("w", w)
    _check("out", out)
    if src_row is not None:
        _check("src_row", src_row, torch.int32, (R,))
    if tensor_cores:
        if not rows_mma_fits(x, w):
            raise L.KernelError("gemm_grouped: the tensor-core kernel needs bfloat16 operands with an inner size that is a multiple of 8")
        L.call("ib_gemm_grouped_mma", x.data_ptr(), _ptr(src_row), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), offsets.data_ptr(), tile_start.data_ptr(), R, E,
               N, K, 1 if gated else 0, _stream())
        return
    L.call("ib_gemm_grouped", x.data_ptr(), dtype_code(x.dtype), _ptr(src_row), w.data_ptr(), dtype_code(w.dtype), out.data_ptr(), dtype_code(out.dtype),
           offsets.data_ptr(), tile_start.data_ptr(), R, E, N, K, 1 if gated else 0, _stream())


def scatter_scaled_rows(x: torch.Tensor, row_of_pair: torch.Tensor, wt: torch.Tensor, out: torch.Tensor) -> None:
    """out[row_of_pair[t * top + k]] = wt[t, k] * x[t]: the step's rows in the experts' order, each scaled by its pair's weight."""
    T, top = wt.shape
    K = x.shape[1]
    _check("x", x, out.dtype, (T, K))
    _check("out", out, None, (T * top, K))
    _check("row_of_pair", row_of_pair, torch.int32, (T * top,))
    _check("wt", wt, torch.float32)
    L.call("ib_scatter_scaled_rows", x.data_ptr(), dtype_code(x.dtype), row_of_pair.data_ptr(), wt.data_ptr(), top, out.data_ptr(), T * top, K, _stream())


def moe_combine(y: torch.Tensor, row_of_pair: torch.Tensor, wt: torch.Tensor, base: Optional[torch.Tensor], out: torch.Tensor, weighted: bool = True) -> None:
    """out[t] = sum_p base[p][t] + sum_k wt[t, k] * y[row_of_pair[t * top + k]]; y float32 [R, H], base float32 [P, T, H] or None.
    weighted=False: the plain sum over a token's choices (wt gives the shape only)."""
    T, top = wt.shape
    H = y.shape[1]
    _check("y", y, torch.float32, (T * top, H))
    _check("out", out, torch.float32, (T, H))
    P = 0
    if base is not None:
        _check("base", base, torch.float32)
        if base.dim() != 3 or tuple(base.shape[1:]) != (T, H):
            raise L.KernelError(f"moe_combine: base must be [P, {T}, {H}], got {tuple(base.shape)}")
        P = base.shape[0]
    L.call("ib_moe_combine", y.data_ptr(), row_of_pair.data_ptr(), wt.data_ptr() if weighted else None, top, _ptr(base), P, T * H, out.data_ptr(), T, H, _stream())


# ---------------------------------------------------------------- layer norm, input convolution, depth average (csrc/layernorm.cu)
L.register("ib_add_layernorm", [L._p, L._p, L._i, L._ll, L._p, L._p, L._p, L._p, L._i, L._p, L._i, L._i, L._f, L._i, L._p, L._i, L._p, L._p, L._p, L._i, L._p, L._ll, L._p])
L.register("ib_causal_conv_rows", [L._p, L._p, L._i, L._p, L._i, L._i, L._i, L._p, L._p, L._p, L._i, L._p, L._ll, L._p])
L.register("ib_depth_average", [L._p, L._p, L._i, L._ll, L._p, L._p, L._p, L._ll, L._i, L._p, L._i, L._i, L._p])
L.register("ib_scale_values", [L._p, L._ll, L._f, L._p])


@dataclass
class ConvLayout:
    """Where `add_layernorm` puts its rows for the convolution over time that follows: every segment's rows preceded by `halo` rows
    of the request's state (its last normed rows of earlier steps). state: float32 [slots, halo, H] (a view of one sublayer's part)."""
    halo: int
    seg_of_token: torch.Tensor
    seg_start: torch.Tensor
    seg_slot: torch.Tensor
    n_segments: int
    state: torch.Tensor
    slot_stride: int        # float32 values between the states of consecutive slots

    def rows(self, T: int) -> int:
        return T + self.halo * self.n_segments


def add_layernorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                  delta_scale: Optional[torch.Tensor] = None, delta_bias: Optional[torch.Tensor] = None, x_copy: Optional[torch.Tensor] = None,
                  layout: Optional[ConvLayout] = None) -> None:
    """v = x + delta_scale * (sum_p delta[p] + delta_bias) (x updated in place unless `rows` gathers); x_copy = v (optional);
    out = w * (v - mean) / sqrt(var + eps). With `layout` out is float32 [T + halo * segments, H] in the layout of `ConvLayout`."""
    T, H = x.shape
    _check("x", x, torch.float32)
    _check("w", w, torch.float32, (H,))
    n_rows = T if rows is None else rows.shape[0]
    _check("out", out, torch.float32 if layout else None, (layout.rows(T) if layout else n_rows, H))
    P, stride = 0, 0
    if delta is not None:
        _check("delta", delta, torch.float32)
        if delta.dim() != 3 or tuple(delta.shape[1:]) != (T, H):
            raise L.KernelError(f"delta must be [P, {T}, {H}], got {tuple(delta.shape)}")
        P, stride = delta.shape[0], T * H
    for name, v in (("delta_scale", delta_scale), ("delta_bias", delta_bias)):
        if v is not None:
            _check(name, v, torch.float32, (H,))
    if x_copy is not None:
        _check("x_copy", x_copy, torch.float32, (T, H))
    if rows is not None:
        _check("rows", rows, torch.int32)
    lay = layout
    L.call("ib_add_layernorm", x.data_ptr(), _ptr(delta), P, stride, _ptr(delta_scale), _ptr(delta_bias), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
           _ptr(rows), n_rows, H, float(eps), 0 if rows is not None else 1, _ptr(x_copy), lay.halo if lay else 0, _ptr(lay.seg_of_token) if lay else None,
           _ptr(lay.seg_start) if lay else None, _ptr(lay.seg_slot) if lay else None, lay.n_segments if lay else 0, _ptr(lay.state) if lay else None,
           lay.slot_stride if lay else 0, _stream())


def causal_conv_rows(ext: torch.Tensor, w: torch.Tensor, out: torch.Tensor, layout: ConvLayout) -> None:
    """out[t] = h[t] + sum_j w[j] h[t - taps + 1 + j] over a request's rows (ext: the normed rows in the layout of `ConvLayout`, taps =
    halo + 1, w float32 [taps, H]: a tap's weights for all channels lie together); the request's state becomes the last `halo` rows of its run."""
    T, H = out.shape
    _check("ext", ext, torch.float32, (layout.rows(T), H))
    _check("w", w, torch.float32, (layout.halo + 1, H))
    _check("out", out)
    L.call("ib_causal_conv_rows", ext.data_ptr(), w.data_ptr(), layout.halo + 1, out.data_ptr(), dtype_code(out.dtype), T, H, layout.seg_of_token.data_ptr(),
           layout.seg_start.data_ptr(), layout.seg_slot.data_ptr(), layout.n_segments, layout.state.data_ptr(), layout.slot_stride, _stream())


L.register("ib_add_layernorm_conv_single", [L._p, L._p, L._i, L._ll, L._p, L._p, L._p, L._f, L._p, L._p, L._i, L._p, L._i, L._i, L._i, L._p, L._p, L._ll, L._p])


def add_layernorm_conv_single(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float, conv_w: torch.Tensor, out: torch.Tensor, layout: ConvLayout,
                              delta_scale: Optional[torch.Tensor] = None, delta_bias: Optional[torch.Tensor] = None, x_copy: Optional[torch.Tensor] = None) -> None:
    """`add_layernorm` and `causal_conv_rows` in one kernel for a step whose segments all bring one token (row t is segment t): the normed row never
    leaves the CTA, and the request's state rows are shifted by one. Sums run in the order of the two kernels."""
    T, H = x.shape
    _check("x", x, torch.float32)
    _check("w", w, torch.float32, (H,))
    _check("conv_w", conv_w, torch.float32, (layout.halo + 1, H))
    _check("out", out, None, (T, H))
    if layout.n_segments != T:
        raise L.KernelError(f"add_layernorm_conv_single: {T} rows in {layout.n_segments} segments (every segment must bring one token)")
    P = 0
    if delta is not None:
        _check("delta", delta, torch.float32)
        if delta.dim() != 3 or tuple(delta.shape[1:]) != (T, H):
            raise L.KernelError(f"delta must be [P, {T}, {H}], got {tuple(delta.shape)}")
        P = delta.shape[0]
    for name, v in (("delta_scale", delta_scale), ("delta_bias", delta_bias)):
        if v is not None:
            _check(name, v, torch.float32, (H,))
    if x_copy is not None:
        _check("x_copy", x_copy, torch.float32, (T, H))
    L.call("ib_add_layernorm_conv_single", x.data_ptr(), _ptr(delta), P, T * H, _ptr(delta_scale), _ptr(delta_bias), w.data_ptr(), float(eps), _ptr(x_copy),
           conv_w.data_ptr(), layout.halo + 1, out.data_ptr(), dtype_code(out.dtype), T, H, layout.seg_slot.data_ptr(), layout.state.data_ptr(), layout.slot_stride, _stream())


def depth_average(x: torch.Tensor, delta: Optional[torch.Tensor], delta_scale: Optional[torch.Tensor], stack: torch.Tensor, k: int, mix: torch.Tensor,
                  delta_bias: Optional[torch.Tensor] = None) -> None:
    """X = x + delta_scale * (sum_p delta[p] + delta_bias); stack[k] = X; x = sum_{j <= k} mix[j] * stack[j] (in place). stack float32 [n, T, H], k >= 1."""
    T, H = x.shape
    _check("x", x, torch.float32)
    _check("stack", stack, torch.float32)
    if stack.dim() != 3 or tuple(stack.shape[1:]) != (T, H) or not 1 <= k < stack.shape[0]:
        raise L.KernelError(f"depth_average: stack must be [more than {k}, {T}, {H}], got {tuple(stack.shape)}")
    _check("mix", mix, torch.float32, (k + 1,))
    P = 0
    if delta is not None:
        _check("delta", delta, torch.float32)
        if delta.dim() != 3 or tuple(delta.shape[1:]) != (T, H):
            raise L.KernelError(f"delta must be [P, {T}, {H}], got {tuple(delta.shape)}")
        P = delta.shape[0]
    for name, v in (("delta_scale", delta_scale), ("delta_bias", delta_bias)):
        if v is not None:
            _check(name, v, torch.float32, (H,))
    L.call("ib_depth_average", x.data_ptr(), _ptr(delta), P, T * H, _ptr(delta_scale), _ptr(delta_bias), stack.data_ptr(), T * H, k, mix.data_ptr(), T, H, _stream())


def scale_values(v: torch.Tensor, s: float) -> None:
    """v *= s, float32, in place."""
    _check("v", v, torch.float32)
    L.call("ib_scale_values", v.data_ptr(), v.numel(), float(s), _stream())


# ---------------------------------------------------------------- gated linear recurrence (csrc/gated_recurrence.cu)
L.register("ib_gated_recurrence", [L._p, L._i, L._ll, L._p, L._p, L._p, L._ll, L._p, L._p, L._i, L._p, L._i, L._i, L._i, L._p, L._p, L._p, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._p])
L.register("ib_recurrence_chunks_finish", [L._p, L._i, L._p, L._i, L._p, L._p, L._ll, L._p, L._p, L._p, L._p, L._i, L._i, L._i, L._p])
L.KERNELS_PER_CALL["ib_recurrence_chunks_finish"] = 2
RECURRENCE_CHUNK = 64   # rows of a chunk of the chunked form (csrc/gated_recurrence.cu: chunk_apply takes 64 rows a CTA)
L.register("ib_head_rmsnorm", [L._p, L._p, L._f, L._p, L._i, L._ll, L._i, L._p])


def gated_recurrence(proj: torch.Tensor, f_bias: torch.Tensor, lower: torch.Tensor, state: torch.Tensor, seg_start: torch.Tensor, seg_slot: torch.Tensor,
                     n_segments: int, out: torch.Tensor, heads: int, dim: int, vdim: int, seg_list: Optional[torch.Tensor] = None,
                     long_segs: Optional[torch.Tensor] = None, chunks: Optional[torch.Tensor] = None, fixed_decay: bool = False,
                     columns: Optional[tuple] = None) -> None:
    """proj float32 [P, T, heads * (2 dim + vdim)] = partial sums of [q | f | v]; state float32 [slots, heads, dim, vdim], advanced in place for the
    step's segments; out float32 [T, heads, vdim] = S^T q after every token.
    fixed_decay: the other form, S <- decay_head S + k v^T with q, k, v = silu of the columns [q | k | v]; `lower` then holds one decay a head
    (float32 [heads]) and f_bias is not read. columns = (q, k or f, v): the projection's row is wider and the parts start there.
    seg_list (int32 [n]): walk only these segments, token by token. long_segs (int32 [n, 3] of (segment, first chunk, chunks)) with chunks
    (int32 [m, 2] of (first row, rows <= RECURRENCE_CHUNK)): these segments in the chunked form instead (every chunk alone from a zero
    state, then the states carried from chunk to chunk, then each chunk's incoming state applied to its rows)."""
    _check("proj", proj, torch.float32)
    P, T, R = proj.shape
    if columns is None and R != heads * (2 * dim + vdim):
        raise L.KernelError(f"gated_recurrence: the projection has {R} columns, expected {heads * (2 * dim + vdim)}")
    if fixed_decay:
        _check("lower", lower, torch.float32, (heads,))
    else:
        _check("f_bias", f_bias, torch.float32, (heads * dim,))
        _check("lower", lower, torch.float32, (heads * dim,))
    form = (1 if fixed_decay else 0, 0, 0, 0, 0) if columns is None else (1 if fixed_decay else 0, R, int(columns[0]), int(columns[1]), int(columns[2]))
    _check("state", state, torch.float32)
    if tuple(state.shape[1:]) != (heads, dim, vdim):
        raise L.KernelError(f"gated_recurrence: the state must be [slots, {heads}, {dim}, {vdim}], got {tuple(state.shape)}")
    _check("out", out, torch.float32, (T, heads, vdim))
    _check("seg_start", seg_start, torch.int32)
    _check("seg_slot", seg_slot, torch.int32)
    common = (proj.data_ptr(), P, T * R, _ptr(f_bias), lower.data_ptr(), state.data_ptr(), heads * dim * vdim, seg_start.data_ptr(), seg_slot.data_ptr())
    if long_segs is None:
        if seg_list is not None:
            _check("seg_list", seg_list, torch.int32)
            n_segments = seg_list.shape[0]
        L.call("ib_gated_recurrence", *common, n_segments, out.data_ptr(), heads, dim, vdim, _ptr(seg_list), None, None, None, None, *form, _stream())
        return
    _check("long_segs", long_segs, torch.int32)
    _check("chunks", chunks, torch.int32)
    if seg_list is not None and seg_list.shape[0]:
        L.call("ib_gated_recurrence", *common, seg_list.shape[0], out.data_ptr(), heads, dim, vdim, seg_list.data_ptr(), None, None, None, None, *form, _stream())
    m = chunks.shape[0]
    chunk_state = torch.empty((m, heads, dim, vdim), dtype=torch.float32, device=proj.device)
    chunk_decay = torch.empty((m, heads, dim), dtype=torch.float32, device=proj.device)
    qa = torch.empty((T, heads, dim), dtype=torch.float32, device=proj.device)
    L.call("ib_gated_recurrence", *common, m, out.data_ptr(), heads, dim, vdim, None, chunks.data_ptr(), chunk_state.data_ptr(), chunk_decay.data_ptr(), qa.data_ptr(),
           *form, _stream())
    L.call("ib_recurrence_chunks_finish", long_segs.data_ptr(), long_segs.shape[0], chunks.data_ptr(), m, seg_slot.data_ptr(), state.data_ptr(), heads * dim * vdim,
           chunk_state.data_ptr(), chunk_decay.data_ptr(), qa.data_ptr(), out.data_ptr(), heads, dim, vdim, _stream())


def head_rmsnorm(o: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[t, a, :] = w * o[t, a, :] / sqrt(mean(o[t, a, :]^2) + eps); o float32 [T, heads, V], out [T, heads * V] in its own dtype."""
    T, heads, V = o.shape
    _check("o", o, torch.float32)
    _check("w", w, torch.float32, (V,))
    _check("out", out, None, (T, heads * V))
    L.call("ib_head_rmsnorm", o.data_ptr(), w.data_ptr(), float(eps), out.data_ptr(), dtype_code(out.dtype), T * heads, V, _stream())


# ---------------------------------------------------------------- token shift, loop entry, gated norm, xIELU (csrc/token_shift.cu)
L.register("ib_token_shift_rows", [L._p, L._p, L._p, L._ll, L._p, L._p, L._p, L._p, L._i, L._i, L._i, L._p])
L.register("ib_add_rmsnorm_ext", [L._p, L._p, L._i, L._ll, L._p, L._p, L._f, L._p, L._p, L._ll, L._p, L._p, L._i, L._i, L._i, L._p])
L.register("ib_loop_pack", [L._p, L._p, L._i, L._ll, L._p, L._p, L._p, L._i, L._i, L._i, L._p])
L.register("ib_add_bias_rows", [L._p, L._p, L._i, L._i, L._p])
L.register("ib_xielu_rows", [L._p, L._i, L._ll, L._p, L._p, L._i, L._i, L._i, L._p])
L.register("ib_gated_rmsnorm", [L._p, L._p, L._f, L._p, L._i, L._ll, L._i, L._f, L._p, L._i, L._i, L._i, L._i, L._p])


def _delta(x: torch.Tensor, delta: Optional[torch.Tensor]) -> tuple:
    """(pointer, partial sums, stride) of float32 partial sums [P, T, H] that belong to the rows of x [T, H]."""
    if delta is None:
        return None, 0, 0
    T, H = x.shape
    _check("delta", delta, torch.float32)
    if delta.dim() != 3 or tuple(delta.shape[1:]) != (T, H):
        raise L.KernelError(f"delta must be [P, {T}, {H}], got {tuple(delta.shape)}")
    return delta.data_ptr(), delta.shape[0], T * H


def token_shift_rows(h: torch.Tensor, mix: torch.Tensor, state: torch.Tensor, seg_of_token: torch.Tensor, seg_start: torch.Tensor, seg_slot: torch.Tensor,
                     out: torch.Tensor) -> None:
    """out[t] = h[t] + (h[t - 1] - h[t]) * mix per channel; the row before a segment's first is state[slot] (float32 [slots, H]), which then
    becomes the segment's last row of h. h float32 [T, H]."""
    T, H = h.shape
    _check("h", h, torch.float32)
    _check("mix", mix, torch.float32, (H,))
    _check("state", state, torch.float32)
    _check("out", out, None, (T, H))
    L.call("ib_token_shift_rows", h.data_ptr(), mix.data_ptr(), state.data_ptr(), state.stride(0), seg_of_token.data_ptr(), seg_start.data_ptr(), seg_slot.data_ptr(),
           out.data_ptr(), dtype_code(out.dtype), T, H, _stream())


def add_rmsnorm_ext(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                    shift: Optional[tuple] = None) -> None:
    """x += sum_p delta[p] + bias (in place); out = w * x / sqrt(mean(x^2) + eps). shift = (mix, state, seg_slot) for a step whose row t is
    segment t: out = h + (state[slot] - h) * mix with h the normed row, which becomes the new state."""
    T, H = x.shape
    _check("x", x, torch.float32)
    _check("w", w, torch.float32, (H,))
    _check("out", out, None, (T, H))
    d_ptr, P, stride = _delta(x, delta)
    if bias is not None:
        _check("bias", bias, torch.float32, (H,))
    mix = state = slots = None
    if shift is not None:
        mix, state, slots = shift
        _check("mix", mix, torch.float32, (H,))
        _check("state", state, torch.float32)
        _check("seg_slot", slots, torch.int32)
    L.call("ib_add_rmsnorm_ext", x.data_ptr(), d_ptr, P, stride, _ptr(bias), w.data_ptr(), float(eps), _ptr(mix), _ptr(state), state.stride(0) if state is not None else 0,
           _ptr(slots), out.data_ptr(), dtype_code(out.dtype), T, H, _stream())


def loop_pack(x: torch.Tensor, delta: Optional[torch.Tensor], x0: torch.Tensor, step: torch.Tensor, packed: torch.Tensor) -> None:
    """packed[t] = [x[t] + sum_p delta[p][t] | x0[t]] in packed's dtype; then x[t] = step (float32 [H])."""
    T, H = x.shape
    _check("x", x, torch.float32)
    _check("x0", x0, torch.float32, (T, H))
    _check("step", step, torch.float32, (H,))
    _check("packed", packed, None, (T, 2 * H))
    d_ptr, P, stride = _delta(x, delta)
    L.call("ib_loop_pack", x.data_ptr(), d_ptr, P, stride, x0.data_ptr(), step.data_ptr(), packed.data_ptr(), dtype_code(packed.dtype), T, H, _stream())


def add_bias_rows(v: torch.Tensor, bias: torch.Tensor) -> None:
    """v[t] += bias, float32 [T, H] in place."""
    T, H = v.shape
    _check("v", v, torch.float32)
    _check("bias", bias, torch.float32, (H,))
    L.call("ib_add_bias_rows", v.data_ptr(), bias.data_ptr(), T, H, _stream())


def xielu_rows(z: torch.Tensor, pq: torch.Tensor, act: torch.Tensor) -> None:
    """act = xielu(sum_p z[p]) with the two numbers pq = (p, q): z > 0: softplus(p) z^2 + z / 2; else (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    _check("z", z, torch.float32)
    P, T, I = z.shape
    _check("pq", pq, torch.float32, (2,))
    _check("act", act, None, (T, I))
    L.call("ib_xielu_rows", z.data_ptr(), P, T * I, pq.data_ptr(), act.data_ptr(), dtype_code(act.dtype), T, I, _stream())


def gated_rmsnorm(o: torch.Tensor, w: torch.Tensor, eps: float, gate: torch.Tensor, gate_col: int, scale: float, out: torch.Tensor, out_col: int = 0) -> None:
    """out[t, out_col : out_col + H] = scale * w * o[t] / sqrt(mean(o[t]^2) + eps) * sigmoid(sum_p gate[p, t, gate_col : gate_col + H]); o float32 [T, H]."""
    T, H = o.shape
    _check("o", o, torch.float32)
    _check("w", w, torch.float32, (H,))
    _check("gate", gate, torch.float32)
    _check("out", out)
    P, Tg, R = gate.shape
    if Tg != T or gate_col + H > R or out.dim() != 2 or out.shape[0] != T or out_col + H > out.shape[1]:
        raise L.KernelError(f"gated_rmsnorm: gate {tuple(gate.shape)} from column {gate_col} and out {tuple(out.shape)} from column {out_col} do not hold {T} rows of {H}")
    L.call("ib_gated_rmsnorm", o.data_ptr(), w.data_ptr(), float(eps), gate.data_ptr() + 4 * gate_col, P, T * R, R, float(scale),
           out.data_ptr() + out.element_size() * out_col, dtype_code(out.dtype), out.shape[1], T, H, _stream())


# ---------------------------------------------------------------- selective scan (csrc/selective_scan.cu)
L.register("ib_conv_silu", [L._p, L._i, L._ll, L._i, L._p, L._p, L._i, L._p, L._ll, L._p, L._p, L._p, L._p, L._p, L._i, L._i, L._i, L._p])
L.register("ib_selective_scan", [L._p, L._p, L._i, L._ll, L._p, L._i, L._ll, L._i, L._p, L._p, L._p, L._p, L._p, L._ll, L._p, L._ll, L._i, L._p, L._p, L._i, L._p, L._i,
                                 L._i, L._i, L._i, L._p, L._p, L._p, L._p, L._i, L._p])
L.register("ib_scan_chunks_carry", [L._p, L._i, L._p, L._p, L._p, L._ll, L._p, L._p, L._p, L._p, L._i, L._ll, L._i, L._p, L._ll, L._i, L._i, L._i, L._p])


def conv_silu(proj: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], conv_state: torch.Tensor, seg_of_token: torch.Tensor, seg_start: torch.Tensor,
              seg_slot: torch.Tensor, xc: torch.Tensor, xa: Optional[torch.Tensor]) -> None:
    """xc[t, c] = silu(bias[c] + sum_j w[j, c] u[t - taps + 1 + j, c]) with u the first `inner` columns of proj (float32 partial sums [P, T, R]) and the rows
    before a segment's first token taken from conv_state (float32 [slots, taps - 1, inner], read only). w float32 [taps, inner]; xa: xc in another dtype."""
    _check("proj", proj, torch.float32)
    P, T, R = proj.shape
    taps, inner = w.shape
    _check("w", w, torch.float32)
    _check("conv_state", conv_state, torch.float32)
    _check("xc", xc, torch.float32, (T, inner))
    if xa is not None:
        _check("xa", xa, None, (T, inner))
    L.call("ib_conv_silu", proj.data_ptr(), P, T * R, R, w.data_ptr(), _ptr(bias), taps, conv_state.data_ptr(), conv_state.stride(0), seg_of_token.data_ptr(),
           seg_start.data_ptr(), seg_slot.data_ptr(), xc.data_ptr(), _ptr(xa), dtype_code(xa.dtype) if xa is not None else L.F32, T, inner, _stream())


def selective_scan(xc: torch.Tensor, low: torch.Tensor, proj: torch.Tensor, wdt: torch.Tensor, dt_bias: torch.Tensor, A: torch.Tensor, D: torch.Tensor,
                   state: torch.Tensor, conv_state: torch.Tensor, taps: int, seg_start: torch.Tensor, seg_slot: torch.Tensor, n_segments: int, out: torch.Tensor,
                   seg_list: Optional[torch.Tensor] = None, long_segs: Optional[torch.Tensor] = None, chunks: Optional[torch.Tensor] = None) -> None:
    """The scan over every segment's tokens, from and into state (float32 [slots, inner, N]); also moves conv_state on to the segment's last taps - 1 inputs.
    seg_list, long_segs, chunks: as for `gated_recurrence`: only the segments of seg_list are walked token by token, those of long_segs go chunk by
    chunk (every chunk alone from a zero state, the states carried from chunk to chunk, every chunk again from its incoming state).
    xc float32 [T, inner]; low float32 partial sums [P, T, rank + 2 N] = [dt_low | B | C]; proj float32 partial sums [P, T, >= 2 inner] = [u | z];
    wdt float32 [inner, rank]; A float32 [inner, N] (negative rates); out [T, inner] = (y + D x) * silu(z)."""
    T, inner = xc.shape
    N, rank = A.shape[1], wdt.shape[1]
    _check("xc", xc, torch.float32)
    _check("low", low, torch.float32)
    _check("proj", proj, torch.float32)
    if tuple(low.shape[1:]) != (T, rank + 2 * N) or proj.shape[1] != T:
        raise L.KernelError(f"selective_scan: low {tuple(low.shape)} must be [P, {T}, {rank + 2 * N}] and proj {tuple(proj.shape)} [P, {T}, >= {2 * inner}]")
    _check("wdt", wdt, torch.float32, (inner, rank))
    _check("dt_bias", dt_bias, torch.float32, (inner,))
    _check("A", A, torch.float32, (inner, N))
    _check("D", D, torch.float32, (inner,))
    _check("state", state, torch.float32)
    _check("conv_state", conv_state, torch.float32)
    _check("out", out, None, (T, inner))
    def scan(n, segs, table, chunk_state, chunk_dt, which):
        L.call("ib_selective_scan", xc.data_ptr(), low.data_ptr(), low.shape[0], T * low.shape[2], proj.data_ptr(), proj.shape[0], T * proj.shape[2], proj.shape[2],
               wdt.data_ptr(), dt_bias.data_ptr(), A.data_ptr(), D.data_ptr(), state.data_ptr(), state.stride(0), conv_state.data_ptr(), conv_state.stride(0), int(taps),
               seg_start.data_ptr(), seg_slot.data_ptr(), n, out.data_ptr(), dtype_code(out.dtype), inner, N, rank, _ptr(segs), _ptr(table), _ptr(chunk_state),
               _ptr(chunk_dt), which, _stream())

    if long_segs is None:
        if seg_list is not None:
            _check("seg_list", seg_list, torch.int32)
            n_segments = seg_list.shape[0]
        scan(n_segments, seg_list, None, None, None, 0)
        return
    _check("long_segs", long_segs, torch.int32)
    _check("chunks", chunks, torch.int32)
    if seg_list is not None and seg_list.shape[0]:
        scan(seg_list.shape[0], seg_list, None, None, None, 0)
    m = chunks.shape[0]
    chunk_state = torch.empty((m, inner, N), dtype=torch.float32, device=xc.device)
    chunk_dt = torch.empty((m, inner), dtype=torch.float32, device=xc.device)
    scan(m, None, chunks, chunk_state, chunk_dt, 1)
    L.call("ib_scan_chunks_carry", long_segs.data_ptr(), long_segs.shape[0], seg_start.data_ptr(), seg_slot.data_ptr(), state.data_ptr(), state.stride(0),
           chunk_state.data_ptr(), chunk_dt.data_ptr(), A.data_ptr(), proj.data_ptr(), proj.shape[0], T * proj.shape[2], proj.shape[2], conv_state.data_ptr(),
           conv_state.stride(0), int(taps), inner, N, _stream())
    scan(m, None, chunks, chunk_state, chunk_dt, 2)


# ---------------------------------------------------------------- attention with sigmoid weights behind a convolution of its projections (csrc/sigmoid_attention.cu)
L.register("ib_qkv_conv", [L._p, L._i, L._ll, L._p, L._p, L._i, L._p, L._ll, L._p, L._p, L._p, L._i, L._p, L._i, L._i, L._i, L._i, L._f, L._i, L._i, L._f, L._p, L._i,
                           C.POINTER(L.KvView), L._p, L._i, L._p])
L.register("ib_sigmoid_attention", [L._p, L._i, C.POINTER(L.KvView), L._p, L._p, L._f, L._p, L._p, L._p, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._i, L._p, L._p])
L.register("ib_sigmoid_attention_mma", [L._p, C.POINTER(L.KvView), L._p, L._p, L._p, L._i, L._i, L._f, L._p, L._p, L._p, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._i, L._p, L._p])
L.KERNELS_PER_CALL["ib_qkv_conv"] = 1   # two with a convolution state; counted by the caller


def qkv_conv(proj: torch.Tensor, bias: Optional[torch.Tensor], conv_w: Optional[torch.Tensor], conv_state: Optional[torch.Tensor], seg_of_token: torch.Tensor,
             seg_start: torch.Tensor, seg_slot: torch.Tensor, n_segments: int, positions: torch.Tensor, q_out: torch.Tensor, kv: KvLayerView, heads: int, qk_dim: int,
             v_dim: int, status: torch.Tensor, q_temp: Optional[tuple] = None, v_norm: bool = False, eps: float = 0.0, single_tokens: bool = False) -> None:
    """proj float32 [P, T, R] with R = [heads x qk_dim | kv_heads x qk_dim | kv_heads x v_dim], bias float32 [R] or None.
    conv_w float32 [taps, R] (a tap's weights for all channels together; the last row is the current token's) or None for no convolution;
    conv_state float32 [slots, taps - 1, R]: the last rows of the biased projection of every request, read for the rows before a segment's
    first token and then replaced by the step's last rows. q_temp = (coef, every): q is multiplied by 1 + coef ln(floor((p + 1) / every) + 1)
    at position p. v_norm: every value head is divided by its root mean square (eps inside the root). Writes q_out [T, heads * qk_dim] in
    the activation dtype and the keys and values into the paged cache. single_tokens: every segment brings one token (a step of decoded
    tokens): the state is replaced inside the one kernel; otherwise a second kernel does it after every reader of the old state."""
    _check("proj", proj, torch.float32)
    P, T, R = proj.shape
    view = kv.c_view()
    if R != (heads + view.kv_heads) * qk_dim + view.kv_heads * v_dim:
        raise L.KernelError(f"qkv_conv: the projection has {R} columns, expected {(heads + view.kv_heads) * qk_dim + view.kv_heads * v_dim}")
    _check("q_out", q_out, None, (T, heads * qk_dim))
    if bias is not None:
        _check("bias", bias, torch.float32, (R,))
    taps = 1
    if conv_w is not None:
        _check("conv_w", conv_w, torch.float32)
        if conv_w.dim() != 2 or conv_w.shape[1] != R:
            raise L.KernelError(f"qkv_conv: conv_w must be [taps, {R}], got {tuple(conv_w.shape)}")
        taps = conv_w.shape[0]
    slot_stride = 0
    if taps > 1:
        _check("conv_state", conv_state, torch.float32)
        if tuple(conv_state.shape[1:]) != (taps - 1, R):
            raise L.KernelError(f"qkv_conv: conv_state must be [slots, {taps - 1}, {R}], got {tuple(conv_state.shape)}")
        slot_stride = conv_state.stride(0)
        if not single_tokens:
            L.launches += 1
    for name, t_, n in (("seg_of_token", seg_of_token, T), ("positions", positions, T), ("seg_start", seg_start, n_segments + 1), ("seg_slot", seg_slot, n_segments)):
        _check(name, t_, torch.int32, (n,))
    coef, every = (0.0, 0) if q_temp is None else (float(q_temp[0]), int(q_temp[1]))
    L.call("ib_qkv_conv", proj.data_ptr(), P, T * R, _ptr(bias), _ptr(conv_w), taps, _ptr(conv_state) if taps > 1 else None, slot_stride, seg_of_token.data_ptr(),
           seg_start.data_ptr(), seg_slot.data_ptr(), n_segments, positions.data_ptr(), T, heads, qk_dim, v_dim, coef, every, 1 if v_norm else 0, float(eps),
           q_out.data_ptr(), dtype_code(q_out.dtype), C.byref(view), status.data_ptr(), 1 if single_tokens else 0, _stream())


def sigmoid_attention_mma_supports(heads: int, kv_heads: int, qk_dim: int, v_dim: int) -> bool:
    return bool(L.load().ib_sigmoid_attention_mma_supports(int(heads), int(kv_heads), int(qk_dim), int(v_dim)))


def sigmoid_attention_mma_rows(qk_dim: int, v_dim: int, rows_wanted: int) -> int:
    """Query rows a CTA of the tensor-core kernel holds (16, 32 or 64) when `rows_wanted` rows of a step can share key and value tiles."""
    return int(L.load().ib_sigmoid_attention_mma_rows(int(qk_dim), int(v_dim), int(rows_wanted)))


def sigmoid_attention(q: torch.Tensor, kv: KvLayerView, positions: torch.Tensor, seg_of_token: torch.Tensor, scale: float, r1: Optional[torch.Tensor],
                      r2: Optional[torch.Tensor], pb: Optional[torch.Tensor], out: torch.Tensor, heads: int, qk_dim: int, v_dim: int, status: torch.Tensor,
                      n_slices: int = 1, slice_keys: int = 1 << 30, part: Optional[torch.Tensor] = None, units: Optional[torch.Tensor] = None,
                      tensor_cores: bool = False, rows: int = 16) -> None:
    """out[t, h] = sum over keys j <= position of sigmoid((q . k_j) * scale - r1[h] ln(1 + r2[h] (position - j)) + pb[h]) v_j: causal attention whose
    weights are sigmoids and are not normalised. r1, r2, pb: float32 [heads] or None. n_slices > 1: the keys are cut into slices of slice_keys whose
    partial sums (`part`, float32, at least T * heads * n_slices * v_dim values) are added in order. tensor_cores: the m16n8k16 kernel (bfloat16; see
    `sigmoid_attention_mma_supports`), with `units` None (a CTA per token and kv head) or int32 [n, 2] of (first token, tokens) runs of consecutive
    tokens of one request, at most rows // (heads // kv_heads) tokens each; rows: query rows a CTA holds (`sigmoid_attention_mma_rows`)."""
    T = q.shape[0]
    view = kv.c_view()
    _check("q", q, None, (T, heads * qk_dim))
    _check("out", out, q.dtype, (T, heads * v_dim))
    _check("positions", positions, torch.int32, (T,))
    _check("seg_of_token", seg_of_token, torch.int32, (T,))
    for name, v in (("r1", r1), ("r2", r2), ("pb", pb)):
        if v is not None:
            _check(name, v, torch.float32, (heads,))
    if n_slices > 1:
        _check("part", part, torch.float32)
        if part.numel() < T * heads * n_slices * v_dim:
            raise L.KernelError("sigmoid_attention: the scratch for the slices is too small")
        L.launches += 1
    if tensor_cores:
        n_units = T
        if units is not None:
            _check("units", units, torch.int32)
            n_units = units.shape[0]
        L.call("ib_sigmoid_attention_mma", q.data_ptr(), C.byref(view), positions.data_ptr(), seg_of_token.data_ptr(), _ptr(units), n_units, int(rows), float(scale), _ptr(r1), _ptr(r2),
               _ptr(pb), out.data_ptr(), _ptr(part), T, heads, qk_dim, v_dim, n_slices, slice_keys, status.data_ptr(), _stream())
        return
    L.call("ib_sigmoid_attention", q.data_ptr(), dtype_code(q.dtype), C.byref(view), positions.data_ptr(), seg_of_token.data_ptr(), float(scale), _ptr(r1), _ptr(r2),
           _ptr(pb), out.data_ptr(), _ptr(part), T, heads, qk_dim, v_dim, n_slices, slice_keys, status.data_ptr(), _stream())
