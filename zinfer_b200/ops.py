"""Python face of the kernel library: one function per kernel entry point.

The library is built on first use (see ``csrc/build.py``) and loaded with ctypes.
Every function takes CUDA tensors, checks what the kernel assumes, launches on the
current torch stream and raises :class:`KernelError` with the kernel's own message
if it refuses.  There is no fallback of any kind: without the library, or with
tensors that are not on a CUDA device, these functions fail.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import profiling as _prof
from .csrc import build as _build


class KernelError(RuntimeError):
    pass


_LIB = None
F32, BF16 = 0, 1


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _build.library_path()
        try:
            _LIB = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        _LIB.zi_last_error.restype = ctypes.c_char_p
        _LIB.zi_gemm_tcgen05_plan.restype = ctypes.c_longlong
        _LIB.zi_attention_decode_workspace_floats.restype = ctypes.c_longlong
    return _LIB


def kernel_status() -> int:
    """Reads and clears the status words of the tcgen05 kernels (synchronises).
    0: every bounded wait inside them completed; else the code of the wait that ran out."""
    return int(lib().zi_gemm_tcgen05_status())   # one word for the products and the tcgen05 attention


def require_kernel_status_ok(where: str) -> None:
    """Raises if a bounded wait inside a tensor-core kernel ran out since the last check (its
    results are then not to be trusted).  Synchronises; the engine calls it where it waits for
    the device anyway, and every so many steps."""
    code = kernel_status()
    if code != 0:
        raise KernelError(f"{where}: a wait inside a tensor-core kernel ran out (code {code}); its results are invalid")


def selftest_wait_runs_out(code: int = 77, tries: int = 4096) -> None:
    """Launches one CTA that waits ``tries`` times on a barrier nobody arrives at, so that the wait
    runs out and the kernel records ``code`` in the status word, the way a stuck product would.
    Returns normally (nothing faults or hangs); :func:`require_kernel_status_ok` then raises."""
    _check(lib().zi_selftest_wait_runs_out(code, tries, _stream()), "selftest_wait_runs_out")


def gemm_pair_kernel(on: bool) -> bool:
    """Switches the matrix product's kernel for CTA pairs (tcgen05 ``cta_group::2``: two SMs on one
    tile of 256 tokens x 256 weight rows, each loading half of the weight rows) on or off for
    products of 256 tokens and more; returns the setting before.  Off unless
    ``ZINFER_B200_GEMM_PAIR=1``: measured equal to the single-CTA kernel inside a prefill step,
    where both run at the pace the power limit allows."""
    return bool(lib().zi_gemm_tcgen05_pair_enable(1 if on else 0))


def library_file() -> str:
    return _build.library_path()


def _tag(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors; there is no CPU path")
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = 0   # kernel launches issued through this module (graph replays are counted by their owner)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        msg = lib().zi_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what}: {msg} (code {code})")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _nb(*tensors) -> int:
    """Bytes of the given tensors (None counts nothing)."""
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")
    return t


class Partials:
    """A split-K matrix product whose partial sums have not been added yet:
    ``data`` [splits, M, N] float32.  The consumers below (residual add + norm, SwiGLU,
    q/k norm + rotary) add the splits themselves, in order, which saves a kernel and a
    round trip through memory; ``sum(dtype)`` adds them for any other consumer."""

    def __init__(self, data: torch.Tensor):
        self.data = data

    @property
    def shape(self):
        return self.data.shape[1:]

    @property
    def splits(self) -> int:
        return self.data.shape[0]

    def sum(self, dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(tuple(self.shape), dtype=dtype, device=self.data.device)
        S, M, N = self.data.shape
        h = torch.zeros((M, N), dtype=torch.float32, device=self.data.device)
        _check(lib().zi_residual_add_partials(_ptr(h), _ptr(self.data), S, ctypes.c_longlong(M * N),
                                              ctypes.c_longlong(M * N), _stream()), "partials.sum")
        return h if dtype == torch.float32 else h.to(dtype)


class Scaled:
    """An update of the residual stream that is multiplied by ``scale`` as it is added (a model's
    residual multiplier): ``delta`` is a tensor or :class:`Partials`."""

    def __init__(self, delta, scale: float):
        self.delta = delta
        self.scale = float(scale)

    @property
    def shape(self):
        return self.delta.shape


class Carried:
    """Nothing is pending: the residual stream is up to date, and ``x`` is that stream in the activations' type (a block
    that made it hands it to the next one, which may read it instead of casting the stream again)."""

    def __init__(self, x: torch.Tensor):
        self.x = x


class Several:
    """Updates of the residual stream that are still to be added, in this order (a block whose sublayers read the
    same stream leaves one per sublayer): each a tensor, :class:`Partials`, or either inside :class:`Scaled`.
    ``row_bias`` (float32 [width]) is a vector that is added to every row with them (an output projection's bias)."""

    def __init__(self, terms, row_bias: Optional[torch.Tensor] = None):
        self.terms = []
        self.row_bias = row_bias
        for t in terms:
            if isinstance(t, Several):        # updates that were pending already come first, in their order
                self.terms += t.terms
                self.row_bias = _sum_row_bias(t.row_bias, self.row_bias)
            elif t is not None and not isinstance(t, Carried):
                self.terms.append(t)

    @property
    def shape(self):
        return self.terms[0].shape


def _sum_row_bias(a: Optional[torch.Tensor], b: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if a is None or b is None:
        return a if b is None else b
    return a + b


def _terms_of(delta) -> list:
    if delta is None or isinstance(delta, Carried):
        return []
    return list(delta.terms) if isinstance(delta, Several) else [delta]


def sum_norm(h: torch.Tensor, delta, w1: torch.Tensor, eps: float, out_dtype: torch.dtype, w2: Optional[torch.Tensor] = None,
             rows: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None):
    """``h += `` every update of ``delta`` (a tensor, :class:`Partials`, :class:`Scaled`, or :class:`Several` of up to
    four of them, added in order) and ``bias``, in place and in 32-bit; then the RMS norm of every row times ``w1`` and,
    with ``w2``, the same norm times ``w2`` as well (two norms of one stream share their root mean square): one
    kernel, one pass.  With ``rows`` the picked rows' norms are returned and ``h`` is left as it is.  Returns the norm,
    or the pair of norms."""
    T, H = h.shape
    terms = _terms_of(delta)
    if isinstance(delta, Several):
        bias = _sum_row_bias(delta.row_bias, bias)
    while len(terms) > 4:               # the kernel adds four at once: the first ones go in by themselves, in order
        _need(rows is None, "more than four updates cannot be added for picked rows")
        residual_add(h, terms.pop(0))
    _need(h.dtype == torch.float32 and h.is_contiguous(), "the residual stream is contiguous float32")
    for w in (w1, w2):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == H), "norm weights are float32 of the row's width")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == H and bias.is_contiguous(), "the bias is float32 of the row's width")
    n_terms = len(terms)
    whole, part = (ctypes.c_void_p * 4)(), (ctypes.c_void_p * 4)()
    dtypes, splits = (ctypes.c_int * 4)(), (ctypes.c_int * 4)()
    zstride, scales = (ctypes.c_longlong * 4)(), (ctypes.c_float * 4)()
    keep, nbytes = [], 0
    for i, term in enumerate(terms):
        t, scales[i] = _unscaled(term)
        if isinstance(t, Partials):
            _need(tuple(t.shape) == (T, H), "an update must match the residual stream")
            part[i], splits[i], zstride[i] = t.data.data_ptr(), t.splits, T * H
            keep.append(t.data)
        else:
            _need(tuple(t.shape) == (T, H) and t.is_contiguous(), "an update must match the residual stream")
            whole[i], dtypes[i] = t.data_ptr(), _tag(t)
            keep.append(t)
        nbytes += _nb(keep[-1])
    n = T if rows is None else _i32(rows, "rows").shape[0]
    out1 = torch.empty((n, H), dtype=out_dtype, device=h.device)
    out2 = torch.empty_like(out1) if w2 is not None else None
    with _prof.region("sum of updates + norm" + (" pair" if w2 is not None else ""),
                      lambda: (2 if rows is None else 1) * n * H * 4 + nbytes + _nb(out1) * (2 if w2 is not None else 1)):
        _check(lib().zi_sum_norm_pair(_ptr(h), n_terms, whole, dtypes, part, splits, zstride, scales, _ptr(bias), _ptr(w1),
                                      _ptr(w2), ctypes.c_float(eps), _ptr(out1), _ptr(out2), _tag(out1), _ptr(rows), n, H,
                                      _stream()), "sum_norm")
    return out1 if w2 is None else (out1, out2)


def add_rmsnorm_pair(h: torch.Tensor, delta, w1: torch.Tensor, w2: torch.Tensor, eps1: float, eps2: float,
                     out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None):
    """Both norms of a block whose two sublayers read the same stream: ``h += delta`` (see :func:`sum_norm`), then
    ``(norm(h) * w1, norm(h) * w2)``; one kernel when both norms have the same eps."""
    if eps1 == eps2:
        return sum_norm(h, delta, w1, eps1, out_dtype, w2=w2, bias=bias)
    x1 = sum_norm(h, delta, w1, eps1, out_dtype, bias=bias)
    return x1, sum_norm(h, None, w2, eps2, out_dtype)


def _unscaled(delta):
    """(update, multiplier) of an update given plain or as :class:`Scaled`; nothing for :class:`Carried`."""
    if isinstance(delta, Carried):
        return None, 1.0
    if isinstance(delta, Scaled):
        return delta.delta, delta.scale
    return delta, 1.0


# ------------------------------------------------------------------ elementwise
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows ``ids`` of ``table`` [V, H] as the 32-bit residual stream [T, H]."""
    V, H = table.shape
    T = ids.shape[0]
    _need(table.is_contiguous(), "embedding table must be contiguous")
    _i32(ids, "ids")
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    with _prof.region("embed_gather", lambda: T * H * table.element_size() + _nb(out, ids)):
        _check(lib().zi_embed_gather(_ptr(out), _ptr(table), _tag(table), _ptr(ids), T, H, V, _stream()), "embed_gather")
    return out


def embed_bigram(table: torch.Tensor, bigram: Optional[torch.Tensor], ids: torch.Tensor, step, last_token: torch.Tensor,
                 scale: float, buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """The 32-bit residual stream ``scale * table[ids] + bigram[row]``: ``row`` is ``(previous token * mul_prev + token *
    mul_cur) mod buckets``, or ``buckets`` (the table's last row) for a request's first token.  The token before a
    portion's first token is ``last_token[slot]`` (int32 [slots, 1], one per request), which then receives the portion's
    last token.  ``bigram`` None: the scaled rows alone."""
    V, H = table.shape
    T = ids.shape[0]
    _need(table.is_contiguous(), "embedding table must be contiguous")
    if bigram is not None:
        _need(bigram.is_contiguous() and bigram.dtype == table.dtype and tuple(bigram.shape) == (buckets + 1, H),
              "the pair table has one row per bucket and one more, in the embedding's type")
    _need(last_token.dtype == torch.int32 and last_token.is_contiguous() and last_token[0].numel() == 1,
          "the last tokens are int32, one per request slot")
    for t, name in ((ids, "ids"), (step.positions, "positions"), (step.cu_q, "cu_q"), (step.state_slots, "state_slots")):
        _i32(t, name)
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    with _prof.region("embed (scaled, with a table of token pairs)", lambda: 2 * T * H * table.element_size() + _nb(out, ids)):
        _check(lib().zi_embed_bigram(_ptr(out), _ptr(table), _ptr(bigram), _tag(table), _ptr(ids), _ptr(step.positions),
                                     _ptr(step.cu_q), _ptr(step.state_slots), _ptr(last_token), step.n_seqs, T, H, V,
                                     ctypes.c_float(scale), int(buckets), ctypes.c_longlong(int(mul_prev)),
                                     ctypes.c_longlong(int(mul_cur)), _stream()), "embed_bigram")
    return out


def patch_tokens(ids: torch.Tensor, prev: torch.Tensor, dst: torch.Tensor, src: torch.Tensor) -> None:
    """``ids[dst[i]] = prev[src[i]]`` where ``dst[i] >= 0``: feeds tokens sampled by the
    step before without a round trip through the host."""
    for t, name in ((ids, "ids"), (prev, "prev"), (dst, "dst"), (src, "src")):
        _i32(t, name)
    _check(lib().zi_patch_tokens(_ptr(ids), _ptr(prev), _ptr(dst), _ptr(src), dst.numel(), _stream()), "patch_tokens")


def add_rmsnorm(h: torch.Tensor, delta, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``h += delta`` in place (32-bit), then RMSNorm of every row.  ``delta`` may be a tensor,
    :class:`Partials`, or either inside :class:`Scaled` (``h += scale * delta``); ``bias`` (float32 [H])
    is added to every row as well.

    ``rows`` (int32, repeats allowed) picks rows instead: the result has one row per entry,
    the norm of ``h[row] + delta[row]``, and ``h`` is left unchanged."""
    T, H = h.shape
    if isinstance(delta, Several):      # several updates at once: the kernel that adds them all in one pass
        _need(out is None, "several updates at once come with a new output tensor")
        return sum_norm(h, delta, weight, eps, out_dtype, rows=rows, bias=bias)
    delta, dscale = _unscaled(delta)
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == H and bias.is_contiguous(), "the bias is float32 of the row's width")
    _need(h.dtype == torch.float32 and h.is_contiguous(), "the residual stream is contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == H, "norm weight must be float32 of the row's width")
    part, splits, zstride = None, 0, 0
    if isinstance(delta, Partials):
        _need(tuple(delta.shape) == tuple(h.shape), "delta must match the residual stream")
        part, splits, zstride, delta = delta.data, delta.splits, T * H, None
    elif delta is not None:
        _need(delta.shape == h.shape and delta.is_contiguous(), "delta must match the residual stream")
    n = T if rows is None else _i32(rows, "rows").shape[0]
    if out is None:
        out = torch.empty((n, H), dtype=out_dtype, device=h.device)
    with _prof.region("add_rmsnorm", lambda: (2 if rows is None else 1) * n * H * 4 + _nb(out, weight)
                      + (n * H * delta.element_size() if delta is not None else 0) + splits * n * H * 4):
        _check(lib().zi_add_rmsnorm_scaled(_ptr(h), _ptr(delta), _tag(delta) if delta is not None else F32, _ptr(part),
                                           splits, ctypes.c_longlong(zstride), ctypes.c_float(dscale), _ptr(bias),
                                           _ptr(weight), ctypes.c_float(eps), _ptr(out), _tag(out), _ptr(rows), n, H,
                                           _stream()), "add_rmsnorm")
    return out


def residual_add(h: torch.Tensor, delta) -> None:
    if isinstance(delta, Several):
        _need(delta.row_bias is None, "residual_add: a vector for every row goes in with a norm's kernel")
        for term in delta.terms:
            residual_add(h, term)
        return
    delta, dscale = _unscaled(delta)
    if isinstance(delta, Partials):
        delta = delta.sum(torch.float32)
    _need(h.dtype == torch.float32 and h.is_contiguous() and delta.is_contiguous() and delta.shape == h.shape,
          "residual_add: shapes must match and be contiguous")
    with _prof.region("residual_add", lambda: 2 * _nb(h) + _nb(delta)):
        _check(lib().zi_residual_add_scaled(_ptr(h), _ptr(delta), _tag(delta), ctypes.c_float(dscale),
                                            ctypes.c_longlong(h.numel()), _stream()), "residual_add")


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """``x *= factor`` in place on a contiguous float32 tensor (a model's multiplier on its logits)."""
    _need(x.dtype == torch.float32 and x.is_contiguous(), "scale_: a contiguous float32 tensor")
    with _prof.region("scale", lambda: 2 * _nb(x)):
        _check(lib().zi_scale_f32(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(factor), _stream()), "scale")
    return x


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, out: Optional[torch.Tensor] = None, group: int = 1) -> torch.Tensor:
    """``x * sigmoid(gate)`` for two [T, width] tensors whose rows may be views of wider rows.  With ``group`` g the
    gate has width / g columns and each gates g neighbouring columns of ``x`` (a gate per head)."""
    T, W = x.shape
    _need(group >= 1 and W % group == 0 and tuple(gate.shape) == (T, W // group) and gate.dtype == x.dtype
          and x.stride(1) == 1 and gate.stride(1) == 1,
          "sigmoid_gate: two tensors of one type with dense rows, the gate with one column per group")
    if out is None:
        out = torch.empty((T, W), dtype=x.dtype, device=x.device)
    with _prof.region("sigmoid gate", lambda: (2 * T * W + T * W // group) * x.element_size()):
        _check(lib().zi_sigmoid_gate_grouped(_ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(gate), gate.stride(0), _tag(x),
                                             T, W, group, _stream()), "sigmoid_gate")
    return out


def clamped_gate(gate_up, limit: float, alpha: float, shift: float, out_dtype: torch.dtype, interleave: int = 0) -> torch.Tensor:
    """``g' * sigmoid(alpha * g') * (u' + shift)`` with ``g' = min(g, limit)`` and ``u' = clamp(u, -limit, limit)`` for
    ``gate_up`` [T, 2I] (gate then up, or interleaved in blocks as :func:`swiglu` has it), a tensor or
    :class:`Partials` whose splits are added in order."""
    part = gate_up if isinstance(gate_up, Partials) else None
    T, two_i = gate_up.shape
    _need(two_i % 2 == 0, "clamped_gate: gate and up side by side")
    I = two_i // 2
    if part is None:
        _need(gate_up.is_contiguous(), "clamped_gate: a contiguous [T, 2I] tensor")
    dev = part.data.device if part is not None else gate_up.device
    out = torch.empty((T, I), dtype=out_dtype, device=dev)
    src = part.data if part is not None else gate_up
    with _prof.region("clamped gate", lambda: _nb(out, src)):
        _check(lib().zi_clamped_gate(_ptr(out), _tag(out), _ptr(None if part is not None else gate_up),
                                     _tag(gate_up) if part is None else F32, _ptr(part.data if part is not None else None),
                                     part.splits if part is not None else 0, ctypes.c_longlong(T * two_i), T, I, interleave,
                                     ctypes.c_float(limit), ctypes.c_float(alpha), ctypes.c_float(shift), _stream()),
               "clamped_gate")
    return out


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """RMS norm of rows of activations ``x`` [T, n] (a view with dense rows; 32-bit or of ``out_dtype``) times ``weight``."""
    T, n = x.shape
    _need(x.stride(1) == 1 and weight.dtype == torch.float32 and weight.numel() == n and weight.is_contiguous(),
          "rmsnorm_rows: dense rows and a float32 weight of their width")
    out = torch.empty((T, n), dtype=out_dtype, device=x.device)
    with _prof.region("rmsnorm of rows", lambda: T * n * (x.element_size() + out.element_size())):
        _check(lib().zi_rmsnorm_rows(_ptr(out), out.stride(0), _tag(out), _ptr(x), x.stride(0), _tag(x), _ptr(weight),
                                     ctypes.c_float(eps), T, n, _stream()), "rmsnorm_rows")
    return out


def rope_table_freqs(n_pos: int, freqs: torch.Tensor, magnitude: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin [positions, len(freqs)] of the angles position * freqs[i] (32-bit products), both times ``magnitude``."""
    _need(freqs.dtype == torch.float32 and freqs.is_contiguous() and freqs.dim() == 1, "frequencies are a float32 vector")
    half = freqs.numel()
    cos = torch.empty((n_pos, half), dtype=torch.float32, device=freqs.device)
    sin = torch.empty_like(cos)
    _check(lib().zi_rope_table_freqs(_ptr(cos), _ptr(sin), n_pos, half, _ptr(freqs), ctypes.c_float(magnitude), _stream()),
           "rope_table_freqs")
    return cos, sin


def qkv_rows_prepare(proj: torch.Tensor, bias: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                     value_dim: int, n_gate: int, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                     eps: float, rot_dims: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                     positions: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor,
                     page_size: int, out_dtype: torch.dtype):
    """What follows a fused projection row [q heads | k heads | v heads | gate columns] when the changes span the whole
    row: ``bias`` (float32, the row's width) is added; ``q_weight`` / ``k_weight`` (float32 [heads * head_dim] and
    [kv heads * head_dim]) norm ALL of q and all of k by their root mean square; the first ``rot_dims`` dimensions of
    every q and k head rotate (pairs (i, i + rot_dims/2)); k and v go into the token's page slot.  ``proj`` may be
    32-bit beside 16-bit results.  Returns (q [T, heads * head_dim], gate [T, n_gate] or None) in ``out_dtype``."""
    T = proj.shape[0]
    qn, kn, vn = num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * value_dim
    width = qn + kn + vn + n_gate
    _need(proj.stride(1) == 1 and proj.shape[1] == width, "qkv_rows_prepare: rows as wide as their parts")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == width and bias.is_contiguous(), "the bias is float32 of the row's width")
    for wt, n in ((q_weight, qn), (k_weight, kn)):
        _need(wt is None or (wt.dtype == torch.float32 and wt.numel() == n and wt.is_contiguous()),
              "the norms' weights are float32, one value per element of q and of k")
    n_table = 0
    if cos is not None:
        _need(cos.shape == sin.shape and cos.shape[1] == rot_dims // 2 and cos.dtype == torch.float32,
              "rotary tables are float32 [positions, rot_dims/2]")
        n_table = cos.shape[0]
    _need(k_cache.dtype == out_dtype and v_cache.dtype == out_dtype and k_cache.is_contiguous() and v_cache.is_contiguous(),
          "cache pages have the activations' dtype")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
          and tuple(v_cache.shape[1:]) == (num_kv_heads, page_size, value_dim), "cache pages are [pages, kv heads, page, size]")
    q = torch.empty((T, qn), dtype=out_dtype, device=proj.device)
    gate = torch.empty((T, n_gate), dtype=out_dtype, device=proj.device) if n_gate else None
    with _prof.region("qkv rows (bias, whole norm, rotation, page write)",
                      lambda: T * width * proj.element_size() + T * width * q.element_size()):
        _check(lib().zi_qkv_rows_prepare(
            _ptr(proj), _tag(proj), proj.stride(0), _ptr(bias), _ptr(q), q.stride(0), _ptr(gate), n_gate, n_gate, _tag(q), T,
            num_heads, num_kv_heads, head_dim, value_dim, _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps),
            rot_dims if cos is not None else 0, _ptr(cos), _ptr(sin), n_table, _ptr(_i32(positions, "positions")),
            _ptr(k_cache), _ptr(v_cache), _ptr(_i32(slots, "slots")), page_size, _stream()), "qkv_rows_prepare")
    return q, gate


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def swiglu(gate_up, out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
           interleave: int = 0, activation: str = "silu") -> torch.Tensor:
    """``act(gate) * up`` for ``gate_up`` [T, 2I]: gate then up (``interleave`` 0), or blocks
    of 2 * ``interleave`` columns holding ``interleave`` gate values and then the up values of
    the same features.  ``activation``: ``silu`` or ``gelu_tanh`` (the tanh form of gelu)."""
    _need(activation in ACTIVATIONS, f"unknown activation {activation!r}")
    act = ACTIVATIONS[activation]
    if isinstance(gate_up, Partials):
        T, two_i = gate_up.shape
        I = two_i // 2
        if I % 4 == 0:
            res = torch.empty((T, I), dtype=out_dtype or torch.bfloat16, device=gate_up.data.device)
            with _prof.region("swiglu (partial sums)", lambda: _nb(res, gate_up.data)):
                _check(lib().zi_gated_act_partials(_ptr(res), _tag(res), _ptr(gate_up.data), gate_up.splits,
                                                   ctypes.c_longlong(T * two_i), T, I, interleave, act, _stream()), "swiglu")
            return res
        gate_up = gate_up.sum(out_dtype or torch.bfloat16)
    T, two_i = gate_up.shape
    _need(two_i % 2 == 0 and gate_up.is_contiguous(), "swiglu input is contiguous [T, 2I]")
    I = two_i // 2
    if out is None:
        out = torch.empty((T, I), dtype=gate_up.dtype, device=gate_up.device)
    with _prof.region("swiglu", lambda: _nb(out, gate_up)):
        _check(lib().zi_gated_act(_ptr(out), _ptr(gate_up), _tag(gate_up), T, I, interleave, act, _stream()), "swiglu")
    return out


SWIGLU_INTERLEAVE = 64   # block of gate rows followed by the up rows of the same features


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = SWIGLU_INTERLEAVE) -> torch.Tensor:
    """[2I, K] with rows in blocks of 2 * block: ``block`` gate rows, then the up rows of the
    same features (what the fused SwiGLU epilogue of the tensor-core product reads)."""
    I, K = gate.shape
    _need(I % block == 0, f"interleaving needs the width {I} to be a multiple of {block}")
    return torch.stack([gate.view(I // block, block, K), up.view(I // block, block, K)], dim=1).reshape(2 * I, K).contiguous()


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                  activation: str = "silu") -> torch.Tensor:
    """``act(x Wg^T) * (x Wu^T)`` for a gate/up weight interleaved by :func:`interleave_gate_up`; ``activation``
    silu (SwiGLU) or gelu_tanh.  On the tensor-core path without a K split the gate runs in the product's
    epilogue; otherwise the product is followed by the gate's kernel."""
    _need(activation in ACTIVATIONS, f"unknown activation {activation!r}")
    M, K = x.shape
    N2 = w_interleaved.shape[0]
    if (GEMM_BACKEND != "simt" and x.dtype == torch.bfloat16 and w_interleaved.dtype == torch.bfloat16 and M > 0
            and x.stride(1) == 1 and w_interleaved.is_contiguous()
            and lib().zi_gemm_tcgen05_supported(_ptr(x), _ptr(w_interleaved), K, x.stride(0), w_interleaved.stride(0))):
        out = torch.empty((M, N2 // 2), dtype=out_dtype or x.dtype, device=x.device)
        with _prof.region(f"linear+swiglu N={N2} K={K}", lambda: _nb(w_interleaved, out) + M * K * 2, 2 * M * N2 * K) as rec:
            code = lib().zi_gemm_tcgen05_gated(_ptr(out), _tag(out), _ptr(x), _ptr(w_interleaved), M, N2, K, x.stride(0),
                                               w_interleaved.stride(0), out.stride(0), ACTIVATIONS[activation],
                                               _sm_count(x.device), _stream())
            rec["keep"] = code != -2      # -2: this shape is better served by the product followed by the SwiGLU kernel
        if code != -2:
            _check(code, "linear_swiglu")
            return out
    gu = linear(x, w_interleaved, out_dtype=out_dtype or x.dtype, allow_partials=True)
    return swiglu(gu, out_dtype=out_dtype or x.dtype, interleave=SWIGLU_INTERLEAVE, activation=activation)


def rope_table(n_pos: int, head_dim: int, theta: float, device, factor: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin [positions, head_dim/2] of the angles position * theta^(-2i/head_dim) / factor (``factor``: linear
    scaling of the positions; 1 for none)."""
    cos = torch.empty((n_pos, head_dim // 2), dtype=torch.float32, device=device)
    sin = torch.empty_like(cos)
    _check(lib().zi_rope_table_scaled(_ptr(cos), _ptr(sin), n_pos, head_dim, ctypes.c_float(theta), ctypes.c_float(factor),
                                      _stream()), "rope_table")
    return cos, sin


def qk_prepare(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, rot_dims: int,
               q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
               cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
               k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], slots: Optional[torch.Tensor],
               page_size: int, values_from_keys: bool = False, write_kv: bool = True,
               value_dim: Optional[int] = None) -> torch.Tensor:
    """The general form of :func:`qk_norm_rope_store`: the rotation turns only the first ``rot_dims`` dimensions of a
    head (pairs (i, i + rot_dims/2), tables [positions, rot_dims/2]), and with ``values_from_keys`` the rows are
    [q heads | k heads] and a token's value is its key AS PROJECTED, before norm and rotation.  Rewrites q in place
    and returns ``qkv``.  ``value_dim``: the size of a value head where it differs from ``head_dim``."""
    T = qkv.shape[0]
    dv = int(value_dim or head_dim)
    width = num_heads * head_dim + ((num_kv_heads * head_dim + (0 if values_from_keys else num_kv_heads * dv)) if write_kv else 0)
    _need(qkv.stride(1) == 1 and qkv.shape[1] >= width, "qk_prepare: dense rows as wide as their heads")
    for wt in (q_weight, k_weight):
        if wt is not None:
            _need(wt.dtype == torch.float32 and wt.numel() == head_dim, "q/k norm weights are float32 [head_dim]")
    n_table = 0
    if cos is not None:
        _need(cos.shape == sin.shape and cos.shape[1] == rot_dims // 2 and cos.dtype == torch.float32,
              "rotary tables are float32 [positions, rot_dims/2]")
        n_table = cos.shape[0]
    _i32(positions, "positions")
    if write_kv:
        _need(k_cache is not None and v_cache is not None and slots is not None, "writing needs pages and slots")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "cache pages have the activations' dtype")
        _i32(slots, "slots")
    with _prof.region("qk_prepare (norm, partial rotation, page write)", lambda: 2 * T * width * qkv.element_size()):
        _check(lib().zi_qk_prepare_v(_ptr(qkv), _tag(qkv), T, qkv.stride(0), _ptr(qkv), qkv.stride(0), num_heads, num_kv_heads,
                                   head_dim, dv, rot_dims, _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps), _ptr(cos), _ptr(sin),
                                   n_table, _ptr(positions), _ptr(k_cache), _ptr(v_cache), _ptr(slots), page_size,
                                   1 if values_from_keys else 0, 1 if write_kv else 0, _stream()), "qk_prepare")
    return qkv


def qk_norm_rope_store(qkv, num_heads: int, num_kv_heads: int, head_dim: int,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       slots: Optional[torch.Tensor], page_size: int, write_kv: bool = True,
                       out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """On the fused projection rows [q heads | k heads | v heads]: per-head RMSNorm of q
    and k (when weights are given), rotary positions (when tables are given); k and v go
    into their page slots.  Returns q [T, >= heads * d]: ``qkv`` itself, rewritten in
    place, or a new tensor when ``qkv`` came as split-K partial sums."""
    width = (num_heads + 2 * num_kv_heads) * head_dim if write_kv else num_heads * head_dim
    part, splits, zstride = None, 0, 0
    if isinstance(qkv, Partials):
        T = qkv.shape[0]
        _need(qkv.shape[1] == width, "partial sums must have exactly the heads' width")
        part, splits, zstride = qkv.data, qkv.splits, T * width
        q_out = torch.empty((T, num_heads * head_dim), dtype=out_dtype or torch.bfloat16, device=part.device)
        src, src_stride, dtype_tag = None, 0, _tag(q_out)
    else:
        T = qkv.shape[0]
        _need(qkv.stride(1) == 1, "qkv rows must be dense")
        _need(qkv.shape[1] >= width, "qkv is narrower than its heads")
        q_out, src, src_stride, dtype_tag = qkv, qkv, qkv.stride(0), _tag(qkv)
    for wt in (q_weight, k_weight):
        if wt is not None:
            _need(wt.dtype == torch.float32 and wt.numel() == head_dim, "q/k norm weights are float32 [head_dim]")
    n_table = 0
    if cos is not None:
        _need(cos.shape == sin.shape and cos.shape[1] == head_dim // 2 and cos.dtype == torch.float32,
              "rotary tables are float32 [positions, head_dim/2]")
        n_table = cos.shape[0]
    _i32(positions, "positions")
    if write_kv:
        _need(k_cache is not None and v_cache is not None and slots is not None, "writing needs pages and slots")
        _need(k_cache.dtype == q_out.dtype and v_cache.dtype == q_out.dtype, "cache pages have the activations' dtype")
        _i32(slots, "slots")
    with _prof.region("qk_norm_rope_store", lambda: (2 * T * width * q_out.element_size() if part is None else
                                                      _nb(part) + T * width * q_out.element_size())):
        _check(lib().zi_qk_norm_rope_store(
            _ptr(src), dtype_tag, T, src_stride, _ptr(part), splits, ctypes.c_longlong(zstride), _ptr(q_out),
            q_out.stride(0), num_heads, num_kv_heads, head_dim, _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps),
            _ptr(cos), _ptr(sin), n_table, _ptr(positions), _ptr(k_cache), _ptr(v_cache), _ptr(slots), page_size,
            1 if write_kv else 0, _stream()), "qk_norm_rope_store")
    return q_out


# ------------------------------------------------------------------------ matrices
_SM_COUNT: dict[int, int] = {}
GEMM_BACKEND = os.environ.get("ZINFER_B200_GEMM", "auto")   # auto | simt  (simt: CUDA cores only, for comparisons)


def _sm_count(device: torch.device) -> int:
    idx = device.index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None, allow_partials: bool = False, fresh_weight: bool = False,
           relu2: bool = False):
    """``x [M, K] @ weight [N, K]^T`` with 32-bit accumulation; with ``relu2`` the square of the product's relu
    (taken on the 32-bit sums: in the tensor-core product's epilogue, or where its K splits are added).

    With ``allow_partials`` a product that was split along K may come back as
    :class:`Partials` (its consumer adds the splits) instead of a tensor.  ``fresh_weight``:
    ``weight`` is no weight but the output of an earlier kernel of this step (the tensor-core kernel
    otherwise requests its first weight tiles before it waits for the kernels before it).

    bfloat16 operands that meet TMA's alignment rules go to the tcgen05 kernel; float32
    operands (the true 32-bit path), mixed types and unaligned shapes go to the
    CUDA-core kernel."""
    M, K = x.shape
    N, K2 = weight.shape
    _need(K == K2, f"linear: x has {K} columns, weight has {K2}")
    _need(x.stride(1) == 1 and weight.stride(1) == 1, "linear: operands must be dense along K")
    _need(not (relu2 and allow_partials), "linear: partial sums cannot carry the square of relu")
    if (GEMM_BACKEND != "simt" and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and M > 0
            and lib().zi_gemm_tcgen05_supported(_ptr(x), _ptr(weight), K, x.stride(0), weight.stride(0))):
        plan = (ctypes.c_int * 3)()
        sms = _sm_count(x.device)
        need = lib().zi_gemm_tcgen05_plan(M, N, K, sms, plan)
        ws = torch.empty((need // 4,), dtype=torch.float32, device=x.device) if need else None
        defer = allow_partials and need > 0 and out is None
        if out is None and not defer:
            out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
        with _prof.region(f"linear{'+relu2' if relu2 else ''} N={N} K={K}",
                          lambda: _nb(weight) + M * K * 2 + (_nb(ws) if defer else _nb(out)), 2 * M * N * K):
            _check(lib().zi_gemm_tcgen05(_ptr(out), _tag(out) if out is not None else BF16, _ptr(x), _ptr(weight), M, N, K,
                                         x.stride(0), weight.stride(0), out.stride(0) if out is not None else N, _ptr(ws),
                                         ctypes.c_longlong(need), sms,
                                         (1 if defer else 0) | (2 if fresh_weight else 0) | (4 if relu2 else 0),
                                         _stream()), "linear (tcgen05)")
        return Partials(ws.view(plan[2], M, N)) if defer else out
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    _need(out.stride(1) == 1, "linear: output rows must be dense")
    with _prof.region(f"linear (CUDA cores) N={N} K={K}", lambda: _nb(weight, out) + M * K * x.element_size(), 2 * M * N * K):
        _check(lib().zi_gemm_simt(_ptr(out), _tag(out), _ptr(x), _tag(x), _ptr(weight), _tag(weight), M, N, K,
                                  x.stride(0), weight.stride(0), out.stride(0), _stream()), "linear")
    if relu2:
        _need(out.is_contiguous(), "linear: the square of relu wants dense results")
        relu2_(out)
    return out


def tensor_core_linear_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether :func:`linear` would run this product on the tcgen05 kernel."""
    return bool(GEMM_BACKEND != "simt" and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] > 0
                and x.stride(1) == 1 and weight.stride(1) == 1
                and lib().zi_gemm_tcgen05_supported(_ptr(x), _ptr(weight), x.shape[1], x.stride(0), weight.stride(0)))


def linear_cuda_cores(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x @ weight^T`` with 32-bit multiply-adds on the CUDA cores whatever the operands' types
    (a router's logits, which are 32-bit also in a bfloat16 run)."""
    M, K = x.shape
    N = weight.shape[0]
    _need(weight.shape[1] == K and x.stride(1) == 1 and weight.is_contiguous(), "linear: operands must be dense along K")
    out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    with _prof.region(f"linear (CUDA cores) N={N} K={K}", lambda: _nb(weight, out) + M * K * x.element_size(), 2 * M * N * K):
        _check(lib().zi_gemm_simt(_ptr(out), _tag(out), _ptr(x), _tag(x), _ptr(weight), _tag(weight), M, N, K,
                                  x.stride(0), weight.stride(0), out.stride(0), _stream()), "linear")
    return out


def linear_argmax(x: torch.Tensor, weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The 32-bit product ``x [M, K] @ weight [N, K]^T`` and each row's argmax (first maximum, NaN
    counted as -inf, as :func:`argmax` has it).  For up to 128 rows on the tensor-core path the
    product's epilogue leaves one candidate per 32 weight rows and a small kernel picks among them,
    so the [M, N] result is not read again; otherwise the product is followed by the argmax kernel."""
    M, K = x.shape
    N = weight.shape[0]
    if (GEMM_BACKEND != "simt" and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and M > 0
            and x.stride(1) == 1 and weight.is_contiguous()
            and lib().zi_gemm_tcgen05_supported(_ptr(x), _ptr(weight), K, x.stride(0), weight.stride(0))):
        units = lib().zi_gemm_argmax_units(N)
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        cand_val = torch.empty((M, units), dtype=torch.float32, device=x.device)
        cand_idx = torch.empty((M, units), dtype=torch.int32, device=x.device)
        with _prof.region(f"linear+argmax N={N} K={K}", lambda: _nb(weight, out) + M * K * 2, 2 * M * N * K) as rec:
            code = lib().zi_gemm_tcgen05_argmax(_ptr(out), _ptr(x), _ptr(weight), M, N, K, x.stride(0), weight.stride(0),
                                                out.stride(0), _ptr(cand_val), _ptr(cand_idx), _sm_count(x.device), _stream())
            rec["keep"] = code != -2      # -2: more than 128 rows, or K would be split
        if code != -2:
            _check(code, "linear_argmax")
            ids = torch.empty((M,), dtype=torch.int32, device=x.device)
            with _prof.region("argmax (candidates)", lambda: _nb(cand_val, cand_idx)):
                _check(lib().zi_argmax_candidates(_ptr(ids), _ptr(cand_val), _ptr(cand_idx), M, units, _stream()),
                       "argmax (candidates)")
            return out, ids
    out = linear(x, weight, out_dtype=torch.float32)
    return out, argmax(out)


def _ll(v: int):
    return ctypes.c_longlong(int(v))


def linear_heads_ok(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether :func:`linear_heads` takes these views: bfloat16, heads side by side in rows that meet TMA's rules."""
    return bool(GEMM_BACKEND != "simt" and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and out.dtype in (torch.bfloat16, torch.float32) and weight.is_contiguous()
                and x.stride(2) == 1 and out.stride(2) == 1 and x.stride(1) % 8 == 0 and x.stride(0) % 8 == 0
                and (x.shape[1] - 1) * x.stride(1) + x.shape[2] <= x.stride(0)
                and lib().zi_gemm_tcgen05_supported(_ptr(x), _ptr(weight), x.shape[2], x.stride(0), weight.shape[2]))


def linear_heads(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[:, n] = x[:, n] @ weight[n]^T`` for every head n in ONE launch of the tcgen05 kernel: ``x`` [T, heads, K]
    and ``out`` [T, heads, N] are views whose heads lie side by side in their rows, ``weight`` [heads, N, K]."""
    T, H, K = x.shape
    N = weight.shape[1]
    _need(weight.shape == (H, N, K) and out.shape == (T, H, N), "linear_heads: shapes")
    with _prof.region(f"linear (per head, tcgen05) heads={H} N={N} K={K}", lambda: _nb(weight) + T * H * (K + N) * 2,
                      2 * T * H * N * K):
        _check(lib().zi_gemm_tcgen05_heads(_ptr(out), _tag(out), _ptr(x), _ptr(weight), T, N, K, x.stride(0), K, out.stride(0),
                                           H, x.stride(1), out.stride(1), _sm_count(x.device), _stream()), "linear_heads")
    return out


def linear_batched(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   relu2: bool = False) -> torch.Tensor:
    """``batch`` independent products ``out[b] = x[b] @ weight[b]^T`` (+ ``bias[b]``) on the CUDA cores with
    32-bit multiply-adds: ``x`` [B, M, K], ``weight`` [B, N, K], ``out`` [B, M, N], each possibly a
    strided view (block-diagonal gate matrices, one projection per head).  Any mix of operand types."""
    B, M, K = x.shape
    _need(weight.shape[0] == B and weight.shape[2] == K and out.shape == (B, M, weight.shape[1]), "linear_batched: shapes")
    N = weight.shape[1]
    _need(x.stride(2) == 1 and weight.stride(2) == 1 and out.stride(2) == 1, "linear_batched: dense along the last axis")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.shape == (B, N) and bias.is_contiguous(), "linear_batched: bias is float32 [B, N]")
    with _prof.region(f"linear (CUDA cores, batch of {B}) N={N} K={K}",
                      lambda: B * (M * K * x.element_size() + N * K * weight.element_size() + M * N * out.element_size()),
                      2 * B * M * N * K):
        _check(lib().zi_gemm_simt_general(
            _ptr(out), _tag(out), _ptr(x), _tag(x), _ptr(weight), _tag(weight), M, N, K, x.stride(1), weight.stride(1),
            out.stride(1), B, _ll(x.stride(0)), _ll(weight.stride(0)), _ll(out.stride(0)), _ptr(bias), _ll(N), None, None,
            None, _ll(0), 1 if relu2 else 0, 64 if M > 16 else 16, _stream()), "linear_batched")
    return out


def linear_grouped(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, row_src: torch.Tensor,
                   tile_group: torch.Tensor, n_tiles: torch.Tensor, tile_rows: int, relu2: bool = False) -> torch.Tensor:
    """Products whose sizes only the device knows: output row r is ``x[row_src[r]] @ weight[g]^T`` with g the
    group (expert) of r's tile of ``tile_rows`` rows (``tile_group``); rows with ``row_src`` -1 and tiles
    at or beyond ``n_tiles[0]`` are left alone.  ``weight`` [G, N, K]; ``out`` [rows, N]."""
    G, N, K = weight.shape
    rows = out.shape[0]
    _need(x.shape[1] == K and out.shape[1] == N and x.stride(1) == 1 and out.stride(1) == 1 and weight.is_contiguous(),
          "linear_grouped: shapes")
    _need(rows % tile_rows == 0 and row_src.numel() >= rows, "linear_grouped: whole tiles of rows")
    for t, name in ((row_src, "row_src"), (tile_group, "tile_group"), (n_tiles, "n_tiles")):
        _i32(t, name)
    pairs = max(1, rows - G * tile_rows)       # about as many rows are in use
    with _prof.region(f"linear (CUDA cores, grouped) N={N} K={K}", lambda: _nb(weight, out) + pairs * K * x.element_size(),
                      2 * pairs * N * K):
        _check(lib().zi_gemm_simt_general(
            _ptr(out), _tag(out), _ptr(x), _tag(x), _ptr(weight), _tag(weight), rows, N, K, x.stride(0), K, out.stride(0),
            1, _ll(0), _ll(0), _ll(0), None, _ll(0), _ptr(row_src), _ptr(tile_group), _ptr(n_tiles), _ll(N * K),
            1 if relu2 else 0, tile_rows, _stream()), "linear_grouped")
    return out


# ---------------------------------------------------------------- mixture of experts
def moe_route(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int,
              renormalize: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Per token: softmax scores over all router outputs, the ``top`` outputs with the largest score +
    correction (int32 [T, top]) and their scores without the correction (float32 [T, top]), divided by
    their sum if ``renormalize``."""
    T, NR = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "router logits are contiguous float32")
    if correction is not None:
        _need(correction.dtype == torch.float32 and correction.numel() == NR, "the correction is float32 [outputs]")
    chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    with _prof.region("moe route", lambda: _nb(logits, chosen, weight)):
        _check(lib().zi_moe_route(_ptr(chosen), _ptr(weight), _ptr(logits), _ptr(correction), T, NR, top,
                                  1 if renormalize else 0, _stream()), "moe_route")
    return chosen, weight


def moe_router(x: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], top: int,
               renormalize: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """The router's product (32-bit multiply-adds whatever the operands' types) and :func:`moe_route` in one
    kernel, one block per token."""
    T, K = x.shape
    NR = w_router.shape[0]
    _need(x.stride(1) == 1 and w_router.is_contiguous() and w_router.shape[1] == K, "moe_router: shapes")
    if correction is not None:
        _need(correction.dtype == torch.float32 and correction.numel() == NR, "the correction is float32 [outputs]")
    chosen = torch.empty((T, top), dtype=torch.int32, device=x.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=x.device)
    with _prof.region(f"moe router N={NR} K={K}", lambda: _nb(w_router) + T * K * x.element_size(), 2 * T * NR * K):
        _check(lib().zi_moe_router(_ptr(chosen), _ptr(weight), _ptr(x), _tag(x), x.stride(0), _ptr(w_router), _tag(w_router),
                                   _ptr(correction), T, K, NR, top, 1 if renormalize else 0, _stream()), "moe_router")
    return chosen, weight


def linear_few_rows_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether :func:`linear_few_rows` takes these operands: one type, rows in whole 16-byte pieces."""
    return bool(x.dtype == weight.dtype and x.shape[1] % 4 == 0 and x.stride(0) % 4 == 0 and x.stride(1) == 1
                and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def linear_few_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, row_src: torch.Tensor,
                    tile_group: torch.Tensor, n_tiles: torch.Tensor, relu2: bool = False) -> torch.Tensor:
    """:func:`linear_grouped` for tiles of 16 rows when the rows are few (a decode step): every weight row is
    streamed once per tile and multiplied with the tile's 16 rows; bound by memory."""
    G, N, K = weight.shape
    rows = out.shape[0]
    _need(rows % MOE_TILE_ROWS_SMALL == 0 and out.shape[1] == N and out.stride(1) == 1, "linear_few_rows: shapes")
    pairs = max(1, rows - G * MOE_TILE_ROWS_SMALL)
    # under the profiler the weights of the tiles in use are counted; their number is read from the device when the
    # profile is summed up, not here, where the read would stall the chain
    with _prof.region(f"linear (grouped, few rows) N={N} K={K}",
                      lambda: (lambda: min(G, pairs, int(n_tiles.item())) * N * K * weight.element_size()
                               + pairs * (K + N) * x.element_size()), 2 * pairs * N * K):
        _check(lib().zi_moe_few_rows(_ptr(out), _tag(out), out.stride(0), _ptr(x), _tag(x), x.stride(0), _ptr(weight),
                                     _ptr(_i32(row_src, "row_src")), _ptr(_i32(tile_group, "tile_group")),
                                     _ptr(_i32(n_tiles, "n_tiles")), rows // MOE_TILE_ROWS_SMALL, N, K, 1 if relu2 else 0,
                                     _stream()), "linear_few_rows")
    return out


MOE_TILE_ROWS_SMALL, MOE_TILE_ROWS, MOE_TILE_ROWS_TENSOR = 16, 64, 128


def moe_align(chosen: torch.Tensor, experts: int, tile_rows: int):
    """Lays the (token, expert) pairs out by expert in whole tiles of ``tile_rows`` rows.  Returns
    ``(row_token, row_self, pair_row, tile_expert, n_tiles)``: the token of every row (-1: padding), the
    row's own index where it is in use, the row of every pair (-1: an identity expert), the expert of
    every tile and the number of tiles (one int32 on the device)."""
    T, top = chosen.shape
    P = T * top
    cap_tiles = -(-P // tile_rows) + experts
    dev = chosen.device
    buf = torch.empty((2 * cap_tiles * tile_rows + P + cap_tiles + 1,), dtype=torch.int32, device=dev)
    n = cap_tiles * tile_rows
    row_token, row_self, pair_row = buf[:n], buf[n:2 * n], buf[2 * n:2 * n + P]
    tile_expert, n_tiles = buf[2 * n + P:2 * n + P + cap_tiles], buf[2 * n + P + cap_tiles:]
    with _prof.region("moe align", lambda: _nb(chosen) + 3 * P * 4):
        _check(lib().zi_moe_align(_ptr(_i32(chosen, "chosen")), P, top, experts, tile_rows, cap_tiles, _ptr(row_token),
                                  _ptr(row_self), _ptr(pair_row), _ptr(tile_expert), _ptr(n_tiles), _stream()), "moe_align")
    return row_token, row_self, pair_row, tile_expert, n_tiles


def gather_rows(x: torch.Tensor, row_src: torch.Tensor) -> torch.Tensor:
    """``out[r] = x[row_src[r]]`` (zeros where ``row_src[r]`` is -1): rows of ``x`` in another order."""
    rows, W = row_src.numel(), x.shape[1]
    _need(x.stride(1) == 1, "gather_rows: dense rows")
    out = torch.empty((rows, W), dtype=x.dtype, device=x.device)
    with _prof.region("gather rows", lambda: 2 * _nb(out)):
        _check(lib().zi_gather_rows(_ptr(out), _ptr(x), _tag(x), _ptr(_i32(row_src, "row_src")), rows, W, x.stride(0),
                                    _stream()), "gather_rows")
    return out


def linear_grouped_tensor_ok(weight: torch.Tensor) -> bool:
    """Whether :func:`linear_grouped_tensor` takes this stacked weight [G, N, K] (bfloat16 that meets TMA's
    alignment rules; its other operand is a fresh contiguous bfloat16 tensor with K columns)."""
    return bool(GEMM_BACKEND != "simt" and weight.dtype == torch.bfloat16 and weight.is_contiguous()
                and lib().zi_gemm_tcgen05_supported(_ptr(weight), _ptr(weight), weight.shape[2], weight.shape[2],
                                                    weight.shape[2]))


def linear_grouped_tensor(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor,
                          relu2: bool = False, pairs: int = 0) -> torch.Tensor:
    """The grouped product on the tcgen05 kernel: every 128 rows of ``x`` [rows, K] (bfloat16, laid out by
    group already) multiply with group ``tile_group[r // 128]`` of ``weight`` [G, N, K]; ``out`` [rows, N].
    Every tile is computed, also those past the rows in use (their results are never read).  ``pairs``:
    rows in use, for the profiler's count of useful operations."""
    G, N, K = weight.shape
    rows = x.shape[0]
    _need(out.shape == (rows, N) and out.stride(1) == 1 and rows % MOE_TILE_ROWS_TENSOR == 0, "linear_grouped_tensor: shapes")
    _need(tile_group.numel() >= rows // MOE_TILE_ROWS_TENSOR, "linear_grouped_tensor: a group per tile")
    with _prof.region(f"linear (grouped, tcgen05) N={N} K={K}", lambda: _nb(weight, out) + rows * K * 2,
                      2 * (pairs or rows) * N * K):
        _check(lib().zi_gemm_tcgen05_grouped(_ptr(out), _tag(out), _ptr(x), _ptr(weight), rows, N, K, x.stride(0), K,
                                             out.stride(0), G, _ptr(_i32(tile_group, "tile_group")), 1 if relu2 else 0,
                                             _sm_count(x.device), _stream()), "linear_grouped_tensor")
    return out


def moe_combine(y: torch.Tensor, x: torch.Tensor, chosen: torch.Tensor, weight: torch.Tensor, pair_row: torch.Tensor,
                experts: int) -> torch.Tensor:
    """``out[t] = sum_k weight[t, k] * (y[pair_row[t, k]] if chosen[t, k] < experts else x[t])``, k ascending."""
    T, H = x.shape
    top = chosen.shape[1]
    _need(y.dtype == torch.float32 and y.is_contiguous() and y.shape[1] == H and x.is_contiguous(), "moe_combine: shapes")
    out = torch.empty((T, H), dtype=x.dtype, device=x.device)
    with _prof.region("moe combine", lambda: T * top * H * 4 + 2 * _nb(out)):
        _check(lib().zi_moe_combine(_ptr(out), _ptr(y), _ptr(x), _tag(x), _ptr(chosen), _ptr(weight), _ptr(pair_row), T,
                                    top, experts, H, _stream()), "moe_combine")
    return out


# ---------------------------------------------------------------- recurrent mixers
RGLRU_CHUNK = 32    # tokens per chunk of the chunked recurrence (bfloat16 steps of 128 tokens and more)


def causal_conv(x: torch.Tensor, x_bias: torch.Tensor, kernel: torch.Tensor, bias: torch.Tensor, state: torch.Tensor,
                step) -> torch.Tensor:
    """Per-channel causal convolution of ``x + x_bias`` ([T, C], rows may be views of wider rows) with
    ``kernel`` [C, taps] (last column: the current token) plus ``bias``; the inputs before a request's
    first token of this step come from ``state`` [slots, taps, C] (rows 0..taps-2).  Returns float32 [T, C];
    the state is left as it is (:func:`rglru_scan` carries it on)."""
    T, C = x.shape
    taps = kernel.shape[1]
    _need(x.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
          and tuple(state.shape[1:]) == (taps, C), "causal_conv: state is float32 [slots, taps, C]")
    for t in (x_bias, kernel, bias):
        _need(t.dtype == torch.float32 and t.is_contiguous(), "causal_conv: float32 parameters")
    u = torch.empty((T, C), dtype=torch.float32, device=x.device)
    with _prof.region("causal conv", lambda: T * C * (x.element_size() * taps + 4)):
        _check(lib().zi_causal_conv(_ptr(u), _ptr(x), x.stride(0), _tag(x), _ptr(x_bias), _ptr(kernel), _ptr(bias),
                                    _ptr(state), C, taps, _ptr(step.cu_q), _ptr(step.state_slots), step.n_seqs, T,
                                    _stream()), "causal_conv")
    return u


def rglru_scan(u: torch.Tensor, gates: torch.Tensor, block_width: int, r_bias: torch.Tensor, i_bias: torch.Tensor,
               lam: torch.Tensor, decay_scale: float, y: torch.Tensor, y_bias: torch.Tensor, x: torch.Tensor,
               x_bias: torch.Tensor, state: torch.Tensor, step) -> torch.Tensor:
    """The real-gated linear recurrence over each request's tokens of this step, from and to ``state``:
    ``a = exp(-decay_scale * sigmoid(g_r + r_bias) * softplus(lam))``,
    ``S = a S + sqrt(1 - a^2) * sigmoid(g_i + i_bias) * u``; returns ``S * gelu_tanh(y + y_bias)`` in ``y``'s
    type.  ``gates`` float32 [T, blocks, 2, block_width] holds g_r and g_i; ``x`` (the convolution's input
    before its bias) is read to carry the convolution's last inputs on.  A bfloat16 step of many tokens
    runs the recurrence in chunks (the same sums, associated per chunk)."""
    T, C = u.shape
    taps = state.shape[1]
    _need(u.dtype == torch.float32 and gates.dtype == torch.float32 and u.is_contiguous() and gates.is_contiguous()
          and gates.numel() == 2 * T * C, "rglru_scan: u [T, C] and gates [T, 2C] are contiguous float32")
    _need(y.dtype == x.dtype and y.stride(1) == 1 and x.stride(1) == 1, "rglru_scan: branch rows are dense")
    out = torch.empty((T, C), dtype=y.dtype, device=y.device)
    if y.dtype == torch.bfloat16 and T >= 4 * RGLRU_CHUNK:
        # a prompt: the recurrence in chunks, so that its tokens do not wait for one another
        need = lib().zi_rglru_chunked_workspace_floats(T, C, step.n_seqs, RGLRU_CHUNK)
        work = torch.empty((need,), dtype=torch.float32, device=y.device)
        with _prof.region("rglru scan (chunks)", lambda: 2 * T * C * (12 + 3 * y.element_size())):
            _check(lib().zi_rglru_scan_chunked(
                _ptr(out), out.stride(0), _ptr(work), _ptr(u), _ptr(gates), block_width, _ptr(r_bias), _ptr(i_bias), _ptr(lam),
                ctypes.c_float(decay_scale), _ptr(y), y.stride(0), _ptr(y_bias), _ptr(x), x.stride(0), _ptr(x_bias), _tag(y),
                _ptr(state), C, taps, _ptr(step.cu_q), _ptr(step.state_slots), step.n_seqs, T, RGLRU_CHUNK, _stream()),
                "rglru_scan_chunked")
        return out
    with _prof.region("rglru scan", lambda: T * C * (12 + 3 * y.element_size())):
        _check(lib().zi_rglru_scan(_ptr(out), out.stride(0), _ptr(u), _ptr(gates), block_width, _ptr(r_bias), _ptr(i_bias),
                                   _ptr(lam), ctypes.c_float(decay_scale), _ptr(y), y.stride(0), _ptr(y_bias), _ptr(x),
                                   x.stride(0), _ptr(x_bias), _tag(y), _ptr(state), C, taps, _ptr(step.cu_q),
                                   _ptr(step.state_slots), step.n_seqs, _stream()), "rglru_scan")
    return out


def rglru_decode(yx: torch.Tensor, y_bias: torch.Tensor, x_bias: torch.Tensor, kernel: torch.Tensor, bias: torch.Tensor,
                 w_gates: torch.Tensor, r_bias: torch.Tensor, i_bias: torch.Tensor, lam: torch.Tensor,
                 decay_scale: float, state: torch.Tensor, step) -> torch.Tensor:
    """:func:`causal_conv`, the gates' products and :func:`rglru_scan` in one kernel, for a step in which every
    request brings one token.  ``yx`` [n, 2C]: the y branch, then the x branch, before their biases;
    ``w_gates`` [blocks, 2 * block_width, block_width]."""
    n, two_c = yx.shape
    C = two_c // 2
    taps = state.shape[1]
    B, two_bw, bw = w_gates.shape
    _need(yx.is_contiguous() and B * bw == C and two_bw == 2 * bw and w_gates.is_contiguous()
          and state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (taps, C),
          "rglru_decode: shapes")
    _need(n == step.n_seqs, "rglru_decode: every request brings exactly one token")
    out = torch.empty((n, C), dtype=yx.dtype, device=yx.device)
    with _prof.region("rglru decode (conv, gates, recurrence)", lambda: _nb(w_gates, yx, out) + 2 * n * taps * C * 4,
                      4 * n * C * bw):
        _check(lib().zi_rglru_decode(_ptr(out), out.stride(0), _ptr(yx), yx.stride(0), _tag(yx), _ptr(y_bias), _ptr(x_bias),
                                     _ptr(kernel), _ptr(bias), _ptr(w_gates), _tag(w_gates), bw, _ptr(r_bias), _ptr(i_bias),
                                     _ptr(lam), ctypes.c_float(decay_scale), _ptr(state), C, taps, _ptr(step.state_slots),
                                     n, _stream()), "rglru_decode")
    return out


# ----------------------------------------------------------------- latent attention
def latent_prepare(proj: torch.Tensor, heads: int, dim: int, rot_dim: int, rank: int, rot_dims: int,
                   c_weight: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
                   q_eff: torch.Tensor, cache: Optional[torch.Tensor], slots: Optional[torch.Tensor]) -> None:
    """From a token's projections [q heads (dim | rot_dim) | rank | rot_dim | ...]: the rotated query part
    of every head goes to ``q_eff[t, h, rank:]``; the RMS-normed latent and the rotated key part go into
    the token's cache row (``cache`` [pages, 1, page_size, rank + rot_dim], row ``slots[t]``)."""
    T = proj.shape[0]
    D = rank + rot_dim
    _need(proj.stride(1) == 1 and proj.shape[1] >= heads * (dim + rot_dim) + D, "latent_prepare: projection rows")
    _need(q_eff.is_contiguous() and q_eff.dtype == proj.dtype and q_eff.numel() == T * heads * D, "latent_prepare: q_eff")
    _need(c_weight.dtype == torch.float32 and c_weight.numel() == rank, "latent_prepare: the latent's norm weight")
    _need(cos.dtype == torch.float32 and cos.shape == sin.shape and cos.shape[1] == rot_dims // 2, "latent_prepare: tables")
    if cache is not None:
        _need(cache.is_contiguous() and cache.dtype == proj.dtype and cache.shape[-1] == D and cache.shape[1] == 1,
              "latent_prepare: cache rows")
        _i32(slots, "slots")
    with _prof.region("latent prepare", lambda: 2 * T * (heads * rot_dim + D) * proj.element_size()):
        _check(lib().zi_latent_prepare(_ptr(proj), proj.stride(0), _tag(proj), T, heads, dim, rot_dim, rank, rot_dims,
                                       _ptr(c_weight), ctypes.c_float(eps), _ptr(cos), _ptr(sin), cos.shape[0],
                                       _ptr(_i32(positions, "positions")), _ptr(q_eff), _ptr(cache), _ptr(slots),
                                       1 if cache is not None else 0, _stream()), "latent_prepare")


def latent_prepare_rows(q: torch.Tensor, kv: torch.Tensor, heads: int, dim: int, rot_dim: int, rank: int, rot_dims: int,
                        neighbours: bool, c_weight: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor,
                        positions: torch.Tensor, q_eff: torch.Tensor, cache: Optional[torch.Tensor],
                        slots: Optional[torch.Tensor]) -> None:
    """:func:`latent_prepare` with the queries [T, heads * (dim + rot_dim)] and the rows [T, rank + rot_dim] in tensors
    (or views) of their own, each 32-bit or of ``q_eff``'s type, and with the rotation's pairs (i, i + rot_dims/2) or, with
    ``neighbours``, (2i, 2i + 1)."""
    T = q.shape[0]
    D = rank + rot_dim
    _need(q.stride(1) == 1 and q.shape[1] >= heads * (dim + rot_dim) and kv.stride(1) == 1 and kv.shape[1] >= D,
          "latent_prepare: projection rows")
    _need(q_eff.is_contiguous() and q_eff.numel() == T * heads * D, "latent_prepare: q_eff")
    _need(c_weight.dtype == torch.float32 and c_weight.numel() == rank, "latent_prepare: the latent's norm weight")
    _need(cos.dtype == torch.float32 and cos.shape == sin.shape and cos.shape[1] == rot_dims // 2, "latent_prepare: tables")
    if cache is not None:
        _need(cache.is_contiguous() and cache.dtype == q_eff.dtype and cache.shape[-1] == D and cache.shape[1] == 1,
              "latent_prepare: cache rows")
        _i32(slots, "slots")
    with _prof.region("latent prepare", lambda: T * (heads * rot_dim * (q.element_size() + q_eff.element_size())
                                                     + D * (kv.element_size() + q_eff.element_size()))):
        _check(lib().zi_latent_prepare_rows(_ptr(q), q.stride(0), _tag(q), _ptr(kv), kv.stride(0), _tag(kv), _tag(q_eff), T, heads,
                                            dim, rot_dim, rank, rot_dims, 1 if neighbours else 0, _ptr(c_weight),
                                            ctypes.c_float(eps), _ptr(cos), _ptr(sin), cos.shape[0],
                                            _ptr(_i32(positions, "positions")), _ptr(q_eff), _ptr(cache), _ptr(slots),
                                            1 if cache is not None else 0, _stream()), "latent_prepare")


# A request that brings this many tokens or more in a bfloat16 step has its latent attention on the
# tensor cores (two products around a causal softmax); fewer go to the exact kernel.
LATENT_TENSOR_MIN_TOKENS = 32
LATENT_QUERY_BLOCK = 512      # queries per pair of products of a long portion


def latent_attention(q_eff: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, step, heads: int, rank: int,
                     page_size: int, window: Optional[int], scale: float,
                     sink_logit: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal softmax attention of ``q_eff`` [T, heads * D] over the latent rows of each request's pages
    (``cache`` [pages, 1, page_size, D]): scores over all D columns, values the first ``rank`` columns.
    Returns [T, heads * rank].

    In float32, and for requests that bring few tokens, the exact kernel on the CUDA cores.  In bfloat16 a
    request's longer portion runs as two tcgen05 products: its cached rows are gathered from the pages (once
    as they are, once with the latent part transposed), S = Q rows^T in 32-bit, a causal softmax in 32-bit
    that writes each weight as a high and a low bfloat16 part (16 bits together: rounding the weights to 8
    bits moved results by more than the rest of a bfloat16 layer does), then [high | low] times the latent
    part held twice.  The scores of a portion against all its keys
    pass through memory; a portion of 2,048 tokens of 16 heads against 2,048 keys holds 268 MB for that."""
    T = q_eff.shape[0]
    D = cache.shape[-1]
    _need(q_eff.shape[1] == heads * D and q_eff.is_contiguous() and cache.is_contiguous() and cache.dtype == q_eff.dtype,
          "latent_attention: shapes")
    out = torch.empty((T, heads * rank), dtype=q_eff.dtype, device=q_eff.device)
    skip_from = skip_single = 0
    n_dec = int(getattr(step, "n_dec", 0) or 0)
    _score_changes_ok(heads, sink_logit, None)
    win = int(window or 0)
    if n_dec > 0 and rank <= 640 and D % 4 == 0 and ATTENTION_BACKEND != "generic":
        # requests that bring one token: split-key kernel, every cached row fetched once for 16 heads
        longest = step.max_kv_len if not win else min(step.max_kv_len or win, win)
        splits = latent_decode_splits(n_dec, -(-heads // 16), _sm_count(q_eff.device), longest,
                                      fixed=q_eff.dtype == torch.float32)
        need = lib().zi_latent_decode_workspace_floats(n_dec, heads, rank, splits)
        ws = torch.empty((need,), dtype=torch.float32, device=q_eff.device) if need else None
        seen = lambda c: min(c + 1, win) if win else c + 1
        with _prof.region("latent attention (decode, split keys)",
                          lambda: sum(seen(c) * D for q_, c in zip(step.q_lens, step.ctx_lens) if q_ == 1) * q_eff.element_size(),
                          sum(2 * heads * seen(c) * (D + rank) for q_, c in zip(step.q_lens, step.ctx_lens) if q_ == 1)):
            _check(lib().zi_latent_decode_mods(
                _ptr(out), out.stride(0), _ptr(ws), _ptr(q_eff), q_eff.stride(0), _tag(q_eff), _ptr(cache),
                _ptr(_i32(block_tables, "block_tables")), block_tables.stride(0), _ptr(step.cu_q), _ptr(step.kv_lens),
                _ptr(step.dec_seq), n_dec, heads, D, rank, page_size, ctypes.c_float(scale), splits, win, _ptr(sink_logit),
                _stream()), "latent_decode")
        if n_dec == step.n_seqs:
            return out
        skip_single = 1
    if (q_eff.dtype == torch.bfloat16 and GEMM_BACKEND != "simt" and ATTENTION_BACKEND != "generic"
            and D % 8 == 0 and rank % 8 == 0 and getattr(step, "q_lens", None)
            and max(step.q_lens) >= LATENT_TENSOR_MIN_TOKENS):
        skip_from = LATENT_TENSOR_MIN_TOKENS
        t0 = 0
        for s, (n, ctx) in enumerate(zip(step.q_lens, step.ctx_lens)):
            if n >= skip_from:
                _latent_attention_portion(q_eff[t0:t0 + n], out[t0:t0 + n], cache, block_tables[s], heads, rank, D,
                                          page_size, ctx, scale, win, sink_logit)
            t0 += n
        if all(n >= skip_from or (n == 1 and skip_single) for n in step.q_lens):
            return out
    with _prof.region("latent attention (exact, CUDA cores)"):
        _check(lib().zi_paged_attention_mods(
            _ptr(out), out.stride(0), _ptr(q_eff), q_eff.stride(0), _tag(q_eff), _ptr(cache), _ptr(cache),
            _ptr(_i32(block_tables, "block_tables")), block_tables.stride(0), _ptr(step.cu_q), _ptr(step.kv_lens),
            _ptr(step.tile_seq), _ptr(step.tile_q0), step.tile_seq.shape[0], heads, 1, D, rank, D, page_size,
            int(window or 0), 0, ctypes.c_float(scale), skip_from, skip_single, ctypes.c_float(0.0), _ptr(sink_logit),
            ctypes.c_float(0.0), None, 0, _stream()), "latent_attention")
    return out


def latent_decode_splits(n_dec: int, head_groups: int, sm_count: int, max_kv_len: Optional[int], fixed: bool = False) -> int:
    """Key splits of the latent decode kernel: its blocks are (split, request, group of 16 heads), two fit on an
    SM, and a block walks its keys in tiles of 32; as many splits as fill the GPU about once, at most one per
    two tiles of the longest request and at most 32.  ``fixed`` (the 32-bit path): always 8, so that the order
    in which a request's keys are added does not depend on what else is in the batch."""
    if fixed:
        return 8
    tiles = -(-(max_kv_len or 2048) // 32)
    want = (2 * sm_count) // max(1, n_dec * head_groups)
    return max(1, min(want, tiles // 2, 32))


def _latent_attention_portion(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                              heads: int, rank: int, D: int, page_size: int, ctx: int, scale: float, window: int = 0,
                              sink_logit: Optional[torch.Tensor] = None) -> None:
    """One request's portion of ``n`` tokens that follow ``ctx`` cached ones, on the tensor cores.  With a window the
    keys are gathered from the first one the portion's first query sees (rounded down to a multiple of 8: rows of 16
    bytes), and a block of queries multiplies with the keys from its own first visible one up to its last position."""
    n = q.shape[0]
    first = max(0, ctx - window + 1) if window else 0        # the first key any query of the portion sees
    start = first // 8 * 8
    kv = ctx + n - start
    kv_pad = -(-kv // 8) * 8                      # rows of 16 bytes for the second product
    dev = q.device
    keys = torch.empty((kv_pad, D), dtype=q.dtype, device=dev)
    values_t = torch.empty((rank, 2 * kv_pad), dtype=q.dtype, device=dev)    # twice: for the weights' high and low parts
    with _prof.region("latent attention: gather rows", lambda: 2 * _nb(keys) + _nb(values_t)):
        _check(lib().zi_latent_gather_from(_ptr(keys), _ptr(values_t), _ptr(cache), _tag(cache),
                                           _ptr(_i32(block_table, "block_table")), page_size, kv, kv_pad, D, rank, start, first,
                                           _stream()), "latent_gather")
    # in blocks of queries: a block multiplies with the keys up to its own last position only (and from its first
    # visible key on), so about five eighths of the rectangle of a whole prompt are computed instead of all of it
    plain = not window and sink_logit is None
    for q0 in range(0, n, LATENT_QUERY_BLOCK):
        q1 = min(n, q0 + LATENT_QUERY_BLOCK)
        rows_b = (q1 - q0) * heads
        k0 = (max(0, ctx + q0 - window + 1) // 8 * 8 - start) if window else 0       # in rows of `keys`
        k0 = max(k0, 0)
        k1 = min(kv_pad, -(-(ctx + q1 - start) // 8) * 8)
        kvb = k1 - k0
        scores = linear(q[q0:q1].view(rows_b, D), keys[k0:k1], out_dtype=torch.float32, fresh_weight=True)
        probs = torch.empty((rows_b, 2 * kvb), dtype=q.dtype, device=dev)
        with _prof.region("latent attention: causal softmax", lambda: _nb(scores, probs)):
            if plain:
                _check(lib().zi_causal_softmax(_ptr(probs), _ptr(scores), _tag(probs), ctypes.c_longlong(rows_b), heads, ctx + q0,
                                               kvb, ctypes.c_float(scale), _stream()), "causal_softmax")
            else:
                _check(lib().zi_window_softmax(_ptr(probs), _ptr(scores), _tag(probs), ctypes.c_longlong(rows_b), heads, ctx + q0,
                                               start + k0, kvb, window, ctypes.c_float(scale), _ptr(sink_logit), _stream()),
                       "window_softmax")
        linear(probs, values_t[:, 2 * k0:2 * k1], out=out[q0:q1].view(rows_b, rank), fresh_weight=True)


# ----------------------------------------------------------------------- attention
def attention_tile_rows() -> int:
    return int(lib().zi_paged_attention_tile_rows())


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                    cu_q: torch.Tensor, kv_lens: torch.Tensor, tile_seq: torch.Tensor, tile_q0: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int],
                    scale: float, out: Optional[torch.Tensor] = None, sink: float = 0.0, keep_first: int = 0,
                    value_dim: Optional[int] = None, sink_logit: Optional[torch.Tensor] = None, softcap: float = 0.0,
                    dist_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of the step's query tokens over their requests' pages.  Changes to the score, each off unless
    given: ``softcap`` c (s <- c tanh(s / c) after the scale); ``dist_bias`` (float32 [heads, n]: entry [h, i - j] is
    added for a key i - j tokens back, distances from n - 1 on share the last entry; neither scaled nor capped);
    ``sink_logit`` (float32 [heads]: exp(sink_logit[h]) joins head h's denominator and has no value).  ``sink``: that many keys of
    score 0 without a value are counted in the softmax's denominator (p_j = exp(s_j) / (sink + sum exp(s))).
    ``keep_first``: with a window, a request's first tokens that stay visible beyond it (query i sees key j <= i if
    i - j < window or j < keep_first).  ``value_dim``: the values' size where it differs from the keys'.

    ``q`` [T, >= num_heads*head_dim] (row stride free), caches [pages, kv heads,
    page_size, head_dim], ``block_tables`` [n, W], ``cu_q`` [n+1] token offsets,
    ``kv_lens`` [n] keys per request including this step's tokens, ``tile_seq`` and
    ``tile_q0`` the request and first token of each query tile."""
    T = q.shape[0]
    _need(q.stride(1) == 1, "q rows must be dense")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache pages must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache pages are [pages, kv heads, page, d]")
    _need(k_cache.dtype == q.dtype, "cache pages have the activations' dtype")
    dv = int(value_dim or head_dim)
    _need(tuple(v_cache.shape[1:]) == (num_kv_heads, page_size, dv) and v_cache.dtype == q.dtype,
          "value pages are [pages, kv heads, page, value size]")
    for name, t in (("block_tables", block_tables), ("cu_q", cu_q), ("kv_lens", kv_lens), ("tile_seq", tile_seq),
                    ("tile_q0", tile_q0)):
        _i32(t, name)
    if out is None:
        out = torch.empty((T, num_heads * dv), dtype=q.dtype, device=q.device)
    _score_changes_ok(num_heads, sink_logit, dist_bias)
    with _prof.region("attention (exact, CUDA cores)"):
        _check(lib().zi_paged_attention_mods(
            _ptr(out), out.stride(0), _ptr(q), q.stride(0), _tag(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
            block_tables.stride(0), _ptr(cu_q), _ptr(kv_lens), _ptr(tile_seq), _ptr(tile_q0), tile_seq.shape[0],
            num_heads, num_kv_heads, head_dim, dv, dv, page_size, int(window or 0), int(keep_first or 0),
            ctypes.c_float(scale), 0, 0, ctypes.c_float(sink), _ptr(sink_logit), ctypes.c_float(softcap), _ptr(dist_bias),
            dist_bias.shape[1] if dist_bias is not None else 0, _stream()), "paged_attention")
    return out


def _score_changes_ok(num_heads: int, sink_logit: Optional[torch.Tensor], dist_bias: Optional[torch.Tensor]) -> None:
    if sink_logit is not None:
        _need(sink_logit.dtype == torch.float32 and sink_logit.numel() == num_heads and sink_logit.is_contiguous(),
              "a learned sink is float32, one value per query head")
    if dist_bias is not None:
        _need(dist_bias.dtype == torch.float32 and dist_bias.dim() == 2 and dist_bias.shape[0] == num_heads
              and dist_bias.is_contiguous(), "a bias by distance is float32 [heads, distances]")


ATTENTION_BACKEND = os.environ.get("ZINFER_B200_ATTENTION", "auto")   # auto | generic
# Which tensor-core prefill kernel: "tcgen05" (S, P and O in tensor memory, TMA-fed, two query
# tiles per CTA so that one tile's softmax runs under the other's products: 61 us for a prompt of
# 2,048 tokens of 32 heads of 128, head size 128 only) with "mma" (mma.sync flash attention, 160 us)
# for the shapes the first does not take; or "mma" always.
PREFILL_ATTENTION = os.environ.get("ZINFER_B200_PREFILL_ATTENTION", "tcgen05")


def _attention_work(step, decode: bool, num_heads: int, num_kv_heads: int, head_dim: int, elt: int,
                    window: int = 0, keep_first: int = 0) -> tuple[int, int]:
    """(bytes, flops) of the attention of a step's decode requests (one token) or of its others:
    every key and value that those requests' queries can see once (all of them, or with a window the last
    ``window`` + q - 1 and the first ``keep_first``), their queries and outputs; 4 d per visible (query, key) pair."""
    nbytes = flops = 0
    for q, c in zip(step.q_lens, step.ctx_lens):
        if (q == 1) != decode:
            continue
        keys = c + q
        pairs = q * c + q * (q + 1) // 2
        if window and window > 0:
            keys = min(keys, window + q - 1 + int(keep_first or 0))
            pairs = sum(min(p + 1, window + min(int(keep_first or 0), max(0, p + 1 - window))) for p in range(c, c + q))
        nbytes += 2 * keys * num_kv_heads * head_dim * elt + 2 * q * num_heads * head_dim * elt
        flops += 4 * num_heads * head_dim * pairs
    return nbytes, flops


def attention_prefill_tile_rows() -> int:
    return int(lib().zi_attention_prefill_tile_rows())


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor, step,
              num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int],
              scale: float, sink: float = 0.0, keep_first: int = 0, value_dim: Optional[int] = None,
              sink_logit: Optional[torch.Tensor] = None, softcap: float = 0.0,
              dist_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of a step's query tokens over their pages, by the fastest kernel that
    takes the shape: in bfloat16 with head sizes 64/128 (decode also 256) the
    tensor-core kernels (requests that bring one token go to the split-key decode
    kernel, the others to the prefill kernel); otherwise, and always in float32, the
    exact CUDA-core kernel.  ``step`` is the StepContext (its request arrays)."""
    T = q.shape[0]
    L = lib()
    keep_first = int(keep_first or 0) if window else 0
    same_size = value_dim is None or int(value_dim) == head_dim
    # the tensor-core kernels take values of the keys' size; kept first tokens only in the form with a sink
    changed = sink_logit is not None or bool(softcap) or dist_bias is not None
    fast = ATTENTION_BACKEND != "generic" and q.dtype == torch.bfloat16 and same_size and (not keep_first or bool(sink)) \
        and not (changed and (sink or keep_first))
    dec_ok = fast and step.n_dec > 0 and L.zi_attention_mma_supported(num_heads, num_kv_heads, head_dim, 1)
    pf_ok = fast and step.n_pf_tiles > 0 and L.zi_attention_mma_supported(num_heads, num_kv_heads, head_dim, 0) \
        and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
    if (step.n_dec > 0 and not dec_ok) or (step.n_pf_tiles > 0 and not pf_ok):
        return paged_attention(q, k_cache, v_cache, block_tables, step.cu_q, step.kv_lens, step.tile_seq, step.tile_q0,
                               num_heads, num_kv_heads, head_dim, page_size, window, scale, sink=sink,
                               keep_first=keep_first, value_dim=value_dim, sink_logit=sink_logit, softcap=softcap,
                               dist_bias=dist_bias)
    _need(q.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous(), "attention: dense operands")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim) and k_cache.dtype == q.dtype,
          "cache pages are [pages, kv heads, page, d] in the activations' dtype")
    out = torch.empty((T, num_heads * head_dim), dtype=q.dtype, device=q.device)
    win = int(window or 0)
    work = lambda decode: _attention_work(step, decode, num_heads, num_kv_heads, head_dim, q.element_size(), win, keep_first) \
        if _prof.ACTIVE is not None else (0, 0)
    if changed:
        # changed scores (a cap, a bias by distance, a learned sink): the mma.sync kernels' form with exact weights
        _score_changes_ok(num_heads, sink_logit, dist_bias)
        n_dist = dist_bias.shape[1] if dist_bias is not None else 0
        if step.n_pf_tiles > 0:
            with _prof.region("attention (prefill, mma.sync, changed scores)", *work(False)):
                _check(L.zi_attention_prefill_mma_mods(
                    _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                    block_tables.stride(0), _ptr(step.cu_q), _ptr(step.kv_lens), _ptr(step.pf_tile_seq), _ptr(step.pf_tile_q0),
                    step.n_pf_tiles, num_heads, num_kv_heads, head_dim, page_size, win, ctypes.c_float(scale),
                    _ptr(sink_logit), ctypes.c_float(softcap), _ptr(dist_bias), n_dist, _stream()),
                    "attention (prefill, changed scores)")
        if step.n_dec > 0:
            splits = decode_splits(step.n_dec, num_kv_heads, _sm_count(q.device), step.max_kv_len if not win else min(step.max_kv_len or win, win))
            need = L.zi_attention_decode_workspace_floats(step.n_dec, num_heads, num_kv_heads, head_dim, splits)
            ws = torch.empty((need,), dtype=torch.float32, device=q.device) if need else None
            with _prof.region("attention (decode, changed scores)", *work(True)):
                _check(L.zi_attention_decode_mma_mods(
                    _ptr(out), out.stride(0), _ptr(ws), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache),
                    ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables), block_tables.stride(0), _ptr(step.cu_q),
                    _ptr(step.kv_lens), _ptr(step.dec_seq), step.n_dec, num_heads, num_kv_heads, head_dim, page_size, win,
                    ctypes.c_float(scale), splits, _ptr(sink_logit), ctypes.c_float(softcap), _ptr(dist_bias), n_dist,
                    _stream()), "attention (decode, changed scores)")
        return out
    if sink:
        # a softmax with a sink: the mma.sync kernels' form whose weights meet the values as two bfloat16 parts (a design
        # that has a sink also wants its softmax weights in 32-bit) and whose denominator counts the sink
        if step.n_pf_tiles > 0:
            with _prof.region("attention (prefill, mma.sync, sink)", *work(False)):
                _check(L.zi_attention_prefill_mma_mask(
                    _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                    block_tables.stride(0), _ptr(step.cu_q), _ptr(step.kv_lens), _ptr(step.pf_tile_seq), _ptr(step.pf_tile_q0),
                    step.n_pf_tiles, num_heads, num_kv_heads, head_dim, page_size, win, keep_first, ctypes.c_float(scale),
                    ctypes.c_float(sink), _stream()), "attention (prefill, sink)")
        if step.n_dec > 0:
            splits = decode_splits(step.n_dec, num_kv_heads, _sm_count(q.device), step.max_kv_len)
            need = L.zi_attention_decode_workspace_floats(step.n_dec, num_heads, num_kv_heads, head_dim, splits)
            ws = torch.empty((need,), dtype=torch.float32, device=q.device) if need else None
            with _prof.region("attention (decode, sink)", *work(True)):
                _check(L.zi_attention_decode_mma_mask(
                    _ptr(out), out.stride(0), _ptr(ws), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache),
                    ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables), block_tables.stride(0), _ptr(step.cu_q),
                    _ptr(step.kv_lens), _ptr(step.dec_seq), step.n_dec, num_heads, num_kv_heads, head_dim, page_size, win,
                    keep_first, ctypes.c_float(scale), splits, ctypes.c_float(sink), _stream()), "attention (decode, sink)")
        return out
    if step.n_pf_tiles > 0 and PREFILL_ATTENTION == "tcgen05" and L.zi_attention_prefill_tcgen05_supported(
            num_heads, num_kv_heads, head_dim, page_size, _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache)):
        with _prof.region("attention (prefill, tcgen05)", *work(False)):
            _check(L.zi_attention_prefill_tcgen05(
                _ptr(out), out.stride(0), _ptr(q), q.stride(0), T, _ptr(k_cache), _ptr(v_cache),
                ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables), block_tables.stride(0), _ptr(step.cu_q),
                _ptr(step.kv_lens), _ptr(step.pf_tile_seq), _ptr(step.pf_tile_q0), step.n_pf_tiles, num_heads, num_kv_heads,
                head_dim, page_size, win, ctypes.c_float(scale), _stream()), "attention (prefill, tcgen05)")
    elif step.n_pf_tiles > 0:
        with _prof.region("attention (prefill, mma.sync)", *work(False)):
            _check(L.zi_attention_prefill_mma(
                _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                block_tables.stride(0), _ptr(step.cu_q), _ptr(step.kv_lens), _ptr(step.pf_tile_seq), _ptr(step.pf_tile_q0),
                step.n_pf_tiles, num_heads, num_kv_heads, head_dim, page_size, win, ctypes.c_float(scale), _stream()),
                "attention (prefill)")
    if step.n_dec > 0:
        splits = decode_splits(step.n_dec, num_kv_heads, _sm_count(q.device), step.max_kv_len)
        need = L.zi_attention_decode_workspace_floats(step.n_dec, num_heads, num_kv_heads, head_dim, splits)
        ws = torch.empty((need,), dtype=torch.float32, device=q.device) if need else None
        with _prof.region("attention (decode)", *work(True)):
            _check(L.zi_attention_decode_mma(
                _ptr(out), out.stride(0), _ptr(ws), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache),
                ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables),
                block_tables.stride(0), _ptr(step.cu_q), _ptr(step.kv_lens), _ptr(step.dec_seq), step.n_dec, num_heads,
                num_kv_heads, head_dim, page_size, win, ctypes.c_float(scale), splits, _stream()), "attention (decode)")
    return out


def decode_splits(n_dec: int, num_kv_heads: int, sm_count: int, max_kv_len: Optional[int] = None,
                  fixed_us: float = 3.0) -> int:
    """Key splits of the decode attention.  Its blocks are (request, kv head, split), two fit on an SM
    at once, and a block costs a fixed time (``fixed_us``: launch, prologue, merge; more in the fused
    kernel, which also makes q, k and v) plus its share of the walk over the keys (about 0.02 us a key
    for a block's four warps).  Any split costs the kernel that merges the splits: about 5 us in the
    chain of a decode step, and 0.25 us more per split.  The split count (at most 32, never more than
    tiles of 64 keys) that makes the sum smallest; one, when the blocks already fill more than half of
    the GPU and the keys are few (measured at 24 to 128 requests of 2,048 keys: no split is 4 to 6 %
    of a layer faster than any split; at 16 requests two splits win, at 8 four, at one 12 to 16)."""
    slots, units = 2 * sm_count, max(1, n_dec * num_kv_heads)
    keys = max_kv_len if max_kv_len and max_kv_len > 0 else 2048
    if 2 * units > slots and keys <= 4096:
        return 1
    limit = max(1, min(32, -(-keys // 64)))
    walk = 0.02 * keys
    best, best_cost = 1, float("inf")
    for s in range(1, limit + 1):
        waves = -(-units * s // slots)
        cost = waves * (fixed_us + walk / s) + (5.0 + 0.25 * s if s > 1 else 0.0)
        if cost < best_cost:
            best, best_cost = s, cost
    return best


def decode_tma(mode) -> int:
    """The decode attention's keys and values by TMA (``cp.async.bulk.tensor`` page boxes, a few lanes
    issuing side by side; pages of 8, 16, 32, ... tokens) or by ``cp.async`` from every lane: 1 (the
    default) TMA for up to 16 requests, where it measured slightly faster, 2 or True always, 0 or False
    never.  Returns the setting before.  For tests and timing comparisons."""
    mode = 2 if mode is True else (0 if mode is False else int(mode))
    return int(lib().zi_attention_decode_tma(mode))


def decode_transposed_tile(on: bool) -> bool:
    """The decode attention's tile for groups of at most 8 query heads: with the keys on the MMA's rows
    (on, the default: half the MMAs and a quarter of the exponentials) or with the heads on them as
    for larger groups (off).  Returns the setting before.  For tests and timing comparisons."""
    return bool(lib().zi_attention_decode_transposed(1 if on else 0))


def decode_fused_ok(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int, step) -> bool:
    """Whether a step can use :func:`attention_decode_fused`: bfloat16, every request brings
    one token, and the split-key decode kernel takes the shape."""
    if not (ATTENTION_BACKEND != "generic" and dtype == torch.bfloat16 and step.n_pf_tiles == 0
            and step.n_dec > 0 and step.n_dec == step.n_seqs and torch.cuda.is_available()
            and lib().zi_attention_mma_supported(num_heads, num_kv_heads, head_dim, 1)):
        return False
    # Worth it while all blocks run at once (few requests: the step is a chain of short
    # kernels and one kernel less counts).  With more blocks than fit, the work every block
    # repeats before it streams its keys costs more than the separate kernel (measured at 64 requests).
    return step.n_dec * num_kv_heads <= 2 * _sm_count(torch.device("cuda", torch.cuda.current_device()))


def attention_decode_fused(qkv, num_heads: int, num_kv_heads: int, head_dim: int, q_weight: Optional[torch.Tensor],
                           k_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                           sin: Optional[torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor,
                           slots: torch.Tensor, block_tables: torch.Tensor, step, page_size: int,
                           window: Optional[int], scale: float) -> torch.Tensor:
    """q/k RMSNorm, rotary positions, the write of each token's key and value into its page
    and the attention itself in ONE kernel, for steps in which every request brings a single
    token.  ``qkv`` is the fused projection row as a tensor or as split-K partial sums."""
    L = lib()
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if isinstance(qkv, Partials):
        T = qkv.shape[0]
        _need(qkv.shape[1] == width, "partial sums must have exactly the heads' width")
        src, src_stride, part, psplits, pz = None, 0, qkv.data, qkv.splits, T * width
        device = qkv.data.device
    else:
        T = qkv.shape[0]
        _need(qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] >= width, "qkv rows are dense bfloat16")
        src, src_stride, part, psplits, pz = qkv, qkv.stride(0), None, 0, 0
        device = qkv.device
    _need(T == step.n_dec, "every request brings exactly one token")
    for wt in (q_weight, k_weight):
        if wt is not None:
            _need(wt.dtype == torch.float32 and wt.numel() == head_dim, "q/k norm weights are float32 [head_dim]")
    n_table = 0
    if cos is not None:
        _need(cos.shape == sin.shape and cos.shape[1] == head_dim // 2 and cos.dtype == torch.float32,
              "rotary tables are float32 [positions, head_dim/2]")
        n_table = cos.shape[0]
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == torch.bfloat16
          and tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache pages are bfloat16 [pages, kv heads, page, d]")
    _i32(slots, "slots")
    out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=device)
    splits = decode_splits(step.n_dec, num_kv_heads, _sm_count(device), step.max_kv_len, fixed_us=8.0)
    need = L.zi_attention_decode_workspace_floats(step.n_dec, num_heads, num_kv_heads, head_dim, splits)
    ws = torch.empty((need,), dtype=torch.float32, device=device) if need else None
    work = _attention_work(step, True, num_heads, num_kv_heads, head_dim, 2) if _prof.ACTIVE is not None else (0, 0)
    with _prof.region("attention (decode, fused with q/k norm, rotary, cache write)", work[0] + _nb(part), work[1]):
        _check(L.zi_attention_decode_fused(
            _ptr(out), out.stride(0), _ptr(ws), _ptr(src), src_stride, _ptr(part), psplits, ctypes.c_longlong(pz),
            _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps), _ptr(cos), _ptr(sin), n_table, _ptr(step.positions),
            _ptr(slots), _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables),
            block_tables.stride(0), _ptr(step.cu_q),
            _ptr(step.kv_lens), _ptr(step.dec_seq), step.n_dec, num_heads, num_kv_heads, head_dim, page_size,
            int(window or 0), ctypes.c_float(scale), splits, _stream()), "attention (fused decode)")
    return out


# ------------------------------------------------- norm of a sublayer's output, small elementwise
def norm_residual(h: torch.Tensor, a, weight: torch.Tensor, eps: float, out_dtype: torch.dtype, b=None) -> torch.Tensor:
    """``h += rmsnorm(a + b) * weight`` in place, the norm taken over the sublayer's OUTPUT (``a``, and ``b`` if given:
    tensors, :class:`Partials` whose splits the kernel adds in order, or either inside :class:`Scaled`).  Returns ``h``
    in ``out_dtype``: what the next sublayer reads (``h`` itself for float32)."""
    T, H = h.shape
    _need(h.dtype == torch.float32 and h.is_contiguous(), "the residual stream is contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == H, "norm weight must be float32 of the row's width")

    def operand(delta):
        """(tensor, tag, partial sums, splits, stride between splits, multiplier)"""
        if delta is None:
            return None, F32, None, 0, 0, 0.0
        delta, scale = _unscaled(delta)
        if isinstance(delta, Partials):
            _need(tuple(delta.shape) == (T, H), "an update must match the residual stream")
            return None, F32, delta.data, delta.splits, T * H, scale
        _need(tuple(delta.shape) == (T, H) and delta.is_contiguous(), "an update must match the residual stream")
        return delta, _tag(delta), None, 0, 0, scale

    at, atag, ap, asplits, az, sa = operand(a)
    bt, btag, bp, bsplits, bz, sb = operand(b)
    _need(at is not None or ap is not None, "norm_residual: no update given")
    x = None if out_dtype == torch.float32 else torch.empty((T, H), dtype=out_dtype, device=h.device)
    with _prof.region("norm of the output + residual add", lambda: 2 * _nb(h) + _nb(at, bt, ap, bp, x)):
        _check(lib().zi_norm_residual(_ptr(h), _ptr(at), atag, _ptr(ap), asplits, _ll(az), ctypes.c_float(sa), _ptr(bt), btag,
                                      _ptr(bp), bsplits, _ll(bz), ctypes.c_float(sb), _ptr(weight), ctypes.c_float(eps), _ptr(x),
                                      _tag(x) if x is not None else F32, T, H, _stream()), "norm_residual")
    return h if x is None else x


def cast_rows(h: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The 32-bit residual stream in the activations' type (itself for float32)."""
    if dtype == torch.float32:
        return h
    _need(h.dtype == torch.float32 and h.is_contiguous(), "cast_rows: contiguous float32")
    out = torch.empty(h.shape, dtype=dtype, device=h.device)
    with _prof.region("cast", lambda: _nb(h, out)):
        _check(lib().zi_cast_rows(_ptr(out), _tag(out), _ptr(h), ctypes.c_longlong(h.numel()), _stream()), "cast_rows")
    return out


def relu2_(x: torch.Tensor) -> torch.Tensor:
    """``x = relu(x)^2`` in place."""
    _need(x.is_contiguous(), "relu2: a contiguous tensor")
    with _prof.region("relu2", lambda: 2 * _nb(x)):
        _check(lib().zi_relu2(_ptr(x), _tag(x), ctypes.c_longlong(x.numel()), _stream()), "relu2")
    return x


# ------------------------------------------- mixers with a matrix-valued state per head
def _slot_view(state: torch.Tensor, name: str):
    """(tensor, elements from one slot to the next) of a float32 per-request state that may be a view of wider rows."""
    if state.numel() == 0:
        return state, 0
    _need(state.dtype == torch.float32 and state.dim() >= 2 and all(
        state.stride(i) == state.stride(i + 1) * state.shape[i + 1] for i in range(1, state.dim() - 1)) and state.stride(-1) == 1,
        f"{name}: a float32 state whose slots are dense")
    return state, state.stride(0)


def short_conv(x: torch.Tensor, kernel: torch.Tensor, tail: torch.Tensor, step, activation: Optional[str] = "silu") -> torch.Tensor:
    """Causal convolution per channel over the last ``taps`` tokens of each request: ``x`` [T, C] (rows may be views of
    wider rows), ``kernel`` float32 [C, taps] (last column: the current token), no bias; the inputs before a
    request's first token of this step come from ``tail`` [slots, taps-1, C] (oldest first; zero at a request's
    start).  Returns float32 [T, C], with ``silu`` applied if asked.  The tail is left as it is
    (:func:`short_conv_carry` moves it on, after every reader of the old one)."""
    T, C = x.shape
    taps = kernel.shape[1]
    tail, stride = _slot_view(tail, "short_conv")
    _need(x.stride(1) == 1 and kernel.dtype == torch.float32 and kernel.is_contiguous() and kernel.shape[0] == C
          and tuple(tail.shape[1:]) == (max(taps - 1, 0), C), "short_conv: kernel float32 [C, taps], tail [slots, taps-1, C]")
    _need(activation in (None, "silu"), f"short_conv: unknown activation {activation!r}")
    y = torch.empty((T, C), dtype=torch.float32, device=x.device)
    with _prof.region("short convolution", lambda: T * C * (x.element_size() * taps + 4)):
        _check(lib().zi_short_conv(_ptr(y), y.stride(0), _ptr(x), x.stride(0), _tag(x), _ptr(kernel), _ptr(tail), _ll(stride), C,
                                   taps, 1 if activation == "silu" else 0, _ptr(step.cu_q), _ptr(step.state_slots), step.n_seqs,
                                   T, _stream()), "short_conv")
    return y


def short_conv_carry(x: torch.Tensor, taps: int, tail: torch.Tensor, step) -> None:
    """Moves ``tail`` on to the last ``taps - 1`` inputs of every request after this step's tokens."""
    T, C = x.shape
    if taps <= 1:
        return
    tail, stride = _slot_view(tail, "short_conv_carry")
    _need(x.stride(1) == 1 and tuple(tail.shape[1:]) == (taps - 1, C), "short_conv_carry: tail [slots, taps-1, C]")
    with _prof.region("short convolution (carry)", lambda: 2 * step.n_seqs * (taps - 1) * C * 4):
        _check(lib().zi_short_conv_carry(_ptr(tail), _ll(stride), _ptr(x), x.stride(0), _tag(x), C, taps, _ptr(step.cu_q),
                                         _ptr(step.state_slots), step.n_seqs, _stream()), "short_conv_carry")


def decay_sigmoid_root_(z: torch.Tensor, bias: Optional[torch.Tensor], tau: float) -> torch.Tensor:
    """In place on float32 [T, N]: ``sigmoid(z + bias)^(1/tau)``, as ``exp(log_sigmoid(z + bias) / tau)``."""
    _need(z.dtype == torch.float32 and z.is_contiguous(), "decay: contiguous float32")
    N = z.shape[-1]
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N, "decay: bias float32 [N]")
    with _prof.region("decay", lambda: 2 * _nb(z)):
        _check(lib().zi_decay(_ptr(z), _ll(z.numel() // N), N, N, _ptr(bias), None, ctypes.c_float(1.0 / tau), 0, _stream()), "decay")
    return z


def decay_exp_softplus_(z: torch.Tensor, bias: Optional[torch.Tensor], a_log: torch.Tensor, head_dim: int) -> torch.Tensor:
    """In place on float32 [T, heads * head_dim]: ``exp(-exp(a_log[head]) * softplus(z + bias))``."""
    _need(z.dtype == torch.float32 and z.is_contiguous(), "decay: contiguous float32")
    N = z.shape[-1]
    _need(a_log.dtype == torch.float32 and a_log.numel() * head_dim == N, "decay: a_log float32 [heads]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N, "decay: bias float32 [N]")
    with _prof.region("decay", lambda: 2 * _nb(z)):
        _check(lib().zi_decay(_ptr(z), _ll(z.numel() // N), N, head_dim, _ptr(bias), _ptr(a_log), ctypes.c_float(1.0), 1,
                              _stream()), "decay")
    return z


def unit_norm_(x: torch.Tensor, heads: int, head_dim: int, eps: float, scale: float = 1.0) -> torch.Tensor:
    """In place on float32 rows [T, >= heads * head_dim]: every head ``scale * x / sqrt(sum(x^2) + eps)``."""
    _need(x.dtype == torch.float32 and x.stride(1) == 1 and x.shape[1] >= heads * head_dim, "unit_norm: float32 rows")
    with _prof.region("unit norm", lambda: 2 * x.shape[0] * heads * head_dim * 4):
        _check(lib().zi_unit_norm(_ptr(x), x.stride(0), x.shape[0], heads, head_dim, ctypes.c_float(eps), ctypes.c_float(scale),
                                  _stream()), "unit_norm")
    return x


def sigmoid_rows(x: torch.Tensor) -> torch.Tensor:
    """float32 ``sigmoid(x)`` of [T, W] rows that may be views of wider rows."""
    T, W = x.shape
    _need(x.stride(1) == 1, "sigmoid_rows: dense rows")
    out = torch.empty((T, W), dtype=torch.float32, device=x.device)
    with _prof.region("sigmoid", lambda: T * W * (4 + x.element_size())):
        _check(lib().zi_sigmoid_rows(_ptr(out), W, _ptr(x), x.stride(0), _tag(x), T, W, _stream()), "sigmoid_rows")
    return out


def linear_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: Optional[torch.Tensor],
                      q_scale: float, state: torch.Tensor, heads: int, key_heads: int, dim: int, vdim: int, step) -> torch.Tensor:
    """Per request and head, over the step's tokens, from and to ``state`` [slots, heads, dim, vdim] (float32):
    ``S = diag(decay_t) S``; ``u = v_t`` or, with ``beta``, ``beta_t (v_t - S^T k_t)`` (the delta rule);
    ``S += k_t u^T``; ``o_t = S^T (q_scale q_t)``.  ``q``, ``k`` [T, key_heads * dim] (head h reads key head
    h // (heads / key_heads)), ``v`` [T, heads * vdim], ``decay`` float32 [T, heads * dim], ``beta`` float32 [T, heads];
    rows may be views of wider rows.  Returns float32 [T, heads * vdim]."""
    T = q.shape[0]
    state, stride = _slot_view(state, "linear_recurrence")
    _need(state[0].numel() == heads * dim * vdim, "linear_recurrence: state [slots, heads, dim, vdim]")
    _need(q.dtype == k.dtype and q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
          and q.shape[1] == key_heads * dim and k.shape[1] == key_heads * dim and v.shape[1] == heads * vdim,
          "linear_recurrence: q, k [T, key heads * dim], v [T, heads * vdim] with dense rows")
    _need(decay.dtype == torch.float32 and decay.stride(1) == 1 and decay.shape[1] == heads * dim, "linear_recurrence: decay")
    if beta is not None:
        _need(beta.dtype == torch.float32 and beta.stride(1) == 1 and beta.shape[1] == heads, "linear_recurrence: beta")
    out = torch.empty((T, heads * vdim), dtype=torch.float32, device=q.device)
    with _prof.region("linear recurrence" + (" (delta rule)" if beta is not None else ""),
                      lambda: _nb(q, k, v, decay, out) + 2 * step.n_seqs * heads * dim * vdim * 4, 6 * T * heads * dim * vdim):
        _check(lib().zi_linear_recurrence(
            _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _tag(q), _ptr(v), v.stride(0), _tag(v),
            _ptr(decay), decay.stride(0), _ptr(beta), beta.stride(0) if beta is not None else 0, ctypes.c_float(q_scale),
            _ptr(state), _ll(stride), heads, key_heads, dim, vdim, 1 if beta is not None else 0, _ptr(step.cu_q),
            _ptr(step.state_slots), step.n_seqs, _stream()), "linear_recurrence")
    return out


def head_norm_gate(o: torch.Tensor, weight: torch.Tensor, eps: float, gate: torch.Tensor, gate_kind: str, heads: int, vdim: int,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """Every head of float32 ``o`` [T, heads * vdim] divided by its root mean square (``eps`` inside the root), times
    ``weight`` [vdim], times ``silu(gate)`` or ``sigmoid(gate)`` (``gate`` [T, heads * vdim], rows may be views)."""
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and gate.stride(1) == 1 and gate.shape[1] == heads * vdim
          and weight.dtype == torch.float32 and weight.numel() == vdim, "head_norm_gate: shapes")
    _need(gate_kind in ("silu", "sigmoid"), f"head_norm_gate: unknown gate {gate_kind!r}")
    out = torch.empty((T, heads * vdim), dtype=out_dtype, device=o.device)
    with _prof.region("head norm + gate", lambda: _nb(o, out) + T * heads * vdim * gate.element_size()):
        _check(lib().zi_head_norm_gate(_ptr(out), _tag(out), out.stride(0), _ptr(o), o.stride(0), _ptr(weight), ctypes.c_float(eps),
                                       _ptr(gate), _tag(gate), gate.stride(0), 0 if gate_kind == "silu" else 1, T, heads, vdim,
                                       _stream()), "head_norm_gate")
    return out


def moe_router_grouped(x: torch.Tensor, w_router: torch.Tensor, top: int, score: str = "sigmoid", groups: int = 1, keep: int = 1,
                       scale: float = 1.0, renormalize: bool = False,
                       correction: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """The router's product (32-bit multiply-adds whatever the operands' types) and :func:`moe_route_grouped` in one
    kernel, one block per token."""
    if correction is not None:
        _need(correction.dtype == torch.float32 and correction.numel() == w_router.shape[0] and correction.is_contiguous(),
              "the correction is float32, one value per router output")
    T, K = x.shape
    NR = w_router.shape[0]
    _need(x.stride(1) == 1 and w_router.is_contiguous() and w_router.shape[1] == K, "moe_router: shapes")
    _need(score in ("softmax", "sigmoid"), f"unknown router score {score!r}")
    chosen = torch.empty((T, top), dtype=torch.int32, device=x.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=x.device)
    with _prof.region(f"moe router (groups) N={NR} K={K}", lambda: _nb(w_router) + T * K * x.element_size(), 2 * T * NR * K):
        _check(lib().zi_moe_router_grouped_c(_ptr(chosen), _ptr(weight), _ptr(x), _tag(x), x.stride(0), _ptr(w_router),
                                           _tag(w_router), _ptr(correction), T, K, NR, top, 1 if renormalize else 0,
                                           1 if score == "sigmoid" else 0, groups, keep, ctypes.c_float(scale), _stream()),
               "moe_router_grouped")
    return chosen, weight


def moe_router_top_logits(x: torch.Tensor, w_router: torch.Tensor, bias: Optional[torch.Tensor], top: int):
    """The router that chooses by its logits: ``z = x @ w_router^T + bias`` in 32-bit, the ``top`` largest chosen (ties to
    the lower index), weights = the softmax over the chosen logits alone; product and choice in one kernel.  Rows too
    long for its shared memory take the CUDA-core product and the choice as two kernels."""
    T, K = x.shape
    NR = w_router.shape[0]
    _need(x.stride(1) == 1 and w_router.is_contiguous() and w_router.shape[1] == K, "moe_router: shapes")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == NR and bias.is_contiguous(), "the router's bias is float32, one value per output")
    chosen = torch.empty((T, top), dtype=torch.int32, device=x.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=x.device)
    if K > 32768:
        logits = linear_cuda_cores(x, w_router, out_dtype=torch.float32)
        with _prof.region("moe route (largest logits)", lambda: _nb(logits, chosen, weight)):
            _check(lib().zi_moe_route_top_logits(_ptr(chosen), _ptr(weight), _ptr(logits), _ptr(bias), T, NR, top, _stream()),
                   "moe_route_top_logits")
        return chosen, weight
    with _prof.region(f"moe router (largest logits) N={NR} K={K}", lambda: _nb(w_router) + T * K * x.element_size(), 2 * T * NR * K):
        _check(lib().zi_moe_router_top_logits(_ptr(chosen), _ptr(weight), _ptr(x), _tag(x), x.stride(0), _ptr(w_router),
                                              _tag(w_router), _ptr(bias), T, K, NR, top, _stream()), "moe_router_top_logits")
    return chosen, weight


def moe_route_grouped(logits: torch.Tensor, top: int, score: str = "sigmoid", groups: int = 1, keep: int = 1,
                      scale: float = 1.0, renormalize: bool = False,
                      correction: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Per token: scores ``sigmoid(z)`` or ``softmax(z)``; the outputs form ``groups`` equal groups of neighbours, a
    group's score is the sum of its two largest scores, and the ``top`` largest scores are chosen among the outputs of
    the ``keep`` best groups (int32 [T, top]); their weights are the scores times ``scale`` (float32 [T, top]),
    divided by the chosen scores' sum first if ``renormalize``.  ``correction`` (float32 [outputs]) is added to the scores
    wherever they are compared, never to the weights."""
    T, NR = logits.shape
    if correction is not None:
        _need(correction.dtype == torch.float32 and correction.numel() == NR and correction.is_contiguous(),
              "the correction is float32, one value per router output")
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "router logits are contiguous float32")
    _need(score in ("softmax", "sigmoid"), f"unknown router score {score!r}")
    chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    with _prof.region("moe route (groups)", lambda: _nb(logits, chosen, weight)):
        _check(lib().zi_moe_route_grouped_c(_ptr(chosen), _ptr(weight), _ptr(logits), _ptr(correction), T, NR, top, 1 if renormalize else 0,
                                          1 if score == "sigmoid" else 0, groups, keep, ctypes.c_float(scale), _stream()),
               "moe_route_grouped")
    return chosen, weight


# ------------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits are float32 with dense rows")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    chunks = lib().zi_argmax_chunks(R, V)
    ws = torch.empty((2 * R * chunks,), dtype=torch.int32, device=logits.device) if chunks else None
    with _prof.region("argmax", lambda: R * V * 4):
        _check(lib().zi_argmax(_ptr(out), _ptr(logits), R, V, logits.stride(0), _ptr(ws), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, seeds: torch.Tensor, draw_index: torch.Tensor,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           min_p: Optional[torch.Tensor] = None, repetition_penalty: Optional[torch.Tensor] = None,
           presence_penalty: Optional[torch.Tensor] = None, frequency_penalty: Optional[torch.Tensor] = None,
           count_rows: Optional[torch.Tensor] = None, counts: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row.  Per-row parameters are device tensors: float32 for
    ``temperature``/``top_p``/``min_p``/penalties, int32 for ``top_k``,
    ``draw_index`` and ``count_rows``, int64 for ``seeds``.  ``counts`` [slots, V]
    int32 holds how often each token occurred in a request; the row named by
    ``count_rows`` is read for the penalties and incremented at the drawn token."""
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits are float32 with dense rows")
    for t in (temperature, top_p, min_p, repetition_penalty, presence_penalty, frequency_penalty):
        if t is not None:
            _need(t.dtype == torch.float32 and t.numel() == R, "per-row float parameters are float32 [rows]")
    for t in (top_k, draw_index, count_rows):
        if t is not None:
            _need(t.dtype == torch.int32 and t.numel() == R, "per-row integer parameters are int32 [rows]")
    _need(seeds.dtype == torch.int64 and seeds.numel() == R, "seeds are int64 [rows]")
    if counts is not None:
        _need(counts.dtype == torch.int32 and counts.shape[1] == V and counts.is_contiguous(), "counts are int32 [slots, V]")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    with _prof.region("sample", lambda: R * V * 4 * (2 if counts is not None else 1)):
        _check(lib().zi_sample(_ptr(out), _ptr(logits), R, V, logits.stride(0), _ptr(temperature), _ptr(top_k),
                               _ptr(top_p), _ptr(min_p), _ptr(repetition_penalty), _ptr(presence_penalty),
                               _ptr(frequency_penalty), _ptr(count_rows), _ptr(counts), _ptr(seeds), _ptr(draw_index),
                               _stream()), "sample")
    return out


def count_tokens(counts_row: torch.Tensor, tokens: torch.Tensor) -> None:
    _need(counts_row.dtype == torch.int32 and counts_row.is_contiguous(), "counts row is contiguous int32")
    _i32(tokens, "tokens")
    _check(lib().zi_count_tokens(_ptr(counts_row), _ptr(tokens), tokens.numel(), counts_row.numel(), _stream()),
           "count_tokens")
