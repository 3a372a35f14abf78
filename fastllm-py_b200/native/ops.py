"""Python faces of the CUDA launchers: torch tensors in, one kernel launch each.

Every function launches on torch's current stream, allocates nothing (outputs
are passed in) and raises if the launch fails.  There is no other
implementation behind these names: without the compiled libraries they raise.
Tensors must live on the CUDA device; strides are passed as leading dimensions,
so row-padded buffers and column slices of wider buffers are fine as long as
the last dimension is contiguous.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_long, c_void_p

import torch

from .build import load_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream():
    """The current CUDA stream's handle for a launch.  `torch.cuda.current_stream()` asks the
    driver how many devices there are on every call (20 us): a step launched kernel by kernel
    spent more time there than on its kernels, so the raw handle is asked for instead."""
    global _device_index
    if _raw_stream is None:
        return c_void_p(torch.cuda.current_stream().cuda_stream)
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return c_void_p(_raw_stream(_device_index))


def _ld(t: torch.Tensor) -> int:
    """Leading dimension (elements between rows) of a 2-D view with a dense last axis."""
    if t.dim() != 2:
        raise KernelError(f"expected a 2-D tensor, got shape {tuple(t.shape)}")
    if t.shape[1] > 1 and t.stride(1) != 1:
        raise KernelError("the last dimension must be contiguous")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


class _Counter:
    """Kernels launched by this process through these wrappers (a graph replay
    adds the number of kernels captured in it)."""
    launches = 0


counter = _Counter()


def _check(rc: int, what: str, kernels: int = 1) -> None:
    if rc != 0:
        raise KernelError(f"{what}: CUDA error {rc} at launch")
    counter.launches += kernels


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the engine's kernels run on a CUDA device only; got a CPU tensor")


_fns: dict = {}
_launches: dict = {}        # operands' places and sizes -> (launcher, converted arguments) of wrappers that remember


def _fn(lib_name: str, fn_name: str, argtypes, defines=None):
    """The launcher `fn_name` of a library with its signature set, looked up once (a step calls
    these wrappers a few hundred times and is short of host time when its kernels are small)."""
    if defines is None:
        fn = _fns.get(fn_name)
        if fn is not None:
            return fn
    key = (lib_name, tuple(sorted((defines or {}).items())), fn_name)
    fn = _fns.get(key)
    if fn is None:
        fn = getattr(load_library(lib_name, defines), fn_name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _fns[key] = fn
        if defines is None:
            _fns[fn_name] = fn
    return fn


# ---------------------------------------------------------------- elementwise

def embed(table, ids, out, status, fed=None, scale=1.0):
    """out[t] = table[ids[t]] * scale as float32; an id outside the table sets status[0] = t + 1.
    With `fed` (int32 on the device), an id -1 - r is replaced by fed[r]."""
    _require_cuda(table, ids, out, status, fed)
    fn = _fn("elementwise", "fl_embed", [c_void_p, c_int, c_long, c_void_p, c_void_p, c_long, c_int,
                                         c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p])
    if out.dtype != torch.float32 or ids.dtype != torch.int32 or (fed is not None and fed.dtype != torch.int32):
        raise KernelError("embed: out must be float32, ids (and fed) int32")
    _check(fn(_ptr(table), dtype_code(table), _ld(table), _ptr(ids), _ptr(out), _ld(out),
              ids.numel(), table.shape[1], table.shape[0], _ptr(status), _ptr(fed),
              0 if fed is None else fed.numel(), float(scale), _stream()), "embed")


def rmsnorm(x, weight, out, eps, rows=None):
    """out[r] = rmsnorm(x[rows[r] if rows else r]) * weight."""
    _require_cuda(x, weight, out, rows)
    fn = _fn("elementwise", "fl_rmsnorm", [c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_int,
                                           c_long, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(x), dtype_code(x), _ld(x), _ptr(weight), dtype_code(weight), _ptr(out),
              dtype_code(out), _ld(out), out.shape[0], x.shape[1], float(eps), _ptr(rows), _stream()),
           "rmsnorm")


def add_rmsnorm(resid, delta, weight, out, eps, rows=None):
    """resid += delta (float32, written back unless rows are gathered); out = rmsnorm(resid) * weight."""
    _require_cuda(resid, delta, weight, out, rows)
    if resid.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream must be float32")
    fn = _fn("elementwise", "fl_add_rmsnorm", [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p,
                                               c_int, c_void_p, c_int, c_long, c_int, c_int, c_float,
                                               c_void_p, c_void_p])
    _check(fn(_ptr(resid), _ld(resid), _ptr(delta), dtype_code(delta), _ld(delta), _ptr(weight),
              dtype_code(weight), _ptr(out), dtype_code(out), _ld(out), out.shape[0], resid.shape[1],
              float(eps), _ptr(rows), _stream()), "add_rmsnorm")


def add_rmsnorm_partial(resid, partial, weight, out, eps):
    """resid += (split-K partial sums, added in slab order); out = rmsnorm(resid) * weight."""
    partial.check()
    # (the same operands in the same places, as in every layer of every step of a size: launched from
    # what the first such call converted; see gemm_tc.gemm)
    key = ("add_rmsnorm_partial", resid.data_ptr(), resid.shape, resid.stride(0), partial.data.data_ptr(),
           partial.splits, partial.split_stride, partial.ld, weight.data_ptr(), weight.dtype, out.data_ptr(),
           out.shape, out.stride(0), out.dtype, eps)
    known = _launches.get(key)
    if known is not None:
        _check(known[0](*known[1], _stream()), "add_rmsnorm_partial")
        return
    _require_cuda(resid, weight, out)
    fn = _fn("elementwise", "fl_add_rmsnorm_partial", [c_void_p, c_long, c_void_p, c_int, c_long, c_long,
                                                       c_void_p, c_int, c_void_p, c_int, c_long, c_int,
                                                       c_int, c_float, c_void_p])
    args = (_ptr(resid), _ld(resid), _ptr(partial.data), partial.splits, partial.split_stride,
            partial.ld, _ptr(weight), dtype_code(weight), _ptr(out), dtype_code(out), _ld(out),
            out.shape[0], resid.shape[1], float(eps))
    _check(fn(*args, _stream()), "add_rmsnorm_partial")
    if len(_launches) > 8192:
        _launches.clear()
    _launches[key] = (fn, args)


def swiglu_partial(partial, out):
    """swiglu over gate|up columns given as split-K partial sums."""
    _require_cuda(out)
    partial.check()
    fn = _fn("elementwise", "fl_swiglu_partial", [c_void_p, c_int, c_long, c_long, c_void_p, c_int, c_long,
                                                  c_int, c_int, c_void_p])
    _check(fn(_ptr(partial.data), partial.splits, partial.split_stride, partial.ld, _ptr(out),
              dtype_code(out), _ld(out), out.shape[0], out.shape[1], _stream()), "swiglu_partial")


def rope_kv_write_partial(partial, q_out, n_heads, n_kv_heads, head_dim, rot_dim, cos, sin, positions,
                          slots, cache, page_size):
    """rope_kv_write reading q|k|v as split-K partial sums; rotated queries go to q_out."""
    _require_cuda(q_out, cos, sin, positions, slots, cache)
    partial.check()
    fn = _fn("rope_kv", "fl_rope_kv_write_partial",
             [c_void_p, c_int, c_long, c_long, c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int,
              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p])
    if cache is not None:
        if cache.dtype != q_out.dtype:
            raise KernelError("rope_kv_write: cache and activations must have one dtype")
        k_ptr = c_void_p(cache.data_ptr())
        v_ptr = c_void_p(cache.data_ptr() + cache.stride(1) * cache.element_size())
        page_stride = cache.stride(0)
    else:
        k_ptr = v_ptr = None
        page_stride = 0
    _check(fn(_ptr(partial.data), partial.splits, partial.split_stride, partial.ld, _ptr(q_out),
              dtype_code(q_out), _ld(q_out), q_out.shape[0], n_heads, n_kv_heads, head_dim, rot_dim,
              _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slots), k_ptr, v_ptr, page_stride, page_size,
              0 if cache is None else 1, _stream()), "rope_kv_write_partial")


def residual_add(resid, delta):
    _require_cuda(resid, delta)
    if resid.dtype != torch.float32:
        raise KernelError("residual_add: the residual stream must be float32")
    fn = _fn("elementwise", "fl_residual_add", [c_void_p, c_long, c_void_p, c_int, c_long, c_int, c_int,
                                                c_void_p])
    _check(fn(_ptr(resid), _ld(resid), _ptr(delta), dtype_code(delta), _ld(delta), resid.shape[0],
              resid.shape[1], _stream()), "residual_add")


def swiglu(gate_up, out):
    """out[:, i] = silu(gate_up[:, i]) * gate_up[:, I + i], I = out.shape[1]."""
    _require_cuda(gate_up, out)
    if gate_up.dtype != out.dtype:
        raise KernelError("swiglu: input and output must have one dtype")
    fn = _fn("elementwise", "fl_swiglu", [c_void_p, c_int, c_long, c_void_p, c_long, c_int, c_int,
                                          c_void_p])
    _check(fn(_ptr(gate_up), dtype_code(gate_up), _ld(gate_up), _ptr(out), _ld(out), out.shape[0],
              out.shape[1], _stream()), "swiglu")


def glu(gate_up, out, activation: str = "silu", params=(0.0, 0.0)):
    """out[:, i] = f(gate_up[:, i], gate_up[:, I + i]), I = out.shape[1]; f: see ACTIVATIONS."""
    _require_cuda(gate_up, out)
    if gate_up.dtype != out.dtype:
        raise KernelError("glu: input and output must have one dtype")
    fn = _fn("elementwise", "fl_glu", [c_void_p, c_int, c_long, c_void_p, c_long, c_int, c_int, c_int, c_float, c_float,
                                       c_void_p])
    _check(fn(_ptr(gate_up), dtype_code(gate_up), _ld(gate_up), _ptr(out), _ld(out), out.shape[0],
              out.shape[1], activation_code(activation), float(params[0]), float(params[1]), _stream()), "glu")


# Gated units f(g, u) of a gate value and an up value.  silu, relu, gelu_tanh, relu_squared: act(g) * u.
# clamped_swish with params (limit, slope): g' = min(g, limit), u' = clamp(u, -limit, limit),
# f = g' * sigmoid(slope * g') * (u' + 1).
ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "clamped_swish": 3, "relu_squared": 4}


def activation_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation {name!r} is not one of {sorted(ACTIVATIONS)}") from None


def sandwich_norm(resid, y, w_post, eps_post, w_pre, eps_pre, out, rows=None):
    """resid += rmsnorm(y) * w_post (written back unless rows are gathered); out = rmsnorm(resid) * w_pre.
    With `out` None only the first half is done."""
    _require_cuda(resid, y, w_post, w_pre, out, rows)
    if resid.dtype != torch.float32:
        raise KernelError("sandwich_norm: the residual stream must be float32")
    if w_pre is not None and w_pre.dtype != w_post.dtype:
        raise KernelError("sandwich_norm: both norm weights must be stored in one dtype")
    fn = _fn("elementwise", "fl_sandwich_norm", [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p, c_float, c_void_p,
                                                 c_float, c_int, c_void_p, c_int, c_long, c_int, c_int, c_void_p,
                                                 c_void_p])
    n_rows = resid.shape[0] if rows is None else rows.numel()
    _check(fn(_ptr(resid), _ld(resid), _ptr(y), dtype_code(y), _ld(y), _ptr(w_post), float(eps_post), _ptr(w_pre),
              float(eps_pre), dtype_code(w_post), _ptr(out), F32 if out is None else dtype_code(out),
              0 if out is None else _ld(out), n_rows, resid.shape[1], _ptr(rows), _stream()), "sandwich_norm")


def sandwich_norm_partial(resid, partial, w_post, eps_post, w_pre, eps_pre, out):
    """`sandwich_norm` with the sublayer's output given as split-K partial sums (added in slab order)."""
    partial.check()
    _require_cuda(resid, w_post, w_pre, out)
    if resid.dtype != torch.float32 or w_pre.dtype != w_post.dtype:
        raise KernelError("sandwich_norm_partial: float32 residual stream, norm weights of one dtype")
    fn = _fn("elementwise", "fl_sandwich_norm_partial", [c_void_p, c_long, c_void_p, c_int, c_long, c_long, c_void_p,
                                                         c_float, c_void_p, c_float, c_int, c_void_p, c_int, c_long,
                                                         c_int, c_int, c_void_p])
    _check(fn(_ptr(resid), _ld(resid), _ptr(partial.data), partial.splits, partial.split_stride, partial.ld,
              _ptr(w_post), float(eps_post), _ptr(w_pre), float(eps_pre), dtype_code(w_post), _ptr(out),
              dtype_code(out), _ld(out), resid.shape[0], resid.shape[1], _stream()), "sandwich_norm_partial")


def softcap(logits, cap: float):
    """logits <- cap * tanh(logits / cap), in place (float32)."""
    _require_cuda(logits)
    if logits.dtype != torch.float32:
        raise KernelError("softcap: logits must be float32")
    fn = _fn("elementwise", "fl_softcap", [c_void_p, c_long, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(logits), _ld(logits), logits.shape[0], logits.shape[1], float(cap), _stream()), "softcap")


def norm_pair(resid, d1, d2, w1, w2, out1, out2, eps, rows=None):
    """resid += d1 + d2 (each may be None; written back unless rows are gathered); r = rms of the row;
    out1 = resid / r * w1 and, when given, out2 = resid / r * w2: two norms of one row in one pass."""
    _require_cuda(resid, d1, d2, w1, w2, out1, out2, rows)
    if resid.dtype != torch.float32:
        raise KernelError("norm_pair: the residual stream must be float32")
    if (d1 is not None and d2 is not None and d1.dtype != d2.dtype) or (w2 is not None and w2.dtype != w1.dtype) or \
            (out2 is not None and out2.dtype != out1.dtype) or (w2 is None) != (out2 is None):
        raise KernelError("norm_pair: both sums, both weights and both outputs share a dtype each")
    fn = _fn("elementwise", "fl_norm_pair", [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p,
                                             c_void_p, c_int, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                             c_float, c_void_p, c_void_p])
    d = d1 if d1 is not None else d2
    _check(fn(_ptr(resid), _ld(resid), _ptr(d1), 0 if d1 is None else _ld(d1), _ptr(d2), 0 if d2 is None else _ld(d2),
              F32 if d is None else dtype_code(d), _ptr(w1), _ptr(w2), dtype_code(w1), _ptr(out1), _ld(out1),
              _ptr(out2), 0 if out2 is None else _ld(out2), dtype_code(out1), out1.shape[0], resid.shape[1],
              float(eps), _ptr(rows), _stream()), "norm_pair")


# ------------------------------------------------------ differential attention

def diff_prep(proj, heads, kv_heads, dim, vdim, rot, cos, sin, positions, slots, cache, page_size):
    """proj columns q (heads x 2 maps x dim) | k (kv_heads x 2 x dim) | v (kv_heads x vdim): rotates the first `rot`
    dimensions of every query map in place (pairs (i, i + rot/2)); rotates the key maps into each token's cache
    row and copies its value behind them.  `cache`: one layer's [pages, kv_heads, page_size, 2 dim + vdim]."""
    _require_cuda(proj, cos, sin, positions, slots, cache)
    if cache is not None and (cache.dtype != proj.dtype or not cache.is_contiguous()):
        raise KernelError("diff_prep: the cache must be contiguous and of the activations' dtype")
    fn = _fn("diff_attention", "fl_diff_prep", [c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int,
                                                c_void_p])
    _check(fn(_ptr(proj), dtype_code(proj), _ld(proj), proj.shape[0], heads, kv_heads, dim, vdim, rot, _ptr(cos),
              _ptr(sin), _ptr(positions), _ptr(slots), _ptr(cache), 0 if cache is None else cache.stride(0), page_size,
              _stream()), "diff_prep")


def diff_attention_simt(q, out, cache, block_table, tok_req, positions, heads, kv_heads, dim, vdim, window, scale,
                        lam, eps, out_scale, page_size):
    """Differential attention of every token over its request's cache rows on CUDA cores: per head
    o = softmax-map 1 - lam * softmax-map 2 (both over the same values), out = o / rms(o) * out_scale."""
    _require_cuda(q, out, cache, block_table, tok_req, positions)
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("diff_attention: q, cache and out share a dtype")
    fn = _fn("diff_attention", "fl_diff_attention_simt",
             [c_void_p, c_int, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_void_p])
    _check(fn(_ptr(q), dtype_code(q), _ld(q), _ptr(out), _ld(out), _ptr(cache), cache.stride(0), page_size,
              _ptr(block_table), block_table.stride(0), _ptr(tok_req), _ptr(positions), q.shape[0], heads, kv_heads,
              dim, vdim, int(window or 0), float(scale), float(lam), float(eps), float(out_scale), _stream()),
           "diff_attention_simt")


def diff_tc_takes(dtype, dim: int, vdim: int) -> bool:
    """Whether the tensor-core differential attention serves this number format and these sizes."""
    return dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 128 and 16 <= vdim <= 128


def diff_tc_library(dim: int, vdim: int):
    return "diff_attention_tc", {"DIFF_DIM": dim, "DIFF_VDIM": vdim}


def diff_attention_tc(q, out, cache, block_table, step, heads, kv_heads, dim, vdim, window, scale, lam, eps, out_scale,
                      page_size, include_single=True):
    """`diff_attention_simt` on the tensor cores for bfloat16: 64 rows of a request and one head per block, both
    maps against the same staged cache rows; one build per (dim, vdim).  Prompt portions and, unless
    `include_single` is False, requests that bring a single token."""
    _require_cuda(q, out, cache, block_table)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("diff_attention_tc: q, cache and out must be bfloat16")
    name, defines = diff_tc_library(dim, vdim)
    fn = _fn(name, "fl_diff_attention_tc", [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_int,
                                            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                            c_float, c_float, c_float, c_void_p], defines)
    _check(fn(_ptr(q), _ld(q), _ptr(out), _ld(out), _ptr(cache), cache.stride(0), page_size, _ptr(block_table),
              block_table.stride(0), _ptr(step.req_start), _ptr(step.req_ctx), _ptr(step.req_qlen), step.n_requests,
              q.shape[0], int(include_single), heads, kv_heads, int(window or 0), float(scale), float(lam), float(eps), float(out_scale),
              _stream()), "diff_attention_tc")


DIFF_SPLIT = 128                 # keys per block of the split-key kernel for single tokens


def diff_decode_takes(heads: int, kv_heads: int, dim: int, vdim: int) -> bool:
    """Whether the split-key kernels for single tokens serve these sizes (groups of up to 8 query heads)."""
    fn = load_library("diff_attention").fl_diff_decode_takes
    fn.argtypes, fn.restype = [c_int, c_int, c_int, c_int], c_int
    return bool(fn(heads, kv_heads, dim, vdim))


def diff_decode(q, out, cache, block_table, tok_req, positions, decode_tokens, partial, n_splits, heads, kv_heads, dim,
                vdim, window, scale, lam, eps, out_scale, page_size):
    """Differential attention for the rows `decode_tokens` of q (each the single token of its request), the keys
    shared out over `n_splits` blocks of DIFF_SPLIT keys at fixed positions, which must reach every token's last
    key ((longest visible span - 1) // DIFF_SPLIT + 2 does); a cache row is read once for all query heads of its
    group.  `partial`: float32, n_decode * heads * 2 * n_splits * (vdim + 2).  Other rows of `out` are left alone."""
    _require_cuda(q, out, cache, block_table, tok_req, positions, decode_tokens, partial)
    n = decode_tokens.numel()
    if partial is None or partial.numel() < n * heads * 2 * n_splits * (vdim + 2):
        raise KernelError("diff_decode: the buffer for the splits' results is too small")
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("diff_decode: q, cache and out share a dtype")
    fn = _fn("diff_attention", "fl_diff_decode",
             [c_void_p, c_int, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float,
              c_void_p])
    _check(fn(_ptr(q), dtype_code(q), _ld(q), _ptr(out), _ld(out), _ptr(cache), cache.stride(0), page_size,
              _ptr(block_table), block_table.stride(0), _ptr(tok_req), _ptr(positions), _ptr(decode_tokens), n,
              _ptr(partial), int(n_splits), heads, kv_heads, dim, vdim, int(window or 0), float(scale), float(lam),
              float(eps), float(out_scale), _stream()), "diff_decode", 2)


# ------------------------------------------------------------------ retention

def retention_prep(proj, work, heads, dim, vdim, rot, cos, sin, positions, k_scale):
    """proj columns q (heads x dim) | k (heads x dim) | v (heads x vdim) | ...: q and k rotated (pairs (i, i + rot/2) of
    the first `rot` dimensions), k times `k_scale`, v as it is, into the float32 columns q | k | v of `work`."""
    _require_cuda(proj, work, cos, sin, positions)
    if work.dtype != torch.float32:
        raise KernelError("retention_prep: the work buffer must be float32")
    fn = _fn("retention", "fl_retention_prep", [c_void_p, c_int, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int,
                                                c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p])
    _check(fn(_ptr(proj), dtype_code(proj), _ld(proj), _ptr(work), _ld(work), proj.shape[0], heads, dim, vdim, rot,
              _ptr(cos), _ptr(sin), _ptr(positions), float(k_scale), _stream()), "retention_prep")


_sm_counts: dict = {}


def retention_scan(work, o, state, decay, step, heads, dim, vdim, fixed_order=False):
    """Per request and head S <- decay S + k v^T, o = S^T q over the step's tokens; q | k | v are the float32 columns
    of `work`, `o` float32 [N, heads * vdim]; state rows [heads, vdim, dim] float32 are read (unless the request
    starts) and written.  `fixed_order`: the read-out's sum keeps one order whatever the step's shape (otherwise a
    lone prompt spreads a column over more lanes than a batch does)."""
    _require_cuda(work, o, state, decay)
    if work.dtype != torch.float32 or o.dtype != torch.float32 or state.dtype != torch.float32 or \
            decay.dtype != torch.float32:
        raise KernelError("retention_scan: work, o, state and decay must be float32")
    sms = _sm_counts.get(work.device)
    if sms is None:
        sms = _sm_counts[work.device] = torch.cuda.get_device_properties(work.device).multi_processor_count
    fn = _fn("retention", "fl_retention_scan", [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p,
                                                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                c_int, c_void_p])
    _check(fn(_ptr(work), _ld(work), _ptr(o), _ld(o), _ptr(state), state.stride(0), _ptr(decay), _ptr(step.req_start),
              _ptr(step.req_ctx), _ptr(step.req_qlen), _ptr(step.req_slot), step.n_requests, heads, dim, vdim, sms,
              int(fixed_order), _stream()), "retention_scan")


def retention_gated_norm(o, proj, gate_col, out, heads, vdim, eps):
    """out[t, h] = o[t, h] / rms(o[t, h]) * silu(gate[t, h]); gate are the columns of `proj` from `gate_col` on."""
    _require_cuda(o, proj, out)
    if proj.dtype != out.dtype or o.dtype != torch.float32:
        raise KernelError("retention_gated_norm: gate and out share a dtype, o is float32")
    fn = _fn("retention", "fl_retention_gated_norm", [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p, c_long, c_int,
                                                      c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(o), _ld(o), c_void_p(proj.data_ptr() + proj.element_size() * gate_col), dtype_code(proj), _ld(proj),
              _ptr(out), _ld(out), out.shape[0], heads, vdim, float(eps), _stream()), "retention_gated_norm")


# ---------------------------------------------------------------- delta rule

def delta_prep(proj, conv_w, a_log, dt_bias, state, tail_off, step, work, heads, kv_heads, dim, vdim, taps,
               unit_eps, q_scale):
    """Convolution, silu, unit norms, beta and decay of every token of the step (and the requests' new
    convolution tails); proj columns are q | k | v | gate | b | a, state rows [S | tail] float32, work
    rows q | k | v | beta | decay | o float32."""
    _require_cuda(proj, conv_w, a_log, dt_bias, state, work)
    if state.dtype != torch.float32 or work.dtype != torch.float32:
        raise KernelError("delta_prep: state and work buffer must be float32")
    if not (conv_w.dtype == a_log.dtype == dt_bias.dtype):
        raise KernelError("delta_prep: the mixer's small tensors must be stored in one dtype")
    fn = _fn("delta_rule", "fl_delta_prep", [c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                             c_long, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_int,
                                             c_int, c_float, c_float, c_void_p])
    _check(fn(_ptr(proj), dtype_code(proj), _ld(proj), _ptr(conv_w), _ptr(a_log), _ptr(dt_bias), dtype_code(conv_w),
              _ptr(state), state.stride(0), tail_off, _ptr(step.tok_req), _ptr(step.positions), _ptr(step.req_start),
              _ptr(step.req_ctx), _ptr(step.req_qlen), _ptr(step.req_slot), _ptr(work), _ld(work),
              proj.shape[0], step.n_requests, heads, kv_heads, dim, vdim, taps, float(unit_eps), float(q_scale),
              _stream()), "delta_prep", 1 if taps == 1 else 2)


def delta_scan(work, state, step, heads, kv_heads, dim, vdim):
    """The recurrence over each request's tokens of the step; state rows are read (unless the request
    starts) and written; the o columns of `work` are filled."""
    _require_cuda(work, state)
    fn = _fn("delta_rule", "fl_delta_scan", [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(work), _ld(work), _ptr(state), state.stride(0), _ptr(step.req_start), _ptr(step.req_ctx),
              _ptr(step.req_qlen), _ptr(step.req_slot), step.n_requests, heads, kv_heads, dim, vdim,
              int(work.shape[0] == step.n_requests), _stream()), "delta_scan")


def delta_gated_norm(work, o_col, proj, gate_col, weight, out, heads, vdim, eps):
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * silu(gate[t, h]); o are the float32 columns of `work`
    from `o_col` on, gate the columns of `proj` from `gate_col` on."""
    _require_cuda(work, proj, weight, out)
    if proj.dtype != out.dtype or work.dtype != torch.float32:
        raise KernelError("delta_gated_norm: gate and out share a dtype, o is float32")
    fn = _fn("delta_rule", "fl_delta_gated_norm", [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p, c_int, c_void_p,
                                                   c_long, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(c_void_p(work.data_ptr() + 4 * o_col), _ld(work), c_void_p(proj.data_ptr() + proj.element_size() * gate_col),
              dtype_code(proj), _ld(proj), _ptr(weight), dtype_code(weight), _ptr(out), _ld(out),
              out.shape[0], heads, vdim, float(eps), _stream()), "delta_gated_norm")


# ---------------------------------------------------------- latent attention

def latent_prep(proj, q_out, heads, dim, rot, rank, norm_w, eps, cos, sin, positions, slots, cache, kv=None,
                interleaved=False):
    """The queries' rotated parts, turned, go to the last `rot` columns of each head's block of `q_out`
    ([N, heads * (rank + rot)], float32 or bfloat16); with `cache` ([pages, page_size, rank + rot]), each token's latent
    is normed and written with the rotated key part into the token's row.  The latent and the key part follow the
    queries in `proj`'s rows, or are the rows of `kv` ([N, rank + rot]).  Rotary pairs are (i, i + rot/2), with
    `interleaved` (2i, 2i + 1)."""
    _require_cuda(proj, q_out, norm_w, cos, sin, positions, slots, cache, kv)
    if kv is not None and kv.dtype != proj.dtype:
        raise KernelError("latent_prep: queries and latents must have one dtype")
    if cache is not None and (cache.dtype != proj.dtype or not cache.is_contiguous()):
        raise KernelError("latent_prep: the cache must be contiguous and of the activations' dtype")
    fn = _fn("latent_attention", "fl_latent_prep", [c_void_p, c_int, c_long, c_void_p, c_long, c_int, c_void_p, c_int, c_long, c_int, c_int, c_int, c_int,
                                                    c_int, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p,
                                                    c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(proj), dtype_code(proj), _ld(proj), _ptr(kv), 0 if kv is None else _ld(kv), int(bool(interleaved)),
              _ptr(q_out), dtype_code(q_out), _ld(q_out), proj.shape[0], heads,
              dim, rot, rank,
              _ptr(norm_w), F32 if norm_w is None else dtype_code(norm_w), float(eps), _ptr(cos), _ptr(sin),
              _ptr(positions), _ptr(slots), _ptr(cache), 0 if cache is None else 1, _stream()), "latent_prep")


def latent_attention(q, out, cache, block_table, tok_req, positions, heads, rank, rot, window, scale, page_size):
    """Attention of every token over its request's cache rows; q [N, heads * (rank + rot)] (float32 or
    bfloat16) and out [N, heads * rank] float32.  CUDA cores, any sizes, both number formats."""
    _require_cuda(q, out, cache, block_table, tok_req, positions)
    if out.dtype != torch.float32:
        raise KernelError("latent_attention: out must be float32")
    fn = _fn("latent_attention", "fl_latent_attention", [c_void_p, c_int, c_long, c_void_p, c_long, c_void_p, c_int, c_int,
                                                         c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                         c_int, c_float, c_void_p])
    _check(fn(_ptr(q), dtype_code(q), _ld(q), _ptr(out), _ld(out), _ptr(cache), dtype_code(cache), page_size,
              _ptr(block_table), block_table.stride(0), _ptr(tok_req), _ptr(positions), q.shape[0], heads, rank, rot,
              int(window or 0), float(scale), _stream()), "latent_attention")


def latent_tc_takes(dtype, rank: int, rot: int) -> bool:
    """Whether the tensor-core latent attention serves this number format and these sizes."""
    return dtype == torch.bfloat16 and rank % 32 == 0 and (rank + rot) % 16 == 0 and rank <= 1024


def latent_tc_library(rank: int, rot: int):
    return "latent_attention_tc", {"LAT_RANK": rank, "LAT_ROT": rot}


def latent_attention_tc(q, out, cache, block_table, tok_req, positions, heads, rank, rot, window, scale, page_size,
                        split_keys=0, n_splits=1, partial=None):
    """The same on tensor cores: q and cache bfloat16, out float32 or bfloat16; one build per (rank, rot).  With
    `split_keys` (a multiple of 32) each token's keys are shared out over `n_splits` blocks, which must reach
    every token's last key ((longest visible span - 1) // split_keys + 2 does), and merged from `partial`
    (float32, N * heads * n_splits * (rank + 2))."""
    _require_cuda(q, out, cache, block_table, tok_req, positions)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("latent_attention_tc: q and cache must be bfloat16")
    name, defines = latent_tc_library(rank, rot)
    if split_keys and (partial is None or partial.numel() < q.shape[0] * heads * n_splits * (rank + 2)):
        raise KernelError("latent_attention_tc: the buffer for the splits' results is too small")
    fn = _fn(name, "fl_latent_attention_tc", [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_int,
                                              c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                              c_void_p], defines)
    _check(fn(_ptr(q), _ld(q), _ptr(out), dtype_code(out), _ld(out), _ptr(cache), page_size, _ptr(block_table), block_table.stride(0),
              _ptr(tok_req), _ptr(positions), q.shape[0], heads, int(window or 0), float(scale), int(split_keys),
              int(n_splits), _ptr(partial), _stream()), "latent_attention_tc", 2 if split_keys else 1)


def gemm_simt_batched(a, a_batch, w, out, out_batch):
    """out[:, b * out_batch : b * out_batch + N] = a[:, b * a_batch : b * a_batch + K] @ w[b]^T for every b:
    w is [batch, N, K]; a and out are 2-D buffers whose column blocks are the batch."""
    _require_cuda(a, w, out)
    batch, n, k = w.shape
    if not w.is_contiguous():
        raise KernelError("gemm_simt_batched: the weights must be contiguous")
    fn = _fn("gemm_simt", "fl_gemm_simt_batched", [c_void_p, c_int, c_long, c_long, c_void_p, c_int, c_long, c_long,
                                                   c_void_p, c_int, c_long, c_long, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(a), dtype_code(a), _ld(a), a_batch, _ptr(w), dtype_code(w), k, n * k, _ptr(out), dtype_code(out),
              _ld(out), out_batch, a.shape[0], n, k, batch, _stream()), "gemm_simt_batched")


def gemm_batched(a, a_batch, w, out, out_batch, gate=None):
    """`gemm_simt_batched` with the kernel chosen by the operands: bfloat16 a and w with K a multiple of 32
    and 16-byte aligned column blocks go to the tensor cores, everything else to the CUDA cores.  `gate` (shaped and
    typed like `out`): out *= sigmoid(gate), in the tensor-core kernel's epilogue or by a kernel of its own."""
    batch, n, k = w.shape
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 32 == 0 and a_batch % 8 == 0 \
            and _ld(a) % 8 == 0 and a.data_ptr() % 16 == 0 and w.is_contiguous():
        _require_cuda(a, w, out, gate)
        if gate is not None and (gate.dtype != out.dtype or gate.shape != out.shape):
            raise KernelError("gemm_batched: the gate shares the output's shape and dtype")
        fn = _fn("gemm_mma", "fl_gemm_mma_batched", [c_void_p, c_long, c_long, c_void_p, c_void_p, c_int, c_long, c_long,
                                                     c_int, c_int, c_int, c_int, c_void_p, c_long, c_long, c_void_p])
        _check(fn(_ptr(a), _ld(a), a_batch, _ptr(w), _ptr(out), dtype_code(out), _ld(out), out_batch, a.shape[0], n, k,
                  batch, _ptr(gate), 0 if gate is None else _ld(gate), out_batch, _stream()), "gemm_mma_batched")
        return
    gemm_simt_batched(a, a_batch, w, out, out_batch)
    if gate is not None:
        sigmoid_gate(out, gate)


# ------------------------------------------ post-norm block with input convolution; paired-token embedding

def input_conv(x, w, taps, ring, step, h, hc):
    """hc[t] = x[t] + sum_j w[:, j] x[t - taps + 1 + j] over the request's own rows (zeros before position 0; rows of
    earlier steps from `ring`, [slots, (taps - 1) * width] float32 filed by position mod (taps - 1)); h[t] = x[t] in the
    activation type (None: not wanted).  x float32 [N, width], w float32 [width, taps]."""
    _require_cuda(x, w, ring, h, hc)
    if x.dtype != torch.float32 or w.dtype != torch.float32 or (ring is not None and ring.dtype != torch.float32):
        raise KernelError("input_conv: the stream, the taps and the kept rows must be float32")
    if h is not None and h.dtype != hc.dtype:
        raise KernelError("input_conv: both outputs share a dtype")
    fn = _fn("gated_block", "fl_input_conv", [c_void_p, c_long, c_void_p, c_int, c_void_p, c_long, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                              c_void_p])
    _check(fn(_ptr(x), _ld(x), _ptr(w), int(taps), _ptr(ring), 0 if ring is None else ring.stride(0), _ptr(step.positions),
              _ptr(step.tok_req), _ptr(step.req_start), _ptr(step.req_slot), _ptr(h), 0 if h is None else _ld(h), _ptr(hc),
              _ld(hc), dtype_code(hc), x.shape[0], x.shape[1], _stream()), "input_conv")


def gated_norm_add(x, y, gate, gate_bias, w, eps, step, ring=None, taps=1, dtype=None):
    """x += rmsnorm(y * sigmoid(gate + gate_bias)) * w (no gate: rmsnorm(y) * w).  y and gate are matrices of one
    dtype, or products left as split-K partial sums (`gemm_tc.Partial`), which the kernel adds up as it reads them
    and rounds to `dtype` (the type the matrix would have had; needed when neither is a matrix).  With `ring`, the
    rows of x as they were before the add are filed for the request's last taps - 1 rows of the step (see
    `input_conv`)."""
    def operand(v):
        if v is None:
            return None, 0, 0, 0, None
        if isinstance(v, torch.Tensor):
            return v, _ld(v), 0, 0, v.dtype
        v.check()
        if (v.rows, v.cols) != tuple(x.shape):
            raise KernelError("gated_norm_add: partial sums must have the stream's shape")
        return v.data, v.ld, v.splits, v.split_stride, None

    y_data, y_ld, y_splits, y_stride, y_dt = operand(y)
    g_data, g_ld, g_splits, g_stride, g_dt = operand(gate)
    dt = y_dt or g_dt or dtype
    if dt is None or (y_dt or dt) != dt or (g_dt or dt) != dt:
        raise KernelError("gated_norm_add: the sublayer's result and the gate share one dtype (name it for partial sums)")
    _require_cuda(x, y_data, g_data, gate_bias, w, ring)
    if x.dtype != torch.float32 or w.dtype != torch.float32 or (gate_bias is not None and gate_bias.dtype != torch.float32):
        raise KernelError("gated_norm_add: float32 stream, weights and bias")
    fn = _fn("gated_block", "fl_gated_norm_add", [c_void_p, c_long, c_void_p, c_long, c_int, c_long, c_void_p, c_long, c_int,
                                                  c_long, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_long,
                                                  c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(x), _ld(x), _ptr(y_data), y_ld, y_splits, y_stride, _ptr(g_data), g_ld, g_splits, g_stride,
              _CODES[dt], _ptr(gate_bias), _ptr(w), float(eps), x.shape[0], x.shape[1], _ptr(ring),
              0 if ring is None else ring.stride(0), int(taps), _ptr(step.positions), _ptr(step.tok_req),
              _ptr(step.req_start), _ptr(step.req_qlen), _ptr(step.req_slot), _stream()), "gated_norm_add")


def sigmoid_gate(a, g):
    """a *= sigmoid(g), element by element, in float."""
    _require_cuda(a, g)
    if a.dtype != g.dtype or a.shape != g.shape:
        raise KernelError("sigmoid_gate: both operands share shape and dtype")
    fn = _fn("gated_block", "fl_sigmoid_gate", [c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(a), _ld(a), _ptr(g), _ld(g), dtype_code(a), a.shape[0], a.shape[1], _stream()), "sigmoid_gate")


def pair_embed(table, pairs, out, step, last_token, buckets, mul_prev, mul_cur, scale):
    """out[t] = table[id_t] * scale + pairs[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets] (row `buckets` for a
    request's first token).  `last_token` ([slots] int32) keeps each request's last token between steps."""
    _require_cuda(table, pairs, out, last_token)
    fed = getattr(step, "token_feed", None)
    if out.dtype != torch.float32 or table.dtype != pairs.dtype or last_token.dtype != torch.int32:
        raise KernelError("pair_embed: out float32, both tables of one dtype, last_token int32")
    fn = _fn("gated_block", "fl_pair_embed", [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_void_p, c_long, c_int,
                                              c_int, c_int, c_int, c_long, c_long, c_float, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(table), _ld(table), _ptr(pairs), _ld(pairs), dtype_code(table), _ptr(step.token_ids), _ptr(out), _ld(out),
              step.token_ids.numel(), table.shape[1], table.shape[0], int(buckets), int(mul_prev), int(mul_cur),
              float(scale), _ptr(step.tok_req), _ptr(step.req_start), _ptr(step.req_ctx), _ptr(step.req_qlen),
              _ptr(step.req_slot), _ptr(last_token), _ptr(step.status), _ptr(fed), 0 if fed is None else fed.numel(),
              _stream()), "pair_embed")


# ------------------------------------------------- attention with soft cap, distance bias, kept first tokens, sink

def sink_prep(proj, bias, q_w, k_w, eps, q_out, heads, kv_heads, dim, vdim, v_mode, lam, v_first, slots, cache, page_size):
    """Biases, the whole-projection norms of q and k, the blend of v with `v_first` (v_mode 0: none, 1: v is kept in
    v_first, 2: v <- (1 - lam) v + lam v_first); q to `q_out`, k and v into the tokens' rows of `cache`
    ([pages, kv_heads, page_size, dim + vdim])."""
    _require_cuda(proj, bias, q_w, k_w, q_out, v_first, slots, cache)
    if cache.dtype != proj.dtype or not cache.is_contiguous():
        raise KernelError("sink_prep: the cache must be contiguous and of the activations' dtype")
    for v in (bias, q_w, k_w, v_first):
        if v is not None and v.dtype != torch.float32:
            raise KernelError("sink_prep: biases, norm weights and the first values are float32")
    fn = _fn("sink_attention", "fl_sink_prep", [c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                                                c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                                c_long, c_void_p, c_void_p, c_long, c_int, c_void_p])
    _check(fn(_ptr(proj), dtype_code(proj), _ld(proj), _ptr(bias), _ptr(q_w), _ptr(k_w), float(eps), _ptr(q_out),
              dtype_code(q_out), _ld(q_out), proj.shape[0], heads, kv_heads, dim, vdim, int(v_mode), float(lam),
              _ptr(v_first), 0 if v_first is None else _ld(v_first), _ptr(slots), _ptr(cache), cache.stride(0), page_size,
              _stream()), "sink_prep")


def sink_attention_simt(q, out, cache, block_table, tok_req, positions, heads, kv_heads, dim, vdim, window, keep_first,
                        scale, cap, bucket_of, rel, sink, page_size, chunk=None):
    """Attention of every token over its request's visible keys (the last `window` and the first `keep_first`), scores
    capped (`cap` None or 0: not), biased by `rel[bucket_of[distance]]` and with `sink` in the denominator (each may be
    None).  With `chunk` a query sees only keys at or after the last multiple of `chunk` at or below its own position.
    CUDA cores, any sizes, both number formats."""
    _require_cuda(q, out, cache, block_table, tok_req, positions, bucket_of, rel, sink)
    if vdim > 256:
        raise KernelError(f"sink_attention: value size {vdim} is beyond the kernel's limit of 256")
    fn = _fn("sink_attention", "fl_sink_attention_simt",
             [c_void_p, c_int, c_long, c_void_p, c_long, c_void_p, c_int, c_long, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p])
    _check(fn(_ptr(q), dtype_code(q), _ld(q), _ptr(out), _ld(out), _ptr(cache), dtype_code(cache), cache.stride(0), page_size,
              _ptr(block_table), block_table.stride(0), _ptr(tok_req), _ptr(positions), q.shape[0], heads, kv_heads, dim,
              vdim, int(window or 0), int(keep_first or 0), int(chunk or 0), float(scale), float(cap or 0.0), _ptr(bucket_of),
              0 if bucket_of is None else bucket_of.numel(), _ptr(rel), _ptr(sink), _stream()), "sink_attention_simt")


def sink_tc_takes(dtype, dim: int, vdim: int) -> bool:
    """Whether the tensor-core sink attention serves this number format and these sizes."""
    return dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 128 and 16 <= vdim <= 128


def sink_tc_library(dim: int, vdim: int):
    return "sink_attention_tc", {"SINK_DIM": dim, "SINK_VDIM": vdim}


def sink_attention_tc(q, out, cache, block_table, step, heads, kv_heads, dim, vdim, window, keep_first, scale, cap,
                      bucket_of, rel, sink, page_size, include_single=True, chunk=None):
    """`sink_attention_simt` on tensor cores: q, cache and out bfloat16; one build per (dim, vdim); 64 rows of a
    request and one head per block, single tokens as tiles of one row (left out with include_single=False)."""
    _require_cuda(q, out, cache, block_table, bucket_of, rel, sink)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("sink_attention_tc: q, cache and out must be bfloat16")
    name, defines = sink_tc_library(dim, vdim)
    fn = _fn(name, "fl_sink_attention_tc", [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_int,
                                            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                            c_int, c_float, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p], defines)
    _check(fn(_ptr(q), _ld(q), _ptr(out), _ld(out), _ptr(cache), cache.stride(0), page_size, _ptr(block_table),
              block_table.stride(0), _ptr(step.req_start), _ptr(step.req_ctx), _ptr(step.req_qlen), step.n_requests,
              q.shape[0], int(include_single), heads, kv_heads, int(window or 0), int(keep_first or 0), int(chunk or 0),
              float(scale), float(cap or 0.0), _ptr(bucket_of), 0 if bucket_of is None else bucket_of.numel(), _ptr(rel), _ptr(sink),
              _stream()), "sink_attention_tc")


SINK_SPLIT = 128                 # keys of one split of the single-token kernel


def sink_decode_takes(heads: int, kv_heads: int, dim: int, vdim: int) -> bool:
    """Whether the split-key kernels for single tokens serve these sizes (up to eight query heads a key/value head)."""
    fn = _fn("sink_attention", "fl_sink_decode_takes", [c_int, c_int, c_int, c_int])
    return bool(fn(heads, kv_heads, dim, vdim))


def sink_decode_splits(window, keep_first: int, longest: int, chunk=None):
    """(splits in all, splits that walk the kept first tokens) for single tokens of sequences up to `longest`."""
    kept = -(-int(keep_first or 0) // SINK_SPLIT) if window else 0
    span = min(int(window), longest) if window else longest
    if chunk:
        span = min(span, int(chunk))
    return kept + (max(span, 1) - 1) // SINK_SPLIT + 2, kept


def sink_decode(q, out, cache, block_table, tok_req, positions, decode_tokens, partial, n_splits, kept_splits, heads,
                kv_heads, dim, vdim, window, keep_first, scale, cap, bucket_of, rel, sink, page_size, chunk=None):
    """Sink attention for the rows `decode_tokens` of q (each the single token of its request): the keys split over
    blocks of 128, every query head of a key/value head served by the block that reads its rows, then a merge with
    the sink.  partial: float32, decode tokens * heads * n_splits * (vdim + 2)."""
    _require_cuda(q, out, cache, block_table, tok_req, positions, decode_tokens, partial, bucket_of, rel, sink)
    n = decode_tokens.numel()
    if partial.dtype != torch.float32 or partial.numel() < n * heads * n_splits * (vdim + 2):
        raise KernelError("sink_decode: the buffer for the splits' results is too small")
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("sink_decode: q, cache and out share a dtype")
    fn = _fn("sink_attention", "fl_sink_decode",
             [c_void_p, c_int, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
              c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(q), dtype_code(q), _ld(q), _ptr(out), _ld(out), _ptr(cache), cache.stride(0), page_size,
              _ptr(block_table), block_table.stride(0), _ptr(tok_req), _ptr(positions), _ptr(decode_tokens), n,
              _ptr(partial), int(n_splits), int(kept_splits), heads, kv_heads, dim, vdim, int(window or 0),
              int(keep_first or 0), int(chunk or 0), float(scale), float(cap or 0.0), _ptr(bucket_of),
              0 if bucket_of is None else bucket_of.numel(), _ptr(rel), _ptr(sink), _stream()), "sink_decode", 2)


def head_prep(proj, bias, q_w, k_w, norm_mode, eps, rot, interleaved, cos, sin, positions, temp, v_from_k, q_out, heads,
              kv_heads, dim, vdim, slots, cache, page_size):
    """The preparation of attention head by head: biases; norm_mode 1: an RMS norm of every query and key head times
    q_w / k_w ([dim] float, or None) before the rotation, 2: one without weight after it, 0: none; the rotation of a
    head's first `rot` dimensions, pairs (2i, 2i + 1) with `interleaved`, else (i, i + rot / 2); queries times
    1 + coef * ln(floor((position + 1) / every) + 1) with temp = (coef, every); q to `q_out`, k and v into the tokens'
    rows of `cache` ([pages, kv_heads, page_size, dim + vdim]); with `v_from_k` the value is the key as projected."""
    _require_cuda(proj, bias, q_w, k_w, cos, sin, positions, q_out, slots, cache)
    if cache.dtype != proj.dtype or not cache.is_contiguous():
        raise KernelError("head_prep: the cache must be contiguous and of the activations' dtype")
    for v in (bias, q_w, k_w, cos, sin):
        if v is not None and v.dtype != torch.float32:
            raise KernelError("head_prep: biases, norm weights and the rotation's tables are float32")
    if rot and cos.shape[1] != rot // 2:
        raise KernelError("head_prep: the rotation's tables do not fit the rotated dimensions")
    coef, every = temp if temp is not None else (0.0, 0)
    fn = _fn("sink_attention", "fl_head_prep",
             [c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
              c_float, c_int, c_int, c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_long,
              c_int, c_void_p])
    _check(fn(_ptr(proj), dtype_code(proj), _ld(proj), _ptr(bias), _ptr(q_w), _ptr(k_w), int(norm_mode), float(eps),
              int(rot or 0), int(bool(interleaved)), _ptr(cos) if rot else None, _ptr(sin) if rot else None,
              _ptr(positions), float(coef), int(every), int(bool(v_from_k)), _ptr(q_out), dtype_code(q_out), _ld(q_out),
              proj.shape[0], heads, kv_heads, dim, vdim, _ptr(slots), _ptr(cache), cache.stride(0), page_size, _stream()),
           "head_prep")


def head_gate(x, gate, heads, vdim):
    """x[t, h * vdim + d] *= sigmoid(gate[t, h])."""
    _require_cuda(x, gate)
    if x.dtype != gate.dtype:
        raise KernelError("head_gate: x and the gate share a dtype")
    fn = _fn("sink_attention", "fl_head_gate", [c_void_p, c_int, c_long, c_void_p, c_long, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), dtype_code(x), _ld(x), _ptr(gate), _ld(gate), x.shape[0], heads, vdim, _stream()), "head_gate")


# ----------------------------------------------- layer norm, mixes, activation

def _summand(x):
    """(pointer, row pitch, splits, floats between slabs, dtype code) of a tensor, or of split-K partial sums (an
    object with data, splits, split_stride, ld and check()) that a kernel adds up while it reads."""
    if x is None:
        return None, 0, 0, 0, F32
    if isinstance(x, torch.Tensor):
        return _ptr(x), _ld(x), 0, 0, dtype_code(x)
    x.check()
    return _ptr(x.data), x.ld, x.splits, x.split_stride, F32


def add_layernorm(resid, delta, scale, weight, bias, out, eps, rows=None):
    """resid += scale * delta (float32, written back unless rows are gathered; delta None: nothing to add; delta may
    be split-K partial sums, added up while they are read); out = (resid - mean) / sqrt(var + eps) * weight + bias."""
    _require_cuda(resid, weight, bias, out, rows)
    if resid.dtype != torch.float32 or (bias is not None and bias.dtype != weight.dtype):
        raise KernelError("add_layernorm: the residual stream is float32; weight and bias share a dtype")
    d_ptr, d_ld, splits, stride, d_code = _summand(delta)
    fn = _fn("norm_mix", "fl_add_layernorm", [c_void_p, c_long, c_void_p, c_int, c_long, c_float, c_void_p, c_void_p, c_int,
                                              c_void_p, c_int, c_long, c_int, c_int, c_float, c_void_p, c_int, c_long,
                                              c_void_p])
    _check(fn(_ptr(resid), _ld(resid), d_ptr, d_code, d_ld, float(scale), _ptr(weight), _ptr(bias), dtype_code(weight),
              _ptr(out), dtype_code(out), _ld(out), out.shape[0], resid.shape[1], float(eps), _ptr(rows), splits, stride,
              _stream()), "add_layernorm")


def rms_mix(a, b, w_a, w_b, out, eps, weight=0.5):
    """out = weight * (a / rms(a) * w_a + b / rms(b) * w_b), row by row.  a and b are tensors of out's dtype or
    split-K partial sums, added up while they are read."""
    _require_cuda(w_a, w_b, out)
    for x in (a, b):
        if isinstance(x, torch.Tensor) and x.dtype != out.dtype:
            raise KernelError("rms_mix: a, b and out share a dtype")
    if w_a.dtype != w_b.dtype:
        raise KernelError("rms_mix: the weights share a dtype")
    a_ptr, a_ld, a_splits, a_stride, _ = _summand(a)
    b_ptr, b_ld, b_splits, b_stride, _ = _summand(b)
    fn = _fn("norm_mix", "fl_rms_mix", [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                        c_long, c_int, c_int, c_float, c_float, c_int, c_long, c_int, c_long, c_void_p])
    _check(fn(a_ptr, a_ld, b_ptr, b_ld, dtype_code(out), _ptr(w_a), _ptr(w_b), dtype_code(w_a), _ptr(out), _ld(out),
              out.shape[0], out.shape[1], float(eps), float(weight), a_splits, a_stride, b_splits, b_stride, _stream()),
           "rms_mix")


def scaled_add(resid, delta, scale):
    """resid += scale * delta."""
    _require_cuda(resid, delta)
    if resid.dtype != torch.float32:
        raise KernelError("scaled_add: the residual stream must be float32")
    fn = _fn("norm_mix", "fl_scaled_add", [c_void_p, c_long, c_void_p, c_int, c_long, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(resid), _ld(resid), _ptr(delta), dtype_code(delta), _ld(delta), resid.shape[0], resid.shape[1],
              float(scale), _stream()), "scaled_add")


def activation(x, out, name: str, params=(0.0, 0.0)):
    """out = f(x, 1) for the gated units' f (ACTIVATIONS): an activation of one argument."""
    _require_cuda(x, out)
    if x.dtype != out.dtype:
        raise KernelError("activation: input and output must have one dtype")
    fn = _fn("norm_mix", "fl_activation", [c_void_p, c_int, c_long, c_void_p, c_long, c_int, c_int, c_int, c_float, c_float,
                                           c_void_p])
    _check(fn(_ptr(x), dtype_code(x), _ld(x), _ptr(out), _ld(out), x.shape[0], x.shape[1], activation_code(name),
              float(params[0]), float(params[1]), _stream()), "activation")


# ---------------------------------------------- gated recurrence per channel

def rglru(proj, bias, conv_w, conv_b, w_a, w_i, b_a, b_i, rate, state, step, u, a, bx, out, width, blocks, taps,
          fixed_order=False):
    """The gated linear recurrence per channel over the step's tokens.  proj [N, 2 width] = gate branch | input branch
    before their biases (`bias`, float32 [2 width]); the input branch passes a causal convolution (`conv_w`
    [width, taps], `conv_b`), the gates r and i are sigmoids of block-diagonal products of it (`w_a`, `w_i`
    [blocks, width / blocks, width / blocks], `b_a`, `b_i` [width]), a = exp(rate * r), S <- a S + sqrt(1 - a^2) i u;
    out = S * gelu_tanh(gate branch).  state rows: [S | the last taps - 1 inputs] float32; u, a, bx: float32 [N, width].
    `fixed_order`: the recurrence runs token by token whatever the step's shape (otherwise a prompt portion's tokens run
    in segments side by side, and the sums' order follows the cut)."""
    _require_cuda(proj, bias, conv_w, conv_b, w_a, w_i, b_a, b_i, rate, state, u, a, bx, out)
    for v in (bias, conv_w, conv_b, b_a, b_i, rate, state, u, a, bx):
        if v.dtype != torch.float32:
            raise KernelError("rglru: biases, convolution, rates, state and scratch are float32")
    if w_a.dtype != w_i.dtype or not w_a.is_contiguous() or not w_i.is_contiguous() or out.dtype != proj.dtype:
        raise KernelError("rglru: the gate matrices share a dtype and are contiguous; out has the activations' dtype")
    if state.stride(0) < width * taps or _ld(u) != _ld(a) or _ld(u) != _ld(bx):
        raise KernelError("rglru: state rows hold width * taps floats; u, a and bx share a row pitch")
    fn = _fn("rglru", "fl_rglru", [c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_long, c_int,
                                   c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(proj), dtype_code(proj), _ld(proj), _ptr(bias), _ptr(conv_w), _ptr(conv_b), _ptr(w_a), _ptr(w_i),
              dtype_code(w_a), _ptr(b_a), _ptr(b_i), _ptr(rate), _ptr(state), state.stride(0), _ptr(step.tok_req),
              _ptr(step.positions), _ptr(step.req_start), _ptr(step.req_ctx), _ptr(step.req_qlen), _ptr(step.req_slot),
              proj.shape[0], step.n_requests, _ptr(u), _ptr(a), _ptr(bx), _ld(u), _ptr(out), _ld(out), width, blocks, taps,
              int(fixed_order), _stream()), "rglru", 3)


# ---------------------------------------------------- gated linear attention

def gla_prep(proj, w2, b2, work, heads, dim, vdim, rank, q_scale, tau):
    """proj columns q | k (heads x dim each) | v | gate (heads x vdim each) | low (rank): q times `q_scale`, k, the decay
    alpha = sigmoid(W_2 low + b_2)^(1 / tau) per key channel and v into the float32 columns q | k | alpha | v of `work`.
    `w2` is W_2 transposed: [rank, heads * dim]."""
    _require_cuda(proj, w2, b2, work)
    if work.dtype != torch.float32 or w2.dtype != torch.float32 or b2.dtype != torch.float32 or not w2.is_contiguous() \
            or tuple(w2.shape) != (rank, heads * dim):
        raise KernelError("gla_prep: the work buffer, W_2 (transposed: [rank, heads * dim]) and b_2 are float32")
    fn = _fn("gla", "fl_gla_prep", [c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_int,
                                    c_int, c_float, c_float, c_void_p])
    _check(fn(_ptr(proj), dtype_code(proj), _ld(proj), _ptr(w2), _ptr(b2), _ptr(work), _ld(work), proj.shape[0], heads, dim,
              vdim, rank, float(q_scale), float(tau), _stream()), "gla_prep")


def gla_scan(work, o, state, step, heads, dim, vdim, fixed_order=False):
    """Per request and head S <- diag(alpha) S + k v^T, o = S^T q over the step's tokens; q | k | alpha | v are the
    float32 columns of `work`, `o` float32 [N, heads * vdim]; state rows [heads, vdim, dim] float32 are read (unless
    the request starts) and written.  `fixed_order`: the read-out's sum keeps one order whatever the step's shape
    (otherwise a lone prompt spreads a column over more lanes than a batch does)."""
    _require_cuda(work, o, state)
    if work.dtype != torch.float32 or o.dtype != torch.float32 or state.dtype != torch.float32:
        raise KernelError("gla_scan: work, o and state must be float32")
    sms = _sm_counts.get(work.device)
    if sms is None:
        sms = _sm_counts[work.device] = torch.cuda.get_device_properties(work.device).multi_processor_count
    fn = _fn("gla", "fl_gla_scan", [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(work), _ld(work), _ptr(o), _ld(o), _ptr(state), state.stride(0), _ptr(step.req_start),
              _ptr(step.req_ctx), _ptr(step.req_qlen), _ptr(step.req_slot), step.n_requests, heads, dim, vdim, sms,
              int(fixed_order), _stream()), "gla_scan")


def gla_gated_norm(o, gate, weight, out, heads, vdim, eps):
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * silu(gate[t, h]); weight [vdim] (or None) is shared by the heads."""
    _require_cuda(o, gate, weight, out)
    if gate.dtype != out.dtype or o.dtype != torch.float32:
        raise KernelError("gla_gated_norm: gate and out share a dtype, o is float32")
    fn = _fn("gla", "fl_gla_gated_norm", [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_long, c_int,
                                          c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(o), _ld(o), _ptr(gate), dtype_code(gate), _ld(gate), _ptr(weight),
              F32 if weight is None else dtype_code(weight), _ptr(out), _ld(out), out.shape[0], heads, vdim, float(eps),
              _stream()), "gla_gated_norm")


# ------------------------------------------------------------- routed experts

def moe_pick(logits, bias, chosen, weights, top, softmax_scores=False, renormalise=False, groups=None, keep=None,
             renormalise_eps=0.0, group_top=1, weight_scale=1.0):
    """Per token, from the router's float32 logits [N, experts]: the `top` experts by score + bias (int32
    `chosen` [N, top]) and their scores (`weights`, divided by their sum + `renormalise_eps` with
    `renormalise`); scores are sigmoids, or a softmax over the experts.  With `groups` the experts form that
    many equal groups of neighbours and only those of the `keep` groups with the largest score can be chosen, a
    group's score being the sum of its `group_top` largest score + bias (1: its best).  The weights are multiplied
    by `weight_scale` at the end."""
    _require_cuda(logits, bias, chosen, weights)
    if logits.dtype != torch.float32 or chosen.shape[1] != top or not chosen.is_contiguous() or not weights.is_contiguous():
        raise KernelError("moe_pick: logits float32, chosen and weights contiguous [N, top]")
    fn = _fn("moe", "fl_moe_pick", [c_void_p, c_long, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_float, c_int, c_float, c_void_p])
    _check(fn(_ptr(logits), _ld(logits), _ptr(bias), F32 if bias is None else dtype_code(bias), _ptr(chosen),
              _ptr(weights), logits.shape[0], logits.shape[1], top, int(softmax_scores), int(renormalise),
              int(groups or 1), int(keep or groups or 1), float(renormalise_eps), int(group_top), float(weight_scale),
              _stream()), "moe_pick")


def moe_experts(h, w_gate_up, w_down, chosen, weights, act_buf, out, activation="silu", params=(0.0, 0.0), gated=True,
                accumulate=False):
    """out[t] = sum_k weights[t, k] * down[e](f(gate[e] h[t], up[e] h[t])), e = chosen[t, k], f as in ACTIVATIONS;
    w_gate_up [E, 2 ff, width], w_down [E, width, ff]; act_buf float32 [N * top, ff].  Without a gate
    (`gated=False`) w_gate_up is the up matrices alone, [E, ff, width], and the unit is f(up[e] h[t], 1).  With
    `accumulate` the sum is added to what `out` holds."""
    _require_cuda(h, w_gate_up, w_down, chosen, weights, act_buf, out)
    experts, ff2, width = w_gate_up.shape
    if not gated:
        ff2 *= 2
    fn = _fn("moe", "fl_moe_experts", [c_void_p, c_int, c_long, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p])
    _check(fn(_ptr(h), dtype_code(h), _ld(h), _ptr(w_gate_up), _ptr(w_down), dtype_code(w_gate_up), _ptr(chosen),
              _ptr(weights), _ptr(act_buf), _ptr(out), _ld(out), h.shape[0], width, ff2 // 2, chosen.shape[1],
              activation_code(activation), float(params[0]), float(params[1]), int(gated), int(accumulate), _stream()),
           "moe_experts", 2)


def moe_group_rows(n_tokens: int, top: int, experts: int) -> int:
    """Rows of the expert-ordered buffers for a step of `n_tokens` (every expert's rows end on a tile)."""
    fn = load_library("moe").fl_moe_group_rows
    fn.argtypes, fn.restype = [c_int, c_int, c_int], c_long
    return int(fn(n_tokens, top, experts))


def moe_group_takes(h_dtype, w_dtype, width: int, ff: int) -> bool:
    """Whether the grouped tensor-core path serves these types and sizes."""
    if h_dtype not in _CODES or w_dtype not in _CODES:
        return False
    fn = load_library("moe").fl_moe_group_takes
    fn.argtypes, fn.restype = [c_int, c_int, c_int, c_int], c_int
    return bool(fn(_CODES[h_dtype], _CODES[w_dtype], width, ff))


def moe_experts_grouped(h, w_gate_up, w_down, chosen, weights, ints, act, y, out, activation="silu", params=(0.0, 0.0),
                        gated=True, accumulate=False):
    """The same sum as `moe_experts` for many tokens: pairs ordered by expert, two tensor-core products
    over tiles of 64 rows, then the weighted sum per token.  All bfloat16; `ints` int32
    [rows + N * top + rows / 64 + 1], `act` bfloat16 [rows, ff], `y` float32 [rows, width] with
    rows = moe_group_rows(N, top, experts).  `gated=False`: as in `moe_experts`."""
    _require_cuda(h, w_gate_up, w_down, chosen, weights, ints, act, y, out)
    experts, ff2, width = w_gate_up.shape
    if not gated:
        ff2 *= 2
    fn = _fn("moe", "fl_moe_experts_grouped", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int,
                                               c_int, c_float, c_float, c_int, c_int, c_void_p])
    _check(fn(_ptr(h), _ld(h), _ptr(w_gate_up), _ptr(w_down), _ptr(chosen), _ptr(weights), _ptr(ints), _ptr(act),
              _ptr(y), _ptr(out), _ld(out), h.shape[0], width, ff2 // 2, chosen.shape[1], experts,
              activation_code(activation), float(params[0]), float(params[1]), int(gated), int(accumulate), _stream()),
           "moe_experts_grouped", 4)


# -------------------------------------------------------------- rope + cache

def rope_kv_write(qkv, n_heads, n_kv_heads, head_dim, rot_dim, cos, sin, positions, slots, cache,
                  page_size):
    """Rotate q in place; rotate k and copy v of each token into its cache slot.

    `cache` is one layer's [pages, 2, kv_heads, page_size, head_dim] tensor, or
    None when the rows hold queries only (a layer that reads another's cache)."""
    _require_cuda(qkv, cos, sin, positions, slots, cache)
    fn = _fn("rope_kv", "fl_rope_kv_write", [c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int,
                                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_long, c_int, c_int, c_void_p])
    if cache is not None:
        if cache.dtype != qkv.dtype:
            raise KernelError("rope_kv_write: cache and activations must have one dtype")
        k_ptr = c_void_p(cache.data_ptr())
        v_ptr = c_void_p(cache.data_ptr() + cache.stride(1) * cache.element_size())
        page_stride = cache.stride(0)
    else:
        k_ptr = v_ptr = None
        page_stride = 0
    _check(fn(_ptr(qkv), dtype_code(qkv), _ld(qkv), qkv.shape[0], n_heads, n_kv_heads, head_dim,
              rot_dim, _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slots), k_ptr, v_ptr, page_stride,
              page_size, 0 if cache is None else 1, _stream()), "rope_kv_write")


# ------------------------------------------------------------------ attention

def paged_attention_simt(q, out, cache, block_table, tok_req, positions, n_heads, n_kv_heads,
                         head_dim, window, scale, page_size):
    """Causal attention of every token in q over its request's cached keys (CUDA cores)."""
    _require_cuda(q, out, cache, block_table, tok_req, positions)
    if head_dim > 256:
        raise KernelError(f"attention: head_dim {head_dim} is beyond the kernel's limit of 256")
    fn = _fn("attention_simt", "fl_paged_attention_simt",
             [c_void_p, c_int, c_long, c_void_p, c_long, c_void_p, c_void_p, c_long, c_int, c_void_p,
              c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    k_ptr = c_void_p(cache.data_ptr())
    v_ptr = c_void_p(cache.data_ptr() + cache.stride(1) * cache.element_size())
    _check(fn(_ptr(q), dtype_code(q), _ld(q), _ptr(out), _ld(out), k_ptr, v_ptr, cache.stride(0),
              page_size, _ptr(block_table), block_table.stride(0), _ptr(tok_req), _ptr(positions),
              q.shape[0], n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _stream()),
           "paged_attention_simt")


# ----------------------------------------------------------------------- GEMM

def gemm_simt(a, w, out):
    """out[M, N] = a[M, K] @ w[N, K]^T, float accumulation on CUDA cores, any dtypes."""
    _require_cuda(a, w, out)
    if a.shape[1] != w.shape[1] or out.shape[0] != a.shape[0] or out.shape[1] != w.shape[0]:
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_simt", "fl_gemm_simt", [c_void_p, c_int, c_long, c_void_p, c_int, c_long, c_void_p,
                                           c_int, c_long, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(a), dtype_code(a), _ld(a), _ptr(w), dtype_code(w), _ld(w), _ptr(out),
              dtype_code(out), _ld(out), a.shape[0], w.shape[0], a.shape[1], _stream()), "gemm_simt")


# ------------------------------------------------------------------- sampling

def sample(logits, out, temperature=None, top_k=None, top_p=None, min_p=None, uniform=None):
    """One token per logits row into `out` (int32); null temperature = greedy everywhere."""
    _require_cuda(logits, out, temperature, top_k, top_p, min_p, uniform)
    if logits.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("sample: logits must be float32 and out int32")
    if temperature is not None and uniform is None:
        raise KernelError("sample: temperature sampling needs uniform numbers")
    fn = _fn("sampling", "fl_sample", [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), _ld(logits), logits.shape[0], logits.shape[1], _ptr(temperature),
              _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform), _ptr(out), _stream()), "sample")


def apply_penalties(logits, rows, tokens, counts, repetition, frequency, presence):
    _require_cuda(logits, rows, tokens, counts, repetition, frequency, presence)
    fn = _fn("sampling", "fl_apply_penalties", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int,
                                                c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(logits), _ld(logits), _ptr(rows), _ptr(tokens), _ptr(counts), rows.numel(),
              _ptr(repetition), _ptr(frequency), _ptr(presence), logits.shape[1], _stream()),
           "apply_penalties")


# ---------------------------------------------------------------------- build

BASE_LIBRARIES = ["elementwise", "gemm_simt", "sampling"]      # every model; a part names what else it needs
BF16_LIBRARIES = ["gemm_tcgen05"]
