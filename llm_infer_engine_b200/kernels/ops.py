"""Python faces of the CUDA kernels: argument checks, then one ctypes call per launch.

Every function takes CUDA tensors, checks dtype / shape / contiguity on the host (the checks
stand in for a memory checker: no kernel is ever launched on sizes it was not written for),
launches on torch's current stream and returns without synchronising. There is no CPU or
library fallback: a tensor that is not on a GPU, or a kernel library that cannot be built,
raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build, trace

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_ERRORS = {-1: "bad argument", -2: "size not supported by this kernel", -3: "pointer not aligned",
           -4: "dtype not supported"}
F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_fn_cache = {}


class KernelError(RuntimeError):
    pass


PDL = True        # programmatic dependent launch between this library's kernels (see csrc/common.cuh)


def set_pdl(on: bool) -> None:
    """Turns programmatic dependent launch on or off for every kernel library, loaded or yet to be."""
    global PDL
    PDL = bool(on)
    for family in list(_pdl_state):
        _apply_pdl(family)


_pdl_state = {}


def _apply_pdl(family: str) -> None:
    if _pdl_state.get(family) != PDL:
        lib = build.load(family)
        lib.llmie_set_pdl.argtypes = [_c_int]
        lib.llmie_set_pdl.restype = None
        lib.llmie_set_pdl(1 if PDL else 0)
        _pdl_state[family] = PDL


def _fn(family: str, name: str, argtypes, query: bool = False):
    """The exported function `name` of a kernel family. `query=True` marks a host-side question (no launch),
    which the per-kernel timer leaves alone."""
    key = (family, name)
    f = _fn_cache.get(key)
    if f is None:
        lib = build.load(family)
        raw = getattr(lib, name)
        raw.argtypes = argtypes
        raw.restype = _c_int
        _apply_pdl(family)
        short = name[6:] if name.startswith("llmie_") else name
        if query:
            _fn_cache[key] = raw
            return raw

        def f(*args, _raw=raw, _name=short):
            t = trace.timer
            return _raw(*args) if t is None else t.run(_name, _raw, args)

        _fn_cache[key] = f
    return f


def _work(nbytes: float = 0.0, flops: float = 0.0) -> None:
    """Tells an installed per-kernel timer what the next launch moves and computes."""
    if trace.timer is not None:
        trace.timer.note(nbytes, flops)


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def library_mm(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [T, K] @ w[N, K]^T through the library GEMM (cuBLAS), for the products the reference leaves to
    nn.Linear; seen by the per-kernel timer like this library's own launches."""
    def run():
        if out_dtype == x.dtype:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out_dtype=out_dtype)
    t = trace.timer
    if t is None:
        return run()
    T, K = x.shape
    N = w.shape[0]
    t.note(_nbytes(x, w) + T * N * (2 if out_dtype == torch.bfloat16 else 4), 2.0 * T * N * K)
    return t.run("library_mm", run, ())


LAUNCHES = 0      # kernels of this library launched so far (captured launches count once, at capture)


def _check(status: int, name: str) -> None:
    if status == 0:
        global LAUNCHES
        LAUNCHES += 1
        return
    if status < 0:
        raise KernelError(f"{name}: {_ERRORS.get(status, 'error ' + str(status))}")
    raise KernelError(f"{name}: CUDA error {status} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream of the current device as a raw handle."""
    if _raw_stream is not None:
        return _raw_stream(_get_device() if _get_device is not None else torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor, what: str) -> int:
    code = _DT.get(t.dtype)
    if code is None:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)")
    return code


def _need(t: torch.Tensor, what: str, dtype=None, shape=None) -> None:
    """The checks every launch makes of every tensor it is given (written for speed: an eager step makes
    several hundred of them)."""
    if not t.is_cuda:
        raise KernelError(f"{what}: must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{what}: must be contiguous")
    if dtype is not None and t.dtype is not dtype:
        raise KernelError(f"{what}: dtype {t.dtype}, expected {dtype}")
    if shape is not None:
        have = t.shape
        bad = len(have) != len(shape)
        if not bad:
            for want, got in zip(shape, have):
                if want is not None and want != got:
                    bad = True
                    break
        if bad:
            raise KernelError(f"{what}: shape {tuple(have)}, expected {tuple(shape)}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ------------------------------------------------------------------------------------------
def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tokens[t]] as float32. tokens int32 [T]; table [V, d]; out float32 [T, d]."""
    T = tokens.shape[0]
    V, d = table.shape
    _need(tokens, "tokens", torch.int32, (T,))
    _need(table, "table")
    _need(out, "out", torch.float32, (T, d))
    _work(T * 4 + T * d * table.element_size() + _nbytes(out))
    f = _fn("elementwise", "llmie_embedding",
            [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(tokens.data_ptr(), table.data_ptr(), _dt(table, "table"), out.data_ptr(), T, d, V, _stream()),
           "embedding")
    return out


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h += delta (float32, in place, when rows is None); out = rmsnorm(h) * weight.

    h float32 [T, d]; delta [T, d] of out's dtype or None; weight float32 [d]; out [n_out, d].
    With `rows` (int32 [n_out]) only those rows of h (+ delta) are normalised and h is left as it is."""
    T, d = h.shape
    n_out = T if rows is None else rows.shape[0]
    _need(h, "h", torch.float32)
    _need(weight, "weight", torch.float32, (d,))
    _need(out, "out", None, (n_out, d))
    if delta is not None:
        _need(delta, "delta", out.dtype, (T, d))
    if rows is not None:
        _need(rows, "rows", torch.int32, (n_out,))
    _work((2 * _nbytes(h) if rows is None else n_out * d * 4) + _nbytes(delta, out))
    f = _fn("elementwise", "llmie_add_rmsnorm",
            [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_float, _c_int, _c_void_p])
    _check(f(h.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(), _ptr(rows), n_out, d, float(eps),
             _dt(out, "out"), _stream()), "add_rmsnorm")
    return out


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """h += delta; h float32, delta float32 or bfloat16 of the same shape."""
    _need(h, "h", torch.float32)
    _need(delta, "delta", None, tuple(h.shape))
    f = _fn("elementwise", "llmie_residual_add", [_c_void_p, _c_void_p, ctypes.c_longlong, _c_int, _c_void_p])
    _check(f(h.data_ptr(), delta.data_ptr(), h.numel(), _dt(delta, "delta"), _stream()), "residual_add")
    return h


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, j] = silu(gate_up[t, j]) * gate_up[t, ff + j]; gate_up [T, 2 ff], out [T, ff]."""
    T, ff = out.shape
    _need(out, "out")
    _need(gate_up, "gate_up", out.dtype, (T, 2 * ff))
    _work(_nbytes(gate_up, out))
    f = _fn("elementwise", "llmie_swiglu", [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(gate_up.data_ptr(), out.data_ptr(), T, ff, _dt(out, "out"), _stream()), "swiglu")
    return out


def rope_store(qkv, q_out, k_cache, v_cache, table, tok_pos, tok_seq, seq_slot, block_table, page_size: int,
               n_q: int, n_kv: int, head_dim: int, rot_dim: int, write_kv: bool = True,
               v_head_dim: Optional[int] = None):
    """Rotates q and k by position and writes k, v into the paged cache.

    qkv [T, (n_q + n_kv) hd + n_kv hdv]; q_out [T, n_q hd]; caches [n_pages, n_kv, page_size, hd] (same dtype), the
    value cache with hdv (`v_head_dim`, default hd) in place of hd;
    table float32 [max_pos, rot_dim / 2, 2] of (cos, sin) or None for no rotation;
    tok_pos, tok_seq int32 [T]; seq_slot int32 [n]; block_table int32 [n_slots, max_pages]."""
    T = qkv.shape[0]
    hdv = head_dim if v_head_dim is None else int(v_head_dim)
    _need(qkv, "qkv", None, (T, (n_q + n_kv) * head_dim + n_kv * hdv))
    _need(q_out, "q_out", qkv.dtype, (T, n_q * head_dim))
    _need(tok_pos, "tok_pos", torch.int32)
    _need(tok_seq, "tok_seq", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if tok_pos.shape[0] < T or tok_seq.shape[0] < T:
        raise KernelError("rope_store: tok_pos / tok_seq shorter than the token count")
    table_len = 0
    if table is not None:
        _need(table, "table", torch.float32, (None, rot_dim // 2, 2))
        table_len = table.shape[0]
    if write_kv:
        _need(k_cache, "k_cache", qkv.dtype, (None, n_kv, page_size, head_dim))
        _need(v_cache, "v_cache", qkv.dtype, tuple(k_cache.shape[:-1]) + (hdv,))
    _work(_nbytes(qkv, q_out) + (T * n_kv * (head_dim + hdv) * qkv.element_size() if write_kv else 0))
    f = _fn("elementwise", "llmie_rope_store_ex",
            [_c_void_p] * 9 + [_c_int] * 11 + [_c_void_p])
    _check(f(qkv.data_ptr(), q_out.data_ptr(), _ptr(k_cache) if write_kv else None,
             _ptr(v_cache) if write_kv else None, _ptr(table), tok_pos.data_ptr(), tok_seq.data_ptr(),
             seq_slot.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, T, n_q,
             n_kv, head_dim, hdv, rot_dim, table_len, 1 if write_kv else 0, _dt(qkv, "qkv"), _stream()), "rope_store")
    return q_out


def attention_paged(q, k_cache, v_cache, out, tok_pos, tok_seq, seq_slot, block_table, page_size: int,
                    n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0, keep_first: int = 0,
                    sink: bool = False, gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                    dist_bias: Optional[torch.Tensor] = None, sink_values: Optional[torch.Tensor] = None,
                    sigmoid_bias: Optional[torch.Tensor] = None):
    """Plain attention over the paged cache, one warp per (token, query head).
    q [T, n_q hd]; out [T, n_q hdv]; k_cache [n_pages, n_kv, page_size, hd]; v_cache the same with hdv (the value
    head size, read from its shape). window 0 = all earlier keys; the first `keep_first` keys of a sequence stay
    visible behind the window; `sink` adds a key of score 0 without a value to the softmax; `gate` (rows of
    n_q hdv elements, possibly a column slice of a wider tensor) multiplies the output by its sigmoid. `softcap` c > 0
    turns a scaled score s into c tanh(s / c); `dist_bias` (float32 [n_q, L]) adds a number per head and distance
    (query position - key position; distances >= L - 1 share the last column), after the cap and unscaled;
    `sink_values` (float32 [n_q]) are the sink's score per head instead of 0. v_cache may be a view of the first hdv
    columns of k_cache's rows (a latent that is key and value at once). `sigmoid_bias` (float32 [n_q]): no softmax;
    a visible key's weight is sigmoid(score + sigmoid_bias[head]), not normalised over the keys."""
    T = q.shape[0]
    hdv = v_cache.shape[-1]
    _need(q, "q", None, (T, n_q * head_dim))
    _need(out, "out", q.dtype, (T, n_q * hdv))
    _need(k_cache, "k_cache", q.dtype, (None, n_kv, page_size, head_dim))
    if v_cache.is_contiguous():
        _need(v_cache, "v_cache", q.dtype, (k_cache.shape[0], n_kv, page_size, hdv))
        v_ld = hdv
    else:
        # rows of hdv elements inside wider rows: every row must start v_ld elements after the one before
        v_ld = v_cache.stride(-2)
        if (v_cache.dtype is not q.dtype or tuple(v_cache.shape) != (k_cache.shape[0], n_kv, page_size, hdv)
                or v_cache.stride(-1) != 1 or v_ld < hdv
                or v_cache.stride() != (n_kv * page_size * v_ld, page_size * v_ld, v_ld, 1)):
            raise KernelError("attention_paged: v_cache must be contiguous or a column range of contiguous rows")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if head_dim > 1024 or hdv > 1024:
        raise KernelError(f"attention_paged: head sizes {head_dim} / {hdv} must be at most 1024")
    bias_len = 0
    if dist_bias is not None:
        _need(dist_bias, "dist_bias", torch.float32, (n_q, None))
        bias_len = dist_bias.shape[1]
    if sink_values is not None:
        _need(sink_values, "sink_values", torch.float32, (n_q,))
        sink = True
    if sigmoid_bias is not None:
        _need(sigmoid_bias, "sigmoid_bias", torch.float32, (n_q,))
        if sink:
            raise KernelError("attention_paged: sigmoid weights have no denominator for a sink to enter")
    gate_ld = 0
    if gate is not None:
        gate_ld = _row_slice(gate, "gate", q.dtype, T, n_q * hdv)
    _work(2 * _nbytes(q) + 1.0 * STEP_HINT["kv_total"] * n_kv * (head_dim + hdv) * q.element_size(),
          2.0 * n_q * (head_dim + hdv) * STEP_HINT["pairs"])
    f = _fn("attention_simt", "llmie_attention_paged_sig",
            [_c_void_p] * 8 + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_float,
                                              _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p])
    _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), tok_pos.data_ptr(),
             tok_seq.data_ptr(), seq_slot.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, T,
             n_q, n_kv, head_dim, hdv, float(scale), int(window), int(keep_first), 1 if sink else 0, _ptr(gate),
             gate_ld, int(v_ld), float(softcap or 0.0), _ptr(dist_bias), bias_len, _ptr(sink_values),
             _ptr(sigmoid_bias), _dt(q, "q"), _stream()), "attention_paged")
    return out


def _row_slice(t: torch.Tensor, what: str, dtype, rows: int, cols: int) -> int:
    """Checks a [rows, cols] tensor that may be a column slice of a wider contiguous one; returns its row stride."""
    if not t.is_cuda:
        raise KernelError(f"{what}: must be a CUDA tensor")
    if t.dtype is not dtype:
        raise KernelError(f"{what}: dtype {t.dtype}, expected {dtype}")
    if t.dim() != 2 or t.shape[0] != rows or t.shape[1] != cols:
        raise KernelError(f"{what}: shape {tuple(t.shape)}, expected {(rows, cols)}")
    if t.stride(1) != 1 or (rows > 1 and t.stride(0) < cols):
        raise KernelError(f"{what}: rows must be contiguous runs of {cols} elements")
    return t.stride(0) if rows > 1 else max(t.stride(0), cols)


ACT_NONE, ACT_RELU, ACT_RELU2, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3, 4
ACTIVATIONS = {"none": ACT_NONE, "relu": ACT_RELU, "relu2": ACT_RELU2, "gelu_tanh": ACT_GELU_TANH, "silu": ACT_SILU}


def scale_pos_norm(h, scale: float, pos_table, tok_pos, norm_w, eps: float, act=None):
    """h (float32 [T, d], in place) = norm(h * scale + pos_table[tok_pos]); pos_table [P, d] (float32 or bfloat16)
    and norm_w (float32 [d]) are optional; act (optional, [T, d]) receives h rounded to its dtype."""
    T, d = h.shape
    _need(h, "h", torch.float32)
    if pos_table is not None:
        _need(pos_table, "pos_table", None, (None, d))
        _need(tok_pos, "tok_pos", torch.int32)
        if tok_pos.shape[0] < T:
            raise KernelError("scale_pos_norm: tok_pos shorter than the token count")
    if norm_w is not None:
        _need(norm_w, "norm_w", torch.float32, (d,))
    if act is not None:
        _need(act, "act", None, (T, d))
    _work(2 * _nbytes(h) + _nbytes(act) + (T * d * pos_table.element_size() if pos_table is not None else 0))
    f = _fn("branch_elementwise", "llmie_scale_pos_norm",
            [_c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_int,
             _c_int, _c_void_p])
    _check(f(h.data_ptr(), float(scale), _ptr(pos_table), _dt(pos_table, "pos_table") if pos_table is not None else 0,
             pos_table.shape[0] if pos_table is not None else 0, _ptr(tok_pos) if pos_table is not None else None,
             _ptr(norm_w), float(eps), _ptr(act), _dt(act, "act") if act is not None else 0, T, d, _stream()),
           "scale_pos_norm")
    return h


def branch_norm_add(h, y, bias, weight, eps: float, act=None):
    """h (float32 [T, d]) += rmsnorm(y + bias) * weight: the norm sits on a branch's output. y [T, d] float32 or
    bfloat16; bias float32 [d] or None; act (optional [T, d]) receives the new h rounded to its dtype."""
    T, d = h.shape
    _need(h, "h", torch.float32)
    _need(y, "y", None, (T, d))
    _need(weight, "weight", torch.float32, (d,))
    if bias is not None:
        _need(bias, "bias", torch.float32, (d,))
    if act is not None:
        _need(act, "act", None, (T, d))
    _work(2 * _nbytes(h) + _nbytes(y, act))
    f = _fn("branch_elementwise", "llmie_branch_norm_add",
            [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(h.data_ptr(), y.data_ptr(), _dt(y, "y"), _ptr(bias), weight.data_ptr(), float(eps), _ptr(act),
             _dt(act, "act") if act is not None else 0, T, d, _stream()), "branch_norm_add")
    return h


def bias_act(u, bias, out, act: int):
    """out[T, n] = act(u[T, n] + bias[n]); bias float32 or None; act one of the ACT_* codes."""
    T, n = u.shape
    _need(u, "u")
    _need(out, "out", None, (T, n))
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    _work(_nbytes(u, out))
    f = _fn("branch_elementwise", "llmie_bias_act",
            [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(u.data_ptr(), _dt(u, "u"), _ptr(bias), out.data_ptr(), _dt(out, "out"), T, n, int(act), _stream()),
           "bias_act")
    return out


def cast_rows(x, out):
    """out = x (float32) rounded to out's dtype."""
    _need(x, "x", torch.float32)
    _need(out, "out", None, tuple(x.shape))
    _work(_nbytes(x, out))
    f = _fn("branch_elementwise", "llmie_cast_rows", [_c_void_p, _c_void_p, _c_int, ctypes.c_longlong, _c_void_p])
    _check(f(x.data_ptr(), out.data_ptr(), _dt(out, "out"), x.numel(), _stream()), "cast_rows")
    return out


def sigmoid_gate(out, gate, group: int = 1):
    """out[T, n] *= sigmoid(gate[T, n / group]) with every gate serving a run of `group` columns (group 1: a gate per
    element; group = a head's value size: one gate per head); gate may be a column slice of a wider tensor."""
    T, n = out.shape
    _need(out, "out")
    if group <= 0 or n % group:
        raise KernelError(f"sigmoid_gate: rows of {n} elements are not whole groups of {group}")
    ld = _row_slice(gate, "gate", out.dtype, T, n // group)
    _work(2 * _nbytes(out) + T * (n // group) * out.element_size())
    f = _fn("branch_elementwise", "llmie_sigmoid_gate_grouped",
            [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(out.data_ptr(), gate.data_ptr(), ld, T, n, int(group), _dt(out, "out"), _stream()), "sigmoid_gate")
    return out


def scaled_sum_norm(h, y, scale, alpha: float, weight, eps: float, act=None):
    """Norm after the residual sum: h (float32 [T, d]) = rmsnorm(alpha * h + scale (.) y) * weight, in place. y [T, d]
    float32 or bfloat16; scale float32 [d] (a learned number per channel) or None; act (optional [T, d]) receives the
    new h rounded to its dtype."""
    T, d = h.shape
    _need(h, "h", torch.float32)
    _need(y, "y", None, (T, d))
    _need(weight, "weight", torch.float32, (d,))
    if scale is not None:
        _need(scale, "scale", torch.float32, (d,))
    if act is not None:
        _need(act, "act", None, (T, d))
    _work(2 * _nbytes(h) + _nbytes(y, act))
    f = _fn("branch_elementwise", "llmie_scaled_sum_norm",
            [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_float, _c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_int,
             _c_void_p])
    _check(f(h.data_ptr(), y.data_ptr(), _dt(y, "y"), _ptr(scale), float(alpha), weight.data_ptr(), float(eps),
             _ptr(act), _dt(act, "act") if act is not None else 0, T, d, _stream()), "scaled_sum_norm")
    return h


def rmsnorm_cols(src, off: int, n: int, weight, eps: float, out):
    """out [T, n] = RMS norm of the columns off .. off + n - 1 of src [T, ld], times weight float32 [n]; float32
    arithmetic, out of src's dtype."""
    T, ld = src.shape
    _need(src, "src")
    _need(out, "out", src.dtype, (T, n))
    _need(weight, "weight", torch.float32, (n,))
    if off < 0 or off + n > ld:
        raise KernelError("rmsnorm_cols: the columns do not fit the rows of src")
    _work(T * n * 2 * src.element_size())
    f = _fn("branch_elementwise", "llmie_rmsnorm_cols",
            [_c_void_p, _c_int, _c_int, _c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(src.data_ptr(), ld, int(off), weight.data_ptr(), float(eps), out.data_ptr(), T, n, _dt(src, "src"),
             _stream()), "rmsnorm_cols")
    return out


def qk_norm_store(proj, q_out, k_cache, v_cache, q_w, k_w, eps: float, tok_pos, tok_seq, seq_slot, block_table,
                  page_size: int, n_q: int, n_kv: int, head_dim: int, v_head_dim: int, write_kv: bool = True,
                  lam: Optional[torch.Tensor] = None, v_first: Optional[torch.Tensor] = None,
                  temp_coef: float = 0.0, temp_every: int = 0):
    """RMS norm over the WHOLE query projection and over the whole key projection (not per head), value blending,
    and the cache write. proj [T, >= n_q hd + n_kv hd + n_kv hdv] holds [q | k | v | ...] per row; q_out [T, n_q hd];
    q_w / k_w float32 weights of the norms (None: that projection is copied as it is); with `v_first` (rows of
    n_kv hdv values, possibly a column slice) the stored values are (1 - lam) v + lam v_first, lam a float32 scalar
    on the device. With `temp_every` > 0 the queries of position p are also multiplied by
    1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (a temperature that grows with the position)."""
    T, ld = proj.shape
    nq, nk, nv = n_q * head_dim, n_kv * head_dim, n_kv * v_head_dim
    _need(proj, "proj")
    if ld < nq + nk + nv:
        raise KernelError(f"qk_norm_store: rows of {ld} elements cannot hold q, k and v ({nq} + {nk} + {nv})")
    _need(q_out, "q_out", proj.dtype, (T, nq))
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if tok_pos.shape[0] < T or tok_seq.shape[0] < T:
        raise KernelError("qk_norm_store: tok_pos / tok_seq shorter than the token count")
    if q_w is not None:
        _need(q_w, "q_w", torch.float32, (nq,))
    if k_w is not None:
        _need(k_w, "k_w", torch.float32, (nk,))
    if write_kv:
        _need(k_cache, "k_cache", proj.dtype, (None, n_kv, page_size, head_dim))
        _need(v_cache, "v_cache", proj.dtype, (k_cache.shape[0], n_kv, page_size, v_head_dim))
    vf_ld = 0
    if v_first is not None:
        vf_ld = _row_slice(v_first, "v_first", proj.dtype, T, nv)
        if lam is None:
            raise KernelError("qk_norm_store: v_first needs lam")
        _need(lam, "lam", torch.float32)
        if lam.numel() != 1:
            raise KernelError("qk_norm_store: lam must hold one number")
    _work((T * (nq + nk + nv) + T * nq + (T * (nk + nv) if write_kv else 0)) * proj.element_size())
    f = _fn("branch_elementwise", "llmie_qk_norm_store_temp",
            [_c_void_p, _c_int] + [_c_void_p] * 5 + [_c_float, _c_void_p, _c_void_p, _c_int] + [_c_void_p] * 4 +
            [_c_int] * 9 + [_c_float, _c_int, _c_void_p])
    _check(f(proj.data_ptr(), ld, q_out.data_ptr(), _ptr(k_cache) if write_kv else None,
             _ptr(v_cache) if write_kv else None, _ptr(q_w), _ptr(k_w), float(eps), _ptr(lam) if v_first is not None else None,
             _ptr(v_first), vf_ld, tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), block_table.data_ptr(),
             block_table.shape[1], page_size, T, n_q, n_kv, head_dim, v_head_dim, 1 if write_kv else 0,
             _dt(proj, "proj"), float(temp_coef), int(temp_every), _stream()), "qk_norm_store")
    return q_out


def attention_decode_supported(head_dim: int, dtype: torch.dtype) -> bool:
    """The head sizes attention_decode.cu is instantiated for. Answered here, without loading the library: a model
    whose sizes it does not take never has it compiled."""
    return dtype in _DT and head_dim in (16, 32, 64, 128)


def attention_decode_run_len(n_seqs: int, head_dim: int, dtype: torch.dtype) -> int:
    """Keys per block that attention_decode wants for this many sequences (a multiple of the page size)."""
    lib = build.load("attention_decode")
    lib.llmie_attention_decode_run_len.argtypes = [_c_int, _c_int, _c_int]
    lib.llmie_attention_decode_run_len.restype = _c_int
    return int(lib.llmie_attention_decode_run_len(n_seqs, head_dim, _DT[dtype]))


def decode_scratch_floats(n_seqs: int, n_q: int, head_dim: int, n_runs: int) -> int:
    """float32 elements of scratch that attention_decode needs."""
    return n_seqs * n_q * n_runs * (head_dim + 2)


def decode_counter_ints(n_seqs: int, n_q: int, n_kv: int) -> int:
    """int32 counters that the one-launch form of attention_decode needs (all zero, left zero)."""
    g = n_q // n_kv
    return n_seqs * n_kv * ((g + 3) // 4 if g <= 4 else (g + 7) // 8)


def attention_decode(q, k_cache, v_cache, out, seq_slot, seq_kvlen, block_table, page_size: int, n_q: int,
                     n_kv: int, head_dim: int, scale: float, window: int, run_len: int, n_runs: int,
                     scratch: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None):
    """Split-KV attention for a step in which every sequence brings one token.

    q, out [n, n_q hd]; seq_kvlen int32 [n] = keys each sequence holds INCLUDING this step's;
    n_runs * run_len must be at least the longest length that seq_kvlen can name; run_len is the
    page size. scratch: float32 with decode_scratch_floats(...) elements (allocated here if None).
    With `counters` (int32 zeros, decode_counter_ints(...) of them) the runs are merged by the last
    block of the same launch instead of a second kernel."""
    n = q.shape[0]
    _need(q, "q", None, (n, n_q * head_dim))
    _need(out, "out", q.dtype, (n, n_q * head_dim))
    _need(k_cache, "k_cache", q.dtype, (None, n_kv, page_size, head_dim))
    _need(v_cache, "v_cache", q.dtype, tuple(k_cache.shape))
    for name, t in (("seq_slot", seq_slot), ("seq_kvlen", seq_kvlen), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if seq_slot.numel() < n or seq_kvlen.numel() < n:
        raise KernelError("attention_decode: seq_slot / seq_kvlen shorter than the number of sequences")
    need = decode_scratch_floats(n, n_q, head_dim, n_runs)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    _need(scratch, "scratch", torch.float32)
    if scratch.numel() < need:
        raise KernelError(f"attention_decode: scratch holds {scratch.numel()} floats, {need} are needed")
    n_ml = n * n_q * n_runs
    base = scratch.data_ptr()
    if counters is not None:
        _need(counters, "counters", torch.int32)
        if counters.numel() < decode_counter_ints(n, n_q, n_kv):
            raise KernelError("attention_decode: too few counters")
        _work(2 * _nbytes(q) + 2.0 * STEP_HINT["kv_total"] * n_kv * head_dim * q.element_size(),
              4.0 * n_q * head_dim * STEP_HINT["pairs"])
        f = _fn("attention_decode", "llmie_attention_decode_fused",
                [_c_void_p] * 11 + [_c_int] * 6 + [_c_float] + [_c_int] * 4 + [_c_void_p])
        _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), base, base + 4 * n_ml,
                 base + 8 * n_ml, counters.data_ptr(), seq_slot.data_ptr(), seq_kvlen.data_ptr(),
                 block_table.data_ptr(), block_table.shape[1], page_size, n, n_q, n_kv, head_dim, float(scale),
                 int(window), int(run_len), int(n_runs), _dt(q, "q"), _stream()), "attention_decode")
        return out
    f = _fn("attention_decode", "llmie_attention_decode",
            [_c_void_p] * 10 + [_c_int] * 6 + [_c_float] + [_c_int] * 4 + [_c_void_p])
    _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), base, base + 4 * n_ml,
             base + 8 * n_ml, seq_slot.data_ptr(), seq_kvlen.data_ptr(), block_table.data_ptr(),
             block_table.shape[1], page_size, n, n_q, n_kv, head_dim, float(scale), int(window), int(run_len),
             int(n_runs), _dt(q, "q"), _stream()), "attention_decode")
    return out


# What a step's attention really reads is known to the caller, not to the launcher (which is sized for upper
# bounds): when a per-kernel timer is installed the engine leaves here, for the timer's counts, the keys all
# sequences of the step hold together and the (query, key) pairs the step's causal attention visits.
STEP_HINT = {"kv_total": 0, "pairs": 0}

MMA_MAX_BLOCKS = 148 * 2        # blocks the decode attention aims at: two per SM


def attention_decode_mma_supported(head_dim: int, dtype: torch.dtype, page_size: int) -> bool:
    """The sizes attention_decode_mma.cu is instantiated for (answered without loading the library)."""
    return dtype == torch.bfloat16 and page_size == 64 and head_dim in (64, 128)


def attention_decode_mma_pages(n_seqs: int, n_q: int, n_kv: int, max_kv_len: int,
                               max_blocks: Optional[int] = None) -> int:
    """Cache pages per block that attention_decode_mma wants for this step's shape."""
    groups = n_kv * ((n_q // n_kv + 15) // 16)
    f = _fn("attention_decode_mma", "llmie_attention_decode_mma_pages", [_c_int] * 4, query=True)
    return int(f(n_seqs, groups, max_kv_len, MMA_MAX_BLOCKS if max_blocks is None else max_blocks))


def attention_decode_mma(q, k_cache, v_cache, out, seq_slot, seq_kvlen, block_table, page_size: int, n_q: int,
                         n_kv: int, head_dim: int, scale: float, window: int, pages_per_run: int, n_runs: int,
                         counters: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None,
                         keep_first: int = 0, sink: bool = False, gate: Optional[torch.Tensor] = None,
                         softcap: float = 0.0, dist_bias: Optional[torch.Tensor] = None,
                         sink_values: Optional[torch.Tensor] = None, sigmoid_bias: Optional[torch.Tensor] = None):
    """Attention for a one-token step on the tensor cores (bfloat16): a warp per cache page, the warps of a
    block merged in shared memory. Arguments as attention_decode; n_runs * pages_per_run pages must cover
    the longest sequence. With n_runs == 1 neither scratch nor counters are touched. keep_first, sink and gate
    as in attention_paged. With sigmoid_bias (float32 [n_q]) there is no softmax: the weight of a visible key is
    sigmoid(scaled score + sigmoid_bias[head]), not normalised (no sink, cap or bias by distance with it)."""
    n = q.shape[0]
    gate_ld = _row_slice(gate, "gate", torch.bfloat16, n, n_q * head_dim) if gate is not None else 0
    _need(q, "q", torch.bfloat16, (n, n_q * head_dim))
    _need(out, "out", torch.bfloat16, (n, n_q * head_dim))
    _need(k_cache, "k_cache", torch.bfloat16, (None, n_kv, page_size, head_dim))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    for name, t in (("seq_slot", seq_slot), ("seq_kvlen", seq_kvlen), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if seq_slot.numel() < n or seq_kvlen.numel() < n:
        raise KernelError("attention_decode_mma: seq_slot / seq_kvlen shorter than the number of sequences")
    base = n_ml = 0
    cptr = None
    if n_runs > 1:
        need = decode_scratch_floats(n, n_q, head_dim, n_runs)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError(f"attention_decode_mma: scratch holds {scratch.numel()} floats, {need} are needed")
        if counters is None or counters.numel() < n * n_kv * ((n_q // n_kv + 15) // 16):
            raise KernelError("attention_decode_mma: counters are needed when a sequence spans several runs")
        _need(counters, "counters", torch.int32)
        base, n_ml, cptr = scratch.data_ptr(), n * n_q * n_runs, counters.data_ptr()
    _work(2 * _nbytes(q) + 2.0 * STEP_HINT["kv_total"] * n_kv * head_dim * 2, 4.0 * n_q * head_dim * STEP_HINT["pairs"])
    f = _fn("attention_decode_mma", "llmie_attention_decode_mma_ex",
            [_c_void_p] * 11 + [_c_int] * 6 + [_c_float] + [_c_int] * 5 + [_c_void_p, _c_int, _c_float, _c_void_p,
                                                                            _c_int, _c_void_p, _c_void_p, _c_void_p])
    if sigmoid_bias is not None:
        if sink or softcap or dist_bias is not None or sink_values is not None:
            raise KernelError("attention_decode_mma: sigmoid weights take no sink, cap or bias by distance")
        _need(sigmoid_bias, "sigmoid_bias", torch.float32, (n_q,))
    bias_len = 0
    if dist_bias is not None:
        _need(dist_bias, "dist_bias", torch.float32, (n_q, None))
        bias_len = dist_bias.shape[1]
    if sink_values is not None:
        _need(sink_values, "sink_values", torch.float32, (n_q,))
        sink = True
    _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), base or None,
             (base + 4 * n_ml) or None, (base + 8 * n_ml) or None, cptr, seq_slot.data_ptr(), seq_kvlen.data_ptr(),
             block_table.data_ptr(), block_table.shape[1], page_size, n, n_q, n_kv, head_dim, float(scale),
             int(window), int(pages_per_run), int(n_runs), int(keep_first), 1 if sink else 0, _ptr(gate), gate_ld,
             float(softcap or 0.0), _ptr(dist_bias), bias_len, _ptr(sink_values), _ptr(sigmoid_bias), _stream()),
           "attention_decode_mma")
    return out


def attention_decode_mma_rope(qkv, k_cache, v_cache, out, table, seq_slot, seq_kvlen, block_table, page_size: int,
                              n_q: int, n_kv: int, head_dim: int, scale: float, window: int, pages_per_run: int,
                              n_runs: int, write_kv: bool = True, counters: Optional[torch.Tensor] = None,
                              scratch: Optional[torch.Tensor] = None):
    """attention_decode_mma with the position encoding and the cache write inside: qkv bfloat16
    [n, (n_q + 2 n_kv) hd] holds the step's raw q, k and v heads; table float32 [max_pos, hd / 2, 2] is the
    (cos, sin) table of a rotation over the whole head size. Sequence i's new key and value are taken for
    position seq_kvlen[i] - 1 and, with write_kv, written into the cache there."""
    n = qkv.shape[0]
    _need(qkv, "qkv", torch.bfloat16, (n, (n_q + 2 * n_kv) * head_dim))
    _need(out, "out", torch.bfloat16, (n, n_q * head_dim))
    _need(k_cache, "k_cache", torch.bfloat16, (None, n_kv, page_size, head_dim))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _need(table, "table", torch.float32, (None, head_dim // 2, 2))
    for name, t in (("seq_slot", seq_slot), ("seq_kvlen", seq_kvlen), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if seq_slot.numel() < n or seq_kvlen.numel() < n:
        raise KernelError("attention_decode_mma_rope: seq_slot / seq_kvlen shorter than the number of sequences")
    base = n_ml = 0
    cptr = None
    if n_runs > 1:
        need = decode_scratch_floats(n, n_q, head_dim, n_runs)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=qkv.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError(f"attention_decode_mma_rope: scratch holds {scratch.numel()} floats, {need} are needed")
        if counters is None or counters.numel() < n * n_kv * ((n_q // n_kv + 15) // 16):
            raise KernelError("attention_decode_mma_rope: counters are needed when a sequence spans several runs")
        _need(counters, "counters", torch.int32)
        base, n_ml, cptr = scratch.data_ptr(), n * n_q * n_runs, counters.data_ptr()
    _work(_nbytes(qkv, out) + 2.0 * STEP_HINT["kv_total"] * n_kv * head_dim * 2, 4.0 * n_q * head_dim * STEP_HINT["pairs"])
    f = _fn("attention_decode_mma", "llmie_attention_decode_mma_rope",
            [_c_void_p] * 5 + [_c_int] + [_c_void_p] * 7 + [_c_int] * 6 + [_c_float] + [_c_int] * 4 + [_c_void_p])
    _check(f(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[0],
             base or None, (base + 4 * n_ml) or None, (base + 8 * n_ml) or None, cptr, seq_slot.data_ptr(),
             seq_kvlen.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, n, n_q, n_kv, head_dim,
             float(scale), int(window), int(pages_per_run), int(n_runs), 1 if write_kv else 0, _stream()),
           "attention_decode_mma_rope")
    return out


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FMA on CUDA cores, fixed summation order)."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", torch.float32)
    _need(w, "w", torch.float32, (N, K))
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _need(out, "out", torch.float32, (M, N))
    _work(_nbytes(a, w) + a.shape[0] * w.shape[0] * 4, 2.0 * a.shape[0] * w.shape[0] * w.shape[1])
    f = _fn("gemm_simt", "llmie_gemm_f32_nt", [_c_void_p] * 3 + [_c_int] * 6 + [_c_void_p])
    _check(f(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, K, K, N, _stream()), "gemm_f32_nt")
    return out


SKINNY_STORE_BF16, SKINNY_STORE_F32, SKINNY_ADD_F32, SKINNY_SWIGLU = 0, 1, 2, 3
SKINNY_MAX_BATCH = 32          # what the kernel takes
SKINNY_BEST_BATCH = 8          # up to here it beats the library GEMM (measured on B200)
SKINNY_ADD_BEST_BATCH = 16     # the `h +=` form saves a pass over h as well: 3.7 / 9.6 us against 5.5 / 13.2 us for the
                               # library product of the output / down projection at 16 rows (1B shape); equal at 32


def gemm_skinny_add_wins(rows: int, n: int, k: int, device) -> bool:
    """Whether `h += x w^T` is better done by gemm_skinny than by the library product followed by the add in the
    next norm kernel. Up to 8 rows always. From 9 to 16 rows only for up to one block (16 weight rows) an SM, the
    1B shape's 2,048 outputs: there it takes 4.0 / 9.3 us (output / down projection, 16 rows) against the library's
    5.7 / 12.9 us. Wider outputs were measured inside whole steps (3B shape, 16 sequences of 1,400 tokens): library
    for both 2.254 ms a step, this kernel for the output projection 2.286 ms, for both 2.329 ms, although alone the
    kernel is level with the library there (3,072 x 3,072: 6.6 against 7.0 us)."""
    if rows <= SKINNY_BEST_BATCH:
        return True
    return rows <= SKINNY_ADD_BEST_BATCH and n // 16 <= _sms(device)


def gemm_skinny_ok(batch: int, n: int, k: int, epilogue: int = SKINNY_STORE_BF16) -> bool:
    """Whether gemm_skinny takes this shape (else the caller uses a tiled GEMM)."""
    if not 0 < batch <= SKINNY_MAX_BATCH or k % 32:
        return False
    return (n % 2 == 0 and (n // 2) % 8 == 0) if epilogue == SKINNY_SWIGLU else n % 16 == 0


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> torch.Tensor:
    """y = x w^T for a few rows of x and a large bfloat16 w [N, K] that is read once.

    epilogue SKINNY_STORE_BF16 / SKINNY_STORE_F32: out [batch, N] = y;  SKINNY_ADD_F32: out (float32) += y;
    SKINNY_SWIGLU: w = [gate rows; up rows], out bfloat16 [batch, N / 2] = silu(gate) * up."""
    batch, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16, (N, K))
    if not gemm_skinny_ok(batch, N, K, epilogue):
        raise KernelError(f"gemm_skinny: shape batch={batch}, N={N}, K={K} is not supported")
    cols = N // 2 if epilogue == SKINNY_SWIGLU else N
    want = torch.float32 if epilogue in (SKINNY_STORE_F32, SKINNY_ADD_F32) else torch.bfloat16
    _need(out, "out", want, (batch, cols))
    _work(_nbytes(x, w, out), 2.0 * x.shape[0] * w.shape[0] * w.shape[1])
    f = _fn("gemm_skinny", "llmie_gemm_skinny", [_c_void_p] * 3 + [_c_int] * 5 + [_c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), out.data_ptr(), batch, N, K, cols, epilogue, _stream()), "gemm_skinny")
    return out


def gemm_skinny_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act: int) -> torch.Tensor:
    """out (bfloat16 [batch, N / 2]) = act(x Wg^T) * (x Wu^T) for w = [gate rows; up rows] in one kernel, for a few
    rows of x; act an ACT_* code."""
    batch, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16, (N, K))
    if act == ACT_NONE or not gemm_skinny_ok(batch, N, K, SKINNY_SWIGLU):
        raise KernelError(f"gemm_skinny_gated: shape batch={batch}, N={N}, K={K} or activation {act} is not supported")
    _need(out, "out", torch.bfloat16, (batch, N // 2))
    _work(_nbytes(x, w, out), 2.0 * batch * N * K)
    f = _fn("gemm_skinny", "llmie_gemm_skinny_gated", [_c_void_p] * 3 + [_c_int] * 5 + [_c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), out.data_ptr(), batch, N, K, N // 2, int(act), _stream()), "gemm_skinny_gated")
    return out


def gemm_skinny_bias_act(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                         act: int) -> torch.Tensor:
    """out (bfloat16 [batch, N]) = act(x w^T + bias) in one kernel, for a few rows of x; bias float32 [N] or None."""
    batch, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16, (N, K))
    _need(out, "out", torch.bfloat16, (batch, N))
    if bias is not None:
        _need(bias, "bias", torch.float32, (N,))
    if not gemm_skinny_ok(batch, N, K):
        raise KernelError(f"gemm_skinny_bias_act: shape batch={batch}, N={N}, K={K} is not supported")
    _work(_nbytes(x, w, out), 2.0 * batch * N * K)
    f = _fn("gemm_skinny", "llmie_gemm_skinny_bias_act", [_c_void_p] * 3 + [_c_int] * 4 + [_c_void_p, _c_int, _c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), out.data_ptr(), batch, N, K, N, _ptr(bias), int(act), _stream()),
           "gemm_skinny_bias_act")
    return out


def norm_gemm_supported(batch: int, k: int) -> bool:
    """Whether the fused norm + product kernels of one-token steps take this many rows and this width."""
    return 1 <= batch <= 8 and k % 32 == 0 and 8 * (k + 32) * 2 + 12 * 1024 <= 200 * 1024


def _norm_gemm_common(h, norm_w, w, what):
    batch, K = h.shape
    _need(h, "h", torch.float32)
    _need(norm_w, "norm_w", torch.float32, (K,))
    _need(w, "w", torch.bfloat16, (None, K))
    if not norm_gemm_supported(batch, K):
        raise KernelError(f"{what}: {batch} rows of width {K} are not supported")
    return batch, K


def norm_gate_swiglu(h, norm_w, eps: float, w_gate_up, act):
    """act[b, j] = silu(x Wg^T) * (x Wu^T) with x = rmsnorm(h) * norm_w, in one kernel.
    h float32 [batch <= 8, K]; w_gate_up bfloat16 [2 ff, K] = [gate rows; up rows]; act bfloat16 [batch, ff]."""
    batch, K = _norm_gemm_common(h, norm_w, w_gate_up, "norm_gate_swiglu")
    ff = w_gate_up.shape[0] // 2
    _need(act, "act", torch.bfloat16, (batch, ff))
    if w_gate_up.shape[0] % 2 or ff % 8:
        raise KernelError("norm_gate_swiglu: the feed-forward width must be a multiple of 8")
    _work(_nbytes(h, w_gate_up, act), 2.0 * batch * w_gate_up.shape[0] * K)
    f = _fn("gemm_fused_decode", "llmie_norm_gate_swiglu",
            [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(h.data_ptr(), norm_w.data_ptr(), float(eps), w_gate_up.data_ptr(), act.data_ptr(), batch, ff, K,
             _stream()), "norm_gate_swiglu")
    return act


# Up to how many rows folding the branch-closing add into the next product pays. Measured on a B200, captured steps,
# 4 layers: 1B layer sizes, 1 row 0.206 -> 0.201 ms a step, 8 rows 0.214 -> 0.242 ms; 8B sizes 0.461 -> 0.452 and
# 0.490 -> 0.522. Every block of the product derives its input rows from the float32 stream and branch output (three
# reads of 4 bytes an element where the unfused product reads 2), which two saved launches repay only for a row or two.
BRANCH_FOLD_BEST_ROWS = 2


def branch_norm_gemm(h, y, y_bias, norm_w, eps: float, h_out, w, out, out_bias=None, act: Optional[int] = None):
    """The add that closes a branch, folded into the product that opens the next one (one-token steps of layers
    whose norm sits on the branch's output): h_out = h + rmsnorm(y + y_bias) * norm_w in float32 (h_out must not be
    h), and out (bfloat16 [batch, N]) = h_out w^T, or act(h_out w^T + out_bias) when `act` is an ACT_* code.
    h, y, h_out float32 [batch <= 8, K]; y_bias float32 [K] or None; out_bias float32 [N] or None."""
    batch, K = _norm_gemm_common(h, norm_w, w, "branch_norm_gemm")
    N = w.shape[0]
    _need(y, "y", torch.float32, (batch, K))
    _need(h_out, "h_out", torch.float32, (batch, K))
    _need(out, "out", torch.bfloat16, (batch, N))
    if h_out.data_ptr() == h.data_ptr():
        raise KernelError("branch_norm_gemm: h_out must be another buffer than h")
    if y_bias is not None:
        _need(y_bias, "y_bias", torch.float32, (K,))
    if out_bias is not None:
        _need(out_bias, "out_bias", torch.float32, (N,))
    if N % 16:
        raise KernelError("branch_norm_gemm: N must be a multiple of 16")
    _work(_nbytes(h, y, h_out, w, out), 2.0 * batch * N * K)
    f = _fn("gemm_fused_decode", "llmie_branch_norm_gemm",
            [_c_void_p] * 4 + [_c_float] + [_c_void_p] * 4 + [_c_int] * 5 + [_c_void_p])
    _check(f(h.data_ptr(), y.data_ptr(), _ptr(y_bias), norm_w.data_ptr(), float(eps), h_out.data_ptr(), w.data_ptr(),
             out.data_ptr(), _ptr(out_bias), int(act or 0), 0 if act is None else 1, batch, N, K, _stream()),
           "branch_norm_gemm")
    return out


def norm_gemm_f32(h, norm_w, eps: float, w, out):
    """out[batch, N] float32 = (rmsnorm(h) * norm_w) w^T in one kernel (final norm + LM head)."""
    batch, K = _norm_gemm_common(h, norm_w, w, "norm_gemm_f32")
    N = w.shape[0]
    _need(out, "out", torch.float32, (batch, N))
    if N % 16:
        raise KernelError("norm_gemm_f32: N must be a multiple of 16")
    _work(_nbytes(h, w, out), 2.0 * batch * w.shape[0] * K)
    f = _fn("gemm_fused_decode", "llmie_norm_gemm_f32",
            [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(h.data_ptr(), norm_w.data_ptr(), float(eps), w.data_ptr(), out.data_ptr(), batch, N, K, _stream()),
           "norm_gemm_f32")
    return out


def norm_qkv_rope(h, norm_w, eps: float, w_qkv, q_out, k_cache, v_cache, table, tok_pos, tok_seq, seq_slot,
                  block_table, page_size: int, n_q: int, n_kv: int, head_dim: int, write_kv: bool = True):
    """RMSNorm, the packed q/k/v product, rotation of q and k and the KV-cache write in one kernel.
    h float32 [batch <= 8, K]; w_qkv bfloat16 [(n_q + 2 n_kv) hd, K]; q_out bfloat16 [batch, n_q hd];
    table float32 [max_pos, hd / 2, 2] (the whole head is rotated)."""
    batch, K = _norm_gemm_common(h, norm_w, w_qkv, "norm_qkv_rope")
    if w_qkv.shape[0] != (n_q + 2 * n_kv) * head_dim or head_dim % 16:
        raise KernelError("norm_qkv_rope: weight rows do not match the head layout")
    _need(q_out, "q_out", torch.bfloat16, (batch, n_q * head_dim))
    _need(table, "table", torch.float32, (None, head_dim // 2, 2))
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if write_kv:
        _need(k_cache, "k_cache", torch.bfloat16, (None, n_kv, page_size, head_dim))
        _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _work(_nbytes(h, w_qkv, q_out) + 2 * batch * n_kv * head_dim * 2, 2.0 * batch * w_qkv.shape[0] * K)
    f = _fn("gemm_fused_decode", "llmie_norm_qkv_rope",
            [_c_void_p, _c_void_p, _c_float] + [_c_void_p] * 9 + [_c_int] * 9 + [_c_void_p])
    _check(f(h.data_ptr(), norm_w.data_ptr(), float(eps), w_qkv.data_ptr(), q_out.data_ptr(),
             _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None, table.data_ptr(),
             tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), block_table.data_ptr(),
             block_table.shape[1], page_size, batch, n_q, n_kv, head_dim, K, table.shape[0], 1 if write_kv else 0,
             _stream()), "norm_qkv_rope")
    return q_out


_tc_status = {}
_TC_STATUS_TEXT = {1: "a TMA load did not arrive", 2: "the tensor cores did not release a stage",
                   3: "the accumulators were not completed"}


def tc_status_word(device) -> torch.Tensor:
    """One int32 per device that the tensor-core kernels set when a bounded wait gives up."""
    key = torch.device(device).index or 0
    t = _tc_status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _tc_status[key] = t
    return t


def check_tc_status(device) -> None:
    """Reads the status word (this synchronises) and raises if a tensor-core kernel gave up a wait."""
    t = tc_status_word(device)
    code = int(t.item())
    if code:
        t.zero_()
        raise KernelError(f"a tensor-core kernel timed out: {_TC_STATUS_TEXT.get(code, code)}")


def tc_wait_probe(device, limit: int = 1000) -> None:
    """Launches one block that waits, for at most `limit` polls, on a barrier at which nothing arrives, gives
    up, records the status of a load that did not arrive, frees its tensor memory and returns. The next
    `check_tc_status` then raises. For tests of the give-up path; it never hangs."""
    f = _fn("gemm_tc", "llmie_tc_wait_probe", [_c_void_p, _c_int, _c_void_p])
    with torch.cuda.device(device):
        _check(f(tc_status_word(device).data_ptr(), int(limit), _stream()), "tc_wait_probe")


def attention_prefill_tc_supported(head_dim: int, page_size: int, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size == 64


def attention_prefill_tc(q, k_cache, v_cache, out, cu_q, seq_slot, seq_start, block_table, page_size: int,
                         n_seqs: int, max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float,
                         window: int = 0, keep_first: int = 0, sink: bool = False,
                         gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                         dist_bias: Optional[torch.Tensor] = None, sink_values: Optional[torch.Tensor] = None,
                         sigmoid_bias: Optional[torch.Tensor] = None):
    """Causal attention for runs of new tokens on the tcgen05 tensor cores, K and V read from the
    paged cache by TMA. q, out bfloat16 [T, n_q hd] with sequences packed (cu_q int32 [n + 1]);
    seq_start int32 [n]: tokens each sequence held before this step. The caches' last page must be
    a scratch page. head_dim 64 or 128, pages of 64. keep_first, sink and gate as in attention_paged (the gate's
    rows must start on 16 bytes). With sigmoid_bias (float32 [n_q]) there is no softmax: the weight of a visible key is
    sigmoid(scaled score + sigmoid_bias[head]), not normalised (no sink, cap or bias by distance with it)."""
    T = q.shape[0]
    gate_ld = _row_slice(gate, "gate", torch.bfloat16, T, n_q * head_dim) if gate is not None else 0
    if gate is not None and (gate_ld % 8 or gate.data_ptr() % 16):
        raise KernelError("attention_prefill_tc: the gate's rows must start on 16-byte boundaries")
    _need(q, "q", torch.bfloat16, (T, n_q * head_dim))
    _need(out, "out", torch.bfloat16, (T, n_q * head_dim))
    _need(k_cache, "k_cache", torch.bfloat16, (None, n_kv, page_size, head_dim))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    for name, t in (("cu_q", cu_q), ("seq_slot", seq_slot), ("seq_start", seq_start), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if not attention_prefill_tc_supported(head_dim, page_size, q.dtype):
        raise KernelError(f"attention_prefill_tc: head_dim {head_dim} / page size {page_size} is not supported")
    if cu_q.numel() < n_seqs + 1 or seq_slot.numel() < n_seqs or seq_start.numel() < n_seqs:
        raise KernelError("attention_prefill_tc: a per-sequence array is shorter than n_seqs")
    if not scale > 0:
        raise KernelError(f"attention_prefill_tc: the scale must be positive, got {scale}")
    _work(2 * _nbytes(q) + 2.0 * STEP_HINT["kv_total"] * n_kv * head_dim * 2, 4.0 * n_q * head_dim * STEP_HINT["pairs"])
    if sigmoid_bias is not None:
        if softcap or dist_bias is not None or sink_values is not None or sink:
            raise KernelError("attention_prefill_tc: sigmoid weights take no sink, cap or bias by distance")
        _need(sigmoid_bias, "sigmoid_bias", torch.float32, (n_q,))
        f = _fn("attention_prefill_tc", "llmie_attention_prefill_tc_sigmoid",
                [_c_void_p] * 8 + [_c_int] * 8 + [_c_float, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                                  _c_void_p])
        _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), cu_q.data_ptr(),
                 seq_slot.data_ptr(), seq_start.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                 k_cache.shape[0], T, n_seqs, max_q_len, n_q, n_kv, head_dim, float(scale), int(window),
                 int(keep_first), _ptr(gate), gate_ld, tc_status_word(q.device).data_ptr(), sigmoid_bias.data_ptr(),
                 _stream()), "attention_prefill_tc_sigmoid")
        return out
    if softcap or dist_bias is not None or sink_values is not None:
        # the options that change single scores: a cap, a bias by distance [n_q, L], the sink's score per head
        bias_len = 0
        if dist_bias is not None:
            _need(dist_bias, "dist_bias", torch.float32, (n_q, None))
            bias_len = dist_bias.shape[1]
        if sink_values is not None:
            _need(sink_values, "sink_values", torch.float32, (n_q,))
            sink = True
        f = _fn("attention_prefill_tc", "llmie_attention_prefill_tc_scored",
                [_c_void_p] * 8 + [_c_int] * 8 + [_c_float, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_float,
                                                  _c_void_p, _c_int, _c_void_p, _c_void_p])
        _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), cu_q.data_ptr(),
                 seq_slot.data_ptr(), seq_start.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                 k_cache.shape[0], T, n_seqs, max_q_len, n_q, n_kv, head_dim, float(scale), int(window),
                 int(keep_first), 1 if sink else 0, _ptr(gate), gate_ld, tc_status_word(q.device).data_ptr(),
                 float(softcap or 0.0), _ptr(dist_bias), bias_len, _ptr(sink_values), _stream()),
               "attention_prefill_tc_scored")
        return out
    f = _fn("attention_prefill_tc", "llmie_attention_prefill_tc",
            [_c_void_p] * 8 + [_c_int] * 8 + [_c_float, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p])
    _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), cu_q.data_ptr(),
             seq_slot.data_ptr(), seq_start.data_ptr(), block_table.data_ptr(), block_table.shape[1],
             k_cache.shape[0], T, n_seqs, max_q_len, n_q, n_kv, head_dim, float(scale), int(window), int(keep_first),
             1 if sink else 0, _ptr(gate), gate_ld, tc_status_word(q.device).data_ptr(), _stream()),
           "attention_prefill_tc")
    return out


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores; a, w bfloat16, out bfloat16 or float32."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16, (N, K))
    _need(out, "out", None, (M, N))
    if K % 8 or N % 8:
        raise KernelError(f"gemm_tc: K ({K}) and N ({N}) must be multiples of 8")
    _work(_nbytes(a, w, out), 2.0 * M * N * K)
    f = _fn("gemm_tc", "llmie_gemm_tc", [_c_void_p] * 3 + [_c_int] * 5 + [_c_void_p, _c_void_p])
    _check(f(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, N, _dt(out, "out"),
             tc_status_word(a.device).data_ptr(), _stream()), "gemm_tc")
    return out


_argmax_parts = {}


STREAM_STORE_BF16, STREAM_STORE_F32, STREAM_ADD_F32 = 0, 1, 2
STREAM_MAX_ROWS = 64
_sm_count = {}


def _sms(device) -> int:
    key = torch.device(device).index or 0
    n = _sm_count.get(key)
    if n is None:
        n = torch.cuda.get_device_properties(key).multi_processor_count
        _sm_count[key] = n
    return n


def gemm_stream_ok(rows: int, n: int, k: int) -> bool:
    """Whether gemm_stream takes this shape: up to 64 rows, K a multiple of 8."""
    return 0 < rows <= STREAM_MAX_ROWS and k % 8 == 0 and n > 0


def gemm_stream_wins(rows: int, n: int, k: int) -> bool:
    """Where gemm_stream beat the library GEMM when measured on a B200 (captured launches, weights rotated through
    more than the L2 holds): only very tall matrices at 33 to 64 rows (a 128,256 x 2,048 head: 84 us against
    92 us). From 9 to 32 rows and for the layer matrices (2,048 to 28,672 rows of weights) the library is equal
    or faster (qkv 6 us against 9-12 us, down 13 us against 13-18 us), so those stay with it."""
    return 32 < rows <= STREAM_MAX_ROWS and k % 8 == 0 and n * k >= 128 * 1024 * 1024


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = STREAM_STORE_BF16,
                splits: int = 0) -> torch.Tensor:
    """out = x @ w^T (mode STREAM_STORE_BF16 / STREAM_STORE_F32) or out += x @ w^T (STREAM_ADD_F32, out float32)
    for up to 64 rows of x, on the tcgen05 tensor cores with the weights as the streamed operand. x [M, K] and
    w [N, K] bfloat16. Needs no workspace: slices of K meet in the shared memory of a thread-block cluster.
    splits: 0 = the launcher chooses into how many slices K is cut; 1, 2, 4 or 8 fixes it."""
    M, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16, (N, K))
    _need(out, "out", torch.bfloat16 if mode == STREAM_STORE_BF16 else torch.float32, (M, N))
    if not gemm_stream_ok(M, N, K):
        raise KernelError(f"gemm_stream: {M} rows x K {K} is not supported (up to {STREAM_MAX_ROWS} rows, K % 8 == 0)")
    _work(_nbytes(x, w, out) + (_nbytes(out) if mode == STREAM_ADD_F32 else 0), 2.0 * M * N * K)
    f = _fn("gemm_stream", "llmie_gemm_stream", [_c_void_p] * 3 + [_c_int] * 6 + [_c_void_p, _c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, int(mode), _sms(x.device), int(splits),
             tc_status_word(x.device).data_ptr(), _stream()), "gemm_stream")
    return out


def _check_query(status: int, name: str) -> None:
    if status != 0:
        raise KernelError(f"{name}: {_ERRORS.get(status, 'error ' + str(status))}")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Greedy token per row of float32 logits [R, V] (lowest index wins a tie), many blocks per row."""
    R, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out, "out", torch.int32)
    if out.shape[0] < R:
        raise KernelError("argmax: out is shorter than the number of rows")
    slices = max(1, min(128, V // 1024, max(8, 1184 // R)))     # about a thousand blocks, each with a few thousand logits
    key = (logits.device, R * slices)
    parts = _argmax_parts.get(key)
    if parts is None:        # kept: a generation loop calls this once per step (calls on one stream are ordered)
        parts = (torch.empty(R * slices, dtype=torch.float32, device=logits.device),
                 torch.empty(R * slices, dtype=torch.int32, device=logits.device))
        _argmax_parts[key] = parts
    part_val, part_idx = parts
    _work(R * V * 4)
    f = _fn("sampling", "llmie_argmax", [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                         _c_void_p])
    _check(f(logits.data_ptr(), R, V, logits.stride(0), slices, part_val.data_ptr(), part_idx.data_ptr(),
             out.data_ptr(), _stream()), "argmax")
    return out


def sampling_words(temperature: float, top_p: float, seed: int) -> list:
    """The four 32-bit words (as Python ints) that `sample(..., params=)` reads from device memory."""
    import struct
    t, p = struct.unpack("<2I", struct.pack("<2f", float(temperature), float(top_p)))
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    as_i32 = lambda w: w - (1 << 32) if w >= (1 << 31) else w
    return [as_i32(t), as_i32(p), as_i32(seed & 0xFFFFFFFF), as_i32(seed >> 32)]


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float = 0.0, top_p: float = 1.0, seed: int = 0,
           seq_ids: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None,
           params: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V]: argmax when temperature <= 0 (lowest index wins a
    tie), else a draw from softmax(logits / T) cut by top_p, with the uniform number of
    (seed, seq_ids[r], counters[r]); counters[r] is then incremented. out int32 [R].
    With `params` (int32 [4] on the device, filled from `sampling_words`) temperature, top_p and seed
    are read from there when the kernel runs, so a captured launch serves any setting."""
    R, V = logits.shape
    if params is not None:
        _need(params, "params", torch.int32, (4,))
        if seq_ids is None or counters is None:
            raise KernelError("sample: seq_ids and counters are required with params")
    elif temperature <= 0 and V >= 4096 and logits.is_contiguous():
        return argmax(logits, out)
    _need(logits, "logits", torch.float32)
    _need(out, "out", torch.int32)
    if out.shape[0] < R:
        raise KernelError("sample: out is shorter than the number of rows")
    if temperature > 0 or params is not None:
        if seq_ids is None or counters is None:
            raise KernelError("sample: seq_ids and counters are required when temperature > 0")
        _need(seq_ids, "seq_ids", torch.int32)
        _need(counters, "counters", torch.int32)
        if seq_ids.shape[0] < R or counters.shape[0] < R:
            raise KernelError("sample: seq_ids / counters shorter than the number of rows")
    _work(R * V * 4)
    f = _fn("sampling", "llmie_sample",
            [_c_void_p, _c_int, _c_int, _c_int, _c_float, _c_float, ctypes.c_ulonglong, _c_void_p, _c_void_p,
             _c_void_p, _c_void_p, _c_void_p])
    _check(f(logits.data_ptr(), R, V, logits.stride(0), float(temperature), float(top_p),
             int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(params), _ptr(seq_ids), _ptr(counters), out.data_ptr(), _stream()),
           "sample")
    return out


def copy_int(src: torch.Tensor, dst: torch.Tensor, n: int) -> None:
    _need(src, "src", torch.int32)
    _need(dst, "dst", torch.int32)
    if src.numel() < n or dst.numel() < n:
        raise KernelError("copy_int: n exceeds a buffer")
    f = _fn("sampling", "llmie_copy_int", [_c_void_p, _c_void_p, _c_int, _c_void_p])
    _check(f(src.data_ptr(), dst.data_ptr(), n, _stream()), "copy_int")


def prepare_decode(slots, seq_lens, tok_pos, tok_seq, cu_q, seq_start, seq_kvlen, n: int) -> None:
    """Per-lane metadata of a one-token step from the device-resident lengths."""
    for name, t in (("slots", slots), ("seq_lens", seq_lens), ("tok_pos", tok_pos), ("tok_seq", tok_seq),
                    ("cu_q", cu_q), ("seq_start", seq_start), ("seq_kvlen", seq_kvlen)):
        _need(t, name, torch.int32)
    if min(slots.numel(), tok_pos.numel(), tok_seq.numel(), seq_start.numel(), seq_kvlen.numel()) < n \
            or cu_q.numel() < n + 1:
        raise KernelError("prepare_decode: a buffer is shorter than n")
    f = _fn("elementwise", "llmie_prepare_decode", [_c_void_p] * 7 + [_c_int, _c_void_p])
    _check(f(slots.data_ptr(), seq_lens.data_ptr(), tok_pos.data_ptr(), tok_seq.data_ptr(), cu_q.data_ptr(),
             seq_start.data_ptr(), seq_kvlen.data_ptr(), n, _stream()), "prepare_decode")


def advance_lengths(slots, seq_kvlen, seq_lens, n: int, scratch_slot: int) -> None:
    """seq_lens[slots[i]] = seq_kvlen[i] for the n lanes of a step, except the scratch slot."""
    for name, t in (("slots", slots), ("seq_kvlen", seq_kvlen), ("seq_lens", seq_lens)):
        _need(t, name, torch.int32)
    f = _fn("elementwise", "llmie_advance_lengths", [_c_void_p] * 3 + [_c_int, _c_int, _c_void_p])
    _check(f(slots.data_ptr(), seq_kvlen.data_ptr(), seq_lens.data_ptr(), n, scratch_slot, _stream()),
           "advance_lengths")


# ------------------------------------------------------------------------------------------ parallel blocks
def add_dyt(h, d1, d2, alpha, weight, bias, out, rows=None):
    """h (float32 [T, d]) += d1 + d2 in place when rows is None (either may be None; float32 or bfloat16), then
    out = tanh(alpha * h) * weight + bias (Dynamic Tanh: a norm that reduces nothing). alpha float32 [1] on the
    device; weight, bias float32 [d]; out [n_out, d]. With `rows` (int32 [n_out]) only those rows of h + d1 + d2
    are produced and h is left as it is."""
    T, d = h.shape
    n_out = T if rows is None else rows.shape[0]
    _need(h, "h", torch.float32)
    _need(alpha, "alpha", torch.float32, (1,))
    _need(weight, "weight", torch.float32, (d,))
    _need(bias, "bias", torch.float32, (d,))
    _need(out, "out", None, (n_out, d))
    for name, t in (("d1", d1), ("d2", d2)):
        if t is not None:
            _need(t, name, None, (T, d))
    if rows is not None:
        _need(rows, "rows", torch.int32, (n_out,))
    _work((2 * _nbytes(h) if rows is None else n_out * d * 4) + _nbytes(d1, d2, out))
    f = _fn("parallel_elementwise", "llmie_add_dyt",
            [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
             _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(h.data_ptr(), _ptr(d1), _dt(d1, "d1") if d1 is not None else 0, _ptr(d2),
             _dt(d2, "d2") if d2 is not None else 0, alpha.data_ptr(), weight.data_ptr(), bias.data_ptr(),
             out.data_ptr(), _dt(out, "out"), _ptr(rows), n_out, d, _stream()), "add_dyt")
    return out


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, act: int) -> torch.Tensor:
    """out[t, j] = act(gate_up[t, j]) * gate_up[t, ff + j]; gate_up [T, 2 ff], out [T, ff]; act an ACT_* code."""
    T, ff = out.shape
    _need(out, "out")
    _need(gate_up, "gate_up", out.dtype, (T, 2 * ff))
    _work(_nbytes(gate_up, out))
    f = _fn("parallel_elementwise", "llmie_gated_act", [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(gate_up.data_ptr(), out.data_ptr(), T, ff, int(act), _dt(out, "out"), _stream()), "gated_act")
    return out


def scale_rows(x: torch.Tensor, scale: float) -> torch.Tensor:
    """x (float32) *= scale in place."""
    _need(x, "x", torch.float32)
    _work(2 * _nbytes(x))
    f = _fn("parallel_elementwise", "llmie_scale_rows", [_c_void_p, _c_float, ctypes.c_longlong, _c_void_p])
    _check(f(x.data_ptr(), float(scale), x.numel(), _stream()), "scale_rows")
    return x


def cap_rows(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap) in place; x float32, cap > 0."""
    _need(x, "x", torch.float32)
    if not cap > 0:
        raise KernelError(f"cap_rows: the cap must be positive, got {cap}")
    _work(2 * _nbytes(x))
    f = _fn("parallel_elementwise", "llmie_cap_rows", [_c_void_p, _c_float, ctypes.c_longlong, _c_void_p])
    _check(f(x.data_ptr(), float(cap), x.numel(), _stream()), "cap_rows")
    return x


# ------------------------------------------------------------------------------------------ grouped products
_c_ll = ctypes.c_longlong
_GROUPED_ARGS = [_c_void_p, _c_ll, _c_ll, _c_void_p, _c_void_p, _c_ll, _c_ll, _c_void_p, _c_ll, _c_ll, _c_void_p,
                 _c_void_p] + [_c_int] * 10 + [_c_void_p]
GROUPED_SMALL_ROWS = 64        # up to this many rows the tiles of 16 rows are used


def grouped_tile_rows(small: bool) -> int:
    """Rows per tile of the grouped product's two forms (the sort of a routed call uses the same number)."""
    return 16 if small else 64


def _cols(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-d tensor whose rows are contiguous runs (possibly a column range of a wider tensor)."""
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: must be a 2-d CUDA tensor with contiguous rows")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def batched_gemm_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, a_group_cols: int, out_group_cols: int,
                    k: int) -> torch.Tensor:
    """For every group g < G: out[:, g * out_group_cols : + N] = a[:, g * a_group_cols : + k] @ w[g]^T.
    a [T, >= (G-1) a_group_cols + k] and out [T, >= (G-1) out_group_cols + N] may be column ranges of wider tensors;
    w [G, N, k] contiguous, of a's dtype (float32, or bfloat16 with bfloat16 or float32 out). float32 accumulation in
    the order of k."""
    G, N, K = w.shape
    T = a.shape[0]
    if K != k or a.shape[1] < (G - 1) * a_group_cols + k or out.shape[1] < (G - 1) * out_group_cols + N \
            or out.shape[0] != T:
        raise KernelError(f"batched_gemm_nt: shapes a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} "
                          f"do not fit (group columns {a_group_cols} / {out_group_cols})")
    _need(w, "w", a.dtype)
    lda, ldc = _cols(a, "a"), _cols(out, "out")
    _work(_nbytes(w) + T * G * (K * a.element_size() + N * out.element_size()), 2.0 * T * G * N * K)
    f = _fn("grouped_gemm", "llmie_grouped_gemm_nt", _GROUPED_ARGS)
    _check(f(a.data_ptr(), lda, a_group_cols, None, w.data_ptr(), N * K, K, out.data_ptr(), ldc, out_group_cols, None,
             None, 0, G, T, N, K, 0, 0, 1 if T <= GROUPED_SMALL_ROWS else 0, _dt(a, "a"), _dt(out, "out"), _stream()),
           "batched_gemm_nt")
    return out


def routed_gemm_nt(a, a_rows, w, out, out_rows, tile_group, n_positions: int, small: bool, dual: bool = False,
                   act: int = ACT_NONE):
    """The routed form: sorted position p (of n_positions, in tiles of grouped_tile_rows(small)) reads row a_rows[p]
    of a (p itself when a_rows is None), multiplies by w[tile_group[p // tile]]^T and writes row out_rows[p] of out
    (p itself when None); -1 anywhere = nothing there. w [E, N or 2 N, K]; dual: w holds [gate | up] rows and the
    result is act(gate) * up."""
    E, rows_w, K = w.shape
    N = rows_w // 2 if dual else rows_w
    _need(w, "w", a.dtype)
    _need(tile_group, "tile_group", torch.int32)
    lda, ldc = _cols(a, "a"), _cols(out, "out")
    if a.shape[1] != K or out.shape[1] != N:
        raise KernelError(f"routed_gemm_nt: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    tile = grouped_tile_rows(small)
    n_tiles = tile_group.shape[0]
    if n_positions > n_tiles * tile:
        raise KernelError("routed_gemm_nt: more positions than the tiles hold")
    for name, t in (("a_rows", a_rows), ("out_rows", out_rows)):
        if t is not None:
            _need(t, name, torch.int32)
            if t.shape[0] < n_positions:
                raise KernelError(f"routed_gemm_nt: {name} shorter than the positions")
    # what is read of the weights is not known on the host: the count assumes the tiles' groups all differ, up to E
    touched = min(E, n_tiles) / E
    _work(touched * _nbytes(w) + n_positions * (K * a.element_size() + N * out.element_size()),
          2.0 * n_positions * rows_w * K)
    f = _fn("grouped_gemm", "llmie_grouped_gemm_nt", _GROUPED_ARGS)
    _check(f(a.data_ptr(), lda, 0, _ptr(a_rows), w.data_ptr(), rows_w * K, K, out.data_ptr(), ldc, 0, _ptr(out_rows),
             tile_group.data_ptr(), n_tiles, E, n_positions, N, K, 1 if dual else 0, int(act), 1 if small else 0,
             _dt(a, "a"), _dt(out, "out"), _stream()), "routed_gemm_nt")
    return out


# ------------------------------------------------------------------------------------------ routed feed-forward
ROUTE_SOFTMAX_TOP, ROUTE_SOFTMAX_ALL, ROUTE_SIGMOID = 0, 1, 2


def moe_route(x, w, bias, ids, weights, scores_over_all=False, correction=None, out_scale: float = 1.0):
    """Router of a mixture of experts: logits = x @ w^T + bias in float32; ids int32 [T, top] receive the `top`
    largest (ties: the lower index), weights float32 [T, top] the softmax over those logits alone.
    x [T, d] float32 or bfloat16; w float32 [E, d]; bias float32 [E] or None.
    `scores_over_all`: the scores are the softmax over ALL logits, the choice goes by score + correction (float32 [E]
    or None) and the weights are the chosen scores / (their sum + 1e-20) * out_scale. `scores_over_all` may also be one
    of the ROUTE_* codes; ROUTE_SIGMOID: the `top` largest logits choose and the weights are sigmoid(logit) * out_scale of
    the chosen ones, not normalised."""
    T, d = x.shape
    E = w.shape[0]
    top = ids.shape[1]
    _need(x, "x")
    _need(w, "w", torch.float32, (E, d))
    if bias is not None:
        _need(bias, "bias", torch.float32, (E,))
    _need(ids, "ids", torch.int32, (T, top))
    _need(weights, "weights", torch.float32, (T, top))
    if correction is not None:
        _need(correction, "correction", torch.float32, (E,))
    _work(_nbytes(x, w, ids, weights), 2.0 * T * E * d)
    f = _fn("moe", "llmie_moe_route_ex", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p] + [_c_int] * 5 +
            [_c_void_p, _c_float, _c_void_p])
    _check(f(x.data_ptr(), _dt(x, "x"), w.data_ptr(), _ptr(bias), ids.data_ptr(), weights.data_ptr(), T, d, E, top,
             int(scores_over_all), _ptr(correction), float(out_scale), _stream()), "moe_route")


def moe_max_tiles(n_pairs: int, n_experts: int, tile: int) -> int:
    """Tiles that the sorted pairs can need at most: every expert may end with a tile that is partly padding."""
    return n_pairs // tile + min(n_pairs, n_experts)


def moe_sort(ids, n_experts: int, tile: int, sorted_token, sorted_pair, tile_group, group_end=None, pair_pos=None):
    """Groups the (token, choice) pairs of ids int32 [T, top] by expert into tiles of `tile` positions: sorted_pair[p]
    = token * top + choice at position p, sorted_token[p] = token, -1 = padding; tile_group[i] = expert of tile i, -1 =
    unused. The arrays are sized for moe_max_tiles. Optional: group_end int32 [E] receives where each expert's
    positions end (padding included), pair_pos int32 [T * top] the position of every pair."""
    T, top = ids.shape
    n_tiles = tile_group.shape[0]
    _need(ids, "ids", torch.int32)
    _need(tile_group, "tile_group", torch.int32, (n_tiles,))
    _need(sorted_token, "sorted_token", torch.int32, (n_tiles * tile,))
    _need(sorted_pair, "sorted_pair", torch.int32, (n_tiles * tile,))
    if group_end is not None:
        _need(group_end, "group_end", torch.int32, (n_experts,))
    if pair_pos is not None:
        _need(pair_pos, "pair_pos", torch.int32, (T * top,))
    f = _fn("moe", "llmie_moe_sort", [_c_void_p] + [_c_int] * 5 + [_c_void_p] * 6)
    _check(f(ids.data_ptr(), T * top, top, n_experts, tile, n_tiles, sorted_token.data_ptr(), sorted_pair.data_ptr(),
             tile_group.data_ptr(), _ptr(group_end), _ptr(pair_pos), _stream()), "moe_sort")


def moe_combine(y, weights, shared_out, out, pair_pos=None):
    """out[t] = sum_k weights[t, k] * y[row of pair t * top + k] (+ shared_out[t]); the row of a pair is the pair's
    own number, or pair_pos[pair] when that is given (y then holds the pairs in sorted order). y float32 or bfloat16
    [rows, d]; out float32 [T, d]. `weights` may be the number of choices a token (an int) instead of a tensor: every
    weight is then one (designs whose weight has already multiplied what the expert read)."""
    d = out.shape[1]
    if isinstance(weights, int):
        T, top, weights = out.shape[0], weights, None
    else:
        T, top = weights.shape
        _need(weights, "weights", torch.float32)
    _need(y, "y", None, (None if pair_pos is not None else T * top, d))
    _need(out, "out", torch.float32, (T, d))
    if shared_out is not None:
        _need(shared_out, "shared_out", None, (T, d))
    if pair_pos is not None:
        _need(pair_pos, "pair_pos", torch.int32, (T * top,))
    _work(T * top * d * y.element_size() + _nbytes(weights, shared_out, out))
    f = _fn("moe", "llmie_moe_combine", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                         _c_int, _c_int, _c_void_p])
    _check(f(y.data_ptr(), _dt(y, "y"), _ptr(pair_pos), _ptr(weights), _ptr(shared_out),
             _dt(shared_out, "shared_out") if shared_out is not None else 0, out.data_ptr(), T, d, top, _stream()),
           "moe_combine")
    return out


def moe_combine_identity(y, weights, ids, n_real: int, x, out, pair_pos=None):
    """The combine for routers some of whose outputs stand for experts that return their input: a choice with
    ids[t, k] >= n_real adds weights[t, k] * x[t] and has no row in y; the others as in `moe_combine`.
    ids int32 [T, top]; x [T, d] float32 or bfloat16."""
    T, top = weights.shape
    d = out.shape[1]
    _need(y, "y", None, (None if pair_pos is not None else T * top, d))
    _need(weights, "weights", torch.float32)
    _need(ids, "ids", torch.int32, (T, top))
    _need(x, "x", None, (T, d))
    _need(out, "out", torch.float32, (T, d))
    if pair_pos is not None:
        _need(pair_pos, "pair_pos", torch.int32, (T * top,))
    _work(T * top * d * y.element_size() + _nbytes(weights, x, out))
    f = _fn("moe", "llmie_moe_combine_identity", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                                                  _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(y.data_ptr(), _dt(y, "y"), _ptr(pair_pos), weights.data_ptr(), ids.data_ptr(), int(n_real), x.data_ptr(),
             _dt(x, "x"), out.data_ptr(), T, d, top, _stream()), "moe_combine_identity")
    return out


def moe_gather_rows(x, rows, out):
    """out[p] = x[rows[p]] (zeros where rows[p] < 0); bfloat16 rows of a multiple of 8 elements."""
    P, d = out.shape
    _need(x, "x", torch.bfloat16, (None, d))
    _need(out, "out", torch.bfloat16)
    _need(rows, "rows", torch.int32)
    if rows.shape[0] < P:
        raise KernelError("moe_gather_rows: rows shorter than the output")
    _work(2 * _nbytes(out))
    f = _fn("moe", "llmie_moe_gather_rows", [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(x.data_ptr(), rows.data_ptr(), out.data_ptr(), P, d, _stream()), "moe_gather_rows")
    return out


def moe_gather_scaled(x, sorted_token, sorted_pair, weights, out):
    """out[p] = weights[sorted_pair[p]] * x[sorted_token[p]] (zeros where sorted_token[p] < 0): the rows of the sorted
    positions, each times its pair's weight (float32 product, one rounding). x [T, d] and out [P, d] float32 or
    bfloat16; weights float32 [T, top]."""
    P, d = out.shape
    _need(x, "x", None, (None, d))
    _need(out, "out")
    _need(sorted_token, "sorted_token", torch.int32)
    _need(sorted_pair, "sorted_pair", torch.int32)
    _need(weights, "weights", torch.float32)
    if sorted_token.shape[0] < P or sorted_pair.shape[0] < P:
        raise KernelError("moe_gather_scaled: index arrays shorter than the output")
    _work(2 * _nbytes(out))
    f = _fn("moe", "llmie_moe_gather_scaled", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                               _c_int, _c_int, _c_void_p])
    _check(f(x.data_ptr(), _dt(x, "x"), sorted_token.data_ptr(), sorted_pair.data_ptr(), weights.data_ptr(),
             out.data_ptr(), _dt(out, "out"), P, d, _stream()), "moe_gather_scaled")
    return out


def library_grouped_mm(x: torch.Tensor, w: torch.Tensor, group_end: torch.Tensor) -> torch.Tensor:
    """Rows [group_end[e-1], group_end[e]) of x [P, K] times w[e]^T (w [E, N, K]) through the library's grouped GEMM
    (bfloat16 in and out, float32 accumulation); rows beyond group_end[-1] are left as they are. Like `library_mm`
    this is the product that prompts leave to the vendor library; the offsets stay on the device."""
    def run():
        return torch._grouped_mm(x, w.transpose(-2, -1), offs=group_end)
    t = trace.timer
    if t is None:
        return run()
    P, K = x.shape
    t.note(_nbytes(x, w) + P * w.shape[1] * 2, 2.0 * P * w.shape[1] * K)
    return t.run("library_grouped_mm", run, ())


def library_grouped_mm_ok(n_pairs: int, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    """Whether the routed products of a prompt go to the library: bfloat16, enough pairs for tiles of 64 to fill, and
    rows that start on 16 bytes."""
    return (hasattr(torch, "_grouped_mm") and w_gate_up.dtype == torch.bfloat16 and n_pairs > GROUPED_SMALL_ROWS * 4
            and w_gate_up.shape[2] % 8 == 0 and w_down.shape[2] % 8 == 0 and w_down.shape[1] % 8 == 0)


# ------------------------------------------------------------------------------------------ latent attention
def latent_prepare(proj, q_off: int, dkv_off: int, q_out, cache, norm_w, eps: float, table, rot_dims: int, tok_pos,
                   tok_seq, seq_slot, block_table, page_size: int, n_heads: int, dim: int, rot: int, rank: int,
                   write: bool, q_src=None):
    """Per token: the latent's RMS norm, the rotation of the shared key part and of every head's rotated query part,
    the cache write (rows [latent | rotated key part]) and the rotated query parts into the last `rot` columns of each
    head of q_out [T, n_heads (rank + rot)]. proj [T, ld] holds the queries from column q_off (heads of dim + rot) and,
    if `write`, the latent projection from dkv_off (rank + rot). table float32 [P, rot_dims / 2, 2] of (cos, sin).
    `q_src` ([T, >= q_off + n_heads (dim + rot)], proj's dtype): the queries are read from there instead of proj."""
    T, ld = proj.shape
    _need(proj, "proj")
    qs = proj if q_src is None else q_src
    if q_src is not None:
        _need(q_src, "q_src", proj.dtype, (T, None))
    _need(q_out, "q_out", proj.dtype, (T, n_heads * (rank + rot)))
    _need(table, "table", torch.float32, (None, rot_dims // 2, 2))
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if q_off + n_heads * (dim + rot) > qs.shape[1] or (write and dkv_off + rank + rot > ld):
        raise KernelError("latent_prepare: the projections do not fit the rows of proj")
    if write:
        _need(cache, "cache", proj.dtype, (None, 1, page_size, rank + rot))
        _need(norm_w, "norm_w", torch.float32, (rank,))
    _work(T * (n_heads * 2 * rot + (2 * (rank + rot) if write else 0)) * proj.element_size())
    f = _fn("latent", "llmie_latent_prepare_from",
            [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p,
             _c_int, _c_int] + [_c_void_p] * 4 + [_c_int] * 9 + [_c_void_p])
    _check(f(proj.data_ptr(), ld, qs.data_ptr(), qs.shape[1], q_off, dkv_off if write else 0, q_out.data_ptr(),
             _ptr(cache) if write else None,
             _ptr(norm_w) if write else None, float(eps), table.data_ptr(), table.shape[0], rot_dims,
             tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), block_table.data_ptr(), block_table.shape[1],
             page_size, T, n_heads, dim, rot, rank, 1 if write else 0, _dt(proj, "proj"), _stream()), "latent_prepare")
    return q_out


# ------------------------------------------------------------------------------------------ attention by rows
def attention_rows_mma_supported(head_dim: int, v_head_dim: int, page_size: int, dtype: torch.dtype,
                                 shared_rows: bool) -> bool:
    """The sizes attention_rows_mma.cu takes (answered without loading the library): bfloat16, a head size that is a
    multiple of 16 up to 1024, a value size that is a multiple of 8 up to 512, pages of whole tiles of 32 keys, and
    about 200 KB of shared memory for the staged tiles."""
    if dtype != torch.bfloat16 or head_dim <= 0 or head_dim % 16 or head_dim > 1024 or v_head_dim <= 0 \
            or v_head_dim % 8 or v_head_dim > 512 or page_size % 32 or (shared_rows and v_head_dim > head_dim):
        return False
    kp, vp = head_dim + 8, v_head_dim + 8
    smem = 32 * kp * 2 + 2 * 32 * kp * 2 + (0 if shared_rows else 2 * 32 * vp * 2) + 4 * 32 * 33 * 4 + 32 * 40 * 2 + 32 * 4
    return smem <= 200 * 1024


def attention_rows_mma(q, k_cache, v_cache, out, cu_q, seq_slot, seq_start, block_table, page_size: int, n_seqs: int,
                       max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0,
                       softcap: float = 0.0, dist_bias: Optional[torch.Tensor] = None,
                       sink_values: Optional[torch.Tensor] = None, sink: bool = False,
                       sigmoid_bias: Optional[torch.Tensor] = None):
    """Attention on the tensor cores with the (token, head) pairs of a key/value head as rows (bfloat16): prompts and
    one-token steps, any head size that is a multiple of 16, a value size of its own, values that are columns of the
    key rows (v_cache a view into k_cache), scale, window, cap, bias by distance, sink and sigmoid weights as in
    attention_paged."""
    T = q.shape[0]
    hdv = v_cache.shape[-1]
    _need(q, "q", torch.bfloat16, (T, n_q * head_dim))
    _need(out, "out", torch.bfloat16, (T, n_q * hdv))
    _need(k_cache, "k_cache", torch.bfloat16, (None, n_kv, page_size, head_dim))
    shared_rows = False
    if v_cache.is_contiguous():
        _need(v_cache, "v_cache", torch.bfloat16, (k_cache.shape[0], n_kv, page_size, hdv))
        v_ld = hdv
    else:
        v_ld = v_cache.stride(-2)
        if (v_cache.dtype is not torch.bfloat16 or tuple(v_cache.shape) != (k_cache.shape[0], n_kv, page_size, hdv)
                or v_cache.stride() != (n_kv * page_size * v_ld, page_size * v_ld, v_ld, 1)):
            raise KernelError("attention_rows_mma: v_cache must be contiguous or a column range of contiguous rows")
        shared_rows = v_cache.data_ptr() == k_cache.data_ptr() and v_ld == head_dim
    for name, t in (("cu_q", cu_q), ("seq_slot", seq_slot), ("seq_start", seq_start), ("block_table", block_table)):
        _need(t, name, torch.int32)
    bias_len = 0
    if dist_bias is not None:
        _need(dist_bias, "dist_bias", torch.float32, (n_q, None))
        bias_len = dist_bias.shape[1]
    if sink_values is not None:
        _need(sink_values, "sink_values", torch.float32, (n_q,))
        sink = True
    if sigmoid_bias is not None:
        _need(sigmoid_bias, "sigmoid_bias", torch.float32, (n_q,))
    _work(2 * _nbytes(q) + 1.0 * STEP_HINT["kv_total"] * n_kv * (head_dim + (0 if shared_rows else hdv)) * 2,
          2.0 * n_q * (head_dim + hdv) * STEP_HINT["pairs"])
    f = _fn("attention_rows_mma", "llmie_attention_rows_mma",
            [_c_void_p] * 8 + [_c_int] * 10 + [_c_float, _c_int, _c_float, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                                               _c_void_p])
    _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), cu_q.data_ptr(), seq_slot.data_ptr(),
             seq_start.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, n_seqs, max_q_len, n_q, n_kv,
             head_dim, hdv, int(v_ld), 1 if shared_rows else 0, float(scale), int(window), float(softcap or 0.0),
             _ptr(dist_bias), bias_len, _ptr(sink_values), 1 if sink else 0, _ptr(sigmoid_bias), _stream()),
           "attention_rows_mma")
    return out


# ------------------------------------------------------------------------------------------ scaled branches, PolyNorm
def scaled_add_rmsnorm(h, d1, c1: float, d2, c2: float, scale, weight, eps: float, out, rows=None):
    """h += scale (.) (c1 d1 + c2 d2) (float32, in place, when rows is None); out = rmsnorm(h) * weight.
    h float32 [T, d]; d1, d2 [T, d] float32 or bfloat16 (d2 or both may be None); scale float32 [d] or None; weight
    float32 [d] with out [n_out, d], or both None (the add alone). With `rows` (int32 [n_out]) only those rows are
    produced and h stays as it is."""
    T, d = h.shape
    n_out = T if rows is None else rows.shape[0]
    _need(h, "h", torch.float32)
    for name, t in (("d1", d1), ("d2", d2)):
        if t is not None:
            _need(t, name, None, (T, d))
    if scale is not None:
        _need(scale, "scale", torch.float32, (d,))
    if (weight is None) != (out is None):
        raise KernelError("scaled_add_rmsnorm: weight and out go together")
    if out is not None:
        _need(weight, "weight", torch.float32, (d,))
        _need(out, "out", None, (n_out, d))
    if rows is not None:
        _need(rows, "rows", torch.int32, (n_out,))
        if n_out == 0:
            return out                   # no row is wanted and h stays as it is
    _work((2 * _nbytes(h) if rows is None else n_out * d * 4) + _nbytes(d1, d2, out))
    f = _fn("scaled_elementwise", "llmie_scaled_add_rmsnorm",
            [_c_void_p, _c_void_p, _c_int, _c_float, _c_void_p, _c_int, _c_float, _c_void_p, _c_void_p, _c_float,
             _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(h.data_ptr(), _ptr(d1), _dt(d1, "d1") if d1 is not None else 0, float(c1), _ptr(d2),
             _dt(d2, "d2") if d2 is not None else 0, float(c2), _ptr(scale), _ptr(weight), float(eps), _ptr(out),
             _dt(out, "out") if out is not None else 0, _ptr(rows), n_out, d, _stream()), "scaled_add_rmsnorm")
    return out


def poly_norm(z, coef, eps: float, out):
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row, N(t) = t / sqrt(mean(t^2) + eps); coef float32 [4] = (a, b, c, e)
    on the device; z, out [T, n] of one dtype; float32 arithmetic."""
    T, n = z.shape
    _need(z, "z")
    _need(out, "out", z.dtype, (T, n))
    _need(coef, "coef", torch.float32, (4,))
    _work(_nbytes(z, out))
    f = _fn("scaled_elementwise", "llmie_poly_norm", [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_int,
                                                      _c_void_p])
    _check(f(z.data_ptr(), coef.data_ptr(), float(eps), out.data_ptr(), T, n, _dt(z, "z"), _stream()), "poly_norm")
    return out


# ------------------------------------------------------------------------------------------ recurrent mixers
def matrix_gates(proj, q_off: int, f_off: int, f_bias, lower, q_out, f_out):
    """q_out = silu(proj[:, q_off : q_off + n]); f_out = lower + (1 - lower) sigmoid(proj[:, f_off : f_off + n] + f_bias).
    proj [T, ld] float32 or bfloat16; f_bias, lower float32 [n]; q_out, f_out float32 [T, n]."""
    T, n = q_out.shape
    _need(proj, "proj", None, (T, None))
    _need(f_bias, "f_bias", torch.float32, (n,))
    _need(lower, "lower", torch.float32, (n,))
    _need(q_out, "q_out", torch.float32)
    _need(f_out, "f_out", torch.float32, (T, n))
    _work(2 * T * n * proj.element_size() + _nbytes(q_out, f_out))
    f = _fn("recurrent", "llmie_matrix_gates", [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                                _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(proj.data_ptr(), proj.shape[1], int(q_off), int(f_off), f_bias.data_ptr(), lower.data_ptr(),
             q_out.data_ptr(), f_out.data_ptr(), T, n, _dt(proj, "proj"), _stream()), "matrix_gates")


# Long pieces of the recurrences run as chunks side by side. Which arithmetic a sequence gets depends on its own piece
# alone, never on what else is in the step: the matrix scan cuts every piece at multiples of SCAN_CHUNK tokens and a
# piece of one chunk goes through the very operations of the unchunked kernel; the unit scan cuts a piece into
# UNIT_CHUNKS equal chunks and a piece of up to UNIT_CHUNKS tokens does the same. So the chunked kernels are launched
# whenever the step's longest piece has more than one chunk. (Only a step whose chunks' starting states would pass
# SCAN_SCRATCH_BYTES gets longer chunks.)
SCAN_CHUNK = 64
UNIT_CHUNKS = 32
SCAN_SCRATCH_BYTES = 1 << 30


def matrix_scan(q, f, v, state, cu_q, seq_slot, out, n_seqs: int, heads: int, dim: int, vdim: int,
                write_state: bool = True, max_len: int = 0, head_decay: Optional[torch.Tensor] = None):
    """Per sequence and head, from the state S [dim, vdim] the slot holds: S <- diag(f_t) S + (1 - f_t) v_t^T and
    out_t = S^T q_t for each of the step's tokens in order; the new S is written back. q, f float32 [T, heads dim];
    v [T, heads vdim] (possibly a column slice) float32 or bfloat16; state float32 [slots, heads, dim, vdim];
    out float32 [T, heads vdim]. `max_len`: an upper bound of the longest piece, if the caller knows one; long pieces
    are cut into chunks that run side by side (each chunk from zero, a chain over the chunks' ends, each chunk again
    from its true start), which changes rounding only. With `head_decay` (float32 [heads]) the recurrence is the
    keyed one, S <- head_decay[h] S + k_t v_t^T, and `f` holds the keys k (linear attention with a constant decay)."""
    T = q.shape[0]
    if head_decay is not None:
        _need(head_decay, "head_decay", torch.float32, (heads,))
    _need(q, "q", torch.float32, (T, heads * dim))
    _need(f, "f", torch.float32, (T, heads * dim))
    _need(state, "state", torch.float32, (None, heads, dim, vdim))
    _need(out, "out", torch.float32, (T, heads * vdim))
    _need(cu_q, "cu_q", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    v_ld = _row_slice(v, "v", v.dtype, T, heads * vdim)
    _work(_nbytes(q, f, out) + T * heads * vdim * v.element_size() + 2.0 * n_seqs * heads * dim * vdim * 4,
          4.0 * T * heads * dim * vdim)
    if max_len > SCAN_CHUNK and n_seqs > 0:
        chunk, per_chunk = SCAN_CHUNK, n_seqs * heads * dim * vdim * 4
        while -(-max_len // chunk) * per_chunk > SCAN_SCRATCH_BYTES and chunk < max_len:
            chunk *= 2
        n_chunks = -(-max_len // chunk)
        if 2 <= n_chunks and n_seqs * n_chunks <= 65535:
            ws = torch.empty((n_seqs, n_chunks, heads, dim, vdim), dtype=torch.float32, device=q.device)
            decay = torch.empty((n_seqs, n_chunks, heads, dim), dtype=torch.float32, device=q.device)
            _work(3.0 * _nbytes(ws) + _nbytes(f) + T * heads * vdim * v.element_size(), 4.0 * T * heads * dim * vdim)
            f_ = _fn("recurrent", "llmie_matrix_scan_chunked_ex",
                     [_c_void_p, _c_void_p, _c_void_p, _c_int] + [_c_void_p] * 6 + [_c_int] * 8 + [_c_void_p, _c_void_p])
            _check(f_(q.data_ptr(), f.data_ptr(), v.data_ptr(), v_ld, state.data_ptr(), cu_q.data_ptr(),
                      seq_slot.data_ptr(), out.data_ptr(), ws.data_ptr(), decay.data_ptr(), n_seqs, heads, dim, vdim,
                      chunk, n_chunks, 1 if write_state else 0, _dt(v, "v"), _ptr(head_decay), _stream()),
                   "matrix_scan_chunked")
            return out
    f_ = _fn("recurrent", "llmie_matrix_scan_ex", [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                                   _c_void_p, _c_void_p] + [_c_int] * 6 + [_c_void_p, _c_void_p])
    _check(f_(q.data_ptr(), f.data_ptr(), v.data_ptr(), v_ld, state.data_ptr(), cu_q.data_ptr(), seq_slot.data_ptr(),
              out.data_ptr(), n_seqs, heads, dim, vdim, 1 if write_state else 0, _dt(v, "v"), _ptr(head_decay),
              _stream()), "matrix_scan")
    return out


def head_rmsnorm(o, weight, eps: float, out, vdim: int, gate=None):
    """out = o / sqrt(mean(o^2) + eps) * weight over every run of vdim columns (a head; vdim = the row's width: the
    concatenated heads together, with a weight per column); o float32 [T, heads vdim]; weight float32 [vdim]; out of
    the activation type. `gate` ([T, heads vdim] of out's type, possibly a column slice): out is also multiplied by
    sigmoid(gate)."""
    T, n = o.shape
    _need(o, "o", torch.float32)
    _need(weight, "weight", torch.float32, (vdim,))
    _need(out, "out", None, (T, n))
    if n % vdim:
        raise KernelError("head_rmsnorm: the row is not a whole number of heads")
    gate_ld = _row_slice(gate, "gate", out.dtype, T, n) if gate is not None else 0
    _work(_nbytes(o, out) + (T * n * out.element_size() if gate is not None else 0))
    f = _fn("recurrent", "llmie_head_rmsnorm_gated", [_c_void_p, _c_void_p, _c_float, _c_void_p, ctypes.c_longlong, _c_int,
                                                      _c_int, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(o.data_ptr(), weight.data_ptr(), float(eps), out.data_ptr(), T * (n // vdim), vdim, _dt(out, "out"),
             _ptr(gate), gate_ld, n // vdim, _stream()), "head_rmsnorm")
    return out


def act_columns(proj, runs, act: int):
    """Float32 copies of up to three runs of columns of proj [T, ld] (float32 or bfloat16), each through the activation
    `act` (an ACT_* code): `runs` is a list of (first column, float32 out [T, n]); out[t, c] = act(proj[t, first + c])."""
    T, ld = proj.shape
    _need(proj, "proj")
    if not 1 <= len(runs) <= 3:
        raise KernelError("act_columns: one to three runs of columns")
    args = []
    for off, out in runs:
        _need(out, "out", torch.float32, (T, None))
        if off < 0 or off + out.shape[1] > ld:
            raise KernelError("act_columns: a run of columns does not fit the rows of proj")
        args += [int(off), out.shape[1], out.data_ptr()]
    args += [0, 0, None] * (3 - len(runs))
    total = sum(out.shape[1] for _, out in runs)
    _work(T * total * (proj.element_size() + 4))
    f = _fn("recurrent", "llmie_act_columns", [_c_void_p, _c_int] + [_c_int, _c_int, _c_void_p] * 3 +
            [_c_int, _c_int, _c_int, _c_void_p])
    _check(f(proj.data_ptr(), ld, *args, int(act), T, _dt(proj, "proj"), _stream()), "act_columns")


def causal_conv(proj, x_off: int, x_bias, taps, conv_bias, conv_state, cu_q, tok_seq, seq_slot, out):
    """out[t, c] = conv_bias[c] + sum_j taps[c, K-1-j] x[t-j, c] with x = proj[:, x_off + c] + x_bias[c]; inputs from
    before the step are the slot's conv_state (its last K-1 inputs, zeros at a sequence's start).
    taps float32 [C, K]; conv_state float32 [slots, K-1, C]; out float32 [T, C]."""
    T, C = out.shape
    K = taps.shape[1]
    _need(proj, "proj", None, (T, None))
    _need(taps, "taps", torch.float32, (C, K))
    _need(conv_state, "conv_state", torch.float32, (None, K - 1, C))
    _need(out, "out", torch.float32)
    for name, t in (("x_bias", x_bias), ("conv_bias", conv_bias)):
        if t is not None:
            _need(t, name, torch.float32, (C,))
    for name, t in (("cu_q", cu_q), ("tok_seq", tok_seq), ("seq_slot", seq_slot)):
        _need(t, name, torch.int32)
    _work(T * C * (proj.element_size() + 4))
    f = _fn("recurrent", "llmie_causal_conv", [_c_void_p, _c_int, _c_int] + [_c_void_p] * 8 + [_c_int] * 4 + [_c_void_p])
    _check(f(proj.data_ptr(), proj.shape[1], int(x_off), _ptr(x_bias), taps.data_ptr(), _ptr(conv_bias),
             conv_state.data_ptr(), cu_q.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), out.data_ptr(), T, C, K,
             _dt(proj, "proj"), _stream()), "causal_conv")
    return out


def unit_gate_values(gates, u, r_bias, i_bias, lam, c_decay: float, block_width: int):
    """gates float32 [T, 2 C], per group of block_width channels the pre-activations of r and then of i, become in place
    a = exp(-c_decay sigmoid(r + r_bias) softplus(lam)) and sqrt(1 - a^2) sigmoid(i + i_bias) u. u float32 [T, C]."""
    T, C = u.shape
    _need(u, "u", torch.float32)
    _need(gates, "gates", torch.float32, (T, 2 * C))
    for name, t in (("r_bias", r_bias), ("i_bias", i_bias), ("lam", lam)):
        _need(t, name, torch.float32, (C,))
    _work(2 * _nbytes(gates) + _nbytes(u))
    f = _fn("recurrent", "llmie_unit_gate_values", [_c_void_p] * 5 + [_c_float, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(gates.data_ptr(), u.data_ptr(), r_bias.data_ptr(), i_bias.data_ptr(), lam.data_ptr(), float(c_decay), T, C,
             int(block_width), _stream()), "unit_gate_values")


def unit_scan(gates, proj, y_off: int, x_off: int, y_bias, x_bias, act: int, state, conv_state, cu_q, seq_slot, out,
              n_seqs: int, block_width: int, write_state: bool = True, max_len: int = 0):
    """Per sequence and channel, from the slot's state S: S <- a_t S + drive_t, out_t = S * act(proj[t, y_off + c] +
    y_bias[c]) for the step's tokens in order (gates as `unit_gate_values` leaves them); the new S and the last K-1
    inputs of the convolution (proj[:, x_off + c] + x_bias) are written back. state float32 [slots, C]; conv_state
    float32 [slots, K-1, C]; out [T, C] of proj's dtype. `max_len`: an upper bound of the longest piece, if the caller
    knows one; long pieces run as 32 chunks side by side, which changes rounding only."""
    T, C = out.shape
    K = conv_state.shape[1] + 1
    _need(gates, "gates", torch.float32, (T, 2 * C))
    _need(proj, "proj", None, (T, None))
    _need(out, "out", proj.dtype)
    _need(state, "state", torch.float32, (None, C))
    _need(conv_state, "conv_state", torch.float32, (state.shape[0], K - 1, C))
    for name, t in (("y_bias", y_bias), ("x_bias", x_bias)):
        if t is not None:
            _need(t, name, torch.float32, (C,))
    _need(cu_q, "cu_q", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    _work(_nbytes(gates, out) + T * C * proj.element_size())
    f = _fn("recurrent", "llmie_unit_scan", [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                                             _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p] + [_c_int] * 7 +
            [_c_void_p])
    _check(f(gates.data_ptr(), proj.data_ptr(), proj.shape[1], int(y_off), int(x_off), _ptr(y_bias), _ptr(x_bias),
             int(act), state.data_ptr(), conv_state.data_ptr(), cu_q.data_ptr(), seq_slot.data_ptr(), out.data_ptr(),
             n_seqs, C, int(block_width), K, 1 if write_state else 0, 1 if max_len > UNIT_CHUNKS else 0,
             _dt(proj, "proj"), _stream()), "unit_scan")
    return out
