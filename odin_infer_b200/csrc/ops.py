"""Python bindings of the kernels: torch tensors in, raw pointers out.

Every function launches on torch's current CUDA stream (so a CUDA graph
capture records it), checks its arguments on the host, and raises on any
error code.  There is no fallback of any kind: a tensor that is not on a
CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build

PAGE = 64  # tokens per cache page

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"unsupported element type {dt}; kernels take float32 and bfloat16") from None


def _ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernel argument is not on a CUDA device (there is no CPU path)")
    return c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_ERRORS = {-1: "unsupported size or element type", -2: "bad argument", -3: "device wait ran out"}


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far (kernels inside replayed CUDA graphs included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code != 0:
        msg = _ERRORS.get(code, f"CUDA error {code}")
        raise KernelError(f"{what}: {msg}")
    _launches += kernels


def _fn(group: str, name: str):
    """A launcher of the kernel libraries."""
    f = getattr(build.load(group), name)
    f.restype = c_int
    return f


# ----------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] = table[ids[t], :] * scale as 32-bit floats; ids int32 [T]."""
    T, d = out.shape
    assert out.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == d
    assert table.is_contiguous() and out.is_contiguous()
    _check(_fn("elementwise", "odin_embed")(
        _ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(out), c_int(T), c_int(d),
        c_int(table.shape[0]), c_float(scale), _stream()), "embed")


def embed_pair(table: torch.Tensor, pair: torch.Tensor, ids: torch.Tensor, tok_seq: torch.Tensor, seq_start: torch.Tensor,
               seq_slots: torch.Tensor, state: torch.Tensor, n_seqs: int, buckets: int, mul_prev: int, mul_cur: int,
               out: torch.Tensor, scale: float = 1.0, single_rows: bool = False) -> None:
    """out[t] = table[ids[t]] * scale + pair[(prev * mul_prev + ids[t] * mul_cur) mod buckets] as 32-bit floats, prev the
    token before in the sequence: the row above, or what `state` (int32 [slots, >= 1], any row stride) holds for the
    sequence's slot (token + 1; 0: the sequence starts here, and row `buckets` of `pair` stands in).  A second kernel
    then stores every sequence's last token of this step in `state`.  Rows of sequence -1 become zeros.
    single_rows: every sequence brings exactly one row; the one kernel then stores the token itself."""
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and ids.dtype == torch.int32
    assert table.shape[1] == d and tuple(pair.shape) == (buckets + 1, d) and pair.dtype == table.dtype
    assert table.is_contiguous() and pair.is_contiguous() and state.dtype == torch.int32 and state.stride(1) == 1
    _check(_fn("elementwise", "odin_embed_pair")(
        _ptr(table), _ptr(pair), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(tok_seq), _ptr(seq_start), _ptr(seq_slots),
        _ptr(state), c_longlong(state.stride(0)), c_int(n_seqs), c_int(buckets), c_longlong(mul_prev), c_longlong(mul_cur),
        _ptr(out), c_int(T), c_int(d), c_int(table.shape[0]), c_float(scale), c_int(1 if single_rows else 0), _stream()),
        "embed_pair", kernels=1 if single_rows else 2)


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """x += sum of delta's leading splits (in place, 32-bit); out = RMSNorm(x) * weight.

    x: [n, d] float32.  delta: None, [n, d] or [splits, n, d].  rows: None, or
    int32 row numbers to gather (then x is left as it is).
    """
    d = x.shape[-1]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n_split, stride = 1, 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-1] == d
        if delta.dim() == 3:
            n_split, stride = delta.shape[0], delta.shape[1] * d
            assert delta.shape[1] == x.shape[0]
        else:
            assert delta.shape[0] == x.shape[0]
    n_rows = out.shape[0]
    if rows is None:
        assert n_rows == x.shape[0]
    else:
        assert rows.dtype == torch.int32 and rows.numel() == n_rows
    assert weight.numel() == d
    _check(_fn("elementwise", "odin_add_rmsnorm")(
        _ptr(x), _ptr(delta), c_int(dtype_code(delta.dtype) if delta is not None else 0), c_int(n_split),
        c_longlong(stride), _ptr(weight), c_int(dtype_code(weight.dtype)), c_float(eps), _ptr(out),
        c_int(dtype_code(out.dtype)), _ptr(rows), c_int(n_rows), c_int(d), _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate) * up for gate_up = [T, 2I] (gate columns first), or for the sum of
    its leading parts when gate_up is [parts, T, 2I] (float32 partial sums of a split product)."""
    T, I = out.shape
    assert gate_up.is_contiguous() and out.is_contiguous() and tuple(gate_up.shape[-2:]) == (T, 2 * I)
    n_split, stride = (gate_up.shape[0], T * 2 * I) if gate_up.dim() == 3 else (1, 0)
    _check(_fn("elementwise", "odin_swiglu")(
        _ptr(gate_up), c_int(dtype_code(gate_up.dtype)), c_int(n_split), c_longlong(stride), _ptr(out),
        c_int(dtype_code(out.dtype)), c_int(T), c_int(I), _stream()), "swiglu")


def random_fill(out: torch.Tensor, key: int, mean: float, scale: float) -> None:
    """out.flatten()[i] = mean + scale * (centred sum of eight 16-bit uniforms of stream `key` at i): the
    device side of the counter-based random weights (weights/random_init.py has the host side)."""
    assert out.is_contiguous()
    _check(_fn("elementwise", "odin_random_fill")(
        _ptr(out), c_int(dtype_code(out.dtype)), c_longlong(out.numel()), ctypes.c_ulonglong(key & ((1 << 64) - 1)),
        c_float(mean), c_float(scale), _stream()), "random_fill")


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    assert src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel()
    _check(_fn("elementwise", "odin_cast")(
        _ptr(src), c_int(dtype_code(src.dtype)), _ptr(dst), c_int(dtype_code(dst.dtype)),
        c_longlong(src.numel()), _stream()), "cast")


ACTIVATIONS = {"tanh": 0, "silu": 1, "gelu_tanh": 2, "xielu": 3, "relu2": 4}   # relu2: max(z, 0)^2


def _parts(t: torch.Tensor, rows: int, cols: int) -> tuple[int, int]:
    """(number of partial sums, their distance in elements) of a product's output [rows, cols] or [parts, rows, cols]."""
    assert t.is_contiguous() and tuple(t.shape[-2:]) == (rows, cols)
    return (t.shape[0], rows * cols) if t.dim() == 3 else (1, 0)


def row_update(x: torch.Tensor, delta, bias: torch.Tensor | None, weight: torch.Tensor | None,
               eps: float, groups: int, out: torch.Tensor | None, rows: torch.Tensor | None = None,
               normalise: bool = True, scale: float = 1.0, weight2: torch.Tensor | None = None,
               out2: torch.Tensor | None = None) -> None:
    """x += sum of delta's parts + bias (in place, 32-bit; not with a row gather), then
    normalise: out = weight * x / rms, the root mean square taken over each of `groups` equal
    consecutive parts of the row by itself (out may be x: in place); else out = x converted
    (out None: the update alone).  delta may be a list of up to three updates (each [n, d] or
    [parts, n, d]; all but the first 32-bit), which are added in their order.  scale != 1: the updates (and the
    bias) are added up by themselves and x += scale * their sum.  out2 with weight2: a second norm of the same row,
    out2 = weight2 * x / rms with the root mean square formed once (out's dtype and shape)."""
    d = x.shape[-1]
    assert x.dtype == torch.float32 and x.is_contiguous()
    more = []
    if isinstance(delta, (list, tuple)):
        delta, more = (delta[0], list(delta[1:])) if delta else (None, [])
    n_split, stride = (1, 0)
    if delta is not None:
        n_split, stride = _parts(delta, x.shape[0], d)
    if more or (scale != 1.0 and delta is not None) or out2 is not None:
        assert len(more) <= 2 and all(m.dtype == torch.float32 for m in more)
        if out2 is not None:
            assert normalise and weight2 is not None and weight2.numel() == d and out is not None
            assert out2.is_contiguous() and out2.shape == out.shape and out2.dtype == out.dtype
            assert out2.data_ptr() not in (x.data_ptr(), out.data_ptr())
        extra = []
        for m in more + [None] * (2 - len(more)):
            ns, st = _parts(m, x.shape[0], d) if m is not None else (0, 0)
            extra += [_ptr(m), c_int(ns), c_longlong(st)]
        if out is not None:
            assert out.is_contiguous() and out.shape[-1] == d
        n_rows = x.shape[0] if rows is None else rows.numel()
        if rows is not None:
            assert rows.dtype == torch.int32 and out is not None and out.shape[0] == n_rows
        if normalise:
            assert weight is not None and weight.numel() == d and out is not None and d % groups == 0
        _check(_fn("rowwise", "odin_row_update_several")(
            _ptr(x), _ptr(delta), c_int(dtype_code(delta.dtype) if delta is not None else 0), c_int(n_split),
            c_longlong(stride), *extra,
            _ptr(bias), c_int(dtype_code(bias.dtype) if bias is not None else 0), _ptr(weight),
            c_int(dtype_code(weight.dtype) if weight is not None else 0), c_float(eps), c_int(groups),
            c_int(0 if normalise else 1), _ptr(out), c_int(dtype_code(out.dtype) if out is not None else 0), _ptr(rows),
            c_int(n_rows), c_int(d), c_float(scale), _ptr(weight2),
            c_int(dtype_code(weight2.dtype) if weight2 is not None else 0), _ptr(out2), _stream()), "row_update")
        return
    if out is not None:
        assert out.is_contiguous() and out.shape[-1] == d
    n_rows = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        assert rows.dtype == torch.int32 and out is not None and out.shape[0] == n_rows
    if normalise:
        assert weight is not None and weight.numel() == d and out is not None and d % groups == 0
    if bias is not None:
        assert bias.numel() == d
    _check(_fn("rowwise", "odin_row_update")(
        _ptr(x), _ptr(delta), c_int(dtype_code(delta.dtype) if delta is not None else 0), c_int(n_split),
        c_longlong(stride), _ptr(bias), c_int(dtype_code(bias.dtype) if bias is not None else 0), _ptr(weight),
        c_int(dtype_code(weight.dtype) if weight is not None else 0), c_float(eps), c_int(groups),
        c_int(0 if normalise else 1), _ptr(out), c_int(dtype_code(out.dtype) if out is not None else 0), _ptr(rows),
        c_int(n_rows), c_int(d), _stream()), "row_update")


def normed_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, tok_seq: torch.Tensor | None = None) -> None:
    """x += weight * y / rms(y) row by row; y may be [parts, n, d] partial sums.  Rows of sequence -1 are skipped."""
    n, d = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and weight.numel() == d
    n_split, stride = _parts(y, n, d)
    _check(_fn("rowwise", "odin_normed_add")(
        _ptr(x), _ptr(y), c_int(dtype_code(y.dtype)), c_int(n_split), c_longlong(stride), _ptr(weight),
        c_int(dtype_code(weight.dtype)), c_float(eps), _ptr(tok_seq), c_int(n), c_int(d), _stream()), "normed_add")


def activation(src: torch.Tensor, kind: str, out: torch.Tensor, params: torch.Tensor | None = None,
               row_scale: torch.Tensor | None = None) -> None:
    """out = act(src) element by element; src [T, n] (a strided view is fine) or [parts, T, n] partial sums,
    added first.  kind: tanh, silu, gelu_tanh, or xielu with params = (p, q):
    z > 0: softplus(p) z^2 + z/2, else (1/2 + softplus(q)) (e^z - 1 - z) + z/2; relu2: max(z, 0)^2.
    row_scale: float32 [T]; row t of the result is multiplied by row_scale[t]."""
    T, n = out.shape
    if row_scale is not None:
        assert row_scale.dtype == torch.float32 and row_scale.is_contiguous() and row_scale.numel() == T
    assert out.stride(1) == 1 and src.stride(-1) == 1 and tuple(src.shape[-2:]) == (T, n)
    if src.dim() == 3:
        assert src.is_contiguous()
        n_split, stride, row = src.shape[0], T * n, n
    else:
        n_split, stride, row = 1, 0, src.stride(0)
    _check(_fn("rowwise", "odin_activation")(
        _ptr(src), c_int(dtype_code(src.dtype)), c_int(n_split), c_longlong(stride), c_longlong(row),
        c_int(ACTIVATIONS[kind]), _ptr(params), c_int(dtype_code(params.dtype) if params is not None else 0), _ptr(out),
        c_int(dtype_code(out.dtype)), c_longlong(out.stride(0)), c_int(T), c_int(n), _ptr(row_scale), _stream()), "activation")


def gated_activation(gate_up: torch.Tensor, kind: str, out: torch.Tensor) -> None:
    """out[t, c] = act(gate[t, c]) * up[t, c] for gate_up = [T, 2 n] (the n gate columns first), or for the sum of
    its leading parts when it is [parts, T, 2 n]; kind: silu (SwiGLU) or gelu_tanh (GeGLU)."""
    T, n = out.shape
    assert out.stride(1) == 1 and gate_up.stride(-1) == 1 and tuple(gate_up.shape[-2:]) == (T, 2 * n)
    if gate_up.dim() == 3:
        assert gate_up.is_contiguous()
        n_split, stride, row = gate_up.shape[0], T * 2 * n, 2 * n
    else:
        n_split, stride, row = 1, 0, gate_up.stride(0)
    _check(_fn("rowwise", "odin_gated_activation")(
        _ptr(gate_up), c_int(dtype_code(gate_up.dtype)), c_int(n_split), c_longlong(stride), c_longlong(row),
        c_int(ACTIVATIONS[kind]), _ptr(out), c_int(dtype_code(out.dtype)), c_longlong(out.stride(0)), c_int(T), c_int(n),
        _stream()), "gated_activation")


def sigmoid_gate(o: torch.Tensor, gate: torch.Tensor, n_heads: int, v_head_dim: int, per_head: bool) -> None:
    """o[t, h, c] *= sigmoid(gate[t, h]) (per_head) or sigmoid(gate[t, h, c]), in place; gate: columns of a product's
    output, [T, n] (a strided view is fine) or [parts, T, n] partial sums (a view of whole rows' columns)."""
    T = o.shape[0]
    n = n_heads if per_head else n_heads * v_head_dim
    assert o.stride(1) == 1 and o.shape[1] == n_heads * v_head_dim and gate.stride(-1) == 1
    assert tuple(gate.shape[-2:]) == (T, n)
    if gate.dim() == 3:
        n_split, stride, row = gate.shape[0], gate.stride(0), gate.stride(1)
    else:
        n_split, stride, row = 1, 0, gate.stride(0)
    _check(_fn("rowwise", "odin_sigmoid_gate")(
        _ptr(o), c_int(dtype_code(o.dtype)), c_longlong(o.stride(0)), _ptr(gate), c_int(dtype_code(gate.dtype)),
        c_int(n_split), c_longlong(stride), c_longlong(row), c_int(1 if per_head else 0), c_int(T), c_int(n_heads),
        c_int(v_head_dim), _stream()), "sigmoid_gate")


def softcap(z: torch.Tensor, cap: float, scale: float = 1.0) -> None:
    """z <- scale * cap * tanh(z / cap) in place (cap 0: z <- scale * z); z float32 [rows, n]."""
    assert z.dtype == torch.float32 and z.dim() == 2 and z.stride(1) == 1
    _check(_fn("rowwise", "odin_softcap")(_ptr(z), c_longlong(z.stride(0)), c_int(z.shape[0]), c_int(z.shape[1]),
                                          c_float(cap), c_float(scale), _stream()), "softcap")


class Term:
    """One term of a combined update (see `combine_add`): `value` [n, d] or [parts, n, d] partial sums, times `scale`,
    times row_scale[r] (float32 [n]) where given; with norm_weight ([d]) the summed row is first divided by its root mean
    square (norm_eps inside the root) and multiplied by that weight."""

    def __init__(self, value: torch.Tensor, scale: float = 1.0, row_scale: torch.Tensor | None = None,
                 norm_weight: torch.Tensor | None = None, norm_eps: float = 0.0):
        self.value, self.scale, self.row_scale = value, float(scale), row_scale
        self.norm_weight, self.norm_eps = norm_weight, float(norm_eps)


def combine_add(x: torch.Tensor | None, terms: list, post_weight: torch.Tensor | None = None, post_eps: float = 0.0,
                next_weight: torch.Tensor | None = None, next_eps: float = 0.0, out: torch.Tensor | None = None,
                rows: torch.Tensor | None = None, tok_seq: torch.Tensor | None = None) -> None:
    """y = the sum of up to four `Term`s; x += post_weight * y / rms(y) (post_weight None: x += y), in place unless `rows`
    gathers; then out = next_weight * x / rms(x) where next_weight is given.  x None: out (float32) = y.  Rows of sequence
    -1 (tok_seq) are skipped.  All sums 32-bit, in an order that the width fixes."""
    assert 0 < len(terms) <= 4
    ref = x if x is not None else out
    d = ref.shape[-1]
    n_all = x.shape[0] if x is not None else out.shape[0]
    n_rows = n_all if rows is None else rows.numel()
    if x is not None:
        assert x.dtype == torch.float32 and x.is_contiguous()
    if out is not None:
        assert out.is_contiguous() and tuple(out.shape) == (n_rows, d)
    if rows is not None:
        assert rows.dtype == torch.int32
    n = len(terms)
    ptrs, dts, nsp, sst, scl = (c_void_p * n)(), (c_int * n)(), (c_int * n)(), (c_longlong * n)(), (c_float * n)()
    rsc, nws, nwd, nep = (c_void_p * n)(), (c_void_p * n)(), (c_int * n)(), (c_float * n)()
    for i, t in enumerate(terms):
        v = t.value
        ns, st = _parts(v, n_all, d)
        ptrs[i], dts[i], nsp[i], sst[i], scl[i] = _ptr(v), dtype_code(v.dtype), ns, st, t.scale
        if t.row_scale is not None:
            assert t.row_scale.dtype == torch.float32 and t.row_scale.is_contiguous() and t.row_scale.numel() == n_all
        rsc[i] = _ptr(t.row_scale)
        if t.norm_weight is not None:
            assert t.norm_weight.numel() == d and t.norm_weight.is_contiguous()
        nws[i], nwd[i] = _ptr(t.norm_weight), dtype_code(t.norm_weight.dtype) if t.norm_weight is not None else 0
        nep[i] = t.norm_eps
    for w in (post_weight, next_weight):
        assert w is None or (w.numel() == d and w.is_contiguous())
    _check(_fn("rowwise", "odin_combine_add")(
        _ptr(x), c_int(n), ptrs, dts, nsp, sst, scl, rsc, nws, nwd, nep, _ptr(post_weight),
        c_int(dtype_code(post_weight.dtype) if post_weight is not None else 0), c_float(post_eps), _ptr(next_weight),
        c_int(dtype_code(next_weight.dtype) if next_weight is not None else 0), c_float(next_eps), _ptr(out),
        c_int(dtype_code(out.dtype) if out is not None else 0), _ptr(rows), _ptr(tok_seq), c_int(n_rows), c_int(d),
        _stream()), "combine_add")


def moe_router(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, top: int, always: int,
               tok_seq: torch.Tensor | None, ids: torch.Tensor, wts: torch.Tensor, logits: torch.Tensor | None = None,
               score: str = "softmax_of_chosen", groups: int = 1, keep: int = 1, route_scale: float = 1.0,
               gate_row: bool = False, gate_out: torch.Tensor | None = None, n_real: int | None = None,
               pass_out: torch.Tensor | None = None) -> None:
    """Per token: logits W h + bias in 32-bit, the `top` largest chosen, weights = softmax over the chosen logits;
    `always` further choices name the experts E, E + 1, ... with weight 1.  ids int32, wts float32: [T, top + always];
    rows of sequence -1 get expert -1.  logits: W h where a product has formed it already (float32 [T, rows of W]).

    score "sigmoid_in_groups": scores sigmoid(z); the experts form `groups` equal groups of neighbours, a group's score
    is the sum of its two largest scores, only experts of the `keep` best groups can be chosen (the `top` largest
    scores among them); weights = chosen scores / (their sum + 1e-20) * route_scale.
    score "softmax_corrected_in_groups": scores softmax(z) over all rows; an expert is chosen by score + bias (a correction
    that the weights do not see), a group's score is its largest choice score, weights = chosen scores / (their sum +
    1e-20) * route_scale.  n_real: the first n_real rows of W have experts behind them; a token that chooses a later row
    gets its own input back times that weight: such places name expert -1 with weight 0, and the token's summed weight of
    them goes to pass_out (float32 [T]).  The `always` choices name the experts n_real, n_real + 1, ...
    gate_row: W has one row more than there are experts, g; the `always` choices are weighted by sigmoid(g . h),
    which also goes to gate_out (float32 [T]) where given."""
    T, d = h.shape
    E = w.shape[0] - (1 if gate_row else 0)
    assert h.stride(1) == 1 and w.is_contiguous() and w.shape[1] == d
    assert ids.dtype == torch.int32 and wts.dtype == torch.float32 and ids.is_contiguous() and wts.is_contiguous()
    assert tuple(ids.shape) == tuple(wts.shape) == (T, top + always)
    if bias is not None:
        assert bias.numel() == E and bias.is_contiguous()
    if logits is not None:
        assert logits.dtype == torch.float32 and logits.is_contiguous() and tuple(logits.shape) == (T, w.shape[0])
    if gate_out is not None:
        assert gate_row and gate_out.dtype == torch.float32 and gate_out.is_contiguous() and gate_out.numel() == T
    n_real = E if n_real is None else n_real
    if pass_out is not None:
        assert pass_out.dtype == torch.float32 and pass_out.is_contiguous() and pass_out.numel() == T
    _check(_fn("moe", "odin_moe_router")(
        _ptr(h), c_int(dtype_code(h.dtype)), c_longlong(h.stride(0)), _ptr(w), c_int(dtype_code(w.dtype)), _ptr(bias),
        c_int(dtype_code(bias.dtype) if bias is not None else 0), c_int(T), c_int(E), c_int(d), c_int(top), c_int(always),
        _ptr(tok_seq), _ptr(ids), _ptr(wts), _ptr(logits), c_int(ROUTER_SCORES[score]), c_int(groups), c_int(keep),
        c_float(route_scale), c_int(1 if gate_row else 0), _ptr(gate_out), c_int(n_real), _ptr(pass_out), _stream()),
        "moe_router")


ROUTER_SCORES = {"softmax_of_chosen": 0, "sigmoid_in_groups": 1, "softmax_corrected_in_groups": 2}


def moe_gate_up(h: torch.Tensor, w: torch.Tensor, ids: torch.Tensor, kind: str, out: torch.Tensor, gated: bool = True) -> None:
    """out[t * per + k, :] = act(Wg[e] h[t]) * (Wu[e] h[t]) with e = ids[t, k]; w: [experts, 2 ff, d], gate rows first.
    Not gated: out[t * per + k, :] = act(W[e] h[t]), w: [experts, ff, d]."""
    T, d = h.shape
    per, ff = ids.shape[1], out.shape[1]
    assert h.stride(1) == 1 and w.is_contiguous() and tuple(w.shape[1:]) == ((2 if gated else 1) * ff, d) and out.is_contiguous()
    assert out.shape[0] == T * per and out.dtype == h.dtype and ids.dtype == torch.int32 and ids.is_contiguous()
    _check(_fn("moe", "odin_moe_gate_up")(
        _ptr(h), c_int(dtype_code(h.dtype)), c_longlong(h.stride(0)), _ptr(w), c_int(dtype_code(w.dtype)), _ptr(ids),
        c_int(T), c_int(per), c_int(ff), c_int(d), c_int(ACTIVATIONS[kind]), c_int(1 if gated else 0), _ptr(out),
        _stream()), "moe_gate_up")


def moe_down(a: torch.Tensor, w: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, out: torch.Tensor) -> None:
    """out[k, t, :] = wts[t, k] * Wd[e] a[t * per + k] with e = ids[t, k]; w: [experts, d, ff]; out float32 [per, T, d]:
    partial sums of the tokens' update."""
    T, per = ids.shape
    ff, d = a.shape[1], w.shape[1]
    assert a.is_contiguous() and a.shape[0] == T * per and w.is_contiguous() and w.shape[2] == ff
    assert out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (per, T, d)
    _check(_fn("moe", "odin_moe_down")(
        _ptr(a), c_int(dtype_code(a.dtype)), _ptr(w), c_int(dtype_code(w.dtype)), _ptr(ids), _ptr(wts), c_int(T),
        c_int(per), c_int(ff), c_int(d), _ptr(out), _stream()), "moe_down")


def moe_places(rows: int, n_experts: int) -> int:
    """Places that `rows` rows take at most once every expert's rows are padded to whole tiles of 128."""
    return (rows + n_experts * 127 + 127) // 128 * 128


def moe_grouped_supported(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    """Shapes and types that the grouped tensor-core products take (bfloat16, rows of whole 16 bytes)."""
    d, inner = w_gate_up.shape[2], w_down.shape[2]
    return (h.dtype == w_gate_up.dtype == w_down.dtype == torch.bfloat16 and d % 8 == 0 and inner % 8 == 0
            and h.stride(1) == 1 and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0)


def moe_plan(ids: torch.Tensor, n_experts: int, place_of_row: torch.Tensor, row_of_place: torch.Tensor,
             tile_expert: torch.Tensor) -> None:
    """The rows (token, choice) of ids [T, per] in the order of their experts, every expert's rows padded to whole
    tiles of 128 places: place_of_row [T * per] (-1: the row has no expert), row_of_place [places] (-1: padding),
    tile_expert [places / 128] (-1: a tile that no rows reach).  Which place a row gets among its expert's is not
    fixed; nothing that is computed from a row depends on it."""
    rows = ids.numel()
    assert ids.dtype == torch.int32 and ids.is_contiguous() and place_of_row.numel() == rows
    assert row_of_place.numel() >= moe_places(rows, n_experts) and tile_expert.numel() * 128 == row_of_place.numel()
    _check(_fn("moe_tc", "odin_moe_plan")(_ptr(ids), c_int(rows), c_int(n_experts), _ptr(place_of_row), _ptr(row_of_place),
                                          c_int(row_of_place.numel()), _ptr(tile_expert), _stream()), "moe_plan")


def moe_gather(h: torch.Tensor, row_of_place: torch.Tensor, per: int, out: torch.Tensor) -> None:
    """out[place] = h[row_of_place[place] // per] (bfloat16), zeros where the place is padding."""
    assert h.dtype == out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == (row_of_place.numel(), h.shape[1])
    _check(_fn("moe_tc", "odin_moe_gather")(_ptr(h), c_longlong(h.stride(0)), _ptr(row_of_place), c_int(out.shape[0]),
                                            c_int(per), c_int(h.shape[1]), _ptr(out), _stream()), "moe_gather")


def moe_grouped(a: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, out: torch.Tensor, kind: str | None = None,
                gated: bool = True) -> None:
    """Every tile of 128 sorted rows of a [places, K] times the matrix of the tile's own expert (tcgen05).
    kind None: w [experts, N, K], out float32 [places, N] = a W[e]^T.  kind silu / gelu_tanh: w [experts, 2 N, K]
    (gate rows first), out bfloat16 [places, N] = act(a Wg[e]^T) * (a Wu[e]^T).  kind with gated=False (also relu2):
    w [experts, N, K], out bfloat16 [places, N] = act(a W[e]^T), the activation applied as the sums are read back."""
    places, K = a.shape
    n_e, rpe = w.shape[0], w.shape[1]
    N = out.shape[1]
    dual = kind is not None and gated
    if kind is not None and not gated:
        assert a.dtype == w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous() and w.shape[2] == K
        assert out.is_contiguous() and out.shape[0] == places and out.dtype == torch.bfloat16
        assert tile_expert.numel() * 128 == places and rpe == N
        _check(_fn("moe_tc", "odin_moe_grouped")(
            _ptr(a), c_longlong(a.stride(0)), _ptr(w), c_longlong(K), c_int(n_e), c_int(rpe), c_int(places), c_int(N), c_int(K),
            c_int(0), c_int(ACTIVATIONS[kind]), _ptr(tile_expert), _ptr(out), c_longlong(out.stride(0)), _stream()),
            "moe_grouped")
        return
    assert a.dtype == w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous() and w.shape[2] == K
    assert out.is_contiguous() and out.shape[0] == places and out.dtype == (torch.bfloat16 if dual else torch.float32)
    assert tile_expert.numel() * 128 == places and rpe == (2 * N if dual else N)
    _check(_fn("moe_tc", "odin_moe_grouped")(
        _ptr(a), c_longlong(a.stride(0)), _ptr(w), c_longlong(K), c_int(n_e), c_int(rpe), c_int(places), c_int(N), c_int(K),
        c_int(1 if dual else 0), c_int(ACTIVATIONS[kind] if dual else 0), _ptr(tile_expert), _ptr(out),
        c_longlong(out.stride(0)), _stream()), "moe_grouped")


def moe_combine(c: torch.Tensor, place_of_row: torch.Tensor, wts: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = sum_k wts[t, k] * c[place_of_row[t * per + k]] (float32), the choices in their order."""
    T, per = wts.shape
    d = c.shape[1]
    assert c.dtype == out.dtype == wts.dtype == torch.float32 and c.is_contiguous() and out.is_contiguous()
    assert tuple(out.shape) == (T, d) and place_of_row.numel() == T * per and wts.is_contiguous()
    _check(_fn("moe_tc", "odin_moe_combine")(_ptr(c), _ptr(place_of_row), _ptr(wts), c_int(T), c_int(per), c_int(d),
                                             _ptr(out), _stream()), "moe_combine")


def moe_tc_check() -> None:
    """Raise if a grouped product gave up a bounded wait since the last check (synchronises)."""
    f = build.load("moe_tc").odin_moe_tc_error
    f.restype = c_int
    if f() != 0:
        raise KernelError("moe_grouped: a device-side wait ran out (pipeline stalled); results are invalid")


def gated_lookup(gate: torch.Tensor, kind: str, table: torch.Tensor, col0: int, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, c] = act(gate[t, c]) * table[ids[t], col0 + c]; gate may be [parts, T, n] partial sums."""
    T, n = out.shape
    assert out.is_contiguous() and table.stride(1) == 1 and ids.dtype == torch.int32 and col0 + n <= table.shape[1]
    n_split, stride = _parts(gate, T, n)
    _check(_fn("rowwise", "odin_gated_lookup")(
        _ptr(gate), c_int(dtype_code(gate.dtype)), c_int(n_split), c_longlong(stride), c_int(ACTIVATIONS[kind]),
        _ptr(table), c_int(dtype_code(table.dtype)), c_longlong(table.stride(0)), c_int(col0), c_int(table.shape[0]),
        _ptr(ids), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(n), _stream()), "gated_lookup")


def token_shift(h: torch.Tensor, state: torch.Tensor, mu: torch.Tensor, out: torch.Tensor, tok_seq: torch.Tensor,
                seq_start: torch.Tensor, seq_slots: torch.Tensor) -> None:
    """out[s, t] = h[t] + (before - h[t]) * mu[s]: `before` is the row above in the same sequence or, for a
    sequence's first row of this step, the row of `state` (float32 [slots, >= d], any row stride) of its slot."""
    T, d = h.shape
    n_mix = mu.shape[0]
    assert h.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (n_mix, T, d) and out.dtype == h.dtype
    assert mu.is_contiguous() and mu.shape[1] == d and state.dtype == torch.float32 and state.stride(1) == 1
    _check(_fn("recurrent", "odin_token_shift")(
        _ptr(h), c_int(dtype_code(h.dtype)), _ptr(state), c_longlong(state.stride(0)), _ptr(mu),
        c_int(dtype_code(mu.dtype)), c_int(n_mix), _ptr(out), _ptr(tok_seq), _ptr(seq_start), _ptr(seq_slots),
        c_int(T), c_int(d), _stream()), "token_shift")


RECURRENCE_MODES = {"bonus": 0, "gated": 1, "fixed": 2, "gla": 3, "ssd": 4}


def linear_recurrence(mode: str, q: torch.Tensor, k: torch.Tensor | None, g: torch.Tensor | None, v: torch.Tensor,
                      c0: torch.Tensor, c1: torch.Tensor, out: torch.Tensor, state: torch.Tensor,
                      seq_start: torch.Tensor, seq_slots: torch.Tensor, n_seqs: int, n_heads: int, dk: int, dv: int,
                      shift_src: torch.Tensor | None = None, shift_state: torch.Tensor | None = None,
                      block_len: int = 0, max_new: int = 0, q_scale: float = 1.0, heads_per_group: int = 1) -> None:
    """The recurrence over a matrix-valued state per (sequence, head), S: [dk, dv] in `state`
    (float32 [slots, >= H dk dv], any row stride), sequence b's rows being seq_start[b] .. seq_start[b+1]:

    "bonus": w = exp(-exp(g + c0)); o = (S + diag(c1) k v^T)^T q; S = diag(w) S + k v^T
    "gated": f = c1 + (1 - c1) sigmoid(g + c0); S = diag(f) S + (1 - f) v^T; o = S^T silu(q)
    "fixed": S = c0 S + k v^T; o = S^T q (one constant decay per head, c0: [H]; g and c1 unused)
    "gla":   w = sigmoid(g + c0)^c1 (as exp(c1 logsigmoid(g + c0))); S = diag(w) S + k v^T; o = S^T (q_scale q)
    "ssd":   per head and token dt = softplus(g[t, head] + c1[head]), w = exp(-exp(c0[head]) dt) (g: [T, H], c0, c1: [H]);
             S = w S + (dt k) v^T; o = S^T q; q and k are [T, (H / heads_per_group) dk]: heads_per_group heads share them

    q, k, g: float32 [T, H dk] (strided views are fine), v, out: float32 [T, H dv].
    shift_src / shift_state: after the walk the last row of shift_src of every sequence is stored
    (as float32) in its slot's row of shift_state.

    block_len > 0 (with max_new, the most rows any sequence brings): every sequence's rows are cut into blocks
    of block_len tokens that are walked side by side from a state of zeros; two small kernels then carry the
    state from block to block and add each block's incoming state to its tokens' outputs.  The same values up
    to rounding (sums in another order); for long prompts, which one walk per head cannot fill the GPU with."""
    if g is None:
        assert mode == "fixed"
        g = q
    for t in (q, g, v, out) + ((k,) if k is not None else ()):
        assert t.dtype == torch.float32 and t.stride(1) == 1
    assert state.dtype == torch.float32 and state.stride(1) == 1 and c0.dtype == c1.dtype
    per = n_heads if mode in ("fixed", "ssd") else n_heads * dk
    assert c0.numel() == per and c1.numel() == per
    kk = k if k is not None else q
    width = 0
    if shift_src is not None:
        assert shift_state is not None and shift_src.is_contiguous() and shift_state.dtype == torch.float32
        width = shift_src.shape[1]
    n_blocks, qp, s_loc, d_tot, kernels = 0, None, None, None, 1
    if block_len > 0:
        assert max_new > 0
        n_blocks = (max_new + block_len - 1) // block_len
        T = q.shape[0]
        qp = torch.empty(T, n_heads * dk, dtype=torch.float32, device=q.device)
        s_loc = torch.empty(n_seqs * n_blocks, n_heads * dk * dv, dtype=torch.float32, device=q.device)
        d_tot = torch.empty(n_seqs * n_blocks, n_heads * dk, dtype=torch.float32, device=q.device)
        kernels = 3
    _check(_fn("recurrent", "odin_linear_recurrence")(
        c_int(RECURRENCE_MODES[mode]), _ptr(q), c_longlong(q.stride(0)), _ptr(kk), c_longlong(kk.stride(0)),
        _ptr(g), c_longlong(g.stride(0)), _ptr(v), c_longlong(v.stride(0)), _ptr(c0), _ptr(c1),
        c_int(dtype_code(c0.dtype)), _ptr(out), c_longlong(out.stride(0)), _ptr(state), c_longlong(state.stride(0)),
        _ptr(seq_start), _ptr(seq_slots), c_int(n_seqs), c_int(n_heads), c_int(dk), c_int(dv), _ptr(shift_src),
        c_int(dtype_code(shift_src.dtype) if shift_src is not None else 0), _ptr(shift_state),
        c_longlong(shift_state.stride(0) if shift_state is not None else 0), c_int(width), c_int(block_len),
        c_int(n_blocks), _ptr(qp), _ptr(s_loc), _ptr(d_tot), c_float(q_scale), c_int(heads_per_group), _stream()),
        "linear_recurrence", kernels=kernels)


def causal_conv(src: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, silu: bool, state: torch.Tensor,
                tok_seq: torch.Tensor, seq_start: torch.Tensor, seq_slots: torch.Tensor, n_seqs: int, out: torch.Tensor,
                single_rows: bool = False) -> None:
    """out[t, c] = act(bias[c] + sum_j weight[c, j] src[t - (taps - 1 - j), c]) over each sequence's rows (act: SiLU or
    none); the rows before a step's first one come from `state` (float32 [slots, >= (taps - 1) C], any row stride: the
    sequence's last taps - 1 inputs, oldest first; zeros at its start), into which a second kernel stores the step's last
    inputs.  src: [T, C], a strided view is fine.  single_rows: every sequence brings exactly one row; the one kernel
    then stores the memory itself."""
    T, C = out.shape
    taps = weight.shape[1]
    assert src.stride(1) == 1 and tuple(src.shape) == (T, C) and out.stride(1) == 1
    assert weight.is_contiguous() and weight.shape[0] == C and state.dtype == torch.float32 and state.stride(1) == 1
    assert state.shape[1] >= (taps - 1) * C
    if bias is not None:
        assert bias.numel() == C and bias.is_contiguous()
    _check(_fn("state_space", "odin_causal_conv")(
        _ptr(src), c_int(dtype_code(src.dtype)), c_longlong(src.stride(0)), _ptr(weight), c_int(dtype_code(weight.dtype)),
        _ptr(bias), c_int(dtype_code(bias.dtype) if bias is not None else 0), c_int(taps), c_int(1 if silu else 0),
        _ptr(state), c_longlong(state.stride(0)), _ptr(tok_seq), _ptr(seq_start), _ptr(seq_slots), c_int(n_seqs), _ptr(out),
        c_int(dtype_code(out.dtype)), c_longlong(out.stride(0)), c_int(T), c_int(C), c_int(1 if single_rows else 0),
        _stream()), "causal_conv", kernels=2 if (taps > 1 and not single_rows) else 1)


def selective_scan(x: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor | None, B: torch.Tensor, C: torch.Tensor,
                   A_log: torch.Tensor, D: torch.Tensor | None, z: torch.Tensor | None, state: torch.Tensor,
                   out: torch.Tensor, seq_start: torch.Tensor, seq_slots: torch.Tensor, n_seqs: int,
                   block_len: int = 0, max_new: int = 0) -> None:
    """Per channel c and state index n, over each sequence's rows in order: step = softplus(dt + dt_bias),
    S[c, n] = exp(step_c A[c, n]) S[c, n] + step_c x_c B_n with A = -exp(A_log); out_c = (sum_n S[c, n] C_n + D_c x_c) *
    silu(z_c).  x, z: [T, inner] in one element type (views are fine); dt float32 [T, inner]; B, C float32 [T, N] views of
    one row stride; state float32 [slots, >= inner N], any row stride.  Everything inside is 32-bit.

    block_len > 0 (with max_new, the most rows any sequence brings): every sequence's rows are cut into blocks of block_len
    tokens that are walked side by side from a state of zeros; a second kernel carries the state from block to block, a
    third adds each block's incoming state to its tokens' outputs.  The same values up to rounding; for long prompts."""
    T, inner = out.shape
    N = A_log.shape[1]
    assert tuple(x.shape) == (T, inner) and x.stride(1) == 1 and dt.dtype == torch.float32 and dt.stride(1) == 1
    assert B.dtype == C.dtype == torch.float32 and B.stride(0) == C.stride(0) and B.stride(1) == C.stride(1) == 1
    assert tuple(B.shape) == tuple(C.shape) == (T, N) and A_log.is_contiguous() and A_log.shape[0] == inner
    assert state.dtype == torch.float32 and state.stride(1) == 1 and state.shape[1] >= inner * N and out.stride(1) == 1
    ws = [w for w in (A_log, D, dt_bias) if w is not None]
    assert len({w.dtype for w in ws}) == 1 and all(w.is_contiguous() for w in ws)
    if z is not None:
        assert z.dtype == x.dtype and z.stride(1) == 1 and tuple(z.shape) == (T, inner)
    n_blocks, ytmp, cumdt, s_loc, dtot, kernels = 0, None, None, None, None, 1
    if block_len > 0:
        assert max_new > 0
        n_blocks = (max_new + block_len - 1) // block_len
        ytmp = torch.empty(T, inner, dtype=torch.float32, device=out.device)
        cumdt = torch.empty(T, inner, dtype=torch.float32, device=out.device)
        s_loc = torch.empty(n_seqs * n_blocks, inner * N, dtype=torch.float32, device=out.device)
        dtot = torch.empty(n_seqs * n_blocks, inner, dtype=torch.float32, device=out.device)
        kernels = 3
    _check(_fn("state_space", "odin_selective_scan")(
        _ptr(x), c_int(dtype_code(x.dtype)), c_longlong(x.stride(0)), _ptr(dt), c_longlong(dt.stride(0)), _ptr(dt_bias),
        _ptr(B), _ptr(C), c_longlong(B.stride(0)), _ptr(A_log), _ptr(D), c_int(dtype_code(A_log.dtype)), _ptr(z),
        c_longlong(z.stride(0) if z is not None else 0), _ptr(state), c_longlong(state.stride(0)), _ptr(out),
        c_int(dtype_code(out.dtype)), c_longlong(out.stride(0)), _ptr(seq_start), _ptr(seq_slots), c_int(n_seqs),
        c_int(inner), c_int(N), c_int(block_len), c_int(n_blocks), _ptr(ytmp), _ptr(cumdt), _ptr(s_loc), _ptr(dtot),
        _stream()), "selective_scan", kernels=kernels)


def skip_gate_norm(o: torch.Tensor, x: torch.Tensor | None, D: torch.Tensor | None, head_dim: int, z: torch.Tensor | None,
                   weight: torch.Tensor | None, groups: int, eps: float, out: torch.Tensor) -> None:
    """out = weight * grouped_rms((o + D[head] x) * silu(z)): the row of `inner` elements (heads of head_dim) is cut into
    `groups` equal consecutive parts, each divided by its own root mean square.  o float32 [T, inner] contiguous; x float32
    view; z any view; D [heads] and weight [inner] of one element type; D (with x), z and weight are optional."""
    T, inner = o.shape
    assert o.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (T, inner)
    if D is not None:
        assert x is not None and x.dtype == torch.float32 and x.stride(1) == 1 and D.numel() * head_dim == inner
    if weight is not None:
        assert weight.numel() == inner and (D is None or D.dtype == weight.dtype)
    zd = z.dtype if z is not None else torch.float32
    wd = weight.dtype if weight is not None else (D.dtype if D is not None else torch.float32)
    _check(_fn("state_space", "odin_skip_gate_norm")(
        _ptr(o), _ptr(x if D is not None else None), c_longlong(x.stride(0) if D is not None else 0), _ptr(D),
        c_int(head_dim), _ptr(z), c_int(dtype_code(zd)), c_longlong(z.stride(0) if z is not None else 0), _ptr(weight),
        c_int(dtype_code(wd)), c_int(groups), c_float(eps), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(inner),
        _stream()), "skip_gate_norm")


def head_unit_scale(o: torch.Tensor, weight: torch.Tensor | None, per_head_weight: bool, gate: torch.Tensor | None,
                    eps: float, out: torch.Tensor, n_heads: int, dv: int) -> None:
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * silu(gate[t, h]) per head of dv elements; weight is
    [H dv] (per_head_weight) or [dv] shared by the heads, or None (no weight); gate (float32, optional) may be a
    strided view."""
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (T, n_heads * dv)
    assert weight is None or weight.numel() == (n_heads * dv if per_head_weight else dv)
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1
    _check(_fn("recurrent", "odin_head_unit_scale")(
        _ptr(o), _ptr(weight), c_int(dtype_code(weight.dtype) if weight is not None else 0),
        c_int(dv if per_head_weight else 0), _ptr(gate),
        c_longlong(gate.stride(0) if gate is not None else 0), c_float(eps), _ptr(out), c_int(dtype_code(out.dtype)),
        c_int(T), c_int(n_heads), c_int(dv), _stream()), "head_unit_scale")


def latent_prep(down: torch.Tensor, q_rank: int, kv_rank: int, rot: int, pairs: bool, q_norm: torch.Tensor | None,
                c_norm: torch.Tensor, eps: float, cq: torch.Tensor | None, cos: torch.Tensor, sin: torch.Tensor,
                tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor, cache: torch.Tensor | None,
                write_cache: bool = True) -> None:
    """A row of the fused down projection, down = [T, q_rank + kv_rank + rot] (or float32 partial sums [parts, T, ...]),
    is [query latent | key/value latent | key part that is rotated]: cq [T, q_rank] = RMSNorm(query latent) * q_norm;
    the cache row of the token's position, [kv_rank + rot] wide, becomes [RMSNorm(key/value latent) * c_norm | the key
    part rotated by the position] (pairs: elements 2i with 2i + 1, else i with i + rot / 2).
    cache: [pages, 1, PAGE, kv_rank + rot] of cq's type; cos, sin: float32 [positions, rot / 2]."""
    n = q_rank + kv_rank + rot
    if down.dim() == 3:
        n_split, T = down.shape[0], down.shape[1]
        assert down.is_contiguous() and down.shape[2] == n
        split_stride, row_stride = T * n, n
    else:
        n_split, T, split_stride, row_stride = 1, down.shape[0], 0, down.stride(0)
        assert down.stride(1) == 1 and down.shape[1] == n
    out_dtype = cq.dtype if cq is not None else cache.dtype
    if q_rank:
        assert cq is not None and cq.is_contiguous() and tuple(cq.shape) == (T, q_rank) and q_norm.numel() == q_rank
        assert q_norm.dtype == c_norm.dtype
    assert c_norm.numel() == kv_rank and cos.dtype == sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    assert rot == 0 or cos.shape[1] == rot // 2
    if write_cache:
        assert cache is not None and cache.is_contiguous() and cache.dtype == out_dtype
        assert tuple(cache.shape[1:]) == (1, PAGE, kv_rank + rot), "the latent cache is [page][1][64][kv_rank + rot]"
    _check(_fn("latent", "odin_latent_prep")(
        _ptr(down), c_int(dtype_code(down.dtype)), c_int(n_split), c_longlong(split_stride), c_longlong(row_stride),
        c_int(T), c_int(q_rank), c_int(kv_rank), c_int(rot), c_int(1 if pairs else 0), _ptr(q_norm), _ptr(c_norm),
        c_int(dtype_code(c_norm.dtype)), c_float(eps), _ptr(cq), c_int(dtype_code(out_dtype)), _ptr(cos), _ptr(sin),
        c_int(cos.shape[0]), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), c_int(block_table.stride(0)), _ptr(cache),
        c_int(PAGE), c_int(1 if write_cache else 0), _stream()), "latent_prep")


def heads_linear(a: torch.Tensor, a_head_stride: int, w: torch.Tensor, out: torch.Tensor, out_head_stride: int) -> None:
    """A product per head: out[t, h * out_head_stride + n] = sum_k a[t, h * a_head_stride + k] * w[h, k, n] for
    w [H, K, N] (input channel before output channel); a and out may be views with any row stride."""
    H, K, N = w.shape
    T = a.shape[0]
    assert w.is_contiguous() and a.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == T
    assert a.shape[1] >= (H - 1) * a_head_stride + K and out.shape[1] >= (H - 1) * out_head_stride + N
    _check(_fn("latent", "odin_heads_linear")(
        _ptr(a), c_int(dtype_code(a.dtype)), c_longlong(a.stride(0)), c_longlong(a_head_stride), _ptr(w),
        c_int(dtype_code(w.dtype)), _ptr(out), c_int(dtype_code(out.dtype)), c_longlong(out.stride(0)),
        c_longlong(out_head_stride), c_int(T), c_int(H), c_int(N), c_int(K), _stream()), "heads_linear")


def rope_heads(src: torch.Tensor, src_head_stride: int, dst: torch.Tensor, dst_head_stride: int, n_heads: int, width: int,
               rot: int, pairs: bool, cos: torch.Tensor, sin: torch.Tensor, tok_pos: torch.Tensor, scale: float = 1.0,
               scale_from_head: int | None = None) -> None:
    """dst[t, h, :width] = src[t, h, :width] with the first `rot` elements of every head turned by tok_pos[t] (pairs:
    element 2i with 2i + 1, else i with i + rot / 2) and the rest copied; heads from scale_from_head on are multiplied
    by `scale`.  src and dst: views with any row stride, heads src_head_stride / dst_head_stride elements apart; they
    may be the same memory."""
    T = src.shape[0]
    assert src.stride(1) == 1 and dst.stride(1) == 1 and dst.shape[0] == T
    assert src.shape[1] >= (n_heads - 1) * src_head_stride + width and dst.shape[1] >= (n_heads - 1) * dst_head_stride + width
    assert cos.dtype == sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    assert rot == 0 or cos.shape[1] == rot // 2
    _check(_fn("latent", "odin_rope_heads")(
        _ptr(src), c_int(dtype_code(src.dtype)), c_longlong(src.stride(0)), c_longlong(src_head_stride), _ptr(dst),
        c_int(dtype_code(dst.dtype)), c_longlong(dst.stride(0)), c_longlong(dst_head_stride), c_int(T), c_int(n_heads),
        c_int(width), c_int(rot), c_int(1 if pairs else 0), c_float(scale),
        c_int(n_heads if scale_from_head is None else scale_from_head), _ptr(cos), _ptr(sin), c_int(cos.shape[0]),
        _ptr(tok_pos), _stream()), "rope_heads")


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the CUDA cores with 32-bit accumulation."""
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(_fn("gemm_plain", "odin_gemm_plain")(
        _ptr(a), c_int(dtype_code(a.dtype)), _ptr(w), c_int(dtype_code(w.dtype)), _ptr(out),
        c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)),
        c_longlong(w.stride(0)), c_longlong(out.stride(0)), _stream()), "gemm_plain")


def gemm_tc_splits(K: int, n_split: int) -> int:
    """How many K parts `gemm_tc` really uses when asked for n_split."""
    f = build.load("gemm_tc").odin_gemm_tc_splits
    f.restype = c_int
    return int(f(c_int(K), c_int(n_split)))


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes and strides that the tensor-core kernel takes (TMA wants 16-byte rows)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
            and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, bn: int, n_split: int = 1,
            stages: int = 0, staged: int = 0) -> None:
    """out = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores (bfloat16 in, 32-bit accumulation).

    mode 0: tokens on the 128-row side of the MMA, tiles of bn weight rows.
    mode 1: weight rows on the 128-row side, tiles of bn tokens (M <= bn is usual).
    n_split > 1: out is float32 [n_split, M, N]; slice s holds the partial sum of K part s.
    stages: length of the kernel's ring of shared-memory stages; 0: as many as fit, fewer to
    leave room on the SM for a CTA of the neighbouring kernel.
    staged (mode 1): K blocks of every CTA's first item whose weights are fetched into tensor memory
    while the kernel before this one still runs; changes no bit of the result.
    """
    M, K = a.shape
    N = w.shape[0]
    if not gemm_tc_supported(a, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows (K and strides multiples of 8)")
    assert w.shape[1] == K and out.stride(-1) == 1
    if n_split > 1 or out.dim() == 3:
        assert out.dtype == torch.float32 and out.dim() == 3 and tuple(out.shape[1:]) == (M, N)
        assert out.shape[0] == gemm_tc_splits(K, n_split), "allocate gemm_tc_splits(K, n_split) slices"
        ldc, stride = out.stride(1), out.stride(0)
    else:
        assert tuple(out.shape) == (M, N)
        ldc, stride = out.stride(0), 0
    _check(_fn("gemm_tc", "odin_gemm_tc")(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(ldc), c_int(mode), c_int(bn), c_int(n_split),
        c_longlong(stride), c_int(stages), c_int(staged), _stream()), "gemm_tc")


GATE_ACTS = {"silu": 0, "gelu_tanh": 1}   # what the gate of a gated product's epilogue goes through


def gemm_tc_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[M, I] = act(a Wg^T) * (a Wu^T) for w_gate_up = [Wg; Wu] ([2 I, K]) in one tcgen05 kernel; act: silu
    (SwiGLU) or gelu_tanh (GeGLU)."""
    M, K = a.shape
    I = out.shape[1]
    if not gemm_tc_supported(a, w_gate_up):
        raise KernelError("gemm_tc_swiglu: operands must be bfloat16 with 16-byte aligned rows")
    assert w_gate_up.shape == (2 * I, K) and out.shape[0] == M and out.stride(1) == 1
    _check(_fn("gemm_tc", "odin_gemm_tc_gated")(
        _ptr(a), _ptr(w_gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(I), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w_gate_up.stride(0)), c_longlong(out.stride(0)),
        c_int(GATE_ACTS[activation]), _stream()), "gemm_tc_swiglu")


def gemm_tc2(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out = a[M, K] @ w[N, K]^T on pairs of SMs (tcgen05 cta_group::2, tiles of 256 x 256): for many tokens.
    accumulate: out (float32) += the product."""
    M, K = a.shape
    N = w.shape[0]
    if not gemm_tc_supported(a, w):
        raise KernelError("gemm_tc2: operands must be bfloat16 with 16-byte aligned rows (K and strides multiples of 8)")
    assert w.shape[1] == K and tuple(out.shape) == (M, N) and out.stride(1) == 1
    _check(_fn("gemm_tc", "odin_gemm_tc2")(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)), c_int(1 if accumulate else 0),
        _stream()), "gemm_tc2")


def gemm_tc2_wide(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n_split: int = 1) -> None:
    """out = a[M, K] @ w[N, K]^T for some hundred tokens on pairs of SMs, the weights on the wide side of the
    MMA and the tokens in tiles of 256 on its N side: out is [M, N], or float32 [n_split, M, N] partial sums of
    the K parts (as `gemm_tc`)."""
    M, K = a.shape
    N = w.shape[0]
    if not gemm_tc_supported(a, w):
        raise KernelError("gemm_tc2_wide: operands must be bfloat16 with 16-byte aligned rows (K and strides multiples of 8)")
    assert w.shape[1] == K and out.stride(-1) == 1
    if out.dim() == 3:
        assert out.dtype == torch.float32 and tuple(out.shape[1:]) == (M, N)
        assert out.shape[0] == gemm_tc_splits(K, n_split), "allocate gemm_tc_splits(K, n_split) slices"
        ldc, stride = out.stride(1), out.stride(0)
    else:
        assert tuple(out.shape) == (M, N) and n_split == 1
        ldc, stride = out.stride(0), 0
    _check(_fn("gemm_tc", "odin_gemm_tc2_wide")(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(ldc), c_int(n_split), c_longlong(stride),
        _stream()), "gemm_tc2_wide")


def gemm_tc2_swiglu_supported(inner: int) -> bool:
    return inner % 64 == 0


def gemm_tc2_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[M, I] = act(a Wg^T) * (a Wu^T) for w_gate_up = [Wg; Wu] ([2 I, K]) on pairs of SMs; I a multiple of 64;
    act: silu or gelu_tanh."""
    M, K = a.shape
    I = out.shape[1]
    if not gemm_tc_supported(a, w_gate_up):
        raise KernelError("gemm_tc2_swiglu: operands must be bfloat16 with 16-byte aligned rows")
    assert w_gate_up.shape == (2 * I, K) and out.shape[0] == M and out.stride(1) == 1
    _check(_fn("gemm_tc", "odin_gemm_tc2_gated")(
        _ptr(a), _ptr(w_gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(I), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w_gate_up.stride(0)), c_longlong(out.stride(0)),
        c_int(GATE_ACTS[activation]), _stream()), "gemm_tc2_swiglu")


def gemm_tc_check() -> None:
    """Raise if a tensor-core kernel gave up a bounded wait since the last check (synchronises)."""
    lib = build.load("gemm_tc")
    detail = (c_int * 8)()
    lib.odin_gemm_tc_error_detail.restype = c_int
    lib.odin_gemm_tc_error_detail(detail)
    f = lib.odin_gemm_tc_error
    f.restype = c_int
    if f() != 0:
        raise KernelError("gemm_tc: a device-side wait ran out (pipeline stalled); results are invalid "
                          f"[wait, block, item, k block, slot, mode, tile, grid] = {list(detail)}")
    lib.odin_gemm_tc2_error.restype = c_int
    if lib.odin_gemm_tc2_error(detail) != 0:
        raise KernelError("gemm_tc2: a device-side wait ran out (pipeline stalled); results are invalid "
                          f"[wait, block, tile, k block, slot, 2, tile, grid] = {list(detail)}")


def head_prep(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int, q_norm: torch.Tensor | None,
              k_norm: torch.Tensor | None, eps: float, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int,
              tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
              k_cache: torch.Tensor | None, v_cache: torch.Tensor | None, write_kv: bool = True,
              q_out: torch.Tensor | None = None, bias: torch.Tensor | None = None, unit_norm_after: bool = False,
              v_head_dim: int | None = None, whole_norm: bool = False, pairs: bool = False) -> torch.Tensor:
    """Per-head RMSNorm and rotation of q and k, and the cache write of k and v.

    bias: one value per column of the projection, added first.  unit_norm_after: instead of the
    weighted norm before the rotation, q and k heads are divided by their root mean square after it
    (q_norm and k_norm are then None).  v_head_dim: size of a value head when it differs from head_dim.
    whole_norm: the norm before the rotation runs over the token's whole q projection at once (and its whole k projection),
    with q_norm [n_q head_dim] and k_norm [n_kv head_dim].  pairs: the rotation pairs element 2i with 2i + 1.

    qkv: [T, (n_q + 2 n_kv) head_dim], or float32 partial sums [parts, T, ...] of a split
    product (added first).  q goes to q_out ([T, n_q head_dim], of the cache's type); without
    q_out it is written back into qkv (one part only).  Returns the tensor that holds q."""
    vd = head_dim if v_head_dim is None else v_head_dim
    width = (n_q + n_kv) * head_dim + n_kv * vd
    if qkv.dim() == 3:
        n_split, T = qkv.shape[0], qkv.shape[1]
        assert qkv.is_contiguous() and qkv.shape[2] >= width   # further columns (a gate's) are left alone
        split_stride, row_stride = T * qkv.shape[2], qkv.shape[2]
        assert q_out is not None, "partial sums need a separate q_out"
    else:
        n_split, T, split_stride, row_stride = 1, qkv.shape[0], 0, qkv.stride(0)
        assert qkv.stride(1) == 1 and qkv.shape[1] >= width
    if q_out is None:
        q_out = qkv[:, : n_q * head_dim]
    assert q_out.stride(1) == 1 and tuple(q_out.shape) == (T, n_q * head_dim)
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32
    assert tok_pos.dtype == torch.int32 and tok_seq.dtype == torch.int32 and block_table.dtype == torch.int32
    has_norm = q_norm is not None
    if has_norm:
        assert k_norm is not None and q_norm.dtype == k_norm.dtype and not unit_norm_after
        if whole_norm:
            assert q_norm.numel() == n_q * head_dim and (n_kv == 0 or k_norm.numel() == n_kv * head_dim)
        else:
            assert q_norm.numel() == head_dim and k_norm.numel() == head_dim
    if bias is not None:
        assert bias.numel() == width and bias.is_contiguous()
    if write_kv:
        assert k_cache is not None and v_cache is not None
        assert k_cache.dtype == q_out.dtype and v_cache.dtype == q_out.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim), "cache layout is [page][kv head][64][hd]"
        assert tuple(v_cache.shape[1:]) == (n_kv, PAGE, vd), "value cache layout is [page][kv head][64][vd]"
    _check(_fn("head_prep", "odin_head_prep")(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_int(n_split), c_longlong(split_stride), _ptr(q_out),
        c_longlong(q_out.stride(0)), c_int(dtype_code(q_out.dtype)), c_int(T), c_int(n_q), c_int(n_kv),
        c_int(head_dim), c_int(vd), c_longlong(row_stride), _ptr(bias),
        c_int(dtype_code(bias.dtype) if bias is not None else 0), _ptr(q_norm), _ptr(k_norm),
        c_int(dtype_code(q_norm.dtype) if has_norm else 0), c_int(2 if unit_norm_after else ((3 if whole_norm else 1) if has_norm else 0)),
        c_float(eps),
        _ptr(cos), _ptr(sin), c_int(rotary_dim), c_int(cos.shape[0]), _ptr(tok_pos), _ptr(tok_seq),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(k_cache), _ptr(v_cache), c_int(PAGE),
        c_int(1 if write_kv else 0), c_int(1 if pairs else 0), _stream()), "head_prep")
    return q_out


def attention_plain(q: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                    block_table: torch.Tensor, window: int = 0, chunk: int = 0, scale: float = 0.0,
                    softcap: float = 0.0, v_head_dim: int | None = None, sink: torch.Tensor | None = None) -> None:
    """Causal attention of each token over its sequence's cache; q may be a strided view.
    sink: float32 [n_q]; exp(sink[h]) joins the softmax's denominator of head h (no key, no value).

    window > 0: only the last `window` keys; chunk > 0: only the keys of the query's own chunk of
    `chunk` positions; scale > 0 replaces 1 / sqrt(head_dim); softcap > 0: scores pass through
    softcap * tanh(score / softcap); v_head_dim: size of a value head when it differs."""
    T = q.shape[0]
    vd = head_dim if v_head_dim is None else v_head_dim
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_cache.dtype
    assert q.shape[1] == n_q * head_dim and out.shape == (T, n_q * vd)
    assert tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim) and k_cache.is_contiguous()
    assert tuple(v_cache.shape[1:]) == (n_kv, PAGE, vd) and v_cache.is_contiguous()
    _check(_fn("attention_plain", "odin_attention_plain")(
        _ptr(q), c_longlong(q.stride(0)), _ptr(out), c_longlong(out.stride(0)), c_int(dtype_code(q.dtype)),
        c_int(T), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(vd), _ptr(k_cache), _ptr(v_cache), c_int(PAGE),
        _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), c_int(block_table.stride(0)), c_int(window), c_int(chunk),
        c_float(scale), c_float(softcap), _ptr(_sink(sink, n_q)), _stream()), "attention_plain")


def _sink(sink: torch.Tensor | None, n_q: int) -> torch.Tensor | None:
    if sink is not None:
        assert sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == n_q
    return sink


def attention_decode_supported(head_dim: int) -> bool:
    return head_dim in (16, 32, 64, 128, 256)


def attention_decode_scratch(n_tokens: int, n_q: int, head_dim: int, n_split: int) -> int:
    """Floats of scratch that `attention_decode` needs."""
    return n_tokens * n_q * n_split * (head_dim + 2)


def attention_decode(q: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                     k_cache: torch.Tensor, v_cache: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                     block_table: torch.Tensor, window: int, scratch: torch.Tensor, n_split: int, chunk: int = 0,
                     scale: float = 0.0, softcap: float = 0.0, sink: torch.Tensor | None = None) -> None:
    """One query token per row over its sequence's bfloat16 cache, keys split n_split ways.
    chunk, scale, softcap, sink: as `attention_plain` takes them.

    The counters on which a launch's key splits meet are one array of the library: all
    decode-attention launches of a process must be ordered on the GPU (one stream, or events
    between streams); two that overlap would mix their arrivals."""
    B = q.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
    assert q.shape[1] == n_q * head_dim and out.shape == (B, n_q * head_dim)
    assert tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim) and k_cache.is_contiguous()
    assert scratch.dtype == torch.float32 and scratch.numel() >= attention_decode_scratch(B, n_q, head_dim, n_split)
    _check(_fn("attention_decode", "odin_attention_decode_masked")(
        _ptr(q), c_longlong(q.stride(0)), _ptr(out), c_longlong(out.stride(0)), c_int(B), c_int(n_q), c_int(n_kv),
        c_int(head_dim), _ptr(k_cache), _ptr(v_cache), c_int(PAGE), c_int(k_cache.shape[0]), _ptr(tok_pos),
        _ptr(tok_seq), _ptr(block_table), c_int(block_table.stride(0)), c_int(window), c_int(chunk), c_float(scale),
        c_float(softcap), _ptr(_sink(sink, n_q)), _ptr(scratch), c_int(n_split), _stream()), "attention_decode", kernels=1 if head_dim in (64, 128) and n_q // n_kv <= 16 else 2)


def attention_decode_fused(qkv: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                           q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, eps: float, cos: torch.Tensor,
                           sin: torch.Tensor, rotary_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor, window: int,
                           scratch: torch.Tensor, n_split: int, write_kv: bool = True) -> bool:
    """`head_prep` and `attention_decode` in one kernel, for one token per sequence: qkv is the
    fused projection's output ([B, width] bfloat16, or float32 partial sums [parts, B, width]).
    Returns False, and launches nothing, where the tensor-core kernel does not apply; the
    caller then runs the two kernels."""
    width = (n_q + 2 * n_kv) * head_dim
    if qkv.dim() == 3:
        parts, B = qkv.shape[0], qkv.shape[1]
        if not (qkv.is_contiguous() and qkv.shape[2] == width and qkv.dtype == torch.float32):
            return False
        part_stride, row_stride = B * width, width
    else:
        parts, B, part_stride, row_stride = 1, qkv.shape[0], 0, qkv.stride(0)
        if not (qkv.stride(1) == 1 and qkv.shape[1] == width and qkv.dtype in (torch.bfloat16, torch.float32)):
            return False
    if not (out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16 and out.stride(1) == 1
            and tuple(out.shape) == (B, n_q * head_dim) and k_cache.is_contiguous() and v_cache.is_contiguous()
            and tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim) and cos.dtype == sin.dtype == torch.float32):
        return False
    has_norm = q_norm is not None
    if has_norm and not (k_norm is not None and q_norm.dtype == k_norm.dtype and q_norm.numel() == head_dim
                         and k_norm.numel() == head_dim):
        return False
    assert scratch.dtype == torch.float32 and scratch.numel() >= attention_decode_scratch(B, n_q, head_dim, n_split)
    code = _fn("attention_decode", "odin_attention_decode_fused")(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_int(parts), c_longlong(part_stride), c_longlong(row_stride),
        _ptr(out), c_longlong(out.stride(0)), c_int(B), c_int(n_q), c_int(n_kv), c_int(head_dim), _ptr(q_norm),
        _ptr(k_norm), c_int(dtype_code(q_norm.dtype) if has_norm else 0), c_int(1 if has_norm else 0), c_float(eps),
        _ptr(cos), _ptr(sin), c_int(rotary_dim), c_int(cos.shape[0]), _ptr(k_cache), _ptr(v_cache), c_int(PAGE),
        c_int(k_cache.shape[0]), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), c_int(block_table.stride(0)),
        c_int(window), _ptr(scratch), c_int(n_split), c_int(1 if write_kv else 0), _stream())
    if code == -1:  # unsupported: nothing was launched
        return False
    _check(code, "attention_decode_fused")
    return True


def attention_decode_check() -> None:
    f = build.load("attention_decode").odin_attention_decode_error
    f.restype = c_int
    if f() != 0:
        raise KernelError("attention_decode: a device-side wait ran out; results are invalid")


def attention_prefill_supported(head_dim: int) -> bool:
    return head_dim in (64, 128)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_new: int, n_q: int, n_kv: int,
                      head_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_start: torch.Tensor,
                      seq_len_after: torch.Tensor, block_table: torch.Tensor, window: int = 0, chunk: int = 0,
                      scale: float = 0.0, softcap: float = 0.0, sink: torch.Tensor | None = None) -> None:
    """Flash attention of each sequence's new tokens (rows seq_start[b]..seq_start[b+1] of q) over its
    bfloat16 cache, which already holds this step's keys and values: tcgen05.mma with accumulators in
    tensor memory."""
    T = q.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == n_q * head_dim and out.shape == (T, n_q * head_dim)
    assert tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim) and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert seq_start.dtype == torch.int32 and seq_len_after.dtype == torch.int32 and block_table.dtype == torch.int32
    _check(_fn("attention_prefill", "odin_attention_prefill_tc_masked")(
        _ptr(q), c_longlong(q.stride(0)), _ptr(out), c_longlong(out.stride(0)), c_int(n_seqs), c_int(max_new),
        c_int(n_q), c_int(n_kv), c_int(head_dim), _ptr(k_cache), _ptr(v_cache), c_int(k_cache.shape[0]),
        _ptr(seq_start), _ptr(seq_len_after), _ptr(block_table), c_int(block_table.stride(0)), c_int(window),
        c_int(chunk), c_float(scale), c_float(softcap), _ptr(_sink(sink, n_q)), _stream()), "attention_prefill")


def attention_prefill_check() -> None:
    detail = (c_int * 32)()
    build.load("attention_prefill").odin_attention_prefill_tc_error_detail(detail)
    for name in ("odin_attention_prefill_tc_error",):
        f = getattr(build.load("attention_prefill"), name)
        f.restype = c_int
        code = f()
        if code != 0:
            raise KernelError(f"attention_prefill ({name}): a device-side wait ran out or the kernel refused to run "
                              f"(code {code}); results are invalid; [wait, head, sequence, tile, iteration, pages, thread] = "
                              f"{list(detail)[:7]}; kinds that ran out (bit mask) {detail[7]:#x}, their last iterations + 1: {list(detail)[9:17]}")


def mma_probe(pattern: int, n: int = 64, b_mn: bool = False, commits: int = 0, per_sm: int = 1,
              iters: int = 4096) -> tuple[float, float]:
    """Cycles of the SM clock per MMA (patterns 0 and 1), per page / page pair (2 and 3) or per group of eight
    MMAs with its commit and wait (4 and 5) that the median CTA of the measuring kernel in mma_probe.cu took,
    and (4 and 5) the part of it until the eighth MMA was issued; per_sm CTAs share every SM's tensor core."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    grid = sms * per_sm
    cycles = torch.zeros(2 * grid, dtype=torch.int64, device="cuda:0")
    _check(_fn("mma_probe", "odin_mma_probe")(
        c_int(pattern), c_int(n), c_int(1 if b_mn else 0), c_int(commits), c_int(per_sm), c_int(iters),
        _ptr(cycles), _stream()), "mma_probe")
    torch.cuda.synchronize()
    f = build.load("mma_probe").odin_mma_probe_error
    f.restype = c_int
    if f() != 0:
        raise KernelError("mma_probe: a device-side wait ran out")
    whole, issue = cycles[:grid].sort().values, cycles[grid:].sort().values
    return float(whole[grid // 2].item()) / iters, float(issue[grid // 2].item()) / iters


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = index of the first maximum of logits[b, :] (float32)."""
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    _check(_fn("sampling", "odin_argmax")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(B), c_int(V), _ptr(out), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: float, top_p: float, coins: torch.Tensor,
           out: torch.Tensor) -> None:
    """Temperature (and top-p) draw, one coin in [0, 1) per row."""
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert coins.dtype == torch.float32 and coins.numel() >= B and out.dtype == torch.int32
    _check(_fn("sampling", "odin_sample")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(B), c_int(V), c_float(temperature),
        c_float(top_p), _ptr(coins), _ptr(out), _stream()), "sample")


def repetition_penalty(logits: torch.Tensor, recent: torch.Tensor, penalty: float) -> None:
    """In place on logits (a copy of the model's): recent is int32 [B, W], negative = empty."""
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert recent.dtype == torch.int32 and recent.is_contiguous() and recent.shape[0] == B
    _check(_fn("sampling", "odin_repetition_penalty")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(B), c_int(V), _ptr(recent),
        c_int(recent.shape[1]), c_float(penalty), _stream()), "repetition_penalty")
