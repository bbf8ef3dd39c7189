"""Python face of the CUDA kernels: loads each kernel module through ctypes at its
first use (building it if needed) and wraps the launchers.

There is no fallback: on a machine with a GPU a missing or unbuildable library
raises, and no operator here has a PyTorch or CPU stand-in.  Matrix products of
the bfloat16 path are this package's tcgen05 kernels for steps of up to 32 rows and,
from 128 rows, for the gate|up product (``KVB200_WIDE=all``: for every product); the
others go to the library (cuBLAS through ``torch.nn.functional.linear``) as all of
upstream's do (cublasGemmEx, base/src/engine.cu:653-671).  Everything else, and
every matrix product of the float32 path, is a kernel of this package.
"""

from __future__ import annotations

import collections
import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p
from typing import Dict, Optional

import torch

from . import build

_libs: Dict[str, ctypes.CDLL] = {}
launch_count = 0  # kernels of this package launched so far (library calls are not counted)
# Which kernel the dispatch below picked, how often (a launch that is captured into a graph counts
# once, at capture): what a test reads to see that the path it means to check is the one that ran.
choices: "collections.Counter[str]" = collections.Counter()

_ERR = {-1: "unsupported dtype", -2: "a size this kernel refuses", -3: "misaligned pointer or stride"}

STATUS_TEXT = {
    1: "a kernel met a position whose cache page is not mapped",
    2: "a kernel met a position outside the position-encoding table",
    3: "a kernel met a token id outside the vocabulary",
    4: "a bounded wait inside a kernel ran out",
}


class KernelError(RuntimeError):
    pass


def lib(name: str) -> ctypes.CDLL:
    got = _libs.get(name)
    if got is None:
        build.ensure_built([name])
        path = build.kernel_lib_path(name)
        try:
            got = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"the kernel library {path} cannot be loaded: {e}") from e
        _libs[name] = got
    return got


def prepare(names) -> None:
    """Builds (in parallel) and loads the named kernel modules."""
    build.ensure_built(list(names))
    for n in names:
        lib(n)


def loaded_libraries():
    return {n: str(build.kernel_lib_path(n)) for n in _libs}


def _check(rc: int, what: str) -> None:
    global launch_count
    if rc != 0:
        if rc < 0:
            raise KernelError(f"{what}: {_ERR.get(rc, rc)}")
        raise KernelError(f"{what}: CUDA error {rc} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")
    launch_count += 1
    if _marks is not None:
        _mark(what)


_marks = None      # while a step is being timed operator by operator: [(name, event after its launch)]


def _mark(name: str) -> None:
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    _marks.append((name, ev))


class timed_operators:
    """While active, an event is recorded behind every launch of this package and behind every
    library product; ``times`` afterwards maps operator name -> (launches, milliseconds), each
    interval running from the event before to the operator's own.  For steps whose kernels are
    long enough that the host is not the bound (prompt portions); not inside a graph capture."""

    def __enter__(self):
        global _marks
        _marks = []
        _mark("start")
        return self

    def __exit__(self, *exc):
        global _marks
        marks, _marks = _marks, None
        torch.cuda.synchronize()
        self.times = {}
        for (_, before), (name, ev) in zip(marks, marks[1:]):
            n, ms = self.times.get(name, (0, 0.0))
            self.times[name] = (n + 1, ms + before.elapsed_time(ev))
        return False


_step_stream: Optional[c_void_p] = None     # the stream of the running forward pass, looked up once
_step_capturing: Optional[bool] = None


class use_current_stream:
    """While active, the operators launch on the stream that was current at entry (and know whether
    it is being captured) without asking torch at every launch: the lookup costs 15 us, a step
    of a small model has a hundred launches."""

    def __enter__(self):
        global _step_stream, _step_capturing
        self.before = (_step_stream, _step_capturing)
        _step_stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        _step_capturing = torch.cuda.is_current_stream_capturing()
        return self

    def __exit__(self, *exc):
        global _step_stream, _step_capturing
        _step_stream, _step_capturing = self.before
        return False


def _stream() -> c_void_p:
    return _step_stream if _step_stream is not None else c_void_p(torch.cuda.current_stream().cuda_stream)


def _capturing() -> bool:
    return _step_capturing if _step_capturing is not None else torch.cuda.is_current_stream_capturing()


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_sm_count: Dict[int, int] = {}


def sm_count(device) -> int:
    """SMs of the device (asked once): what the dispatch compares a step's tiles with."""
    idx = torch.device(device).index or 0
    if idx not in _sm_count:
        _sm_count[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _sm_count[idx]


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {dt} has no kernels (float32 and bfloat16 do)")


_arena = None      # the running step's arena (engine/arena.py), None outside a step


class use_arena:
    """While active, the tensors that the operators below produce come out of ``arena``
    instead of the allocator."""

    def __init__(self, arena):
        self.arena = arena

    def __enter__(self):
        global _arena
        self.before, _arena = _arena, self.arena
        return self.arena

    def __exit__(self, *exc):
        global _arena
        _arena = self.before
        return False


def new(shape, dtype: torch.dtype, device) -> torch.Tensor:
    """An uninitialised result tensor: out of the running step's arena when there is one (on
    its device), otherwise from the allocator (operators called on their own)."""
    a = _arena
    if a is not None and a.device == device:
        return a.new(shape, dtype)
    return torch.empty(tuple(shape), dtype=dtype, device=device)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels of this package run on CUDA tensors only; there is no CPU path")


# ------------------------------------------------------------------ elementwise

def embed_gather(table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor,
                 sampled: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """float32 residual rows ``table[ids] * scale`` (the factor applied in float32).  With ``sampled`` (int32), an id ``-(1 + r)``
    stands for ``sampled[r]``: a token that is still on the device."""
    _need_cuda(table, ids, sampled)
    assert sampled is None or (sampled.dtype == torch.int32 and sampled.is_contiguous())
    V, H = table.shape
    T = ids.numel()
    out = new((T, H), torch.float32, table.device)
    rc = lib("elementwise").kvb_embed_gather(_p(table), dtype_code(table.dtype), _p(ids), _p(sampled),
                                             c_int(0 if sampled is None else sampled.numel()), _p(out),
                                             c_int(T), c_int(H), c_int(V), c_float(scale), _p(status), _stream())
    _check(rc, "embed_gather")
    return out


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``resid += delta`` (when given, in float32, in place unless ``rows`` selects),
    then RMSNorm of the sum times ``weight`` (no weight: ``None``); ``rows`` (int32) picks the rows to
    produce, in order, leaving ``resid`` untouched."""
    _need_cuda(resid)
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == resid.shape[1])
    T, H = resid.shape
    n = T if rows is None else rows.numel()
    out = new((n, H), out_dtype, resid.device)
    if delta is not None:
        assert delta.shape == resid.shape and delta.dtype == out_dtype and delta.is_contiguous()
    rc = lib("elementwise").kvb_add_rmsnorm(_p(resid), _p(delta), _p(weight), _p(out), _p(rows), c_int(n),
                                            c_int(H), c_float(eps), c_int(dtype_code(out_dtype)), _stream())
    _check(rc, "add_rmsnorm")
    return out


def silu_mul(gate_up: torch.Tensor, block: Optional[int] = None) -> torch.Tensor:
    """``silu(gate) * up`` for rows that hold gate and up in alternating blocks of
    ``block`` features ([gate | up] as a whole when ``block`` is None)."""
    _need_cuda(gate_up)
    assert gate_up.is_contiguous()
    T, two_i = gate_up.shape
    I = two_i // 2
    out = new((T, I), gate_up.dtype, gate_up.device)
    rc = lib("elementwise").kvb_silu_mul(_p(gate_up), _p(out), c_int(T), c_int(I), c_int(block or I),
                                         c_int(dtype_code(gate_up.dtype)), _stream())
    _check(rc, "silu_mul")
    return out


def rope_kv_write(qkv, positions, token_req, cos, sin, k_pages, v_pages, block_table, page_size,
                  nq, nkv, d, rot, status) -> None:
    """Rotates q (in place) and k, writes k and v into their pages.  ``k_pages`` None:
    only q is rotated.  ``cos`` None: no rotation."""
    _need_cuda(qkv)
    assert qkv.is_contiguous() and qkv.shape[1] == (nq + 2 * nkv) * d
    T = qkv.shape[0]
    table_len = 0 if cos is None else cos.shape[0]
    num_pages = 0 if k_pages is None else k_pages.shape[0]
    if k_pages is not None:
        assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == qkv.dtype
        assert tuple(k_pages.shape[1:]) == (nkv, page_size, d), (k_pages.shape, nkv, page_size, d)
    max_pages = block_table.shape[1]
    rc = lib("elementwise").kvb_rope_kv_write(
        _p(qkv), _p(positions), _p(token_req), _p(cos), _p(sin), c_int(table_len), _p(k_pages),
        _p(v_pages), _p(block_table), c_int(max_pages), c_int(page_size), c_int(num_pages), c_int(T),
        c_int(nq), c_int(nkv), c_int(d), c_int(rot), c_int(dtype_code(qkv.dtype)), _p(status), _stream())
    _check(rc, "rope_kv_write")


# ------------------------------------------------------------------ norms around a branch, gated activations

NORM_KINDS = {None: 0, "none": 0, "copy": 0, "layer": 1, "rms": 2}


class PostNormed:
    """A branch's output that still has to pass a norm of its own before it joins the residual
    stream: ``delta`` [T, H] (plus ``bias`` [H], float32, if the branch's last product has one),
    the norm's ``kind`` ("layer" or "rms"), its float32 ``weight`` (a per-channel scale of the
    branch is multiplied into it) and ``eps``.  The norm that follows (:func:`add_norm`) carries
    it out in the kernel that also adds the result to the residual; ``materialize`` does it alone."""
    __slots__ = ("delta", "bias", "kind", "weight", "eps")

    def __init__(self, delta, bias, kind, weight, eps):
        self.delta, self.bias, self.kind, self.weight, self.eps = delta, bias, kind, weight, float(eps)

    def materialize(self) -> torch.Tensor:
        """The normed branch output as a tensor of its own, for a norm that cannot take it in."""
        zero = torch.zeros(self.delta.shape, dtype=torch.float32, device=self.delta.device)
        add_norm(zero, self, None, None, 0.0, self.delta.dtype)
        return zero.to(self.delta.dtype)


def add_norm(resid: torch.Tensor, pending, kind: Optional[str], weight: Optional[torch.Tensor], eps: float,
             out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``resid += post(pending)`` in float32 (in place unless ``rows`` selects), then the norm
    ``kind`` ("layer": (v - mean) / sqrt(var + eps), "rms": v / sqrt(mean(v^2) + eps)) of the sum
    times ``weight``.  ``pending``: None, a tensor [T, H] that is added as it is, or a
    :class:`PostNormed`.  ``kind`` None: only the residual is brought up to date; "copy": the sum itself comes back
    in ``out_dtype`` (for a sublayer that reads the stream without a norm in front)."""
    _need_cuda(resid)
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    T, H = resid.shape
    delta = bias = post_w = None
    post_kind, post_eps = 0, 0.0
    if isinstance(pending, PostNormed):
        delta, bias, post_w = pending.delta, pending.bias, pending.weight
        post_kind, post_eps = NORM_KINDS[pending.kind], pending.eps
    elif pending is not None:
        delta = pending
    if delta is not None:
        assert delta.shape == resid.shape and delta.is_contiguous() and delta.dtype in (torch.float32, torch.bfloat16)
        assert delta.dtype == out_dtype
    n = T if rows is None else rows.numel()
    out = new((n, H), out_dtype, resid.device) if kind is not None else None
    rc = lib("rowwise").kvb_add_norm(_p(resid), _p(delta), _p(bias), _p(post_w), c_int(post_kind), c_float(post_eps),
                                     _p(weight), c_int(NORM_KINDS[kind]), c_float(eps), _p(out), _p(rows), c_int(n),
                                     c_int(H), c_int(dtype_code(out_dtype)), _stream())
    _check(rc, "add_norm")
    return out


ACT_KINDS = {"silu": 0, "gelu_tanh": 1}


def bias_act_mul(gate_up: torch.Tensor, bias: Optional[torch.Tensor], act: str) -> torch.Tensor:
    """``act(gate + b_gate) * (up + b_up)`` for rows that hold [gate | up]; ``bias`` float32 [2 I] or None."""
    _need_cuda(gate_up)
    assert gate_up.is_contiguous() and (bias is None or (bias.dtype == torch.float32 and bias.numel() == gate_up.shape[1]))
    T, two_i = gate_up.shape
    out = new((T, two_i // 2), gate_up.dtype, gate_up.device)
    rc = lib("rowwise").kvb_bias_act_mul(_p(gate_up), _p(bias), _p(out), c_int(T), c_int(two_i // 2),
                                         c_int(ACT_KINDS[act]), c_int(dtype_code(gate_up.dtype)), _stream())
    _check(rc, "bias_act_mul")
    return out


def scale_softcap(x: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
    """``x <- cap * tanh(x * scale / cap)`` in place on a float32 tensor (``cap`` 0: only the factor)."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    rc = lib("rowwise").kvb_scale_softcap(_p(x), ctypes.c_size_t(x.numel()), c_float(scale), c_float(cap), _stream())
    _check(rc, "scale_softcap")
    return x


def tanh_slice(x: torch.Tensor, first: int, n: int) -> torch.Tensor:
    """``tanh(x[:, first:first + n])`` as a dense tensor."""
    _need_cuda(x)
    assert x.stride(1) == 1
    out = new((x.shape[0], n), x.dtype, x.device)
    rc = lib("rowwise").kvb_tanh_slice(c_void_p(x.data_ptr() + first * x.element_size()), c_int(x.stride(0)), _p(out),
                                       c_int(x.shape[0]), c_int(n), c_int(dtype_code(x.dtype)), _stream())
    _check(rc, "tanh_slice")
    return out


class PendingSum:
    """What still has to join the float32 residual stream before the next norm reads it: up to two
    branch outputs ``deltas`` [T, H] of the compute type (a layer whose mixer and feed-forward read
    the same normed input hands on both), float32 ``rows`` [T, H] (the embedding's output entering
    the stream again at the start of a repeated run of layers) and a float32 ``vector`` [H] added to
    every row.  :func:`join_norm` adds them all and norms the sum in one kernel."""
    __slots__ = ("deltas", "rows", "vector")

    def __init__(self, deltas=(), rows=None, vector=None):
        self.deltas = tuple(d for d in deltas if d is not None)
        assert len(self.deltas) <= 2
        self.rows, self.vector = rows, vector

    def plus(self, rows=None, vector=None) -> "PendingSum":
        assert (rows is None or self.rows is None) and (vector is None or self.vector is None)
        return PendingSum(self.deltas, self.rows if rows is None else rows, self.vector if vector is None else vector)


def join_norm(resid: torch.Tensor, pending: Optional[PendingSum], kind: Optional[str], weight: Optional[torch.Tensor],
              eps: float, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
              compute_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """``resid += sum of pending`` in float32 (in place unless ``rows`` selects), then the norm ``kind``
    ("rms", "layer" or None for no output) of the sum times ``weight``.  ``out_dtype`` may be float32
    whatever the type of the pending branch outputs (``compute_dtype`` names that type when there
    are none)."""
    _need_cuda(resid)
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    T, H = resid.shape
    deltas = pending.deltas if pending is not None else ()
    e = pending.rows if pending is not None else None
    vec = pending.vector if pending is not None else None
    dt = deltas[0].dtype if deltas else (compute_dtype or out_dtype)
    for d in deltas:
        assert d.shape == resid.shape and d.is_contiguous() and d.dtype == dt
    assert e is None or (e.dtype == torch.float32 and e.shape == resid.shape and e.is_contiguous())
    assert vec is None or (vec.dtype == torch.float32 and vec.numel() == H and vec.is_contiguous())
    assert out_dtype in (dt, torch.float32)
    n = T if rows is None else rows.numel()
    out = new((n, H), out_dtype, resid.device) if kind is not None else None
    rc = lib("rowwise").kvb_join_norm(_p(resid), _p(deltas[0] if deltas else None), _p(deltas[1] if len(deltas) > 1 else None),
                                      _p(e), _p(vec), _p(weight), c_int(NORM_KINDS[kind]), c_float(eps), _p(out),
                                      c_int(1 if out_dtype == torch.float32 else 0), _p(rows), c_int(n), c_int(H),
                                      c_int(dtype_code(dt)), _stream())
    _check(rc, "join_norm")
    return out


# ------------------------------------------------------------------ mixers with a matrix state (delta-rule family)

class _DeltaArgs(ctypes.Structure):
    _fields_ = [("r", c_void_p), ("ld_r", c_int), ("k", c_void_p), ("ld_k", c_int), ("v", c_void_p), ("ld_v", c_int),
                ("gate", c_void_p), ("ld_gate", c_int), ("decay", c_void_p), ("ld_decay", c_int),
                ("aux", c_void_p), ("ld_aux", c_int), ("decay_bias", c_void_p), ("aux_bias", c_void_p),
                ("head_rate", c_void_p), ("norm_w", c_void_p), ("norm_per_head", c_int), ("state", c_void_p),
                ("slot_stride", c_longlong), ("out", c_void_p), ("ld_out", c_int), ("q_start", c_void_p),
                ("req_start", c_void_p), ("slots", c_void_p), ("H", c_int), ("G", c_int), ("Dk", c_int), ("Dv", c_int),
                ("eps", c_float), ("o_raw", c_void_p), ("decay_per_head", c_int), ("gate_silu", c_int)]


_key_pad: Dict[int, int] = {}


def delta_key_pad(dk: int) -> int:
    """Floats per column of a head's state for key size ``dk`` (the kernel pads it), 0 if refused."""
    if dk not in _key_pad:
        _key_pad[dk] = int(lib("delta_rule").kvb_delta_key_pad(c_int(int(dk))))
    return _key_pad[dk]


def _at(t: torch.Tensor, col: int) -> int:
    return t.data_ptr() + col * t.element_size()


def delta_scan(mode: str, batch, state: torch.Tensor, r, k, v, gate, decay, aux, decay_bias, aux_bias, head_rate,
               norm_w, norm_per_head: bool, heads: int, key_heads: int, dk: int, dv: int, eps: float,
               decay_per_head: bool = False, gate_act: str = "sigmoid") -> torch.Tensor:
    """One step of a delta-rule mixer for every request of the batch: walks each request's new
    tokens in order from the state in its slot (zero for a request that starts at position 0)
    and leaves the new state there.  ``r, k, v, gate, decay, aux``: (tensor, first column) pairs
    naming where each projection lies in a [T, *] tensor of the compute type.  ``state``:
    float32 [slots, >= heads * dv * delta_key_pad(dk)], a request's slot row starting with the
    matrix states.  ``mode``: "general" or "gated" (see csrc/kernels/delta_rule.cu).
    ``decay_per_head`` ("gated"): ``decay`` is [T, heads] and ``decay_bias`` [heads], one decay for all key
    channels of a head.  ``gate_act``: "sigmoid" or "silu", the function applied to the output gate.
    Returns the gated, normed read-out [T, heads * dv]."""
    x0 = r[0]
    _need_cuda(x0, state)
    T = x0.shape[0]
    assert state.dtype == torch.float32 and state.stride(-1) == 1
    out = new((T, heads * dv), x0.dtype, x0.device)
    a = _DeltaArgs()
    for name, (t, col) in (("r", r), ("k", k), ("v", v), ("gate", gate), ("decay", decay), ("aux", aux)):
        assert t.dtype == x0.dtype and t.stride(1) == 1 and t.shape[0] == T
        setattr(a, name, _at(t, col))
        setattr(a, "ld_" + name, t.stride(0))
    for name, t in (("decay_bias", decay_bias), ("aux_bias", aux_bias), ("head_rate", head_rate), ("norm_w", norm_w)):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
        setattr(a, name, 0 if t is None else t.data_ptr())
    a.norm_per_head = 1 if norm_per_head else 0
    a.state, a.slot_stride = state.data_ptr(), state.stride(0)
    a.out, a.ld_out = out.data_ptr(), out.stride(0)
    a.q_start, a.req_start, a.slots = batch.q_start.data_ptr(), batch.req_start.data_ptr(), batch.slots.data_ptr()
    a.H, a.G, a.Dk, a.Dv, a.eps = heads, key_heads, dk, dv, eps
    a.o_raw = new((T, heads * dv), torch.float32, x0.device).data_ptr()
    a.decay_per_head = 1 if decay_per_head else 0
    a.gate_silu = {"sigmoid": 0, "silu": 1}[gate_act]
    rc = lib("delta_rule").kvb_delta_scan(ctypes.byref(a), c_int({"general": 0, "gated": 1}[mode]),
                                          c_int(batch.num_reqs), c_int(T), c_int(int(getattr(batch, "max_q_len", 0) or 0)),
                                          c_int(dtype_code(x0.dtype)), _stream())
    _check(rc, "delta_scan")
    global launch_count
    launch_count += 1       # the scan and the read-outs' norm
    choices["delta_scan_" + mode] += 1
    return out


class _AppendArgs(ctypes.Structure):
    _fields_ = [("pages", c_void_p), ("block_table", c_void_p), ("max_pages", c_int), ("page_size", c_int),
                ("num_pages", c_int), ("k_off", c_int), ("v_off", c_int), ("kv_heads", c_int), ("Dk", c_int), ("Dv", c_int),
                ("status", c_void_p)]


def conv_can_append(x: torch.Tensor, first: int, channels: int, k_off: int, v_off: int, dk: int, dv: int) -> bool:
    """Whether :func:`conv_silu` can write keys and values into their pages itself: every run of channels starts and
    ends on a 16-byte boundary."""
    vec = 16 // x.element_size()
    return (channels % vec == 0 and x.stride(0) % vec == 0 and _at(x, first) % 16 == 0 and dk % vec == 0 and dv % vec == 0
            and k_off % vec == 0 and v_off % vec == 0)


def conv_silu(x: torch.Tensor, first: int, channels: int, w: torch.Tensor, tails: Optional[torch.Tensor],
              batch, act: str = "silu", append=None, in_bias: Optional[torch.Tensor] = None,
              out_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu`` (``act`` "none": nothing) of a short causal convolution over time per channel of ``x[:, first:first + channels]``.
    ``w`` float32 [channels, taps], last column for the token itself.  ``tails``: float32
    [slots, >= (taps - 1) * channels], a view whose row r starts with request slot r's last
    ``taps - 1`` inputs; it is read for the inputs in front of the step's tokens and brought up to date.
    ``append``: (pages, block_table, k_off, v_off, kv_heads, dk, dv): the results from channel ``k_off`` on are
    ``kv_heads`` keys of ``dk``, those from ``v_off`` on values of ``dv``, and they are also written into the requests'
    pages [num_pages, kv_heads, page_size, dk + dv] (only when :func:`conv_can_append` says so).
    ``in_bias`` (float32 [channels]) joins every input before it is weighed, except the zeros that stand before a
    sequence's start; ``out_bias`` (float32 [channels]) joins the sum before the activation."""
    _need_cuda(x, w)
    taps = w.shape[1]
    for b in (in_bias, out_bias):
        assert b is None or (b.dtype == torch.float32 and b.is_contiguous() and b.numel() == channels)
    assert w.dtype == torch.float32 and w.is_contiguous() and x.stride(1) == 1
    assert taps == 1 or (tails is not None and tails.dtype == torch.float32 and tails.stride(-1) == 1)
    out = new((x.shape[0], channels), x.dtype, x.device)
    ap = None
    if append is not None:
        pages, table, k_off, v_off, kv_heads, dk, dv = append
        assert pages.is_contiguous() and pages.dtype == x.dtype and tuple(pages.shape[1:]) == (kv_heads, pages.shape[2], dk + dv)
        ap = _AppendArgs(pages.data_ptr(), table.data_ptr(), table.shape[1], pages.shape[2], pages.shape[0], k_off, v_off,
                         kv_heads, dk, dv, batch.status.data_ptr())
    rc = lib("delta_rule").kvb_conv_silu(
        c_void_p(_at(x, first)), c_int(x.stride(0)), _p(w), c_int(taps), _p(tails),
        c_longlong(0 if tails is None else tails.stride(0)), _p(out), c_int(channels), c_int(x.shape[0]),
        c_int(batch.num_reqs), _p(batch.positions), _p(batch.token_req), _p(batch.q_start), _p(batch.req_start),
        _p(batch.ctx_len), _p(batch.slots), c_int({"silu": 0, "none": 1}[act]),
        ctypes.byref(ap) if ap is not None else None, _p(in_bias), _p(out_bias), c_int(dtype_code(x.dtype)), _stream())
    _check(rc, "conv_silu")
    global launch_count
    launch_count += 1 if taps > 1 else 0   # the convolution and the tails' update
    return out


# ------------------------------------------------------------------ attention over a cached latent

def latent_prep(d_in: torch.Tensor, q_rank: int, kv_off: int, rank: int, rot: int, rdims: int, wq, wkv, eps: float,
                cos, sin, batch, block_table, pages: torch.Tensor, write: bool) -> torch.Tensor:
    """RMS norm of the query latent (returned, [T, q_rank]); RMS norm of the key/value latent and
    interleaved rotary encoding of the shared key part, both written to the token's cache row."""
    _need_cuda(d_in, pages)
    assert d_in.stride(1) == 1 and pages.is_contiguous() and pages.dtype == d_in.dtype
    assert pages.shape[1] == 1 and pages.shape[3] == rank + rot
    T = d_in.shape[0]
    cq = new((T, q_rank), d_in.dtype, d_in.device)
    rc = lib("latent_attention").kvb_latent_prep(
        _p(d_in), c_int(d_in.stride(0)), c_int(q_rank), c_int(kv_off), c_int(rank), c_int(rot), c_int(rdims), _p(wq),
        _p(wkv), c_float(eps), _p(cos), _p(sin), c_int(0 if cos is None else cos.shape[0]), _p(batch.positions),
        _p(batch.token_req), _p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[2]), c_int(pages.shape[0]),
        _p(cq), _p(pages), c_int(1 if write else 0), c_int(T), c_int(dtype_code(d_in.dtype)), _p(batch.status), _stream())
    _check(rc, "latent_prep")
    return cq


HEAD_GEMM_LIBRARY_MIN_ROWS = int(os.environ.get('KVB200_HEAD_GEMM_LIBRARY_MIN_ROWS', '128'))


def head_gemm(x: torch.Tensor, first: int, head_stride: int, w: torch.Tensor) -> torch.Tensor:
    """A product per head: ``out[t, h, :] = w[h] @ x[t, first + h * head_stride : ... + K]`` with
    ``w`` [H, N, K].  float32, and bfloat16 steps of fewer than 128 rows: this package's FMA kernel, float32
    sums in ascending k; bfloat16 with more rows: the library's batched product.  Returns [T, H * N]."""
    _need_cuda(x, w)
    H, N, K = w.shape
    assert w.is_contiguous() and w.dtype == x.dtype and x.stride(1) == 1
    out = new((x.shape[0], H * N), x.dtype, x.device)
    T = x.shape[0]
    if x.dtype == torch.bfloat16 and T >= HEAD_GEMM_LIBRARY_MIN_ROWS:
        # many rows: the library's batched product (tensor cores, float32 sums), as the other products of such steps
        xv = torch.as_strided(x, (H, T, K), (head_stride, x.stride(0), 1), x.storage_offset() + first)
        tmp = new((H, T, N), x.dtype, x.device)
        torch.bmm(xv, w.transpose(1, 2), out=tmp)
        out.view(T, H, N).copy_(tmp.permute(1, 0, 2))
        if _marks is not None:
            _mark("head_gemm_library")
        choices["head_gemm_library"] += 1
        return out
    rc = lib("latent_attention").kvb_head_gemm(c_void_p(_at(x, first)), c_int(x.stride(0)), c_int(head_stride), _p(w),
                                               _p(out), c_int(out.stride(0)), c_int(N), c_int(x.shape[0]), c_int(N),
                                               c_int(K), c_int(H), c_int(dtype_code(x.dtype)), _stream())
    _check(rc, "head_gemm")
    return out


LATENT_TC = os.environ.get('KVB200_LATENT_TC', '1') != '0'
_latent_tc_ok: Dict[tuple, bool] = {}
_latent_tpt: Dict[int, int] = {}


def latent_attention_tc_supported(rank: int, rot: int) -> bool:
    """Whether the tensor-core form of the latent attention takes these sizes (bfloat16 only)."""
    key = (int(rank), int(rot))
    if key not in _latent_tc_ok:
        _latent_tc_ok[key] = bool(lib("latent_attention").kvb_latent_attention_tc_supported(c_int(key[0]), c_int(key[1])))
    return _latent_tc_ok[key]


def latent_tokens_per_tile(heads: int) -> int:
    """Tokens in one tile of the tensor-core latent attention (a tile holds up to 64 (token, head) rows)."""
    if heads not in _latent_tpt:
        _latent_tpt[heads] = int(lib("latent_attention").kvb_latent_attention_tc_tokens_per_tile(c_int(int(heads))))
    return _latent_tpt[heads]


def _query_tiles(batch, nt: int) -> torch.Tensor:
    """[n, 4] int32 tiles (request row, first token row, tokens, 0) of at most ``nt`` consecutive tokens of one
    request: the ones the batch was laid out with, or built here for a batch that was made without them."""
    ready = (getattr(batch, "tiles", None) or {}).get(nt)
    if ready is not None:
        return ready
    cache = batch.host.setdefault("query_tiles", {})
    got = cache.get(nt)
    if got is None:
        import numpy as np
        qs = batch.host["q_start"]
        rows = []
        for r in range(batch.num_reqs):
            a, b = int(qs[r]), int(qs[r + 1])
            starts = np.arange(a, b, nt, dtype=np.int32)
            tile = np.zeros((len(starts), 4), dtype=np.int32)
            tile[:, 0], tile[:, 1], tile[:, 2] = r, starts, np.minimum(nt, b - starts)
            rows.append(tile)
        host = torch.from_numpy(np.concatenate(rows)).pin_memory()
        got = host.to(batch.token_ids.device, non_blocking=True)
        cache[nt], cache[("host", nt)] = got, host      # the pinned source lives until the step is over
    return got


def latent_attention(q_abs: torch.Tensor, q: torch.Tensor, rot_first: int, q_head_stride: int, cos, sin, rdims: int,
                     pages: torch.Tensor, block_table, batch, sink: torch.Tensor, scale: float, heads: int,
                     rank: int, rot: int) -> torch.Tensor:
    """Causal attention of every token over its request's cached rows [latent | rotated part],
    all heads sharing the rows; softmax with a sink per head.  ``q_abs`` [T, heads * rank]: the
    queries' plain parts moved into the latent's space; ``q`` holds head h's part to be rotated at
    ``rot_first + h * q_head_stride``.  Returns the attended latents [T, heads * rank]."""
    _need_cuda(q_abs, pages)
    assert q_abs.is_contiguous() and q.stride(1) == 1 and pages.is_contiguous() and sink.dtype == torch.float32
    T = q_abs.shape[0]
    out = new((T, heads * rank), q_abs.dtype, q_abs.device)
    if q_abs.dtype == torch.bfloat16 and LATENT_TC and latent_attention_tc_supported(rank, rot):
        nt = latent_tokens_per_tile(heads)
        if batch.decode_only:
            tiles, n_tiles = None, batch.num_reqs           # one tile per request, found in the kernel
        else:
            tiles = _query_tiles(batch, nt)
            n_tiles = tiles.shape[0]
        rc = lib("latent_attention").kvb_latent_attention_tc(
            _p(q_abs), c_int(q_abs.stride(0)), c_int(rank), c_void_p(_at(q, rot_first)), c_int(q.stride(0)),
            c_int(q_head_stride), _p(cos), _p(sin), c_int(0 if cos is None else cos.shape[0]), c_int(rdims), _p(pages),
            _p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[2]), c_int(pages.shape[0]),
            _p(batch.positions), _p(batch.q_start), _p(tiles), c_int(n_tiles), _p(sink), c_float(scale), _p(out),
            c_int(out.stride(0)), c_int(rank), c_int(heads), c_int(rank), c_int(rot), _p(batch.status), _stream())
        _check(rc, "latent_attention_tc")
        choices["latent_attention_tc"] += 1
        return out
    rc = lib("latent_attention").kvb_latent_attention(
        _p(q_abs), c_int(q_abs.stride(0)), c_int(rank), c_void_p(_at(q, rot_first)), c_int(q.stride(0)),
        c_int(q_head_stride), _p(cos), _p(sin), c_int(0 if cos is None else cos.shape[0]), c_int(rdims), _p(pages),
        _p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[2]), c_int(pages.shape[0]), _p(batch.positions),
        _p(batch.token_req), _p(sink), c_float(scale), _p(out), c_int(out.stride(0)), c_int(rank), c_int(T),
        c_int(heads), c_int(rank), c_int(rot), c_int(dtype_code(q_abs.dtype)), _p(batch.status), _stream())
    _check(rc, "latent_attention")
    choices["latent_attention"] += 1
    return out


# ------------------------------------------------------------------ attention

def paged_attention_generic(qkv, k_pages, v_pages, block_table, positions, token_req, nq, nkv, d,
                            scale, window, status) -> torch.Tensor:
    """Attention of every token in ``qkv`` (q part) over its request's cached keys."""
    _need_cuda(qkv, k_pages)
    T = qkv.shape[0]
    out = new((T, nq * d), qkv.dtype, qkv.device)
    page_size = k_pages.shape[2]
    rc = lib("attention").kvb_paged_attention_generic(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), _p(block_table),
        c_int(block_table.shape[1]), c_int(page_size), c_int(k_pages.shape[0]), _p(positions),
        _p(token_req), _p(out), c_int(T), c_int(nq), c_int(nkv), c_int(d), c_float(scale),
        c_int(int(window or 0)), c_int(dtype_code(qkv.dtype)), _p(status), _stream())
    _check(rc, "paged_attention_generic")
    choices["paged_attention_generic"] += 1
    return out


def kv_rows_append(src: torch.Tensor, k_off: int, v_off: int, pages: torch.Tensor, block_table, batch,
                   kv_heads: int, dk: int, dv: int) -> None:
    """Writes the step's keys (``src[:, k_off : k_off + kv_heads * dk]``) and values (from ``v_off``) into the
    requests' pages, whose rows hold a token's key and value side by side:
    ``pages`` [num_pages, kv_heads, page_size, dk + dv]."""
    _need_cuda(src, pages)
    assert src.stride(1) == 1 and pages.is_contiguous() and pages.dtype == src.dtype
    assert tuple(pages.shape[1:]) == (kv_heads, pages.shape[2], dk + dv)
    rc = lib("window_attention").kvb_kv_rows_append(
        _p(src), c_int(src.stride(0)), c_int(k_off), c_int(v_off), _p(pages), _p(block_table), c_int(block_table.shape[1]),
        c_int(pages.shape[2]), c_int(pages.shape[0]), _p(batch.positions), _p(batch.token_req), c_int(src.shape[0]),
        c_int(kv_heads), c_int(dk), c_int(dv), c_int(dtype_code(src.dtype)), _p(batch.status), _stream())
    _check(rc, "kv_rows_append")


def window_attention(q: torch.Tensor, q_off: int, pages: torch.Tensor, block_table, batch, heads: int, kv_heads: int,
                     dk: int, dv: int, scale: float, window: int, keep_first: int, one_more: bool,
                     head_scale: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None,
                     softcap: float = 0.0, out_scale: float = 1.0, sinks: Optional[torch.Tensor] = None,
                     chunk: int = 0, gate=None) -> torch.Tensor:
    """Attention of every token (queries at ``q[:, q_off : q_off + heads * dk]``) over its request's cached
    rows [key | value]: query i sees key j when ``j <= i and (i - j < window or j < keep_first)`` (``window``
    0: every key up to i); ``one_more``: the softmax's denominator is ``1 + sum exp(s)``.  Positions do
    not enter the scores unless ``slopes`` is given.  On its way to the softmax a score ``(q . k) * scale`` is
    multiplied by ``head_scale[h]`` (float32 [heads]), capped as ``softcap * tanh(s / softcap)`` (``softcap`` 0: not),
    and lowered by ``slopes[h] * (i - j)`` (float32 [heads]); the result is multiplied by ``out_scale``.
    ``sinks`` (float32 [heads]): ``exp(sinks[h])`` joins the softmax's denominator once, without a value.  ``chunk`` > 0:
    query i sees key j <= i only when ``i // chunk == j // chunk``, blocks counted from the sequence's start.
    ``gate``: (tensor, first column) of rows in the activations' type by whose sigmoid the result is multiplied.
    Returns [T, heads * dv]."""
    _need_cuda(q, pages)
    assert q.stride(1) == 1 and pages.is_contiguous() and pages.dtype == q.dtype
    T = q.shape[0]
    out = new((T, heads * dv), q.dtype, q.device)
    if sinks is not None or chunk or gate is not None:
        for v in (head_scale, slopes, sinks):
            assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == heads)
        gate_at, gate_ld = 0, 0
        if gate is not None:
            gt, gcol = gate
            assert gt.dtype == q.dtype and gt.stride(1) == 1 and gt.shape[0] == T and gt.shape[1] >= gcol + heads * dv
            gate_at, gate_ld = _at(gt, gcol), gt.stride(0)
        rc = lib("window_attention").kvb_window_attention_masked(
            c_void_p(_at(q, q_off)), c_int(q.stride(0)), _p(pages), _p(block_table), c_int(block_table.shape[1]),
            c_int(pages.shape[2]), c_int(pages.shape[0]), _p(batch.positions), _p(batch.token_req), _p(out), c_int(T),
            c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv), c_float(scale), c_int(int(window or 0)),
            c_int(int(keep_first or 0)), c_int(1 if one_more else 0), _p(head_scale), _p(slopes), c_float(float(softcap or 0.0)),
            c_float(float(out_scale)), _p(sinks), c_int(int(chunk or 0)), c_void_p(gate_at), c_int(gate_ld),
            c_int(dtype_code(q.dtype)), _p(batch.status), _stream())
        _check(rc, "window_attention")
        choices["window_attention"] += 1
        choices["window_attention_masked"] += 1
        return out
    if head_scale is not None or slopes is not None or softcap or out_scale != 1.0:
        for v in (head_scale, slopes):
            assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == heads)
        rc = lib("window_attention").kvb_window_attention_shaped(
            c_void_p(_at(q, q_off)), c_int(q.stride(0)), _p(pages), _p(block_table), c_int(block_table.shape[1]),
            c_int(pages.shape[2]), c_int(pages.shape[0]), _p(batch.positions), _p(batch.token_req), _p(out), c_int(T),
            c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv), c_float(scale), c_int(int(window or 0)),
            c_int(int(keep_first or 0)), c_int(1 if one_more else 0), _p(head_scale), _p(slopes), c_float(float(softcap or 0.0)),
            c_float(float(out_scale)), c_int(dtype_code(q.dtype)), _p(batch.status), _stream())
        _check(rc, "window_attention")
        choices["window_attention"] += 1
        choices["window_attention_shaped"] += 1
        return out
    rc = lib("window_attention").kvb_window_attention(
        c_void_p(_at(q, q_off)), c_int(q.stride(0)), _p(pages), _p(block_table), c_int(block_table.shape[1]),
        c_int(pages.shape[2]), c_int(pages.shape[0]), _p(batch.positions), _p(batch.token_req), _p(out), c_int(T),
        c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv), c_float(scale), c_int(int(window or 0)),
        c_int(int(keep_first or 0)), c_int(1 if one_more else 0), c_int(dtype_code(q.dtype)), _p(batch.status), _stream())
    _check(rc, "window_attention")
    choices["window_attention"] += 1
    return out


def flash_attention_rows_supported(dk: int, dv: int, group: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core form of :func:`window_attention` takes these sizes: bfloat16, key and value
    size equal and 64 or 128, pages of a power of two."""
    return dtype == torch.bfloat16 and dk == dv and flash_attention_supported(dk, group, page_size)


# Which form the tensor-core attention over [key | value] rows takes: None: chosen from the step's size as for the
# rotary attention (128-row tiles on tcgen05 when they fill the GPU, else 64-row tiles on mma.sync); 0, 1 or 3 forces
# 64-row tiles, 128-row tiles on mma.sync, or the tcgen05 form with roles.
FLASH_ROWS_WIDE = {"": None, "0": 0, "1": 1, "3": 3}[os.environ.get('KVB200_FLASH_ROWS_WIDE', '')]


def flash_attention_rows(q: torch.Tensor, pages: torch.Tensor, block_table, batch, heads: int, kv_heads: int, d: int,
                         scale: float, window: int, keep_first: int, one_more: bool,
                         wide: Optional[int] = None) -> torch.Tensor:
    """:func:`window_attention` on tensor cores for steps with runs of query tokens (bfloat16, key and value
    size ``d`` both): tiles of 64 or 128 (token, head of a group) rows against tiles of 64 keys, the tiles that
    hold kept first keys in front of the window's own.  Queries at ``q[:, : heads * d]``.  ``wide``: 0: 64-row tiles
    (mma.sync); 1: 128-row tiles (mma.sync); 3: 128-row tiles on tcgen05 with roles (pages of at least 8 rows);
    None: chosen from the step's size."""
    _need_cuda(q, pages)
    assert q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16 and pages.is_contiguous() and q.stride(1) == 1
    assert tuple(pages.shape[1:]) == (kv_heads, pages.shape[2], 2 * d)
    T = q.shape[0]
    group = heads // kv_heads
    if wide is None:
        wide = FLASH_ROWS_WIDE
    if wide is None:
        wide = FLASH_WIDE and (T // flash_tokens_per_tile(group, True)) * kv_heads >= (2 if d == 64 else 1) * sm_count(q.device)
        if wide and FLASH_TC and FLASH_TC_ROLES:
            wide = 3
    wide = int(wide)
    if wide == 3 and not (pages.shape[2] >= 8 and q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0):
        wide = 1
    tiles = flash_tiles(batch, group, bool(wide))
    out = new((T, heads * d), q.dtype, q.device)
    rc = lib("flash_attention").kvb_paged_flash_attention_rows(
        _p(q), c_int(q.stride(0)), _p(pages), _p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[2]),
        c_int(pages.shape[0]), _p(batch.positions), _p(tiles), c_int(tiles.shape[0]), c_int(wide), _p(out),
        c_int(heads), c_int(kv_heads), c_int(d), c_float(scale), c_int(int(window or 0)), c_int(int(keep_first or 0)),
        c_int(1 if one_more else 0), _p(batch.status), _stream())
    _check(rc, "flash_attention_rows")
    choices["flash_attention_rows"] += 1
    choices[f"flash_attention_rows_{wide}"] += 1
    return out


def flash_attention_rows_masked_wanted(batch, heads: int, kv_heads: int, dk: int, dv: int, page_size: int,
                                       dtype: torch.dtype, q: Optional[torch.Tensor] = None) -> bool:
    """Whether a step's attention over blocks of positions goes to the tcgen05 kernel with roles: bfloat16, key and value
    size both 64 or both 128, pages of at least 8 rows, and 128-row tiles enough to fill the GPU (twice over at head
    size 64), as for the other designs' prompt portions."""
    if not (dtype == torch.bfloat16 and dk == dv and dk in (64, 128) and page_size >= 8 and FLASH_WIDE and FLASH_TC
            and FLASH_TC_ROLES and FLASH_ROWS_WIDE in (None, 3)):
        return False
    group = heads // kv_heads
    if not flash_attention_supported(dk, group, page_size):
        return False
    if q is not None and not (q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0):
        return False
    if FLASH_ROWS_WIDE == 3:
        return True
    return (batch.num_tokens // flash_tokens_per_tile(group, True)) * kv_heads >= (2 if dk == 64 else 1) * sm_count(batch.token_ids.device)


def flash_attention_rows_masked(q: torch.Tensor, pages: torch.Tensor, block_table, batch, heads: int, kv_heads: int,
                                d: int, scale: float, chunk: int = 0, sinks: Optional[torch.Tensor] = None,
                                softcap: float = 0.0, gate=None) -> torch.Tensor:
    """:func:`window_attention` with a mask by blocks of ``chunk`` positions, ``sinks``, a ``softcap`` and a ``gate`` (as
    there) on the tcgen05 kernel with roles: bfloat16 steps with runs of query tokens, key and value size ``d`` both
    (64 or 128), 128-row tiles, pages of at least 8 rows.  Queries at ``q[:, : heads * d]``.  Returns [T, heads * d]."""
    _need_cuda(q, pages)
    assert q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16 and pages.is_contiguous() and q.stride(1) == 1
    assert tuple(pages.shape[1:]) == (kv_heads, pages.shape[2], 2 * d)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == heads)
    T = q.shape[0]
    gate_at, gate_ld = 0, 0
    if gate is not None:
        gt, gcol = gate
        assert gt.dtype == q.dtype and gt.stride(1) == 1 and gt.shape[0] == T and gt.shape[1] >= gcol + heads * d
        gate_at, gate_ld = _at(gt, gcol), gt.stride(0)
    tiles = flash_tiles(batch, heads // kv_heads, True)
    out = new((T, heads * d), q.dtype, q.device)
    rc = lib("flash_attention").kvb_paged_flash_attention_rows_masked(
        _p(q), c_int(q.stride(0)), _p(pages), _p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[2]),
        c_int(pages.shape[0]), _p(batch.positions), _p(tiles), c_int(tiles.shape[0]), _p(out), c_int(heads), c_int(kv_heads),
        c_int(d), c_float(scale), c_int(int(chunk or 0)), _p(sinks), c_float(float(softcap or 0.0)), c_void_p(gate_at),
        c_int(gate_ld), _p(batch.status), _stream())
    _check(rc, "flash_attention_rows")
    choices["flash_attention_rows"] += 1
    choices["flash_attention_rows_masked"] += 1
    return out


def qk_norm_append(p: torch.Tensor, first: int, k_off: int, v_off: int, bq, bk, bv, qw, kw, eps: float, pages: torch.Tensor,
                   block_table, batch, heads: int, kv_heads: int, dk: int, dv: int, write: bool = True) -> torch.Tensor:
    """What lies between the q|k|v product and an attention over [key | value] rows: the biases (float32, each may
    be None) join their projections, every query and key head is divided by its root mean square (eps inside the
    root) and multiplied by a weight of ``dk`` shared by the heads (``qw``, ``kw``; None: no norm), the keys and
    values go into the requests' pages.  ``p`` [T, *]: queries from column ``first``, keys ``k_off`` columns further,
    values ``v_off`` columns further.  Returns the queries [T, heads * dk]."""
    _need_cuda(p, pages)
    assert p.stride(1) == 1 and pages.is_contiguous() and pages.dtype == p.dtype
    assert tuple(pages.shape[1:]) == (kv_heads, pages.shape[2], dk + dv)
    for v, n in ((bq, heads * dk), (bk, kv_heads * dk), (bv, kv_heads * dv), (qw, dk), (kw, dk)):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == n)
    T = p.shape[0]
    q = new((T, heads * dk), p.dtype, p.device)
    rc = lib("window_attention").kvb_qk_norm_append(
        c_void_p(_at(p, first)), c_int(p.stride(0)), c_int(k_off), c_int(v_off), _p(bq), _p(bk), _p(bv), _p(qw), _p(kw),
        c_float(eps), _p(q),
        _p(pages), _p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[2]), c_int(pages.shape[0]),
        _p(batch.positions), _p(batch.token_req), c_int(T), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv),
        c_int(1 if write else 0), c_int(dtype_code(p.dtype)), _p(batch.status), _stream())
    _check(rc, "qk_norm_append")
    return q


class _QkRotArgs(ctypes.Structure):
    _fields_ = [("src", c_void_p), ("ld", c_int), ("k_off", c_int), ("v_off", c_int), ("bq", c_void_p), ("bk", c_void_p),
                ("bv", c_void_p), ("qw", c_void_p), ("kw", c_void_p), ("eps", c_float), ("cos_t", c_void_p),
                ("sin_t", c_void_p), ("table_len", c_int), ("rot", c_int), ("layout", c_int), ("q_out", c_void_p),
                ("pages", c_void_p), ("block_table", c_void_p), ("max_pages", c_int), ("page_size", c_int),
                ("num_pages", c_int), ("positions", c_void_p), ("token_req", c_void_p), ("nq", c_int), ("nkv", c_int),
                ("Dk", c_int), ("Dv", c_int), ("write", c_int), ("status", c_void_p)]


ROTARY_LAYOUTS = {"half": 0, "pairs": 1}


def qk_rot_append(p: torch.Tensor, first: int, k_off: int, v_off: int, bq, bk, bv, qw, kw, eps: float, cos, sin,
                  rot: int, layout: str, pages: torch.Tensor, block_table, batch, heads: int, kv_heads: int, dk: int,
                  dv: int, write: bool = True) -> torch.Tensor:
    """From a product's rows to queries and cached rows.  ``p[:, first:]`` holds a token's ``heads`` queries of
    ``dk``, its ``kv_heads`` keys ``k_off`` columns further and its values ``v_off`` columns further.  Each gets its
    bias (float32 or None); with ``qw`` (float32 [heads * dk]) all queries of a token together are divided by their
    root mean square (``eps`` inside the root) and multiplied by ``qw``, likewise the keys with ``kw``; then the
    first ``rot`` channels of every query and key head turn by the token's position (``cos``, ``sin``: float32
    [positions, rot / 2]; ``layout`` "half": pair (i, i + rot / 2), "pairs": (2 i, 2 i + 1)).  Keys and values go
    into the request's pages as rows [key | value].  Returns the queries [T, heads * dk]."""
    _need_cuda(p, pages)
    assert p.stride(1) == 1 and pages.is_contiguous() and pages.dtype == p.dtype
    assert tuple(pages.shape[1:]) == (kv_heads, pages.shape[2], dk + dv)
    for v, n in ((bq, heads * dk), (bk, kv_heads * dk), (bv, kv_heads * dv), (qw, heads * dk), (kw, kv_heads * dk)):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == n)
    table_len = 0
    if rot:
        assert cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] == rot // 2
        table_len = cos.shape[0]
    T = p.shape[0]
    q = new((T, heads * dk), p.dtype, p.device)
    a = _QkRotArgs(_at(p, first), p.stride(0), k_off, v_off, *(0 if v is None else v.data_ptr() for v in (bq, bk, bv, qw, kw)),
                   float(eps), cos.data_ptr() if rot else 0, sin.data_ptr() if rot else 0, table_len, int(rot),
                   ROTARY_LAYOUTS[layout], q.data_ptr(), pages.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                   pages.shape[2], pages.shape[0], batch.positions.data_ptr(), batch.token_req.data_ptr(), heads, kv_heads,
                   dk, dv, 1 if write else 0, batch.status.data_ptr())
    rc = lib("window_attention").kvb_qk_rot_append(ctypes.byref(a), c_int(T), c_int(dtype_code(p.dtype)), _stream())
    _check(rc, "qk_rot_append")
    return q


def rows_tokens_per_tile(group: int, wide: bool) -> int:
    """Query tokens in one tile of :func:`window_flash_attention`: 64 (``wide``: 128) rows over the group of query
    heads padded to a power of two."""
    gp = 1
    while gp < group:
        gp <<= 1
    return max(1, (128 if wide else 64) // gp)


def window_flash_attention_supported(dk: int, dv: int, group: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core form of :func:`window_attention` for steps with runs of tokens takes these sizes:
    bfloat16, key and value sizes that are multiples of 8 up to 128, at most 64 query heads per key/value head, pages
    of a power of two."""
    return (dtype == torch.bfloat16 and 8 <= dk <= 128 and dk % 8 == 0 and 8 <= dv <= 128 and dv % 8 == 0
            and 1 <= group <= 64 and page_size >= 1 and page_size & (page_size - 1) == 0)


# Which tiles the tensor-core attention over [key | value] rows of unequal sizes cuts a step into: "" chosen from the
# step's size (128 rows when such tiles fill the GPU twice over), "0" 64 rows, "1" 128 rows.
WINDOW_FLASH_WIDE = {"": None, "0": False, "1": True}[os.environ.get('KVB200_WINDOW_FLASH_WIDE', '')]


def window_flash_attention(q: torch.Tensor, pages: torch.Tensor, block_table, batch, heads: int, kv_heads: int, dk: int,
                           dv: int, scale: float, window: int, keep_first: int, one_more: bool,
                           head_scale: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None,
                           softcap: float = 0.0, out_scale: float = 1.0, wide: Optional[bool] = None,
                           sinks: Optional[torch.Tensor] = None, chunk: int = 0, gate=None) -> torch.Tensor:
    """:func:`window_attention` on tensor cores for bfloat16 steps with runs of query tokens: the same mask (window or
    blocks of ``chunk`` positions), softmax (``sinks`` included), shaping of the scores (float32) and output ``gate``,
    the two products on ``mma.sync`` with the probabilities rounded to bfloat16.
    Queries at ``q[:, : heads * dk]``; ``pages`` [num_pages, kv_heads, page_size, dk + dv].  Returns [T, heads * dv]."""
    _need_cuda(q, pages)
    assert q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16 and pages.is_contiguous() and q.stride(1) == 1
    assert tuple(pages.shape[1:]) == (kv_heads, pages.shape[2], dk + dv)
    for v in (head_scale, slopes, sinks):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == heads)
    gate_at, gate_ld = 0, 0
    if gate is not None:
        gt, gcol = gate
        assert gt.dtype == q.dtype and gt.stride(1) == 1 and gt.shape[0] == q.shape[0] and gt.shape[1] >= gcol + heads * dv
        assert gcol % 2 == 0 and gt.stride(0) % 2 == 0
        gate_at, gate_ld = _at(gt, gcol), gt.stride(0)
    T = q.shape[0]
    group = heads // kv_heads
    if wide is None:
        wide = WINDOW_FLASH_WIDE
    if wide is None:
        wide = (T // rows_tokens_per_tile(group, True)) * kv_heads >= 2 * sm_count(q.device)
    tiles = tiles_of_height(batch, rows_tokens_per_tile(group, bool(wide)))
    out = new((T, heads * dv), q.dtype, q.device)
    rc = lib("window_flash_attention").kvb_window_flash_attention_masked(
        _p(q), c_int(q.stride(0)), _p(pages), _p(block_table), c_int(block_table.shape[1]), c_int(pages.shape[2]),
        c_int(pages.shape[0]), _p(batch.positions), _p(tiles), c_int(tiles.shape[0]), c_int(1 if wide else 0), _p(out),
        c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv), c_float(scale), c_int(int(window or 0)),
        c_int(int(keep_first or 0)), c_int(1 if one_more else 0), _p(head_scale), _p(slopes), c_float(float(softcap or 0.0)),
        c_float(float(out_scale)), _p(sinks), c_int(int(chunk or 0)), c_void_p(gate_at), c_int(gate_ld), _p(batch.status),
        _stream())
    _check(rc, "window_flash_attention")
    choices["window_flash_attention"] += 1
    return out


# ------------------------------------------------------------------ several residual streams, token shift, xIELU

class _HyperArgs(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("y", c_void_p), ("y2", c_void_p), ("mix", c_void_p), ("out_w", c_void_p),
                ("in_w", c_void_p), ("weight", c_void_p), ("rows", c_void_p), ("out", c_void_p), ("n", c_int), ("S", c_int),
                ("W", c_int), ("eps", c_float), ("one_plus", c_int), ("out_f32", c_int), ("shift", c_void_p),
                ("shift_state", c_void_p), ("slot_stride", c_longlong), ("slots", c_void_p), ("positions", c_void_p),
                ("prev", c_void_p), ("token_req", c_void_p), ("q_start", c_void_p)]


class PendingStreams:
    """A sublayer's output that has not been written into the residual streams yet: up to two tensors ``ys`` [T, W]
    of the compute type (two mixers that ran side by side hand on both), the mixing matrix ``mix`` [S, S] (indexed
    [from, to]) and the weights ``out_w`` [S] of the write  x_t <- sum_s mix[s, t] x_s + out_w[t] * sum(ys).
    :func:`hyper_norm` carries it out in the kernel that also makes the next sublayer's input."""
    __slots__ = ("ys", "mix", "out_w")

    def __init__(self, ys, mix, out_w):
        self.ys = tuple(y for y in ys if y is not None)
        assert 1 <= len(self.ys) <= 2
        self.mix, self.out_w = mix, out_w


def embed_sinusoid_streams(table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, streams: int,
                           status: torch.Tensor, sampled: Optional[torch.Tensor] = None,
                           base: float = 10000.0) -> torch.Tensor:
    """float32 [T, streams, W]: ``table[ids]`` plus the sinusoidal vector of each token's position (entry 2i:
    ``sin(p base^(-2i / W))``, entry 2i + 1 the cosine of the same angle), the same row in every stream.  Ids below
    zero name tokens still on the device, as for :func:`embed_gather`."""
    _need_cuda(table, ids, sampled)
    V, W = table.shape
    T = ids.numel()
    out = new((T, streams, W), torch.float32, table.device)
    rc = lib("streams").kvb_embed_sinusoid_streams(
        _p(table), dtype_code(table.dtype), _p(ids), _p(sampled), c_int(0 if sampled is None else sampled.numel()),
        _p(positions), _p(out), c_int(T), c_int(streams), c_int(W), c_int(V), c_float(base), _p(status), _stream())
    _check(rc, "embed_sinusoid_streams")
    return out


def hyper_norm(x: torch.Tensor, pending: Optional[PendingStreams], in_w: Optional[torch.Tensor],
               weight: Optional[torch.Tensor], eps: float, one_plus: bool, out_dtype: Optional[torch.dtype],
               compute_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, shift: Optional[torch.Tensor] = None,
               shift_state: Optional[torch.Tensor] = None, batch=None, stage_prev: bool = False):
    """One launch around the residual streams ``x`` (float32 [T, S, W], updated in place unless ``rows`` selects):
    the pending write of the sublayer before, the read ``u = sum_s in_w[s] x_s`` (``in_w`` None: the plain sum) and
    its RMS norm times ``weight`` (``one_plus``: times 1 + weight).  ``out_dtype`` None: only the write.
    With ``shift`` (float32 [W]) and a step in which every request brings one token, the token shift follows in the
    same launch: ``h + (h_before - h) * shift`` with ``h_before`` from ``shift_state[slot]`` (zero at position 0),
    which then takes the unshifted row.  ``stage_prev``: for steps with runs of tokens; the row in front of every
    run's first token is copied out of the slots and returned as the second result, for :func:`token_shift`."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 3
    T, S, W = x.shape
    a = _HyperArgs()
    a.x = x.data_ptr()
    if pending is not None:
        for i, y in enumerate(pending.ys):
            assert y.shape == (T, W) and y.is_contiguous() and y.dtype == compute_dtype
            setattr(a, "y" if i == 0 else "y2", y.data_ptr())
        for v, n in ((pending.mix, S * S), (pending.out_w, S)):
            assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == n)
        a.mix = 0 if pending.mix is None else pending.mix.data_ptr()
        a.out_w = 0 if pending.out_w is None else pending.out_w.data_ptr()
    for v, n in ((in_w, S), (weight, W), (shift, W)):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == n)
    a.in_w = 0 if in_w is None else in_w.data_ptr()
    a.weight = 0 if weight is None else weight.data_ptr()
    n = T if rows is None else rows.numel()
    a.rows = 0 if rows is None else rows.data_ptr()
    out = prev = None
    if out_dtype is not None:
        out = new((n, W), out_dtype, x.device)
        a.out = out.data_ptr()
    a.n, a.S, a.W, a.eps, a.one_plus = n, S, W, eps, 1 if one_plus else 0
    a.out_f32 = 1 if out_dtype == torch.float32 else 0
    if shift is not None or stage_prev:
        assert rows is None and shift_state is not None and shift_state.dtype == torch.float32 and shift_state.stride(1) == 1
        a.shift_state, a.slot_stride = shift_state.data_ptr(), shift_state.stride(0)
        a.slots, a.positions = batch.slots.data_ptr(), batch.positions.data_ptr()
        if stage_prev:
            prev = new((batch.num_reqs, W), torch.float32, x.device)
            a.prev, a.token_req, a.q_start = prev.data_ptr(), batch.token_req.data_ptr(), batch.q_start.data_ptr()
        else:
            assert batch.num_reqs == T
            a.shift = shift.data_ptr()
    rc = lib("streams").kvb_hyper_norm(ctypes.byref(a), c_int(dtype_code(compute_dtype)), _stream())
    _check(rc, "hyper_norm")
    return (out, prev) if stage_prev else out


def token_shift(h: torch.Tensor, prev: torch.Tensor, shift: torch.Tensor, state: torch.Tensor, batch,
                out_dtype: torch.dtype) -> torch.Tensor:
    """``h[t] + (h[t - 1] - h[t]) * shift`` along each request's run of tokens (``h`` float32 [T, W]); the row in front
    of a run's first token is ``prev[request]``; the run's last row goes to ``state[slot]``."""
    _need_cuda(h, prev, state)
    assert h.dtype == torch.float32 and h.is_contiguous() and prev.is_contiguous() and state.stride(1) == 1
    T, W = h.shape
    out = new((T, W), out_dtype, h.device)
    rc = lib("streams").kvb_token_shift(_p(h), _p(prev), _p(shift), _p(state), c_longlong(state.stride(0)), _p(batch.slots),
                                        _p(batch.token_req), _p(batch.q_start), _p(out), c_int(T), c_int(W),
                                        c_int(dtype_code(out_dtype)), _stream())
    _check(rc, "token_shift")
    return out


def xielu(x: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """``z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2`` with ``pq`` = (p, q),
    float32 on the device."""
    _need_cuda(x, pq)
    assert x.is_contiguous() and pq.dtype == torch.float32 and pq.numel() == 2
    out = new(tuple(x.shape), x.dtype, x.device)
    rc = lib("streams").kvb_xielu(_p(x), _p(out), c_longlong(x.numel()), _p(pq), c_int(dtype_code(x.dtype)), _stream())
    _check(rc, "xielu")
    return out


# ------------------------------------------------------------------ linear recurrences with a decay per token

GATE_SUMS_LIBRARY_MIN_ROWS = int(os.environ.get('KVB200_GATE_SUMS_LIBRARY_MIN_ROWS', '128'))


def gate_coeffs(u: torch.Tensor, w: torch.Tensor, br: torch.Tensor, bi: torch.Tensor, lam: torch.Tensor,
                decay_scale: float):
    """The coefficients of a gated diagonal recurrence.  ``u`` [T, C]; ``w`` [blocks, 2 bw, bw] of the compute type,
    block b's rows 0 .. bw-1 making the decay gate r and the rest the input gate i from ``u``'s block b; ``br``, ``bi``,
    ``lam`` float32 [C].  Returns float32 ``a = exp(-decay_scale r softplus(lam))`` and ``b = sqrt(1 - a^2) i u``,
    both [T, C].  The gates' sums are float32 (this package's FMA kernel; for bfloat16 steps of many rows the
    library's batched product with float32 output)."""
    _need_cuda(u, w)
    nb, two_bw, bw = w.shape
    assert two_bw == 2 * bw and u.shape[1] == nb * bw and u.stride(1) == 1 and w.is_contiguous() and w.dtype == u.dtype
    T, C = u.shape
    a = new((T, C), torch.float32, u.device)
    b = new((T, C), torch.float32, u.device)
    if u.dtype == torch.bfloat16 and T >= GATE_SUMS_LIBRARY_MIN_ROWS and _bmm_f32_ok():
        pre = new((nb, T, 2 * bw), torch.float32, u.device)
        uv = torch.as_strided(u, (nb, T, bw), (bw, u.stride(0), 1), u.storage_offset())
        torch.bmm(uv, w.transpose(1, 2), out_dtype=torch.float32, out=pre)
        if _marks is not None:
            _mark("gate_sums_library")
        choices["gate_sums_library"] += 1
        rc = lib("recurrence").kvb_coeffs_from_sums(_p(pre), _p(u), c_int(u.stride(0)), _p(br), _p(bi), _p(lam),
                                                    c_float(decay_scale), _p(a), _p(b), c_int(T), c_int(nb), c_int(bw),
                                                    c_int(dtype_code(u.dtype)), _stream())
        _check(rc, "coeffs_from_sums")
        return a, b
    rc = lib("recurrence").kvb_gate_coeffs(_p(u), c_int(u.stride(0)), _p(w), _p(br), _p(bi), _p(lam), c_float(decay_scale),
                                           _p(a), _p(b), c_int(T), c_int(nb), c_int(bw), c_int(dtype_code(u.dtype)), _stream())
    _check(rc, "gate_coeffs")
    return a, b


_bmm_f32: Optional[bool] = None


def _bmm_f32_ok() -> bool:
    """Whether the library's batched product writes float32 from bfloat16 operands (asked once, on tiny tensors)."""
    global _bmm_f32
    if _bmm_f32 is None:
        if _capturing():
            return False
        try:
            x = torch.zeros((1, 8, 8), dtype=torch.bfloat16, device="cuda")
            torch.bmm(x, x, out_dtype=torch.float32, out=torch.empty((1, 8, 8), dtype=torch.float32, device="cuda"))
            _bmm_f32 = True
        except (TypeError, RuntimeError, NotImplementedError):
            _bmm_f32 = False
    return _bmm_f32


# Runs of at least this many tokens are cut into chunks that the scans below walk side by side (the states that
# the chunks begin with then come from per-chunk summaries, which rounds differently from one walk).
SCAN_CHUNK_MIN_RUN = int(os.environ.get('KVB200_SCAN_CHUNK_MIN_RUN', '256'))


def _chunk_rows(batch, chunk: int):
    """For a step whose runs are cut into chunks of ``chunk`` tokens: (rows of per-chunk scratch, first request row
    that may have more than one chunk).  Request row r's chunk that begins at token row t uses scratch row
    ``r - first + t // chunk``."""
    first = 0
    qs = batch.host.get("q_start") if getattr(batch, "host", None) else None
    if qs is not None:
        runs = qs[1:batch.num_reqs + 1] - qs[:batch.num_reqs]
        long_runs = (runs > chunk).nonzero()[0]
        first = int(long_runs[0]) if len(long_runs) else batch.num_reqs
    return batch.num_reqs - first + batch.num_tokens // chunk + 1, first


class _DiagArgs(ctypes.Structure):
    _fields_ = [("a", c_void_p), ("b", c_void_p), ("y", c_void_p), ("ld_y", c_int), ("y_bias", c_void_p),
                ("out_scale", c_float), ("out", c_void_p), ("state", c_void_p), ("slot_stride", c_longlong),
                ("q_start", c_void_p), ("req_start", c_void_p), ("slots", c_void_p), ("C", c_int),
                ("chunked", c_int), ("row_off", c_int), ("sum_a", c_void_p), ("sum_b", c_void_p), ("begin", c_void_p)]


def diag_scan(a: torch.Tensor, b: torch.Tensor, y, y_bias: Optional[torch.Tensor], out_scale: float,
              state: torch.Tensor, batch, out_dtype: torch.dtype) -> torch.Tensor:
    """``S_t = a_t S_{t-1} + b_t`` per channel along every request's tokens of the step, from the state in the
    request's slot (zero for a request that starts at position 0), which is left up to date.  ``y``: (tensor,
    first column) of the gate branch [T, C] before its activation.  Returns
    ``S_t * gelu_tanh(y_t + y_bias) * out_scale`` [T, C].  A step with a run of ``SCAN_CHUNK_MIN_RUN`` tokens or
    more walks chunks of its runs side by side."""
    _need_cuda(a, b, state)
    T, C = a.shape
    yt, ycol = y
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous()
    assert yt.dtype == out_dtype and yt.stride(1) == 1 and state.dtype == torch.float32 and state.stride(1) == 1
    out = new((T, C), out_dtype, a.device)
    max_run = int(getattr(batch, "max_q_len", 0) or 0)
    chunked = max_run >= SCAN_CHUNK_MIN_RUN and not _capturing()
    sa = sb = begin = first = 0
    if chunked:
        rows, first = _chunk_rows(batch, lib("recurrence").kvb_diag_chunk())
        pairs = new((2, rows, C), torch.float32, a.device)
        begin_t = new((batch.num_reqs, C), torch.float32, a.device)
        sa, sb, begin = pairs[0].data_ptr(), pairs[1].data_ptr(), begin_t.data_ptr()
        choices["diag_scan_chunked"] += 1
    p = _DiagArgs(a.data_ptr(), b.data_ptr(), _at(yt, ycol), yt.stride(0), 0 if y_bias is None else y_bias.data_ptr(),
                  float(out_scale), out.data_ptr(), state.data_ptr(), state.stride(0), batch.q_start.data_ptr(),
                  batch.req_start.data_ptr(), batch.slots.data_ptr(), C, int(chunked), first, sa, sb, begin)
    rc = lib("recurrence").kvb_diag_scan(ctypes.byref(p), c_int(batch.num_reqs), c_int(max_run),
                                         c_int(dtype_code(out_dtype)), _stream())
    _check(rc, "diag_scan")
    return out


class _SsdArgs(ctypes.Structure):
    _fields_ = [("xbc", c_void_p), ("ld_xbc", c_int), ("dt", c_void_p), ("ld_dt", c_int), ("dt_bias", c_void_p),
                ("A_log", c_void_p), ("D", c_void_p), ("state", c_void_p), ("slot_stride", c_longlong), ("y", c_void_p),
                ("q_start", c_void_p), ("req_start", c_void_p), ("slots", c_void_p), ("H", c_int), ("G", c_int),
                ("N", c_int), ("Dv", c_int), ("cols", c_int), ("chunk", c_int), ("row_off", c_int),
                ("local", c_void_p), ("carry", c_void_p), ("decay", c_void_p)]


def ssd_scan(xbc: torch.Tensor, dt, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, batch, heads: int, groups: int, n: int, dv: int) -> torch.Tensor:
    """A matrix state ``S`` [n, dv] per head with one decay per head and token, along every request's tokens of the
    step:  ``dt = softplus(dt_raw + dt_bias)``, ``S <- exp(-exp(A_log) dt) S + dt B x^T``, ``y = S^T C + D x``.
    ``xbc`` [T, heads dv + 2 groups n]: x | B | C (head h reads group ``h // (heads / groups)``); ``dt``: (tensor, first
    column) of the raw step sizes [T, heads].  ``state``: float32 [slots, >= heads * dv * n], zero for a request
    that starts at position 0.  Returns float32 y [T, heads * dv].  A step with a run of ``SCAN_CHUNK_MIN_RUN``
    tokens or more walks chunks of its runs side by side (64 tokens a chunk, 128 from runs of 1024 on)."""
    _need_cuda(xbc, state)
    T = xbc.shape[0]
    dtt, dcol = dt
    assert xbc.stride(1) == 1 and dtt.stride(1) == 1 and dtt.dtype == xbc.dtype and state.dtype == torch.float32
    assert state.stride(1) == 1 and xbc.shape[1] >= heads * dv + 2 * groups * n
    for v in (dt_bias, a_log, d_skip):
        assert v.dtype == torch.float32 and v.is_contiguous() and v.numel() == heads
    y = new((T, heads * dv), torch.float32, xbc.device)
    max_run = int(getattr(batch, "max_q_len", 0) or 0)
    chunk = first = local = carry = decay = 0
    if max_run >= SCAN_CHUNK_MIN_RUN and not _capturing():
        chunk = 128 if max_run >= 1024 else 64
        rows, first = _chunk_rows(batch, chunk)
        mats = new((2, rows, heads * dv * n), torch.float32, xbc.device)
        decay_t = new((rows, heads), torch.float32, xbc.device)
        local, carry, decay = mats[0].data_ptr(), mats[1].data_ptr(), decay_t.data_ptr()
        choices["ssd_scan_chunked"] += 1
    p = _SsdArgs(xbc.data_ptr(), xbc.stride(0), _at(dtt, dcol), dtt.stride(0), dt_bias.data_ptr(), a_log.data_ptr(),
                 d_skip.data_ptr(), state.data_ptr(), state.stride(0), y.data_ptr(), batch.q_start.data_ptr(),
                 batch.req_start.data_ptr(), batch.slots.data_ptr(), heads, groups, n, dv, 0, chunk, first, local, carry, decay)
    rc = lib("recurrence").kvb_ssd_scan(ctypes.byref(p), c_int(batch.num_reqs), c_int(max_run),
                                        c_int(dtype_code(xbc.dtype)), _stream())
    _check(rc, "ssd_scan")
    return y


class _MlstmArgs(ctypes.Structure):
    _fields_ = [("qkv", c_void_p), ("ld", c_int), ("q_off", c_int), ("k_off", c_int), ("v_off", c_int),
                ("gates", c_void_p), ("ld_g", c_int), ("bi", c_void_p), ("bf", c_void_p), ("cap", c_float),
                ("q_scale", c_float), ("state", c_void_p), ("slot_stride", c_longlong), ("y", c_void_p),
                ("q_start", c_void_p), ("req_start", c_void_p), ("slots", c_void_p), ("H", c_int), ("N", c_int),
                ("Dv", c_int), ("chunk", c_int), ("row_off", c_int), ("local", c_void_p), ("carry", c_void_p),
                ("fsum", c_void_p)]


def mlstm_state_floats(heads: int, n: int, dv: int) -> int:
    """float32 numbers of one request's state of :func:`mlstm_scan`: the matrices [heads, dv, n], then the vector n
    and the maximum m once per block of 64 value columns."""
    splits = -(-dv // 64)
    return heads * dv * n + heads * splits * (n + 1)


def mlstm_scan(p: torch.Tensor, q_off: int, k_off: int, v_off: int, gates: torch.Tensor, bi: torch.Tensor,
               bf: torch.Tensor, cap: float, q_scale: float, state: torch.Tensor, batch, heads: int, n: int,
               dv: int) -> torch.Tensor:
    """A matrix memory ``C`` [n, dv] per head with exponential gates and a running maximum ``m``, along every
    request's tokens of the step::

        i = cap tanh((a + bi) / cap),  f = logsigmoid(cap tanh((b + bf) / cap)),  m' = max(f + m, i)
        C <- exp(f + m - m') C + exp(i - m') k v^T,  n <- (likewise with k),  y = C^T q / (max(|n . q|, exp(-m')) + 1e-6)

    ``p`` [T, ...] holds q (``heads * n`` from column ``q_off``; multiplied by ``q_scale``), k and v; ``gates`` float32
    [T, 2 heads]: the raw a, then the raw b.  ``state``: float32 [slots, >= mlstm_state_floats], empty (m = 0) for a
    request that starts at position 0.  Returns float32 y [T, heads * dv].  A step with a run of
    ``SCAN_CHUNK_MIN_RUN`` tokens or more walks chunks of 64 tokens side by side."""
    _need_cuda(p, gates, state)
    T = p.shape[0]
    assert p.stride(1) == 1 and gates.dtype == torch.float32 and gates.stride(1) == 1 and gates.shape[1] >= 2 * heads
    assert state.dtype == torch.float32 and state.stride(1) == 1 and state.shape[1] >= mlstm_state_floats(heads, n, dv)
    for v in (bi, bf):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == heads)
    y = new((T, heads * dv), torch.float32, p.device)
    max_run = int(getattr(batch, "max_q_len", 0) or 0)
    chunk = first = local = carry = fsum = 0
    if max_run >= SCAN_CHUNK_MIN_RUN and not _capturing():
        chunk = 64
        rows, first = _chunk_rows(batch, chunk)
        per = mlstm_state_floats(heads, n, dv)
        mats = new((2, rows, per), torch.float32, p.device)
        fsum_t = new((rows, heads), torch.float32, p.device)
        local, carry, fsum = mats[0].data_ptr(), mats[1].data_ptr(), fsum_t.data_ptr()
        choices["mlstm_scan_chunked"] += 1
    a = _MlstmArgs(p.data_ptr(), p.stride(0), q_off, k_off, v_off, gates.data_ptr(), gates.stride(0),
                   0 if bi is None else bi.data_ptr(), 0 if bf is None else bf.data_ptr(), float(cap), float(q_scale),
                   state.data_ptr(), state.stride(0), y.data_ptr(), batch.q_start.data_ptr(), batch.req_start.data_ptr(),
                   batch.slots.data_ptr(), heads, n, dv, chunk, first, local, carry, fsum)
    rc = lib("mlstm").kvb_mlstm_scan(ctypes.byref(a), c_int(batch.num_reqs), c_int(max_run), c_int(dtype_code(p.dtype)),
                                     _stream())
    _check(rc, "mlstm_scan")
    return y


def head_norm_gate(y: torch.Tensor, gate, weight: torch.Tensor, heads: int, eps: float,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """Every head of ``y`` (float32 [T, heads * dv]) divided by its own root mean square (eps inside the root), times
    ``weight`` (float32 [heads * dv]), times the sigmoid of ``gate``: (tensor, first column), compute type."""
    _need_cuda(y, weight)
    T, width = y.shape
    gt, gcol = gate
    assert y.dtype == torch.float32 and y.is_contiguous() and gt.stride(1) == 1 and gt.dtype == out_dtype
    assert weight.dtype == torch.float32 and weight.numel() == width and width % heads == 0
    out = new((T, width), out_dtype, y.device)
    rc = lib("mlstm").kvb_head_norm_gate(_p(y), c_void_p(_at(gt, gcol)), c_int(gt.stride(0)), _p(weight), _p(out),
                                         c_int(T), c_int(heads), c_int(width // heads), c_float(eps),
                                         c_int(dtype_code(out_dtype)), _stream())
    _check(rc, "head_norm_gate")
    return out


def gated_group_norm(y: torch.Tensor, z, weight: torch.Tensor, groups: int, eps: float,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """``v = y * silu(z)``, then each of ``groups`` equal parts of a row divided by its own root mean square (eps
    inside the root), times ``weight``.  ``y`` float32 [T, width]; ``z``: (tensor, first column), compute type."""
    _need_cuda(y, weight)
    T, width = y.shape
    zt, zcol = z
    assert y.dtype == torch.float32 and y.is_contiguous() and zt.stride(1) == 1 and zt.dtype == out_dtype
    assert weight.dtype == torch.float32 and weight.numel() == width
    out = new((T, width), out_dtype, y.device)
    rc = lib("recurrence").kvb_gated_group_norm(_p(y), c_void_p(_at(zt, zcol)), c_int(zt.stride(0)), _p(weight), _p(out),
                                                c_int(T), c_int(width), c_int(groups), c_float(eps),
                                                c_int(dtype_code(out_dtype)), _stream())
    _check(rc, "gated_group_norm")
    return out


# ------------------------------------------------------------------ routed experts

def route(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], experts: int, identity: int, top: int,
          scale: float, logits: Optional[torch.Tensor] = None, score: str = "softmax", renormalize: bool = True):
    """The router of a feed-forward of many experts.  ``w_router`` float32 [experts + identity, K],
    ``correction`` float32 [experts + identity] (added to the scores for the choice only).  Returns
    ``gate`` float32 [T, experts + identity], a token's weight for every expert (0 where not chosen), and
    float32 [T], the summed weights of its identity experts (None without any).  ``logits``: float32
    [T, experts + identity], the products ``h . w_router^T`` if the caller has made them already (by a matrix
    product that adds up in float32; further columns behind them are left alone), in which case the kernel only
    chooses.  ``score`` "softmax": the scores are the logits' softmax over all experts; "sigmoid": each logit's sigmoid.
    ``renormalize`` False: a chosen expert's weight is its score times ``scale``, not divided by the chosen scores' sum.
    ``correction`` None: the choice goes by the scores alone."""
    _need_cuda(h, w_router)
    T, K = h.shape
    n_all = experts + identity
    assert logits is not None or w_router is not None
    assert w_router is None or (w_router.dtype == torch.float32 and w_router.is_contiguous()
                                and tuple(w_router.shape) == (n_all, K))
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == n_all)
    assert h.stride(1) == 1
    assert logits is None or (logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[0] == T
                              and logits.shape[1] >= n_all)
    gate = new((T, n_all), torch.float32, h.device)
    idw = new((T,), torch.float32, h.device) if identity else None
    rc = lib("experts").kvb_route(_p(h), c_int(h.stride(0)), _p(w_router), _p(logits),
                                  c_int(0 if logits is None else logits.stride(0)), _p(correction), _p(gate), _p(idw), c_int(T),
                                  c_int(K), c_int(experts), c_int(identity), c_int(top), c_float(scale),
                                  c_int({"softmax": 0, "sigmoid": 1}[score]), c_int(1 if renormalize else 0),
                                  c_int(dtype_code(h.dtype)), _stream())
    _check(rc, "route")
    return gate, idw


def expert_act(p: torch.Tensor, gate: torch.Tensor, experts: int, ff: int, shared_ff: int) -> torch.Tensor:
    """``relu(p)^2`` times each routed expert's weight for the token (``p`` [T, experts * ff + shared_ff]:
    the experts' first products side by side, then those of an expert that every token uses)."""
    _need_cuda(p, gate)
    assert p.is_contiguous() and p.shape[1] == experts * ff + shared_ff and gate.dtype == torch.float32
    out = new(tuple(p.shape), p.dtype, p.device)
    rc = lib("experts").kvb_expert_act(_p(p), _p(gate), c_int(gate.stride(0)), _p(out), c_int(p.shape[0]), c_int(experts),
                                       c_int(ff), c_int(shared_ff), c_int(dtype_code(p.dtype)), _stream())
    _check(rc, "expert_act")
    return out


def limited_act(p: torch.Tensor, gate: torch.Tensor, shared_logit: Optional[torch.Tensor], experts: int, ff: int,
                shared_ff: int, pad: int, limit: float, shared_limit: float, alpha: float) -> torch.Tensor:
    """The activation of experts ``down(a(g) (u + 1))`` with ``g = min(w gate.h, limit)``, ``u = clamp(w up.h, +-limit)``,
    ``a(g) = g sigmoid(alpha g)`` and ``w`` the token's weight for the expert (``gate`` float32 [T, >= experts], 0 where
    not chosen).  ``p`` [T, 2 (experts ff + shared_ff)]: per expert its gate product, then its up product; behind
    them those of an expert that every token uses, whose result is multiplied by ``sigmoid(shared_logit[t])`` (float32
    column, may be a strided view; None: by 1).  Returns [T, experts ff + shared_ff + pad], the padding zero."""
    _need_cuda(p, gate)
    assert p.stride(1) == 1 and gate.dtype == torch.float32 and gate.stride(1) == 1
    assert shared_logit is None or (shared_logit.dtype == torch.float32 and shared_logit.shape[0] == p.shape[0])
    width = experts * ff + shared_ff + pad
    out = new((p.shape[0], width), p.dtype, p.device)
    rc = lib("experts").kvb_limited_act(_p(p), c_int(p.stride(0)), _p(gate), c_int(gate.stride(0)), _p(shared_logit),
                                        c_int(0 if shared_logit is None else shared_logit.stride(0)), _p(out),
                                        c_int(p.shape[0]), c_int(experts), c_int(ff), c_int(shared_ff), c_int(pad),
                                        c_float(limit), c_float(shared_limit), c_float(alpha), c_int(dtype_code(p.dtype)),
                                        _stream())
    _check(rc, "limited_act")
    return out


def row_axpy(y: torch.Tensor, x: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """``y[t] += c[t] * x[t]`` in place (``c`` float32 [T])."""
    _need_cuda(y, x, c)
    assert y.is_contiguous() and x.stride(1) == 1 and x.dtype == y.dtype and x.shape == y.shape and c.dtype == torch.float32
    rc = lib("experts").kvb_row_axpy(_p(y), _p(x), c_int(x.stride(0)), _p(c), c_int(y.shape[0]), c_int(y.shape[1]),
                                     c_int(dtype_code(y.dtype)), _stream())
    _check(rc, "row_axpy")
    return y


# ------------------------------------------------------------------ matrix products

SKINNY_MAX_ROWS = int(os.environ.get('KVB200_SKINNY_MAX_ROWS', '32'))   # measured: the library product wins beyond
_status_word: Dict[int, torch.Tensor] = {}


def kernel_status(device) -> torch.Tensor:
    """The device word into which kernels report impossible indices and waits that ran
    out; one per device, shared by every engine in the process."""
    idx = torch.device(device).index or 0
    t = _status_word.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status_word[idx] = t
    return t


class Folded:
    """What a product hands on in place of its output once it has added that output into
    the float32 residual itself: ``xb``, the new residual rows in bfloat16, and ``sumsq``
    [rows, parts], partial sums of their squares, from which the next norm's 1/rms follows."""
    __slots__ = ("xb", "sumsq")

    def __init__(self, xb: torch.Tensor, sumsq: torch.Tensor):
        self.xb, self.sumsq = xb, sumsq


class PendingNorm:
    """A weightless RMSNorm that has not been carried out (the norm's weight has been
    multiplied into the matrices that read its result): the float32 rows, their bfloat16
    copy and partial sums of squares, and eps.  ``linear`` and ``linear_swiglu`` take it in
    place of a tensor: they multiply the bare rows and scale each row of the result by its
    1/rms.  ``materialize`` runs the norm as a kernel of its own for everything else."""
    __slots__ = ("resid", "xb", "sumsq", "eps", "dtype")

    def __init__(self, resid, xb, sumsq, eps, dtype):
        self.resid, self.xb, self.sumsq, self.eps, self.dtype = resid, xb, sumsq, eps, dtype

    @property
    def shape(self):
        return self.resid.shape

    def materialize(self) -> torch.Tensor:
        return add_rmsnorm(self.resid, None, None, self.eps, self.dtype)


FUSED_NORM = os.environ.get('KVB200_FUSED_NORM', '1') != '0'


def fused_norm_rows(rows: int, dtype: torch.dtype) -> bool:
    """Whether products over ``rows`` rows fold the residual add and the norm into themselves."""
    return FUSED_NORM and dtype == torch.bfloat16 and rows <= min(SKINNY_MAX_ROWS, FUSED_EPILOGUE_MAX_ROWS)


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, into: Optional[torch.Tensor] = None):
    """``x . w^T`` with ``w`` [out, in].
    float32: this package's FMA kernel (true 32-bit).
    bfloat16, few rows (decode and short portions): this package's tcgen05/TMA
    kernel, which streams the weights.  bfloat16 with more rows (long prompt portions):
    the library product, float32 accumulation, as upstream's cublasGemmEx.

    ``x`` may be a :class:`PendingNorm`.  ``into``: a float32 residual [rows, out] the
    caller is going to add the result to; where the tensor-core kernel can, it adds the
    product there itself and a :class:`Folded` comes back instead of a tensor."""
    if isinstance(x, PendingNorm):
        if into is None and fused_norm_rows(x.xb.shape[0], x.dtype) and w.dtype == torch.bfloat16:
            return gemm_skinny_fused(x.xb, w, kernel_status(w.device), row_scale=x,
                                     x_is_static=_capturing())
        if (into is None and wide_fused_rows(x.xb.shape[0], x.dtype) and _wide_ok(x.xb, w, 8)
                and (out_dtype is None or out_dtype == x.dtype)):
            return gemm_wide(x.xb, w, kernel_status(w.device), row_scale=x)
        x = x.materialize()
    _need_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == w.dtype
    if (into is not None and fused_norm_rows(M, x.dtype) and _skinny_ok(x, FUSED_EPILOGUE_MAX_ROWS) and N % 8 == 0
            and into.dtype == torch.float32 and into.shape == (M, N) and into.is_contiguous()):
        return gemm_skinny_fused(x, w, kernel_status(w.device), into=into,
                                 x_is_static=_capturing())
    if (into is not None and wide_fused_rows(M, x.dtype) and _wide_ok(x, w, 8) and into.dtype == torch.float32
            and into.shape == (M, N) and into.is_contiguous() and N % 4 == 0):
        return gemm_wide(x, w, kernel_status(w.device), into=into)
    if x.dtype == torch.float32:
        assert x.stride(1) == 1 and w.stride(1) == 1
        out = new((M, N), torch.float32, x.device)
        rc = lib("gemm_f32").kvb_sgemm_nt(_p(x), c_int(x.stride(0)), _p(w), c_int(w.stride(0)), _p(out),
                                          c_int(N), c_int(M), c_int(N), c_int(K), _stream())
        _check(rc, "sgemm_nt")
        choices["sgemm_nt"] += 1
        return out
    if M <= SKINNY_MAX_ROWS and K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        return gemm_skinny(x, w, out_dtype or x.dtype, kernel_status(x.device),
                           x_is_static=_capturing())
    if WIDE == "all" and _wide_ok(x, w, 8) and (out_dtype is None or out_dtype == x.dtype):
        return gemm_wide(x, w, kernel_status(x.device))
    choices["library_product"] += 1
    return _library_product(x, w, out_dtype or x.dtype)


_mm_takes_out_with_dtype = True    # whether torch.mm accepts out= together with out_dtype= (found out at first use)


def _library_product(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``x . w^T`` by the library (cuBLAS, float32 accumulation), written into a tensor of the
    step's arena."""
    global _mm_takes_out_with_dtype
    out = new((x.shape[0], w.shape[0]), out_dtype, x.device)
    if out_dtype == x.dtype:
        torch.matmul(x, w.t(), out=out)
        if _marks is not None:
            _mark("library_product")
        return out
    if _mm_takes_out_with_dtype:
        try:
            return torch.mm(x, w.t(), out_dtype=out_dtype, out=out)
        except (TypeError, RuntimeError, NotImplementedError):
            _mm_takes_out_with_dtype = False
    return torch.mm(x, w.t(), out_dtype=out_dtype)


# Which products of steps with many rows run on this package's tcgen05 kernel (gemm_bf16_wide.cu):
#   "auto"  those it is faster for on a B200 at every number of rows: the gate|up product, whose
#           SiLU * up it does as its epilogue (at 2048 rows it is level with the library for the
#           others, at 512 rows the library's split of K wins for the down product)
#   "all"   every one (no library product in a bfloat16 step)
#   "off"   none (the library product, then the activation kernel)
WIDE = os.environ.get('KVB200_WIDE', 'auto')
WIDE_MIN_ROWS = 128
# From this many rows on the products of a step also take the residual add and the RMSNorm into
# themselves (as the products of few rows do), which makes every product of the step this
# package's: below it the library's split of K is the faster way through the narrow products.  0: never.
WIDE_FUSED_MIN_ROWS = int(os.environ.get('KVB200_WIDE_FUSED_MIN_ROWS', '0'))


def wide_fused_rows(rows: int, dtype: torch.dtype) -> bool:
    """Whether products over ``rows`` rows (many) fold the residual add and the norm into themselves."""
    return (FUSED_NORM and WIDE != "off" and WIDE_FUSED_MIN_ROWS > 0 and dtype == torch.bfloat16
            and rows >= WIDE_FUSED_MIN_ROWS)


def _wide_ok(x: torch.Tensor, w: torch.Tensor, n_multiple: int) -> bool:
    """Whether the tcgen05 kernel for steps of many rows takes this product."""
    return (x.shape[0] >= WIDE_MIN_ROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.shape[1] % 8 == 0 and w.shape[0] % n_multiple == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _skinny_ok(x: torch.Tensor, rows_limit: int) -> bool:
    return (x.dtype == torch.bfloat16 and x.shape[0] <= rows_limit and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)


def linear_swiglu(x: torch.Tensor, gate_up: torch.Tensor, block: int) -> torch.Tensor:
    """``silu(x . gate^T) * (x . up^T)`` with gate and up stored as one matrix whose rows
    alternate in blocks of ``block`` features.  Few bfloat16 rows (SKINNY_MAX_ROWS) with blocks of 64:
    one kernel (the activation is the product's epilogue); otherwise product, then
    activation kernel."""
    I = gate_up.shape[0] // 2
    if isinstance(x, PendingNorm):
        if fused_norm_rows(x.xb.shape[0], x.dtype) and gate_up.dtype == torch.bfloat16:
            st, static = kernel_status(gate_up.device), _capturing()
            if block == 64 and gate_up.shape[0] % 128 == 0:
                return gemm_skinny_fused(x.xb, gate_up, st, row_scale=x, epilogue="swiglu", x_is_static=static)
            return silu_mul(gemm_skinny_fused(x.xb, gate_up, st, row_scale=x, x_is_static=static),
                            block=block if block != I else None)
        if wide_fused_rows(x.xb.shape[0], x.dtype) and block == 64 and _wide_ok(x.xb, gate_up, 128):
            return gemm_wide(x.xb, gate_up, kernel_status(gate_up.device), epilogue="swiglu", row_scale=x)
        x = x.materialize()
    if block == 64 and _skinny_ok(x, min(SKINNY_MAX_ROWS, FUSED_EPILOGUE_MAX_ROWS)) \
            and gate_up.shape[0] % 128 == 0:
        return gemm_skinny(x, gate_up, x.dtype, kernel_status(x.device),
                           x_is_static=_capturing(), epilogue="swiglu")
    if WIDE != "off" and block == 64 and _wide_ok(x, gate_up, 128):
        return gemm_wide(x, gate_up, kernel_status(x.device), epilogue="swiglu")
    return silu_mul(linear(x, gate_up), block=block if block != I else None)


_scratch: Dict[tuple, torch.Tensor] = {}


def scratch(key: tuple, shape, dtype, device) -> torch.Tensor:
    """A buffer that lives as long as the process, one per key: kernels that need
    global memory beyond their inputs and outputs get it here, so that captured
    graphs see fixed addresses and steps allocate nothing."""
    t = _scratch.get(key)
    if t is None or t.shape != tuple(shape):
        t = torch.empty(shape, dtype=dtype, device=device)
        _scratch[key] = t
    return t


def decode_key_blocks(max_positions: int):
    """(keys per block, number of blocks) of the split decode kernel for an engine that
    allows ``max_positions`` tokens: at most 64 blocks, 128 keys or a multiple."""
    kb = 128 * max(1, -(-max_positions // (128 * 64)))
    return kb, -(-max_positions // kb)


def decode_attention_supported(d: int, group: int) -> bool:
    return bool(lib("attention").kvb_decode_attention_supported(c_int(d), c_int(group)))


def decode_attention(qkv, k_pages, v_pages, block_table, q_start, ctx_len, nq, nkv, d, scale, window,
                     max_positions, status, reqs_capacity=None) -> torch.Tensor:
    """One query token per request, split over key blocks, all heads of a group together."""
    _need_cuda(qkv, k_pages)
    R = ctx_len.numel()
    T = qkv.shape[0]
    kb, nb = decode_key_blocks(max_positions)
    cap = max(R, reqs_capacity or 0)
    part_o = scratch(("dec_o", qkv.device.index, cap, nq, nb, d), (cap, nq, nb, d), torch.float32, qkv.device)
    part_ml = scratch(("dec_ml", qkv.device.index, cap, nq, nb), (cap, nq, nb, 2), torch.float32, qkv.device)
    out = new((T, nq * d), qkv.dtype, qkv.device)
    rc = lib("attention").kvb_decode_attention(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]),
        c_int(k_pages.shape[2]), c_int(k_pages.shape[0]), _p(q_start), _p(ctx_len), _p(out), _p(part_o),
        _p(part_ml), c_int(R), c_int(nq), c_int(nkv), c_int(d), c_float(scale), c_int(int(window or 0)),
        c_int(kb), c_int(nb), c_int(dtype_code(qkv.dtype)), _p(status), _stream())
    _check(rc, "decode_attention")
    global launch_count
    launch_count += 1  # split and combine
    return out


FLASH_WIDE = os.environ.get('KVB200_FLASH_WIDE', '1') != '0'
FLASH_TC = os.environ.get('KVB200_FLASH_TC', '1') != '0'
FLASH_TC_ROLES = os.environ.get('KVB200_FLASH_TC_ROLES', '1') != '0'


def flash_attention_supported(d: int, group: int, page_size: int) -> bool:
    if d not in (64, 128):      # answered here, so that a model of another head size never builds the module
        return False
    return bool(lib("flash_attention").kvb_flash_attention_supported(c_int(d), c_int(group), c_int(page_size)))


_tokens_per_tile: Dict[tuple, int] = {}


def flash_tokens_per_tile(group: int, wide: bool) -> int:
    """Query tokens in one tile of the tensor-core attention for prompt portions: 64 rows
    (``wide`` False) or 128 rows of (token, head of the group) pairs."""
    key = (int(group), bool(wide))
    if key not in _tokens_per_tile:
        _tokens_per_tile[key] = int(lib("flash_attention").kvb_flash_attention_tokens_per_tile(
            c_int(key[0]), c_int(1 if wide else 0)))
    return _tokens_per_tile[key]


def flash_tiles(batch, group: int, wide: bool) -> torch.Tensor:
    """The query tiles of a step for a group size: [n, 4] int32 rows (request row, first
    token row, tokens, 0), each tile holding consecutive tokens of one request.  Built
    once per step, group size and tile height, kept on the batch."""
    return tiles_of_height(batch, flash_tokens_per_tile(group, bool(wide)))


def tiles_of_height(batch, nt: int) -> torch.Tensor:
    """The step's runs of tokens cut into query tiles of at most ``nt`` tokens: [n, 4] int32 rows (request row, first
    token row, tokens, 0)."""
    ready = (getattr(batch, "tiles", None) or {}).get(nt)
    if ready is not None:
        return ready            # laid out with the batch's other arrays and copied with them
    cache = batch.host.setdefault("flash_tiles", {})
    got = cache.get(nt)
    if got is None:
        import numpy as np
        qs = batch.host["q_start"]
        rows = []
        for r in range(batch.num_reqs):
            a, b = int(qs[r]), int(qs[r + 1])
            starts = np.arange(a, b, nt, dtype=np.int32)
            tile = np.zeros((len(starts), 4), dtype=np.int32)
            tile[:, 0] = r
            tile[:, 1] = starts
            tile[:, 2] = np.minimum(nt, b - starts)
            rows.append(tile)
        host = torch.from_numpy(np.concatenate(rows)).pin_memory()
        got = host.to(batch.token_ids.device, non_blocking=True)
        cache[nt] = got
        cache[("host", nt)] = host   # keep the pinned source alive until the step is over
    return got


def flash_attention(qkv, k_pages, v_pages, block_table, batch, nq, nkv, d, scale, window,
                    wide: Optional[bool] = None, skip_single: bool = False,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-core attention for steps with runs of query tokens (bfloat16).  ``wide``:
    False: 64 query rows per block (mma.sync); True: 128 rows (mma.sync); 2: 128 rows on
    tcgen05 with the scores in tensor memory (head size 64); 3: the same with roles (a TMA
    loader warp, two issuing warps, four softmax warps; head size 64 or 128, pages of at least
    8 rows); None:
    chosen from the step's size, the head size and the page size.  ``skip_single``: the step's
    leading single tokens (``batch.num_single``) are somebody else's: their tiles are left out.
    ``out``: where the rows go; made here if not given."""
    _need_cuda(qkv, k_pages)
    skip = int(batch.num_single) if skip_single else 0
    T = qkv.shape[0] - skip
    # 128-row tiles when there are enough of them to keep every SM busy, else 64-row tiles
    nt128 = flash_tokens_per_tile(nq // nkv, True)
    if wide is None:
        # 128-row tiles when they fill the GPU: two blocks per SM at head size 64, one at 128
        wide = FLASH_WIDE and (T // nt128) * nkv >= (2 if d == 64 else 1) * sm_count(qkv.device)
        if wide and FLASH_TC:
            roles = (FLASH_TC_ROLES and k_pages.shape[2] >= 8 and k_pages.data_ptr() % 16 == 0
                     and v_pages.data_ptr() % 16 == 0 and qkv.data_ptr() % 16 == 0 and qkv.stride(0) % 8 == 0)
            if roles:
                wide = 3
            elif d == 64:
                wide = 2
    tiles = flash_tiles(batch, nq // nkv, wide)[skip:]      # a single token is one tile, and they come first
    if out is None:
        out = new((qkv.shape[0], nq * d), qkv.dtype, qkv.device)
    rc = lib("flash_attention").kvb_paged_flash_attention(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]),
        c_int(k_pages.shape[2]), c_int(k_pages.shape[0]), _p(batch.positions), _p(tiles), c_int(tiles.shape[0]),
        c_int(int(wide)), _p(out), c_int(nq), c_int(nkv), c_int(d), c_float(scale), c_int(int(window or 0)), _p(batch.status),
        _stream())
    _check(rc, "paged_flash_attention")
    choices[f"flash_attention_{int(wide)}"] += 1
    return out


def decode_attention_fused(qkv, k_pages, v_pages, write_kv, block_table, q_start, ctx_len, cos, sin, rot,
                           nq, nkv, d, scale, window, max_positions, status, trace=None) -> torch.Tensor:
    """The whole attention of a decode step in one launch: rotary encoding of query and
    new key, the write of key and value into their page, split attention, merge."""
    _need_cuda(qkv, k_pages)
    R = ctx_len.numel()
    T = qkv.shape[0]
    kb, nb = decode_key_blocks(max_positions)
    dev = qkv.device
    part_o = scratch(("dec_o", dev.index, R, nq, nb, d), (R, nq, nb, d), torch.float32, dev)
    part_ml = scratch(("dec_ml", dev.index, R, nq, nb), (R, nq, nb, 2), torch.float32, dev)
    counters = _scratch.get(("dec_counters", dev.index))
    if counters is None or counters.numel() < R * nkv:
        counters = torch.zeros(max(R * nkv, 4096), dtype=torch.int32, device=dev)
        _scratch[("dec_counters", dev.index)] = counters
    out = new((T, nq * d), qkv.dtype, dev)
    rc = lib("attention").kvb_decode_attention_fused(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), c_int(1 if write_kv else 0), _p(block_table),
        c_int(block_table.shape[1]), c_int(k_pages.shape[2]), c_int(k_pages.shape[0]), _p(q_start), _p(ctx_len),
        _p(cos), _p(sin), c_int(0 if cos is None else cos.shape[0]), c_int(rot), _p(out), _p(part_o), _p(part_ml),
        _p(counters), c_int(R), c_int(nq), c_int(nkv), c_int(d), c_float(scale), c_int(int(window or 0)),
        c_int(kb), c_int(nb), c_int(dtype_code(qkv.dtype)), _p(status), _p(trace), _stream())
    _check(rc, "decode_attention_fused")
    choices["decode_attention_fused"] += 1
    return out


def decode_attention_mma_supported(d: int, group: int, page_size: int) -> bool:
    if d not in (64, 128):      # answered here, so that a model of another head size never builds the module
        return False
    return bool(lib("decode_attention").kvb_decode_attention_mma_supported(c_int(d), c_int(group), c_int(page_size)))


def decode_context_class(max_ctx: int) -> int:
    """The classes of 128-key tiles (4, 8 or 16) that the longest context of a decode step
    needs in the tensor-core decode attention.  The launch (kernel variant, blocks per request)
    depends on it, the results do not; steps are replayed from graphs captured per class."""
    from .engine.batch import CONTEXT_CLASS_BOUNDS as bounds   # the block tables' widths follow the same classes
    return 4 if max_ctx <= bounds[0] else (8 if max_ctx <= bounds[1] else 16)


def decode_launch_context(batch) -> int:
    """The context length a decode step's launches are sized for: the upper end of the class
    of the step's longest context, so that every step of a class launches alike (a captured
    graph is replayed for all of them)."""
    from .engine.batch import CONTEXT_CLASS_BOUNDS as bounds
    c = decode_context_class(int(batch.max_ctx_len))
    return bounds[0] if c == 4 else (bounds[1] if c == 8 else 1 << 30)


def decode_attention_mma(qkv, k_pages, v_pages, write_kv, block_table, q_start, ctx_len, cos, sin, rot,
                         nq, nkv, d, scale, window, status, max_ctx: int = 0,
                         trace: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The attention of a bfloat16 decode step in one launch on tensor cores: rotary
    encoding of query and new key, cache write, attention over 128-key tiles spread over
    a cluster of blocks, merge through distributed shared memory.  No scratch.
    A token's tiles fall into 4 classes below position 2048, 8 below 8192, 16 beyond (head
    size 64), whatever the batch; up to that many blocks share a (request, kv head).
    ``max_ctx``: the longest context of the step if the host knows it (the launch is sized
    for it), 0 otherwise.  ``out``: where the rows go ([tokens, nq d], the rows of the requests'
    tokens are written); made here if not given."""
    _need_cuda(qkv, k_pages)
    assert qkv.dtype == torch.bfloat16
    R = ctx_len.numel()
    if out is None:
        out = new((qkv.shape[0], nq * d), qkv.dtype, qkv.device)
    rc = lib("decode_attention").kvb_decode_attention_mma(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), c_int(1 if write_kv else 0), _p(block_table),
        c_int(block_table.shape[1]), c_int(k_pages.shape[2]), c_int(k_pages.shape[0]), _p(q_start), _p(ctx_len),
        _p(cos), _p(sin), c_int(0 if cos is None else cos.shape[0]), c_int(rot), _p(out), c_int(R), c_int(nq),
        c_int(nkv), c_int(d), c_float(scale), c_int(int(window or 0)), c_int(int(max_ctx)),
        _p(status), _p(trace), _stream())
    _check(rc, "decode_attention_mma")
    choices["decode_attention_mma"] += 1
    return out


def attention_step(qkv, k_pages, v_pages, write_kv, block_table, batch, nq, nkv, d, scale, window, max_positions,
                   cos, sin, rot) -> torch.Tensor:
    """Everything between the q|k|v projection and the output projection: rotary
    encoding, the write of keys and values into their pages, attention over the pages.
    Picks the kernels:
    * float32: rotary/write kernel, then the general kernel, whose sums follow absolute
      positions in one fixed order whatever the shape of the step;
    * bfloat16, single tokens only: one fused launch, on tensor cores where the sizes allow
      (head size 64/128), else the FMA form (head size 32);
    * bfloat16, runs of tokens: rotary/write kernel, then the tensor-core kernel; single tokens
      beside them (they are the step's first rows) go to the fused launch of decode steps;
    * sizes neither takes: rotary/write kernel, then the general kernel."""
    group, page_size = nq // nkv, k_pages.shape[2]
    if qkv.dtype == torch.bfloat16 and batch.decode_only and decode_attention_mma_supported(d, group, page_size):
        return decode_attention_mma(qkv, k_pages, v_pages, write_kv, block_table, batch.q_start, batch.ctx_len,
                                    cos, sin, rot, nq, nkv, d, scale, window, batch.status,
                                    max_ctx=decode_launch_context(batch))
    if qkv.dtype == torch.bfloat16 and batch.decode_only and decode_attention_supported(d, group):
        return decode_attention_fused(qkv, k_pages, v_pages, write_kv, block_table, batch.q_start, batch.ctx_len,
                                      cos, sin, rot, nq, nkv, d, scale, window, max_positions, batch.status)
    ns = int(getattr(batch, "num_single", 0))
    if (qkv.dtype == torch.bfloat16 and ns > 0 and flash_attention_supported(d, group, page_size)
            and decode_attention_mma_supported(d, group, page_size)):
        # Single tokens beside runs: the single tokens (the step's first rows) go to the kernel of
        # decode steps, which rotates, writes and attends in one launch, the runs to the two kernels
        # for runs.  As a tile of the kernel for runs a single token would fill 4 of 128 rows.
        out = new((qkv.shape[0], nq * d), qkv.dtype, qkv.device)
        decode_attention_mma(qkv, k_pages, v_pages, write_kv, block_table[:ns], batch.q_start[:ns + 1], batch.ctx_len[:ns],
                             cos, sin, rot, nq, nkv, d, scale, window, batch.status,
                             max_ctx=decode_launch_context(batch), out=out)
        rope_kv_write(qkv[ns:], batch.positions[ns:], batch.token_req[ns:], cos, sin, k_pages if write_kv else None,
                      v_pages if write_kv else None, block_table, page_size, nq, nkv, d, rot, batch.status)
        return flash_attention(qkv, k_pages, v_pages, block_table, batch, nq, nkv, d, scale, window,
                               skip_single=True, out=out)
    rope_kv_write(qkv, batch.positions, batch.token_req, cos, sin, k_pages if write_kv else None,
                  v_pages if write_kv else None, block_table, page_size, nq, nkv, d, rot, batch.status)
    if qkv.dtype == torch.bfloat16 and not batch.decode_only and flash_attention_supported(d, group, page_size):
        return flash_attention(qkv, k_pages, v_pages, block_table, batch, nq, nkv, d, scale, window)
    return paged_attention_generic(qkv, k_pages, v_pages, block_table, batch.positions, batch.token_req,
                                   nq, nkv, d, scale, window, batch.status)


# ------------------------------------------------------------------ sampling

def sample(logits, temperature, seed, key, pos, penalty, mask, slots, out=None, status=None,
           status_at: int = 0) -> torch.Tensor:
    """One token id per row of float32 ``logits``.  ``temperature`` None: greedy for all
    rows; ``penalty``/``mask`` None: no repetition penalty.  ``status``: the kernels' error
    word, copied to ``out[status_at]`` so that it travels with the tokens."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    R, V = logits.shape
    if out is None:
        out = new((R,), torch.int32, logits.device)
    rc = lib("sampling").kvb_sample(_p(logits), c_int(R), c_int(V), _p(temperature), _p(seed), _p(key),
                                    _p(pos), _p(penalty), _p(mask), _p(slots), _p(out), _p(status),
                                    c_int(status_at), _stream())
    _check(rc, "sample")
    return out


def reset_mask(mask: torch.Tensor, slot: int, tokens: Optional[torch.Tensor]) -> None:
    """Clears the slot's row of produced-token marks and marks ``tokens`` (int32, device)."""
    n = 0 if tokens is None else tokens.numel()
    rc = lib("sampling").kvb_reset_mask(_p(mask), c_int(slot), c_int(mask.shape[1]), _p(tokens), c_int(n),
                                        _stream())
    _check(rc, "reset_mask")


# ------------------------------------------------------------------ bfloat16 matrix products (tcgen05)

def gemm_skinny_plan(M: int, N: int, K: int):
    """(blocks along K, tiles along N) of the skinny tensor-core kernel, or None if it
    does not take the sizes."""
    splits, tiles = c_int(0), c_int(0)
    rc = lib("gemm_bf16").kvb_gemm_skinny_plan(c_int(M), c_int(N), c_int(K), ctypes.byref(splits), ctypes.byref(tiles))
    if rc != 0:
        return None
    return splits.value, tiles.value


FUSED_EPILOGUE_MAX_ROWS = int(os.environ.get('KVB200_FUSED_MAX_ROWS', '32'))   # the kernel takes up to 64


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, status: torch.Tensor,
                x_is_static: bool = False, trace: Optional[torch.Tensor] = None, epilogue: str = "store") -> torch.Tensor:
    """``x . w^T`` for few rows (M <= 256) on tcgen05 tensor cores, weights streamed by TMA.

    ``epilogue``: "store", or "swiglu": ``w`` holds gate and up rows in alternating blocks
    of 64 and ``silu(gate) * up`` [M, N/2] is returned (up to 64 rows)."""
    _need_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    code = {"store": 0, "swiglu": 1}[epilogue]
    out = new((M, N // 2 if code == 1 else N), out_dtype, x.device)
    rc = lib("gemm_bf16").kvb_gemm_skinny(
        _p(x), c_int(x.stride(0)), _p(w), c_int(w.stride(0)), _p(out), c_int(1 if out_dtype == torch.float32 else 0),
        c_int(M), c_int(N), c_int(K), c_int(1 if x_is_static else 0), c_int(code), _p(status), _p(trace),
        _stream())
    if rc == -2:
        raise KernelError(f"gemm_skinny refuses M={M}, N={N}, K={K} (M <= 256 and K a multiple of 8 are required)")
    _check(rc, "gemm_skinny")
    choices["gemm_skinny"] += 1
    return out


def gemm_skinny_fused(x: torch.Tensor, w: torch.Tensor, status: torch.Tensor, row_scale: Optional[PendingNorm] = None,
                      into: Optional[torch.Tensor] = None, epilogue: str = "store", x_is_static: bool = False,
                      trace: Optional[torch.Tensor] = None):
    """The skinny product (up to 64 rows) with the residual stream's add and RMSNorm folded around it.

    ``row_scale``: every row of ``x . w^T`` is multiplied by the 1/rms that follows from the
    pending norm's partial sums (``x`` is then its bare bfloat16 rows, and ``w`` has the
    norm's weight multiplied into its columns).  ``into``: the product is added into this
    float32 residual in place and a :class:`Folded` is returned; otherwise the product
    (``epilogue`` "store" or "swiglu") as a bfloat16 tensor."""
    _need_cuda(x, w)
    N, K = w.shape
    M = x.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    assert x.shape[1] == K and M <= 64
    ss, parts, eps = None, 0, 0.0
    if row_scale is not None:
        ss, eps = row_scale.sumsq, row_scale.eps
        assert into is None and ss.dtype == torch.float32 and ss.is_contiguous() and ss.shape[0] == M
        parts = ss.shape[1]
    out = sumsq = xb = None
    if into is not None:
        assert epilogue == "store" and into.dtype == torch.float32 and into.shape == (M, N) and into.stride(1) == 1
        code = 2
        sumsq = new((M, -(-N // 128)), torch.float32, x.device)
        xb = new((M, N), torch.bfloat16, x.device)
    else:
        code = {"store": 0, "swiglu": 1}[epilogue]
        out = new((M, N // 2 if code == 1 else N), torch.bfloat16, x.device)
    rc = lib("gemm_bf16").kvb_gemm_skinny_fused(
        _p(x), c_int(x.stride(0)), _p(w), c_int(w.stride(0)), _p(out), c_int(M), c_int(N), c_int(K),
        c_int(1 if x_is_static else 0), c_int(code), _p(ss), c_int(parts), c_float(eps),
        _p(into), c_int(into.stride(0) if into is not None else 0), _p(xb), _p(sumsq), _p(status), _p(trace),
        _stream())
    if rc == -2:
        raise KernelError(f"gemm_skinny_fused refuses M={M}, N={N}, K={K}, epilogue {epilogue}")
    _check(rc, "gemm_skinny_fused")
    choices["gemm_skinny_fused"] += 1
    return Folded(xb, sumsq) if into is not None else out


def gemm_wide(x: torch.Tensor, w: torch.Tensor, status: torch.Tensor, epilogue: str = "store",
              tile=(0, 0), row_scale: Optional[PendingNorm] = None, into: Optional[torch.Tensor] = None):
    """``x . w^T`` for steps of many rows on tcgen05 tensor cores: a persistent kernel with a TMA
    loader warp, an issuing warp and four epilogue warps, two accumulators in tensor memory.

    ``epilogue``: "store", or "swiglu": ``w`` holds gate and up rows in alternating blocks
    of 64 and ``silu(gate) * up`` [M, N/2] is returned.  ``tile``: (rows of x, features) per
    tile, one of (128, 64), (128, 128), (128, 256), (256, 256); (256, 256, 1): such a tile shared
    by the two blocks of a cluster; (0, 0) for the kernel's own choice.

    ``row_scale``: every row of ``x . w^T`` is multiplied by the 1/rms that follows from the
    pending norm's partial sums (``x`` is then its bare bfloat16 rows, and ``w`` has the
    norm's weight multiplied into its columns).  ``into``: the product is added into this
    float32 residual in place and a :class:`Folded` is returned."""
    _need_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    assert w.shape[1] == K
    ss, parts, eps = None, 0, 0.0
    if row_scale is not None:
        ss, eps = row_scale.sumsq, row_scale.eps
        assert into is None and ss.dtype == torch.float32 and ss.is_contiguous() and ss.shape[0] == M
        parts = ss.shape[1]
    out = xb = sumsq = None
    if into is not None:
        assert epilogue == "store" and into.dtype == torch.float32 and into.shape == (M, N) and into.stride(1) == 1
        code = 2
        sumsq = new((M, -(-N // 256)), torch.float32, x.device)
        xb = new((M, N), torch.bfloat16, x.device)
    else:
        code = {"store": 0, "swiglu": 1}[epilogue]
        out = new((M, N // 2 if code == 1 else N), torch.bfloat16, x.device)
    rc = lib("gemm_bf16_wide").kvb_gemm_wide_fused(
        _p(x), c_int(x.stride(0)), _p(w), c_int(w.stride(0)), _p(out), c_int(out.stride(0) if out is not None else 0),
        c_int(M), c_int(N), c_int(K), c_int(code), c_int(tile[0]), c_int(tile[1]),
        c_int(tile[2] if len(tile) > 2 else 0), _p(ss), c_int(parts), c_float(eps), _p(into),
        c_int(into.stride(0) if into is not None else 0), _p(xb), _p(sumsq), _p(status), _stream())
    if rc in (-2, -3):
        raise KernelError(f"gemm_wide refuses M={M}, N={N}, K={K}, epilogue {epilogue}, tile {tile} (K and N "
                          "multiples of 8, N a multiple of 128 for swiglu, 16-byte aligned rows are required)")
    _check(rc, "gemm_wide")
    choices["gemm_wide"] += 1
    return Folded(xb, sumsq) if into is not None else out


def wait_selftest(polls: int, status: torch.Tensor) -> None:
    """Lets the product kernels' bounded barrier wait run out on a barrier that nothing
    completes: ``status`` receives the wait-timeout code, the kernel returns."""
    rc = lib("gemm_bf16").kvb_wait_selftest(ctypes.c_uint(int(polls)), _p(status), _stream())
    _check(rc, "wait_selftest")


def decode_wait_selftest(polls: int, status: torch.Tensor) -> torch.Tensor:
    """Runs the decode attention's bounded wait (head size 128 waits for its pages on mbarriers) against barriers
    that nothing completes: one warp gives up after ``polls`` polls, reports KVB_STATUS_WAIT_TIMEOUT in ``status``
    and raises the block's flag, by which the other warp leaves.  Returns [flag, whether the other warp's wait
    claimed success] as an int32 tensor."""
    flags = torch.full((2,), -1, dtype=torch.int32, device=status.device)
    rc = lib("decode_attention").kvb_decode_wait_selftest(ctypes.c_uint(int(polls)), _p(status), _p(flags), _stream())
    _check(rc, "decode_wait_selftest")
    return flags
