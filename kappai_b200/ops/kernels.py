"""Python faces of the CUDA kernels.

Each function checks its tensors (device, dtype, layout), launches on the
current CUDA stream and raises on any error.  There is no CPU path: a tensor
that is not on a CUDA device is refused.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .build import is_loaded, load_library

F32, BF16 = 0, 1
EPI_STORE, EPI_STORE_F32, EPI_ACCUM_F32 = 0, 1, 2


MAX_STEP_ROWS = 65535     # rows of one step: the row-wise kernels put rows on a grid axis that ends there

LAUNCHES = [0]      # kernel launchers called so far (a launcher may launch more than one kernel)
LAUNCHES_BY = {}    # the same by launcher name


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dt}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current CUDA stream of the current device (asked of torch's C layer directly where it offers that:
    this runs once per kernel launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor (kappai_b200 has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: expected a contiguous tensor")


class _Stream:
    """Stands for "the current stream" among a launcher's arguments."""


STREAM = _Stream()


class KernelTimer:
    """Device time by kernel class: while one is installed (``TIMER[0]``), every launcher call is put between
    two CUDA events on its stream; ``report`` adds them up by class.  The reference keeps per-stage counters of
    the same kind (src/profile.h:9-47,77-88) and prints them with ``--time`` (src/profile.c:65-110).  A class is
    the launcher's name, for matrix products with the weight's shape.  Only launches made one by one are seen:
    the engine runs its steps eagerly (no captured graphs) while it is timed, so the times of small kernels
    include the gap the host leaves before them."""

    FOLD_AT = 8192

    def __init__(self):
        self._open = []                    # (class, event before, event after, flops, bytes)
        self.totals = {}                   # class -> [calls, ms, flops, bytes]

    def add(self, key, e0, e1, work) -> None:
        self._open.append((key, e0, e1, work))
        if len(self._open) >= self.FOLD_AT:
            self.fold()

    def fold(self) -> None:
        if not self._open:
            return
        self._open[-1][2].synchronize()
        for key, e0, e1, work in self._open:
            t = self.totals.setdefault(key, [0, 0.0, 0, 0])
            t[0] += 1
            t[1] += e0.elapsed_time(e1)
            if work:
                t[2] += work[0]
                t[3] += work[1]
        self._open = []

    def report(self):
        """Rows (class, calls, ms, microseconds a call, share in per cent, TFLOP/s or None, GB/s or None),
        the class that took longest first."""
        self.fold()
        total = sum(t[1] for t in self.totals.values()) or 1.0
        rows = []
        for key, (calls, ms, flops, nbytes) in sorted(self.totals.items(), key=lambda kv: -kv[1][1]):
            rows.append((key, calls, ms, ms * 1e3 / calls, 100.0 * ms / total,
                         flops / (ms * 1e-3) / 1e12 if flops and ms > 0 else None,
                         nbytes / (ms * 1e-3) / 1e9 if nbytes and ms > 0 else None))
        return rows

    def format(self, label: str = "kernels") -> str:
        rows = self.report()
        total = sum(r[2] for r in rows)
        out = [f"[profile] {label}  accounted={total * 1e3:.0f} us",
               f"  {'class':<34} {'ms':>10} {'calls':>8} {'us/call':>9} {'share':>7} {'TFLOP/s':>8} {'GB/s':>8}"]
        for key, calls, ms, per, share, tf, gb in rows:
            out.append(f"  {key:<34} {ms:>10.3f} {calls:>8d} {per:>9.2f} {share:>6.2f}% "
                       f"{'' if tf is None else format(tf, '8.1f'):>8} {'' if gb is None else format(gb, '8.1f'):>8}")
        return "\n".join(out)


TIMER = [None]         # the KernelTimer that watches the launches, if any


def _run(what: str, fn, *args, tag: str = "", work=None) -> None:
    """The one door to the kernel libraries: call the launcher ``fn`` on the current stream and check its
    answer.  ``tag`` and ``work`` = (flops, bytes) describe the call to a :class:`KernelTimer`."""
    timer = TIMER[0]
    if timer is None:
        _check(fn(*[_stream() if a is STREAM else a for a in args]), what)
        if LAUNCH_LOG[0] is not None and tag:
            LAUNCH_LOG[0][-1] += tag
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    _check(fn(*[_stream() if a is STREAM else a for a in args]), what)
    e1.record()
    timer.add(what + tag, e0, e1, work)


def _gemm_work(M: int, N: int, K: int, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor):
    return (2 * M * N * K, M * K * a.element_size() + N * K * w.element_size() + out.numel() * out.element_size())


LAUNCH_LOG = [None]        # a list: every launch appends its name (bench.py --probe timeline names a step's kernels by it)


def _check(status: int, what: str) -> None:
    LAUNCHES[0] += 1
    LAUNCHES_BY[what] = LAUNCHES_BY.get(what, 0) + 1
    if LAUNCH_LOG[0] is not None:
        LAUNCH_LOG[0].append(what)
    if status != 0:
        if status == -95:
            raise KernelError(f"{what}: size not supported by this kernel")
        if status == -22:
            raise KernelError(f"{what}: bad argument")
        raise KernelError(f"{what}: CUDA error {status}")


def _rows_2d(t: torch.Tensor, name: str) -> int:
    """Leading dimension (in elements) of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name}: expected a 2-D tensor with contiguous rows")
    return t.stride(0)


# --------------------------------------------------------------- status words
# Kernels that wait on a barrier wait with a limit; one that gives up sets its library's status word, stops
# issuing work and returns.  The engine reads the words of a step with the step's own device-to-host copy.

_STATUS_LIBS = (("gemm_tc", "tc"), ("gemm_stream", "stream"), ("attention_mma", "attention_mma"),
                ("attention_tc", "attention_tc"), ("moe", "moe_tc"))


def read_status() -> dict:
    """Library -> status word (0, or 1 if a bounded wait gave up since the last call) of every kernel library
    that is loaded and has one; the words are cleared.  Synchronises the device."""
    return {lib: _read_one(lib, name) for lib, name in _STATUS_LIBS if is_loaded(lib)}


def _read_one(lib: str, name: str) -> int:
    return int(getattr(load_library(lib), f"kp_{name}_status")()) if is_loaded(lib) else 0


def tc_status() -> int:
    """0, or 1 if a bounded wait of the tcgen05 product kernel gave up since the last call (synchronises)."""
    return _read_one("gemm_tc", "tc")


def stream_status() -> int:
    return _read_one("gemm_stream", "stream")


def attention_tc_status() -> int:
    return _read_one("attention_tc", "attention_tc")


def attention_mma_status() -> int:
    return _read_one("attention_mma", "attention_mma")


class StatusGather:
    """Collects the status words of the loaded kernel libraries (and one word of its own, ``injected``, that
    the host may set: a stand-in for a kernel failure where the real one cannot be made) into one device
    word, with one small kernel behind a step."""

    def __init__(self, device: torch.device):
        self.device = device
        self.injected = torch.zeros(1, dtype=torch.int32, device=device)
        self._libs = None
        self._addrs: Optional[torch.Tensor] = None

    def _refresh(self) -> None:
        libs = tuple(lib for lib, _ in _STATUS_LIBS if is_loaded(lib))
        if libs == self._libs:
            return
        addrs = [self.injected.data_ptr()]
        for lib, name in _STATUS_LIBS:
            if lib in libs:
                fn = getattr(load_library(lib), f"kp_{name}_status_address")
                fn.restype = ctypes.c_void_p
                a = fn()
                if not a:
                    raise KernelError(f"{lib}: no address for its status word")
                addrs.append(int(a))
        self._addrs = torch.tensor(addrs, dtype=torch.int64).to(self.device)
        self._libs = libs

    def gather(self, out: torch.Tensor) -> None:
        """out[0] (int32, on the device) = OR of the status words, in stream order."""
        _need(out, "out", torch.int32)
        self._refresh()
        _run("gather_status", load_library("rowwise").kp_gather_status, _ptr(self._addrs), self._addrs.numel(), _ptr(out), STREAM)

    def clear(self) -> dict:
        """Read and clear every word (synchronises); returns what was set."""
        st = read_status()
        if int(self.injected.item()):
            st["injected"] = 1
            self.injected.zero_()
        return {k: v for k, v in st.items() if v}


# -------------------------------------------------------------------- rowwise

def step_tables(src_pinned: torch.Tensor, dst: torch.Tensor, tokens: Optional[torch.Tensor] = None, tok_off: int = 0) -> None:
    """The int32 tables of a captured step from their staging buffer in pinned host memory to the device buffer
    ``dst`` by a kernel (the device reads the host buffer itself), and with them ``tokens`` (int32, on the device)
    to words ``tok_off`` ... of ``dst``."""
    if src_pinned.dtype != torch.int32 or not src_pinned.is_pinned() or src_pinned.numel() != dst.numel():
        raise KernelError("step_tables: the source is an int32 tensor in pinned memory, as long as the destination")
    _need(dst, "dst", torch.int32)
    n_tok = 0
    if tokens is not None:
        _need(tokens, "tokens", torch.int32)
        n_tok = tokens.numel()
    _run("step_tables", load_library("rowwise").kp_step_tables, ctypes.c_void_p(src_pinned.data_ptr()), _ptr(dst), dst.numel(),
         _ptr(tokens), tok_off, n_tok, STREAM)


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
               pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = table[ids[r]] * scale (+ pos_table[positions[r]], a table of learned position vectors)."""
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    n, d = out.shape
    if table.shape[1] != d or ids.numel() != n:
        raise KernelError("embed_rows: shape mismatch")
    if pos_table is not None:
        _need(pos_table, "pos_table", table.dtype); _need(positions, "positions", torch.int32)
        if pos_table.shape[1] != d or positions.numel() != n:
            raise KernelError("embed_rows: position table shape mismatch")
    lib = load_library("rowwise")
    _run("embed_rows", lib.kp_embed_rows, _ptr(table), _ptr(ids), _ptr(out), n, d, ctypes.c_float(scale),
         _ptr(pos_table), _ptr(positions if pos_table is not None else None), dtype_code(table.dtype), STREAM)
    return out


def rmsnorm_rows(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = rmsnorm(x[rows[r]] if rows is given else x[r])."""
    _need(x, "x", torch.float32); _need(w, "w", torch.float32); _need(out, "out")
    n, d = out.shape
    if x.shape[1] != d or w.numel() != d:
        raise KernelError("rmsnorm_rows: shape mismatch")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() != n:
            raise KernelError("rmsnorm_rows: rows/out mismatch")
    elif x.shape[0] != n:
        raise KernelError("rmsnorm_rows: x/out mismatch")
    lib = load_library("rowwise")
    _run("rmsnorm_rows", lib.kp_rmsnorm_rows, _ptr(x), _ptr(w), _ptr(out), _ptr(rows), n, d, ctypes.c_float(eps),
                               dtype_code(out.dtype), STREAM)
    return out


def layernorm_rows(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
                   rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = (x - mean) / sqrt(var + eps) * w of the float32 row x[rows[r]] (x[r] without ``rows``): a weighted layer
    norm without a shift, the variance taken about the mean."""
    _need(x, "x", torch.float32); _need(w, "w", torch.float32); _need(out, "out")
    n, d = out.shape
    if x.shape[1] != d or w.numel() != d:
        raise KernelError("layernorm_rows: shape mismatch")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() != n:
            raise KernelError("layernorm_rows: rows/out mismatch")
    elif x.shape[0] != n:
        raise KernelError("layernorm_rows: x/out mismatch")
    if n > MAX_STEP_ROWS:
        raise KernelError("layernorm_rows: too many rows")
    _run("layernorm_rows", load_library("rowwise").kp_layernorm_rows, _ptr(x), _ptr(w), _ptr(out), _ptr(rows), n, d,
         ctypes.c_float(eps), dtype_code(out.dtype), STREAM)
    return out


GATE_ACTS = {"silu": 0, "sigmoid": 1}


def group_norm_gate_rows(o: torch.Tensor, w: Optional[torch.Tensor], g: torch.Tensor, eps: float, out: torch.Tensor,
                         groups: int, gate_first: bool, gate_act: str = "silu") -> torch.Tensor:
    """The float32 rows ``o`` [n, c] RMS-normed in ``groups`` stretches of equal width (a mean square a stretch), with a
    gate ``act(g)`` (silu or sigmoid; ``g`` [n, c] in the storage type, rows may be strided) and an optional weight
    ``w`` [c]: ``gate_first`` -> ``norm(o * act(g)) * w``, else ``norm(o) * w * act(g)``."""
    _need(o, "o", torch.float32); _need(out, "out"); _need(g, "g", out.dtype, contiguous=False)
    n, c = o.shape
    if tuple(out.shape) != (n, c) or tuple(g.shape) != (n, c) or groups < 1 or c % groups:
        raise KernelError("group_norm_gate_rows: shape mismatch")
    if w is not None:
        _need(w, "w", torch.float32)
        if w.numel() != c:
            raise KernelError("group_norm_gate_rows: weight size")
    if gate_act not in GATE_ACTS:
        raise KernelError(f"group_norm_gate_rows: gate '{gate_act}' (silu or sigmoid)")
    if n > MAX_STEP_ROWS:
        raise KernelError("group_norm_gate_rows: too many rows")
    _run("group_norm_gate_rows", load_library("rowwise").kp_group_norm_gate_rows, _ptr(o), c, _ptr(w), _ptr(g), _rows_2d(g, "g"),
         _ptr(out), c, n, int(groups), c // int(groups), ctypes.c_float(eps), int(bool(gate_first)), GATE_ACTS[gate_act],
         dtype_code(out.dtype), STREAM)
    return out


def head_gate(o: torch.Tensor, g: torch.Tensor, H: int, hd: int) -> torch.Tensor:
    """o[r, h hd + i] *= sigmoid(g[r, h]) in place: one gate a head (``g`` [n, H], rows may be strided)."""
    _need(o, "o"); _need(g, "g", o.dtype, contiguous=False)
    n = o.shape[0]
    if tuple(o.shape) != (n, H * hd) or tuple(g.shape) != (n, H):
        raise KernelError("head_gate: shape mismatch")
    _run("head_gate", load_library("rowwise").kp_head_gate, _ptr(o), H * hd, _ptr(g), _rows_2d(g, "g"), n, H, hd,
         dtype_code(o.dtype), STREAM)
    return o


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (float32)."""
    _need(x, "x", torch.float32)
    if not cap > 0:
        raise KernelError("softcap: the cap must be positive")
    _run("softcap", load_library("rowwise").kp_softcap, _ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), STREAM)
    return x


def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float, shift: float) -> torch.Tensor:
    """out = g sigmoid(alpha g) (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit), rows [gate | up]."""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    n, ff = out.shape
    if gate_up.shape != (n, 2 * ff):
        raise KernelError("glu_clamped: shape mismatch")
    _run("glu_clamped", load_library("rowwise").kp_glu_clamped, _ptr(gate_up), _ptr(out), n, ff, ctypes.c_float(limit),
         ctypes.c_float(alpha), ctypes.c_float(shift), dtype_code(out.dtype), STREAM)
    return out


ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2}     # codes of the gated units' activations (csrc/common.cuh)


def activation_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation '{name}': expected one of {', '.join(ACTIVATIONS)}") from None


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """out = act(gate) * up for rows [gate | up]."""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    n, ff = out.shape
    if gate_up.shape != (n, 2 * ff):
        raise KernelError("swiglu: shape mismatch")
    lib = load_library("rowwise")
    _run("swiglu", lib.kp_swiglu, _ptr(gate_up), _ptr(out), n, ff, activation_code(activation), dtype_code(out.dtype), STREAM)
    return out


def postnorm_rows(acc: torch.Tensor, w: torch.Tensor, eps: float, x_out: Optional[torch.Tensor] = None,
                  h_out: Optional[torch.Tensor] = None, scaled_out: Optional[torch.Tensor] = None,
                  alpha: float = 1.0) -> None:
    """y = rmsnorm(acc) * w for the float32 rows of ``acc``; y goes to ``x_out`` (float32), ``h_out`` (any
    storage type) and, times ``alpha``, to ``scaled_out`` (float32), whichever are given (each may be ``acc``)."""
    _need(acc, "acc", torch.float32); _need(w, "w", torch.float32)
    n, d = acc.shape
    if w.numel() != d:
        raise KernelError("postnorm_rows: weight size")
    for t, nm, dt in ((x_out, "x_out", torch.float32), (h_out, "h_out", None), (scaled_out, "scaled_out", torch.float32)):
        if t is not None:
            _need(t, nm, dt)
            if tuple(t.shape) != (n, d):
                raise KernelError(f"postnorm_rows: {nm} shape")
    if n > MAX_STEP_ROWS:
        raise KernelError("postnorm_rows: too many rows")
    code = dtype_code(h_out.dtype) if h_out is not None else F32
    _run("postnorm_rows", load_library("rowwise").kp_postnorm_rows, _ptr(acc), _ptr(w), _ptr(x_out), _ptr(h_out),
         _ptr(scaled_out), n, d, ctypes.c_float(eps), ctypes.c_float(alpha), code, STREAM)


def scale_cast(x: torch.Tensor, h_out: Optional[torch.Tensor], scaled_out: torch.Tensor, alpha: float) -> None:
    """h_out = x in h_out's type (if given), scaled_out = alpha * x (float32)."""
    _need(x, "x", torch.float32); _need(scaled_out, "scaled_out", torch.float32)
    if h_out is not None:
        _need(h_out, "h_out")
        if h_out.numel() != x.numel():
            raise KernelError("scale_cast: size mismatch")
    if scaled_out.numel() != x.numel():
        raise KernelError("scale_cast: size mismatch")
    code = dtype_code(h_out.dtype) if h_out is not None else F32
    _run("scale_cast", load_library("rowwise").kp_scale_cast, _ptr(x), _ptr(h_out), _ptr(scaled_out),
         ctypes.c_longlong(x.numel()), ctypes.c_float(alpha), code, STREAM)


def sigmoid_gate(o: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """o *= sigmoid(g), element by element; both 2-D with contiguous rows (``g`` may be columns of a wider tensor)."""
    _need(o, "o", contiguous=False); _need(g, "g", o.dtype, contiguous=False)
    if o.shape != g.shape:
        raise KernelError("sigmoid_gate: shape mismatch")
    _run("sigmoid_gate", load_library("rowwise").kp_sigmoid_gate, _ptr(o), _rows_2d(o, "o"), _ptr(g), _rows_2d(g, "g"),
         o.shape[0], o.shape[1], dtype_code(o.dtype), STREAM)
    return o


def rmsnorm_cols(x: torch.Tensor, stretches, eps: float) -> None:
    """RMS norm of one or two column stretches of the rows of ``x`` (storage type), each on its own:
    ``stretches`` = [(first column, weight float32 [width], out [n, width] in x's type), ...]."""
    _need(x, "x", contiguous=False)
    if not 1 <= len(stretches) <= 2:
        raise KernelError("rmsnorm_cols: one or two stretches")
    n = x.shape[0]
    args = []
    for col, w, out in stretches:
        _need(w, "weight", torch.float32); _need(out, "out", x.dtype, contiguous=False)
        width = w.numel()
        if col < 0 or col + width > x.shape[1] or tuple(out.shape) != (n, width):
            raise KernelError("rmsnorm_cols: shape mismatch")
        args += [int(col), width, _ptr(w), _ptr(out), _rows_2d(out, "out")]
    if len(stretches) == 1:
        args += [0, 0, _ptr(None), _ptr(None), 0]
    _run("rmsnorm_cols", load_library("rowwise").kp_rmsnorm_cols, _ptr(x), _rows_2d(x, "x"), n, ctypes.c_float(eps), *args,
         dtype_code(x.dtype), STREAM)


def norm_gate_rows(o: torch.Tensor, w: torch.Tensor, g: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = rmsnorm(o) * w * sigmoid(g): float32 rows ``o`` normed whole, gated by columns ``g`` of a wider row."""
    _need(o, "o", torch.float32); _need(w, "w", torch.float32); _need(g, "g", contiguous=False)
    _need(out, "out", g.dtype, contiguous=False)
    n, d = o.shape
    if w.numel() != d or tuple(g.shape) != (n, d) or tuple(out.shape) != (n, d):
        raise KernelError("norm_gate_rows: shape mismatch")
    _run("norm_gate_rows", load_library("rowwise").kp_norm_gate_rows, _ptr(o), _ptr(w), _ptr(g), _rows_2d(g, "g"), _ptr(out),
         _rows_2d(out, "out"), n, d, ctypes.c_float(eps), dtype_code(g.dtype), STREAM)
    return out


def token_gate(gate: torch.Tensor, table: torch.Tensor, col0: int, ids: torch.Tensor, out: torch.Tensor,
               activation: str = "gelu_tanh") -> torch.Tensor:
    """out[r, c] = act(gate[r, c]) * table[ids[r], col0 + c]."""
    _need(gate, "gate", contiguous=False); _need(table, "table", gate.dtype, contiguous=False)
    _need(ids, "ids", torch.int32); _need(out, "out", gate.dtype)
    n, dim = gate.shape
    if tuple(out.shape) != (n, dim) or ids.numel() != n or col0 < 0 or col0 + dim > table.shape[1]:
        raise KernelError("token_gate: shape mismatch")
    _run("token_gate", load_library("rowwise").kp_token_gate, _ptr(gate), _rows_2d(gate, "gate"), _ptr(table),
         _rows_2d(table, "table"), int(col0), _ptr(ids), _ptr(out), n, dim, activation_code(activation),
         dtype_code(gate.dtype), STREAM)
    return out


def rmsnorm_add_rows(y: torch.Tensor, w: torch.Tensor, eps: float, x: torch.Tensor) -> torch.Tensor:
    """x += rmsnorm(y) * w (all float32)."""
    _need(y, "y", torch.float32); _need(w, "w", torch.float32); _need(x, "x", torch.float32)
    n, d = x.shape
    if tuple(y.shape) != (n, d) or w.numel() != d:
        raise KernelError("rmsnorm_add_rows: shape mismatch")
    _run("rmsnorm_add_rows", load_library("rowwise").kp_rmsnorm_add_rows, _ptr(y), _ptr(w), _ptr(x), n, d, ctypes.c_float(eps), STREAM)
    return x


def rmsnorm_add_norm_rows(y: torch.Tensor, w_branch: torch.Tensor, eps_branch: float, x: torch.Tensor,
                          w_next: Optional[torch.Tensor] = None, eps_next: float = 0.0,
                          h_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += rmsnorm(y) * w_branch (float32), y cleared; with ``w_next`` and ``h_out`` also
    ``h_out = rmsnorm(x) * w_next`` of the new x, in ``h_out``'s type: the norms behind one sublayer and in front
    of the next in one launch."""
    _need(y, "y", torch.float32); _need(w_branch, "w_branch", torch.float32); _need(x, "x", torch.float32)
    n, d = x.shape
    if tuple(y.shape) != (n, d) or w_branch.numel() != d or (w_next is None) != (h_out is None):
        raise KernelError("rmsnorm_add_norm_rows: shape mismatch")
    if n > MAX_STEP_ROWS:
        raise KernelError("rmsnorm_add_norm_rows: too many rows")
    if h_out is not None:
        _need(w_next, "w_next", torch.float32); _need(h_out, "h_out")
        if tuple(h_out.shape) != (n, d) or w_next.numel() != d:
            raise KernelError("rmsnorm_add_norm_rows: shape mismatch")
    _run("rmsnorm_add_norm_rows", load_library("rowwise").kp_rmsnorm_add_norm_rows, _ptr(y), _ptr(w_branch),
         ctypes.c_float(eps_branch), _ptr(x), _ptr(w_next), ctypes.c_float(eps_next), _ptr(h_out), n, d,
         dtype_code(h_out.dtype if h_out is not None else torch.float32), STREAM)
    return x


def row_gate_add(h: torch.Tensor, w_gate: torch.Tensor, y: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] += sigmoid(h[r] . w_gate) * y[r]: ``w_gate`` float32 [d], ``y`` and ``out`` float32 [n, d]."""
    _need(h, "h", contiguous=False); _need(w_gate, "w_gate", torch.float32); _need(y, "y", torch.float32)
    _need(out, "out", torch.float32)
    n, d = h.shape
    if w_gate.numel() != d or tuple(y.shape) != (n, d) or tuple(out.shape) != (n, d):
        raise KernelError("row_gate_add: shape mismatch")
    _run("row_gate_add", load_library("rowwise").kp_row_gate_add, _ptr(h), _rows_2d(h, "h"), _ptr(w_gate), _ptr(y), _ptr(out),
         n, d, dtype_code(h.dtype), STREAM)
    return out


def cast(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    _need(src, "src"); _need(dst, "dst")
    if src.numel() != dst.numel():
        raise KernelError("cast: size mismatch")
    lib = load_library("rowwise")
    _run("cast", lib.kp_cast, _ptr(src), _ptr(dst), ctypes.c_longlong(src.numel()), dtype_code(src.dtype),
                       dtype_code(dst.dtype), STREAM)
    return dst


# ----------------------------------------------------------------------- gemm

def gemm_nt_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 accumulate: bool = False) -> torch.Tensor:
    """out = a @ w.T (+ bias); with ``accumulate`` out (float32) += that."""
    _need(a, "a", contiguous=False); _need(w, "w", a.dtype, contiguous=False); _need(out, "out", contiguous=False)
    lda, ldw, ldc = _rows_2d(a, "a"), _rows_2d(w, "w"), _rows_2d(out, "out")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("gemm: bias size")
    if accumulate:
        if out.dtype != torch.float32:
            raise KernelError("gemm: accumulation needs a float32 output")
        epi = EPI_ACCUM_F32
    elif out.dtype == a.dtype:
        epi = EPI_STORE
    elif out.dtype == torch.float32:
        epi = EPI_STORE_F32
    else:
        raise KernelError("gemm: output dtype must be the operand dtype or float32")
    lib = load_library("gemm_simt")
    _run("gemm_nt_simt", lib.kp_gemm_nt_simt, _ptr(a), _ptr(w), _ptr(bias), _ptr(out), M, N, K, lda, ldw, ldc, epi,
         dtype_code(a.dtype), STREAM, tag=f" {N}x{K}", work=_gemm_work(M, N, K, a, w, out))
    return out


# ------------------------------------------------------------------ shortconv

def shortconv_forward(p: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                      row_seg: torch.Tensor, cu_rows: torch.Tensor, seg_pos: torch.Tensor,
                      seg_slot: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(p, "p", contiguous=False); _need(w, "w", torch.float32); _need(state, "state", torch.float32)
    _need(out, "out", p.dtype, contiguous=False)
    for t, nm in ((row_seg, "row_seg"), (cu_rows, "cu_rows"), (seg_pos, "seg_pos"), (seg_slot, "seg_slot")):
        _need(t, nm, torch.int32)
    n, d = out.shape
    K = w.shape[1]
    if p.shape != (n, 3 * d) or w.shape[0] != d or state.shape[1:] != (K - 1, d):
        raise KernelError("shortconv_forward: shape mismatch")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    lib = load_library("shortconv")
    _run("shortconv_forward", lib.kp_shortconv_forward, _ptr(p), _rows_2d(p, "p"), _ptr(w), _ptr(bias), _ptr(state), _ptr(row_seg),
                                    _ptr(cu_rows), _ptr(seg_pos), _ptr(seg_slot), _ptr(out), _rows_2d(out, "out"),
                                    n, d, K, dtype_code(p.dtype), STREAM)
    return out


def shortconv_decode(p: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                     seg_pos: torch.Tensor, seg_slot: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Output and state update in one launch, for steps in which every segment is one row."""
    _need(p, "p", contiguous=False); _need(w, "w", torch.float32); _need(state, "state", torch.float32)
    _need(out, "out", p.dtype, contiguous=False)
    _need(seg_pos, "seg_pos", torch.int32); _need(seg_slot, "seg_slot", torch.int32)
    n, d = out.shape
    K = w.shape[1]
    if p.shape != (n, 3 * d) or w.shape[0] != d or state.shape[1:] != (K - 1, d) or seg_pos.numel() != n:
        raise KernelError("shortconv_decode: shape mismatch")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    lib = load_library("shortconv")
    _run("shortconv_decode", lib.kp_shortconv_decode, _ptr(p), _rows_2d(p, "p"), _ptr(w), _ptr(bias), _ptr(state), _ptr(seg_pos),
                                   _ptr(seg_slot), _ptr(out), _rows_2d(out, "out"), n, d, K, dtype_code(p.dtype),
                                   STREAM)
    return out


def shortconv_update_state(p: torch.Tensor, state: torch.Tensor, cu_rows: torch.Tensor, seg_pos: torch.Tensor,
                           seg_slot: torch.Tensor, n_seg: int) -> None:
    _need(p, "p", contiguous=False); _need(state, "state", torch.float32)
    d = p.shape[1] // 3
    K = state.shape[1] + 1
    if state.shape[2] != d:
        raise KernelError("shortconv_update_state: shape mismatch")
    lib = load_library("shortconv")
    _run("shortconv_update_state", lib.kp_shortconv_update_state, _ptr(p), _rows_2d(p, "p"), _ptr(state), _ptr(cu_rows), _ptr(seg_pos),
                                         _ptr(seg_slot), n_seg, d, K, dtype_code(p.dtype), STREAM)


# ------------------------------------------------------------------ linear attention with decay

LIGHTNING_MAX_DIM = 256    # key rows of a head's state that the scan keeps in registers


def lightning_scan(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, decay_hi: torch.Tensor, decay_lo: torch.Tensor,
                   state: torch.Tensor, cu_rows: torch.Tensor, seg_pos: torch.Tensor, seg_slot: torch.Tensor,
                   out: torch.Tensor, n_seg: int, H: int, dim: int, vdim: int, activation: Optional[str] = "silu",
                   write_state: bool = True, rotary=None, k_scale: float = 1.0) -> torch.Tensor:
    """``S <- a_h S + k v^T; o = S^T q`` row after row of every segment, from the state in the segment's slot (zero at
    position 0) and back into it.  q, k (H heads of ``dim``) and v (H heads of ``vdim``) are columns of ``qkv`` in
    the storage type with ``activation`` (silu or None) applied here; ``out`` float32 [n, H vdim];
    ``state`` float32 [slots, H, dim, vdim]; the decays as float32 pairs hi + lo [H].  ``rotary`` = (cos, sin,
    rotated dimensions): q and k are rotated by position as they are read (dimension i paired with i + half; tables
    float32 [positions, half]); ``k_scale`` multiplies k behind the rotation."""
    _need(qkv, "qkv", contiguous=False); _need(out, "out", torch.float32); _need(state, "state", torch.float32)
    _need(decay_hi, "decay_hi", torch.float32); _need(decay_lo, "decay_lo", torch.float32)
    for t, nm in ((cu_rows, "cu_rows"), (seg_pos, "seg_pos"), (seg_slot, "seg_slot")):
        _need(t, nm, torch.int32)
    n = qkv.shape[0]
    if (tuple(out.shape) != (n, H * vdim) or tuple(state.shape[1:]) != (H, dim, vdim) or decay_hi.numel() != H
            or decay_lo.numel() != H or max(q_col, k_col) + H * dim > qkv.shape[1] or v_col + H * vdim > qkv.shape[1]):
        raise KernelError("lightning_scan: shape mismatch")
    if activation not in ("silu", None):
        raise KernelError("lightning_scan: activation is silu or none")
    if dim > LIGHTNING_MAX_DIM:
        raise KernelError(f"lightning_scan: dim={dim} exceeds {LIGHTNING_MAX_DIM}")
    cos, sin, rot = _lightning_rotary(rotary, dim, "lightning_scan")
    _run("lightning_scan", load_library("lightning").kp_lightning_scan, _ptr(qkv), _rows_2d(qkv, "qkv"), int(q_col), int(k_col),
         int(v_col), _ptr(decay_hi), _ptr(decay_lo), _ptr(state), _ptr(cu_rows), _ptr(seg_pos), _ptr(seg_slot), _ptr(out),
         _rows_2d(out, "out"), int(n_seg), H, dim, vdim, 0 if activation == "silu" else 1, int(bool(write_state)),
         _ptr(cos), _ptr(sin), rot, ctypes.c_float(k_scale), dtype_code(qkv.dtype), STREAM, work=(4 * n * H * dim * vdim, 0))
    return out


def _lightning_rotary(rotary, dim: int, what: str):
    """(cos, sin, rotated dimensions) checked; (None, None, 0) for no rotation."""
    if rotary is None:
        return None, None, 0
    cos, sin, rot = rotary
    if cos is None or not rot:
        return None, None, 0
    _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32)
    rot = int(rot)
    if rot < 2 or rot % 2 or rot > dim or cos.dim() != 2 or cos.shape[1] != rot // 2 or sin.shape != cos.shape:
        raise KernelError(f"{what}: rotation of {rot} dimensions does not go with heads of {dim} and tables {tuple(cos.shape)}")
    return cos, sin, rot


LIGHTNING_CHUNK_MAX_DIM = 128    # key rows of a head that the chunked form holds in shared memory


def lightning_chunk_rows() -> int:
    """Rows of a chunk of :func:`lightning_chunks` (its decay table holds the powers 0 .. rows of every head's decay)."""
    return int(load_library("lightning").kp_lightning_chunk_rows())


def lightning_chunks(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, decay_pow: torch.Tensor, state: torch.Tensor,
                     cu_rows: torch.Tensor, seg_pos: torch.Tensor, seg_slot: torch.Tensor, chunk_seg: torch.Tensor,
                     chunk_row0: torch.Tensor, seg_chunk0: torch.Tensor, n_chunks: int, out: torch.Tensor, n_seg: int,
                     H: int, dim: int, vdim: int, activation: Optional[str] = "silu", write_state: bool = True,
                     rotary=None, k_scale: float = 1.0) -> torch.Tensor:
    """The recurrence of :func:`lightning_scan` for segments of many rows: chunks of rows as small matrix products
    (float32 on the CUDA cores), the chunks of all segments side by side: every chunk's own sum, a short serial pass
    over a segment's chunks for the states at their heads, every chunk's outputs.  ``decay_pow``: float32
    [H, rows + 1], the powers ``a_h^m`` (made in double).  Sums have another order than the scan's.  ``chunk_seg`` /
    ``chunk_row0`` [n_chunks]: a chunk's segment and first row (chunks of at most :func:`lightning_chunk_rows` rows,
    a segment's chunks in order); ``seg_chunk0`` [n_seg + 1]: the first chunk of every segment.  ``rotary`` and
    ``k_scale`` as in :func:`lightning_scan`."""
    _need(qkv, "qkv", contiguous=False); _need(out, "out", torch.float32); _need(state, "state", torch.float32)
    _need(decay_pow, "decay_pow", torch.float32)
    for t, nm in ((cu_rows, "cu_rows"), (seg_pos, "seg_pos"), (seg_slot, "seg_slot"), (chunk_seg, "chunk_seg"),
                  (chunk_row0, "chunk_row0"), (seg_chunk0, "seg_chunk0")):
        _need(t, nm, torch.int32)
    n = qkv.shape[0]
    if (tuple(out.shape) != (n, H * vdim) or tuple(state.shape[1:]) != (H, dim, vdim)
            or tuple(decay_pow.shape) != (H, lightning_chunk_rows() + 1) or chunk_seg.numel() < n_chunks
            or chunk_row0.numel() < n_chunks or seg_chunk0.numel() < n_seg + 1
            or max(q_col, k_col) + H * dim > qkv.shape[1] or v_col + H * vdim > qkv.shape[1]):
        raise KernelError("lightning_chunks: shape mismatch")
    if activation not in ("silu", None):
        raise KernelError("lightning_chunks: activation is silu or none")
    if dim > LIGHTNING_CHUNK_MAX_DIM:
        raise KernelError(f"lightning_chunks: dim={dim} exceeds {LIGHTNING_CHUNK_MAX_DIM}")
    cos, sin, rot = _lightning_rotary(rotary, dim, "lightning_chunks")
    scratch = torch.empty(n_chunks * H * dim * vdim, dtype=torch.float32, device=qkv.device)
    _run("lightning_chunks", load_library("lightning").kp_lightning_chunks, _ptr(qkv), _rows_2d(qkv, "qkv"), int(q_col),
         int(k_col), int(v_col), _ptr(decay_pow), _ptr(state), _ptr(cu_rows), _ptr(seg_pos), _ptr(seg_slot), _ptr(chunk_seg),
         _ptr(chunk_row0), _ptr(seg_chunk0), int(n_chunks), _ptr(scratch), _ptr(out), _rows_2d(out, "out"), int(n_seg), H, dim,
         vdim, 0 if activation == "silu" else 1, int(bool(write_state)), _ptr(cos), _ptr(sin), rot, ctypes.c_float(k_scale),
         dtype_code(qkv.dtype), STREAM, work=(4 * n * H * dim * vdim, 0))
    LAUNCHES[0] += 2
    return out


# ------------------------------------------------------------------ selective state space (mamba2)

SSM_MAX_STATE = 256        # rows of a head's state that the scan keeps in registers
SSM_CHUNK_MAX_STATE = 128  # rows of a head's state that the chunked form holds in shared memory
SSM_MAX_TAPS = 16


def ssm_conv(p: torch.Tensor, conv_col: int, dt_col: int, taps: torch.Tensor, bias: torch.Tensor, dt_bias: torch.Tensor,
             a_log: torch.Tensor, kept: torch.Tensor, row_seg: torch.Tensor, cu_rows: torch.Tensor, seg_pos: torch.Tensor,
             seg_slot: torch.Tensor, out: torch.Tensor, dt_out: torch.Tensor, da_out: torch.Tensor, n_seg: int,
             single_rows: bool, keep: bool = True) -> None:
    """``out = silu(conv(p[:, conv_col : conv_col + C]) + bias)`` (a causal convolution a channel, taps [C, K], the
    last tap on the current row; rows before a segment come from the request's kept inputs, zero at position 0),
    ``dt_out = softplus(p[:, dt_col : dt_col + H] + dt_bias)`` and ``da_out = -exp(a_log) * dt_out`` (float32).
    ``kept``: float32 [slots, stride] whose rows begin with the last K - 1 inputs as [K - 1, C]; renewed unless
    ``keep`` is False (``single_rows``: every segment has one row, and one launch does both)."""
    _need(p, "p", contiguous=False); _need(out, "out", p.dtype); _need(kept, "kept", torch.float32, contiguous=False)
    for t, nm in ((taps, "taps"), (bias, "bias"), (dt_bias, "dt_bias"), (a_log, "a_log"), (dt_out, "dt_out"), (da_out, "da_out")):
        _need(t, nm, torch.float32)
    for t, nm in ((row_seg, "row_seg"), (cu_rows, "cu_rows"), (seg_pos, "seg_pos"), (seg_slot, "seg_slot")):
        _need(t, nm, torch.int32)
    n, C = out.shape
    H, K = dt_bias.numel(), taps.shape[1]
    if (p.shape[0] != n or tuple(taps.shape) != (C, K) or bias.numel() != C or a_log.numel() != H or tuple(dt_out.shape) != (n, H)
            or tuple(da_out.shape) != (n, H) or conv_col + C > p.shape[1] or dt_col + H > p.shape[1] or kept.dim() != 2
            or kept.stride(1) != 1 or kept.shape[1] < (K - 1) * C):
        raise KernelError("ssm_conv: shape mismatch")
    if K > SSM_MAX_TAPS:
        raise KernelError(f"ssm_conv: {K} taps exceed {SSM_MAX_TAPS}")
    _run("ssm_conv", load_library("ssm").kp_ssm_conv, _ptr(p), _rows_2d(p, "p"), int(conv_col), int(dt_col), _ptr(taps), _ptr(bias),
         _ptr(dt_bias), _ptr(a_log), _ptr(kept), ctypes.c_longlong(kept.stride(0)), _ptr(row_seg), _ptr(cu_rows), _ptr(seg_pos),
         _ptr(seg_slot), _ptr(out), _ptr(dt_out), _ptr(da_out), n, int(n_seg), C, H, K, int(bool(single_rows)), int(bool(keep)),
         dtype_code(p.dtype), STREAM)
    if keep and not single_rows and K > 1:
        LAUNCHES[0] += 1


def _ssm_check(what, xbc, dt, da, D, state, y, H, G, N, P):
    _need(xbc, "xbc", contiguous=False); _need(y, "y", torch.float32); _need(state, "state", torch.float32, contiguous=False)
    for t, nm in ((dt, "dt"), (da, "da"), (D, "D")):
        _need(t, nm, torch.float32)
    n = xbc.shape[0]
    if (tuple(y.shape) != (n, H * P) or tuple(dt.shape) != (n, H) or tuple(da.shape) != (n, H) or D.numel() != H or H % G
            or xbc.shape[1] < H * P + 2 * G * N or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < H * N * P):
        raise KernelError(f"{what}: shape mismatch")
    return n


def ssm_scan(xbc: torch.Tensor, dt: torch.Tensor, da: torch.Tensor, D: torch.Tensor, state: torch.Tensor, cu_rows: torch.Tensor,
             seg_pos: torch.Tensor, seg_slot: torch.Tensor, y: torch.Tensor, n_seg: int, H: int, G: int, N: int, P: int,
             write_state: bool = True) -> torch.Tensor:
    """``S <- exp(da) S + dt B x^T; y = S^T C + D x`` row after row of every segment, from the state in the segment's
    slot (zero at position 0) and back into it.  ``xbc`` rows hold [x: H heads of P | B: G groups of N | C: the same]
    in the storage type; ``dt``, ``da`` float32 [n, H]; ``state`` float32 [slots, stride] whose rows begin with
    [H, N, P]; ``y`` float32 [n, H P]."""
    n = _ssm_check("ssm_scan", xbc, dt, da, D, state, y, H, G, N, P)
    for t, nm in ((cu_rows, "cu_rows"), (seg_pos, "seg_pos"), (seg_slot, "seg_slot")):
        _need(t, nm, torch.int32)
    if N > SSM_MAX_STATE:
        raise KernelError(f"ssm_scan: state={N} exceeds {SSM_MAX_STATE}")
    _run("ssm_scan", load_library("ssm").kp_ssm_scan, _ptr(xbc), _rows_2d(xbc, "xbc"), H * P, H * P + G * N, _ptr(dt), _ptr(da),
         _ptr(D), _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(cu_rows), _ptr(seg_pos), _ptr(seg_slot), _ptr(y),
         _rows_2d(y, "y"), int(n_seg), H, G, N, P, int(bool(write_state)), dtype_code(xbc.dtype), STREAM,
         work=(4 * n * H * N * P, 0))
    return y


def ssm_chunk_rows() -> int:
    return int(load_library("ssm").kp_ssm_chunk_rows())


def ssm_chunks(xbc: torch.Tensor, dt: torch.Tensor, da: torch.Tensor, D: torch.Tensor, state: torch.Tensor, cu_rows: torch.Tensor,
               seg_pos: torch.Tensor, seg_slot: torch.Tensor, chunk_seg: torch.Tensor, chunk_row0: torch.Tensor,
               seg_chunk0: torch.Tensor, n_chunks: int, y: torch.Tensor, n_seg: int, H: int, G: int, N: int, P: int,
               write_state: bool = True) -> torch.Tensor:
    """The recurrence of :func:`ssm_scan` for segments of many rows, chunks of rows as small float32 matrix products,
    the chunks of all segments side by side (C B^T a group, sums, a serial pass over a segment's chunks, outputs).  The chunk lists
    as in :func:`lightning_chunks`.  Sums have another order than the scan's."""
    n = _ssm_check("ssm_chunks", xbc, dt, da, D, state, y, H, G, N, P)
    for t, nm in ((cu_rows, "cu_rows"), (seg_pos, "seg_pos"), (seg_slot, "seg_slot"), (chunk_seg, "chunk_seg"),
                  (chunk_row0, "chunk_row0"), (seg_chunk0, "seg_chunk0")):
        _need(t, nm, torch.int32)
    if chunk_seg.numel() < n_chunks or chunk_row0.numel() < n_chunks or seg_chunk0.numel() < n_seg + 1:
        raise KernelError("ssm_chunks: chunk lists too short")
    if N > SSM_CHUNK_MAX_STATE:
        raise KernelError(f"ssm_chunks: state={N} exceeds {SSM_CHUNK_MAX_STATE}")
    lib = load_library("ssm")
    lib.kp_ssm_chunks_scratch.restype = ctypes.c_longlong
    scratch = torch.empty(int(lib.kp_ssm_chunks_scratch(int(n_chunks), H, G, N, P)), dtype=torch.float32, device=xbc.device)
    _run("ssm_chunks", load_library("ssm").kp_ssm_chunks, _ptr(xbc), _rows_2d(xbc, "xbc"), H * P, H * P + G * N, _ptr(dt), _ptr(da),
         _ptr(D), _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(cu_rows), _ptr(seg_pos), _ptr(seg_slot), _ptr(chunk_seg),
         _ptr(chunk_row0), _ptr(seg_chunk0), int(n_chunks), _ptr(scratch), _ptr(y), _rows_2d(y, "y"), int(n_seg), H, G, N, P,
         int(bool(write_state)), dtype_code(xbc.dtype), STREAM, work=(4 * n * H * N * P, 0))
    LAUNCHES[0] += 3
    return y


# ------------------------------------------------------------------ attention

def qk_norm_rope_kv(qkv: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
                    cos_tab: Optional[torch.Tensor], sin_tab: Optional[torch.Tensor], rotary_dim: int,
                    interleaved: bool, positions: torch.Tensor, slot_map: Optional[torch.Tensor],
                    q_out: Optional[torch.Tensor], cache: Optional[torch.Tensor], page_size: int, H: int, G: int,
                    hd: int, v_col: Optional[int] = None, norm_dim: Optional[int] = None,
                    q_temp: Optional[Tuple[float, float]] = None) -> Optional[torch.Tensor]:
    """Norm + rotate q and k; write q to ``q_out`` and, if ``cache`` is given,
    k and v to their pages.  ``cache`` is one layer's [pages, 2, G, page_size, hd].
    With ``q_out`` None, q and k are changed in place and no cache is written.
    ``v_col``: the column of a row at which the values start (default: behind the keys, ``(H + G) * hd``;
    ``H * hd`` makes the values the key projections themselves, before norm and rotation).  Columns behind
    q, k and v are left alone.  ``norm_dim``: the number the norm's mean is taken over where a head is stored
    wider than it is (zeros behind its own columns; default ``hd``).  ``q_temp`` = (coef, every): the queries of
    the row at position p leave multiplied by ``1 + coef ln(floor((p + 1) / every) + 1)`` (float32)."""
    _need(qkv, "qkv", contiguous=False)
    _need(positions, "positions", torch.int32)
    n = qkv.shape[0]
    if v_col is None:
        v_col = (H + G) * hd
    if qkv.shape[1] < (H + G) * hd or not (0 <= v_col <= qkv.shape[1] - G * hd):
        raise KernelError("qk_norm_rope_kv: shape mismatch")
    if q_out is None and v_col < (H + G) * hd:
        raise KernelError("qk_norm_rope_kv: the in-place form would change the values it shares with the keys")
    if q_out is not None:
        _need(q_out, "q_out", qkv.dtype, contiguous=False)
        if q_out.shape != (n, H * hd):
            raise KernelError("qk_norm_rope_kv: q_out shape")
    elif cache is not None:
        raise KernelError("qk_norm_rope_kv: the in-place form writes no cache")
    for t, nm in ((q_w, "q_w"), (k_w, "k_w")):
        if t is not None:
            _need(t, nm, torch.float32)
            if t.numel() != hd:
                raise KernelError(f"qk_norm_rope_kv: {nm} size")
    if cos_tab is not None:
        _need(cos_tab, "cos_tab", torch.float32); _need(sin_tab, "sin_tab", torch.float32)
        if cos_tab.shape[1] != rotary_dim // 2:
            raise KernelError("qk_norm_rope_kv: table width")
    write_kv = cache is not None
    if write_kv:
        _need(cache, "cache", qkv.dtype); _need(slot_map, "slot_map", torch.int32)
        if tuple(cache.shape[1:]) != (2, G, page_size, hd):
            raise KernelError(f"qk_norm_rope_kv: cache layout {tuple(cache.shape)}")
    nd = hd if norm_dim is None else int(norm_dim)
    if not (1 <= nd <= hd):
        raise KernelError("qk_norm_rope_kv: norm_dim")
    coef, every = (0.0, 0.0) if q_temp is None else (float(q_temp[0]), float(q_temp[1]))
    if q_temp is not None and not every > 0:
        raise KernelError("qk_norm_rope_kv: the query temperature's period must be positive")
    lib = load_library("qkrope")
    _run("qk_norm_rope_kv", lib.kp_qk_norm_rope_kv_temp, _ptr(qkv), _rows_2d(qkv, "qkv"), _ptr(q_w), _ptr(k_w), ctypes.c_float(eps),
                                  _ptr(cos_tab), _ptr(sin_tab), rotary_dim, int(interleaved), _ptr(positions),
                                  _ptr(slot_map), _ptr(q_out), 0 if q_out is None else _rows_2d(q_out, "q_out"), _ptr(cache),
                                  page_size,
                                  n, H, G, hd, int(write_kv), int(v_col), nd, ctypes.c_float(coef), ctypes.c_float(every),
                                  dtype_code(qkv.dtype), STREAM)
    return q_out


def qk_rownorm_kv(qkv: torch.Tensor, k_col: int, v_col: int, q_w: torch.Tensor, k_w: Optional[torch.Tensor], eps: float,
                  count_q: int, count_k: int, slot_map: Optional[torch.Tensor], q_out: torch.Tensor,
                  cache: Optional[torch.Tensor], page_size: int, H: int, G: int, hd: int) -> torch.Tensor:
    """RMS norm of q and of k each over its whole projection (all heads at once, weights as long as the projections),
    no rotation; q to ``q_out``, and with ``cache`` given the normed k and v to their pages.  Rows hold q at column
    0 (H heads stored ``hd`` wide), k at ``k_col`` and v at ``v_col`` (G heads each).  ``count_q`` / ``count_k``: the
    numbers the means are taken over (smaller than H hd and G hd where heads are stored wider than they are, with
    zeros behind)."""
    _need(qkv, "qkv", contiguous=False); _need(q_out, "q_out", qkv.dtype); _need(q_w, "q_w", torch.float32)
    n = qkv.shape[0]
    if tuple(q_out.shape) != (n, H * hd) or q_w.numel() != H * hd or H * hd > qkv.shape[1]:
        raise KernelError("qk_rownorm_kv: shape mismatch")
    write_kv = cache is not None
    if write_kv:
        _need(cache, "cache", qkv.dtype); _need(slot_map, "slot_map", torch.int32); _need(k_w, "k_w", torch.float32)
        if (tuple(cache.shape[1:]) != (2, G, page_size, hd) or k_w.numel() != G * hd
                or max(k_col, v_col) + G * hd > qkv.shape[1] or min(k_col, v_col) < H * hd):
            raise KernelError(f"qk_rownorm_kv: cache layout {tuple(cache.shape)} or columns")
    if n > MAX_STEP_ROWS:
        raise KernelError("qk_rownorm_kv: too many rows")
    _run("qk_rownorm_kv", load_library("qkrope").kp_qk_rownorm_kv, _ptr(qkv), _rows_2d(qkv, "qkv"), int(k_col), int(v_col),
         _ptr(q_w), _ptr(k_w if write_kv else None), ctypes.c_float(eps), ctypes.c_float(count_q), ctypes.c_float(count_k),
         _ptr(slot_map if write_kv else None), _ptr(q_out), H * hd, _ptr(cache), page_size, n, H, G, hd, int(write_kv),
         dtype_code(qkv.dtype), STREAM)
    return q_out


def _check_sink(sink: Optional[torch.Tensor], H: int, keep_first: int, window: Optional[int], block: Optional[int], what: str) -> None:
    if sink is not None:
        _need(sink, "sink", torch.float32)
        if sink.numel() != H:
            raise KernelError(f"{what}: one sink a query head")
    if keep_first and (keep_first < 0 or block):
        raise KernelError(f"{what}: keep_first must not be negative and does not go with blocks of positions")


def attention_rows(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, row_seg: torch.Tensor,
                   positions: torch.Tensor, out: torch.Tensor, scale: float, window: Optional[int],
                   page_size: int, H: int, G: int, hd: int, block: Optional[int] = None, keep_first: int = 0,
                   sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``block``: a row reads no key from before the start of its own block of that many positions.
    ``keep_first``: behind its window a row still reads the first that many keys of its sequence.  ``sink``
    (float32 [H]): ``exp(sink_h)`` joins the softmax's denominator, a key with a score and no value."""
    _need(q, "q", contiguous=False); _need(cache, "cache", q.dtype); _need(out, "out", q.dtype, contiguous=False)
    _need(block_table, "block_table", torch.int32); _need(row_seg, "row_seg", torch.int32)
    _need(positions, "positions", torch.int32)
    n = q.shape[0]
    if q.shape[1] != H * hd or out.shape != (n, H * hd) or tuple(cache.shape[1:]) != (2, G, page_size, hd):
        raise KernelError("attention_rows: shape mismatch")
    _check_sink(sink, H, keep_first, window, block, "attention_rows")
    lib = load_library("attention")
    _run("attention_rows", lib.kp_attention_rows_sink, _ptr(q), _rows_2d(q, "q"), _ptr(cache), _ptr(block_table),
         block_table.shape[1], _ptr(row_seg), _ptr(positions), _ptr(out), _rows_2d(out, "out"), ctypes.c_float(scale),
         int(window or 0), int(block or 0), int(keep_first or 0), _ptr(sink), page_size, n, H, G, hd, dtype_code(q.dtype), STREAM)
    return out


SPLIT_CHUNK = 256          # keys a chunk of the split-KV attention
SPLIT_CHUNK_MMA = 256       # keys a chunk of its tensor-core form: 64, 128 or 256 (a divisor of SPLIT_CHUNK)
SPLIT_MAX_RATIO = 8        # query heads per kv head it takes


def attention_split_scratch(n_rows: int, H: int, hd: int, n_chunks: int, keep_first: int = 0) -> int:
    """Float elements of scratch that :func:`attention_split` needs (``keep_first``: with slots for the chunks of
    that many kept first keys)."""
    slots = n_chunks * (SPLIT_CHUNK // min(SPLIT_CHUNK, SPLIT_CHUNK_MMA)) + -(-int(keep_first or 0) // SPLIT_CHUNK)
    return n_rows * H * slots * (hd + 2)


def attention_split(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, row_seg: torch.Tensor,
                    positions: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, n_chunks: int, scale: float,
                    window: Optional[int], page_size: int, H: int, G: int, hd: int,
                    block: Optional[int] = None, exact_weights: bool = False, keep_first: int = 0,
                    sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Split-KV attention (chunks of 256 keys, merged in order).  ``n_chunks``
    must cover the largest position of the batch; ``scratch`` is float32.
    ``block``: a row reads no key from before the start of its own block of that many positions.
    ``exact_weights``: the softmax weights enter the product with V whole (the scalar kernel always does so; the
    tensor-core form then multiplies their three bfloat16 parts one after the other) instead of rounded to bfloat16.
    ``keep_first`` / ``sink``: as in :func:`attention_rows`; the sink enters in the merge, once a row; kept first
    keys behind a window are computed by a second small launch where the tensor-core form (which knows nothing of
    them) computes the window's chunks."""
    _need(q, "q", contiguous=False); _need(cache, "cache", q.dtype); _need(out, "out", q.dtype, contiguous=False)
    _need(block_table, "block_table", torch.int32); _need(row_seg, "row_seg", torch.int32)
    _need(positions, "positions", torch.int32); _need(scratch, "scratch", torch.float32)
    n = q.shape[0]
    if q.shape[1] != H * hd or out.shape != (n, H * hd) or tuple(cache.shape[1:]) != (2, G, page_size, hd):
        raise KernelError("attention_split: shape mismatch")
    keep_first = int(keep_first or 0) if window else 0
    if scratch.numel() < attention_split_scratch(n, H, hd, n_chunks, keep_first):
        raise KernelError("attention_split: scratch too small")
    _check_sink(sink, H, keep_first, window, block, "attention_split")
    lib = load_library("attention_decode")
    if USE_MMA_ATTENTION and q.dtype == torch.bfloat16 and hd in (64, 128) and q.stride(0) % 2 == 0:
        # tensor-core chunk pass over smaller chunks, then the same merge; kept first keys get slots behind the window's
        # chunks (for the chunk pass they are chunks beyond every position: it leaves them alone)
        front0 = n_chunks * (SPLIT_CHUNK // SPLIT_CHUNK_MMA)
        parts = front0 + -(-keep_first // SPLIT_CHUNK)
        if keep_first:
            _run("attention_front_chunks", lib.kp_attention_front_chunks, _ptr(q), _rows_2d(q, "q"), _ptr(cache), _ptr(block_table),
                 block_table.shape[1], _ptr(row_seg), _ptr(positions), _ptr(scratch), parts, front0, ctypes.c_float(scale),
                 int(window), keep_first, page_size, n, H, G, hd, dtype_code(q.dtype), STREAM)
        _run("attention_split_mma", load_library("attention_mma").kp_attention_split_mma_masked,
            _ptr(q), _rows_2d(q, "q"), _ptr(cache), ctypes.c_longlong(cache.shape[0] if USE_TMA_ATTENTION else 0),
            _ptr(block_table), block_table.shape[1], _ptr(row_seg),
            _ptr(positions), _ptr(scratch), parts, SPLIT_CHUNK_MMA, ctypes.c_float(scale), int(window or 0), int(block or 0),
            int(bool(exact_weights)), page_size, n, H, G, hd, STREAM)
        _run("attention_merge", lib.kp_attention_merge_sink, _ptr(positions), _ptr(out), _rows_2d(out, "out"), _ptr(scratch),
             parts, SPLIT_CHUNK_MMA, int(window or 0), int(block or 0), keep_first, _ptr(sink), front0 if keep_first else -1, n, H, hd,
             dtype_code(q.dtype), STREAM)
        return out
    _run("attention_split", lib.kp_attention_split_sink, _ptr(q), _rows_2d(q, "q"), _ptr(cache), _ptr(block_table),
         block_table.shape[1], _ptr(row_seg), _ptr(positions), _ptr(out), _rows_2d(out, "out"), _ptr(scratch),
         n_chunks, ctypes.c_float(scale), int(window or 0), int(block or 0), keep_first, _ptr(sink), page_size, n, H, G, hd,
         dtype_code(q.dtype), STREAM)
    LAUNCHES[0] += 1
    return out


USE_TMA_ATTENTION = True       # its key/value tiles come by TMA where the page size allows
USE_MMA_ATTENTION = True       # bfloat16 attention with head size 64 or 128 runs on the tensor cores
PREFILL_TILE = 64              # query rows a CTA of the prefill attention kernel


USE_TC_ATTENTION = True        # prompt portions with head size 64 run on the tcgen05 tensor cores


def attention_prefill_tc_ok(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_size: int, hd: int) -> bool:
    """Can the tcgen05 prefill attention take this call (head size 64, 16-byte aligned rows, a page size
    that is a multiple of 8 and divides 128 or is a multiple of it)?"""
    return (USE_TC_ATTENTION and hd == 64 and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and cache.data_ptr() % 16 == 0
            and page_size % 8 == 0 and (page_size % 128 == 0 or 128 % page_size == 0)
            and cache.shape[0] * cache.shape[1] * cache.shape[2] * page_size < 2 ** 31 - 1)


def attention_prefill_ok(q: torch.Tensor, hd: int) -> bool:
    return USE_MMA_ATTENTION and q.dtype == torch.bfloat16 and hd in (64, 128) and q.stride(0) % 2 == 0


def attention_prefill(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, cu_rows: torch.Tensor,
                      seg_pos: torch.Tensor, tile_seg: torch.Tensor, tile_row0: torch.Tensor, out: torch.Tensor,
                      scale: float, window: Optional[int], page_size: int, H: int, G: int, hd: int,
                      big_tile_seg: Optional[torch.Tensor] = None, big_tile_row0: Optional[torch.Tensor] = None,
                      block: Optional[int] = None, exact_weights: bool = False, keep_first: int = 0,
                      sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-core causal attention for segments of many rows.  ``tile_seg`` / ``tile_row0`` list, for every
    tile of 64 consecutive rows of a segment, its segment and its first row; ``big_tile_seg`` /
    ``big_tile_row0`` the same for tiles of 128 rows, the tile that reads the most keys first (with them the
    tcgen05 kernel runs where it takes the sizes).  ``block``: a row reads no key from before the start of its own
    block of that many positions.  ``exact_weights``: the softmax weights enter the product with V whole, as three
    bfloat16 parts multiplied one after the other (the mma.sync kernel; the tcgen05 kernel, whose weights pass
    through shared memory as one bfloat16 operand, is then not taken).  ``keep_first`` / ``sink``: as in
    :func:`attention_rows` (the mma.sync kernel has them, the tcgen05 kernel is then not taken)."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(cache, "cache", torch.bfloat16)
    _need(out, "out", torch.bfloat16, contiguous=False)
    for t_, nm in ((block_table, "block_table"), (cu_rows, "cu_rows"), (seg_pos, "seg_pos"), (tile_seg, "tile_seg"),
                   (tile_row0, "tile_row0")):
        _need(t_, nm, torch.int32)
    n = q.shape[0]
    if q.shape[1] != H * hd or out.shape != (n, H * hd) or tuple(cache.shape[1:]) != (2, G, page_size, hd):
        raise KernelError("attention_prefill: shape mismatch")
    if tile_seg.numel() != tile_row0.numel():
        raise KernelError("attention_prefill: tile lists differ in length")
    _check_sink(sink, H, keep_first, window, block, "attention_prefill")
    keep_first = int(keep_first or 0) if window else 0
    if (big_tile_seg is not None and not exact_weights and not keep_first and sink is None
            and attention_prefill_tc_ok(q, out, cache, page_size, hd)):
        _need(big_tile_seg, "big_tile_seg", torch.int32); _need(big_tile_row0, "big_tile_row0", torch.int32)
        if big_tile_seg.numel() != big_tile_row0.numel():
            raise KernelError("attention_prefill: tile lists differ in length")
        _run("attention_prefill_tc", load_library("attention_tc").kp_attention_prefill_tc_masked,
            _ptr(q), _rows_2d(q, "q"), n, _ptr(cache), ctypes.c_longlong(cache.shape[0]), _ptr(block_table),
            block_table.shape[1], _ptr(cu_rows), _ptr(seg_pos), _ptr(big_tile_seg), _ptr(big_tile_row0),
            big_tile_seg.numel(),
            _ptr(out), _rows_2d(out, "out"), ctypes.c_float(scale), int(window or 0), int(block or 0), page_size, H, G, hd,
            STREAM)
        return out
    _run("attention_prefill_mma", load_library("attention_mma").kp_attention_prefill_mma_sink,
        _ptr(q), _rows_2d(q, "q"), _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(cu_rows), _ptr(seg_pos),
        _ptr(tile_seg), _ptr(tile_row0), tile_seg.numel(), _ptr(out), _rows_2d(out, "out"), ctypes.c_float(scale),
        int(window or 0), int(block or 0), keep_first, _ptr(sink), int(bool(exact_weights)), page_size, H, G, hd, STREAM)
    return out


# ---------------------------------------------------------------- skinny gemm

SKINNY_MAX_M = 64
EPI_SWIGLU = 3


def skinny_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Can the weight-streaming kernel take this product?"""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] <= SKINNY_MAX_M
            and a.shape[1] % 32 == 0 and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


USE_TC = True              # bfloat16 products of more than 64 rows (and some of fewer) run on tcgen05 tensor cores


TC_HEAD_FROM_M = 2         # rows from which a 65536-row head goes to the tcgen05 kernel (measured: one row ties)
TC_SPLIT_FROM_M = 17       # rows from which every product goes to the tcgen05 kernel (cut along K where that pays)


def tc_pays_for_few_rows(M: int, N: int, swiglu: bool) -> bool:
    """Few-row products that the tcgen05 kernel runs faster than the weight-streaming
    kernels (measured on B200, K = 2048, inside a decode step): the 65536-row head from
    2 rows on (a step of 2 rows 638 -> 602 us, of 4 rows 661 -> 624; one row ties), every
    product from 17 rows on (there the kernel cuts the product along K: a step of 64 rows
    1600 -> 1320 us), and below that wide products from 32 rows on."""
    if M >= TC_SPLIT_FROM_M:
        return True
    if swiglu:
        return N >= 8192 and M >= 32        # gate/up 11264 x 2048: 19.9 us against 22.9 at 32 rows, 19.8 against 32.1 at 64
    return (N >= 32768 and M >= TC_HEAD_FROM_M) or (N >= 4096 and M >= 32)


def tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Can the tcgen05 kernel take this product (bfloat16, 16-byte aligned rows, K a multiple of 8)?"""
    return (USE_TC and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            accumulate: bool = False, swiglu: bool = False, split: bool = True, activation: str = "silu",
            glu: Optional[Tuple[float, float, float]] = None) -> torch.Tensor:
    """out = a @ w.T (+ bias) on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory); with
    ``swiglu`` ``w`` holds gate rows then up rows and out = silu(gate) * up (or ``activation``; with ``glu`` =
    (limit, alpha, shift) the gated unit with limits of :func:`glu_clamped`).  With ``split`` a product of 17 to
    1024 rows is cut along K where that brings fewer bytes into the busiest SM (the parts of a tile are a
    thread-block cluster and are added in a fixed order)."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(w, "w", torch.bfloat16, contiguous=False)
    _need(out, "out", contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or out.shape != (M, n_out):
        raise KernelError(f"gemm_tc: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("gemm_tc: bias size")
    lib = load_library("gemm_tc")
    if swiglu and glu is not None:
        epi = _skinny_epilogue(out, accumulate, swiglu) | (ACT_GLU_CLAMPED << 8)
        _run("gemm_tc", lib.kp_gemm_tc_split_glu, _ptr(a), _rows_2d(a, "a"), _ptr(w), _rows_2d(w, "w"), _ptr(bias), _ptr(out),
             _rows_2d(out, "out"), M, N, K, epi, 1 if split else 0, *_glu_floats(glu), STREAM, tag=f" {N}x{K}",
             work=_gemm_work(M, N, K, a, w, out))
        return out
    epi = _skinny_epilogue(out, accumulate, swiglu) | (_fused_activation(activation) << 8 if swiglu else 0)
    _run("gemm_tc", lib.kp_gemm_tc_split, _ptr(a), _rows_2d(a, "a"), _ptr(w), _rows_2d(w, "w"), _ptr(bias), _ptr(out),
         _rows_2d(out, "out"), M, N, K, epi, 1 if split else 0, STREAM, tag=f" {N}x{K}",
         work=_gemm_work(M, N, K, a, w, out))
    return out


STREAM_MAX_M = 64          # rows up to which the bulk-copy kernel is preferred
USE_STREAM = True         # few-row products go to the bulk-copy kernel where their shape fits it


def stream_fits(K: int, swiglu: bool) -> bool:
    """The bulk-copy kernel streams W in chunks of 512 columns."""
    return K >= 512 and K % 512 == 0


def stream_pays(N: int, K: int) -> bool:
    """Measured on B200 (8 rows, back to back in a graph): the bulk-copy kernel wins or ties with the
    register-streaming kernel for the layer products (6144 x 2048: 8.0 against 8.1 us; gate/up 11264 x 2048:
    9.5 against 16.0; 2048 x 5632: 10.2 against 8.9; 2048 x 2048: 4.6 against 4.4) and, because its producer
    fills the ring before it waits for the kernel before it, overlaps that kernel's tail inside a model step.
    It loses on the huge grid of a 65536-row head (65 against 48 us)."""
    return N <= 16384


CONV_STEP_MAX_M = 16       # rows up to which the conv step runs in in_proj's epilogue (measured: batch 8 703 -> 672 us a
                           # step, batch 16 776 -> 741; at 64 rows the tensor-core in_proj and the separate conv kernel win)


def conv_step_fusable(a: torch.Tensor, w_in: torch.Tensor, conv_k: int) -> bool:
    """Can the weight-streaming kernel run the conv step of a decode step in in_proj's epilogue?"""
    return (USE_STREAM and skinny_ok(a, w_in) and a.shape[0] <= CONV_STEP_MAX_M and stream_fits(a.shape[1], False)
            and w_in.shape[0] % 3 == 0 and 2 <= conv_k <= 16)


def gemm_stream_conv_step(a: torch.Tensor, w_in: torch.Tensor, bias: Optional[torch.Tensor], conv_w: torch.Tensor,
                          conv_bias: Optional[torch.Tensor], state: torch.Tensor, seg_pos: torch.Tensor,
                          seg_slot: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = C * conv(B * X)`` for one-row segments, with ``[B | C | X] = a @ w_in.T (+ bias)`` never written
    out: the product's tile holds the matching rows of B, C and X and its epilogue runs the conv step and the
    state update of :func:`shortconv_decode` (same arithmetic, same bits)."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(w_in, "w_in", torch.bfloat16, contiguous=False)
    _need(out, "out", torch.bfloat16, contiguous=False)
    _need(conv_w, "conv_w", torch.float32); _need(state, "state", torch.float32)
    _need(seg_pos, "seg_pos", torch.int32); _need(seg_slot, "seg_slot", torch.int32)
    M, K = a.shape
    N = w_in.shape[0]
    d, conv_k = N // 3, conv_w.shape[1]
    if (w_in.shape[1] != K or N != 3 * d or out.shape != (M, d) or conv_w.shape[0] != d
            or tuple(state.shape[1:]) != (conv_k - 1, d) or seg_pos.numel() != M or seg_slot.numel() != M):
        raise KernelError("gemm_stream_conv_step: shape mismatch")
    for t, nm, n in ((bias, "bias", N), (conv_bias, "conv_bias", d)):
        if t is not None:
            _need(t, nm, torch.float32)
            if t.numel() != n:
                raise KernelError(f"gemm_stream_conv_step: {nm} size")
    lib = load_library("gemm_stream")
    _run("gemm_stream_conv_step", lib.kp_gemm_stream_conv_step, _ptr(a), _rows_2d(a, "a"), _ptr(w_in), _rows_2d(w_in, "w_in"),
         _ptr(bias), _ptr(out), _rows_2d(out, "out"), M, N, K, _ptr(conv_w), _ptr(conv_bias), _ptr(state), _ptr(seg_pos),
         _ptr(seg_slot), conv_k, STREAM, tag=f" {N}x{K}", work=_gemm_work(M, N, K, a, w_in, out))
    return out


FUSED_ACTIVATIONS = ("silu", "relu", "gelu_tanh")     # what the products' gated epilogues compute themselves
ACT_GLU_CLAMPED = 3        # the epilogues' code of the gated unit with limits (csrc/common.cuh); its constants travel beside it


def _glu_floats(glu):
    limit, alpha, shift = glu
    if not limit > 0:
        raise KernelError("the gated unit's limit must be positive")
    return ctypes.c_float(limit), ctypes.c_float(alpha), ctypes.c_float(shift)


def _fused_activation(name: str) -> int:
    if name not in FUSED_ACTIVATIONS:
        raise KernelError(f"the gated epilogue computes {', '.join(FUSED_ACTIVATIONS)}, not '{name}'")
    return activation_code(name)


def _skinny_epilogue(out: torch.Tensor, accumulate: bool, swiglu: bool) -> int:
    if swiglu:
        if out.dtype != torch.bfloat16:
            raise KernelError("gemm_skinny: the SwiGLU epilogue writes bfloat16")
        return EPI_SWIGLU
    if accumulate:
        if out.dtype != torch.float32:
            raise KernelError("gemm_skinny: accumulation needs a float32 output")
        return EPI_ACCUM_F32
    if out.dtype == torch.bfloat16:
        return EPI_STORE
    if out.dtype == torch.float32:
        return EPI_STORE_F32
    raise KernelError("gemm_skinny: output dtype")


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                accumulate: bool = False, swiglu: bool = False, activation: str = "silu",
                glu: Optional[Tuple[float, float, float]] = None) -> torch.Tensor:
    """out = a @ w.T (+ bias) for up to 64 rows of bfloat16 ``a``.  With
    ``swiglu`` ``w`` holds gate rows then up rows and out = silu(gate) * up (or ``activation``; with ``glu`` =
    (limit, alpha, shift) the gated unit with limits of :func:`glu_clamped`)."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(w, "w", torch.bfloat16, contiguous=False)
    _need(out, "out", contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or out.shape != (M, n_out):
        raise KernelError(f"gemm_skinny: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("gemm_skinny: bias size")
    if swiglu:
        if out.dtype != torch.bfloat16:
            raise KernelError("gemm_skinny: the SwiGLU epilogue writes bfloat16")
        epi = EPI_SWIGLU | ((ACT_GLU_CLAMPED if glu is not None else _fused_activation(activation)) << 8)
    elif accumulate:
        if out.dtype != torch.float32:
            raise KernelError("gemm_skinny: accumulation needs a float32 output")
        epi = EPI_ACCUM_F32
    elif out.dtype == torch.bfloat16:
        epi = EPI_STORE
    elif out.dtype == torch.float32:
        epi = EPI_STORE_F32
    else:
        raise KernelError("gemm_skinny: output dtype")
    consts = _glu_floats(glu) if swiglu and glu is not None else ()
    if USE_STREAM and stream_fits(K, swiglu) and stream_pays(N, K) and M <= STREAM_MAX_M:
        lib = load_library("gemm_stream")
        _run("gemm_stream", lib.kp_gemm_stream_glu if consts else lib.kp_gemm_stream, _ptr(a), _rows_2d(a, "a"), _ptr(w),
             _rows_2d(w, "w"), _ptr(bias), _ptr(out), _rows_2d(out, "out"), M, N, K, epi, *consts, STREAM, tag=f" {N}x{K}",
             work=_gemm_work(M, N, K, a, w, out))
        return out
    lib = load_library("gemm_skinny")
    _run("gemm_skinny", lib.kp_gemm_skinny_glu if consts else lib.kp_gemm_skinny, _ptr(a), _rows_2d(a, "a"), _ptr(w),
         _rows_2d(w, "w"), _ptr(bias), _ptr(out), _rows_2d(out, "out"), M, N, K, epi, *consts, STREAM, tag=f" {N}x{K}",
         work=_gemm_work(M, N, K, a, w, out))
    return out


# ------------------------------------------------------------------ mixture of experts

MOE_MAX_TOP = 32           # experts a row can use
MOE_MAX_EXPERTS = 1536     # experts the routing kernels hold in shared memory


def moe_layout_ints(n: int, E: int, top: int) -> int:
    """int32 words of the device-side layout of one step (see :func:`moe_route`)."""
    return 3 * (E + 1) + 2 * n * top


MOE_ROUTINGS = {"top_logits": 0, "softmax_all": 1, "sigmoid": 2}


def _moe_routing(routing: str) -> int:
    try:
        return MOE_ROUTINGS[routing]
    except KeyError:
        raise KernelError(f"moe: routing '{routing}' (expected one of {', '.join(MOE_ROUTINGS)})") from None


def moe_route(logits: torch.Tensor, top: int, idx: torch.Tensor, weights: torch.Tensor, layout: torch.Tensor,
              bias: Optional[torch.Tensor] = None, routing: str = "top_logits", scale: float = 1.0,
              n_identity: int = 0) -> None:
    """Router logits [n, E] (float32) -> the ``top`` experts of every row (``idx`` int32 [n, top], largest
    first, the lower index on ties), their weights (float32 [n, top]) and the
    layout of the (row, choice) pairs by expert (``layout``, int32, :func:`moe_layout_ints` words), which the
    grouped products read.  Nothing returns to the host.  ``routing`` ``top_logits``: the largest logits (+ ``bias``),
    weighted by the softmax over the chosen logits alone; ``softmax_all``: scores = softmax over all E outputs, the
    largest score + ``bias`` are chosen and weighted by their score times ``scale``; ``sigmoid``: the largest logits
    are chosen and each weighted by its own ``sigmoid(logit)`` times ``scale``.  The last ``n_identity``
    outputs stand for experts without weights (places in the layout, no tiles)."""
    _need(logits, "logits", torch.float32); _need(idx, "idx", torch.int32); _need(weights, "weights", torch.float32)
    _need(layout, "layout", torch.int32)
    n, E = logits.shape
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != E:
            raise KernelError("moe_route: bias size")
    if not (1 <= top <= min(E, MOE_MAX_TOP)) or E > MOE_MAX_EXPERTS:
        raise KernelError(f"moe_route: top={top} of {E} experts is not supported (top <= {MOE_MAX_TOP}, experts <= {MOE_MAX_EXPERTS})")
    if idx.numel() != n * top or weights.numel() != n * top or layout.numel() < moe_layout_ints(n, E, top):
        raise KernelError("moe_route: output sizes")
    _run("moe_route", load_library("moe").kp_moe_route, _ptr(logits), _ptr(bias), n, E, top, _moe_routing(routing),
         ctypes.c_float(scale), int(n_identity), _ptr(idx), _ptr(weights), _ptr(layout), STREAM)
    LAUNCHES[0] += 1


MOE_TC_MIN_PAIRS = [512]   # (row, expert) pairs of a step from which the experts' products run on tcgen05 tiles


def moe_set_tc_min_pairs(v: int) -> None:
    """For measurements and tests: the number of pairs from which the tcgen05 path is taken."""
    MOE_TC_MIN_PAIRS[0] = int(v)
    load_library("moe").kp_moe_set_tc_min_pairs(ctypes.c_longlong(int(v)))


def moe_tc_status() -> int:
    return _read_one("moe", "moe_tc")


def moe_router_ok(d: int, E: int) -> bool:
    """Can the fused router kernel take rows of ``d`` elements and ``E`` experts (a row, its logits and its scores in shared memory)?"""
    return d % 4 == 0 and E <= MOE_MAX_EXPERTS and (d + 2 * E) * 4 <= 200 * 1024


def moe_router(h: torch.Tensor, w_router: torch.Tensor, bias: Optional[torch.Tensor], top: int, idx: torch.Tensor,
               weights: torch.Tensor, layout: torch.Tensor, routing: str = "top_logits", scale: float = 1.0,
               n_identity: int = 0) -> None:
    """The router in one go: logits ``h w_router^T`` in float32 (``w_router`` [E, d] and ``bias`` are float32;
    ``h`` is widened from its storage type), the choice and the layout as :func:`moe_route` leaves them."""
    _need(h, "h", contiguous=False); _need(w_router, "w_router", torch.float32)
    _need(idx, "idx", torch.int32); _need(weights, "weights", torch.float32); _need(layout, "layout", torch.int32)
    n, d = h.shape
    E = w_router.shape[0]
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != E:
            raise KernelError("moe_router: bias size")
    if w_router.shape[1] != d or not moe_router_ok(d, E) or not (1 <= top <= min(E, MOE_MAX_TOP)):
        raise KernelError("moe_router: sizes not supported")
    if idx.numel() != n * top or weights.numel() != n * top or layout.numel() < moe_layout_ints(n, E, top):
        raise KernelError("moe_router: output sizes")
    _run("moe_router", load_library("moe").kp_moe_router, _ptr(h), _rows_2d(h, "h"), _ptr(w_router), _ptr(bias), n, E, d, top,
         _moe_routing(routing), ctypes.c_float(scale), int(n_identity), _ptr(idx), _ptr(weights), _ptr(layout), dtype_code(h.dtype), STREAM,
         work=(2 * n * E * d, n * d * h.element_size() + E * d * 4))
    LAUNCHES[0] += 1


def moe_experts(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, layout: torch.Tensor,
                weights: torch.Tensor, top: int, out: torch.Tensor, activation: str = "silu", n_identity: int = 0,
                idx: Optional[torch.Tensor] = None, weight_input: bool = False) -> torch.Tensor:
    """out[r] += sum_j weights[r, j] * Wd_e (act(Wg_e h[r]) * (Wu_e h[r])), e = the j-th expert of row r as laid out
    by :func:`moe_route`.  ``w_gate_up``: [E, 2 ff, d] (gate rows, then up rows); ``w_down``: [E, d, ff]; ``out``
    float32 [n, d].  bfloat16 operands run on the tensor cores, float32 ones on the CUDA cores in true 32-bit.
    With ``n_identity`` the router had that many outputs more than there are experts here; a pair that chose one of
    them (``idx`` [n, top] says so) adds ``weight * h[r]``.  ``weight_input``: the weight multiplies the unit's
    input instead, ``out[r] += sum_j Wd_e (act(Wg_e w_j h[r]) * (Wu_e w_j h[r]))`` (the product ``w_j h[r]`` in
    float32, rounded to the storage type as a matrix operand)."""
    _need(h, "h", contiguous=False); _need(w_gate_up, "w_gate_up", h.dtype); _need(w_down, "w_down", h.dtype)
    _need(layout, "layout", torch.int32); _need(weights, "weights", torch.float32); _need(out, "out", torch.float32)
    n, d = h.shape
    E_real, ff2, d2 = w_gate_up.shape
    E = E_real + int(n_identity)
    ff = ff2 // 2
    if d2 != d or ff2 != 2 * ff or tuple(w_down.shape) != (E_real, d, ff) or tuple(out.shape) != (n, d):
        raise KernelError("moe_experts: shape mismatch")
    if weights.numel() != n * top or layout.numel() < moe_layout_ints(n, E, top):
        raise KernelError("moe_experts: routing tables do not fit")
    if n_identity:
        _need(idx, "idx", torch.int32)
        if idx.numel() != n * top:
            raise KernelError("moe_experts: idx size")
        if weight_input:
            raise KernelError("moe_experts: weights on the inputs do not go with identity experts")
    act = torch.empty((n * top, ff), dtype=h.dtype, device=h.device)
    y = torch.empty((n * top, d), dtype=torch.float32, device=h.device)
    # (many rows, 16-bit: the tcgen05 tiles read the rows laid out place by place)
    hs = (torch.empty((n * top, d), dtype=h.dtype, device=h.device)
          if (weight_input or (h.dtype == torch.bfloat16 and n * top >= MOE_TC_MIN_PAIRS[0])) else None)
    _run("moe_experts", load_library("moe").kp_moe_experts_weighted, _ptr(h), _rows_2d(h, "h"), _ptr(w_gate_up), _ptr(w_down), _ptr(layout),
         _ptr(weights), _ptr(act), _ptr(y), _ptr(out), _ptr(hs), n, E, top, d, ff, activation_code(activation), dtype_code(h.dtype),
         int(n_identity), _ptr(idx if n_identity else None), int(bool(weight_input)), STREAM, tag=f" {E}x{ff}x{d}",
         work=(6 * n * top * ff * d, min(E, n * top) * 3 * ff * d * h.element_size()))     # (bytes: the experts a step can touch)
    LAUNCHES[0] += 2
    return out
