"""Python face of the hand-written CUDA kernels (sm_100a).

Each function checks its tensors (device, dtype, contiguity, shapes), passes raw pointers and the
current CUDA stream to an ``extern "C"`` entry point through ctypes, and raises ``KernelError`` with the
library's message on a non-zero return.  There is no CPU or PyTorch fallback: if a library cannot be
compiled or loaded the first call that needs it raises.
"""
import ctypes
import os
from ctypes import c_float, c_int, c_void_p

import torch

from .build import BuildError, build_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt):
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dt}")


_P, _I, _F = c_void_p, c_int, c_float

_SIGNATURES = {
    "core": {
        "forge_embedding": [_P, _P, _I, _P, _I, _I, _I, _P, _P],
        "forge_rmsnorm": [_P, _P, _P, _I, _P, _I, _I, _F, _P],
        "forge_rope_kv_write": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
        "forge_rope_table": [_P, _P, _I, _I, _F, _I, _P],
        "forge_silu_mul_interleaved": [_P, _P, _I, _I, _I, _P],
        "forge_gemm_simt": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "forge_paged_attention_simt": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P],
        "forge_argmax": [_P, _P, _I, _I, _P],
        "forge_repeat_penalty": [_P, _P, _P, _P, _P, _I, _I, _P],
        "forge_sample": [_P, _P, _P, _P, _P, _P, _I, _I, _P],
        "forge_history_penalty": [_P, _P, _P, _P, _I, _I, _P],
        "forge_history_add": [_P, _P, _P, _P, _I, _I, _P],
    },
    "gemm_sm100": {
        "forge_gemm_sm100": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
        "forge_gemm_sm100_set_workspace": [_P, ctypes.c_longlong],
        "forge_gemm_sm100_qkv_rope": [_P] * 8 + [_I] * 7 + [_P],
    },
    "attention_mma": {
        "forge_paged_attention_mma": [_P] * 10 + [_I] * 9 + [_F, _P],
        "forge_decode_attention_fused": [_P] * 6 + [_I] * 8 + [_F, _F, _I, _P],
        "forge_decode_attention_stream": [_P] * 7 + [_I] * 9 + [_F, _F, _I, _I, _P],
    },
    "attention_sm100": {
        "forge_paged_attention_sm100": [_P] * 10 + [_I] + [_P] * 3 + [_I] * 9 + [_F, _P],
    },
    "decode_layers": {
        "forge_decode_layers_desc_bytes": [],
        "forge_decode_layers_supports": [_I] * 6,
        "forge_decode_layers_describe": [_P, _I] + [_P] * 8 + [_I] * 5,
        "forge_decode_layers": [_P, _I] + [_P] * 12 + [_I] * 10 + [_F, _F, _F, _I, _P, _P],
        "forge_decode_layers_barrier_probe": [_P, _P, ctypes.c_ulonglong, _P],
    },
}

_libs = {}

# FORGE_CHECKS=1: every library is built with index checks (csrc/checks.cuh): page ids, slots and token indices are
# tested before use, a bad one raises bit 4 of the step's status word and is skipped.  The entries that tell a
# library the bounds, per library (one per source file that checks):
_CHECK_ENTRIES = {"core": ["forge_checks_configure_rope", "forge_checks_configure_attention_simt"],
                  "gemm_sm100": ["forge_checks_configure_gemm_sm100"],
                  "attention_mma": ["forge_checks_configure_attention_mma", "forge_checks_configure_attention_decode_stream"],
                  "attention_sm100": ["forge_checks_configure_attention_sm100"]}
_check_bounds = [None]          # (num_pages, page_size, num_tokens, status tensor, first_bad tensor) of the current step


def checks_enabled():
    return os.environ.get("FORGE_CHECKS", "0") == "1"


def _configure_library_checks(name, lib):
    b = _check_bounds[0]
    if b is None:
        return
    for fn in _CHECK_ENTRIES.get(name, []):
        f = getattr(lib, fn)
        f.argtypes = [_I, _I, _I, _P, _P, _P]
        f.restype = c_int
        rc = f(b[0], b[1], b[2], b[3].data_ptr(), b[4].data_ptr(), _stream())
        if rc != 0:
            raise KernelError(f"{fn}: {lib.forge_last_error().decode(errors='replace')}")


def configure_checks(num_pages, page_size, num_tokens, status, first_bad):
    """(checks build) Gives every loaded library the bounds of the step that is about to run; libraries loaded later
    get them when they load.  ``status``: int32 [1]; ``first_bad``: int32 [3] (kind, value, limit of the first offender)."""
    if not checks_enabled():
        return
    _check_bounds[0] = (int(num_pages), int(page_size), int(num_tokens), status, first_bad)
    for (name, defines), lib in _libs.items():
        if ("FORGE_CHECKS", 1) in defines:
            _configure_library_checks(name, lib)


def library(name, defines=None):
    """Loads (building first if needed) kernel library ``name`` (variant ``defines``) and returns its
    ctypes handle."""
    if checks_enabled() and name in _CHECK_ENTRIES:
        defines = dict(defines or {}, FORGE_CHECKS=1)
    key = (name, tuple(sorted((defines or {}).items())))
    lib = _libs.get(key)
    if lib is not None:
        return lib
    if not torch.cuda.is_available():
        raise KernelError("forge_b200 runs on a CUDA device (B200, sm_100a) only; no device is visible")
    try:
        path = build_library(name, defines=defines)
    except BuildError as e:
        raise KernelError(f"kernel library '{name}' is not available: {e}") from e
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        raise KernelError(f"cannot load {path}: {e}") from e
    for fn, argtypes in _SIGNATURES[name].items():
        f = getattr(lib, fn)
        f.argtypes = argtypes
        f.restype = c_int
        setattr(lib, fn, _Entry(lib, fn, f, argtypes))
    lib.forge_last_error.restype = ctypes.c_char_p
    _libs[key] = lib
    if defines and defines.get("FORGE_CHECKS") == 1:
        _configure_library_checks(name, lib)
    return lib


_launches = [0]

# ----------------------------------------------------------------------------- a layer's launches, noted and repeated
# The layers of a model mostly differ in nothing but the addresses of their weights and caches, while the host's share
# of a launch (choosing the kernel, checking the arguments, cutting outputs from the workspace, the foreign call) costs
# about 17 us against 3 to 10 us of device time at few tokens: a prompt of 128 tokens took 2.7 ms for 0.9 ms of device
# work.  So a model whose layers declare it (parts.base.replay_of) runs ONE layer through Python with the calls into
# the libraries noted, and repeats the noted calls for the other layers with the layer's own addresses in place.
# Launches that make what the whole step shares happen inside the layer that first needs it; they are marked
# (once_per_step) and left out of the notes.
_recording = [None]
_once = [0, 0]          # depth of open ``once_per_step`` blocks; launches counted inside them while a recording is open


class _OncePerStep:
    def __enter__(self):
        _once[0] += 1

    def __exit__(self, *exc):
        _once[0] -= 1
        return False


def once_per_step():
    """``with once_per_step():`` around launches that make something the whole step shares (a table of angles, a
    workspace handed to a library): a recording that is open leaves them out, and they are not repeated with the
    layer they happened to be made in."""
    return _OncePerStep()


class _Entry:
    """A library function that notes its calls while a recording is open."""
    __slots__ = ("lib", "name", "fn", "pointer_args")

    def __init__(self, lib, name, fn, argtypes):
        self.lib, self.name, self.fn = lib, name, fn
        self.pointer_args = tuple(i for i, t in enumerate(argtypes) if t is _P)

    def __call__(self, *args):
        rec = _recording[0]
        if rec is not None and not _once[0]:
            rec.append((self, args))
        return self.fn(*args)


class _Recording:
    def __enter__(self):
        self.calls, self.launches0 = [], _launches[0]
        _recording[0] = self.calls
        _once[1] = 0
        return self

    def __exit__(self, *exc):
        _recording[0] = None
        self.launches = _launches[0] - self.launches0 - _once[1]
        return False


def record_launches():
    """``with record_launches() as rec:`` notes every call into the kernel libraries made inside (``rec.calls``) and how
    many launches they counted for (``rec.launches``)."""
    return _Recording()


class LayerReplay:
    """The launches of one layer, to be repeated for layers of the same shape.  ``source``: the device tensors of the
    recorded layer (weights, cache), None where an optional one is absent; every pointer argument that points into one
    of them is exchanged for the same offset into the other layer's tensor."""

    def __init__(self, recording, source):
        spans = [(t.data_ptr(), t.data_ptr() + t.numel() * t.element_size(), i) for i, t in enumerate(source) if t is not None]
        self.calls = [(entry, list(args)) for entry, args in recording.calls]
        self.patches = []                       # (call, argument, tensor, byte offset)
        for ci, (entry, args) in enumerate(self.calls):
            for ai in entry.pointer_args:
                v = args[ai]
                if not v:
                    continue
                for lo, hi, ti in spans:
                    if lo <= v < hi:
                        self.patches.append((ci, ai, ti, v - lo))
                        break
        self.launches = recording.launches
        self.source_kinds = [t is None for t in source]

    def run(self, tensors):
        """Repeats the launches with ``tensors`` (same order and kinds as the source) in the recorded tensors' place."""
        if [t is None for t in tensors] != self.source_kinds:
            raise KernelError("a layer's launches cannot be repeated for a layer with other optional tensors")
        base = [0 if t is None else t.data_ptr() for t in tensors]
        calls = self.calls
        for ci, ai, ti, off in self.patches:
            calls[ci][1][ai] = base[ti] + off
        for entry, args in calls:
            rc = entry.fn(*args)
            if rc != 0:
                raise KernelError(f"{entry.name}: {entry.lib.forge_last_error().decode(errors='replace')} (code {rc})")
        _launches[0] += self.launches


def launch_count():
    """How many kernels of these libraries have been launched (graph replays add their kernels)."""
    return _launches[0]


def count_launches(n):
    _launches[0] += n


def _check(lib, rc, what):
    _launches[0] += 1
    if _once[0]:
        _once[1] += 1
    if rc != 0:
        raise KernelError(f"{what}: {lib.forge_last_error().decode(errors='replace')} (code {rc})")
    if _profile["on"]:
        _profile_mark(what)


# ------------------------------------------------------------------------------------------ timing
# A per-kernel-class timing table in the manner of the reference's PerfProfiler (include/forge/perf_profiler.h:28-218,
# src/bindings/profiler.cpp): while it is enabled an event is recorded after every launch, and a kernel's time is the
# time from the end of its predecessor on the stream to its own end (so it includes the hand-over between the two).
# Decode steps are launched kernel by kernel meanwhile (a CUDA graph replay has no launches to put events between).
_profile = {"on": False, "last": None, "pending": [], "records": {}}


def profiler_enable():
    _profile["on"] = True
    _profile["last"] = None


def profiler_disable():
    _profile["on"] = False


def profiler_enabled():
    return _profile["on"]


def profiler_reset():
    _profile["pending"].clear()
    _profile["records"].clear()
    _profile["last"] = None


def profiler_step_begin():
    """The time before a step's first kernel belongs to nobody."""
    if _profile["on"]:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        _profile["last"] = e


def _profile_mark(what):
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    if _profile["last"] is not None:
        _profile["pending"].append((what, _profile["last"], e))
    _profile["last"] = e


def profiler_summary():
    """{kernel class: {count, total_ms, avg_ms, min_ms, max_ms, last_ms}} (the reference's field names)."""
    if _profile["pending"]:
        torch.cuda.synchronize()
        for what, e0, e1 in _profile["pending"]:
            ms = e0.elapsed_time(e1)
            r = _profile["records"].setdefault(what, {"count": 0, "total_ms": 0.0, "min_ms": float("inf"), "max_ms": 0.0, "last_ms": 0.0})
            r["count"] += 1
            r["total_ms"] += ms
            r["min_ms"], r["max_ms"], r["last_ms"] = min(r["min_ms"], ms), max(r["max_ms"], ms), ms
        _profile["pending"].clear()
    return {k: dict(v, avg_ms=v["total_ms"] / v["count"]) for k, v in _profile["records"].items()}


def profiler_print(file=None):
    import sys
    rows = sorted(profiler_summary().items(), key=lambda kv: -kv[1]["total_ms"])
    total = sum(r["total_ms"] for _, r in rows) or 1.0
    out = file or sys.stderr
    print(f"{'kernel':<28}{'count':>8}{'total ms':>12}{'avg us':>10}{'min us':>10}{'max us':>10}{'share':>8}", file=out)
    for name, r in rows:
        print(f"{name:<28}{r['count']:>8}{r['total_ms']:>12.3f}{1e3 * r['avg_ms']:>10.1f}{1e3 * r['min_ms']:>10.1f}"
              f"{1e3 * r['max_ms']:>10.1f}{100 * r['total_ms'] / total:>7.1f}%", file=out)


# The current stream's handle, asked for once per kernel launch: torch's two C entry points answer in a fraction of a
# microsecond, torch.cuda.current_stream() takes several (a prompt step of a 22-layer model launches 180 kernels and
# is as long on the host as on the device).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need(t, name, dtype=None, ndim=None):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dims, got shape {tuple(t.shape)}")
    return t.data_ptr()


def _opt(t, name, dtype=None):
    return None if t is None else _need(t, name, dtype)


# ----------------------------------------------------------------------------------- step workspace

class StepWorkspace:
    """One device buffer that the outputs of a step's kernels are cut from, instead of one trip to the allocator per
    kernel output (the reference allocates device memory for every operator output, src/core/tensor.cpp:86-107).

    While a step is open (``with ws.step():``) every tensor that the functions of this module would allocate is a
    view into the buffer.  What lives for one layer is handed out front to back, and ``mark`` / ``release`` give a
    layer's intermediates back when the layer is done; what lives for the whole step (a step's tile lists, its table
    of rotary angles: made inside the first layer that needs them, used by all) is handed out from the back and
    stays until the step closes.  So the buffer holds one layer's worth plus the step's own.  The buffer is as large
    as the largest step so far needed: a step that outgrows it gets ordinary allocations for the overflow, and the
    buffer is enlarged after that step.  ``reserve(nbytes)`` sizes it ahead of time.  Tensors cut from it are dead
    when the next step opens; what a caller keeps (logits) must not come from here (``paused``)."""
    ALIGN = 256

    def __init__(self, device):
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.buf = None
        self.typed = {}
        self.capacity = 0
        self.offset = 0          # next free byte at the front (may run past capacity: then it only measures)
        self.back = 0            # bytes handed out from the back
        self.high = 0
        self.open = False
        self.hold = 0            # > 0: paused
        self.allocations = 0     # outputs that had to come from the allocator while a step was open

    ITEMSIZE = {torch.float32: 4, torch.bfloat16: 2, torch.int32: 4, torch.float16: 2, torch.int64: 8, torch.uint8: 1}

    CANARY_BYTE = 0xA5

    def reserve(self, nbytes):
        nbytes = -(-int(nbytes) // self.ALIGN) * self.ALIGN
        if nbytes > self.capacity:
            whole = torch.empty(nbytes + self.ALIGN, dtype=torch.uint8, device=self.device)
            whole[nbytes:].fill_(self.CANARY_BYTE)              # canary words behind the buffer: nothing ever writes them
            self._whole, self.buf = whole, whole[:nbytes]
            self.capacity = nbytes
            self.typed = {dt: self.buf.view(dt) for dt in self.ITEMSIZE}     # one view per element type to slice from

    def canary_intact(self):
        """False if a kernel wrote past the end of the buffer (synchronises)."""
        return self.capacity == 0 or bool((self._whole[self.capacity:] == self.CANARY_BYTE).all())

    def step(self):
        return _OpenStep(self)

    def paused(self):
        return _Paused(self)

    def mark(self):
        return self.offset

    def release(self, mark):
        self.offset = mark

    def take(self, shape, dtype, whole_step=False):
        n = 1
        for d in shape:
            n *= d
        size = self.ITEMSIZE[dtype]
        nbytes = n * size
        padded = -(-nbytes // self.ALIGN) * self.ALIGN
        if whole_step:
            self.back += padded
            start = self.capacity - self.back
        else:
            start = self.offset
            self.offset += padded
        self.high = max(self.high, self.offset + self.back)
        if self.offset + self.back > self.capacity:
            self.allocations += 1
            return None
        first = start // size                        # start is a multiple of ALIGN, so of every element size
        return self.typed[dtype][first:first + n].view(shape)


class _OpenStep:
    def __init__(self, ws):
        self.ws = ws

    def __enter__(self):
        ws = self.ws
        ws.offset, ws.back, ws.high, ws.open = 0, 0, 0, True
        _active_workspace[0] = ws
        return ws

    def __exit__(self, *exc):
        ws = self.ws
        ws.open = False
        _active_workspace[0] = None
        if ws.high > ws.capacity:          # the next step of this size fits
            ws.reserve(ws.high + ws.high // 8)
        return False


class _Paused:
    def __init__(self, ws):
        self.ws = ws

    def __enter__(self):
        self.ws.hold += 1

    def __exit__(self, *exc):
        self.ws.hold -= 1
        return False


_active_workspace = [None]


def new_tensor(shape, dtype, device, whole_step=False):
    """An uninitialised tensor for a kernel's output: from the open step's workspace if there is one (and it is
    not paused, and lives on this device), else from the allocator.  ``whole_step``: the tensor is kept for the rest
    of the step (in the batch's plan, say), not only for the layer that makes it."""
    ws = _active_workspace[0]
    if ws is not None and ws.hold == 0 and device == ws.device:      # (a step is never open during a graph capture)
        t = ws.take(shape, dtype, whole_step)
        if t is not None:
            return t
    return torch.empty(tuple(shape), dtype=dtype, device=device)


def new_ints(values, device):
    """int32 device tensor of a host list (a step's tile lists and the like), kept for the whole step."""
    host = torch.tensor(values, dtype=torch.int32)
    out = new_tensor(host.shape, torch.int32, device, whole_step=True)
    out.copy_(host)
    return out


# ---------------------------------------------------------------------------------------------- core

def embedding(ids, table, out=None, status=None):
    """out[t,:] = table[ids[t],:] as float32 [T,H]; ids int32 [T]; table [V,H] float32 or bfloat16."""
    lib = library("core")
    T, (V, H) = ids.numel(), table.shape
    if out is None:
        out = new_tensor((T, H), torch.float32, table.device)
    _check(lib, lib.forge_embedding(_need(ids, "ids", torch.int32), _need(table, "table", ndim=2),
                                    dtype_code(table.dtype), _need(out, "out", torch.float32), T, H, V,
                                    _opt(status, "status", torch.int32), _stream()), "embedding")
    return out


def rmsnorm(x, weight, eps, out_dtype, rows=None, out=None):
    """y = x * rsqrt(mean(x^2)+eps) * w over the last dim of float32 x [T,H]; ``rows`` (int32) picks rows."""
    lib = library("core")
    H = x.shape[-1]
    R = x.shape[0] if rows is None else rows.numel()
    if weight.numel() != H:
        raise KernelError(f"rmsnorm: weight has {weight.numel()} elements, rows have {H}")
    if out is None:
        out = new_tensor((R, H), out_dtype, x.device)
    _check(lib, lib.forge_rmsnorm(_need(x, "x", torch.float32, 2), _need(weight, "weight", torch.float32),
                                  _need(out, "out", out_dtype), dtype_code(out_dtype),
                                  _opt(rows, "rows", torch.int32), R, H, float(eps), _stream()), "rmsnorm")
    return out


def rope_table(positions, head_dim, theta, by_pair=False):
    """float32 [T, head_dim/2, 2]: (cos, sin) of position / theta^(2d/head_dim) for the step's tokens; computed once
    per step and shared by every head of every layer with the same head size and base.  ``by_pair``: laid out
    [head_dim/2, T, 2] instead, which is what the projection whose epilogue rotates reads (a thread per token there,
    so neighbouring threads read neighbouring tokens of one pair)."""
    lib = library("core")
    T = positions.numel()
    shape = (head_dim // 2, T, 2) if by_pair else (T, head_dim // 2, 2)
    table = new_tensor(shape, torch.float32, positions.device, whole_step=True)
    with once_per_step():
        _check(lib, lib.forge_rope_table(_need(positions, "positions", torch.int32), _need(table, "table"), T, head_dim,
                                         float(theta), 1 if by_pair else 0, _stream()), "rope_table")
    return table


def rope_kv_write(qkv, positions, slot_mapping, kv_cache, n_heads, n_kv_heads, head_dim, page_size, theta,
                  act_dtype, rotary=True, q_out=None, table=None):
    """Rotates q and k of float32 qkv [T,(NH+2NKV)*HD], returns q [T,NH*HD] in ``act_dtype`` and writes
    k, v into ``kv_cache`` [pages,2,NKV,page,HD] at ``slot_mapping`` (int32 [T]; None or negative: no write)."""
    lib = library("core")
    T = qkv.shape[0]
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"rope_kv_write: qkv has width {qkv.shape[1]}, expected {width}")
    if q_out is None:
        q_out = new_tensor((T, n_heads * head_dim), act_dtype, qkv.device)
    if kv_cache is not None and kv_cache.dtype != act_dtype:
        raise KernelError("rope_kv_write: cache and activation dtypes differ")
    if kv_cache is None:
        slot_mapping = None
    _check(lib, lib.forge_rope_kv_write(_need(qkv, "qkv", torch.float32, 2), _need(positions, "positions", torch.int32),
                                        _opt(slot_mapping, "slot_mapping", torch.int32), _need(q_out, "q_out", act_dtype),
                                        _opt(kv_cache, "kv_cache"), dtype_code(act_dtype), T, n_heads, n_kv_heads,
                                        head_dim, page_size, float(theta), 1 if rotary else 0,
                                        _opt(table, "table", torch.float32), _stream()),
           "rope_kv_write")
    return q_out


def silu_mul_interleaved(gu, out_dtype, out=None):
    """out[t,j] = silu(gu[t,2j]) * gu[t,2j+1]; gu float32 [T,2I]."""
    lib = library("core")
    T, two_i = gu.shape
    if out is None:
        out = new_tensor((T, two_i // 2), out_dtype, gu.device)
    _check(lib, lib.forge_silu_mul_interleaved(_need(gu, "gu", torch.float32, 2), _need(out, "out", out_dtype),
                                               dtype_code(out_dtype), T, two_i // 2, _stream()), "silu_mul_interleaved")
    return out


def gemm_simt(a, w, bias=None, out=None, accumulate=False):
    """float32 C[M,N] = a[M,K] . w[N,K]^T (+bias) (+C when ``accumulate``), true fp32 FMA; a, w same dtype."""
    lib = library("core")
    (M, K), (N, K2) = a.shape, w.shape
    if K != K2 or a.dtype != w.dtype:
        raise KernelError(f"gemm_simt: a {tuple(a.shape)} {a.dtype} does not match w {tuple(w.shape)} {w.dtype}")
    if out is None:
        if accumulate:
            raise KernelError("gemm_simt: accumulate needs an output tensor")
        out = new_tensor((M, N), torch.float32, a.device)
    elif tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_simt: out has shape {tuple(out.shape)}, expected {(M, N)}")
    _check(lib, lib.forge_gemm_simt(_need(a, "a", ndim=2), _need(w, "w", ndim=2), _opt(bias, "bias", torch.float32),
                                    _need(out, "out", torch.float32), dtype_code(a.dtype), M, N, K,
                                    1 if accumulate else 0, _stream()), "gemm_simt")
    return out


def paged_attention_simt(q, kv_cache, block_table, tok_req, positions, n_heads, n_kv_heads, head_dim, page_size,
                         window=0, scale=None, out=None):
    """Causal GQA over the paged cache, fp32 arithmetic; q [T,NH*HD]; block_table int32 [S,max_pages];
    tok_req / positions int32 [T] give each token's row of the table and its position."""
    lib = library("core")
    T = q.shape[0]
    if out is None:
        out = new_tensor(q.shape, q.dtype, q.device)
    if kv_cache.dtype != q.dtype:
        raise KernelError("paged_attention_simt: q and cache dtypes differ")
    scale = head_dim ** -0.5 if scale is None else scale
    _check(lib, lib.forge_paged_attention_simt(
        _need(q, "q", ndim=2), _need(kv_cache, "kv_cache"), _need(block_table, "block_table", torch.int32, 2),
        _need(tok_req, "tok_req", torch.int32), _need(positions, "positions", torch.int32), _need(out, "out", q.dtype),
        dtype_code(q.dtype), T, n_heads, n_kv_heads, head_dim, page_size, block_table.shape[1], int(window or 0),
        float(scale), _stream()), "paged_attention_simt")
    return out


def argmax(logits, out=None):
    """int32 [R]: index of the largest of each row of float32 logits [R,V]; lowest index wins a tie."""
    lib = library("core")
    R, V = logits.shape
    if out is None:
        out = new_tensor((R,), torch.int32, logits.device)
    _check(lib, lib.forge_argmax(_need(logits, "logits", torch.float32, 2), _need(out, "out", torch.int32), R, V,
                                 _stream()), "argmax")
    return out


def repeat_penalty(logits, tokens, counts, offsets, penalty):
    """In place: for row r and each (token, count) in [offsets[r], offsets[r+1]): logit>0 ? /pen : *pen, count times."""
    lib = library("core")
    R, V = logits.shape
    _check(lib, lib.forge_repeat_penalty(_need(logits, "logits", torch.float32, 2), _need(tokens, "tokens", torch.int32),
                                         _need(counts, "counts", torch.int32), _need(offsets, "offsets", torch.int32),
                                         _need(penalty, "penalty", torch.float32), R, V, _stream()), "repeat_penalty")
    return logits


def history_penalty(logits, counts, slot_of_row, penalty):
    """The repeat penalty with the history on the device: ``counts`` int32 [slots, V] (how often each token was
    generated, per request slot), ``slot_of_row`` int32 [R], ``penalty`` fp32 [R] (1 = none).  In place."""
    lib = library("core")
    R, V = logits.shape
    _check(lib, lib.forge_history_penalty(_need(logits, "logits", torch.float32, 2), _need(counts, "counts", torch.int32, 2),
                                          _need(slot_of_row, "slot_of_row", torch.int32), _need(penalty, "penalty", torch.float32),
                                          R, V, _stream()), "history_penalty")
    return logits


def history_add(counts, slot_of_row, tokens, penalty):
    """counts[slot_of_row[r], tokens[r]] += 1 for the rows with a penalty."""
    lib = library("core")
    R, V = tokens.numel(), counts.shape[1]
    _check(lib, lib.forge_history_add(_need(counts, "counts", torch.int32, 2), _need(slot_of_row, "slot_of_row", torch.int32),
                                      _need(tokens, "tokens", torch.int32), _need(penalty, "penalty", torch.float32), R, V,
                                      _stream()), "history_add")


def sample(logits, temperature, top_k, top_p, u, out=None):
    """int32 [R]: temperature / top-k / top-p sampling of each row with the caller's uniform numbers u [R]."""
    lib = library("core")
    R, V = logits.shape
    if out is None:
        out = new_tensor((R,), torch.int32, logits.device)
    _check(lib, lib.forge_sample(_need(logits, "logits", torch.float32, 2), _need(temperature, "temperature", torch.float32),
                                 _need(top_k, "top_k", torch.int32), _need(top_p, "top_p", torch.float32),
                                 _need(u, "u", torch.float32), _need(out, "out", torch.int32), R, V, _stream()), "sample")
    return out


# ------------------------------------------------------------------------------- tensor-core kernels

def gemm_sm100_supports(n, k):
    """The tcgen05 kernel reads rows by TMA: a row of K bfloat16 must be a multiple of 16 bytes."""
    return _TENSOR_CORE_GEMM and k % 8 == 0 and n >= 1


def attention_mma_supports(head_dim, group, page_size):
    """Head sizes in steps of 16 up to 256, any group size, any page size; other shapes use the fp32 kernel."""
    return _TENSOR_CORE_ATTENTION and head_dim % 16 == 0 and 16 <= head_dim <= 256


BQ_ROWS = 64        # query rows (token, head-of-group pairs) per attention tile
KV_TILE = 64        # keys per inner iteration
_NUM_SMS = {}


def _sm_count(device):
    key = str(device)
    if key not in _NUM_SMS:
        _NUM_SMS[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _NUM_SMS[key]


TC_ROWS = 128       # query rows per tile of the tcgen05 attention kernel
TC_MIN_ROWS = 64    # requests with at least this many rows in the step go to it


def attention_plan(batch, group, device, only_below=None):
    """How the step's query rows are cut into tiles for the tensor-core attention kernel, and into how
    many slices each tile's keys are cut.  Computed once per step and group size (all layers share it).
    A request with q_len tokens has q_len * group rows; tiles never span requests.  ``only_below``: plan
    only the requests with fewer rows than that (the others are served by the tcgen05 kernel)."""
    key = ("mma", group, only_below)
    plan = batch.attention_plan.get(key)
    if plan is not None:
        return plan
    tile_req, tile_row0, max_rows = [], [], 1
    qs = batch.host_q_start
    for s in range(batch.num_requests):
        rows = (qs[s + 1] - qs[s]) * group
        if only_below is not None and rows >= only_below:
            continue
        for r0 in range(0, rows, BQ_ROWS):
            tile_req.append(s)
            tile_row0.append(r0)
            max_rows = max(max_rows, min(BQ_ROWS, rows - r0))
    max_ctx = getattr(batch, "max_context", None)
    if max_ctx is None:
        max_ctx = max(c + qs[s + 1] - qs[s] for s, c in enumerate(batch.host_context_before))
    plan = {"tile_req": new_ints(tile_req, device), "tile_row0": new_ints(tile_row0, device),
            "num_tiles": len(tile_req), "max_rows": max_rows, "max_kv_tiles": -(-max_ctx // KV_TILE), "scratch": {}}
    batch.attention_plan[key] = plan
    return plan


TC_MIN_SHARE = 8     # key tiles (of 64 keys) that a share of a tile's keys holds at least
TC_MAX_SHARES = 32


def attention_plan_tc(batch, group, device, n_kv_heads=1, head_dim=64, window=0, shares=None):
    """Tiles of (128 // group) whole tokens, that is up to 128 rows, for the requests that bring at least TC_MIN_ROWS
    rows, heaviest (most keys) first.  When the step has at most half as many (tile, kv head) pairs as the GPU has
    places for the kernel's CTAs, the keys of the long tiles are cut into shares, in proportion to their length, so that the places
    are taken (a short portion on a long context); ``shares`` forces a number for every tile (tests)."""
    key = ("tc", group, n_kv_heads, head_dim, window, shares)
    plan = batch.attention_plan.get(key)
    if plan is not None:
        return plan
    tiles, qs = [], batch.host_q_start
    tile_rows = (TC_ROWS // group) * group
    for s in range(batch.num_requests):
        rows = (qs[s + 1] - qs[s]) * group
        if rows < TC_MIN_ROWS:
            continue
        ctx = batch.host_context_before[s]
        for r0 in range(0, rows, tile_rows):
            kv_hi = ctx + (min(rows, r0 + tile_rows) - 1) // group + 1
            kv_lo = max(0, ctx + r0 // group - window + 1) if window else 0
            tiles.append((-(-kv_hi // KV_TILE) - kv_lo // KV_TILE, s, r0))
    places = _sm_count(device) * (2 if head_dim <= 64 else 1)
    total = max(1, sum(t[0] for t in tiles) * n_kv_heads)

    def worth(n, scale):        # n / (total / places): how many places this tile's keys are worth
        return max(1, min(n // TC_MIN_SHARE, n * places * scale // (10 * total), TC_MAX_SHARES))
    if shares is not None:
        cut = [max(1, min(int(shares), t[0], TC_MAX_SHARES)) for t in tiles]
    else:
        cut = [1] * len(tiles)
        # (with more than half of the places taken already there is nothing to gain that pays for the second kernel)
        for scale in range(10, 4, -1) if 2 * len(tiles) * n_kv_heads <= places else ():
            # short tiles count as one whole place each: shrink the others' worth until all fit
            trial = [worth(t[0], scale) for t in tiles]
            if sum(trial) * n_kv_heads <= places:
                cut = trial
                break
    entries, merges, slots = [], [], 0
    for (n, s, r0), z in zip(tiles, cut):
        if z > 1:
            merges.append((s, r0, slots, z))
        entries += [(n / z, s, r0, i, z, slots if z > 1 else 0) for i in range(z)]
        slots += z if z > 1 else 0
    entries.sort(key=lambda e: (-e[0], e[1], e[2], e[3]))
    plan = {"tile_req": new_ints([e[1] for e in entries], device), "tile_row0": new_ints([e[2] for e in entries], device),
            "num_tiles": len(entries), "num_merge": len(merges), "tile_cut": None, "merge_list": None, "part_o": None, "part_ml": None}
    if merges:
        plan["tile_cut"] = new_ints([v for e in entries for v in e[3:6]], device)
        plan["merge_list"] = new_ints([v for m in merges for v in m], device)
        plan["part_o"] = new_tensor((slots * n_kv_heads * TC_ROWS * head_dim,), torch.float32, device, whole_step=True)
        plan["part_ml"] = new_tensor((slots * n_kv_heads * TC_ROWS * 2,), torch.float32, device, whole_step=True)
    batch.attention_plan[key] = plan
    return plan


def attention_sm100_supports(head_dim, group, page_size):
    """Head sizes 64 and 128, any group of up to 128 query heads per kv head, pages of 8 to 64 tokens."""
    return _TENSOR_CORE_ATTENTION and head_dim in (64, 128) and 1 <= group <= TC_ROWS and page_size in (8, 16, 32, 64)


def paged_attention_sm100(q, kv_cache, group_batch, batch, n_heads, n_kv_heads, head_dim, page_size, window=0,
                          scale=None, out=None, shares=None):
    """tcgen05/TMEM attention for the requests of the step that bring many rows (prompt portions).  Writes
    only those requests' rows of ``out``.  Returns (out, number of tiles run: a tile whose keys are cut into
    shares counts once per share)."""
    lib = library("attention_sm100", {"FORGE_ATT_HD": head_dim})
    plan = attention_plan_tc(batch, n_heads // n_kv_heads, q.device, n_kv_heads, head_dim, int(window or 0), shares)
    if out is None:
        out = new_tensor(q.shape, q.dtype, q.device)
    if plan["num_tiles"] == 0:
        return out, 0
    scale = head_dim ** -0.5 if scale is None else scale
    _check(lib, lib.forge_paged_attention_sm100(
        _need(q, "q", torch.bfloat16, 2), _need(kv_cache, "kv_cache", torch.bfloat16), _need(out, "out", torch.bfloat16),
        _need(group_batch.block_table, "block_table", torch.int32, 2), _need(plan["tile_req"], "tile_req"),
        _need(plan["tile_row0"], "tile_row0"), _opt(plan["tile_cut"], "tile_cut"), _opt(plan["part_o"], "part_o"),
        _opt(plan["part_ml"], "part_ml"), _opt(plan["merge_list"], "merge_list"), plan["num_merge"],
        _need(batch.q_start, "q_start", torch.int32),
        _need(batch.context_before, "context_before", torch.int32), _need(_gemm_status(q.device), "status", torch.int32),
        plan["num_tiles"], q.shape[0], kv_cache.shape[0], n_heads, n_kv_heads, head_dim, page_size,
        group_batch.block_table.shape[1], int(window or 0), float(scale), _stream()), "paged_attention_sm100")
    if plan["num_merge"]:
        count_launches(1)      # the kernel that adds the shares up
    return out, plan["num_tiles"]


def paged_attention_mma(q, kv_cache, group_batch, batch, n_heads, n_kv_heads, head_dim, page_size, window=0,
                        scale=None, out=None, num_splits=None, only_below=None):
    """bf16 tensor-core attention over the paged cache for every token of the step (or, with ``only_below``,
    for the requests that bring fewer rows than that)."""
    lib = library("attention_mma", {"FORGE_ATT_HD": head_dim})
    plan = attention_plan(batch, n_heads // n_kv_heads, q.device, only_below)
    if out is None:
        out = new_tensor(q.shape, q.dtype, q.device)
    if plan["num_tiles"] == 0:
        return out
    if num_splits is None:
        # decode-like steps (every tile is one warp with small buffers, ten of which fit an SM): slice the
        # keys until about eight CTAs per SM exist, so that enough loads are in flight to hide their latency
        base = plan["num_tiles"] * n_kv_heads
        num_splits = 1
        if plan["max_rows"] <= 16:
            num_splits = max(1, min(plan["max_kv_tiles"], -(-8 * _sm_count(q.device) // base)))
    part_o = part_ml = None
    if num_splits > 1:
        pr = 16 if plan["max_rows"] <= 16 else BQ_ROWS
        sk = (num_splits, head_dim, pr)
        if sk not in plan["scratch"]:
            n = plan["num_tiles"] * n_kv_heads * num_splits * pr
            plan["scratch"][sk] = (new_tensor((n * head_dim,), torch.float32, q.device, whole_step=True),
                                   new_tensor((n * 2,), torch.float32, q.device, whole_step=True))
        part_o, part_ml = plan["scratch"][sk]
    if out is None:
        out = new_tensor(q.shape, q.dtype, q.device)
    scale = head_dim ** -0.5 if scale is None else scale
    _check(lib, lib.forge_paged_attention_mma(
        _need(q, "q", torch.bfloat16, 2), _need(kv_cache, "kv_cache", torch.bfloat16), _need(out, "out", torch.bfloat16),
        _opt(part_o, "part_o"), _opt(part_ml, "part_ml"), _need(group_batch.block_table, "block_table", torch.int32, 2),
        _need(plan["tile_req"], "tile_req"), _need(plan["tile_row0"], "tile_row0"),
        _need(batch.q_start, "q_start", torch.int32), _need(batch.context_before, "context_before", torch.int32),
        plan["num_tiles"], plan["max_rows"], n_heads, n_kv_heads, head_dim, page_size, group_batch.block_table.shape[1],
        int(window or 0), int(num_splits), float(scale), _stream()), "paged_attention_mma")
    if num_splits > 1:
        count_launches(1)      # the merge kernel
    return out


def decode_attention_fused_supports(dtype, head_dim, group, num_requests, n_kv_heads, max_context, page_size=None):
    """One launch for rotary encoding + cache write + attention of a decode step: bfloat16, head sizes in steps
    of 16 up to 128, at most 16 query heads per kv head.  With few requests and long contexts the
    sliced kernel (keys spread over many CTAs) is the better choice."""
    if not (_TENSOR_CORE_ATTENTION and dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128 and group <= 16):
        return False
    # with few requests the kernel spreads a request's keys over a cluster of up to 4 CTAs; measured (22 layers, 4 kv
    # heads, 8 requests x 6,000 cached tokens) 1.10 ms per step against 1.26 for the sliced kernel + merge.  Beyond
    # 16k cached tokens with a handful of CTAs the sliced kernel's many CTAs are the better choice again.
    if page_size is not None and decode_attention_stream_supports(head_dim, page_size, group):
        # the kernel that streams the cache spreads a request over up to 8 CTAs and keeps a ring of tiles in flight:
        # the sliced kernel only wins with at most 16 (request, kv head) pairs beyond 16k tokens (measured: 4 pairs x
        # 32k tokens 25 against 18 us, 16 pairs 46 against 38; 32 pairs 50 against 63)
        return not (num_requests * n_kv_heads <= 16 and max_context > 16384)
    return not (num_requests * n_kv_heads < 64 and max_context > 16384)


# The decode attention that streams the cache through a TMA ring pays where a request has many tiles of 64 keys, or
# where there are more (request, kv head) pairs than SMs; with few pairs and fewer than this many cached tokens (an
# upper bound known on the host) the kernel with one buffer pair per warp, which asks for a short context's tiles
# before its dependency wait, is the faster one inside a step (measured, 8 requests x 540 tokens: 0.826 against
# 0.846 ms per step; 64 requests: 48.6 against 49.9 thousand tokens a second the other way round).
STREAM_ATTENTION_MIN_CONTEXT = int(os.environ.get("FORGE_STREAM_ATTENTION_MIN_CONTEXT", "2048"))
STREAM_ATTENTION_MANY_PAIRS = 148


def decode_attention_stream_supports(head_dim, page_size, group):
    return _TENSOR_CORE_ATTENTION and head_dim in (64, 128) and page_size in (16, 32, 64) and group <= 16


def decode_attention_stream(qkv, kv_cache, block_table, positions, slot_mapping, n_heads, n_kv_heads, head_dim, page_size,
                            theta, rotary=True, window=0, scale=None, out=None, max_context=0, ksplit=0):
    """The same step as ``decode_attention_fused`` with the keys and values brought by TMA into a ring of tiles
    (csrc/attention_decode_stream.cu): head sizes 64 and 128, pages of 16, 32 or 64 tokens.  ``ksplit``: CTAs that
    share a request's keys (0: chosen from ``max_context``)."""
    lib = library("attention_mma", {"FORGE_ATT_HD": head_dim})
    S = qkv.shape[0]
    if out is None:
        out = new_tensor((S, n_heads * head_dim), torch.bfloat16, qkv.device)
    scale = head_dim ** -0.5 if scale is None else scale
    _check(lib, lib.forge_decode_attention_stream(
        _need(qkv, "qkv", torch.float32, 2), _need(kv_cache, "kv_cache", torch.bfloat16), _need(out, "out", torch.bfloat16),
        _need(block_table, "block_table", torch.int32, 2), _need(positions, "positions", torch.int32),
        _need(slot_mapping, "slot_mapping", torch.int32), _need(_gemm_status(qkv.device), "status", torch.int32), S, n_heads,
        n_kv_heads, head_dim, page_size, block_table.shape[1], kv_cache.shape[0], int(window or 0), 1 if rotary else 0,
        float(theta), float(scale), int(max_context or 0), int(ksplit), _stream()), "decode_attention_stream")
    return out


def decode_attention_fused(qkv, kv_cache, block_table, positions, slot_mapping, n_heads, n_kv_heads, head_dim, page_size,
                           theta, rotary=True, window=0, scale=None, out=None, max_context=0):
    """qkv fp32 [S,(NH+2NKV)*HD], one new token per request: rotates q and k (``rotary``), writes k and v into
    the cache at ``slot_mapping`` and returns the attention output bf16 [S, NH*HD], all in one kernel.
    ``max_context``: an upper bound of any request's cached tokens + 1, if known: with few requests and many keys
    the kernel then spreads a request's keys over 2 or 4 CTAs."""
    pairs = qkv.shape[0] * n_kv_heads
    # (beyond some 768 pairs with short contexts the per-warp kernel is ahead again: 256 requests x 1,024 tokens 60 against 67 us)
    if ((max_context or 0) >= STREAM_ATTENTION_MIN_CONTEXT or STREAM_ATTENTION_MANY_PAIRS < pairs <= 768) and \
            decode_attention_stream_supports(head_dim, page_size, n_heads // n_kv_heads):
        return decode_attention_stream(qkv, kv_cache, block_table, positions, slot_mapping, n_heads, n_kv_heads, head_dim,
                                       page_size, theta, rotary=rotary, window=window, scale=scale, out=out, max_context=max_context)
    lib = library("attention_mma", {"FORGE_ATT_HD": head_dim})
    S = qkv.shape[0]
    if out is None:
        out = new_tensor((S, n_heads * head_dim), torch.bfloat16, qkv.device)
    scale = head_dim ** -0.5 if scale is None else scale
    _check(lib, lib.forge_decode_attention_fused(
        _need(qkv, "qkv", torch.float32, 2), _need(kv_cache, "kv_cache", torch.bfloat16), _need(out, "out", torch.bfloat16),
        _need(block_table, "block_table", torch.int32, 2), _need(positions, "positions", torch.int32),
        _need(slot_mapping, "slot_mapping", torch.int32), S, n_heads, n_kv_heads, head_dim, page_size, block_table.shape[1],
        int(window or 0), 1 if rotary else 0, float(theta), float(scale), int(max_context or 0), _stream()),
        "decode_attention_fused")
    return out


class DecodeLayers:
    """All layers of a decode step as one persistent kernel (csrc/decode_layers.cu).

    Made once per model from the layers' device tensors; ``run`` then takes the residual stream of a step of
    at most ``max_tokens`` single tokens through every layer, in place.  The object owns the kernel's scratch
    (fp32 results of the projections, attention output, barrier words), so calls must not overlap on the GPU.
    """
    MAX_TOKENS = 16

    @staticmethod
    def supports(hidden, intermediate, n_heads, n_kv_heads, head_dim, tokens=1):
        if not (_TENSOR_CORE_GEMM and _TENSOR_CORE_ATTENTION) or head_dim % 16 != 0 or not 16 <= head_dim <= 128:
            return False
        lib = library("decode_layers", {"FORGE_ATT_HD": head_dim})
        return bool(lib.forge_decode_layers_supports(int(tokens), hidden, intermediate, n_heads, n_kv_heads, head_dim))

    def __init__(self, layers, hidden, intermediate, n_heads, n_kv_heads, head_dim, page_size, theta, rotary, eps,
                 window=0, scale=None, max_tokens=MAX_TOKENS):
        """layers: per layer a dict of device tensors: wqkv bf16 [(NH+2NKV)*HD, H], wo [H, NH*HD], wgu [2I, H] (gate and
        up rows interleaved), wdown [H, I], norm1 / norm2 fp32 [H], bias fp32 [(NH+2NKV)*HD] or None, kv (the layer's
        cache [pages, 2, NKV, page_size, HD] bf16)."""
        self.lib = lib = library("decode_layers", {"FORGE_ATT_HD": head_dim})
        self.dims = (hidden, intermediate, n_heads, n_kv_heads, head_dim)
        self.page_size, self.theta, self.rotary, self.eps, self.window = int(page_size), float(theta), bool(rotary), float(eps), int(window or 0)
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.max_tokens = min(int(max_tokens), self.MAX_TOKENS)
        # weights are asked into L2 two or three products ahead of their use (0: off); a layer's matrices must fit
        # the L2 beside what is in use for that to pay
        self.prefetch_units = int(os.environ.get("FORGE_DECODE_PREFETCH_UNITS", "1"))
        dev = layers[0]["wqkv"].device
        self.num_layers = len(layers)
        nbytes = lib.forge_decode_layers_desc_bytes()
        self.descs = torch.zeros(self.num_layers * nbytes, dtype=torch.uint8, device=dev)
        self._keep = layers                                    # the maps hold raw pointers into these tensors
        with torch.cuda.device(dev):
            for i, t in enumerate(layers):
                rc = lib.forge_decode_layers_describe(
                    self.descs.data_ptr(), i, _need(t["wqkv"], "wqkv", torch.bfloat16, 2), _need(t["wo"], "wo", torch.bfloat16, 2),
                    _need(t["wgu"], "wgu", torch.bfloat16, 2), _need(t["wdown"], "wdown", torch.bfloat16, 2),
                    _need(t["norm1"], "norm1", torch.float32), _need(t["norm2"], "norm2", torch.float32),
                    _opt(t.get("bias"), "bias", torch.float32), _need(t["kv"], "kv", torch.bfloat16), hidden, intermediate,
                    n_heads, n_kv_heads, head_dim)
                if rc != 0:
                    raise KernelError(f"decode_layers: {lib.forge_last_error().decode(errors='replace')} (code {rc})")
        B, qkv = self.max_tokens, (n_heads + 2 * n_kv_heads) * head_dim
        self.qkv_acc = torch.zeros(B * qkv, dtype=torch.float32, device=dev)
        self.gu_acc = torch.zeros(B * 2 * intermediate, dtype=torch.float32, device=dev)
        self.ssq = torch.zeros(128, dtype=torch.float32, device=dev)
        self.rope_tab = torch.zeros(B * head_dim, dtype=torch.float32, device=dev)
        self.part_o = torch.zeros(B * n_kv_heads * 4 * 16 * head_dim, dtype=torch.float32, device=dev)
        self.part_ml = torch.zeros(B * n_kv_heads * 4 * 16 * 2, dtype=torch.float32, device=dev)
        self.barrier = torch.zeros(4, dtype=torch.int32, device=dev)

    def run(self, residual, block_table, positions, slot_mapping, timeline=None):
        """residual fp32 [B, H], updated in place; block_table int32 [B, max_pages]; positions, slot_mapping int32 [B].
        ``timeline``: an int64 tensor [SMs, 1 + 5 * layers, 2] that receives when each CTA reached and left each of
        the kernel's barriers (ns of the device's clock), for a look at where a step's time goes."""
        H, I, NH, NKV, HD = self.dims
        B = residual.shape[0]
        if B > self.max_tokens or residual.shape[1] != H:
            raise KernelError(f"decode_layers: residual {tuple(residual.shape)} does not fit ({self.max_tokens} tokens of {H})")
        lib = self.lib
        _check(lib, lib.forge_decode_layers(
            self.descs.data_ptr(), self.num_layers, _need(residual, "residual", torch.float32, 2), self.qkv_acc.data_ptr(),
            self.gu_acc.data_ptr(), self.ssq.data_ptr(), self.rope_tab.data_ptr(), self.part_o.data_ptr(),
            self.part_ml.data_ptr(), _need(block_table, "block_table", torch.int32, 2),
            _need(positions, "positions", torch.int32), _need(slot_mapping, "slot_mapping", torch.int32), self.barrier.data_ptr(),
            _need(_gemm_status(residual.device), "status", torch.int32), B, H, I, NH, NKV, HD, self.page_size,
            block_table.shape[1], self.window, 1 if self.rotary else 0, self.theta, self.scale, self.eps, self.prefetch_units,
            _opt(timeline, "timeline", torch.int64), _stream()), "decode_layers")
        return residual

    def reset_after_error(self):
        """After a wait ran out the barrier words are left as they were; clear them before the next step."""
        self.barrier.zero_()


def paged_attention(q, kv_cache, group_batch, batch, n_heads, n_kv_heads, head_dim, page_size, window=None,
                    scale=None):
    """Attention of every token of the step over its request's pages; picks the kernel by dtype and shape."""
    if q.dtype == torch.bfloat16 and attention_mma_supports(head_dim, n_heads // n_kv_heads, page_size):
        group = n_heads // n_kv_heads
        if attention_sm100_supports(head_dim, group, page_size) and not getattr(batch, "decode_only", False):
            out, n = paged_attention_sm100(q, kv_cache, group_batch, batch, n_heads, n_kv_heads, head_dim, page_size,
                                           window=window or 0, scale=scale)
            if n:       # the requests with few rows (decode tokens, short portions) use the mma.sync kernel
                return paged_attention_mma(q, kv_cache, group_batch, batch, n_heads, n_kv_heads, head_dim, page_size,
                                           window=window or 0, scale=scale, out=out, only_below=TC_MIN_ROWS)
        return paged_attention_mma(q, kv_cache, group_batch, batch, n_heads, n_kv_heads, head_dim, page_size,
                                   window=window or 0, scale=scale)
    return paged_attention_simt(q, kv_cache, group_batch.block_table, batch.tok_req, batch.positions, n_heads,
                                n_kv_heads, head_dim, page_size, window=window or 0, scale=scale)


EPILOGUES = {"none": 0, "accumulate": 1, "cast": 2, "swiglu": 3}


def gemm_sm100(x, w, bias=None, accumulate_into=None, epilogue="none", tile_n=0, status=None, out=None):
    """bf16 x [M,K] . w [N,K]^T on the tcgen05 tensor cores, fp32 accumulation.
    epilogue "none": fp32 [M,N] (added into ``accumulate_into`` when given); "cast": bf16 [M,N];
    "swiglu": bf16 [M,N/2] = silu(y[:,2j]) * y[:,2j+1]."""
    lib = library("gemm_sm100")
    (M, K), (N, K2) = x.shape, w.shape
    if K != K2:
        raise KernelError(f"gemm_sm100: x {tuple(x.shape)} does not match w {tuple(w.shape)}")
    if epilogue == "none":
        if accumulate_into is not None:
            out, code = accumulate_into, EPILOGUES["accumulate"]
        else:
            out = new_tensor((M, N), torch.float32, x.device) if out is None else out
            code = EPILOGUES["none"]
        want_shape, want_dtype = (M, N), torch.float32
    elif epilogue == "cast":
        out = new_tensor((M, N), torch.bfloat16, x.device) if out is None else out
        code, want_shape, want_dtype = EPILOGUES["cast"], (M, N), torch.bfloat16
    elif epilogue == "swiglu":
        out = new_tensor((M, N // 2), torch.bfloat16, x.device) if out is None else out
        code, want_shape, want_dtype = EPILOGUES["swiglu"], (M, N // 2), torch.bfloat16
    else:
        raise KernelError(f"gemm_sm100: unknown epilogue {epilogue!r}")
    if tuple(out.shape) != want_shape:
        raise KernelError(f"gemm_sm100: output has shape {tuple(out.shape)}, expected {want_shape}")
    if status is None:
        status = _gemm_status(x.device)
    _gemm_workspace(lib, x.device)
    _check(lib, lib.forge_gemm_sm100(_need(x, "x", torch.bfloat16, 2), _need(w, "w", torch.bfloat16, 2),
                                     _opt(bias, "bias", torch.float32), _need(out, "out", want_dtype),
                                     _need(status, "status", torch.int32), M, N, K, code, int(tile_n), None, _stream()),
           "gemm_sm100")
    return out


def gemm_sm100_qkv_rope_supports(rows, head_dim, k):
    """The projection whose epilogue rotates and stores: prompt portions (more than 128 rows), head sizes 64 and 128."""
    return _TENSOR_CORE_GEMM and rows > 128 and head_dim in (64, 128) and k % 8 == 0


def gemm_sm100_qkv_rope(x, w, bias, rope_table, slot_mapping, kv_cache, n_heads, n_kv_heads, head_dim, page_size, q_out=None,
                        tile=0):
    """bf16 x [M,K] . w [(NH+2NKV)*HD, K]^T (+ bias) on the tensor cores; the epilogue rotates q and k by ``rope_table``
    (fp32 [HD/2, M, 2] of (cos, sin), ``rope_table(..., by_pair=True)``; None: no rotation), returns q bf16 [M, NH*HD] and writes k and v into ``kv_cache``
    at ``slot_mapping`` (None: not written).  The fp32 product never reaches global memory.  ``tile``: 0 lets the
    library choose; 128 / 256 one CTA per tile of that width, 1128 / 1192 / 1256 a pair of CTAs on 256 rows of it."""
    lib = library("gemm_sm100")
    (M, K), (N, K2) = x.shape, w.shape
    if K != K2 or N != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError(f"gemm_sm100_qkv_rope: x {tuple(x.shape)}, w {tuple(w.shape)} do not fit {n_heads}+2*{n_kv_heads} heads of {head_dim}")
    if q_out is None:
        q_out = new_tensor((M, n_heads * head_dim), torch.bfloat16, x.device)
    if kv_cache is None:
        slot_mapping = None
    _check(lib, lib.forge_gemm_sm100_qkv_rope(
        _need(x, "x", torch.bfloat16, 2), _need(w, "w", torch.bfloat16, 2), _opt(bias, "bias", torch.float32),
        _need(q_out, "q_out", torch.bfloat16, 2), _opt(kv_cache, "kv_cache", torch.bfloat16), _opt(rope_table, "rope_table", torch.float32),
        _opt(slot_mapping, "slot_mapping", torch.int32), _need(_gemm_status(x.device), "status", torch.int32), M, K, n_heads,
        n_kv_heads, head_dim, page_size, tile, _stream()), "gemm_sm100_qkv_rope")
    return q_out


_status_words = {}
_workspaces = {}
GEMM_WORKSPACE_BYTES = 48 * 1024 * 1024


def _gemm_workspace(lib, device):
    """One zeroed buffer per device for the few-rows GEMM's partial sums and flags, given to the library once."""
    key = str(device)
    if key not in _workspaces:
        ws = torch.zeros(GEMM_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        with torch.cuda.device(device), once_per_step():
            rc = lib.forge_gemm_sm100_set_workspace(ws.data_ptr(), GEMM_WORKSPACE_BYTES)
        if rc != 0:
            raise KernelError(f"gemm_sm100: {lib.forge_last_error().decode(errors='replace')}")
        _workspaces[key] = ws
    return _workspaces[key]



def _gemm_status(device):
    """One int32 per device on which tensor-core kernels raise bit 1 when a bounded wait runs out."""
    dev = torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    key = str(dev)
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status_words[key]


def check_kernel_status(device="cuda:0"):
    """Synchronises and raises if a tensor-core kernel gave up on a wait since the last check."""
    dev = torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    w = _status_words.get(str(dev))
    if w is not None:
        v = int(w.item())
        if v:
            w.zero_()
            raise KernelError(f"a tensor-core kernel reported status {v:#x} (a bounded wait ran out)")


_TENSOR_CORE_GEMM = True
_TENSOR_CORE_ATTENTION = True
