"""Kernel entry points: checked Python wrappers over the compiled sm_100a libraries.

Every function here launches hand-written CUDA on the current stream of its
tensors' device.  There is no CPU path and no fallback: a tensor that is not on
a CUDA device, or a library that cannot be compiled or loaded, raises.  Shapes,
dtypes, contiguity and size limits are checked here, before the launch, so that
a size a kernel does not take is refused with a message and never computed
wrongly.
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Dict, Iterable, Optional

import torch

from . import build as _build

_libs: Dict[str, ctypes.CDLL] = {}

_F32, _BF16 = 0, 1
_STATUS_TEXT = {
    1: "a block-table entry outside the page pool was met (page not held by the request)",
    2: "a token id outside the vocabulary was met",
    3: "a row index outside its tensor was met",
    4: "a bounded wait inside a kernel ran out",
}


class KernelError(RuntimeError):
    pass


# ------------------------------------------------------------------ loading
def prepare(names: Iterable[str], verbose: bool = False) -> None:
    """Compile (if needed) and load the named libraries; raises if that is impossible."""
    names = [n for n in dict.fromkeys(names) if n not in _libs]
    if not names:
        return
    paths = _build.ensure_built(names, verbose=verbose)
    for n in names:
        try:
            _libs[n] = ctypes.CDLL(paths[n])
        except OSError as e:
            raise KernelError(f"cannot load kernel library '{n}' from {paths[n]}: {e}") from None
        _libs[n].lsb_error_string.restype = ctypes.c_char_p


def loaded_libraries() -> Dict[str, str]:
    return {n: lib._name for n, lib in _libs.items()}


def _lib(name: str) -> ctypes.CDLL:
    if name not in _libs:
        prepare([name])
    return _libs[name]


def check_status() -> None:
    """Read (and clear) every loaded library's status word; raises if a kernel recorded a fault.
    Synchronises the device."""
    for n, lib in _libs.items():
        code = ctypes.c_int(0)
        rc = lib.lsb_take_status(ctypes.byref(code))
        if rc != 0:
            raise KernelError(f"{n}: reading the status word failed: "
                              f"{lib.lsb_error_string(rc).decode()}")
        if code.value != 0:
            raise KernelError(f"{n}: {_STATUS_TEXT.get(code.value, f'status {code.value}')}")


_launches = 0
_scratch: Dict[tuple, torch.Tensor] = {}      # scratch buffers by use and size, kept for reuse


def launch_count() -> int:
    """How many kernel launches this process has made through this module."""
    return _launches


def _call(libname: str, fn: str, *args) -> None:
    global _launches
    lib = _lib(libname)
    _launches += 1
    cfn = getattr(lib, fn)
    rc = cfn(*args)
    if rc != 0:
        raise KernelError(f"{fn} failed: {lib.lsb_error_string(rc).decode()} (code {rc})")
    if _recording is not None:
        _recording.ops.append([cfn, list(args), fn, lib, ()])


# ------------------------------------------------------ a layer's launches, recorded
# The layers of a model are the same sequence of launches with other weights.  What the host does
# per launch (checks, choosing a kernel, sizing grids, allocating the output) is the same work for
# every layer of a step, and in steps that hold prompt portions (launched kernel by kernel, unlike
# decode steps, which replay a captured graph) it is most of the host's time.  So the model records
# the launches of one layer call and repeats them for the calls after it that have the same shape,
# with the pointers of that layer's own tensors (weights, cache pages, the delta coming in and
# going out) exchanged for the next layer's; every other buffer is the recorded layer's, reused in
# stream order.
LAYER_REPLAY = True
_recording: Optional["LayerRecording"] = None


class LayerRecording:
    """The launches of one layer call: C entry points with their packed arguments and, between
    them, stream operations (the second stream of steps that hold decode tokens and portions)."""

    def __init__(self):
        self.ops = []          # [cfunction, args, name, lib, slots] or a callable (a stream operation)
        self.keep = []         # tensors whose memory the recorded launches use
        self._before = None

    def __enter__(self):
        global _recording
        self._before, _recording = _recording, self
        return self

    def __exit__(self, *exc):
        global _recording
        _recording = self._before
        return False

    def bind(self, roles: Dict[int, object]) -> None:
        """``roles``: device address -> name, for every tensor that is the recorded layer's own.
        Arguments that hold such an address become slots that :meth:`replay` fills."""
        for op in self.ops:
            if not callable(op):
                op[4] = tuple((i, roles[a.value]) for i, a in enumerate(op[1])
                              if isinstance(a, ctypes.c_void_p) and a.value in roles)

    def replay(self, addresses: Dict[object, int]) -> None:
        """Launch everything again with the slots pointing at ``addresses[name]``."""
        global _launches
        for op in self.ops:
            if callable(op):
                op()
                continue
            cfn, args, name, lib, slots = op
            for i, role in slots:
                args[i] = ctypes.c_void_p(addresses[role])
            _launches += 1
            rc = cfn(*args)
            if rc != 0:
                raise KernelError(f"{name} failed: {lib.lsb_error_string(rc).decode()} (code {rc})")


def _stream_op(fn) -> None:
    """Do a stream or event operation now and, when a layer is being recorded, again at every replay."""
    fn()
    if _recording is not None:
        _recording.ops.append(fn)


# ------------------------------------------------------------------- helpers
def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _req(t: torch.Tensor, name: str, dtype=None, dim: Optional[int] = None, contiguous=True):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name} must have {dim} dims, got shape {tuple(t.shape)}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def _p(t: Optional[torch.Tensor]):
    if _recording is not None and t is not None:
        _recording.keep.append(t)
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = torch._C._cuda_getCurrentRawStream      # (device index) -> cudaStream_t as int


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(_raw_stream(t.device.index))


_i = ctypes.c_int
_ll = ctypes.c_longlong
_f = ctypes.c_float


# ---------------------------------------------------------------------- ops
def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor) -> None:
    """dst.flat[idx[i]] = val[i]."""
    _req(dst, "dst", torch.int32)
    _req(idx, "idx", torch.int32, 1)
    _req(val, "val", torch.int32, 1)
    if idx.numel() != val.numel():
        raise KernelError("scatter_i32: idx and val differ in length")
    _call("cache_table", "lsb_scatter_i32", _p(dst), _p(idx), _p(val), _i(idx.numel()),
          _ll(dst.numel()), _stream(dst))


def move_i32(dst: torch.Tensor, dst_idx: torch.Tensor, src: torch.Tensor, src_idx: torch.Tensor) -> None:
    """dst[dst_idx[i]] = src[src_idx[i]]."""
    for name, t in (("dst", dst), ("dst_idx", dst_idx), ("src", src), ("src_idx", src_idx)):
        _req(t, name, torch.int32, 1)
    if dst_idx.numel() != src_idx.numel():
        raise KernelError("move_i32: dst_idx and src_idx differ in length")
    _call("cache_table", "lsb_move_i32", _p(dst), _p(dst_idx), _p(src), _p(src_idx), _i(dst_idx.numel()),
          _ll(dst.numel()), _ll(src.numel()), _stream(dst))


def scatter_i32_counted(dst: torch.Tensor, packed: torch.Tensor, cap: int) -> None:
    """dst.flat[idx[i]] = val[i] for i < n, with packed = [n, idx[cap], val[cap]] on the device."""
    _req(dst, "dst", torch.int32)
    _req(packed, "packed", torch.int32, 1)
    if packed.numel() != 1 + 2 * cap:
        raise KernelError("scatter_i32_counted: packed must hold 1 + 2 * cap ints")
    _call("cache_table", "lsb_scatter_i32_counted", _p(dst), _p(packed), _i(cap), _ll(dst.numel()),
          _stream(dst))


def random_normal(out: torch.Tensor, key: int, mean: float, scale: float) -> None:
    """out.flat[i] = mean + scale * normal(key, i): the counter-based stream of the random-weights
    mode (``weights/random_init.py`` states the same arithmetic for the CPU)."""
    _req(out, "out")
    _call("random_init", "lsb_random_normal", _p(out), _i(_dt(out)), _ll(out.numel()),
          ctypes.c_ulonglong(key & ((1 << 64) - 1)), _f(mean), _f(scale), _stream(out))


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] = float(table[ids[t], :]) * scale."""
    _req(table, "table", dim=2)
    _req(ids, "ids", torch.int32, 1)
    _req(out, "out", torch.float32, 2)
    if out.shape != (ids.shape[0], table.shape[1]):
        raise KernelError(f"embedding: out is {tuple(out.shape)}, expected "
                          f"{(ids.shape[0], table.shape[1])}")
    _call("embedding", "lsb_embedding", _p(table), _i(_dt(table)), _p(ids), _p(out),
          _i(ids.shape[0]), _i(table.shape[1]), _i(table.shape[0]), _f(scale), _stream(out))


def embedding_pair(table: torch.Tensor, pair_table: torch.Tensor, ctx, last_token: torch.Tensor, buckets: int,
                   mul_prev: int, mul_cur: int, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] = float(table[id_t, :]) * scale + float(pair_table[row_t, :]) with row_t = (id_(t-1) * mul_prev +
    id_t * mul_cur) mod buckets, and row ``buckets`` for a sequence's first token.  ``last_token`` (int32, one
    per request slot) holds the token before a portion's first and is left holding the portion's last."""
    _req(table, "table", dim=2)
    _req(pair_table, "pair_table", table.dtype, 2)
    _req(last_token, "last_token", torch.int32, 1)
    _req(out, "out", torch.float32, 2)
    T = ctx.n_tokens
    if out.shape != (T, table.shape[1]) or pair_table.shape != (buckets + 1, table.shape[1]):
        raise KernelError("embedding_pair: out must be [tokens, hidden] and the pair table [buckets + 1, hidden]")
    _call("embedding", "lsb_embedding_pair", _p(table), _p(pair_table), _i(_dt(table)), _p(ctx.token_ids),
          _p(ctx.positions), _p(ctx.token_req), _p(ctx.q_start), _p(ctx.table_rows), _p(last_token), _p(out), _i(T),
          _i(table.shape[1]), _i(table.shape[0]), _i(buckets), _ll(mul_prev), _ll(mul_cur), _i(last_token.shape[0]),
          _f(scale), _stream(out))


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor) -> None:
    """residual += delta (in place, 32-bit); out = rmsnorm(residual) * weight."""
    _req(residual, "residual", torch.float32, 2)
    _req(weight, "weight", torch.float32, 1)
    _req(out, "out", dim=2)
    T, H = residual.shape
    if out.shape != (T, H) or weight.shape[0] != H:
        raise KernelError("add_rmsnorm: shapes of residual, weight and out disagree")
    if delta is not None:
        _req(delta, "delta", out.dtype, 2)
        if delta.shape != (T, H):
            raise KernelError("add_rmsnorm: delta has another shape than residual")
    _call("norm", "lsb_add_rmsnorm", _p(residual), _p(delta), _p(weight), _p(out), _i(_dt(out)),
          _i(T), _i(H), _f(eps), _stream(out))


def gather_add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor,
                       weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[i] = rmsnorm(residual[rows[i]] + delta[rows[i]]) * weight; residual unchanged."""
    _req(residual, "residual", torch.float32, 2)
    _req(rows, "rows", torch.int32, 1)
    _req(weight, "weight", torch.float32, 1)
    _req(out, "out", dim=2)
    T, H = residual.shape
    if out.shape != (rows.shape[0], H) or weight.shape[0] != H:
        raise KernelError("gather_add_rmsnorm: shapes disagree")
    if delta is not None:
        _req(delta, "delta", out.dtype, 2)
        if delta.shape != (T, H):
            raise KernelError("gather_add_rmsnorm: delta has another shape than residual")
    _call("norm", "lsb_gather_add_rmsnorm", _p(residual), _p(delta), _p(rows), _p(weight), _p(out),
          _i(_dt(out)), _i(rows.shape[0]), _i(T), _i(H), _f(eps), _stream(out))


ACTIVATIONS = {"silu": 1, "gelu_tanh": 2, "none": 3, "capped_glu": 5}     # act(gate) * up of a gated product
# "capped_glu" has a limit L: min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u, -L, L) + 1).  The tile kernel's
# epilogue knows it (prompt steps, the experts' grouped product) and so does the streaming product's (steps of
# a few rows); where another kernel makes the product (32-bit, sizes those two refuse) it leaves gate and up
# side by side and the activation kernel follows.
UNFUSED_GATED = ("capped_glu",)


def _activation_id(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation '{name}' is not implemented "
                          f"(known: {', '.join(sorted(ACTIVATIONS))})") from None


class NormOut:
    """Rows as they leave an RMS norm that a product folded in.  ``values`` [M, H] is the residual
    row times the norm's weight, rounded to the compute dtype; ``parts`` [P, 16] holds each row's
    sum of squares in P parts (row m in column m), and the factor ``rsqrt(sum / H + eps)`` per row
    is still owed: the next product scales its output rows by it (``linear`` takes a NormOut for
    ``x``), which is the same as normalising first.  ``parts`` None: nothing is owed, ``values``
    are the normalised rows (where no kernel could fold the norm).  ``finish_norm`` gives the
    normalised rows in either case."""
    __slots__ = ("values", "parts", "eps")

    def __init__(self, values: torch.Tensor, parts: Optional[torch.Tensor] = None, eps: float = 0.0):
        self.values, self.parts, self.eps = values, parts, float(eps)

    shape = property(lambda self: self.values.shape)
    dtype = property(lambda self: self.values.dtype)
    device = property(lambda self: self.values.device)


FOLD_NORMS = True               # decode steps fold each norm into the products on either side of it

# Warming.  A streaming product (csrc/gemm_stream.cu) can ask L2, while it ends, for the first
# weights of the streaming product after it, so that HBM works through the gap between the two
# kernels (csrc/stream_warm.cuh).  Which product comes next is not something a part knows; it is
# learnt here: the matrix that followed a matrix the last time is expected to follow it again,
# which holds from a model's second step on (and a decode step runs once before it is captured in
# a graph).  A wrong guess costs a few prefetched bytes; nothing depends on it.  Any other product
# in between (more than 16 rows, the output head) ends the chain.
WARM_NEXT = True
_follows: Dict[int, tuple] = {}         # address of a matrix -> (weak reference to its follower, gated)
_warm_structs: Dict[tuple, object] = {}  # (address, rows, gated) -> (weak reference, filled-in StreamWarm)
_last_streamed: Optional[int] = None


def _warm_after(w: torch.Tensor, gated: bool, M: int):
    """Note that ``w`` is being streamed now; the StreamWarm for what followed it last time, or None."""
    global _last_streamed
    if not WARM_NEXT:
        return None
    here = w.data_ptr()
    if _last_streamed is not None and _last_streamed != here:
        _follows[_last_streamed] = (weakref.ref(w), gated)
    _last_streamed = here
    nxt = _follows.get(here)
    if nxt is None:
        return None
    t = nxt[0]()
    if t is None:
        del _follows[here]
        return None
    key = (t.data_ptr(), M, nxt[1])
    made = _warm_structs.get(key)
    if made is None or made[0]() is not t:
        lib = _lib("gemm_stream")
        buf = ctypes.create_string_buffer(lib.lsb_stream_warm_bytes())
        rc = lib.lsb_gemm_stream_warm(_p(t), _i(M), _i(t.shape[0]), _i(t.shape[1]),
                                      _i(ACTIVATIONS["silu"] if nxt[1] else 0), _i(0), buf)
        made = _warm_structs[key] = (weakref.ref(t), buf if rc == 0 else None)
    return made[1]


def _chain_ends() -> None:
    global _last_streamed
    _last_streamed = None


def folds_norm(rows: int, dtype: torch.dtype) -> bool:
    """Does a step of this many rows fold its norms into the neighbouring products?  (The products
    of at most 16 bfloat16 rows, which one kernel streams: there a norm's own kernel costs more
    than the bytes it moves.)"""
    return FOLD_NORMS and STREAM_PRODUCTS and dtype == torch.bfloat16 and 0 < rows <= 16


def finish_norm(x: NormOut) -> torch.Tensor:
    """The normalised rows a NormOut stands for."""
    if x.parts is None:
        return x.values
    M, H = x.values.shape
    out = torch.empty_like(x.values)
    _call("norm", "lsb_finish_norm", _p(x.values), _p(x.parts), _i(x.parts.shape[0]), _p(out), _i(_dt(out)),
          _i(M), _i(H), _f(x.eps), _stream(out))
    return out


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           gated: bool = False, activation: str = "silu", into=None, limit: float = 0.0):
    """x [M, K] times w [N, K] transposed -> [M, N]; 32-bit accumulation.

    ``x`` may be a ``NormOut`` (the norm before this product, possibly half done: see there).
    ``into = (residual, norm_weight, eps)``: the product is added to ``residual`` ([M, N] 32-bit, in
    place) and what comes back is a ``NormOut``: what follows the RMS norm with that weight.

    float32 operands run on the CUDA cores in true 32-bit.  bfloat16 operands run on the
    tensor cores (tcgen05, accumulators in TMEM) when K is a multiple of 8, else on the CUDA
    cores as well.

    ``gated``: the rows of ``w`` alternate gate_i, up_i and the result is [M, N / 2] with
    ``out[m, i] = act(d[m, 2i]) * d[m, 2i + 1]`` (applied in the product's epilogue on the
    tensor-core path, by the activation kernel otherwise); ``activation`` names act: "silu",
    "gelu_tanh", "none", or "capped_glu" with its ``limit``.
    """
    if gated and activation in UNFUSED_GATED:
        if into is not None:
            raise KernelError("linear: a product into the residual is plain and in the compute dtype")
        if not limit > 0:
            raise KernelError(f"linear: '{activation}' needs a positive limit")
        if isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] > 16 \
                and w.shape[0] % 2 == 0 and tensor_core_gemm_ok(x, w) and (out_dtype or x.dtype) in (x.dtype, torch.float32):
            # the tile kernel's epilogue knows the capped form; steps of a few rows take the plain way below
            _req(w, "w", x.dtype, 2)
            if w.shape[1] != x.shape[1]:
                raise KernelError(f"linear: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
            _chain_ends()
            od = out_dtype or x.dtype
            out = torch.empty((x.shape[0], w.shape[0] // 2), dtype=od, device=x.device)
            _call("gemm_tc", "lsb_gemm_tc", _p(x), _p(w), _p(out), _i(1 if od == torch.float32 else 0),
                  _i(x.shape[0]), _i(w.shape[0]), _i(x.shape[1]), _i(_activation_id(activation)), _f(limit), _stream(out))
            return out
        act5 = _activation_id(activation)
        if isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] <= 16 \
                and STREAM_PRODUCTS and w.dim() == 2 and w.dtype == x.dtype and w.shape[1] == x.shape[1] \
                and (out_dtype or x.dtype) in (x.dtype, torch.float32) and stream_gemm_ok(x, w, act5):
            # a few rows: the streaming product's end knows the capped form too
            od = out_dtype or x.dtype
            out = torch.empty((x.shape[0], w.shape[0] // 2), dtype=od, device=x.device)
            _call("gemm_stream", "lsb_gemm_stream_capped", _p(x), _p(w), _p(out), _i(1 if od == torch.float32 else 0),
                  _i(x.shape[0]), _i(w.shape[0]), _i(x.shape[1]), _f(limit), _warm_after(w, True, x.shape[0]), _stream(out))
            return out
        raw = linear(x, w, out_dtype)
        half = torch.empty((raw.shape[0], raw.shape[1] // 2), dtype=raw.dtype, device=raw.device)
        gated_activation(raw, half, activation, limit)
        return half
    act = _activation_id(activation) if gated else 0
    owed = None
    if isinstance(x, NormOut):
        owed, x = (x if x.parts is not None else None), x.values
    _req(x, "x", dim=2)
    _req(w, "w", x.dtype, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if gated and N % 2:
        raise KernelError("linear: a gated product needs an even number of weight rows")
    out_dtype = out_dtype or x.dtype
    if out_dtype not in (x.dtype, torch.float32):
        raise KernelError(f"linear: output must be {x.dtype} or float32")
    if into is not None:
        residual, norm_w, eps = into
        if gated or out_dtype != x.dtype:
            raise KernelError("linear: a product into the residual is plain and in the compute dtype")
        _req(residual, "residual", torch.float32, 2)
        _req(norm_w, "norm weight", torch.float32, 1)
        if residual.shape != (M, N) or norm_w.shape[0] != N:
            raise KernelError("linear: residual and norm weight do not fit the product")
    if (owed is not None or into is not None) and x.dtype == torch.bfloat16 and STREAM_PRODUCTS \
            and M <= 16 and stream_gemm_ok(x, w, act):
        lib = _lib("gemm_stream")
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        parts = None
        if into is not None:
            parts = torch.empty((lib.lsb_gemm_stream_blocks(_i(M), _i(N), _i(K), _i(act)), 16),
                                dtype=torch.float32, device=x.device)
        _call("gemm_stream", "lsb_gemm_stream_folded", _p(x), _p(w), _p(out),
              _i(1 if out_dtype == torch.float32 else 0), _i(M), _i(N), _i(K), _i(act),
              _p(owed.parts if owed is not None else None), _i(owed.parts.shape[0] if owed is not None else 0),
              _i(K), _f(owed.eps if owed is not None else 0.0),
              _p(into[0] if into is not None else None), _p(into[1] if into is not None else None), _p(parts),
              _warm_after(w, gated, M), _stream(out))
        return NormOut(out, parts, into[2]) if into is not None else out
    if owed is not None:
        x = finish_norm(owed)
    if into is not None:
        delta = linear(x, w, out_dtype)
        out = torch.empty_like(delta)
        add_rmsnorm(into[0], delta, into[1], into[2], out)
        return NormOut(out)
    if x.dtype == torch.bfloat16 and SMALL_PRODUCTS and not gated and M <= 16 and small_gemm_ok(x, w):
        # a few rows times a matrix that fits the chip's shared memory (decode: q/k/v, output
        # projection): weights resident before the previous kernel has ended, no cluster
        _chain_ends()
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        _call("gemm_small", "lsb_gemm_small", _p(x), _p(w), _p(out), _i(1 if out_dtype == torch.float32 else 0),
              _i(M), _i(N), _i(K), _stream(out))
        return out
    if x.dtype == torch.bfloat16 and STREAM_PRODUCTS and M <= 16 and stream_gemm_ok(x, w, act):
        # a few rows times a matrix of any size (decode: gate/up, down): every SM streams its own
        # share of the weight rows, the first chunks before the previous kernel has ended
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        _call("gemm_stream", "lsb_gemm_stream_folded", _p(x), _p(w), _p(out),
              _i(1 if out_dtype == torch.float32 else 0), _i(M), _i(N), _i(K), _i(act), _p(None), _i(0), _i(K),
              _f(0.0), _p(None), _p(None), _p(None), _warm_after(w, gated, M), _stream(out))
        return out
    _chain_ends()
    if x.dtype == torch.bfloat16 and tensor_core_gemm_ok(x, w):
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        _call("gemm_tc", "lsb_gemm_tc", _p(x), _p(w), _p(out), _i(1 if out_dtype == torch.float32 else 0),
              _i(M), _i(N), _i(K), _i(act), _f(0.0), _stream(out))
        return out
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _call("gemm", "lsb_gemm_nt", _p(x), _p(w), _p(out), _i(_dt(x)), _i(_dt(out)), _i(M), _i(N), _i(K),
          _ll(K), _ll(K), _ll(N), _stream(out))
    if gated:
        half = torch.empty((M, N // 2), dtype=out_dtype, device=x.device)
        gated_activation(out, half, activation)
        return half
    return out


SMALL_PRODUCTS = True           # products of at most 16 rows with a small matrix: csrc/gemm_small.cu
STREAM_PRODUCTS = True          # products of at most 16 rows with any matrix: csrc/gemm_stream.cu
STREAM_MAX_ROWS = 65536         # weight rows beyond which the tile kernel's persistent form is used


def stream_gemm_ok(x: torch.Tensor, w: torch.Tensor, act: int = 0) -> bool:
    """Does the streaming kernel take x [M, K] times w [N, K] transposed?  (bfloat16, M <= 16, K a
    multiple of 64; the output head, far more rows than the SMs can share out in a few passes,
    stays with the persistent tile kernel.)"""
    M, K = x.shape
    N = w.shape[0]
    if M > 16 or K % 64 or N > STREAM_MAX_ROWS:
        return False
    return bool(_lib("gemm_stream").lsb_gemm_stream_supported(_p(x), _p(w), _i(M), _i(N), _i(K), _i(act)))



def small_gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Does the small-product kernel take x [M, K] times w [N, K] transposed?  (bfloat16, M <= 16,
    K a multiple of 64, N / SMs rows of w and the rows of x within one block's shared memory.)"""
    M, K = x.shape
    N = w.shape[0]
    per_sm = -(-N // num_sms(x.device))
    if M > 16 or K % 64 or per_sm > 32 or (per_sm + 16) * K * 2 > 180 * 1024:
        return False                                  # cheap refusals first; the library has the last word
    return bool(_lib("gemm_small").lsb_gemm_small_supported(_p(x), _p(w), _i(M), _i(N), _i(K)))


def tensor_core_gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA needs 16-byte aligned bases and row strides: K a multiple of 8 for bfloat16."""
    return (x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gated_activation(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu", limit: float = 0.0) -> None:
    """out[t, i] = act(gate_up[t, 2i]) * gate_up[t, 2i + 1] (gate and up alternate); "capped_glu" with ``limit`` L:
    min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u, -L, L) + 1)."""
    if activation in UNFUSED_GATED and not limit > 0:
        raise KernelError(f"gated_activation: '{activation}' needs a positive limit")
    _req(gate_up, "gate_up", dim=2)
    _req(out, "out", gate_up.dtype, 2)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError(f"gated_activation: gate_up is {tuple(gate_up.shape)}, out is {tuple(out.shape)}")
    _call("activation", "lsb_gated_act", _p(gate_up), _p(out), _i(_dt(out)), _i(T), _i(I),
          _i(_activation_id(activation)), _f(limit), _stream(out))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, 2i]) * gate_up[t, 2i + 1]."""
    gated_activation(gate_up, out, "silu")


def _check_cache(cache, nkv: int, hd: int, dtype) -> None:
    for name in ("k_pages", "v_pages"):
        t = _req(getattr(cache, name), name, dtype, 4)
        if t.shape[1:] != (nkv, cache.page_size, hd):
            raise KernelError(f"{name} is {tuple(t.shape)}, expected [pages, {nkv}, "
                              f"{cache.page_size}, {hd}]")
    _req(cache.block_table, "block_table", torch.int32, 2)


def rope_kv_store(qkv: torch.Tensor, nh: int, nkv: int, hd: int, ctx, cache,
                  inv_freq: Optional[torch.Tensor], rotary_dim: int, store: bool = True,
                  skip_single: bool = False) -> None:
    """Rotate queries and keys of the fused projection in place and write keys and values
    of this step's tokens into their cache pages.  ``skip_single`` leaves the tokens of requests
    that bring one token alone (their attention kernel does the same work itself)."""
    _req(qkv, "qkv", dim=2)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise KernelError(f"qkv is {tuple(qkv.shape)}, expected [T, {(nh + 2 * nkv) * hd}]")
    if hd % 2 or rotary_dim % 2 or rotary_dim > hd:
        raise KernelError(f"rope: head_dim {hd} and rotary_dim {rotary_dim} must be even, "
                          f"rotary_dim <= head_dim")
    if rotary_dim:
        _req(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2:
            raise KernelError("inv_freq must have rotary_dim / 2 entries")
    _check_cache(cache, nkv, hd, qkv.dtype)
    if ctx.n_tokens != T:
        raise KernelError(f"qkv has {T} rows, the step has {ctx.n_tokens} tokens")
    _call("rope_cache", "lsb_rope_kv_store", _p(qkv), _i(_dt(qkv)), _i(T), _i(nh), _i(nkv), _i(hd),
          _p(ctx.positions), _p(ctx.token_req), _p(ctx.table_rows), _p(cache.block_table),
          _i(cache.block_table.shape[1]), _p(inv_freq if rotary_dim else None), _i(rotary_dim),
          _p(cache.k_pages), _p(cache.v_pages), _i(cache.page_size), _i(cache.k_pages.shape[0]),
          _i(1 if store else 0), _p(ctx.q_start if skip_single else None), _stream(qkv))


_sm_counts: Dict[int, int] = {}


def num_sms(device=None) -> int:
    """Streaming multiprocessors of ``device`` (the current one by default), asked once."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


USE_TCGEN05_ATTENTION = True    # prompt portions of 128 tokens and more
FUSE_DECODE_ROPE = True         # single tokens: rotation and cache write inside the decode kernel
_TC_HEAD_DIMS = (64, 128)


_decode_occupancy: Dict[tuple, int] = {}


def decode_splits(n_decode: int, nkv: int, device=None, hd: int = 64, group: int = 4) -> int:
    """How many ways each request's keys are split among thread blocks in the decode kernel: as many
    as fill four fifths of the blocks the SMs hold at once (four an SM at head size 64, two at 128,
    where a block has twice the registers and shared memory), never a second round of blocks.
    Measured inside decode steps at context 4096: head size 64, 8 requests: 7 splits (6: 1 % slower,
    9: 10 %); 32 requests: 2 (1: 14 % slower, 3: 10 %); head size 128, 8 requests: 4 or 5 splits 27 -
    28 us a layer, 7 splits (a second round for four blocks) 42 us; 32 requests: 1 split 84 us, 2
    splits 108 us.  A function of the batch alone, so that a captured launch stays valid as
    sequences grow."""
    key = (hd, group)
    if key not in _decode_occupancy:
        fits = 4
        if hd in _TC_HEAD_DIMS:
            fits = int(_lib("attention_tc").lsb_decode_blocks_per_sm(_i(hd), _i(group)))
        _decode_occupancy[key] = max(1, fits)
    room = _decode_occupancy[key] * num_sms(device)
    return max(1, min(32, int(0.8 * room / max(1, n_decode * nkv) + 0.5)))


_cluster_caps: Dict[int, int] = {}


def _decode_cluster_cap(hd: int) -> int:
    """The largest thread-block cluster the decode kernel can be launched with here (8 or 16)."""
    if hd not in _cluster_caps:
        _cluster_caps[hd] = int(_lib("attention_tc").lsb_decode_max_cluster(_i(hd)))
    return _cluster_caps[hd]


def tensor_core_attention_ok(dtype, hd: int, nh: int, nkv: int) -> bool:
    return dtype == torch.bfloat16 and hd in _TC_HEAD_DIMS and nh // nkv <= 16


OVERLAP_ATTENTION = True        # decode kernel beside the prompt kernels in steps that hold both
_side: Dict[torch.device, tuple] = {}


def _fork_join(ctx, device):
    """(the step's stream, a second stream, two events), looked up once per step."""
    got = getattr(ctx, "_fork_join", None)
    if got is None:
        if device not in _side:
            _side[device] = (torch.cuda.Stream(device), torch.cuda.Event(), torch.cuda.Event())
        got = ctx._fork_join = (torch.cuda.current_stream(device),) + _side[device]
    return got


def _batch_shape(ctx):
    """(single-token requests, first and one past the last request with more tokens) of a step;
    worked out once per step and kept on the context."""
    shape = getattr(ctx, "_batch_shape", None)
    if shape is None:
        many = ctx.h_q_len != 1
        idx = many.nonzero()[0]
        shape = (int(len(many) - len(idx)),) + ((int(idx[0]), int(idx[-1]) + 1) if len(idx) else (0, 0))
        ctx._batch_shape = shape
    return shape


def rope_store_attention(qkv: torch.Tensor, nh: int, nkv: int, hd: int, ctx, cache,
                         inv_freq: Optional[torch.Tensor], rotary_dim: int, store: bool,
                         scale: float, window: int, out: torch.Tensor, softcap: float = 0.0,
                         slopes: Optional[torch.Tensor] = None) -> None:
    """``rope_kv_store`` followed by ``paged_attention``, as one operation.  Where the decode
    kernel can do the rotation and the cache write of single tokens itself (tensor-core path,
    the rotated part of the head a multiple of 16 wide, no score modifier), the separate kernel
    runs only for the tokens of prompt portions, or not at all."""
    if softcap or slopes is not None:
        rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store)
        paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out, softcap=softcap, slopes=slopes)
        return
    fuse = (FUSE_DECODE_ROPE and 0 < rotary_dim <= hd and rotary_dim % 16 == 0 and inv_freq is not None
            and tensor_core_attention_ok(qkv.dtype, hd, nh, nkv))
    n_decode = _batch_shape(ctx)[0] if fuse else 0
    if not n_decode:
        rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store)
        paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out)
        return
    if n_decode < ctx.n_requests:
        if OVERLAP_ATTENTION and not getattr(ctx, "fixed_launch", False):
            # Single tokens and prompt portions are different requests with different pages: the
            # decode kernel (memory-bound) runs on a second stream beside the rotation and the
            # attention of the portions (compute-bound), and the step's stream waits for both.
            main, side, fork, join = _fork_join(ctx, qkv.device)
            _stream_op(lambda: fork.record(main))             # qkv is whole here
            _stream_op(lambda: side.wait_event(fork))
            paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out,
                            decode_rope=(inv_freq, store, rotary_dim), only="single", stream=side.cuda_stream)
            _stream_op(lambda: join.record(side))
            rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store, skip_single=True)
            paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out, only="portions")
            _stream_op(lambda: main.wait_event(join))
            return
        rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store, skip_single=True)
    else:
        _req(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2 or qkv.shape[1] != (nh + 2 * nkv) * hd:
            raise KernelError("rope: inv_freq or qkv do not fit the head size")
    paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out,
                    decode_rope=(inv_freq, store, rotary_dim))


def paged_attention(qkv: torch.Tensor, nh: int, nkv: int, hd: int, ctx, cache, scale: float,
                    window: int, out: torch.Tensor, decode_rope=None, only: Optional[str] = None,
                    stream: Optional[int] = None, softcap: float = 0.0,
                    slopes: Optional[torch.Tensor] = None) -> None:
    """Causal attention of this step's query rows over their requests' cached keys and values.

    Score modifiers: ``softcap`` > 0 replaces a scaled score s by ``softcap * tanh(s / softcap)``;
    ``slopes`` (float32 [heads]) subtracts ``slopes[h] * (query position - key position)``.  A
    call with either runs the generic kernel, whatever the dtype and head size.

    bfloat16 with head size 64 or 128 runs on the tensor cores: single decode tokens in the
    split-KV kernel, prompt portions in the tiled kernel.  Everything else (32-bit, other head
    sizes) runs the generic kernel.  ``decode_rope = (inv_freq, store, rotary_dim)`` says that
    single tokens come unrotated and not yet in the cache (see ``rope_store_attention``).  ``only``: "single"
    or "portions" launches just that kernel; ``stream``: a raw stream to launch on instead of the
    current one."""
    _req(qkv, "qkv", dim=2)
    _req(out, "out", qkv.dtype, 2)
    T = qkv.shape[0]
    if qkv.shape[1] < nh * hd or out.shape != (T, nh * hd):
        raise KernelError(f"attention: qkv {tuple(qkv.shape)} / out {tuple(out.shape)} do not fit "
                          f"{nh} heads of {hd}")
    if hd % 16 or not 16 <= hd <= 256:
        raise KernelError(f"attention: head_dim must be a multiple of 16 in [16, 256], got {hd}")
    if nkv <= 0 or nh % nkv:
        raise KernelError(f"attention: {nh} heads cannot share {nkv} kv heads")
    if ctx.n_requests > 65535 or nh > 65535:
        raise KernelError("attention: at most 65535 requests and heads per step")
    _check_cache(cache, nkv, hd, qkv.dtype)
    common = (_p(qkv), _i(qkv.shape[1]), _p(cache.k_pages), _p(cache.v_pages), _p(ctx.q_start),
              _p(ctx.kv_len), _p(ctx.table_rows), _p(cache.block_table),
              _i(cache.block_table.shape[1]), _p(out))
    tail = (_i(nh), _i(nkv), _i(hd), _i(cache.page_size), _i(cache.k_pages.shape[0]), _f(scale),
            _i(window))
    modified = bool(softcap) or slopes is not None
    if slopes is not None:
        _req(slopes, "slopes", torch.float32, 1)
        if slopes.shape[0] != nh:
            raise KernelError(f"attention: {slopes.shape[0]} slopes for {nh} heads")
    if softcap < 0:
        raise KernelError("attention: the soft cap must be positive (0: none)")
    if modified or not tensor_core_attention_ok(qkv.dtype, hd, nh, nkv):
        if decode_rope is not None:
            raise KernelError("attention: only the tensor-core decode kernel rotates by itself")
        _call("attention", "lsb_paged_attention_generic", *common, _i(_dt(qkv)),
              _i(ctx.n_requests), _i(ctx.max_q_len), *tail, _f(softcap), _p(slopes), _stream(out))
        return
    R = ctx.n_requests
    n_decode, first, last = _batch_shape(ctx)
    on = _stream(out) if stream is None else ctypes.c_void_p(stream)
    if n_decode and only != "portions":
        splits = decode_splits(n_decode, nkv, qkv.device, hd, nh // nkv)
        if not getattr(ctx, "fixed_launch", False):
            splits = min(splits, -(-ctx.max_kv_len // 128))
        cluster_cap = _decode_cluster_cap(hd)
        if cluster_cap >= 16 and splits > 8 and n_decode * nkv <= 16:
            splits = 16                 # a few requests: one 16-block cluster each, no merge kernel
                                        # (with more clusters than that the merge kernel was faster)
        elif splits > 12:
            splits = 12                 # finer splits than this only lengthen the merge
        scratch = None
        if splits > cluster_cap:        # splits of a cluster merge through distributed shared memory
            key = (qkv.device, R, nh, hd, splits)
            scratch = _scratch.get(key)
            if scratch is None:
                scratch = torch.empty(R * nh * splits * (hd + 2), dtype=torch.float32,
                                      device=qkv.device)
                _scratch[key] = scratch
        if decode_rope is None:
            _call("attention_tc", "lsb_decode_attention", *common, _p(scratch), _i(R), *tail,
                  _i(splits), on)
        else:
            _call("attention_tc", "lsb_decode_attention_rope", *common, _p(scratch), _i(R), *tail,
                  _i(splits), _p(decode_rope[0]), _i(decode_rope[2]), _i(1 if decode_rope[1] else 0), on)
    if n_decode < R and only != "single":
        # prompt portions: tcgen05 kernel for long ones (128-row tiles), mma.sync kernel otherwise
        # The grid has a slab of blocks per request, and blocks that find a single token leave at
        # once, but thousands of them still cost tens of microseconds: the kernels get only the
        # requests from the first to the last prompt portion (the scheduler puts single tokens
        # first), by way of offset pointers into the per-request arrays.
        off = 4 * first
        per_request = (ctypes.c_void_p(ctx.q_start.data_ptr() + off),
                       ctypes.c_void_p(ctx.kv_len.data_ptr() + off),
                       ctypes.c_void_p(ctx.table_rows.data_ptr() + off))
        skip = _i(1 if n_decode > first + (R - last) else 0)      # single tokens among them
        if (USE_TCGEN05_ATTENTION and ctx.max_q_len >= 128
                and cache.page_size in (8, 16, 32, 64) and qkv.shape[1] % 8 == 0):
            _call("attention_tc5", "lsb_prefill_attention_tc5", _p(qkv), _i(qkv.shape[1]), _i(T),
                  _p(cache.k_pages), _p(cache.v_pages), *per_request, _p(cache.block_table),
                  _i(cache.block_table.shape[1]), _p(out), _i(last - first), _i(ctx.max_q_len), *tail,
                  skip, _i(0), _p(None), _ll(0), on)
        else:
            _call("attention_tc", "lsb_prefill_attention", _p(qkv), _i(qkv.shape[1]), _p(cache.k_pages),
                  _p(cache.v_pages), *per_request, _p(cache.block_table), _i(cache.block_table.shape[1]),
                  _p(out), _i(last - first), _i(ctx.max_q_len), *tail, skip, on)


# ----------------------------------------------- rows of a stream that is normed after the sum
def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (32-bit) rounded to out's dtype."""
    _req(x, "x", torch.float32)
    _req(out, "out")
    if out.shape != x.shape:
        raise KernelError("cast_rows: shapes differ")
    _call("rownorm", "lsb_cast_rows", _p(x), _p(out), _i(_dt(out)), _ll(x.numel()), _stream(out))


def post_group_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                    groups: int, alpha: float, out: Optional[torch.Tensor], gate: Optional[torch.Tensor] = None,
                    gate_bias: Optional[torch.Tensor] = None, keep_sum: bool = False, dtype=None) -> None:
    """s = alpha * residual + delta * sigmoid(gate + gate_bias); y = the RMS norm of s in ``groups``
    consecutive parts, times weight.  residual <- y (or s with ``keep_sum``), in place, 32-bit;
    out <- y in the compute dtype (``out`` may be None).  ``gate`` may be a column slice of a wider
    tensor (its row stride is passed on)."""
    _req(residual, "residual", torch.float32, 2)
    _req(weight, "weight", torch.float32, 1)
    T, H = residual.shape
    dt = out.dtype if out is not None else (delta.dtype if delta is not None else (dtype or torch.float32))
    if out is not None:
        _req(out, "out", dim=2)
        if out.shape != (T, H):
            raise KernelError("post_group_norm: out has another shape than residual")
    if weight.shape[0] != H or groups <= 0 or H % groups:
        raise KernelError(f"post_group_norm: weight {tuple(weight.shape)} / groups {groups} do not fit width {H}")
    gate_stride = 0
    if delta is not None:
        _req(delta, "delta", dt, 2)
        if delta.shape != (T, H):
            raise KernelError("post_group_norm: delta has another shape than residual")
    if gate is not None:
        _req(gate, "gate", dt, 2, contiguous=False)
        if delta is None or gate.shape != (T, H) or gate.stride(1) != 1:
            raise KernelError("post_group_norm: the gate needs a delta and its shape, with unit column stride")
        gate_stride = gate.stride(0)
        if gate_bias is not None:
            _req(gate_bias, "gate_bias", torch.float32, 1)
    _call("rownorm", "lsb_post_group_norm", _p(residual), _p(delta), _p(gate), _ll(gate_stride), _p(gate_bias),
          _p(weight), _p(out), _i(_F32 if dt == torch.float32 else _BF16), _i(T), _i(H), _i(groups), _f(alpha),
          _f(eps), _i(1 if keep_sum else 0), _stream(residual))


def gather_group_norm(residual: torch.Tensor, rows: torch.Tensor, weight: torch.Tensor, eps: float,
                      groups: int, out: torch.Tensor) -> None:
    """out[i] = group RMS norm of residual[rows[i]], times weight; residual unchanged."""
    _req(residual, "residual", torch.float32, 2)
    _req(rows, "rows", torch.int32, 1)
    _req(weight, "weight", torch.float32, 1)
    _req(out, "out", dim=2)
    T, H = residual.shape
    if out.shape != (rows.shape[0], H) or weight.shape[0] != H or groups <= 0 or H % groups:
        raise KernelError("gather_group_norm: shapes disagree")
    _call("rownorm", "lsb_gather_group_norm", _p(residual), _p(rows), _i(rows.shape[0]), _i(T), _p(weight),
          _p(out), _i(_dt(out)), _i(H), _i(groups), _f(eps), _stream(out))


def unit_add(residual: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
             out: Optional[torch.Tensor]) -> None:
    """residual += y / sqrt(mean(y^2) + eps) * weight (in place, 32-bit); out <- residual rounded."""
    _req(residual, "residual", torch.float32, 2)
    _req(y, "y", dim=2)
    _req(weight, "weight", torch.float32, 1)
    if y.shape != residual.shape or weight.shape[0] != residual.shape[1]:
        raise KernelError("unit_add: shapes disagree")
    if out is not None:
        _req(out, "out", y.dtype, 2)
        if out.shape != residual.shape:
            raise KernelError("unit_add: out has another shape than residual")
    _call("rownorm", "lsb_unit_add", _p(residual), _p(y), _p(weight), _p(out), _i(_dt(y)),
          _i(residual.shape[0]), _i(residual.shape[1]), _f(eps), _stream(residual))


def rows_norm_gate(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float,
                   gate: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = RMS norm of each of the ``groups`` parts of a 32-bit row, times ``weight`` (its index taken
    modulo its length: one weight per part, or one over the row), times sigmoid(gate) if given."""
    _req(x, "x", torch.float32, 2)
    _req(weight, "weight", torch.float32, 1)
    _req(out, "out", dim=2)
    T, n = x.shape
    if out.shape != (T, n) or groups <= 0 or n % groups or n % weight.shape[0]:
        raise KernelError("rows_norm_gate: shapes disagree")
    gate_stride = 0
    if gate is not None:
        _req(gate, "gate", out.dtype, 2, contiguous=False)
        if gate.shape != (T, n) or gate.stride(1) != 1:
            raise KernelError("rows_norm_gate: the gate must have x's shape and unit column stride")
        gate_stride = gate.stride(0)
    _call("rownorm", "lsb_rows_norm_gate", _p(x), _p(weight), _i(weight.shape[0]), _p(gate), _ll(gate_stride),
          _p(out), _i(_dt(out)), _i(T), _i(n), _i(groups), _f(eps), _stream(out))


def token_side_gate(g: torch.Tensor, table: torch.Tensor, token_ids: torch.Tensor, offset: int,
                    activation: str, out: torch.Tensor) -> None:
    """out[t, j] = act(g[t, j]) * table[token_ids[t], offset + j]."""
    _req(g, "g", dim=2)
    _req(table, "table", g.dtype, 2)
    _req(token_ids, "token_ids", torch.int32, 1)
    _req(out, "out", g.dtype, 2)
    T, dim = g.shape
    if out.shape != (T, dim) or token_ids.shape[0] != T or offset < 0 or offset + dim > table.shape[1]:
        raise KernelError("token_side_gate: shapes disagree")
    _call("rownorm", "lsb_token_side_gate", _p(g), _p(table), _p(token_ids), _p(out), _i(_dt(g)), _i(T), _i(dim),
          _i(table.shape[1]), _i(offset), _i(table.shape[0]), _i(ACTIVATIONS.get(activation, 0) if activation != "none" else 0),
          _stream(out))


# ------------------------------------------------------------------ linear recurrence
SCAN_GATES = {"fixed_decay": 0, "forget": 1, "given": 2}
_SCAN_ACTS = {"none": 0, "silu": 1}
SCAN_SEGMENT = 128              # tokens of a segment when long portions are walked in segments (0: never)


def linear_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, key_dim: int,
                value_dim: int, gate: str, decay: Optional[torch.Tensor], f_bias: Optional[torch.Tensor],
                floor: Optional[torch.Tensor], q_act: str, k_act: str, v_act: str, state: torch.Tensor,
                ctx, out: torch.Tensor, keep: Optional[torch.Tensor] = None, write: Optional[torch.Tensor] = None,
                ones: bool = False, q_scale: float = 1.0) -> None:
    """S <- diag(a) S + b v^T, o = S^T q per head and token, each request from its slot's state
    (``state`` [slots, heads, value_dim, key_dim] 32-bit, updated in place); ``proj`` [T, columns] holds
    the projections of q at ``q_off``, of k (or the forget gate) at ``k_off`` and of v at ``v_off``;
    ``out`` [T, heads * value_dim] 32-bit.

    Gate "given": ``keep`` and ``write`` (32-bit [T, heads]) are a and the factor of b for every channel
    of a head.  ``ones``: a value column of ones rides along behind each head's ``value_dim`` columns
    (state and out then have ``value_dim + 1`` columns a head, the last one of out being the
    running sum of b dotted with q).  ``q_scale`` multiplies q."""
    _req(proj, "proj", dim=2)
    _req(state, "state", torch.float32, 4)
    _req(out, "out", torch.float32, 2)
    T, ld = proj.shape
    cols = value_dim + (1 if ones else 0)
    if state.shape[1:] != (heads, cols, key_dim) or out.shape != (T, heads * cols) or ctx.n_tokens != T:
        raise KernelError("linear_scan: state, out or the step do not fit the sizes")
    if max(q_off, k_off) + heads * key_dim > ld or v_off + heads * value_dim > ld or min(q_off, k_off, v_off) < 0:
        raise KernelError("linear_scan: a projection lies outside the rows of proj")
    if gate == "given" and (keep is None or write is None):
        raise KernelError("linear_scan: given gates need keep and write")
    for name, t in (("keep", keep), ("write", write)):
        if t is not None:
            _req(t, name, torch.float32, 2)
            if t.shape != (T, heads):
                raise KernelError(f"linear_scan: {name} must be [tokens, heads]")
    for name, t, n in (("decay", decay, heads), ("f_bias", f_bias, heads * key_dim), ("floor", floor, heads * key_dim)):
        if t is not None:
            _req(t, name, torch.float32, 1)
            if t.shape[0] != n:
                raise KernelError(f"linear_scan: {name} must have {n} entries")
    if not _lib("linear_scan").lsb_linear_scan_supported(_i(key_dim)):
        raise KernelError(f"linear_scan: key_dim {key_dim} is not supported")
    # a few requests with long portions: segments walked side by side (twice the arithmetic, a chain
    # a segment long); many requests, short portions and single tokens: one walk each
    seg, seg_state, seg_decay = 0, None, None
    if SCAN_SEGMENT and ctx.max_q_len >= 2 * SCAN_SEGMENT and ctx.n_requests <= 8:
        seg = SCAN_SEGMENT
        n = ctx.n_requests * -(-ctx.max_q_len // seg)
        seg_state = torch.empty(n * heads * cols * key_dim, dtype=torch.float32, device=proj.device)
        seg_decay = torch.empty(n * heads * key_dim, dtype=torch.float32, device=proj.device)
    _call("linear_scan", "lsb_linear_scan", _p(proj), _i(_dt(proj)), _ll(ld), _i(q_off), _i(k_off), _i(v_off),
          _i(heads), _i(key_dim), _i(value_dim), _i(SCAN_GATES[gate]), _p(decay), _p(f_bias), _p(floor),
          _i(_SCAN_ACTS[q_act]), _i(_SCAN_ACTS[k_act]), _i(_SCAN_ACTS[v_act]), _p(state), _i(state.shape[0]),
          _p(ctx.q_start), _p(ctx.table_rows), _i(ctx.n_requests), _p(out), _i(seg), _i(ctx.max_q_len),
          _p(seg_state), _p(seg_decay), _p(keep), _p(write), _i(1 if ones else 0), _f(q_scale), _stream(out))


# --------------------------------------------------------------------- latent attention
_PAIRINGS = {"half": 0, "adjacent": 1}
LATENT_TENSOR_CORES = True      # bfloat16 latent attention on warp-level MMA (csrc/latent_tc.cu)


def _check_latent_cache(cache, width: int, dtype) -> None:
    t = _req(cache.pages, "pages", dtype, 3)
    if t.shape[1:] != (cache.page_size, width):
        raise KernelError(f"latent pages are {tuple(t.shape)}, expected [pages, {cache.page_size}, {width}]")
    _req(cache.block_table, "block_table", torch.int32, 2)


def latent_prep(down: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, q_weight: torch.Tensor,
                kv_weight: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rot_dims: int,
                pairing: str, ctx, cache, cq: torch.Tensor, write: bool) -> None:
    """Per token: cq = rmsnorm(down[:q_rank]) * q_weight; with ``write`` also the token's cache row:
    rmsnorm(down[q_rank:q_rank + kv_rank]) * kv_weight, then the next rot_dim values rotated by the
    token's position."""
    _req(down, "down", torch.float32, 2)
    _req(q_weight, "q_weight", torch.float32, 1)
    _req(cq, "cq", dim=2)
    T, ld = down.shape
    if cq.shape != (T, q_rank) or q_weight.shape[0] != q_rank or ctx.n_tokens != T:
        raise KernelError("latent_prep: cq, the weight or the step do not fit")
    if write:
        _req(kv_weight, "kv_weight", torch.float32, 1)
        if ld < q_rank + kv_rank + rot_dim or kv_weight.shape[0] != kv_rank:
            raise KernelError("latent_prep: down must hold q_rank + kv_rank + rot_dim columns (more may follow)")
        if rot_dims:
            _req(inv_freq, "inv_freq", torch.float32, 1)
            if inv_freq.shape[0] != rot_dims // 2:
                raise KernelError("latent_prep: inv_freq must have rot_dims / 2 entries")
        _check_latent_cache(cache, kv_rank + rot_dim, cq.dtype)
    elif ld < q_rank:
        raise KernelError("latent_prep: down is narrower than q_rank")
    _call("latent", "lsb_latent_prep", _p(down), _ll(ld), _i(T), _i(q_rank), _i(kv_rank), _i(rot_dim),
          _p(q_weight), _p(kv_weight if write else None), _f(eps), _p(inv_freq if write else None), _i(rot_dims),
          _i(_PAIRINGS[pairing]), _p(ctx.positions), _p(ctx.token_req), _p(ctx.table_rows),
          _p(cache.block_table), _i(cache.block_table.shape[1]), _p(cache.pages), _i(_dt(cq)),
          _i(cache.page_size), _i(cache.pages.shape[0]), _p(cq), _i(1 if write else 0), _stream(cq))


def latent_query_rot(q: torch.Tensor, qf: torch.Tensor, heads: int, plain: int, rot_dim: int, kv_rank: int,
                     inv_freq: Optional[torch.Tensor], rot_dims: int, pairing: str, ctx) -> None:
    """qf[t, h, kv_rank:] = the last rot_dim values of head h of q[t], rotated by the token's position."""
    _req(q, "q", torch.float32, 2)
    _req(qf, "qf", torch.float32, 3)
    T = q.shape[0]
    if q.shape[1] != heads * (plain + rot_dim) or qf.shape != (T, heads, kv_rank + rot_dim):
        raise KernelError("latent_query_rot: q or qf do not fit the sizes")
    if rot_dims:
        _req(inv_freq, "inv_freq", torch.float32, 1)
    _call("latent", "lsb_latent_query_rot", _p(q), _p(qf), _i(T), _i(heads), _i(plain), _i(rot_dim), _i(kv_rank),
          _i(rot_dims), _i(_PAIRINGS[pairing]), _p(inv_freq), _p(ctx.positions), _stream(qf))


def batched_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, exact: bool = False) -> None:
    """out[m, h, :] = a[m, h, :] @ b[h].T for every h: ``a`` [M, H, K] and ``out`` [M, H, N] may be
    views with any row and head strides (unit stride along the last axis), ``b`` [H, N, K] is dense.
    32-bit accumulation.  ``exact``: 32-bit operands of ``a`` are not rounded on their way into the product
    (the CUDA cores' multiply-add), whatever the dtype of ``b``."""
    for name, t in (("a", a), ("out", out)):
        _req(t, name, dim=3, contiguous=False)
        if t.stride(2) != 1:
            raise KernelError(f"batched_nt: {name} needs unit stride along its last axis")
    _req(b, "b", dim=3)
    M, H, K = a.shape
    N = b.shape[1]
    if b.shape != (H, N, K) or out.shape != (M, H, N):
        raise KernelError(f"batched_nt: a {tuple(a.shape)}, b {tuple(b.shape)}, out {tuple(out.shape)} do not fit")
    if LATENT_TENSOR_CORES and b.dtype == torch.bfloat16 and not exact:
        _call("latent_tc", "lsb_batched_nt_tc", _p(a), _i(_dt(a)), _ll(a.stride(0)), _ll(a.stride(1)), _p(b), _p(out),
              _i(_dt(out)), _ll(out.stride(0)), _ll(out.stride(1)), _i(M), _i(N), _i(K), _i(H), _stream(out))
        return
    _call("latent", "lsb_batched_nt", _p(a), _i(_dt(a)), _ll(a.stride(0)), _ll(a.stride(1)), _p(b), _i(_dt(b)),
          _p(out), _i(_dt(out)), _ll(out.stride(0)), _ll(out.stride(1)), _i(M), _i(N), _i(K), _i(H), _stream(out))


def head_gate(x: torch.Tensor, gate: torch.Tensor) -> None:
    """x[t, h, :] *= sigmoid(gate[t, h]) in place; ``gate`` 32-bit [T, heads], rows may be strided."""
    _req(x, "x", dim=3)
    _req(gate, "gate", torch.float32, 2, contiguous=False)
    T, H, D = x.shape
    if gate.shape != (T, H) or gate.stride(1) != 1:
        raise KernelError("head_gate: the gate must be [tokens, heads] with unit column stride")
    _call("latent", "lsb_head_gate", _p(x), _i(_dt(x)), _p(gate), _ll(gate.stride(0)), _i(T), _i(H), _i(D), _stream(x))


# ------------------------------------------------------- gated linear recurrent unit (real gates)
def rglru_conv(proj: torch.Tensor, x_off: int, x_bias: Optional[torch.Tensor], taps_w: torch.Tensor,
               conv_bias: Optional[torch.Tensor], conv_state: torch.Tensor, ctx, u: torch.Tensor,
               split: Optional[torch.Tensor] = None, blocks: int = 1) -> None:
    """u[t, c] = conv_bias[c] + sum_k taps_w[c, k] * xin[t - (taps - 1 - k), c] with xin = proj[:, x_off + c] +
    x_bias[c]; before a portion's first token xin is the request slot's ``conv_state`` [slots, taps - 1, width]
    (zeros before a sequence's start).  All 32-bit.  ``split`` (bfloat16 [T, 2 * width]): u once more as the sum
    of two bfloat16 numbers, per block of ``width / blocks`` channels the rounded values and then the rounded
    rests."""
    _req(proj, "proj", torch.float32, 2)
    if split is not None:
        _req(split, "split", torch.bfloat16, 2)
        if split.shape != (u.shape[0], 2 * u.shape[1]) or blocks <= 0 or u.shape[1] % blocks:
            raise KernelError("rglru_conv: split must be [tokens, 2 * width], the blocks dividing the width")
    _req(taps_w, "taps_w", torch.float32, 2)
    _req(conv_state, "conv_state", torch.float32, 3)
    _req(u, "u", torch.float32, 2)
    T, width = u.shape
    taps = taps_w.shape[1]
    if ctx.n_tokens != T or proj.shape[0] != T or x_off < 0 or x_off + width > proj.shape[1] or taps_w.shape[0] != width \
            or conv_state.shape[1] < taps - 1 or conv_state.shape[2] != width:
        raise KernelError("rglru_conv: proj, the taps, the state and u disagree")
    if taps > 1 and conv_state.shape[1] != taps - 1:
        raise KernelError("rglru_conv: the state must hold taps - 1 inputs")
    for name, t in (("x_bias", x_bias), ("conv_bias", conv_bias)):
        if t is not None:
            _req(t, name, torch.float32, 1)
            if t.shape[0] != width:
                raise KernelError(f"rglru_conv: {name} must have {width} entries")
    _call("rglru", "lsb_rglru_conv", _p(proj), _ll(proj.stride(0)), _i(x_off), _p(x_bias), _p(taps_w), _p(conv_bias),
          _i(taps), _p(conv_state), _p(ctx.token_req), _p(ctx.q_start), _p(ctx.table_rows), _i(conv_state.shape[0]),
          _p(u), _i(width), _i(T), _p(split), _i(blocks), _stream(u))


def rglru_gates(gates: torch.Tensor, r_bias: Optional[torch.Tensor], i_bias: Optional[torch.Tensor],
                lam: torch.Tensor, rate: float, u: torch.Tensor, proj: torch.Tensor, y_off: int,
                y_bias: Optional[torch.Tensor], blocks: int) -> None:
    """In place, 32-bit: with channel c = b * bw + o, ``gates[t, b, o]`` (the decay gate's product) becomes
    a = exp(-rate * sigmoid(. + r_bias) * softplus(lam)), ``gates[t, b, bw + o]`` (the input gate's product) becomes
    sqrt(1 - a^2) * sigmoid(. + i_bias) * u, and ``proj[t, y_off + c]`` becomes gelu_tanh(. + y_bias)."""
    _req(gates, "gates", torch.float32, 2)
    _req(u, "u", torch.float32, 2)
    _req(proj, "proj", torch.float32, 2)
    _req(lam, "lam", torch.float32, 1)
    T, width = u.shape
    if gates.shape != (T, 2 * width) or proj.shape[0] != T or y_off < 0 or y_off + width > proj.shape[1] \
            or lam.shape[0] != width or blocks <= 0 or width % blocks:
        raise KernelError("rglru_gates: gates, u, proj and the decay's parameter disagree")
    for name, t in (("r_bias", r_bias), ("i_bias", i_bias), ("y_bias", y_bias)):
        if t is not None:
            _req(t, name, torch.float32, 1)
            if t.shape[0] != width:
                raise KernelError(f"rglru_gates: {name} must have {width} entries")
    _call("rglru", "lsb_rglru_gates", _p(gates), _p(r_bias), _p(i_bias), _p(lam), _f(rate), _p(u), _p(proj),
          _ll(proj.stride(0)), _i(y_off), _p(y_bias), _i(width), _i(blocks), _i(T), _stream(u))


RGLRU_SEGMENT = 64              # tokens of a segment when long portions of the recurrence are walked in segments (0: never)
RGLRU_SEGMENT_FROM = 256        # ... in steps whose longest portion has at least this many tokens


def rglru_walk(gates: torch.Tensor, proj: torch.Tensor, x_off: int, y_off: int, x_bias: Optional[torch.Tensor],
               taps: int, state: torch.Tensor, conv_state: torch.Tensor, ctx, out: torch.Tensor, blocks: int) -> None:
    """S <- a_t S + in_t token by token for every request and channel, from the slot's ``state`` [slots, width] and
    back into it; out[t] = S_t * proj[t, y_off:] in the compute dtype.  ``gates`` as ``rglru_gates`` left them.  The
    slot's ``conv_state`` is left holding the x branch's last ``taps - 1`` inputs."""
    _req(gates, "gates", torch.float32, 2)
    _req(proj, "proj", torch.float32, 2)
    _req(state, "state", torch.float32, 2)
    _req(conv_state, "conv_state", torch.float32, 3)
    _req(out, "out", dim=2)
    T, width = out.shape
    if gates.shape != (T, 2 * width) or proj.shape[0] != T or ctx.n_tokens != T or state.shape[1] != width \
            or conv_state.shape[0] != state.shape[0] or conv_state.shape[2] != width \
            or (taps > 1 and conv_state.shape[1] != taps - 1) or max(x_off, y_off) + width > proj.shape[1]:
        raise KernelError("rglru_walk: gates, proj, the states and out disagree")
    if RGLRU_SEGMENT and ctx.max_q_len >= RGLRU_SEGMENT_FROM \
            and ctx.n_requests * -(-ctx.max_q_len // RGLRU_SEGMENT) <= 65535:
        # a step with a long portion: every request's tokens in segments walked side by side, chained, and
        # walked again from their starts (the single tokens of other requests are segments of one token)
        segs = -(-ctx.max_q_len // RGLRU_SEGMENT)
        key = ("rglru", out.device, ctx.n_requests * segs * 2 * width)
        scratch = _scratch.get(key)
        if scratch is None:
            scratch = _scratch[key] = torch.empty(key[2], dtype=torch.float32, device=out.device)
        _call("rglru", "lsb_rglru_walk_segments", _p(gates), _p(proj), _ll(proj.stride(0)), _i(x_off), _i(y_off),
              _p(x_bias), _i(taps), _p(state), _p(conv_state), _p(ctx.q_start), _p(ctx.table_rows), _i(state.shape[0]),
              _p(out), _i(_dt(out)), _i(width), _i(blocks), _i(ctx.n_requests), _i(ctx.max_q_len), _i(RGLRU_SEGMENT),
              _p(scratch), _stream(out))
        return
    _call("rglru", "lsb_rglru_walk", _p(gates), _p(proj), _ll(proj.stride(0)), _i(x_off), _i(y_off), _p(x_bias),
          _i(taps), _p(state), _p(conv_state), _p(ctx.q_start), _p(ctx.table_rows), _i(state.shape[0]), _p(out),
          _i(_dt(out)), _i(width), _i(blocks), _i(ctx.n_requests), _stream(out))


def latent_attention(qf: torch.Tensor, ctx, cache, kv_rank: int, rot_dim: int, scale: float,
                     out: torch.Tensor) -> None:
    """Causal softmax attention of this step's rows over their requests' latent cache rows:
    scores (qf . row) * scale over the whole row, values the first kv_rank dims of the rows."""
    _req(qf, "qf", torch.float32, 3)
    _req(out, "out", dim=3)
    T, H, width = qf.shape
    if width != kv_rank + rot_dim or out.shape != (T, H, kv_rank) or ctx.n_tokens != T:
        raise KernelError("latent_attention: qf, out or the step do not fit the sizes")
    _check_latent_cache(cache, width, out.dtype)
    if LATENT_TENSOR_CORES and out.dtype == torch.bfloat16 and \
            _lib("latent_tc").lsb_latent_attention_tc_supported(_i(kv_rank), _i(rot_dim)):
        # 64 (token, head) rows a block; steps of single tokens split each request's keys over
        # blocks so that the SMs are busy (a function of the batch alone: a captured launch stays
        # valid as the sequences grow)
        splits, part_o, part_ml = 1, None, None
        if ctx.max_q_len == 1:
            splits = max(1, min(32, num_sms(qf.device) // (ctx.n_requests * -(-H // 64))))
        if splits > 1:
            part_o = torch.empty(T * H * splits * kv_rank, dtype=torch.float32, device=qf.device)
            part_ml = torch.empty(T * H * splits * 2, dtype=torch.float32, device=qf.device)
        _call("latent_tc", "lsb_latent_attention_tc", _p(qf), _p(cache.pages), _p(ctx.q_start), _p(ctx.kv_len),
              _p(ctx.table_rows), _p(cache.block_table), _i(cache.block_table.shape[1]), _p(out), _p(part_o),
              _p(part_ml), _i(ctx.n_requests), _i(ctx.max_q_len), _i(T), _i(H), _i(kv_rank), _i(rot_dim),
              _i(cache.page_size), _i(cache.pages.shape[0]), _f(scale), _i(splits), _stream(out))
        return
    _call("latent", "lsb_latent_attention", _p(qf), _p(cache.pages), _i(_dt(out)), _p(ctx.q_start), _p(ctx.kv_len),
          _p(ctx.table_rows), _p(cache.block_table), _i(cache.block_table.shape[1]), _p(out), _i(ctx.n_requests),
          _i(ctx.max_q_len), _i(H), _i(kv_rank), _i(rot_dim), _i(cache.page_size), _i(cache.pages.shape[0]),
          _f(scale), _stream(out))


# ------------------------------------------------- a stream whose sublayers are normed on both sides
def stream_norm(residual: torch.Tensor, y: Optional[torch.Tensor], post_weight: Optional[torch.Tensor],
                post_eps: float, mult: float, step: Optional[torch.Tensor], rows: Optional[torch.Tensor],
                next_weight: Optional[torch.Tensor], next_eps: float, out: Optional[torch.Tensor]) -> None:
    """residual += mult * unit(y) * post_weight (+ step, one vector for every row); out = unit(residual) *
    next_weight; unit(z) = z / sqrt(mean(z^2) + eps).  Every piece is optional (``post_weight`` None
    with ``y`` given: a plain sum of mult * y).  ``rows`` (int32): only those rows, into ``out``
    [len(rows), H], the stream untouched."""
    _req(residual, "residual", torch.float32, 2)
    T, H = residual.shape
    n = T if rows is None else rows.shape[0]
    if rows is not None:
        _req(rows, "rows", torch.int32, 1)
    dtype = None
    for name, t in (("y", y), ("out", out)):
        if t is not None:
            _req(t, name, dtype, 2)
            dtype = t.dtype
    if y is not None and y.shape != (T, H):
        raise KernelError("stream_norm: y has another shape than the stream")
    if out is not None and (out.shape != (n, H) or next_weight is None):
        raise KernelError("stream_norm: out must be [rows, H] and needs the weight of its norm")
    for name, t in (("post_weight", post_weight), ("step", step), ("next_weight", next_weight)):
        if t is not None:
            _req(t, name, torch.float32, 1)
            if t.shape[0] != H:
                raise KernelError(f"stream_norm: {name} must have {H} entries")
    if dtype is None:
        if step is None:
            return
        dtype = torch.float32
    _call("sandwich", "lsb_stream_norm", _p(residual), _p(y), _p(post_weight), _f(post_eps), _f(mult), _p(step),
          _p(rows), _i(n), _p(next_weight), _f(next_eps), _p(out), _i(_F32 if dtype == torch.float32 else _BF16),
          _i(T), _i(H), _stream(residual))


def stream_centred_norm(residual: torch.Tensor, y: Optional[torch.Tensor], post_weight: Optional[torch.Tensor],
                        post_bias: Optional[torch.Tensor], post_eps: float, mult: float, rows: Optional[torch.Tensor],
                        next_weight: Optional[torch.Tensor], next_bias: Optional[torch.Tensor], next_eps: float,
                        out: Optional[torch.Tensor]) -> None:
    """residual += mult * (cn(y) * post_weight + post_bias); out = cn(residual) * next_weight + next_bias, with
    cn(z) = (z - mean z) / sqrt(mean((z - mean z)^2) + eps).  Every piece is optional (``post_weight`` None with
    ``y`` given: a plain sum of mult * y).  ``rows`` (int32): only those rows, into ``out`` [len(rows), H], the
    stream untouched."""
    _req(residual, "residual", torch.float32, 2)
    T, H = residual.shape
    n = T if rows is None else rows.shape[0]
    if rows is not None:
        _req(rows, "rows", torch.int32, 1)
    dtype = None
    for name, t in (("y", y), ("out", out)):
        if t is not None:
            _req(t, name, dtype, 2)
            dtype = t.dtype
    if dtype is None:
        return
    if y is not None and y.shape != (T, H):
        raise KernelError("stream_centred_norm: y has another shape than the stream")
    if out is not None and (out.shape != (n, H) or next_weight is None or next_bias is None):
        raise KernelError("stream_centred_norm: out must be [rows, H] and needs the weight and bias of its norm")
    if (post_weight is None) != (post_bias is None):
        raise KernelError("stream_centred_norm: the norm behind the sublayer needs weight and bias")
    for name, t in (("post_weight", post_weight), ("post_bias", post_bias), ("next_weight", next_weight),
                    ("next_bias", next_bias)):
        if t is not None:
            _req(t, name, torch.float32, 1)
            if t.shape[0] != H:
                raise KernelError(f"stream_centred_norm: {name} must have {H} entries")
    _call("sandwich", "lsb_stream_centred_norm", _p(residual), _p(y), _p(post_weight), _p(post_bias), _f(post_eps),
          _f(mult), _p(rows), _i(n), _p(next_weight), _p(next_bias), _f(next_eps), _p(out),
          _i(_F32 if dtype == torch.float32 else _BF16), _i(T), _i(H), _stream(residual))


def branch_mean(ys, weights, eps: float, out: torch.Tensor) -> None:
    """out = mean over the branches b of unit(ys[b]) * weights[b], row by row."""
    _req(out, "out", dim=2)
    n = len(ys)
    if n == 0 or n != len(weights) or n > _lib("sandwich").lsb_branch_max():
        raise KernelError(f"branch_mean: {n} branches with {len(weights)} weights")
    for y, w in zip(ys, weights):
        _req(y, "branch", out.dtype, 2)
        _req(w, "branch weight", torch.float32, 1)
        if y.shape != out.shape or w.shape[0] != out.shape[1]:
            raise KernelError("branch_mean: a branch or its weight does not fit out")
    yp = (ctypes.c_void_p * n)(*[_p(y).value for y in ys])
    wp = (ctypes.c_void_p * n)(*[_p(w).value for w in weights])
    _call("sandwich", "lsb_branch_mean", yp, wp, _i(n), _f(eps), _p(out), _i(_dt(out)), _i(out.shape[0]),
          _i(out.shape[1]), _stream(out))


# ------------------------------------------ attention with key and value sizes of their own
def _check_kv_cache(cache, nkv: int, dk: int, dv: int, dtype) -> None:
    for name, d in (("k_pages", dk), ("v_pages", dv)):
        t = _req(getattr(cache, name), name, dtype, 4)
        if t.shape[1:] != (nkv, cache.page_size, d):
            raise KernelError(f"{name} is {tuple(t.shape)}, expected [pages, {nkv}, {cache.page_size}, {d}]")
    _req(cache.block_table, "block_table", torch.int32, 2)


def attention_prep(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, nh: int, nkv: int, dk: int, dv: int,
                   ctx, cache, q_out: torch.Tensor, *, q_bias=None, k_bias=None, v_bias=None, q_norm=None,
                   k_norm=None, norm_eps: float = 0.0, temp_coef: float = 0.0, temp_every: int = 0,
                   inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0, pairing: str = "half",
                   store: bool = True, norm_all: bool = False, v_unit: bool = False,
                   v_first: Optional[torch.Tensor] = None, v_lambda: Optional[torch.Tensor] = None) -> None:
    """From the rows of ``proj`` (q at ``q_off``, k at ``k_off``, v at ``v_off``) to queries in ``q_out``
    [T, nh * dk] and keys and values in this step's cache places: biases, a norm per head of q and k
    (one weight of head size each), the query temperature ``1 + coef * ln(floor((pos + 1) / every) + 1)``
    and the rotation of the first ``rotary_dim`` dims, each if given.  ``norm_all``: q and k are each
    normed over all their heads at once, with weights as long as the whole projection.  ``v_unit``: every
    value head is divided by its root mean square (eps ``norm_eps``, no weight) on its way into the cache.
    ``v_first`` [T, nkv * dv] (rows may be strided) with ``v_lambda`` (one 32-bit number on the device): the
    values are mixed with those another layer made of the same tokens, v <- (1 - lambda) v + lambda v_first,
    and cached so."""
    _req(proj, "proj", dim=2)
    _req(q_out, "q_out", proj.dtype, 2)
    T, ld = proj.shape
    if ctx.n_tokens != T or q_out.shape != (T, nh * dk):
        raise KernelError("attention_prep: proj, q_out and the step disagree")
    if min(q_off, k_off, v_off) < 0 or q_off + nh * dk > ld or k_off + nkv * dk > ld or v_off + nkv * dv > ld:
        raise KernelError("attention_prep: a projection lies outside the rows of proj")
    if dk > _lib("attention_prep").lsb_attention_prep_max_dim():
        raise KernelError(f"attention_prep: key size {dk} is not supported")
    for name, t, n in (("q_bias", q_bias, nh * dk), ("k_bias", k_bias, nkv * dk), ("v_bias", v_bias, nkv * dv),
                       ("q_norm", q_norm, nh * dk if norm_all else dk),
                       ("k_norm", k_norm, nkv * dk if norm_all else dk)):
        if t is not None:
            _req(t, name, torch.float32, 1)
            if t.shape[0] != n:
                raise KernelError(f"attention_prep: {name} must have {n} entries")
    if rotary_dim:
        _req(inv_freq, "inv_freq", torch.float32, 1)
        if rotary_dim % 2 or rotary_dim > dk or inv_freq.shape[0] != rotary_dim // 2:
            raise KernelError("attention_prep: rotary_dim must be even, at most the key size, with rotary_dim / 2 "
                              "frequencies")
    if norm_all and (q_norm is None) != (k_norm is None):
        raise KernelError("attention_prep: a norm over all heads needs both weights")
    v_first_ld = 0
    if v_first is not None:
        _req(v_first, "v_first", proj.dtype, 2, contiguous=False)
        _req(v_lambda, "v_lambda", torch.float32)
        if v_first.shape != (T, nkv * dv) or v_first.stride(1) != 1 or v_lambda.numel() != 1 or v_unit:
            raise KernelError("attention_prep: v_first must be [T, kv heads * value size] with one mixing number")
        v_first_ld = v_first.stride(0)
    _check_kv_cache(cache, nkv, dk, dv, proj.dtype)
    _call("attention_prep", "lsb_attention_prep", _p(proj), _i(_dt(proj)), _ll(ld), _i(q_off), _i(k_off), _i(v_off),
          _i(T), _i(nh), _i(nkv), _i(dk), _i(dv), _p(q_bias), _p(k_bias), _p(v_bias), _p(q_norm), _p(k_norm),
          _f(norm_eps), _i(1 if norm_all else 0), _i(1 if v_unit else 0), _f(temp_coef), _i(temp_every), _p(inv_freq if rotary_dim else None), _i(rotary_dim),
          _i(_PAIRINGS[pairing]), _p(ctx.positions), _p(ctx.token_req), _p(ctx.table_rows), _p(cache.block_table),
          _i(cache.block_table.shape[1]), _p(q_out), _p(cache.k_pages), _p(cache.v_pages), _i(cache.page_size),
          _i(cache.k_pages.shape[0]), _i(1 if store else 0), _p(v_first), _ll(v_first_ld), _p(v_lambda), _stream(proj))


DV_BLOCK_SHAPE = 0              # 0: by the grid's size; 1: 64-row blocks; 2, 3: 16-row blocks, two or four tiles in flight; 4: as 3, keys shared by three blocks
DV_TENSOR_CORES = True          # bfloat16 heads of multiples of 16 up to 128 on warp-level MMA (csrc/attention_dv.cu)


def attention_dv(q: torch.Tensor, nh: int, nkv: int, dk: int, dv: int, ctx, cache, scale: float, window: int,
                 chunk: int, gate: Optional[torch.Tensor], out: torch.Tensor, sink: bool = False,
                 gate_per_head: bool = False, softcap: float = 0.0, linear_bias: bool = False) -> None:
    """Softmax attention of this step's queries ``q`` [T, nh * dk] over their requests' cached keys (size
    dk) and values (size dv): a query at position p sees ``[lo, p]`` with lo the larger of
    ``p - window + 1`` (window > 0) and the start of p's chunk of ``chunk`` positions (chunk > 0).
    ``gate`` [T, nh * dv] (rows may be strided): out *= sigmoid(gate); with ``gate_per_head`` it is
    [T, nh], one number per head.  ``sink``: one is added to the softmax's denominator (a place with
    score 0 and no value).  ``softcap`` > 0: a scaled score s becomes softcap * tanh(s / softcap).
    ``linear_bias``: head h's score for the key at distance d loses 2^(-8 (h + 1) / nh) * d (after the cap).

    bfloat16 with both sizes multiples of 16 up to 128 runs on the tensor cores (prompt portions in
    tiles of 64 rows, a row being a position and a head of a kv head's group; single tokens with the
    keys of a tile dealt to four warps); everything else runs the generic kernel."""
    _req(q, "q", dim=2)
    _req(out, "out", q.dtype, 2)
    T = q.shape[0]
    if q.shape[1] != nh * dk or out.shape != (T, nh * dv) or ctx.n_tokens != T:
        raise KernelError("attention_dv: q, out and the step disagree")
    if nkv <= 0 or nh % nkv:
        raise KernelError(f"attention_dv: {nh} heads cannot share {nkv} kv heads")
    if max(dk, dv) > _lib("attention_dv").lsb_attention_dv_max_dim():
        raise KernelError(f"attention_dv: head sizes {dk}, {dv} are not supported")
    gate_stride = 0
    if gate is not None:
        _req(gate, "gate", q.dtype, 2, contiguous=False)
        if gate.shape != (T, nh if gate_per_head else nh * dv) or gate.stride(1) != 1:
            raise KernelError("attention_dv: the gate must be [T, heads * value size] (or [T, heads]) with unit column stride")
        gate_stride = gate.stride(0)
    flags = (1 if sink else 0) | (2 if gate is not None and gate_per_head else 0) | (4 if linear_bias else 0)
    softcap = float(softcap or 0.0)
    if softcap < 0:
        raise KernelError("attention_dv: the cap must be positive (0: none)")
    _check_kv_cache(cache, nkv, dk, dv, q.dtype)
    # equal key and value sizes, no chunks, no gate or one number a head: the prompt portions of a step go
    # to the tcgen05 prompt kernel, which takes the sink and that gate in its last step; single tokens,
    # where they all come before the portions (as the scheduler puts them), go on below
    n_req, max_q = ctx.n_requests, ctx.max_q_len
    if (USE_TCGEN05_ATTENTION and DV_TENSOR_CORES and q.dtype == torch.bfloat16 and dk == dv and dk in (64, 128)
            and not chunk and (gate is None or gate_per_head) and ctx.max_q_len >= 128
            and cache.page_size in (8, 16, 32, 64)
            and _lib("attention_tc5").lsb_prefill_attention_tc5_supported(
                _p(q), _i(q.shape[1]), _p(cache.k_pages), _p(cache.v_pages), _i(nh), _i(nkv), _i(dk), _i(cache.page_size))):
        n_decode, first, last = _batch_shape(ctx)
        if n_decode == 0 or (n_decode == first and last == ctx.n_requests):
            off = 4 * first
            _call("attention_tc5", "lsb_prefill_attention_tc5_biased", _p(q), _i(q.shape[1]), _i(T), _p(cache.k_pages),
                  _p(cache.v_pages), ctypes.c_void_p(ctx.q_start.data_ptr() + off),
                  ctypes.c_void_p(ctx.kv_len.data_ptr() + off), ctypes.c_void_p(ctx.table_rows.data_ptr() + off),
                  _p(cache.block_table), _i(cache.block_table.shape[1]), _p(out), _i(ctx.n_requests - first),
                  _i(ctx.max_q_len), _i(nh), _i(nkv), _i(dk), _i(cache.page_size), _i(cache.k_pages.shape[0]), _f(scale),
                  _i(window), _i(0), _i(1 if sink else 0), _p(gate), _ll(gate_stride), _f(softcap),
                  _i(1 if linear_bias else 0), _stream(out))
            if first == 0:
                return
            n_req, max_q = first, 1
    if (DV_TENSOR_CORES and q.dtype == torch.bfloat16 and gate_stride % 2 == 0
            and (gate is None or gate.data_ptr() % 4 == 0)
            and _lib("attention_dv").lsb_attention_dv_mma_supported(_i(dk), _i(dv))):
        # a few blocks only (single tokens, one short portion): the keys of a row tile are shared among
        # several blocks, whose partial sums meet in a scratch buffer kept for reuse
        lib = _lib("attention_dv")
        plan = lib.lsb_attention_dv_mma_plan(_i(n_req), _i(max_q), _i(nh), _i(nkv), _i(chunk),
                                             _i(num_sms(q.device)), _i(DV_BLOCK_SHAPE))
        scratch = None
        if plan >> 8 > 1:
            tiles = -(-max_q * (nh // nkv) // 16)
            key = ("attention_dv", q.device, n_req * nkv * tiles * (plan >> 8) * 16 * (dv + 2))
            scratch = _scratch.get(key)
            if scratch is None:
                scratch = _scratch[key] = torch.empty(key[2], dtype=torch.float32, device=q.device)
        _call("attention_dv", "lsb_attention_dv_mma", _p(q), _p(cache.k_pages), _p(cache.v_pages), _p(ctx.q_start),
              _p(ctx.kv_len), _p(ctx.table_rows), _p(cache.block_table), _i(cache.block_table.shape[1]), _p(gate),
              _ll(gate_stride), _p(out), _i(n_req), _i(max_q), _i(nh), _i(nkv), _i(dk), _i(dv),
              _i(cache.page_size), _i(cache.k_pages.shape[0]), _f(scale), _i(window), _i(chunk), _i(num_sms(q.device)),
              _i(DV_BLOCK_SHAPE), _p(scratch), _i(flags), _f(softcap), _stream(out))
        return
    _call("attention_dv", "lsb_attention_dv_generic", _p(q), _p(cache.k_pages), _p(cache.v_pages), _p(ctx.q_start),
          _p(ctx.kv_len), _p(ctx.table_rows), _p(cache.block_table), _i(cache.block_table.shape[1]), _p(gate),
          _ll(gate_stride), _p(out), _i(_dt(q)), _i(n_req), _i(max_q), _i(nh), _i(nkv), _i(dk),
          _i(dv), _i(cache.page_size), _i(cache.k_pages.shape[0]), _f(scale), _i(window), _i(chunk), _i(flags), _f(softcap),
          _stream(out))


def branch_sum(ys, scales, out: torch.Tensor) -> None:
    """out = sum_b scales[b] * ys[b], summed in 32-bit (mixers side by side whose results are added
    with fixed factors)."""
    n = len(ys)
    if n == 0 or len(scales) != n:
        raise KernelError("branch_sum: one factor per branch")
    _req(out, "out", dim=2)
    for y in ys:
        _req(y, "branch", out.dtype, 2)
        if y.shape != out.shape:
            raise KernelError("branch_sum: every branch must have out's shape")
    yp = (ctypes.c_void_p * n)(*[_p(y).value for y in ys])
    sc = (ctypes.c_float * n)(*[float(x) for x in scales])
    _call("sandwich", "lsb_branch_sum", yp, sc, _i(n), _p(out), _i(_dt(out)), _i(out.shape[0]), _i(out.shape[1]),
          _stream(out))


PLAIN_ACTIVATIONS = {"silu": 1, "gelu_tanh": 2, "none": 3, "bent_square": 4}


def plain_activation(x: torch.Tensor, out: torch.Tensor, activation: str, c_pos: float = 0.0, c_neg: float = 0.0) -> None:
    """out = act(x) element by element, evaluated in 32-bit.  "bent_square": ``c_pos z^2 + z/2`` right of
    zero, ``c_neg (e^z - 1 - z) + z/2`` left of it."""
    _req(x, "x")
    _req(out, "out", x.dtype)
    if out.shape != x.shape or activation not in PLAIN_ACTIVATIONS:
        raise KernelError(f"plain_activation: shapes disagree or '{activation}' is not known")
    _call("activation", "lsb_plain_act", _p(x), _p(out), _i(_dt(x)), _ll(x.numel()), _i(PLAIN_ACTIVATIONS[activation]),
          _f(c_pos), _f(c_neg), _stream(out))


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place (32-bit)."""
    _req(x, "x", torch.float32)
    if not cap > 0:
        raise KernelError("softcap: the cap must be positive")
    _call("activation", "lsb_softcap", _p(x), _ll(x.numel()), _f(cap), _stream(x))


# ---------------------------------------------------------------------- delta-rule memories
def delta_max_key_dim() -> int:
    return int(_lib("delta_rule").lsb_delta_max_key_dim())


def gated_delta_prep(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, key_heads: int, heads: int, key_dim: int,
                     value_dim: int, taps, conv_state: Optional[torch.Tensor], raw: torch.Tensor, a_log: torch.Tensor,
                     dt_bias: torch.Tensor, ctx, qk: torch.Tensor, v: torch.Tensor, scal: torch.Tensor,
                     unit_eps: float = 1e-6) -> None:
    """What a delta-rule memory with scalar gates needs of a step's tokens, in 32-bit.  ``proj`` [T, columns]
    holds the projections of q and k (``key_heads * key_dim`` each) and v (``heads * value_dim``); ``taps`` =
    (q, k, v) filters [channels, n] of a causal convolution over time whose last column meets the current
    token, the n - 1 inputs before a portion coming from ``conv_state`` [slots, n - 1, channels] (updated
    for the next step); then silu; q and k to unit length per head, q also times key_dim^-1/2 -> ``qk``
    [T, 2 * key_heads * key_dim]; v -> ``v`` [T, heads * value_dim].  ``raw`` [T, 2 * heads] 32-bit: the
    projections of beta and of the fade; ``scal`` [T, 2 * heads] receives
    exp(-exp(a_log) * softplus(. + dt_bias)) and then sigmoid(.)."""
    _req(proj, "proj", dim=2)
    T, ld = proj.shape
    GD, HV = key_heads * key_dim, heads * value_dim
    C = 2 * GD + HV
    n = taps[0].shape[1]
    for name, t, rows in (("q taps", taps[0], GD), ("k taps", taps[1], GD), ("v taps", taps[2], HV)):
        _req(t, name, torch.float32, 2)
        if t.shape != (rows, n):
            raise KernelError(f"gated_delta_prep: {name} must be [{rows}, {n}]")
    if n > 1:
        _req(conv_state, "conv_state", torch.float32, 3)
        if conv_state.shape[1:] != (n - 1, C):
            raise KernelError(f"gated_delta_prep: conv_state must be [slots, {n - 1}, {C}]")
    _req(raw, "raw", torch.float32, 2, contiguous=False)
    for name, t, shape in (("qk", qk, (T, 2 * GD)), ("v", v, (T, HV)), ("scal", scal, (T, 2 * heads))):
        _req(t, name, torch.float32, 2)
        if t.shape != shape:
            raise KernelError(f"gated_delta_prep: {name} must be {shape}")
    for name, t in (("a_log", a_log), ("dt_bias", dt_bias)):
        _req(t, name, torch.float32, 1)
        if t.shape[0] != heads:
            raise KernelError(f"gated_delta_prep: {name} must have {heads} entries")
    if (ctx.n_tokens != T or raw.shape != (T, 2 * heads) or raw.stride(1) != 1 or min(q_off, k_off, v_off) < 0
            or max(q_off, k_off) + GD > ld or v_off + HV > ld or heads % key_heads):
        raise KernelError("gated_delta_prep: proj, raw and the step do not fit the sizes")
    _call("delta_rule", "lsb_gated_delta_prep", _p(proj), _i(_dt(proj)), _ll(ld), _i(q_off), _i(k_off), _i(v_off), _i(T),
          _i(ctx.n_requests), _i(key_heads), _i(heads), _i(key_dim), _i(value_dim), _i(n), _p(taps[0]), _p(taps[1]),
          _p(taps[2]), _p(conv_state if n > 1 else None), _i(conv_state.shape[0] if n > 1 else 1 << 30), _p(raw),
          _ll(raw.stride(0)), _p(a_log), _p(dt_bias), _p(ctx.token_req), _p(ctx.q_start), _p(ctx.table_rows), _p(qk), _p(v),
          _p(scal), _f(unit_eps), _stream(proj))


def channel_delta_prep(proj: torch.Tensor, r_off: int, k_off: int, v_off: int, heads: int, key_dim: int, value_dim: int,
                       decay_raw: torch.Tensor, decay_bias: torch.Tensor, remove_raw: torch.Tensor,
                       remove_bias: torch.Tensor, decay_rate: float, vecs: torch.Tensor, v: torch.Tensor,
                       unit_eps: float = 1e-6) -> None:
    """What a delta-rule memory with a gate per key channel needs, in 32-bit: per token and head the read
    vector r, the key k, its unit vector u = k / sqrt(sum k^2 + eps), a * u with a = sigmoid(remove_raw +
    remove_bias) and the decay w = exp(-decay_rate * sigmoid(decay_raw + decay_bias)) -> ``vecs``
    [T, heads, 5, key_dim]; the values -> ``v`` [T, heads * value_dim]."""
    _req(proj, "proj", dim=2)
    T, ld = proj.shape
    HD = heads * key_dim
    for name, t in (("decay_raw", decay_raw), ("remove_raw", remove_raw)):
        _req(t, name, torch.float32, 2, contiguous=False)
        if t.shape != (T, HD) or t.stride(1) != 1:
            raise KernelError(f"channel_delta_prep: {name} must be [T, heads * key_dim] with unit column stride")
    for name, t in (("decay_bias", decay_bias), ("remove_bias", remove_bias)):
        _req(t, name, torch.float32, 1)
        if t.shape[0] != HD:
            raise KernelError(f"channel_delta_prep: {name} must have {HD} entries")
    _req(vecs, "vecs", torch.float32, 4)
    _req(v, "v", torch.float32, 2)
    if (vecs.shape != (T, heads, 5, key_dim) or v.shape != (T, heads * value_dim) or min(r_off, k_off, v_off) < 0
            or max(r_off, k_off) + HD > ld or v_off + heads * value_dim > ld):
        raise KernelError("channel_delta_prep: proj, vecs and v do not fit the sizes")
    _call("delta_rule", "lsb_channel_delta_prep", _p(proj), _i(_dt(proj)), _ll(ld), _i(r_off), _i(k_off), _i(v_off), _i(T),
          _i(heads), _i(key_dim), _i(value_dim), _p(decay_raw), _ll(decay_raw.stride(0)), _p(decay_bias), _p(remove_raw),
          _ll(remove_raw.stride(0)), _p(remove_bias), _f(decay_rate), _f(unit_eps), _p(vecs), _p(v), _stream(proj))


DELTA_SEGMENT = 128             # tokens of a segment when long portions of a delta-rule memory are walked in segments (0: never);
                                # half as many for portions of up to eight segments
DELTA_SEGMENT_REQUESTS = 64     # ... in steps of at most this many requests


def delta_scan(form: str, vecs: torch.Tensor, scal: Optional[torch.Tensor], vals: torch.Tensor, state: torch.Tensor, ctx,
               out: torch.Tensor, heads: int, key_heads: int, key_dim: int, value_dim: int) -> None:
    """The walk of a delta-rule memory, each request from its slot's state (``state`` [slots, heads,
    value_dim, key_dim] 32-bit, updated in place), tokens in order; ``out`` [T, heads * value_dim] 32-bit.
    "scalar": S <- g S; e = beta (v - S^T k); S += k e^T; o = S^T q, with ``vecs`` [T, 2 * key_heads * key_dim]
    (q then k) and ``scal`` [T, 2 * heads] (g then beta).  "channel": S <- diag(w) S - (a * u)(u^T S) + k v^T,
    o = S^T r, with ``vecs`` [T, heads, 5, key_dim] (r, k, u, a * u, w)."""
    if form not in ("scalar", "channel"):
        raise KernelError(f"delta_scan: form '{form}' is not known (scalar, channel)")
    _req(vecs, "vecs", torch.float32)
    _req(vals, "vals", torch.float32, 2)
    _req(state, "state", torch.float32, 4)
    _req(out, "out", torch.float32, 2)
    T = vals.shape[0]
    n_vec = 2 * key_heads * key_dim if form == "scalar" else heads * 5 * key_dim
    if (state.shape[1:] != (heads, value_dim, key_dim) or out.shape != (T, heads * value_dim) or vals.shape != out.shape
            or ctx.n_tokens != T or vecs.numel() != T * n_vec):
        raise KernelError("delta_scan: vecs, vals, state, out or the step do not fit the sizes")
    if form == "scalar":
        _req(scal, "scal", torch.float32, 2)
        if scal.shape != (T, 2 * heads) or heads % key_heads:
            raise KernelError("delta_scan: scal must be [T, 2 * heads]")
    if key_dim > delta_max_key_dim():
        raise KernelError(f"delta_scan: key_dim {key_dim} is not supported (at most {delta_max_key_dim()})")
    # a step with a long portion: every request's tokens in segments walked side by side (three times the
    # arithmetic, a chain a segment long), single tokens beside it included; short portions, single
    # tokens only, or very many requests: one walk each.  Scratch: a row per segment,
    # tokens / segment + requests at most.
    seg, seg_acc, seg_start = 0, None, None
    # (segments half as long for portions up to eight segments: more of them side by side; measured at
    # 8 heads of 128 x 128: 512 tokens 244 us in one walk, 210 in segments of 128, 166 in segments of 64)
    want = 0 if not DELTA_SEGMENT else DELTA_SEGMENT if ctx.max_q_len > 8 * DELTA_SEGMENT else max(1, DELTA_SEGMENT // 2)
    if want and ctx.max_q_len >= 4 * want and ctx.n_requests <= DELTA_SEGMENT_REQUESTS:
        seg = want
        n = T // seg + ctx.n_requests
        seg_acc = torch.empty(n * heads * (value_dim + key_dim) * key_dim, dtype=torch.float32, device=out.device)
        seg_start = torch.empty(n * heads * value_dim * key_dim, dtype=torch.float32, device=out.device)
    _call("delta_rule", "lsb_delta_scan", _i(0 if form == "scalar" else 1), _p(vecs), _p(scal if form == "scalar" else None),
          _p(vals), _p(state), _i(state.shape[0]), _p(ctx.q_start), _p(ctx.table_rows), _i(ctx.n_requests), _p(out),
          _i(heads), _i(key_heads), _i(key_dim), _i(value_dim), _i(seg), _i(ctx.max_q_len), _p(seg_acc), _p(seg_start),
          _stream(out))


_DELTA_GATES = {"none": 0, "sigmoid": 1, "silu": 2}


def delta_output(x: torch.Tensor, weight: torch.Tensor, heads: int, eps: float, gate: Optional[torch.Tensor],
                 gate_act: str, out: torch.Tensor) -> None:
    """out = each head of the 32-bit row ``x`` [T, heads * V] divided by its root mean square, times ``weight``
    (its index taken modulo its length: one weight per head, or one over the row), times sigmoid or silu of
    ``gate`` [T, heads * V] (rows may be strided)."""
    _req(x, "x", torch.float32, 2)
    _req(weight, "weight", torch.float32, 1)
    _req(out, "out", dim=2)
    T, n = x.shape
    if out.shape != (T, n) or heads <= 0 or n % heads or n % weight.shape[0] or gate_act not in _DELTA_GATES:
        raise KernelError("delta_output: shapes disagree")
    gate_stride = 0
    if gate is not None:
        _req(gate, "gate", out.dtype, 2, contiguous=False)
        if gate.shape != (T, n) or gate.stride(1) != 1:
            raise KernelError("delta_output: the gate must have x's shape and unit column stride")
        gate_stride = gate.stride(0)
    _call("delta_rule", "lsb_delta_output", _p(x), _p(weight), _i(weight.shape[0]), _p(gate), _ll(gate_stride),
          _i(_DELTA_GATES[gate_act] if gate is not None else 0), _p(out), _i(_dt(out)), _i(T), _i(heads), _i(n // heads),
          _f(eps), _stream(out))


def tanh_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = tanh(x) in the compute dtype; ``x`` 32-bit [T, n], rows may be strided."""
    _req(x, "x", torch.float32, 2, contiguous=False)
    _req(out, "out", dim=2)
    if out.shape != x.shape or x.stride(1) != 1:
        raise KernelError("tanh_rows: shapes disagree")
    _call("delta_rule", "lsb_tanh_rows", _p(x), _ll(x.stride(0)), _i(0), _i(x.shape[1]), _p(out), _i(_dt(out)),
          _i(x.shape[0]), _stream(out))


# -------------------------------------------------- matrix memory with an exponential input gate
def memory_gates(raw: torch.Tensor, i_bias: Optional[torch.Tensor], f_bias: Optional[torch.Tensor], cap: float,
                 m_state: torch.Tensor, ctx, gates: torch.Tensor) -> None:
    """``raw`` [T, 2 * heads] 32-bit holds the input-gate and then the forget-gate projections.  With
    i = cap * tanh((zi + bi) / cap), f = logsigmoid(cap * tanh((zf + bf) / cap)) and the running
    maximum m_t = max(f + m_(t-1), i) (per request and head, carried in ``m_state`` [slots, heads]),
    ``gates`` [3, T, heads] receives exp(f + m_(t-1) - m_t), exp(i - m_t) and exp(-m_t).  ``raw`` may be
    overwritten (steps with long portions form the gate activations in place)."""
    _req(raw, "raw", torch.float32, 2)
    _req(m_state, "m_state", torch.float32, 2)
    _req(gates, "gates", torch.float32, 3)
    T, heads = raw.shape[0], m_state.shape[1]
    if raw.shape[1] != 2 * heads or gates.shape != (3, T, heads) or ctx.n_tokens != T:
        raise KernelError("memory_gates: raw, m_state, gates and the step disagree")
    for name, t in (("i_bias", i_bias), ("f_bias", f_bias)):
        if t is not None:
            _req(t, name, torch.float32, 1)
            if t.shape[0] != heads:
                raise KernelError(f"memory_gates: {name} must have {heads} entries")
    _call("matrix_memory", "lsb_memory_gates", _p(raw), _p(i_bias), _p(f_bias), _f(cap), _p(m_state),
          _i(m_state.shape[0]), _p(ctx.q_start), _p(ctx.table_rows), _i(ctx.n_requests), _p(gates), _i(T), _i(heads),
          _i(ctx.max_q_len), _stream(gates))


def memory_output(walked: torch.Tensor, floor: torch.Tensor, weight: torch.Tensor, gate: Optional[torch.Tensor],
                  eps: float, out: torch.Tensor) -> None:
    """``walked`` [T, heads * (V + 1)] 32-bit: per head S^T q in V columns and n . q in the last;
    ``floor`` [T, heads].  o = S^T q / (max(|n . q|, floor) + 1e-6); out = unit(o) per head * weight
    [heads * V] * sigmoid(gate)."""
    _req(walked, "walked", torch.float32, 2)
    _req(floor, "floor", torch.float32, 2)
    _req(weight, "weight", torch.float32, 1)
    _req(out, "out", dim=2)
    T, heads = floor.shape
    V = out.shape[1] // max(heads, 1)
    if out.shape != (T, heads * V) or walked.shape != (T, heads * (V + 1)) or weight.shape[0] != heads * V:
        raise KernelError("memory_output: shapes disagree")
    gate_stride = 0
    if gate is not None:
        _req(gate, "gate", out.dtype, 2, contiguous=False)
        if gate.shape != out.shape or gate.stride(1) != 1:
            raise KernelError("memory_output: the gate must have out's shape and unit column stride")
        gate_stride = gate.stride(0)
    _call("matrix_memory", "lsb_memory_output", _p(walked), _p(floor), _p(weight), _p(gate), _ll(gate_stride),
          _p(out), _i(_dt(out)), _i(T), _i(heads), _i(V), _f(eps), _stream(out))


# ------------------------------------------------------------------------ routed experts
MOE_SCORES = {"sigmoid": 0, "softmax": 1}
MOE_TENSOR_CORES = True         # bfloat16 experts on the grouped tcgen05 product


def moe_tile() -> int:
    """Rows an expert's share of a step is padded to."""
    return int(_lib("moe").lsb_moe_tile())


def _route_options(E: int, choice_bias: Optional[torch.Tensor], weight_scale: float, renorm_eps: float):
    if choice_bias is not None:
        _req(choice_bias, "choice_bias", torch.float32, 1)
        if choice_bias.shape[0] != E:
            raise KernelError(f"moe: the choice bias must have {E} entries")
    return _p(choice_bias), _f(weight_scale), _f(renorm_eps)


def moe_route(logits: torch.Tensor, top: int, score: str, renormalize: bool, ids: torch.Tensor,
              weights: torch.Tensor, choice_bias: Optional[torch.Tensor] = None, weight_scale: float = 1.0,
              renorm_eps: float = 0.0) -> None:
    """The ``top`` experts with the largest scores per row of 32-bit ``logits`` and their scores.
    ``choice_bias`` (one number an expert) is added to the scores for the choice only; the weights are the
    chosen scores themselves, divided by their sum + ``renorm_eps`` if ``renormalize``, times ``weight_scale``."""
    _req(logits, "logits", torch.float32, 2)
    _req(ids, "ids", torch.int32, 2)
    _req(weights, "weights", torch.float32, 2)
    T, E = logits.shape
    if ids.shape != (T, top) or weights.shape != (T, top) or not 0 < top <= min(E, 32):
        raise KernelError("moe_route: ids / weights must be [tokens, top], top at most 32")
    _call("moe", "lsb_moe_route", _p(logits), _i(T), _i(E), _i(top), _i(MOE_SCORES[score]),
          _i(1 if renormalize else 0), *_route_options(E, choice_bias, weight_scale, renorm_eps), _p(ids), _p(weights),
          _stream(ids))


MOE_FUSED_ROUTING_TOKENS = 256  # steps of at most this many tokens choose their experts inside the sorting kernel


def moe_routed_experts(x: torch.Tensor, logits: torch.Tensor, top: int, score: str, renormalize: bool,
                       w_gate_up: torch.Tensor, w_down: torch.Tensor, activation: str, weight_on: str,
                       out: torch.Tensor, choice_bias: Optional[torch.Tensor] = None, weight_scale: float = 1.0,
                       renorm_eps: float = 0.0, limit: float = 0.0, add: Optional[torch.Tensor] = None) -> None:
    """``moe_route`` on the 32-bit ``logits`` followed by ``moe_experts``; in a step of few tokens the
    choosing rides in the kernel that sorts the rows by expert (one launch less)."""
    _req(logits, "logits", torch.float32, 2)
    T, E = logits.shape
    ids = torch.empty(T, top, dtype=torch.int32, device=x.device)
    weights = torch.empty(T, top, dtype=torch.float32, device=x.device)
    if not 0 < top <= min(E, 32):
        raise KernelError("moe_routed_experts: top must be in [1, min(experts, 32)]")
    if T <= MOE_FUSED_ROUTING_TOKENS:
        moe_experts(x, ids, weights, w_gate_up, w_down, activation, weight_on, out,
                    route=(logits, MOE_SCORES[score], 1 if renormalize else 0, choice_bias, weight_scale, renorm_eps),
                    limit=limit, add=add)
    else:
        moe_route(logits, top, score, renormalize, ids, weights, choice_bias, weight_scale, renorm_eps)
        moe_experts(x, ids, weights, w_gate_up, w_down, activation, weight_on, out, limit=limit, add=add)


def moe_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, activation: str, weight_on: str, out: torch.Tensor, route=None,
                limit: float = 0.0, add: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum over k of down_e(act(gate_e u) * up_e u), e = ids[t, k], with u = weights[t, k] * x[t]
    (``weight_on`` "input") or u = x[t] and the sum weighted ("output"); plus ``add[t]`` if given (a shared
    expert's rows, or a callable that makes them: it is called behind the experts' products), in the same
    32-bit sum.  ``w_gate_up`` [E, 2F, H] has
    rows alternating gate_i, up_i; ``w_down`` [E, H, F]."""
    _req(x, "x", dim=2)
    _req(ids, "ids", torch.int32, 2)
    _req(weights, "weights", torch.float32, 2)
    _req(w_gate_up, "w_gate_up", x.dtype, 3)
    _req(w_down, "w_down", x.dtype, 3)
    _req(out, "out", x.dtype, 2)
    T, H = x.shape
    E, F2, _ = w_gate_up.shape
    F, top = F2 // 2, ids.shape[1]
    if w_gate_up.shape != (E, 2 * F, H) or w_down.shape != (E, H, F) or out.shape != (T, H) \
            or ids.shape[0] != T or weights.shape != ids.shape or weight_on not in ("input", "output"):
        raise KernelError("moe_experts: shapes disagree")
    # bfloat16 with TMA-friendly sizes: rows gathered in place, two grouped tcgen05 products over
    # 128-row tiles; anything else (32-bit, odd sizes): the plain grouped kernels over 32-row tiles
    tc = MOE_TENSOR_CORES and x.dtype == torch.bfloat16 and H % 8 == 0 and F % 8 == 0
    tile = 128 if tc else moe_tile()
    cap_tiles = -(-T * top // tile) + E
    dev = x.device
    pos = torch.empty(T * top, dtype=torch.int32, device=dev)
    row_token = torch.empty(cap_tiles * tile, dtype=torch.int32, device=dev)
    row_scale = torch.empty(cap_tiles * tile, dtype=torch.float32, device=dev)
    tile_expert = torch.empty(cap_tiles, dtype=torch.int32, device=dev)
    hidden = torch.empty(cap_tiles * tile, F, dtype=x.dtype, device=dev)
    y = torch.empty(cap_tiles * tile, H, dtype=x.dtype if tc else torch.float32, device=dev)
    s = _stream(out)
    on_input = 1 if weight_on == "input" else 0
    r_logits, r_score, r_renorm, r_bias, r_scale, r_eps = (tuple(route) + (None, 1.0, 0.0))[:6] if route is not None \
        else (None, 0, 0, None, 1.0, 0.0)
    if r_logits is not None and r_logits.shape != (T, E):
        raise KernelError("moe_experts: the router's logits must be [tokens, experts]")
    unfused = activation in UNFUSED_GATED
    if unfused and not limit > 0:
        raise KernelError(f"moe_experts: '{activation}' needs a positive limit")
    _call("moe", "lsb_moe_align", _p(ids), _p(weights), _i(T), _i(top), _i(E), _i(cap_tiles), _i(tile), _p(pos),
          _p(row_token), _p(row_scale), _p(tile_expert), _p(r_logits), _i(r_score), _i(r_renorm),
          *_route_options(E, r_bias, r_scale, r_eps), s)
    if tc:
        rows = torch.empty(cap_tiles * tile, H, dtype=x.dtype, device=dev)
        _call("moe", "lsb_moe_gather", _p(x), _i(_dt(x)), _p(pos), _p(weights), _i(on_input), _i(T), _i(top),
              _i(cap_tiles * tile), _i(H), _p(rows), s)
        _chain_ends()
        _call("gemm_tc", "lsb_gemm_tc_grouped", _p(rows), _p(w_gate_up), _p(hidden), _i(0), _i(cap_tiles * tile),
              _i(2 * F), _i(H), _i(E), _p(tile_expert), _i(_activation_id(activation)), _f(limit), s)
        _call("gemm_tc", "lsb_gemm_tc_grouped", _p(hidden), _p(w_down), _p(y), _i(0), _i(cap_tiles * tile),
              _i(H), _i(F), _i(E), _p(tile_expert), _i(0), _f(0.0), s)
    else:
        _call("moe", "lsb_moe_up", _p(x), _i(_dt(x)), _p(row_token), _p(row_scale), _i(on_input), _p(w_gate_up),
              _p(tile_expert), _i(cap_tiles), _p(hidden), _i(F), _i(H), _i(_activation_id(activation)), _f(limit), s)
        _call("moe", "lsb_moe_down", _p(hidden), _i(_dt(x)), _p(row_token), _p(w_down), _p(tile_expert), _i(cap_tiles),
              _p(y), _i(H), _i(F), s)
    if callable(add):           # made now, behind the experts' products (its own products' weights are then the
        add = add()             # last streamed before the next layer's, which they ask L2 for while they end)
    if add is not None:
        _req(add, "add", x.dtype, 2)
        if add.shape != (T, H):
            raise KernelError("moe_experts: add must have out's shape")
    _call("moe", "lsb_moe_combine", _p(y), _i(1 if tc else 0), _p(pos), _p(weights), _i(1 - on_input), _i(T), _i(top),
          _i(H), _i(cap_tiles * tile), _p(out), _i(_dt(out)), _p(add), s)


def sample(logits: torch.Tensor, params: torch.Tensor, top_k: torch.Tensor,
           prev_start: Optional[torch.Tensor], prev_tokens: Optional[torch.Tensor],
           out: torch.Tensor, work: Optional[torch.Tensor] = None) -> None:
    """One token per row of ``logits``.  ``params[r] = (temperature, top_p, repetition_penalty,
    u)``; ``top_k[r]`` (0 = off); ``prev_tokens[prev_start[r]:prev_start[r+1]]`` are the tokens the
    repetition penalty applies to; ``work`` is scratch shaped like ``logits`` (needed only when
    a penalty is in use)."""
    _req(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    _req(params, "params", torch.float32, 2)
    _req(top_k, "top_k", torch.int32, 1)
    _req(out, "out", torch.int32, 1)
    if params.shape != (R, 4) or top_k.shape[0] != R or out.shape[0] != R:
        raise KernelError("sample: per-row arrays do not match the logits")
    if prev_start is not None:
        _req(prev_start, "prev_start", torch.int32, 1)
        _req(prev_tokens, "prev_tokens", torch.int32, 1)
        if work is None:
            work = torch.empty_like(logits)
        _req(work, "work", torch.float32, 2)
        if work.shape != logits.shape:
            raise KernelError("sample: work must be shaped like logits")
    _call("sampling", "lsb_sample", _p(logits), _p(work), _i(R), _i(V), _p(params), _p(top_k),
          _p(prev_start), _p(prev_tokens), _p(out), _stream(out))
