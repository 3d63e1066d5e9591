"""Python faces of the CUDA kernels.

Each function checks its tensors (device, dtype, layout), launches on the
current CUDA stream and raises on any error.  There is no CPU path: a tensor
that is not on a CUDA device is refused.
"""
from __future__ import annotations

import ctypes
from typing import Optional

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
                ("attention_tc", "attention_tc"))


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


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    n, d = out.shape
    if table.shape[1] != d or ids.numel() != n:
        raise KernelError("embed_rows: shape mismatch")
    lib = load_library("rowwise")
    _run("embed_rows", lib.kp_embed_rows, _ptr(table), _ptr(ids), _ptr(out), n, d, ctypes.c_float(scale),
                             dtype_code(table.dtype), STREAM)
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


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    n, ff = out.shape
    if gate_up.shape != (n, 2 * ff):
        raise KernelError("swiglu: shape mismatch")
    lib = load_library("rowwise")
    _run("swiglu", lib.kp_swiglu, _ptr(gate_up), _ptr(out), n, ff, dtype_code(out.dtype), STREAM)
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


# ------------------------------------------------------------------ attention

def qk_norm_rope_kv(qkv: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
                    cos_tab: Optional[torch.Tensor], sin_tab: Optional[torch.Tensor], rotary_dim: int,
                    interleaved: bool, positions: torch.Tensor, slot_map: Optional[torch.Tensor],
                    q_out: Optional[torch.Tensor], cache: Optional[torch.Tensor], page_size: int, H: int, G: int,
                    hd: int) -> Optional[torch.Tensor]:
    """Norm + rotate q and k; write q to ``q_out`` and, if ``cache`` is given,
    k and v to their pages.  ``cache`` is one layer's [pages, 2, G, page_size, hd].
    With ``q_out`` None, q and k are changed in place and no cache is written."""
    _need(qkv, "qkv", contiguous=False)
    _need(positions, "positions", torch.int32)
    n = qkv.shape[0]
    if qkv.shape[1] != (H + 2 * G) * hd:
        raise KernelError("qk_norm_rope_kv: shape mismatch")
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
    lib = load_library("qkrope")
    _run("qk_norm_rope_kv", lib.kp_qk_norm_rope_kv, _ptr(qkv), _rows_2d(qkv, "qkv"), _ptr(q_w), _ptr(k_w), ctypes.c_float(eps),
                                  _ptr(cos_tab), _ptr(sin_tab), rotary_dim, int(interleaved), _ptr(positions),
                                  _ptr(slot_map), _ptr(q_out), 0 if q_out is None else _rows_2d(q_out, "q_out"), _ptr(cache),
                                  page_size,
                                  n, H, G, hd, int(write_kv), dtype_code(qkv.dtype), STREAM)
    return q_out


def attention_rows(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, row_seg: torch.Tensor,
                   positions: torch.Tensor, out: torch.Tensor, scale: float, window: Optional[int],
                   page_size: int, H: int, G: int, hd: int) -> torch.Tensor:
    _need(q, "q", contiguous=False); _need(cache, "cache", q.dtype); _need(out, "out", q.dtype, contiguous=False)
    _need(block_table, "block_table", torch.int32); _need(row_seg, "row_seg", torch.int32)
    _need(positions, "positions", torch.int32)
    n = q.shape[0]
    if q.shape[1] != H * hd or out.shape != (n, H * hd) or tuple(cache.shape[1:]) != (2, G, page_size, hd):
        raise KernelError("attention_rows: shape mismatch")
    lib = load_library("attention")
    _run("attention_rows", lib.kp_attention_rows, _ptr(q), _rows_2d(q, "q"), _ptr(cache), _ptr(block_table), block_table.shape[1],
                                 _ptr(row_seg), _ptr(positions), _ptr(out), _rows_2d(out, "out"),
                                 ctypes.c_float(scale), int(window or 0), page_size, n, H, G, hd,
                                 dtype_code(q.dtype), STREAM)
    return out


SPLIT_CHUNK = 256          # keys a chunk of the split-KV attention
SPLIT_CHUNK_MMA = 256       # keys a chunk of its tensor-core form: 64, 128 or 256 (a divisor of SPLIT_CHUNK)
SPLIT_MAX_RATIO = 8        # query heads per kv head it takes


def attention_split_scratch(n_rows: int, H: int, hd: int, n_chunks: int) -> int:
    """Float elements of scratch that :func:`attention_split` needs."""
    return n_rows * H * n_chunks * (SPLIT_CHUNK // min(SPLIT_CHUNK, SPLIT_CHUNK_MMA)) * (hd + 2)


def attention_split(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, row_seg: torch.Tensor,
                    positions: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, n_chunks: int, scale: float,
                    window: Optional[int], page_size: int, H: int, G: int, hd: int) -> torch.Tensor:
    """Split-KV attention (chunks of 256 keys, merged in order).  ``n_chunks``
    must cover the largest position of the batch; ``scratch`` is float32."""
    _need(q, "q", contiguous=False); _need(cache, "cache", q.dtype); _need(out, "out", q.dtype, contiguous=False)
    _need(block_table, "block_table", torch.int32); _need(row_seg, "row_seg", torch.int32)
    _need(positions, "positions", torch.int32); _need(scratch, "scratch", torch.float32)
    n = q.shape[0]
    if q.shape[1] != H * hd or out.shape != (n, H * hd) or tuple(cache.shape[1:]) != (2, G, page_size, hd):
        raise KernelError("attention_split: shape mismatch")
    if scratch.numel() < attention_split_scratch(n, H, hd, n_chunks):
        raise KernelError("attention_split: scratch too small")
    lib = load_library("attention_decode")
    if USE_MMA_ATTENTION and q.dtype == torch.bfloat16 and hd in (64, 128) and q.stride(0) % 2 == 0:
        # tensor-core chunk pass over smaller chunks, then the same merge
        parts = n_chunks * (SPLIT_CHUNK // SPLIT_CHUNK_MMA)
        _run("attention_split_mma", load_library("attention_mma").kp_attention_split_mma, 
            _ptr(q), _rows_2d(q, "q"), _ptr(cache), ctypes.c_longlong(cache.shape[0] if USE_TMA_ATTENTION else 0),
            _ptr(block_table), block_table.shape[1], _ptr(row_seg),
            _ptr(positions), _ptr(scratch), parts, SPLIT_CHUNK_MMA, ctypes.c_float(scale), int(window or 0), page_size,
            n, H, G, hd, STREAM)
        _run("attention_merge", lib.kp_attention_merge, _ptr(positions), _ptr(out), _rows_2d(out, "out"), _ptr(scratch), parts,
                                      SPLIT_CHUNK_MMA, int(window or 0), n, H, hd, dtype_code(q.dtype), STREAM)
        return out
    _run("attention_split", lib.kp_attention_split, _ptr(q), _rows_2d(q, "q"), _ptr(cache), _ptr(block_table), block_table.shape[1],
                                  _ptr(row_seg), _ptr(positions), _ptr(out), _rows_2d(out, "out"), _ptr(scratch),
                                  n_chunks, ctypes.c_float(scale), int(window or 0), page_size, n, H, G, hd,
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
                      big_tile_seg: Optional[torch.Tensor] = None, big_tile_row0: Optional[torch.Tensor] = None
                      ) -> torch.Tensor:
    """Tensor-core causal attention for segments of many rows.  ``tile_seg`` / ``tile_row0`` list, for every
    tile of 64 consecutive rows of a segment, its segment and its first row; ``big_tile_seg`` /
    ``big_tile_row0`` the same for tiles of 128 rows, the tile that reads the most keys first (with them the
    tcgen05 kernel runs where it takes the sizes)."""
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
    if big_tile_seg is not None and attention_prefill_tc_ok(q, out, cache, page_size, hd):
        _need(big_tile_seg, "big_tile_seg", torch.int32); _need(big_tile_row0, "big_tile_row0", torch.int32)
        if big_tile_seg.numel() != big_tile_row0.numel():
            raise KernelError("attention_prefill: tile lists differ in length")
        _run("attention_prefill_tc", load_library("attention_tc").kp_attention_prefill_tc, 
            _ptr(q), _rows_2d(q, "q"), n, _ptr(cache), ctypes.c_longlong(cache.shape[0]), _ptr(block_table),
            block_table.shape[1], _ptr(cu_rows), _ptr(seg_pos), _ptr(big_tile_seg), _ptr(big_tile_row0),
            big_tile_seg.numel(),
            _ptr(out), _rows_2d(out, "out"), ctypes.c_float(scale), int(window or 0), page_size, H, G, hd, STREAM)
        return out
    _run("attention_prefill_mma", load_library("attention_mma").kp_attention_prefill_mma, 
        _ptr(q), _rows_2d(q, "q"), _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(cu_rows), _ptr(seg_pos),
        _ptr(tile_seg), _ptr(tile_row0), tile_seg.numel(), _ptr(out), _rows_2d(out, "out"), ctypes.c_float(scale),
        int(window or 0), page_size, H, G, hd, STREAM)
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
            accumulate: bool = False, swiglu: bool = False, split: bool = True) -> torch.Tensor:
    """out = a @ w.T (+ bias) on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory); with
    ``swiglu`` ``w`` holds gate rows then up rows and out = silu(gate) * up.  With ``split`` a product of 17 to
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
    epi = _skinny_epilogue(out, accumulate, swiglu)
    lib = load_library("gemm_tc")
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
                accumulate: bool = False, swiglu: bool = False) -> torch.Tensor:
    """out = a @ w.T (+ bias) for up to 64 rows of bfloat16 ``a``.  With
    ``swiglu`` ``w`` holds gate rows then up rows and out = silu(gate) * up."""
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
        epi = EPI_SWIGLU
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
    if USE_STREAM and stream_fits(K, swiglu) and stream_pays(N, K) and M <= STREAM_MAX_M:
        lib = load_library("gemm_stream")
        _run("gemm_stream", lib.kp_gemm_stream, _ptr(a), _rows_2d(a, "a"), _ptr(w), _rows_2d(w, "w"), _ptr(bias), _ptr(out),
             _rows_2d(out, "out"), M, N, K, epi, STREAM, tag=f" {N}x{K}", work=_gemm_work(M, N, K, a, w, out))
        return out
    lib = load_library("gemm_skinny")
    _run("gemm_skinny", lib.kp_gemm_skinny, _ptr(a), _rows_2d(a, "a"), _ptr(w), _rows_2d(w, "w"), _ptr(bias), _ptr(out),
         _rows_2d(out, "out"), M, N, K, epi, STREAM, tag=f" {N}x{K}", work=_gemm_work(M, N, K, a, w, out))
    return out
