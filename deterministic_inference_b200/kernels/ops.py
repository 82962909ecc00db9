"""Python side of the CUDA kernels: argument checks and launches.

Every function takes CUDA tensors, checks dtype, shape and contiguity on the
host, and launches the hand-written kernel on the current stream.  There is no
CPU path and no library fallback: a tensor that is not on a CUDA device raises
``KernelError``, and a missing or unbuildable library raises
``KernelBuildError``.  The one library call is the bfloat16 matrix product of
``linear`` (cuBLAS through ``torch.mm``) for shapes the package's own tcgen05
kernel does not take; the reference uses the library for every matrix product
(sid/model/qwen3.py:38).

The parts call these functions through the module (``ops.rms_norm(...)``), so a
test can substitute plain PyTorch restatements to exercise the engine's host
logic on a machine without a GPU; the package itself never does.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build


class KernelError(RuntimeError):
    pass


_STATUS = {
    -1: "unsupported dtype",
    -2: "a size this kernel refuses",
    -3: "misaligned pointer",
    -4: "kernel launch failed",
    -5: "a bounded wait inside the kernel ran out",
}

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream      # a plain integer handle, cheap
except AttributeError:                                     # pragma: no cover
    _raw_stream = None


def _stream():
    """Handle of the current CUDA stream of the current device."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, what: str, detail: str = "", kernels: int = 1):
    global launch_count
    launch_count += kernels
    if status != 0:
        raise KernelError(f"{what}: {_STATUS.get(status, status)}{(' — ' + detail) if detail else ''}")


def _need(t: torch.Tensor, name: str, dtype=None, ndim=None):
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name} must be a tensor")
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: this package has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous (shape {tuple(t.shape)}, stride {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dims, got shape {tuple(t.shape)}")


def _dt(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DT:
        raise KernelError(f"{name}: dtype {t.dtype} is not supported (float32 or bfloat16)")
    return _DT[t.dtype]


_libs: dict[str, ctypes.CDLL] = {}

# Kernels launched by this module since import (this package's own kernels plus
# the library matrix products it calls); benchmarks read differences of it.
launch_count = 0


def _launched(n: int = 1) -> None:
    global launch_count
    launch_count += n


def _lib(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        lib = build.load_library(name)
        _libs[name] = lib
    return lib


# Libraries whose kernels have bounded waits: name -> (read, clear) of its error word.
_STATUS_FUNCTIONS = {
    "gemm_bf16": ("dib_gemm_bf16_status", "dib_gemm_bf16_status_clear"),
    "gemm_bf16_large": ("dib_gemm_bf16_large_status", "dib_gemm_bf16_large_status_clear"),
    "attention_bf16": ("dib_attention_bf16_status", "dib_attention_bf16_status_clear"),
    "attention_prefill_tc": ("dib_attention_prefill_tc_status", "dib_attention_prefill_tc_status_clear"),
}
_extra_status: dict = {}


def register_kernel_status(name: str, read, clear) -> None:
    """Add the error word of a library loaded from outside this module: ``read()`` gives 0
    or the code of a wait that ran out, ``clear()`` sets it back to 0."""
    _extra_status[name] = (read, clear)


def kernel_status() -> dict:
    """The error words of the libraries with bounded waits that have been loaded: name ->
    0, or the code of a wait that ran out (the results of that launch are not valid).
    Reading them synchronises with the device."""
    out = {}
    for name, (read, _) in _STATUS_FUNCTIONS.items():
        lib = _libs.get(name)
        if lib is not None:
            out[name] = int(getattr(lib, read)())
    for name, (read, _) in _extra_status.items():
        out[name] = int(read())
    return out


def clear_kernel_status() -> None:
    """Set every error word back to 0."""
    for name, (_, clear) in _STATUS_FUNCTIONS.items():
        lib = _libs.get(name)
        if lib is not None:
            getattr(lib, clear)()
    for _, clear in _extra_status.values():
        clear()


def check_kernel_status() -> None:
    """Raise ``KernelError`` if a bounded wait inside a kernel ran out since the last check.
    The words are cleared first, so the failure is reported once and later work is judged
    on its own."""
    bad = {k: v for k, v in kernel_status().items() if v != 0}
    if bad:
        clear_kernel_status()
        raise KernelError(f"a bounded wait inside a kernel ran out (library: code): {bad}; results of "
                          "the steps since the last check are not valid")


# ---------------------------------------------------------------- deferred sums

class SplitSum:
    """A matrix that exists as ``S`` float32 partial products of a split-k matrix
    product, ``parts[s]`` of shape [rows, cols], not yet added.  The kernels that
    read a projection output (residual-add + norm, q/k norm, SiLU gate) take it as
    it is and add the partials in split order while they load, rounding the sum to
    ``dtype`` as a stored product would be; anything else gets a plain tensor from
    ``as_tensor``.  ``hidden`` handed from a block to the next may be one."""

    def __init__(self, parts: torch.Tensor, dtype: torch.dtype):
        self.parts, self.dtype = parts, dtype

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def device(self):
        return self.parts.device

    @property
    def splits(self) -> int:
        return self.parts.shape[0]

    def tensor(self) -> torch.Tensor:
        s, m, n = self.parts.shape
        out = torch.empty(m, n, dtype=self.dtype, device=self.parts.device)
        if (m * n) % 4 == 0:
            st = _lib("elementwise").dib_sum_split(_ptr(self.parts), c_int(s), c_longlong(m * n),
                                                   _ptr(out), c_longlong(m * n),
                                                   c_int(_DT[self.dtype]), _stream())
            _check(st, "sum_split")
            return out
        _launched(1)
        acc = self.parts[0].clone()
        for i in range(1, s):          # split order
            acc += self.parts[i]
        return acc.to(self.dtype)


# Rows up to which the gate of a gated feed-forward is left to the product that follows
# (``GatedSplit``).  The product then stages the partial products of its columns in shared
# memory; with more than a few rows that costs more than the separate gate kernel (B200,
# width 1,024 / 3,072: 6.2 against 7.2 us for both products at 1 row, 8.2 against 7.5 us at 8);
# and with a wide feed-forward too (width 4,096 / 12,288: a decode step of one request 5 %
# slower with it), so it is limited to feed-forwards up to GATE_IN_PRODUCT_WIDTH wide.
GATE_IN_PRODUCT_ROWS = 2
GATE_IN_PRODUCT_WIDTH = 4096


class GatedSplit:
    """silu(gate) * up that is not computed yet: the [gate | up] product exists as the
    split-k partial products ``gate_up`` (a ``SplitSum``, [rows, 2I]).  The matrix product
    that follows makes its operand from them while it loads (``linear``); anything else gets
    the tensor [rows, I] from ``tensor()`` (the gate kernel that reads partials)."""

    def __init__(self, gate_up: SplitSum):
        self.gate_up = gate_up
        self.dtype = gate_up.dtype

    @property
    def shape(self):
        rows, two_i = self.gate_up.shape
        return torch.Size((rows, two_i // 2))

    @property
    def device(self):
        return self.gate_up.device

    def tensor(self) -> torch.Tensor:
        return silu_mul(self.gate_up)


class SplitAttention:
    """The output of the split-KV decode attention before its splits are merged:
    ``part_o`` float32 [sequences, heads, splits, head_dim], ``part_lse`` [sequences, heads,
    splits], the sequences' lengths on the device and the window.  Its logical shape is
    [sequences, heads * head_dim].  The output projection merges while it loads its
    operand (``linear``); ``tensor()`` runs the merge kernel."""

    def __init__(self, part_o, part_lse, seq_lens, num_seqs: int, window: int, dtype):
        self.part_o, self.part_lse, self.seq_lens = part_o, part_lse, seq_lens
        self.num_seqs, self.window, self.dtype = num_seqs, window, dtype
        _, self.num_heads, self.max_splits, self.head_dim = part_o.shape

    @property
    def shape(self):
        return torch.Size((self.num_seqs, self.num_heads * self.head_dim))

    @property
    def device(self):
        return self.part_o.device

    def tensor(self) -> torch.Tensor:
        out = torch.empty(self.num_seqs, self.num_heads, self.head_dim, dtype=self.dtype,
                          device=self.part_o.device)
        st = _lib("attention_bf16").dib_decode_attention_merge(
            _ptr(self.part_o), _ptr(self.part_lse), _ptr(self.seq_lens), _ptr(out), c_int(self.num_seqs),
            c_int(self.max_splits), c_int(self.num_heads), c_int(self.head_dim), c_int(self.window),
            _stream())
        _check(st, "decode_attention_merge")
        return out.view(self.num_seqs, self.num_heads * self.head_dim)


class WeightedSum:
    """sum_i scale_i * term_i that is not computed yet: the outputs of mixers that run side
    by side, each a tensor, a ``SplitSum`` or a ``NormedTerm`` (an output that is RMS-normed
    with a weight of its own before it is scaled).  The norm of a float32 residual stream adds
    the terms to the stream in their order while it loads them; ``tensor()`` gives the sum
    as a float32 tensor."""

    def __init__(self, terms: list):
        if not 1 <= len(terms) <= 2:
            raise KernelError(f"a weighted sum of {len(terms)} terms has no kernel (1 or 2)")
        self.terms = [(float(a), x) for a, x in terms]
        self.dtype = torch.float32

    @property
    def shape(self):
        return self.terms[0][1].shape

    @property
    def device(self):
        return self.terms[0][1].device

    @property
    def normed(self) -> bool:
        return any(isinstance(x, NormedTerm) for _, x in self.terms)

    def tensor(self) -> torch.Tensor:
        rows, width = self.shape
        if self.normed:
            out = torch.zeros(rows, width, dtype=torch.float32, device=self.device)
            _stream_add_normed_terms(out, self.terms, None, 0.0, None)
            return out
        out = torch.empty(rows, width, dtype=torch.float32, device=self.device)
        st = _lib("stream_f32").dib_weighted_sum(c_int(len(self.terms)), *_terms_args(self.terms, 2),
                                                 _ptr(out), c_longlong(rows * width), _stream())
        _check(st, "weighted_sum")
        return out


class NormedTerm:
    """x / sqrt(mean(x^2) + eps) * weight that is not computed yet: the output of a part that is
    normed before it joins a float32 residual stream.  The stream's next norm computes it in float32
    and adds it to the stream without rounding it (``stream_rms_norm``); ``tensor()`` gives it as a
    float32 tensor.  ``x``: a tensor or a ``SplitSum``."""

    def __init__(self, x, weight: torch.Tensor, eps: float):
        self.x, self.weight, self.eps = x, weight, float(eps)
        self.dtype = torch.float32

    @property
    def shape(self):
        return self.x.shape

    @property
    def device(self):
        return self.x.device

    def tensor(self) -> torch.Tensor:
        rows, width = self.shape
        out = torch.zeros(rows, width, dtype=torch.float32, device=self.device)
        return stream_add_(out, self)


_DEFERRED = (SplitSum, GatedSplit, SplitAttention, WeightedSum, NormedTerm)


def _source_args(x):
    """(pointer, kind, splits, stride) of a kernel input that is a float32 or bfloat16
    tensor or the split-k partial products of a matrix product."""
    if isinstance(x, SplitSum):
        s, m, n = x.parts.shape
        return (_ptr(x.parts), c_int(0), c_int(s), c_longlong(m * n))
    if isinstance(x, _DEFERRED):
        x = x.tensor()
    _need(x, "x")
    return (_ptr(x), c_int(_dt(x, "x")), c_int(1), c_longlong(0))


def _terms_args(terms: list, n: int) -> list:
    """Arguments of ``n`` (source, scale) pairs; missing ones are null."""
    out = []
    for i in range(n):
        if i < len(terms):
            a, x = terms[i]
            out += [*_source_args(x), c_float(a)]
        else:
            out += [c_void_p(0), c_int(0), c_int(1), c_longlong(0), c_float(0.0)]
    return out


def _stream_add_normed_terms(stream: torch.Tensor, terms: list, weight, eps: float, out) -> None:
    """stream += sum_i a_i * n_i in place (float32), n_i a ``NormedTerm`` (x / rms(x) * its weight) or a
    plain term; with ``out`` also out = RMSNorm(stream) * weight."""
    rows, w = stream.shape
    args = []
    for i in range(2):
        if i < len(terms):
            a, x = terms[i]
            if tuple(x.shape) != (rows, w):
                raise KernelError(f"a term of shape {tuple(x.shape)} for a stream {(rows, w)}")
            if isinstance(x, NormedTerm):
                _need(x.weight, "term.weight", torch.float32, 1)
                if x.weight.shape[0] != w:
                    raise KernelError(f"a normed term's weight has {x.weight.shape[0]} elements, rows have {w}")
                args += [*_source_args(x.x), c_float(a), _ptr(x.weight), c_float(x.eps)]
            else:
                args += [*_source_args(x), c_float(a), c_void_p(0), c_float(0.0)]
        else:
            args += [c_void_p(0), c_int(0), c_int(1), c_longlong(0), c_float(0.0), c_void_p(0), c_float(0.0)]
    st = _lib("stream_f32").dib_stream_norm_normed_terms(
        _ptr(stream), c_int(len(terms)), *args, _ptr(weight), _ptr(out),
        c_int(_DT[out.dtype] if out is not None else 0), c_int(rows), c_int(w), c_float(eps), _stream())
    _check(st, "stream_rms_norm(normed terms)", f"row width {w}")


def as_tensor(x):
    """A plain tensor, whatever ``x`` is."""
    return x.tensor() if isinstance(x, _DEFERRED) else x


def merge_heads(o):
    """Attention output [T, heads, head_dim] as the output projection's operand
    [T, heads * head_dim] (a ``SplitAttention`` has that shape already)."""
    if isinstance(o, SplitAttention):
        return o
    return o.view(o.shape[0], o.shape[1] * o.shape[2])


# ---------------------------------------------------------------- embedding

def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """out[t] = table[ids[t]]; ids int32 [T], table [V, H]."""
    _need(ids, "ids", torch.int32, 1)
    _need(table, "table", None, 2)
    out = torch.empty(ids.shape[0], table.shape[1], dtype=table.dtype, device=table.device)
    st = _lib("elementwise").dib_embedding(
        _ptr(table), _ptr(ids), _ptr(out), c_int(ids.shape[0]), c_int(table.shape[1]),
        c_int(table.shape[0]), c_int(_dt(table, "table")), _stream())
    _check(st, "embedding")
    return out


def patch_token_ids(input_ids: torch.Tensor, patch_dst: torch.Tensor, patch_src: torch.Tensor,
                    prev_tokens: torch.Tensor) -> None:
    """input_ids[patch_dst[i]] = prev_tokens[patch_src[i]] where patch_dst[i] >= 0 (all
    int32): the tokens the previous step sampled become inputs on the device."""
    for t, n in ((input_ids, "input_ids"), (patch_dst, "patch_dst"), (patch_src, "patch_src"),
                 (prev_tokens, "prev_tokens")):
        _need(t, n, torch.int32, 1)
    st = _lib("elementwise").dib_patch_ids(_ptr(input_ids), _ptr(patch_dst), _ptr(patch_src),
                                           _ptr(prev_tokens), c_int(patch_dst.shape[0]),
                                           c_int(input_ids.shape[0]), c_int(prev_tokens.shape[0]),
                                           _stream())
    _check(st, "patch_token_ids")


# ---------------------------------------------------------------- norms

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * weight over the last dim; weight float32."""
    x = as_tensor(x)
    _need(x, "x")
    _need(weight, "weight", torch.float32, 1)
    h = x.shape[-1]
    if weight.shape[0] != h:
        raise KernelError(f"rms_norm: weight has {weight.shape[0]} elements, rows have {h}")
    out = torch.empty_like(x)
    rows = x.numel() // h if h else 0
    st = _lib("elementwise").dib_rms_norm(_ptr(x), _ptr(weight), _ptr(out), c_int(rows), c_int(h),
                                          c_float(eps), c_int(_dt(x, "x")), _stream())
    _check(st, "rms_norm", f"row width {h}")
    return out


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """In place: residual += x (stored rounded); x = rms_norm(unrounded sum).
    Returns (x, residual).  ``x`` may be a ``SplitSum``; the norm is then written to
    a new tensor."""
    if isinstance(x, SplitSum):
        _need(residual, "residual", x.dtype, 2)
        _need(weight, "weight", torch.float32, 1)
        s_, rows, h = x.parts.shape
        if tuple(residual.shape) != (rows, h) or weight.shape[0] != h:
            raise KernelError(f"add_rms_norm: x {(rows, h)} vs residual {tuple(residual.shape)}, "
                              f"weight {weight.shape[0]}")
        if h % 4 == 0 and h <= (16384 if rows <= 128 else 4096):
            out = torch.empty(rows, h, dtype=x.dtype, device=x.device)
            st = _lib("elementwise").dib_add_rms_norm_split(
                _ptr(x.parts), c_int(s_), c_longlong(rows * h), _ptr(residual), _ptr(weight),
                _ptr(out), c_int(rows), c_int(h), c_float(eps), c_int(_DT[x.dtype]), _stream())
            _check(st, "add_rms_norm(split)", f"row width {h}")
            return out, residual
        x = x.tensor()
    _need(x, "x")
    _need(residual, "residual", x.dtype)
    _need(weight, "weight", torch.float32, 1)
    if x.shape != residual.shape:
        raise KernelError(f"add_rms_norm: x {tuple(x.shape)} vs residual {tuple(residual.shape)}")
    h = x.shape[-1]
    if weight.shape[0] != h:
        raise KernelError(f"add_rms_norm: weight has {weight.shape[0]} elements, rows have {h}")
    rows = x.numel() // h if h else 0
    st = _lib("elementwise").dib_add_rms_norm(_ptr(x), _ptr(residual), _ptr(weight), c_int(rows),
                                              c_int(h), c_float(eps), c_int(_dt(x, "x")), _stream())
    _check(st, "add_rms_norm", f"row width {h}")
    return x, residual


# ------------------------------------------------ q/k norm + rotary + cache

def qk_norm_rope_cache(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                       q_norm_weight, k_norm_weight, eps: float, cos_sin, positions: torch.Tensor,
                       kv_cache, slot_mapping, page_size: int) -> torch.Tensor:
    """From the fused projection row [q heads | k heads | v heads] of each token:
    per-head RMSNorm of q and k (when a weight is given), rotate-half rotation by
    the token's position (when a table [max_pos, rotary_dim] = [cos | sin] is
    given), q to the returned tensor [T, Hq, D], k and v into the token's slot of
    the paged cache [pages, 2, Hkv, page_size, D] (when a cache is given;
    slot = page * page_size + offset, negative = skip)."""
    parts = None
    if isinstance(qkv, SplitSum):
        if head_dim in (64, 128, 256) and (cos_sin is None or cos_sin.shape[1] == head_dim):
            parts = qkv
        else:
            qkv = qkv.tensor()
    if parts is None:
        _need(qkv, "qkv", None, 2)
    t, got_width = qkv.shape
    act_dtype, device = qkv.dtype, qkv.device
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if got_width != width:
        raise KernelError(f"qkv has width {got_width}, expected {width}")
    _need(positions, "positions", torch.int32, 1)
    for w, n in ((q_norm_weight, "q_norm_weight"), (k_norm_weight, "k_norm_weight")):
        if w is not None:
            _need(w, n, torch.float32, 1)
            if w.shape[0] != head_dim:
                raise KernelError(f"{n} has {w.shape[0]} elements, head_dim is {head_dim}")
    rotary_dim, max_pos = 0, 0
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32, 2)
        max_pos, rotary_dim = cos_sin.shape
    num_pages = 0
    if kv_cache is not None:
        _need(kv_cache, "kv_cache", act_dtype, 5)
        _need(slot_mapping, "slot_mapping", torch.int32, 1)
        if tuple(kv_cache.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
            raise KernelError(f"kv_cache shape {tuple(kv_cache.shape)} does not match "
                              f"[pages, 2, {num_kv_heads}, {page_size}, {head_dim}]")
        num_pages = kv_cache.shape[0]
    q = torch.empty(t, num_heads, head_dim, dtype=act_dtype, device=device)
    if parts is not None:
        st = _lib("elementwise").dib_qk_norm_rope_cache_split(
            c_void_p(0), _ptr(parts.parts), c_int(parts.splits), c_longlong(t * width), _ptr(q),
            _ptr(kv_cache), _ptr(q_norm_weight), _ptr(k_norm_weight), c_float(eps), _ptr(cos_sin),
            c_int(rotary_dim), c_int(max_pos), _ptr(positions), _ptr(slot_mapping), c_int(t),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size),
            c_longlong(num_pages), c_int(_DT[parts.dtype]), _stream())
        _check(st, "qk_norm_rope_cache(split)", f"head_dim {head_dim}")
        return q
    st = _lib("elementwise").dib_qk_norm_rope_cache(
        _ptr(qkv), _ptr(q), _ptr(kv_cache), _ptr(q_norm_weight), _ptr(k_norm_weight), c_float(eps),
        _ptr(cos_sin), c_int(rotary_dim), c_int(max_pos), _ptr(positions), _ptr(slot_mapping),
        c_int(t), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size),
        c_longlong(num_pages), c_int(_dt(qkv, "qkv")), _stream())
    _check(st, "qk_norm_rope_cache", f"head_dim {head_dim}, rotary_dim {rotary_dim}")
    return q


def qkv_project(x: torch.Tensor, w_qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                q_norm_weight, k_norm_weight, eps: float, cos_sin, positions: torch.Tensor, kv_cache,
                slot_mapping, page_size: int) -> torch.Tensor:
    """The fused q/k/v projection of the step's tokens followed by ``qk_norm_rope_cache``: returns
    q [T, Hq, D], with k and v in the tokens' cache slots.  Many bfloat16 rows of heads of 128
    run as ONE kernel when the package's many-rows product is in use (``large_products`` "own"
    or "auto"): the product's epilogue norms, rotates and writes the cache, with the bits of
    the two kernels."""
    x = as_tensor(x)
    if x.dtype == torch.bfloat16 and x.is_cuda and head_dim == 128 and kv_cache is not None \
            and (cos_sin is None or cos_sin.shape[1] == head_dim):
        from . import gemm_bf16
        q = gemm_bf16.qkv_large(x, w_qkv, num_heads, num_kv_heads, q_norm_weight, k_norm_weight, eps,
                                cos_sin, positions, kv_cache, slot_mapping, page_size)
        if q is not None:
            return q
    return qk_norm_rope_cache(linear(x, w_qkv), num_heads, num_kv_heads, head_dim, q_norm_weight,
                              k_norm_weight, eps, cos_sin, positions, kv_cache, slot_mapping, page_size)


def reshape_and_cache(k: torch.Tensor, v: torch.Tensor, kv_cache: torch.Tensor,
                      slot_mapping: torch.Tensor) -> None:
    """k, v [T, Hkv, D] into their slots of the paged cache (negative slot: skip)."""
    _need(k, "k", None, 3)
    _need(v, "v", k.dtype, 3)
    _need(kv_cache, "kv_cache", k.dtype, 5)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    t, hkv, d = k.shape
    if v.shape != k.shape or kv_cache.shape[1] != 2 or kv_cache.shape[2] != hkv or kv_cache.shape[4] != d:
        raise KernelError(f"reshape_and_cache: k {tuple(k.shape)}, v {tuple(v.shape)}, "
                          f"cache {tuple(kv_cache.shape)}")
    st = _lib("elementwise").dib_reshape_and_cache(
        _ptr(k), _ptr(v), _ptr(kv_cache), _ptr(slot_mapping), c_int(t), c_int(hkv), c_int(d),
        c_int(kv_cache.shape[3]), c_longlong(kv_cache.shape[0]), c_int(_dt(k, "k")), _stream())
    _check(st, "reshape_and_cache")


# ---------------------------------------------------------------- attention

def paged_attention(q: torch.Tensor, kv_cache: torch.Tensor, meta, scale: float,
                    window=None, defer: bool = False):
    """Causal attention of every token of the step over its sequence's keys in the
    paged cache.  q [T, Hq, D]; kv_cache [pages, 2, Hkv, page_size, D]; ``meta``
    is the step's attention metadata for this cache's group (``AttentionMeta``:
    block_table [B, max_blocks], token_seq [T], positions [T], cu_q_lens [B+1],
    seq_lens [B], host copies of the lengths, number of leading decode
    sequences).  A query at position p sees keys max(0, p-window+1) .. p.
    ``defer``: a step of one-token sequences only may come back as a ``SplitAttention``
    (its splits not yet merged) for the matrix product that follows to merge."""
    _need(q, "q", None, 3)
    _need(kv_cache, "kv_cache", q.dtype, 5)
    t, hq, d = q.shape
    _, two, hkv, page_size, d2 = kv_cache.shape
    if two != 2 or d2 != d or hq % hkv:
        raise KernelError(f"paged_attention: q {tuple(q.shape)} vs cache {tuple(kv_cache.shape)}")
    _need(meta.block_table, "block_table", torch.int32, 2)
    _need(meta.token_seq, "token_seq", torch.int32, 1)
    _need(meta.positions, "positions", torch.int32, 1)
    out = torch.empty_like(q)
    win = int(window) if window else 0
    if q.dtype == torch.bfloat16:
        from . import attention_bf16
        if attention_bf16.supports(hq, hkv, d, page_size):
            deferred = attention_bf16.run(q, out, kv_cache, meta, scale, win, defer)
            return deferred if deferred is not None else out
    st = _lib("attention_generic").dib_paged_attention_generic(
        _ptr(q), _ptr(out), _ptr(kv_cache), _ptr(meta.block_table), c_int(meta.block_table.shape[1]),
        _ptr(meta.token_seq), _ptr(meta.positions), c_int(t), c_int(hq), c_int(hkv), c_int(d),
        c_int(page_size), c_float(scale), c_int(win), c_int(_dt(q, "q")), _stream())
    _check(st, "paged_attention", f"head_dim {d} (at most 256), heads {hq}/{hkv}")
    return out


# ---------------------------------------------------------------- feed-forward

def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] = [gate | up] -> silu(gate) * up, [T, I]."""
    if isinstance(gate_up, SplitSum):
        s_, t, two_i = gate_up.parts.shape
        if two_i % 8 == 0:
            out = torch.empty(t, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
            st = _lib("elementwise").dib_silu_mul_split(
                _ptr(gate_up.parts), c_int(s_), c_longlong(t * two_i), _ptr(out), c_int(t),
                c_int(two_i // 2), c_int(_DT[gate_up.dtype]), _stream())
            _check(st, "silu_mul(split)")
            return out
        gate_up = gate_up.tensor()
    _need(gate_up, "gate_up", None, 2)
    t, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError(f"silu_mul: width {two_i} is odd")
    out = torch.empty(t, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    st = _lib("elementwise").dib_silu_mul(_ptr(gate_up), _ptr(out), c_int(t), c_int(two_i // 2),
                                          c_int(_dt(gate_up, "gate_up")), _stream())
    _check(st, "silu_mul")
    return out


def gather_rows(x: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """out[r] = x[index[r]]; index int32."""
    if isinstance(x, NormedTerm):          # a norm works row by row: gather first
        return NormedTerm(gather_rows(x.x, index), x.weight, x.eps)
    if isinstance(x, WeightedSum) and x.normed:
        return WeightedSum([(a, gather_rows(term, index)) for a, term in x.terms])
    x = as_tensor(x)
    _need(x, "x", None, 2)
    _need(index, "index", torch.int32, 1)
    out = torch.empty(index.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
    st = _lib("elementwise").dib_gather_rows(_ptr(x), _ptr(index), _ptr(out), c_int(index.shape[0]),
                                             c_int(x.shape[1]), c_int(x.shape[0]),
                                             c_int(_dt(x, "x")), _stream())
    _check(st, "gather_rows")
    return out


# ---------------------------------------------------------------- matrix product

def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """y = x @ weight^T; x [M, K], weight [N, K] (checkpoint layout), no bias.

    float32: the package's own CUDA-core kernel (plain FMA, no TF32, fixed k
    order, so a row's bits do not depend on the batch).  bfloat16: float32
    accumulation on the tensor cores; ``out_dtype=torch.float32`` returns the
    accumulator unrounded (used for the logits).  With few rows and a split of k the
    bfloat16 product comes back as a ``SplitSum`` (see there)."""
    if isinstance(x, (GatedSplit, SplitAttention)) and weight.dtype == torch.bfloat16 \
            and tuple(x.shape)[1] == weight.shape[1]:
        from . import gemm_bf16
        y = gemm_bf16.linear_of_deferred(x, weight, out_dtype or torch.bfloat16)
        if y is not None:
            return y
    x = as_tensor(x)
    _need(x, "x", None, 2)
    _need(weight, "weight", x.dtype, 2)
    m, k = x.shape
    n, k2 = weight.shape
    if k != k2:
        raise KernelError(f"linear: x [{m}, {k}] against weight [{n}, {k2}]")
    if x.dtype == torch.float32:
        out = torch.empty(m, n, dtype=torch.float32, device=x.device)
        st = _lib("gemm_fp32").dib_gemm_fp32(_ptr(x), _ptr(weight), _ptr(out), c_int(m), c_int(n),
                                             c_int(k), _stream())
        _check(st, "linear(float32)", f"M={m} N={n} K={k}")
        return out
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: dtype {x.dtype} is not supported")
    from . import gemm_bf16
    return gemm_bf16.linear(x, weight, out_dtype or torch.bfloat16)


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor):
    """silu(x w_gate^T) * (x w_up^T), [M, I], for the concatenated weight
    [w_gate ; w_up] ([2I, K]).  With few bfloat16 rows the gate is applied in the matrix
    product's epilogue, or, when the product comes back as split-k partials, left to the
    reader (a ``GatedSplit``); otherwise this is ``silu_mul(linear(x, w_gate_up))``."""
    x = as_tensor(x)
    if x.dtype == torch.bfloat16 and x.is_cuda:
        _need(x, "x", None, 2)
        _need(w_gate_up, "w_gate_up", x.dtype, 2)
        if x.shape[1] != w_gate_up.shape[1]:
            raise KernelError(f"gated_linear: x {tuple(x.shape)} against weight {tuple(w_gate_up.shape)}")
        from . import gemm_bf16
        out = gemm_bf16.gated_linear(x, w_gate_up)
        if out is not None:
            return out
    y = linear(x, w_gate_up)
    if isinstance(y, SplitSum) and y.dtype == torch.bfloat16 and y.shape[1] % 16 == 0 \
            and y.shape[0] <= GATE_IN_PRODUCT_ROWS and y.shape[1] // 2 <= GATE_IN_PRODUCT_WIDTH:
        return GatedSplit(y)          # the gate is applied by the product that reads it
    return silu_mul(y)


# ---------------------------------------------------------------- sampling

def argmax(logits: torch.Tensor) -> torch.Tensor:
    """int32 [R]: index of the largest logit of each row, lowest index on ties."""
    _need(logits, "logits", torch.float32, 2)
    r, v = logits.shape
    out = torch.empty(r, dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    if v > 8192 and r <= 65535:
        # wide rows: one block per chunk of the row, then a second tiny kernel
        chunks = -(-v // 4096)
        sv = torch.empty(r, chunks, dtype=torch.float32, device=logits.device)
        si = torch.empty(r, chunks, dtype=torch.int32, device=logits.device)
        st = lib.dib_argmax_two_stage(_ptr(logits), _ptr(sv), _ptr(si), _ptr(out), c_int(r), c_int(v),
                                      _stream())
        _check(st, "argmax", kernels=2)
        return out
    st = lib.dib_argmax(_ptr(logits), _ptr(out), c_int(r), c_int(v), _stream())
    _check(st, "argmax")
    return out


def gumbel_sample(logits: torch.Tensor, temperatures: torch.Tensor, seeds: torch.Tensor,
                  sample_positions: torch.Tensor, keep=None, top_ks=None, top_ps=None,
                  return_thresholds: bool = False):
    """int32 [R]: rows with temperature <= 0 take the argmax; the others the
    position-seeded Gumbel-max draw from softmax(logits / temperature), restricted
    to ids with keep != 0 when a mask (uint8 [R, V]) is given.  ``top_ks`` (int64 [R],
    <= 0: off) and ``top_ps`` (float32 [R], >= 1: off): top-k / top-p applied inside the
    kernels by a probability threshold found without a sort (``return_thresholds``: also
    the int32 bits of each row's smallest kept probability, 0 where nothing is dropped)."""
    _need(logits, "logits", torch.float32, 2)
    r, v = logits.shape
    _need(temperatures, "temperatures", torch.float32, 1)
    _need(seeds, "seeds", torch.int64, 1)
    _need(sample_positions, "sample_positions", torch.int64, 1)
    if not (temperatures.shape[0] == seeds.shape[0] == sample_positions.shape[0] == r):
        raise KernelError("gumbel_sample: per-row parameter lengths differ from the number of rows")
    if keep is not None:
        _need(keep, "keep", torch.uint8, 2)
        if tuple(keep.shape) != (r, v):
            raise KernelError(f"gumbel_sample: keep {tuple(keep.shape)} vs logits {(r, v)}")
    out = torch.empty(r, dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    filtered = top_ks is not None or top_ps is not None
    if (v > 8192 or filtered) and r <= 65535:
        # a block per chunk of a row (normaliser, then scores), then the best chunk
        chunks = -(-v // 4096)
        sf = torch.empty(3, r, chunks, dtype=torch.float32, device=logits.device)
        si = torch.empty(r, chunks, dtype=torch.int32, device=logits.device)
        thresh = None
        if top_ks is not None or top_ps is not None:
            _need(top_ks, "top_ks", torch.int64, 1)
            _need(top_ps, "top_ps", torch.float32, 1)
            if top_ks.shape[0] != r or top_ps.shape[0] != r:
                raise KernelError("gumbel_sample: top_ks / top_ps lengths differ from the number of rows")
            thresh = torch.empty(r, dtype=torch.int32, device=logits.device)
            # histograms of the four radix passes: [4, r, 256] 64-bit masses, then 32-bit counts
            hist = torch.empty(4 * r * 256 * 3 // 2, dtype=torch.int64, device=logits.device)
        st = lib.dib_gumbel_sample_chunked(_ptr(logits), _ptr(temperatures), _ptr(seeds),
                                           _ptr(sample_positions), _ptr(keep), _ptr(top_ks),
                                           _ptr(top_ps), _ptr(thresh),
                                           _ptr(hist) if thresh is not None else c_void_p(0),
                                           _ptr(sf), _ptr(si), _ptr(out), c_int(r), c_int(v), _stream())
        _check(st, "gumbel_sample", kernels=3 if thresh is None else 7)
        return (out, thresh) if return_thresholds else out
    if filtered:
        raise KernelError("gumbel_sample: top_ks / top_ps with more than 65535 rows")
    st = lib.dib_gumbel_sample(_ptr(logits), _ptr(temperatures), _ptr(seeds), _ptr(sample_positions),
                               _ptr(keep), _ptr(out), c_int(r), c_int(v), _stream())
    _check(st, "gumbel_sample")
    return out


# ---------------------------------------------------------------- float32 residual stream

def embedding_positions(ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor,
                        pos_table: torch.Tensor) -> torch.Tensor:
    """float32 [T, W]: table[ids[t]] + pos_table[positions[t]]."""
    _need(ids, "ids", torch.int32, 1)
    _need(positions, "positions", torch.int32, 1)
    _need(table, "table", None, 2)
    _need(pos_table, "pos_table", table.dtype, 2)
    if table.shape[1] != pos_table.shape[1] or positions.shape[0] < ids.shape[0]:
        raise KernelError(f"embedding_positions: table {tuple(table.shape)}, positions table "
                          f"{tuple(pos_table.shape)}, {ids.shape[0]} ids, {positions.shape[0]} positions")
    out = torch.empty(ids.shape[0], table.shape[1], dtype=torch.float32, device=table.device)
    st = _lib("stream_f32").dib_embed_pos(_ptr(table), _ptr(pos_table), c_int(_dt(table, "table")), _ptr(ids),
                                          _ptr(positions), _ptr(out), c_int(ids.shape[0]),
                                          c_int(table.shape[1]), c_int(table.shape[0]),
                                          c_int(pos_table.shape[0]), _stream())
    _check(st, "embedding_positions")
    return out


def stream_rms_norm(stream: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype,
                    add=None) -> torch.Tensor:
    """RMSNorm of the float32 residual stream [rows, W], written in ``out_dtype``; with ``add``
    (a tensor, a ``SplitSum`` or a ``WeightedSum``) the stream first takes stream += add in
    place, in float32, and the norm is that of the sum."""
    _need(stream, "stream", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    rows, w = stream.shape
    if weight.shape[0] != w:
        raise KernelError(f"stream_rms_norm: weight has {weight.shape[0]} elements, rows have {w}")
    if isinstance(add, NormedTerm):
        out = torch.empty(rows, w, dtype=out_dtype, device=stream.device)
        stream_add_(stream, add, norm_weight=weight, norm_eps=eps, out=out)
        return out
    if isinstance(add, WeightedSum) and add.normed:
        out = torch.empty(rows, w, dtype=out_dtype, device=stream.device)
        _stream_add_normed_terms(stream, add.terms, weight, eps, out)
        return out
    terms = []
    if add is not None:
        terms = add.terms if isinstance(add, WeightedSum) else [(1.0, add)]
        for _, x in terms:
            if tuple(x.shape) != (rows, w):
                raise KernelError(f"stream_rms_norm: a term of shape {tuple(x.shape)} for a stream {(rows, w)}")
    out = torch.empty(rows, w, dtype=out_dtype, device=stream.device)
    st = _lib("stream_f32").dib_stream_norm(_ptr(stream), c_int(len(terms)), *_terms_args(terms, 2),
                                            _ptr(weight), _ptr(out), c_int(_DT[out_dtype]), c_int(rows),
                                            c_int(w), c_float(eps), _stream())
    _check(st, "stream_rms_norm", f"row width {w}")
    return out


def stream_add_(stream: torch.Tensor, term=None, bias=None, norm_weight=None, norm_eps: float = 0.0,
                out=None) -> torch.Tensor:
    """In place, float32: stream += term (a ``NormedTerm``: computed here, never rounded) + bias (a
    float32 vector added to every row); with ``out`` also out = RMSNorm(stream) * norm_weight (no
    ``norm_weight``: out = the stream in out's type).  Returns the stream."""
    _need(stream, "stream", torch.float32, 2)
    rows, w = stream.shape
    src, wx, eps_x = (c_void_p(0), c_int(0), c_int(1), c_longlong(0)), None, 0.0
    if term is not None:
        if not isinstance(term, NormedTerm) or tuple(term.shape) != (rows, w):
            raise KernelError(f"stream_add_: a normed term of shape {(rows, w)} is needed")
        _need(term.weight, "term.weight", torch.float32, 1)
        src, wx, eps_x = _source_args(term.x), term.weight, term.eps
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != w:
            raise KernelError(f"stream_add_: bias has {bias.shape[0]} elements, rows have {w}")
    if out is not None:
        # (no norm weight: out is the stream itself in out's type, not normed)
        if norm_weight is not None:
            _need(norm_weight, "norm_weight", torch.float32, 1)
        _need(out, "out", None, 2)
    st = _lib("stream_f32").dib_stream_normed_add(
        _ptr(stream), *src, _ptr(wx), c_float(eps_x), _ptr(bias), _ptr(norm_weight), _ptr(out),
        c_int(_DT[out.dtype] if out is not None else 0), c_int(rows), c_int(w), c_float(norm_eps), _stream())
    _check(st, "stream_add_", f"row width {w}")
    return stream


def stream_read(stream: torch.Tensor, term, out_dtype) -> torch.Tensor:
    """The float32 residual stream as the next sublayer reads it: first stream += term in place (a
    ``NormedTerm`` computed in float32 and never rounded, or None), then the stream itself in
    ``out_dtype`` (float32: the stream, no copy)."""
    _need(stream, "stream", torch.float32, 2)
    if out_dtype == torch.float32:
        return stream if term is None else stream_add_(stream, term)
    out = torch.empty(stream.shape, dtype=out_dtype, device=stream.device)
    stream_add_(stream, term, out=out)
    return out


def embedding_scaled(ids: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    """float32 [T, W]: table[ids[t]] * scale."""
    _need(ids, "ids", torch.int32, 1)
    _need(table, "table", None, 2)
    out = torch.empty(ids.shape[0], table.shape[1], dtype=torch.float32, device=table.device)
    st = _lib("stream_f32").dib_embed_scale(_ptr(table), c_int(_dt(table, "table")), _ptr(ids), c_float(scale),
                                            _ptr(out), c_int(ids.shape[0]), c_int(table.shape[1]),
                                            c_int(table.shape[0]), _stream())
    _check(st, "embedding_scaled")
    return out


def limited_gate(gate_up, limit: float, alpha: float, out_dtype) -> torch.Tensor:
    """[T, 2I] = [gate | up] -> [T, I]: g = min(gate, limit), u = clamp(up, -limit, limit),
    g * sigmoid(alpha * g) * (u + 1); float32 arithmetic on the product's accumulator where it is at hand."""
    rows, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError(f"limited_gate: width {two_i} is odd")
    out = torch.empty(rows, two_i // 2, dtype=out_dtype, device=gate_up.device)
    st = _lib("stream_f32").dib_limited_gate(*_source_args(gate_up), c_float(limit), c_float(alpha), _ptr(out),
                                             c_int(_DT[out_dtype]), c_int(rows), c_int(two_i // 2), _stream())
    _check(st, "limited_gate")
    return out


def xielu(z, alpha_p: float, alpha_n: float, out_dtype) -> torch.Tensor:
    """z > 0: alpha_p z^2 + z / 2;  z <= 0: alpha_n (exp(z) - 1 - z) + z / 2; float32 arithmetic."""
    rows, w = z.shape
    out = torch.empty(rows, w, dtype=out_dtype, device=z.device)
    st = _lib("stream_f32").dib_xielu(*_source_args(z), c_float(alpha_p), c_float(alpha_n), _ptr(out),
                                      c_int(_DT[out_dtype]), c_longlong(rows * w), _stream())
    _check(st, "xielu")
    return out


def scale_(x: torch.Tensor, a: float) -> torch.Tensor:
    """x *= a in place (float32)."""
    _need(x, "x", torch.float32)
    st = _lib("stream_f32").dib_scale(_ptr(x), c_float(a), c_longlong(x.numel()), _stream())
    _check(st, "scale_")
    return x


def softcap_(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """In place: cap * tanh(logits / cap)."""
    _need(logits, "logits", torch.float32)
    st = _lib("stream_f32").dib_softcap(_ptr(logits), c_float(cap), c_longlong(logits.numel()), _stream())
    _check(st, "softcap")
    return logits


# ---------------------------------------------------------------- attention without a softmax

def qkv_bias_cache(qkv, bias, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                   kv_cache, slot_mapping, page_size: int, out_dtype) -> torch.Tensor:
    """From the projection row [q heads | k heads | v heads] of each token plus ``bias`` (float32,
    or None): q [T, Hq, D] is returned, k and v go to the token's slot of the paged cache (a page:
    keys [Hkv, page_size, D], then values [Hkv, page_size, Dv]; slot = page * page_size + offset)."""
    t, got = qkv.shape
    width = num_heads * head_dim + num_kv_heads * (head_dim + v_head_dim)
    if got != width:
        raise KernelError(f"qkv has width {got}, expected {width}")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != width:
            raise KernelError(f"qkv bias has {bias.shape[0]} elements, expected {width}")
    num_pages = 0
    if kv_cache is not None:
        _need(kv_cache, "kv_cache", out_dtype)
        _need(slot_mapping, "slot_mapping", torch.int32, 1)
        page_elems = num_kv_heads * page_size * (head_dim + v_head_dim)
        if kv_cache.numel() % page_elems or kv_cache.shape[0] != kv_cache.numel() // page_elems:
            raise KernelError(f"kv_cache shape {tuple(kv_cache.shape)} is not [pages, ...] of pages of "
                              f"{page_elems} elements")
        num_pages = kv_cache.shape[0]
    src = _source_args(qkv)
    q = torch.empty(t, num_heads, head_dim, dtype=out_dtype, device=qkv.device)
    st = _lib("sigmoid_attention").dib_qkv_bias_cache(
        *src, _ptr(bias), _ptr(q), _ptr(kv_cache), _ptr(slot_mapping), c_int(t), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), c_int(v_head_dim), c_int(page_size), c_longlong(num_pages),
        c_int(_DT[out_dtype]), _stream())
    _check(st, "qkv_bias_cache")
    return q


# DIB200_SIGMOID_TC=0 (read once): bfloat16 steps run the float32-arithmetic kernel too
SIGMOID_ATTENTION_TC = __import__("os").environ.get("DIB200_SIGMOID_TC", "1") != "0"
# key tiles of 64 keys per CTA of a decoded token (a constant: where a token's sum over its
# keys is cut depends on its position alone)
SIGMOID_DECODE_CHUNK_TILES = 4


def sigmoid_attention_tiles(q_lens: list, tokens_per_tile: int, device, first: int = 0) -> torch.Tensor:
    """int32 [n, 3] on ``device``: (sequence, first token in the step, tokens) for every run of up
    to ``tokens_per_tile`` consecutive tokens of one sequence, in the step's token order, for the
    sequences from ``first`` on."""
    rows, start = [], 0
    for b, n in enumerate(q_lens):
        for k in range(0, n if b >= first else 0, tokens_per_tile):
            rows.append((b, start + k, min(tokens_per_tile, n - k)))
        start += n
    host = torch.tensor(rows, dtype=torch.int32).view(-1, 3)
    if torch.device(device).type == "cuda":
        return host.pin_memory().to(device, non_blocking=True)
    return host


def sigmoid_attention(q: torch.Tensor, kv_cache: torch.Tensor, meta, scale: float, head_bias,
                      v_head_dim: int, page_size: int, window=None, keep_first: int = 0) -> torch.Tensor:
    """[T, Hq, Dv]: every token's sum over its visible cached keys j of
    sigmoid(q . k_j * scale + head_bias[head]) * v_j (no normalisation over keys).  A query at
    position p sees j <= p with p - j < window or j < keep_first (no window: every j <= p)."""
    _need(q, "q", None, 3)
    _need(kv_cache, "kv_cache", q.dtype)
    t, hq, d = q.shape
    page_elems = kv_cache.numel() // kv_cache.shape[0]
    hkv, rem = divmod(page_elems, page_size * (d + v_head_dim))
    if rem or hkv < 1 or hq % hkv:
        raise KernelError(f"sigmoid_attention: q {tuple(q.shape)}, value size {v_head_dim}, pages of "
                          f"{page_elems} elements at page size {page_size}")
    if head_bias is not None:
        _need(head_bias, "head_bias", torch.float32, 1)
        if head_bias.shape[0] != hq:
            raise KernelError(f"sigmoid_attention: {head_bias.shape[0]} head biases for {hq} heads")
    _need(meta.block_table, "block_table", torch.int32, 2)
    _need(meta.token_seq, "token_seq", torch.int32, 1)
    _need(meta.positions, "positions", torch.int32, 1)
    out = torch.empty(t, hq, v_head_dim, dtype=q.dtype, device=q.device)
    win = int(window) if window else 0
    if q.dtype == torch.bfloat16 and SIGMOID_ATTENTION_TC and d % 16 == 0 and v_head_dim % 16 == 0 \
            and d <= 256 and v_head_dim <= 256 and hq // hkv <= 64 and getattr(meta, "q_lens", None) is not None \
            and getattr(meta, "num_decode", None) is not None and getattr(meta, "kv_lens", None) is not None:
        # the tensor-core form.  The step's leading one-token sequences (decoded tokens) go to
        # CTAs whose warps share a tile's keys; the others to tiles of up to 64 (token,
        # head-of-group) rows of one sequence, or of 128 where a sequence brings that many (the
        # same bits either way).
        group = hq // hkv
        n_dec = meta.num_decode if group <= 16 else 0
        rows = 128 if max(meta.q_lens[n_dec:], default=0) * group > 64 else 64
        lists = meta.scratch.get(("sigmoid_attention_tiles", group, rows))
        if lists is None:
            lists = []
            if n_dec:
                lists.append((16, sigmoid_attention_tiles(meta.q_lens[:n_dec], 1, q.device)))
            if n_dec < len(meta.q_lens):
                lists.append((rows, sigmoid_attention_tiles(meta.q_lens, rows // group, q.device, first=n_dec)))
            meta.scratch[("sigmoid_attention_tiles", group, rows)] = lists
        st = 0
        for form, tiles in lists:
            partial, max_chunks = None, 1
            if form == 16:
                # a decoded token's key tiles in chunks, a CTA each: the most tiles a token can have
                if win:
                    most = -(-int(keep_first) // 64) + win // 64 + 2
                else:
                    most = max(meta.kv_lens[:n_dec]) // 64 + 1
                max_chunks = -(-most // SIGMOID_DECODE_CHUNK_TILES)
                if max_chunks > 1:
                    partial = torch.empty(n_dec, hq, max_chunks, v_head_dim, dtype=torch.float32, device=q.device)
            st = _lib("sigmoid_attention").dib_sigmoid_attention_mma(
                _ptr(q), _ptr(out), _ptr(kv_cache), _ptr(meta.block_table), c_int(meta.block_table.shape[1]),
                _ptr(meta.positions), _ptr(meta.seq_lens), _ptr(tiles), c_int(tiles.shape[0]), _ptr(head_bias),
                c_int(hq), c_int(hkv), c_int(d), c_int(v_head_dim), c_int(page_size), c_float(scale), c_int(win),
                c_int(int(keep_first)), c_int(form), _ptr(partial), c_int(SIGMOID_DECODE_CHUNK_TILES),
                c_int(max_chunks), _stream())
            if st in (-2, -3):
                break
            _check(st, "sigmoid_attention(tensor cores)", f"heads {hq}/{hkv}, sizes {d}/{v_head_dim}")
        if st not in (-2, -3):
            return out
    st = _lib("sigmoid_attention").dib_sigmoid_attention(
        _ptr(q), _ptr(out), _ptr(kv_cache), _ptr(meta.block_table), c_int(meta.block_table.shape[1]),
        _ptr(meta.token_seq), _ptr(meta.positions), _ptr(head_bias), c_int(t), c_int(hq), c_int(hkv), c_int(d),
        c_int(v_head_dim), c_int(page_size), c_float(scale), c_int(int(window) if window else 0),
        c_int(int(keep_first)), c_int(_dt(q, "q")), _stream())
    _check(st, "sigmoid_attention", f"heads {hq}/{hkv}, sizes {d}/{v_head_dim}")
    return out


# ---------------------------------------------------------------- generalised delta rule

# DIB200_DELTA_FORM (read once): 0 / 1 force a form of the recurrence kernel for every sequence
DELTA_FORM = __import__("os").environ.get("DIB200_DELTA_FORM", "auto")


def delta_rule_forms(step) -> list:
    """[(form, first sequence, sequences)] of the recurrence's launches: the step's leading
    one-token sequences (decoded tokens) run on form 0 (a column's rows over 4 lanes: the state
    is read and written once, with the fewest CTAs), the sequences that bring prompt portions on
    form 1 (rows over 16 lanes, a quarter of the instructions per token and warp).  The forms
    order a sum's terms differently, so which one a sequence runs on depends on what IT brings,
    not on the rest of the batch."""
    n = step.num_seqs
    if DELTA_FORM in ("0", "1"):
        return [(int(DELTA_FORM), 0, n)]
    nd = min(int(getattr(step, "num_decode", 0) or 0), n)
    return [(f, a, m) for f, a, m in ((0, 0, nd), (1, nd, n - nd)) if m > 0]


def delta_rule(proj, w2_t: torch.Tensor, w0: torch.Tensor, a_bias, norm_weight: torch.Tensor,
               state: torch.Tensor, step, num_heads: int, head_dim: int, lora_rank: int,
               decay_scale: float, key_eps: float, norm_eps: float, out_dtype) -> torch.Tensor:
    """The recurrence S_t = diag(w) S_(t-1) - (a * u)(u^T S_(t-1)) + k v^T, o_t = S_t^T r per head,
    over every sequence's tokens of the step, from and to ``state`` [slots, H, D, D] (float32,
    rows ``step.state_slots``); then each head's o over its root mean square, times
    ``norm_weight``, times sigmoid(g): [T, H * D] in ``out_dtype``.  ``proj`` rows are
    [r | k | v | g | a | lora hidden]; w = exp(-decay_scale * sigmoid(w2 tanh(lora hidden) + w0)) with
    w2 given transposed (``w2_t`` [lora_rank, H * D]),
    a = sigmoid(a + a_bias), u = k / sqrt(sum(k^2) + key_eps)."""
    t, got = proj.shape
    hd = num_heads * head_dim
    if got != 5 * hd + lora_rank:
        raise KernelError(f"delta_rule: projection rows of {got}, expected {5 * hd + lora_rank}")
    _need(w2_t, "w2_t", None, 2)
    _need(w0, "w0", torch.float32, 1)
    _need(norm_weight, "norm_weight", torch.float32, 1)
    _need(state, "state", torch.float32, 4)
    if tuple(w2_t.shape) != (lora_rank, hd) or w0.shape[0] != hd or norm_weight.shape[0] != hd \
            or tuple(state.shape[1:]) != (num_heads, head_dim, head_dim):
        raise KernelError("delta_rule: a weight or the state does not fit the head count and size")
    if a_bias is not None:
        _need(a_bias, "a_bias", torch.float32, 1)
    lib = _lib("delta_rule")
    src = _source_args(proj)
    dev = state.device
    packed = torch.empty(t, num_heads, 6, head_dim, dtype=torch.float32, device=dev)
    st = lib.dib_delta_prepare(*src, _ptr(w2_t), c_int(_dt(w2_t, "w2_t")), _ptr(w0), _ptr(a_bias), _ptr(packed),
                               c_int(t), c_int(num_heads), c_int(head_dim), c_int(lora_rank),
                               c_float(decay_scale), c_float(key_eps), _stream())
    _check(st, "delta_rule(prepare)", f"heads {num_heads} of {head_dim}, rank {lora_rank}")
    o = torch.empty(t, num_heads, head_dim, dtype=torch.float32, device=dev)
    for form, first, count in delta_rule_forms(step):
        st = lib.dib_delta_recurrence(_ptr(packed), _ptr(state), c_longlong(num_heads * head_dim * head_dim),
                                      _ptr(o), c_void_p(step.cu_q_lens.data_ptr() + 4 * first),
                                      c_void_p(step.state_slots.data_ptr() + 4 * first), c_int(count),
                                      c_int(num_heads), c_int(head_dim), c_int(head_dim), c_int(form), _stream())
        _check(st, "delta_rule(recurrence)", f"heads of {head_dim} (at most 256)")
    out = torch.empty(t, hd, dtype=out_dtype, device=dev)
    st = lib.dib_delta_output(_ptr(o), *src, _ptr(norm_weight), _ptr(out), c_int(_DT[out_dtype]), c_int(t),
                              c_int(num_heads), c_int(head_dim), c_int(lora_rank), c_float(norm_eps), _stream())
    _check(st, "delta_rule(output)")
    return out




# ---------------------------------------------------------------- gated delta rule

def gated_delta_rule(proj, conv_weight: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                     norm_weight: torch.Tensor, state: torch.Tensor, step, num_heads: int, num_kv_heads: int,
                     head_dim: int, v_head_dim: int, taps: int, key_eps: float, norm_eps: float,
                     out_dtype) -> torch.Tensor:
    """The gated delta rule over every sequence's tokens of the step: [T, H * E] in ``out_dtype``.
    ``proj`` rows are [q: G * D | k: G * D | v: H * E | g: H * E | b: H | a: H | padding].  q, k and v pass
    a causal convolution per channel (``conv_weight`` float32 [2 G D + H E, taps], the last tap the
    current token's; the inputs before the step's first token come from the state's tail) and silu;
    q and k become unit vectors per head (``key_eps`` inside the root), q times D^(-1/2); beta =
    sigmoid(b), decay = exp(-exp(a_log) * softplus(a + dt_bias)); per head S <- decay S,
    u = beta (v - S^T k), S <- S + k u^T, o = S^T q; then o over its root mean square (``norm_eps``),
    times ``norm_weight`` [E], times silu(g).  ``state`` float32 [slots, H D E + (taps - 1) channels]:
    the heads' states, then the convolutions' last taps - 1 inputs (rows ``step.state_slots``)."""
    t, width = proj.shape
    h, g, d, e = num_heads, num_kv_heads, head_dim, v_head_dim
    chan = 2 * g * d + h * e
    if width < chan + h * e + 2 * h:
        raise KernelError(f"gated_delta_rule: projection rows of {width}, expected at least {chan + h * e + 2 * h}")
    _need(conv_weight, "conv_weight", torch.float32, 2)
    _need(a_log, "a_log", torch.float32, 1)
    _need(dt_bias, "dt_bias", torch.float32, 1)
    _need(norm_weight, "norm_weight", torch.float32, 1)
    _need(state, "state", torch.float32, 2)
    if tuple(conv_weight.shape) != (chan, taps) or a_log.shape[0] != h or dt_bias.shape[0] != h \
            or norm_weight.shape[0] != e or state.shape[1] != h * d * e + (taps - 1) * chan or h % g:
        raise KernelError("gated_delta_rule: a weight or the state does not fit the head counts and sizes")
    lib = _lib("delta_rule")
    src = _source_args(proj)
    dev = state.device
    slot_stride, tail_at = state.shape[1], h * d * e
    packed = torch.empty(t, h, 5 * d + e, dtype=torch.float32, device=dev)
    st = lib.dib_gated_delta_prepare(*src, c_longlong(width), _ptr(conv_weight), _ptr(a_log), _ptr(dt_bias),
                                     _ptr(state), c_longlong(slot_stride), c_longlong(tail_at), _ptr(step.token_seq),
                                     _ptr(step.cu_q_lens), _ptr(step.state_slots), _ptr(packed), c_int(t), c_int(h),
                                     c_int(g), c_int(d), c_int(e), c_int(taps), c_float(key_eps), _stream())
    _check(st, "gated_delta_rule(prepare)", f"heads {h}/{g} of {d}/{e}, {taps} taps")
    o = torch.empty(t, h, e, dtype=torch.float32, device=dev)
    for form, first, count in delta_rule_forms(step):
        st = lib.dib_delta_recurrence(_ptr(packed), _ptr(state), c_longlong(slot_stride), _ptr(o),
                                      c_void_p(step.cu_q_lens.data_ptr() + 4 * first),
                                      c_void_p(step.state_slots.data_ptr() + 4 * first), c_int(count),
                                      c_int(h), c_int(d), c_int(e), c_int(form), _stream())
        _check(st, "gated_delta_rule(recurrence)", f"heads of {d}/{e} (at most 256)")
    out = torch.empty(t, h * e, dtype=out_dtype, device=dev)
    st = lib.dib_gated_delta_output(_ptr(o), *src, c_longlong(width), _ptr(norm_weight), _ptr(out),
                                    c_int(_DT[out_dtype]), _ptr(state), c_longlong(slot_stride), c_longlong(tail_at),
                                    _ptr(step.cu_q_lens), _ptr(step.state_slots), c_int(t), c_int(step.num_seqs),
                                    c_int(h), c_int(g), c_int(d), c_int(e), c_int(taps), c_float(norm_eps), _stream())
    _check(st, "gated_delta_rule(output)", kernels=2 if taps > 1 else 1)
    return out


# ---------------------------------------------------------------- state-space recurrence, a scalar decay per head

def state_space(proj, conv_weight: torch.Tensor, conv_bias, a_log: torch.Tensor, dt_bias: torch.Tensor,
                d_skip: torch.Tensor, norm_weight: torch.Tensor, state: torch.Tensor, step, num_heads: int,
                head_dim: int, state_dim: int, groups: int, norm_groups: int, taps: int, norm_eps: float,
                out_dtype) -> torch.Tensor:
    """A state-space recurrence with a scalar decay per head over every sequence's tokens of the step:
    [T, H * P] in ``out_dtype``.  ``proj`` rows are [z: H P | x: H P | B: G N | C: G N | dt: H | padding].
    x, B and C together pass a causal convolution per channel (``conv_weight`` float32 [H P + 2 G N, taps],
    the last tap the current token's; the inputs before the step's first token come from the state's tail),
    ``conv_bias`` and silu; dt = softplus(dt + dt_bias); per head h (B and C of group h // (H / G)) with S
    [N, P] from zero: S <- exp(-exp(a_log[h]) dt) S + dt B x^T, y = S^T C + d_skip[h] x.  Then y * silu(z),
    RMS-normed in ``norm_groups`` equal parts (``norm_eps``), times ``norm_weight`` [H P].  ``state`` float32
    [slots, H N P + (taps - 1) channels]: the heads' states, then the convolution's last taps - 1 inputs
    (rows ``step.state_slots``)."""
    t, width = proj.shape
    h, p, n, g = num_heads, head_dim, state_dim, groups
    inner, chan = h * p, h * p + 2 * g * n
    if width < inner + chan + h:
        raise KernelError(f"state_space: projection rows of {width}, expected at least {inner + chan + h}")
    _need(conv_weight, "conv_weight", torch.float32, 2)
    for name, v, size in (("a_log", a_log, h), ("dt_bias", dt_bias, h), ("d_skip", d_skip, h),
                          ("norm_weight", norm_weight, inner)):
        _need(v, name, torch.float32, 1)
        if v.shape[0] != size:
            raise KernelError(f"state_space: {name} has {v.shape[0]} elements, expected {size}")
    if conv_bias is not None:
        _need(conv_bias, "conv_bias", torch.float32, 1)
    _need(state, "state", torch.float32, 2)
    if tuple(conv_weight.shape) != (chan, taps) or (conv_bias is not None and conv_bias.shape[0] != chan) \
            or state.shape[1] != h * n * p + (taps - 1) * chan or h % g or inner % norm_groups:
        raise KernelError("state_space: a weight or the state does not fit the head counts and sizes")
    lib = _lib("state_space")
    src = _source_args(proj)
    dev = state.device
    slot_stride, tail_at = state.shape[1], h * n * p
    xbc = torch.empty(t, chan, dtype=torch.float32, device=dev)
    dtv = torch.empty(t, h, 2, dtype=torch.float32, device=dev)
    st = lib.dib_ssm_prepare(*src, c_longlong(width), _ptr(conv_weight), _ptr(conv_bias), _ptr(a_log), _ptr(dt_bias),
                             _ptr(state), c_longlong(slot_stride), c_longlong(tail_at), _ptr(step.token_seq),
                             _ptr(step.cu_q_lens), _ptr(step.state_slots), _ptr(xbc), _ptr(dtv), c_int(t), c_int(h),
                             c_int(g), c_int(n), c_int(p), c_int(taps), _stream())
    _check(st, "state_space(prepare)", f"{h} heads of {p} in {g} groups, state {n}, {taps} taps")
    y = torch.empty(t, inner, dtype=torch.float32, device=dev)
    st = lib.dib_ssm_recurrence(_ptr(xbc), _ptr(dtv), _ptr(d_skip), _ptr(state), c_longlong(slot_stride), _ptr(y),
                                _ptr(step.cu_q_lens), _ptr(step.state_slots), c_int(step.num_seqs), c_int(h),
                                c_int(g), c_int(n), c_int(p), _stream())
    _check(st, "state_space(recurrence)", f"state {n} (at most 512)")
    out = torch.empty(t, inner, dtype=out_dtype, device=dev)
    st = lib.dib_ssm_output(_ptr(y), *src, c_longlong(width), _ptr(norm_weight), _ptr(out), c_int(_DT[out_dtype]),
                            _ptr(state), c_longlong(slot_stride), c_longlong(tail_at), _ptr(step.cu_q_lens),
                            _ptr(step.state_slots), c_int(t), c_int(step.num_seqs), c_int(h), c_int(g), c_int(n),
                            c_int(p), c_int(norm_groups), c_int(taps), c_float(norm_eps), _stream())
    _check(st, "state_space(output)", kernels=2 if taps > 1 else 1)
    return out


# ---------------------------------------------------------------- gated linear recurrent unit

def gated_linear_recurrence(proj, bias: torch.Tensor, conv_weight: torch.Tensor, conv_bias: torch.Tensor,
                            gates: torch.Tensor, gate_bias: torch.Tensor, neg_rate: torch.Tensor,
                            state: torch.Tensor, step, width: int, blocks: int, taps: int, out_dtype) -> torch.Tensor:
    """[T, C] in ``out_dtype``: S_t * gelu_tanh(y_t) of the recurrent unit over every sequence's tokens
    of the step.  ``proj`` rows are [y: C | x: C], ``bias`` float32 [2 C] is added to them.  u = the
    causal convolution of x per channel (``conv_weight`` float32 [C, taps], the last tap the current
    token's, plus ``conv_bias``; the inputs before the step's first token come from the state's tail).
    In each of the ``blocks`` equal parts of u: r = sigmoid(u_b R_b + c_b), i = sigmoid(u_b I_b + d_b)
    with ``gates`` float32 [2, blocks, in, out] = (R, I) and ``gate_bias`` [2, C]; a = exp(r *
    neg_rate), S_t = a S_(t-1) + sqrt(1 - a^2) * i * u.  ``state`` float32 [slots, taps * C]: S, then the
    convolution's last taps - 1 inputs (rows ``step.state_slots``)."""
    t, got = proj.shape
    c = int(width)
    per = c // blocks
    for v, name, shape in ((bias, "bias", (2 * c,)), (conv_weight, "conv_weight", (c, taps)),
                           (conv_bias, "conv_bias", (c,)), (gates, "gates", (2, blocks, per, per)),
                           (gate_bias, "gate_bias", (2, c)), (neg_rate, "neg_rate", (c,))):
        _need(v, name, torch.float32)
        if tuple(v.shape) != shape:
            raise KernelError(f"gated_linear_recurrence: {name} of shape {tuple(v.shape)}, expected {shape}")
    _need(state, "state", torch.float32, 2)
    if got != 2 * c or state.shape[1] != taps * c or c % blocks:
        raise KernelError(f"gated_linear_recurrence: rows of {got} and state rows of {state.shape[1]} for "
                          f"{c} channels and {taps} taps")
    lib = _lib("linear_recurrence")
    src = _source_args(proj)
    dev = state.device
    u = torch.empty(t, c, dtype=torch.float32, device=dev)
    st = lib.dib_glr_conv(*src, _ptr(bias), _ptr(conv_weight), _ptr(conv_bias), _ptr(state), _ptr(step.token_seq),
                          _ptr(step.cu_q_lens), _ptr(step.state_slots), _ptr(u), c_int(t), c_int(c), c_int(taps),
                          _stream())
    _check(st, "gated_linear_recurrence(convolution)", f"{c} channels, {taps} taps")
    decay_in = torch.empty(2, t, c, dtype=torch.float32, device=dev)
    st = lib.dib_glr_gates(_ptr(u), _ptr(gates), _ptr(gate_bias), _ptr(neg_rate), _ptr(decay_in), c_int(t), c_int(c),
                           c_int(blocks), _stream())
    _check(st, "gated_linear_recurrence(gates)", f"{c} channels in {blocks} blocks")
    out = torch.empty(t, c, dtype=out_dtype, device=dev)
    st = lib.dib_glr_scan(_ptr(decay_in), *src, _ptr(bias), _ptr(state), _ptr(step.cu_q_lens), _ptr(step.state_slots),
                          _ptr(out), c_int(_DT[out_dtype]), c_int(step.num_seqs), c_int(t), c_int(c), c_int(taps),
                          _stream())
    _check(st, "gated_linear_recurrence(scan)")
    return out


# ---------------------------------------------------------------- routed experts

# rows of an expert's tile in the grouped products (every expert's rows are filled up to whole tiles):
# the small tile, and the large one for steps that bring an expert EXPERT_TILE_ROWS_LARGE rows on average.
# A row's bits do not depend on the tile it is computed in.
EXPERT_TILE_ROWS = 16
EXPERT_TILE_ROWS_LARGE = 64
# bfloat16 steps that bring an expert EXPERT_TILE_ROWS_TC rows on average: the sorted rows become a
# matrix of their own and both products run on the tcgen05 kernel of ``gemm_bf16_large`` (a tile of 128
# rows times its expert's matrix).  DIB200_EXPERTS_TC=0 (read once) leaves that form out.
EXPERT_TILE_ROWS_TC = 128
EXPERTS_TC = __import__("os").environ.get("DIB200_EXPERTS_TC", "1") != "0"


ROUTER_SCORES = {"sigmoid": 0, "softmax": 1}


def route_experts(logits, correction: torch.Tensor, num_experts: int, top: int, group_count: int,
                  group_keep: int, scale: float, eps: float, score: str = "sigmoid", group_top: int = 2,
                  normalize: bool = True):
    """(int32 [T, top] chosen experts, float32 [T, top] their weights).  ``logits`` [T, >= E] (a float32
    tensor or split sums; columns from E on are not the router's): s = sigmoid(logits), or (``score``
    "softmax") the softmax of the row's E logits; the choice is made on s + correction: the experts form
    ``group_count`` groups of neighbours, a group's score is the sum of its ``group_top`` (1 or 2)
    largest choice scores, the ``group_keep`` best groups stay, and of their experts the ``top`` largest
    choice scores win (ties: the lower index).  Weights: s of the chosen over their sum (+ eps), times
    ``scale``; with ``normalize`` off s times ``scale``."""
    t, row = logits.shape
    _need(correction, "correction", torch.float32, 1)
    if score not in ROUTER_SCORES or group_top not in (1, 2):
        raise KernelError(f"route_experts: score {score!r} ({sorted(ROUTER_SCORES)}) or group_top {group_top} (1, 2)")
    if correction.shape[0] != num_experts or row < num_experts or num_experts % group_count \
            or not 1 <= group_keep <= group_count or not 1 <= top <= group_keep * (num_experts // group_count):
        raise KernelError(f"route_experts: {num_experts} experts, rows of {row}, {group_count} groups, "
                          f"{group_keep} kept, {top} chosen")
    ids = torch.empty(t, top, dtype=torch.int32, device=logits.device)
    weights = torch.empty(t, top, dtype=torch.float32, device=logits.device)
    st = _lib("routed_experts").dib_moe_route(*_source_args(logits), c_longlong(row), _ptr(correction), _ptr(ids),
                                              _ptr(weights), c_int(t), c_int(num_experts), c_int(top),
                                              c_int(group_count), c_int(group_keep), c_float(scale), c_float(eps),
                                              c_int(ROUTER_SCORES[score]), c_int(group_top),
                                              c_int(1 if normalize else 0), _stream())
    _check(st, "route_experts", f"{num_experts} experts (at most 1024), {top} chosen (at most 32)")
    return ids, weights


def routed_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                   w_down: torch.Tensor, shared, logits, shared_gate_col: int, out_dtype) -> torch.Tensor:
    """float32 [T, W]: sum_j weights[t, j] * down_e(silu(gate_e x_t) * up_e x_t) over the chosen experts
    e = ids[t, j], in the order of j, plus (``shared`` [T, W], a tensor or split sums, given)
    sigmoid(logits[t, shared_gate_col]) * shared[t] (``shared_gate_col`` negative: plus shared[t]).  ``w_gate_up`` [E, 2F, W] (an expert's gate rows,
    then its up rows), ``w_down`` [E, W, F], both of x's type.  The (token, expert) pairs are sorted by
    expert on the device into tiles of EXPERT_TILE_ROWS (or EXPERT_TILE_ROWS_LARGE) rows of one expert; a
    row's sums run over k in an order that its tile does not change, so a token's result does not depend
    on what else is in the step."""
    _need(x, "x", None, 2)
    _need(ids, "ids", torch.int32, 2)
    _need(weights, "weights", torch.float32, 2)
    _need(w_gate_up, "w_gate_up", x.dtype, 3)
    _need(w_down, "w_down", x.dtype, 3)
    t, w = x.shape
    n_exp, two_f, w2 = w_gate_up.shape
    f = two_f // 2
    top = ids.shape[1]
    if w2 != w or tuple(w_down.shape) != (n_exp, w, f) or two_f != 2 * f or tuple(weights.shape) != (t, top) \
            or ids.shape[0] != t:
        raise KernelError(f"routed_experts: x {tuple(x.shape)}, gate/up {tuple(w_gate_up.shape)}, down "
                          f"{tuple(w_down.shape)}, ids {tuple(ids.shape)}")
    lib = _lib("routed_experts")
    dev = x.device
    pairs = t * top
    on_tc = EXPERTS_TC and x.dtype == torch.bfloat16 and pairs >= EXPERT_TILE_ROWS_TC * n_exp \
        and f % 128 == 0 and w % 256 == 0 and x.is_contiguous()
    tile = EXPERT_TILE_ROWS_TC if on_tc \
        else EXPERT_TILE_ROWS_LARGE if pairs >= EXPERT_TILE_ROWS_LARGE * n_exp else EXPERT_TILE_ROWS
    max_tiles = pairs // tile + min(n_exp, pairs) + 1
    order = torch.empty(max_tiles * tile + max_tiles + n_exp + 2, dtype=torch.int32, device=dev)
    st = lib.dib_moe_sort(_ptr(ids), c_int(pairs), c_int(n_exp), c_int(tile), c_int(max_tiles), _ptr(order), _stream())
    _check(st, "routed_experts(sort)", f"{n_exp} experts (at most 1024)")
    per_pair = torch.empty(pairs, w, dtype=torch.float32, device=dev)
    if on_tc:
        from .gemm_bf16 import _sms
        large = _lib("gemm_bf16_large")
        rows = max_tiles * tile
        tile_expert = c_void_p(order.data_ptr() + 4 * rows)
        sorted_x = torch.empty(rows, w, dtype=x.dtype, device=dev)
        st = lib.dib_moe_gather_rows(_ptr(x), _ptr(order), c_longlong(rows), c_int(top), c_int(w), _ptr(sorted_x),
                                     _stream())
        _check(st, "routed_experts(rows in the experts' order)")
        hidden = torch.empty(rows, f, dtype=x.dtype, device=dev)
        st = large.dib_gemm_bf16_large_grouped(_ptr(sorted_x), _ptr(w_gate_up), _ptr(hidden), c_int(rows), c_int(f),
                                               c_int(w), c_int(1), c_int(0), tile_expert, c_int(n_exp),
                                               c_int(_sms(dev)), _stream())
        _check(st, "routed_experts(gate and up, tcgen05)", f"rows {rows}, F {f}, W {w}")
        sorted_y = torch.empty(rows, w, dtype=torch.float32, device=dev)
        st = large.dib_gemm_bf16_large_grouped(_ptr(hidden), _ptr(w_down), _ptr(sorted_y), c_int(rows), c_int(w),
                                               c_int(f), c_int(0), c_int(1), tile_expert, c_int(n_exp),
                                               c_int(_sms(dev)), _stream())
        _check(st, "routed_experts(down, tcgen05)", f"rows {rows}, F {f}, W {w}")
        st = lib.dib_moe_scatter_rows(_ptr(sorted_y), _ptr(order), c_longlong(rows), c_int(w), _ptr(per_pair), _stream())
        _check(st, "routed_experts(rows back to their pairs)")
    else:
        hidden = torch.empty(max_tiles * tile, f, dtype=x.dtype, device=dev)
        st = lib.dib_moe_gate_up(_ptr(x), c_int(_dt(x, "x")), _ptr(order), c_int(max_tiles), c_int(tile), c_int(top),
                                 _ptr(w_gate_up), _ptr(hidden), c_int(f), c_int(w), _stream())
        _check(st, "routed_experts(gate and up)")
        st = lib.dib_moe_down(_ptr(hidden), c_int(_dt(x, "x")), _ptr(order), c_int(max_tiles), c_int(tile), _ptr(w_down),
                              _ptr(per_pair), c_int(f), c_int(w), _stream())
        _check(st, "routed_experts(down)")
    out = torch.empty(t, w, dtype=torch.float32, device=dev)
    if shared is not None:
        if tuple(shared.shape) != (t, w) or logits.shape[0] != t or logits.shape[1] <= shared_gate_col:
            raise KernelError(f"routed_experts: shared output {tuple(shared.shape)}, logits {tuple(logits.shape)}")
        sh, lg, row = _source_args(shared), _source_args(logits), logits.shape[1]
        if shared_gate_col < 0:
            shared_gate_col = -1
    else:
        sh = lg = (c_void_p(0), c_int(0), c_int(1), c_longlong(0))
        row = 0
    st = lib.dib_moe_combine(_ptr(per_pair), _ptr(weights), *sh, *lg, c_longlong(row), c_int(shared_gate_col),
                             _ptr(out), c_int(t), c_int(top), c_int(w), _stream())
    _check(st, "routed_experts(combine)")
    return out


# ---------------------------------------------------------------- softmax attention with a mask kind

MASK_KINDS = {"causal": 0, "window": 1, "chunk": 2}


def _mask_args(mask: str, size) -> tuple:
    if mask not in MASK_KINDS:
        raise KernelError(f"mask {mask!r} is not known: {sorted(MASK_KINDS)}")
    if mask != "causal" and (size is None or int(size) < 1):
        raise KernelError(f"a {mask} mask needs a positive size")
    return MASK_KINDS[mask], int(size) if mask != "causal" else 0


def sequence_tiles(q_lens: list, tokens_per_tile: int, device, first: int = 0, last=None) -> torch.Tensor:
    """int32 [n, 3] on ``device``: (sequence, first token of the tile among the sequence's new tokens,
    tokens) for every run of up to ``tokens_per_tile`` consecutive tokens of the sequences ``first`` ..
    ``last`` - 1.  The lengths may be upper bounds (a captured graph's): the kernel reads the real ones on
    the device and drops what lies beyond them."""
    rows = [(b, k, min(tokens_per_tile, q_lens[b] - k))
            for b in range(first, len(q_lens) if last is None else last)
            for k in range(0, q_lens[b], tokens_per_tile)]
    host = torch.tensor(rows, dtype=torch.int32).view(-1, 3)
    if torch.device(device).type == "cuda":
        return host.pin_memory().to(device, non_blocking=True)
    return host


def _cache_pages(kv_cache, page_elems: int, what: str) -> int:
    if kv_cache.numel() % page_elems or kv_cache.shape[0] != kv_cache.numel() // page_elems:
        raise KernelError(f"{what}: cache of shape {tuple(kv_cache.shape)} is not [pages, ...] of pages of "
                          f"{page_elems} elements")
    return kv_cache.shape[0]


def attn_prepare(proj, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, q_norm_weight,
                 k_norm_weight, eps: float, freq, rotary_dim: int, positions: torch.Tensor, kv_cache,
                 slot_mapping, page_size: int, out_dtype, bias=None, norm_scope: str = "head",
                 rotary_layout: str = "halves", conv_weight=None, conv_state=None, step=None) -> torch.Tensor:
    """From each token's projection row [q heads | k heads | v heads | anything else] (plus ``bias``,
    float32 over q, k and v, when given): RMS norm of q and k (when a weight is given; ``norm_scope``
    "head": per head, weights of head_dim elements; "projection": over all of q's (k's) heads at once,
    weights of that many elements), rotation of the first ``rotary_dim`` elements of each head by the
    token's position (``rotary_layout`` "halves": element i with i + rotary_dim / 2, "pairs": element 2i
    with 2i + 1; angle = position * freq[i], float32), q [T, Hq, D] returned, k and v to the token's slot
    of the paged cache (a page: keys [Hkv, page_size, D], then values [Hkv, page_size, Dv]).
    ``conv_weight`` (float32 [q + k + v channels, taps], the last tap the current token's): each channel
    of q, k and v first passes a causal convolution over its sequence's tokens, before norm and rotation;
    the inputs before the step's first token come from ``conv_state`` (float32 [slots, (taps - 1) *
    channels], rows ``step.state_slots``, oldest input first), which is moved on by the step's tokens."""
    t, width = proj.shape
    need = num_heads * head_dim + num_kv_heads * (head_dim + v_head_dim)
    conv_args = [c_void_p(0), c_int(0), c_void_p(0), c_longlong(0), c_longlong(0), c_void_p(0), c_void_p(0),
                 c_void_p(0), c_int(0)]
    if conv_weight is not None:
        _need(conv_weight, "conv_weight", torch.float32, 2)
        taps = conv_weight.shape[1]
        if conv_weight.shape[0] != need or step is None:
            raise KernelError(f"attn_prepare: convolution weights of shape {tuple(conv_weight.shape)} for {need} "
                              f"channels (and the step's sequences are needed)")
        if taps > 1:
            _need(conv_state, "conv_state", torch.float32, 2)
            if conv_state.shape[1] != (taps - 1) * need:
                raise KernelError(f"attn_prepare: state rows of {conv_state.shape[1]} floats for {taps} taps of "
                                  f"{need} channels")
        conv_args = [_ptr(conv_weight), c_int(taps), _ptr(conv_state if taps > 1 else None),
                     c_longlong(conv_state.shape[1] if taps > 1 else 0), c_longlong(0), _ptr(step.token_seq),
                     _ptr(step.cu_q_lens), _ptr(step.state_slots), c_int(step.num_seqs)]
    if width < need:
        raise KernelError(f"attn_prepare: rows of {width} elements, q, k and v need {need}")
    if norm_scope not in ("head", "projection") or rotary_layout not in ("halves", "pairs"):
        raise KernelError(f"attn_prepare: norm scope {norm_scope!r} or rotary layout {rotary_layout!r}")
    whole = norm_scope == "projection"
    for w, n, heads in ((q_norm_weight, "q_norm_weight", num_heads), (k_norm_weight, "k_norm_weight", num_kv_heads)):
        if w is not None:
            _need(w, n, torch.float32, 1)
            if w.shape[0] != (heads * head_dim if whole else head_dim):
                raise KernelError(f"{n} has {w.shape[0]} elements for {heads} heads of {head_dim} "
                                  f"(norm over the {norm_scope})")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != need:
            raise KernelError(f"attn_prepare: a bias of {bias.shape[0]} elements, q, k and v have {need}")
    if freq is not None:
        _need(freq, "freq", torch.float32, 1)
        if freq.shape[0] * 2 != rotary_dim:
            raise KernelError(f"attn_prepare: {freq.shape[0]} frequencies for {rotary_dim} rotated elements")
    _need(positions, "positions", torch.int32, 1)
    num_pages = 0
    if kv_cache is not None:
        _need(kv_cache, "kv_cache", out_dtype)
        _need(slot_mapping, "slot_mapping", torch.int32, 1)
        num_pages = _cache_pages(kv_cache, num_kv_heads * page_size * (head_dim + v_head_dim), "attn_prepare")
    q = torch.empty(t, num_heads, head_dim, dtype=out_dtype, device=proj.device)
    if bias is not None or whole or rotary_layout == "pairs" or conv_weight is not None:
        # a block per token: it sees all heads of the row at once
        st = _lib("masked_attention").dib_attn_prepare_row(
            *_source_args(proj), c_longlong(width), _ptr(bias), _ptr(q), _ptr(kv_cache), _ptr(q_norm_weight),
            _ptr(k_norm_weight), c_int(1 if whole else 0), c_float(eps), _ptr(freq),
            c_int(rotary_dim if freq is not None else 0), c_int(1 if rotary_layout == "pairs" else 0), _ptr(positions),
            _ptr(slot_mapping), c_int(t), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(v_head_dim),
            c_int(page_size), c_longlong(num_pages), c_int(_DT[out_dtype]), *conv_args, _stream())
        _check(st, "attn_prepare(row)", f"heads {num_heads}/{num_kv_heads} of {head_dim}/{v_head_dim}",
               kernels=2 if conv_weight is not None and conv_weight.shape[1] > 1 else 1)
        return q
    st = _lib("masked_attention").dib_attn_prepare(
        *_source_args(proj), c_longlong(width), _ptr(q), _ptr(kv_cache), _ptr(q_norm_weight), _ptr(k_norm_weight),
        c_float(eps), _ptr(freq), c_int(rotary_dim if freq is not None else 0), _ptr(positions),
        _ptr(slot_mapping), c_int(t), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(v_head_dim),
        c_int(page_size), c_longlong(num_pages), c_int(_DT[out_dtype]), _stream())
    _check(st, "attn_prepare", f"heads {num_heads}/{num_kv_heads} of {head_dim}/{v_head_dim}")
    return q


def latent_prepare(proj, num_heads: int, plain_dim: int, rot_dim: int, rank: int, latent_norm_weight,
                   eps: float, freq, positions, kv_cache, slot_mapping, page_size: int, out_dtype) -> torch.Tensor:
    """From each token's projection row [q: heads of (plain_dim + rot_dim) | latent: rank | rotated key
    part: rot_dim]: the latent, RMS-normed with its weight, and the rotated key part go to the token's
    cache row [rank + rot_dim]; the rotated part of every query head goes to q[t, h, rank:], where q
    [T, H, rank + rot_dim] is returned with its first ``rank`` columns still to be filled (by the
    product of the head's plain part with its key map)."""
    t, width = proj.shape
    if width != num_heads * (plain_dim + rot_dim) + rank + rot_dim:
        raise KernelError(f"latent_prepare: rows of {width} elements, expected "
                          f"{num_heads * (plain_dim + rot_dim) + rank + rot_dim}")
    _need(latent_norm_weight, "latent_norm_weight", torch.float32, 1)
    _need(freq, "freq", torch.float32, 1)
    if freq.shape[0] * 2 != rot_dim or latent_norm_weight.shape[0] != rank:
        raise KernelError("latent_prepare: frequencies or norm weight of the wrong size")
    _need(positions, "positions", torch.int32, 1)
    num_pages = 0
    if kv_cache is not None:
        _need(kv_cache, "kv_cache", out_dtype)
        _need(slot_mapping, "slot_mapping", torch.int32, 1)
        num_pages = _cache_pages(kv_cache, page_size * (rank + rot_dim), "latent_prepare")
    q = torch.empty(t, num_heads, rank + rot_dim, dtype=out_dtype, device=proj.device)
    st = _lib("masked_attention").dib_latent_prepare(
        *_source_args(proj), c_longlong(width), _ptr(q), _ptr(kv_cache), _ptr(latent_norm_weight), c_float(eps),
        _ptr(freq), _ptr(positions), _ptr(slot_mapping), c_int(t), c_int(num_heads), c_int(plain_dim),
        c_int(rot_dim), c_int(rank), c_int(page_size), c_longlong(num_pages), c_int(_DT[out_dtype]), _stream())
    _check(st, "latent_prepare")
    return q


def heads_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[m, h, n] = sum_k x[m, h, k] * weight[h, k, n]: a product per head.  ``x`` [M, H, K] and
    ``out`` [M, H, N] may be views with any row and head stride (their last dimension contiguous);
    ``weight`` [H, K, N] is contiguous.  float32 accumulation, k in ascending order."""
    _need(weight, "weight", x.dtype, 3)
    h, k, n = weight.shape
    for v, name, last in ((x, "x", k), (out, "out", n)):
        if not v.is_cuda or v.dim() != 3 or v.shape[1] != h or v.shape[2] != last or v.stride(2) != 1 \
                or v.dtype != x.dtype:
            raise KernelError(f"heads_linear: {name} of shape {tuple(v.shape)}, stride {v.stride()} against "
                              f"weight {tuple(weight.shape)}")
    if out.shape[0] != x.shape[0]:
        raise KernelError("heads_linear: x and out differ in rows")
    m = x.shape[0]
    if x.dtype == torch.bfloat16 and m > HEADS_LINEAR_LIBRARY_ROWS:
        # many rows: the library's batched product, as for the other products of many rows
        _launched(2)
        out.transpose(0, 1).copy_(torch.bmm(x.transpose(0, 1), weight))
        return out
    st = _lib("masked_attention").dib_heads_linear(
        _ptr(x), c_longlong(x.stride(0)), c_longlong(x.stride(1)), _ptr(weight), _ptr(out),
        c_longlong(out.stride(0)), c_longlong(out.stride(1)), c_int(m), c_int(h), c_int(k), c_int(n),
        c_int(_dt(x, "x")), _stream())
    _check(st, "heads_linear", f"M={m} H={h} K={k} N={n}")
    return out


# DIB200_MASKED_TC=0 (read once): bfloat16 steps run the float32-arithmetic attention kernel too
MASKED_ATTENTION_TC = __import__("os").environ.get("DIB200_MASKED_TC", "1") != "0"
# DIB200_MASKED_MMA=0 (read once): only the mma.sync form of this module is left out
MASKED_ATTENTION_MMA = __import__("os").environ.get("DIB200_MASKED_MMA", "1") != "0"

# key tiles of 64 keys per CTA of a decoded token in the mma.sync form (a constant: where a token's
# sums over its keys are cut depends on its position alone)
MASKED_DECODE_CHUNK_TILES = 2

# bfloat16 rows above which ``heads_linear`` is the library's batched product (DIB200_HEADS_LINEAR_ROWS,
# read once)
HEADS_LINEAR_LIBRARY_ROWS = int(__import__("os").environ.get("DIB200_HEADS_LINEAR_ROWS", "64"))


def masked_attention(q: torch.Tensor, kv_cache: torch.Tensor, meta, scale: float, num_kv_heads: int,
                     v_head_dim: int, page_size: int, mask: str = "causal", mask_size=None, sink=None,
                     gate=None, gate_col: int = 0, values_in_keys: bool = False, keep_first: int = 0,
                     softcap=None) -> torch.Tensor:
    """[T, Hq, Dv]: softmax attention of every token of the step over the keys of its sequence in the
    paged cache that ``mask`` lets it see (a query at position p: "causal" 0 .. p; "window" p - size + 1
    .. p, and with ``keep_first`` also the keys 0 .. keep_first - 1; "chunk" floor(p / size) * size .. p).  ``sink`` float32 [Hq]: the denominator also holds
    exp(sink[h]) as one more term that brings nothing into the output and is taken as it is.  ``gate`` [T, >= gate_col + Hq * Dv] (a tensor or split
    sums): the output is multiplied by sigmoid(gate[t, gate_col + h * Dv + d]).  ``values_in_keys``: the
    cache holds keys only and a key's first Dv elements are its value.  ``softcap`` c: a score (after the
    scale) becomes c * tanh(score / c) before the softmax."""
    cap = 0.0 if softcap is None else float(softcap)
    if cap < 0.0:
        raise KernelError("masked_attention: a soft cap is positive")
    _need(q, "q", None, 3)
    _need(kv_cache, "kv_cache", q.dtype)
    t, hq, dk = q.shape
    dv_stored = 0 if values_in_keys else v_head_dim
    if hq % num_kv_heads:
        raise KernelError(f"masked_attention: {hq} heads over {num_kv_heads} key/value heads")
    _cache_pages(kv_cache, num_kv_heads * page_size * (dk + dv_stored), "masked_attention")
    kind, size = _mask_args(mask, mask_size)
    keep = int(keep_first)
    if keep < 0 or (keep and kind != 1):
        raise KernelError("masked_attention: kept first keys belong to a window mask")
    if sink is not None:
        _need(sink, "sink", torch.float32, 1)
        if sink.shape[0] != hq:
            raise KernelError(f"masked_attention: {sink.shape[0]} sinks for {hq} heads")
    gate_args, gate_row = (c_void_p(0), c_int(0), c_int(1), c_longlong(0)), 0
    if gate is not None:
        if gate.shape[0] != t or gate.shape[1] < gate_col + hq * v_head_dim:
            raise KernelError(f"masked_attention: gate of shape {tuple(gate.shape)}")
        gate_args, gate_row = _source_args(gate), gate.shape[1]
    _need(meta.block_table, "block_table", torch.int32, 2)
    _need(meta.token_seq, "token_seq", torch.int32, 1)
    _need(meta.positions, "positions", torch.int32, 1)
    out = torch.empty(t, hq, v_head_dim, dtype=q.dtype, device=q.device)
    if q.dtype == torch.bfloat16 and MASKED_ATTENTION_TC and not values_in_keys and dk == v_head_dim and not keep \
            and not cap \
            and getattr(meta, "q_lens", None) is not None and getattr(meta, "num_decode", None) is not None:
        # keys and values of one size that the tensor-core kernels of ``attention_bf16`` take: the
        # split-KV decode kernels for the step's one-token sequences, the tcgen05 kernel (heads of
        # 128) or the mma.sync kernel for prompt portions; the mask goes in as a signed size, the sink
        # into the last normalisation; the gate is a kernel of its own behind them
        from . import attention_bf16
        if attention_bf16.supports(hq, num_kv_heads, dk, page_size):
            cache5 = kv_cache.view(kv_cache.shape[0], 2, num_kv_heads, page_size, dk)
            attention_bf16.run(q, out, cache5, meta, scale, {0: 0, 1: size, 2: -size}[kind], False, sink)
            if gate is not None:
                st = _lib("masked_attention").dib_sigmoid_gate_(
                    _ptr(out), *gate_args, c_longlong(gate_row), c_longlong(gate_col), c_int(t),
                    c_int(hq * v_head_dim), c_int(_dt(q, "q")), _stream())
                _check(st, "sigmoid_gate_")
            return out
    group = hq // num_kv_heads
    if q.dtype == torch.bfloat16 and MASKED_ATTENTION_TC and MASKED_ATTENTION_MMA and dk % 16 == 0 and v_head_dim % 16 == 0 \
            and v_head_dim <= 256 and group <= 128 and getattr(meta, "q_lens", None) is not None \
            and getattr(meta, "num_decode", None) is not None and getattr(meta, "kv_lens", None) is not None:
        # the mma.sync form for every other bfloat16 shape of sizes that are multiples of 16: the
        # step's leading one-token sequences on tiles of one token whose keys are cut into chunks,
        # a CTA each; prompt portions on tiles of 64 or 128 (token, head-of-group) rows
        def smem_of(rows):
            return 2 * ((rows + 128) * (dk + 8) + (0 if values_in_keys else 128 * (v_head_dim + 8)))
        n_dec = meta.num_decode
        rows = 128 if (group > 64 or max(meta.q_lens[n_dec:], default=0) * group > 64) else 64
        if smem_of(rows) > 224 * 1024 and group <= 64:
            rows = 64
        dec_rows = 64 if group <= 64 else 128
        if smem_of(rows) <= 224 * 1024 and smem_of(dec_rows) <= 224 * 1024:
            key = ("masked_attention_tiles", group, rows)
            lists = meta.scratch.get(key)
            if lists is None:
                lists = []
                if n_dec:
                    lists.append((dec_rows, True, sequence_tiles(meta.q_lens, 1, q.device, last=n_dec)))
                if n_dec < len(meta.q_lens):
                    lists.append((rows, False, sequence_tiles(meta.q_lens, rows // group, q.device, first=n_dec)))
                meta.scratch[key] = lists
            for form_rows, decoded, tiles in lists:
                part_o = part_ml = None
                max_chunks = 1
                if decoded:
                    # the most key tiles a decoded token can have
                    most = (size // 64 + 2 + -(-keep // 64)) if kind else (max(meta.kv_lens[:n_dec]) // 64 + 1)
                    max_chunks = -(-most // MASKED_DECODE_CHUNK_TILES)
                    if max_chunks > 1:
                        part_o = torch.empty(n_dec, hq, max_chunks, v_head_dim, dtype=torch.float32, device=q.device)
                        part_ml = torch.empty(n_dec, hq, max_chunks, 2, dtype=torch.float32, device=q.device)
                st = _lib("masked_attention").dib_masked_attention_mma(
                    _ptr(q), _ptr(out), _ptr(kv_cache), _ptr(meta.block_table), c_int(meta.block_table.shape[1]),
                    _ptr(meta.positions), _ptr(meta.seq_lens), _ptr(meta.cu_q_lens), _ptr(tiles),
                    c_int(tiles.shape[0]), _ptr(sink),
                    c_int(hq), c_int(num_kv_heads), c_int(dk), c_int(v_head_dim), c_int(dv_stored),
                    c_int(page_size), c_float(scale), c_int(kind), c_int(size), c_int(keep), *gate_args,
                    c_longlong(gate_row), c_longlong(gate_col), c_int(form_rows), _ptr(part_o), _ptr(part_ml),
                    c_int(MASKED_DECODE_CHUNK_TILES), c_int(max_chunks), c_int(n_dec), c_float(cap), _stream())
                _check(st, "masked_attention(tensor cores)", f"heads {hq}/{num_kv_heads}, sizes {dk}/{v_head_dim}",
                       kernels=2 if part_o is not None else 1)
            return out
    st = _lib("masked_attention").dib_masked_attention(
        _ptr(q), _ptr(out), _ptr(kv_cache), _ptr(meta.block_table), c_int(meta.block_table.shape[1]),
        _ptr(meta.token_seq), _ptr(meta.positions), c_int(t), c_int(hq), c_int(num_kv_heads), c_int(dk),
        c_int(v_head_dim), c_int(dv_stored), c_int(page_size), c_float(scale), c_int(kind), c_int(size), c_int(keep),
        _ptr(sink), *gate_args, c_longlong(gate_row), c_longlong(gate_col), c_int(_dt(q, "q")), c_float(cap),
        _stream())
    _check(st, "masked_attention", f"heads {hq}/{num_kv_heads}, sizes {dk}/{v_head_dim}")
    return out
