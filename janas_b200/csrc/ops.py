"""The kernels as Python functions over CUDA tensors.

This module loads the compiled library (building it at the first call) and
checks every argument before handing raw pointers to it.  There is no CPU
fallback and no library model code behind these functions: without a GPU, or
when the library cannot be built or loaded, they raise.

Conventions: the residual stream and every matrix product's output are
float32.  A product's output is a stack ``[S, n, m]`` of S partial sums whose
sum over S is the result (S = 1 unless the product was split over k); the
kernels that consume a product add the partial sums in the order 0 .. S-1.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional, Tuple

import torch

from . import build

PAGE = 64  # positions per cache page; common.cuh has the same number

_DT = {torch.float32: 0, torch.bfloat16: 1}
_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    pass


_C_TYPES = {"int": ctypes.c_int, "int32_t": ctypes.c_int32, "unsigned": ctypes.c_uint,
            "long long": ctypes.c_longlong, "unsigned long long": ctypes.c_ulonglong,
            "float": ctypes.c_float, "double": ctypes.c_double, "size_t": ctypes.c_size_t,
            "cudaStream_t": ctypes.c_void_p}


def _c_type(decl: str, with_name: bool):
    """The ctypes type of a parameter (or return type) as kernels.h writes it."""
    decl = decl.strip()
    if "*" in decl:
        return ctypes.c_void_p
    words = [w for w in decl.split() if w != "const"]     # also folds runs of blanks
    if with_name:
        words = words[:-1]
    return _C_TYPES[" ".join(words)]


def declare(library: ctypes.CDLL, header: str) -> int:
    """Gives every function that ``header`` (the text of kernels.h) declares its
    argument and return types, so that a call converts plain Python numbers (and
    None for a null pointer) by the declared type instead of guessing it from each
    argument: a wrong guess would pass a 64-bit size as 32 bits.  Returns how many
    functions were declared; one that the header has and the library lacks, or a
    type the table above does not know, raises."""
    import re
    text = re.sub(r"//[^\n]*", "", header)
    count = 0
    for ret, name, params in re.findall(
            r"\b((?:unsigned\s+)?(?:long\s+long|int|float|double))\s+(jb_\w+)\s*\(([^)]*)\)\s*;", text):
        fn = getattr(library, name)
        params = params.strip()
        fn.argtypes = [] if params in ("", "void") else [_c_type(p, True)
                                                         for p in params.split(",")]
        fn.restype = _c_type(ret, False)
        count += 1
    return count


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build.library_path()
                try:
                    loaded = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"janas_b200: cannot load {path}: {e}") from None
                import os
                with open(os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                       "kernels.h")) as f:
                    declare(loaded, f.read())
                _lib = loaded
    return _lib


def loaded_library_path() -> Optional[str]:
    return _lib._name if _lib is not None else None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Asked on every launch, so by the short
    way when this PyTorch has it (the Stream object costs several microseconds)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    """A tensor's address for a pointer argument (None: a null pointer)."""
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    """A contiguous CUDA tensor of the given dtype (one, or a tuple of allowed ones)
    and shape (None: any size there).  Called several times per launch, so written
    for speed: dtypes are compared by identity, sizes in a plain loop."""
    try:
        ok = t.is_cuda
    except AttributeError:
        ok = False
    if not ok:
        raise KernelError(f"{name}: a CUDA tensor is needed (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None:
        td = t.dtype
        if td is not dtype and (dtype.__class__ is torch.dtype or td not in dtype):
            raise KernelError(f"{name}: dtype {td}, expected {dtype}")
    if shape is not None:
        ts = t.shape
        bad = len(shape) != len(ts)
        if not bad:
            for s, d in zip(shape, ts):
                if s is not None and s != d:
                    bad = True
                    break
        if bad:
            raise KernelError(f"{name}: shape {tuple(ts)}, expected {tuple(shape)}")


# how many of the library's kernels have been launched (for measurements)
COUNTERS = {"launches": 0}


def _check(code: int, what: str, kernels: int = 1) -> None:
    if code == 0:
        COUNTERS["launches"] += kernels
        return
    if code == -1:
        raise KernelError(f"{what}: the kernel does not take these sizes or types")
    raise KernelError(f"{what}: the launch failed (code {code})")


_FLOATS = (torch.float32, torch.bfloat16)


def stack(t: torch.Tensor) -> torch.Tensor:
    """A product's output as a stack of partial sums: [n, m] -> [1, n, m]."""
    return t if t.dim() == 3 else t.unsqueeze(0)


# ------------------------------------------------------------------ row-wise
def embed(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """x[j, :] = table[tokens[j], :] as float32."""
    _need(table, "embedding table", _FLOATS)
    _need(tokens, "tokens", torch.int32)
    n, dm = tokens.numel(), table.shape[1]
    x = torch.empty((n, dm), dtype=torch.float32, device=table.device)
    _check(lib().jb_embed(_p(table), _DT[table.dtype], _p(tokens), _p(x), n, dm, _stream()),
           "embed")
    return x


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of the rows of x (float32 [n, dm]).

    With ``delta`` (a stack [S, n, dm] of float32 partial sums) x is first
    updated in place, x += delta[0] + ... + delta[S-1].  With ``rows`` (int32
    indices) only those rows are normalized and returned, in that order."""
    _need(x, "x", torch.float32, (None, None))
    n, dm = x.shape
    _need(weight, "norm weight", _FLOATS, (dm,))
    S, stride = 0, 0
    if delta is not None:
        delta = stack(delta)
        _need(delta, "delta", torch.float32, (None, n, dm))
        S, stride = delta.shape[0], n * dm
        if rows is not None:
            raise KernelError("rmsnorm: delta and rows cannot be combined")
    n_out = n
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out = rows.numel()
    out = torch.empty((n_out, dm), dtype=out_dtype, device=x.device)
    _check(lib().jb_rmsnorm(_p(x), _p(delta), S, int(stride), _p(rows),
                            _p(weight), _DT[weight.dtype], _p(out), _DT[out_dtype], n_out, dm,
                            float(eps), _stream()), "rmsnorm")
    return out


def add_(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta[0] + ... + delta[S-1] in place (float32)."""
    _need(x, "x", torch.float32, (None, None))
    n, dm = x.shape
    delta = stack(delta)
    _need(delta, "delta", torch.float32, (None, n, dm))
    _check(lib().jb_rmsnorm(_p(x), _p(delta), delta.shape[0], int(n * dm),
                            _p(None), _p(None), 0, _p(None), 0, n, dm, float(0.0),
                            _stream()), "add")
    return x


def swiglu(gate_up: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """SiLU(gate) * up for a stack [S, n, 2 ff] whose columns are [gate | up]."""
    gate_up = stack(gate_up)
    _need(gate_up, "gate_up", torch.float32, (None, None, None))
    S, n, two_ff = gate_up.shape
    if two_ff % 2:
        raise KernelError("swiglu: the gate_up width must be even")
    ff = two_ff // 2
    out = torch.empty((n, ff), dtype=out_dtype, device=gate_up.device)
    _check(lib().jb_swiglu(_p(gate_up), S, int(n * two_ff), _p(out),
                           _DT[out_dtype], n, ff, _stream()), "swiglu")
    return out


# ------------------------------------------------------------------ position
def rope_table(inv_freq: torch.Tensor, n_pos: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of (float)p * inv_freq[i] for p < n_pos: two [n_pos, half]."""
    _need(inv_freq, "inv_freq", torch.float32)
    half = inv_freq.numel()
    cs = torch.empty((n_pos, half), dtype=torch.float32, device=inv_freq.device)
    sn = torch.empty_like(cs)
    _check(lib().jb_rope_table(_p(cs), _p(sn), _p(inv_freq), n_pos, half, _stream()),
           "rope_table")
    return cs, sn


def qk_norm_rope_append(qkv: torch.Tensor, q_weight: Optional[torch.Tensor],
                        k_weight: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                        row_pos: torch.Tensor, row_seq: torch.Tensor,
                        block_table: torch.Tensor, k_cache: Optional[torch.Tensor],
                        v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                        head_dim: int, out_dtype: torch.dtype) -> torch.Tensor:
    """Per-head RMSNorm of q and k (when weights are given), NeoX rotation by
    the rows' positions (when tables are given), K and V appended to the cache
    pages (when caches are given).  Returns q [n, heads, head_dim].

    qkv: stack [S, n, (heads + 2 kv_heads) head_dim] float32, columns
    [q | k | v].  k_cache, v_cache: [pages, kv_heads, PAGE, head_dim]."""
    qkv = stack(qkv)
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv, "qkv", torch.float32, (None, None, width))
    S, n, _ = qkv.shape
    _need(row_pos, "row_pos", torch.int32, (n,))
    _need(row_seq, "row_seq", torch.int32, (n,))
    _need(block_table, "block_table", torch.int32, (None, None))
    w_dt = 0
    if q_weight is not None:
        _need(q_weight, "q_norm weight", _FLOATS, (head_dim,))
        _need(k_weight, "k_norm weight", q_weight.dtype, (head_dim,))
        w_dt = _DT[q_weight.dtype]
    rot_half = 0
    if cos is not None:
        _need(cos, "cos", torch.float32, (None, head_dim // 2))
        _need(sin, "sin", torch.float32, tuple(cos.shape))
        rot_half = head_dim // 2
    if k_cache is not None:
        _need(k_cache, "k_cache", out_dtype, (None, num_kv_heads, PAGE, head_dim))
        _need(v_cache, "v_cache", out_dtype, tuple(k_cache.shape))
    q = torch.empty((n, num_heads, head_dim), dtype=out_dtype, device=qkv.device)
    _check(lib().jb_qk_norm_rope_append(
        _p(qkv), S, int(n * width), _p(q_weight), _p(k_weight), w_dt,
        float(eps), _p(cos), _p(sin), rot_half, _p(row_pos), _p(row_seq),
        _p(block_table), block_table.shape[1], _p(q), _p(k_cache), _p(v_cache), _DT[out_dtype],
        n, num_heads, num_kv_heads, head_dim, _stream()), "qk_norm_rope_append")
    return q


# ----------------------------------------------------------------- attention
def attention_chunk() -> int:
    return int(lib().jb_attention_chunk())


_ATT_SCRATCH_BYTES = 256 << 20
_att_scratch: dict = {}


def _scratch(device: torch.device, floats: int) -> torch.Tensor:
    buf = _att_scratch.get(device)
    if buf is None or buf.numel() < floats:
        buf = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
        _att_scratch[device] = buf
    return buf


def attention_block_positions(num_heads: int, num_kv_heads: int) -> int:
    """Positions of one sequence that a block of the tensor-core prefill kernel holds."""
    return int(lib().jb_attn_tc_block_positions(num_heads, num_kv_heads))


def attention_blocks(seq_row0, seq_pos0, seq_len, positions_per_block: int,
                     device: torch.device) -> torch.Tensor:
    """The blocks a prefill step is cut into for the tensor-core kernel: int32
    [blocks, 4] = first row, positions, the first row's position, sequence."""
    import numpy as np
    rows = []
    for i, (r0, p0, n) in enumerate(zip(seq_row0, seq_pos0, seq_len)):
        for a in range(0, int(n), positions_per_block):
            rows.append((int(r0) + a, min(positions_per_block, int(n) - a), int(p0) + a, i))
    # the runs that end latest see the most keys and take longest: they start first
    rows.sort(key=lambda b: -(b[2] + b[1]))
    return torch.from_numpy(np.asarray(rows, dtype=np.int32).reshape(-1, 4)).to(device)


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              row_pos: torch.Tensor, row_seq: torch.Tensor, block_table: torch.Tensor,
              window: int, scale: float, max_chunks: int, blocks: Optional[torch.Tensor] = None,
              decode: bool = False, force_simt: bool = False) -> torch.Tensor:
    """Causal GQA attention of every row over its sequence's cache pages.

    q: [n, heads, hd]; caches [pages, kv_heads, PAGE, hd] of q's dtype.  Row r
    is at position row_pos[r] of sequence row_seq[r], whose pages are
    block_table[row_seq[r]]; it sees positions max(0, pos + 1 - window) .. pos
    (all of 0 .. pos when window is 0).  max_chunks: the most chunks of
    ``attention_chunk()`` positions that any row's range touches.

    bfloat16 heads of 64 or 128 values run on the tensor cores when the caller
    says how the rows are arranged: ``decode=True`` (every row is the one new
    token of its sequence) or ``blocks`` (from ``attention_blocks``: runs of
    consecutive positions of one sequence).  Everything else, and float32, runs on
    the plain kernel."""
    _need(q, "q", _FLOATS, (None, None, None))
    n, nh, hd = q.shape
    _need(k_cache, "k_cache", q.dtype, (None, None, PAGE, hd))
    _need(v_cache, "v_cache", q.dtype, tuple(k_cache.shape))
    nkv = k_cache.shape[1]
    _need(row_pos, "row_pos", torch.int32, (n,))
    _need(row_seq, "row_seq", torch.int32, (n,))
    _need(block_table, "block_table", torch.int32, (None, None))
    out = torch.empty_like(q)
    L = lib()
    tc = (not force_simt and q.dtype == torch.bfloat16 and (decode or blocks is not None)
          and bool(L.jb_attn_tc_ok(nh, nkv, hd)))
    if tc and not decode:
        _need(blocks, "blocks", torch.int32, (None, 4))
        _check(L.jb_attn_tc_prefill(_p(q), _p(k_cache), _p(v_cache),
                                    int(k_cache.shape[0]), _p(blocks),
                                    blocks.shape[0], _p(block_table), block_table.shape[1],
                                    _p(out), n, nh, nkv, hd, window, float(scale),
                                    _stream()), "attention (tcgen05, prefill)")
        return out
    if tc:
        # CTAs per (token, KV head): each runs over per_cta chunks and leaves one partial
        if L.jb_attn_tc_decode_runs(nh, nkv, hd):
            parts = _decode_parts(min(n, 4096) * nkv, max_chunks, 2 * _sm_count(q.device))
        else:
            parts = max_chunks
        per_cta = (max_chunks + parts - 1) // parts
        parts = (max_chunks + per_cta - 1) // per_cta
    else:
        parts, per_cta = max_chunks, 1
    per_row = int(L.jb_attention_scratch(1, nh, hd, parts))
    rows_per_call = max(1, min(n, (_ATT_SCRATCH_BYTES // 4) // max(per_row, 1)))
    scratch = _scratch(q.device, per_row * rows_per_call)
    for row0 in range(0, n, rows_per_call):
        cnt = min(rows_per_call, n - row0)
        if tc:
            _check(L.jb_attn_tc_decode(_p(q), _p(k_cache), _p(v_cache),
                                       int(k_cache.shape[0]), _p(row_pos),
                                       _p(row_seq), _p(block_table), block_table.shape[1],
                                       _p(scratch), n, row0, cnt, nh, nkv, hd, window,
                                       float(scale), max_chunks, per_cta, _stream()),
                   "attention (tcgen05, decode)")
            _check(L.jb_attention_merge(_p(scratch), _p(row_pos), _p(out), _DT[q.dtype], row0, cnt,
                                        nh, hd, window, parts, per_cta, _stream()),
                   "attention merge")
        else:
            _check(L.jb_attention(_p(q), _p(k_cache), _p(v_cache), _DT[q.dtype], _p(row_pos),
                                  _p(row_seq), _p(block_table), block_table.shape[1], _p(scratch),
                                  _p(out), row0, cnt, nh, nkv, hd, window, float(scale),
                                  max_chunks, _stream()), "attention", kernels=2)
    return out


def attention_decode_qkv(qkv: torch.Tensor, q_weight: Optional[torch.Tensor],
                         k_weight: Optional[torch.Tensor], eps: float,
                         cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                         k_cache: torch.Tensor, v_cache: torch.Tensor, append: bool,
                         row_pos: torch.Tensor, row_seq: torch.Tensor, block_table: torch.Tensor,
                         window: int, scale: float, max_chunks: int,
                         num_heads: int) -> Optional[torch.Tensor]:
    """``qk_norm_rope_append`` and ``attention(decode=True)`` in one kernel: the
    attention's CTAs make q, and the one that holds the new position's chunk makes
    that position's key and value and writes them to the cache (``append``), from
    the q,k,v product's partial sums ``qkv`` [S, n, (heads + 2 kv_heads) 128].
    Returns the attention's output [n, heads, 128] in bfloat16, or None where the
    kernel does not take these sizes and types (bfloat16 caches, heads of 128
    values in groups of at most 16): the caller then goes the two-kernel way."""
    L = lib()
    if k_cache.dtype != torch.bfloat16 or k_cache.dim() != 4:
        return None
    nkv, hd = k_cache.shape[1], k_cache.shape[3]
    if not L.jb_attn_tc_decode_runs(num_heads, nkv, hd):
        return None
    qkv = stack(qkv)
    width = (num_heads + 2 * nkv) * hd
    _need(qkv, "qkv", torch.float32, (None, None, width))
    S, n, _ = qkv.shape
    _need(k_cache, "k_cache", torch.bfloat16, (None, nkv, PAGE, hd))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _need(row_pos, "row_pos", torch.int32, (n,))
    _need(row_seq, "row_seq", torch.int32, (n,))
    _need(block_table, "block_table", torch.int32, (None, None))
    w_dt = 0
    if q_weight is not None:
        _need(q_weight, "q_norm weight", _FLOATS, (hd,))
        _need(k_weight, "k_norm weight", q_weight.dtype, (hd,))
        w_dt = _DT[q_weight.dtype]
    if cos is not None:
        _need(cos, "cos", torch.float32, (None, hd // 2))
        _need(sin, "sin", torch.float32, tuple(cos.shape))
    parts = _decode_parts(min(n, 4096) * nkv, max_chunks, 2 * _sm_count(qkv.device))
    per_cta = (max_chunks + parts - 1) // parts
    parts = (max_chunks + per_cta - 1) // per_cta
    per_row = int(L.jb_attention_scratch(1, num_heads, hd, parts))
    rows_per_call = max(1, min(n, (_ATT_SCRATCH_BYTES // 4) // max(per_row, 1)))
    scratch = _scratch(qkv.device, per_row * rows_per_call)
    out = torch.empty((n, num_heads, hd), dtype=torch.bfloat16, device=qkv.device)
    for row0 in range(0, n, rows_per_call):
        cnt = min(rows_per_call, n - row0)
        code = L.jb_attn_tc_decode_qkv(
            _p(qkv), S, int(n * width), _p(q_weight), _p(k_weight), w_dt,
            float(eps), _p(cos), _p(sin), _p(k_cache), _p(v_cache), int(bool(append)),
            int(k_cache.shape[0]), _p(row_pos), _p(row_seq), _p(block_table),
            block_table.shape[1], _p(scratch), n, row0, cnt, num_heads, nkv, hd, window,
            float(scale), max_chunks, per_cta, _stream())
        if code == -1 and row0 == 0:
            return None             # an address the kernel's 16-byte loads cannot take
        _check(code, "attention (tcgen05, decode, from the product's sums)")
        _check(L.jb_attention_merge(_p(scratch), _p(row_pos), _p(out), _DT[out.dtype], row0, cnt,
                                    num_heads, hd, window, parts, per_cta, _stream()),
               "attention merge")
    return out


_SM_COUNT = {}


def _sm_count(device: torch.device) -> int:
    key = torch.device(device).index or 0
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _SM_COUNT[key]


def _decode_parts(pairs: int, chunks: int, places: int) -> int:
    """Into how many CTAs the chunks of one (token, KV head) pair are cut.  A CTA
    costs about three chunks' time to set up, and CTAs beyond the device's places
    (two per SM) come in waves: the cut that finishes first by that estimate."""
    sms = places
    best, best_t = 1, None
    for parts in range(1, chunks + 1):
        per_cta = -(-chunks // parts)
        waves = -(-(pairs * -(-chunks // per_cta)) // sms)
        t = waves * (3.0 + per_cta)
        if best_t is None or t < best_t:
            best, best_t = parts, t
    return best


def attn_tc_error() -> int:
    """0, or which bounded wait of a tensor-core attention kernel ran out since
    the last call.  Synchronizes the device."""
    return int(lib().jb_attn_tc_error())


# ------------------------------------------------------------------ products
def _tensor_core_ok(a: torch.Tensor, weight: torch.Tensor) -> bool:
    """What jb_gemm_tc_ok asks (bfloat16 rows of a multiple of 8 values, 16-byte
    aligned bases), asked here: it is on the path of every product."""
    if a.dtype is not torch.bfloat16 or weight.dtype is not torch.bfloat16:
        return False
    k = a.shape[1]
    return (a.shape[0] > 0 and weight.shape[0] > 0 and k >= 8 and k % 8 == 0
            and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


_SPLITS: dict = {}


def _splits(n: int, m: int, k: int, device=None) -> int:
    """jb_gemm_tc_splits, remembered per shape and device (it depends on nothing
    else but the device's SM count)."""
    key = (n, m, k, device)
    s = _SPLITS.get(key)
    if s is None:
        if len(_SPLITS) > 4096:
            _SPLITS.clear()
        s = _SPLITS[key] = int(lib().jb_gemm_tc_splits(n, m, k))
    return s


def linear(a: torch.Tensor, weight: torch.Tensor, force_simt: bool = False,
           whole: bool = False, splits: Optional[int] = None) -> torch.Tensor:
    """a [n, k] . weight[m, k]^T as a stack [S, n, m] of float32 partial sums.

    bfloat16 operands whose rows are a multiple of 8 long go to the tensor-core
    kernel (which may cut k into S parts); everything else (float32 on either
    side, other row lengths) goes to the plain multiply-add kernel, S = 1.
    ``whole=True`` asks for S = 1 in every case (the result itself, not parts).

    The tensor-core kernel starts fetching ``weight`` before the kernel launched
    just before it has finished; weights must therefore not be the output of that
    kernel (model weights never are)."""
    _need(a, "activations", _FLOATS, (None, None))
    _need(weight, "weight", _FLOATS, (None, a.shape[1]))
    n, k = a.shape
    m = weight.shape[0]
    L = lib()
    if not force_simt and n > 0 and _tensor_core_ok(a, weight):
        S = 1 if whole else int(splits or _splits(n, m, k, a.device.index))
        out = torch.empty((S, n, m), dtype=torch.float32, device=a.device)
        _check(L.jb_gemm_tc(_p(a), _p(weight), _p(out), n, m, k, S, _stream()), "linear (tcgen05)")
        return out
    out = torch.empty((1, n, m), dtype=torch.float32, device=a.device)
    need = int(L.jb_gemm_simt_scratch(n, m, k))
    scratch = torch.empty((need,), dtype=torch.float32, device=a.device) if need else None
    _check(L.jb_gemm_simt(_p(a), _DT[a.dtype], _p(weight), _DT[weight.dtype], _p(out), n, m,
                          k, _p(scratch), _stream()), "linear", kernels=2 if need else 1)
    return out


def linear_swiglu(a: torch.Tensor, gate_up: torch.Tensor) -> Optional[torch.Tensor]:
    """SiLU(a . gate^T) * (a . up^T) in one tensor-core kernel, for bfloat16
    a [n, k] and gate_up [2 ff, k] (rows [gate | up]); returns bfloat16 [n, ff],
    or None when the kernel does not take the operands."""
    _need(a, "activations", _FLOATS, (None, None))
    _need(gate_up, "gate_up weight", _FLOATS, (None, a.shape[1]))
    if gate_up.shape[0] % 2 or a.shape[0] == 0 or not _tensor_core_ok(a, gate_up):
        return None
    n, k = a.shape
    ff = gate_up.shape[0] // 2
    out = torch.empty((n, ff), dtype=torch.bfloat16, device=a.device)
    _check(lib().jb_gemm_tc_swiglu(_p(a), _p(gate_up), _p(out), n, ff, k, _stream()),
           "linear_swiglu (tcgen05)")
    return out


def linear_parts(n: int, m: int, k: int) -> int:
    """Into how many parts of k the tensor-core product of n rows with a weight
    [m, k] is cut when the caller leaves it open (see ``linear``)."""
    return _splits(n, m, k)


def gemm_tc_error() -> int:
    """0, or which bounded wait of a tensor-core product ran out since the last
    call (the product's output is then not valid).  Synchronizes the device."""
    return int(lib().jb_gemm_tc_error())


# ------------------------------------------------------------------ sampling
def sample(logits: torch.Tensor, out: Optional[torch.Tensor] = None,
           row_slot: Optional[torch.Tensor] = None,
           temperature: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
           top_p: Optional[torch.Tensor] = None, min_p: Optional[torch.Tensor] = None,
           rng: Optional[torch.Tensor] = None, big_keys: Optional[torch.Tensor] = None,
           big_probs: Optional[torch.Tensor] = None,
           forced: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of logits [rows, V] (float32).

    Without ``temperature`` every row takes the first index of its maximum.
    Otherwise the settings (float32 / int32 arrays) and ``rng`` (int64 array,
    the splitmix64 states) are indexed by row_slot[row]; a row whose
    temperature is 0 is still greedy and leaves its state alone."""
    _need(logits, "logits", torch.float32, (None, None))
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, (rows,))
    for t, name, dt in ((row_slot, "row_slot", torch.int32), (temperature, "temperature",
                        torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (min_p, "min_p", torch.float32),
                        (rng, "rng", torch.int64), (forced, "forced", torch.int32)):
        if t is not None:
            _need(t, name, dt)
    big_cap = 0
    if big_keys is not None:
        _need(big_keys, "big_keys", torch.int64, (None, None))
        _need(big_probs, "big_probs", torch.float32, tuple(big_keys.shape))
        if big_keys.shape[0] < rows:
            raise KernelError("sample: scratch for fewer rows than logits")
        big_cap = big_keys.shape[1]
    if temperature is not None and rng is None:
        raise KernelError("sample: temperature needs the random states")
    L = lib()
    chunk_keys = torch.empty((int(L.jb_sample_scratch(rows, V)),), dtype=torch.int64,
                             device=logits.device)
    launches = int(L.jb_sample_launches(V, int(big_cap), int(temperature is not None)))
    _check(L.jb_sample(_p(logits), rows, V, _p(row_slot), _p(temperature), _p(top_k),
                       _p(top_p), _p(min_p), _p(rng), _p(big_keys), _p(big_probs),
                       int(big_cap), _p(chunk_keys), _p(out), _p(forced), _stream()),
           "sample", kernels=launches)
    return out


def sample_small_cap() -> int:
    return int(lib().jb_sample_small_cap())
