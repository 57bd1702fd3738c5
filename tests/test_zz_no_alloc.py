"""The allocation-free attention entry point, called through its exported C
symbol, against the ordinary entry point.

It is for callers that cannot ask the CUDA allocator for memory (a real-time
loop, a host with a fixed memory budget, a plug-in whose host owns the
allocator): the partial results live in a fixed array inside the library instead
of a buffer the caller brings.  This file is collected last on purpose: should it
fail, a run that stops at the first failure has run everything else already.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(n, nh, nkv, hd, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n, nh, hd, generator=g).to(dtype)
    pages = (n + 63) // 64
    order = np.random.default_rng(seed).permutation(pages + 3)[:pages]
    kc = torch.randn(pages + 3, nkv, 64, hd, generator=g).to(dtype)
    vc = torch.randn(pages + 3, nkv, 64, hd, generator=g).to(dtype)
    bt = torch.full((1, (pages + 7) // 8 * 8), -1, dtype=torch.int32)
    bt[0, :pages] = torch.from_numpy(order.astype(np.int32))
    pos = torch.arange(n, dtype=torch.int32)
    seq = torch.zeros(n, dtype=torch.int32)
    return [t.to(DEV) for t in (q, kc, vc, pos, seq, bt)]


def _call_noalloc(lib, q, kc, vc, pos, seq, bt, window, scale, max_chunks, row0=0, n_rows=None,
                  out=None):
    n, nh, hd = q.shape
    if out is None:
        out = torch.zeros_like(q)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.jb_attention_noalloc(
        p(q), p(kc), p(vc), 0 if q.dtype == torch.float32 else 1, p(pos), p(seq), p(bt),
        bt.shape[1], p(out), row0, n if n_rows is None else n_rows, nh, kc.shape[1], hd, window,
        ctypes.c_float(scale), max_chunks, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_noalloc_attention_equals_the_ordinary_entry_point():
    from janas_b200.csrc import ops
    lib = ops.lib()
    lib.jb_attention_noalloc_error.restype = ctypes.c_char_p
    chunk = ops.attention_chunk()
    cases = [(300, 8, 2, 128, torch.bfloat16, 0), (200, 6, 2, 32, torch.float32, 50)]
    for round_ in range(2):                       # two calls in a row share the fixed array
        for i, (n, nh, nkv, hd, dtype, window) in enumerate(cases):
            q, kc, vc, pos, seq, bt = _inputs(n, nh, nkv, hd, dtype, seed=10 * round_ + i)
            mc = (n - 1) // chunk + 1
            if window:
                mc = min(mc, (window - 1) // chunk + 2)
            scale = 1 / math.sqrt(hd)
            want = ops.attention(q, kc, vc, pos, seq, bt, window, scale, mc)
            out = torch.zeros_like(q)
            torch.cuda.synchronize()
            # what this process has taken from the device, as its allocator sees it (the
            # device-wide figure would also move with other users of the GPU)
            held_before = torch.cuda.memory_reserved()
            rc, got = _call_noalloc(lib, q, kc, vc, pos, seq, bt, window, scale, mc, out=out)
            assert rc == 0, lib.jb_attention_noalloc_error()
            torch.cuda.synchronize()
            assert torch.cuda.memory_reserved() == held_before
            # the same kernels on the same inputs: the same bits (the tests' tolerance
            # for this kernel against its plain reference is 2^-8 / 5e-6)
            assert torch.equal(got, want), (round_, i)
            assert lib.jb_attention_noalloc_error() == b""
            # the rows in two unequal parts (row0 > 0 in the second), into one output:
            # each part's partial results start at the array's beginning
            halves = torch.zeros_like(q)
            cut = n // 3
            for row0, cnt in ((0, cut), (cut, n - cut)):
                rc, _ = _call_noalloc(lib, q, kc, vc, pos, seq, bt, window, scale, mc, row0=row0,
                                      n_rows=cnt, out=halves)
                assert rc == 0, lib.jb_attention_noalloc_error()
            torch.cuda.synchronize()
            assert torch.equal(halves, want), (round_, i)


def test_noalloc_attention_refuses_what_does_not_fit():
    from janas_b200.csrc import ops
    lib = ops.lib()
    lib.jb_attention_noalloc_error.restype = ctypes.c_char_p
    lib.jb_attention_scratch.restype = ctypes.c_longlong
    n, nh, nkv, hd = 4096, 32, 8, 128
    q, kc, vc, pos, seq, bt = _inputs(64, nh, nkv, hd, torch.bfloat16, seed=3)
    # claim 4096 rows of up to 32 chunks: far more than the fixed 8 Mi floats
    assert lib.jb_attention_scratch(n, nh, hd, 32) > 8 * 1024 * 1024
    big_q = torch.zeros(n, nh, hd, dtype=torch.bfloat16, device=DEV)
    big_pos = torch.zeros(n, dtype=torch.int32, device=DEV)
    rc, out = _call_noalloc(lib, big_q, kc, vc, big_pos, big_pos, bt, 0, 0.1, 32)
    assert rc == -3
    msg = lib.jb_attention_noalloc_error().decode()
    assert "fewer rows" in msg and "8388608" in msg
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0          # nothing ran
    # the same rows in two halves fit and are accepted
    rc, _ = _call_noalloc(lib, big_q, kc, vc, big_pos, big_pos, bt, 0, 0.1, 1, row0=0, n_rows=1024)
    assert rc == 0, lib.jb_attention_noalloc_error()
    torch.cuda.synchronize()
