"""The C interface as ctypes sees it: every function of kernels.h gets its
argument and return types from the header's own text."""
import ctypes
import os
import re

import pytest

from janas_b200.csrc import ops

HEADER = os.path.join(os.path.dirname(os.path.abspath(ops.__file__)), "kernels.h")


class _Fn:
    argtypes = None
    restype = None


class _Lib:
    def __init__(self):
        self.fns = {}

    def __getattr__(self, name):
        if not name.startswith("jb_"):
            raise AttributeError(name)
        return self.fns.setdefault(name, _Fn())


def test_every_declaration_is_read():
    text = open(HEADER).read()
    lib = _Lib()
    n = ops.declare(lib, text)
    names = set(re.findall(r"\b(jb_\w+)\s*\(", re.sub(r"//[^\n]*", "", text)))
    assert n == len(names) == len(lib.fns) and n >= 20
    f = lib.fns["jb_rmsnorm"]
    assert f.restype is ctypes.c_int
    assert f.argtypes == [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                          ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    assert lib.fns["jb_attention_scratch"].restype is ctypes.c_longlong
    assert lib.fns["jb_attention_chunk"].argtypes == []
    assert lib.fns["jb_sample"].argtypes[11] is ctypes.c_longlong        # big_cap
    assert lib.fns["jb_sample"].argtypes[8] is ctypes.c_void_p           # unsigned long long *rng


def test_small_headers():
    lib = _Lib()
    assert ops.declare(lib, """
        // int jb_commented_out(int a);
        int jb_one(const float *x, unsigned long long *y, long long n,
                   cudaStream_t st);
        long long jb_two(void);
        unsigned long long jb_three(size_t n, double d, unsigned u, const int32_t *p, int32_t v);
    """) == 3
    assert lib.fns["jb_one"].argtypes == [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
                                          ctypes.c_void_p]
    assert lib.fns["jb_two"].argtypes == [] and lib.fns["jb_two"].restype is ctypes.c_longlong
    assert lib.fns["jb_three"].restype is ctypes.c_ulonglong
    assert lib.fns["jb_three"].argtypes == [ctypes.c_size_t, ctypes.c_double, ctypes.c_uint,
                                            ctypes.c_void_p, ctypes.c_int32]
    with pytest.raises(KeyError):
        ops.declare(_Lib(), "int jb_bad(short s);")      # a type the table does not know
