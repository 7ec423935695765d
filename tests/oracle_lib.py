"""ctypes bindings of the CPU checkers under oracle/_ref/ (test infrastructure only).

`oracle`  : the plain-C restatement (oracle/w4a32_oracle.c), always present after
            `make -C oracle`.
`kai_ref` : the reference's own scalar W4A32 code compiled in place
            (oracle/kai_ref_wrap.cpp); present only where the reference tree was at build time.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")


def _build_if_missing():
    if not os.path.exists(os.path.join(REF_DIR, "liboracle.so")):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")])


def load_oracle():
    _build_if_missing()
    lib = C.CDLL(os.path.join(REF_DIR, "liboracle.so"))
    lib.oracle_cast_bf16_f32.argtypes = [C.c_float, C.c_int]
    lib.oracle_cast_bf16_f32.restype = C.c_uint16
    lib.oracle_cast_f32_bf16.argtypes = [C.c_uint16]
    lib.oracle_cast_f32_bf16.restype = C.c_float
    lib.oracle_cast_f16_f32.argtypes = [C.c_float]
    lib.oracle_cast_f16_f32.restype = C.c_uint16
    lib.oracle_cast_f32_f16.argtypes = [C.c_uint16]
    lib.oracle_cast_f32_f16.restype = C.c_float
    lib.oracle_quant_nxk_qs4c32_f32.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, _f32p, _u8p, _u16p, C.c_int]
    lib.oracle_quant_nxk_qs4c32_f32.restype = None
    lib.oracle_quant_qa8dx_f32.argtypes = [C.c_size_t, C.c_size_t, _f32p, _i8p]
    lib.oracle_quant_qa8dx_f32.restype = None
    lib.oracle_matmul_f32_qa8dx_qs4c32.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, _i8p, _u8p,
                                                   _u16p, C.c_int, C.c_void_p, _f32p, C.c_float, C.c_float]
    lib.oracle_matmul_f32_qa8dx_qs4c32.restype = None
    lib.oracle_fill_uniform_random.argtypes = [C.c_size_t, _f32p, C.c_uint]
    lib.oracle_fill_uniform_random.restype = None
    lib.oracle_num_threads.restype = C.c_int
    return lib


def load_kai_ref():
    path = os.path.join(REF_DIR, "libkai_ref.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    lib.kairef_cast_bf16_f32.argtypes = [C.c_float]
    lib.kairef_cast_bf16_f32.restype = C.c_uint16
    lib.kairef_cast_f32_bf16.argtypes = [C.c_uint16]
    lib.kairef_cast_f32_bf16.restype = C.c_float
    lib.kairef_fill_uniform_random.argtypes = [C.c_size_t, C.c_size_t, _f32p, C.c_size_t]
    lib.kairef_fill_uniform_random.restype = None
    lib.kairef_quant_nxk_qs4c32_f32.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, _f32p, _u8p, _u16p]
    lib.kairef_quant_nxk_qs4c32_f32.restype = None
    lib.kairef_quant_qa8dx_f32.argtypes = [C.c_size_t, C.c_size_t, _f32p, _i8p]
    lib.kairef_quant_qa8dx_f32.restype = None
    lib.kairef_matmul.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, _i8p, _u8p, _u16p, _f32p]
    lib.kairef_matmul.restype = None
    return lib


FLT_MAX = float(np.finfo(np.float32).max)


class Oracle:
    """numpy-level wrapper of the C oracle."""

    def __init__(self):
        self.lib = load_oracle()

    @staticmethod
    def nblocks(k, bl=32):
        return (k + bl - 1) // bl

    def fill_uniform_random(self, count, seed):
        out = np.empty(count, np.float32)
        self.lib.oracle_fill_uniform_random(count, out, seed)
        return out

    def quant_weights(self, w, scale_mode=0):
        n, k = w.shape
        q = np.zeros((n, (k + 1) // 2), np.uint8)
        s = np.zeros((n, self.nblocks(k)), np.uint16)
        self.lib.oracle_quant_nxk_qs4c32_f32(n, k, 32, np.ascontiguousarray(w, np.float32), q, s, scale_mode)
        return q, s

    def quant_act(self, x):
        m, k = x.shape
        out = np.zeros((m, k + 8), np.int8)
        self.lib.oracle_quant_qa8dx_f32(m, k, np.ascontiguousarray(x, np.float32), out)
        return out

    def matmul(self, lhs_q, q, s, k, bias=None, scale_mode=0):
        m = lhs_q.shape[0]
        n = q.shape[0]
        y = np.zeros((m, n), np.float32)
        b = None
        if bias is not None:
            bias = np.ascontiguousarray(bias, np.float32)
            b = bias.ctypes.data_as(C.c_void_p)
        self.lib.oracle_matmul_f32_qa8dx_qs4c32(m, n, k, 32, lhs_q, q, s, scale_mode, b, y, -FLT_MAX, FLT_MAX)
        return y

    def linear(self, x, q, s, bias=None, scale_mode=0):
        x = np.ascontiguousarray(x, np.float32)
        return self.matmul(self.quant_act(x), q, s, x.shape[1], bias, scale_mode)


class OracleW4A16:
    """numpy-level wrapper of the W4A16 restatement (oracle/w4a16_oracle.c)."""

    def __init__(self):
        self.lib = lib = load_oracle()
        _i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
        lib.oracle_w4a16_quant_nxk_qai4c32_f32.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, _f32p, _u8p, _f32p,
                                                           _f32p, _i32p]
        lib.oracle_w4a16_quant_nxk_qai4c32_f32.restype = None
        lib.oracle_w4a16_quant_lhs_f32.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, _f32p, _i8p, _f32p]
        lib.oracle_w4a16_quant_lhs_f32.restype = None
        lib.oracle_w4a16_matmul.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, _i8p, _f32p, _u8p, _f32p,
                                            _f32p, C.c_void_p, _u16p, C.c_float, C.c_float]
        lib.oracle_w4a16_matmul.restype = None
        lib.oracle_w4a16_fill_uniform_random_f16.argtypes = [C.c_size_t, _u16p, C.c_uint]
        lib.oracle_w4a16_fill_uniform_random_f16.restype = None

    @staticmethod
    def nblocks(k, bl=32):
        return (k + bl - 1) // bl

    def fill_uniform_random_f16(self, count, seed):
        out = np.empty(count, np.uint16)
        self.lib.oracle_w4a16_fill_uniform_random_f16(count, out, seed)
        return out.view(np.float16)

    def quant_weights(self, w):
        """-> nibbles u8 [n, ceil(k/2)] (even k in the high half), scales f32, zeros f32, zero points i32."""
        n, k = w.shape
        nb = self.nblocks(k)
        q = np.zeros((n, (k + 1) // 2), np.uint8)
        z = np.zeros((n, nb), np.float32)
        s = np.zeros((n, nb), np.float32)
        zp = np.zeros((n, nb), np.int32)
        self.lib.oracle_w4a16_quant_nxk_qai4c32_f32(n, k, 32, np.ascontiguousarray(w, np.float32), q, z, s, zp)
        return q, s, z, zp

    def quant_act(self, x):
        m, k = x.shape
        nb = self.nblocks(k)
        a_q = np.zeros((m, nb * 32), np.int8)
        a_s = np.zeros((m, nb), np.float32)
        self.lib.oracle_w4a16_quant_lhs_f32(m, k, 32, np.ascontiguousarray(x, np.float32), a_q, a_s)
        return a_q, a_s

    def linear(self, x, q, s, z, bias=None):
        """x: fp32 or fp16 [m,k] (fp16 is widened, exactly) -> fp16 [m,n]."""
        x = np.ascontiguousarray(np.asarray(x).astype(np.float32))
        m, k = x.shape
        n = q.shape[0]
        a_q, a_s = self.quant_act(x)
        y = np.zeros((m, n), np.uint16)
        b = None
        if bias is not None:
            bias = np.ascontiguousarray(bias, np.float32)
            b = bias.ctypes.data_as(C.c_void_p)
        self.lib.oracle_w4a16_matmul(m, n, k, 32, a_q, a_s, q, s, z, b, y, -65504.0, 65504.0)
        return y.view(np.float16)
