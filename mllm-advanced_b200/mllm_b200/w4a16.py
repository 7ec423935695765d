"""Python mirror of the W4A16 entry points of the C ABI (include/mllmb200.h): asymmetric int4 weights with an
fp32 scale and zero term per group of 32, per-block int8 activations, fp16 output
(reference project: KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk, mllm/Backends/Arm/Kernels/kai_linear.cpp:680-951)."""
import ctypes as C

import numpy as np

from .binding import _check, _stream_ptr, lib


def prepack_size(n, k, has_bias):
    out = C.c_size_t()
    _check(lib().mllmb200_w4a16_prepack_size(n, k, int(bool(has_bias)), C.byref(out)), "w4a16_prepack_size")
    return out.value


def quant_prepack(w, bias=None):
    """fp32 [N,K] weights (+ optional fp32 [N] bias) -> W4A16 pre-pack blob (numpy uint8, host)."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    blob = np.empty(prepack_size(n, k, b is not None), np.uint8)
    _check(lib().mllmb200_w4a16_quant_prepack(w.ctypes.data, None if b is None else b.ctypes.data, n, k,
                                              blob.ctypes.data), "w4a16_quant_prepack")
    return blob


def blob_info(blob):
    n, k, hb = C.c_int(), C.c_int(), C.c_int()
    _check(lib().mllmb200_w4a16_blob_info(blob.ctypes.data, blob.size, C.byref(n), C.byref(k), C.byref(hb)),
           "w4a16_blob_info")
    return n.value, k.value, hb.value


def blob_sections(blob):
    """Views of the nibble, scale, zero and bias sections of a host blob."""
    n, k, hb = blob_info(blob)
    a, b, z, c = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
    _check(lib().mllmb200_w4a16_blob_offsets(n, k, hb, C.byref(a), C.byref(b), C.byref(z), C.byref(c)),
           "w4a16_blob_offsets")
    ns, nb = (k + 1) // 2, (k + 31) // 32
    nib = blob[a.value:a.value + n * ns].reshape(n, ns)
    sc = blob[b.value:b.value + n * nb * 4].view(np.float32).reshape(n, nb)
    zr = blob[z.value:z.value + n * nb * 4].view(np.float32).reshape(n, nb)
    bias = blob[c.value:c.value + n * 4].view(np.float32) if hb else None
    return nib, sc, zr, bias


def tiled_size(n, k):
    out = C.c_size_t()
    _check(lib().mllmb200_w4a16_tiled_size(n, k, C.byref(out)), "w4a16_tiled_size")
    return out.value


def workspace_size(m, k, n):
    out = C.c_size_t()
    _check(lib().mllmb200_w4a16_workspace_size(m, k, n, C.byref(out)), "w4a16_workspace_size")
    return out.value


class W4A16Weights:
    """Device-resident W4A16 weights of one linear in the tile layout (optionally a row shard)."""

    def __init__(self, tiled, n, k, has_bias, row_begin=0, n_total=None):
        self.tiled, self.n, self.k, self.has_bias = tiled, n, k, has_bias
        self.row_begin, self.n_total = row_begin, n if n_total is None else n_total

    @staticmethod
    def from_blob(blob, device="cuda", row_begin=0, row_count=None, stream=None):
        import torch
        n, k, hb = blob_info(blob)
        row_count = n - row_begin if row_count is None else row_count
        blob_dev = torch.from_numpy(blob).to(device)
        tiled = torch.empty(tiled_size(row_count, k), dtype=torch.uint8, device=device)
        _check(lib().mllmb200_w4a16_repack_device(blob_dev.data_ptr(), n, k, hb, row_begin, row_count,
                                                  tiled.data_ptr(), _stream_ptr(stream)), "w4a16_repack_device")
        torch.cuda.current_stream().synchronize()  # blob_dev is released when this returns
        return W4A16Weights(tiled, row_count, k, hb, row_begin, n)


KERNEL_AUTO, KERNEL_DP4A, KERNEL_TC_F16 = 0, 2, 4


def linear_forward(x, weights, out=None, workspace=None, stream=None, kernel=KERNEL_AUTO, pdl=False):
    """fp16 y = W4A16 linear of x (torch float32 or float16 [M,K] on the GPU, last dim contiguous).
    kernel: KERNEL_AUTO (tensor cores for M >= 128, or M >= 32 with N >= 8192; else dp4a), KERNEL_DP4A, KERNEL_TC_F16 (M >= 8)."""
    import torch
    assert x.is_cuda and x.dtype in (torch.float32, torch.float16) and x.dim() == 2 and x.stride(1) == 1
    m, k = x.shape
    assert k == weights.k
    if out is None:
        out = torch.empty((m, weights.n), dtype=torch.float16, device=x.device)
    if workspace is None:
        workspace = torch.empty(workspace_size(m, k, weights.n), dtype=torch.uint8, device=x.device)
    _check(lib().mllmb200_w4a16_linear_forward_ex(x.data_ptr(), 1 if x.dtype == torch.float16 else 0,
                                                  weights.tiled.data_ptr(), out.data_ptr(), workspace.data_ptr(), m, k,
                                                  weights.n, x.stride(0), out.stride(0), kernel | (0x100 if pdl else 0),
                                                  _stream_ptr(stream)),
           "w4a16_linear_forward")
    return out


def linear_forward_grouped(x, weights_list, outs=None, workspace=None, stream=None, pdl=False):
    """Several W4A16 linears on the same activations in one call (one launch for M <= 4 on small matrices)."""
    import torch
    assert x.is_cuda and x.dtype in (torch.float32, torch.float16) and x.dim() == 2 and x.stride(1) == 1
    m, k = x.shape
    cnt = len(weights_list)
    assert 1 <= cnt <= 4 and all(w.k == k for w in weights_list)
    if outs is None:
        outs = [torch.empty((m, w.n), dtype=torch.float16, device=x.device) for w in weights_list]
    if workspace is None:
        workspace = torch.empty(max(workspace_size(m, k, w.n) for w in weights_list), dtype=torch.uint8, device=x.device)
    tiled = (C.c_void_p * cnt)(*[w.tiled.data_ptr() for w in weights_list])
    ys = (C.c_void_p * cnt)(*[o.data_ptr() for o in outs])
    ns = (C.c_int * cnt)(*[w.n for w in weights_list])
    ldy = (C.c_int * cnt)(*[o.stride(0) for o in outs])
    _check(lib().mllmb200_w4a16_linear_forward_grouped(x.data_ptr(), 1 if x.dtype == torch.float16 else 0, m, k,
                                                       x.stride(0), cnt, tiled, ys, ns, ldy, workspace.data_ptr(),
                                                       0x100 if pdl else 0, _stream_ptr(stream)),
           "w4a16_linear_forward_grouped")
    return outs
