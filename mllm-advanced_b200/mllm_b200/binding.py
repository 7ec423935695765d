import ctypes as C
import os

import numpy as np

SCALE_BF16_TRUNC, SCALE_BF16_RNE, SCALE_FP16 = 0, 1, 2
KERNEL_AUTO, KERNEL_GEMV, KERNEL_SIMT, KERNEL_TC, KERNEL_TC_F16, KERNEL_FASTEST, KERNEL_GEMV_2LAUNCH, KERNEL_STREAM_TC = 0, 1, 2, 3, 4, 5, 6, 7
KERNEL_FLAG_PDL = 0x100

_HERE = os.path.dirname(os.path.abspath(__file__))


def lib_path():
    return os.path.join(os.path.dirname(_HERE), "lib", "libmllm_b200.so")


class MllmB200Error(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        super().__init__(f"{where}: {status_str(status)} (status {status}, cuda error {lib().mllmb200_last_cuda_error()})")


_lib = None


def lib():
    """Loads libmllm_b200.so.  There is no fallback: without the CUDA library nothing here works."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: build it with mllm-advanced_b200/build.sh "
                          "(or __graft_entry__.build()); there is no CPU fallback")
    L = C.CDLL(path)
    sz_p = C.POINTER(C.c_size_t)
    int_p = C.POINTER(C.c_int)
    vp = C.c_void_p
    sig = {
        "mllmb200_status_str": ([C.c_int], C.c_char_p),
        "mllmb200_last_cuda_error": ([], C.c_int),
        "mllmb200_version": ([], C.c_int),
        "mllmb200_w4a32_prepack_size": ([C.c_int, C.c_int, C.c_int, sz_p], C.c_int),
        "mllmb200_w4a32_quant_prepack": ([vp, vp, C.c_int, C.c_int, C.c_int, vp], C.c_int),
        "mllmb200_w4a32_prepack_from_quantized": ([vp, vp, vp, C.c_int, C.c_int, C.c_int, vp], C.c_int),
        "mllmb200_w4a32_blob_info": ([vp, C.c_size_t, int_p, int_p, int_p, int_p], C.c_int),
        "mllmb200_w4a32_blob_offsets": ([C.c_int, C.c_int, C.c_int, sz_p, sz_p, sz_p], C.c_int),
        "mllmb200_w4a32_tiled_size": ([C.c_int, C.c_int, sz_p], C.c_int),
        "mllmb200_w4a32_repack_device": ([vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp], C.c_int),
        "mllmb200_w4a32_unpack_device": ([vp, C.c_int, C.c_int, vp, vp], C.c_int),
        "mllmb200_w4a32_workspace_size": ([C.c_int, C.c_int, sz_p], C.c_int),
        "mllmb200_w4a32_linear_forward": ([vp, vp, vp, vp] + [C.c_int] * 5 + [vp], C.c_int),
        "mllmb200_w4a32_linear_forward_ex": ([vp, vp, vp, vp] + [C.c_int] * 6 + [vp], C.c_int),
        "mllmb200_w4a32_linear_forward_grouped": ([vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp, vp, vp, vp, C.c_int,
                                                   vp], C.c_int),
        "mllmb200_w4a32_select_kernel": ([C.c_int, C.c_int, C.c_int], C.c_int),
        "mllmb200_w4a32_gemv_trace": ([vp, C.c_int], C.c_int),
        "mllmb200_w4a32_gemv_plan_check": ([C.c_int, C.c_int, int_p, int_p, int_p, int_p, int_p, int_p, sz_p], C.c_int),
        "mllmb200_w4a32_linear_forward_multi": ([C.c_int, vp, int_p, int_p, vp, vp, int_p, int_p, C.c_int, C.c_int, vp], C.c_int),
        "mllmb200_w4a32_quant_activations": ([vp, C.c_int, C.c_int, C.c_int, vp, vp], C.c_int),
        "mllmb200_check_device_status": ([vp], C.c_int),
        "mllmb200_selftest_wait_timeout": ([C.c_longlong, vp, vp], C.c_int),
        "mllmb200_w4a32_tp_init": ([C.c_int, C.c_int, vp, C.POINTER(vp)], C.c_int),
        "mllmb200_w4a32_tp_alloc_output": ([vp, C.c_size_t, C.POINTER(vp), vp], C.c_int),
        "mllmb200_w4a32_tp_ipc_export": ([vp, C.c_size_t, C.POINTER(vp), vp], C.c_int),
        "mllmb200_w4a32_tp_ipc_import": ([vp, vp], C.c_int),
        "mllmb200_w4a32_linear_forward_tp": ([vp, vp, vp, vp] + [C.c_int] * 6 + [vp], C.c_int),
        "mllmb200_w4a32_tp_output": ([vp, C.POINTER(vp), sz_p], C.c_int),
        "mllmb200_w4a32_tp_destroy": ([vp], None),
        "mllmb200_conv3d_w4a32_plan": ([int_p, int_p, int_p, C.c_int, int_p, int_p, sz_p], C.c_int),
        "mllmb200_conv3d_w4a32_forward": ([vp, vp, vp, vp, int_p, int_p, int_p, C.c_int, vp], C.c_int),
        "mllmb200_w4a16_prepack_size": ([C.c_int, C.c_int, C.c_int, sz_p], C.c_int),
        "mllmb200_w4a16_quant_prepack": ([vp, vp, C.c_int, C.c_int, vp], C.c_int),
        "mllmb200_w4a16_blob_info": ([vp, C.c_size_t, int_p, int_p, int_p], C.c_int),
        "mllmb200_w4a16_blob_offsets": ([C.c_int, C.c_int, C.c_int, sz_p, sz_p, sz_p, sz_p], C.c_int),
        "mllmb200_w4a16_tiled_size": ([C.c_int, C.c_int, sz_p], C.c_int),
        "mllmb200_w4a16_repack_device": ([vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp], C.c_int),
        "mllmb200_w4a16_workspace_size": ([C.c_int, C.c_int, C.c_int, sz_p], C.c_int),
        "mllmb200_w4a16_linear_forward": ([vp, C.c_int, vp, vp, vp] + [C.c_int] * 5 + [vp], C.c_int),
        "mllmb200_w4a16_linear_forward_ex": ([vp, C.c_int, vp, vp, vp] + [C.c_int] * 6 + [vp], C.c_int),
        "mllmb200_w4a16_linear_forward_grouped": ([vp] + [C.c_int] * 5 + [vp, vp, vp, vp, vp, C.c_int, vp], C.c_int),
    }
    for name, (args, res) in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = res
    _lib = L
    return L


def status_str(status):
    return lib().mllmb200_status_str(int(status)).decode()


def _check(status, where):
    if status != 0:
        raise MllmB200Error(status, where)


def prepack_size(n, k, has_bias):
    out = C.c_size_t()
    _check(lib().mllmb200_w4a32_prepack_size(n, k, int(bool(has_bias)), C.byref(out)), "prepack_size")
    return out.value


def tiled_size(n, k):
    out = C.c_size_t()
    _check(lib().mllmb200_w4a32_tiled_size(n, k, C.byref(out)), "tiled_size")
    return out.value


def workspace_size(m, k):
    out = C.c_size_t()
    _check(lib().mllmb200_w4a32_workspace_size(m, k, C.byref(out)), "workspace_size")
    return out.value


def quant_prepack(w, bias=None, scale_mode=SCALE_BF16_TRUNC):
    """fp32 [N,K] weights (+ optional fp32 [N] bias) -> pre-pack blob (numpy uint8, host)."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    blob = np.empty(prepack_size(n, k, b is not None), np.uint8)
    _check(lib().mllmb200_w4a32_quant_prepack(w.ctypes.data, None if b is None else b.ctypes.data, n, k, scale_mode,
                                              blob.ctypes.data), "quant_prepack")
    return blob


def prepack_from_quantized(nibbles, scales, n, k, bias=None, scale_mode=SCALE_BF16_TRUNC):
    nibbles = np.ascontiguousarray(nibbles, np.uint8)
    scales = np.ascontiguousarray(scales, np.uint16)
    assert nibbles.size == n * ((k + 1) // 2) and scales.size == n * ((k + 31) // 32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    blob = np.empty(prepack_size(n, k, b is not None), np.uint8)
    _check(lib().mllmb200_w4a32_prepack_from_quantized(nibbles.ctypes.data, scales.ctypes.data,
                                                       None if b is None else b.ctypes.data, n, k, scale_mode,
                                                       blob.ctypes.data), "prepack_from_quantized")
    return blob


def blob_info(blob):
    n, k, sm, hb = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    _check(lib().mllmb200_w4a32_blob_info(blob.ctypes.data, blob.size, C.byref(n), C.byref(k), C.byref(sm),
                                          C.byref(hb)), "blob_info")
    return n.value, k.value, sm.value, hb.value


def blob_sections(blob):
    """Views of the nibble, scale and bias sections of a host blob."""
    n, k, _, hb = blob_info(blob)
    a, b, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
    _check(lib().mllmb200_w4a32_blob_offsets(n, k, hb, C.byref(a), C.byref(b), C.byref(c)), "blob_offsets")
    ns, nb = (k + 1) // 2, (k + 31) // 32
    nib = blob[a.value:a.value + n * ns].reshape(n, ns)
    sc = blob[b.value:b.value + n * nb * 2].view(np.uint16).reshape(n, nb)
    bias = blob[c.value:c.value + n * 4].view(np.float32) if hb else None
    return nib, sc, bias


def _stream_ptr(stream):
    import torch
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


class W4A32Weights:
    """Device-resident weights of one linear in the tile layout (optionally a row shard)."""

    def __init__(self, tiled, n, k, scale_mode, has_bias, row_begin=0, n_total=None):
        self.tiled, self.n, self.k = tiled, n, k
        self.scale_mode, self.has_bias = scale_mode, has_bias
        self.row_begin, self.n_total = row_begin, n if n_total is None else n_total

    @staticmethod
    def from_blob(blob, device="cuda", row_begin=0, row_count=None, stream=None):
        import torch
        n, k, sm, hb = blob_info(blob)
        row_count = n - row_begin if row_count is None else row_count
        blob_dev = torch.from_numpy(blob).to(device)
        tiled = torch.empty(tiled_size(row_count, k), dtype=torch.uint8, device=device)
        _check(lib().mllmb200_w4a32_repack_device(blob_dev.data_ptr(), n, k, sm, hb, row_begin, row_count,
                                                  tiled.data_ptr(), _stream_ptr(stream)), "repack_device")
        torch.cuda.current_stream().synchronize()  # blob_dev is released when this returns
        return W4A32Weights(tiled, row_count, k, sm, hb, row_begin, n)

    def unpack(self, stream=None):
        """Tile layout -> host blob (inverse of the repack), for round-trip checks."""
        import torch
        out = torch.zeros(prepack_size(self.n, self.k, self.has_bias), dtype=torch.uint8, device=self.tiled.device)
        _check(lib().mllmb200_w4a32_unpack_device(self.tiled.data_ptr(), self.n, self.k, out.data_ptr(),
                                                  _stream_ptr(stream)), "unpack_device")
        return out.cpu().numpy()


_ws_cache = {}


def _workspace_for(m, k, device):
    """One cached workspace per device, grown on demand (the op keeps its own in the C++ backend)."""
    import torch
    need = workspace_size(m, k)
    key = str(device)
    ws = _ws_cache.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        _ws_cache[key] = ws
    return ws


def linear_forward(x, weights, out=None, workspace=None, kernel=KERNEL_AUTO, stream=None, pdl=False):
    """y = W4A32 linear of x (torch float32 [M,K] on the GPU, last dim contiguous)."""
    import torch
    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    m, k = x.shape
    assert k == weights.k
    if out is None:
        out = torch.empty((m, weights.n), dtype=torch.float32, device=x.device)
    if workspace is None:
        workspace = _workspace_for(m, k, x.device)
    _check(lib().mllmb200_w4a32_linear_forward_ex(x.data_ptr(), weights.tiled.data_ptr(), out.data_ptr(),
                                                  workspace.data_ptr(), m, k, weights.n, x.stride(0), out.stride(0),
                                                  kernel | (KERNEL_FLAG_PDL if pdl else 0), _stream_ptr(stream)),
           "linear_forward")
    return out


def linear_forward_grouped(x, weights_list, outs=None, workspace=None, stream=None, pdl=False, policy=KERNEL_AUTO):
    """Several linears on the same activations in one call (one launch for M <= 4; one shared
    quantization for larger M).  policy: KERNEL_AUTO or KERNEL_FASTEST."""
    import torch
    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    m, k = x.shape
    cnt = len(weights_list)
    assert 1 <= cnt <= 4 and all(w.k == k for w in weights_list)
    if outs is None:
        outs = [torch.empty((m, w.n), dtype=torch.float32, device=x.device) for w in weights_list]
    if workspace is None:
        workspace = _workspace_for(m, k, x.device)
    tiled = (C.c_void_p * cnt)(*[w.tiled.data_ptr() for w in weights_list])
    ys = (C.c_void_p * cnt)(*[o.data_ptr() for o in outs])
    ns = (C.c_int * cnt)(*[w.n for w in weights_list])
    ldy = (C.c_int * cnt)(*[o.stride(0) for o in outs])
    _check(lib().mllmb200_w4a32_linear_forward_grouped(x.data_ptr(), m, k, x.stride(0), cnt, tiled, ys, ns, ldy,
                                                       workspace.data_ptr(), (KERNEL_FLAG_PDL if pdl else 0) | policy,
                                                       _stream_ptr(stream)), "linear_forward_grouped")
    return outs


def gemv_plan_check(m, ks, ns):
    """Host-only replay of the streaming GEMV's work decomposition for matrices [ns[i], ks[i]] with activations
    [m, ks[i]] (ks may be one int for all).  Returns a dict (clusters, cluster_size, cells_per_stage, stages, smem)
    or None when the call has no GEMV plan; raises when the replay finds a cell or panel not covered exactly once."""
    cnt = len(ns)
    if isinstance(ks, int):
        ks = [ks] * cnt
    karr = (C.c_int * cnt)(*ks)
    arr = (C.c_int * cnt)(*ns)
    c, s, cpc, st, sm = C.c_int(), C.c_int(), C.c_int(), C.c_int(), C.c_size_t()
    r = lib().mllmb200_w4a32_gemv_plan_check(m, cnt, karr, arr, C.byref(c), C.byref(s), C.byref(cpc), C.byref(st), C.byref(sm))
    if r == 2:
        return None
    if r != 0:
        raise MllmB200Error(r, f"gemv_plan_check failed check {r - 100}")
    return {"clusters": c.value, "cluster_size": s.value, "cells_per_stage": cpc.value, "stages": st.value, "smem": sm.value}


def linear_forward_multi(xs, weights_list, outs=None, stream=None, pdl=False):
    """Several independent linears (each its own x [M, K_i]) in one launch; M <= 4, at most 8 of them."""
    import torch
    cnt = len(weights_list)
    m = xs[0].shape[0]
    assert len(xs) == cnt and all(x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1 and
                                   x.shape[0] == m and x.shape[1] == w.k for x, w in zip(xs, weights_list))
    if outs is None:
        outs = [torch.empty((m, w.n), dtype=torch.float32, device=xs[0].device) for w in weights_list]
    xp = (C.c_void_p * cnt)(*[x.data_ptr() for x in xs])
    ldx = (C.c_int * cnt)(*[x.stride(0) for x in xs])
    ks = (C.c_int * cnt)(*[w.k for w in weights_list])
    tiled = (C.c_void_p * cnt)(*[w.tiled.data_ptr() for w in weights_list])
    ys = (C.c_void_p * cnt)(*[o.data_ptr() for o in outs])
    ns = (C.c_int * cnt)(*[w.n for w in weights_list])
    ldy = (C.c_int * cnt)(*[o.stride(0) for o in outs])
    _check(lib().mllmb200_w4a32_linear_forward_multi(cnt, xp, ldx, ks, tiled, ys, ns, ldy, m, KERNEL_FLAG_PDL if pdl else 0,
                                                     _stream_ptr(stream)), "linear_forward_multi")
    return outs


def quant_activations(x, stream=None):
    """Device activation quantization in the reference's row layout: numpy int8 [M, K+8]."""
    import torch
    m, k = x.shape
    out = torch.empty((m, k + 8), dtype=torch.int8, device=x.device)
    _check(lib().mllmb200_w4a32_quant_activations(x.data_ptr(), m, k, x.stride(0), out.data_ptr(), _stream_ptr(stream)),
           "quant_activations")
    return out.cpu().numpy()


def check_device_status(stream=None):
    _check(lib().mllmb200_check_device_status(_stream_ptr(stream)), "device status")


def conv3d_forward(x, weights, kernel, stride, stream=None):
    """Conv3D (no padding, dilation 1) as a W4A32 linear: x [B, C, T, H, W] fp32 on the device,
    weights = W4A32Weights of the [out_ch, C*kt*kh*kw] matrix.  Returns [B, out_ch, T', H', W']."""
    import torch
    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 5 and x.is_contiguous()
    shp = (C.c_int * 5)(*x.shape)
    ker = (C.c_int * 3)(*kernel)
    strd = (C.c_int * 3)(*stride)
    m, k, wsb = C.c_int(), C.c_int(), C.c_size_t()
    _check(lib().mllmb200_conv3d_w4a32_plan(shp, ker, strd, weights.n, C.byref(m), C.byref(k), C.byref(wsb)), "conv3d_plan")
    assert k.value == weights.k, (k.value, weights.k)
    ot, oh, ow = [(x.shape[2 + i] - kernel[i]) // stride[i] + 1 for i in range(3)]
    y = torch.empty((x.shape[0], weights.n, ot, oh, ow), dtype=torch.float32, device=x.device)
    ws = torch.empty(wsb.value + 256, dtype=torch.uint8, device=x.device)
    off = (-ws.data_ptr()) % 256
    _check(lib().mllmb200_conv3d_w4a32_forward(x.data_ptr(), weights.tiled.data_ptr(), y.data_ptr(), ws.data_ptr() + off,
                                               shp, ker, strd, weights.n, _stream_ptr(stream)), "conv3d_forward")
    return y
