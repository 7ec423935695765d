"""Conv3D as a W4A32 linear (Qwen2VL patch embedding, K = 1176): CUDA path against the numpy
restatement oracle/conv3d_oracle.py whose linear is the pinned W4A32 C oracle.  Bar: the linear's
1e-3 * rms; im2col and the output permutation are pure data movement (checked exactly on CPU)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
from conv3d_oracle import conv3d_as_linear, im2col  # noqa: E402
from oracle_lib import Oracle  # noqa: E402


def test_im2col_matches_direct_convolution():
    """The restated im2col + a dense fp64 product equals a directly written 3-D convolution."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 3, 4, 9, 8)).astype(np.float32)
    w = rng.standard_normal((5, 3, 2, 3, 4)).astype(np.float32)
    kernel, stride = (2, 3, 4), (1, 2, 2)
    y = conv3d_as_linear(x, lambda z: (z.astype(np.float64) @ w.reshape(5, -1).astype(np.float64).T), 5, kernel, stride)
    ot, oh, ow = y.shape[2:]
    ref = np.zeros_like(y, dtype=np.float64)
    for b in range(2):
        for o in range(5):
            for it in range(ot):
                for ih in range(oh):
                    for iw in range(ow):
                        patch = x[b, :, it:it + 2, ih * 2:ih * 2 + 3, iw * 2:iw * 2 + 4]
                        ref[b, o, it, ih, iw] = float((patch.astype(np.float64) * w[o]).sum())
    assert np.allclose(y, ref, rtol=1e-12, atol=1e-12)


def test_plan_reports_the_implied_linear():
    import ctypes as C
    import mllm_b200 as mb
    m, k, ws = C.c_int(), C.c_int(), C.c_size_t()
    shp, ker = (C.c_int * 5)(7, 3, 2, 14, 14), (C.c_int * 3)(2, 14, 14)
    assert mb.lib().mllmb200_conv3d_w4a32_plan(shp, ker, ker, 1280, C.byref(m), C.byref(k), C.byref(ws)) == 0
    assert (m.value, k.value) == (7, 1176) and ws.value >= 7 * 1176 * 4 + 7 * 1280 * 4
    bad = (C.c_int * 3)(3, 14, 14)  # kernel deeper than the input
    assert mb.lib().mllmb200_conv3d_w4a32_plan(shp, bad, ker, 1280, None, None, None) != 0


@pytest.mark.gpu
@pytest.mark.parametrize("shape,kernel,stride,out_ch", [
    ((1, 3, 2, 14, 14), (2, 14, 14), (2, 14, 14), 1280),    # one Qwen2VL patch: M = 1 (GEMV), K = 1176
    ((40, 3, 2, 14, 14), (2, 14, 14), (2, 14, 14), 1280),   # a batch of patches: tcgen05 path
    ((2, 3, 4, 28, 28), (2, 14, 14), (2, 14, 14), 96),      # several output positions per image: M = 16
    ((3, 2, 3, 10, 9), (2, 3, 4), (1, 2, 2), 33),           # overlapping windows, odd sizes
])
def test_conv3d_matches_oracle(shape, kernel, stride, out_ch):
    import torch
    import mllm_b200 as mb
    orc = Oracle()
    rng = np.random.default_rng(sum(shape) + out_ch)
    x = rng.standard_normal(shape).astype(np.float32)
    k = shape[1] * kernel[0] * kernel[1] * kernel[2]
    w = (rng.standard_normal((out_ch, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(out_ch) * 0.1).astype(np.float32)
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    q, s = np.ascontiguousarray(q), np.ascontiguousarray(s)
    ref = conv3d_as_linear(x, lambda z: orc.linear(z, q, s, b), out_ch, kernel, stride)
    y = mb.conv3d_forward(torch.from_numpy(x).cuda(), mb.W4A32Weights.from_blob(blob), kernel, stride)
    torch.cuda.synchronize()
    mb.check_device_status()
    y = y.cpu().numpy()
    assert y.shape == ref.shape
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    assert float(np.max(np.abs(y - ref))) <= 1e-3 * rms
    # the data movement alone is exact: the device im2col feeds the same linear as the oracle's
    z, _ = im2col(x, kernel, stride)
    y_lin = mb.linear_forward(torch.from_numpy(z).cuda(), mb.W4A32Weights.from_blob(blob)).cpu().numpy()
    ot, oh, ow = ref.shape[2:]
    assert np.array_equal(y, np.transpose(y_lin.reshape(shape[0], ot, oh, ow, out_ch), (0, 4, 1, 2, 3)))
