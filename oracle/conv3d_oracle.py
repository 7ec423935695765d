"""CPU restatement (numpy) of the reference project's Conv3D-as-linear flow.

TEST INFRASTRUCTURE ONLY: the checker for the CUDA path; nothing shipped imports it.

Follows mllm/Backends/Arm/Ops/Conv3DOp.cpp:31-170 of the reference project: im2col of the fp32
activation (mllm/Backends/Arm/Kernels/conv3d.cpp:15-79: no padding, dilation 1, column order
c, kt, kh, kw; rows ordered b, t', h', w'), the W4A32 linear on the im2col matrix (passed in as a
callable: the tests bind it to the pinned C oracle), and the permutation {0, 4, 1, 2, 3} of the
[B, T', H', W', O] result to [B, O, T', H', W'].  Loops are written out as in the reference (plain
Python, small cases only).  The reference's vectorized inner copy takes its trip count from the
image width instead of the kernel width; the two agree whenever kernel width == image width (the
Qwen2VL patch embedding) and the scalar definition below is the intended one otherwise.
"""
import numpy as np


def im2col(x, kernel, stride):
    B, C, T, H, W = x.shape
    kt, kh, kw = kernel
    st, sh, sw = stride
    ot, oh, ow = (T - kt) // st + 1, (H - kh) // sh + 1, (W - kw) // sw + 1
    z = np.zeros((B * ot * oh * ow, C * kt * kh * kw), np.float32)
    for b in range(B):
        for it in range(ot):
            for ih in range(oh):
                for iw in range(ow):
                    row = ((b * ot + it) * oh + ih) * ow + iw
                    for c in range(C):
                        for a in range(kt):
                            for e in range(kh):
                                z0 = c * kt * kh * kw + a * kh * kw + e * kw
                                z[row, z0:z0 + kw] = x[b, c, it * st + a, ih * sh + e, iw * sw:iw * sw + kw]
    return z, (ot, oh, ow)


def conv3d_as_linear(x, linear, out_ch, kernel, stride):
    z, (ot, oh, ow) = im2col(np.asarray(x, np.float32), kernel, stride)
    y = linear(z)                                            # [B*ot*oh*ow, out_ch]
    y = y.reshape(x.shape[0], ot, oh, ow, out_ch)
    return np.ascontiguousarray(np.transpose(y, (0, 4, 1, 2, 3)))
