"""GPU parity tests: every result comes from libmllm_b200.so through the C ABI and is compared
with the CPU oracle (oracle/w4a32_oracle.c) on the same seeded inputs.

Bars: packing, repacking and activation quantization bit-exact; outputs max|diff| <= 1e-3 * rms(y)
(the fp32-accumulate bar; the integer group sums are exact, only the order of the fp32 additions
and the factored zero-point term differ from the scalar reference)."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import mllm_b200 as mb  # noqa: E402
from oracle_lib import Oracle  # noqa: E402

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "kai_ref_golden.npz"))
TOL = 1e-3  # times rms(y)


@pytest.fixture(scope="module")
def orc():
    return Oracle()


@pytest.fixture(scope="module", autouse=True)
def _device():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    mb.lib()
    yield
    mb.check_device_status()


def make_case(rng, m, n, k, bias=True, x_scale=1.0, w_scale=0.02):
    x = (rng.standard_normal((m, k)) * x_scale).astype(np.float32)
    w = (rng.standard_normal((n, k)) * w_scale).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32) * 0.1 if bias else None
    return x, w, b


def gpu_forward(x, blob, kernel=mb.KERNEL_AUTO, **kw):
    wt = mb.W4A32Weights.from_blob(blob)
    y = mb.linear_forward(torch.from_numpy(x).cuda(), wt, kernel=kernel, **kw)
    torch.cuda.synchronize()
    mb.check_device_status()
    return y.cpu().numpy()


def assert_close(y, ref, what=""):
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    err = float(np.max(np.abs(y.astype(np.float64) - ref)))
    assert np.all(np.isfinite(y)), what
    assert err <= TOL * max(rms, 1e-30), f"{what}: max|diff| {err:.3e} > {TOL} * rms {rms:.3e}"


# ------------------------------------------------------------------ packing
@pytest.mark.parametrize("n,k,mode,bias", [(8960, 1536, 0, False), (1536, 8960, 0, True), (256, 1536, 1, True),
                                           (33, 257, 2, True), (5, 70, 0, False), (9, 71, 0, True), (64, 1176, 0, True),
                                           (1, 32, 0, False), (31, 31, 0, True)])
def test_repack_unpack_roundtrip_bit_exact(n, k, mode, bias):
    rng = np.random.default_rng(n + k)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32) if bias else None
    blob = mb.quant_prepack(w, b, mode)
    wt = mb.W4A32Weights.from_blob(blob)
    back = wt.unpack()
    assert np.array_equal(back, blob)


def test_repack_row_shards_roundtrip():
    rng = np.random.default_rng(5)
    n, k = 200, 160
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    blob = mb.quant_prepack(w, b)
    nib, sc, bias = mb.blob_sections(blob)
    for r0, cnt in [(0, 50), (50, 97), (147, 53)]:
        wt = mb.W4A32Weights.from_blob(blob, row_begin=r0, row_count=cnt)
        n2, s2, b2 = mb.blob_sections(wt.unpack())
        assert np.array_equal(n2, nib[r0:r0 + cnt]) and np.array_equal(s2, sc[r0:r0 + cnt])
        assert np.array_equal(b2, bias[r0:r0 + cnt])


# ------------------------------------------------------------------ activation quantization
@pytest.mark.parametrize("m,k", [(1, 1536), (4, 8960), (3, 71), (7, 1000), (2, 32), (5, 1176)])
def test_activation_quant_bit_exact(orc, m, k):
    rng = np.random.default_rng(m * 31 + k)
    x = (rng.standard_normal((m, k)) * rng.uniform(0.05, 8.0)).astype(np.float32)
    if m > 1:
        x[1] = np.abs(x[1])          # all positive
    if m > 2:
        x[2] = 0.0                   # degenerate row
    got = mb.quant_activations(torch.from_numpy(x).cuda())
    assert np.array_equal(got, orc.quant_act(x))


def test_activation_quant_fixture_golden():
    x = Oracle().fill_uniform_random(1024, 4568).reshape(1, 1024)
    got = mb.quant_activations(torch.from_numpy(x).cuda())
    assert np.array_equal(got, GOLD["fixture_a"])


# ------------------------------------------------------------------ forward: reference fixture + goldens
def test_reference_fixture(orc):
    """The reference's own test of this path: M=1, K=N=1024, srand 4568/4572, |ref-act| <= 1e-4
    (tests/Arm/KaiLinearTest.hpp:387-463 of the reference project)."""
    x = orc.fill_uniform_random(1024, 4568).reshape(1, 1024)
    w = orc.fill_uniform_random(1024 * 1024, 4572).reshape(1024, 1024)
    y = gpu_forward(x, mb.quant_prepack(w))
    assert np.max(np.abs(y - GOLD["fixture_y"])) <= 1e-4
    assert_close(y, GOLD["fixture_y"], "fixture")


@pytest.mark.parametrize("name", sorted({k[:-2] for k in GOLD.files if k.startswith("r_") and k.endswith("_x")}))
@pytest.mark.parametrize("kernel", [mb.KERNEL_AUTO, mb.KERNEL_SIMT])
def test_ragged_goldens(name, kernel):
    x, w = GOLD[name + "_x"], GOLD[name + "_w"]
    y = gpu_forward(x, mb.quant_prepack(w), kernel)
    ref = GOLD[name + "_y"]
    assert_close(y, ref, name)


# ------------------------------------------------------------------ forward: decode GEMV
QWEN_SHAPES = [(1536, 1536), (1536, 256), (1536, 8960), (8960, 1536)]  # K -> N


@pytest.mark.parametrize("k,n", QWEN_SHAPES + [(1024, 1024), (32, 32), (64, 40), (4096, 96), (1176, 1280)])
@pytest.mark.parametrize("m", [1, 2, 3, 4])
def test_gemv_vs_oracle(orc, m, k, n):
    rng = np.random.default_rng(k * 7 + n + m)
    x, w, b = make_case(rng, m, n, k, bias=(n % 512 == 0))
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
    y = gpu_forward(x, blob, mb.KERNEL_GEMV)
    assert_close(y, ref, f"gemv m={m} k={k} n={n}")
    y2 = gpu_forward(x, blob, mb.KERNEL_GEMV, pdl=True)
    assert np.array_equal(y, y2)


@pytest.mark.parametrize("k,n", QWEN_SHAPES + [(64, 40), (1176, 1280)])
@pytest.mark.parametrize("m", [1, 4])
def test_gemv_two_launch_path_vs_oracle(orc, m, k, n):
    """The activation-quantization kernel + one-shot GEMV pair (kernel 6; what the decoder's graph mode is built
    from) against the oracle, and against the single-launch kernel within the same bar."""
    rng = np.random.default_rng(k * 5 + n + m)
    x, w, b = make_case(rng, m, n, k, bias=(n % 512 == 0))
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
    y = gpu_forward(x, blob, mb.KERNEL_GEMV_2LAUNCH)
    assert_close(y, ref, f"two-launch gemv m={m} k={k} n={n}")
    assert_close(gpu_forward(x, blob, mb.KERNEL_GEMV), y, "single launch vs two launches")


LAYER7 = [(1536, 1536, True), (1536, 256, True), (1536, 256, True), (1536, 1536, False), (1536, 8960, False),
          (1536, 8960, False), (8960, 1536, False)]  # K, N, bias of q k v o gate up down


@pytest.mark.parametrize("m", [1, 3])
def test_gemv_multi_layer_vs_oracle(orc, m):
    """BASELINE config 1 at decode: the seven linears of a decoder layer, each with its OWN activations, in ONE
    launch (mllmb200_w4a32_linear_forward_multi), every output against the oracle; with programmatic dependent
    launch the result is the same bit for bit."""
    rng = np.random.default_rng(700 + m)
    xs, wts, refs = [], [], []
    for k, n, bias in LAYER7:
        x, w, b = make_case(rng, m, n, k, bias=bias)
        blob = mb.quant_prepack(w, b)
        q, s, _ = mb.blob_sections(blob)
        refs.append(orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b))
        xs.append(torch.from_numpy(x).cuda())
        wts.append(mb.W4A32Weights.from_blob(blob))
    outs = mb.linear_forward_multi(xs, wts)
    torch.cuda.synchronize()
    mb.check_device_status()
    for (k, n, _), o, ref in zip(LAYER7, outs, refs):
        assert_close(o.cpu().numpy(), ref, f"multi m={m} k={k} n={n}")
    outs2 = mb.linear_forward_multi(xs, wts, pdl=True)
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(outs, outs2))


def test_gemv_multi_ragged_vs_oracle(orc):
    """Odd sizes side by side in one launch: K with a short last group, odd K, N below a panel, one matrix twice."""
    rng = np.random.default_rng(811)
    shapes = [(33, 40, True), (1176, 1280, False), (64, 7, True), (4096, 96, False), (71, 9, True), (32, 32, False),
              (257, 33, True), (8960, 64, False)]
    m = 2
    xs, wts, refs = [], [], []
    for k, n, bias in shapes:
        x, w, b = make_case(rng, m, n, k, bias=bias)
        blob = mb.quant_prepack(w, b)
        q, s, _ = mb.blob_sections(blob)
        refs.append(orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b))
        xs.append(torch.from_numpy(x).cuda())
        wts.append(mb.W4A32Weights.from_blob(blob))
    outs = mb.linear_forward_multi(xs, wts)
    torch.cuda.synchronize()
    mb.check_device_status()
    for (k, n, _), o, ref in zip(shapes, outs, refs):
        assert_close(o.cpu().numpy(), ref, f"multi ragged k={k} n={n}")


def test_gemv_multi_refuses_what_it_cannot_do():
    rng = np.random.default_rng(5)
    x, w, b = make_case(rng, 5, 64, 64)
    wt = mb.W4A32Weights.from_blob(mb.quant_prepack(w, b))
    with pytest.raises(mb.MllmB200Error) as e:
        mb.linear_forward_multi([torch.from_numpy(x).cuda()], [wt])  # M = 5: not a GEMV
    assert e.value.status == 2  # MLLMB200_UNSUPPORTED


def test_gemv_trace_records_ordered_stamps():
    """The profiling aid: with a trace buffer set, a launch leaves increasing global-timer values."""
    import ctypes as C
    rng = np.random.default_rng(6)
    x, w, b = make_case(rng, 1, 1536, 1536)
    wt = mb.W4A32Weights.from_blob(mb.quant_prepack(w, b))
    xd = torch.from_numpy(x).cuda()
    buf = torch.zeros(1 + 20 * 2, dtype=torch.int64, device="cuda")
    assert mb.lib().mllmb200_w4a32_gemv_trace(C.c_void_p(buf.data_ptr()), 2) == 0
    try:
        for _ in range(3):  # the third launch finds the buffer full and records nothing
            mb.linear_forward(xd, wt, kernel=mb.KERNEL_GEMV)
        torch.cuda.synchronize()
    finally:
        assert mb.lib().mllmb200_w4a32_gemv_trace(None, 0) == 0
    t = buf.cpu().numpy()[1:].reshape(2, 2, 10)
    for launch in range(2):
        first = t[launch, 0, :8]
        assert first[0] > 0 and np.all(np.diff(first) >= 0), first
    mb.check_device_status()


def test_cfg0_int4_uniform_fp16_scales(orc):
    """BASELINE config 0: x ~ N(0,1) [1,1536]; q uniform in [-8,7]; scales |N(0,0.02)|/7 as fp16."""
    g = torch.Generator().manual_seed(0)
    n, k = 8960, 1536
    x = torch.randn((1, k), generator=g).numpy()
    qv = torch.randint(-8, 8, (n, k), generator=g).numpy()
    sc = (torch.randn((n, k // 32), generator=g).abs() * 0.02 / 7)
    u = (qv + 8).astype(np.uint8)
    nib = (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)
    for mode, s16 in ((mb.SCALE_FP16, sc.to(torch.float16).view(torch.int16).numpy().view(np.uint16)),
                      (mb.SCALE_BF16_TRUNC, (sc.numpy().view(np.uint32) >> 16).astype(np.uint16))):
        blob = mb.prepack_from_quantized(nib, s16, n, k, None, mode)
        ref = orc.linear(x, nib, np.ascontiguousarray(s16), None, mode)
        y = gpu_forward(x, blob)
        assert_close(y, ref, f"cfg0 mode {mode}")


def test_negative_zero_and_huge_activations(orc):
    rng = np.random.default_rng(11)
    m, n, k = 4, 96, 256
    x, w, b = make_case(rng, m, n, k)
    x[0] *= 1e4
    x[1] = np.abs(x[1]) + 3.0      # zero point pinned at -128
    x[2] = -np.abs(x[2]) - 3.0     # zero point pinned at 127
    x[3] = 0.0
    w[3] = 0.0                      # all scales -0.0
    w[4, :32] = np.abs(w[4, :32])   # forces a negative scale in group 0
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
    for kern in (mb.KERNEL_GEMV, mb.KERNEL_SIMT):
        y = gpu_forward(x, blob, kern)
        for r in range(m):  # per row: the rows have very different magnitudes
            assert_close(y[r:r + 1], ref[r:r + 1], f"row {r} kernel {kern}")


# ------------------------------------------------------------------ forward: GEMM paths
@pytest.mark.parametrize("m,k,n", [(5, 1536, 256), (33, 1536, 1536), (64, 8960, 1536), (64, 1536, 8960),
                                   (17, 1176, 1280), (100, 70, 45), (128, 1536, 256)])
def test_simt_gemm_vs_oracle(orc, m, k, n):
    rng = np.random.default_rng(m + k + n)
    x, w, b = make_case(rng, m, n, k, x_scale=rng.uniform(0.2, 3.0))
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
    y = gpu_forward(x, blob, mb.KERNEL_SIMT)
    assert_close(y, ref, f"simt m={m} k={k} n={n}")


@pytest.mark.parametrize("m,k,n", [(5, 1536, 256), (8, 1536, 1536), (9, 64, 40), (16, 1176, 1280), (17, 1536, 256),
                                   (24, 8960, 1536), (32, 4096, 96), (33, 1536, 1536), (40, 32, 33), (64, 1536, 8960),
                                   (64, 8960, 1536), (64, 70, 45), (63, 8192, 512), (64, 12288, 64)])
def test_streaming_small_batch_gemm_vs_oracle(orc, m, k, n):
    """The streaming tensor-core GEMM for 5 <= M <= 64 (mma.sync u8 x s8 per K-group, clusters split K where the
    activations of a whole row do not fit one CTA): exact int32 group sums, fp32 scale-accumulate; against the
    oracle, and the default policy must pick it for these batch sizes."""
    rng = np.random.default_rng(m * 5 + k + n)
    x, w, b = make_case(rng, m, n, k, bias=(n % 2 == 0), x_scale=rng.uniform(0.2, 3.0))
    if m > 8:
        x[7] = np.abs(x[7]) + 1.0   # zero point -128
        x[8] = 0.0
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
    y = gpu_forward(x, blob, mb.KERNEL_STREAM_TC)
    assert_close(y, ref, f"streaming tensor-core m={m} k={k} n={n}")
    assert mb.lib().mllmb200_w4a32_select_kernel(m, k, n) == mb.KERNEL_STREAM_TC
    y2 = gpu_forward(x, blob, mb.KERNEL_AUTO, pdl=True)
    assert np.array_equal(y, y2), "default policy / dependent launch must give the same bits"
    assert_close(y, gpu_forward(x, blob, mb.KERNEL_SIMT), "streaming tensor-core vs simt")
    mb.check_device_status()


def test_streaming_small_batch_gemm_grouped_and_scale_modes(orc):
    """q, k, v sharing one quantization and ONE launch at M = 64, and the other two scale encodings."""
    rng = np.random.default_rng(64)
    k, ns, m = 1536, (1536, 256, 256), 64
    x = rng.standard_normal((m, k)).astype(np.float32)
    ws = [make_case(rng, 1, n, k)[1:] for n in ns]
    wts = [mb.W4A32Weights.from_blob(mb.quant_prepack(w, b)) for w, b in ws]
    outs = mb.linear_forward_grouped(torch.from_numpy(x).cuda(), wts)
    for (w, b), wt, o in zip(ws, wts, outs):
        single = mb.linear_forward(torch.from_numpy(x).cuda(), wt, kernel=mb.KERNEL_STREAM_TC)
        assert torch.equal(o, single)
        q, s, _ = mb.blob_sections(mb.quant_prepack(w, b))
        assert_close(o.cpu().numpy(), orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b), "grouped small batch")
    for mode in (mb.SCALE_BF16_RNE, mb.SCALE_FP16):
        w, b = ws[1]
        blob = mb.quant_prepack(w, b, scale_mode=mode)
        y = gpu_forward(x[:20], blob, mb.KERNEL_STREAM_TC)
        assert_close(y, gpu_forward(x[:20], blob, mb.KERNEL_SIMT), f"scale mode {mode}")
    mb.check_device_status()


@pytest.mark.parametrize("m,k,n", [(128, 128, 128), (17, 1536, 256), (33, 1536, 1536), (64, 8960, 1536),
                                   (128, 1536, 8960), (100, 70, 45), (200, 1176, 1280), (512, 1536, 256),
                                   (300, 4096, 96), (129, 32, 33)])
def test_tcgen05_gemm_vs_oracle(orc, m, k, n):
    """tcgen05 kind::i8 path: exact int32 group sums on the tensor cores, fp32 scale-accumulate in K order."""
    rng = np.random.default_rng(m * 3 + k + n)
    x, w, b = make_case(rng, m, n, k, x_scale=rng.uniform(0.2, 3.0))
    if m > 40:
        x[7] = np.abs(x[7]) + 1.0   # zero point -128
        x[8] = 0.0
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
    y = gpu_forward(x, blob, mb.KERNEL_TC)
    assert_close(y, ref, f"tcgen05 m={m} k={k} n={n}")
    y2 = gpu_forward(x, blob, mb.KERNEL_SIMT)
    assert_close(y, y2, "tcgen05 vs simt")


@pytest.mark.parametrize("m,k,n", [(128, 128, 128), (64, 1536, 256), (100, 70, 45), (200, 1176, 1280), (512, 1536, 256),
                                   (300, 4096, 96), (129, 32, 33), (256, 1536, 8960), (512, 8960, 1536),
                                   (384, 1536, 12800)])
def test_tcgen05_fp16_gemm_vs_oracle(orc, m, k, n):
    """tcgen05 fp16 path: group scales folded into an exact fp16 weight operand, fp32 accumulation over
    all of K in tensor memory.  Products are exact; the stated bound is the common 1e-3 * rms."""
    rng = np.random.default_rng(m * 5 + k + n)
    x, w, b = make_case(rng, m, n, k, x_scale=rng.uniform(0.2, 3.0))
    x[7] = np.abs(x[7]) + 1.0   # zero point -128
    x[8] = 0.0
    w[3] *= 1e-3                # a row of small scales next to ordinary ones
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
    y = gpu_forward(x, blob, mb.KERNEL_TC_F16)
    assert_close(y, ref, f"tcgen05 fp16 m={m} k={k} n={n}")
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    print(f"tcgen05 fp16 m={m} k={k} n={n}: max|diff| / rms = {float(np.max(np.abs(y - ref))) / rms:.2e}")


@pytest.mark.parametrize("m,k,n", [(128, 1056, 200), (512, 8960, 1536), (260, 2080, 384), (64, 4128, 96), (128, 1024, 256),
                                   (256, 1056, 9600)])
def test_tcgen05_fp16_gemm_k_split(orc, m, k, n):
    """Launches that would leave most SMs idle split K between two CTAs per output tile (and so do the tiles left over
    after the last full wave - the last case: 150 tiles on 148 SMs); the half that finishes first parks its sums in
    the tile's place in y.  Odd and ragged K-tile counts, an output buffer that starts as NaN
    (nothing may depend on what y held), a row stride wider than N, and the same bits on every repeat whichever
    half finishes first."""
    rng = np.random.default_rng(m + 3 * k + n)
    x, w, b = make_case(rng, m, n, k, x_scale=rng.uniform(0.3, 2.0))
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
    wt = mb.W4A32Weights.from_blob(blob)
    xd = torch.from_numpy(x).cuda()
    buf = torch.full((m, n + 24), float("nan"), device="cuda")
    y = buf[:, :n]
    first = None
    for _ in range(6):
        buf.fill_(float("nan"))
        mb.linear_forward(xd, wt, out=y, kernel=mb.KERNEL_TC_F16)
        torch.cuda.synchronize()
        mb.check_device_status()
        if first is None:
            first = y.clone()
            assert_close(first.cpu().numpy(), ref, f"k-split m={m} k={k} n={n}")
        else:
            assert torch.equal(y, first)
        assert bool(torch.isnan(buf[:, n:]).all()), "wrote outside the N columns"


@pytest.mark.parametrize("mode", [mb.SCALE_BF16_RNE, mb.SCALE_FP16])
@pytest.mark.parametrize("m,k,n", [(128, 1536, 256), (512, 1536, 8960), (256, 8960, 1536), (200, 1176, 1280)])
def test_tcgen05_fp16_gemm_other_scale_encodings(orc, m, k, n, mode):
    """The fp16 tensor-core path (kernel 4, and policy 5 which picks it for M >= 128) under the other two scale
    encodings.  bf16 scales (either rounding): the weight operand (u-8) * s is exact in fp16, bar 1e-3 * rms as
    everywhere.  fp16-encoded scales (the encoding BASELINE config 0 states): the product needs up to 14 bits and
    is rounded to fp16's 11 - relative error <= 2^-12 per weight; stated bar for that mode 2e-3 * rms(y)."""
    rng = np.random.default_rng(m + k + n + mode)
    x, w, b = make_case(rng, m, n, k, x_scale=rng.uniform(0.5, 2.0))
    blob = mb.quant_prepack(w, b, scale_mode=mode)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b, mode)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    bar = (2e-3 if mode == mb.SCALE_FP16 else TOL) * rms
    for kern in (mb.KERNEL_TC_F16, mb.KERNEL_FASTEST):
        y = gpu_forward(x, blob, kern)
        err = float(np.max(np.abs(y.astype(np.float64) - ref)))
        print(f"fp16 tensor-core path, scale mode {mode}, kernel {kern}, m={m} k={k} n={n}: max|diff| / rms = {err / rms:.2e}")
        assert np.all(np.isfinite(y)) and err <= bar, (mode, kern, err / rms)
    # the exact int8 path under the same encoding meets the common bar
    assert_close(gpu_forward(x, blob, mb.KERNEL_TC), ref, f"int8 tensor-core path, scale mode {mode}")


@pytest.mark.parametrize("policy", [0, 5])
def test_grouped_prefill_shares_quantization(orc, policy):
    """q/k/v and gate/up at prefill size through the grouped call equal single calls bit for bit:
    policy 0 = one shared quantization, then one int8 tensor-core launch per matrix; policy 5 = one
    shared quantization and ONE fp16 tensor-core launch for all matrices (same tile width as the
    single fp16 calls here, hence the same order of additions)."""
    rng = np.random.default_rng(91)
    m, k = 300, 1536
    x = rng.standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    for ns in ((1536, 256, 256), (8960, 8960)):
        wts = []
        for n in ns:
            w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
            wts.append(mb.W4A32Weights.from_blob(mb.quant_prepack(w, None)))
        outs = mb.linear_forward_grouped(xd, wts, policy=policy)
        torch.cuda.synchronize()
        for wt, o in zip(wts, outs):
            single = mb.linear_forward(xd, wt, kernel=mb.KERNEL_TC_F16 if policy == 5 else policy)
            torch.cuda.synchronize()
            assert torch.equal(o, single), (policy, wt.n)
    mb.check_device_status()


def test_tcgen05_prefill_layer_shapes_full_size():
    """All seven linears of a decoder layer at M=512 (BASELINE config 1): tcgen05 vs SIMT path."""
    rng = np.random.default_rng(77)
    for k, n in QWEN_SHAPES:
        x, w, b = make_case(rng, 512, n, k)
        blob = mb.quant_prepack(w, b)
        y = gpu_forward(x, blob, mb.KERNEL_TC)
        y2 = gpu_forward(x, blob, mb.KERNEL_SIMT)
        assert_close(y, y2, f"prefill k={k} n={n}")


def test_config1_prefill_full_size_vs_oracle(orc):
    """BASELINE config 1 at prefill, full size (M = 512, the four shapes of the 1.5B layer), every kernel policy
    against the ORACLE: an output row depends on its own activation row only, so the oracle computes 64 of the
    512 rows (spread over all four 128-row tiles) and those rows of every GPU result are compared."""
    rng = np.random.default_rng(512)
    sel = np.sort(rng.choice(512, 64, replace=False))
    sel[0], sel[-1] = 0, 511
    for k, n in QWEN_SHAPES:
        x, w, b = make_case(rng, 512, n, k, bias=(n != 8960))
        blob = mb.quant_prepack(w, b)
        q, s, _ = mb.blob_sections(blob)
        ref = orc.linear(np.ascontiguousarray(x[sel]), np.ascontiguousarray(q), np.ascontiguousarray(s), b)
        for kern in (mb.KERNEL_AUTO, mb.KERNEL_TC, mb.KERNEL_TC_F16, mb.KERNEL_FASTEST, mb.KERNEL_SIMT):
            y = gpu_forward(x, blob, kern)
            assert_close(y[sel], ref, f"config 1 prefill k={k} n={n} kernel {kern}")


def test_config4_full_size_vs_oracle(orc):
    """BASELINE config 4's matrix (W [28672, 8192], int4 + bf16 scales drawn directly): the GEMV at M = 2 against the
    oracle on every output; the GEMM at M = 2048 (int8 and fp16 tensor-core kernels) against the oracle on 96
    activation rows x 512 weight rows (rows of y depend on their own x row, columns on their own weight row)."""
    n, k = 28672, 8192
    g = torch.Generator().manual_seed(4)
    nib = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g).numpy()
    sc = (torch.randn((n, k // 32), generator=g).abs() * (0.02 / 7)).numpy()
    s16 = (sc.view(np.uint32) >> 16).astype(np.uint16)
    blob = mb.prepack_from_quantized(nib, s16, n, k, None, mb.SCALE_BF16_TRUNC)
    wt = mb.W4A32Weights.from_blob(blob)
    x2 = torch.randn((2, k), generator=g).numpy()
    ref2 = orc.linear(x2, nib, s16, None)
    y2 = mb.linear_forward(torch.from_numpy(x2).cuda(), wt, kernel=mb.KERNEL_GEMV).cpu().numpy()
    mb.check_device_status()
    assert_close(y2, ref2, "config 4 GEMV M=2")
    m = 2048
    xm = torch.randn((m, k), generator=g).numpy()
    rng = np.random.default_rng(44)
    xsel = np.sort(rng.choice(m, 96, replace=False))
    wsel = np.sort(rng.choice(n, 512, replace=False))
    xsel[0], xsel[-1], wsel[0], wsel[-1] = 0, m - 1, 0, n - 1
    ref = orc.linear(np.ascontiguousarray(xm[xsel]), np.ascontiguousarray(nib[wsel]), np.ascontiguousarray(s16[wsel]), None)
    xd = torch.from_numpy(xm).cuda()
    for kern in (mb.KERNEL_TC, mb.KERNEL_TC_F16):
        y = mb.linear_forward(xd, wt, kernel=kern)
        torch.cuda.synchronize()
        mb.check_device_status()
        got = y[torch.from_numpy(xsel).cuda()][:, torch.from_numpy(wsel).cuda()].cpu().numpy()
        assert_close(got, ref, f"config 4 GEMM M=2048 kernel {kern}")
        del y


def test_strided_input_and_output(orc):
    rng = np.random.default_rng(21)
    m, n, k = 3, 64, 128
    x, w, b = make_case(rng, m, n, k)
    blob = mb.quant_prepack(w, b)
    q, s, _ = mb.blob_sections(blob)
    ref = orc.linear(x, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
    wt = mb.W4A32Weights.from_blob(blob)
    xb = torch.zeros((m, k + 24), device="cuda")
    xb[:, :k] = torch.from_numpy(x).cuda()
    yb = torch.full((m, n + 8), -7.0, device="cuda")
    for kern in (mb.KERNEL_GEMV, mb.KERNEL_SIMT):
        yb.fill_(-7.0)
        mb.linear_forward(xb[:, :k], wt, out=yb[:, :n], kernel=kern)
        torch.cuda.synchronize()
        assert_close(yb[:, :n].cpu().numpy(), ref, f"strided kernel {kern}")
        assert torch.all(yb[:, n:] == -7.0)


# ------------------------------------------------------------------ size-independent properties at full size
def test_row_shards_concatenate_to_full_result():
    """Column (output-channel) sharding: each shard's output is bit-identical to that slice of the
    unsharded output, for 2/4/8 shards - the tensor-parallel path needs no reduction."""
    rng = np.random.default_rng(33)
    n, k = 8960, 1536
    x, w, b = make_case(rng, 1, n, k)
    blob = mb.quant_prepack(w, b)
    full = gpu_forward(x, blob)
    xd = torch.from_numpy(x).cuda()
    for g in (2, 4, 8):
        per = n // g
        parts = [mb.linear_forward(xd, mb.W4A32Weights.from_blob(blob, row_begin=r * per, row_count=per)).cpu().numpy()
                 for r in range(g)]
        assert np.array_equal(np.concatenate(parts, axis=1), full)


def test_batch_rows_match_single_rows():
    """Each activation row is quantized on its own: row r of an M=4 call equals the M=1 call on that row."""
    rng = np.random.default_rng(34)
    n, k = 1536, 8960
    x, w, b = make_case(rng, 4, n, k)
    blob = mb.quant_prepack(w, b)
    y4 = gpu_forward(x, blob, mb.KERNEL_GEMV)
    for r in range(4):
        y1 = gpu_forward(x[r:r + 1], blob, mb.KERNEL_GEMV)
        assert np.array_equal(y1[0], y4[r])
    ys = gpu_forward(x, blob, mb.KERNEL_SIMT)
    assert_close(ys, y4, "simt vs gemv")


@pytest.mark.parametrize("m", [1, 3, 4, 9])
def test_grouped_equals_single_calls(m):
    """q/k/v and gate/up style groups: one launch, results bit-identical to separate calls for the
    same kernel family."""
    rng = np.random.default_rng(40 + m)
    k = 1536
    x = rng.standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    for ns in ((1536, 256, 256), (8960, 8960), (40,), (64, 8960, 32, 1536)):
        ws = [mb.W4A32Weights.from_blob(mb.quant_prepack(*make_case(rng, 1, n, k, bias=(i % 2 == 0))[1:]))
              for i, n in enumerate(ns)]
        outs = mb.linear_forward_grouped(xd, ws)
        torch.cuda.synchronize()
        mb.check_device_status()
        for w, o in zip(ws, outs):
            single = mb.linear_forward(xd, w)
            if m <= 4:
                assert_close(o.cpu().numpy(), single.cpu().numpy(), f"grouped m={m} n={w.n}")
            else:
                assert torch.equal(o, single)


def test_zero_input_gives_bias():
    rng = np.random.default_rng(35)
    n, k = 512, 1536
    _, w, b = make_case(rng, 2, n, k)
    blob = mb.quant_prepack(w, b)
    for kern in (mb.KERNEL_GEMV, mb.KERNEL_SIMT):
        y = gpu_forward(np.zeros((2, k), np.float32), blob, kern)
        assert np.array_equal(y, np.broadcast_to(b, (2, n)))


def test_deterministic_repeat():
    rng = np.random.default_rng(36)
    x, w, b = make_case(rng, 1, 8960, 1536)
    blob = mb.quant_prepack(w, b)
    wt = mb.W4A32Weights.from_blob(blob)
    xd = torch.from_numpy(x).cuda()
    y0 = mb.linear_forward(xd, wt).clone()
    for _ in range(5):
        assert torch.equal(mb.linear_forward(xd, wt), y0)


def test_bad_header_reports_status():
    """Calling forward with N/K that do not match the tiled buffer is caught on the device and
    reported as a status, not a fault."""
    rng = np.random.default_rng(37)
    x, w, b = make_case(rng, 1, 64, 64)
    wt = mb.W4A32Weights.from_blob(mb.quant_prepack(w, b))
    wt.n = 32  # lie about N (stays inside the buffer)
    mb.linear_forward(torch.from_numpy(x).cuda(), wt, kernel=mb.KERNEL_GEMV)
    with pytest.raises(mb.MllmB200Error) as e:
        mb.check_device_status()
    assert e.value.status == 5
    mb.check_device_status()  # cleared


def test_bounded_wait_gives_up_and_reports_timeout():
    """Every device-side wait of the library is bounded.  A test kernel waits, with a short tick limit, for bytes
    that nobody sends: it must come back (no hang), the status word must say MLLMB200_TIMEOUT exactly once, and
    the GPU must be usable right after."""
    import ctypes as C
    mb.check_device_status()  # clean before
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = mb.lib().mllmb200_selftest_wait_timeout(1 << 20, C.c_void_p(flag.data_ptr()), None)  # ~0.5 ms of ticks
    assert st == 0, mb.status_str(st)
    with pytest.raises(mb.MllmB200Error) as e:
        mb.check_device_status()
    assert e.value.status == 4  # MLLMB200_TIMEOUT
    assert int(flag.item()) == 1
    mb.check_device_status()  # the word was cleared by the read
    rng = np.random.default_rng(1)
    x, w, b = make_case(rng, 1, 64, 64)
    y = gpu_forward(x, mb.quant_prepack(w, b))  # the context is intact
    assert np.all(np.isfinite(y))
