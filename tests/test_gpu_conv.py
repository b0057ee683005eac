"""GPU: Conv2d_q through the C ABI -- against the fixtures generated from the reference build, against the CPU oracle
on other shapes, and through size-independent properties where the oracle would take too long."""
import ctypes as C

import numpy as np
import pytest

from helpers import iter_conv_cases, ltq_qp, qp_of

pytestmark = pytest.mark.gpu


def _conv(cuda, ltq, c, qps, flags=0, out_mode=0, bias=None):
    h = ltq.ConvHandle(0, c["Cin"], c["Cout"], c["kh"], c["kw"], c["ph"], c["pw"], c["sh"], c["sw"])
    w = cuda.from_numpy(np.ascontiguousarray(c["w"])).cuda()
    b = None if bias is None else cuda.from_numpy(bias).cuda()
    h.set_weights(w, b)
    h.set_qparams(*qps)
    y = h.forward(cuda.from_numpy(np.ascontiguousarray(c["x"])).cuda(), out_mode, flags)
    cuda.cuda.synchronize()
    return y.cpu().numpy()


@pytest.mark.parametrize("force", ["auto", "simt"])
def test_conv_matches_golden(cuda, golden, force):
    import ltq
    g = golden("conv2d.npz")
    flags = ltq.FLAG_FORCE_SIMT if force == "simt" else 0
    for c in iter_conv_cases(g):
        y = _conv(cuda, ltq, c, [ltq_qp(r) for r in c["qp"]], flags=flags, bias=c["bias"])
        # left to itself the library computes every one of the reference's cases without a patch buffer
        assert ltq.last_kernel().startswith("conv_direct_kernel<") == (force == "auto"), (c["key"], ltq.last_kernel())
        np.testing.assert_array_equal(y, c["y"], err_msg=c["key"])
    assert ltq.lib().ltq_device_check(0, None) == 0


def test_im2col_t_is_the_transposed_padded_reference_buffer(cuda, golden):
    import ltq
    g = golden("conv2d.npz")
    for c in iter_conv_cases(g):
        K, N = c["col0"].shape
        Kp = (K + 15) // 16 * 16
        x = cuda.from_numpy(np.ascontiguousarray(c["x"])).cuda()
        col = cuda.full((c["B"], N, Kp), 0xEE, dtype=cuda.uint8, device="cuda")
        ltq._binding.check(ltq.lib().ltq_im2col_t_u8(x.data_ptr(), c["B"], c["Cin"], c["H"], c["W"], c["kh"], c["kw"],
                                                     c["ph"], c["pw"], c["sh"], c["sw"], col.data_ptr(), Kp, 0, None))
        cuda.cuda.synchronize()
        col = col.cpu().numpy()
        np.testing.assert_array_equal(col[0, :, :K], c["col0"].T, err_msg=c["key"])
        assert not col[:, :, K:].any(), "padding bytes must be zero"


@pytest.mark.parametrize("shape", [
    # B, Cin, H, W, Cout, kh, kw, ph, pw, sh, sw
    (2, 32, 20, 20, 160, 3, 3, 1, 1, 1, 1),      # 160 x 400 x 288: tensor-core path, two row tiles
    (3, 8, 33, 31, 12, 4, 4, 0, 0, 1, 1),        # M = 12, K = 128: eligible for the skinny kernel
    (1, 3, 40, 40, 64, 7, 7, 3, 3, 2, 2),        # K = 147 -> padded to 160
    (5, 1, 28, 28, 10, 5, 5, 2, 2, 1, 1),
])
def test_conv_matches_oracle(cuda, oracle, shape):
    import ltq
    B, Cin, H, W, Cout, kh, kw, ph, pw, sh, sw = shape
    rng = np.random.default_rng(sum(shape))
    c = dict(Cin=Cin, Cout=Cout, kh=kh, kw=kw, ph=ph, pw=pw, sh=sh, sw=sw,
             x=rng.integers(0, 256, (B, Cin, H, W), dtype=np.uint8),
             w=rng.integers(0, 256, (Cout, Cin * kh * kw), dtype=np.uint8))
    rows = [(0.02, 128), (0.005, 127), (0.6, 3)]
    want = oracle.port.conv2d_q(c["x"], c["w"], Cout, kh, kw, *[qp_of(oracle, r) for r in rows], ph=ph, pw=pw, sh=sh,
                                sw=sw)
    got = _conv(cuda, ltq, c, [ltq_qp(r) for r in rows])
    # these stride-1 layers take the kernel without a patch buffer whatever the channel counts (they are padded); the 7 x 7
    # stride-2 layer's weights and regions do not fit its shared memory and go through the patch buffer
    assert ltq.last_kernel().startswith("conv_direct_kernel<") == (sh == 1 and sw == 1), ltq.last_kernel()
    np.testing.assert_array_equal(got, want)
    # one bias per output channel (the library's option; the oracle restates the same arithmetic)
    bias = rng.integers(-30000, 30000, Cout, dtype=np.int32)
    want = oracle.port.conv2d_q(c["x"], c["w"], Cout, kh, kw, *[qp_of(oracle, r) for r in rows], bias=bias, ph=ph,
                                pw=pw, sh=sh, sw=sw, bias_per_channel=True)
    got = _conv(cuda, ltq, c, [ltq_qp(r) for r in rows], flags=ltq.FLAG_BIAS_PER_CHANNEL, bias=bias)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("shape", [
    # B, Cin, H, W, Cout, kh, kw, ph, pw
    (2, 64, 12, 20, 32, 3, 3, 1, 1),       # 32 slots per row: 4 output rows per tile, three tiles per image
    (3, 64, 56, 56, 64, 3, 3, 1, 1),       # the benchmark's geometry: 2 rows of 56 (64 slots each) per tile
    (1, 128, 9, 9, 48, 3, 3, 0, 0),        # two channel chunks, no padding, 7 x 7 output in one tile of 8 rows x 16 slots
    (5, 64, 7, 7, 16, 1, 1, 0, 0),         # 1 x 1 kernel
    (2, 64, 30, 30, 32, 5, 5, 2, 2),       # 25 taps (77 KB of reordered weights resident)
    (1, 64, 5, 128, 16, 3, 3, 1, 0),       # Wo = 126: one output row per tile of 128 slots; padding in y only
    (2, 64, 14, 14, 256, 3, 3, 1, 1),      # 256 output channels: three launches (96 + 96 + 64 channels)
    (1, 128, 10, 12, 128, 3, 3, 1, 1),     # 128 -> 128 channels: two channel chunks, two launches of 64 channels
    (2, 64, 9, 16, 32, 3, 3, 1, 1),        # image rows of two 8-byte units: gathered by the kernel itself
    (1, 100, 10, 24, 24, 3, 3, 0, 1),      # gathered, two channel chunks, the second one 36 channels + padding
    (3, 3, 11, 64, 16, 3, 3, 1, 1),        # gathered, 64-byte rows (a full scratch line), three channels
    (2, 64, 6, 8, 16, 1, 1, 0, 0),         # one unit per row, 16 image rows per tile: the scratch lines do not fit, NHWC copy
    (1, 70, 40, 40, 40, 3, 3, 1, 1),       # gathered, many tiles per CTA-less grid (20 tiles), 70 channels
])
@pytest.mark.parametrize("mode", ["u8", "f32", "i32"])
def test_conv_without_patch_buffer_matches_oracle(cuda, oracle, shape, mode):
    # the shapes whose NCHW input the kernel transposes itself while it loads (strides 1, rows of whole 8-byte units up to 64
    # bytes, scratch lines that fit beside the weights); the others go through the NHWC copy
    GATHERED = {(3, 64, 56, 56, 64, 3, 3, 1, 1), (2, 64, 9, 16, 32, 3, 3, 1, 1), (1, 100, 10, 24, 24, 3, 3, 0, 1),
                (3, 3, 11, 64, 16, 3, 3, 1, 1), (1, 70, 40, 40, 40, 3, 3, 1, 1)}
    """Stride 1 and a multiple of 64 input channels take the kernel that never builds the patches (K walked as kernel row,
    kernel column, channel; patch sums from an all-ones weight row).  Against the oracle, bit for bit, with and without
    the per-channel bias and ReLU, and against the patch-buffer path on the same device."""
    import ltq
    B, Cin, H, W, Cout, kh, kw, ph, pw = shape
    rng = np.random.default_rng(sum(shape) + len(mode))
    c = dict(Cin=Cin, Cout=Cout, kh=kh, kw=kw, ph=ph, pw=pw, sh=1, sw=1,
             x=rng.integers(0, 256, (B, Cin, H, W), dtype=np.uint8),
             w=rng.integers(0, 256, (Cout, Cin * kh * kw), dtype=np.uint8))
    rows = [(0.02, 128), (0.005, 127), (4.0, 3)]
    qps = [ltq_qp(r) for r in rows]
    out_mode = {"u8": ltq.OUT_U8, "f32": ltq.OUT_F32, "i32": ltq.OUT_I32}[mode]
    bias = rng.integers(-30000, 30000, Cout, dtype=np.int32)
    for use_bias, relu in ((False, False), (True, False), (True, True)):
        flags = (ltq.FLAG_BIAS_PER_CHANNEL if use_bias else 0) | (ltq.FLAG_RELU if relu else 0)
        got = _conv(cuda, ltq, c, qps, flags=flags, out_mode=out_mode, bias=bias if use_bias else None)
        assert ltq.last_kernel().startswith("conv_direct_kernel<"), ltq.last_kernel()
        # image rows of whole words are transposed by the kernel itself while it loads; the others go through the NHWC copy
        assert ("NCHW input gathered" in ltq.last_kernel()) == (shape in GATHERED), ltq.last_kernel()
        old = _conv(cuda, ltq, c, qps, flags=flags | ltq.FLAG_FORCE_SIMT, out_mode=out_mode, bias=bias if use_bias else None)
        assert not ltq.last_kernel().startswith("conv_direct_kernel<")
        np.testing.assert_array_equal(got.view(np.uint32) if mode == "f32" else got, old.view(np.uint32) if mode == "f32" else old)
        if mode == "u8" and not relu:
            want = oracle.port.conv2d_q(c["x"], c["w"], Cout, kh, kw, *[qp_of(oracle, r) for r in rows], bias=bias if use_bias else None,
                                        ph=ph, pw=pw, sh=1, sw=1, bias_per_channel=use_bias)
            np.testing.assert_array_equal(got, want)
    assert ltq.lib().ltq_device_check(0, None) == 0


@pytest.mark.parametrize("shape", [
    # B, Cin, H, W, Cout, kh, kw, ph, pw, sh, sw
    (2, 64, 16, 16, 32, 3, 3, 1, 1, 2, 2),       # the usual down-sampling layer: four planes of equal residues
    (1, 32, 15, 17, 48, 3, 3, 1, 1, 2, 2),       # odd image size: the planes differ by a row / a column
    (2, 64, 14, 14, 64, 1, 1, 0, 0, 2, 2),       # 1 x 1 kernel: only one of the four planes is read
    (3, 8, 21, 30, 24, 3, 5, 1, 2, 2, 1),        # different strides per direction
    (1, 64, 56, 56, 64, 3, 3, 1, 1, 2, 2),       # 28 x 28 output
    (1, 16, 23, 23, 16, 4, 4, 0, 0, 3, 3),       # stride 3, no padding
])
def test_strided_conv_without_patch_buffer_matches_oracle(cuda, oracle, shape):
    """Strides: the channels-last copy is kept as sh * sw planes of equal residues and every kernel tap reads one plane
    with a constant shift.  Against the oracle and the patch-buffer path, bit for bit."""
    import ltq
    B, Cin, H, W, Cout, kh, kw, ph, pw, sh, sw = shape
    rng = np.random.default_rng(sum(shape))
    c = dict(Cin=Cin, Cout=Cout, kh=kh, kw=kw, ph=ph, pw=pw, sh=sh, sw=sw,
             x=rng.integers(0, 256, (B, Cin, H, W), dtype=np.uint8),
             w=rng.integers(0, 256, (Cout, Cin * kh * kw), dtype=np.uint8))
    rows = [(0.02, 128), (0.005, 127), (4.0, 3)]
    qps = [ltq_qp(r) for r in rows]
    bias = rng.integers(-30000, 30000, Cout, dtype=np.int32)
    got = _conv(cuda, ltq, c, qps, flags=ltq.FLAG_BIAS_PER_CHANNEL, bias=bias)
    assert ltq.last_kernel().startswith("conv_direct_kernel<"), ltq.last_kernel()
    want = oracle.port.conv2d_q(c["x"], c["w"], Cout, kh, kw, *[qp_of(oracle, r) for r in rows], bias=bias, ph=ph, pw=pw, sh=sh,
                                sw=sw, bias_per_channel=True)
    np.testing.assert_array_equal(got, want)
    for mode in (ltq.OUT_I32, ltq.OUT_F32):
        a = _conv(cuda, ltq, c, qps, flags=ltq.FLAG_RELU, out_mode=mode)
        b = _conv(cuda, ltq, c, qps, flags=ltq.FLAG_RELU | ltq.FLAG_FORCE_SIMT, out_mode=mode)
        np.testing.assert_array_equal(a.view(np.uint32), b.view(np.uint32))
    assert ltq.lib().ltq_device_check(0, None) == 0


@pytest.mark.parametrize("shape", [(2, 64, 12, 20, 32, 3, 3, 1, 1), (1, 128, 10, 12, 128, 3, 3, 1, 1), (2, 64, 14, 14, 256, 1, 1, 0, 0)])
@pytest.mark.parametrize("mode", ["u8", "f32", "i32"])
def test_conv_channels_last_in_and_out(cuda, shape, mode):
    """LTQ_FLAG_NHWC_IN / LTQ_FLAG_NHWC_OUT: the same values as the NCHW call, only placed channels-last, in every
    combination of the two flags; refused where the layer is not computed from a channels-last copy."""
    import ltq
    B, Cin, H, W, Cout, kh, kw, ph, pw = shape
    rng = np.random.default_rng(sum(shape))
    x = cuda.from_numpy(rng.integers(0, 256, (B, Cin, H, W), dtype=np.uint8)).cuda()
    w = cuda.from_numpy(rng.integers(0, 256, (Cout, Cin * kh * kw), dtype=np.uint8)).cuda()
    bias = cuda.from_numpy(rng.integers(-30000, 30000, Cout, dtype=np.int32)).cuda()
    h = ltq.ConvHandle(0, Cin, Cout, kh, kw, ph, pw, 1, 1)
    h.set_weights(w, bias)
    h.set_qparams(ltq.QParams(0.02, 128), ltq.QParams(0.005, 127), ltq.QParams(4.0, 3))
    out_mode = {"u8": ltq.OUT_U8, "f32": ltq.OUT_F32, "i32": ltq.OUT_I32}[mode]
    base = ltq.FLAG_BIAS_PER_CHANNEL | ltq.FLAG_RELU
    ref = h.forward(x, out_mode, base)
    x_cl = x.permute(0, 2, 3, 1).contiguous()
    for fin, fout in ((True, False), (False, True), (True, True)):
        flags = base | (ltq.FLAG_NHWC_IN if fin else 0) | (ltq.FLAG_NHWC_OUT if fout else 0)
        y = h.forward(x_cl if fin else x, out_mode, flags)
        assert ltq.last_kernel().startswith("conv_direct_kernel<")
        want = ref.permute(0, 2, 3, 1).contiguous() if fout else ref
        assert cuda.equal(y, want), (fin, fout)
    if mode == "u8":
        # the same through the layer class with the reference's surface
        conv = ltq.Conv2d_q(Cin, Cout, True, kh, kw, ph, pw)
        conv.init()
        conv.get_all_weights()[0].copy_(w.view(Cout, Cin, kh * kw).cpu())
        conv.get_all_weights()[1].copy_(bias.view(1, Cout, 1, 1).cpu())
        conv.set_qparams_in(ltq.QParams(0.02, 128))
        conv.set_qparams_out(ltq.QParams(4.0, 3))
        conv.set_qparams_params([ltq.QParams(0.005, 127)], 1)
        conv.set_output(ltq.OUT_U8, relu=True, bias_per_channel=True)
        conv.to("cuda", 0)
        conv.set_layout(True, True)
        assert cuda.equal(conv.forward(x_cl), ref.permute(0, 2, 3, 1).contiguous())
    with pytest.raises(ltq.LtqError, match="channels-last"):
        h.forward(x, out_mode, base | ltq.FLAG_NHWC_OUT | ltq.FLAG_FORCE_SIMT)
    odd = ltq.ConvHandle(0, 3, 16, 3, 3, 1, 1, 1, 1)           # 3 input channels: patch-buffer path only
    odd.set_weights(cuda.zeros((16, 27), dtype=cuda.uint8, device="cuda"))
    with pytest.raises(ltq.LtqError, match="channels-last"):
        odd.forward(cuda.zeros((1, 8, 8, 3), dtype=cuda.uint8, device="cuda"), out_mode, ltq.FLAG_NHWC_IN)
    assert ltq.lib().ltq_device_check(0, None) == 0


def test_reference_bias_indexing_is_refused_beyond_its_tensor(cuda):
    import ltq
    h = ltq.ConvHandle(0, 2, 4, 3, 3)
    w = cuda.zeros((4, 18), dtype=cuda.uint8, device="cuda")
    b = cuda.zeros(4, dtype=cuda.int32, device="cuda")
    h.set_weights(w, b)
    x = cuda.zeros((1, 2, 8, 8), dtype=cuda.uint8, device="cuda")       # 36 output positions > 4 channels
    with pytest.raises(ltq.LtqError, match="output position"):
        h.forward(x)
    assert h.forward(x, flags=ltq.FLAG_BIAS_PER_CHANNEL).shape == (1, 4, 6, 6)


def test_geometry_errors(cuda):
    import ltq
    h = ltq.ConvHandle(0, 1, 1, 5, 5)
    with pytest.raises(ltq.LtqError, match="smaller than the kernel"):
        h.output_size(4, 10)
    hp = C.c_void_p()
    assert ltq.lib().ltq_conv2d_create(C.byref(hp), 0, 1, 1, 3, 3, 0, 0, 0, 1) == -1   # stride 0
    h.set_weights(cuda.zeros((1, 25), dtype=cuda.uint8, device="cuda"))
    assert h.forward(cuda.zeros((0, 1, 8, 8), dtype=cuda.uint8, device="cuda")).shape == (0, 1, 4, 4)


def test_float_and_int32_outputs_and_relu(cuda, oracle):
    """out_mode / ReLU act on the convolution exactly as on the linear layer: int32 is the corrected accumulator,
    float = (s_wt*s_in)*acc, ReLU clamps the accumulator first."""
    import ltq
    rng = np.random.default_rng(12)
    c = dict(Cin=4, Cout=9, kh=3, kw=3, ph=1, pw=1, sh=1, sw=1, x=rng.integers(0, 256, (2, 4, 10, 10), dtype=np.uint8),
             w=rng.integers(0, 256, (9, 36), dtype=np.uint8))
    rows = [(0.02, 128), (0.005, 127), (1.0, 0)]
    qps = [ltq_qp(r) for r in rows]
    acc = _conv(cuda, ltq, c, qps, out_mode=ltq.OUT_I32)
    want = np.empty_like(acc)
    for b in range(2):
        col = oracle.port.im2col(c["x"][b], 3, 3, 1, 1, 1, 1)
        want[b] = oracle.port.acc_i32(c["w"], col, 9, 100, 36, 127, 128, tA=False, tB=False).reshape(9, 10, 10)
    np.testing.assert_array_equal(acc, want)
    f = _conv(cuda, ltq, c, qps, out_mode=ltq.OUT_F32, flags=ltq.FLAG_RELU)
    sab = np.float32(0.005) * np.float32(0.02)
    np.testing.assert_array_equal(f, sab * np.maximum(want, 0).astype(np.float32))


def test_large_batch_is_processed_in_chunks_and_equals_per_image_calls(cuda):
    """Property at a size the CPU oracle cannot reach: a batch whose patch buffer exceeds one pass (256 MiB) gives, image
    by image, what single-image calls give (different chunking, different buffer offsets, same arithmetic)."""
    import ltq
    g = cuda.Generator(device="cuda").manual_seed(3)
    B, Cin, H, W, Cout = 180, 64, 56, 56, 64           # patch rows: 3136 x 576 B = 1.8 MB per image -> 148 images per pass
    x = cuda.randint(0, 256, (B, Cin, H, W), dtype=cuda.uint8, device="cuda", generator=g)
    w = cuda.randint(0, 256, (Cout, Cin * 9), dtype=cuda.uint8, device="cuda", generator=g)
    h = ltq.ConvHandle(0, Cin, Cout, 3, 3, 1, 1, 1, 1)
    h.set_weights(w)
    h.set_qparams(ltq.QParams(0.02, 128), ltq.QParams(0.005, 127), ltq.QParams(0.1, 5))
    y = h.forward(x)
    assert tuple(y.shape) == (B, Cout, H, W)
    for b in (0, 1, 147, 148, 179):
        yb = h.forward(x[b:b + 1].contiguous())
        assert cuda.equal(yb[0], y[b]), f"image {b}"
    # and the simplest cross-kernel check: the generic kernel on one image agrees with the tensor-core result
    y0 = h.forward(x[179:180].contiguous(), flags=ltq.FLAG_FORCE_SIMT)
    assert cuda.equal(y0[0], y[179])
    assert ltq.lib().ltq_device_check(0, None) == 0
