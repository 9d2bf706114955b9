"""GPU: a tensor larger than 4 GiB through the tensor-core 1x1 kernel: pixel indices beyond 2^26 and byte offsets beyond 2^32
on both sides (TMA coordinates, the output stage's pointer arithmetic), checked on sampled pixels against the CPU checker."""
import numpy as np
import pytest

from support import ACT_RELU, ConvCase, run_port

pytestmark = pytest.mark.gpu


def test_one_by_one_layer_beyond_4_gib():
    from gpu_support import make_layer
    from tensor_b200 import S8_NHWC, Context
    c = 64
    case = ConvCase("big_pw", c, c, 1, n=1, h=8, w=8, int8_scale_term=101, act_type=ACT_RELU, s8_input=True, seed=123).make()
    n, h, w = 17, 2048, 2048  # 71.3 M pixels x 64 B = 4.56 GB in, as much out
    pixels = n * h * w
    block_px = 1 << 22          # the input is one random 256 MiB block repeated: pixel p holds block[p % block_px]
    block = np.random.default_rng(99).integers(-127, 128, size=(block_px, c), dtype=np.int8)
    with Context(0) as ctx:
        layer = make_layer(ctx, case, 0)
        xd, od = ctx.malloc(pixels * c), ctx.malloc(pixels * c)
        try:
            import ctypes as C
            for p0 in range(0, pixels, block_px):
                m = min(block_px, pixels - p0)
                ctx.check(ctx.lib.ott_memcpy_h2d(ctx.h, C.c_void_p(xd + p0 * c), block.ctypes.data_as(C.c_void_p), m * c))
            ctx.sync()
            ctx.memset(od, 0x7B, pixels * c)
            layer.forward(xd, S8_NHWC, n, h, w, od, S8_NHWC)
            ctx.sync()
            edge = (1 << 32) // c  # first pixel whose byte offset needs 33 bits
            rng = np.random.default_rng(100)
            sample = np.unique(np.concatenate([np.arange(0, 130), np.arange(edge - 130, edge + 130), np.arange(pixels - 130, pixels),
                                               rng.integers(0, pixels, size=600)]))
            got = np.stack([ctx.to_host(od + int(p) * c, (c,), np.int8) for p in sample])
            probe = ConvCase("big_pw_probe", c, c, 1, n=1, h=1, w=len(sample), int8_scale_term=101, act_type=ACT_RELU, s8_input=True, seed=123).make()
            probe.weight, probe.bias, probe.w_scales = case.weight, case.bias, case.w_scales
            probe.in_scales, probe.out_scales = case.in_scales, case.out_scales
            probe.x_s8 = np.ascontiguousarray(block[sample % block_px].T.reshape(1, c, 1, len(sample)))
            want = run_port(probe, 0, want_acc=False)["y"]  # [1, c, 1, S]
            assert np.array_equal(got, want[0, :, 0, :].T)
            assert np.count_nonzero(got) > got.size // 8  # a real result, not the fill or zeros
        finally:
            ctx.free(xd)
            ctx.free(od)
            layer.close()


@pytest.mark.parametrize("tensor_cores", [2, 0], ids=["dw_umma", "depthwise_tiled"])
def test_depthwise_layer_beyond_4_gib(tensor_cores):
    """The same for a depthwise 3x3 layer on either kernel (tensor cores: 4-D TMA boxes per image; CUDA cores: plane tiles):
    sampled interior pixels, their 3x3 neighbourhoods cut out as 3x3 images for the checker (no padding, one output each)."""
    import ctypes as C
    from gpu_support import make_layer
    from tensor_b200 import S8_NHWC, Context
    c = 64
    kw = dict(groups=c, int8_scale_term=101, act_type=ACT_RELU, s8_input=True, w_std=0.1, seed=124)
    case = ConvCase("big_dw", c, c, 3, pad=1, n=1, h=8, w=8, **kw).make()
    n, h, w = 17, 2048, 2048
    pixels, img_px = n * h * w, h * w
    image = np.random.default_rng(98).integers(-127, 128, size=(h, w, c), dtype=np.int8)  # every image of the batch is this one
    with Context(0) as ctx:
        ctx.check(ctx.lib.ott_set_depthwise_tensor_cores(ctx.h, tensor_cores))
        layer = make_layer(ctx, case, 0)
        xd, od = ctx.malloc(pixels * c), ctx.malloc(pixels * c)
        try:
            for i in range(n):
                ctx.check(ctx.lib.ott_memcpy_h2d(ctx.h, C.c_void_p(xd + i * img_px * c), image.ctypes.data_as(C.c_void_p), img_px * c))
            ctx.sync()
            ctx.memset(od, 0x7B, pixels * c)
            layer.forward(xd, S8_NHWC, n, h, w, od, S8_NHWC)
            ctx.sync()
            edge = (1 << 32) // c
            rng = np.random.default_rng(101)
            cand = np.unique(np.concatenate([np.arange(edge - 200, edge + 200), np.arange(pixels - 3 * w, pixels - w),
                                             rng.integers(0, pixels, size=800)]))
            yy, xx = (cand % img_px) // w, cand % w
            sample = cand[(yy >= 1) & (yy < h - 1) & (xx >= 1) & (xx < w - 1)]
            assert len(sample) > 600 and (sample > edge).any() and (sample < edge).any()
            got = np.stack([ctx.to_host(od + int(p) * c, (c,), np.int8) for p in sample])
            sy, sx = (sample % img_px) // w, sample % w
            patches = np.stack([image[y - 1:y + 2, x - 1:x + 2, :] for y, x in zip(sy, sx)])  # [S, 3, 3, c]
            probe = ConvCase("big_dw_probe", c, c, 3, pad=0, n=len(sample), h=3, w=3, **kw).make(dry_run=False)
            probe.weight, probe.bias, probe.w_scales = case.weight, case.bias, case.w_scales
            probe.in_scales, probe.out_scales = case.in_scales, case.out_scales
            probe.x_s8 = np.ascontiguousarray(patches.transpose(0, 3, 1, 2))
            want = run_port(probe, 0, want_acc=False)["y"]  # [S, c, 1, 1]
            assert np.array_equal(got, want[:, :, 0, 0])
            assert np.count_nonzero(got) > got.size // 8
        finally:
            ctx.free(xd)
            ctx.free(od)
            layer.close()
