"""GPU: the guard bands every device block carries in these tests (tests/conftest.py sets OTT_DEBUG_GUARD_BYTES; the contexts
check the bands when they are closed). Here: the check itself sees a write one byte outside a block, on either side, and a whole
forward of the benchmark graph through every kernel family leaves all bands intact."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GUARD = int(os.environ.get("OTT_DEBUG_GUARD_BYTES", "0"))


@pytest.mark.skipif(GUARD <= 0, reason="guard bands switched off")
@pytest.mark.parametrize("side", ["after", "before"])
def test_check_sees_a_write_outside_a_block(side):
    from tensor_b200 import Context, OtterB200Error
    with Context(0) as ctx:
        p = ctx.malloc(1024)  # 1024 is a whole allocation granule: the band begins right behind it
        ctx.memset(p, 0x11, 1024)
        ctx.check_guards()
        at = p + 1024 if side == "after" else p - 1
        ctx.memset(at, 0x00, 1)  # inside the allocation the driver made, outside the block the caller got
        with pytest.raises(OtterB200Error, match="outside their bounds"):
            ctx.check_guards()
        ctx.memset(at, 0xC5, 1)  # put the band back so that closing the context finds nothing
        ctx.check_guards()
        ctx.free(p)


@pytest.mark.skipif(GUARD <= 0, reason="guard bands switched off")
def test_benchmark_graph_writes_inside_its_blocks():
    """ShuffleNetV2 at the benchmarked 320x320 (first layer + pool, routed 1x1 layers, both depthwise kernels, conv5) and the
    detector (5x5 depthwise, upsample, heads): every blob, weight panel and staging block keeps its bands."""
    import bench
    for name, batch in (("shufflenetv2_320", 3), ("nanodet_plus_320", 2)):
        cfg = bench.NET_WORKLOADS[name]
        net, layers, params = bench.build_calibrated_net(cfg, batch, 0)
        try:
            x = np.random.default_rng(5).random((batch, 3, cfg["height"], cfg["width"]), dtype=np.float32)
            outs = cfg["outputs"]
            for _ in range(2):
                net.forward("data", x, list(outs))
            net.context().check_guards()
        finally:
            net.close()
