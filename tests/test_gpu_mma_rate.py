"""GPU: the measurement hook behind the tile-shape arguments (ott_debug_mma_rate) runs, returns plausible numbers and leaves
the context usable: an N = 256 int8 MMA occupies the tensor pipe for about 128 cycles (8192 multiply-adds per cycle and SM),
narrow ones cost more than their share."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


def test_mma_rate_probe():
    from tensor_b200 import Context, OtterB200Error
    with Context(0) as ctx:
        def rate(n, warps, lanes, ctas):
            v = C.c_float()
            ctx.check(ctx.lib.ott_debug_mma_rate(ctx.h, n, warps, lanes, ctas, 1024, C.byref(v)))
            return v.value
        wide = rate(256, 1, 1, 1)
        narrow = rate(32, 4, 1, 1)
        assert 100.0 < wide < 180.0, wide
        assert 16.0 <= narrow < wide / 2, (narrow, wide)   # 16 cycles would be the N = 32 share of the full rate
        with pytest.raises(OtterB200Error):
            ctx.check(ctx.lib.ott_debug_mma_rate(ctx.h, 24, 1, 1, 1, 1024, C.byref(C.c_float())))
        ctx.sync()
