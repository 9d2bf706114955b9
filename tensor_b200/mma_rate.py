"""Prints the table behind the tile-shape arguments of the tensor-core kernels: cycles one tcgen05.mma kind::i8 (M = 128,
K = 32) occupies an SM, by N, issuing warps x lanes and CTAs per SM (ott_debug_mma_rate).

    python -m tensor_b200.mma_rate
"""
import ctypes as C

from .capi import Context


def table(device=0, reps=2048):
    rows = []
    with Context(device) as ctx:
        for ctas in (1, 2):
            for n in (32, 64, 128, 256):
                for warps, lanes in ((1, 1), (1, 2), (2, 1), (4, 1)):
                    v = C.c_float()
                    ctx.check(ctx.lib.ott_debug_mma_rate(ctx.h, n, warps, lanes, ctas, reps, C.byref(v)))
                    rows.append((n, warps, lanes, ctas, v.value))
    return rows


if __name__ == "__main__":
    print("N  issuing_warps  lanes_per_warp  ctas_per_sm  cycles_per_mma_per_sm")
    for n, warps, lanes, ctas, cyc in table():
        print(f"{n:<3d} {warps:<14d} {lanes:<15d} {ctas:<12d} {cyc:.1f}")
