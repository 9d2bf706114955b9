"""Freeze the reference's own answer for the detector it ships (benchmark/nanodet-plus-m-1.5x_416_int8_fused.otter) as a
golden fixture: graph_support.shipped_nanodet_case (that graph, seeded parameters, one 416x416 image) through the compiled
reference's Net (oracle/_ref/libotter_ref.so: load_otter -> Extractor).

    python tests/golden/make_golden_shipped.py

Writes tests/golden/net_nanodet_shipped_416.npz: the heads of the three coarser levels in full, a SHA-256 digest of every
head (the stride-8 head is 1.2 MB; its digest is enough for a bit-exact comparison) and a digest of the inputs.
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent.parent))
from graph_support import reference_net_forward, shipped_nanodet_case  # noqa: E402
from support import GOLDEN_DIR  # noqa: E402


def sha(a) -> np.ndarray:
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest().encode(), dtype=np.uint8)


def main():
    L, params, x, heads = shipped_nanodet_case()
    got = reference_net_forward(L, params, x, heads)
    h = hashlib.sha256(np.ascontiguousarray(x).tobytes())
    for k in sorted(params):
        h.update(np.ascontiguousarray(params[k]["weight"]).tobytes())
        h.update(np.ascontiguousarray(params[k]["in_scales"]).tobytes())
    out = {"input_sha256": np.frombuffer(h.hexdigest().encode(), dtype=np.uint8)}
    for name in heads:
        out[name + "_sha256"] = sha(got[name])
        out[name + "_shape"] = np.array(got[name].shape, np.int32)
        if name != heads[0]:
            out[name] = got[name]
    np.savez_compressed(GOLDEN_DIR / "net_nanodet_shipped_416.npz", **out)
    print("net_nanodet_shipped_416.npz", (GOLDEN_DIR / "net_nanodet_shipped_416.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
