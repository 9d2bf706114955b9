"""The C restatement (oracle/) against the frozen outputs of the compiled reference (tests/golden/)."""
import ctypes as C
import hashlib

import numpy as np
import pytest

from cases import small_cases
from support import GOLDEN_DIR, ROUND_ADD_HALF_TRUNC, ROUND_HALF_AWAY, _p, load_port, rounding_for, run_port

GOLD = np.load(GOLDEN_DIR / "conv_int8_small.npz")
ADV = np.load(GOLDEN_DIR / "epilogue_adversarial.npz")


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def bits(a):
    return a.view(np.int32) if a.dtype == np.float32 else a


@pytest.mark.parametrize("case,path", small_cases(), ids=[c.name for c, _ in small_cases()])
def test_port_matches_golden(case, path):
    case.make()
    want_inputs = bytes(GOLD[case.name + "/inputs_sha256"]).decode()
    assert digest(case.weight, case.bias, case.w_scales, case.in_scales, case.out_scales, case.x_f32, case.x_s8) == want_inputs, \
        "seeded inputs differ from the ones the fixtures were generated with (numpy random stream changed?)"
    rounding = rounding_for(path)
    got = run_port(case, rounding)
    assert digest(got["xq"]) == bytes(GOLD[case.name + "/xq_sha256"]).decode()
    assert digest(got["acc"]) == bytes(GOLD[case.name + "/acc_sha256"]).decode()
    want = GOLD[case.name + "/y"]
    assert got["y"].dtype == want.dtype and got["y"].shape == want.shape
    assert np.array_equal(bits(got["y"]), bits(want))  # bit-exact, fp32 included


def test_adversarial_set_is_adversarial():
    """The fixture must contain accumulators on which a separate multiply+add differs from the fused one."""
    acc, s, b = ADV["acc"], ADV["scale_in"], ADV["bias"]
    mul_add = (acc.astype(np.float32) * s[:, None, None]) + b[:, None, None]
    assert (mul_add.view(np.int32) != ADV["dequant_packed"].view(np.int32)).sum() > 10


@pytest.mark.parametrize("tag,rounding", [("packed", ROUND_ADD_HALF_TRUNC), ("unpacked", ROUND_HALF_AWAY)])
def test_port_epilogues_match_golden(tag, rounding):
    lib = load_port()
    acc, s, b, so = ADV["acc"], ADV["scale_in"], ADV["bias"], ADV["scale_out"]
    c, _, hw = acc.shape
    y = np.empty((1, c, hw), np.float32)
    lib.orc_dequantize(_p(acc, C.c_int32), 1, c, hw, _p(s, C.c_float), c, _p(b, C.c_float), c, 0, C.c_float(0), _p(y, C.c_float))
    assert np.array_equal(y.reshape(c, 1, hw).view(np.int32), ADV[f"dequant_{tag}"].view(np.int32))
    for act, slope in ((0, 0.0), (1, 0.0), (2, 0.1), (3, 0.0)):
        q = np.empty((1, c, hw), np.int8)
        lib.orc_requantize(_p(acc, C.c_int32), 1, c, hw, _p(s, C.c_float), c, _p(so, C.c_float), 1, _p(b, C.c_float), c,
                           act, C.c_float(slope), rounding, _p(q, C.c_int8))
        assert np.array_equal(q.reshape(c, 1, hw), ADV[f"requant_act{act}_{tag}"]), f"act {act}"


@pytest.mark.parametrize("tag,rounding", [("packed", ROUND_ADD_HALF_TRUNC), ("unpacked", ROUND_HALF_AWAY)])
def test_port_quantize_ties(tag, rounding):
    lib = load_port()
    ties = ADV["ties"]
    q = np.empty(ties.shape, np.int8)
    one = np.ones((1,), np.float32)
    lib.orc_quantize(_p(ties, C.c_float), 1, ties.shape[0], ties.shape[1], ties.shape[2], _p(one, C.c_float), 1, rounding, _p(q, C.c_int8))
    want = ADV[f"ties_q_{tag}"]
    # |x| >= 2^31 is outside every real activation range; the reference's answer there is an x86 artefact
    ok = np.abs(ties) < 2.0e9
    assert np.array_equal(q[ok], want[ok])


def test_two_rounding_rules_differ_only_at_one_float():
    lib = load_port()
    v = np.float32(0.49999997)
    assert lib.orc_float2int8(v, ROUND_ADD_HALF_TRUNC) == 1 and lib.orc_float2int8(v, ROUND_HALF_AWAY) == 0
    xs = np.linspace(-130, 130, 100001, dtype=np.float32)
    for x in xs[::97]:
        assert lib.orc_float2int8(float(x), 0) == lib.orc_float2int8(float(x), 1)
    assert lib.orc_float2int8(-1000.0, 0) == -127 and lib.orc_float2int8(1000.0, 1) == 127
