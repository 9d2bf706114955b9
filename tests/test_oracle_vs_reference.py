"""The C restatement against the compiled reference, live. Skipped where oracle/_ref/ has not been
built (it needs the reference's sources); the frozen fixtures in tests/golden/ cover that situation."""
import numpy as np
import pytest

from cases import small_cases
from support import ROUND_ADD_HALF_TRUNC, ROUND_HALF_AWAY, ConvCase, ACT_RELU, have_ref, run_port, run_ref

pytestmark = pytest.mark.skipif(not have_ref(), reason="oracle/_ref/libotter_ref.so not built")


def bits(a):
    return a.view(np.int32) if a.dtype == np.float32 else a


@pytest.mark.parametrize("case,path", [cp for cp in small_cases() if not cp[1].startswith("port")],
                         ids=[c.name for c, p in small_cases() if not p.startswith("port")])
def test_port_equals_reference(case, path):
    case.make()
    packed = path.startswith("packed")
    got = run_port(case, ROUND_ADD_HALF_TRUNC if packed else ROUND_HALF_AWAY)
    want = run_ref(case, packed)
    for k in ("xq", "acc", "y"):
        assert np.array_equal(bits(got[k]), bits(want[k])), k


def test_packed_and_unpacked_reference_agree_where_both_valid():
    case = ConvCase("both", 64, 64, 3, 1, 1, n=1, h=12, w=12, int8_scale_term=101, act_type=ACT_RELU, seed=77).make()
    a, b = run_ref(case, True), run_ref(case, False)
    assert np.array_equal(a["acc"], b["acc"]) and np.array_equal(a["y"], b["y"])


def test_batch_is_a_loop_of_single_images():
    case = ConvCase("batch", 32, 32, 3, 1, 1, n=3, h=6, w=6, int8_scale_term=2, seed=78).make()
    whole = run_port(case)
    for i in range(case.n):
        one = ConvCase("one", 32, 32, 3, 1, 1, n=1, h=6, w=6, int8_scale_term=2, seed=78).make()
        one.x_f32 = np.ascontiguousarray(case.x_f32[i:i + 1])
        one.in_scales = case.in_scales
        ref = run_ref(one, True)
        assert np.array_equal(whole["y"][i:i + 1].view(np.int32), ref["y"].view(np.int32))
