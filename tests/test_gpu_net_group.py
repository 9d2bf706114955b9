"""GPU: a group of Net replicas behind one forward call (ott_net_group_*). Two replicas, each with its own context, stream,
allocator and weights, are built on device 0 (the box has one GPU; on a multi-GPU box the same code takes distinct devices);
a host batch is cut between them and the gathered outputs must equal the unsharded forward bit for bit."""
import numpy as np
import pytest

from graph_walk import calibrate
from tensor_b200 import graphs

pytestmark = pytest.mark.gpu


def _build_group(L, params, n_members):
    from tensor_b200 import NetGroup
    group = NetGroup([0] * n_members)
    for net in group.members:
        for l in L:
            net.add_layer(**l)
        net.compile()
        for name, p in params.items():
            net.set_conv_params(name, p["weight"], p["bias"], p["w_scales"], p["in_scales"], p["out_scales"])
    return group


@pytest.mark.parametrize("n,members", [(5, 2), (3, 3), (1, 2), (261, 2)])
def test_group_forward_equals_unsharded_forward(n, members):
    from graph_support import build_net, oracle_conv_for_calibration
    L = graphs.shufflenetv2_layers(64, 64, batch=1, stage_repeats=(2, 2, 2))
    params = graphs.make_params(L, seed=41)
    x4 = np.random.default_rng(42).uniform(0, 1, size=(4, 3, 64, 64)).astype(np.float32)
    calibrate(L, params, x4[:1], oracle_conv_for_calibration)
    x = np.ascontiguousarray(x4[np.arange(n) % 4])
    blobs = ["s3b1_shuf", "conv5"]
    single = build_net(L, params)
    want = single.forward("data", x4, blobs)
    single.close()
    group = _build_group(L, params, members)
    for _ in range(2):  # the second call reuses what the first one set up (captured chunk forwards for the 261-image case)
        got = group.forward("data", x, blobs)
        for b, g, w in zip(blobs, got, want):
            assert g.shape == (n,) + w.shape[1:], b
            for i in range(n):
                assert np.array_equal(g[i].view(np.int32), w[i % 4].view(np.int32)), f"blob {b}, image {i}"
    group.close()


def test_group_reports_a_member_s_failure():
    from tensor_b200 import NetGroup, OtterB200Error
    group = NetGroup([0, 0])
    with pytest.raises(OtterB200Error):  # nothing compiled yet: the blob is unknown
        group.forward("data", np.zeros((2, 3, 8, 8), np.float32), ["nope"])
    group.close()
