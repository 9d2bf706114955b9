"""The `.otter` model-structure reader (C++ side) against the writer in tensor_b200.graphs and, where the reference
checkout is present, against the reference's own shipped int8 graph file."""
import os
from pathlib import Path

import pytest

from tensor_b200 import graphs
from tensor_b200.capi import parse_otter_text

REF_GRAPH = Path(os.environ.get("OTTER_REFERENCE", "/root/reference")) / "benchmark" / "nanodet-plus-m-1.5x_416_int8_fused.otter"


@pytest.fixture(scope="module", autouse=True)
def built():
    from tensor_b200.build import build
    build()


def test_writer_reader_round_trip():
    layers = graphs.shufflenetv2_layers(96, 128, batch=4)
    got = parse_otter_text(graphs.to_otter_text(layers))
    assert len(got) == len(layers)
    for want, g in zip(layers, got):
        assert {k: str(v) for k, v in want.items()} == g


def test_syntax_details():
    text = '''name: "a file-level key is ignored"
    # a comment line
    Convolution { name: c1  input: "a, b"   Param { out_channels: 8  kernel: 3 } activation: LRelu }
    Concat{name:cat input:"c1,c1" Param{axis:1}}
    $ Input { name: never_read }
    '''
    got = parse_otter_text(text)
    assert got == [dict(type="Convolution", name="c1", input="a, b", out_channels="8", kernel="3", activation="LRelu"),
                   dict(type="Concat", name="cat", input="c1,c1", axis="1")]
    from tensor_b200 import OtterB200Error
    with pytest.raises(OtterB200Error):
        parse_otter_text("Convolution { name c1 }")


@pytest.mark.skipif(not REF_GRAPH.exists(), reason="reference checkout not present")
def test_reads_the_reference_s_own_int8_graph():
    got = parse_otter_text(REF_GRAPH.read_text())
    kinds = {}
    for l in got:
        kinds[l["type"]] = kinds.get(l["type"], 0) + 1
    assert kinds == {"Input": 1, "Convolution": 110, "MaxPool": 1, "Concat": 28, "ChannelShuffle": 16, "Crop": 26, "ShortCut": 5,
                     "Upsample": 2, "NanodetPlusDetectionOutput": 1}
    conv4 = next(l for l in got if l.get("name") == "conv_4")
    assert conv4["int8_scale_term"] == "102" and conv4["activation"] == "LRelu" and conv4["input"] == "pool_1"
    cat = next(l for l in got if l.get("name") == "concat_1")
    assert cat["input"] == "conv_3, conv_6"


def _canonical(layers):
    """Layers with blob names replaced by the index of the layer that produced them, so that two files which differ only in
    names compare equal."""
    ids, out = {}, []
    for l in layers:
        ins = [t.strip() for t in l.get("input", "").split(",") if t.strip()]
        sig = {k: (f"{float(v):.6f}" if k.endswith("_threshold") else v) for k, v in l.items() if k not in ("name", "input", "output", "batchsize")}
        sig["in"] = tuple(ids[i] for i in ins)
        ids[l.get("output", l.get("name"))] = len(ids)
        out.append(sig)
    return out


@pytest.mark.skipif(not REF_GRAPH.exists(), reason="reference checkout not present")
@pytest.mark.parametrize("flavour", ["fused", "mixed"])
def test_generator_reproduces_the_reference_s_shipped_detector(flavour):
    """graphs.shipped_nanodet_plus_layers is layer for layer (types, parameters, wiring; 190 layers) the graph the reference
    ships as benchmark/nanodet-plus-m-1.5x_416_int8_{fused,mixed}.otter, so the GPU parity test of that description
    (tests/test_gpu_bench_geometry.py) runs the reference's own model structure."""
    ref = parse_otter_text(REF_GRAPH.with_name(f"nanodet-plus-m-1.5x_416_int8_{flavour}.otter").read_text())
    gen = parse_otter_text(graphs.to_otter_text(graphs.shipped_nanodet_plus_layers(mixed=flavour == "mixed")))
    assert len(ref) == len(gen) == 190
    for i, (a, b) in enumerate(zip(_canonical(ref), _canonical(gen))):
        assert a == b, f"layer {i} ({ref[i].get('name')}) differs"
