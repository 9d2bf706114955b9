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
