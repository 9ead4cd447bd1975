"""musa_graph_optimizer: the GraphDef wire codec, the fusion patterns and the
driver, through the C ABI on serialised GraphDef bytes.  No GPU.

Structure follows the reference's fusion tests
(test/fusion/linear_relu_fusion_test.py:56-271): a positive case per pattern
with a downstream consumer, a negative case where an intervening node blocks
the match, dtype coverage, and a check that the fused op appears under the
original node name."""
import os

import pytest

import graph_proto as gp
from graph_proto import Builder, by_name, parse
from tensorflow_musa_extension_b200 import _graph_optimizer as go
from tensorflow_musa_extension_b200 import errors


def run(builder_or_bytes, **kw):
    data = builder_or_bytes.bytes() if isinstance(builder_or_bytes, Builder) else builder_or_bytes
    out, report = go.optimize_graph_def(data, **kw)
    return parse(out), report


def bias_relu_graph(dtype=gp.DT_FLOAT, device=gp.MUSA, fmt=None):
    g = Builder()
    g.node("x", "Placeholder", device=device, dtype=dtype, shape=[8, 16])
    g.node("b", "Const", device=device, dtype=dtype)
    extra = {"data_format": fmt} if fmt else {}
    g.node("bias_add", "BiasAdd", ["x", "b"], device, T=dtype, **extra)
    g.node("act", "Relu", ["bias_add"], device, T=dtype)
    g.node("two", "Const", device=device, dtype=dtype)
    g.node("out", "Mul", ["act", "two"], device, T=dtype)   # downstream reader
    return g


# ------------------------------------------------------------------ codec --

def test_codec_round_trip_preserves_everything():
    g = Builder()
    n = g.node("weird", "SomeOp", ["a:1", "^ctrl"], gp.CPU, T=gp.DT_HALF, flag=True,
               count=-7, ratio=0.25, label="hello", shape=[2, -1, 3])
    n.attr["types"].list.type.extend([1, 19, 14])
    n.attr["names"].list.s.extend([b"p", b"q"])
    g.node("a", "Placeholder", device="", dtype=gp.DT_FLOAT)
    g.graph.version = 3
    g.graph.versions.bad_consumers.extend([5, 6])
    out, report = run(g, parameters={"disabled_fusion_patterns": "all"})
    assert report["applied"] == 0
    assert out == g.graph                     # message equality, field by field
    # and a second trip through the C++ codec is byte-stable
    again, _ = go.optimize_graph_def(out.SerializeToString(),
                                     parameters={"disabled_fusion_patterns": "all"})
    assert parse(again) == g.graph


def test_malformed_bytes_are_rejected():
    with pytest.raises(errors.InvalidArgumentError, match="malformed GraphDef"):
        go.optimize_graph_def(b"\x0a\xff\xff\xff\xff\x0f\x01")
    with pytest.raises(errors.InvalidArgumentError, match="unknown"):
        go.optimize_graph_def(b"", parameters={"no_such_parameter": "1"})


def test_empty_graph_is_a_no_op():
    out, report = run(b"")
    assert len(out.node) == 0 and report["applied"] == 0


# ---------------------------------------------------------- BiasAdd + Relu --

@pytest.mark.parametrize("dtype", [gp.DT_FLOAT, gp.DT_HALF, gp.DT_BFLOAT16])
def test_bias_add_relu_is_fused(dtype):
    out, report = run(bias_relu_graph(dtype, fmt="NHWC"))
    nodes = by_name(out)
    assert report["applied"] == 1 and report["patterns"] == {"MusaBiasAddReluFusion": 1}
    fused = nodes["act"]                       # fused op sits under the original name
    assert fused.op == "MusaBiasAddRelu" and list(fused.input) == ["x", "b"]
    assert fused.device == gp.MUSA
    assert fused.attr["T"].type == dtype and fused.attr["data_format"].s == b"NHWC"
    assert "bias_add" not in nodes and "act_original" not in nodes
    assert list(nodes["out"].input) == ["act", "two"]      # reader untouched
    assert out.versions.producer == 808


def test_bias_add_v1_and_default_format():
    g = Builder()
    g.node("x", "Placeholder", dtype=gp.DT_FLOAT)
    g.node("b", "Const", dtype=gp.DT_FLOAT)
    g.node("ba", "BiasAddV1", ["x:0", "b"], T=gp.DT_FLOAT)
    g.node("r", "Relu", ["ba:0"], T=gp.DT_FLOAT)
    nodes = by_name(run(g)[0])
    assert nodes["r"].op == "MusaBiasAddRelu" and list(nodes["r"].input) == ["x:0", "b"]
    assert nodes["r"].attr["data_format"].s == b"NHWC"


def test_intervening_identity_blocks_fusion():
    g = Builder()
    g.node("x", "Placeholder", dtype=gp.DT_FLOAT)
    g.node("b", "Const", dtype=gp.DT_FLOAT)
    g.node("ba", "BiasAdd", ["x", "b"], T=gp.DT_FLOAT)
    g.node("id", "Identity", ["ba"], T=gp.DT_FLOAT)
    g.node("r", "Relu", ["id"], T=gp.DT_FLOAT)
    out, report = run(g)
    assert report["applied"] == 0 and out == g.graph


def test_second_reader_of_bias_add_blocks_fusion():
    g = bias_relu_graph()
    g.node("peek", "Identity", ["bias_add"], T=gp.DT_FLOAT)
    out, report = run(g)
    assert report["applied"] == 0 and by_name(out)["act"].op == "Relu"
    # a control edge is a reader too
    g2 = bias_relu_graph()
    g2.node("later", "NoOp", ["^bias_add"])
    assert run(g2)[1]["applied"] == 0


@pytest.mark.parametrize("mutate", ["cpu_relu", "cpu_bias", "int32", "original_suffix",
                                    "port_one"])
def test_non_matching_variants(mutate):
    g = Builder()
    dt = gp.DT_INT32 if mutate == "int32" else gp.DT_FLOAT
    g.node("x", "Placeholder", dtype=dt)
    g.node("b", "Const", dtype=dt)
    g.node("ba", "BiasAdd", ["x", "b"], gp.CPU if mutate == "cpu_bias" else gp.MUSA, T=dt)
    name = "r_original" if mutate == "original_suffix" else "r"
    g.node(name, "Relu", ["ba:1" if mutate == "port_one" else "ba"],
           gp.CPU if mutate == "cpu_relu" else gp.MUSA, T=dt)
    out, report = run(g)
    assert report["applied"] == 0 and out == g.graph


def test_control_inputs_are_carried_over():
    g = Builder()
    g.node("x", "Placeholder", dtype=gp.DT_FLOAT)
    g.node("b", "Const", dtype=gp.DT_FLOAT)
    g.node("init", "NoOp")
    g.node("ba", "BiasAdd", ["x", "b", "^init"], T=gp.DT_FLOAT)
    g.node("r", "Relu", ["ba"], T=gp.DT_FLOAT)
    nodes = by_name(run(g)[0])
    assert list(nodes["r"].input) == ["x", "b", "^init"] and "init" in nodes


def test_optimizer_is_idempotent():
    once, _ = go.optimize_graph_def(bias_relu_graph().bytes())
    twice, report = go.optimize_graph_def(once)
    assert report["applied"] == 0 and parse(twice) == parse(once)


# ---------------------------------------------------------------- swish ----

@pytest.mark.parametrize("x_first", [True, False])
@pytest.mark.parametrize("dtype", [gp.DT_FLOAT, gp.DT_HALF, gp.DT_BFLOAT16])
def test_swish_chain_is_fused(x_first, dtype):
    g = Builder()
    g.node("x", "Placeholder", dtype=dtype)
    g.node("b", "Const", dtype=dtype)
    g.node("ba", "BiasAdd", ["x", "b"], T=dtype, data_format="NHWC")
    g.node("sig", "Sigmoid", ["ba"], T=dtype)
    g.node("y", "Mul", ["x", "sig"] if x_first else ["sig", "x:0"], T=dtype)
    g.node("sink", "Identity", ["y"], T=dtype)
    out, report = run(g)
    nodes = by_name(out)
    assert report["patterns"] == {"MusaBiasAddSwishFusion": 1}
    assert nodes["y"].op == "MusaBiasAddSwish" and list(nodes["y"].input) == ["x", "b"]
    assert set(nodes) == {"x", "b", "y", "sink"}


def test_swish_needs_the_same_tensor_on_both_sides():
    g = Builder()
    g.node("x", "Placeholder", dtype=gp.DT_FLOAT)
    g.node("z", "Placeholder", dtype=gp.DT_FLOAT)
    g.node("b", "Const", dtype=gp.DT_FLOAT)
    g.node("ba", "BiasAdd", ["x", "b"], T=gp.DT_FLOAT)
    g.node("sig", "Sigmoid", ["ba"], T=gp.DT_FLOAT)
    g.node("y", "Mul", ["z", "sig"], T=gp.DT_FLOAT)
    nodes = by_name(run(g)[0])
    # not a swish; the Sigmoid(BiasAdd) inside it is still a chain of its own
    assert nodes["y"].op == "Mul" and nodes["sig"].op == "MusaBiasAddSigmoid"
    assert list(nodes["y"].input) == ["z", "sig"]


def test_sigmoid_chain_and_priorities():
    names = [(n, p) for n, p, _ in go.list_fusion_patterns()]
    assert names == [("MusaBiasAddSwishFusion", 56), ("MusaBiasAddReluFusion", 55),
                     ("MusaBiasAddSigmoidFusion", 54), ("MusaBiasAddReluGradFusion", 53),
                     ("MusaAdamMixedFusion", 40)]
    g = Builder()
    g.node("x", "Placeholder", dtype=gp.DT_HALF)
    g.node("b", "Const", dtype=gp.DT_HALF)
    g.node("ba", "BiasAdd", ["x", "b"], T=gp.DT_HALF)
    g.node("s", "Sigmoid", ["ba"], T=gp.DT_HALF)
    nodes = by_name(run(g)[0])
    assert nodes["s"].op == "MusaBiasAddSigmoid" and "ba" not in nodes


# ---------------------------------------------------------------- Adam -----

def adam_graph(src=gp.DT_BFLOAT16, extra_cast_reader=False, adam_t=gp.DT_FLOAT):
    g = Builder()
    for n in ("var", "m", "v"):
        g.node(n, "VarHandleOp", dtype=gp.DT_FLOAT)
    for n in ("b1p", "b2p", "lr", "b1", "b2", "eps"):
        g.node(n, "Const", dtype=gp.DT_FLOAT)
    g.node("grad16", "Placeholder", dtype=src)
    g.node("cast", "Cast", ["grad16"], SrcT=src, DstT=gp.DT_FLOAT)
    g.node("adam", "ResourceApplyAdam",
           ["var", "m", "v", "b1p", "b2p", "lr", "b1", "b2", "eps", "cast"],
           T=adam_t, use_locking=True, use_nesterov=False)
    if extra_cast_reader:
        g.node("norm", "L2Loss", ["cast"], T=gp.DT_FLOAT)
    return g


@pytest.mark.parametrize("src", [gp.DT_BFLOAT16, gp.DT_HALF])
def test_adam_mixed_rewrite(src):
    out, report = run(adam_graph(src))
    nodes = by_name(out)
    assert report["patterns"] == {"MusaAdamMixedFusion": 1}
    adam = nodes["adam"]
    assert adam.op == "MusaResourceApplyAdamMixed" and adam.attr["T"].type == src
    assert adam.input[9] == "grad16" and len(adam.input) == 10
    assert adam.attr["use_locking"].b is True and adam.attr["use_nesterov"].b is False
    assert "cast" not in nodes and "grad16" in nodes


def test_adam_keeps_a_cast_that_has_another_reader():
    nodes = by_name(run(adam_graph(extra_cast_reader=True))[0])
    assert nodes["adam"].op == "MusaResourceApplyAdamMixed"
    assert "cast" in nodes and list(nodes["norm"].input) == ["cast"]


def test_adam_not_rewritten_for_float_grad_or_16bit_state():
    assert run(adam_graph(src=gp.DT_FLOAT))[1]["applied"] == 0
    assert run(adam_graph(adam_t=gp.DT_BFLOAT16))[1]["applied"] == 0
    g = adam_graph()
    by_name(g.graph)["adam"].device = gp.CPU
    assert run(g)[1]["applied"] == 0


def test_adam_kill_switch(monkeypatch):
    monkeypatch.setenv("MUSA_DISABLE_ADAM_MIXED_FUSION", "1")
    out, report = run(adam_graph())
    assert report["applied"] == 0 and report["fallbacks"] >= 1
    assert by_name(out)["adam"].op == "ResourceApplyAdam"
    monkeypatch.setenv("MUSA_DISABLE_ADAM_MIXED_FUSION", "0")
    assert run(adam_graph())[1]["applied"] == 1


# ---------------------------------------------------- driver and parameters --

def many_chains(n):
    g = Builder()
    g.node("b", "Const", dtype=gp.DT_FLOAT)
    prev = "x0"
    g.node(prev, "Placeholder", dtype=gp.DT_FLOAT)
    for i in range(n):
        g.node("ba%d" % i, "BiasAdd", [prev, "b"], T=gp.DT_FLOAT)
        g.node("r%d" % i, "Relu", ["ba%d" % i], T=gp.DT_FLOAT)
        prev = "r%d" % i
    return g


def test_fixed_point_over_many_chains():
    out, report = run(many_chains(40))
    nodes = by_name(out)
    assert report["applied"] == 40 and not report["hit_iteration_limit"]
    assert all(nodes["r%d" % i].op == "MusaBiasAddRelu" for i in range(40))
    assert nodes["r5"].input[0] == "r4" and len(nodes) == 42


@pytest.mark.parametrize("value,fused", [
    ("MusaBiasAddReluFusion", False), ("  musabiasaddrelufusion ,MusaAdamMixedFusion", False),
    ("all", False), (" ALL ", False), ("MusaAdamMixedFusion", True), ("", True)])
def test_disabled_fusion_patterns_parameter(value, fused):
    out, _ = run(bias_relu_graph(), parameters={"disabled_fusion_patterns": value})
    assert (by_name(out)["act"].op == "MusaBiasAddRelu") == fused


def test_set_pattern_enabled():
    lib = go._graph_lib()
    assert lib.MusaGraphSetPatternEnabled(b"NoSuchPattern", 0) == 5
    assert lib.MusaGraphSetPatternEnabled(b"MusaBiasAddReluFusion", 0) == 0
    try:
        assert run(bias_relu_graph())[1]["applied"] == 0
    finally:
        lib.MusaGraphSetPatternEnabled(b"MusaBiasAddReluFusion", 1)
    assert run(bias_relu_graph())[1]["applied"] == 1


def test_biasadd_kill_switch(monkeypatch):
    monkeypatch.setenv("MUSA_DISABLE_BIASADD_ACT_FUSION", "true")
    assert run(bias_relu_graph())[1]["applied"] == 0


# ------------------------------------------- ReluGrad -> BiasAddGrad backward --

def relu_grad_graph(dtype=gp.DT_FLOAT, fmt=None, reader=True, relu_grad_reader=True,
                    bias_grad_device=gp.MUSA):
    g = Builder()
    g.node("dy", "Placeholder", dtype=dtype)
    g.node("y", "Placeholder", dtype=dtype)
    g.node("w", "Placeholder", dtype=dtype)
    g.node("dz", "ReluGrad", ["dy", "y"], T=dtype)
    extra = {"data_format": fmt} if fmt else {}
    g.node("db", "BiasAddGrad", ["dz"], bias_grad_device, T=dtype, **extra)
    if relu_grad_reader:
        g.node("dx", "MatMul", ["dz", "w"], T=dtype)       # the layer's input gradient
    if reader:
        g.node("lr", "Const", dtype=dtype)
        g.node("step", "Mul", ["db", "lr"], T=dtype)       # reads the bias gradient
    return g


@pytest.mark.parametrize("dtype", [gp.DT_FLOAT, gp.DT_HALF, gp.DT_BFLOAT16])
@pytest.mark.parametrize("fmt", [None, "NHWC", "NCHW"])
def test_relu_grad_bias_add_grad_is_fused(dtype, fmt):
    out, report = run(relu_grad_graph(dtype, fmt))
    nodes = by_name(out)
    assert report["patterns"] == {"MusaBiasAddReluGradFusion": 1}
    fused = nodes["dz"]                        # takes the ReluGrad's name
    assert fused.op == "MusaBiasAddReluGrad" and list(fused.input) == ["dy", "y"]
    assert fused.device == gp.MUSA and fused.attr["T"].type == dtype
    assert fused.attr["data_format"].s == (fmt or "NHWC").encode()
    assert "db" not in nodes and "dz_original" not in nodes
    assert list(nodes["dx"].input) == ["dz", "w"]          # output 0: backprops
    assert list(nodes["step"].input) == ["dz:1", "lr"]     # output 1: bias gradient


def test_relu_grad_fusion_moves_control_edges():
    g = relu_grad_graph()
    g.node("gate", "NoOp")
    g.node("late", "NoOp", ["^db"])
    for n in g.graph.node:
        if n.name == "db":
            n.input.append("^gate")
    nodes = by_name(run(g)[0])
    assert list(nodes["dz"].input) == ["dy", "y", "^gate"]
    assert list(nodes["late"].input) == ["^dz"]


@pytest.mark.parametrize("kw", [dict(reader=False), dict(bias_grad_device=gp.CPU),
                                dict(dtype=gp.DT_DOUBLE)])
def test_relu_grad_fusion_non_matching_variants(kw):
    g = relu_grad_graph(**kw)
    out, report = run(g)
    assert report["patterns"].get("MusaBiasAddReluGradFusion", 0) == 0
    assert by_name(out)["db"].op == "BiasAddGrad"


def test_bias_add_grad_of_another_producer_is_left_alone():
    g = Builder()
    g.node("dy", "Placeholder", dtype=gp.DT_FLOAT)
    g.node("db", "BiasAddGrad", ["dy"], T=gp.DT_FLOAT)
    g.node("lr", "Const", dtype=gp.DT_FLOAT)
    g.node("step", "Mul", ["db", "lr"], T=gp.DT_FLOAT)
    assert run(g)[1]["applied"] == 0


def test_relu_grad_fusion_is_idempotent_and_has_a_kill_switch(monkeypatch):
    once, _ = go.optimize_graph_def(relu_grad_graph().bytes())
    twice, report = go.optimize_graph_def(once)
    assert report["applied"] == 0 and parse(twice) == parse(once)
    monkeypatch.setenv("MUSA_DISABLE_BIASADD_RELU_GRAD_FUSION", "1")
    assert run(relu_grad_graph())[1]["applied"] == 0


def test_forward_and_backward_chains_fuse_in_one_run():
    g = Builder()
    for name in ("x", "b", "dy", "w"):
        g.node(name, "Placeholder", dtype=gp.DT_HALF)
    g.node("z", "BiasAdd", ["x", "b"], T=gp.DT_HALF)
    g.node("y", "Relu", ["z"], T=gp.DT_HALF)
    g.node("dz", "ReluGrad", ["dy", "y"], T=gp.DT_HALF)
    g.node("db", "BiasAddGrad", ["dz"], T=gp.DT_HALF)
    g.node("dx", "MatMul", ["dz", "w"], T=gp.DT_HALF)
    g.node("loss", "Mul", ["y", "db"], T=gp.DT_HALF)
    out, report = run(g)
    assert report["patterns"] == {"MusaBiasAddReluFusion": 1, "MusaBiasAddReluGradFusion": 1}
    nodes = by_name(out)
    assert nodes["y"].op == "MusaBiasAddRelu" and nodes["dz"].op == "MusaBiasAddReluGrad"
    assert list(nodes["dz"].input) == ["dy", "y"] and list(nodes["loss"].input) == ["y", "dz:1"]


# ------------------------------------------------------ Python config layer --

def test_config_helpers_mirror_the_reference_api():
    cfg = go.enable_musa_graph_optimizer(add_to_optimizer_list=True,
                                         disabled_fusion_patterns=[" A ", "b,c", "A"])
    ro = cfg.graph_options.rewrite_options
    assert go.is_musa_graph_optimizer_enabled(cfg)
    assert ro.optimizers == [go.MUSA_GRAPH_OPTIMIZER_NAME]
    assert go.get_musa_disabled_fusion_patterns(cfg) == ["A", "b", "c"]
    go.set_musa_disabled_fusion_patterns(cfg, "x, all ,y")
    assert go.get_musa_disabled_fusion_patterns(cfg) == ["all"]
    go.clear_musa_disabled_fusion_patterns(cfg)
    assert go.get_musa_disabled_fusion_patterns(cfg) == []
    go.enable_musa_graph_optimizer(cfg)       # enabling twice keeps one entry
    assert len(ro.custom_optimizers) == 1
    go.disable_musa_graph_optimizer(cfg)
    assert not go.is_musa_graph_optimizer_enabled(cfg) and ro.optimizers == []
    assert go._graph_lib().MusaGraphOptimizerName() == b"musa_graph_optimizer"


def test_config_drives_the_optimizer():
    data = bias_relu_graph().bytes()
    off = go.disable_musa_graph_optimizer()
    assert go.optimize_graph_def(data, config=off)[0] == data
    on = go.enable_musa_graph_optimizer()
    assert by_name(parse(go.optimize_graph_def(data, config=on)[0]))["act"].op == "MusaBiasAddRelu"
    go.disable_musa_fusion_patterns("MusaBiasAddReluFusion", on)
    assert by_name(parse(go.optimize_graph_def(data, config=on)[0]))["act"].op == "Relu"


# ------------------------------------------------------------ graph dumps --

def test_graph_dump_files(tmp_path):
    d = tmp_path / "dumps"
    go.enable_musa_graph_dump(str(d), dump_text=True, dump_slim=True)
    try:
        assert go.is_musa_graph_dump_enabled() and go.get_musa_graph_dump_directory() == str(d)
        assert go.is_musa_graph_dump_text_enabled() and go.is_musa_graph_dump_slim_enabled()
        g = bias_relu_graph(gp.DT_HALF, fmt="NHWC")
        out, report = run(g)
        assert report["applied"] == 1
        names = sorted(p.name for p in d.iterdir())
        ids = {n.split("_")[3] for n in names}
        assert len(ids) == 1 and len(next(iter(ids))) == 4          # one run, id width 4
        rid = next(iter(ids))
        for stage in ("initial", "before_fusion", "after_fusion", "final"):
            for ext in (".pb", ".slim.pb", ".pbtxt"):
                assert "musa_graph_optimizer_%s_%s%s" % (rid, stage, ext) in names
        base = d / ("musa_graph_optimizer_%s_" % rid)
        # the binary dumps are the graphs themselves
        assert parse((d / ("musa_graph_optimizer_%s_initial.pb" % rid)).read_bytes()) == g.graph
        assert parse((d / ("musa_graph_optimizer_%s_final.pb" % rid)).read_bytes()) == out
        text = (d / ("musa_graph_optimizer_%s_final.pbtxt" % rid)).read_text()
        assert 'op: "MusaBiasAddRelu"' in text and 'name: "act"' in text
        assert 's: "NHWC"' in text and "type: DT_HALF" in text
        slim = parse((d / ("musa_graph_optimizer_%s_initial.slim.pb" % rid)).read_bytes())
        full = {n.name: n for n in g.graph.node}
        for n in slim.node:
            assert n.op == full[n.name].op and list(n.input) == list(full[n.name].input)
            assert "shape" not in n.attr                               # non-scalar attrs dropped
        assert any("shape" in n.attr for n in g.graph.node)
        # a second run gets the next id
        run(g)
        ids2 = {p.name.split("_")[3] for p in d.iterdir()}
        assert len(ids2) == 2
    finally:
        go.clear_musa_graph_dump_config()


def test_graph_dump_environment_and_override(tmp_path, monkeypatch):
    go.clear_musa_graph_dump_config()
    monkeypatch.delenv("MUSA_DUMP_GRAPHDEF", raising=False)
    assert not go.is_musa_graph_dump_enabled() and go.get_musa_graph_dump_directory() == "."
    monkeypatch.setenv("MUSA_DUMP_GRAPHDEF", "1")
    monkeypatch.setenv("MUSA_DUMP_GRAPHDEF_DIR", str(tmp_path))
    monkeypatch.setenv("MUSA_DUMP_GRAPHDEF_SLIM", "true")
    assert go.is_musa_graph_dump_enabled() and go.get_musa_graph_dump_directory() == str(tmp_path)
    assert go.is_musa_graph_dump_slim_enabled() and not go.is_musa_graph_dump_text_enabled()
    run(bias_relu_graph())
    assert any(p.name.endswith("_final.pb") for p in tmp_path.iterdir())
    # the programmatic setting wins over the environment until it is cleared
    go.disable_musa_graph_dump()
    try:
        assert not go.is_musa_graph_dump_enabled()
        before = len(list(tmp_path.iterdir()))
        run(bias_relu_graph())
        assert len(list(tmp_path.iterdir())) == before
    finally:
        go.clear_musa_graph_dump_config()
    assert go.is_musa_graph_dump_enabled()


def test_allow_growth_switch(monkeypatch):
    monkeypatch.delenv("TF_FORCE_GPU_ALLOW_GROWTH", raising=False)
    go.set_musa_allow_growth(False)
    assert not go.get_musa_allow_growth()
    go.set_musa_allow_growth(True)
    assert go.get_musa_allow_growth()
    monkeypatch.setenv("TF_FORCE_GPU_ALLOW_GROWTH", "false")
    assert not go.get_musa_allow_growth()                  # the environment wins
    monkeypatch.setenv("TF_FORCE_GPU_ALLOW_GROWTH", "maybe")
    assert go.get_musa_allow_growth()                      # unparsable: ignored
    go.set_musa_allow_growth(False)
