"""The rewritten graph computes what the original graph computes: both are run
node by node through the op front end on the GPU (the reference's fusion tests
compare the fused run with the un-fused CPU run and look for the fused op in
the executed graph, test/fusion/linear_relu_fusion_test.py:104-141)."""
import numpy as np
import pytest

import graph_proto as gp
from graph_proto import Builder, parse
from helpers import RTOL, assert_close, np_dtype, to_numpy, to_torch
from oracle import np_ref
from tensorflow_musa_extension_b200 import _graph_optimizer as go
from tensorflow_musa_extension_b200 import raw_ops

pytestmark = pytest.mark.gpu

OPS = {
    "BiasAdd": lambda n, a: raw_ops.BiasAdd(a[0], a[1]),
    "Relu": lambda n, a: raw_ops.Relu(a[0]),
    "Sigmoid": lambda n, a: raw_ops.Sigmoid(a[0]),
    "Mul": lambda n, a: a[0] * a[1],
    "MusaBiasAddRelu": lambda n, a: raw_ops.MusaBiasAddRelu(a[0], a[1]),
    "MusaBiasAddSwish": lambda n, a: raw_ops.MusaBiasAddSwish(a[0], a[1]),
    "MusaBiasAddSigmoid": lambda n, a: raw_ops.MusaBiasAddSigmoid(a[0], a[1]),
    "ReluGrad": lambda n, a: raw_ops.ReluGrad(a[0], a[1]),
    "BiasAddGrad": lambda n, a: raw_ops.BiasAddGrad(a[0]),
    "MusaBiasAddReluGrad": lambda n, a: tuple(raw_ops.MusaBiasAddReluGrad(a[0], a[1])),
    "Add": lambda n, a: a[0] + a[1],
}


def execute(graph, feeds, fetch):
    nodes = {n.name: n for n in graph.node}
    values = dict(feeds)
    executed = []

    def value(tensor):
        name, _, port = tensor.partition(":")
        if name not in values:
            n = nodes[name]
            args = [value(i) for i in n.input if not i.startswith("^")]
            values[name] = OPS[n.op](n, args)
            executed.append(n.op)
        out = values[name]
        if isinstance(out, tuple):
            return out[int(port or 0)]
        assert not port or port == "0"
        return out

    return value(fetch), executed


@pytest.mark.parametrize("dtype,code", [("float32", gp.DT_FLOAT), ("float16", gp.DT_HALF),
                                        ("bfloat16", gp.DT_BFLOAT16)])
def test_fused_graph_matches_unfused_graph(kernel_lib, dtype, code):
    g = Builder()
    g.node("x", "Placeholder", dtype=code)
    g.node("b1", "Placeholder", dtype=code)
    g.node("b2", "Placeholder", dtype=code)
    g.node("ba1", "BiasAdd", ["x", "b1"], T=code)
    g.node("h", "Relu", ["ba1"], T=code)
    g.node("ba2", "BiasAdd", ["h", "b2"], T=code)
    g.node("sig", "Sigmoid", ["ba2"], T=code)
    g.node("y", "Mul", ["h", "sig"], T=code)
    rewritten, report = go.optimize_graph_def(g.bytes())
    assert report["patterns"] == {"MusaBiasAddReluFusion": 1, "MusaBiasAddSwishFusion": 1}

    rng = np.random.default_rng(5)
    dt = np_dtype(dtype)
    x = rng.standard_normal((300, 64)).astype(dt)
    b1 = rng.normal(0, 0.3, 64).astype(dt)
    b2 = rng.normal(0, 0.3, 64).astype(dt)
    feeds = {"x": to_torch(x), "b1": to_torch(b1), "b2": to_torch(b2)}
    plain, ops_plain = execute(g.graph, feeds, "y")
    fused, ops_fused = execute(parse(rewritten), feeds, "y")
    assert sorted(ops_fused) == ["MusaBiasAddRelu", "MusaBiasAddSwish"]
    assert len(ops_plain) == 5
    rt, at = (RTOL["f32_elementwise"], 1e-6) if dtype == "float32" else (RTOL["lowp"], 1e-3)
    assert_close(to_numpy(fused), to_numpy(plain), rt, at, "fused vs un-fused")
    h = np_ref.bias_add_relu(x, b1)
    assert_close(to_numpy(fused), np_ref.bias_add_swish(h, b2), rt, at, "fused vs oracle")


@pytest.mark.parametrize("dtype,code", [("float32", gp.DT_FLOAT), ("float16", gp.DT_HALF),
                                        ("bfloat16", gp.DT_BFLOAT16)])
def test_fused_backward_graph_matches_unfused_graph(kernel_lib, dtype, code):
    """Forward chain and its backward in one graph; the fetched value depends
    on both outputs of the fused backward op."""
    g = Builder()
    for name in ("x", "b", "dy"):
        g.node(name, "Placeholder", dtype=code)
    g.node("z", "BiasAdd", ["x", "b"], T=code)
    g.node("y", "Relu", ["z"], T=code)
    g.node("dz", "ReluGrad", ["dy", "y"], T=code)
    g.node("db", "BiasAddGrad", ["dz"], T=code)
    g.node("out", "Add", ["dz", "db"], T=code)       # broadcasts db over the rows
    rewritten, report = go.optimize_graph_def(g.bytes())
    assert report["patterns"] == {"MusaBiasAddReluFusion": 1, "MusaBiasAddReluGradFusion": 1}

    rng = np.random.default_rng(6)
    dt = np_dtype(dtype)
    x = rng.standard_normal((500, 48)).astype(dt)
    b = rng.normal(0, 0.3, 48).astype(dt)
    dy = rng.standard_normal((500, 48)).astype(dt)
    feeds = {"x": to_torch(x), "b": to_torch(b), "dy": to_torch(dy)}
    plain, ops_plain = execute(g.graph, feeds, "out")
    fused, ops_fused = execute(parse(rewritten), feeds, "out")
    assert sorted(ops_fused) == ["Add", "MusaBiasAddRelu", "MusaBiasAddReluGrad"]
    assert sorted(ops_plain) == ["Add", "BiasAdd", "BiasAddGrad", "Relu", "ReluGrad"]
    rt, at = (RTOL["f32_bn"], 1e-4) if dtype == "float32" else (RTOL["lowp"], 0.15)
    assert_close(to_numpy(fused), to_numpy(plain), rt, at, "fused vs un-fused")
    want_dx, want_db = np_ref.bias_add_relu_grad(dy, np_ref.bias_add_relu(x, b))
    want = want_dx.astype(np.float64) + want_db.astype(np.float64)
    assert_close(to_numpy(fused), want, rt, at, "fused vs oracle")
