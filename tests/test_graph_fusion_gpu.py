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
}


def execute(graph, feeds, fetch):
    nodes = {n.name: n for n in graph.node}
    values = dict(feeds)
    executed = []

    def value(name):
        name = name.split(":")[0]
        if name not in values:
            n = nodes[name]
            args = [value(i) for i in n.input if not i.startswith("^")]
            values[name] = OPS[n.op](n, args)
            executed.append(n.op)
        return values[name]

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
