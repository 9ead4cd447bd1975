"""Generates the golden vectors under tests/golden/ (run once, by hand, on a
machine that has the reference checkout; the .npz files are committed).

    python tests/golden/make_golden.py /path/to/reference [adam|bn|elementwise|bias_grad|optimizers|row_norm|adagrad ...]

What pins what:
  adam_reference_numpy.npz
      Expected values computed by the REFERENCE's own NumPy statement of the
      Adam update, `MusaResourceSparseApplyAdamTest._compute_expected`
      (test/ops/musa_resource_sparse_apply_adam_op_test.py:35-69), taken from
      the reference file with `ast` (the module itself imports TensorFlow, which
      is not installed) and run on seeded inputs with indices = arange(n), i.e.
      as a dense update.  Includes the |1 - beta1^t| < 1e-10 first-step case.
  bn_torch_cpu.npz
      FusedBatchNorm forward/gradient cases at the shapes of the reference
      tests (test/ops/fused_batchnorm_op_test.py:25-55, 97-141, 178-216,
      358-448; test/ops/fused_batchnorm_hcnw_op_test.py:86-107), answered by an
      INDEPENDENT implementation: PyTorch's CPU batch_norm in float64 and its
      autograd.  TensorFlow's CPU kernel, the stated oracle, is not available;
      these vectors pin the restatement to a second implementation, not to
      TensorFlow.
  elementwise_literals.npz
      The literal inputs of the reference's Relu / Sigmoid / BiasAdd tests
      (test/ops/relu_op_test.py:58-96, test/ops/sigmoid_op_test.py:58-93,
      test/ops/biasadd_op_test.py:74-116) with closed-form float64 answers.
  bias_grad_torch_cpu.npz
      BiasAddGrad / ReluGrad cases at the shapes of the reference test
      (test/ops/biasadd_grad_op_test.py:16-86: NHWC [2,8,8,32], NCHW
      [2,32,8,8]) plus a ragged 2-D case, answered by PyTorch's CPU autograd of
      relu(x + b) in float64: an independent implementation, not TensorFlow.
  optimizer_cases.npz
      Nadam at the shapes and hyper-parameters of the reference test
      (test/ops/resource_apply_nadam_op_test.py:26-40, 88-106) with the formula
      that test states (:57-67), RMSProp / centered RMSProp and gradient descent
      at the literal inputs of their tests (test/ops/apply_rmsprop_op_test.py:
      77-199, 256-330; test/ops/apply_gradient_descent_op_test.py:64-78,
      97-101), all evaluated in float64.  The reference tests compare with
      TensorFlow's CPU ops on a live device and hold no expected values.
  adagrad_reference_numpy.npz
      AdagradV2 answered by the REFERENCE's own NumPy statement of the update,
      `_expected_apply_adagrad_v2` (test/ops/apply_adagrad_op_test.py:53-62),
      taken from the reference file with `ast` and evaluated in float64 on the
      test's literal cases and on seeded random inputs.
  row_norm_torch_cpu.npz
      LayerNorm forward / gradient at shapes of the reference test
      (test/ops/layernorm_op_test.py:143-157, 211-240: [16,32], [8,16,32],
      [32,128], [2,4,8,16], [100,1], [100,2], [1,1], [10,8192] (2 rows of it)) and RMSNorm
      forward / gradient, answered by PyTorch's CPU layer_norm / rms_norm in
      float64 and its autograd: an independent implementation.
"""
import ast
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_adam_fn(reference_root):
    path = os.path.join(reference_root, "test", "ops",
                        "musa_resource_sparse_apply_adam_op_test.py")
    tree = ast.parse(open(path).read())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "_compute_expected":
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"np": np}
            exec(compile(mod, path, "exec"), ns)
            return ns["_compute_expected"]
    raise RuntimeError("_compute_expected not found in " + path)


def make_adam(reference_root):
    fn = reference_adam_fn(reference_root)
    rng = np.random.default_rng(3)
    out = {}
    cases = [
        # name, n, beta1_power, beta2_power
        ("step10", 4099, 0.9 ** 10, 0.999 ** 10),
        ("first_step_guard", 257, 1.0, 1.0),
        ("step1", 1024, 0.9, 0.999),
    ]
    for name, n, b1p, b2p in cases:
        var = rng.normal(0, 0.05, n).astype(np.float32)
        m = rng.normal(0, 1e-4, n).astype(np.float32)
        v = rng.uniform(0, 1e-6, n).astype(np.float32)
        grad = rng.normal(0, 1e-3, n).astype(np.float32)
        lr, b1, b2, eps = (np.float32(1e-3), np.float32(0.9), np.float32(0.999),
                           np.float32(1e-7))
        ev, em, evv = fn(None, var, m, v, lr, b1, b2, eps, np.float32(b1p),
                         np.float32(b2p), grad, np.arange(n))
        out.update({
            name + "/var": var, name + "/m": m, name + "/v": v, name + "/grad": grad,
            name + "/scalars": np.array([b1p, b2p, lr, b1, b2, eps], np.float32),
            name + "/expected_var": ev.astype(np.float32),
            name + "/expected_m": em.astype(np.float32),
            name + "/expected_v": evv.astype(np.float32),
        })
    np.savez_compressed(os.path.join(HERE, "adam_reference_numpy.npz"), **out)


def make_bn():
    import torch
    import torch.nn.functional as F

    rng = np.random.default_rng(11)
    out = {}
    # name, shape, data_format, mean, std
    cases = [
        ("nhwc_2x2x2x4", (2, 2, 2, 4), "NHWC", 0.0, 1.0),
        ("nhwc_4x5x3x16", (4, 5, 3, 16), "NHWC", 0.5, 2.0),
        ("keras2d_512x64", (512, 1, 1, 64), "NHWC", 0.0, 1.0),
        ("nchw_2x3x4x5", (2, 3, 4, 5), "NCHW", 0.0, 1.0),
        ("nchw_2x32x1x1", (2, 32, 1, 1), "NCHW", 0.0, 1.0),
        ("nhwc_2x1x1x32", (2, 1, 1, 32), "NHWC", 0.0, 1.0),
        ("nchw_large_var_8x6x16x16", (8, 6, 16, 16), "NCHW", 3.0, 30.0),
        ("nhwc_large_mean_64x3x3x8", (64, 3, 3, 8), "NHWC", 1000.0, 1.0),
    ]
    eps = 1e-3
    for name, shape, fmt, mu, sd in cases:
        x = (rng.standard_normal(shape) * sd + mu).astype(np.float32)
        c = shape[-1] if fmt == "NHWC" else shape[1]
        scale = rng.uniform(0.5, 1.5, c).astype(np.float32)
        offset = rng.normal(0, 0.1, c).astype(np.float32)
        dy = rng.standard_normal(shape).astype(np.float32)
        xt = torch.from_numpy(x).double()
        if fmt == "NHWC":
            xt = xt.permute(0, 3, 1, 2)
            dyt = torch.from_numpy(dy).double().permute(0, 3, 1, 2)
        else:
            dyt = torch.from_numpy(dy).double()
        xt = xt.contiguous().requires_grad_(True)
        st = torch.from_numpy(scale).double().requires_grad_(True)
        ot = torch.from_numpy(offset).double().requires_grad_(True)
        y = F.batch_norm(xt, None, None, st, ot, training=True, eps=eps)
        y.backward(dyt.contiguous())
        red = (0, 2, 3)
        mean = xt.detach().mean(dim=red)
        var = xt.detach().var(dim=red, unbiased=False)
        count = xt.numel() // c
        unbiased = var * count / (count - 1) if count > 1 else var

        def back(t):
            t = t.detach()
            if fmt == "NHWC":
                t = t.permute(0, 2, 3, 1)
            return t.contiguous().numpy().astype(np.float32)

        out.update({
            name + "/x": x, name + "/scale": scale, name + "/offset": offset,
            name + "/dy": dy, name + "/format": np.array(fmt),
            name + "/y": back(y), name + "/mean": mean.numpy().astype(np.float32),
            name + "/var_pop": var.numpy().astype(np.float32),
            name + "/var_unbiased": unbiased.numpy().astype(np.float32),
            name + "/dx": back(xt.grad),
            name + "/dscale": st.grad.numpy().astype(np.float32),
            name + "/doffset": ot.grad.numpy().astype(np.float32),
        })
    np.savez_compressed(os.path.join(HERE, "bn_torch_cpu.npz"), **out)


def make_elementwise():
    out = {}
    relu_in = np.array([-2.0, -1.0, 0.0, 1.0, 2.0], np.float32)
    out["relu/in"] = relu_in
    out["relu/out"] = np.array([0.0, 0.0, 0.0, 1.0, 2.0], np.float32)
    sig_in = np.array([-100.0, -10.0, -1.0, 0.0, 1.0, 10.0, 100.0], np.float64)
    out["sigmoid/in"] = sig_in.astype(np.float32)
    with np.errstate(over="ignore"):
        out["sigmoid/out"] = 1.0 / (1.0 + np.exp(-sig_in))
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    b = np.array([0.5, -1.0, 2.0, 10.0], np.float32)
    out["biasadd/x"] = x
    out["biasadd/b"] = b
    out["biasadd/out_nhwc"] = x + b
    xn = np.arange(48, dtype=np.float32).reshape(2, 3, 2, 4)
    bn = np.array([1.0, -2.0, 3.0], np.float32)
    out["biasadd/x_nchw"] = xn
    out["biasadd/b_nchw"] = bn
    out["biasadd/out_nchw"] = xn + bn.reshape(1, 3, 1, 1)
    xi = np.arange(12, dtype=np.int32).reshape(3, 4)
    bi = np.array([1, -1, 2, -2], np.int32)
    out["biasadd/x_i32"] = xi
    out["biasadd/b_i32"] = bi
    out["biasadd/out_i32"] = xi + bi
    np.savez_compressed(os.path.join(HERE, "elementwise_literals.npz"), **out)


def make_bias_grad():
    import torch
    rng = np.random.default_rng(77)
    out = {}
    cases = [("nhwc", (2, 8, 8, 32), "NHWC"), ("nchw", (2, 32, 8, 8), "NCHW"),
             ("ragged2d", (37, 24), "NHWC")]
    for name, shape, fmt in cases:
        ax = 1 if fmt == "NCHW" else len(shape) - 1
        for dt_name, tdt in (("f32", torch.float32), ("f16", torch.float16),
                             ("bf16", torch.bfloat16)):
            # Inputs are rounded to the storage type first, so every dtype sees
            # values that it can hold exactly.
            x = torch.from_numpy(rng.standard_normal(shape)).to(tdt)
            b = torch.from_numpy(rng.standard_normal(shape[ax]) * 0.5).to(tdt)
            dy = torch.from_numpy(rng.standard_normal(shape)).to(tdt)
            view = [1] * len(shape)
            view[ax] = shape[ax]
            z = (x.double() + b.double().reshape(view)).to(tdt)  # BiasAdd in T
            zt = z.double().requires_grad_(True)
            y = torch.relu(zt)
            y.backward(dy.double())
            dz = zt.grad                      # = ReluGrad(dy, y)
            red = [i for i in range(len(shape)) if i != ax]
            db = dz.sum(dim=red)              # = BiasAddGrad(dz)
            key = "%s/%s" % (name, dt_name)
            out[key + "/features"] = y.detach().float().numpy()
            out[key + "/gradients"] = dy.float().numpy()
            out[key + "/backprops"] = dz.float().numpy()
            out[key + "/bias_grad"] = db.numpy()
            out[key + "/dy_colsum"] = dy.double().sum(dim=red).numpy()
    np.savez_compressed(os.path.join(HERE, "bias_grad_torch_cpu.npz"), **out)


def reference_method(reference_root, rel_path, name):
    """A method of a reference test class, taken out of its file with `ast`
    (the module itself imports TensorFlow) and turned into a plain function."""
    path = os.path.join(reference_root, *rel_path.split("/"))
    tree = ast.parse(open(path).read())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == name:
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"np": np}
            exec(compile(mod, path, "exec"), ns)
            return ns[name]
    raise RuntimeError("%s not found in %s" % (name, path))


def make_adagrad(reference_root):
    """Expected values from the REFERENCE's own NumPy statement of AdagradV2
    (test/ops/apply_adagrad_op_test.py:53-62), on the literal cases of that
    test (:94-112) and on seeded inputs as its shape test draws them
    (:136-147)."""
    fn = reference_method(reference_root, "test/ops/apply_adagrad_op_test.py",
                          "_expected_apply_adagrad_v2")
    out = {}
    cases = {
        "vector": ([1.0, -2.0, 3.5, -4.5], [0.1, 0.2, 0.3, 0.4], 0.01, 1e-7,
                   [0.5, -1.0, 2.0, 0.25]),
        "matrix": ([[1.0, 2.0], [3.0, 4.0]], [[0.1, 0.1], [0.1, 0.1]], 0.01, 1e-7,
                   [[0.2, 0.4], [0.6, 0.8]]),
    }
    rng = np.random.default_rng(42)
    for shape in ((1024,), (33, 65), (4, 8, 16)):
        cases["random_" + "x".join(map(str, shape))] = (
            rng.random(shape), rng.random(shape) + 0.01, 0.01, 1e-7, rng.random(shape) * 0.1)
    for name, (var, accum, lr, eps, grad) in cases.items():
        var, accum, grad = (np.asarray(a, np.float32) for a in (var, accum, grad))
        want_var, want_accum = fn(None, var.astype(np.float64), accum.astype(np.float64),
                                  np.float64(np.float32(lr)), np.float64(np.float32(eps)),
                                  grad.astype(np.float64))
        k = "adagrad/" + name
        out.update({k + "/var": var, k + "/accum": accum, k + "/grad": grad,
                    k + "/hyper": np.array([np.float32(lr), np.float32(eps)], np.float64),
                    k + "/var_out": want_var, k + "/accum_out": want_accum})
    np.savez_compressed(os.path.join(HERE, "adagrad_reference_numpy.npz"), **out)


def make_optimizers():
    out = {}
    rng = np.random.default_rng(123)
    f8 = np.float64
    # Nadam: uniform inputs as the reference test draws them.
    for name, shape in (("basic", (128, 128)), ("small", (7,)), ("half", (64, 64))):
        var = rng.uniform(-1, 1, shape).astype(np.float32)
        m = rng.uniform(-1, 1, shape).astype(np.float32)
        v = rng.uniform(0.1, 1, shape).astype(np.float32)
        g = rng.uniform(-1, 1, shape).astype(np.float32)
        b1p, b2p, lr, b1, b2, eps = 0.9, 0.99, 0.01, 0.9, 0.99, 1e-8
        m_new = b1 * m.astype(f8) + (1 - b1) * g.astype(f8)
        v_new = b2 * v.astype(f8) + (1 - b2) * np.square(g.astype(f8))
        m_hat = (b1 * m_new + (1 - b1) * g.astype(f8)) / (1 - b1p)
        v_hat = v_new / (1 - b2p)
        var_new = var.astype(f8) - lr * m_hat / (np.sqrt(v_hat) + eps)
        k = "nadam/" + name
        out.update({k + "/var": var, k + "/m": m, k + "/v": v, k + "/grad": g,
                    k + "/hyper": np.array([b1p, b2p, lr, b1, b2, eps]),
                    k + "/var_out": var_new, k + "/m_out": m_new, k + "/v_out": v_new})
    # RMSProp: literal cases of the reference test.
    rms_cases = {
        "basic": ([1.0, 2.0, 3.0, 4.0], [0, 0, 0, 0], [0, 0, 0, 0], [0.1, 0.2, 0.3, 0.4],
                  (0.01, 0.9, 0.9, 1e-8)),
        "dtypes": ([1.0, 2.0, 3.0, 4.0], [0.1, 0.2, 0.3, 0.4], [0, 0, 0, 0],
                   [0.1, 0.2, 0.3, 0.4], (0.01, 0.9, 0.9, 1e-7)),
        "zero_grad": ([1.0, 2.0, 3.0, 4.0], [0.5, 0.6, 0.7, 0.8], [0, 0, 0, 0], [0, 0, 0, 0],
                      (0.01, 0.9, 0.9, 1e-7)),
        "negative_grad": ([1.0, 2.0, 3.0, 4.0], [0, 0, 0, 0], [0, 0, 0, 0],
                          [-10.0, -5.0, -2.0, -1.0], (0.01, 0.9, 0.9, 1e-7)),
    }
    for name, (var, ms, mom, g, (lr, rho, mo, eps)) in rms_cases.items():
        var, ms, mom, g = (np.array(a, np.float32) for a in (var, ms, mom, g))
        ms_new = rho * ms.astype(f8) + (1 - rho) * np.square(g.astype(f8))
        mom_new = mo * mom.astype(f8) + lr * g.astype(f8) / np.sqrt(ms_new + eps)
        k = "rmsprop/" + name
        out.update({k + "/var": var, k + "/ms": ms, k + "/mom": mom, k + "/grad": g,
                    k + "/hyper": np.array([lr, rho, mo, eps]),
                    k + "/var_out": var.astype(f8) - mom_new, k + "/ms_out": ms_new,
                    k + "/mom_out": mom_new})
    crms_cases = {
        "basic": ([1.0, 2.0, 3.0, 4.0], [0] * 4, [0] * 4, [0] * 4, [0.1, 0.2, 0.3, 0.4],
                  (0.01, 0.9, 0.9, 1e-8)),
        "dtypes": ([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [0] * 6, [0.1, 0.2, 0.3, 0.4, 0.5, 0.6],
                   [0] * 6, [0.1, 0.2, 0.3, 0.4, 0.5, 0.6], (0.01, 0.9, 0.9, 1e-7)),
    }
    for name, (var, mg, ms, mom, g, (lr, rho, mo, eps)) in crms_cases.items():
        var, mg, ms, mom, g = (np.array(a, np.float32) for a in (var, mg, ms, mom, g))
        mg_new = rho * mg.astype(f8) + (1 - rho) * g.astype(f8)
        ms_new = rho * ms.astype(f8) + (1 - rho) * np.square(g.astype(f8))
        mom_new = mo * mom.astype(f8) + lr * g.astype(f8) / np.sqrt(
            ms_new - np.square(mg_new) + eps)
        k = "centered_rmsprop/" + name
        out.update({k + "/var": var, k + "/mg": mg, k + "/ms": ms, k + "/mom": mom,
                    k + "/grad": g, k + "/hyper": np.array([lr, rho, mo, eps]),
                    k + "/var_out": var.astype(f8) - mom_new, k + "/mg_out": mg_new,
                    k + "/ms_out": ms_new, k + "/mom_out": mom_new})
    sgd_cases = {
        "vector": ([1.0, -2.0, 3.5, -4.5], 0.1, [0.5, -1.0, 2.0, 0.25]),
        "matrix": ([[1.0, 2.0], [3.0, 4.0]], 0.25, [[0.2, 0.4], [0.6, 0.8]]),
        "locking": ([1.25, -2.5, 5.0, -10.0], 0.5, [0.5, 0.25, -1.0, 2.0]),
    }
    for name, (var, alpha, g) in sgd_cases.items():
        var, g = np.array(var, np.float32), np.array(g, np.float32)
        k = "sgd/" + name
        out.update({k + "/var": var, k + "/grad": g, k + "/alpha": np.float64(alpha),
                    k + "/var_out": var.astype(f8) - np.float64(np.float32(alpha)) * g.astype(f8)})
    np.savez_compressed(os.path.join(HERE, "optimizer_cases.npz"), **out)


def make_row_norm():
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(321)
    out = {}
    shapes = {"s16x32": (16, 32), "s8x16x32": (8, 16, 32), "s32x128": (32, 128),
              "s2x4x8x16": (2, 4, 8, 16), "s100x1": (100, 1), "s100x2": (100, 2),
              "s1x1": (1, 1), "s2x8192": (2, 8192), "s7x1000": (7, 1000)}
    for name, shape in shapes.items():
        n = shape[-1]
        x = rng.uniform(-2, 2, shape).astype(np.float32)
        dy = rng.uniform(-1, 1, shape).astype(np.float32)
        gamma = rng.uniform(0.5, 1.5, n).astype(np.float32)
        beta = rng.uniform(-0.5, 0.5, n).astype(np.float32)
        eps = 1e-5
        xt = torch.from_numpy(x).double().requires_grad_(True)
        gt = torch.from_numpy(gamma).double().requires_grad_(True)
        bt = torch.from_numpy(beta).double().requires_grad_(True)
        y = F.layer_norm(xt, (n,), gt, bt, eps)
        y.backward(torch.from_numpy(dy).double())
        k = "layer_norm/" + name
        out.update({k + "/x": x, k + "/dy": dy, k + "/gamma": gamma, k + "/beta": beta,
                    k + "/y": y.detach().numpy(), k + "/dx": xt.grad.numpy(),
                    k + "/dgamma": gt.grad.numpy(), k + "/dbeta": bt.grad.numpy()})
        xt2 = torch.from_numpy(x).double().requires_grad_(True)
        g2 = torch.from_numpy(gamma).double()
        y2 = F.rms_norm(xt2, (n,), g2, eps)
        y2.backward(torch.from_numpy(dy).double())
        inv = torch.rsqrt(xt2.detach().pow(2).mean(-1, keepdim=True) + eps)
        k = "rms_norm/" + name
        out.update({k + "/y": y2.detach().numpy(), k + "/normalized": (xt2.detach() * inv).numpy(),
                    k + "/inv_rms": inv.numpy(), k + "/dx": xt2.grad.numpy()})
    np.savez_compressed(os.path.join(HERE, "row_norm_torch_cpu.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    which = sys.argv[2:] or ["adam", "bn", "elementwise", "bias_grad", "optimizers", "row_norm", "adagrad"]
    if "adam" in which:
        make_adam(sys.argv[1])
    if "bn" in which:
        make_bn()
    if "elementwise" in which:
        make_elementwise()
    if "bias_grad" in which:
        make_bias_grad()
    if "optimizers" in which:
        make_optimizers()
    if "row_norm" in which:
        make_row_norm()
    if "adagrad" in which:
        make_adagrad(sys.argv[1])
    print("wrote golden vectors to", HERE)
