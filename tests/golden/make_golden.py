"""Build the committed golden vectors for the matmul hot path.

Run in a checkout that has the reference mounted:

    python tests/golden/make_golden.py <path to the Tensotron checkout>

Two sources go into tests/golden/*.json:

1. The reference's own torch fixtures that pin this path
   (tests/Tensotron.Tests/Fixtures/{matmul,matmul_nd,add,unary,losses,optim,conv}.json).
   Only the cases on the path are kept.  Every kept case is re-computed with the
   local torch (same version as the fixtures' torch_version) and must reproduce the
   recorded output and gradients, so a drifted fixture cannot slip in.
2. Larger seeded cases the reference tests only against an in-test naive loop with
   .NET's System.Random (TiledMatMulTests 96x80x112, MatMulNtOpTests 5x7x3,
   BatchedCuBlasMatMulTests 3x64x64x80, the Linear fwd+bwd config).  The .NET bit
   stream cannot be regenerated without .NET, so these use the same shapes with
   numpy-seeded inputs; expected values come from torch float64 on those inputs.

The tests read only the JSON; nothing at test time needs the reference tree.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _t(x):
    return {"shape": list(x.shape), "data": [float(v) for v in x.detach().reshape(-1).tolist()]}


def _close(a, b, what):
    a = torch.as_tensor(a, dtype=torch.float32).reshape(-1)
    b = torch.as_tensor(b, dtype=torch.float32).reshape(-1)
    assert a.shape == b.shape, what
    assert torch.allclose(a, b, atol=1e-6, rtol=1e-6), what


def _inputs(case):
    return [torch.tensor(i["data"], dtype=torch.float32).reshape(i["shape"]).requires_grad_(True)
            for i in case["inputs"]]


def _recheck(case, fn):
    ins = _inputs(case)
    out = fn(*ins)
    go = torch.tensor(case["grad_output"]["data"], dtype=torch.float32).reshape(case["grad_output"]["shape"])
    out.backward(go)
    _close(out, case["output"]["data"], case["name"] + " output")
    for i, g in zip(ins, case["grads"]):
        _close(i.grad, g["data"], case["name"] + " grad")


def from_reference(ref_root):
    fx = os.path.join(ref_root, "tests", "Tensotron.Tests", "Fixtures")
    load = lambda op: json.load(open(os.path.join(fx, op + ".json")))
    out = {"torch_version": torch.__version__, "tolerance": {"atol": 2e-4, "rtol": 2e-4}, "groups": {}}

    mm = load("matmul")
    assert mm["torch_version"].split("+")[0] == torch.__version__.split("+")[0]
    for c in mm["cases"]:
        _recheck(c, lambda a, b: a @ b)
    out["groups"]["matmul"] = mm["cases"]

    nd = load("matmul_nd")
    for c in nd["cases"]:
        _recheck(c, (lambda a, b: torch.outer(a, b)) if c["meta"]["op"] == "outer" else (lambda a, b: a @ b))
    out["groups"]["matmul_nd"] = nd["cases"]

    add = [c for c in load("add")["cases"] if c["name"] == "2x3 + 3 (broadcast row)"]
    assert len(add) == 1
    _recheck(add[0], lambda a, b: a + b)
    out["groups"]["bias_add"] = add

    un = [c for c in load("unary")["cases"] if c["meta"]["op"] in ("relu", "tanh")]
    assert len(un) == 3
    for c in un:
        _recheck(c, torch.relu if c["meta"]["op"] == "relu" else torch.tanh)
    out["groups"]["activation"] = un

    ce = [c for c in load("losses")["cases"] if c["meta"]["op"] == "cross_entropy"]
    assert len(ce) == 2
    for c in ce:
        idx = torch.tensor(c["meta"]["index"])
        _recheck(c, lambda x, idx=idx, red=c["meta"]["reduction"]:
                 torch.nn.functional.cross_entropy(x, idx, reduction=red))
    out["groups"]["cross_entropy"] = ce

    adam = [c for c in load("optim")["cases"] if c["name"] in ("adam lr0.05", "adam wd")]
    assert len(adam) == 2
    for c in adam:
        cfg = c["meta"]["config"]
        p = torch.tensor(c["inputs"][0]["data"]).reshape(c["inputs"][0]["shape"]).requires_grad_(True)
        tgt = torch.tensor(c["inputs"][1]["data"]).reshape(c["inputs"][1]["shape"])
        opt = torch.optim.Adam([p], lr=cfg["lr"], weight_decay=cfg.get("weight_decay", 0.0))
        for _ in range(int(cfg["steps"])):
            opt.zero_grad()
            (0.5 * ((p - tgt) ** 2).sum()).backward()
            opt.step()
        _close(p, c["output"]["data"], c["name"])
    out["groups"]["adam"] = adam

    conv = [c for c in load("conv")["cases"] if c["meta"]["op"] == "conv2d"]
    assert len(conv) == 5
    for c in conv:
        cfg = c["meta"]["config"]
        _recheck(c, lambda x, w, b=None, cfg=cfg: torch.nn.functional.conv2d(
            x, w, b, stride=cfg["stride"], padding=cfg["padding"], dilation=cfg["dilation"]))
    out["groups"]["conv2d"] = conv
    return out


def seeded_cases():
    """Shapes of the reference's tolerance tests with numpy-seeded inputs; expected
    values from float64 torch, rounded once to float32."""
    rng = np.random.default_rng(20240607)
    cases = []

    def u(*shape):
        return torch.tensor(rng.uniform(-0.5, 0.5, size=shape).astype(np.float32))

    def mm_case(name, a, b, layout):
        a64, b64 = a.double().requires_grad_(True), b.double().requires_grad_(True)
        out = a64 @ (b64.transpose(-1, -2) if layout == "NT" else b64)
        go = u(*out.shape)
        out.backward(go.double())
        cases.append({"name": name, "layout": layout, "inputs": [_t(a), _t(b)], "grad_output": _t(go),
                      "output": _t(out.float()), "grads": [_t(a64.grad.float()), _t(b64.grad.float())]})

    # tests/Tensotron.Tests/TiledMatMulTests.cs:34-75 -- NN fwd + dA/dB, M,K,N = 96,80,112
    mm_case("tiled 96x80 @ 80x112", u(96, 80), u(80, 112), "NN")
    # tests/Tensotron.Tests/MatMulNtOpTests.cs:12-48 -- NT vs MatMul(a, b.T())
    mm_case("nt 5x7 . (3x7)^T", u(5, 7), u(3, 7), "NT")
    mm_case("nt 96x80 . (112x80)^T", u(96, 80), u(112, 80), "NT")
    # tests/Tensotron.Tests/BatchedCuBlasMatMulTests.cs:55-118 -- Bt=3, 64x64x80
    mm_case("bmm 3x64x64 @ 3x64x80", u(3, 64, 64), u(3, 64, 80), "NN")
    mm_case("bcast 64x64 @ 3x64x80", u(64, 64), u(3, 64, 80), "NN")
    return cases


def linear_case():
    """nn.Linear forward+backward, batch 64, 128 -> 64, ReLU and Tanh variants:
    X~N(0,1), W Kaiming-uniform(a=sqrt5) = U(+-1/sqrt(in)), dY~N(0,1).  One variant
    keeps the zero bias of the benchmark config, one uses a non-zero bias."""
    rng = np.random.default_rng(7)
    out = []
    for name, act, zero_bias in (("linear relu zero-bias", "relu", True), ("linear tanh bias", "tanh", False),
                                 ("linear none bias", "none", False)):
        x = torch.tensor(rng.standard_normal((64, 128)).astype(np.float32))
        bound = 1.0 / np.sqrt(128.0)
        w = torch.tensor(rng.uniform(-bound, bound, size=(64, 128)).astype(np.float32))
        b = torch.zeros(64) if zero_bias else torch.tensor(rng.uniform(-bound, bound, size=(64,)).astype(np.float32))
        dy = torch.tensor(rng.standard_normal((64, 64)).astype(np.float32))
        x64, w64, b64 = (t.double().requires_grad_(True) for t in (x, w, b))
        z = torch.nn.functional.linear(x64, w64, b64)
        y = torch.relu(z) if act == "relu" else torch.tanh(z) if act == "tanh" else z
        y.backward(dy.double())
        out.append({"name": name, "act": act, "inputs": [_t(x), _t(w), _t(b)], "grad_output": _t(dy),
                    "output": _t(y.float()),
                    "grads": [_t(x64.grad.float()), _t(w64.grad.float()), _t(b64.grad.float())]})
    return out


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to the Tensotron checkout>")
    ref_root = sys.argv[1]
    ref = from_reference(ref_root)
    json.dump(ref, open(os.path.join(HERE, "reference_fixtures.json"), "w"), indent=1)
    # The seeded cases are ~0.4 M floats: stored as float32 binary (.npz) plus a small index.
    arrays, index = {}, {"torch_version": torch.__version__, "matmul": [], "linear": []}
    for group, cases in (("matmul", seeded_cases()), ("linear", linear_case())):
        for ci, c in enumerate(cases):
            entry = {k: v for k, v in c.items() if k not in ("inputs", "grad_output", "output", "grads")}
            for key in ("inputs", "grads"):
                entry[key] = []
                for ti, t in enumerate(c[key]):
                    name = "%s%d_%s%d" % (group, ci, key, ti)
                    arrays[name] = np.asarray(t["data"], dtype=np.float32).reshape(t["shape"])
                    entry[key].append(name)
            for key in ("grad_output", "output"):
                name = "%s%d_%s" % (group, ci, key)
                arrays[name] = np.asarray(c[key]["data"], dtype=np.float32).reshape(c[key]["shape"])
                entry[key] = name
            index[group].append(entry)
    np.savez(os.path.join(HERE, "seeded_cases.npz"), **arrays)
    json.dump(index, open(os.path.join(HERE, "seeded_cases.json"), "w"), indent=1)
    print("wrote reference_fixtures.json (%d groups), seeded_cases.json and seeded_cases.npz"
          % len(ref["groups"]))


if __name__ == "__main__":
    main()
