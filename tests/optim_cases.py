"""Replays homura's bitwise Adam / AdamW fixtures (protocol of tests/optim.rs:159-244) on a backend."""
from __future__ import annotations

import numpy as np

from golden_io import Golden
from optim_protocol import Adam
from values import assert_same

PARAMS = ["a", "b", "c"]
STEPS = 5


def _scalar(g: Golden, case: str, name: str) -> float:
    return float(g.get(f"{case}/opt.{name}")[2].reshape(-1)[0])


def _build(be, g, case, groups):
    kind = case.split(".")[0].split("_")[0]
    return Adam(be, groups, betas=(_scalar(g, case, "beta1"), _scalar(g, case, "beta2")), eps=_scalar(g, case, "eps"),
                weight_decay=_scalar(g, case, "weight_decay"), amsgrad=_scalar(g, case, "amsgrad") != 0.0,
                maximize=_scalar(g, case, "maximize") != 0.0, decoupled=kind == "adamw")


def _check_state(be, g, case, t, n, p, opt, used):
    names = g.names(case)
    def compare(key, actual):
        used.add(key)
        dt, shape, raw = g.get(f"{case}/{key}")
        assert_same(be.download(actual).reshape(shape), raw, dt, f"{case}/{key}")
    compare(f"after{t}.{n}", p)
    st = opt.state.get(id(p))
    stored = [k for k in names if k.startswith(f"after{t}.{n}.")]
    have = {} if st is None else {"exp_avg": st.exp_avg, "exp_avg_sq": st.exp_avg_sq}
    if st is not None and st.max_exp_avg_sq is not None:
        have["max_exp_avg_sq"] = st.max_exp_avg_sq
    assert len(stored) == (len(have) + 1 if st is not None else 0), f"{case}: state of {n} after step {t}"
    for s, value in have.items():
        compare(f"after{t}.{n}.{s}", value)
    if st is not None:
        key = f"after{t}.{n}.step"
        used.add(key)
        assert float(g.get(f"{case}/{key}")[2].reshape(-1)[0]) == st.step


def multi_step(be, case: str, fused_kernel: bool = False):
    g = Golden("adam_steps.safetensors")
    names, used = g.names(case), set()
    def load(key):
        used.add(key)
        dt, shape, raw = g.get(f"{case}/{key}")
        return be.upload(raw, dt, shape)
    params = [load(f"init.{p}") for p in PARAMS]
    lr = _scalar(g, case, "lr")
    opt = _build(be, g, case, [(lr, [params[0], params[2]]), (2.0 * lr, [params[1]])])
    for t in range(STEPS):
        if t == 2:
            opt.groups[0][0] *= 0.5
        grads = {}
        for p, n in zip(params, PARAMS):
            key = f"grad{t}.{n}"
            if key in names:
                grads[id(p)] = load(key)
        opt.step(grads, fused_kernel=fused_kernel)
        for p, n in zip(params, PARAMS):
            _check_state(be, g, case, t, n, p, opt, used)
    for n in names:
        assert n in used or n.startswith("opt."), f"golden tensor {case}/{n} was not used"


def edge_values(be, case: str, fused_kernel: bool = False):
    g = Golden("adam_edges.safetensors")
    names, used = g.names(case), set()
    dt, shape, raw = g.get(f"{case}/init.p")
    p = be.upload(raw, dt, shape)
    opt = _build(be, g, case, [(_scalar(g, case, "lr"), [p])])
    t = 0
    while f"grad{t}.p" in names:
        gd = g.get(f"{case}/grad{t}.p")
        opt.step({id(p): be.upload(gd[2], gd[0], gd[1])}, fused_kernel=fused_kernel)
        _check_state(be, g, case, t, "p", p, opt, used)
        t += 1
    assert t > 0


def cases(file: str):
    return Golden(file).cases()


def fusable(file: str, case: str) -> bool:
    g = Golden(file)
    return case.startswith("adamw_") and _scalar(g, case, "amsgrad") == 0.0 and _scalar(g, case, "maximize") == 0.0
