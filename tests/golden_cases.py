"""Runs homura's golden cases of the hot path (the handlers of its tests/golden_ops.rs:22-351, restated) on
a backend and compares with the stored PyTorch results at homura's tolerances (tests/common/mod.rs:104-161)."""
from __future__ import annotations

import numpy as np

from frontend import T, where
from golden_io import Golden
from homura_b200.host import BF16, BOOL, F16, F32, F64, I32, I64, is_float
from values import storage_to_f64

TOL = {F16: (2.0 ** -10, 1e-7), BF16: (2.0 ** -7, 1e-7), F32: (1e-6, 1e-6), F64: (1e-12, 1e-12)}


def assert_close(actual: T, expected, what: str):
    dt, shape, raw = expected
    assert actual.shape == tuple(shape), f"{what}: shape {actual.shape} vs {shape}"
    assert actual.dtype == dt, f"{what}: dtype {actual.dtype} vs {dt}"
    got = actual.raw()
    if not is_float(dt):
        assert (got.astype(np.int64) == raw.astype(np.int64)).all(), f"{what}: integers differ\n{got}\n{raw}"
        return
    rtol, atol = TOL[dt]
    x, y = storage_to_f64(got, dt).reshape(-1), storage_to_f64(raw, dt).reshape(-1)
    nan = np.isnan(x) | np.isnan(y)
    assert (np.isnan(x) == np.isnan(y)).all(), f"{what}: NaN placement"
    inf = (np.isinf(x) | np.isinf(y)) & ~nan
    assert (x[inf] == y[inf]).all(), f"{what}: infinities"
    ok = ~(nan | inf)
    bad = np.abs(x[ok] - y[ok]) > atol + rtol * np.abs(y[ok])
    assert not bad.any(), f"{what}: got {x[ok][bad][:4]}, expected {y[ok][bad][:4]}"


class Case:
    def __init__(self, be, golden: Golden, name: str):
        self.be, self.golden, self.name = be, golden, name
        self.used = set()

    def input(self, n: str) -> T:
        self.used.add(n)
        dt, shape, raw = self.golden.get(f"{self.name}/{n}")
        return T(self.be, self.be.upload(raw, dt, shape))

    def check(self, n: str, actual: T):
        self.used.add(n)
        assert_close(actual, self.golden.get(f"{self.name}/{n}"), f"{self.name}/{n}")

    def assert_all_used(self):
        for n in self.golden.names(self.name):
            assert n in self.used, f"golden tensor {self.name}/{n} was not used"


def _unary(op: str, x: T):
    table = {"neg": x.neg, "abs": x.abs, "exp": x.exp, "log": x.log, "sqrt": x.sqrt, "rsqrt": x.rsqrt,
             "reciprocal": x.reciprocal, "sin": x.sin, "cos": x.cos, "tanh": x.tanh, "sigmoid": x.sigmoid,
             "relu": x.relu, "silu": x.silu, "gelu": lambda: x.gelu("none"), "gelu_tanh": lambda: x.gelu("tanh"),
             "pow3": lambda: x.pow(3), "clamp_float": lambda: x.clamp(-1.5, 2.5), "clamp_int": lambda: x.clamp(-1, 2)}
    return table[op]() if op in table else None


def run(c: Case) -> bool:
    """True if the case has a handler (tests/golden_ops.rs `run`)."""
    name = c.name
    cat = name.split(".")[0]
    op = name.split(".", 1)[1] if "." in name else ""
    x = lambda: c.input("x")
    a, b = (lambda: c.input("a")), (lambda: c.input("b"))
    out = lambda t: c.check("out", t)
    if cat in ("unary", "unary_wide", "unary_special", "unary_f16", "unary_bf16", "unary_f64", "unary_int"):
        t = _unary(op, x())
        if t is None:
            return False
        out(t)
    elif cat == "pow":
        out({"scalar2": lambda: x().pow(2), "scalar3": lambda: x().pow(3), "half": lambda: x().pow(0.5),
             "neg": lambda: x().pow(-1.5)}[op]())
    elif cat == "clamp":
        out({"both": lambda: x().clamp(-0.5, 0.5), "min": lambda: x().clamp_min(0.2), "max": lambda: x().clamp_max(-0.1),
             "special": lambda: x().clamp(-1.0, 1.0), "inverted": lambda: x().clamp(0.5, -0.5)}[op]())
    elif cat == "logical_not":
        out(x().logical_not())
    elif cat in ("binary", "binary_f16", "binary_bf16"):
        out({"add": lambda: a().add(b()), "sub": lambda: a().sub(b()), "mul": lambda: a().mul(b()),
             "div": lambda: a().div(b()), "maximum": lambda: a().maximum(b()), "minimum": lambda: a().minimum(b()),
             "pow": lambda: a().pow(b()), "rsub": lambda: x().rsub(1.0), "rdiv": lambda: x().rdiv(2.0),
             "add_scalar": lambda: x().add(2.5), "div_zero": lambda: a().div(b())}[op]())
    elif cat == "compare":
        out({"gt": lambda: a().greater(b()), "ge": lambda: a().greater_equal(b()), "lt": lambda: a().less(b()),
             "le": lambda: a().less_equal(b()), "eq": lambda: a().equal(b()), "ne": lambda: a().not_equal(b()),
             "mixed_lt": lambda: a().less(b()), "scalar_ge": lambda: a().greater_equal(2.5)}[op]())
    elif cat == "logical":
        out({"and": lambda: a().logical_and(b()), "or": lambda: a().logical_or(b())}[op]())
    elif cat == "promote":
        if op in ("i32_f16", "u8_i8", "f32_f64_zero_dim", "i64_f64_zero_dim", "i8_overflow", "bool_add"):
            out(a().add(b()))
        elif op in ("bool_mul", "i8_mul_overflow"):
            out(a().mul(b()))
        elif op in ("i64_float_scalar", "f16_float_scalar"):
            out(a().mul(2.5))
        elif op == "int_div":
            out(a().div(b()))
        elif op == "bool_int_scalar":
            out(a().add(1))
        elif op == "u8_minus_one":
            out(a().sub(1))
        else:
            return False
    elif cat == "where":
        cond = c.input("cond")
        if op in ("tensors", "promote"):
            out(where(cond, x(), c.input("y")))
        elif op == "scalar":
            out(where(cond, x(), 0.5))
        else:
            return False
    elif cat == "masked_fill":
        out({"broadcast": lambda: x().masked_fill(c.input("mask"), -1e9), "int": lambda: x().masked_fill(c.input("mask"), 7)}[op]())
    elif cat in ("reduce", "ties", "nan", "var", "std", "bool", "float", "int", "reduce_f16", "reduce_bf16"):
        def vi(pair):
            c.check("values", pair[0])
            c.check("indices", pair[1])
        table = {
            "maximum": lambda: out(a().maximum(b())), "minimum": lambda: out(a().minimum(b())),
            "sum": lambda: out(x().sum()), "sum_dims_keepdim": lambda: out(x().sum_dim([0, 2], True)),
            "sum_last": lambda: out(x().sum_dim(-1)), "sum_negative_dims": lambda: out(x().sum_dim([-1, -3])),
            "sum_dim": lambda: out(x().sum_dim(0 if cat in ("nan", "int") else -1)),
            "mean": lambda: out(x().mean()), "mean_dim_keepdim": lambda: out(x().mean_dim(1, True)),
            "prod": lambda: out(x().prod()), "prod_dim": lambda: out(x().prod_dim(1)),
            "max": lambda: out(x().max()), "min": lambda: out(x().min()),
            "max_dim": lambda: vi(x().max_dim(1)), "min_dim": lambda: vi(x().min_dim(0)),
            "min_dim_keepdim": lambda: vi(x().min_dim(-1, True)),
            "argmax": lambda: out(x().argmax()), "argmax_dim": lambda: out(x().argmax_dim(1)),
            "argmin_dim": lambda: out(x().argmin_dim(1 if cat == "ties" else 2)),
            "default": lambda: out(x().var(1)), "dim_c0_keepdim": lambda: out(x().var_dim(1, 0, True)),
            "single": lambda: out(x().var(1)), "dims": lambda: out(x().std_dim([0, 2], 1)),
            "dim_c2": lambda: out(x().std_dim(2, 2)), "var_dim": lambda: out(x().var_dim(1, 1)),
            "all": lambda: out(x().all()), "any": lambda: out(x().any()), "any_dim": lambda: out(x().any_dim(1)),
            "all_dim_keepdim": lambda: out(x().all_dim(0, True)),
        }
        if op not in table:
            return False
        table[op]()
    elif cat == "softmax":
        out({"last": lambda: x().softmax(-1), "f16": lambda: x().softmax(-1), "inf": lambda: x().softmax(-1),
             "first": lambda: x().softmax(0)}[op]())
    elif cat == "log_softmax":
        out({"mid": lambda: x().log_softmax(1), "inf": lambda: x().log_softmax(-1)}[op]())
    elif cat == "addcmul":
        out(c.input("input").addcmul(c.input("t1"), c.input("t2"), 0.5))
    elif cat == "addcdiv":
        out(c.input("input").addcdiv(c.input("t1"), c.input("t2"), -2))
    elif cat == "lerp":
        start, end = c.input("start"), c.input("end")
        out({"low": lambda: start.lerp(end, 0.3), "high": lambda: start.lerp(end, 0.7),
             "tensor": lambda: start.lerp(end, c.input("weight"))}[op]())
    elif cat == "cast":
        target = {"f32_i32": I32, "f32_i64": I64, "f32_bool": BOOL, "f32_f16": F16, "f16_rounding": F16, "f32_bf16": BF16,
                  "bf16_rounding": BF16, "i64_f32": F32, "bool_f32": F32, "f16_f32": F32}
        if op not in target:
            return False
        out(x().to(target[op]))
    elif cat == "erf":
        out(x().erf())
    elif cat == "sign":
        out(x().sign())
    elif cat == "sum_to_size":
        size = {"leading": [3, 4], "ones": [2, 1, 4], "mixed": [3, 1], "scalar": [], "same": [2, 3, 4], "int": [1, 5],
                "empty": [1, 3], "f16": [4]}
        if op not in size:
            return False
        out(x().sum_to_size(size[op]))
    else:
        return False
    c.assert_all_used()
    return True


def run_all(be, only=None):
    g = Golden("ops_hotpath.safetensors")
    count = 0
    for name in g.cases():
        if only is not None and name.split(".")[0] not in only:
            continue
        assert run(Case(be, g, name)), f"no handler for golden case {name!r}"
        count += 1
    return count
