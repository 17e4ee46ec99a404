"""The CUDA library against the CPU checker at the full sizes of the benchmark configurations, on the same bits:

* elementwise / broadcast: x bf16 [8192, 8192], bias f32 [8192, 1], scale bf16 [1, 8192]; silu, * scale, + bias with
  promotion, the same on x.t(), and the bf16 -> f32 cast, every element of every result;
* reductions: f32 and i32 [16384, 4096], every reduction of the configuration in full;
* softmax / log_softmax: the causally masked f32 [8, 32, 2048, 2048] tensor is computed in full on the GPU and 8192
  of its 524288 rows (every position within the causal matrices occurs) are checked, rows being independent; the
  row mean of squares of bf16 [32768, 4096] in full;
* the sharded configuration, one GPU's share: a * b + c on 2^29 f32 elements, its sum and maximum, and the AdamW
  step over the 291 Llama-3-8B-shaped tensors (an eighth of the rows of each) in one launch against the per-tensor
  kernel (every element) and against the CPU's op-by-op optimizer on chunks of several tensors.

Bars: integers, indices, casts and IEEE float operations bit for bit; the half types' silu within one ulp (special
function unit); f32 reductions and softmax within two ulps of the CPU's f64-accumulated result."""
import numpy as np
import pytest

from frontend import T
from homura_b200 import ffi
from homura_b200.host import BF16, BOOL, F32, F64, I32, I64, Generator, TensorData
from test_gpu_full_size import equal_bits
from values import assert_bitwise, assert_ulp, storage_to_f64

pytestmark = pytest.mark.gpu


def philox_normal(n, seed):
    return np.random.Generator(np.random.Philox(seed)).standard_normal(n, dtype=np.float32)


def bf16_bits(f):
    x = f.astype(np.float32).view(np.uint32).astype(np.uint64)
    return ((x + 0x7FFF + ((x >> 16) & 1)) >> 16).astype(np.uint16)


def pair(oracle, cuda, raw, dtype, shape=None):
    return T(oracle, oracle.upload(raw, dtype, shape)), T(cuda, cuda.upload(raw, dtype, shape))


def test_elementwise_broadcast_step_at_8192x8192(oracle, cuda):
    n = 8192
    x = bf16_bits(philox_normal(n * n, 11)).reshape(n, n)
    bias = philox_normal(n, 12).reshape(n, 1)
    scale = bf16_bits(philox_normal(n, 13)).reshape(1, n)
    (ox, gx), (ob, gb), (osc, gsc) = pair(oracle, cuda, x, BF16), pair(oracle, cuda, bias, F32), pair(oracle, cuda, scale, BF16)
    tr = lambda d: d.t()
    # silu, contiguous and through the tiled kernel: bf16 results of an f32 evaluation with the special function
    # unit, within one ulp; both GPU kernels agree bit for bit
    so, sg = ox.silu(), gx.silu()
    worst, differ = assert_ulp(sg.raw(), so.raw(), BF16, 1, "silu(x)")
    sto, stg = ox.view(tr).silu(), gx.view(tr).silu()
    assert_ulp(stg.raw(), sto.raw(), BF16, 1, "silu(x.t())")
    assert equal_bits(cuda, stg.data, sg.data.t()), "the tiled kernel differs from the contiguous one"
    print(f"silu bf16 [8192, 8192]: {differ} of {n * n} elements one ulp from the CPU's")
    # the arithmetic after it from the CPU's silu on both sides: every bit
    s_on_gpu = T(cuda, cuda.upload(so.raw(), BF16))
    yo, yg = so.mul(osc).add(ob), s_on_gpu.mul(gsc).add(gb)
    assert yo.dtype == yg.dtype == F32
    assert_bitwise(yg.raw(), yo.raw(), F32, "silu(x) * scale + bias")
    st_on_gpu = T(cuda, cuda.upload(sto.raw(), BF16))
    scale_t = lambda t: t.view(lambda d: d.reshape(n, 1))
    bias_t = lambda t: t.view(lambda d: d.reshape(1, n))
    yto, ytg = sto.mul(scale_t(osc)).add(bias_t(ob)), st_on_gpu.mul(scale_t(gsc)).add(bias_t(gb))
    assert_bitwise(ytg.raw(), yto.raw(), F32, "silu(x.t()) * scale + bias")
    assert_bitwise(gx.to(F32).raw(), ox.to(F32).raw(), F32, "cast bf16 -> f32")
    assert_bitwise(gx.view(tr).to(F32).raw(), ox.view(tr).to(F32).raw(), F32, "cast of x.t()")
    # the whole expression in one kernel, contiguous and on x.t(): the bits of the three GPU kernels run in turn
    three, three_t = sg.mul(gsc).add(gb), stg.mul(scale_t(gsc)).add(bias_t(gb))
    fused = cuda.empty((n, n), F32)
    codes = (ffi.HMC_UNARY_SILU, ffi.HMC_BINARY_MUL, ffi.HMC_BINARY_ADD)
    cuda.unary_binary_binary(*codes, fused, gx.data, gsc.data, gb.data)
    assert equal_bits(cuda, fused, three.data), "the fused expression differs from its three kernels"
    cuda.unary_binary_binary(*codes, fused, gx.view(tr).data, scale_t(gsc).data, bias_t(gb).data)
    assert equal_bits(cuda, fused, three_t.data), "the fused expression on x.t() differs from its three kernels"
    cuda.allocator.empty_cache()


def test_reductions_at_16384x4096(oracle, cuda):
    r, c = 16384, 4096
    x = philox_normal(r * c, 21).reshape(r, c)
    i = np.random.Generator(np.random.Philox(22)).integers(-1000, 1001, size=(r, c), dtype=np.int32)
    ox, gx = pair(oracle, cuda, x, F32)
    oi, gi = pair(oracle, cuda, i, I32)
    for name, f in (("sum rows", lambda t: t.sum_dim([1])), ("mean rows", lambda t: t.mean_dim([1])),
                    ("var rows", lambda t: t.var_dim([1], 1)), ("sum cols", lambda t: t.sum_dim([0])),
                    ("mean cols", lambda t: t.mean_dim([0])), ("var cols", lambda t: t.var_dim([0], 1)),
                    ("std rows", lambda t: t.std_dim([1], 1)), ("full sum", lambda t: t.sum()), ("full mean", lambda t: t.mean())):
        assert_ulp(f(gx).raw(), f(ox).raw(), F32, 2, name)
    (ov, on), (gv, gn) = ox.max_dim(1), gx.max_dim(1)
    assert_bitwise(gv.raw(), ov.raw(), F32, "max rows")
    assert_bitwise(gn.raw(), on.raw(), I64, "argmax rows")
    assert_bitwise(gx.argmax_dim(0).raw(), ox.argmax_dim(0).raw(), I64, "argmax cols")
    assert_bitwise(gx.max().raw(), ox.max().raw(), F32, "full max")
    for name, f in (("sum rows", lambda t: t.sum_dim([1])), ("sum cols", lambda t: t.sum_dim([0])), ("full sum", lambda t: t.sum())):
        w = f(oi)
        assert w.dtype == I64
        assert_bitwise(f(gi).raw(), w.raw(), I64, "i32 " + name)
    (ov, on), (gv, gn) = oi.max_dim(1), gi.max_dim(1)
    assert_bitwise(gv.raw(), ov.raw(), I32, "i32 max rows")
    assert_bitwise(gn.raw(), on.raw(), I64, "i32 argmax rows (first of equals)")
    cuda.allocator.empty_cache()


def test_softmax_of_masked_logits_8x32x2048x2048_on_sampled_rows(oracle, cuda):
    b, n = 256, 2048
    x = cuda.empty((b * n * n,), F32)
    cuda.random_normal(x, Generator(31), 0.0, 3.0)
    x = x.reshape(b, n, n)
    mask = cuda.upload(np.triu(np.ones((n, n), dtype=np.uint8), 1), BOOL)
    cuda.where_constant(x, mask.reshape(1, n, n).expand(b, n, n), float("-inf"), x)
    soft, logsoft = cuda.empty((b, n, n), F32), cuda.empty((b, n, n), F32)
    cuda.softmax(soft, x, 2, False)
    cuda.softmax(logsoft, x, 2, True)
    # 8192 rows, one in every 64: within its group of 64 the k-th row sits at (k div 32) mod 64, so every position of
    # a row inside its causal matrix of 2048 rows turns up (four times)
    k = np.arange(8192, dtype=np.int64)
    rows = k * 64 + (k // 32) % 64
    assert len(set((rows % n).tolist())) == n
    index = cuda.upload(rows, I64)
    def sample(t):
        out = cuda.empty((rows.size, n), F32)
        cuda.index_select(out, t.reshape(b * n, n), 0, index)
        return cuda.download(out)
    xs, got_soft, got_log = sample(x), sample(soft), sample(logsoft)
    assert np.isneginf(xs).sum() == int(((n - 1) - (rows % n)).sum()), "the causal mask is not where it should be"
    ox = T(oracle, oracle.upload(xs, F32))
    from frontend import softmax_op
    want_soft = oracle.download(softmax_op(oracle, ox.data, 1, False))
    want_log = oracle.download(softmax_op(oracle, ox.data, 1, True))
    assert_ulp(got_soft, want_soft, F32, 2, "softmax")
    assert_ulp(got_log, want_log, F32, 2, "log_softmax")
    assert (got_soft[np.isneginf(xs)] == 0).all() and np.isneginf(got_log[np.isneginf(xs)]).all()
    cuda.allocator.empty_cache()


def test_row_mean_of_squares_of_bf16_32768x4096(oracle, cuda):
    r, c = 32768, 4096
    h = cuda.empty((r * c,), BF16)
    cuda.random_normal(h, Generator(32), 0.0, 1.0)
    raw = cuda.download(h).reshape(r, c)
    oh, gh = T(oracle, oracle.upload(raw, BF16)), T(cuda, h.reshape(r, c))
    # as homura's rms_norm composes it: to(F32), pow(2), mean over the last dimension (kept)
    o32, g32 = oh.to(F32), gh.to(F32)
    assert_bitwise(g32.raw(), o32.raw(), F32, "to f32")
    op, gp = o32.pow(2.0), g32.pow(2.0)
    assert_bitwise(gp.raw(), op.raw(), F32, "pow 2")
    assert_ulp(gp.mean_dim([1], True).raw(), op.mean_dim([1], True).raw(), F32, 2, "row mean of squares")
    # and the direct bf16 composition x.pow(2).mean_dim(-1, true)
    ob, gb = oh.pow(2.0), gh.pow(2.0)
    assert_bitwise(gb.raw(), ob.raw(), BF16, "bf16 pow 2")
    assert_ulp(gb.mean_dim([1], True).raw(), ob.mean_dim([1], True).raw(), BF16, 2, "bf16 row mean of squares")
    cuda.allocator.empty_cache()


def test_flat_elementwise_sum_and_max_at_2_to_the_29(oracle, cuda):
    n = 1 << 29
    a, b, c = (cuda.empty((n,), F32) for _ in range(3))
    for t, seed in ((a, 41), (b, 42), (c, 43)):
        cuda.random_normal(t, Generator(seed), 0.0, 1.0)
    t1, t2 = cuda.empty((n,), F32), cuda.empty((n,), F32)
    cuda.binary(ffi.HMC_BINARY_MUL, t1, a, b)
    cuda.binary(ffi.HMC_BINARY_ADD, t2, t1, c)
    total, top, where = cuda.empty((), F32), cuda.empty((), F32), cuda.empty((), I64)
    cuda.reduce(ffi.HMC_REDUCE_SUM, total, t2, [True])
    cuda.arg_reduce(top, where, t2, 0, True)
    # chunks of the elementwise results on the CPU checker: the start, an odd offset in the middle, the end
    for start, length in ((0, 1 << 22), ((1 << 28) + 12345, (1 << 22) + 7), (n - (1 << 22) - 3, (1 << 22) + 3)):
        oa, ob_, oc = (T(oracle, oracle.upload(cuda.download(t.narrow(0, start, length)), F32)) for t in (a, b, c))
        assert_bitwise(cuda.download(t2.narrow(0, start, length)), oa.mul(ob_).add(oc).raw(), F32, f"a * b + c at {start}")
    # every element: IEEE single-precision multiply and add, which numpy performs exactly as the CPU backend does
    ha, hb = cuda.download(a), cuda.download(b)
    want = ha * hb
    del ha, hb
    want += cuda.download(c)
    got = cuda.download(t2)
    assert (got.view(np.uint32) == want.view(np.uint32)).all(), "a * b + c differs somewhere in 2^29 elements"
    del want
    # the sum and the maximum of the GPU's tensor, folded by the CPU checker in its own (sequential, f64) order
    ot = T(oracle, oracle.upload(got, F32))
    assert_ulp(cuda.download(total), ot.sum().raw(), F32, 2, "sum of 2^29")
    assert_bitwise(cuda.download(top), ot.max().raw(), F32, "max of 2^29")
    assert int(cuda.download(where)) == int(np.argmax(got)), "argmax of 2^29"
    cuda.allocator.empty_cache()


def test_adamw_over_the_llama_3_8b_tensors_one_eighth_of_each(oracle, cuda):
    from bench import llama3_8b_shapes
    from optim_protocol import Adam
    shapes = [(s[0] // 8,) + tuple(s[1:]) for s in llama3_8b_shapes()]
    assert len(shapes) == 291 and sum(int(np.prod(s)) for s in shapes) * 8 == 8_030_261_248
    hyper = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
    base_n = (1 << 22) + 11   # not a multiple of any row length: every tensor sees the pattern at another phase
    p0 = cuda.upload(0.02 * philox_normal(base_n, 51), F32)
    g0 = cuda.upload(1e-3 * philox_normal(base_n, 52), F32)

    def tile(big, small, phase):
        flat, n = big.reshape(big.numel), small.numel
        phase %= n
        first = min(flat.numel, n - phase)
        cuda.copy(flat.narrow(0, 0, first), small.narrow(0, phase, first))
        done = first
        reps = (flat.numel - done) // n
        if reps:
            cuda.copy(flat.narrow(0, done, reps * n).reshape(reps, n), small.reshape(1, n).expand(reps, n))
            done += reps * n
        if done < flat.numel:
            cuda.copy(flat.narrow(0, done, flat.numel - done), small.narrow(0, 0, flat.numel - done))

    def make():
        out = []
        for i, shape in enumerate(shapes):
            p, g, m, v = (cuda.empty(shape, F32) for _ in range(4))
            tile(p, p0, 7919 * i)
            tile(g, g0, 104729 * i)
            cuda.fill(m, 0.0)
            cuda.fill(v, 0.0)
            out.append((p, g, m, v))
        return out

    many, single = make(), make()
    # chunks for the CPU's op-by-op optimizer: (tensor, first element, length), taken before the first step
    picks = [(0, 0, 1 << 16), (0, shapes[0][0] * 4096 - 50_000, 50_000), (1, 123_457, 1 << 16), (8, 0, 512), (9, 0, 512),
             (7, 4096 * 14336 // 8 - 4099, 4099), (289, 0, 512), (290, (1 << 20) + 3, 1 << 16)]
    cpu_runs = []
    for t, start, length in picks:
        p, g = (cuda.download(x.reshape(x.numel).narrow(0, start, length)) for x in many[t][:2])
        cpu_runs.append((oracle.upload(p, F32), g))
    group = cuda.adamw_group(many, with_grad_sq=True)
    assert len(group.flat) == 291 and not group.strided
    steps = 3
    for t in range(1, steps + 1):
        group.step(step=float(t), **hyper)
        for p, g, m, v in single:
            cuda.adamw_step(p, g, m, v, step=float(t), **hyper)
    for i, (a, b) in enumerate(zip(many, single)):
        for x, y, what in zip(a, b, ("param", "grad", "exp_avg", "exp_avg_sq")):
            assert equal_bits(cuda, x, y), f"tensor {i} {shapes[i]} {what}: one launch for all differs from a launch per tensor"
    # the CPU's optimizer, op by op with its temporaries and in-place copies, on the chunks
    for (t, start, length), (op, g) in zip(picks, cpu_runs):
        opt = Adam(oracle, [(hyper["lr"], [op])], betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, amsgrad=False,
                   maximize=False, decoupled=True)
        for _ in range(steps):
            opt.step({id(op): oracle.upload(g, F32)})
        st = opt.state[id(op)]
        for want, x, what in ((op, many[t][0], "param"), (st.exp_avg, many[t][2], "exp_avg"), (st.exp_avg_sq, many[t][3], "exp_avg_sq")):
            got = cuda.download(x.reshape(x.numel).narrow(0, start, length))
            assert_bitwise(got, oracle.download(want), F32, f"tensor {t} [{start}, +{length}) {what} after {steps} steps")
    # sums of squared gradients: per tensor the f64 sum of the f32 squares; against g.mul(g).sum() on the GPU (two
    # ulps of f32 after its rounding) and, for the small tensors, the CPU checker's
    squares = group.grad_squares()
    assert squares.shape == (291,) and (squares > 0).all()
    for t in (0, 1, 5, 7, 8, 290):
        g = T(cuda, many[t][1])
        want = g.mul(g).sum().raw()
        assert_ulp(np.array([squares[t]], dtype=np.float32), want.reshape(1), F32, 2, f"sum of squares of tensor {t}")
    for t in (8, 9, 289):
        og = T(oracle, oracle.upload(cuda.download(many[t][1]), F32))
        want = float(np.sum(storage_to_f64(og.mul(og).raw(), F32)))
        assert abs(squares[t] - want) <= 1e-12 * want
    # the norm: the partials folded in tensor order in f64
    total = cuda.empty((), F64)
    cuda.reduce(ffi.HMC_REDUCE_SUM, total, TensorData(group.grad_sq, F64, (291,), (1,)), [True])
    assert abs(float(cuda.download(total)) - float(np.sum(squares))) <= 1e-12 * float(np.sum(squares))
    del many, single, group
    cuda.allocator.empty_cache()
