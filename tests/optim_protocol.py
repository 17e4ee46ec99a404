"""homura's Adam / AdamW step (src/optim/adam.rs:125-171) written against the backend functions, op by op,
and the protocol of its multi-step golden tests (tests/optim.rs:159-290), so that the bitwise optimizer
fixtures can be replayed on the CPU checker and on the CUDA library. TEST INFRASTRUCTURE."""
from __future__ import annotations

from homura_b200 import ffi
from homura_b200.host import BF16, F16, TensorData
from frontend import binary_op, unary_op


class AdamState:
    def __init__(self, be, p: TensorData, amsgrad: bool):
        zeros = lambda: _filled(be, p, 0.0)
        self.step = 0.0
        self.exp_avg, self.exp_avg_sq = zeros(), zeros()
        self.max_exp_avg_sq = zeros() if amsgrad else None


def _filled(be, like: TensorData, value: float) -> TensorData:
    t = be.empty(like.shape, like.dtype)
    be.fill(t, value)
    return t


def _fused(be, op, value, a, b, c=None) -> TensorData:
    out = be.empty(a.shape, a.dtype)
    be.fused(op, value, out, a, b, c)
    return out


def _inplace(be, target: TensorData, result: TensorData):
    """An in-place op: the result is computed out of place, then copied into the target
    (src/ops/binary.rs:568-587)."""
    be.copy(target, result)


class Adam:
    def __init__(self, be, groups, *, betas, eps, weight_decay, amsgrad, maximize, decoupled):
        """groups: [(lr, [params])]."""
        self.be, self.groups = be, [[lr, ps] for lr, ps in groups]
        self.betas, self.eps, self.weight_decay = betas, eps, weight_decay
        self.amsgrad, self.maximize, self.decoupled = amsgrad, maximize, decoupled
        self.state = {}

    def step(self, grads: dict, fused_kernel: bool = False):
        """grads: id(param) -> gradient TensorData (parameters without one are skipped)."""
        be = self.be
        for lr, params in self.groups:
            for p in params:
                g = grads.get(id(p))
                if g is None:
                    continue
                st = self.state.setdefault(id(p), AdamState(be, p, self.amsgrad))
                st.step += 1.0
                beta1, beta2 = self.betas
                if fused_kernel:
                    assert self.decoupled and not self.amsgrad and not self.maximize
                    be.adamw_step(p, g, st.exp_avg, st.exp_avg_sq, lr=lr, beta1=beta1, beta2=beta2, eps=self.eps,
                                  weight_decay=self.weight_decay, step=st.step)
                    continue
                grad = unary_op(be, "neg", g) if self.maximize else g
                if self.weight_decay != 0.0:
                    if self.decoupled:
                        _inplace(be, p, binary_op(be, "mul", p, 1.0 - lr * self.weight_decay))
                    else:
                        grad = _fused(be, ffi.HMC_FUSED_SCALED_ADD, self.weight_decay, grad, p)
                _inplace(be, st.exp_avg, _fused(be, ffi.HMC_FUSED_LERP, 1.0 - beta1, st.exp_avg, grad))
                _inplace(be, st.exp_avg_sq, binary_op(be, "mul", st.exp_avg_sq, beta2))
                _inplace(be, st.exp_avg_sq, _fused(be, ffi.HMC_FUSED_ADDCMUL, 1.0 - beta2, st.exp_avg_sq, grad, grad))
                bias_correction2 = 1.0 - beta2 ** st.step
                step_size = lr / (1.0 - beta1 ** st.step)
                bias_correction2_sqrt = bias_correction2 ** 0.5
                second = st.exp_avg_sq
                if self.amsgrad:
                    _inplace(be, st.max_exp_avg_sq, binary_op(be, "maximum", st.max_exp_avg_sq, st.exp_avg_sq))
                    second = st.max_exp_avg_sq
                denom = binary_op(be, "div", unary_op(be, "sqrt", second), bias_correction2_sqrt)
                _inplace(be, denom, binary_op(be, "add", denom, self.eps))
                _inplace(be, p, _fused(be, ffi.HMC_FUSED_ADDCDIV, -step_size, p, st.exp_avg, denom))
