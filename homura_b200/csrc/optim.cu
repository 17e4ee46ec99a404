// The decoupled-weight-decay Adam update of one parameter in a single kernel.
//
// homura's optimizer (src/optim/adam.rs:125-171) issues about fourteen elementwise kernels and six
// temporaries per parameter: p *= 1 - lr*wd; exp_avg = lerp(exp_avg, g, 1 - beta1);
// exp_avg_sq *= beta2; exp_avg_sq = addcmul(exp_avg_sq, g, g, 1 - beta2);
// denom = sqrt(exp_avg_sq) / sqrt(bias2) + eps; p = addcdiv(p, exp_avg, denom, -step_size).
// Every one of those kernels rounds its result to the parameter's dtype. This kernel performs the
// same operations in the same order on registers and rounds at the same points, so the three
// updated tensors carry the bits of the op-by-op path while reading and writing each of them once
// (28 bytes per f32 element instead of ~130).
#include "functors.cuh"

namespace hmc {
namespace {

template <class T>
struct AdamW {
    using C = typename Comp<T>::C;
    C decay, lerp_coeff, beta2, one_minus_beta2, bias2_sqrt, eps, neg_step_size;
    bool has_decay, lerp_small;

    // Rounds to the dtype and widens again: the store and reload between two of homura's kernels.
    __device__ __forceinline__ static C rt(C c) { return up(down<T>(c)); }

    __device__ __forceinline__ void operator()(T &p, T g0, T &m0, T &v0) const {
        C x = up(p);
        const C g = up(g0);
        const C m = up(m0);
        const C v = up(v0);
        if (has_decay) x = rt(x * decay);
        const C m1 = rt(m_fma(lerp_coeff, g - m, lerp_small ? m : g));
        const C v1 = rt(v * beta2);
        const C v2 = rt(m_fma(one_minus_beta2 * g, g, v1));
        const C s = rt(m_sqrt(v2));
        const C d = rt(s / bias2_sqrt);
        const C d2 = rt(d + eps);
        const C x1 = x + neg_step_size * m1 / d2;
        p = down<T>(x1);
        m0 = down<T>(m1);
        v0 = down<T>(v2);
    }
};

// Same walk as map_kernel (operand 0 param, 1 grad, 2 exp_avg, 3 exp_avg_sq), three of them written.
template <class T>
__global__ void __launch_bounds__(kThreads) adamw_kernel(const __grid_constant__ MapArgs a, const AdamW<T> f) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int UNR = 2;
    const int tpr = 1 << a.tpr_log2;
    const int lane = threadIdx.x & (tpr - 1);
    const int rib = threadIdx.x >> a.tpr_log2;
    const int rpb = kThreads >> a.tpr_log2;
    const int64_t step = static_cast<int64_t>(tpr) * VEC;
    int mode[kOperands];
#pragma unroll
    for (int k = 0; k < kOperands; ++k) mode[k] = operand_mode(a, k);
    for (int64_t item = blockIdx.x; item < a.items; item += gridDim.x) {
        int64_t rg, seg;
        if (a.rows == 1) { rg = 0; seg = item; }
        else if (a.segs == 1) { rg = item; seg = 0; }
        else if (a.segs_shift != 0) {
            rg = static_cast<int64_t>((static_cast<uint64_t>(item) * a.segs_magic) >> a.segs_shift);
            seg = item - rg * a.segs;
        } else { rg = item / a.segs; seg = item - rg * a.segs; }
        const int64_t row = rg * rpb + rib;
        if (row >= a.rows) continue;
        int64_t off[kOperands];
        row_offsets(a, row, off);
        T *pp = operand_row<T>(a, 0, off[0]);
        const T *pg = operand_row<T>(a, 1, off[1]);
        T *pm = operand_row<T>(a, 2, off[2]);
        T *pv = operand_row<T>(a, 3, off[3]);
        const int64_t i0 = seg * (step * UNR) + static_cast<int64_t>(lane) * VEC;
        Pack<T, VEC> vp[UNR], vg[UNR], vm[UNR], vv[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t idx = i0 + u * step;
            if (idx < a.n0) {
                load_operand<T, VEC>(vp[u], a, 0, mode[0], pp, idx);
                load_operand<T, VEC>(vg[u], a, 1, mode[1], pg, idx);
                load_operand<T, VEC>(vm[u], a, 2, mode[2], pm, idx);
                load_operand<T, VEC>(vv[u], a, 3, mode[3], pv, idx);
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t idx = i0 + u * step;
            if (idx < a.n0) {
#pragma unroll
                for (int j = 0; j < VEC; ++j) f(vp[u].v[j], vg[u].v[j], vm[u].v[j], vv[u].v[j]);
                store_operand<T, VEC>(vp[u], a, 0, mode[0], pp, idx);
                store_operand<T, VEC>(vm[u], a, 2, mode[2], pm, idx);
                store_operand<T, VEC>(vv[u], a, 3, mode[3], pv, idx);
            }
        }
    }
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_adamw_step(hmc_context_t ctx, const hmc_tensor_desc *param, const hmc_tensor_desc *grad,
                                  const hmc_tensor_desc *exp_avg, const hmc_tensor_desc *exp_avg_sq,
                                  const hmc_adamw_scalars *scalars) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (scalars == nullptr) return fail(HMC_INVALID, "null scalars");
        const hmc_tensor_desc *d[4] = {param, grad, exp_avg, exp_avg_sq};
        for (int k = 0; k < 4; ++k) {
            if (d[k] == nullptr) return fail(HMC_INVALID, "null description");
        }
        int64_t n = 0;
        hmc_status s = check_operands(d, 4, &n);
        if (s != HMC_OK) return s;
        const int dt = param->dtype;
        if (!dtype_is_float(dt) || grad->dtype != dt || exp_avg->dtype != dt || exp_avg_sq->dtype != dt) {
            return fail(HMC_INVALID, "an AdamW step takes floating point tensors of one dtype");
        }
        if (n == 0) return HMC_OK;
        return dispatch_float(dt, [&](auto t) -> hmc_status {
            using T = decltype(t);
            using C = typename Comp<T>::C;
            AdamW<T> f;
            f.decay = static_cast<C>(scalars->decay);
            f.lerp_coeff = static_cast<C>(scalars->lerp_coeff);
            f.beta2 = static_cast<C>(scalars->beta2);
            f.one_minus_beta2 = static_cast<C>(scalars->one_minus_beta2);
            f.bias2_sqrt = static_cast<C>(scalars->bias2_sqrt);
            f.eps = static_cast<C>(scalars->eps);
            f.neg_step_size = static_cast<C>(scalars->neg_step_size);
            f.has_decay = scalars->has_decay != 0;
            f.lerp_small = scalars->lerp_small != 0;
            MapOperand in[3] = {tensor_operand(grad), tensor_operand(exp_avg), tensor_operand(exp_avg_sq)};
            MapArgs a;
            build_map_args(a, param, in, 3, 16 / static_cast<int>(sizeof(T)), 2);
            const int64_t cap = static_cast<int64_t>(ctx->sm_count) * 16;
            const unsigned grid = static_cast<unsigned>(a.items < cap ? a.items : cap);
            adamw_kernel<T><<<grid, kThreads, 0, ctx->stream>>>(a, f);
            return launch_status("adamw kernel launch");
        });
    });
}
