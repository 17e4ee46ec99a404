// softmax / log_softmax along rows, in f64 like homura's CPU kernel (src/backend/cpu/misc.rs:13-51):
// row maximum (a NaN never wins the comparison), sum of exp(x - max), then exp(x - max) / sum or
// x - max - log(sum), rounded to the dtype once. Stands in for hmr_softmax of csrc/reduce.hip.
//
// A row is handled by a group of G = 32 or 256 lanes. Its elements are cut into 16-byte vectors;
// vector v belongs to lane v mod G. When a lane owns at most 8 vectors the row lives in registers:
// the source is read from HBM once, exp runs once per element, and the output is written once,
// which is the algorithmic minimum of traffic. Longer rows are streamed in three passes (the
// second and third find the row in cache when it fits). Rows whose elements are not adjacent, or
// not 16-byte aligned, take scalar accesses with the same lane assignment and give the same bits.
// exp is skipped for x - max = -inf (a masked logit), whose result is exactly +0.
#include <math_constants.h>

#include <algorithm>
#include <cstdlib>
#include <string>

#include "map.cuh"
#include "math.cuh"
#include "reduce.cuh"

namespace hmc {
namespace {

struct SoftmaxArgs {
    hmc_tensor_desc out_rows;
    hmc_tensor_desc src_rows;
    int64_t nrows, n, so, si;
};

struct SoftmaxPlan {
    int kind;   // 0: row in registers, 1: streaming
    int group;  // 32, 128 or 256
    int cache;  // vectors a lane keeps (kind 0)
};

SoftmaxPlan softmax_plan(int dtype, int64_t n) {
    const int64_t vec = 16 / element_size(dtype);
    const int64_t nvec = ceil_div(n, vec);
    SoftmaxPlan p{};
    // a warp for short rows; 128 lanes (two rows per block) while a lane then holds at most four vectors: the work
    // done once per row and lane (reductions, the reciprocal, addresses) is then spread over twice the elements
    p.group = nvec <= 64 ? 32 : (nvec <= 4 * 128 ? 128 : 256);
    const int64_t per = ceil_div(nvec, p.group);
    p.kind = per <= 8 ? 0 : 1;
    p.cache = 0;
    if (p.kind == 0) {
        p.cache = 1;
        while (p.cache < per) p.cache *= 2;
    }
    return p;
}

// A barrier over the G lanes of a row: the whole block for 256, a named barrier per row for 128 (two rows share
// a block and may take different paths), nothing for a warp.
template <int G>
__device__ __forceinline__ void row_barrier() {
    if constexpr (G == 256) {
        __syncthreads();
    } else if constexpr (G == 128) {
        // (barrier numbers as immediates: a number in a register makes the compiler reserve all sixteen)
        if (threadIdx.x < 128) asm volatile("bar.sync 1, 128;" ::: "memory");
        else asm volatile("bar.sync 2, 128;" ::: "memory");
    }
}
// The warps of a row: W = G / 32 of them, the first at index `first` of the block's eight.
template <int G>
__device__ __forceinline__ double group_max(double v, double *scratch) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        double o = __shfl_xor_sync(0xFFFFFFFFu, v, d);
        v = o > v ? o : v;
    }
    if constexpr (G > 32) {
        constexpr int W = G / 32;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, first = warp / W * W;
        row_barrier<G>();
        if (lane == 0) scratch[warp] = v;
        row_barrier<G>();
        v = scratch[first];
        for (int w = 1; w < W; ++w) v = scratch[first + w] > v ? scratch[first + w] : v;
    }
    return v;
}

template <int G>
__device__ __forceinline__ double group_sum(double v, double *scratch) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, d);
    if constexpr (G > 32) {
        constexpr int W = G / 32;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, first = warp / W * W;
        row_barrier<G>();
        if (lane == 0) scratch[warp] = v;
        row_barrier<G>();
        v = scratch[first];
        for (int w = 1; w < W; ++w) v += scratch[first + w];
    }
    return v;
}

// The same reductions for the rows that live in registers as f32 values: the maximum in f32 (exact), one
// barrier per reduction (the two scratch arrays alternate, so a warp that runs ahead cannot overwrite values
// another warp still reads).
template <int G>
__device__ __forceinline__ float row_max_f32(float v, float *scratch) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
    if constexpr (G > 32) {
        constexpr int W = G / 32;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, first = warp / W * W;
        if (lane == 0) scratch[warp] = v;
        row_barrier<G>();
        v = scratch[first + (lane & (W - 1))];
#pragma unroll
        for (int d = W / 2; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
    }
    return v;
}
template <int G>
__device__ __forceinline__ double row_sum_f64(double v, double *scratch) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, d);
    if constexpr (G > 32) {
        constexpr int W = G / 32;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, first = warp / W * W;
        if (lane == 0) scratch[warp] = v;
        row_barrier<G>();
        // a butterfly over the warps' partial sums: every lane adds the same pairs, so all lanes hold the same bits
        v = scratch[first + (lane & (W - 1))];
#pragma unroll
        for (int d = W / 2; d > 0; d >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, d);
    }
    return v;
}
// max(x, y) that keeps a NaN (fmaxf drops it).
__device__ __forceinline__ float max_keep_nan(float x, float y) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(x), "f"(y));
    return r;
}

// exp(d) for d = x - max <= 0, or NaN. exp(-inf) is +0 without evaluating anything. Rows of F16, BF16 and
// F32 tensors are rounded to at most 24 bits at the end, so their exponentials need 40 good bits, not 53:
// they take the short polynomial; F64 rows take the full f64 exp.
template <class T>
__device__ __forceinline__ double exp_shifted(double d) {
    if (d == -CUDART_INF) return 0.0;
    if constexpr (std::is_same_v<T, double>) return exp(d);
    else return exp_lite(d);
}

// f64 -> T with the hardware's round-to-nearest conversion (through f32 for the half types, as the CPU does);
// a NaN comes out as the hardware's canonical NaN, which no softmax result is compared on.
template <class T> __device__ __forceinline__ T round_f64(double v);
template <> __device__ __forceinline__ float round_f64<float>(double v) { return __double2float_rn(v); }
template <> __device__ __forceinline__ F16 round_f64<F16>(double v) { return down<F16>(__double2float_rn(v)); }
template <> __device__ __forceinline__ BF16 round_f64<BF16>(double v) { return down<BF16>(__double2float_rn(v)); }

// Rows are handled one after the other inside a block (load, max, exp, sum, store are dependent phases), so
// throughput is rows in flight per SM: the register budget keeps three blocks resident while a lane caches up
// to two vectors (plus the two of the row it loads ahead), two blocks beyond that.
constexpr int softmax_min_blocks(int cv) { return cv <= 2 ? 3 : 2; }

template <class T, int G, int CV, bool LOG>
__global__ void __launch_bounds__(kRThreads, softmax_min_blocks(CV)) softmax_kernel(const __grid_constant__ SoftmaxArgs a) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int P = kRThreads / G;
    constexpr int NV = CV > 0 ? CV : 1;
    __shared__ double scratch[8];
    __shared__ double scratch_sum[8];
    __shared__ float scratch_max[8];
    const int lane = threadIdx.x % G;
    const int slot = threadIdx.x / G;
    const int64_t tiles = (a.nrows + P - 1) / P;
    const T *src = static_cast<const T *>(a.src_rows.data);
    T *dst = static_cast<T *>(a.out_rows.data);
    const int64_t nvec = (a.n + VEC - 1) / VEC;
    const double ninf = -CUDART_INF;
    // The vectors of the row a lane handles next, loaded while the current row is computed (rows are dependent
    // phases, so a block with a single row in flight leaves the memory system idle most of the time).
    RVec<T, VEC> ahead[NV];
    bool have_ahead = false;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t r = tile * P + slot;
        const bool valid = r < a.nrows;
        const int64_t rr = valid ? r : 0;
        const T *ps = src + a.src_rows.offset + decompose(a.src_rows, rr, a.src_rows.ndim);
        T *po = dst + a.out_rows.offset + decompose(a.out_rows, rr, a.out_rows.ndim);
        const bool fast_in = a.si == 1 && (reinterpret_cast<uintptr_t>(ps) & 15) == 0;
        const bool fast_out = a.so == 1 && (reinterpret_cast<uintptr_t>(po) & 15) == 0;
        auto load_vec = [&](int64_t v, RVec<T, VEC> &x) {
            const int64_t i0 = v * VEC;
            if (fast_in && i0 + VEC <= a.n) {
                x = *reinterpret_cast<const RVec<T, VEC> *>(ps + i0);
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) x.v[e] = i0 + e < a.n ? ps[(i0 + e) * a.si] : T{};
            }
        };
        auto store_vec = [&](int64_t v, const RVec<T, VEC> &y) {
            const int64_t i0 = v * VEC;
            if (fast_out && i0 + VEC <= a.n) {
                *reinterpret_cast<RVec<T, VEC> *>(po + i0) = y;
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e)
                    if (i0 + e < a.n) po[(i0 + e) * a.so] = y.v[e];
            }
        };
        if constexpr (CV > 0 && !std::is_same_v<T, double>) {
            // Rows of whole, aligned vectors of F16, BF16 or F32: the row is kept as f32 values (its maximum is
            // exact in f32), no element needs a bounds check, and the exponentials take the short f64 polynomial.
            // An element more than 200 below the maximum is moved up to there: its exponential, below 1e-86, still
            // rounds to 0 in the output and vanishes in the sum, and exp_short needs no range check.
            if (fast_in && fast_out && a.n % VEC == 0) {
                float xf[NV][VEC];
                float vmax[NV];  // the vector's maximum, NaN if it holds one
                bool on[NV];
                float mxf = -CUDART_INF_F;
#pragma unroll
                for (int c = 0; c < NV; ++c) {
                    const int64_t v = lane + static_cast<int64_t>(c) * G;
                    on[c] = valid && v < nvec;
                    if (on[c]) {
                        if (!have_ahead) ahead[c] = *reinterpret_cast<const RVec<T, VEC> *>(ps + v * VEC);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) xf[c][e] = up(ahead[c].v[e]);
                        vmax[c] = xf[c][0];
#pragma unroll
                        for (int e = 1; e < VEC; ++e) vmax[c] = max_keep_nan(vmax[c], xf[c][e]);
                        mxf = fmaxf(mxf, vmax[c]);  // a NaN loses here; it reaches the sum below
                    }
                }
                have_ahead = false;
                if (tile + gridDim.x < tiles) {
                    const int64_t rn = (tile + gridDim.x) * P + slot;
                    const bool valid_n = rn < a.nrows;
                    const T *pn = src + a.src_rows.offset + decompose(a.src_rows, valid_n ? rn : 0, a.src_rows.ndim);
                    if ((reinterpret_cast<uintptr_t>(pn) & 15) == 0) {
#pragma unroll
                        for (int c = 0; c < NV; ++c) {
                            const int64_t v = lane + static_cast<int64_t>(c) * G;
                            if (valid_n && v < nvec) ahead[c] = *reinterpret_cast<const RVec<T, VEC> *>(pn + v * VEC);
                        }
                        have_ahead = true;
                    }
                }
                mxf = row_max_f32<G>(mxf, scratch_max);
                const float floor_x = mxf - 200.0f;
                const double mx = static_cast<double>(mxf);
                double ex[LOG ? 1 : NV][LOG ? 1 : VEC];
                double sum = 0.0;
#pragma unroll
                for (int c = 0; c < NV; ++c) {
                    if (!on[c]) continue;
                    if (vmax[c] < floor_x) {
                        // a vector of masked logits: its exponentials round to 0 and vanish in the sum
                        if constexpr (!LOG) {
#pragma unroll
                            for (int e = 0; e < VEC; ++e) ex[c][e] = 0.0;
                        }
                        continue;
                    }
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        const double ev = exp_short(static_cast<double>(max_keep_nan(xf[c][e], floor_x)) - mx);
                        sum += ev;
                        if constexpr (!LOG) ex[c][e] = ev;
                    }
                }
                sum = row_sum_f64<G>(sum, scratch_sum);
                const double log_sum = LOG ? log(sum) : 0.0;
                const double inv = LOG ? 0.0 : reciprocal_short(sum);
#pragma unroll
                for (int c = 0; c < NV; ++c) {
                    if (on[c]) {
                        const int64_t v = lane + static_cast<int64_t>(c) * G;
                        RVec<T, VEC> y;
#pragma unroll
                        for (int e = 0; e < VEC; ++e) {
                            if constexpr (LOG) y.v[e] = from_f64<T>((static_cast<double>(xf[c][e]) - mx) - log_sum);
                            else y.v[e] = from_f64<T>(ex[c][e] * inv);
                        }
                        *reinterpret_cast<RVec<T, VEC> *>(po + v * VEC) = y;
                    }
                }
                continue;
            }
        }
        have_ahead = false;  // (the paths below load for themselves)
        if constexpr (CV > 0) {
            double x[NV][VEC];
            double mx = ninf;
            {
                RVec<T, VEC> raw[NV];
#pragma unroll
                for (int c = 0; c < NV; ++c) {
                    const int64_t v = lane + static_cast<int64_t>(c) * G;
                    if (valid && v < nvec) load_vec(v, raw[c]);
                }
#pragma unroll
                for (int c = 0; c < NV; ++c) {
                    const int64_t v = lane + static_cast<int64_t>(c) * G;
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        const bool in = valid && v < nvec && v * VEC + e < a.n;
                        x[c][e] = in ? to_f64(raw[c].v[e]) : ninf;
                        if (in && x[c][e] > mx) mx = x[c][e];
                    }
                }
            }
            mx = group_max<G>(mx, scratch);
            double sum = 0.0;
#pragma unroll
            for (int c = 0; c < NV; ++c) {
                const int64_t v = lane + static_cast<int64_t>(c) * G;
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const bool in = valid && v < nvec && v * VEC + e < a.n;
                    if (in) {
                        const double d = x[c][e] - mx;
                        if constexpr (LOG) {
                            sum += exp_shifted<T>(d);
                            x[c][e] = d;
                        } else {
                            x[c][e] = exp_shifted<T>(d);
                            sum += x[c][e];
                        }
                    }
                }
            }
            sum = group_sum<G>(sum, scratch);
            const double log_sum = LOG ? log(sum) : 0.0;
            // One division per row for the narrower dtypes: e * (1 / sum) differs from e / sum by an f64 ulp,
            // far below their rounding. F64 rows divide element by element like the CPU.
            constexpr bool kReciprocal = !std::is_same_v<T, double>;
            const double inv = kReciprocal ? 1.0 / sum : 0.0;
#pragma unroll
            for (int c = 0; c < NV; ++c) {
                const int64_t v = lane + static_cast<int64_t>(c) * G;
                if (valid && v < nvec) {
                    RVec<T, VEC> y;
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        y.v[e] = from_f64<T>(LOG ? x[c][e] - log_sum : (kReciprocal ? x[c][e] * inv : x[c][e] / sum));
                    }
                    store_vec(v, y);
                }
            }
        } else {
            double mx = ninf;
            for (int64_t v = lane; valid && v < nvec; v += G) {
                RVec<T, VEC> raw;
                load_vec(v, raw);
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    if (v * VEC + e < a.n) {
                        const double xv = to_f64(raw.v[e]);
                        if (xv > mx) mx = xv;
                    }
                }
            }
            mx = group_max<G>(mx, scratch);
            double sum = 0.0;
            for (int64_t v = lane; valid && v < nvec; v += G) {
                RVec<T, VEC> raw;
                load_vec(v, raw);
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    if (v * VEC + e < a.n) sum += exp_shifted<T>(to_f64(raw.v[e]) - mx);
                }
            }
            sum = group_sum<G>(sum, scratch);
            const double log_sum = LOG ? log(sum) : 0.0;
            for (int64_t v = lane; valid && v < nvec; v += G) {
                RVec<T, VEC> raw, y;
                load_vec(v, raw);
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const double d = to_f64(raw.v[e]) - mx;
                    y.v[e] = from_f64<T>(LOG ? d - log_sum : exp_shifted<T>(d) / sum);
                }
                store_vec(v, y);
            }
        }
    }
}


// ---- rows staged in shared memory, a warp per row ----
//
// For F16, BF16 and F32 rows of whole, aligned vectors (the attention-logit case). The kernel above keeps a row
// in registers, so the bytes a block has in flight are bounded by its registers and the phases of a row (load,
// maximum, exponentials, sum, store) leave the memory system idle in between. Here a warp owns a row and a ring
// of two row buffers in shared memory: while it computes one row from its buffer, the next row is on its way
// from HBM into the other one by asynchronous copies (cp.async, 16 bytes per lane and copy), which need no
// registers. Vector v of a row belongs to lane v mod 32, for the copy and for every pass, so a lane only ever
// reads what it copied itself: cp.async.wait_group is all the synchronisation there is, no barrier. A row is
// read from HBM once and written once.
//
// The maths is the CPU's in f64 (src/backend/cpu/misc.rs:15-51): the maximum is exact in f32; exp(x - max) is
// 2^(k/32) from a table times a cubic in the remainder (relative error below 2^-35, for results that are rounded
// to 24 bits or fewer), ten f64 operations; the sum is added per lane in vector order and folded over the lanes
// by a butterfly. For softmax the exponentials are evaluated a second time for the output instead of being kept
// (64 of them per lane for a row of 2048 would cost 128 registers); a second evaluation gives the same bits. An
// element more than 200 below the maximum is moved up to there (its exponential, below 1e-86, rounds to 0 in the
// output and vanishes in the sum), which keeps 2^k a normal number; a vector that lies entirely below, such as the
// masked half of causal logits, is skipped and stored as zeros.
struct RowExp {
    double mx;  // the row's maximum
    // exp(x - mx). The difference is taken first, in f64 (exact whenever it matters: the maximum itself gives 0 and
    // its exponential exactly 1, as on the CPU, which a row with a single live element shows in log_softmax).
    __device__ __forceinline__ double operator()(float x, const uint64_t *table) const {
        const double t = (static_cast<double>(x) - mx) * (0x1.71547652b82fep+0 * 32.0);
        const double shift = 0x1.8p+52;
        double kd = t + shift;
        const uint32_t ki = static_cast<uint32_t>(__double2loint(kd));
        kd -= shift;
        const double r = t - kd;
        const uint64_t entry = table[ki & 31u];
        const double s = __hiloint2double(static_cast<int>(static_cast<uint32_t>(entry >> 32) + (ki << 15)),
                                          static_cast<int>(static_cast<uint32_t>(entry)));
        const double q = __fma_rn(0x1.c6af84b912394p-5 / 32768.0, r, 0x1.ebfce50fac4f3p-3 / 1024.0);
        const double r2 = r * r;
        double y = __fma_rn(0x1.62e42ff0c52d6p-1 / 32.0, r, 1.0);
        y = __fma_rn(q, r2, y);
        return y * s;
    }
};

// CU vectors of a lane (vectors lane + 32 * (c0 + u), u = 0..CU-1: sixteen elements) as f32 values; vectors beyond
// the row read as -inf. Returns the largest value, NaN if one of them is a NaN.
template <class T, int VEC, int CU>
__device__ __forceinline__ float load_chunk(const RVec<T, VEC> *row, int lane, int c0, int nvec, float (&xf)[CU][VEC]) {
    float top = -CUDART_INF_F;
#pragma unroll
    for (int u = 0; u < CU; ++u) {
        const int v = lane + 32 * (c0 + u);
        if (v < nvec) {
            const RVec<T, VEC> x = row[v];
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                xf[u][e] = up(x.v[e]);
                top = max_keep_nan(top, xf[u][e]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) xf[u][e] = -CUDART_INF_F;
        }
    }
    return top;
}

template <class T, bool LOG>
__global__ void __launch_bounds__(kRThreads, 1) softmax_staged_kernel(const __grid_constant__ SoftmaxArgs a, const int row_bytes) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int CU = 16 / VEC;  // vectors per chunk: sixteen elements
    extern __shared__ __align__(16) unsigned char staged[];
    __shared__ uint64_t table[32];
    if (threadIdx.x < 32) table[threadIdx.x] = lm::kExp2Table[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    unsigned char *ring = staged + static_cast<size_t>(warp) * 2 * row_bytes;
    const int nvec = static_cast<int>(a.n / VEC);
    const int per_lane = (nvec + 31) / 32;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * warps;
    const T *src = static_cast<const T *>(a.src_rows.data) + a.src_rows.offset;
    T *dst = static_cast<T *>(a.out_rows.data) + a.out_rows.offset;
    auto fetch = [&](int64_t r, int stage) {
        const T *ps = src + decompose(a.src_rows, r, a.src_rows.ndim);
        unsigned char *buf = ring + static_cast<size_t>(stage) * row_bytes;
        for (int v = lane; v < nvec; v += 32) async_copy_16(buf + 16 * v, ps + static_cast<size_t>(v) * VEC);
    };
    int64_t r = static_cast<int64_t>(blockIdx.x) * warps + warp;
    if (r < a.nrows) fetch(r, 0);
    async_copy_commit();
    int stage = 0;
    for (; r < a.nrows; r += stride, stage ^= 1) {
        if (r + stride < a.nrows) fetch(r + stride, stage ^ 1);
        async_copy_commit();
        async_copy_wait(1);  // everything but the copies just issued has landed: this row is in its buffer
        const RVec<T, VEC> *row = reinterpret_cast<const RVec<T, VEC> *>(ring + static_cast<size_t>(stage) * row_bytes);
        T *po = dst + decompose(a.out_rows, r, a.out_rows.ndim);
        // pass 1: the maximum (a NaN never wins; it reaches the sum below)
        float mxf = -CUDART_INF_F;
#pragma unroll 4
        for (int v = lane; v < nvec; v += 32) {
            const RVec<T, VEC> x = row[v];
#pragma unroll
            for (int e = 0; e < VEC; ++e) mxf = fmaxf(mxf, up(x.v[e]));
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) mxf = fmaxf(mxf, __shfl_xor_sync(0xFFFFFFFFu, mxf, d));
        const float floor_x = mxf - 200.0f;
        const double mx = static_cast<double>(mxf);
        const RowExp ex{mx};
        // pass 2: the sum of the exponentials, sixteen independent evaluations at a time; a chunk that lies below
        // the floor altogether adds nothing, an element below it inside a live chunk adds less than 1e-86
        double sum = 0.0;
        for (int c0 = 0; c0 < per_lane; c0 += CU) {
            float xf[CU][VEC];
            const float top = load_chunk<T, VEC, CU>(row, lane, c0, nvec, xf);
            if (top < floor_x) continue;  // (false for a NaN)
            double ev[CU][VEC];
#pragma unroll
            for (int u = 0; u < CU; ++u)
#pragma unroll
                for (int e = 0; e < VEC; ++e) ev[u][e] = ex(max_keep_nan(xf[u][e], floor_x), table);
#pragma unroll
            for (int u = 0; u < CU; ++u) {
                // (a vector beyond the row holds -inf, whose clamped exponential is as good as zero; when the whole
                // row is -inf the floor is -inf too and every exponential a NaN, as on the CPU)
                double part = ev[u][0];
#pragma unroll
                for (int e = 1; e < VEC; ++e) part += ev[u][e];
                sum += part;
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
        // pass 3: the outputs
        if constexpr (LOG) {
            const double log_sum = log(sum);
#pragma unroll 4
            for (int v = lane; v < nvec; v += 32) {
                const RVec<T, VEC> x = row[v];
                RVec<T, VEC> y;
#pragma unroll
                for (int e = 0; e < VEC; ++e) y.v[e] = round_f64<T>((static_cast<double>(up(x.v[e])) - mx) - log_sum);
                *reinterpret_cast<RVec<T, VEC> *>(po + static_cast<size_t>(v) * VEC) = y;
            }
        } else {
            const double inv = reciprocal_short(sum);
            // what a skipped element gets: +0, or NaN when the row's sum is one
            const T nothing = round_f64<T>(0.0 * inv);
            for (int c0 = 0; c0 < per_lane; c0 += CU) {
                float xf[CU][VEC];
                const float top = load_chunk<T, VEC, CU>(row, lane, c0, nvec, xf);
                RVec<T, VEC> y[CU];
                if (top < floor_x) {
#pragma unroll
                    for (int u = 0; u < CU; ++u)
#pragma unroll
                        for (int e = 0; e < VEC; ++e) y[u].v[e] = nothing;
                } else {
#pragma unroll
                    for (int u = 0; u < CU; ++u)
#pragma unroll
                        for (int e = 0; e < VEC; ++e) y[u].v[e] = round_f64<T>(ex(max_keep_nan(xf[u][e], floor_x), table) * inv);
                }
#pragma unroll
                for (int u = 0; u < CU; ++u) {
                    const int v = lane + 32 * (c0 + u);
                    if (v < nvec) *reinterpret_cast<RVec<T, VEC> *>(po + static_cast<size_t>(v) * VEC) = y[u];
                }
            }
        }
    }
    async_copy_wait(0);
}

// Whether the staged kernel takes these rows: unit stride inside a row, whole vectors, every row of source and
// output starting on a 16-byte boundary, rows of 256 bytes to 48 KB.
template <class T>
bool staged_rows(const SoftmaxArgs &a) {
    constexpr int VEC = 16 / sizeof(T);
    if (a.si != 1 || a.so != 1 || a.n % VEC != 0) return false;
    const int64_t bytes = a.n * static_cast<int64_t>(sizeof(T));
    if (bytes < 256 || bytes > 48 * 1024) return false;
    for (const hmc_tensor_desc *d : {&a.src_rows, &a.out_rows}) {
        if ((reinterpret_cast<uintptr_t>(d->data) + static_cast<uintptr_t>(d->offset) * sizeof(T)) % 16 != 0) return false;
        for (int k = 0; k < d->ndim; ++k)
            if (d->sizes[k] > 1 && d->strides[k] % VEC != 0) return false;
    }
    return true;
}

template <class T>
hmc_status launch_softmax_staged(hmc_context_t ctx, const SoftmaxArgs &a, bool log) {
    const int row_bytes = static_cast<int>(a.n * sizeof(T));
    // as many warps per block as two row buffers each allow within ~96 KB, so that two blocks share an SM
    int warps = 8;
    const int budget = 96 * 1024;
    while (warps > 1 && static_cast<int64_t>(warps) * 2 * row_bytes > budget) warps >>= 1;
    const size_t shared = static_cast<size_t>(warps) * 2 * row_bytes;
    int per_sm = std::max<int>(1, std::min<int>(8, static_cast<int>((220 * 1024) / (shared + 1024))));
    const int64_t blocks_needed = ceil_div(a.nrows, warps);
    const unsigned grid = clamp_grid(blocks_needed, static_cast<int64_t>(ctx->sm_count) * per_sm);
    auto kernel = log ? softmax_staged_kernel<T, true> : softmax_staged_kernel<T, false>;
    if (shared > 48 * 1024) {
        HMC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)),
                 "shared memory size of the softmax kernel");
    }
    kernel<<<grid, warps * 32, shared, ctx->stream>>>(a, row_bytes);
    return launch_status("softmax kernel launch");
}

// ---- a few very long rows: three launches ----
//
// A row per block leaves most of the GPU idle when there are only a handful of rows, however long. Such
// reductions are split like any other: (1) the rows' maxima by the reduction engine, whose plan cuts each row
// into chunks until the GPU is full, (2) the rows' sums of exp(x - max) the same way, both kept in f64 in the
// caller's workspace, (3) an elementwise pass over all elements that writes exp(x - max) / sum or
// (x - max) - ln(sum). Three reads of the source instead of one, on every SM instead of on four.
// (homura's ROCm layer splits the same way: csrc/reduce.hip:283-300, 348-361.)
template <class TT>
struct MaxSkippingNaN {
    using T = TT;
    using Acc = double;
    __device__ __forceinline__ Acc init() const { return -CUDART_INF; }
    __device__ __forceinline__ Acc load(T x, int64_t, int64_t) const { return to_f64(x); }
    // (a NaN never wins the comparison: src/backend/cpu/misc.rs:25-30)
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return b > a ? b : a; }
};
template <class TT>
struct ExpSum {
    using T = TT;
    using Acc = double;
    const double *maxima;
    double mx;
    __device__ __forceinline__ Acc init() const { return 0.0; }
    __device__ __forceinline__ Acc load(T x, int64_t o, int64_t) const {
        return exp_shifted<T>(to_f64(x) - (maxima != nullptr ? maxima[o] : mx));
    }
    __device__ __forceinline__ ExpSum bound(int64_t o) const { return ExpSum{nullptr, maxima != nullptr ? maxima[o] : mx}; }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return a + b; }
};
struct KeepF64 {
    double *out;
    __device__ __forceinline__ void put(int64_t o, double a, int64_t) const { out[o] = a; }
};

// Grid: (segments of a row, rows). A thread takes 16-byte vectors of its row when both sides allow.
template <class T, bool LOG>
__global__ void __launch_bounds__(kRThreads) softmax_normalize_kernel(const __grid_constant__ SoftmaxArgs a, const double *maxima,
                                                                      const double *sums) {
    constexpr int VEC = 16 / sizeof(T);
    const T *src = static_cast<const T *>(a.src_rows.data);
    T *dst = static_cast<T *>(a.out_rows.data);
    for (int64_t r = blockIdx.y; r < a.nrows; r += gridDim.y) {
        const T *ps = src + a.src_rows.offset + decompose(a.src_rows, r, a.src_rows.ndim);
        T *po = dst + a.out_rows.offset + decompose(a.out_rows, r, a.out_rows.ndim);
        const double mx = maxima[r], sum = sums[r];
        const double log_sum = LOG ? log(sum) : 0.0;
        constexpr bool kReciprocal = !std::is_same_v<T, double>;
        const double inv = (!LOG && kReciprocal) ? 1.0 / sum : 0.0;
        auto one = [&](T x) {
            const double d = to_f64(x) - mx;
            if constexpr (LOG) return from_f64<T>(d - log_sum);
            else return from_f64<T>(kReciprocal ? exp_shifted<T>(d) * inv : exp_shifted<T>(d) / sum);
        };
        const bool vectors = a.si == 1 && a.so == 1 && (reinterpret_cast<uintptr_t>(ps) & 15) == 0 && (reinterpret_cast<uintptr_t>(po) & 15) == 0;
        const int64_t nvec = vectors ? a.n / VEC : 0;
        const int64_t stride = static_cast<int64_t>(gridDim.x) * kRThreads;
        for (int64_t v = static_cast<int64_t>(blockIdx.x) * kRThreads + threadIdx.x; v < nvec; v += stride) {
            const RVec<T, VEC> x = *reinterpret_cast<const RVec<T, VEC> *>(ps + v * VEC);
            RVec<T, VEC> y;
#pragma unroll
            for (int e = 0; e < VEC; ++e) y.v[e] = one(x.v[e]);
            *reinterpret_cast<RVec<T, VEC> *>(po + v * VEC) = y;
        }
        for (int64_t i = nvec * VEC + static_cast<int64_t>(blockIdx.x) * kRThreads + threadIdx.x; i < a.n; i += stride) {
            po[i * a.so] = one(ps[i * a.si]);
        }
    }
}

// The rows as a reduction: kept = the rows' dimensions, reduced = the n elements of a row.
void rows_as_reduction(const SoftmaxArgs &a, ReduceArgs &r) {
    r.kept = a.src_rows;
    r.red = hmc_tensor_desc{};
    r.red.dtype = a.src_rows.dtype;
    r.red.ndim = 1;
    r.red.sizes[0] = a.n;
    r.red.strides[0] = a.si;
    r.plan = make_reduce_plan(r.kept, r.red);
    r.partials = nullptr;
    r.tickets = nullptr;
}

// Few rows, each long enough that cutting it fills the GPU better than a block per row does.
bool split_rows_plan(int64_t nrows, int64_t n) { return nrows <= 128 && n >= (int64_t{1} << 16); }

// Workspace of the split plan: the f64 maxima and sums (256-byte aligned blocks), then the reductions' partials.
int64_t split_bytes(const SoftmaxArgs &a) {
    ReduceArgs r;
    rows_as_reduction(a, r);
    const int64_t block = (a.nrows * 8 + 255) / 256 * 256;
    return 2 * block + plan_partial_bytes(r.plan);
}

template <class T>
hmc_status launch_softmax_split(hmc_context_t ctx, const SoftmaxArgs &a, bool log, void *workspace, int64_t workspace_bytes) {
    const int64_t need = split_bytes(a);
    if (workspace == nullptr || workspace_bytes < need) {
        return fail(HMC_INVALID, "the workspace of softmax is too small: " + std::to_string(need) + " bytes needed");
    }
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return fail(HMC_INVALID, "the workspace of softmax must be 16-byte aligned");
    ReduceArgs r;
    rows_as_reduction(a, r);
    const int64_t block = (a.nrows * 8 + 255) / 256 * 256;
    double *maxima = static_cast<double *>(workspace);
    double *sums = reinterpret_cast<double *>(static_cast<char *>(workspace) + block);
    r.partials = static_cast<char *>(workspace) + 2 * block;
    r.tickets = ctx->tickets;
    hmc_status s = launch_reduce(r, MaxSkippingNaN<T>{}, KeepF64{maxima}, ctx->stream);
    if (s != HMC_OK) return s;
    s = launch_reduce(r, ExpSum<T>{maxima, 0.0}, KeepF64{sums}, ctx->stream);
    if (s != HMC_OK) return s;
    const int64_t per_row = ceil_div(ceil_div(a.n, 16 / static_cast<int64_t>(sizeof(T))), kRThreads * 4);
    const int64_t want = ceil_div(static_cast<int64_t>(ctx->sm_count) * 8, a.nrows);
    dim3 grid(clamp_grid(per_row < want ? per_row : want, 1 << 16), clamp_grid(a.nrows, 65535));
    if (log) softmax_normalize_kernel<T, true><<<grid, kRThreads, 0, ctx->stream>>>(a, maxima, sums);
    else softmax_normalize_kernel<T, false><<<grid, kRThreads, 0, ctx->stream>>>(a, maxima, sums);
    return launch_status("softmax normalize kernel launch");
}

template <class T, int G, int CV>
hmc_status launch_softmax_cv(hmc_context_t ctx, const SoftmaxArgs &a, bool log) {
    constexpr int P = kRThreads / G;
    const int64_t tiles = (a.nrows + P - 1) / P;
    const unsigned grid = clamp_grid(tiles, static_cast<int64_t>(ctx->sm_count) * 32);
    if (log) softmax_kernel<T, G, CV, true><<<grid, kRThreads, 0, ctx->stream>>>(a);
    else softmax_kernel<T, G, CV, false><<<grid, kRThreads, 0, ctx->stream>>>(a);
    return launch_status("softmax kernel launch");
}

template <class T, int G>
hmc_status launch_softmax_g(hmc_context_t ctx, const SoftmaxArgs &a, const SoftmaxPlan &p, bool log) {
    if constexpr (G == 128) {
        // the plan gives 128 lanes only to rows that fit four vectors per lane
        switch (p.cache) {
            case 1: return launch_softmax_cv<T, G, 1>(ctx, a, log);
            case 2: return launch_softmax_cv<T, G, 2>(ctx, a, log);
            default: return launch_softmax_cv<T, G, 4>(ctx, a, log);
        }
    }
    switch (p.kind == 0 ? p.cache : 0) {
        case 1: return launch_softmax_cv<T, G, 1>(ctx, a, log);
        case 2: return launch_softmax_cv<T, G, 2>(ctx, a, log);
        case 4: return launch_softmax_cv<T, G, 4>(ctx, a, log);
        case 8: return launch_softmax_cv<T, G, 8>(ctx, a, log);
        default: return launch_softmax_cv<T, G, 0>(ctx, a, log);
    }
}

hmc_status check_lines(const hmc_tensor_desc *out_rows, const hmc_tensor_desc *src_rows, int64_t n, int64_t so,
                       int64_t si, int64_t *nrows) {
    const hmc_tensor_desc *d[2] = {out_rows, src_rows};
    hmc_status s = check_operands(d, src_rows != nullptr && out_rows != nullptr ? 2 : 0, nrows);
    if (s != HMC_OK) return s;
    if (n < 0 || so < 0 || si < 0) return fail(HMC_INVALID, "negative row length or stride");
    return HMC_OK;
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_softmax_workspace(const hmc_tensor_desc *src_rows, int64_t n, int64_t src_stride,
                                         int64_t *bytes) {
    return guarded([&]() -> hmc_status {
        if (bytes == nullptr) return fail(HMC_INVALID, "null output");
        hmc_status s = check_desc(src_rows, "the rows");
        if (s != HMC_OK) return s;
        if (n < 0 || src_stride < 0) return fail(HMC_INVALID, "negative row length or stride");
        *bytes = 0;  // the other plans work in registers, shared memory and caches
        int64_t nrows = 1;
        for (int k = 0; k < src_rows->ndim; ++k) nrows *= src_rows->sizes[k];
        if (dtype_is_float(src_rows->dtype) && nrows > 0 && split_rows_plan(nrows, n)) {
            SoftmaxArgs a{*src_rows, *src_rows, nrows, n, src_stride, src_stride};
            *bytes = split_bytes(a);
        }
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_test_softmax_plan(const hmc_tensor_desc *src_rows, int64_t n, int64_t src_stride,
                                         int32_t *kind, int32_t *group, int32_t *cache) {
    return guarded([&]() -> hmc_status {
        if (kind == nullptr || group == nullptr || cache == nullptr) return fail(HMC_INVALID, "null output");
        hmc_status s = check_desc(src_rows, "the rows");
        if (s != HMC_OK) return s;
        if (!dtype_is_float(src_rows->dtype)) return fail(HMC_INVALID, "softmax needs a floating point tensor");
        SoftmaxPlan p = softmax_plan(src_rows->dtype, n);
        *kind = p.kind;
        *group = p.group;
        *cache = p.cache;
        int64_t nrows = 1;
        for (int k = 0; k < src_rows->ndim; ++k) nrows *= src_rows->sizes[k];
        if (nrows > 0 && split_rows_plan(nrows, n)) {
            *kind = 3;
            *group = 256;
            *cache = 0;
            return HMC_OK;
        }
        if (src_rows->dtype != HMC_F64) {
            // the plan for rows like these when the output has the same layout: a warp per row, staged in shared memory
            SoftmaxArgs a{*src_rows, *src_rows, 1, n, src_stride, src_stride};
            const bool staged = dispatch_float(src_rows->dtype, [&](auto t) -> hmc_status {
                using T = decltype(t);
                if constexpr (std::is_same_v<T, double>) return HMC_INVALID;
                else return staged_rows<T>(a) ? HMC_OK : HMC_INVALID;
            }) == HMC_OK;
            if (staged) {
                *kind = 2;
                *group = 32;
                *cache = 0;
            }
        }
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_softmax(hmc_context_t ctx, const hmc_tensor_desc *out_rows, const hmc_tensor_desc *src_rows,
                               int64_t n, int64_t out_stride, int64_t src_stride, int32_t log, void *workspace,
                               int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (out_rows == nullptr || src_rows == nullptr) return fail(HMC_INVALID, "null description");
        int64_t nrows = 0;
        hmc_status s = check_lines(out_rows, src_rows, n, out_stride, src_stride, &nrows);
        if (s != HMC_OK) return s;
        if (!dtype_is_float(src_rows->dtype) || out_rows->dtype != src_rows->dtype) {
            return fail(HMC_INVALID, "softmax takes a floating point tensor and writes its dtype");
        }
        if (nrows == 0 || n == 0) return HMC_OK;
        SoftmaxArgs a{*out_rows, *src_rows, nrows, n, out_stride, src_stride};
        const SoftmaxPlan p = softmax_plan(src_rows->dtype, n);
        return dispatch_float(src_rows->dtype, [&](auto t) -> hmc_status {
            using T = decltype(t);
            if (split_rows_plan(nrows, n)) return launch_softmax_split<T>(ctx, a, log != 0, workspace, workspace_bytes);
            if constexpr (!std::is_same_v<T, double>) {
                if (staged_rows<T>(a)) return launch_softmax_staged<T>(ctx, a, log != 0);
            }
            if (p.group == 32) return launch_softmax_g<T, 32>(ctx, a, p, log != 0);
            if (p.group == 128) return launch_softmax_g<T, 128>(ctx, a, p, log != 0);
            return launch_softmax_g<T, 256>(ctx, a, p, log != 0);
        });
    });
}
