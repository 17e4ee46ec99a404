// Float sum / prod / mean and var / std.
#include "math.cuh"
#include "reduce.cuh"

namespace hmc {

hmc_status reduce_float(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, ReduceArgs &a) {
    return dispatch_float(a.kept.dtype, [&](auto t) {
        using T = decltype(t);
        T *o = static_cast<T *>(out->data) + out->offset;
        if (op == HMC_REDUCE_PROD) return launch_reduce(a, FloatFold<T, true>{}, FloatSink<T>{o, nullptr, 0}, ctx->stream);
        return launch_reduce(a, FloatFold<T, false>{}, FloatSink<T>{o, nullptr, op == HMC_REDUCE_MEAN ? 1 : 0}, ctx->stream);
    });
}

hmc_status reduce_float_partial(hmc_context_t ctx, int32_t op, double *partial, ReduceArgs &a) {
    return dispatch_float(a.kept.dtype, [&](auto t) {
        using T = decltype(t);
        if (op == HMC_REDUCE_PROD) return launch_reduce(a, FloatFold<T, true>{}, FloatSink<T>{nullptr, partial, 3}, ctx->stream);
        return launch_reduce(a, FloatFold<T, false>{}, FloatSink<T>{nullptr, partial, 3}, ctx->stream);
    });
}

// The f64 sums of squared deviations from given f64 means, one per output (a shard's share of a variance).
hmc_status reduce_var_partial(hmc_context_t ctx, double *partial, ReduceArgs &a, const double *means) {
    return dispatch_float(a.kept.dtype, [&](auto t) {
        using T = decltype(t);
        return launch_reduce(a, SquaredDeviation<T>{means, 0.0}, FloatSink<T>{nullptr, partial, 3}, ctx->stream);
    });
}

namespace {

// Sum, mean and squared deviations of each output in one kernel, for plans without chunks: the
// second walk over the row finds it in cache. The folds and the team's order are those of the two
// separate reductions, so both routes give the same bits. Grid: one block per 256 / G outputs.
template <int G, class T>
__global__ void __launch_bounds__(kRThreads) deviations_kernel(const __grid_constant__ ReduceArgs a, const VarSink<T> sink) {
    constexpr int kTeams = kRThreads / G;
    const ReducePlan &p = a.plan;
    const int lane = threadIdx.x % G;
    const int team = threadIdx.x / G;
    __shared__ double mean_of[kTeams];
    const FloatFold<T, false> fold;
    const int64_t o = static_cast<int64_t>(blockIdx.x) * kTeams + team;
    const bool live = o < p.nout;
    const int64_t base = live ? a.kept.offset + decompose(a.kept, o, a.kept.ndim) : 0;
    double sum = live ? fold_span<G>(fold, a, o, base, 0, p.nred, lane) : 0.0;
    sum = fold_team<G>(fold, sum);
    if (lane == 0) mean_of[team] = sum / static_cast<double>(p.nred);
    if constexpr (G == 32) __syncwarp();
    else __syncthreads();
    const SquaredDeviation<T> dev{nullptr, mean_of[team]};
    double sq = live ? fold_span<G>(dev, a, o, base, 0, p.nred, lane) : 0.0;
    sq = fold_team<G>(dev, sq);
    if (lane == 0 && live) sink.put(o, sq, p.nred);
}


// ---- variance in one pass ----
// The CPU takes two passes (the mean, then the squared deviations from it, src/backend/cpu/reduce.rs:135-170).
// One pass is enough when the deviations are taken from a nearby constant instead: with c the first value a thread
// meets, d = x - c, s = sum of d and q = sum of d * d, the sum of squared deviations from the true mean is
// M2 = q - s * s / n and the mean is c + s / n. Because c is one of the values, (mean - c)^2 is at most M2, so
// q = M2 + n (mean - c)^2 <= (n + 1) M2: the subtraction cancels at most log2(n + 1) bits of an f64, which leaves
// 30 and more for ranges up to 2^20 values per thread where F16, BF16 and F32 results need 24 (F64 tensors keep
// the two passes). Four f64 operations an element (widen, subtract, add, fused multiply-add), none of them
// waiting for the previous element's result except its own running sum. The moments (count, mean, M2) of
// threads, warps and chunks are then merged pairwise in a fixed order with the update of Chan, Golub and
// LeVeque: mean += d n_b / n, M2 += M2_b + d^2 n_a n_b / n with d = mean_b - mean.
struct alignas(16) Moments {
    double mean, m2;
};
static_assert(sizeof(Moments) == kPartialBytes, "the moments of a chunk are one partial");

__device__ __forceinline__ void merge_moments(double &n, double &mean, double &m2, double nb, double mean_b, double m2_b) {
    if (nb == 0.0) return;
    const double total = n + nb;
    const double d = mean_b - mean;
    const double w = nb * reciprocal_short(total);  // counts are small whole numbers: an ulp or two off nb / total
    mean = n == 0.0 ? mean_b : mean + d * w;
    m2 = n == 0.0 ? m2_b : m2 + m2_b + d * d * n * w;
    n = total;
}

// A thread's share of the chunks' partials of output o in the fold of a strip (see strip_share): chunks h, h + H, ...
// in order, four loads in flight. With a shift common to all chunks the partials are the sums (s, q) themselves
// and simply add up (n counts nothing then); otherwise they are (mean, M2) pairs merged with their counts, which
// follow from the plan.
struct MomentShare {
    double n, a, b;
};
template <int W>
__device__ __forceinline__ MomentShare moment_share(const Moments *partials, int64_t o, bool live, int h, const ReducePlan &p,
                                                    bool common_shift) {
    constexpr int H = kRThreads / W;
    constexpr int B = 4;
    MomentShare r{0.0, 0.0, 0.0};
    if (!live) return r;
    for (int64_t c0 = h; c0 < p.splits; c0 += static_cast<int64_t>(B) * H) {
        Moments m[B];
#pragma unroll
        for (int u = 0; u < B; ++u) {
            if (c0 + u * H < p.splits) m[u] = load_partial(partials + (c0 + u * H) * p.nout + o);
        }
#pragma unroll
        for (int u = 0; u < B; ++u) {
            const int64_t c = c0 + u * H;
            if (c < p.splits) {
                if (common_shift) {
                    r.a += m[u].mean;
                    r.b += m[u].m2;
                } else {
                    const int64_t j0 = c * p.chunk;
                    const int64_t j1 = j0 + p.chunk < p.nred ? j0 + p.chunk : p.nred;
                    merge_moments(r.n, r.a, r.b, static_cast<double>(j1 - j0), m[u].mean, m[u].m2);
                }
            }
        }
    }
    return r;
}

// The strip's fold, by every thread of a block; `memory` holds 3 * (H - 1) * W doubles.
template <int W, class Sink>
__device__ __forceinline__ void fold_moment_strip(const ReduceArgs &a, int64_t outer, int64_t tile, bool common_shift, double *memory,
                                                  const Sink &sink) {
    constexpr int H = kRThreads / W;
    const ReducePlan &p = a.plan;
    const int w = threadIdx.x % W, h = threadIdx.x / W;
    const int64_t c = tile * W + w;
    const bool live = c < p.ncols;
    const int64_t o = outer * p.ncols + c;
    MomentShare r = moment_share<W>(static_cast<const Moments *>(a.partials), live ? o : 0, live, h, p, common_shift);
    if constexpr (H > 1) {
        if (h > 0) {
            double *slot = memory + (static_cast<size_t>(h - 1) * W + w) * 3;
            slot[0] = r.n;
            slot[1] = r.a;
            slot[2] = r.b;
        }
        __syncthreads();
        if (h == 0) {
#pragma unroll
            for (int k = 1; k < H; ++k) {
                const double *slot = memory + (static_cast<size_t>(k - 1) * W + w) * 3;
                if (common_shift) {
                    r.a += slot[1];
                    r.b += slot[2];
                } else {
                    merge_moments(r.n, r.a, r.b, slot[0], slot[1], slot[2]);
                }
            }
        }
    }
    if (h == 0 && live) {
        double m2 = r.b;
        if (common_shift) {
            // (s, q) over the whole column about one shift: M2 = q - s^2 / n
            const double spread = r.b - r.a * r.a * reciprocal_short(static_cast<double>(p.nred));
            m2 = spread > 0.0 ? spread : (spread == spread ? 0.0 : spread);
        }
        sink.put(o, m2, p.nred);
    }
}

// Block 32 x 8 as in the column kernel of the engine: thread (tx, ty) owns VC adjacent columns of its strip and the rows
// j0 + ty, j0 + ty + 8, ... of its chunk. The rows in flight sit in a ring of kVarStages 16-byte slots per thread in
// shared memory, filled by asynchronous copies, so that a thread has 256 bytes on their way at any time without a
// register spent on them (with the loads in registers beside the twelve f64 accumulators of four columns, the
// compiler could keep only half as many in flight).
constexpr int kVarStages = 16;
constexpr int kKnownDevices = 64;
constexpr int64_t kSharedShiftRows = 4096;
constexpr int64_t kCommonShiftRows = int64_t{1} << 18;
constexpr int64_t kRowShiftElements = int64_t{1} << 16;
constexpr int kVarBatch = 4;  // slots consumed and refilled at a time
constexpr size_t kVarSharedBytes = static_cast<size_t>(kVarStages) * kRThreads * 16;

template <class T>
__global__ void __launch_bounds__(kRThreads, 3) var_columns_kernel(const __grid_constant__ ReduceArgs a, const VarSink<T> sink) {
    constexpr int VC = (16 / sizeof(T)) > 8 ? 8 : (16 / sizeof(T));
    const ReducePlan &p = a.plan;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t chunk = blockIdx.y;
    const int64_t j0 = chunk * p.chunk;
    const int64_t j1 = j0 + p.chunk < p.nred ? j0 + p.chunk : p.nred;
    const int last = a.kept.ndim - 1;
    extern __shared__ __align__(16) unsigned char var_shared[];
    // during the walk: the ring; afterwards: the warps' moments on their way to warp 0
    RVec<T, VC> *ring = reinterpret_cast<RVec<T, VC> *>(var_shared) + threadIdx.x;
    static_assert(sizeof(RVec<T, VC>) == 16, "a slot is 16 bytes");
    double(*stage_mean)[32 * VC] = reinterpret_cast<double(*)[32 * VC]>(var_shared);
    double(*stage_m2)[32 * VC] = stage_mean + 7;
    double *stage_n = reinterpret_cast<double *>(stage_m2 + 7);
    static_assert((14 * 32 * VC + 8) * sizeof(double) <= kVarSharedBytes, "the moments fit into the ring's memory");
    // Grid: (kouter * xtiles, splits), one block per strip of 32 * VC outputs and chunk.
    const int64_t outer = blockIdx.x / p.xtiles;
    const int64_t tile = blockIdx.x - outer * p.xtiles;
    const int64_t c0 = tile * (32 * VC) + static_cast<int64_t>(tx) * VC;
    const int64_t base = a.kept.offset + (last > 0 ? decompose(a.kept, outer, last) : 0);
    const int64_t o0 = outer * p.ncols + c0;
    const T *src = static_cast<const T *>(a.kept.data) + base + c0;
    double n = 0.0, mean[VC], m2[VC], held[VC];  // (held: warp 0's shifts when the block shares them)
#pragma unroll
    for (int e = 0; e < VC; ++e) mean[e] = m2[e] = held[e] = 0.0;
    const bool in_range = c0 < p.ncols;
    const bool whole = c0 + VC <= p.ncols;
    // Chunks of up to kSharedShiftRows rows take one shift per column for the whole block: the warps' sums then simply
    // add up, which spares every block eight merges and a division at its end (the cancellation in q - s^2 / n grows
    // with the number of values that share a shift: at most log2(rows + 1) bits, 12 of an f64's 53 here).
    const bool shared_shift = j1 - j0 <= kSharedShiftRows;
    // With several chunks of a column that is not too long, all of them take the column's first value: their sums
    // (s, q) then add up across chunks as well, and the fold at the end needs no merges (the cancellation bound
    // becomes log2(nred + 1) bits, 18 at most here, of which the accumulation error of a thread's 512 rows leaves 26).
    const bool common_shift = (p.chunk < p.nred ? p.chunk : p.nred) <= kSharedShiftRows && p.splits > 1 && p.nred <= kCommonShiftRows;
    if (in_range && j0 + ty < j1) {
        const int64_t stride = a.red.strides[0];
        const bool single = a.red.ndim == 1;
        const bool walk = single && whole && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                          (stride * static_cast<int64_t>(sizeof(T))) % 16 == 0 && j1 - j0 < (int64_t{1} << 31);
        auto red_off = [&](int64_t j) { return single ? j * stride : decompose(a.red, j, a.red.ndim); };
        // the shift of each column: the first value of the chunk (shared by the block's warps), or, for long chunks, the
        // first value this thread meets
        double shift[VC], s[VC], q[VC];
        {
            const T *first = src + red_off(common_shift ? 0 : (shared_shift ? j0 : j0 + ty));
#pragma unroll
            for (int e = 0; e < VC; ++e) {
                shift[e] = c0 + e < p.ncols ? to_f64(first[e]) : 0.0;
                s[e] = q[e] = 0.0;
            }
        }
        auto take = [&](const RVec<T, VC> &x) {
#pragma unroll
            for (int e = 0; e < VC; ++e) {
                const double d = to_f64(x.v[e]) - shift[e];
                s[e] += d;
                q[e] = __fma_rn(d, d, q[e]);
            }
        };
        if (walk) {
            // whole aligned vectors along one reduced dimension: this thread's rows are r = 0 .. rows - 1 at ptr + r * step
            const T *ptr = src + (j0 + ty) * stride;
            const int64_t step = 8 * stride;
            const int rows = static_cast<int>((j1 - (j0 + ty) + 7) / 8);  // (32-bit counters: the loop's bookkeeping is a third of its instructions otherwise)
            static_assert(kVarStages % kVarBatch == 0, "a batch never wraps round the ring");
            // (the copies walk a pointer of their own, kVarStages rows ahead of the row that is consumed)
            const T *ahead = ptr;
            int to_copy = rows;
            auto request = [&](int slot) {  // (a group is committed also when there is nothing left to copy)
                if (to_copy > 0) {
                    ring_copy_16(ring + slot * kRThreads, ahead);
                    ahead += step;
                    --to_copy;
                }
                ring_commit();
            };
            for (int slot = 0; slot < kVarStages; ++slot) request(slot);
            int r = 0;
            int slot = 0;  // of row r
            for (; r + kVarBatch <= rows; r += kVarBatch) {
                ring_wait<kVarStages - kVarBatch>();
                RVec<T, VC> x[kVarBatch];
#pragma unroll
                for (int u = 0; u < kVarBatch; ++u) x[u] = ring[(slot + u) * kRThreads];
#pragma unroll
                for (int u = 0; u < kVarBatch; ++u) take(x[u]);
#pragma unroll
                for (int u = 0; u < kVarBatch; ++u) request(slot + u);
                slot = slot + kVarBatch == kVarStages ? 0 : slot + kVarBatch;
            }
            ring_wait<0>();
            for (; r < rows; ++r, ++slot) take(ring[slot * kRThreads]);
            n = static_cast<double>(rows);
        } else {
            for (int64_t j = j0 + ty; j < j1; j += 8) {
                const T *row = src + red_off(j);
#pragma unroll
                for (int e = 0; e < VC; ++e) {
                    if (c0 + e < p.ncols) {
                        const double d = to_f64(row[e]) - shift[e];
                        s[e] += d;
                        q[e] = __fma_rn(d, d, q[e]);
                    }
                }
                n += 1.0;
            }
        }
        if (shared_shift) {
            // (s, q) travel as they are; warp 0 keeps the shifts for when it has the block's sums
#pragma unroll
            for (int e = 0; e < VC; ++e) {
                mean[e] = s[e];
                m2[e] = q[e];
                held[e] = shift[e];
            }
        } else {
            const double inv = 1.0 / n;
#pragma unroll
            for (int e = 0; e < VC; ++e) {
                mean[e] = shift[e] + s[e] * inv;
                const double spread = q[e] - s[e] * s[e] * inv;
                m2[e] = spread > 0.0 ? spread : (spread == spread ? 0.0 : spread);  // (rounding may leave -0.0...; a NaN stays)
            }
        }
    }
    __syncthreads();  // every thread is done with its ring: the memory now carries the warps' moments
    if (ty > 0) {
#pragma unroll
        for (int e = 0; e < VC; ++e) {
            stage_mean[ty - 1][tx * VC + e] = mean[e];
            stage_m2[ty - 1][tx * VC + e] = m2[e];
        }
    }
    if (tx == 0) stage_n[ty] = n;
    __syncthreads();
    if (ty == 0 && in_range) {
#pragma unroll
        for (int e = 0; e < VC; ++e) {
            if (c0 + e >= p.ncols) continue;
            double cn = n, cm = mean[e], c2 = m2[e];
            if (shared_shift) {
                // the warps' sums in warp order, then the chunk's moments from them
                for (int w = 0; w < 7; ++w) {
                    cm += stage_mean[w][tx * VC + e];
                    c2 += stage_m2[w][tx * VC + e];
                }
                if (!common_shift) {
                    const double rows = static_cast<double>(j1 - j0);
                    const double inv = reciprocal_short(rows);
                    const double spread = c2 - cm * cm * inv;
                    c2 = spread > 0.0 ? spread : (spread == spread ? 0.0 : spread);
                    cm = held[e] + cm * inv;
                }
            } else {
                for (int w = 0; w < 7; ++w) merge_moments(cn, cm, c2, stage_n[w + 1], stage_mean[w][tx * VC + e], stage_m2[w][tx * VC + e]);
            }
            if (p.splits == 1) sink.put(o0 + e, c2, p.nred);
            else static_cast<Moments *>(a.partials)[chunk * p.nout + o0 + e] = Moments{cm, c2};
        }
    }
    if (p.splits == 1 || a.tickets == nullptr || !drew_last_ticket(a.tickets)) return;
    // this block is the last of its strip's (and every thread is past the staging area): fold the strip
    fold_moment_strip<32 * VC>(a, outer, tile, common_shift, reinterpret_cast<double *>(var_shared), sink);
}

// The same fold as a kernel of its own (more chunks than a last block folds, or no counters). Grid: one block per strip.
template <class T>
__global__ void __launch_bounds__(kRThreads) var_combine_kernel(const __grid_constant__ ReduceArgs a, const VarSink<T> sink) {
    constexpr int VC = (16 / sizeof(T)) > 8 ? 8 : (16 / sizeof(T));
    constexpr int W = 32 * VC, H = kRThreads / W;
    __shared__ double memory[3 * (H > 1 ? H - 1 : 1) * W];
    const ReducePlan &p = a.plan;
    const int64_t outer = blockIdx.x / p.xtiles;
    const int64_t tile = blockIdx.x - outer * p.xtiles;
    const int64_t chunk_rows = p.chunk < p.nred ? p.chunk : p.nred;
    const bool common_shift = chunk_rows <= kSharedShiftRows && p.splits > 1 && p.nred <= kCommonShiftRows;
    fold_moment_strip<W>(a, outer, tile, common_shift, memory, sink);
}

// ---- variance over rows in one pass ----
// The same for rows that are one unit-stride run of whole, aligned 32-byte pieces (plan.simple): piece w belongs to
// lane w mod G, read by one 256-bit load, four in flight; a lane takes the shift from its first element and keeps
// four (s, q) pairs, so that consecutive elements add to different running sums; the pairs share the shift and
// simply add up. The lanes of a row are merged in lane
// order by shuffles and, for 256 lanes, the warps in warp order through shared memory. The row is read once; the
// two-pass kernel above reads it twice and misses the caches for part of the second walk.
// Grid: one block per 256 / G rows.
template <int G, class T>
__global__ void __launch_bounds__(kRThreads, 4) var_rows_kernel(const __grid_constant__ ReduceArgs a, const VarSink<T> sink) {
    constexpr int kTeams = kRThreads / G;
    constexpr int N = Piece<T>::N;  // elements of a 32-byte piece
    constexpr int K = 4;            // running sums per lane: element e of a piece adds to pair e % K
    constexpr int UNR = 4;          // pieces in flight
    const ReducePlan &p = a.plan;
    const int lane = threadIdx.x % G;
    __shared__ double warp_n[8], warp_mean[8], warp_m2[8];
    const uint32_t pieces = static_cast<uint32_t>(p.nred) / N;
    const int64_t o = static_cast<int64_t>(blockIdx.x) * kTeams + threadIdx.x / G;
    const bool live = o < p.nout;
    double n = 0.0, mean = 0.0, m2 = 0.0;
    // Rows of up to kRowShiftElements share one shift, the row's first element: the lanes' sums then simply add up
    // (shuffles and additions instead of five merges with a reciprocal each per row), at a cancellation of at most
    // log2(nred + 1) = 16 bits, of which the accumulation error of a lane's 2048 elements leaves 26.
    const bool row_shift = p.nred <= kRowShiftElements;
    if (live && static_cast<uint32_t>(lane) < pieces) {
        const T *row = static_cast<const T *>(a.kept.data) + a.kept.offset + decompose(a.kept, o, a.kept.ndim);
        const double shift = to_f64(row[row_shift ? 0 : static_cast<size_t>(lane) * N]);
        double s[K], q[K];
#pragma unroll
        for (int k = 0; k < K; ++k) s[k] = q[k] = 0.0;
        auto take = [&](const Piece<T> &x) {
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const double d = to_f64(x.v[e]) - shift;
                s[e % K] += d;
                q[e % K] = __fma_rn(d, d, q[e % K]);
            }
        };
        uint32_t w = lane, taken = 0;
        for (; w + (UNR - 1) * G < pieces; w += UNR * G, taken += UNR) {
            Piece<T> x[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u) x[u] = load_piece(row + static_cast<size_t>(w + u * G) * N);
#pragma unroll
            for (int u = 0; u < UNR; ++u) take(x[u]);
        }
        for (; w < pieces; w += G, ++taken) take(load_piece(row + static_cast<size_t>(w) * N));
        double st = (s[0] + s[1]) + (s[2] + s[3]), qt = (q[0] + q[1]) + (q[2] + q[3]);
        if (row_shift) {
            mean = st;  // (the sums travel in the places of mean and M2)
            m2 = qt;
        } else {
            n = static_cast<double>(taken) * N;
            mean = shift + st / n;
            const double spread = qt - st * st / n;
            m2 = spread > 0.0 ? spread : (spread == spread ? 0.0 : spread);
        }
    }
    if (row_shift) {
        // the lanes' sums in lane order, the warps' in warp order, then the row's M2 from them
        if constexpr (G > 1) {
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                mean += __shfl_down_sync(0xFFFFFFFFu, mean, d);
                m2 += __shfl_down_sync(0xFFFFFFFFu, m2, d);
            }
        }
        if constexpr (G == 256) {
            const int warp = threadIdx.x >> 5;
            if ((threadIdx.x & 31) == 0) {
                warp_mean[warp] = mean;
                warp_m2[warp] = m2;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < 8; ++w) {
                    mean += warp_mean[w];
                    m2 += warp_m2[w];
                }
            }
        }
        if (lane == 0 && live) {
            const double spread = m2 - mean * mean * reciprocal_short(static_cast<double>(p.nred));
            sink.put(o, spread > 0.0 ? spread : (spread == spread ? 0.0 : spread), p.nred);
        }
        return;
    }
    if constexpr (G > 1) {
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const double on = __shfl_down_sync(0xFFFFFFFFu, n, d);
            const double om = __shfl_down_sync(0xFFFFFFFFu, mean, d);
            const double o2 = __shfl_down_sync(0xFFFFFFFFu, m2, d);
            merge_moments(n, mean, m2, on, om, o2);
        }
    }
    if constexpr (G == 256) {
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) {
            warp_n[warp] = n;
            warp_mean[warp] = mean;
            warp_m2[warp] = m2;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < 8; ++w) merge_moments(n, mean, m2, warp_n[w], warp_mean[w], warp_m2[w]);
        }
    }
    if (lane == 0 && live) sink.put(o, m2, p.nred);
}

}  // namespace

hmc_status reduce_var(hmc_context_t ctx, const hmc_tensor_desc *out, ReduceArgs &a, double correction, int take_sqrt,
                      double *means) {
    return dispatch_float(a.kept.dtype, [&](auto t) -> hmc_status {
        using T = decltype(t);
        const ReducePlan &p = a.plan;
        T *o = static_cast<T *>(out->data) + out->offset;
        double divisor = static_cast<double>(p.nred) - correction;
        if (!(divisor > 0.0)) divisor = 0.0;
        VarSink<T> sink{o, divisor, take_sqrt};
        if (p.kind == 0 && p.splits == 1) {
            if constexpr (!std::is_same_v<T, double>) {
                // every row one aligned run of whole pieces: the one-pass kernel
                bool aligned = p.simple && p.group > 1 &&
                               (reinterpret_cast<uintptr_t>(a.kept.data) + static_cast<uintptr_t>(a.kept.offset) * sizeof(T)) % 32 == 0;
                for (int k = 0; k < a.kept.ndim; ++k) aligned = aligned && (a.kept.strides[k] * static_cast<int64_t>(sizeof(T))) % 32 == 0;
                if (aligned) {
                    const int64_t per = kRThreads / p.group;
                    if ((p.nout + per - 1) / per > 0x7FFFFFFF) return fail(HMC_INVALID, "a reduction with more than 2^31 blocks of outputs");
                    const unsigned g = static_cast<unsigned>((p.nout + per - 1) / per);
                    if (p.group == 256) var_rows_kernel<256, T><<<g, kRThreads, 0, ctx->stream>>>(a, sink);
                    else var_rows_kernel<32, T><<<g, kRThreads, 0, ctx->stream>>>(a, sink);
                    return launch_status("var kernel launch");
                }
            }
            const int64_t per_block = kRThreads / p.group;
            const int64_t blocks = (p.nout + per_block - 1) / per_block;
            if (blocks > 0x7FFFFFFF) return fail(HMC_INVALID, "a reduction with more than 2^31 blocks of outputs");
            const unsigned grid = static_cast<unsigned>(blocks);
            if (p.group == 256) deviations_kernel<256, T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
            else if (p.group == 32) deviations_kernel<32, T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
            else deviations_kernel<1, T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
            return launch_status("var kernel launch");
        }
        if constexpr (!std::is_same_v<T, double>) {
            if (p.kind == 1) {
                const int64_t strips = p.kouter * p.xtiles;
                if (strips > 0x7FFFFFFF) return fail(HMC_INVALID, "a reduction with more than 2^31 strips of outputs");
                ReduceArgs args = a;
                const ReducePlan &q = args.plan;
                dim3 grid(static_cast<unsigned>(strips), static_cast<unsigned>(q.splits));
                // few chunks: the block that finishes last merges its strip's; else a second kernel (same order)
                const bool self_merge = q.splits > 1 && a.tickets != nullptr && strips <= kTickets && q.splits <= kSelfFoldSplits;
                if (!self_merge) args.tickets = nullptr;
                static bool raised[kKnownDevices] = {};  // (a race between threads only repeats the call)
                if (ctx->device >= kKnownDevices || !raised[ctx->device]) {
                    HMC_CUDA(cudaFuncSetAttribute(var_columns_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  static_cast<int>(kVarSharedBytes)),
                             "shared memory size of the variance kernel");
                    if (ctx->device < kKnownDevices) raised[ctx->device] = true;
                }
                var_columns_kernel<T><<<grid, kRThreads, kVarSharedBytes, ctx->stream>>>(args, sink);
                hmc_status s1 = launch_status("var kernel launch");
                if (s1 != HMC_OK || q.splits == 1 || self_merge) return s1;
                var_combine_kernel<T><<<static_cast<unsigned>(strips), kRThreads, 0, ctx->stream>>>(args, sink);
                return launch_status("var combine kernel launch");
            }
        }
        hmc_status s = launch_reduce(a, FloatFold<T, false>{}, FloatSink<T>{nullptr, means, 2}, ctx->stream);
        if (s != HMC_OK) return s;
        return launch_reduce(a, SquaredDeviation<T>{means, 0.0}, sink, ctx->stream);
    });
}

}  // namespace hmc
