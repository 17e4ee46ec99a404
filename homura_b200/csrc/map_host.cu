// Host side of the elementwise engine: validation of descriptions and the launch geometry.
#include "map.cuh"

#include <algorithm>
#include <utility>

namespace hmc {

hmc_status check_desc(const hmc_tensor_desc *d, const char *what) {
    if (d == nullptr) return fail(HMC_INVALID, std::string("null description of ") + what);
    if (!dtype_valid(d->dtype)) return fail(HMC_INVALID, std::string("unknown dtype code for ") + what);
    if (d->ndim < 0 || d->ndim > HMC_MAX_DIMS) {
        return fail(HMC_INVALID, std::string(what) + " has " + std::to_string(d->ndim) + " dimensions, the limit is " +
                                     std::to_string(HMC_MAX_DIMS));
    }
    if (d->offset < 0) return fail(HMC_INVALID, std::string("negative offset of ") + what);
    for (int k = 0; k < d->ndim; ++k) {
        if (d->sizes[k] < 0) return fail(HMC_INVALID, std::string("negative size in ") + what);
        if (d->strides[k] < 0) return fail(HMC_INVALID, std::string("negative stride in ") + what);
    }
    return HMC_OK;
}

hmc_status check_operands(const hmc_tensor_desc *const *descs, int n, int64_t *count) {
    static const char *names[] = {"the output", "the first input", "the second input", "the third input"};
    const hmc_tensor_desc *first = nullptr;
    for (int i = 0; i < n; ++i) {
        if (descs[i] == nullptr) continue;  // an absent (constant) operand
        hmc_status s = check_desc(descs[i], names[i < 4 ? i : 3]);
        if (s != HMC_OK) return s;
        if (first == nullptr) {
            first = descs[i];
            continue;
        }
        if (descs[i]->ndim != first->ndim) return fail(HMC_INVALID, "operands differ in their number of dimensions");
        for (int k = 0; k < first->ndim; ++k) {
            if (descs[i]->sizes[k] != first->sizes[k]) return fail(HMC_INVALID, "operands differ in their sizes");
        }
    }
    if (first == nullptr) return fail(HMC_INVALID, "no operands");
    int64_t total = 1;
    for (int k = 0; k < first->ndim; ++k) {
        if (first->sizes[k] == 0) {
            total = 0;
            break;
        }
        if (__builtin_mul_overflow(total, first->sizes[k], &total)) {
            return fail(HMC_INVALID, "the number of elements overflows 63 bits");
        }
    }
    if (total > 0) {
        for (int i = 0; i < n; ++i) {
            if (descs[i] != nullptr && descs[i]->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        }
    }
    *count = total;
    return HMC_OK;
}

void build_map_args(MapArgs &a, const hmc_tensor_desc *out, const MapOperand *inputs, int ninputs, int vec, int unr) {
    a = MapArgs{};
    const hmc_tensor_desc *descs[kOperands] = {out, nullptr, nullptr, nullptr};
    for (int k = 0; k < ninputs && k < 3; ++k) {
        if (inputs[k].constant) {
            a.constant_mask |= 1u << (k + 1);
            a.constant[k + 1] = inputs[k].bits;
        } else {
            descs[k + 1] = inputs[k].desc;
        }
    }
    int nd = out->ndim;
    if (nd == 0) {
        a.ndim = 1;
        a.sizes[0] = 1;
        for (int k = 0; k < kOperands; ++k) a.strides[k][0] = 1;
    } else {
        a.ndim = nd;
        for (int d = 0; d < nd; ++d) a.sizes[d] = out->sizes[d];
        for (int k = 0; k < kOperands; ++k) {
            if (descs[k] == nullptr) continue;
            for (int d = 0; d < nd; ++d) a.strides[k][d] = descs[k]->strides[d];
        }
    }
    for (int k = 0; k < kOperands; ++k) {
        if (descs[k] == nullptr) continue;
        a.base[k] = static_cast<char *>(descs[k]->data) + descs[k]->offset * element_size(descs[k]->dtype);
    }
    // Elementwise work may visit the dimensions in any order: put the output's unit-stride dimension last,
    // so that stores are always coalesced and an operand that runs against the grain becomes "transposed".
    if (a.ndim >= 2 && a.strides[0][a.ndim - 1] != 1) {
        for (int d = a.ndim - 2; d >= 0; --d) {
            if (a.strides[0][d] == 1) {
                const int last = a.ndim - 1;
                std::swap(a.sizes[d], a.sizes[last]);
                for (int k = 0; k < kOperands; ++k) std::swap(a.strides[k][d], a.strides[k][last]);
                break;
            }
        }
    }
    // The tiled kernel: some input has unit stride along the second-to-last dimension and not along the last.
    if (a.ndim >= 2 && a.strides[0][a.ndim - 1] == 1 && a.sizes[a.ndim - 1] >= 16 && a.sizes[a.ndim - 2] >= 16) {
        const int da = a.ndim - 2, db = a.ndim - 1;
        for (int k = 1; k < kOperands; ++k) {
            if (descs[k] == nullptr) continue;
            if (a.strides[k][da] == 1 && a.strides[k][db] > 1) a.tile_mask |= 1u << k;
        }
        // (the launch, which knows the tile edge of its element types, counts the tiles)
    }
    a.n0 = a.sizes[a.ndim - 1];
    a.rows = 1;
    for (int d = 0; d < a.ndim - 1; ++d) a.rows *= a.sizes[d];
    if (a.n0 == 0 || a.rows == 0) {
        a.items = 0;
        return;
    }
    int64_t lanes = ceil_div(a.n0, vec);
    int log2 = 0;
    while ((int64_t{1} << log2) < lanes && log2 < 8) ++log2;
    a.tpr_log2 = log2;
    int64_t tpr = int64_t{1} << log2;
    a.segs = ceil_div(a.n0, tpr * vec * unr);
    int64_t rpb = kThreads / tpr;
    a.items = ceil_div(a.rows, rpb) * a.segs;
    a.rows_fit32 = a.rows < (int64_t{1} << 31) ? 1 : 0;
    // Division of an item index below 2^31 by segs as a multiplication: with l = ceil(log2(segs)) and
    // M = floor(2^(31+l) / segs) + 1, floor(n / segs) = (n * M) >> (31 + l) for every n < 2^31.
    if (a.segs > 1 && a.items < (int64_t{1} << 31)) {
        int l = 0;
        while ((int64_t{1} << l) < a.segs) ++l;
        a.segs_shift = 31 + l;
        a.segs_magic = static_cast<uint64_t>((static_cast<unsigned __int128>(1) << a.segs_shift) / static_cast<uint64_t>(a.segs)) + 1;
    }
}

bool build_lean_args(LeanArgs &lean, const MapArgs &a, const int *elem_size, int vec) {
    if (a.ndim > 2 || a.n0 >= (int64_t{1} << 31)) return false;
    // short rows leave most of a block idle here; the general kernel packs several rows into a block
    if (a.rows > 1 && a.n0 < 64 * static_cast<int64_t>(vec)) return false;
    const int last = a.ndim - 1;
    lean = LeanArgs{};
    lean.n0 = static_cast<uint32_t>(a.n0);
    lean.rows = a.rows;
    lean.constant_mask = a.constant_mask;
    for (int k = 0; k < kOperands; ++k) {
        if (elem_size[k] == 0) continue;  // an absent input
        lean.constant[k] = a.constant[k];
        if (a.constant_mask & (1u << k)) continue;
        const int64_t inner = a.strides[k][last];
        const int64_t row_stride = a.ndim == 2 ? a.strides[k][0] : 0;
        if (inner != 1 && !(inner == 0 && k > 0)) return false;
        const int64_t vec_bytes = std::min<int64_t>(16, static_cast<int64_t>(vec) * elem_size[k]);
        if (inner == 1) {
            if (reinterpret_cast<uintptr_t>(a.base[k]) % vec_bytes != 0) return false;
            if (a.rows > 1 && (row_stride * elem_size[k]) % vec_bytes != 0) return false;
        }
        if (inner == 1 && reinterpret_cast<uintptr_t>(a.base[k]) % 32 == 0 && (a.rows == 1 || (row_stride * elem_size[k]) % 32 == 0))
            lean.wide_mask |= 1u << k;
        lean.base[k] = a.base[k];
        lean.row_stride[k] = row_stride;
        lean.inner[k] = inner == 1 ? 1u : 0u;
    }
    return true;
}

}  // namespace hmc
