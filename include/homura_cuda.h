/*
 * homura_cuda.h: the C ABI of homura's CUDA backend for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a `cuda` feature of homura binds, next to its `rocm` one: the Rust side
 * (the files of src/backend/cuda and the generated ffi.rs) sees exactly these symbols. Each entry point names the
 * declaration of homura's ROCm boundary (csrc/homura_rocm.h) it stands in for.
 *
 * Rules every entry point keeps:
 *  - plain C: only <stddef.h> and <stdint.h>; pointers, sizes and int32 codes;
 *  - the return value is an hmc_status; after a failure hmc_last_error() gives the calling
 *    thread's message until that thread calls the library again;
 *  - no C++ exception leaves the library;
 *  - an entry that works on a device makes it the thread's current CUDA device for the call only;
 *  - a failed entry has queued nothing, and the CUDA runtime's own "last error" is cleared;
 *  - kernels are queued on the context's stream and the entry returns without waiting.
 */
#ifndef HOMURA_CUDA_H
#define HOMURA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status (csrc/homura_rocm.h:26-40) ---- */
#define HMC_OK 0
#define HMC_OUT_OF_MEMORY 1  /* device or pinned host memory exhausted */
#define HMC_INVALID 2        /* bad argument, unsupported op/dtype pair, unsupported GPU */
#define HMC_CUDA_ERROR 3     /* the CUDA runtime (or NCCL) reported an error */
#define HMC_INTERNAL_ERROR 4 /* a fault inside this library, e.g. a caught C++ exception */

typedef int32_t hmc_status;

/* csrc/homura_rocm.h:40 */
const char *hmc_last_error(void);

/* ---- devices (csrc/homura_rocm.h:42-64) ---- */
#define HMC_NAME_LEN 256
#define HMC_ARCH_LEN 64

typedef struct hmc_device_properties {
    char name[HMC_NAME_LEN]; /* e.g. "NVIDIA B200" */
    char arch[HMC_ARCH_LEN]; /* e.g. "sm_100" */
    int32_t multiprocessor_count;
    int32_t warp_size;
    uint64_t total_memory;
} hmc_device_properties;

/* Visible CUDA devices; 0 with HMC_OK when there is no driver or no device.
 * csrc/homura_rocm.h:59 */
hmc_status hmc_device_count(int32_t *count);
/* csrc/homura_rocm.h:61 */
hmc_status hmc_device_properties_get(int32_t device, hmc_device_properties *out);
/* cudaMemGetInfo. csrc/homura_rocm.h:64 */
hmc_status hmc_mem_get_info(int32_t device, uint64_t *free_bytes, uint64_t *total_bytes);

/* ---- context: one device, one non-blocking stream (csrc/homura_rocm.h:66-79) ---- */
typedef struct hmc_context *hmc_context_t;

/* Refuses a GPU whose architecture the library holds no code for (HMC_INVALID), creates the
 * stream, and runs a probe kernel whose answer is checked. Nothing stays allocated on failure. */
hmc_status hmc_context_create(int32_t device, hmc_context_t *out);
hmc_status hmc_context_destroy(hmc_context_t ctx);
hmc_status hmc_context_synchronize(hmc_context_t ctx);

/* ---- memory for the caller's caching allocator (csrc/homura_rocm.h:81-100, 144-146) ---- */
hmc_status hmc_malloc(int32_t device, uint64_t nbytes, void **out);
hmc_status hmc_free(int32_t device, void *ptr);
/* cudaMemsetAsync on the context's stream. */
hmc_status hmc_memset(hmc_context_t ctx, void *ptr, uint8_t value, uint64_t nbytes);
/* Stream-ordered copies between host memory and the device that have completed on return. */
hmc_status hmc_copy_to_host(hmc_context_t ctx, void *dst, const void *src, uint64_t nbytes);
hmc_status hmc_copy_from_host(hmc_context_t ctx, void *dst, const void *src, uint64_t nbytes);
/* Async device-to-device copy of non-overlapping ranges. */
hmc_status hmc_copy_device(hmc_context_t ctx, void *dst, const void *src, uint64_t nbytes);

/* ---- dtypes, numbered as homura's DType (csrc/homura_rocm.h:102-113) ----
 * Bool is a byte 0/1; F16 and BF16 are their 16-bit patterns. */
#define HMC_BOOL 0
#define HMC_U8 1
#define HMC_I8 2
#define HMC_I16 3
#define HMC_I32 4
#define HMC_I64 5
#define HMC_F16 6
#define HMC_BF16 7
#define HMC_F32 8
#define HMC_F64 9

#define HMC_MAX_DIMS 25

/* A strided view of device memory (csrc/homura_rocm.h:118-130). Element (i_0..i_{ndim-1}) lives at
 * element index offset + sum_k i_k * strides[k] of the `dtype` array at `data`. Offsets and
 * strides count elements, not bytes. ndim 0 is one element. The caller has already dropped
 * size-1 dimensions and merged neighbours (src/backend/rocm/copy.rs:34-57). */
typedef struct hmc_tensor_desc {
    void *data;
    int64_t offset;
    int32_t dtype;
    int32_t ndim;
    int64_t sizes[HMC_MAX_DIMS];
    int64_t strides[HMC_MAX_DIMS];
} hmc_tensor_desc;

/* dst[i] = cast(src[i]) with homura's Element::to_element rules (src/dtype.rs:144-273); equal
 * dtypes copy bytes. Same ndim and sizes; src strides may be 0. csrc/homura_rocm.h:138 */
hmc_status hmc_copy(hmc_context_t ctx, const hmc_tensor_desc *dst, const hmc_tensor_desc *src);
/* Every element of dst becomes the low bytes of `bits` (little endian). csrc/homura_rocm.h:142 */
hmc_status hmc_fill(hmc_context_t ctx, const hmc_tensor_desc *dst, uint64_t bits);

/* ---- elementwise (csrc/homura_rocm.h:148-255) ----
 * Results are those of homura's CPU backend (src/backend/cpu/mod.rs): float maths in f32 for
 * F16/BF16/F32 and in f64 for F64 with a single rounding to the dtype; integer arithmetic wraps.
 * Operands share ndim and sizes; inputs may have zero strides; the output's elements are distinct
 * and an input either is the output view itself or does not touch it. */
#define HMC_UNARY_NEG 0
#define HMC_UNARY_ABS 1
#define HMC_UNARY_SIGN 2
#define HMC_UNARY_RELU 3
#define HMC_UNARY_EXP 4
#define HMC_UNARY_LOG 5
#define HMC_UNARY_SQRT 6
#define HMC_UNARY_RSQRT 7
#define HMC_UNARY_RECIPROCAL 8
#define HMC_UNARY_SIN 9
#define HMC_UNARY_COS 10
#define HMC_UNARY_ERF 11
#define HMC_UNARY_TANH 12
#define HMC_UNARY_SIGMOID 13
#define HMC_UNARY_LOG_SIGMOID 14
#define HMC_UNARY_SILU 15
#define HMC_UNARY_GELU 16
#define HMC_UNARY_GELU_TANH 17
#define HMC_UNARY_LOGICAL_NOT 18
#define HMC_UNARY_COUNT 19

#define HMC_BINARY_ADD 0
#define HMC_BINARY_SUB 1
#define HMC_BINARY_MUL 2
#define HMC_BINARY_DIV 3
#define HMC_BINARY_POW 4
#define HMC_BINARY_MAXIMUM 5
#define HMC_BINARY_MINIMUM 6
#define HMC_BINARY_GREATER 7
#define HMC_BINARY_GREATER_EQUAL 8
#define HMC_BINARY_LESS 9
#define HMC_BINARY_LESS_EQUAL 10
#define HMC_BINARY_EQUAL 11
#define HMC_BINARY_NOT_EQUAL 12
#define HMC_BINARY_LOGICAL_AND 13
#define HMC_BINARY_LOGICAL_OR 14
#define HMC_BINARY_COUNT 15

#define HMC_FUSED_SCALED_ADD 0
#define HMC_FUSED_LERP 1
#define HMC_FUSED_ADDCMUL 2
#define HMC_FUSED_ADDCDIV 3

/* out = op(src); LogicalNot writes Bool, everything else src's dtype. csrc/homura_rocm.h:202 */
hmc_status hmc_unary(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                     const hmc_tensor_desc *src);
/* out = op(a, b), a and b of one dtype; comparisons and logical ops write Bool.
 * csrc/homura_rocm.h:206 */
hmc_status hmc_binary(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                      const hmc_tensor_desc *a, const hmc_tensor_desc *b);
/* hmc_binary with one operand replaced by the element of a's dtype held in the low bytes of
 * `bits`; constant_first puts it on the left. csrc/homura_rocm.h:212 */
hmc_status hmc_binary_constant(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                               const hmc_tensor_desc *a, uint64_t bits, int32_t constant_first);
/* MUL or DIV of a float tensor with a scalar kept in the computation type (f32 for F16, BF16,
 * F32): a*s, a/s, or s/a with scalar_first. csrc/homura_rocm.h:217 */
hmc_status hmc_binary_scalar(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                             const hmc_tensor_desc *a, double s, int32_t scalar_first);
/* The optimizers' single-rounding steps on float operands of one dtype; c is NULL for SCALED_ADD
 * and LERP. `coefficient` is exact in the computation type.
 *   SCALED_ADD fma(b, k, a) | LERP fma(k, b - a, small ? a : b)
 *   ADDCMUL fma(k * b, c, a) | ADDCDIV a + k * b / c (no fma)
 * csrc/homura_rocm.h:227 */
hmc_status hmc_fused(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                     const hmc_tensor_desc *a, const hmc_tensor_desc *b,
                     const hmc_tensor_desc *c, double coefficient, int32_t small);
/* out = cond ? x : y with a Bool cond. csrc/homura_rocm.h:247 */
hmc_status hmc_where(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *cond,
                     const hmc_tensor_desc *x, const hmc_tensor_desc *y);
/* hmc_where where a NULL branch is the constant in x_bits / y_bits. csrc/homura_rocm.h:253 */
hmc_status hmc_where_constant(hmc_context_t ctx, const hmc_tensor_desc *out,
                              const hmc_tensor_desc *cond, const hmc_tensor_desc *x,
                              uint64_t x_bits, const hmc_tensor_desc *y, uint64_t y_bits);

/* ---- reductions (csrc/homura_rocm.h:297-346) ----
 * `kept`: kept dimensions with the source's strides, data, offset, dtype. `red`: reduced
 * dimensions with the source's strides. Outputs are contiguous over the kept sizes. The order in
 * which an output's elements are folded is a function of the sizes and strides only, so results
 * repeat from run to run. A plan may need scratch memory: ask hmc_reduce_workspace (var = 1 for
 * hmc_var) and pass at least that many bytes (NULL is fine for 0). */
#define HMC_REDUCE_SUM 0
#define HMC_REDUCE_PROD 1
#define HMC_REDUCE_MEAN 2
#define HMC_REDUCE_MAX 3
#define HMC_REDUCE_MIN 4
#define HMC_REDUCE_ALL 5
#define HMC_REDUCE_ANY 6

/* csrc/homura_rocm.h:315 */
hmc_status hmc_reduce_workspace(const hmc_tensor_desc *kept, const hmc_tensor_desc *red,
                                int32_t var, int64_t *bytes);
/* cpu::reduce (src/backend/cpu/reduce.rs:92-131): float sum/prod/mean in f64, integer and bool
 * sum/prod wrapping into I64, max/min in the dtype (first NaN, then first of equals), all/any to
 * Bool (U8 stays U8). csrc/homura_rocm.h:321 */
hmc_status hmc_reduce(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                      const hmc_tensor_desc *kept, const hmc_tensor_desc *red, void *workspace,
                      int64_t workspace_bytes);
/* cpu::var (src/backend/cpu/reduce.rs:135-170): two passes in f64, divisor max(0, n - correction),
 * NaN for n = 0, sqrt on request. csrc/homura_rocm.h:327 */
hmc_status hmc_var(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *kept,
                   const hmc_tensor_desc *red, double correction, int32_t take_sqrt,
                   void *workspace, int64_t workspace_bytes);
/* cpu::arg_reduce (src/backend/cpu/reduce.rs:175-225): I64 index along the reduced dimension and,
 * unless `values` is NULL, the value. csrc/homura_rocm.h:333 */
hmc_status hmc_arg_reduce(hmc_context_t ctx, const hmc_tensor_desc *values,
                          const hmc_tensor_desc *indices, const hmc_tensor_desc *kept,
                          const hmc_tensor_desc *red, int32_t is_max, void *workspace,
                          int64_t workspace_bytes);
/* cpu::softmax (src/backend/cpu/misc.rs:15-51) on rows of n elements that are out_stride /
 * src_stride apart; out_rows / src_rows describe all other dimensions.
 * csrc/homura_rocm.h:341-346 */
hmc_status hmc_softmax_workspace(const hmc_tensor_desc *src_rows, int64_t n, int64_t src_stride,
                                 int64_t *bytes);
hmc_status hmc_softmax(hmc_context_t ctx, const hmc_tensor_desc *out_rows,
                       const hmc_tensor_desc *src_rows, int64_t n, int64_t out_stride,
                       int64_t src_stride, int32_t log, void *workspace,
                       int64_t workspace_bytes);

/* ---- the callers either side of the path: samplers and the mask builder ---- */

/* Random sampling with the Philox4x32-10 counter of src/ops/random.rs:29-51: block n has the counter
 * [n, n >> 32, 0, 0] under the key [seed, seed >> 32]; the caller reserves the blocks of a call from
 * `offset` on, as the CPU does (random.rs:65-83), and advances its generator. `out` is flat and
 * contiguous (ndim <= 1, stride 1).
 * hmc_random_uniform (sample_float, random.rs:162-183; the clamp at random.rs:268-277): from + u * (to - from)
 *   in f64 for a float `out`; u comes from 53 bits (two words per value, two values per block) for F64 and
 *   from the dtype's significand bits (one word per value, four per block) otherwise; the result is rounded
 *   to the dtype, and one that reaches `to` (with from < to) becomes `from`. Bit for bit the CPU's samples.
 * hmc_random_normal (random.rs:184-197): Box-Muller in f64, two values per block (cosine, then sine),
 *   rounded to the dtype; log, cos and sin are this library's, so a sample may differ from the CPU's in the
 *   last place.
 * csrc/homura_rocm.h:265-281 */
hmc_status hmc_random_uniform(hmc_context_t ctx, const hmc_tensor_desc *out, uint64_t seed, uint64_t offset,
                              double from, double to);
hmc_status hmc_random_normal(hmc_context_t ctx, const hmc_tensor_desc *out, uint64_t seed, uint64_t offset,
                             double mean, double std);

/* The Philox blocks of one tile of hmc_random_int. */
#define HMC_RANDOM_INT_TILE 256

/* One batch of the CPU's integer rejection sampling (sample_int, random.rs:213-238): the 64-bit words of
 * `blocks` blocks from `offset` on, two per block, [w0 w1] then [w2 w3]; the words >= `threshold`, in that
 * order, become low + word % range (wrapping) and fill the I64 `out` until it is full; the rest are dropped.
 * With threshold 0 every word is taken and `workspace` may be NULL. Otherwise `workspace` holds
 * 2 * tiles + 1 64-bit words of device memory, tiles = ceil(blocks / HMC_RANDOM_INT_TILE), and the number of
 * words >= threshold of the batch (which may exceed out's elements) is left in its last word. Elements of out at
 * and beyond that number are unspecified after the call (a later batch fills them).
 * csrc/homura_rocm.h:283-295 */
hmc_status hmc_random_int(hmc_context_t ctx, const hmc_tensor_desc *out, uint64_t seed, uint64_t offset,
                          uint64_t blocks, int64_t low, uint64_t range, uint64_t threshold, void *workspace);

/* cpu::triangle (src/backend/cpu/misc.rs:347-381): out = src where the column minus the row index (the last
 * two dimensions, ndim >= 2) is at least (upper) or at most `diagonal`, else 0; tril / triu, and the causal
 * mask in front of a softmax. csrc/homura_rocm.h:257-260 */
hmc_status hmc_triangle(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src,
                        int64_t diagonal, int32_t upper);

/* cpu::flip (src/backend/cpu/misc.rs:384-411): out = src for one dtype, where src's strides may be negative
 * (the flipped dimensions, with the offset at the element that comes first). csrc/homura_rocm.h:262-263 */
hmc_status hmc_flip(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src);

/* cpu::addr (src/backend/cpu/linalg.rs:227-410): out[i][j] = beta * input[i][j] + alpha * v1[i] * v2[j] with the
 * steps of the CPU kernel, for every dtype. All four descriptions have the output's two dimensions [n, m]: v1 with
 * stride 0 along the columns, v2 along the rows, and the input broadcast; `input` is NULL when beta is zero (it is
 * not read).
 *   floats (coefficients rounded to the dtype, in `alpha` and `beta`): a = alpha * v1[i] (skipped for alpha == 1),
 *     p = a * v2[j], out = p or (beta == 1 ? c : beta * c) + p, each step in the computation type rounded to the dtype;
 *   integers (`alpha_int`, `beta_int`): wrapping, alpha * (v1[i] * v2[j]) + beta * c;
 *   Bool (`alpha_int`, `beta_int` 0 or 1): (v1[i] and alpha and v2[j]) or c.
 * csrc/homura_rocm.h:231-244 */
hmc_status hmc_addr(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *v1, const hmc_tensor_desc *v2,
                    const hmc_tensor_desc *input, double alpha, double beta, int64_t alpha_int, int64_t beta_int);

/* cpu::exclusive_cumprod (src/backend/cpu/reduce.rs:286-329) along lines of `n` elements, described as for
 * hmc_softmax: element k of a line gets the product of the elements before it (after it with `reverse`), 1 for
 * the first (last); the product is accumulated one element at a time in f32 for F16 / BF16 and f64 for F32 / F64 and
 * rounded to the dtype as it is written. Floats only. csrc/homura_rocm.h:348-351 */
hmc_status hmc_exclusive_cumprod(hmc_context_t ctx, const hmc_tensor_desc *out_lines, const hmc_tensor_desc *src_lines,
                                 int64_t n, int64_t out_stride, int64_t src_stride, int32_t reverse);

/* ---- gathers (the read side of csrc/index.hip). Index tensors are I32 or I64; positions are checked first
 * (hmc_index_check), so the gathers take them as valid. ---- */

/* The first element of `index`, in row-major order of its logical positions, that is outside [low, high) and,
 * if has_exempt, not equal to `exempt`: queues writing its position to slot[0] (UINT64_MAX if there is none) and
 * its value to slot[1]. `slot` is two 64-bit words of device memory. csrc/homura_rocm.h:357-363 */
hmc_status hmc_index_check(hmc_context_t ctx, const hmc_tensor_desc *index, int64_t low, int64_t high,
                           int32_t has_exempt, int64_t exempt, uint64_t *slot);

/* cpu::index_select (src/backend/cpu/misc.rs:77-103; an embedding lookup is this along dimension 0): out (src's
 * sizes but `index`'s length along dim) gets the slices of src along dim at the positions of the 1-D `index`,
 * negative ones counted from the end if wrap_negative. out and src have the same number of dimensions.
 * csrc/homura_rocm.h:365-370 */
hmc_status hmc_index_select(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src,
                            const hmc_tensor_desc *index, int32_t dim, int32_t wrap_negative);

/* cpu::gather (src/backend/cpu/misc.rs:319-342): out (index's sizes) gets src at each index position with the
 * coordinate along dim replaced by the index element. csrc/homura_rocm.h:372-375 */
hmc_status hmc_gather(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src,
                      const hmc_tensor_desc *index, int32_t dim);

/* cpu::index_overwrite (src/backend/cpu/misc.rs:105-125): slice i of src along dim is copied to slice positions[i] of
 * out, the last of repeated positions winning; slices of out that no position names are left as they are. `positions`
 * is a contiguous 1-D I64 tensor of valid positions; the workspace has hmc_index_overwrite_workspace bytes for out's
 * size along dim. csrc/homura_rocm.h:383-390 */
hmc_status hmc_index_overwrite_workspace(int64_t size, int64_t *bytes);
hmc_status hmc_index_overwrite(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src,
                               const hmc_tensor_desc *positions, int32_t dim, void *workspace, int64_t workspace_bytes);

/* cpu::index_add (src/backend/cpu/misc.rs:258-293): slice i of src along dim is added into slice index[i] of out, each
 * element of out summed in f64 (floats; integers wrap in i64, a Bool is the or) from its own value, in the order of i,
 * and rounded once. `index` is a 1-D I32 or I64 tensor of m positions (negative ones count from the end; one outside
 * the dimension adds nothing); the workspace has hmc_index_add_workspace bytes. csrc/homura_rocm.h:390-397 */
hmc_status hmc_index_add_workspace(int64_t m, int64_t size, int64_t *bytes);
hmc_status hmc_index_add(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src,
                         const hmc_tensor_desc *index, int32_t dim, void *workspace, int64_t workspace_bytes);

/* cpu::scatter_add (src/backend/cpu/misc.rs:295-317): src at each index position is added into out at that position
 * with the coordinate along dim replaced by the index element, summed as hmc_index_add sums, in row-major order of the
 * index positions. The three descriptions have the same number of dimensions; `index` gives the walked sizes, out its
 * own size along dim. The workspace has hmc_scatter_add_workspace bytes for the index's number of elements.
 * csrc/homura_rocm.h:399-406 */
hmc_status hmc_scatter_add_workspace(int64_t n, int64_t *bytes);
hmc_status hmc_scatter_add(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src,
                           const hmc_tensor_desc *index, int32_t dim, void *workspace, int64_t workspace_bytes);

/* One indexed dimension of advanced indexing (cpu::index_positions, src/backend/cpu/misc.rs:154-204): out (I64) = (if
 * first) or += coord * stride, the coordinate wrapped by `size` when negative; `coord` (I32 or I64) has out's sizes,
 * broadcast by strides of 0. csrc/homura_rocm.h:376-380 */
hmc_status hmc_index_positions(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *coord,
                               int64_t size, int64_t stride, int32_t first);

/* cpu::mask_coordinates (src/backend/cpu/misc.rs:127-151; PyTorch's nonzero, transposed) in two calls:
 * hmc_mask_count queues counting the true elements of the BOOL mask, whose number it leaves at 64-bit word
 * total_word of the workspace (hmc_mask_workspace bytes for the mask's number of elements); hmc_mask_coordinates
 * then writes coordinate d of the k-th true element, in row-major order, to out[d][k] (I64, contiguous, the mask's
 * rank x the number: a two-dimensional description, whose second size bounds what is written). The mask's
 * description keeps the dimensions whose coordinates are wanted (it is not merged).
 * csrc/homura_rocm.h:420-429 */
hmc_status hmc_mask_workspace(int64_t n, int64_t *bytes, int64_t *total_word);
hmc_status hmc_mask_count(hmc_context_t ctx, const hmc_tensor_desc *mask, void *workspace, int64_t workspace_bytes);
hmc_status hmc_mask_coordinates(hmc_context_t ctx, const hmc_tensor_desc *mask, void *workspace, int64_t workspace_bytes,
                                const hmc_tensor_desc *out);

/* ---- additions of this backend (no counterpart in csrc/homura_rocm.h) ---- */

/* hmc_reduce without a workspace argument, for callers that cannot allocate one when they need the
 * reduction (an out-of-memory handler, a loop that must stay clear of the allocator and of driver
 * allocations, a host whose device memory is all in its own arena). No counterpart in homura's ROCm
 * boundary, where the Rust side always brings the workspace. The partials live in an array of
 * HMC_NOALLOC_SCRATCH_BYTES built into the library's device image (held on every GPU that loads the
 * library until the process exits); a reduction whose plan needs more is refused with HMC_INVALID.
 * Same results, bit for bit, as hmc_reduce. The entry point allocates nothing. All calls share the one
 * array: calls that overlap on a GPU race, calls on one context are ordered by its stream. The array's
 * device address is looked up when a context is created on the device (which makes the runtime load the
 * module that holds the array then, not under memory pressure later), else by the first call on that
 * device, which should then come before any stream capture. The runtime loads a kernel's code the first
 * time it is launched unless the process runs with CUDA_MODULE_LOADING=EAGER, and that takes device
 * memory: a caller that must not allocate later makes one call per (op, dtype, layout class) it will
 * need while starting up; from then on a call leaves the device's free memory unchanged. */
#define HMC_NOALLOC_SCRATCH_BYTES 1048576
hmc_status hmc_reduce_noalloc(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                              const hmc_tensor_desc *kept, const hmc_tensor_desc *red);

/* out = a + b where a and b may differ in float dtype and out has the promoted dtype
 * (src/dtype.rs:429-470): the same bits as homura's "cast both with hmc_copy, then hmc_binary ADD"
 * (src/ops/binary.rs:55-60, 132-136) without the temporaries. Also MUL/SUB. */
hmc_status hmc_binary_promoted(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                               const hmc_tensor_desc *a, const hmc_tensor_desc *b);

/* out = (unary(x) first_op b) second_op c in one kernel, with the roundings of the three elementwise kernels
 * homura's front end would issue for it (src/ops/unary.rs:18-57, src/ops/binary.rs:70-143): unary(x) and the
 * first binary result are rounded to the dtype T of x and b, then both operands of the second op are converted to
 * the promoted dtype of (T, dtype of c), which `out` has. The output has the bits of hmc_unary, hmc_binary and
 * hmc_binary_promoted run one after the other, with neither intermediate written to memory. unary_op: RELU, EXP,
 * TANH, SIGMOID, SILU, GELU or GELU_TANH; the binary ops: ADD, SUB or MUL; T: F16, BF16 or F32 with c of the same
 * dtype, or F16 / BF16 with an F32 c. Operands broadcast by stride 0 as everywhere. */
hmc_status hmc_unary_binary_binary(hmc_context_t ctx, int32_t unary_op, int32_t first_op, int32_t second_op,
                                   const hmc_tensor_desc *out, const hmc_tensor_desc *x,
                                   const hmc_tensor_desc *b, const hmc_tensor_desc *c);

/* Scalars of one AdamW step (src/optim/adam.rs:125-171), each already rounded to the parameter
 * dtype's computation type by the caller, as the op-by-op path rounds them. */
typedef struct hmc_adamw_scalars {
    double decay;       /* 1 - lr * weight_decay, multiplies the parameter (skipped when 1) */
    double lerp_coeff;  /* Lerp coefficient for exp_avg: w or w - 1, w = 1 - beta1 */
    int32_t lerp_small; /* |w| < 0.5 */
    int32_t has_decay;  /* weight_decay != 0 */
    double beta2;       /* multiplies exp_avg_sq */
    double one_minus_beta2;
    double bias2_sqrt;  /* divides sqrt(exp_avg_sq) */
    double eps;
    double neg_step_size; /* -lr / (1 - beta1^t) */
} hmc_adamw_scalars;

/* One kernel for the whole decoupled-weight-decay Adam update of one parameter: the same
 * roundings, in the same order, as the sequence of hmc_binary_constant / hmc_fused / hmc_unary /
 * hmc_copy calls that src/optim/adam.rs:139-170 issues. param, exp_avg and exp_avg_sq are
 * updated in place; all four operands have one float dtype, equal sizes, any strides. */
hmc_status hmc_adamw_step(hmc_context_t ctx, const hmc_tensor_desc *param,
                          const hmc_tensor_desc *grad, const hmc_tensor_desc *exp_avg,
                          const hmc_tensor_desc *exp_avg_sq, const hmc_adamw_scalars *scalars);

/* The same update for all tensors of a parameter group (one set of scalars) in one launch, for
 * optimizers that step hundreds of tensors, some of a few hundred elements: homura's loop over the
 * parameters (src/optim/adam.rs:125-171) issues the per-parameter sequence once per tensor. Each entry
 * names four contiguous tensors of n elements of `dtype`; tensors that are views with other strides go
 * through hmc_adamw_step, which gives the same bits (the update must not depend on the layout,
 * tests/optim.rs:430-480). With grad_sq non-null (device memory, `count` doubles) the call also leaves,
 * per tensor, the f64 sum of the squares of its gradient, each square rounded to `dtype` first: what
 * `g.mul(&g).sum()` accumulates before its final rounding, for a gradient norm; the sums are the same on
 * every run. The table is read during the call only. The workspace (device memory, 256-byte aligned,
 * hmc_adamw_step_many_workspace bytes) is used by the kernels of this call; a later call on the same
 * context may reuse it. */
typedef struct hmc_adamw_tensor {
    void *param;
    const void *grad;
    void *exp_avg;
    void *exp_avg_sq;
    int64_t n;
} hmc_adamw_tensor;
hmc_status hmc_adamw_step_many_workspace(int32_t dtype, const hmc_adamw_tensor *tensors, int64_t count,
                                         int32_t with_grad_sq, int64_t *bytes);
hmc_status hmc_adamw_step_many(hmc_context_t ctx, int32_t dtype, const hmc_adamw_tensor *tensors,
                               int64_t count, const hmc_adamw_scalars *scalars, double *grad_sq,
                               void *workspace, int64_t workspace_bytes);

/* Pinned host memory for transfers that should run at link speed. */
hmc_status hmc_host_alloc(uint64_t nbytes, void **out);
hmc_status hmc_host_free(void *ptr);

/* The raw cudaStream_t of a context, for callers that order their own work behind it. */
hmc_status hmc_context_stream(hmc_context_t ctx, void **stream);

/* Elapsed-time markers on the context's stream (cudaEvent_t underneath), so that callers time
 * kernels on the stream they run on. */
typedef struct hmc_event *hmc_event_t;
hmc_status hmc_event_create(hmc_context_t ctx, hmc_event_t *out);
hmc_status hmc_event_record(hmc_context_t ctx, hmc_event_t ev);
hmc_status hmc_event_elapsed_ms(hmc_event_t start, hmc_event_t stop, float *ms);
hmc_status hmc_event_destroy(hmc_event_t ev);

/* ---- introspection (csrc/homura_rocm.h:589-610) ---- */
const char *hmc_built_archs(void);

typedef struct hmc_abi_info {
    uint32_t abi_info_size;
    uint32_t properties_size;
    uint32_t properties_align;
    uint32_t properties_offsets[5];
    int32_t status_values[5];
    int32_t name_len;
    int32_t arch_len;
    uint32_t desc_size;
    uint32_t desc_align;
    uint32_t desc_offsets[6];
    int32_t dtype_values[10];
    int32_t max_dims;
    uint32_t adamw_scalars_size;
    uint32_t adamw_scalars_align;
} hmc_abi_info;

void hmc_abi_check(hmc_abi_info *out);

/* ---- testing hooks, not part of the supported interface (csrc/homura_rocm.h:612-666) ----
 * fail_stream_create(n): the thread's next n stream creations fail with HMC_OUT_OF_MEMORY.
 * fail_after_probe(n): the next n context creations fail late, after stream and probe succeeded.
 * fail_properties(n): the next n hmc_device_properties_get fail with HMC_CUDA_ERROR.
 * fail_data(n, oom): the next n data operations fail before queueing anything.
 * reduce_plan / softmax_plan: which plan the library picks, so tests can reach every path.
 *   reduce: kind (0 rows, 1 columns, 2 generic), splits of the reduced range, elements per split.
 *   softmax: kind (0 row in registers, 1 streaming, 2 row staged in shared memory by a warp, 3 few long
 *   rows split into three launches), lanes per row, vectors a lane keeps.
 * live_streams: streams the thread created and has not destroyed. */
void hmc_test_fail_stream_create(int32_t n);
void hmc_test_fail_after_probe(int32_t n);
void hmc_test_fail_properties(int32_t n);
void hmc_test_fail_data(int32_t n, int32_t out_of_memory);
hmc_status hmc_test_reduce_plan(const hmc_tensor_desc *kept, const hmc_tensor_desc *red,
                                int64_t *kind, int64_t *splits, int64_t *chunk);
hmc_status hmc_test_softmax_plan(const hmc_tensor_desc *src_rows, int64_t n, int64_t src_stride,
                                 int32_t *kind, int32_t *group, int32_t *cache);
/* The second step of hmc_index_check alone: if slot[0] (a logical position of `index`, set by the caller) is not
 * UINT64_MAX, writes the value there to slot[1]: to test positions far beyond what a check could reach in a test
 * (2^60 and more, in views with zero strides). `slot` is device memory. csrc/homura_rocm.h:631-634, 657-658 */
hmc_status hmc_test_index_value(hmc_context_t ctx, const hmc_tensor_desc *index, uint64_t *slot);
int32_t hmc_test_live_streams(void);
hmc_status hmc_test_current_device(int32_t *device);
hmc_status hmc_test_set_current_device(int32_t device);
hmc_status hmc_test_fail(const char *message);

#ifdef __cplusplus
}
#endif

#endif /* HOMURA_CUDA_H */
