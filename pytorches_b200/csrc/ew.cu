// Elementwise kernels of the B200 plugin: unary ops, binary ops with N-d strided broadcasting,
// AXPY, FILL, RAND_NORMAL. They take the place of plugins/cpu/src/ew.rs in the reference CPU plugin.
//
// All of this is HBM-bound streaming work, so the design is about bytes in flight, not math:
//   * 128-bit (float4) coalesced accesses; every thread issues all loads of its UNROLL work items
//     before the first use, so a CTA keeps BLOCK*UNROLL*16 bytes per operand in flight;
//   * a "flat" kernel for fully contiguous operands (and scalar broadcasts);
//   * a "rows" kernel for everything whose innermost coalesced dim has operand strides 0 or 1: the
//     work item is one float4 of one row; the row number is split over the outer dims with exact
//     multiply-high division, and the dim tables travel in the kernel's constant parameter bank;
//   * a "tile" kernel for operands whose unit stride sits in another dim than the output's
//     (transposed views): 32x32 tiles go through padded shared memory so both sides stay coalesced;
//   * a generic gather kernel for whatever is left.
// Outputs are always contiguous (docs/plugin-abi.md:169). Buffers start on 256-byte boundaries
// (handles are never offset by the host, docs/plugin-abi.md:119-122), so float4 access at a multiple
// of 4 elements is always aligned.
//
// Arithmetic is one IEEE operation per element, written with the __f*_rn intrinsics so that no
// multiply-add contraction can change bits relative to the reference.
#include "common.cuh"
#include "vecmath.cuh"

namespace b200 {

namespace {

enum : uint32_t {
    OP_NEG = 1, OP_EXP = 2, OP_LOG = 3, OP_RELU = 4, OP_TANH = 5, OP_STEP = 6,
    OP_ADD = 100, OP_SUB = 101, OP_MUL = 102, OP_DIV = 103, OP_COPY = 300,
    OP_RELU_GRAD = 501, OP_ADD_RELU = 502, OP_SUB_EXP = 503,
};

// ---- per-element functors ------------------------------------------------------------------------
// Unary semantics follow plugins/cpu/src/ew.rs:96-106 (RELU is max(v, 0) with NaN -> 0; STEP is v > 0).
template <uint32_t OP> struct UnaryFn;
template <> struct UnaryFn<OP_NEG> { static constexpr bool SPLIT = false; __device__ __forceinline__ static float f(float v) { return -v; } };
template <> struct UnaryFn<OP_RELU> { static constexpr bool SPLIT = false; __device__ __forceinline__ static float f(float v) { return v > 0.0f ? v : 0.0f; } };
template <> struct UnaryFn<OP_STEP> { static constexpr bool SPLIT = false; __device__ __forceinline__ static float f(float v) { return v > 0.0f ? 1.0f : 0.0f; } };
template <> struct UnaryFn<OP_COPY> { static constexpr bool SPLIT = false; __device__ __forceinline__ static float f(float v) { return v; } };
// EXP/LOG/TANH: `f` is the reference's vector polynomial. `libm` stands in for the C library call the
// reference makes on the elements its 8-wide vector loop does not cover (plugins/cpu/src/ew.rs:114-138):
// evaluated in double and rounded once, it is correctly rounded in all but vanishingly rare cases and
// so within an ulp or two of any good libm.
template <> struct UnaryFn<OP_EXP> {
    static constexpr bool SPLIT = true;
    __device__ __forceinline__ static float f(float v) { return exp_ref(v); }
    __device__ __noinline__ static float libm(float v) { return (float)exp((double)v); }
};
template <> struct UnaryFn<OP_LOG> {
    static constexpr bool SPLIT = true;
    __device__ __forceinline__ static float f(float v) { return log_ref(v); }
    __device__ __noinline__ static float libm(float v) { return (float)log((double)v); }
};
template <> struct UnaryFn<OP_TANH> {
    static constexpr bool SPLIT = true;
    __device__ __forceinline__ static float f(float v) { return tanh_ref(v); }
    __device__ __noinline__ static float libm(float v) { return (float)tanh((double)v); }
};

// Which elements of a unary op the reference computes with libm instead of its vector polynomial.
// The reference cuts the output into chunks of 65536 elements (the whole tensor below 32768,
// ew.rs:13-15,160), walks each chunk as runs of the innermost dim (ew.rs:46-87), and per run:
//   inner stride 1: polynomial on the first len/8*8 elements of the run, libm on the rest;
//   inner stride 0: one value, computed alone, hence by libm (ew.rs:168-172);
//   other strides:  the run is gathered 256 elements at a time and each piece is split the same way.
struct LibmSplit {
    uint64_t n;      // output elements
    uint64_t inner;  // size of the innermost coalesced dim (n if there is just one)
    int mode;        // 0: inner stride 1, 1: always libm, 2: gathered in 256s
    __device__ __forceinline__ bool uses_libm(uint64_t pos) const {
        if (mode == 1) return true;
        const uint64_t chunk = n < 32768 ? n : 65536;
        const uint64_t c_lo = pos / chunk * chunk, r_lo = pos / inner * inner;
        uint64_t lo = c_lo > r_lo ? c_lo : r_lo;
        uint64_t hi = c_lo + chunk < r_lo + inner ? c_lo + chunk : r_lo + inner;
        if (hi > n) hi = n;
        if (mode == 2) {
            lo += (pos - lo) / 256 * 256;
            if (hi > lo + 256) hi = lo + 256;
        }
        return pos - lo >= ((hi - lo) & ~7ull);
    }
};

template <class Fn> __device__ __forceinline__ float apply_unary(float v, bool libm) {
    if constexpr (Fn::SPLIT) {
        if (libm) return Fn::libm(v);
    }
    return Fn::f(v);
}

// TAIL: the op ends in EXP, whose last (n mod 8) output elements the reference computes with libm.
template <uint32_t OP> struct BinaryFn;
template <> struct BinaryFn<OP_ADD> { static constexpr bool TAIL = false; __device__ __forceinline__ static float f(float a, float b) { return __fadd_rn(a, b); } };
template <> struct BinaryFn<OP_SUB> { static constexpr bool TAIL = false; __device__ __forceinline__ static float f(float a, float b) { return __fsub_rn(a, b); } };
template <> struct BinaryFn<OP_MUL> { static constexpr bool TAIL = false; __device__ __forceinline__ static float f(float a, float b) { return __fmul_rn(a, b); } };
template <> struct BinaryFn<OP_DIV> { static constexpr bool TAIL = false; __device__ __forceinline__ static float f(float a, float b) { return __fdiv_rn(a, b); } };
// The appended fused ops: each is the two reference ops it names, applied one after the other to the
// element, so the result carries the bits of the two-op sequence (the intermediate of that sequence
// is an f32 tensor; here it is an f32 register).
//   RELU_GRAD = MUL(g, STEP(x)): a real multiply by 1 or 0, so that g = -3 gives -0 and g = inf gives NaN
//   exactly as the sequence does.
template <> struct BinaryFn<OP_RELU_GRAD> {
    static constexpr bool TAIL = false;
    __device__ __forceinline__ static float f(float g, float x) { return __fmul_rn(g, UnaryFn<OP_STEP>::f(x)); }
};
template <> struct BinaryFn<OP_ADD_RELU> {
    static constexpr bool TAIL = false;
    __device__ __forceinline__ static float f(float a, float b) { return UnaryFn<OP_RELU>::f(__fadd_rn(a, b)); }
};
// SUB_EXP = EXP(SUB(a, b)). The EXP of the sequence reads a contiguous intermediate, so the reference
// computes all but the last (n mod 8) elements of the whole output with its polynomial and those few
// with libm (plugins/cpu/src/ew.rs:114-138,160); `libm` is applied to them by a second, tiny launch.
template <> struct BinaryFn<OP_SUB_EXP> {
    static constexpr bool TAIL = true;
    __device__ __forceinline__ static float f(float a, float b) { return exp_ref(__fsub_rn(a, b)); }
    __device__ __noinline__ static float libm(float a, float b) { return UnaryFn<OP_EXP>::libm(__fsub_rn(a, b)); }
};

// ---- memory access helpers --------------------------------------------------------------------------
// Inputs are read once: bypass L1 allocation. Outputs are written once: streaming stores.
__device__ __forceinline__ float4 ld4(const float *p) { return __ldcs(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float ld1(const float *p) { return __ldcs(p); }
__device__ __forceinline__ void st4(float *p, float4 v) { __stcs(reinterpret_cast<float4 *>(p), v); }
__device__ __forceinline__ void st1(float *p, float v) { __stcs(p, v); }

constexpr int EW_BLOCK = 256;
constexpr int EW_UNROLL = 4;

// Grid for a kernel whose CTAs each take BLOCK*UNROLL work items.
inline unsigned tiles_for(uint64_t items, int per_cta) { return (unsigned)((items + per_cta - 1) / per_cta); }

// ---- flat kernels: contiguous operands, optional scalar broadcast ------------------------------------
// MODE 0: out[i] = f(a[i], b[i]);  1: f(a[i], b[0]);  2: f(a[0], b[i]);  3: f(a[0], b[0]).
// A work item is 4 consecutive elements; the last item may be partial and is done element by element.
template <class Fn, int MODE>
__global__ void __launch_bounds__(EW_BLOCK) binary_flat_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                                               float *__restrict__ out, uint64_t n) {
    ordered_start();
    const uint64_t items = (n + 3) >> 2;
    const uint64_t tile = (uint64_t)blockIdx.x * (EW_BLOCK * EW_UNROLL) + threadIdx.x;
    float4 va[EW_UNROLL], vb[EW_UNROLL];
    float sa = 0.0f, sb = 0.0f;
    if (MODE & 2) sa = a[0];
    if (MODE & 1) sb = b[0];
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const uint64_t w = tile + (uint64_t)k * EW_BLOCK;
        if (w < items && (w << 2) + 4 <= n) {
            if (!(MODE & 2)) va[k] = ld4(a + (w << 2));
            if (!(MODE & 1)) vb[k] = ld4(b + (w << 2));
        }
    }
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const uint64_t w = tile + (uint64_t)k * EW_BLOCK;
        if (w >= items) continue;
        const uint64_t i = w << 2;
        if (i + 4 <= n) {
            const float4 x = (MODE & 2) ? make_float4(sa, sa, sa, sa) : va[k];
            const float4 y = (MODE & 1) ? make_float4(sb, sb, sb, sb) : vb[k];
            st4(out + i, make_float4(Fn::f(x.x, y.x), Fn::f(x.y, y.y), Fn::f(x.z, y.z), Fn::f(x.w, y.w)));
        } else {
            for (uint64_t j = i; j < n; ++j) out[j] = Fn::f((MODE & 2) ? sa : a[j], (MODE & 1) ? sb : b[j]);
        }
    }
}

// Elements at positions >= n_poly are the ones the reference computes with libm (see LibmSplit);
// n_poly is a multiple of 8, so a 4-element work item never straddles it.
template <class Fn>
__global__ void __launch_bounds__(EW_BLOCK) unary_flat_kernel(const float *__restrict__ x, float *__restrict__ out, uint64_t n,
                                                              uint64_t n_poly) {
    ordered_start();
    const uint64_t items = (n + 3) >> 2;
    const uint64_t tile = (uint64_t)blockIdx.x * (EW_BLOCK * EW_UNROLL) + threadIdx.x;
    float4 v[EW_UNROLL];
    // Every CTA but the last lies wholly below n_poly: no bounds to check and no element for libm, so
    // its sixteen evaluations per thread are one straight-line block that the compiler interleaves.
    // With the per-element choice between polynomial and (out-of-line) libm inside the loop it cannot,
    // and exp, log and tanh, which are bound by instruction issue, lose 5-20%.
    if (((uint64_t)blockIdx.x + 1) * (EW_BLOCK * EW_UNROLL * 4) <= n_poly) {
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k) v[k] = ld4(x + ((tile + (uint64_t)k * EW_BLOCK) << 2));
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            st4(out + ((tile + (uint64_t)k * EW_BLOCK) << 2), make_float4(Fn::f(v[k].x), Fn::f(v[k].y), Fn::f(v[k].z), Fn::f(v[k].w)));
        return;
    }
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const uint64_t w = tile + (uint64_t)k * EW_BLOCK;
        if (w < items && (w << 2) + 4 <= n) v[k] = ld4(x + (w << 2));
    }
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const uint64_t w = tile + (uint64_t)k * EW_BLOCK;
        if (w >= items) continue;
        const uint64_t i = w << 2;
        const bool lm = i >= n_poly;
        if (i + 4 <= n) {
            st4(out + i, make_float4(apply_unary<Fn>(v[k].x, lm), apply_unary<Fn>(v[k].y, lm), apply_unary<Fn>(v[k].z, lm),
                                     apply_unary<Fn>(v[k].w, lm)));
        } else {
            for (uint64_t j = i; j < n; ++j) out[j] = apply_unary<Fn>(x[j], lm);
        }
    }
}

// ---- rows kernel: innermost strides in {0,1}, any outer strides --------------------------------------
// Work item w = (row, c): row over the outer dims, c over the inner dim in steps of VEC elements.
// NOPS operands (1 = unary, 2 = binary). I = uint32_t while the item count fits, else uint64_t.
template <typename I, int NOPS> struct RowsPlan {
    I items;                       // rows * cols
    I inner;                       // elements in the innermost dim
    Divider<I> cols;               // items per row = ceil(inner / VEC)
    int n_outer;                   // outer dims (>= 1), listed innermost-outer first
    Divider<I> outer[MAX_DIMS];    // their sizes (the last listed, outermost, is never divided by)
    uint64_t ostride[NOPS][MAX_DIMS];
    uint32_t istride[NOPS];        // 0 or 1
};

template <typename I, int NOPS>
__device__ __forceinline__ void rows_offsets(const RowsPlan<I, NOPS> &p, I row, uint64_t (&off)[NOPS]) {
#pragma unroll
    for (int o = 0; o < NOPS; ++o) off[o] = 0;
    for (int d = 0; d < p.n_outer - 1; ++d) {
        I q, r;
        p.outer[d].divmod(row, q, r);
        row = q;
#pragma unroll
        for (int o = 0; o < NOPS; ++o) off[o] += (uint64_t)r * p.ostride[o][d];
    }
#pragma unroll
    for (int o = 0; o < NOPS; ++o) off[o] += (uint64_t)row * p.ostride[o][p.n_outer - 1];
}

template <typename I, int VEC> struct Pack;
template <typename I> struct Pack<I, 4> {
    float4 v;
    __device__ __forceinline__ void load(const float *base, uint32_t istride, I c) {
        if (istride) v = ld4(base + (uint64_t)c * 4);
        else { const float s = __ldg(base); v = make_float4(s, s, s, s); }
    }
};
template <typename I> struct Pack<I, 1> {
    float v;
    __device__ __forceinline__ void load(const float *base, uint32_t istride, I c) { v = istride ? ld1(base + c) : __ldg(base); }
};

// WARPROW: the row length in items is a multiple of 128, so the 128 consecutive items a warp takes
// (lane + 32 k, k = 0..3) lie in ONE row: the row is decomposed once per thread instead of once per
// item, and an operand that is broadcast along the row (inner stride 0: a column vector) is loaded
// once. Otherwise item k of a thread is 256 items further on and may sit in another row each time.
template <class Fn, typename I, int VEC, bool WARPROW>
__global__ void __launch_bounds__(EW_BLOCK) binary_rows_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                                               float *__restrict__ out,
                                                               const __grid_constant__ RowsPlan<I, 2> p) {
    ordered_start();
    Pack<I, VEC> va[EW_UNROLL], vb[EW_UNROLL];
    uint64_t oo[EW_UNROLL];
    if constexpr (WARPROW) {
        const I first = (I)blockIdx.x * (I)(EW_BLOCK * EW_UNROLL) + (I)((threadIdx.x >> 5) * (32 * EW_UNROLL) + (threadIdx.x & 31));
        const bool live = first < p.items;  // items is a multiple of 128 here: a warp is live or not as a whole
        if (live) {
            I row, c;
            p.cols.divmod(first, row, c);
            uint64_t off[2];
            rows_offsets<I, 2>(p, row, off);
            const uint64_t o0 = (uint64_t)row * p.inner + (uint64_t)c * VEC;
            Pack<I, VEC> sa, sb;
            if (!p.istride[0]) sa.load(a + off[0], 0, c);
            if (!p.istride[1]) sb.load(b + off[1], 0, c);
#pragma unroll
            for (int k = 0; k < EW_UNROLL; ++k) {
                if (p.istride[0]) va[k].load(a + off[0], 1, c + (I)(32 * k)); else va[k] = sa;
                if (p.istride[1]) vb[k].load(b + off[1], 1, c + (I)(32 * k)); else vb[k] = sb;
                oo[k] = o0 + (uint64_t)(32 * k) * VEC;
            }
#pragma unroll
            for (int k = 0; k < EW_UNROLL; ++k) {
                if constexpr (VEC == 4) {
                    const float4 x = va[k].v, y = vb[k].v;
                    st4(out + oo[k], make_float4(Fn::f(x.x, y.x), Fn::f(x.y, y.y), Fn::f(x.z, y.z), Fn::f(x.w, y.w)));
                } else {
                    st1(out + oo[k], Fn::f(va[k].v, vb[k].v));
                }
            }
        }
        return;
    }
    const I tile = (I)blockIdx.x * (I)(EW_BLOCK * EW_UNROLL) + threadIdx.x;
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const I w = tile + (I)(k * EW_BLOCK);
        if (w < p.items) {
            I row, c;
            p.cols.divmod(w, row, c);
            uint64_t off[2];
            rows_offsets<I, 2>(p, row, off);
            va[k].load(a + off[0], p.istride[0], c);
            vb[k].load(b + off[1], p.istride[1], c);
            oo[k] = (uint64_t)row * p.inner + (uint64_t)c * VEC;
        }
    }
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const I w = tile + (I)(k * EW_BLOCK);
        if (w < p.items) {
            if constexpr (VEC == 4) {
                const float4 x = va[k].v, y = vb[k].v;
                st4(out + oo[k], make_float4(Fn::f(x.x, y.x), Fn::f(x.y, y.y), Fn::f(x.z, y.z), Fn::f(x.w, y.w)));
            } else {
                st1(out + oo[k], Fn::f(va[k].v, vb[k].v));
            }
        }
    }
}

template <class Fn, typename I, int VEC>
__global__ void __launch_bounds__(EW_BLOCK) unary_rows_kernel(const float *__restrict__ x, float *__restrict__ out,
                                                              const __grid_constant__ RowsPlan<I, 1> p, const LibmSplit split) {
    ordered_start();
    const I tile = (I)blockIdx.x * (I)(EW_BLOCK * EW_UNROLL) + threadIdx.x;
    Pack<I, VEC> v[EW_UNROLL];
    uint64_t oo[EW_UNROLL];
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const I w = tile + (I)(k * EW_BLOCK);
        if (w < p.items) {
            I row, c;
            p.cols.divmod(w, row, c);
            uint64_t off[1];
            rows_offsets<I, 1>(p, row, off);
            v[k].load(x + off[0], p.istride[0], c);
            oo[k] = (uint64_t)row * p.inner + (uint64_t)c * VEC;
        }
    }
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const I w = tile + (I)(k * EW_BLOCK);
        if (w < p.items) {
            // Row starts, chunk starts and split points are all multiples of 4 when VEC is 4, so one
            // test covers the whole work item.
            const bool lm = Fn::SPLIT && split.uses_libm(oo[k]);
            if constexpr (VEC == 4) {
                const float4 t = v[k].v;
                st4(out + oo[k], make_float4(apply_unary<Fn>(t.x, lm), apply_unary<Fn>(t.y, lm), apply_unary<Fn>(t.z, lm), apply_unary<Fn>(t.w, lm)));
            } else {
                st1(out + oo[k], apply_unary<Fn>(v[k].v, lm));
            }
        }
    }
}

// ---- tile kernel: an operand whose unit stride lies in a non-innermost dim --------------------------
// The output's innermost dim is I (size ni); dim F (size nf) is where a "transposed" operand has
// stride 1. A CTA handles a 32(F) x 32(I) tile of one batch entry (all other dims). Transposed
// operands are read coalesced along F into padded shared memory and consumed along I; "direct"
// operands (inner stride 0 or 1) are read in output orientation. Output writes are coalesced along I.
template <int NOPS> struct TilePlan {
    uint32_t nf, ni;               // sizes of dims F and I
    uint32_t tiles_f, tiles_i;
    uint64_t out_fstride;          // output stride of dim F (dim I has stride 1)
    int n_batch;                   // remaining dims, listed innermost first
    Divider<uint64_t> batch[MAX_DIMS];
    uint64_t out_bstride[MAX_DIMS];
    uint64_t bstride[NOPS][MAX_DIMS];
    uint64_t fstride[NOPS], istride[NOPS];
    uint32_t transposed[NOPS];     // 1: via shared memory (fstride == 1)
};

constexpr int TILE = 32;
constexpr int TILE_ROWS = 8;  // CTA is 32 x 8 threads

template <class Fn, int NOPS>
__global__ void __launch_bounds__(TILE *TILE_ROWS) tile_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                                               float *__restrict__ out,
                                                               const __grid_constant__ TilePlan<NOPS> p, const LibmSplit split) {
    ordered_start();
    __shared__ float sm[NOPS][TILE][TILE + 1];
    const float *src[2] = {a, b};
    // blockIdx.x enumerates (batch, tile_f, tile_i) with tile_i fastest.
    uint64_t t = blockIdx.x;
    const uint32_t ti = (uint32_t)(t % p.tiles_i);
    t /= p.tiles_i;
    const uint32_t tf = (uint32_t)(t % p.tiles_f);
    uint64_t bidx = t / p.tiles_f;
    uint64_t boff[NOPS], oboff = 0;
#pragma unroll
    for (int o = 0; o < NOPS; ++o) boff[o] = 0;
    for (int d = 0; d < p.n_batch; ++d) {
        uint64_t q, r;
        p.batch[d].divmod(bidx, q, r);
        bidx = q;
        oboff += r * p.out_bstride[d];
#pragma unroll
        for (int o = 0; o < NOPS; ++o) boff[o] += r * p.bstride[o][d];
    }
    const uint32_t f0 = tf * TILE, i0 = ti * TILE;
    const int tx = threadIdx.x, ty = threadIdx.y;
    // Stage transposed operands: thread (tx, ty) reads element (f = f0 + tx, i = i0 + ty + 8k).
#pragma unroll
    for (int o = 0; o < NOPS; ++o) {
        if (p.transposed[o]) {
#pragma unroll
            for (int k = 0; k < TILE; k += TILE_ROWS) {
                const uint32_t f = f0 + tx, i = i0 + ty + k;
                if (f < p.nf && i < p.ni) sm[o][ty + k][tx] = src[o][boff[o] + (uint64_t)f * p.fstride[o] + (uint64_t)i * p.istride[o]];
            }
        }
    }
    __syncthreads();
    // Consume: thread (tx, ty) produces element (f = f0 + ty + 8k, i = i0 + tx).
#pragma unroll
    for (int k = 0; k < TILE; k += TILE_ROWS) {
        const uint32_t f = f0 + ty + k, i = i0 + tx;
        if (f < p.nf && i < p.ni) {
            float v[NOPS];
#pragma unroll
            for (int o = 0; o < NOPS; ++o)
                v[o] = p.transposed[o] ? sm[o][tx][ty + k] : src[o][boff[o] + (uint64_t)f * p.fstride[o] + (uint64_t)i * p.istride[o]];
            const uint64_t pos = oboff + (uint64_t)f * p.out_fstride + i;
            float r;
            if constexpr (NOPS == 2) r = Fn::f(v[0], v[1]);
            else r = apply_unary<Fn>(v[0], Fn::SPLIT && split.uses_libm(pos));
            out[pos] = r;
        }
    }
}

// ---- wide tile kernel: the same job with 64x64 tiles and 128-bit accesses ----------------------------
// Used when sizes and strides allow float4 on every side (F and I sizes multiples of 4, 16-byte
// aligned rows). 256 threads; a thread moves four float4 per operand and issues all of its global
// loads before anything else. Transposed operands: float4 along F, scattered into padded shared
// memory, read back along I. Direct operands: float4 along I (mode 1) or four scalars (mode 2,
// broadcast or unaligned rows). Output: float4 along I. blockIdx.x walks the tiles of one batch
// entry (I fastest), blockIdx.y the batch entries, whose index is split with multiply-high division.
constexpr int WT = 64;
template <int NOPS> struct WideTilePlan {
    uint32_t nf, ni, tiles_i, batches;
    uint64_t out_fstride;
    int n_batch;                   // remaining dims, innermost first
    Divider<uint32_t> batch[MAX_DIMS];
    uint64_t out_bstride[MAX_DIMS];
    uint64_t bstride[NOPS][MAX_DIMS];
    uint64_t fstride[NOPS], istride[NOPS];
    uint32_t mode[NOPS];           // 0: transposed through shared memory, 1: direct float4, 2: direct scalars
};

template <class Fn, int NOPS>
__global__ void __launch_bounds__(256) wide_tile_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out,
                                                        const __grid_constant__ WideTilePlan<NOPS> p, const LibmSplit split) {
    ordered_start();
    __shared__ float sm[NOPS][WT][WT + 1];
    const float *src[2] = {a, b};
    const uint32_t ti = blockIdx.x % p.tiles_i, tf = blockIdx.x / p.tiles_i;
    const uint32_t f0 = tf * WT, i0 = ti * WT;
    const uint32_t q_hi = threadIdx.x >> 4, q_lo = (threadIdx.x & 15) * 4;  // (row 0..15, float4 column 0..60) of a 16-row slab
    for (uint32_t bidx = blockIdx.y; bidx < p.batches; bidx += gridDim.y) {
        uint64_t boff[NOPS], oboff = 0;
#pragma unroll
        for (int o = 0; o < NOPS; ++o) boff[o] = 0;
        uint32_t rem = bidx;
        for (int d = 0; d < p.n_batch; ++d) {
            uint32_t q, r;
            p.batch[d].divmod(rem, q, r);
            rem = q;
            oboff += (uint64_t)r * p.out_bstride[d];
#pragma unroll
            for (int o = 0; o < NOPS; ++o) boff[o] += (uint64_t)r * p.bstride[o][d];
        }
        float4 v[NOPS][4];
        // Phase 1: every global load of this thread.
#pragma unroll
        for (int o = 0; o < NOPS; ++o) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t row = q_hi + 16 * k;  // 0..63
                if (p.mode[o] == 0) {
                    const uint32_t i = i0 + row, f = f0 + q_lo;  // 64 floats along F per I-row
                    if (i < p.ni && f < p.nf) v[o][k] = ld4(src[o] + boff[o] + (uint64_t)i * p.istride[o] + f);
                } else {
                    const uint32_t f = f0 + row, i = i0 + q_lo;  // 64 floats along I per F-row
                    if (f < p.nf && i < p.ni) {
                        const float *q = src[o] + boff[o] + (uint64_t)f * p.fstride[o] + (uint64_t)i * p.istride[o];
                        if (p.mode[o] == 1) v[o][k] = ld4(q);
                        else v[o][k] = make_float4(q[0], q[p.istride[o]], q[2 * p.istride[o]], q[3 * p.istride[o]]);
                    }
                }
            }
        }
        // Phase 2: transposed operands go through shared memory.
#pragma unroll
        for (int o = 0; o < NOPS; ++o) {
            if (p.mode[o] == 0) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t il = q_hi + 16 * k;
                    sm[o][q_lo + 0][il] = v[o][k].x;
                    sm[o][q_lo + 1][il] = v[o][k].y;
                    sm[o][q_lo + 2][il] = v[o][k].z;
                    sm[o][q_lo + 3][il] = v[o][k].w;
                }
            }
        }
        __syncthreads();
        // Phase 3: compute and store along I.
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t fl = q_hi + 16 * k, f = f0 + fl, i = i0 + q_lo;
            if (f < p.nf && i < p.ni) {
                float4 x[NOPS];
#pragma unroll
                for (int o = 0; o < NOPS; ++o)
                    x[o] = p.mode[o] == 0 ? make_float4(sm[o][fl][q_lo], sm[o][fl][q_lo + 1], sm[o][fl][q_lo + 2], sm[o][fl][q_lo + 3]) : v[o][k];
                const uint64_t pos = oboff + (uint64_t)f * p.out_fstride + i;
                float4 r;
                if constexpr (NOPS == 2) {
                    r = make_float4(Fn::f(x[0].x, x[1].x), Fn::f(x[0].y, x[1].y), Fn::f(x[0].z, x[1].z), Fn::f(x[0].w, x[1].w));
                } else {
                    r = make_float4(apply_unary<Fn>(x[0].x, Fn::SPLIT && split.uses_libm(pos)), apply_unary<Fn>(x[0].y, Fn::SPLIT && split.uses_libm(pos + 1)),
                                    apply_unary<Fn>(x[0].z, Fn::SPLIT && split.uses_libm(pos + 2)), apply_unary<Fn>(x[0].w, Fn::SPLIT && split.uses_libm(pos + 3)));
                }
                st4(out + pos, r);
            }
        }
        __syncthreads();
    }
}

// ---- generic gather kernel: any strides, one element per thread --------------------------------------
template <int NOPS> struct GatherPlan {
    uint64_t n;
    int nd;                        // dims listed innermost first
    Divider<uint64_t> size[MAX_DIMS];
    uint64_t stride[NOPS][MAX_DIMS];
};

template <class Fn, int NOPS>
__global__ void __launch_bounds__(EW_BLOCK) gather_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                                          float *__restrict__ out, const __grid_constant__ GatherPlan<NOPS> p,
                                                          const LibmSplit split) {
    ordered_start();
    const uint64_t i = (uint64_t)blockIdx.x * EW_BLOCK + threadIdx.x;
    if (i >= p.n) return;
    uint64_t rem = i, off[NOPS];
#pragma unroll
    for (int o = 0; o < NOPS; ++o) off[o] = 0;
    for (int d = 0; d < p.nd; ++d) {
        uint64_t q, r;
        p.size[d].divmod(rem, q, r);
        rem = q;
#pragma unroll
        for (int o = 0; o < NOPS; ++o) off[o] += r * p.stride[o][d];
    }
    if constexpr (NOPS == 2) out[i] = Fn::f(a[off[0]], b[off[1]]);
    else out[i] = apply_unary<Fn>(a[off[0]], Fn::SPLIT && split.uses_libm(i));
}

// The last (n mod 8) elements of a binary op that ends in a libm-split function: one thread each.
template <class Fn>
__global__ void __launch_bounds__(32) binary_tail_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out,
                                                         const __grid_constant__ GatherPlan<2> p, uint64_t first) {
    ordered_start();
    const uint64_t i = first + threadIdx.x;
    if (i >= p.n) return;
    uint64_t rem = i, off[2] = {0, 0};
    for (int d = 0; d < p.nd; ++d) {
        uint64_t q, r;
        p.size[d].divmod(rem, q, r);
        rem = q;
        off[0] += r * p.stride[0][d];
        off[1] += r * p.stride[1][d];
    }
    if constexpr (Fn::TAIL) out[i] = Fn::libm(a[off[0]], b[off[1]]);
}

// ---- AXPY, FILL, RAND_NORMAL --------------------------------------------------------------------------
// out = a + alpha*b. The reference fuses the multiply-add (one rounding) for every element except
// the last n mod 8, which it computes with two roundings (plugins/cpu/src/ew.rs:316-329; its chunks
// of 65536 are multiples of 8, so only the global tail is unfused). `out` may alias `a`.
__global__ void __launch_bounds__(EW_BLOCK) axpy_kernel(const float *a, const float *b, float *out, float alpha, uint64_t n) {
    ordered_start();
    const uint64_t n_fused = n - (n & 7);
    const uint64_t items = (n + 3) >> 2;
    const uint64_t tile = (uint64_t)blockIdx.x * (EW_BLOCK * EW_UNROLL) + threadIdx.x;
    float4 va[EW_UNROLL], vb[EW_UNROLL];
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const uint64_t w = tile + (uint64_t)k * EW_BLOCK;
        if (w < items && (w << 2) + 4 <= n) {
            va[k] = ld4(a + (w << 2));
            vb[k] = ld4(b + (w << 2));
        }
    }
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const uint64_t w = tile + (uint64_t)k * EW_BLOCK;
        if (w >= items) continue;
        const uint64_t i = w << 2;
        if (i + 4 <= n) {
            const float4 x = va[k], y = vb[k];
            float4 r;
            if (i < n_fused) {
                r = make_float4(__fmaf_rn(alpha, y.x, x.x), __fmaf_rn(alpha, y.y, x.y), __fmaf_rn(alpha, y.z, x.z), __fmaf_rn(alpha, y.w, x.w));
            } else {
                r = make_float4(__fadd_rn(x.x, __fmul_rn(alpha, y.x)), __fadd_rn(x.y, __fmul_rn(alpha, y.y)),
                                __fadd_rn(x.z, __fmul_rn(alpha, y.z)), __fadd_rn(x.w, __fmul_rn(alpha, y.w)));
            }
            st4(out + i, r);
        } else {
            for (uint64_t j = i; j < n; ++j)
                out[j] = j < n_fused ? __fmaf_rn(alpha, b[j], a[j]) : __fadd_rn(a[j], __fmul_rn(alpha, b[j]));
        }
    }
}

__global__ void __launch_bounds__(EW_BLOCK) fill_kernel(float *__restrict__ out, uint64_t n, float v) {
    ordered_start();
    const uint64_t items = (n + 3) >> 2;
    const uint64_t tile = (uint64_t)blockIdx.x * (EW_BLOCK * EW_UNROLL) + threadIdx.x;
#pragma unroll
    for (int k = 0; k < EW_UNROLL; ++k) {
        const uint64_t w = tile + (uint64_t)k * EW_BLOCK;
        if (w >= items) continue;
        const uint64_t i = w << 2;
        if (i + 4 <= n) st4(out + i, make_float4(v, v, v, v));
        else for (uint64_t j = i; j < n; ++j) out[j] = v;
    }
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// The counter-based Box-Muller recipe of crates/plugin-abi/src/lib.rs:99-107. The integer hash is
// exact; ln/cos come from CUDA's math library and may differ from the CPU's libm in the last ulp.
__device__ __forceinline__ float rand_normal(uint64_t seed, uint64_t i) {
    const uint64_t h = splitmix64(seed ^ (i * 0x9E3779B97F4A7C15ull));
    const float u1 = __fdiv_rn((float)((h >> 40) + 1), 16777216.0f);
    const float u2 = __fdiv_rn((float)(h & 0xFFFFFFull), 16777216.0f);
    const float rad = sqrtf(__fmul_rn(-2.0f, logf(u1)));
    const float ang = __fmul_rn(__fmul_rn(2.0f, 3.14159265358979323846264338327950288f), u2);
    return __fmul_rn(rad, cosf(ang));
}

__global__ void __launch_bounds__(EW_BLOCK) randn_kernel(float *__restrict__ out, uint64_t n, uint64_t seed) {
    ordered_start();
    const uint64_t items = (n + 3) >> 2;
    const uint64_t w = (uint64_t)blockIdx.x * EW_BLOCK + threadIdx.x;
    if (w >= items) return;
    const uint64_t i = w << 2;
    if (i + 4 <= n) {
        st4(out + i, make_float4(rand_normal(seed, i), rand_normal(seed, i + 1), rand_normal(seed, i + 2), rand_normal(seed, i + 3)));
    } else {
        for (uint64_t j = i; j < n; ++j) out[j] = rand_normal(seed, j);
    }
}

// RAND_UNIFORM (appended op): lo + scale * u with u = (hash >> 40) / 2^24, counters first, first + 1, ...
__device__ __forceinline__ float rand_uniform(uint64_t seed, uint64_t i, float lo, float scale) {
    const uint64_t h = splitmix64(seed ^ (i * 0x9E3779B97F4A7C15ull));
    const float u = __fdiv_rn((float)(h >> 40), 16777216.0f);
    return __fadd_rn(lo, __fmul_rn(scale, u));
}

__global__ void __launch_bounds__(EW_BLOCK) rand_uniform_kernel(float *__restrict__ out, uint64_t n, uint64_t seed, float lo, float scale,
                                                                uint64_t first) {
    ordered_start();
    const uint64_t items = (n + 3) >> 2;
    const uint64_t w = (uint64_t)blockIdx.x * EW_BLOCK + threadIdx.x;
    if (w >= items) return;
    const uint64_t i = w << 2, c = first + i;
    if (i + 4 <= n) {
        st4(out + i, make_float4(rand_uniform(seed, c, lo, scale), rand_uniform(seed, c + 1, lo, scale), rand_uniform(seed, c + 2, lo, scale),
                                 rand_uniform(seed, c + 3, lo, scale)));
    } else {
        for (uint64_t j = i; j < n; ++j) out[j] = rand_uniform(seed, first + j, lo, scale);
    }
}

// ---- required MATMUL: correctness only, outside the measured path --------------------------------------
// 32x32 shared-memory tiles, k in order with one fused multiply-add per step; any operand strides.
__global__ void __launch_bounds__(TILE *TILE) matmul_kernel(const float *__restrict__ a, uint64_t ars, uint64_t acs,
                                                             const float *__restrict__ b, uint64_t brs, uint64_t bcs,
                                                             float *__restrict__ c, uint64_t m, uint64_t n, uint64_t k, uint32_t tiles_n) {
    ordered_start();
    __shared__ float sa[TILE][TILE + 1], sb[TILE][TILE + 1];
    // Tiles are numbered along one grid axis (row-major), which has room for 2^31 - 1 of them.
    const uint32_t tile_row = blockIdx.x / tiles_n, tile_col = blockIdx.x - tile_row * tiles_n;
    const uint64_t row = (uint64_t)tile_row * TILE + threadIdx.y, col = (uint64_t)tile_col * TILE + threadIdx.x;
    float acc = 0.0f;
    for (uint64_t k0 = 0; k0 < k; k0 += TILE) {
        const uint64_t ka = k0 + threadIdx.x, kb = k0 + threadIdx.y;
        sa[threadIdx.y][threadIdx.x] = (row < m && ka < k) ? a[row * ars + ka * acs] : 0.0f;
        sb[threadIdx.y][threadIdx.x] = (kb < k && col < n) ? b[kb * brs + col * bcs] : 0.0f;
        __syncthreads();
#pragma unroll
        for (int p = 0; p < TILE; ++p) acc = __fmaf_rn(sa[threadIdx.y][p], sb[p][threadIdx.x], acc);
        __syncthreads();
    }
    if (row < m && col < n) c[row * n + col] = acc;
}

// ---- host side: choose a kernel for a coalesced problem --------------------------------------------

template <int NOPS> bool inner_is_unit_or_zero(const EwProblem &p) {
    for (int o = 0; o < NOPS; ++o)
        if (p.dim[p.nd - 1].stride[o] > 1) return false;
    return true;
}

template <typename I, int NOPS> RowsPlan<I, NOPS> make_rows_plan(const EwProblem &p, int vec) {
    RowsPlan<I, NOPS> r{};
    const EwDim &in = p.dim[p.nd - 1];
    const uint64_t cols = (in.size + vec - 1) / vec;
    r.inner = (I)in.size;
    r.cols = Divider<I>(cols);
    r.n_outer = p.nd - 1;
    uint64_t rows = 1;
    for (int d = 0; d < r.n_outer; ++d) {
        const EwDim &od = p.dim[p.nd - 2 - d];  // innermost-outer first
        r.outer[d] = Divider<I>(od.size);
        for (int o = 0; o < NOPS; ++o) r.ostride[o][d] = od.stride[o];
        rows *= od.size;
    }
    for (int o = 0; o < NOPS; ++o) r.istride[o] = (uint32_t)in.stride[o];
    r.items = (I)(rows * cols);
    return r;
}

// The rows kernels index with 32 bits while both the work-item count (plus one grid's worth of
// overshoot) and the inner dim's element count fit: with 4 elements per item the inner dim can reach
// 2^32 elements while the items still number fewer than 2^32.
bool rows_plan_fits_32bit(uint64_t items, uint64_t inner) {
    return items + (uint64_t)EW_BLOCK * EW_UNROLL < (1ull << 32) && inner < (1ull << 32);
}

// float4 access needs: inner size a multiple of 4 and, for operands read with inner stride 1, every
// outer stride a multiple of 4 (row starts stay 16-byte aligned).
template <int NOPS> int rows_vec_width(const EwProblem &p) {
    const EwDim &in = p.dim[p.nd - 1];
    if (in.size % 4) return 1;
    for (int o = 0; o < NOPS; ++o) {
        if (in.stride[o] != 1) continue;
        for (int d = 0; d < p.nd - 1; ++d)
            if (p.dim[d].stride[o] % 4) return 1;
    }
    return 4;
}

// Finds the dim (other than the innermost) in which operand o has stride 1, or -1.
int unit_stride_dim(const EwProblem &p, int o) {
    for (int d = 0; d < p.nd - 1; ++d)
        if (p.dim[d].stride[o] == 1 && p.dim[d].size > 1) return d;
    return -1;
}

// Tries to express the problem for the tile kernel. Every operand must be either "direct" (inner
// stride 0 or 1) or "transposed" with its unit stride in one common dim F.
template <int NOPS> bool make_tile_plan(const EwProblem &p, TilePlan<NOPS> &t, uint64_t &ctas) {
    if (p.nd < 2) return false;
    int F = -1;
    for (int o = 0; o < NOPS; ++o) {
        const uint64_t is = p.dim[p.nd - 1].stride[o];
        if (is <= 1) { t.transposed[o] = 0; continue; }
        const int f = unit_stride_dim(p, o);
        if (f < 0 || (F >= 0 && f != F)) return false;
        F = f;
        t.transposed[o] = 1;
    }
    if (F < 0) return false;
    const EwDim &df = p.dim[F], &di = p.dim[p.nd - 1];
    if (df.size > UINT32_MAX || di.size > UINT32_MAX) return false;
    t.nf = (uint32_t)df.size;
    t.ni = (uint32_t)di.size;
    t.tiles_f = (t.nf + TILE - 1) / TILE;
    t.tiles_i = (t.ni + TILE - 1) / TILE;
    // Output strides: contiguous over the coalesced dims.
    uint64_t ostride[MAX_DIMS], acc = 1;
    for (int d = p.nd - 1; d >= 0; --d) { ostride[d] = acc; acc *= p.dim[d].size; }
    t.out_fstride = ostride[F];
    for (int o = 0; o < NOPS; ++o) { t.fstride[o] = df.stride[o]; t.istride[o] = di.stride[o]; }
    t.n_batch = 0;
    uint64_t batches = 1;
    for (int d = p.nd - 2; d >= 0; --d) {
        if (d == F) continue;
        const int j = t.n_batch++;
        t.batch[j] = Divider<uint64_t>(p.dim[d].size);
        t.out_bstride[j] = ostride[d];
        for (int o = 0; o < NOPS; ++o) t.bstride[o][j] = p.dim[d].stride[o];
        batches *= p.dim[d].size;
    }
    ctas = batches * t.tiles_f * t.tiles_i;
    return ctas <= 0x7fffffffull;
}

// The wide tile kernel's plan, or false when sizes / strides do not allow 128-bit accesses throughout.
template <int NOPS> bool make_wide_tile_plan(const EwProblem &p, WideTilePlan<NOPS> &t, dim3 &grid) {
    if (p.nd < 2) return false;
    int F = -1;
    for (int o = 0; o < NOPS; ++o) {
        if (p.dim[p.nd - 1].stride[o] <= 1) continue;
        const int f = unit_stride_dim(p, o);
        if (f < 0 || (F >= 0 && f != F)) return false;
        F = f;
    }
    if (F < 0) return false;
    const EwDim &df = p.dim[F], &di = p.dim[p.nd - 1];
    if (df.size % 4 || di.size % 4 || df.size > UINT32_MAX || di.size > UINT32_MAX) return false;
    t.nf = (uint32_t)df.size;
    t.ni = (uint32_t)di.size;
    const uint64_t tiles_f = (t.nf + WT - 1) / WT;
    t.tiles_i = (t.ni + WT - 1) / WT;
    if (tiles_f * t.tiles_i > 0x7fffffffull) return false;
    uint64_t ostride[MAX_DIMS], acc = 1;
    for (int d = p.nd - 1; d >= 0; --d) { ostride[d] = acc; acc *= p.dim[d].size; }
    t.out_fstride = ostride[F];
    t.n_batch = 0;
    uint64_t batches = 1;
    for (int d = p.nd - 2; d >= 0; --d) {
        if (d == F) continue;
        const int j = t.n_batch++;
        t.batch[j] = Divider<uint32_t>(p.dim[d].size);
        t.out_bstride[j] = ostride[d];
        for (int o = 0; o < NOPS; ++o) t.bstride[o][j] = p.dim[d].stride[o];
        batches *= p.dim[d].size;
    }
    if (batches > UINT32_MAX) return false;
    t.batches = (uint32_t)batches;
    for (int o = 0; o < NOPS; ++o) {
        t.fstride[o] = df.stride[o];
        t.istride[o] = di.stride[o];
        bool aligned = true;  // every batch offset keeps 16-byte alignment
        for (int j = 0; j < t.n_batch; ++j) aligned = aligned && t.bstride[o][j] % 4 == 0;
        if (di.stride[o] > 1) {  // transposed: float4 along F at offset i*istride + f
            if (!aligned || di.stride[o] % 4) return false;
            t.mode[o] = 0;
        } else {
            t.mode[o] = (di.stride[o] == 1 && aligned && df.stride[o] % 4 == 0) ? 1 : 2;
        }
    }
    grid = dim3((unsigned)(tiles_f * t.tiles_i), (unsigned)(batches < 65535 ? batches : 65535));
    return true;
}

template <int NOPS> GatherPlan<NOPS> make_gather_plan(const EwProblem &p) {
    GatherPlan<NOPS> g{};
    g.n = p.n;
    g.nd = p.nd;
    for (int d = 0; d < p.nd; ++d) {
        const EwDim &src = p.dim[p.nd - 1 - d];
        g.size[d] = Divider<uint64_t>(src.size);
        for (int o = 0; o < NOPS; ++o) g.stride[o][d] = src.stride[o];
    }
    return g;
}

template <class Fn> cudaError_t run_binary_body(const float *a, const float *b, float *out, const EwProblem &p, cudaStream_t s) {
    // Flat: one dim (or none) and inner strides in {0,1}.
    if (p.nd <= 1) {
        const uint64_t sa = p.nd ? p.dim[0].stride[0] : 0, sb = p.nd ? p.dim[0].stride[1] : 0;
        if (sa <= 1 && sb <= 1) {
            const unsigned grid = tiles_for((p.n + 3) / 4, EW_BLOCK * EW_UNROLL);
            const int mode = (sa ? 0 : 2) | (sb ? 0 : 1);
            switch (mode) {
                case 0: B200_LAUNCH_ORDERED((binary_flat_kernel<Fn, 0>), grid, EW_BLOCK, 0, s, a, b, out, p.n); break;
                case 1: B200_LAUNCH_ORDERED((binary_flat_kernel<Fn, 1>), grid, EW_BLOCK, 0, s, a, b, out, p.n); break;
                case 2: B200_LAUNCH_ORDERED((binary_flat_kernel<Fn, 2>), grid, EW_BLOCK, 0, s, a, b, out, p.n); break;
                default: B200_LAUNCH_ORDERED((binary_flat_kernel<Fn, 3>), grid, EW_BLOCK, 0, s, a, b, out, p.n); break;
            }
            return cudaGetLastError();
        }
    } else if (inner_is_unit_or_zero<2>(p)) {
        const int vec = rows_vec_width<2>(p);
        uint64_t rows = p.n / p.dim[p.nd - 1].size;
        const uint64_t items = rows * ((p.dim[p.nd - 1].size + vec - 1) / vec);
        const unsigned grid = tiles_for(items, EW_BLOCK * EW_UNROLL);
        const bool warprow = vec == 4 && (p.dim[p.nd - 1].size / 4) % (32 * EW_UNROLL) == 0;  // a warp's 128 items share a row
        if (rows_plan_fits_32bit(items, p.dim[p.nd - 1].size)) {
            auto plan = make_rows_plan<uint32_t, 2>(p, vec);
            if (warprow) B200_LAUNCH_ORDERED((binary_rows_kernel<Fn, uint32_t, 4, true>), grid, EW_BLOCK, 0, s, a, b, out, plan);
            else if (vec == 4) B200_LAUNCH_ORDERED((binary_rows_kernel<Fn, uint32_t, 4, false>), grid, EW_BLOCK, 0, s, a, b, out, plan);
            else B200_LAUNCH_ORDERED((binary_rows_kernel<Fn, uint32_t, 1, false>), grid, EW_BLOCK, 0, s, a, b, out, plan);
        } else {
            auto plan = make_rows_plan<uint64_t, 2>(p, vec);
            if (warprow) B200_LAUNCH_ORDERED((binary_rows_kernel<Fn, uint64_t, 4, true>), grid, EW_BLOCK, 0, s, a, b, out, plan);
            else if (vec == 4) B200_LAUNCH_ORDERED((binary_rows_kernel<Fn, uint64_t, 4, false>), grid, EW_BLOCK, 0, s, a, b, out, plan);
            else B200_LAUNCH_ORDERED((binary_rows_kernel<Fn, uint64_t, 1, false>), grid, EW_BLOCK, 0, s, a, b, out, plan);
        }
        return cudaGetLastError();
    } else {
        WideTilePlan<2> w{};
        dim3 wgrid;
        if (make_wide_tile_plan<2>(p, w, wgrid)) {
            B200_LAUNCH_ORDERED((wide_tile_kernel<Fn, 2>), wgrid, 256, 0, s, a, b, out, w, LibmSplit{});
            return cudaGetLastError();
        }
        TilePlan<2> t{};
        uint64_t ctas = 0;
        if (make_tile_plan<2>(p, t, ctas)) {
            B200_LAUNCH_ORDERED((tile_kernel<Fn, 2>), (unsigned)ctas, dim3(TILE, TILE_ROWS), 0, s, a, b, out, t, LibmSplit{});
            return cudaGetLastError();
        }
    }
    auto g = make_gather_plan<2>(p);
    B200_LAUNCH_ORDERED((gather_kernel<Fn, 2>), tiles_for(p.n, EW_BLOCK), EW_BLOCK, 0, s, a, b, out, g, LibmSplit{});
    return cudaGetLastError();
}

template <class Fn> cudaError_t run_binary(const float *a, const float *b, float *out, const EwProblem &p, cudaStream_t s) {
    cudaError_t e = run_binary_body<Fn>(a, b, out, p, s);
    if constexpr (Fn::TAIL) {
        if (e == cudaSuccess && (p.n & 7)) {  // ordered behind the body on the same stream: overwrites its last few elements
            auto g = make_gather_plan<2>(p);
            B200_LAUNCH_ORDERED((binary_tail_kernel<Fn>), 1, 32, 0, s, a, b, out, g, p.n - (p.n & 7));
            e = cudaGetLastError();
        }
    }
    return e;
}

template <class Fn> cudaError_t run_unary(const float *x, float *out, const EwProblem &p, cudaStream_t s) {
    LibmSplit split{};
    split.n = p.n;
    split.inner = p.nd ? p.dim[p.nd - 1].size : 1;
    const uint64_t ist = p.nd ? p.dim[p.nd - 1].stride[0] : 0;  // no dims left: the reference sees stride 0
    split.mode = ist == 1 ? 0 : ist == 0 ? 1 : 2;
    if (p.nd <= 1 && (p.nd == 0 || p.dim[0].stride[0] == 1)) {
        const uint64_t n_poly = p.nd == 0 ? 0 : p.n - (p.n & 7);
        B200_LAUNCH_ORDERED((unary_flat_kernel<Fn>), tiles_for((p.n + 3) / 4, EW_BLOCK * EW_UNROLL), EW_BLOCK, 0, s, x, out, p.n, n_poly);
        return cudaGetLastError();
    }
    if (p.nd >= 2 && inner_is_unit_or_zero<1>(p)) {
        const int vec = rows_vec_width<1>(p);
        const uint64_t rows = p.n / p.dim[p.nd - 1].size;
        const uint64_t items = rows * ((p.dim[p.nd - 1].size + vec - 1) / vec);
        const unsigned grid = tiles_for(items, EW_BLOCK * EW_UNROLL);
        if (rows_plan_fits_32bit(items, p.dim[p.nd - 1].size)) {
            auto plan = make_rows_plan<uint32_t, 1>(p, vec);
            if (vec == 4) B200_LAUNCH_ORDERED((unary_rows_kernel<Fn, uint32_t, 4>), grid, EW_BLOCK, 0, s, x, out, plan, split);
            else B200_LAUNCH_ORDERED((unary_rows_kernel<Fn, uint32_t, 1>), grid, EW_BLOCK, 0, s, x, out, plan, split);
        } else {
            auto plan = make_rows_plan<uint64_t, 1>(p, vec);
            if (vec == 4) B200_LAUNCH_ORDERED((unary_rows_kernel<Fn, uint64_t, 4>), grid, EW_BLOCK, 0, s, x, out, plan, split);
            else B200_LAUNCH_ORDERED((unary_rows_kernel<Fn, uint64_t, 1>), grid, EW_BLOCK, 0, s, x, out, plan, split);
        }
        return cudaGetLastError();
    }
    if (p.nd >= 2) {
        WideTilePlan<1> w{};
        dim3 wgrid;
        if (make_wide_tile_plan<1>(p, w, wgrid)) {
            B200_LAUNCH_ORDERED((wide_tile_kernel<Fn, 1>), wgrid, 256, 0, s, x, nullptr, out, w, split);
            return cudaGetLastError();
        }
        TilePlan<1> t{};
        uint64_t ctas = 0;
        if (make_tile_plan<1>(p, t, ctas)) {
            B200_LAUNCH_ORDERED((tile_kernel<Fn, 1>), (unsigned)ctas, dim3(TILE, TILE_ROWS), 0, s, x, nullptr, out, t, split);
            return cudaGetLastError();
        }
    }
    auto g = make_gather_plan<1>(p);
    B200_LAUNCH_ORDERED((gather_kernel<Fn, 1>), tiles_for(p.n, EW_BLOCK), EW_BLOCK, 0, s, x, nullptr, out, g, split);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_unary(uint32_t op, const float *x, float *out, const EwProblem &p, cudaStream_t s) {
    switch (op) {
        case OP_NEG: return run_unary<UnaryFn<OP_NEG>>(x, out, p, s);
        case OP_EXP: return run_unary<UnaryFn<OP_EXP>>(x, out, p, s);
        case OP_LOG: return run_unary<UnaryFn<OP_LOG>>(x, out, p, s);
        case OP_RELU: return run_unary<UnaryFn<OP_RELU>>(x, out, p, s);
        case OP_TANH: return run_unary<UnaryFn<OP_TANH>>(x, out, p, s);
        case OP_STEP: return run_unary<UnaryFn<OP_STEP>>(x, out, p, s);
        case OP_COPY: return run_unary<UnaryFn<OP_COPY>>(x, out, p, s);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_binary(uint32_t op, const float *a, const float *b, float *out, const EwProblem &p, cudaStream_t s) {
    switch (op) {
        case OP_ADD: return run_binary<BinaryFn<OP_ADD>>(a, b, out, p, s);
        case OP_SUB: return run_binary<BinaryFn<OP_SUB>>(a, b, out, p, s);
        case OP_MUL: return run_binary<BinaryFn<OP_MUL>>(a, b, out, p, s);
        case OP_DIV: return run_binary<BinaryFn<OP_DIV>>(a, b, out, p, s);
        case OP_RELU_GRAD: return run_binary<BinaryFn<OP_RELU_GRAD>>(a, b, out, p, s);
        case OP_ADD_RELU: return run_binary<BinaryFn<OP_ADD_RELU>>(a, b, out, p, s);
        case OP_SUB_EXP: return run_binary<BinaryFn<OP_SUB_EXP>>(a, b, out, p, s);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_axpy(const float *a, const float *b, float *out, float alpha, uint64_t n, cudaStream_t s) {
    B200_LAUNCH_ORDERED(axpy_kernel, tiles_for((n + 3) / 4, EW_BLOCK * EW_UNROLL), EW_BLOCK, 0, s, a, b, out, alpha, n);
    return cudaGetLastError();
}

cudaError_t launch_fill(float *out, uint64_t n, float v, cudaStream_t s) {
    B200_LAUNCH_ORDERED(fill_kernel, tiles_for((n + 3) / 4, EW_BLOCK * EW_UNROLL), EW_BLOCK, 0, s, out, n, v);
    return cudaGetLastError();
}

cudaError_t launch_randn(float *out, uint64_t n, uint64_t seed, cudaStream_t s) {
    B200_LAUNCH_ORDERED(randn_kernel, tiles_for((n + 3) / 4, EW_BLOCK), EW_BLOCK, 0, s, out, n, seed);
    return cudaGetLastError();
}

cudaError_t launch_rand_uniform(float *out, uint64_t n, uint64_t seed, float lo, float scale, uint64_t first, cudaStream_t s) {
    B200_LAUNCH_ORDERED(rand_uniform_kernel, tiles_for((n + 3) / 4, EW_BLOCK), EW_BLOCK, 0, s, out, n, seed, lo, scale, first);
    return cudaGetLastError();
}

cudaError_t launch_matmul(const float *a, uint64_t ars, uint64_t acs, const float *b, uint64_t brs, uint64_t bcs, float *c,
                          uint64_t m, uint64_t n, uint64_t k, cudaStream_t s) {
    const uint64_t tiles_n = (n + TILE - 1) / TILE, tiles_m = (m + TILE - 1) / TILE;
    if (tiles_n * tiles_m > 0x7fffffffull) return cudaErrorInvalidValue;  // an output of more than 2^41 elements
    B200_LAUNCH_ORDERED(matmul_kernel, (unsigned)(tiles_n * tiles_m), dim3(TILE, TILE), 0, s, a, ars, acs, b, brs, bcs, c, m, n, k, (uint32_t)tiles_n);
    return cudaGetLastError();
}

}  // namespace b200
