// TEST INFRASTRUCTURE ONLY (CPU oracle; see pool.hpp).
//
// Elementwise and reduction kernels of the reference CPU plugin, restated in C++:
//   plugins/cpu/src/ew.rs      coalesce, rows, unary, transpose, binary, axpy, fill, randn
//   plugins/cpu/src/reduce.rs  sum_axis (row path and column path)
// The chunk sizes, the AVX2-body / scalar-tail split and every association order are kept, because
// they decide the bits. Build with -ffp-contract=off: the Rust original never contracts a*b+c.
//
// max_axis / argmax_axis at the end have NO counterpart in the reference (parity unpinned there);
// they are plain scans with torch-CPU semantics and are pinned against torch in the tests.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "pool.hpp"
#include "vecmath.hpp"

namespace cpuref {

enum : uint32_t {
    OP_NEG = 1, OP_EXP = 2, OP_LOG = 3, OP_RELU = 4, OP_TANH = 5, OP_STEP = 6,
    OP_ADD = 100, OP_SUB = 101, OP_MUL = 102, OP_DIV = 103,
    OP_MATMUL = 200, OP_SUM_AXIS = 201, OP_MATMUL_T = 202, OP_MAX_AXIS = 203, OP_ARGMAX_AXIS = 204,
    OP_MAX_ARGMAX_AXIS = 205, OP_ARGMAX_COMBINE = 206,
    OP_COPY = 300, OP_FILL = 400, OP_RAND_NORMAL = 401, OP_RAND_UNIFORM = 402, OP_AXPY = 500,
    OP_RELU_GRAD = 501, OP_ADD_RELU = 502, OP_SUB_EXP = 503,  // appended fused ops (not in the reference)
};

constexpr size_t CHUNK = size_t(1) << 16;    // ew.rs:13
constexpr size_t PAR_MIN = size_t(1) << 15;  // ew.rs:15
constexpr size_t BLOCK = size_t(1) << 16;    // reduce.rs:10
constexpr size_t COLS = 2048;                // reduce.rs:12

#define CPUREF_AVX2 __attribute__((target("avx2,fma")))
#define CPUREF_INLINE inline __attribute__((always_inline))

// One dimension after coalescing: size and the element stride of each of the N operands (ew.rs:18).
template <int N> struct Dim {
    size_t size;
    size_t st[N];
};

// ew.rs:22-43: drop size-1 dims; merge a dim into the previous one when, for every operand,
// previous stride == this stride * this size.
template <int N>
std::vector<Dim<N>> coalesce(const uint64_t *shape, size_t nd, const uint64_t *const strides[N]) {
    std::vector<Dim<N>> v;
    for (size_t d = 0; d < nd; ++d) {
        size_t s = (size_t)shape[d];
        if (s == 1) continue;
        Dim<N> cur;
        cur.size = s;
        for (int k = 0; k < N; ++k) cur.st[k] = (size_t)strides[k][d];
        if (!v.empty()) {
            Dim<N> &last = v.back();
            bool merge = true;
            for (int k = 0; k < N; ++k) merge = merge && (last.st[k] == cur.st[k] * s);
            if (merge) {
                last.size *= s;
                for (int k = 0; k < N; ++k) last.st[k] = cur.st[k];
                continue;
            }
        }
        v.push_back(cur);
    }
    return v;
}

// ew.rs:46-87: calls row(out_offset, operand_offsets, len) for each maximal inner run of [lo, hi).
template <int N, class F> void rows(const std::vector<Dim<N>> &dims, size_t lo, size_t hi, F &&row) {
    size_t offs[N];
    for (int k = 0; k < N; ++k) offs[k] = 0;
    if (dims.empty()) {
        row(lo, offs, hi - lo);
        return;
    }
    const size_t nd = dims.size();
    std::vector<size_t> idx(nd, 0);
    size_t rem = lo;
    for (size_t d = nd; d-- > 0;) {
        idx[d] = rem % dims[d].size;
        rem /= dims[d].size;
    }
    for (size_t d = 0; d < nd; ++d)
        for (int k = 0; k < N; ++k) offs[k] += idx[d] * dims[d].st[k];
    const size_t inner = dims[nd - 1].size;
    size_t pos = lo;
    while (pos < hi) {
        size_t len = std::min(inner - idx[nd - 1], hi - pos);
        row(pos, offs, len);
        pos += len;
        idx[nd - 1] += len;
        for (int k = 0; k < N; ++k) offs[k] += len * dims[nd - 1].st[k];
        size_t d = nd - 1;
        while (d > 0 && idx[d] == dims[d].size) {
            for (int k = 0; k < N; ++k) offs[k] -= dims[d].size * dims[d].st[k];
            idx[d] = 0;
            d -= 1;
            idx[d] += 1;
            for (int k = 0; k < N; ++k) offs[k] += dims[d].st[k];
        }
    }
}

// ---- unary (ew.rs:95-188) ----------------------------------------------------------------------

// ew.rs:96-106. RELU is Rust's f32::max(v, 0.0): a NaN input gives 0.0; the sign of the zero
// returned for v = -0.0 is unspecified there, +0.0 here.
CPUREF_INLINE void unary_generic(uint32_t op, const float *x, float *o, size_t n) {
    switch (op) {
        case OP_NEG: for (size_t i = 0; i < n; ++i) o[i] = -x[i]; break;
        case OP_RELU: for (size_t i = 0; i < n; ++i) o[i] = x[i] > 0.0f ? x[i] : 0.0f; break;
        case OP_STEP: for (size_t i = 0; i < n; ++i) o[i] = x[i] > 0.0f ? 1.0f : 0.0f; break;
        case OP_EXP: for (size_t i = 0; i < n; ++i) o[i] = std::exp(x[i]); break;
        case OP_LOG: for (size_t i = 0; i < n; ++i) o[i] = std::log(x[i]); break;
        case OP_TANH: for (size_t i = 0; i < n; ++i) o[i] = std::tanh(x[i]); break;
        default: std::memmove(o, x, n * sizeof(float)); break;  // COPY
    }
}

inline void unary_plain(uint32_t op, const float *x, float *o, size_t n) { unary_generic(op, x, o, n); }

// ew.rs:112-138: polynomial for the first n/8*8 elements of THIS call, libm for the rest.
CPUREF_AVX2 inline void unary_avx2(uint32_t op, const float *x, float *o, size_t n) {
    const size_t n8 = n / 8 * 8;
    switch (op) {
        case OP_EXP: for (size_t i = 0; i < n8; i += 8) _mm256_storeu_ps(o + i, exp256(_mm256_loadu_ps(x + i))); break;
        case OP_LOG: for (size_t i = 0; i < n8; i += 8) _mm256_storeu_ps(o + i, log256(_mm256_loadu_ps(x + i))); break;
        case OP_TANH: for (size_t i = 0; i < n8; i += 8) _mm256_storeu_ps(o + i, tanh256(_mm256_loadu_ps(x + i))); break;
        default: unary_generic(op, x, o, n); return;
    }
    unary_generic(op, x + n8, o + n8, n - n8);
}

inline void unary_dispatch(uint32_t op, const float *x, float *o, size_t n) {
    if (has_avx2()) return unary_avx2(op, x, o, n);
    unary_plain(op, x, o, n);
}

// ew.rs:197-219: blocked transpose of a contiguous [rows, cols] matrix into [cols, rows].
inline void transpose(const float *src, size_t nrows, size_t ncols, float *out) {
    constexpr size_t T = 32;
    const size_t tile_rows = (nrows + T - 1) / T;
    const size_t tasks = nrows * ncols < PAR_MIN ? 1 : tile_rows;
    const size_t per = (tile_rows + tasks - 1) / tasks;
    Pool::get().run_tasks(tasks, [&](size_t t) {
        for (size_t tr = t * per; tr < std::min((t + 1) * per, tile_rows); ++tr) {
            size_t i0 = tr * T, i1 = std::min(i0 + T, nrows);
            for (size_t j0 = 0; j0 < ncols; j0 += T) {
                size_t j1 = std::min(j0 + T, ncols);
                for (size_t i = i0; i < i1; ++i)
                    for (size_t j = j0; j < j1; ++j) out[j * nrows + i] = src[i * ncols + j];
            }
        }
    });
}

// ew.rs:149-188
inline void unary(uint32_t op, const float *x, const uint64_t *shape, const uint64_t *strides, size_t nd, float *out) {
    size_t n = 1;
    for (size_t d = 0; d < nd; ++d) n *= (size_t)shape[d];
    if (n == 0) return;
    const uint64_t *sts[1] = {strides};
    auto dims = coalesce<1>(shape, nd, sts);
    // ew.rs:192-194: a COPY whose merged dims are (c,[1]),(r,[c]) is a plain 2-D transpose.
    if (op == OP_COPY && dims.size() == 2 && dims[0].st[0] == 1 && dims[1].st[0] == dims[0].size)
        return transpose(x, dims[1].size, dims[0].size, out);
    const size_t st = dims.empty() ? 0 : dims.back().st[0];
    const size_t chunk = n < PAR_MIN ? n : CHUNK;
    Pool::get().for_chunks(n, chunk, [&](size_t lo, size_t hi) {
        rows<1>(dims, lo, hi, [&](size_t oo, const size_t *offs, size_t len) {
            float *dst = out + oo;
            if (st == 1) {
                unary_dispatch(op, x + offs[0], dst, len);
            } else if (st == 0) {
                float v = x[offs[0]], tmp = 0.0f;
                unary_dispatch(op, &v, &tmp, 1);
                std::fill(dst, dst + len, tmp);
            } else {
                float buf[256];  // gather so the math still runs on contiguous data (ew.rs:174-184)
                size_t done = 0;
                while (done < len) {
                    size_t m = std::min(len - done, (size_t)256);
                    for (size_t i = 0; i < m; ++i) buf[i] = x[offs[0] + (done + i) * st];
                    unary_dispatch(op, buf, dst + done, m);
                    done += m;
                }
            }
        });
    });
}

// ---- binary (ew.rs:223-300) --------------------------------------------------------------------

template <class F>
CPUREF_INLINE void binary_row_op(F f, const float *a, size_t sa, const float *b, size_t sb, float *o, size_t len) {
    if (sa == 1 && sb == 1) {
        for (size_t i = 0; i < len; ++i) o[i] = f(a[i], b[i]);
    } else if (sa == 1 && sb == 0) {
        const float y = *b;
        for (size_t i = 0; i < len; ++i) o[i] = f(a[i], y);
    } else if (sa == 0 && sb == 1) {
        const float x = *a;
        for (size_t i = 0; i < len; ++i) o[i] = f(x, b[i]);
    } else {
        for (size_t i = 0; i < len; ++i) o[i] = f(a[i * sa], b[i * sb]);
    }
}

CPUREF_INLINE void binary_row_impl(uint32_t op, const float *a, size_t sa, const float *b, size_t sb, float *o, size_t len) {
    switch (op) {
        case OP_ADD: binary_row_op([](float x, float y) { return x + y; }, a, sa, b, sb, o, len); break;
        case OP_SUB: binary_row_op([](float x, float y) { return x - y; }, a, sa, b, sb, o, len); break;
        case OP_MUL: binary_row_op([](float x, float y) { return x * y; }, a, sa, b, sb, o, len); break;
        default: binary_row_op([](float x, float y) { return x / y; }, a, sa, b, sb, o, len); break;
    }
}
inline void binary_row_plain(uint32_t op, const float *a, size_t sa, const float *b, size_t sb, float *o, size_t len) {
    binary_row_impl(op, a, sa, b, sb, o, len);
}
CPUREF_AVX2 inline void binary_row_avx2(uint32_t op, const float *a, size_t sa, const float *b, size_t sb, float *o, size_t len) {
    binary_row_impl(op, a, sa, b, sb, o, len);
}

inline void binary(uint32_t op, const float *a, const uint64_t *sta, const float *b, const uint64_t *stb,
                   const uint64_t *shape, size_t nd, float *out) {
    size_t n = 1;
    for (size_t d = 0; d < nd; ++d) n *= (size_t)shape[d];
    if (n == 0) return;
    const uint64_t *sts[2] = {sta, stb};
    auto dims = coalesce<2>(shape, nd, sts);
    const size_t ia = dims.empty() ? 0 : dims.back().st[0];
    const size_t ib = dims.empty() ? 0 : dims.back().st[1];
    const bool avx = has_avx2();
    const size_t chunk = n < PAR_MIN ? n : CHUNK;
    Pool::get().for_chunks(n, chunk, [&](size_t lo, size_t hi) {
        rows<2>(dims, lo, hi, [&](size_t oo, const size_t *offs, size_t len) {
            if (avx) binary_row_avx2(op, a + offs[0], ia, b + offs[1], ib, out + oo, len);
            else binary_row_plain(op, a + offs[0], ia, b + offs[1], ib, out + oo, len);
        });
    });
}

// ---- axpy, fill, random (ew.rs:304-380) --------------------------------------------------------

inline void axpy_impl(const float *a, const float *b, float *o, float alpha, size_t len) {
    for (size_t i = 0; i < len; ++i) o[i] = a[i] + alpha * b[i];  // two roundings (no contraction)
}

// ew.rs:316-329: one-rounding FMA for the first len/8*8 elements, unfused tail.
CPUREF_AVX2 inline void axpy_avx2(const float *a, const float *b, float *o, float alpha, size_t len) {
    const __m256 va = _mm256_set1_ps(alpha);
    const size_t n8 = len / 8 * 8;
    for (size_t i = 0; i < n8; i += 8)
        _mm256_storeu_ps(o + i, _mm256_fmadd_ps(va, _mm256_loadu_ps(b + i), _mm256_loadu_ps(a + i)));
    axpy_impl(a + n8, b + n8, o + n8, alpha, len - n8);
}

inline void axpy(const float *a, const float *b, float *out, float alpha, size_t n) {
    const bool avx = has_avx2();
    const size_t chunk = n < PAR_MIN ? std::max(n, (size_t)1) : CHUNK;
    Pool::get().for_chunks(n, chunk, [&](size_t lo, size_t hi) {
        if (avx) axpy_avx2(a + lo, b + lo, out + lo, alpha, hi - lo);
        else axpy_impl(a + lo, b + lo, out + lo, alpha, hi - lo);
    });
}

inline void fill(float *out, size_t n, float v) {
    const size_t chunk = n < PAR_MIN ? std::max(n, (size_t)1) : CHUNK;
    Pool::get().for_chunks(n, chunk, [&](size_t lo, size_t hi) { std::fill(out + lo, out + hi, v); });
}

inline uint64_t splitmix64(uint64_t x) {  // ew.rs:356-361
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

inline float rand_normal(uint64_t seed, uint64_t i) {  // ew.rs:364-369
    const uint64_t h = splitmix64(seed ^ (i * 0x9E3779B97F4A7C15ull));
    const float u1 = (float)((h >> 40) + 1) / 16777216.0f;
    const float u2 = (float)(h & 0xFFFFFFull) / 16777216.0f;
    return std::sqrt(-2.0f * std::log(u1)) * std::cos(2.0f * 3.14159265358979323846264338327950288f * u2);
}

inline void randn(float *out, size_t n, uint64_t seed) {  // ew.rs:371-380
    const size_t chunk = n < PAR_MIN ? std::max(n, (size_t)1) : (size_t(1) << 14);
    Pool::get().for_chunks(n, chunk, [&](size_t lo, size_t hi) {
        for (size_t i = lo; i < hi; ++i) out[i] = rand_normal(seed, (uint64_t)i);
    });
}

// RAND_UNIFORM (appended op, not in the reference): the same counter hash, u = (h >> 40) / 2^24,
// out = lo + scale * u with the multiply and the add rounded separately.
inline void rand_uniform(float *out, size_t n, uint64_t seed, float lo, float scale, uint64_t first) {
    const size_t chunk = n < PAR_MIN ? std::max(n, (size_t)1) : (size_t(1) << 14);
    Pool::get().for_chunks(n, chunk, [&](size_t b, size_t e) {
        for (size_t i = b; i < e; ++i) {
            const uint64_t h = splitmix64(seed ^ ((first + (uint64_t)i) * 0x9E3779B97F4A7C15ull));
            const float u = (float)(h >> 40) / 16777216.0f;
            const float scaled = scale * u;
            out[i] = lo + scaled;
        }
    });
}

// ---- sum over an axis (reduce.rs) --------------------------------------------------------------

inline float sum_slice_plain(const float *x, size_t n) {  // reduce.rs:15-32
    float acc[16] = {0};
    size_t n16 = n / 16 * 16;
    for (size_t i = 0; i < n16; i += 16)
        for (int k = 0; k < 16; ++k) acc[k] += x[i + k];
    float s = 0.0f;
    for (int k = 0; k < 16; ++k) s += acc[k];
    for (size_t i = n16; i < n; ++i) s += x[i];
    return s;
}

// reduce.rs:36-61. Element i of the slice goes to accumulator slot i mod 32 (4 registers x 8
// lanes); the slots are then combined as ((a0+a1)+(a2+a3)), high half onto low half, lanes
// (0+2),(1+3), and finally those two; the last n mod 32 elements are added one by one.
CPUREF_AVX2 inline float sum_slice_avx2(const float *p, size_t n) {
    __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0;
    const size_t n32 = n / 32 * 32;
    for (size_t i = 0; i < n32; i += 32) {
        a0 = _mm256_add_ps(a0, _mm256_loadu_ps(p + i));
        a1 = _mm256_add_ps(a1, _mm256_loadu_ps(p + i + 8));
        a2 = _mm256_add_ps(a2, _mm256_loadu_ps(p + i + 16));
        a3 = _mm256_add_ps(a3, _mm256_loadu_ps(p + i + 24));
    }
    const __m256 v = _mm256_add_ps(_mm256_add_ps(a0, a1), _mm256_add_ps(a2, a3));
    const __m128 lo = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
    __m128 sh = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
    sh = _mm_add_ss(sh, _mm_shuffle_ps(sh, sh, 1));
    float s = _mm_cvtss_f32(sh);
    for (size_t i = n32; i < n; ++i) s += p[i];
    return s;
}

inline float sum_slice(const float *x, size_t n) {
    if (has_avx2()) return sum_slice_avx2(x, n);
    return sum_slice_plain(x, n);
}

// reduce.rs:100-146: out[o*inner + i] = sum_j x[(o*n + j)*inner + i].
inline void sum_axis(const float *x, size_t outer, size_t n, size_t inner, float *out) {
    const size_t total = outer * inner;
    if (total == 0) return;
    if (n == 0) {
        std::fill(out, out + total, 0.0f);
        return;
    }
    if (inner == 1) {
        // Rows are cut into BLOCK-element pieces summed independently, then added in block order.
        const size_t blocks = (n + BLOCK - 1) / BLOCK;
        std::vector<float> partial(outer * blocks, 0.0f);
        Pool::get().run_tasks(outer * blocks, [&](size_t t) {
            size_t row = t / blocks, b = t % blocks;
            size_t lo = b * BLOCK, hi = std::min(lo + BLOCK, n);
            partial[t] = sum_slice(x + row * n + lo, hi - lo);
        });
        for (size_t row = 0; row < outer; ++row) {
            float s = 0.0f;
            for (size_t b = 0; b < blocks; ++b) s += partial[row * blocks + b];
            out[row] = s;
        }
        return;
    }
    // inner > 1: each output column accumulates rows j = 0..n-1 in order, starting from 0.0.
    const size_t chunks = (inner + COLS - 1) / COLS;
    Pool::get().run_tasks(outer * chunks, [&](size_t t) {
        size_t o = t / chunks, c = t % chunks;
        size_t i0 = c * COLS, len = std::min(i0 + COLS, inner) - i0;
        float *dst = out + o * inner + i0;
        std::fill(dst, dst + len, 0.0f);
        for (size_t j = 0; j < n; ++j) {
            const float *src = x + (o * n + j) * inner + i0;
            for (size_t i = 0; i < len; ++i) dst[i] += src[i];
        }
    });
}

// ---- max / argmax over an axis: NOT in the reference ----------------------------------------------
// torch CPU semantics: a NaN wins (first NaN position for argmax); ties keep the lowest index.
inline void max_scan(const float *p, size_t stride, size_t lo, size_t hi, float &best, int64_t &bi) {
    best = p[lo * stride];
    bi = (int64_t)lo;
    for (size_t j = lo + 1; j < hi && !(best != best); ++j) {
        const float v = p[j * stride];
        if (v > best || v != v) {
            best = v;
            bi = (int64_t)j;
        }
    }
}

inline void max_axis(const float *x, size_t outer, size_t n, size_t inner, float *out_val, int64_t *out_idx, int64_t idx_offset = 0) {
    const size_t total = outer * inner;
    if (inner == 1 && n > BLOCK) {
        // Long rows: scan BLOCK-sized pieces in parallel, then keep the first best piece. The result
        // does not depend on the split, so this is the same function as the plain scan below.
        const size_t blocks = (n + BLOCK - 1) / BLOCK;
        std::vector<float> pv(outer * blocks);
        std::vector<int64_t> pi(outer * blocks);
        Pool::get().run_tasks(outer * blocks, [&](size_t t) {
            const size_t row = t / blocks, b = t % blocks;
            max_scan(x + row * n, 1, b * BLOCK, std::min((b + 1) * BLOCK, n), pv[t], pi[t]);
        });
        for (size_t row = 0; row < outer; ++row) {
            float best = pv[row * blocks];
            int64_t bi = pi[row * blocks];
            for (size_t b = 1; b < blocks && !(best != best); ++b) {
                const float v = pv[row * blocks + b];
                if (v > best || v != v) {
                    best = v;
                    bi = pi[row * blocks + b];
                }
            }
            if (out_val) out_val[row] = best;
            if (out_idx) out_idx[row] = bi + idx_offset;
        }
        return;
    }
    Pool::get().for_chunks(total, 256, [&](size_t lo, size_t hi) {
        for (size_t t = lo; t < hi; ++t) {
            const size_t o = t / inner, i = t % inner;
            float best;
            int64_t bi;
            max_scan(x + o * n * inner + i, inner, 0, n, best, bi);
            if (out_val) out_val[t] = best;
            if (out_idx) out_idx[t] = bi + idx_offset;
        }
    });
}

// Picks, per column, the best of G candidates (value, position): NaN wins, then the larger value,
// then the lower position. Combines per-shard results of a sharded argmax. NOT in the reference.
inline void argmax_combine(const float *vals, const int64_t *idx, size_t g, size_t m, int64_t *out) {
    for (size_t j = 0; j < m; ++j) {
        float bv = vals[j];
        int64_t bi = idx[j];
        for (size_t r = 1; r < g; ++r) {
            const float v = vals[r * m + j];
            const int64_t i = idx[r * m + j];
            const bool vn = v != v, bn = bv != bv;
            const bool better = (vn || bn) ? (vn && (!bn || i < bi)) : (v > bv || (v == bv && i < bi));
            if (better) {
                bv = v;
                bi = i;
            }
        }
        out[j] = bi;
    }
}

// ---- matmul: required by the ABI, outside the measured path ------------------------------------------
// A plain f32 dot product per output (k in order, FMA). It does NOT follow the blocking of
// plugins/cpu/src/gemm.rs, so its bits differ from the reference; tests compare with f64 at the
// reference's tolerance (plugins/cpu/tests/kernels.rs:102).
inline void matmul(size_t m, size_t n, size_t k, const float *a, size_t ars, size_t acs, const float *b,
                   size_t brs, size_t bcs, float *c) {
    Pool::get().for_chunks(m, 4, [&](size_t lo, size_t hi) {
        for (size_t i = lo; i < hi; ++i)
            for (size_t j = 0; j < n; ++j) {
                float s = 0.0f;
                for (size_t p = 0; p < k; ++p) s = std::fma(a[i * ars + p * acs], b[p * brs + j * bcs], s);
                c[i * n + j] = s;
            }
    });
}

}  // namespace cpuref
