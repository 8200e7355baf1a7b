// TEST INFRASTRUCTURE ONLY (CPU oracle; see pool.hpp).
//
// AVX2+FMA exp/log/tanh, restating plugins/cpu/src/simd.rs:23-118 intrinsic for intrinsic: every
// `_mm256_*` call of the Rust source has the same-named C intrinsic here, in the same order, so a
// build with AVX2+FMA produces the same bits as the reference on an AVX2+FMA host. Constants are
// written as the decimal literals of simd.rs; both compilers round them to the nearest f32.
#pragma once
#include <immintrin.h>
#include <limits>

namespace cpuref {

// simd.rs:6-15: the AVX2 paths are taken when the CPU has both AVX2 and FMA.
inline bool has_avx2() {
    static const bool ok = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
    return ok;
}

// simd.rs:23-48
__attribute__((target("avx2,fma"))) inline __m256 exp256(__m256 x) {
    const __m256 nan = _mm256_cmp_ps(x, x, _CMP_UNORD_Q);
    const __m256 too_big = _mm256_cmp_ps(x, _mm256_set1_ps(88.72284f), _CMP_GT_OQ);
    const __m256 xc = _mm256_max_ps(_mm256_min_ps(x, _mm256_set1_ps(88.72284f)), _mm256_set1_ps(-103.97208f));
    const __m256 n = _mm256_round_ps(_mm256_mul_ps(xc, _mm256_set1_ps(1.44269504088896340736f)),
                                     _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
    __m256 r = _mm256_fnmadd_ps(n, _mm256_set1_ps(0.6933594f), xc);
    r = _mm256_fnmadd_ps(n, _mm256_set1_ps(-2.1219444e-4f), r);
    __m256 y = _mm256_set1_ps(1.9875691e-4f);
    y = _mm256_fmadd_ps(y, r, _mm256_set1_ps(1.3981999e-3f));
    y = _mm256_fmadd_ps(y, r, _mm256_set1_ps(8.333452e-3f));
    y = _mm256_fmadd_ps(y, r, _mm256_set1_ps(4.1665796e-2f));
    y = _mm256_fmadd_ps(y, r, _mm256_set1_ps(1.6666665e-1f));
    y = _mm256_fmadd_ps(y, r, _mm256_set1_ps(5.0000001e-1f));
    y = _mm256_fmadd_ps(y, _mm256_mul_ps(r, r), r);
    y = _mm256_add_ps(y, _mm256_set1_ps(1.0f));
    const __m256i ni = _mm256_cvtps_epi32(n);
    const __m256i n1 = _mm256_srai_epi32(ni, 1);
    const __m256i n2 = _mm256_sub_epi32(ni, n1);
    const __m256 s1 = _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_add_epi32(n1, _mm256_set1_epi32(127)), 23));
    const __m256 s2 = _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_add_epi32(n2, _mm256_set1_epi32(127)), 23));
    __m256 res = _mm256_mul_ps(_mm256_mul_ps(y, s1), s2);
    res = _mm256_blendv_ps(res, _mm256_set1_ps(std::numeric_limits<float>::infinity()), too_big);
    return _mm256_blendv_ps(res, x, nan);
}

// simd.rs:52-97
__attribute__((target("avx2,fma"))) inline __m256 log256(__m256 x) {
    const __m256 zero = _mm256_setzero_ps();
    const __m256 is_nan = _mm256_cmp_ps(x, x, _CMP_UNORD_Q);
    const __m256 neg = _mm256_cmp_ps(x, zero, _CMP_LT_OQ);
    const __m256 is_zero = _mm256_cmp_ps(x, zero, _CMP_EQ_OQ);
    const __m256 is_inf = _mm256_cmp_ps(x, _mm256_set1_ps(std::numeric_limits<float>::infinity()), _CMP_EQ_OQ);
    const __m256 denorm = _mm256_cmp_ps(x, _mm256_castsi256_ps(_mm256_set1_epi32(0x00800000)), _CMP_LT_OQ);
    const __m256 xs = _mm256_blendv_ps(x, _mm256_mul_ps(x, _mm256_set1_ps(8388608.0f)), denorm);
    const __m256 adj = _mm256_and_ps(denorm, _mm256_set1_ps(23.0f));

    const __m256i bits = _mm256_castps_si256(xs);
    const __m256i emm = _mm256_srli_epi32(bits, 23);
    const __m256 m = _mm256_castsi256_ps(
        _mm256_or_si256(_mm256_and_si256(bits, _mm256_set1_epi32(0x007fffff)), _mm256_set1_epi32(0x3f000000)));
    const __m256 one = _mm256_set1_ps(1.0f);
    __m256 e = _mm256_cvtepi32_ps(_mm256_sub_epi32(emm, _mm256_set1_epi32(0x7f)));
    e = _mm256_sub_ps(_mm256_add_ps(e, one), adj);
    const __m256 mask = _mm256_cmp_ps(m, _mm256_set1_ps(0.707106781186547524400844362104849039f), _CMP_LT_OQ);
    const __m256 tmp = _mm256_and_ps(m, mask);
    __m256 x1 = _mm256_sub_ps(m, one);
    e = _mm256_sub_ps(e, _mm256_and_ps(one, mask));
    x1 = _mm256_add_ps(x1, tmp);
    const __m256 z = _mm256_mul_ps(x1, x1);
    __m256 y = _mm256_set1_ps(7.0376836e-2f);
    y = _mm256_fmadd_ps(y, x1, _mm256_set1_ps(-1.151461e-1f));
    y = _mm256_fmadd_ps(y, x1, _mm256_set1_ps(1.1676999e-1f));
    y = _mm256_fmadd_ps(y, x1, _mm256_set1_ps(-1.2420141e-1f));
    y = _mm256_fmadd_ps(y, x1, _mm256_set1_ps(1.4249323e-1f));
    y = _mm256_fmadd_ps(y, x1, _mm256_set1_ps(-1.6668058e-1f));
    y = _mm256_fmadd_ps(y, x1, _mm256_set1_ps(2.0000715e-1f));
    y = _mm256_fmadd_ps(y, x1, _mm256_set1_ps(-2.4999994e-1f));
    y = _mm256_fmadd_ps(y, x1, _mm256_set1_ps(3.3333332e-1f));
    y = _mm256_mul_ps(_mm256_mul_ps(y, x1), z);
    y = _mm256_fmadd_ps(e, _mm256_set1_ps(-2.1219444e-4f), y);
    y = _mm256_fnmadd_ps(z, _mm256_set1_ps(0.5f), y);
    __m256 res = _mm256_add_ps(x1, y);
    res = _mm256_fmadd_ps(e, _mm256_set1_ps(0.6933594f), res);

    res = _mm256_blendv_ps(res, _mm256_set1_ps(std::numeric_limits<float>::infinity()), is_inf);
    res = _mm256_blendv_ps(res, _mm256_set1_ps(-std::numeric_limits<float>::infinity()), is_zero);
    res = _mm256_blendv_ps(res, _mm256_set1_ps(std::numeric_limits<float>::quiet_NaN()), neg);
    return _mm256_blendv_ps(res, x, is_nan);
}

// simd.rs:103-118
__attribute__((target("avx2,fma"))) inline __m256 tanh256(__m256 x) {
    const __m256 nan = _mm256_cmp_ps(x, x, _CMP_UNORD_Q);
    const __m256 lim = _mm256_set1_ps(7.905311f);
    const __m256 xc = _mm256_max_ps(_mm256_min_ps(x, lim), _mm256_sub_ps(_mm256_setzero_ps(), lim));
    const __m256 x2 = _mm256_mul_ps(xc, xc);
    __m256 p = _mm256_set1_ps(-2.7607685e-16f);
    static const float pc[6] = {2.0001879e-13f, -8.604672e-11f, 5.122297e-8f, 1.4857224e-5f, 6.3726193e-4f, 4.8935245e-3f};
    for (float c : pc) p = _mm256_fmadd_ps(p, x2, _mm256_set1_ps(c));
    p = _mm256_mul_ps(p, xc);
    __m256 q = _mm256_set1_ps(1.1982584e-6f);
    static const float qc[3] = {1.185347e-4f, 2.2684346e-3f, 4.893525e-3f};
    for (float c : qc) q = _mm256_fmadd_ps(q, x2, _mm256_set1_ps(c));
    return _mm256_blendv_ps(_mm256_div_ps(p, q), x, nan);
}

}  // namespace cpuref
