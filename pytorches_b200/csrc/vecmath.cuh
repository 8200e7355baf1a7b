// exp / log / tanh for the B200 plugin.
//
// These are scalar restatements of the reference CPU plugin's AVX2+FMA polynomials
// (plugins/cpu/src/simd.rs:23-118), one lane at a time: every fused multiply-add of the original is
// an explicit __fmaf_rn here, every separately rounded multiply/add/divide an explicit
// __fmul_rn/__fadd_rn/__fdiv_rn (which the compiler never contracts or approximates), and the
// integer exponent manipulation is the same. On every input the result therefore carries the bits
// the reference computes in its vector body. The reference hands the last (len mod 8) elements of a
// row to libm instead; for those few elements this code may differ from it by an ulp or two.
#pragma once
#include <cuda_runtime.h>

namespace b200 {

// simd.rs:23-48, every input. Kept out of line: it runs only for the inputs exp_ref's short form
// does not take (|x| >= 86, NaN).
__device__ __noinline__ float exp_ref_full(float x) {
    const bool is_nan = x != x;
    const bool too_big = x > 88.72284f;
    // min(x, c) as SSE/AVX define it yields c for a NaN x; so does fminf, which is one instruction.
    // (What a NaN lane computes is discarded anyway; xc itself is never NaN for the max.)
    const float xc = fmaxf(fminf(x, 88.72284f), -103.97208f);
    const float n = rintf(__fmul_rn(xc, 1.44269504088896340736f));
    float r = __fmaf_rn(-n, 0.6933594f, xc);
    r = __fmaf_rn(-n, -2.1219444e-4f, r);
    float y = 1.9875691e-4f;
    y = __fmaf_rn(y, r, 1.3981999e-3f);
    y = __fmaf_rn(y, r, 8.333452e-3f);
    y = __fmaf_rn(y, r, 4.1665796e-2f);
    y = __fmaf_rn(y, r, 1.6666665e-1f);
    y = __fmaf_rn(y, r, 5.0000001e-1f);
    y = __fmaf_rn(y, __fmul_rn(r, r), r);
    y = __fadd_rn(y, 1.0f);
    // 2^n as two factors so that n in [-150, 128] never overflows the exponent field.
    const int ni = __float2int_rn(n);
    const int n1 = ni >> 1;
    const int n2 = ni - n1;
    const float s1 = __int_as_float((n1 + 127) << 23);
    const float s2 = __int_as_float((n2 + 127) << 23);
    float res = __fmul_rn(__fmul_rn(y, s1), s2);
    res = too_big ? __int_as_float(0x7f800000) : res;
    return is_nan ? x : res;
}

// The same function for |x| < 86, which is where nearly every input of a real workload lies, in
// about half the instructions and with the same bits (checked against exp_ref_full on every such
// float). What the range buys: the clamps, the NaN and overflow selects never act; n = rint(x*log2e)
// has |n| <= 125, so (a) adding and subtracting 1.5*2^23 rounds to the nearest integer exactly as
// rintf does (ties to even) and leaves that integer in the low bits of the intermediate, and (b)
// y * 2^n neither overflows nor goes subnormal (y is in [0.7, 1.42]), so the two exact multiplies of
// the full form equal one integer add of n into y's exponent field. (t << 23 drops the constant:
// its low 9 bits are zero.)
__device__ __forceinline__ float exp_ref(float x) {
    if (!(fabsf(x) < 86.0f)) return exp_ref_full(x);
    const float magic = 12582912.0f;
    const float t = __fadd_rn(__fmul_rn(x, 1.44269504088896340736f), magic);
    const float n = __fsub_rn(t, magic);
    float r = __fmaf_rn(-n, 0.6933594f, x);
    r = __fmaf_rn(-n, -2.1219444e-4f, r);
    float y = 1.9875691e-4f;
    y = __fmaf_rn(y, r, 1.3981999e-3f);
    y = __fmaf_rn(y, r, 8.333452e-3f);
    y = __fmaf_rn(y, r, 4.1665796e-2f);
    y = __fmaf_rn(y, r, 1.6666665e-1f);
    y = __fmaf_rn(y, r, 5.0000001e-1f);
    y = __fmaf_rn(y, __fmul_rn(r, r), r);
    y = __fadd_rn(y, 1.0f);
    return __int_as_float(__float_as_int(y) + (__float_as_int(t) << 23));
}

// simd.rs:52-97 from the mantissa/exponent split on: m in [0.5, 1), e the matching exponent.
__device__ __forceinline__ float log_ref_tail(float m, float e) {
    const bool below = m < 0.707106781186547524400844362104849039f;
    const float tmp = below ? m : 0.0f;
    float x1 = __fsub_rn(m, 1.0f);
    e = __fsub_rn(e, below ? 1.0f : 0.0f);
    x1 = __fadd_rn(x1, tmp);
    const float z = __fmul_rn(x1, x1);
    float y = 7.0376836e-2f;
    y = __fmaf_rn(y, x1, -1.151461e-1f);
    y = __fmaf_rn(y, x1, 1.1676999e-1f);
    y = __fmaf_rn(y, x1, -1.2420141e-1f);
    y = __fmaf_rn(y, x1, 1.4249323e-1f);
    y = __fmaf_rn(y, x1, -1.6668058e-1f);
    y = __fmaf_rn(y, x1, 2.0000715e-1f);
    y = __fmaf_rn(y, x1, -2.4999994e-1f);
    y = __fmaf_rn(y, x1, 3.3333332e-1f);
    y = __fmul_rn(__fmul_rn(y, x1), z);
    y = __fmaf_rn(e, -2.1219444e-4f, y);
    y = __fmaf_rn(-z, 0.5f, y);
    const float res = __fadd_rn(x1, y);
    return __fmaf_rn(e, 0.6933594f, res);
}

// simd.rs:52-97, every input; out of line, for what log_ref's short form does not take.
__device__ __noinline__ float log_ref_full(float x) {
    const bool is_nan = x != x;
    const bool neg = x < 0.0f;
    const bool is_zero = x == 0.0f;
    const bool is_inf = x == __int_as_float(0x7f800000);
    const bool denorm = x < __int_as_float(0x00800000);
    const float xs = denorm ? __fmul_rn(x, 8388608.0f) : x;
    const float adj = denorm ? 23.0f : 0.0f;
    const unsigned bits = (unsigned)__float_as_int(xs);
    const int emm = (int)(bits >> 23);
    const float m = __int_as_float((int)((bits & 0x007fffffu) | 0x3f000000u));
    float e = __int2float_rn(emm - 0x7f);
    e = __fsub_rn(__fadd_rn(e, 1.0f), adj);
    float res = log_ref_tail(m, e);
    res = is_inf ? __int_as_float(0x7f800000) : res;
    res = is_zero ? __int_as_float(0xff800000) : res;
    res = neg ? __int_as_float(0x7fc00000) : res;
    return is_nan ? x : res;
}

// Positive, normal, finite x (one unsigned compare decides): no rescaling, no special value applies
// and the exponent is (bits >> 23) - 126 as an exact small integer. Same bits as log_ref_full on
// every such float (checked exhaustively).
__device__ __forceinline__ float log_ref(float x) {
    const unsigned bits = (unsigned)__float_as_int(x);
    if (bits - 0x00800000u >= 0x7f000000u) return log_ref_full(x);
    const float m = __int_as_float((int)((bits & 0x007fffffu) | 0x3f000000u));
    return log_ref_tail(m, __int2float_rn((int)(bits >> 23) - 126));
}

// simd.rs:103-118
__device__ __forceinline__ float tanh_ref(float x) {
    const bool is_nan = x != x;
    const float lim = 7.905311f;
    const float xc = fmaxf(fminf(x, lim), -lim);  // NaN x -> lim, like the AVX min; the lane is replaced below
    const float x2 = __fmul_rn(xc, xc);
    float p = -2.7607685e-16f;
    p = __fmaf_rn(p, x2, 2.0001879e-13f);
    p = __fmaf_rn(p, x2, -8.604672e-11f);
    p = __fmaf_rn(p, x2, 5.122297e-8f);
    p = __fmaf_rn(p, x2, 1.4857224e-5f);
    p = __fmaf_rn(p, x2, 6.3726193e-4f);
    p = __fmaf_rn(p, x2, 4.8935245e-3f);
    p = __fmul_rn(p, xc);
    float q = 1.1982584e-6f;
    q = __fmaf_rn(q, x2, 1.185347e-4f);
    q = __fmaf_rn(q, x2, 2.2684346e-3f);
    q = __fmaf_rn(q, x2, 4.893525e-3f);
    const float res = __fdiv_rn(p, q);
    return is_nan ? x : res;
}

}  // namespace b200
