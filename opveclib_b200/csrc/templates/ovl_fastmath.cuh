// Tolerance-bounded fp32 math for generated kernels (sm_100a): the `math='tolerance'` lowering.
//
// The exact lowering calls CUDA's libm and IEEE division so that results track the reference's C++ operator to
// the last bit or two; a fused chain with several transcendentals then spends its time issuing instructions, not
// moving bytes.  The routines here spend the error budget the backend is allowed (element-wise fp32 within
// 2 units in the last place, transcendental results within rtol 1e-5) on fewer instructions:
//
//   division   n * rcp.approx(d)                                      relative error <= 2^-23 + 2^-24 (1.8e-7)
//              (compile with -DOVL_TOL_DIV_NEWTON=1 for one residual correction in explicit fma: <= 1 ulp)
//   exp        ex2.approx of x * log2(e)                              <= 2^-22 + 6e-8 * |x| relative
//   log        exponent split + degree-7 polynomial on [2/3, 4/3)     <= 2 ulp, also next to 1
//   tanh       odd polynomial below 0.55, 1 - 2 / (exp(2x) + 1) above <= 6e-7 relative
//   log10      log * log10(e)                                         <= 3 ulp
//   sqrt       sqrt.approx                                            <= 2^-23 relative
//
// NaN, +-inf and zero arguments give what the exact functions give.  Subnormal arguments (of log, too: its result
// is then -inf) and subnormal results of exp and of the division count as zero (the approximate instructions flush
// them).  The user's own +, -, * stay separate,
// exactly rounded operations (no contraction); explicit fma appears only inside these routines, as in any libm.
//
// Everything exists twice: for one float, and for a pair of floats held in one 64-bit register, where additions,
// multiplications and fused multiply-adds are the packed `*.f32x2` instructions of sm_100 - one issue slot for
// two elements.  Comparisons, selects, the special-function unit and the integer steps of log work per element.
#pragma once
#include <stdint.h>
#include <math.h>

namespace ovl {
namespace tol {

#ifndef OVL_TOL_DIV_NEWTON
#define OVL_TOL_DIV_NEWTON 0
#endif

// ---------------------------------------------------------------------------------------------------------
// special-function unit
__device__ __forceinline__ float mufu_rcp(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float mufu_sqrt(float x) {
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float mufu_ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// ---------------------------------------------------------------------------------------------------------
// constants
#define OVL_TOL_LOG2E 1.4426950408889634f
#define OVL_TOL_LN2 0.6931471805599453f
// log(1 + f) = f + f^2 * Q(f) on f in [-1/3, 1/3]; weighted minimax fit, relative error 2.6e-8
#define OVL_TOL_LQ0 -0.49999936078009044f
#define OVL_TOL_LQ1 0.3333319813734399f
#define OVL_TOL_LQ2 -0.25007818964199596f
#define OVL_TOL_LQ3 0.2001116865627148f
#define OVL_TOL_LQ4 -0.16415959265035213f
#define OVL_TOL_LQ5 0.13995807124828513f
#define OVL_TOL_LQ6 -0.15388548689958223f
#define OVL_TOL_LQ7 0.14026358592156937f
// tanh(x) = x + x^3 * P(x^2) on |x| <= 0.55; relative error 3.7e-8
#define OVL_TOL_TP0 -0.3333294663423962f
#define OVL_TOL_TP1 0.13320725002921485f
#define OVL_TOL_TP2 -0.05267181011464024f
#define OVL_TOL_TP3 0.01643757460070023f
#define OVL_TOL_TANH_SPLIT 0.55f
// alternative (-DOVL_TOL_TANH_RATIONAL=1): tanh(x) = x * P(x^2) / Q(x^2) on |x| <= 9 (tanh is 1 in fp32 beyond), both of
// degree 4, relative error 2.1e-8 before rounding; P is scaled by 1 - 3e-7 so that rounding cannot carry a result
// past 1
#define OVL_TOL_TR_SCALE 0.9999997f
#define OVL_TOL_TRP0 (0.9999999794560867f * OVL_TOL_TR_SCALE)
#define OVL_TOL_TRP1 (0.13381027540820747f * OVL_TOL_TR_SCALE)
#define OVL_TOL_TRP2 (0.003495590311460851f * OVL_TOL_TR_SCALE)
#define OVL_TOL_TRP3 (2.0609115037626294e-05f * OVL_TOL_TR_SCALE)
#define OVL_TOL_TRP4 (1.3354700564421183e-08f * OVL_TOL_TR_SCALE)
#define OVL_TOL_TRQ1 0.46714343135843744f
#define OVL_TOL_TRQ2 0.02587699070470303f
#define OVL_TOL_TRQ3 0.00032856382533732716f
#define OVL_TOL_TRQ4 7.776575625539569e-07f
#ifndef OVL_TOL_TANH_RATIONAL
#define OVL_TOL_TANH_RATIONAL 0
#endif

// ---------------------------------------------------------------------------------------------------------
// one float

__device__ __forceinline__ float fdiv(float n, float d) {
    const float r = mufu_rcp(d);
    float q = n * r;
#if OVL_TOL_DIV_NEWTON
    // n - d * q is exact in fma; where d or the quotient is 0, inf or NaN the residual is NaN and q already is
    // the answer
    const float e = __fmaf_rn(-d, q, n);
    if (e == e) q = __fmaf_rn(e, r, q);
#endif
    return q;
}

__device__ __forceinline__ float fexp(float x) { return mufu_ex2(x * OVL_TOL_LOG2E); }

__device__ __forceinline__ float flog_poly(float f, float kf) {
    float q = OVL_TOL_LQ7;
    q = __fmaf_rn(q, f, OVL_TOL_LQ6);
    q = __fmaf_rn(q, f, OVL_TOL_LQ5);
    q = __fmaf_rn(q, f, OVL_TOL_LQ4);
    q = __fmaf_rn(q, f, OVL_TOL_LQ3);
    q = __fmaf_rn(q, f, OVL_TOL_LQ2);
    q = __fmaf_rn(q, f, OVL_TOL_LQ1);
    q = __fmaf_rn(q, f, OVL_TOL_LQ0);
    const float r = __fmaf_rn(f * f, q, f);
    return __fmaf_rn(kf, OVL_TOL_LN2, r);
}

// x = 2^k * m with m in [2/3, 4/3): the bits of m, and k as 12582912 + k in float (12582912 = 1.5 * 2^23, so the
// integer add lands in the mantissa).  Returns true when x is NOT a positive normal number (zero, subnormal,
// negative, inf, NaN): one unsigned comparison of ix - 0x00800000.
// The two other integer steps are multiply-adds, which run beside the logic unit instead of on it:
// with t = ix - 0x3f2aaaab (the bits of 2/3), k = t >> 23 is the high word of t * 2^9, computed from
// ix - 0x00800000 by folding the difference of the two offsets and the 0x4b400000 into the 64-bit addend; and
// ix - (k << 23) = ix + kb * (-2^23) because 0x4b400000 << 23 is 0 modulo 2^32.
__device__ __forceinline__ bool flog_split(float x, float& m, float& kbiased) {
    const int ix = __float_as_int(x);
    const int t2 = ix - 0x00800000;
    long long wide;
    // -(0x3eaaaaab * 512) + (0x4b400000 << 32)
    asm("mad.wide.s32 %0, %1, 512, %2;" : "=l"(wide) : "r"(t2), "l"(0x4b3fff82aaaaaa00ll));
    const int kb = (int)(wide >> 32);
    int im;
    asm("mad.lo.s32 %0, %1, -8388608, %2;" : "=r"(im) : "r"(kb), "r"(ix));
    m = __int_as_float(im);
    kbiased = __int_as_float(kb);
    return (unsigned)t2 >= 0x7f000000u;
}

// log of an argument that is not a positive normal number: -inf for zero and (counted as zero) subnormals, +inf
// for +inf, NaN for negative arguments and NaN (x * inf + inf gives the last three)
__device__ __forceinline__ float flog_special(float x) {
    return fabsf(x) < 1.17549435e-38f ? -INFINITY : __fmaf_rn(x, INFINITY, INFINITY);
}

__device__ __forceinline__ float flog(float x) {
    float m, kb;
    const bool odd = flog_split(x, m, kb);
    const float kf = kb - 12582912.0f;
    float r = flog_poly(m - 1.0f, kf);
    if (odd) r = flog_special(x);
    return r;
}

// clamp that keeps NaN (fminf / fmaxf drop it)
__device__ __forceinline__ float clamp_nan(float x, float lo, float hi) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(x), "f"(lo));
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(r), "f"(hi));
    return r;
}

__device__ __forceinline__ float flog10(float x) { return flog(x) * 0.4342944819032518f; }
// sqrt.approx: relative error <= 2^-23 (one ulp); -0 gives -0, negative arguments NaN, subnormal ones zero
__device__ __forceinline__ float fsqrt(float x) { return mufu_sqrt(x); }

__device__ __forceinline__ float ftanh(float x) {
#if OVL_TOL_TANH_RATIONAL
    const float c = clamp_nan(x, -9.0f, 9.0f);
    const float zz = c * c;
    float pp = OVL_TOL_TRP4, qq = OVL_TOL_TRQ4;
    pp = __fmaf_rn(pp, zz, OVL_TOL_TRP3);
    qq = __fmaf_rn(qq, zz, OVL_TOL_TRQ3);
    pp = __fmaf_rn(pp, zz, OVL_TOL_TRP2);
    qq = __fmaf_rn(qq, zz, OVL_TOL_TRQ2);
    pp = __fmaf_rn(pp, zz, OVL_TOL_TRP1);
    qq = __fmaf_rn(qq, zz, OVL_TOL_TRQ1);
    pp = __fmaf_rn(pp, zz, OVL_TOL_TRP0);
    qq = __fmaf_rn(qq, zz, 1.0f);
    return (c * pp) * mufu_rcp(qq);
#endif
    const float z = x * x;
    float p = OVL_TOL_TP3;
    p = __fmaf_rn(p, z, OVL_TOL_TP2);
    p = __fmaf_rn(p, z, OVL_TOL_TP1);
    p = __fmaf_rn(p, z, OVL_TOL_TP0);
    const float small = __fmaf_rn(z * x, p, x);
    // 1 - 2 / (e^2x + 1) holds for either sign: e^2x = inf gives 1, e^2x = 0 gives -1
    const float e = mufu_ex2(x * (2.0f * OVL_TOL_LOG2E));
    const float big = __fmaf_rn(mufu_rcp(e + 1.0f), -2.0f, 1.0f);
    // (NaN compares false and takes `big`, which is NaN then)
    return fabsf(x) < OVL_TOL_TANH_SPLIT ? small : big;
}

// ---------------------------------------------------------------------------------------------------------
// a pair of floats
struct f2 {
    float x, y;
};

__device__ __forceinline__ f2 make2(float x, float y) {
    f2 r;
    r.x = x;
    r.y = y;
    return r;
}
__device__ __forceinline__ f2 splat(float v) { return make2(v, v); }

__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
    f2 r;
    asm("{\n\t.reg .b64 a, b, c, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\tmov.b64 c, {%6, %7};\n\t"
        "fma.rn.f32x2 d, a, b, c;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return r;
}

// The operator language's own +, - and * must round once each, like the scalar code built without contraction.  The
// assembler merges a packed multiplication and a packed addition that follows it into one packed fused
// multiply-add even when both carry an explicit rounding mode and contraction is switched off (measured: all 2^20
// random triples gave the fused result; the same when the two are spelled a * b + (-0) and a * 1 + b).  So packed
// additions and subtractions are fused multiply-adds by a 1.0 that the assembler cannot know to be 1.0 - the bits of
// 1.0f plus (number of blocks along y) - 1, and every launch of these kernels is one-dimensional: a * one + b and
// b * (-one) + a round exactly like a + b and a - b and can absorb no multiplication (checked the same way: every
// triple equal to the separately rounded result).
__device__ __forceinline__ float opaque_one() {
    unsigned g;
    asm("mov.u32 %0, %%nctaid.y;" : "=r"(g));
    return __uint_as_float(0x3f800000u + (g - 1u));
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
    f2 r;
    asm("{\n\t.reg .b64 a, b, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\tmul.rn.f32x2 d, a, b;\n\t"
        "mov.b64 {%0, %1}, d;\n\t}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ f2 add2(f2 a, f2 b) { return fma2(a, splat(opaque_one()), b); }
__device__ __forceinline__ f2 sub2(f2 a, f2 b) { return fma2(b, splat(-opaque_one()), a); }

__device__ __forceinline__ f2 fdiv(f2 n, f2 d) {
    const f2 r = make2(mufu_rcp(d.x), mufu_rcp(d.y));
    f2 q = mul2(n, r);
#if OVL_TOL_DIV_NEWTON
    const f2 e = fma2(mul2(d, splat(-1.0f)), q, n);
    const f2 c = fma2(e, r, q);
    if (e.x == e.x) q.x = c.x;
    if (e.y == e.y) q.y = c.y;
#endif
    return q;
}

__device__ __forceinline__ f2 fexp(f2 x) {
    const f2 t = mul2(x, splat(OVL_TOL_LOG2E));
    return make2(mufu_ex2(t.x), mufu_ex2(t.y));
}

__device__ __forceinline__ f2 flog(f2 x) {
    f2 m, kb;
    const bool odd_x = flog_split(x.x, m.x, kb.x);
    const bool odd_y = flog_split(x.y, m.y, kb.y);
    const f2 kf = sub2(kb, splat(12582912.0f));
    const f2 f = sub2(m, splat(1.0f));
    f2 q = splat(OVL_TOL_LQ7);
    q = fma2(q, f, splat(OVL_TOL_LQ6));
    q = fma2(q, f, splat(OVL_TOL_LQ5));
    q = fma2(q, f, splat(OVL_TOL_LQ4));
    q = fma2(q, f, splat(OVL_TOL_LQ3));
    q = fma2(q, f, splat(OVL_TOL_LQ2));
    q = fma2(q, f, splat(OVL_TOL_LQ1));
    q = fma2(q, f, splat(OVL_TOL_LQ0));
    f2 r = fma2(mul2(f, f), q, f);
    r = fma2(kf, splat(OVL_TOL_LN2), r);
    if (odd_x | odd_y) {
        if (odd_x) r.x = flog_special(x.x);
        if (odd_y) r.y = flog_special(x.y);
    }
    return r;
}

__device__ __forceinline__ f2 flog10(f2 x) { return mul2(flog(x), splat(0.4342944819032518f)); }
__device__ __forceinline__ f2 fsqrt(f2 x) { return make2(mufu_sqrt(x.x), mufu_sqrt(x.y)); }

__device__ __forceinline__ f2 ftanh(f2 x) {
#if OVL_TOL_TANH_RATIONAL
    const f2 c = make2(clamp_nan(x.x, -9.0f, 9.0f), clamp_nan(x.y, -9.0f, 9.0f));
    const f2 zz = mul2(c, c);
    f2 pp = splat(OVL_TOL_TRP4), qq = splat(OVL_TOL_TRQ4);
    pp = fma2(pp, zz, splat(OVL_TOL_TRP3));
    qq = fma2(qq, zz, splat(OVL_TOL_TRQ3));
    pp = fma2(pp, zz, splat(OVL_TOL_TRP2));
    qq = fma2(qq, zz, splat(OVL_TOL_TRQ2));
    pp = fma2(pp, zz, splat(OVL_TOL_TRP1));
    qq = fma2(qq, zz, splat(OVL_TOL_TRQ1));
    pp = fma2(pp, zz, splat(OVL_TOL_TRP0));
    qq = fma2(qq, zz, splat(1.0f));
    return mul2(mul2(c, pp), make2(mufu_rcp(qq.x), mufu_rcp(qq.y)));
#endif
    const f2 z = mul2(x, x);
    f2 p = splat(OVL_TOL_TP3);
    p = fma2(p, z, splat(OVL_TOL_TP2));
    p = fma2(p, z, splat(OVL_TOL_TP1));
    p = fma2(p, z, splat(OVL_TOL_TP0));
    const f2 small = fma2(mul2(z, x), p, x);
    const f2 t = mul2(x, splat(2.0f * OVL_TOL_LOG2E));
    const f2 s = add2(make2(mufu_ex2(t.x), mufu_ex2(t.y)), splat(1.0f));
    const f2 big = fma2(make2(mufu_rcp(s.x), mufu_rcp(s.y)), splat(-2.0f), splat(1.0f));
    return make2(fabsf(x.x) < OVL_TOL_TANH_SPLIT ? small.x : big.x, fabsf(x.y) < OVL_TOL_TANH_SPLIT ? small.y : big.y);
}

// ---- what the emitter needs beyond arithmetic: comparisons give 1.0f / 0.0f in the operand's type, as every
// comparison of the operator language does; conditions are "value != 0" per element
struct b2 {
    bool x, y;
};
__device__ __forceinline__ b2 truth(f2 v) {
    b2 r;
    r.x = v.x != 0.0f;
    r.y = v.y != 0.0f;
    return r;
}
__device__ __forceinline__ b2 both(b2 a, b2 b) {
    b2 r;
    r.x = a.x && b.x;
    r.y = a.y && b.y;
    return r;
}
__device__ __forceinline__ b2 andnot(b2 a, b2 b) {
    b2 r;
    r.x = a.x && !b.x;
    r.y = a.y && !b.y;
    return r;
}
__device__ __forceinline__ f2 pick(b2 m, f2 a, f2 b) { return make2(m.x ? a.x : b.x, m.y ? a.y : b.y); }

#define OVL_TOL_CMP(name, op)                                                                  \
    __device__ __forceinline__ f2 name(f2 a, f2 b) {                                           \
        return make2((a.x op b.x) ? 1.0f : 0.0f, (a.y op b.y) ? 1.0f : 0.0f);                  \
    }
OVL_TOL_CMP(eq2, ==)
OVL_TOL_CMP(ne2, !=)
OVL_TOL_CMP(lt2, <)
OVL_TOL_CMP(le2, <=)
OVL_TOL_CMP(gt2, >)
OVL_TOL_CMP(ge2, >=)
#undef OVL_TOL_CMP
__device__ __forceinline__ f2 and2(f2 a, f2 b) {
    return make2((a.x != 0.0f && b.x != 0.0f) ? 1.0f : 0.0f, (a.y != 0.0f && b.y != 0.0f) ? 1.0f : 0.0f);
}
__device__ __forceinline__ f2 or2(f2 a, f2 b) {
    return make2((a.x != 0.0f || b.x != 0.0f) ? 1.0f : 0.0f, (a.y != 0.0f || b.y != 0.0f) ? 1.0f : 0.0f);
}
__device__ __forceinline__ f2 not2(f2 a) { return make2(a.x == 0.0f ? 1.0f : 0.0f, a.y == 0.0f ? 1.0f : 0.0f); }
__device__ __forceinline__ f2 min2(f2 a, f2 b) { return make2(a.x < b.x ? a.x : b.x, a.y < b.y ? a.y : b.y); }
__device__ __forceinline__ f2 max2(f2 a, f2 b) { return make2(a.x > b.x ? a.x : b.x, a.y > b.y ? a.y : b.y); }
__device__ __forceinline__ f2 neg2(f2 a) { return make2(-a.x, -a.y); }
__device__ __forceinline__ f2 abs2(f2 a) { return make2(fabsf(a.x), fabsf(a.y)); }
// isinf(a) && a > 0 in one comparison
__device__ __forceinline__ f2 isposinf2(f2 a) {
    return make2(a.x == INFINITY ? 1.0f : 0.0f, a.y == INFINITY ? 1.0f : 0.0f);
}
__device__ __forceinline__ f2 isinf2(f2 a) { return make2(isinf(a.x) ? 1.0f : 0.0f, isinf(a.y) ? 1.0f : 0.0f); }
__device__ __forceinline__ f2 isnan2(f2 a) { return make2(isnan(a.x) ? 1.0f : 0.0f, isnan(a.y) ? 1.0f : 0.0f); }
__device__ __forceinline__ f2 isfinite2(f2 a) {
    return make2(isfinite(a.x) ? 1.0f : 0.0f, isfinite(a.y) ? 1.0f : 0.0f);
}

}  // namespace tol
}  // namespace ovl
