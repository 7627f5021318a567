// TEST INFRASTRUCTURE: host stand-in for csrc/templates/ovl_fastmath.cuh (see ovl_common.cuh beside it).  The pair
// type and its operations with the meaning the device versions have: +, -, * rounded once each, comparisons giving
// 1.0f / 0.0f, selects per element.  Division and the three functions use the host's libm here - what is under test
// on the host is the code generator's use of these operations, not their device implementation.
#pragma once
#include "ovl_common.cuh"

namespace ovl {
namespace tol {

inline float fdiv(float n, float d) { return n / d; }
inline float fexp(float x) { return expf(x); }
inline float flog(float x) { return logf(x); }
inline float ftanh(float x) { return tanhf(x); }
inline float flog10(float x) { return log10f(x); }
inline float fsqrt(float x) { return sqrtf(x); }

struct f2 {
    float x, y;
};
struct b2 {
    bool x, y;
};
inline f2 make2(float x, float y) { f2 r; r.x = x; r.y = y; return r; }
inline f2 splat(float v) { return make2(v, v); }
inline f2 add2(f2 a, f2 b) { volatile float x = a.x + b.x, y = a.y + b.y; return make2(x, y); }
inline f2 sub2(f2 a, f2 b) { volatile float x = a.x - b.x, y = a.y - b.y; return make2(x, y); }
inline f2 mul2(f2 a, f2 b) { volatile float x = a.x * b.x, y = a.y * b.y; return make2(x, y); }
inline f2 fma2(f2 a, f2 b, f2 c) { return make2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y)); }
inline f2 fdiv(f2 n, f2 d) { return make2(n.x / d.x, n.y / d.y); }
inline f2 fexp(f2 x) { return make2(expf(x.x), expf(x.y)); }
inline f2 flog(f2 x) { return make2(logf(x.x), logf(x.y)); }
inline f2 ftanh(f2 x) { return make2(tanhf(x.x), tanhf(x.y)); }
inline f2 flog10(f2 x) { return make2(log10f(x.x), log10f(x.y)); }
inline f2 fsqrt(f2 x) { return make2(sqrtf(x.x), sqrtf(x.y)); }
inline b2 truth(f2 v) { b2 r; r.x = v.x != 0.0f; r.y = v.y != 0.0f; return r; }
inline b2 both(b2 a, b2 b) { b2 r; r.x = a.x && b.x; r.y = a.y && b.y; return r; }
inline b2 andnot(b2 a, b2 b) { b2 r; r.x = a.x && !b.x; r.y = a.y && !b.y; return r; }
inline f2 pick(b2 m, f2 a, f2 b) { return make2(m.x ? a.x : b.x, m.y ? a.y : b.y); }
#define OVL_HOST_CMP(name, op) \
    inline f2 name(f2 a, f2 b) { return make2((a.x op b.x) ? 1.0f : 0.0f, (a.y op b.y) ? 1.0f : 0.0f); }
OVL_HOST_CMP(eq2, ==)
OVL_HOST_CMP(ne2, !=)
OVL_HOST_CMP(lt2, <)
OVL_HOST_CMP(le2, <=)
OVL_HOST_CMP(gt2, >)
OVL_HOST_CMP(ge2, >=)
#undef OVL_HOST_CMP
inline f2 and2(f2 a, f2 b) { return make2((a.x != 0.0f && b.x != 0.0f) ? 1.0f : 0.0f, (a.y != 0.0f && b.y != 0.0f) ? 1.0f : 0.0f); }
inline f2 or2(f2 a, f2 b) { return make2((a.x != 0.0f || b.x != 0.0f) ? 1.0f : 0.0f, (a.y != 0.0f || b.y != 0.0f) ? 1.0f : 0.0f); }
inline f2 not2(f2 a) { return make2(a.x == 0.0f ? 1.0f : 0.0f, a.y == 0.0f ? 1.0f : 0.0f); }
inline f2 min2(f2 a, f2 b) { return make2(a.x < b.x ? a.x : b.x, a.y < b.y ? a.y : b.y); }
inline f2 max2(f2 a, f2 b) { return make2(a.x > b.x ? a.x : b.x, a.y > b.y ? a.y : b.y); }
inline f2 neg2(f2 a) { return make2(-a.x, -a.y); }
inline f2 abs2(f2 a) { return make2(fabsf(a.x), fabsf(a.y)); }
inline f2 isposinf2(f2 a) { return make2(a.x == INFINITY ? 1.0f : 0.0f, a.y == INFINITY ? 1.0f : 0.0f); }
inline f2 isinf2(f2 a) { return make2(std::isinf(a.x) ? 1.0f : 0.0f, std::isinf(a.y) ? 1.0f : 0.0f); }
inline f2 isnan2(f2 a) { return make2(std::isnan(a.x) ? 1.0f : 0.0f, std::isnan(a.y) ? 1.0f : 0.0f); }
inline f2 isfinite2(f2 a) { return make2(std::isfinite(a.x) ? 1.0f : 0.0f, std::isfinite(a.y) ? 1.0f : 0.0f); }

}  // namespace tol
}  // namespace ovl
