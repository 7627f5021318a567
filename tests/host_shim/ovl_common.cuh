// TEST INFRASTRUCTURE: stands in for csrc/templates/ovl_common.cuh when a generated kernel is compiled for the HOST,
// so that the statement-level output of the code generator (bodies, hoisted vector accesses, packed pairs, masks)
// can be executed and compared with the CPU oracle on a machine without a GPU.  Never part of the product path.
#pragma once
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <cfloat>
#include <cmath>

struct ovl_host_dim3 {
    unsigned x, y, z;
};
extern thread_local ovl_host_dim3 blockIdx, threadIdx, gridDim, blockDim;

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __restrict__
#define __launch_bounds__(...)

using std::isfinite;
using std::isinf;
using std::isnan;

static inline float __fmaf_rn(float a, float b, float c) { return fmaf(a, b, c); }
static inline float __int_as_float(int v) { float f; memcpy(&f, &v, 4); return f; }
static inline int __float_as_int(float f) { int v; memcpy(&v, &f, 4); return v; }
static inline float __uint_as_float(unsigned v) { float f; memcpy(&f, &v, 4); return f; }

namespace ovl {

inline int8_t abs_8(const int8_t x) { return (x < 0) ? -x : x; }
inline int16_t abs_16(const int16_t x) { return (x < 0) ? -x : x; }

template <typename T, int N>
struct Vec {
    T v[N];
};
template <typename T, int N>
inline Vec<T, N> load_vec(const T* p) {
    Vec<T, N> r;
    memcpy(&r, p, sizeof(r));
    return r;
}
template <typename T, int N>
inline void store_vec(T* p, const Vec<T, N>& v) {
    memcpy(p, &v, sizeof(v));
}

}  // namespace ovl
