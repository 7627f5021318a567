// Common device helpers shared by every generated kernel (sm_100a).
#pragma once
#include <stdint.h>
#include <cfloat>

namespace ovl {

// integer absolute values for types narrower than int, with the meaning of the reference's helpers
// (opveclib/expression.py:599-600)
__device__ __forceinline__ int8_t abs_8(const int8_t x) { return (x < 0) ? -x : x; }
__device__ __forceinline__ int16_t abs_16(const int16_t x) { return (x < 0) ? -x : x; }

// N consecutive elements moved with one memory instruction (16 bytes when sizeof(T) * N == 16)
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
    T v[N];
};

template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_vec(const T* __restrict__ p) {
    return *reinterpret_cast<const Vec<T, N>*>(p);
}

// streaming variant: read-only path, do not keep the line in L1
template <int N>
__device__ __forceinline__ Vec<float, N> load_vec_stream(const float* __restrict__ p);

template <>
__device__ __forceinline__ Vec<float, 4> load_vec_stream<4>(const float* __restrict__ p) {
    Vec<float, 4> r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3])
                 : "l"(p));
    return r;
}

template <typename T, int N>
__device__ __forceinline__ void store_vec(T* __restrict__ p, const Vec<T, N>& v) {
    *reinterpret_cast<Vec<T, N>*>(p) = v;
}

// Asynchronous copy of one vector (BYTES = 4, 8 or 16) from global to shared memory, and the group fence.
template <int BYTES>
__device__ __forceinline__ void cp_async_vec(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(d), "l"(gmem_src), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

}  // namespace ovl
