// Inclusive scan along an axis that is NOT the contiguous one (sm_100a).
//
// The operator language scans along any axis with one worker per line (opveclib/examples/test_accumulate.py:22-78;
// the reference's own timing harness scans fp64 [10000, 1000] along axis 0,
// opveclib/examples/test_perf_accumulate.py:35-48).  Seen as [outer, n, inner] with the scan along n and inner > 1,
// neighbouring lines are neighbouring columns, so a warp that walks down the rows of a strip of columns reads and
// writes whole contiguous row segments.  The rows are cut into chunks so that there are enough (chunk, strip)
// tiles to fill the device; three streaming passes, none of which waits for another block:
//   col_aggregates   every tile: the per-column totals of its rows                       -> agg[outer][chunk][inner]
//   col_prefixes     every column: exclusive scan of its chunk totals, in place           (tiny)
//   col_scan         every tile: running values seeded with the chunk's prefix, rounded on store
// Accumulation is in Acc (double for floating-point data), as in the scans along the contiguous axis.
#pragma once
#include "ovl_scan.cuh"

namespace ovl {

constexpr int kColBlock = 256;        // threads per block: 8 warps, one tile each
constexpr int kColRows = 64;          // rows per chunk

__host__ __device__ constexpr uint64_t col_chunks(uint64_t n) { return (n + kColRows - 1) / kColRows; }

// One warp per tile; lane L owns columns strip * 32 * VEC + L * VEC .. + VEC - 1.  VEC > 1 needs inner % VEC == 0
// and 16-byte aligned base pointers (then every row segment is aligned).
template <typename T, typename Acc, class Op, int VEC, bool WRITE>
__device__ __forceinline__ void col_tiles(const T* __restrict__ in, T* __restrict__ out, Acc* __restrict__ agg, const uint64_t outer,
                                          const uint64_t n, const uint64_t inner) {
    const uint64_t chunks = col_chunks(n);
    const uint64_t strips = (inner + 32 * VEC - 1) / (32 * VEC);
    const uint64_t tiles = outer * chunks * strips;
    const int lane = threadIdx.x & 31;
    const uint64_t warps = (uint64_t)gridDim.x * (kColBlock / 32);
    for (uint64_t tile = (uint64_t)blockIdx.x * (kColBlock / 32) + (threadIdx.x >> 5); tile < tiles; tile += warps) {
        const uint64_t strip = tile % strips;
        const uint64_t chunk = (tile / strips) % chunks;
        const uint64_t o = tile / (strips * chunks);
        const uint64_t col = strip * 32 * VEC + (uint64_t)lane * VEC;
        if (col >= inner) continue;
        const uint64_t row0 = chunk * kColRows;
        const uint64_t rows = (n - row0 < (uint64_t)kColRows) ? n - row0 : (uint64_t)kColRows;
        const T* src = in + (o * n + row0) * inner + col;
        Acc* a = agg + (o * chunks + chunk) * inner + col;
        Acc run[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) run[e] = WRITE ? a[e] : Op::template identity<Acc>();
        T* dst = WRITE ? out + (o * n + row0) * inner + col : nullptr;
        uint64_t r = 0;
        // eight rows in flight
        for (; r + 8 <= rows; r += 8) {
            Vec<T, VEC> v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = load_vec<T, VEC>(src + (r + u) * inner);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                Vec<T, VEC> w;
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    run[e] = Op::apply(run[e], (Acc)v[u].v[e]);
                    w.v[e] = (T)run[e];
                }
                if (WRITE) store_vec<T, VEC>(dst + (r + u) * inner, w);
            }
        }
        for (; r < rows; ++r) {
            const Vec<T, VEC> v = load_vec<T, VEC>(src + r * inner);
            Vec<T, VEC> w;
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                run[e] = Op::apply(run[e], (Acc)v.v[e]);
                w.v[e] = (T)run[e];
            }
            if (WRITE) store_vec<T, VEC>(dst + r * inner, w);
        }
        if (!WRITE) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) a[e] = run[e];
        }
    }
}

// agg[o][chunk][col] becomes the reduction of the chunks before `chunk` in the same column (exclusive scan along
// the chunks).  One warp per column: lane L owns a contiguous run of the column's chunks, scans it locally, and the
// lane totals are scanned across the warp, so a column costs two trips to memory whatever its length.
template <typename Acc, class Op>
__device__ __forceinline__ void col_prefixes(Acc* __restrict__ agg, const uint64_t outer, const uint64_t n, const uint64_t inner) {
    constexpr int PER = 8;                      // chunks per lane and round
    const uint64_t chunks = col_chunks(n);
    const uint64_t columns = outer * inner;
    const int lane = threadIdx.x & 31;
    const uint64_t warps = (uint64_t)gridDim.x * (kColBlock / 32);
    for (uint64_t c = (uint64_t)blockIdx.x * (kColBlock / 32) + (threadIdx.x >> 5); c < columns; c += warps) {
        const uint64_t o = c / inner, col = c - o * inner;
        Acc* a = agg + o * chunks * inner + col;
        Acc carry = Op::template identity<Acc>();
        for (uint64_t k0 = 0; k0 < chunks; k0 += 32 * PER) {
            const uint64_t mine = k0 + (uint64_t)lane * PER;
            Acc v[PER];
#pragma unroll
            for (int i = 0; i < PER; ++i) v[i] = (mine + i < chunks) ? a[(mine + i) * inner] : Op::template identity<Acc>();
            Acc t = v[0];
#pragma unroll
            for (int i = 1; i < PER; ++i) t = Op::apply(t, v[i]);
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const Acc y = shfl_up_any(t, d);
                if (lane >= d) t = Op::apply(y, t);
            }
            Acc run = shfl_up_any(t, 1);
            if (lane == 0) run = Op::template identity<Acc>();
            run = Op::apply(carry, run);
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                if (mine + i < chunks) a[(mine + i) * inner] = run;
                run = Op::apply(run, v[i]);
            }
            carry = Op::apply(carry, shfl_any(t, 31));
        }
    }
}

}  // namespace ovl
