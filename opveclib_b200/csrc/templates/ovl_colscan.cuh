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
//
// When the tensor has enough columns, one launch does it (`col_walk`): the columns are cut into strips of C
// neighbouring columns, and one thread block walks down ALL rows of its strip, tile after tile, with the strip's
// running totals in registers - no block ever needs anything from another block, every element is read once and
// written once.  Inside a block the rows of a tile are split over the warps (and, for narrow strips, over groups of
// lanes), combined through shuffles and a few words of shared memory; the loads of the next tile are in flight
// while the current one is scanned.
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

// ---------------------------------------------------------------------------------------------------------
// One block per strip of C columns (C a power of two, 4..32).  A warp's 32 lanes are G = 32 / C groups of C lanes:
// lane = g * C + c owns column c of the strip and, per tile, the U consecutive rows of row-worker (warp * G + g).
// A tile is WARPS * G * U rows.  Per tile: every lane totals its U rows, the totals are scanned across the groups of
// the warp (shuffles) and across the warps (shared memory, double-buffered so that one barrier per tile is enough),
// which gives every lane the value in front of its first row; it then writes its U running values.
template <typename T, typename Acc, class Op, int C, int WARPS, int U>
__device__ __forceinline__ void col_walk(const T* __restrict__ in, T* __restrict__ out, const uint64_t outer, const uint64_t n,
                                         const uint64_t inner) {
    constexpr int G = 32 / C;
    constexpr int TILE_ROWS = WARPS * G * U;
    __shared__ Acc s_tot[2][WARPS][C];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = lane % C, g = lane / C;
    const uint64_t strips_per = (inner + C - 1) / C;
    const uint64_t strips = outer * strips_per;
    for (uint64_t strip = blockIdx.x; strip < strips; strip += gridDim.x) {
        const uint64_t o = strip / strips_per;
        const uint64_t col = (strip - o * strips_per) * C + c;
        const bool live = col < inner;
        const T* src = in + o * n * inner + col;
        T* dst = out + o * n * inner + col;
        const uint64_t my_row = (uint64_t)(warp * G + g) * U;       // first row of this lane inside a tile
        Acc carry = Op::template identity<Acc>();                   // everything above the current tile, this column
        T next[U];
        auto fetch = [&](uint64_t row0) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint64_t r = row0 + my_row + u;
                next[u] = (live && r < n) ? src[r * inner] : (T)Op::template identity<Acc>();
            }
        };
        fetch(0);
        int buf = 0;
        for (uint64_t row0 = 0; row0 < n; row0 += TILE_ROWS, buf ^= 1) {
            T cur[U];
#pragma unroll
            for (int u = 0; u < U; ++u) cur[u] = next[u];
            if (row0 + TILE_ROWS < n) fetch(row0 + TILE_ROWS);      // the next tile travels while this one is scanned
            Acc part = Op::template identity<Acc>();
#pragma unroll
            for (int u = 0; u < U; ++u) part = Op::apply(part, (Acc)cur[u]);
            // inclusive scan of the groups' totals inside the warp (same column: lanes C apart)
            Acc incl = part;
#pragma unroll
            for (int d = C; d < 32; d <<= 1) {
                const Acc y = shfl_up_any(incl, d);
                if (lane >= d) incl = Op::apply(y, incl);
            }
            if (g == G - 1) s_tot[buf][warp][c] = incl;             // the warp's total for column c
            __syncthreads();
            Acc seed = carry, all = carry;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const Acc t = s_tot[buf][w][c];
                if (w < warp) seed = Op::apply(seed, t);
                all = Op::apply(all, t);
            }
            carry = all;
            // what lies in front of this lane's rows: the earlier warps, then the earlier groups of this warp
            Acc before = shfl_up_any(incl, C);
            if (g == 0) before = Op::template identity<Acc>();
            Acc run = Op::apply(seed, before);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                run = Op::apply(run, (Acc)cur[u]);
                const uint64_t r = row0 + my_row + u;
                if (live && r < n) dst[r * inner] = (T)run;
            }
        }
        __syncthreads();       // (the next strip starts with buffer 0 again)
    }
}

}  // namespace ovl
