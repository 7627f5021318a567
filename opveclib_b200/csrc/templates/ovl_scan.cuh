// Cooperative inclusive scan along contiguous lines: single pass, decoupled look-back (sm_100a).
//
// The operator language expresses a scan as one worker walking a whole line serially
// (opveclib/examples/test_accumulate.py:22-78).  Here a line of n elements is cut into tiles of
// BLOCK * VPT * VEC elements; thread blocks scan their tile in registers (serial scan inside each 128-bit
// vector, warp-shuffle scan across lanes, shared-memory scan across warps).  Lines that fit one tile need nothing
// else.  For longer lines every block publishes its tile aggregate and
// obtains the prefix of everything to their left in the same line by looking back over the descriptors of
// earlier tiles: aggregates are summed until a tile that already knows its inclusive prefix is met; several
// warps inspect consecutive windows of 32 descriptors at once, because the rate at which prefixes can travel
// along the line is (tiles inspected per round) / (one L2 round trip).  Every element is read once and
// written once.
//
// Accumulation runs in the wider type Acc (double for fp32 data), so results do not depend on how the line was
// cut and are the correctly rounded exact scan rather than a re-association of fp32 partial sums.
//
// Every wait on another block is bounded: when the bound expires the block records OVL_ERR_TIMEOUT in the status
// word at the start of the scratch buffer and carries on with the identity as prefix; the host reports the
// error after the launch.  Nothing traps.
#pragma once
#include "ovl_common.cuh"

namespace ovl {

constexpr int kScanBlock = 512;          // threads per block when a line fits one tile (no look-back)
constexpr int kScanBlockLookback = 256;  // threads per block for longer lines: more blocks per SM hide look-back waits
constexpr int kScanVpt = 4;              // 128-bit vectors per thread
constexpr int kScanLookbackWarps = 8;    // look-back windows (of 32 tiles each) inspected in parallel
constexpr uint32_t kScanSpinLimit = 1u << 22;
constexpr int32_t kErrTimeout = 8;  // OVL_ERR_TIMEOUT
constexpr int kScanOneTile = 0, kScanLookback = 1, kScanPrefixed = 2;

template <typename A> struct IsDouble { static constexpr bool value = false; };
template <> struct IsDouble<double> { static constexpr bool value = true; };
#define OVL_IS_DOUBLE(A) (ovl::IsDouble<A>::value)

struct OpAdd {
    template <typename A> static __device__ __forceinline__ A identity() { return A(0); }
    template <typename A> static __device__ __forceinline__ A apply(A a, A b) { return a + b; }
};
struct OpMul {
    template <typename A> static __device__ __forceinline__ A identity() { return A(1); }
    template <typename A> static __device__ __forceinline__ A apply(A a, A b) { return a * b; }
};

// scratch layout: header, then one descriptor per tile
struct ScanHeader {
    int32_t status;         // 0, or an error code set by a block whose wait expired
    uint32_t reserved;
    uint32_t pad[2];
};
template <typename Acc>
struct alignas(16) TileDesc {
    Acc aggregate;   // reduction of the tile alone            (valid when flag >= 1)
    Acc prefix;      // reduction of the line up to tile's end (valid when flag == 2)
    uint32_t flag;   // 0 empty, 1 aggregate published, 2 inclusive prefix published
    uint32_t pad;
};

template <typename Acc>
__host__ __device__ constexpr uint64_t scan_scratch_bytes(uint64_t total_tiles) {
    return sizeof(ScanHeader) + total_tiles * sizeof(TileDesc<Acc>);
}

__device__ __forceinline__ uint32_t ld_flag(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_flag(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <typename A>
__device__ __forceinline__ A shfl_up_any(A v, int delta) {
    if constexpr (sizeof(A) == 8 && !OVL_IS_DOUBLE(A)) {
        long long x = *reinterpret_cast<long long*>(&v);
        x = __shfl_up_sync(0xffffffffu, x, delta);
        return *reinterpret_cast<A*>(&x);
    } else {
        return __shfl_up_sync(0xffffffffu, v, delta);
    }
}
template <typename A>
__device__ __forceinline__ A shfl_down_any(A v, int delta) {
    if constexpr (sizeof(A) == 8 && !OVL_IS_DOUBLE(A)) {
        long long x = *reinterpret_cast<long long*>(&v);
        x = __shfl_down_sync(0xffffffffu, x, delta);
        return *reinterpret_cast<A*>(&x);
    } else {
        return __shfl_down_sync(0xffffffffu, v, delta);
    }
}
template <typename A>
__device__ __forceinline__ A shfl_any(A v, int lane) {
    if constexpr (sizeof(A) == 8 && !OVL_IS_DOUBLE(A)) {
        long long x = *reinterpret_cast<long long*>(&v);
        x = __shfl_sync(0xffffffffu, x, lane);
        return *reinterpret_cast<A*>(&x);
    } else {
        return __shfl_sync(0xffffffffu, v, lane);
    }
}

template <typename A>
__device__ __forceinline__ A shfl_xor_any(A v, int mask) {
    if constexpr (sizeof(A) == 8 && !OVL_IS_DOUBLE(A)) {
        long long x = *reinterpret_cast<long long*>(&v);
        x = __shfl_xor_sync(0xffffffffu, x, mask);
        return *reinterpret_cast<A*>(&x);
    } else {
        return __shfl_xor_sync(0xffffffffu, v, mask);
    }
}

// Tile data of one thread: VPT vectors of VEC elements, warp-striped (lane L owns vector j at
// warp_off + (j*32 + L) * VEC).  Elements past the end of the line hold the identity.
//
// stage_tile starts bringing a tile into the thread's own slots of the shared staging buffer (asynchronous copies
// for whole vectors when ALIGNED, plain loads otherwise); fetch_tile waits for the thread's own copies and moves
// the slots into registers.  Slots are private to a thread, so no block-wide barrier is involved.
template <typename T, class Op, int VEC, int VPT, int BLOCK, bool ALIGNED>
__device__ __forceinline__ void stage_tile(const T* __restrict__ in, uint64_t line_base, uint64_t warp_off, uint64_t n, int lane,
                                           Vec<T, VEC> (*stage)[BLOCK]) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const uint64_t off = warp_off + (uint64_t)(j * 32 + lane) * VEC;
        if (ALIGNED && off + VEC <= n) {
            cp_async_vec<(int)(sizeof(T) * VEC)>(&stage[j][threadIdx.x], in + line_base + off);
        } else {
            Vec<T, VEC> v;
#pragma unroll
            for (int e = 0; e < VEC; ++e) v.v[e] = (off + e < n) ? in[line_base + off + e] : Op::template identity<T>();
            stage[j][threadIdx.x] = v;
        }
    }
    cp_async_commit();
}

template <typename T, int VEC, int VPT, int BLOCK>
__device__ __forceinline__ void fetch_tile(Vec<T, VEC> (*stage)[BLOCK], T (&raw)[VPT][VEC]) {
    cp_async_wait_all();
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const Vec<T, VEC> v = stage[j][threadIdx.x];
#pragma unroll
        for (int e = 0; e < VEC; ++e) raw[j][e] = v.v[e];
    }
}

// One launch scans `lines` lines of `n` elements.
//  ALIGNED    every line start is VEC-aligned (n % VEC == 0 or a single line) and the base pointers are 16-byte
//             aligned, so whole vectors move with one instruction.
//  MODE       kScanOneTile: every line fits one tile; nothing is published, no block waits for another.
//             kScanPrefixed: lines are cut into several tiles and the prefix in front of every tile is already
//             known (array of Acc after the scratch header, written by tile_aggregates + scan_aggregates); again
//             no block waits for another.
//             kScanLookback: several tiles per line, single pass: prefixes travel from tile to tile through
//             descriptors (decoupled look-back); blocks wait for the aggregates of earlier tiles, so the whole
//             grid must be resident (cooperative launch).
// Tiles are handed out statically (blockIdx, blockIdx + gridDim, ...).  While a block works on one tile, the data of its next tile is already on its way into shared memory
// (cp.async), so global loads overlap the scan, the look-back and the stores of the current tile.
template <typename T, typename Acc, class Op, int VEC, bool ALIGNED, bool HAS_CARRY, int MODE>
__device__ __forceinline__ void scan_lines(const T* __restrict__ in, T* __restrict__ out, const Acc* __restrict__ carry,
                                           const uint64_t lines, const uint64_t n, void* scratch) {
    constexpr bool LOOKBACK = MODE == kScanLookback;
    constexpr bool PREFIXED = MODE == kScanPrefixed;
    constexpr int BLOCK = LOOKBACK ? kScanBlockLookback : kScanBlock;
    constexpr int VPT = kScanVpt;
    constexpr int WARPS = BLOCK / 32;
    constexpr int LBW = kScanLookbackWarps;
    constexpr uint32_t TILE = BLOCK * VPT * VEC;
    constexpr uint32_t WARP_ELEMS = 32 * VPT * VEC;

    ScanHeader* hdr = reinterpret_cast<ScanHeader*>(scratch);
    TileDesc<Acc>* desc = reinterpret_cast<TileDesc<Acc>*>(hdr + 1);
    const Acc* tile_prefix = reinterpret_cast<const Acc*>(hdr + 1);
    const uint64_t tiles_per_line = (LOOKBACK || PREFIXED) ? (n + TILE - 1) / TILE : 1;
    const uint64_t total_tiles = tiles_per_line * lines;

    __shared__ Vec<T, VEC> s_stage[VPT][BLOCK];   // staging slots, [j][thread]
    __shared__ Acc s_warp_total[2][WARPS];        // double buffered by iteration parity
    __shared__ Acc s_win_sum[LBW];
    __shared__ int s_win_found[LBW];

    const int lane = threadIdx.x & 31;
    const int wid = threadIdx.x >> 5;
    int parity = 0;

    // ---- tiles are handed out statically: blockIdx, blockIdx + gridDim, ...  The sequence is known in advance,
    // so the next tile is staged while the current one is processed.  With look-back, a tile waits for the
    // aggregates of the tiles before it, which other blocks are working on at the same moment: every block of
    // the grid must be resident (the launcher starts look-back kernels as cooperative launches with
    // grid <= resident blocks), and blocks then advance in step, tile t-1 being published about when tile t
    // needs it.
    uint64_t tile = blockIdx.x;
    if (tile < total_tiles) {
        const uint64_t line = tile / tiles_per_line;
        stage_tile<T, Op, VEC, VPT, BLOCK, ALIGNED>(in, line * n, (tile - line * tiles_per_line) * TILE + (uint64_t)wid * WARP_ELEMS,
                                                    n, lane, s_stage);
    }

    while (tile < total_tiles) {
        const uint64_t line = tile / tiles_per_line;
        const uint64_t tile_in_line = tile - line * tiles_per_line;
        const uint64_t line_base = line * n;
        const uint64_t warp_off = tile_in_line * TILE + (uint64_t)wid * WARP_ELEMS;

        T raw[VPT][VEC];
        fetch_tile<T, VEC, VPT, BLOCK>(s_stage, raw);

        const uint64_t next = tile + gridDim.x;
        if (next < total_tiles) {
            const uint64_t nline = next / tiles_per_line;
            stage_tile<T, Op, VEC, VPT, BLOCK, ALIGNED>(in, nline * n,
                                                        (next - nline * tiles_per_line) * TILE + (uint64_t)wid * WARP_ELEMS, n, lane,
                                                        s_stage);
        }

        // ---- pass 1: totals of each vector, scanned across the warp; base[j] = prefix in front of vector j
        Acc base[VPT];
        Acc run = Op::template identity<Acc>();
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            Acc t = (Acc)raw[j][0];
#pragma unroll
            for (int e = 1; e < VEC; ++e) t = Op::apply(t, (Acc)raw[j][e]);
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const Acc y = shfl_up_any(t, d);
                if (lane >= d) t = Op::apply(y, t);
            }
            Acc excl = shfl_up_any(t, 1);
            if (lane == 0) excl = Op::template identity<Acc>();
            base[j] = Op::apply(run, excl);
            run = Op::apply(run, shfl_any(t, 31));
        }
        if (lane == 0) s_warp_total[parity][wid] = run;
        __syncthreads();

        // ---- prefix of the warps to the left inside the tile, and the tile aggregate
        Acc warp_excl = Op::template identity<Acc>();
        Acc aggregate = Op::template identity<Acc>();
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const Acc v = s_warp_total[parity][w];
            if (w < wid) warp_excl = Op::apply(warp_excl, v);
            aggregate = Op::apply(aggregate, v);
        }
        parity ^= 1;

        // ---- prefix of the tiles to the left inside the line
        Acc exclusive = Op::template identity<Acc>();
        if (PREFIXED) {
            exclusive = tile_prefix[tile];      // carry already folded in by scan_aggregates
        } else if (tile_in_line == 0) {
            if (HAS_CARRY) exclusive = *carry;
            if (LOOKBACK && threadIdx.x == 0) {
                desc[tile].prefix = Op::apply(exclusive, aggregate);
                st_flag(&desc[tile].flag, 2u);
            }
        } else if (LOOKBACK) {
            // decoupled look-back: LBW warps inspect LBW consecutive windows of 32 earlier tiles at once
            if (threadIdx.x == 0) {
                desc[tile].aggregate = aggregate;
                st_flag(&desc[tile].flag, 1u);
            }
            const int64_t first = (int64_t)(tile - tile_in_line);   // first tile of this line
            int64_t wbase = (int64_t)tile - 1;                      // nearest tile of window 0
            bool done = false;
            while (!done) {
                if (wid < LBW) {
                    const int64_t mine = wbase - 32 * wid - lane;
                    uint32_t flag = 2u;                              // left of the line start: nothing to add
                    Acc val = Op::template identity<Acc>();
                    if (mine >= first) {
                        uint32_t spins = 0;
                        flag = ld_flag(&desc[mine].flag);
                        while (flag == 0u && spins < kScanSpinLimit) {
                            if (spins > 8) __nanosleep(32);
                            flag = ld_flag(&desc[mine].flag);
                            ++spins;
                        }
                        if (flag == 0u) {
                            atomicExch(&hdr->status, kErrTimeout);
                            flag = 2u;                               // give up: behave as if the line started here
                        } else {
                            val = (flag == 2u) ? *(volatile Acc*)&desc[mine].prefix : *(volatile Acc*)&desc[mine].aggregate;
                        }
                    }
                    // the nearest lane holding an inclusive prefix ends this window
                    const uint32_t has_prefix = __ballot_sync(0xffffffffu, flag == 2u);
                    const int stop = __ffs(has_prefix) - 1;
                    const int last = (stop >= 0) ? stop : 31;
                    // combine left to right: lane `last` (farthest) ... lane 0 (nearest); an order-preserving tree:
                    // after step d lane k holds v[k+2d-1] (+) ... (+) v[k]
                    Acc window = (lane <= last) ? val : Op::template identity<Acc>();
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const Acc far = shfl_down_any(window, d);
                        if (lane + d < 32) window = Op::apply(far, window);
                    }
                    if (lane == 0) {
                        s_win_sum[wid] = window;
                        s_win_found[wid] = (stop >= 0) ? 1 : 0;
                    }
                }
                __syncthreads();
#pragma unroll
                for (int w = 0; w < LBW; ++w) {
                    if (!done) {
                        exclusive = Op::apply(s_win_sum[w], exclusive);
                        if (s_win_found[w]) done = true;
                    }
                }
                wbase -= 32 * LBW;
                if (!done) __syncthreads();     // the window slots are rewritten in the next round
            }
            if (threadIdx.x == 0) {
                desc[tile].prefix = Op::apply(exclusive, aggregate);
                st_flag(&desc[tile].flag, 2u);
            }
        }
        const Acc offset = Op::apply(exclusive, warp_excl);

        // ---- pass 2: running values, rounded to T on store
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const uint64_t off = warp_off + (uint64_t)(j * 32 + lane) * VEC;
            Acc p = Op::apply(offset, base[j]);
            if (ALIGNED && off + VEC <= n) {
                Vec<T, VEC> v;
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    p = Op::apply(p, (Acc)raw[j][e]);
                    v.v[e] = (T)p;
                }
                store_vec<T, VEC>(out + line_base + off, v);
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    p = Op::apply(p, (Acc)raw[j][e]);
                    if (off + e < n) out[line_base + off + e] = (T)p;
                }
            }
        }
        tile = next;
    }
    cp_async_wait_all();
}

// ---------------------------------------------------------------------------------------------------------
// Scan in three passes for lines of several tiles, with no waiting between blocks:
//   tile_aggregates   reads every tile once and writes its reduction (Acc) to agg[tile]            4 B/elem
//   scan_aggregates   turns agg[] into the exclusive prefix in front of every tile, per line      (tiny)
//   scan_lines<kScanPrefixed>  scans every tile seeded with its prefix                              8 B/elem
// Twelve bytes per element instead of the single pass's eight, but every pass streams at copy speed, which on
// this device beats handing prefixes from block to block through L2.
template <typename T, typename Acc, class Op, int VEC, bool ALIGNED>
__device__ __forceinline__ void tile_aggregates(const T* __restrict__ in, const uint64_t lines, const uint64_t n,
                                                Acc* __restrict__ agg) {
    constexpr int BLOCK = kScanBlock;
    constexpr int VPT = kScanVpt;
    constexpr int WARPS = BLOCK / 32;
    constexpr uint32_t TILE = BLOCK * VPT * VEC;
    constexpr uint32_t WARP_ELEMS = 32 * VPT * VEC;
    __shared__ Vec<T, VEC> s_stage[VPT][BLOCK];
    __shared__ Acc s_part[2][WARPS];
    const uint64_t tiles_per_line = (n + TILE - 1) / TILE;
    const uint64_t total_tiles = tiles_per_line * lines;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int parity = 0;
    uint64_t tile = blockIdx.x;
    if (tile < total_tiles) {
        const uint64_t line = tile / tiles_per_line;
        stage_tile<T, Op, VEC, VPT, BLOCK, ALIGNED>(in, line * n, (tile - line * tiles_per_line) * TILE + (uint64_t)wid * WARP_ELEMS,
                                                    n, lane, s_stage);
    }
    while (tile < total_tiles) {
        T raw[VPT][VEC];
        fetch_tile<T, VEC, VPT, BLOCK>(s_stage, raw);
        const uint64_t next = tile + gridDim.x;
        if (next < total_tiles) {
            const uint64_t nline = next / tiles_per_line;
            stage_tile<T, Op, VEC, VPT, BLOCK, ALIGNED>(in, nline * n,
                                                        (next - nline * tiles_per_line) * TILE + (uint64_t)wid * WARP_ELEMS, n, lane,
                                                        s_stage);
        }
        // thread-local sum of the 16 values, then one tree over the warp.  (The summation order differs from the
        // scan pass; in fp64 that changes the aggregate by parts in 1e16, far below the rounding to T.)
        Acc run = (Acc)raw[0][0];
#pragma unroll
        for (int j = 0; j < VPT; ++j)
#pragma unroll
            for (int e = (j == 0 ? 1 : 0); e < VEC; ++e) run = Op::apply(run, (Acc)raw[j][e]);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) run = Op::apply(run, shfl_down_any(run, d));
        if (lane == 0) s_part[parity][wid] = run;
        __syncthreads();
        if (threadIdx.x == 0) {
            Acc a = Op::template identity<Acc>();
#pragma unroll
            for (int w = 0; w < WARPS; ++w) a = Op::apply(a, s_part[parity][w]);
            agg[tile] = a;
        }
        parity ^= 1;
        tile = next;
    }
    cp_async_wait_all();
}

// One block per line (grid-stride over lines): agg[line][0..tiles) becomes the exclusive prefix of the tile
// aggregates, seeded with *carry when HAS_CARRY (single line).  total_out[line] (optional) receives the
// reduction of the whole line without the carry.  WRITE_PREFIX = false only computes the totals.
// The line is walked in rounds of BLOCK * IPT consecutive values (coalesced), each round a block-wide scan.
template <typename Acc, class Op, bool HAS_CARRY, bool WRITE_PREFIX>
__device__ __forceinline__ void scan_aggregates(Acc* __restrict__ agg, const uint64_t lines, const uint64_t tiles_per_line,
                                                const Acc* __restrict__ carry, Acc* __restrict__ total_out) {
    constexpr int BLOCK = kScanBlock;
    constexpr int WARPS = BLOCK / 32;
    constexpr int IPT = 8;
    __shared__ Acc s_warp[2][WARPS];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int parity = 0;
    for (uint64_t line = blockIdx.x; line < lines; line += gridDim.x) {
        Acc* a = agg + line * tiles_per_line;
        Acc running = Op::template identity<Acc>();     // everything before the current round (without carry)
        for (uint64_t round0 = 0; round0 < tiles_per_line; round0 += (uint64_t)BLOCK * IPT) {
            const uint64_t lo = round0 + (uint64_t)threadIdx.x * IPT;
            Acc v[IPT];
#pragma unroll
            for (int k = 0; k < IPT; ++k) v[k] = (lo + k < tiles_per_line) ? a[lo + k] : Op::template identity<Acc>();
            Acc mine = v[0];
#pragma unroll
            for (int k = 1; k < IPT; ++k) mine = Op::apply(mine, v[k]);
            Acc t = mine;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const Acc y = shfl_up_any(t, d);
                if (lane >= d) t = Op::apply(y, t);
            }
            if (lane == 31) s_warp[parity][wid] = t;
            __syncthreads();
            Acc before = Op::template identity<Acc>();
            Acc round_total = Op::template identity<Acc>();
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const Acc x = s_warp[parity][w];
                if (w < wid) before = Op::apply(before, x);
                round_total = Op::apply(round_total, x);
            }
            parity ^= 1;
            if (WRITE_PREFIX) {
                Acc excl = shfl_up_any(t, 1);
                if (lane == 0) excl = Op::template identity<Acc>();
                Acc p = Op::apply(Op::apply(running, before), excl);
                if (HAS_CARRY) p = Op::apply(*carry, p);
#pragma unroll
                for (int k = 0; k < IPT; ++k) {
                    if (lo + k < tiles_per_line) a[lo + k] = p;
                    p = Op::apply(p, v[k]);
                }
            }
            running = Op::apply(running, round_total);
        }
        if (total_out != nullptr && threadIdx.x == 0) total_out[line] = running;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Many lines: one WARP per line, no cooperation between warps at all.
//
// When there are thousands of lines, a warp can walk down its line alone: chunks of 32 lanes x kWarpScanVecs vectors
// (warp-striped, every access a coalesced 128-bit vector), the running prefix of the line carried in a register, the
// next chunk already requested while the current one is scanned.  No shared memory, no barrier, nothing published:
// the only waits are a warp's own loads, and the other warps of the SM cover them.  Lines of any length (vectors
// must not straddle line ends: n % VEC == 0 and 16-byte aligned bases for VEC > 1).
constexpr int kWarpScanBlock = 256;
constexpr int kWarpScanVecs = 4;

// Launch shape for `lines` lines on `sms` SMs: every warp walks whole lines one after the other, so the kernel takes
// as long as the warp with the most lines.  Among 12 to 21 resident warps per SM (two to four blocks of four to eight
// warps; the kernel's registers allow no more) take the shape that leaves the fewest warp slots idle in the last
// round, and among equals the one with the most warps.
struct WarpScanShape {
    uint32_t grid, block;
};
constexpr uint64_t kWarpScanManyLines = 32768;
__host__ __device__ inline WarpScanShape warp_scan_shape(uint64_t lines, uint32_t sms) {
    // tens of thousands of (then short) lines: one line per warp in blocks of four warps, handed out by the hardware
    // as earlier blocks finish (fp32 [131072, 512]: 0.081 ms against 0.091 ms with resident warps walking the lines)
    if (lines >= kWarpScanManyLines) return WarpScanShape{(uint32_t)((lines + 3) / 4), 128};
    const uint32_t shapes[][2] = {{3, 7}, {4, 5}, {3, 6}, {2, 8}, {2, 7}, {3, 5}, {2, 6}, {3, 4}};   // {blocks per SM, warps}
    double best = -1.0;
    WarpScanShape pick = {1, 32};
    for (int i = 0; i < 8; ++i) {
        const uint64_t slots = (uint64_t)sms * shapes[i][0] * shapes[i][1];
        const uint64_t rounds = (lines + slots - 1) / slots;
        const double used = (double)lines / (double)(rounds * slots);
        if (used > best + 0.02) {
            best = used;
            const uint64_t blocks = (lines + shapes[i][1] - 1) / shapes[i][1];
            const uint64_t cap = (uint64_t)sms * shapes[i][0];
            pick.grid = (uint32_t)(blocks < cap ? blocks : cap);
            pick.block = shapes[i][1] * 32;
        }
    }
    return pick;
}

template <typename T, typename Acc, class Op, int VEC>
__device__ __forceinline__ void scan_lines_warp(const T* __restrict__ in, T* __restrict__ out, const uint64_t lines,
                                                const uint64_t n) {
    constexpr int U = kWarpScanVecs;
    constexpr uint64_t CHUNK = 32ull * VEC * U;
    const int lane = threadIdx.x & 31;
    // (the block may be launched with fewer warps than kWarpScanBlock / 32: the host sizes blocks and grid so that
    // the lines divide evenly among the resident warps)
    const uint64_t per_block = blockDim.x >> 5;
    const uint64_t warps = (uint64_t)gridDim.x * per_block;
    for (uint64_t line = (uint64_t)blockIdx.x * per_block + (threadIdx.x >> 5); line < lines; line += warps) {
        const T* src = in + line * n;
        T* dst = out + line * n;
        Acc carry = Op::template identity<Acc>();
        // one chunk ahead: the loads of chunk k + 1 are in flight while chunk k is scanned
        Vec<T, VEC> nxt[U];
        auto fetch = [&](const uint64_t from) {
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const uint64_t at = from + ((uint64_t)j * 32 + lane) * VEC;
                if (at < n) {
                    nxt[j] = load_vec<T, VEC>(src + at);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) nxt[j].v[e] = Op::template identity<T>();
                }
            }
        };
        fetch(0);
        for (uint64_t base = 0; base < n; base += CHUNK) {
            Vec<T, VEC> cur[U];
#pragma unroll
            for (int j = 0; j < U; ++j) cur[j] = nxt[j];
            if (base + CHUNK < n) fetch(base + CHUNK);
            // running values inside each of the lane's vectors (every element is widened once), then U independent
            // inclusive scans of the vector totals across the lanes
            Acc part[U][VEC], inc[U];
#pragma unroll
            for (int j = 0; j < U; ++j) {
                part[j][0] = (Acc)cur[j].v[0];
#pragma unroll
                for (int e = 1; e < VEC; ++e) part[j][e] = Op::apply(part[j][e - 1], (Acc)cur[j].v[e]);
                inc[j] = part[j][VEC - 1];
            }
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    const Acc y = shfl_up_any(inc[j], d);
                    if (lane >= d) inc[j] = Op::apply(y, inc[j]);
                }
            }
            // vector j covers elements [j * 32 * VEC, (j + 1) * 32 * VEC) of the chunk
#pragma unroll
            for (int j = 0; j < U; ++j) {
                Acc before = shfl_up_any(inc[j], 1);
                if (lane == 0) before = Op::template identity<Acc>();
                const Acc lead = Op::apply(carry, before);
                Vec<T, VEC> w;
#pragma unroll
                for (int e = 0; e < VEC; ++e) w.v[e] = (T)Op::apply(lead, part[j][e]);
                const uint64_t at = base + ((uint64_t)j * 32 + lane) * VEC;
                if (at < n) store_vec<T, VEC>(dst + at, w);
                carry = Op::apply(carry, shfl_any(inc[j], 31));
            }
        }
    }
}


// Lines of at most 128 vectors (2 KB), any whole number of vectors long: the tensor is walked as one flat array of
// vectors.  A warp's chunk (kWarpScanVecs rows of 32 lanes) takes as many WHOLE lines as fit into its 128 vectors - they
// follow each other in memory, so the warp streams one contiguous piece and the next chunk starts right behind it; a
// line is a run of neighbouring lanes that may continue from one row into the next.  The shuffle scans stop at line
// starts (a lane takes from the lane d to its left only if that lane holds the same line), the total of the line that
// is still open at the end of a row is handed to the next row, and nothing is carried from chunk to chunk.  With a
// power-of-two number of vectors per line every lane of every chunk is used; otherwise the last up-to-(line - 1)
// vectors of a chunk idle.
template <typename T, typename Acc, class Op, int VEC>
__device__ __forceinline__ void scan_lines_short(const T* __restrict__ in, T* __restrict__ out, const uint64_t lines,
                                                 const uint32_t n) {
    constexpr int U = kWarpScanVecs;
    const uint32_t per_line = n / VEC;                          // vectors per line: 1 ... 128
    const uint32_t lines_per_chunk = (32u * U) / per_line;
    const uint32_t used = lines_per_chunk * per_line;           // vectors of a chunk that hold data
    const int lane = threadIdx.x & 31;
    uint32_t pos[U];                                            // this lane's vectors: how far into their lines
#pragma unroll
    for (int j = 0; j < U; ++j) pos[j] = (uint32_t)(j * 32 + lane) % per_line;
    const uint64_t chunks = (lines + lines_per_chunk - 1) / lines_per_chunk;
    const uint64_t vectors = lines * per_line;
    const uint64_t per_block = blockDim.x >> 5;
    const uint64_t step = (uint64_t)gridDim.x * per_block;
    for (uint64_t chunk = (uint64_t)blockIdx.x * per_block + (threadIdx.x >> 5); chunk < chunks; chunk += step) {
        const uint64_t base = chunk * used;
        Acc part[U][VEC], inc[U];
        bool live[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const uint32_t c = (uint32_t)(j * 32 + lane);
            live[j] = c < used && base + c < vectors;
            Vec<T, VEC> cur;
            if (live[j]) {
                cur = load_vec<T, VEC>(in + (base + c) * VEC);
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) cur.v[e] = Op::template identity<T>();
            }
            part[j][0] = (Acc)cur.v[0];
#pragma unroll
            for (int e = 1; e < VEC; ++e) part[j][e] = Op::apply(part[j][e - 1], (Acc)cur.v[e]);
            inc[j] = part[j][VEC - 1];
        }
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            if ((uint32_t)d < per_line) {                       // (the same for every thread)
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    const Acc y = shfl_up_any(inc[j], d);
                    if (lane >= d && pos[j] >= (uint32_t)d) inc[j] = Op::apply(y, inc[j]);
                }
            }
        }
        Acc open_total = Op::template identity<Acc>();          // of the line that runs on from the row before
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const bool continues = pos[j] > (uint32_t)lane;     // the line began in an earlier row
            const Acc incl = continues ? Op::apply(open_total, inc[j]) : inc[j];
            Acc before = shfl_up_any(incl, 1);
            if (lane == 0) before = open_total;
            if (pos[j] == 0) before = Op::template identity<Acc>();
            Vec<T, VEC> w;
#pragma unroll
            for (int e = 0; e < VEC; ++e) w.v[e] = (T)Op::apply(before, part[j][e]);
            if (live[j]) store_vec<T, VEC>(out + (base + (uint32_t)(j * 32 + lane)) * VEC, w);
            if (per_line > 1) open_total = shfl_any(incl, 31);
        }
    }
}
// lines of n elements (vectors of VEC) that scan_lines_short takes
__host__ __device__ constexpr bool scan_short_line(uint64_t n, uint32_t vec) {
    return n >= vec && n % vec == 0 && n / vec <= 32 * kWarpScanVecs;
}
constexpr int kShortScanBlock = 128;
constexpr uint64_t kShortScanMinElements = 1ull << 16;


// ---------------------------------------------------------------------------------------------------------
// Ring scan: long lines in a single launch; every element is read from memory once and written once
// (8 bytes per fp32 element) and no thread block ever waits for the block before it.
//
// One persistent block per SM.  Tiles are numbered line by line; tile t belongs to block t % gridDim.x; the tiles b, b + G, b + 2G ... of block b
// are its "waves" 0, 1, 2 ...  A tile travels through a ring of kRingSlots tile-sized slots in shared memory.
// The block's warps have five roles, coupled only through shared-memory barriers (mbarrier):
//   copy warp      one thread streams the block's tiles into free slots with bulk asynchronous copies
//                  (cp.async.bulk, completion counted on the slot's `full` barrier), up to a whole ring ahead;
//   reduce warps   as soon as a tile has landed they total its sixteen chunks (`reduced` barrier) and publish the sum
//                  of those, the tile aggregate, to global memory;
//   chunk warp     scans the sixteen chunk totals exclusively (`chunked` barrier);
//   prefix warp    for every wave, gathers the aggregates all blocks published for that wave and forms
//                  carry-so-far (+) aggregates of the blocks to the left; each block keeps its own copy of the carry
//                  over the waves, computed in the same order everywhere, so no block depends on a value another
//                  block derived - only on the aggregates themselves.  It then leaves the prefix in front of every
//                  chunk of the tile in shared memory (`ready` barrier).  Its loop is the critical path of the whole
//                  grid - every scan waits for it - which is why the part that does not need the other blocks'
//                  aggregates is the chunk warp's;
//   scan warps     each scans one chunk of the tile out of its slot, seeded with the chunk's prefix, stores the
//                  result and releases the slot (`empty` barrier); the sixteen scan warps never wait for each other.
// Reduction runs ahead of the scan by as many tiles as the ring holds, which hides the trip of the aggregates
// through L2; in steady state nobody waits.  Aggregates travel as two 8-byte words, each carrying 32 payload bits
// and a 32-bit tag, so a word is valid on its own whenever its tag is set and no fence is needed; the host clears
// the words before the launch.
//
// All blocks must be resident (cooperative launch, grid <= number of SMs).  Every wait is bounded: when one
// expires the block records OVL_ERR_TIMEOUT in the status word, raises its abort flag, lets copies in flight
// land, and leaves; nothing traps.
constexpr int kRingSlots = 6;
constexpr int kRingScanWarps = kScanBlock / 32;    // 16 warps scan a tile (VPT vectors per thread)
constexpr int kRingReduceWarps = 8;                // 8 warps reduce a tile (2 * VPT vectors per thread)
constexpr int kRingThreads = (kRingScanWarps + kRingReduceWarps + 3) * 32;   // + copy, chunk and prefix warps
constexpr int kRingMaxGrid = 256;
constexpr int kRingGather = 5;                     // aggregates fetched per lane and round by the prefix warp (160 a round)
constexpr long long kRingWaitCycles = 1ll << 32;   // bound of every wait, in SM clock cycles (about two seconds)
constexpr long long kRingSelfTestWaitCycles = 1ll << 27;   // the same bound in the expiry self-test (about 70 ms)
constexpr uint32_t kRingCtlBytes = 4096;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bulk asynchronous copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned); completion
// is counted in bytes on `bar`
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
template <int ID, int THREADS>
__device__ __forceinline__ void named_bar_sync() {
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(THREADS) : "memory");
}

template <typename Acc>
struct RingCtl {
    Acc wprefix[kRingSlots][kRingScanWarps];       // exclusive prefix of each scan warp's chunk of the tile in the slot
    Acc ctot[kRingSlots][kRingScanWarps];          // totals of those chunks
    Acc rpart[2][kRingReduceWarps];                // per-warp partials of the tile being reduced
    uint64_t full[kRingSlots];                     // slot holds its tile             (copy thread + bytes landed)
    uint64_t reduced[kRingSlots];                  // ctot[slot] is valid             (one arrival per reduce warp)
    uint64_t ready[kRingSlots];                    // wprefix[slot] is valid          (prefix warp)
    uint64_t empty[kRingSlots];                    // slot has been read for the scan (one arrival per scan warp)
    Acc cexcl[kRingSlots][kRingScanWarps];         // exclusive scan of the chunk totals inside the tile
    uint64_t chunked[kRingSlots];                  // cexcl[slot] is valid            (chunk warp)
    int abort;
    int rstop[2];                                  // abort flag as latched for the reduce warps' current step
};

// bounded wait on a shared-memory barrier; gives up at once when the block is aborting
__device__ __forceinline__ bool ring_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, const long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (clock64() - t0 < limit) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void ring_fail(ScanHeader* hdr, volatile int* abort_flag) {
    if (!*abort_flag) {
        atomicExch(&hdr->status, kErrTimeout);
        *abort_flag = 1;
    }
}

template <typename Acc>
__device__ __forceinline__ void ring_publish(uint64_t* desc, uint64_t tile, Acc a) {
    uint64_t bits = 0;
    memcpy(&bits, &a, sizeof(Acc));
    const uint64_t w0 = (1ull << 32) | (bits & 0xffffffffull), w1 = (1ull << 32) | (bits >> 32);
    asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(desc + 2 * tile), "l"(w0), "l"(w1) : "memory");
}
__device__ __forceinline__ void ring_peek(const uint64_t* desc, uint64_t tile, uint64_t& w0, uint64_t& w1) {
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(desc + 2 * tile) : "memory");
}

// ---------------------------------------------------------------------------------------------------------
// Exchange of shard totals between the GPUs of one box through peer memory (a scan along an axis that is split
// over several GPUs).  Every GPU owns one exchange buffer; `slots[p]` is the buffer of rank p as mapped into this
// process (an IPC mapping for p != rank).  A buffer holds, for each of two epoch parities and each source rank,
// two 8-byte words that carry 32 payload bits and the 32-bit epoch as a tag: a word is valid on its own when its
// tag equals the epoch of the call, so no fence and no reset between calls is needed.  The reduction kernel of
// rank r stores its total into slot [epoch & 1][r] of EVERY rank's buffer (plain stores over NVLink); the scan
// kernel of every rank polls its OWN buffer (local memory) until all `world` totals of the epoch are there, and
// folds those of the ranks before it, in rank order, into its carry.  Waiting for all ranks, not only for the
// earlier ones, keeps any rank from running more than one call ahead of another, which is what makes two
// parities enough.  The wait is bounded like every other wait of the ring scan.
constexpr int kMaxPeers = 8;
struct PeerExchange {
    uint64_t* slots[kMaxPeers];
    uint32_t world;
    uint32_t rank;
    uint32_t epoch;      // 1, 2, 3, ... (0 is the tag of a cleared buffer)
    uint32_t pad;
};
constexpr uint32_t kPeerBufferWords = 2 * kMaxPeers * 2;

template <typename Acc>
__device__ __forceinline__ void peer_publish(const PeerExchange& px, Acc total) {
    static_assert(sizeof(Acc) == 8, "totals travel as two tagged 32-bit halves");
    uint64_t bits = 0;
    memcpy(&bits, &total, sizeof(Acc));
    const uint64_t tag = (uint64_t)px.epoch << 32;
    const uint64_t w0 = tag | (bits & 0xffffffffull), w1 = tag | (bits >> 32);
    const uint32_t at = ((px.epoch & 1u) * kMaxPeers + px.rank) * 2;
    for (uint32_t p = 0; p < px.world; ++p)
        asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(px.slots[p] + at), "l"(w0), "l"(w1) : "memory");
}

// called by one whole warp; returns false when the totals did not arrive within `limit` clock cycles
template <typename Acc, class Op>
__device__ __forceinline__ bool peer_carry(const PeerExchange& px, const int lane, const long long limit, Acc& carry) {
    const uint64_t* mine = px.slots[px.rank] + (px.epoch & 1u) * kMaxPeers * 2;
    uint64_t w0 = 0, w1 = 0;
    bool have = lane >= (int)px.world;
    const long long t0 = clock64();
    bool all = false;
    while (true) {
        if (!have) {
            asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(mine + 2 * lane) : "memory");
            have = (uint32_t)(w0 >> 32) == px.epoch && (uint32_t)(w1 >> 32) == px.epoch;
        }
        all = __all_sync(0xffffffffu, have);
        if (all || clock64() - t0 >= limit) break;
    }
    const uint64_t bits = (w0 & 0xffffffffull) | (w1 << 32);
    carry = Op::template identity<Acc>();
    for (uint32_t r = 0; r < px.rank; ++r) {
        const uint64_t b = __shfl_sync(0xffffffffu, bits, (int)r);
        Acc t;
        memcpy(&t, &b, sizeof(Acc));
        carry = Op::apply(carry, t);
    }
    return all;
}

// slot index and barrier phase of a role's current wave, advanced without divisions
struct RingCursor {
    int slot;
    uint32_t phase;
    __device__ __forceinline__ RingCursor() : slot(0), phase(0) {}
    __device__ __forceinline__ void advance() {
        if (++slot == kRingSlots) {
            slot = 0;
            phase ^= 1u;
        }
    }
};

// Position of a role's current tile: tiles are numbered line by line (tiles_per_line per line, the last tile of a
// line possibly ragged); a role visits tiles b, b + G, b + 2G ... and keeps (line, tile in line) without divisions.
// With a single line (MULTI = false) the line stays 0 and nothing but an addition is left.
template <bool MULTI>
struct RingTile {
    uint64_t line, q, tiles_per_line;
    uint64_t dl, dq;
    __device__ __forceinline__ RingTile(uint64_t tile, uint64_t tpl, uint32_t G)
        : line(MULTI ? tile / tpl : 0), q(MULTI ? tile % tpl : tile), tiles_per_line(tpl), dl(MULTI ? G / tpl : 0),
          dq(MULTI ? G % tpl : G) {}
    __device__ __forceinline__ void advance() {
        q += dq;
        if (MULTI) {
            line += dl;
            if (q >= tiles_per_line) {
                q -= tiles_per_line;
                ++line;
            }
        }
    }
    __device__ __forceinline__ bool last_of_line() const { return q + 1 == tiles_per_line; }
    __device__ __forceinline__ uint64_t first_element(uint64_t n, uint32_t tile_elems) const {
        return (MULTI ? line * n : 0) + q * tile_elems;
    }
};

template <bool MULTI, bool GROUPED>
struct RingTileOf {
    typedef RingTile<MULTI> type;
};

// Several lines, GROUPED layout: the grid is cut into groups of `g` consecutive blocks and every group scans whole
// lines on its own - group k takes the lines k, k + groups, k + 2 groups ... one after the other, each exactly like
// a single line scanned by a grid of g blocks (tile t of a line belongs to member t % g; a wave is g tiles of one
// line).  Groups never wait for each other, and a block's prefix warp gathers g aggregates instead of a whole
// grid's; with g = 1 a block walks down its lines alone.  Tiles keep their line-by-line numbers in the scratch.
struct RingGroupTile {
    uint64_t line, q, tiles_per_line;
    uint32_t member, g, groups;
    __device__ __forceinline__ RingGroupTile(uint32_t block, uint64_t tpl, uint32_t group_size, uint32_t n_groups)
        : line(block / group_size), q(block % group_size), tiles_per_line(tpl), member(block % group_size), g(group_size),
          groups(n_groups) {}
    __device__ __forceinline__ void advance() {
        q += g;
        if (q >= tiles_per_line) {
            q = member;
            line += groups;
        }
    }
    __device__ __forceinline__ bool last_of_line() const { return q + 1 == tiles_per_line; }
    __device__ __forceinline__ uint64_t first_element(uint64_t n, uint32_t tile_elems) const { return line * n + q * tile_elems; }
    __device__ __forceinline__ uint64_t number() const { return line * tiles_per_line + q; }
};

// Blocks per group for `lines` lines of `tpl` tiles on a grid of G blocks: as many as the grid has per line, at most
// one per tile of a line.  The share of the grid's block-time that does useful work with that layout (lines that do
// not fill the last round of groups, blocks left over) decides whether the grouped layout is used at all.
__host__ __device__ inline uint32_t ring_group_size(uint32_t G, uint64_t lines, uint64_t tpl) {
    uint64_t g = lines >= G ? 1 : G / lines;
    if (g > tpl) g = tpl;
    return (uint32_t)(g < 1 ? 1 : g);
}
__host__ __device__ inline double ring_group_efficiency(uint32_t G, uint64_t lines, uint64_t tpl) {
    const uint32_t g = ring_group_size(G, lines, tpl);
    const uint64_t groups = G / g;
    const uint64_t rounds = (lines + groups - 1) / groups;
    return (double)lines / (double)(rounds * groups) * (double)(groups * g) / (double)G;
}
// (measured on fp32: groups that keep the whole grid busy run at 5.5 TB/s against 5.0 TB/s for waves across line
// ends - 16 lines of 2^27, 148 lines of 2^22, 1024 lines of 2^20 - but at 86 % occupancy, 64 or 256 lines, they lose)
constexpr double kRingGroupedMinEfficiency = 0.93;
template <bool MULTI>
struct RingTileOf<MULTI, true> {
    typedef RingGroupTile type;
};

// SELFTEST: the bounded-wait self-test (one block withholds its aggregates; every wait uses the short bound).
// PEER: the carry comes from the totals that all ranks published into this rank's exchange buffer (`px`).
// GROUPED: several lines in the grouped layout above (MULTI must then be false: no wave crosses a line end).
template <typename T, typename Acc, class Op, int VEC, bool HAS_CARRY, bool MULTI, bool SELFTEST = false, bool PEER = false,
          bool GROUPED = false>
__device__ __forceinline__ void scan_ring(const T* __restrict__ in, T* __restrict__ out, const Acc* __restrict__ carry_in,
                                          const uint64_t lines, const uint64_t n, void* scratch,
                                          const int withhold_block = -1, const PeerExchange* px = nullptr) {
    constexpr int VPT = kScanVpt;
    constexpr int SW = kRingScanWarps, RW = kRingReduceWarps;
    constexpr int CPR = SW / RW;                   // chunks (one per scan warp) handled by one reduce warp
    constexpr int R = kRingSlots;
    constexpr uint32_t TILE = kScanBlock * VPT * VEC;
    constexpr uint32_t TILE_BYTES = TILE * sizeof(T);
    static_assert(sizeof(RingCtl<Acc>) <= kRingCtlBytes, "control block too large");
    static_assert(TILE_BYTES % 16 == 0, "tiles must be whole 16-byte units");
    static_assert(SW <= 32 && (SW & (SW - 1)) == 0 && SW % RW == 0, "chunk totals are scanned by one warp");

    extern __shared__ __align__(128) unsigned char ring_smem[];
    RingCtl<Acc>* ctl = reinterpret_cast<RingCtl<Acc>*>(ring_smem + (size_t)R * TILE_BYTES);
    volatile int* abort_flag = &ctl->abort;
    // (the self-test that withholds one block's aggregates lets every wait run out: it uses a short bound)
    constexpr long long wait_limit = SELFTEST ? kRingSelfTestWaitCycles : kRingWaitCycles;

    ScanHeader* hdr = reinterpret_cast<ScanHeader*>(scratch);
    uint64_t* desc = reinterpret_cast<uint64_t*>(hdr + 1);
    const uint64_t tiles_per_line = (n + TILE - 1) / TILE;
    static_assert(!(GROUPED && (MULTI || HAS_CARRY || SELFTEST || PEER)), "the grouped layout stands alone");
    const uint64_t total_tiles = tiles_per_line * (MULTI ? lines : 1);
    const uint32_t G = gridDim.x, b = blockIdx.x;
    // grouped layout: g blocks per group, `groups` groups, this block is member `me` of group b / g
    const uint32_t g = GROUPED ? ring_group_size(G, lines, tiles_per_line) : G;
    const uint32_t groups = GROUPED ? G / g : 1u;
    const uint32_t me = GROUPED ? b % g : b;
    uint32_t my_tiles = (total_tiles > b) ? (uint32_t)((total_tiles - b + G - 1) / G) : 0u;
    if (GROUPED) {
        const uint32_t group = b / g;
        const uint64_t my_lines = (group < groups && lines > group) ? (lines - group + groups - 1) / groups : 0;
        my_tiles = (uint32_t)(my_lines * ((tiles_per_line - me + g - 1) / g));      // (g <= tiles_per_line)
    }
    using Tile = typename RingTileOf<MULTI, GROUPED>::type;
    auto first_tile = [&]() {
        if constexpr (GROUPED) {
            return RingGroupTile(b, tiles_per_line, g, groups);
        } else {
            return RingTile<MULTI>(b, tiles_per_line, G);
        }
    };
    const uint32_t tail = (uint32_t)(n - (tiles_per_line - 1) * TILE);   // valid elements of a line's last tile
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        for (int s = 0; s < R; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->reduced[s], RW);
            mbar_init(&ctl->chunked[s], 1);
            mbar_init(&ctl->ready[s], 1);
            mbar_init(&ctl->empty[s], SW);
        }
        ctl->abort = 0;
        ctl->rstop[0] = ctl->rstop[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (wid < SW) {
        // --------------------------------------------------------------------------------------- scan warps
        // warp `wid` scans chunk `wid` (32 * VPT vectors) of every tile of the block, on its own: the prefix in
        // front of the chunk is already in shared memory when the warp starts, so warps never wait for each other
        RingCursor cur;
        Tile at = first_tile();
        const uint32_t v0 = (uint32_t)wid * 32 * VPT + lane;            // this thread's vectors: v0 + 32 j
        for (uint32_t k = 0; k < my_tiles; ++k, at.advance(), cur.advance()) {
            if (!ring_wait(&ctl->full[cur.slot], cur.phase, abort_flag, wait_limit)) ring_fail(hdr, abort_flag);
            if (!ring_wait(&ctl->ready[cur.slot], cur.phase, abort_flag, wait_limit)) ring_fail(hdr, abort_flag);
            if (*abort_flag) break;
            const bool whole = !at.last_of_line() || tail == TILE;
            const Vec<T, VEC>* sv = reinterpret_cast<const Vec<T, VEC>*>(ring_smem + (size_t)cur.slot * TILE_BYTES);
            Acc av[VPT][VEC];                                           // the chunk's values, widened once
            if (whole) {
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    const Vec<T, VEC> v = sv[v0 + j * 32];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) av[j][e] = (Acc)v.v[e];
                }
            } else {
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    const Vec<T, VEC> v = sv[v0 + j * 32];
#pragma unroll
                    for (int e = 0; e < VEC; ++e)
                        av[j][e] = ((v0 + j * 32) * VEC + e < tail) ? (Acc)v.v[e] : Op::template identity<Acc>();
                }
            }
            const Acc offset = ctl->wprefix[cur.slot][wid];
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->empty[cur.slot]);          // this warp is done with the slot
            // sweep 1: totals of each vector, scanned across the warp; base[j] = prefix in front of vector j
            Acc base[VPT];
            Acc run = offset;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                Acc t = av[j][0];
#pragma unroll
                for (int e = 1; e < VEC; ++e) t = Op::apply(t, av[j][e]);
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const Acc y = shfl_up_any(t, d);
                    if (lane >= d) t = Op::apply(y, t);
                }
                Acc excl = shfl_up_any(t, 1);
                if (lane == 0) excl = Op::template identity<Acc>();
                base[j] = Op::apply(run, excl);
                if (j + 1 < VPT) run = Op::apply(run, shfl_any(t, 31));
            }
            // sweep 2: running values, rounded to T on store
            T* dst = out + at.first_element(n, TILE);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const uint32_t off = (v0 + j * 32) * VEC;
                Acc p = base[j];
                if (whole) {
                    Vec<T, VEC> v;
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        p = Op::apply(p, av[j][e]);
                        v.v[e] = (T)p;
                    }
                    store_vec<T, VEC>(dst + off, v);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        p = Op::apply(p, av[j][e]);
                        if (off + e < tail) dst[off + e] = (T)p;
                    }
                }
            }
        }
    } else if (wid < SW + RW) {
        // ------------------------------------------------------------------------------------- reduce warps
        // reduce warp rw totals the chunks CPR*rw .. CPR*rw + CPR - 1 of every tile as soon as it has landed
        RingCursor cur;
        int parity = 0;
        const int rw = wid - SW;
        uint64_t tile = b;
        Tile at = first_tile();
        for (uint32_t k = 0; k < my_tiles; ++k, tile += G, at.advance(), cur.advance(), parity ^= 1) {
            if (!ring_wait(&ctl->full[cur.slot], cur.phase, abort_flag, wait_limit)) ring_fail(hdr, abort_flag);
            const bool whole = !at.last_of_line() || tail == TILE;
            const Vec<T, VEC>* sv = reinterpret_cast<const Vec<T, VEC>*>(ring_smem + (size_t)cur.slot * TILE_BYTES);
            Acc part[CPR];
#pragma unroll
            for (int q = 0; q < CPR; ++q) {
                const uint32_t v0 = (uint32_t)(rw * CPR + q) * 32 * VPT + lane;
                Acc pj[VPT];
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    const Vec<T, VEC> v = sv[v0 + j * 32];
                    pj[j] = Op::template identity<Acc>();
#pragma unroll
                    for (int e = 0; e < VEC; ++e)
                        if (whole || (v0 + j * 32) * VEC + e < tail) pj[j] = Op::apply(pj[j], (Acc)v.v[e]);
                }
                part[q] = pj[0];
#pragma unroll
                for (int j = 1; j < VPT; ++j) part[q] = Op::apply(part[q], pj[j]);
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1)
#pragma unroll
                for (int q = 0; q < CPR; ++q) part[q] = Op::apply(part[q], shfl_down_any(part[q], d));
            if (lane == 0) {
                Acc sum = part[0];
                ctl->ctot[cur.slot][rw * CPR] = part[0];
#pragma unroll
                for (int q = 1; q < CPR; ++q) {
                    ctl->ctot[cur.slot][rw * CPR + q] = part[q];
                    sum = Op::apply(sum, part[q]);
                }
                ctl->rpart[parity][rw] = sum;
                mbar_arrive(&ctl->reduced[cur.slot]);
                if (rw == 0) ctl->rstop[parity] = *abort_flag;
            }
            named_bar_sync<2, RW * 32>();
            if (ctl->rstop[parity]) break;                              // same value for every reduce thread
            if (rw == 0 && lane == 0) {
                Acc a = ctl->rpart[parity][0];
#pragma unroll
                for (int w = 1; w < RW; ++w) a = Op::apply(a, ctl->rpart[parity][w]);
                // (self-test of the bounded waits: one block may be told to keep its aggregates to itself)
                if constexpr (GROUPED) {
                    ring_publish<Acc>(desc, at.number(), a);
                } else {
                    if (!SELFTEST || (int)b != withhold_block) ring_publish<Acc>(desc, tile, a);
                }
            }
        }
    } else if (wid == SW + RW) {
        // ---------------------------------------------------------------------------------------- copy warp
        if (lane == 0) {
            RingCursor cur;
            uint32_t issued = 0;
            Tile at = first_tile();
            for (uint32_t k = 0; k < my_tiles; ++k, at.advance(), cur.advance()) {
                // second and later uses of a slot: wait until the scan of its previous tile has read it
                if (k >= (uint32_t)R && !ring_wait(&ctl->empty[cur.slot], cur.phase ^ 1u, abort_flag, wait_limit)) {
                    ring_fail(hdr, abort_flag);
                    break;
                }
                const uint32_t valid = at.last_of_line() ? tail : TILE;
                const uint32_t bulk = (uint32_t)(valid * sizeof(T)) & ~15u;
                const T* src = in + at.first_element(n, TILE);
                T* slot_data = reinterpret_cast<T*>(ring_smem + (size_t)cur.slot * TILE_BYTES);
                for (uint32_t i = bulk / (uint32_t)sizeof(T); i < valid; ++i) slot_data[i] = src[i];   // ragged end
                if (bulk) {
                    mbar_arrive_expect_tx(&ctl->full[cur.slot], bulk);
                    bulk_load(slot_data, src, bulk, &ctl->full[cur.slot]);
                } else {
                    mbar_arrive(&ctl->full[cur.slot]);
                }
                issued = k + 1;
            }
            if (*abort_flag) {
                // let the copies that may still be in flight land before the block gives up its shared memory
                const long long t0 = clock64();
                for (uint32_t k = (issued > (uint32_t)R) ? issued - R : 0; k < issued; ++k)
                    while (!mbar_try_wait(&ctl->full[k % R], (k / R) & 1u) && clock64() - t0 < wait_limit) {
                    }
            }
        }
    } else if (wid == SW + RW + 1) {
        // --------------------------------------------------------------------------------------- chunk warp
        // scans the sixteen chunk totals of a tile as soon as the reduce warps have written them and leaves the
        // exclusive values in shared memory - work that does not need the other blocks, taken off the prefix warp
        RingCursor cur;
        for (uint32_t k = 0; k < my_tiles; ++k, cur.advance()) {
            // the chunk totals have been written - which also means that the slot's previous tile has been scanned, so
            // that its prefixes (wprefix, cexcl) are no longer needed; the prefix warp relies on this
            if (!ring_wait(&ctl->reduced[cur.slot], cur.phase, abort_flag, wait_limit) ||
                (k >= (uint32_t)R && !ring_wait(&ctl->empty[cur.slot], cur.phase ^ 1u, abort_flag, wait_limit))) {
                if (lane == 0) ring_fail(hdr, abort_flag);
                break;
            }
            Acc c = (lane < SW) ? ctl->ctot[cur.slot][lane] : Op::template identity<Acc>();
#pragma unroll
            for (int d = 1; d < SW; d <<= 1) {
                const Acc y = shfl_up_any(c, d);
                if (lane >= d) c = Op::apply(y, c);
            }
            Acc cexcl = shfl_up_any(c, 1);
            if (lane == 0) cexcl = Op::template identity<Acc>();
            if (lane < SW) ctl->cexcl[cur.slot][lane] = cexcl;
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->chunked[cur.slot]);
        }
    } else {
        // -------------------------------------------------------------------------------------- prefix warp
        RingCursor cur;
        Acc carry = Op::template identity<Acc>();
        if (HAS_CARRY) {
            if (PEER) {
                // the carry is the combination of the totals that the ranks before this one published
                if (!peer_carry<Acc, Op>(*px, lane, wait_limit, carry)) ring_fail(hdr, abort_flag);
            } else {
                carry = *carry_in;
            }
        }
        // With several lines, `carry` is the reduction of the tiles before the current wave that belong to the line
        // in which the wave starts, and prefixes restart at every line start.  Which tiles of a wave belong to which
        // line follows from the positions of the wave's first tile, of this block's tile and of the next wave's
        // first tile inside their lines.  (With a single line all of this is constant and the masks disappear.)
        // (Grouped layout: a wave is the g tiles of ONE line that the group's members hold at the same time; the carry
        // restarts with every line and no masks are needed.)
        uint64_t first = 0;
        RingTile<MULTI> wave(0, tiles_per_line, G);
        Tile mine = first_tile();
        for (uint32_t j = 0; j < my_tiles; ++j, first += G, cur.advance(), mine.advance()) {
            if (*abort_flag) break;
            uint32_t gj;
            bool same_line_next;
            if constexpr (GROUPED) {
                const uint64_t wave_q = mine.q - me;                        // the wave's first tile inside the line
                first = mine.line * tiles_per_line + wave_q;
                gj = (uint32_t)((tiles_per_line - wave_q < g) ? (tiles_per_line - wave_q) : g);
                same_line_next = mine.q + g < tiles_per_line;               // this block's next tile: same line?
                if (wave_q == 0) carry = Op::template identity<Acc>();
            } else {
                gj = (uint32_t)((total_tiles - first < G) ? (total_tiles - first) : G);
                const uint64_t line_first = wave.line;
                wave.advance();                                             // now the next wave's first tile
                same_line_next = !MULTI || wave.line == line_first;         // the wave lies in one line that goes on
            }
            const uint32_t next_lo = same_line_next ? 0u : (uint32_t)(G - wave.q);   // wave tiles from here on: next wave's line
            const bool mine_in_first = !MULTI || mine.q >= b;               // my line began at or before the wave's start
            const uint32_t mine_lo = mine_in_first ? 0u : (uint32_t)(b - mine.q);    // wave tiles from here to b: my line
            Acc excl = Op::template identity<Acc>(), tot = Op::template identity<Acc>();
            bool failed = false;
            for (uint32_t base_i = 0; base_i < gj; base_i += 32 * kRingGather) {
                uint64_t w0[kRingGather], w1[kRingGather];
                bool missing = false;
#pragma unroll
                for (int i = 0; i < kRingGather; ++i) {
                    const uint32_t idx = base_i + i * 32 + lane;
                    w0[i] = w1[i] = 1ull << 32;                         // (slots past the wave's end: valid, identity)
                    if (idx < gj) ring_peek(desc, first + idx, w0[i], w1[i]);
                }
#pragma unroll
                for (int i = 0; i < kRingGather; ++i) missing |= (w0[i] >> 32) == 0 || (w1[i] >> 32) == 0;
                if (__any_sync(0xffffffffu, missing)) {
                    // not all there yet: poll the missing ones, with a bound
                    const long long t0 = clock64();
#pragma unroll
                    for (int i = 0; i < kRingGather; ++i) {
                        const uint32_t idx = base_i + i * 32 + lane;
                        uint32_t spins = 0;
                        while (((w0[i] >> 32) == 0 || (w1[i] >> 32) == 0) && clock64() - t0 < wait_limit && !*abort_flag) {
                            if (++spins > 4) __nanosleep(64);
                            ring_peek(desc, first + idx, w0[i], w1[i]);
                        }
                        failed |= (w0[i] >> 32) == 0 || (w1[i] >> 32) == 0;
                    }
                }
#pragma unroll
                for (int i = 0; i < kRingGather; ++i) {
                    const uint32_t idx = base_i + i * 32 + lane;
                    if (idx < gj) {
                        const uint64_t bits = (w0[i] & 0xffffffffull) | (w1[i] << 32);
                        Acc v;
                        memcpy(&v, &bits, sizeof(Acc));
                        if (!MULTI || idx >= next_lo) tot = Op::apply(tot, v);
                        if (idx < me && (!MULTI || idx >= mine_lo)) excl = Op::apply(excl, v);
                    }
                }
            }
            if (__any_sync(0xffffffffu, failed)) {
                if (lane == 0) ring_fail(hdr, abort_flag);
                break;
            }
            // lanes hold interleaved partial results, combined in a fixed butterfly
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) excl = Op::apply(excl, shfl_xor_any(excl, d));
            // this tile's chunk prefixes are ready (and with that, wprefix[slot] of the slot's previous tile was read)
            if (!ring_wait(&ctl->chunked[cur.slot], cur.phase, abort_flag, wait_limit)) {
                if (lane == 0) ring_fail(hdr, abort_flag);
                break;
            }
            const Acc before = mine_in_first ? Op::apply(carry, excl) : excl;
            if (lane < SW) ctl->wprefix[cur.slot][lane] = Op::apply(before, ctl->cexcl[cur.slot][lane]);
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->ready[cur.slot]);
            // the carry of the next wave, off the path of this wave's scans (the same butterfly in every block, so
            // every block derives the same value)
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) tot = Op::apply(tot, shfl_xor_any(tot, d));
            carry = (same_line_next || GROUPED) ? Op::apply(carry, tot) : tot;
        }
    }
    __syncthreads();
}

// Reduction of n elements to one Acc, combination order fixed by the launch shape: per-thread strided partials,
// block tree, then the last block to finish combines the per-block partials in block order.
// scratch: [uint32 done_counter, pad to 16 bytes][Acc partial per block]
//
// Every block totals ONE chunk of kReduceChunk consecutive elements (the grid is one block per chunk and the
// hardware hands chunks to SMs as earlier blocks finish, so no SM waits behind a slow one); the block that finishes
// last combines the per-chunk partials - all of its threads, in an order fixed by the chunk count alone, so the
// result does not depend on which block that was or on how the blocks were scheduled.
// (Visiting the chunks from the end of the array to its start, so that the caches would still hold the START of the
// array for a scan that follows, was measured and is not done: the reversed walk itself runs at 5.6 TB/s against
// 6.9 TB/s forward, more than the warm start gives back.)  `px` (optional): publish the total to the GPUs of the
// exchange as well.
constexpr uint64_t kReduceChunk = 1ull << 17;

__host__ __device__ constexpr uint64_t reduce_chunks(uint64_t n) { return (n + kReduceChunk - 1) / kReduceChunk; }

template <typename Acc, class Op, int BLOCK>
__device__ __forceinline__ Acc block_total(Acc t, Acc* s_part) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) t = Op::apply(t, shfl_down_any(t, d));
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) s_part[wid] = t;
    __syncthreads();
    Acc b = Op::template identity<Acc>();
    if (threadIdx.x == 0)
        for (int w = 0; w < BLOCK / 32; ++w) b = Op::apply(b, s_part[w]);
    return b;       // valid in thread 0
}

template <typename T, typename Acc, class Op, int VEC, bool ALIGNED>
__device__ __forceinline__ void reduce_all(const T* __restrict__ in, const uint64_t n, Acc* __restrict__ out_total,
                                           void* scratch, const PeerExchange* px = nullptr) {
    constexpr int BLOCK = kScanBlock;
    __shared__ Acc s_part[BLOCK / 32];
    __shared__ bool s_last;
    uint32_t* counter = reinterpret_cast<uint32_t*>(scratch);
    Acc* partials = reinterpret_cast<Acc*>(reinterpret_cast<char*>(scratch) + 16);

    const uint64_t chunks = gridDim.x;
    const uint64_t chunk = blockIdx.x;
    const uint64_t begin = chunk * kReduceChunk;
    const uint64_t len = (n - begin < kReduceChunk) ? n - begin : kReduceChunk;
    const T* src = in + begin;          // (a chunk starts on a 16-byte boundary whenever the array does)
    Acc acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = Op::template identity<Acc>();
    const uint64_t nvec = ALIGNED ? len / VEC : 0;
    uint64_t g = threadIdx.x;
    // four independent vectors in flight per thread
    for (; g + 3 * BLOCK < nvec; g += 4 * BLOCK) {
        Vec<T, VEC> v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = load_vec<T, VEC>(src + (g + u * BLOCK) * VEC);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[u] = Op::apply(acc[u], (Acc)v[u].v[e]);
    }
    for (; g < nvec; g += BLOCK) {
        const Vec<T, VEC> v = load_vec<T, VEC>(src + g * VEC);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[0] = Op::apply(acc[0], (Acc)v.v[e]);
    }
    for (uint64_t i = nvec * VEC + threadIdx.x; i < len; i += BLOCK) acc[0] = Op::apply(acc[0], (Acc)src[i]);
    const Acc mine = block_total<Acc, Op, BLOCK>(Op::apply(Op::apply(acc[0], acc[1]), Op::apply(acc[2], acc[3])), s_part);
    if (threadIdx.x == 0) {
        partials[chunk] = mine;
        __threadfence();
        const uint32_t ticket = atomicAdd(counter, 1u);
        s_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    // the last block to finish: thread t folds partials t, t + BLOCK, ... (chunk order), then the threads are combined
    __threadfence();
    Acc t = Op::template identity<Acc>();
    for (uint64_t c = threadIdx.x; c < chunks; c += BLOCK) t = Op::apply(t, *(volatile Acc*)&partials[c]);
    __syncthreads();                    // (s_part is reused)
    const Acc total = block_total<Acc, Op, BLOCK>(t, s_part);
    if (threadIdx.x == 0) {
        *out_total = total;
        if (px != nullptr) peer_publish<Acc>(*px, total);
    }
}

}  // namespace ovl
