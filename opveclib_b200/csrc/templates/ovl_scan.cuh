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
    if constexpr (sizeof(A) == 8) {
        long long x = *reinterpret_cast<long long*>(&v);
        x = __shfl_up_sync(0xffffffffu, x, delta);
        return *reinterpret_cast<A*>(&x);
    } else {
        return __shfl_up_sync(0xffffffffu, v, delta);
    }
}
template <typename A>
__device__ __forceinline__ A shfl_down_any(A v, int delta) {
    if constexpr (sizeof(A) == 8) {
        long long x = *reinterpret_cast<long long*>(&v);
        x = __shfl_down_sync(0xffffffffu, x, delta);
        return *reinterpret_cast<A*>(&x);
    } else {
        return __shfl_down_sync(0xffffffffu, v, delta);
    }
}
template <typename A>
__device__ __forceinline__ A shfl_any(A v, int lane) {
    if constexpr (sizeof(A) == 8) {
        long long x = *reinterpret_cast<long long*>(&v);
        x = __shfl_sync(0xffffffffu, x, lane);
        return *reinterpret_cast<A*>(&x);
    } else {
        return __shfl_sync(0xffffffffu, v, lane);
    }
}

// Asynchronous copy of one vector (BYTES = 4, 8 or 16) from global to shared memory, and the group fence.
template <int BYTES>
__device__ __forceinline__ void cp_async_vec(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(d), "l"(gmem_src), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

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
//  LOOKBACK   lines are longer than one tile.  false: one tile per line, tiles are handed out statically
//             (blockIdx, blockIdx + gridDim, ...), nothing is published and no block ever waits for another.
//             true: tiles are claimed in order from the atomic counter and prefixes travel through descriptors.
// While a block works on one tile, the data of its next tile is already on its way into shared memory
// (cp.async), so global loads overlap the scan, the look-back and the stores of the current tile.
template <typename T, typename Acc, class Op, int VEC, bool ALIGNED, bool HAS_CARRY, bool LOOKBACK>
__device__ __forceinline__ void scan_lines(const T* __restrict__ in, T* __restrict__ out, const Acc* __restrict__ carry,
                                           const uint64_t lines, const uint64_t n, void* scratch) {
    constexpr int BLOCK = LOOKBACK ? kScanBlockLookback : kScanBlock;
    constexpr int VPT = kScanVpt;
    constexpr int WARPS = BLOCK / 32;
    constexpr int LBW = kScanLookbackWarps;
    constexpr uint32_t TILE = BLOCK * VPT * VEC;
    constexpr uint32_t WARP_ELEMS = 32 * VPT * VEC;

    ScanHeader* hdr = reinterpret_cast<ScanHeader*>(scratch);
    TileDesc<Acc>* desc = reinterpret_cast<TileDesc<Acc>*>(hdr + 1);
    const uint64_t tiles_per_line = LOOKBACK ? (n + TILE - 1) / TILE : 1;
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
        if (tile_in_line == 0) {
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
// One long line: wave scan.
//
// Look-back hands prefixes from tile to tile through L2, a window of descriptors per round trip; for a single
// line of millions of tiles that relay, not HBM, sets the pace.  Here the blocks of a (cooperative, fully
// resident) grid advance in waves: in wave w block b owns tile w*G + b.  Every block publishes its tile
// aggregate in slot b of a wave buffer (16-byte {value, wave tag} written and read as one transaction), then
// reads ALL G slots of the wave once: the ordered sum of the slots before b is its prefix inside the wave, the
// sum of all slots advances the running prefix that every block keeps for itself in a register.  Nothing is
// relayed: one publish and one gather per wave, independent of the line's length.  Two wave buffers alternate;
// a block can only publish into a buffer again after a complete gather of the wave in between, which in turn
// needs every block to have finished reading the older wave.
constexpr int kWaveMaxBlocks = 1024;   // slots per wave buffer
constexpr int kWaveSlotsPerThread = kWaveMaxBlocks / kScanBlockLookback;

__host__ __device__ constexpr uint64_t wave_scratch_bytes() { return sizeof(ScanHeader) + 2ull * kWaveMaxBlocks * 16ull; }

__device__ __forceinline__ void st_slot(void* p, unsigned long long value_bits, unsigned long long tag) {
    asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(value_bits), "l"(tag) : "memory");
}
__device__ __forceinline__ void ld_slot(const void* p, unsigned long long& value_bits, unsigned long long& tag) {
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(value_bits), "=l"(tag) : "l"(p) : "memory");
}
template <typename Acc>
__device__ __forceinline__ unsigned long long acc_bits(Acc v) {
    unsigned long long b = 0;
    memcpy(&b, &v, sizeof(Acc));
    return b;
}
template <typename Acc>
__device__ __forceinline__ Acc bits_acc(unsigned long long b) {
    Acc v;
    memcpy(&v, &b, sizeof(Acc));
    return v;
}

template <typename T, typename Acc, class Op, int VEC, bool ALIGNED, bool HAS_CARRY>
__device__ __forceinline__ void scan_long_line(const T* __restrict__ in, T* __restrict__ out, const Acc* __restrict__ carry,
                                               const uint64_t n, void* scratch) {
    constexpr int BLOCK = kScanBlockLookback;
    constexpr int VPT = kScanVpt;
    constexpr int WARPS = BLOCK / 32;
    constexpr int SPT = kWaveSlotsPerThread;
    constexpr uint32_t TILE = BLOCK * VPT * VEC;
    constexpr uint32_t WARP_ELEMS = 32 * VPT * VEC;

    ScanHeader* hdr = reinterpret_cast<ScanHeader*>(scratch);
    char* slots = reinterpret_cast<char*>(hdr + 1);
    const uint64_t total_tiles = (n + TILE - 1) / TILE;
    const uint32_t G = gridDim.x;                      // <= kWaveMaxBlocks, all resident
    const uint32_t b = blockIdx.x;

    __shared__ Vec<T, VEC> s_stage[VPT][BLOCK];
    __shared__ Acc s_warp_total[2][WARPS];
    __shared__ Acc s_gather_lt[2][WARPS];
    __shared__ Acc s_gather_all[2][WARPS];

    const int lane = threadIdx.x & 31;
    const int wid = threadIdx.x >> 5;
    int parity = 0;
    Acc running = Op::template identity<Acc>();        // prefix of all complete waves so far
    if (HAS_CARRY) running = *carry;

    uint64_t tile = b;
    if (tile < total_tiles) stage_tile<T, Op, VEC, VPT, BLOCK, ALIGNED>(in, 0, tile * TILE + (uint64_t)wid * WARP_ELEMS, n, lane, s_stage);

    for (uint64_t wave = 0; wave * G < total_tiles; ++wave, tile += G) {
        const bool active = tile < total_tiles;
        const uint64_t remaining = total_tiles - wave * G;
        const uint32_t in_wave = (uint32_t)(remaining < G ? remaining : G);    // tiles of this wave
        const uint64_t warp_off = tile * TILE + (uint64_t)wid * WARP_ELEMS;

        T raw[VPT][VEC];
        Acc base[VPT];
        Acc warp_excl = Op::template identity<Acc>();
        if (active) {
            fetch_tile<T, VEC, VPT, BLOCK>(s_stage, raw);
            const uint64_t next = tile + G;
            if (next < total_tiles)
                stage_tile<T, Op, VEC, VPT, BLOCK, ALIGNED>(in, 0, next * TILE + (uint64_t)wid * WARP_ELEMS, n, lane, s_stage);

            // ---- pass 1
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
        }
        __syncthreads();
        if (active) {
            Acc aggregate = Op::template identity<Acc>();
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const Acc v = s_warp_total[parity][w];
                if (w < wid) warp_excl = Op::apply(warp_excl, v);
                aggregate = Op::apply(aggregate, v);
            }
            if (threadIdx.x == 0)
                st_slot(slots + ((wave & 1) * kWaveMaxBlocks + b) * 16ull, acc_bits<Acc>(aggregate), wave + 1);
        }

        // ---- gather the wave: thread t owns slots [t*SPT, (t+1)*SPT)
        Acc lt = Op::template identity<Acc>();      // ordered sum of my slots that lie before block b
        Acc all = Op::template identity<Acc>();     // ordered sum of all my slots
#pragma unroll
        for (int k = 0; k < SPT; ++k) {
            const uint32_t slot = threadIdx.x * SPT + k;
            if (slot < in_wave) {
                const char* p = slots + ((wave & 1) * kWaveMaxBlocks + slot) * 16ull;
                unsigned long long bits, tag;
                uint32_t spins = 0;
                ld_slot(p, bits, tag);
                while (tag != wave + 1 && spins < kScanSpinLimit) {
                    if (spins > 8) __nanosleep(32);
                    ld_slot(p, bits, tag);
                    ++spins;
                }
                Acc v = bits_acc<Acc>(bits);
                if (tag != wave + 1) {
                    atomicExch(&hdr->status, kErrTimeout);
                    v = Op::template identity<Acc>();
                }
                all = Op::apply(all, v);
                if (slot < b) lt = Op::apply(lt, v);
            }
        }
        // ordered block reduction of both sums (threads hold consecutive slot ranges)
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const Acc far_lt = shfl_down_any(lt, d);
            const Acc far_all = shfl_down_any(all, d);
            if (lane + d < 32) {
                lt = Op::apply(lt, far_lt);
                all = Op::apply(all, far_all);
            }
        }
        if (lane == 0) {
            s_gather_lt[parity][wid] = lt;
            s_gather_all[parity][wid] = all;
        }
        __syncthreads();
        Acc in_wave_excl = Op::template identity<Acc>();
        Acc wave_total = Op::template identity<Acc>();
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            in_wave_excl = Op::apply(in_wave_excl, s_gather_lt[parity][w]);
            wave_total = Op::apply(wave_total, s_gather_all[parity][w]);
        }
        const Acc offset = Op::apply(Op::apply(running, in_wave_excl), warp_excl);
        running = Op::apply(running, wave_total);
        parity ^= 1;

        // ---- pass 2
        if (active) {
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
                    store_vec<T, VEC>(out + off, v);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        p = Op::apply(p, (Acc)raw[j][e]);
                        if (off + e < n) out[off + e] = (T)p;
                    }
                }
            }
        }
    }
    cp_async_wait_all();
}

// Reduction of n elements to one Acc, combination order fixed by the launch shape: per-thread strided partials,
// block tree, then the last block to finish combines the per-block partials in block order.
// scratch: [uint32 done_counter, pad to 16 bytes][Acc partial per block]
template <typename T, typename Acc, class Op, int VEC, bool ALIGNED>
__device__ __forceinline__ void reduce_all(const T* __restrict__ in, const uint64_t n, Acc* __restrict__ out_total,
                                           void* scratch) {
    constexpr int BLOCK = kScanBlock;
    __shared__ Acc s_part[BLOCK / 32];
    __shared__ bool s_last;
    uint32_t* counter = reinterpret_cast<uint32_t*>(scratch);
    Acc* partials = reinterpret_cast<Acc*>(reinterpret_cast<char*>(scratch) + 16);

    Acc acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = Op::template identity<Acc>();
    const uint64_t nvec = ALIGNED ? n / VEC : 0;
    const uint64_t stride = (uint64_t)gridDim.x * BLOCK;
    uint64_t g = (uint64_t)blockIdx.x * BLOCK + threadIdx.x;
    // four independent vectors in flight per thread
    for (; g + 3 * stride < nvec; g += 4 * stride) {
        Vec<T, VEC> v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = load_vec<T, VEC>(in + (g + u * stride) * VEC);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[u] = Op::apply(acc[u], (Acc)v[u].v[e]);
    }
    for (; g < nvec; g += stride) {
        const Vec<T, VEC> v = load_vec<T, VEC>(in + g * VEC);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[0] = Op::apply(acc[0], (Acc)v.v[e]);
    }
    for (uint64_t i = nvec * VEC + (uint64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += stride)
        acc[0] = Op::apply(acc[0], (Acc)in[i]);
    Acc t = Op::apply(Op::apply(acc[0], acc[1]), Op::apply(acc[2], acc[3]));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        Acc y;
        if constexpr (sizeof(Acc) == 8) {
            long long xx = *reinterpret_cast<long long*>(&t);
            xx = __shfl_down_sync(0xffffffffu, xx, d);
            y = *reinterpret_cast<Acc*>(&xx);
        } else {
            y = __shfl_down_sync(0xffffffffu, t, d);
        }
        t = Op::apply(t, y);
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) s_part[wid] = t;
    __syncthreads();
    if (threadIdx.x == 0) {
        Acc b = Op::template identity<Acc>();
        for (int w = 0; w < BLOCK / 32; ++w) b = Op::apply(b, s_part[w]);
        partials[blockIdx.x] = b;
        __threadfence();
        const uint32_t ticket = atomicAdd(counter, 1u);
        s_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        __threadfence();
        Acc total = Op::template identity<Acc>();
        for (uint32_t b = 0; b < gridDim.x; ++b) total = Op::apply(total, *(volatile Acc*)&partials[b]);
        *out_total = total;
    }
}

}  // namespace ovl
