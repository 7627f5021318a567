// Cooperative per-worker reduction loops (sm_100a).
//
// The operator language writes a reduction as one worker folding a term into an accumulator over a counted loop
// (opveclib/test/test_dot_product.py:18-34).  The generated `_red` kernels give the loop of one worker to a group
// of threads - a warp, or a whole block for long loops: member m evaluates the terms m, m + GROUP, m + 2 GROUP ...
// (neighbouring members touch neighbouring elements, so row-major reads coalesce), keeps a private partial result
// and group_reduce combines the partials in a fixed order.  Partials are kept in the accumulator's own type:
// integer results are exactly those of the serial loop; floating-point results differ from it only by the order
// of the additions.  Loops whose reads are strided along the loop variable but contiguous across workers (column
// sums) get the other layout, written out by the code generator: a warp is 32 neighbouring workers, the block's warps
// take slices of the loop and the slices meet in shared memory.  When the workers are too few to occupy the device
// and their loops are long, the code generator also cuts every loop into slices for different blocks: a block leaves
// its slice's result in the worker's row of a scratch array and takes a ticket from the worker's counter; the block
// with the last ticket folds the row in slice order and finishes the worker.
#pragma once
#include "ovl_scan.cuh"

namespace ovl {

// Combination of the partials of GROUP consecutive threads (GROUP = 32: a warp; otherwise the whole block, which
// must then have exactly GROUP threads and call this from converged code).  Every member receives the result.
// `smem` holds one value per warp of the block.
template <typename A, class Op, int GROUP>
__device__ __forceinline__ A group_reduce(A v, A* smem) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = Op::template apply<A>(v, shfl_xor_any(v, d));
    if constexpr (GROUP == 32) {
        return v;
    } else {
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
        if (lane == 0) smem[wid] = v;
        __syncthreads();
        A t = smem[0];
#pragma unroll
        for (int w = 1; w < GROUP / 32; ++w) t = Op::template apply<A>(t, smem[w]);
        __syncthreads();            // the next call may overwrite smem
        return t;
    }
}

}  // namespace ovl
