// libovl_b200.so - C-ABI launcher for generated sm_100a kernels plus the built-in fp32 scans.
// Interface and the reference code each entry point replaces: include/ovl_b200.h.
//
// Uses the CUDA runtime only (statically linked): cubins are loaded with cudaLibraryLoadData and launched with
// cudaLaunchKernel on the caller's stream, in the caller's (primary) context - no private context, unlike the
// reference harness (opveclib/testcudaop.cc:69-75).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <mutex>
#include <string>
#include <atomic>
#include <vector>

#include "../../include/ovl_b200.h"
#include "templates/ovl_scan.cuh"

namespace {

thread_local int g_last_cuda_error = 0;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    (void)cudaGetLastError();   // the runtime also remembers the error; clear it so that a later, unrelated
                                // cudaGetLastError() after a kernel launch does not report it again
    return OVL_ERR_CUDA;
}
#define OVL_CUDA(call)                                   \
    do {                                                 \
        cudaError_t e__ = (call);                        \
        if (e__ != cudaSuccess) return cuda_fail(e__);   \
    } while (0)

size_t dtype_size(int32_t d) {
    switch (d) {
        case OVL_FLOAT16: case OVL_INT16: case OVL_UINT16: return 2;
        case OVL_FLOAT32: case OVL_INT32: case OVL_UINT32: return 4;
        case OVL_FLOAT64: case OVL_INT64: case OVL_UINT64: return 8;
        case OVL_INT8: case OVL_UINT8: return 1;
        default: return 0;
    }
}

}  // namespace

struct OvlModule {
    cudaLibrary_t lib;
};

struct OvlKernel {
    cudaKernel_t fn;
    std::string symbol;
    uint32_t grid_x, block_x, dynamic_smem;
    std::vector<int32_t> dtypes;
    std::vector<uint64_t> lens;
    std::vector<uint32_t> align;
    uint32_t n_in, n_out;
    uint64_t scratch_bytes, scratch_zero_bytes;
    bool cooperative;
};

extern "C" const char* ovl_version(void) { return "ovl_b200 0.1.0 (sm_100a)"; }

extern "C" const char* ovl_status_string(int s) {
    switch (s) {
        case OVL_OK: return "ok";
        case OVL_ERR_ARITY: return "wrong number of input or output tensors";
        case OVL_ERR_LENGTH: return "tensor element count does not match the kernel signature";
        case OVL_ERR_DTYPE: return "tensor dtype does not match the kernel signature";
        case OVL_ERR_NULL: return "null pointer";
        case OVL_ERR_CUDA: return "CUDA error";
        case OVL_ERR_NOT_FOUND: return "kernel symbol not found in module";
        case OVL_ERR_SCRATCH: return "scratch buffer missing, too small or misaligned";
        case OVL_ERR_TIMEOUT: return "bounded device-side wait expired";
        case OVL_ERR_ALIGNMENT: return "tensor pointer alignment too small for this kernel";
        case OVL_ERR_TOO_LARGE: return "size beyond what this entry point supports";
        case OVL_ERR_INVALID: return "malformed specification";
        default: return "unknown status";
    }
}

extern "C" int ovl_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int ovl_device_sm_count(int* out_count) {
    if (!out_count) return OVL_ERR_NULL;
    int dev = 0;
    OVL_CUDA(cudaGetDevice(&dev));
    OVL_CUDA(cudaDeviceGetAttribute(out_count, cudaDevAttrMultiProcessorCount, dev));
    return OVL_OK;
}

extern "C" int ovl_module_load(const void* image, size_t size, OvlModule** out_module) {
    (void)size;
    if (!image || !out_module) return OVL_ERR_NULL;
    cudaLibrary_t lib;
    OVL_CUDA(cudaLibraryLoadData(&lib, image, nullptr, nullptr, 0, nullptr, nullptr, 0));
    *out_module = new OvlModule{lib};
    return OVL_OK;
}

extern "C" int ovl_module_load_file(const char* path, OvlModule** out_module) {
    if (!path || !out_module) return OVL_ERR_NULL;
    cudaLibrary_t lib;
    OVL_CUDA(cudaLibraryLoadFromFile(&lib, path, nullptr, nullptr, 0, nullptr, nullptr, 0));
    *out_module = new OvlModule{lib};
    return OVL_OK;
}

extern "C" int ovl_module_unload(OvlModule* module) {
    if (!module) return OVL_ERR_NULL;
    cudaError_t e = cudaLibraryUnload(module->lib);
    delete module;
    if (e != cudaSuccess) return cuda_fail(e);
    return OVL_OK;
}

extern "C" int ovl_kernel_create(OvlModule* module, const OvlKernelSpec* spec, OvlKernel** out_kernel) {
    if (!module || !spec || !out_kernel || !spec->symbol) return OVL_ERR_NULL;
    const uint32_t n = spec->n_inputs + spec->n_outputs;
    if (spec->grid_x == 0 || spec->block_x == 0 || spec->block_x > 1024) return OVL_ERR_INVALID;
    if (n > 0 && (!spec->dtypes || !spec->lens)) return OVL_ERR_NULL;
    if (spec->scratch_zero_bytes > spec->scratch_bytes) return OVL_ERR_INVALID;
    cudaKernel_t fn;
    cudaError_t e = cudaLibraryGetKernel(&fn, module->lib, spec->symbol);
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        (void)cudaGetLastError();
        return OVL_ERR_NOT_FOUND;
    }
    OvlKernel* k = new OvlKernel();
    k->fn = fn;
    k->symbol = spec->symbol;
    k->grid_x = spec->grid_x;
    k->block_x = spec->block_x;
    k->dynamic_smem = spec->dynamic_smem_bytes;
    k->n_in = spec->n_inputs;
    k->n_out = spec->n_outputs;
    k->dtypes.assign(spec->dtypes, spec->dtypes + n);
    k->lens.assign(spec->lens, spec->lens + n);
    if (spec->align_bytes) k->align.assign(spec->align_bytes, spec->align_bytes + n);
    else k->align.assign(n, 0);
    k->scratch_bytes = spec->scratch_bytes;
    k->scratch_zero_bytes = spec->scratch_zero_bytes;
    k->cooperative = (spec->flags & OVL_KERNEL_COOPERATIVE) != 0;
    if (k->dynamic_smem > 48u * 1024u) {
        // beyond the default limit: opt in, for the current device
        e = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k->dynamic_smem);
        if (e != cudaSuccess) {
            delete k;
            return cuda_fail(e);
        }
    }
    for (uint32_t i = 0; i < n; ++i)
        if (dtype_size(k->dtypes[i]) == 0) {
            delete k;
            return OVL_ERR_DTYPE;
        }
    *out_kernel = k;
    return OVL_OK;
}

extern "C" int ovl_kernel_destroy(OvlKernel* kernel) {
    if (!kernel) return OVL_ERR_NULL;
    delete kernel;
    return OVL_OK;
}

namespace {

// signature checks of the reference's generated stub (opveclib/expression.py:662-663, 622, 639), plus dtype,
// null and alignment checks
int validate(const OvlKernel* k, const OvlTensor* in, size_t n_in, const OvlTensor* out, size_t n_out, const void* scratch,
             uint64_t scratch_bytes) {
    if (!k) return OVL_ERR_NULL;
    if (n_in != k->n_in || n_out != k->n_out) return OVL_ERR_ARITY;
    if ((n_in && !in) || (n_out && !out)) return OVL_ERR_NULL;
    for (size_t i = 0; i < n_in + n_out; ++i) {
        const OvlTensor& t = (i < n_in) ? in[i] : out[i - n_in];
        if (t.len != k->lens[i]) return OVL_ERR_LENGTH;
        if (t.dtype != k->dtypes[i]) return OVL_ERR_DTYPE;
        if (!t.data) return OVL_ERR_NULL;
        if (k->align[i] > 1 && ((uintptr_t)t.data % k->align[i]) != 0) return OVL_ERR_ALIGNMENT;
    }
    if (k->scratch_bytes) {
        if (!scratch || scratch_bytes < k->scratch_bytes || ((uintptr_t)scratch % 16) != 0) return OVL_ERR_SCRATCH;
    }
    return OVL_OK;
}

int enqueue(const OvlKernel* k, const OvlTensor* in, size_t n_in, const OvlTensor* out, size_t n_out, void* scratch,
            cudaStream_t stream) {
    void* ptrs[64];
    void* args[64];
    size_t n = 0;
    if (n_in + n_out + 1 > 64) return OVL_ERR_TOO_LARGE;
    for (size_t i = 0; i < n_in; ++i) ptrs[n++] = in[i].data;
    for (size_t i = 0; i < n_out; ++i) ptrs[n++] = out[i].data;
    if (k->scratch_bytes) ptrs[n++] = scratch;
    for (size_t i = 0; i < n; ++i) args[i] = &ptrs[i];
    if (k->scratch_zero_bytes) OVL_CUDA(cudaMemsetAsync(scratch, 0, k->scratch_zero_bytes, stream));
    if (k->cooperative)
        OVL_CUDA(cudaLaunchCooperativeKernel((const void*)k->fn, dim3(k->grid_x), dim3(k->block_x), args, k->dynamic_smem, stream));
    else
        OVL_CUDA(cudaLaunchKernel((const void*)k->fn, dim3(k->grid_x), dim3(k->block_x), args, k->dynamic_smem, stream));
    return OVL_OK;
}

}  // namespace

extern "C" int ovl_launch(OvlKernel* kernel, const OvlTensor* inputs, size_t n_inputs, const OvlTensor* outputs,
                          size_t n_outputs, void* scratch, uint64_t scratch_bytes, void* cuda_stream) {
    int st = validate(kernel, inputs, n_inputs, outputs, n_outputs, scratch, scratch_bytes);
    if (st != OVL_OK) return st;
    return enqueue(kernel, inputs, n_inputs, outputs, n_outputs, scratch, (cudaStream_t)cuda_stream);
}

extern "C" int ovl_profile(OvlKernel* kernel, const OvlTensor* inputs, size_t n_inputs, const OvlTensor* outputs,
                           size_t n_outputs, void* scratch, uint64_t scratch_bytes, void* cuda_stream,
                           uint32_t iterations, float* ms) {
    int st = validate(kernel, inputs, n_inputs, outputs, n_outputs, scratch, scratch_bytes);
    if (st != OVL_OK) return st;
    if (iterations && !ms) return OVL_ERR_NULL;
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    cudaEvent_t a, b;
    OVL_CUDA(cudaEventCreate(&a));
    OVL_CUDA(cudaEventCreate(&b));
    int rc = OVL_OK;
    for (uint32_t it = 0; it < iterations && rc == OVL_OK; ++it) {
        cudaEventRecord(a, stream);
        rc = enqueue(kernel, inputs, n_inputs, outputs, n_outputs, scratch, stream);
        cudaEventRecord(b, stream);
        cudaError_t e = cudaEventSynchronize(b);
        if (rc == OVL_OK && e != cudaSuccess) rc = cuda_fail(e);
        if (rc == OVL_OK) cudaEventElapsedTime(&ms[it], a, b);
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    return rc;
}

extern "C" int ovl_run_host(OvlKernel* kernel, const OvlTensor* host_inputs, size_t n_inputs,
                            const OvlTensor* host_outputs, size_t n_outputs, uint32_t iterations, float* ms) {
    if (!kernel) return OVL_ERR_NULL;
    if (n_inputs != kernel->n_in || n_outputs != kernel->n_out) return OVL_ERR_ARITY;
    if ((n_inputs && !host_inputs) || (n_outputs && !host_outputs)) return OVL_ERR_NULL;
    std::vector<OvlTensor> din(n_inputs), dout(n_outputs);
    std::vector<void*> owned;
    void* scratch = nullptr;
    int rc = OVL_OK;
    auto cleanup = [&]() {
        for (void* p : owned) cudaFree(p);
    };
    for (size_t i = 0; i < n_inputs + n_outputs && rc == OVL_OK; ++i) {
        const bool is_in = i < n_inputs;
        const OvlTensor& h = is_in ? host_inputs[i] : host_outputs[i - n_inputs];
        if (!h.data) { rc = OVL_ERR_NULL; break; }
        const size_t bytes = (size_t)h.len * dtype_size(h.dtype);
        void* d = nullptr;
        cudaError_t e = cudaMalloc(&d, bytes ? bytes : 1);
        if (e != cudaSuccess) { rc = cuda_fail(e); break; }
        owned.push_back(d);
        if (is_in) e = cudaMemcpy(d, h.data, bytes, cudaMemcpyHostToDevice);
        else e = cudaMemset(d, 0xFE, bytes);   // unwritten elements show up as 0xFE, as in testcudaop.cc:186-196
        if (e != cudaSuccess) { rc = cuda_fail(e); break; }
        OvlTensor t = {d, h.dtype, h.len};
        if (is_in) din[i] = t; else dout[i - n_inputs] = t;
    }
    if (rc == OVL_OK && kernel->scratch_bytes) {
        cudaError_t e = cudaMalloc(&scratch, kernel->scratch_bytes);
        if (e != cudaSuccess) rc = cuda_fail(e);
        else owned.push_back(scratch);
    }
    if (rc == OVL_OK) {
        if (iterations == 0) iterations = 1;
        std::vector<float> local(iterations);
        rc = ovl_profile(kernel, din.data(), n_inputs, dout.data(), n_outputs, scratch, kernel->scratch_bytes, nullptr,
                         iterations, local.data());
        if (rc == OVL_OK && ms) memcpy(ms, local.data(), iterations * sizeof(float));
    }
    if (rc == OVL_OK && kernel->scratch_bytes) {
        int32_t status = 0;
        rc = ovl_read_kernel_status(scratch, nullptr, &status);
        if (rc == OVL_OK && status != 0) rc = status;
    }
    for (size_t i = 0; i < n_outputs && rc == OVL_OK; ++i) {
        const size_t bytes = (size_t)host_outputs[i].len * dtype_size(host_outputs[i].dtype);
        cudaError_t e = cudaMemcpy(host_outputs[i].data, dout[i].data, bytes, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) rc = cuda_fail(e);
    }
    cleanup();
    return rc;
}

extern "C" int ovl_read_kernel_status(const void* scratch, void* cuda_stream, int32_t* out_status) {
    if (!scratch || !out_status) return OVL_ERR_NULL;
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    OVL_CUDA(cudaMemcpyAsync(out_status, scratch, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    OVL_CUDA(cudaStreamSynchronize(stream));
    return OVL_OK;
}

// ---------------------------------------------------------------------------------------------------------
// built-in fp32 scans and reductions

namespace {

template <class Op, bool ALIGNED, bool HAS_CARRY, int MODE>
__global__ void __launch_bounds__(MODE == ovl::kScanLookback ? ovl::kScanBlockLookback : ovl::kScanBlock,
                                  MODE == ovl::kScanLookback ? 4 : 2)
    scan_f32_kernel(const float* __restrict__ in, float* __restrict__ out, const double* __restrict__ carry, uint64_t lines,
                    uint64_t n, void* scratch) {
    ovl::scan_lines<float, double, Op, 4, ALIGNED, HAS_CARRY, MODE>(in, out, carry, lines, n, scratch);
}

template <class Op, bool ALIGNED>
__global__ void __launch_bounds__(ovl::kScanBlock, 2) tile_aggregates_f32_kernel(const float* __restrict__ in, uint64_t lines,
                                                                                uint64_t n, double* __restrict__ agg) {
    ovl::tile_aggregates<float, double, Op, 4, ALIGNED>(in, lines, n, agg);
}

template <class Op, bool HAS_CARRY, bool WRITE_PREFIX>
__global__ void __launch_bounds__(ovl::kScanBlock) scan_aggregates_f64_kernel(double* __restrict__ agg, uint64_t lines,
                                                                             uint64_t tiles_per_line,
                                                                             const double* __restrict__ carry,
                                                                             double* __restrict__ total_out) {
    ovl::scan_aggregates<double, Op, HAS_CARRY, WRITE_PREFIX>(agg, lines, tiles_per_line, carry, total_out);
}

template <class Op, bool ALIGNED>
__global__ void __launch_bounds__(ovl::kScanBlock) reduce_f32_kernel(const float* __restrict__ in, uint64_t n,
                                                                    double* __restrict__ out_total, void* scratch) {
    ovl::reduce_all<float, double, Op, 4, ALIGNED>(in, n, out_total, scratch);
}

template <class Op, bool HAS_CARRY, bool MULTI>
__global__ void __launch_bounds__(ovl::kRingThreads, 1) scan_ring_f32_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                            const double* __restrict__ carry, uint64_t lines,
                                                                            uint64_t n, void* scratch) {
    ovl::scan_ring<float, double, Op, 4, HAS_CARRY, MULTI>(in, out, carry, lines, n, scratch);
}

// several lines, each scanned by a group of blocks of its own (or by one block)
template <class Op>
__global__ void __launch_bounds__(ovl::kRingThreads, 1) scan_ring_grouped_f32_kernel(const float* __restrict__ in,
                                                                                    float* __restrict__ out,
                                                                                    const double* __restrict__ carry,
                                                                                    uint64_t lines, uint64_t n, void* scratch) {
    ovl::scan_ring<float, double, Op, 4, false, false, false, false, true>(in, out, nullptr, lines, n, scratch);
}

// the bounded-wait self-test: block `withhold_block` keeps its aggregates to itself, waits use the short bound
template <class Op>
__global__ void __launch_bounds__(ovl::kRingThreads, 1) scan_ring_selftest_f32_kernel(const float* __restrict__ in,
                                                                                     float* __restrict__ out, uint64_t n,
                                                                                     void* scratch, int withhold_block) {
    ovl::scan_ring<float, double, Op, 4, false, false, true>(in, out, nullptr, 1, n, scratch, withhold_block);
}

// the pair of a sharded scan whose totals travel through peer memory (the exchange is a __grid_constant__ parameter:
// its address can be taken without every thread copying it to local memory)
template <class Op>
__global__ void __launch_bounds__(ovl::kScanBlock) reduce_publish_f32_kernel(const float* __restrict__ in, uint64_t n,
                                                                            double* __restrict__ out_total, void* scratch,
                                                                            const __grid_constant__ ovl::PeerExchange px) {
    ovl::reduce_all<float, double, Op, 4, true>(in, n, out_total, scratch, &px);
}

template <class Op>
__global__ void __launch_bounds__(ovl::kRingThreads, 1) scan_ring_peer_f32_kernel(const float* __restrict__ in,
                                                                                 float* __restrict__ out, uint64_t n,
                                                                                 void* scratch,
                                                                                 const __grid_constant__ ovl::PeerExchange px) {
    ovl::scan_ring<float, double, Op, 4, true, false, false, true>(in, out, nullptr, 1, n, scratch, -1, &px);
}

template <class Op>
__global__ void __launch_bounds__(ovl::kWarpScanBlock) scan_warp_f32_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                          uint64_t lines, uint64_t n) {
    ovl::scan_lines_warp<float, double, Op, 4>(in, out, lines, n);
}

template <class Op>
__global__ void __launch_bounds__(ovl::kShortScanBlock) scan_short_f32_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                             uint64_t lines, uint32_t n) {
    ovl::scan_lines_short<float, double, Op, 4>(in, out, lines, n);
}

// from this many lines on (all starting on 16-byte boundaries) a warp scans a whole line by itself
constexpr uint64_t kWarpScanMinLines = 2048;

// a line of at most kTile elements is one tile; longer lines are cut into tiles of kTile elements (three-pass
// scan) or kTileLookback elements (single-pass look-back scan)
constexpr uint64_t kTile = (uint64_t)ovl::kScanBlock * ovl::kScanVpt * 4;
constexpr uint64_t kTileLookback = (uint64_t)ovl::kScanBlockLookback * ovl::kScanVpt * 4;

inline uint64_t tiles_per_line(uint64_t n, bool lookback) {
    if (n <= kTile) return 1;
    const uint64_t t = lookback ? kTileLookback : kTile;
    return (n + t - 1) / t;
}

// SM count of the current device (looked up once per device)
int sm_count_cached() {
    constexpr int kMaxDevices = 64;
    static std::atomic<int> sms[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    int v = sms[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
        sms[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

// How a single line of several tiles is scanned.  Default: the ring scan (one launch, 8 bytes per element).
// OVL_SCAN_MODE=threepass selects the three streaming passes (12 bytes per element; also what lines that are not
// 16-byte aligned and several long lines in one call use), OVL_SCAN_MODE=lookback the single-pass decoupled
// look-back kernel.
enum { kModeRing = 0, kModeThreePass = 1, kModeLookback = 2 };
int long_line_mode() {
    static int cached = -1;
    if (cached < 0) {
        const char* e = getenv("OVL_SCAN_MODE");
        if (e && strcmp(e, "lookback") == 0) cached = kModeLookback;
        else if (e && strcmp(e, "threepass") == 0) cached = kModeThreePass;
        else cached = kModeRing;
    }
    return cached;
}
bool use_lookback() { return long_line_mode() == kModeLookback; }

inline uint32_t clamp_grid(uint64_t tiles, uint64_t per_sm) {
    const uint64_t cap = (uint64_t)sm_count_cached() * per_sm;
    const uint64_t g = tiles < cap ? tiles : cap;
    return (uint32_t)(g ? g : 1);
}

// pass 1 of the three-pass scan: per-tile aggregates into the scratch (after the header)
template <class Op>
cudaError_t launch_tile_aggregates(const float* in, uint64_t lines, uint64_t n, void* scratch, bool aligned,
                                   cudaStream_t stream) {
    double* agg = reinterpret_cast<double*>(reinterpret_cast<char*>(scratch) + sizeof(ovl::ScanHeader));
    const uint32_t grid = clamp_grid(tiles_per_line(n, false) * lines, 2);
    if (aligned) tile_aggregates_f32_kernel<Op, true><<<grid, ovl::kScanBlock, 0, stream>>>(in, lines, n, agg);
    else tile_aggregates_f32_kernel<Op, false><<<grid, ovl::kScanBlock, 0, stream>>>(in, lines, n, agg);
    return cudaGetLastError();
}

// pass 2: exclusive prefixes of the aggregates (optionally seeded with the carry), and/or the line totals
template <class Op>
cudaError_t launch_scan_aggregates(void* scratch, uint64_t lines, uint64_t n, const double* carry, double* total_out,
                                   bool write_prefix, cudaStream_t stream) {
    double* agg = reinterpret_cast<double*>(reinterpret_cast<char*>(scratch) + sizeof(ovl::ScanHeader));
    const uint64_t tpl = tiles_per_line(n, false);
    const uint32_t grid = clamp_grid(lines, 4);
    if (write_prefix) {
        if (carry) scan_aggregates_f64_kernel<Op, true, true><<<grid, ovl::kScanBlock, 0, stream>>>(agg, lines, tpl, carry, total_out);
        else scan_aggregates_f64_kernel<Op, false, true><<<grid, ovl::kScanBlock, 0, stream>>>(agg, lines, tpl, carry, total_out);
    } else {
        scan_aggregates_f64_kernel<Op, false, false><<<grid, ovl::kScanBlock, 0, stream>>>(agg, lines, tpl, carry, total_out);
    }
    return cudaGetLastError();
}

template <class Op, bool ALIGNED, bool HAS_CARRY>
cudaError_t launch_scan_mode(const float* in, float* out, uint64_t lines, uint64_t n, const double* carry, void* scratch,
                             int mode, cudaStream_t stream) {
    if (mode == ovl::kScanOneTile) {
        scan_f32_kernel<Op, ALIGNED, HAS_CARRY, ovl::kScanOneTile><<<clamp_grid(lines, 2), ovl::kScanBlock, 0, stream>>>(
            in, out, carry, lines, n, scratch);
        return cudaGetLastError();
    }
    if (mode == ovl::kScanPrefixed) {
        scan_f32_kernel<Op, ALIGNED, false, ovl::kScanPrefixed>
            <<<clamp_grid(tiles_per_line(n, false) * lines, 2), ovl::kScanBlock, 0, stream>>>(in, out, nullptr, lines, n, scratch);
        return cudaGetLastError();
    }
    // look-back: blocks wait for each other's aggregates, so all of them must be resident at once - a
    // cooperative launch with the grid clamped to what the device holds
    auto kernel = scan_f32_kernel<Op, ALIGNED, HAS_CARRY, ovl::kScanLookback>;
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, ovl::kScanBlockLookback, 0);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    const uint32_t grid = clamp_grid(tiles_per_line(n, true) * lines, (uint64_t)per_sm);
    void* args[] = {(void*)&in, (void*)&out, (void*)&carry, (void*)&lines, (void*)&n, (void*)&scratch};
    return cudaLaunchCooperativeKernel((const void*)kernel, dim3(grid), dim3(ovl::kScanBlockLookback), args, 0, stream);
}

template <class Op>
cudaError_t launch_scan_pass(const float* in, float* out, uint64_t lines, uint64_t n, const double* carry, void* scratch,
                             bool aligned, int mode, cudaStream_t stream) {
    if (aligned) {
        if (carry) return launch_scan_mode<Op, true, true>(in, out, lines, n, carry, scratch, mode, stream);
        return launch_scan_mode<Op, true, false>(in, out, lines, n, carry, scratch, mode, stream);
    }
    if (carry) return launch_scan_mode<Op, false, true>(in, out, lines, n, carry, scratch, mode, stream);
    return launch_scan_mode<Op, false, false>(in, out, lines, n, carry, scratch, mode, stream);
}

// ring scan of long lines: clear the aggregate words, then one cooperative launch with a block per SM
template <class Op>
int launch_ring(const float* in, float* out, uint64_t lines, uint64_t n, const double* carry, void* scratch,
                cudaStream_t stream, int withhold_block = -1) {
    const uint64_t tiles = ((n + kTile - 1) / kTile) * lines;
    uint64_t cap = (uint64_t)sm_count_cached();
    if (cap > (uint64_t)ovl::kRingMaxGrid) cap = ovl::kRingMaxGrid;
    const uint32_t grid = (uint32_t)(tiles < cap ? tiles : cap);
    const size_t smem = (size_t)ovl::kRingSlots * kTile * sizeof(float) + ovl::kRingCtlBytes;
    // (a carry is only accepted together with a single line)
    if (withhold_block >= 0) {
        const void* kernel = (const void*)scan_ring_selftest_f32_kernel<Op>;
        OVL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        OVL_CUDA(cudaMemsetAsync(scratch, 0, sizeof(ovl::ScanHeader) + tiles * 16, stream));
        void* args[] = {(void*)&in, (void*)&out, (void*)&n, (void*)&scratch, (void*)&withhold_block};
        OVL_CUDA(cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(ovl::kRingThreads), args, smem, stream));
        return OVL_OK;
    }
    // several lines: groups of blocks that take whole lines when that keeps the grid busy, else waves across line ends
    const bool grouped = lines > 1 && getenv("OVL_RING_LAYOUT") == nullptr &&
                         ovl::ring_group_efficiency(grid, lines, (n + kTile - 1) / kTile) >= ovl::kRingGroupedMinEfficiency;
    const void* kernel = grouped   ? (const void*)scan_ring_grouped_f32_kernel<Op>
                         : lines > 1 ? (const void*)scan_ring_f32_kernel<Op, false, true>
                         : carry   ? (const void*)scan_ring_f32_kernel<Op, true, false>
                                   : (const void*)scan_ring_f32_kernel<Op, false, false>;
    OVL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    OVL_CUDA(cudaMemsetAsync(scratch, 0, sizeof(ovl::ScanHeader) + tiles * 16, stream));
    void* args[] = {(void*)&in, (void*)&out, (void*)&carry, (void*)&lines, (void*)&n, (void*)&scratch};
    OVL_CUDA(cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(ovl::kRingThreads), args, smem, stream));
    return OVL_OK;
}

int check_scan_args(int op, const void* in, uint64_t lines, uint64_t n, const double* carry, const void* scratch,
                    uint64_t scratch_bytes) {
    if (!in) return OVL_ERR_NULL;
    if (op != 0 && op != 1) return OVL_ERR_INVALID;
    if (lines == 0 || n == 0) return OVL_ERR_INVALID;
    if (carry && lines != 1) return OVL_ERR_INVALID;
    if (!scratch || scratch_bytes < ovl_scan_f32_scratch_bytes(lines, n) || ((uintptr_t)scratch % 16) != 0)
        return OVL_ERR_SCRATCH;
    if (tiles_per_line(n, true) * lines >= (1ull << 32) - 65536) return OVL_ERR_TOO_LARGE;
    return OVL_OK;
}

}  // namespace

extern "C" uint64_t ovl_scan_f32_scratch_bytes(uint64_t lines, uint64_t n) {
    // header + one 32-byte slot per tile; sized for the finer (look-back) tiling so either scan mode fits
    return ovl::scan_scratch_bytes<double>(tiles_per_line(n, true) * lines);
}

namespace {

// second half of a scan: prefixes of the tile aggregates (seeded with the carry), then the seeded tile scans
template <class Op>
int finish_scan(const float* in, float* out, uint64_t lines, uint64_t n, const double* carry, void* scratch, bool aligned,
                cudaStream_t stream) {
    cudaError_t e = launch_scan_aggregates<Op>(scratch, lines, n, carry, nullptr, true, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    e = launch_scan_pass<Op>(in, out, lines, n, nullptr, scratch, aligned, ovl::kScanPrefixed, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    return OVL_OK;
}

template <class Op>
int run_scan(const float* in, float* out, uint64_t lines, uint64_t n, const double* carry, void* scratch, bool aligned,
             cudaStream_t stream) {
    if (aligned && !carry && ovl::scan_short_line(n, 4) && lines * n >= ovl::kShortScanMinElements &&
        long_line_mode() == kModeRing) {
        // short lines: the tensor streamed as a flat array, as many whole lines per warp as fit into 128 vectors
        const uint64_t per_chunk = 128 / (n / 4);
        const uint64_t spans = ((lines + per_chunk - 1) / per_chunk + 3) / 4;       // four warps per block
        const uint64_t cap = (uint64_t)sm_count_cached() * 128;
        scan_short_f32_kernel<Op><<<(uint32_t)(spans < cap ? spans : cap), ovl::kShortScanBlock, 0, stream>>>(in, out, lines,
                                                                                                            (uint32_t)n);
        cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? OVL_OK : cuda_fail(e);
    }
    if (aligned && !carry && lines >= kWarpScanMinLines && n % 4 == 0 && long_line_mode() == kModeRing) {
        const ovl::WarpScanShape shape = ovl::warp_scan_shape(lines, (uint32_t)sm_count_cached());
        scan_warp_f32_kernel<Op><<<shape.grid, shape.block, 0, stream>>>(in, out, lines, n);
        cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? OVL_OK : cuda_fail(e);
    }
    if (n <= kTile) {
        cudaError_t e = launch_scan_pass<Op>(in, out, lines, n, carry, scratch, aligned, ovl::kScanOneTile, stream);
        return e == cudaSuccess ? OVL_OK : cuda_fail(e);
    }
    if (aligned && long_line_mode() == kModeRing) return launch_ring<Op>(in, out, lines, n, carry, scratch, stream);
    if (use_lookback()) {
        // the descriptors must start out empty
        OVL_CUDA(cudaMemsetAsync(scratch, 0, ovl_scan_f32_scratch_bytes(lines, n), stream));
        cudaError_t e = launch_scan_pass<Op>(in, out, lines, n, carry, scratch, aligned, ovl::kScanLookback, stream);
        return e == cudaSuccess ? OVL_OK : cuda_fail(e);
    }
    cudaError_t e = launch_tile_aggregates<Op>(in, lines, n, scratch, aligned, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    return finish_scan<Op>(in, out, lines, n, carry, scratch, aligned, stream);
}

}  // namespace

extern "C" int ovl_scan_f32(int op, const float* in, float* out, uint64_t lines, uint64_t n, const double* carry,
                            void* scratch, uint64_t scratch_bytes, void* cuda_stream) {
    if (!out) return OVL_ERR_NULL;
    int st = check_scan_args(op, in, lines, n, carry, scratch, scratch_bytes);
    if (st != OVL_OK) return st;
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const bool aligned = ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0) && (lines == 1 || n % 4 == 0);
    OVL_CUDA(cudaMemsetAsync(scratch, 0, sizeof(ovl::ScanHeader), stream));   // status word
    if (op == 0) return run_scan<ovl::OpAdd>(in, out, lines, n, carry, scratch, aligned, stream);
    return run_scan<ovl::OpMul>(in, out, lines, n, carry, scratch, aligned, stream);
}

extern "C" int ovl_selftest_scan_timeout(const float* in, float* out, uint64_t n, void* scratch, uint64_t scratch_bytes,
                                         void* cuda_stream) {
    if (!out) return OVL_ERR_NULL;
    int st = check_scan_args(0, in, 1, n, nullptr, scratch, scratch_bytes);
    if (st != OVL_OK) return st;
    if (n <= kTile || ((uintptr_t)in % 16) != 0 || ((uintptr_t)out % 16) != 0) return OVL_ERR_INVALID;
    return launch_ring<ovl::OpAdd>(in, out, 1, n, nullptr, scratch, (cudaStream_t)cuda_stream, /*withhold_block=*/0);
}

namespace {

// total of n elements into *out_total; `scratch` holds ovl_reduce_f32_scratch_bytes(n) bytes
int launch_reduce(int op, const float* in, uint64_t n, double* out_total, void* scratch, cudaStream_t stream) {
    const bool aligned = ((uintptr_t)in % 16 == 0);
    const uint32_t grid = (uint32_t)ovl::reduce_chunks(n);       // one block per chunk
    OVL_CUDA(cudaMemsetAsync(scratch, 0, 16, stream));
    if (op == 0) {
        if (aligned) reduce_f32_kernel<ovl::OpAdd, true><<<grid, ovl::kScanBlock, 0, stream>>>(in, n, out_total, scratch);
        else reduce_f32_kernel<ovl::OpAdd, false><<<grid, ovl::kScanBlock, 0, stream>>>(in, n, out_total, scratch);
    } else {
        if (aligned) reduce_f32_kernel<ovl::OpMul, true><<<grid, ovl::kScanBlock, 0, stream>>>(in, n, out_total, scratch);
        else reduce_f32_kernel<ovl::OpMul, false><<<grid, ovl::kScanBlock, 0, stream>>>(in, n, out_total, scratch);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e);
    return OVL_OK;
}

// The begin/finish pair of a shard: when the shard can be scanned by the ring scan, `begin` only needs the
// shard's total (one streaming read) and `finish` is the ring scan seeded with the carry; otherwise `begin` leaves
// per-tile aggregates in the scratch for the seeded tile scans of `finish`.  Both sides evaluate this predicate.
bool shard_uses_ring(const float* in, uint64_t n) {
    return long_line_mode() == kModeRing && n > kTile && ((uintptr_t)in % 16 == 0) &&
           ovl_scan_f32_scratch_bytes(1, n) >= sizeof(ovl::ScanHeader) + ovl_reduce_f32_scratch_bytes(n);
}

}  // namespace

extern "C" int ovl_scan_f32_begin(int op, const float* in, uint64_t n, double* out_total, void* scratch,
                                  uint64_t scratch_bytes, void* cuda_stream) {
    if (!out_total) return OVL_ERR_NULL;
    int st = check_scan_args(op, in, 1, n, nullptr, scratch, scratch_bytes);
    if (st != OVL_OK) return st;
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const bool aligned = ((uintptr_t)in % 16 == 0);
    OVL_CUDA(cudaMemsetAsync(scratch, 0, sizeof(ovl::ScanHeader), stream));
    if (shard_uses_ring(in, n))
        return launch_reduce(op, in, n, out_total, reinterpret_cast<char*>(scratch) + sizeof(ovl::ScanHeader), stream);
    cudaError_t e = (op == 0) ? launch_tile_aggregates<ovl::OpAdd>(in, 1, n, scratch, aligned, stream)
                              : launch_tile_aggregates<ovl::OpMul>(in, 1, n, scratch, aligned, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    e = (op == 0) ? launch_scan_aggregates<ovl::OpAdd>(scratch, 1, n, nullptr, out_total, false, stream)
                  : launch_scan_aggregates<ovl::OpMul>(scratch, 1, n, nullptr, out_total, false, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    return OVL_OK;
}

extern "C" int ovl_scan_f32_finish(int op, const float* in, float* out, uint64_t n, const double* carry, void* scratch,
                                   uint64_t scratch_bytes, void* cuda_stream) {
    if (!out) return OVL_ERR_NULL;
    int st = check_scan_args(op, in, 1, n, carry, scratch, scratch_bytes);
    if (st != OVL_OK) return st;
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const bool aligned = ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0);
    if (shard_uses_ring(in, n)) {
        // `begin` left no tile aggregates: the ring scan, or (output not aligned) the three passes from the start
        OVL_CUDA(cudaMemsetAsync(scratch, 0, sizeof(ovl::ScanHeader), stream));
        if (op == 0) return run_scan<ovl::OpAdd>(in, out, 1, n, carry, scratch, aligned, stream);
        return run_scan<ovl::OpMul>(in, out, 1, n, carry, scratch, aligned, stream);
    }
    if (op == 0) return finish_scan<ovl::OpAdd>(in, out, 1, n, carry, scratch, aligned, stream);
    return finish_scan<ovl::OpMul>(in, out, 1, n, carry, scratch, aligned, stream);
}

// ---------------------------------------------------------------------------------------------------------
// Sharded scan whose shard totals travel through peer memory instead of a collective library call.

extern "C" uint64_t ovl_peer_buffer_bytes(void) { return (uint64_t)ovl::kPeerBufferWords * sizeof(uint64_t); }

extern "C" int ovl_peer_alloc(void** out_ptr, unsigned char* out_handle) {
    if (!out_ptr || !out_handle) return OVL_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == OVL_PEER_HANDLE_BYTES, "handle size");
    void* p = nullptr;
    OVL_CUDA(cudaMalloc(&p, ovl_peer_buffer_bytes()));
    cudaError_t e = cudaMemset(p, 0, ovl_peer_buffer_bytes());
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return cuda_fail(e);
    }
    memcpy(out_handle, &h, sizeof(h));
    *out_ptr = p;
    return OVL_OK;
}

extern "C" int ovl_peer_open(const unsigned char* handle, void** out_ptr) {
    if (!handle || !out_ptr) return OVL_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    OVL_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *out_ptr = p;
    return OVL_OK;
}

extern "C" int ovl_peer_close(void* ptr) {
    if (!ptr) return OVL_ERR_NULL;
    OVL_CUDA(cudaIpcCloseMemHandle(ptr));
    return OVL_OK;
}

extern "C" int ovl_peer_free(void* ptr) {
    if (!ptr) return OVL_ERR_NULL;
    OVL_CUDA(cudaFree(ptr));
    return OVL_OK;
}

namespace {

int check_peer_args(int op, const float* in, uint64_t n, const void* scratch, uint64_t scratch_bytes,
                    const OvlPeerExchange* px) {
    if (!px) return OVL_ERR_NULL;
    int st = check_scan_args(op, in, 1, n, nullptr, scratch, scratch_bytes);
    if (st != OVL_OK) return st;
    if (px->world == 0 || px->world > (uint32_t)ovl::kMaxPeers || px->rank >= px->world || px->epoch == 0)
        return OVL_ERR_INVALID;
    for (uint32_t p = 0; p < px->world; ++p)
        if (!px->buffers[p] || ((uintptr_t)px->buffers[p] % 16) != 0) return OVL_ERR_NULL;
    // only shards that the ring scan takes: longer than a tile, 16-byte aligned
    if (!shard_uses_ring(in, n)) return OVL_ERR_ALIGNMENT;
    return OVL_OK;
}

ovl::PeerExchange device_exchange(const OvlPeerExchange* px) {
    ovl::PeerExchange d;
    memset(&d, 0, sizeof(d));
    for (uint32_t p = 0; p < px->world; ++p) d.slots[p] = reinterpret_cast<uint64_t*>(px->buffers[p]);
    d.world = px->world;
    d.rank = px->rank;
    d.epoch = px->epoch;
    return d;
}

}  // namespace

extern "C" int ovl_scan_f32_begin_peer(int op, const float* in, uint64_t n, double* out_total, void* scratch,
                                       uint64_t scratch_bytes, const OvlPeerExchange* px, void* cuda_stream) {
    if (!out_total) return OVL_ERR_NULL;
    int st = check_peer_args(op, in, n, scratch, scratch_bytes, px);
    if (st != OVL_OK) return st;
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const uint32_t grid = (uint32_t)ovl::reduce_chunks(n);
    // status word of the scan and the reduction's block counter sit side by side: one clear for both
    OVL_CUDA(cudaMemsetAsync(scratch, 0, sizeof(ovl::ScanHeader) + 16, stream));
    void* red = reinterpret_cast<char*>(scratch) + sizeof(ovl::ScanHeader);
    const ovl::PeerExchange d = device_exchange(px);
    if (op == 0) reduce_publish_f32_kernel<ovl::OpAdd><<<grid, ovl::kScanBlock, 0, stream>>>(in, n, out_total, red, d);
    else reduce_publish_f32_kernel<ovl::OpMul><<<grid, ovl::kScanBlock, 0, stream>>>(in, n, out_total, red, d);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? OVL_OK : cuda_fail(e);
}

extern "C" int ovl_scan_f32_finish_peer(int op, const float* in, float* out, uint64_t n, void* scratch,
                                        uint64_t scratch_bytes, const OvlPeerExchange* px, void* cuda_stream) {
    if (!out) return OVL_ERR_NULL;
    int st = check_peer_args(op, in, n, scratch, scratch_bytes, px);
    if (st != OVL_OK) return st;
    if (((uintptr_t)out % 16) != 0) return OVL_ERR_ALIGNMENT;
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const uint64_t tiles = (n + kTile - 1) / kTile;
    uint64_t cap = (uint64_t)sm_count_cached();
    if (cap > (uint64_t)ovl::kRingMaxGrid) cap = ovl::kRingMaxGrid;
    const uint32_t grid = (uint32_t)(tiles < cap ? tiles : cap);
    const size_t smem = (size_t)ovl::kRingSlots * kTile * sizeof(float) + ovl::kRingCtlBytes;
    const void* kernel = op == 0 ? (const void*)scan_ring_peer_f32_kernel<ovl::OpAdd>
                                 : (const void*)scan_ring_peer_f32_kernel<ovl::OpMul>;
    OVL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    OVL_CUDA(cudaMemsetAsync(scratch, 0, sizeof(ovl::ScanHeader) + tiles * 16, stream));
    ovl::PeerExchange d = device_exchange(px);
    void* args[] = {(void*)&in, (void*)&out, (void*)&n, (void*)&scratch, (void*)&d};
    OVL_CUDA(cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(ovl::kRingThreads), args, smem, stream));
    return OVL_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant of ovl_scan_f32: the tile descriptors live in a file-scope device array instead of
// caller-provided scratch, for hosts that are not allowed (or cannot afford) to allocate device memory.

static __device__ __align__(256) unsigned char g_scan_static_scratch[OVL_SCAN_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the array on the current device.  In host code the array's name is only a handle for the
// runtime, not an address a kernel could use; the address comes from cudaGetSymbolAddress, once per device.
int static_scratch_address(void** out_ptr) {
    int dev = 0;
    OVL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return OVL_ERR_INVALID;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        OVL_CUDA(cudaGetSymbolAddress(&p, g_scan_static_scratch));
        if (!p) return OVL_ERR_NULL;
        g_static_ptr[dev] = p;
    }
    *out_ptr = g_static_ptr[dev];
    return OVL_OK;
}

}  // namespace

extern "C" int ovl_scan_f32_static(int op, const float* in, float* out, uint64_t lines, uint64_t n, const double* carry,
                                   void* cuda_stream) {
    if (!in || !out) return OVL_ERR_NULL;
    if (op != 0 && op != 1) return OVL_ERR_INVALID;
    if (lines == 0 || n == 0) return OVL_ERR_INVALID;
    if (carry && lines != 1) return OVL_ERR_INVALID;
    // size check first, in a form that cannot overflow
    const uint64_t per_line = tiles_per_line(n, true);
    const uint64_t max_tiles = (OVL_SCAN_STATIC_SCRATCH_BYTES - sizeof(ovl::ScanHeader)) / sizeof(ovl::TileDesc<double>);
    if (per_line > max_tiles || lines > max_tiles / per_line) return OVL_ERR_TOO_LARGE;
    void* scratch = nullptr;
    int st = static_scratch_address(&scratch);
    if (st != OVL_OK) return st;
    // ovl_scan_f32 clears the part of the scratch this launch uses and enqueues the kernel; it allocates nothing
    return ovl_scan_f32(op, in, out, lines, n, carry, scratch, OVL_SCAN_STATIC_SCRATCH_BYTES, cuda_stream);
}

extern "C" int ovl_scan_f32_static_status(void* cuda_stream, int32_t* out_status) {
    if (!out_status) return OVL_ERR_NULL;
    void* scratch = nullptr;
    int st = static_scratch_address(&scratch);
    if (st != OVL_OK) return st;
    return ovl_read_kernel_status(scratch, cuda_stream, out_status);
}

extern "C" uint64_t ovl_reduce_f32_scratch_bytes(uint64_t n) {
    // block counter + one partial per chunk
    return 16 + ovl::reduce_chunks(n ? n : 1) * sizeof(double);
}

extern "C" int ovl_reduce_f32(int op, const float* in, uint64_t n, double* out_total, void* scratch, uint64_t scratch_bytes,
                              void* cuda_stream) {
    if (!in || !out_total) return OVL_ERR_NULL;
    if (op != 0 && op != 1) return OVL_ERR_INVALID;
    if (n == 0) return OVL_ERR_INVALID;
    const uint64_t need = ovl_reduce_f32_scratch_bytes(n);
    if (!scratch || scratch_bytes < need || ((uintptr_t)scratch % 16) != 0) return OVL_ERR_SCRATCH;
    return launch_reduce(op, in, n, out_total, scratch, (cudaStream_t)cuda_stream);
}
