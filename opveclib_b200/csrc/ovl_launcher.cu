// libovl_b200.so - C-ABI launcher for generated sm_100a kernels plus the built-in fp32 scans.
// Interface and the reference code each entry point replaces: include/ovl_b200.h.
//
// Uses the CUDA runtime only (statically linked): cubins are loaded with cudaLibraryLoadData and launched with
// cudaLaunchKernel on the caller's stream, in the caller's (primary) context - no private context, unlike the
// reference harness (opveclib/testcudaop.cc:69-75).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/ovl_b200.h"
#include "templates/ovl_scan.cuh"

namespace {

thread_local int g_last_cuda_error = 0;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
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
    uint32_t cooperative;
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
    k->cooperative = spec->cooperative;
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
    if (k->cooperative) {
        // blocks of this kernel wait for one another: all of them have to be resident
        uint32_t grid = k->grid_x;
        int per_sm = 0, dev = 0, sms = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)k->fn, (int)k->block_x, k->dynamic_smem) ==
                cudaSuccess && per_sm > 0 && cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) {
            const uint64_t cap = (uint64_t)per_sm * (uint64_t)sms;
            if (grid > cap) grid = (uint32_t)cap;
        } else {
            (void)cudaGetLastError();
        }
        OVL_CUDA(cudaLaunchCooperativeKernel((const void*)k->fn, dim3(grid), dim3(k->block_x), args, k->dynamic_smem, stream));
        return OVL_OK;
    }
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

template <class Op, bool ALIGNED, bool HAS_CARRY, bool LOOKBACK>
__global__ void __launch_bounds__(LOOKBACK ? ovl::kScanBlockLookback : ovl::kScanBlock, LOOKBACK ? 4 : 2) scan_f32_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                     const double* __restrict__ carry, uint64_t lines,
                                                                     uint64_t n, void* scratch) {
    ovl::scan_lines<float, double, Op, 4, ALIGNED, HAS_CARRY, LOOKBACK>(in, out, carry, lines, n, scratch);
}

template <class Op, bool ALIGNED, bool HAS_CARRY>
__global__ void __launch_bounds__(ovl::kScanBlockLookback, 4) scan_f32_wave_kernel(const float* __restrict__ in,
                                                                                  float* __restrict__ out,
                                                                                  const double* __restrict__ carry, uint64_t n,
                                                                                  void* scratch) {
    ovl::scan_long_line<float, double, Op, 4, ALIGNED, HAS_CARRY>(in, out, carry, n, scratch);
}

template <class Op, bool ALIGNED>
__global__ void __launch_bounds__(ovl::kScanBlock) reduce_f32_kernel(const float* __restrict__ in, uint64_t n,
                                                                    double* __restrict__ out_total, void* scratch) {
    ovl::reduce_all<float, double, Op, 4, ALIGNED>(in, n, out_total, scratch);
}

// a line of at most kTile elements is one tile; longer lines are cut into tiles of kTileLookback elements
constexpr uint64_t kTile = (uint64_t)ovl::kScanBlock * ovl::kScanVpt * 4;
constexpr uint64_t kTileLookback = (uint64_t)ovl::kScanBlockLookback * ovl::kScanVpt * 4;

inline uint64_t tiles_per_line(uint64_t n) { return n <= kTile ? 1 : (n + kTileLookback - 1) / kTileLookback; }

int sm_count_cached() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
            sms = v;
        else
            return 148;
    }
    return sms;
}

template <class Op, bool ALIGNED, bool HAS_CARRY>
cudaError_t launch_scan_lb(const float* in, float* out, uint64_t lines, uint64_t n, const double* carry, void* scratch,
                           uint64_t tiles, bool lookback, cudaStream_t stream) {
    const uint64_t sms = (uint64_t)sm_count_cached();
    if (!lookback) {
        const uint64_t max_grid = sms * 2;
        const uint32_t grid = (uint32_t)(tiles < max_grid ? tiles : max_grid);
        scan_f32_kernel<Op, ALIGNED, HAS_CARRY, false><<<grid, ovl::kScanBlock, 0, stream>>>(in, out, carry, lines, n, scratch);
        return cudaGetLastError();
    }
    if (lines == 1) {
        // one long line: wave scan (cooperative launch, at most kWaveMaxBlocks resident blocks)
        auto wave_kernel = scan_f32_wave_kernel<Op, ALIGNED, HAS_CARRY>;
        int wave_per_sm = 0;
        cudaError_t we = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&wave_per_sm, wave_kernel, ovl::kScanBlockLookback, 0);
        if (we != cudaSuccess) return we;
        if (wave_per_sm < 1) return cudaErrorLaunchOutOfResources;
        uint64_t cap = sms * (uint64_t)wave_per_sm;
        if (cap > (uint64_t)ovl::kWaveMaxBlocks) cap = ovl::kWaveMaxBlocks;
        const uint32_t wave_grid = (uint32_t)(tiles < cap ? tiles : cap);
        void* wave_args[] = {(void*)&in, (void*)&out, (void*)&carry, (void*)&n, (void*)&scratch};
        return cudaLaunchCooperativeKernel((const void*)wave_kernel, dim3(wave_grid), dim3(ovl::kScanBlockLookback), wave_args,
                                           0, stream);
    }
    // look-back: blocks wait for each other's aggregates, so all of them must be resident at once - a
    // cooperative launch with the grid clamped to what the device holds
    auto kernel = scan_f32_kernel<Op, ALIGNED, HAS_CARRY, true>;
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, ovl::kScanBlockLookback, 0);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    const uint64_t max_grid = sms * (uint64_t)per_sm;
    const uint32_t grid = (uint32_t)(tiles < max_grid ? tiles : max_grid);
    void* args[] = {(void*)&in, (void*)&out, (void*)&carry, (void*)&lines, (void*)&n, (void*)&scratch};
    return cudaLaunchCooperativeKernel((const void*)kernel, dim3(grid), dim3(ovl::kScanBlockLookback), args, 0, stream);
}

template <class Op>
int launch_scan(const float* in, float* out, uint64_t lines, uint64_t n, const double* carry, void* scratch, uint64_t tiles,
                bool aligned, bool lookback, cudaStream_t stream) {
    cudaError_t e;
    if (aligned) {
        if (carry) e = launch_scan_lb<Op, true, true>(in, out, lines, n, carry, scratch, tiles, lookback, stream);
        else e = launch_scan_lb<Op, true, false>(in, out, lines, n, carry, scratch, tiles, lookback, stream);
    } else {
        if (carry) e = launch_scan_lb<Op, false, true>(in, out, lines, n, carry, scratch, tiles, lookback, stream);
        else e = launch_scan_lb<Op, false, false>(in, out, lines, n, carry, scratch, tiles, lookback, stream);
    }
    if (e != cudaSuccess) return cuda_fail(e);
    return OVL_OK;
}

}  // namespace

extern "C" uint64_t ovl_scan_f32_scratch_bytes(uint64_t lines, uint64_t n) {
    if (lines == 1 && n > kTile) return ovl::wave_scratch_bytes();   // one long line: two wave buffers
    return ovl::scan_scratch_bytes<double>(tiles_per_line(n) * lines);
}

extern "C" int ovl_scan_f32(int op, const float* in, float* out, uint64_t lines, uint64_t n, const double* carry,
                            void* scratch, uint64_t scratch_bytes, void* cuda_stream) {
    if (!in || !out) return OVL_ERR_NULL;
    if (op != 0 && op != 1) return OVL_ERR_INVALID;
    if (lines == 0 || n == 0) return OVL_ERR_INVALID;
    if (carry && lines != 1) return OVL_ERR_INVALID;
    const uint64_t need = ovl_scan_f32_scratch_bytes(lines, n);
    if (!scratch || scratch_bytes < need || ((uintptr_t)scratch % 16) != 0) return OVL_ERR_SCRATCH;
    const uint64_t tiles = tiles_per_line(n) * lines;
    if (tiles >= (1ull << 32) - 65536) return OVL_ERR_TOO_LARGE;   // the tile counter is 32 bits wide
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const bool aligned = ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0) && (lines == 1 || n % 4 == 0);
    const bool lookback = n > kTile;
    // lines of at most one tile publish nothing: only the header (status word) has to be clear
    OVL_CUDA(cudaMemsetAsync(scratch, 0, lookback ? need : sizeof(ovl::ScanHeader), stream));
    if (op == 0) return launch_scan<ovl::OpAdd>(in, out, lines, n, carry, scratch, tiles, aligned, lookback, stream);
    return launch_scan<ovl::OpMul>(in, out, lines, n, carry, scratch, tiles, aligned, lookback, stream);
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
    const uint64_t per_line = tiles_per_line(n);
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
    (void)n;
    return 16 + (uint64_t)sm_count_cached() * 8 * sizeof(double);
}

extern "C" int ovl_reduce_f32(int op, const float* in, uint64_t n, double* out_total, void* scratch, uint64_t scratch_bytes,
                              void* cuda_stream) {
    if (!in || !out_total) return OVL_ERR_NULL;
    if (op != 0 && op != 1) return OVL_ERR_INVALID;
    if (n == 0) return OVL_ERR_INVALID;
    const uint64_t need = ovl_reduce_f32_scratch_bytes(n);
    if (!scratch || scratch_bytes < need || ((uintptr_t)scratch % 16) != 0) return OVL_ERR_SCRATCH;
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const bool aligned = ((uintptr_t)in % 16 == 0);
    const uint64_t want = (n / 4 + ovl::kScanBlock - 1) / ovl::kScanBlock;
    const uint64_t max_grid = (uint64_t)sm_count_cached() * 8;
    uint32_t grid = (uint32_t)(want < max_grid ? want : max_grid);
    if (grid == 0) grid = 1;
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
