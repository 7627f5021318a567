// TEST INFRASTRUCTURE - CPU oracle harness, never part of the product path.
//
// Runs one oracle operator (emitted by cpp_emit.py) on host threads with the reference harness's contract
// (opveclib/testcop.cc:183-219): dlopen the operator library, then for every iteration start one task per
// thread index, join them all, and record the iteration's wall-clock milliseconds.  Thread t of T handles the
// t-th contiguous block of workers; the split itself lives in the generated entry point.
#include <dlfcn.h>
#include <stdint.h>
#include <chrono>
#include <thread>
#include <vector>

typedef void (*ovl_oracle_fn)(const void* const*, void* const*, uint32_t, uint32_t);

extern "C" int ovl_oracle_run(const char* lib_path, const char* fn_name, const void* const* ins, void* const* outs,
                              uint32_t num_threads, double* ms, uint32_t iterations) {
    void* handle = dlopen(lib_path, RTLD_NOW | RTLD_LOCAL);
    if (!handle) return 1;
    ovl_oracle_fn fn = (ovl_oracle_fn)dlsym(handle, fn_name);
    if (!fn) return 2;
    if (num_threads == 0) num_threads = std::thread::hardware_concurrency();
    if (num_threads == 0) num_threads = 1;
    for (uint32_t it = 0; it < iterations; ++it) {
        auto t0 = std::chrono::steady_clock::now();
        std::vector<std::thread> pool;
        pool.reserve(num_threads);
        for (uint32_t t = 1; t < num_threads; ++t) pool.emplace_back(fn, ins, outs, num_threads, t);
        fn(ins, outs, num_threads, 0);
        for (auto& th : pool) th.join();
        auto t1 = std::chrono::steady_clock::now();
        if (ms) ms[it] = std::chrono::duration<double, std::milli>(t1 - t0).count();
    }
    return 0;
}

extern "C" uint32_t ovl_oracle_hardware_threads() { return std::thread::hardware_concurrency(); }
