// TEST INFRASTRUCTURE - never part of the product path.
//
// TensorFlow-free stand-in for the reference's standalone C++ test harness (opveclib/testcop.cc:36-226), which
// cannot be built without TensorFlow headers (testcop.cc:20-21).  Same exported entry point and contract, so
// that the reference's own ``profile(..., target_language='cpp')`` (opveclib/operator.py:2164-2198, 2310-2314)
// loads it from its cache directory in place of libtestcop.so: wrap raw buffers in the reference's typed
// parameter carriers, fill outputs with 0xFE, dlopen the generated operator library, and for every iteration
// run the operator once per thread index on hardware_concurrency() threads, timing the iteration.
// Built against the reference's own dynamiclibop.h (passed with -I from where the reference lies).
#include <dlfcn.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <chrono>
#include <iostream>
#include <memory>
#include <thread>
#include <vector>
#include "dynamiclibop.h"

namespace {
// wire values of the language's DType enum (opveclib/language.proto:16-37)
enum RefDType { F16 = 1, F32 = 2, F64 = 3, I8 = 4, I16 = 5, I32 = 6, I64 = 7, U8 = 8, U16 = 9, U32 = 10, U64 = 11 };

struct TensorParam {
    void* data;
    int dtype;
    size_t len;
};

typedef void (*OpFn)(std::vector<std::shared_ptr<const InputParameter>>, std::vector<std::shared_ptr<OutputParameter>>,
                     uint32_t, uint32_t, uint16_t*);

template <typename T>
void add_input(std::vector<std::shared_ptr<const InputParameter>>& v, const TensorParam& p) {
    v.emplace_back(new TypedInput<T>(static_cast<const T*>(p.data), p.len));
}
template <typename T>
void add_output(std::vector<std::shared_ptr<OutputParameter>>& v, const TensorParam& p) {
    memset(p.data, 0xFE, p.len * sizeof(T));
    v.emplace_back(new TypedOutput<T>(static_cast<T*>(p.data), p.len));
}
}  // namespace

extern "C" int32_t testCOperatorThreads(const char* lib_path, const char* fn_name, const TensorParam* ins, size_t n_in,
                                        TensorParam* outs, size_t n_out, double* ms, size_t iterations,
                                        uint32_t num_threads) {
    std::vector<std::shared_ptr<const InputParameter>> inputs;
    for (size_t i = 0; i < n_in; ++i) {
        switch (ins[i].dtype) {
            case F32: add_input<float>(inputs, ins[i]); break;
            case F64: add_input<double>(inputs, ins[i]); break;
            case I8: add_input<int8_t>(inputs, ins[i]); break;
            case I16: add_input<int16_t>(inputs, ins[i]); break;
            case I32: add_input<int32_t>(inputs, ins[i]); break;
            case I64: add_input<int64_tf>(inputs, ins[i]); break;
            case U8: add_input<uint8_t>(inputs, ins[i]); break;
            case U16: add_input<uint16_t>(inputs, ins[i]); break;
            case U32: add_input<uint32_t>(inputs, ins[i]); break;
            case U64: add_input<uint64_t>(inputs, ins[i]); break;
            default: return 1;
        }
    }
    std::vector<std::shared_ptr<OutputParameter>> outputs;
    for (size_t i = 0; i < n_out; ++i) {
        switch (outs[i].dtype) {
            case F32: add_output<float>(outputs, outs[i]); break;
            case F64: add_output<double>(outputs, outs[i]); break;
            case I8: add_output<int8_t>(outputs, outs[i]); break;
            case I16: add_output<int16_t>(outputs, outs[i]); break;
            case I32: add_output<int32_t>(outputs, outs[i]); break;
            case I64: add_output<int64_tf>(outputs, outs[i]); break;
            case U8: add_output<uint8_t>(outputs, outs[i]); break;
            case U16: add_output<uint16_t>(outputs, outs[i]); break;
            case U32: add_output<uint32_t>(outputs, outs[i]); break;
            case U64: add_output<uint64_t>(outputs, outs[i]); break;
            default: return 1;
        }
    }
    void* handle = dlopen(lib_path, RTLD_LAZY);
    if (!handle) {
        std::cerr << "***ERROR - Unable to find operator library " << lib_path << '\n';
        return 1;
    }
    OpFn fn = reinterpret_cast<OpFn>(dlsym(handle, fn_name));
    if (!fn) {
        std::cerr << "***ERROR - Unable to find operator function " << fn_name << '\n';
        return 1;
    }
    if (num_threads == 0) {
        const char* env = getenv("OVL_REF_THREADS");
        num_threads = env ? (uint32_t)atoi(env) : 0;
    }
    if (num_threads == 0) num_threads = std::thread::hardware_concurrency();
    if (num_threads == 0) num_threads = 1;
    uint16_t err = 0;
    for (size_t it = 0; it < iterations; ++it) {
        auto t1 = std::chrono::steady_clock::now();
        {
            std::vector<std::thread> pool;
            for (uint32_t t = 0; t < num_threads; ++t) pool.emplace_back(fn, inputs, outputs, num_threads, t, &err);
            for (auto& th : pool) th.join();
        }
        auto t2 = std::chrono::steady_clock::now();
        ms[it] = std::chrono::duration<double, std::milli>(t2 - t1).count();
    }
    if (err != 0) std::cerr << "***ERROR - Generated operator function execution error code: " << err << '\n';
    return err;
}

extern "C" int32_t testCOperator(const char* lib_path, const char* fn_name, const TensorParam* ins, size_t n_in,
                                 TensorParam* outs, size_t n_out, double* ms, size_t iterations) {
    return testCOperatorThreads(lib_path, fn_name, ins, n_in, outs, n_out, ms, iterations, 0);
}

extern "C" uint32_t refHardwareThreads() { return std::thread::hardware_concurrency(); }
