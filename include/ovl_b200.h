/*
 * ovl_b200.h - C ABI of the B200 operator launcher (libovl_b200.so).
 *
 * This library is what a host program binds to run OVL operators on a B200.  It replaces the reference's
 * native glue for the evaluate path:
 *   - the per-operator C++ entry point `<name>_generic_cuda(std::vector<std::shared_ptr<const InputParameter>>,
 *     std::vector<std::shared_ptr<OutputParameter>>, CUstream, uint16_t threads_per_block, uint16_t* err)`
 *     generated at opveclib/expression.py:685-699 (C++ STL types across a dlopen boundary, not a C ABI);
 *   - the standalone CUDA harness `testCUDAOperator` (opveclib/testcudaop.cc:60-395);
 *   - the launcher half of the TensorFlow custom op (opveclib/dynamiclibop.cc:127-171).
 * Signatures use plain pointers and sizes only.  The callee never owns tensor memory (as in
 * opveclib/dynamiclibop.h:48,77); modules and kernels live until destroyed or process exit.  Every function
 * returns an OvlStatus; nothing calls exit() (the reference's harness does, opveclib/testcudaop.cc:22-43).
 * Launches are asynchronous on the caller's stream and the library is re-entrant, like the reference's GPU
 * launcher (opveclib/dynamiclibop.cc:161-171).
 */
#ifndef OVL_B200_H_
#define OVL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element type codes: wire values of the language's DType enum (opveclib/language.proto:16-37). */
enum OvlDType {
    OVL_FLOAT16 = 1, OVL_FLOAT32 = 2, OVL_FLOAT64 = 3, OVL_INT8 = 4, OVL_INT16 = 5, OVL_INT32 = 6, OVL_INT64 = 7,
    OVL_UINT8 = 8, OVL_UINT16 = 9, OVL_UINT32 = 10, OVL_UINT64 = 11
};

/* Status codes.  OVL_ERR_ARITY / OVL_ERR_LENGTH correspond to the reference's `*err = 1` on a wrong number of
 * tensors or a wrong element count (opveclib/expression.py:622, 639, 662-663). */
enum OvlStatus {
    OVL_OK = 0,
    OVL_ERR_ARITY = 1,       /* wrong number of input or output tensors */
    OVL_ERR_LENGTH = 2,      /* a tensor's element count differs from the kernel's signature */
    OVL_ERR_DTYPE = 3,       /* a tensor's dtype differs from the kernel's signature */
    OVL_ERR_NULL = 4,        /* a required pointer is null */
    OVL_ERR_CUDA = 5,        /* a CUDA call failed; see ovl_last_cuda_error() */
    OVL_ERR_NOT_FOUND = 6,   /* kernel symbol not present in the module */
    OVL_ERR_SCRATCH = 7,     /* scratch buffer missing, too small or misaligned */
    OVL_ERR_TIMEOUT = 8,     /* a bounded device-side wait expired (reported through the kernel's status word) */
    OVL_ERR_ALIGNMENT = 9,   /* a tensor pointer does not meet the alignment the kernel was built for */
    OVL_ERR_TOO_LARGE = 10,  /* size beyond what the entry point supports */
    OVL_ERR_INVALID = 11     /* malformed specification */
};

/* A tensor argument: borrowed device (or host, where stated) memory, dtype code and element count.
 * Same fields as the reference's `_TensorParam` / `TensorParam` (opveclib/operator.py:128-131,
 * opveclib/testcop.cc:28-32). */
typedef struct OvlTensor {
    void* data;
    int32_t dtype;
    uint64_t len;
} OvlTensor;

typedef struct OvlModule OvlModule; /* a loaded cubin */
typedef struct OvlKernel OvlKernel; /* one kernel of a module together with its signature and launch shape */

/* Launch description of one generated kernel.  Kernel parameters are, in order: the input pointers, the
 * output pointers, then the scratch pointer if scratch_bytes > 0.  More than 48 KiB of dynamic shared memory is
 * opted into when the kernel is created. */
typedef struct OvlKernelSpec {
    const char* symbol;          /* name of the __global__ function inside the module */
    uint32_t grid_x;             /* number of thread blocks */
    uint32_t block_x;            /* threads per block */
    uint32_t dynamic_smem_bytes; /* dynamic shared memory per block */
    uint32_t n_inputs;
    uint32_t n_outputs;
    const int32_t* dtypes;       /* n_inputs + n_outputs dtype codes, inputs first */
    const uint64_t* lens;        /* n_inputs + n_outputs element counts */
    const uint32_t* align_bytes; /* n_inputs + n_outputs required pointer alignments (0 or 1 = none) */
    uint64_t scratch_bytes;      /* device scratch the kernel needs (0 = none); provided by the caller */
    uint64_t scratch_zero_bytes; /* leading part of the scratch that must be zero when the kernel starts;
                                    ovl_launch clears it on the stream before the kernel */
    uint32_t flags;              /* OVL_KERNEL_* bits */
} OvlKernelSpec;

/* The kernel's blocks wait for one another (always with a bound), so the whole grid must be resident at once:
 * launched with cudaLaunchCooperativeKernel, which refuses a grid the device cannot hold. */
#define OVL_KERNEL_COOPERATIVE 1u

/* Library / device ------------------------------------------------------------------------------------- */
const char* ovl_version(void);
const char* ovl_status_string(int status);
/* CUDA error code of the calling thread's most recent OVL_ERR_CUDA (a cudaError_t value), 0 if none. */
int ovl_last_cuda_error(void);
/* Number of streaming multiprocessors of the current device. */
int ovl_device_sm_count(int* out_count);

/* Modules and kernels ---------------------------------------------------------------------------------- */
/* Load an sm_100a cubin image from memory / from a file into the current device's context. */
int ovl_module_load(const void* image, size_t size, OvlModule** out_module);
int ovl_module_load_file(const char* path, OvlModule** out_module);
int ovl_module_unload(OvlModule* module);
/* Look up spec->symbol and bind it to a copy of the specification. */
int ovl_kernel_create(OvlModule* module, const OvlKernelSpec* spec, OvlKernel** out_kernel);
int ovl_kernel_destroy(OvlKernel* kernel);

/* Launching -------------------------------------------------------------------------------------------- */
/* Validate the tensors against the kernel's signature (arity, element counts, dtypes, alignment), clear the
 * zeroed part of the scratch and enqueue one launch on `cuda_stream` (a cudaStream_t; NULL = default stream).
 * Tensors are DEVICE pointers.  Replaces `<name>_generic_cuda` (opveclib/expression.py:685-699). */
int ovl_launch(OvlKernel* kernel, const OvlTensor* inputs, size_t n_inputs, const OvlTensor* outputs,
               size_t n_outputs, void* scratch, uint64_t scratch_bytes, void* cuda_stream);

/* Timed launches: `iterations` launches, each bracketed by CUDA events on `cuda_stream`; milliseconds per
 * launch are written to ms[0..iterations).  Synchronises the stream.  Replaces the timing loop of
 * opveclib/testcudaop.cc:294-304. */
int ovl_profile(OvlKernel* kernel, const OvlTensor* inputs, size_t n_inputs, const OvlTensor* outputs,
                size_t n_outputs, void* scratch, uint64_t scratch_bytes, void* cuda_stream, uint32_t iterations,
                float* ms);

/* Host-buffer convenience with the contract of the reference harness (opveclib/testcudaop.cc:60-395):
 * tensors are HOST pointers; the call stages inputs to device memory it allocates, fills outputs with 0xFE
 * bytes, runs `iterations` timed launches, copies outputs back, frees the staging memory and synchronises.
 * `ms` may be NULL. */
int ovl_run_host(OvlKernel* kernel, const OvlTensor* host_inputs, size_t n_inputs, const OvlTensor* host_outputs,
                 size_t n_outputs, uint32_t iterations, float* ms);

/* Read the 32-bit status word a kernel keeps at the start of its scratch buffer (0 = no error; otherwise an
 * OvlStatus such as OVL_ERR_TIMEOUT).  Synchronises the stream. */
int ovl_read_kernel_status(const void* scratch, void* cuda_stream, int32_t* out_status);

/* Built-in scans ----------------------------------------------------------------------------------------- */
/* Inclusive scan (op: 0 = sum, 1 = product) of `lines` contiguous lines of `n` fp32 elements each, device
 * memory in and out, with the same cooperative kernels the code generator uses for recognised accumulate loops
 * (the reference's one-worker-per-line loop: opveclib/examples/test_accumulate.py:22-78).  Accumulation is in
 * fp64.  Lines of at most 8192 elements are scanned in one pass by one thread block each - or, with 16-byte
 * aligned line starts, by one warp each from 2048 lines on, and as one flat array of vectors (several lines per
 * warp) when a line has at most 512 elements and a multiple of four of them.  Longer lines whose
 * starts are 16-byte aligned (aligned pointers and, with several lines, n divisible by four) are scanned by the
 * ring scan: one cooperative launch (a block per SM, so nothing else should occupy the device's SMs meanwhile)
 * that reads and writes every element once (several lines: a group of blocks per line when that keeps the grid
 * busy, else waves of tiles that cross line ends).  Other long lines take three streaming passes (tile aggregates,
 * prefixes of the aggregates, seeded tile scans).  The environment variable OVL_SCAN_MODE=threepass forces the
 * three passes, OVL_SCAN_MODE=lookback selects a single pass with decoupled look-back.
 * `carry` (device pointer to one double, or NULL) is combined into every element of a single line (lines
 * must be 1 when it is given).  `scratch` must hold ovl_scan_f32_scratch_bytes(lines, n) bytes. */
uint64_t ovl_scan_f32_scratch_bytes(uint64_t lines, uint64_t n);
int ovl_scan_f32(int op, const float* in, float* out, uint64_t lines, uint64_t n, const double* carry, void* scratch,
                 uint64_t scratch_bytes, void* cuda_stream);
/* The same scan of ONE line split at the point where ranks of a sharded scan exchange their totals:
 * ovl_scan_f32_begin reads the shard once and writes the shard's total to *out_total (device memory); after the
 * carry has been formed from the totals of the ranks before, ovl_scan_f32_finish produces the result.  The pair
 * moves 12 bytes per element (4 for the total, 8 for the scan): a shard's total is only known after all of it has
 * been read, so every shard but the first must be read twice.  Pass the same `in`, `n` and scratch to both calls
 * (the scratch carries state from one to the other). */
int ovl_scan_f32_begin(int op, const float* in, uint64_t n, double* out_total, void* scratch, uint64_t scratch_bytes,
                       void* cuda_stream);
int ovl_scan_f32_finish(int op, const float* in, float* out, uint64_t n, const double* carry, void* scratch,
                        uint64_t scratch_bytes, void* cuda_stream);
/* The same pair for GPUs of one box that exchange their totals through peer memory, without a collective library
 * call between the two kernels (the reference has no multi-GPU support; this is the shard-boundary exchange of a
 * scan along an axis split over 2 to 8 GPUs).  Every rank allocates one exchange buffer (ovl_peer_alloc: device
 * memory plus a 64-byte handle that another process of the same box turns into a mapping with ovl_peer_open) and
 * fills OvlPeerExchange with all ranks' buffers as mapped in its own process, its rank, the number of ranks and
 * an epoch that starts at 1 and grows by one with every begin/finish pair - the same on all ranks.
 * ovl_scan_f32_begin_peer reads the shard once and stores its total into every rank's buffer (plain stores over
 * NVLink, also into *out_total); ovl_scan_f32_finish_peer scans the shard in one cooperative launch whose first
 * step waits - bounded, OVL_ERR_TIMEOUT in the scratch's status word on expiry - until the totals of all ranks of
 * this epoch have arrived in its own buffer, and combines those of the ranks before it, in rank order, into its
 * carry.  Only shards that the ring scan takes are accepted: more than 8192 elements, `in` and `out` 16-byte
 * aligned; OVL_ERR_ALIGNMENT otherwise - use the plain pair with a collective then.  All ranks must call both
 * functions once per epoch; kernels of different ranks wait for each other, so each rank needs its own GPU (on one
 * GPU, enqueue every rank's begin before any rank's finish). */
#define OVL_PEER_HANDLE_BYTES 64
#define OVL_MAX_PEERS 8
typedef struct OvlPeerExchange {
    void* buffers[OVL_MAX_PEERS]; /* rank p's exchange buffer as mapped in this process */
    uint32_t world;               /* number of ranks, 1..8 */
    uint32_t rank;                /* this rank */
    uint32_t epoch;               /* 1, 2, 3, ...: one per begin/finish pair, equal on all ranks */
} OvlPeerExchange;
uint64_t ovl_peer_buffer_bytes(void);
int ovl_peer_alloc(void** out_ptr, unsigned char* out_handle /* OVL_PEER_HANDLE_BYTES */);
int ovl_peer_open(const unsigned char* handle, void** out_ptr);
int ovl_peer_close(void* ptr);
int ovl_peer_free(void* ptr);
int ovl_scan_f32_begin_peer(int op, const float* in, uint64_t n, double* out_total, void* scratch,
                            uint64_t scratch_bytes, const OvlPeerExchange* px, void* cuda_stream);
int ovl_scan_f32_finish_peer(int op, const float* in, float* out, uint64_t n, void* scratch, uint64_t scratch_bytes,
                             const OvlPeerExchange* px, void* cuda_stream);

/* Reduce `n` fp32 elements to one double (sum or product, fixed combination order): the shard total that
 * ranks exchange before a scan that crosses shard boundaries.  `scratch` must hold
 * ovl_reduce_f32_scratch_bytes(n) bytes. */
uint64_t ovl_reduce_f32_scratch_bytes(uint64_t n);
int ovl_reduce_f32(int op, const float* in, uint64_t n, double* out_total, void* scratch, uint64_t scratch_bytes,
                   void* cuda_stream);

/* Self-test of the bounded device-side waits (no counterpart in the reference).  Runs the ring scan (cumsum of one
 * line of n > 8192 fp32 elements, 16-byte aligned pointers) with the first thread block keeping its tile aggregates
 * to itself, so that every block's wait for them runs into its limit (about two seconds).  Nothing hangs or traps:
 * the kernel ends, `out` is unspecified, and ovl_read_kernel_status(scratch, ...) then reports OVL_ERR_TIMEOUT;
 * the context stays usable.  For hosts that want to check their error path. */
int ovl_selftest_scan_timeout(const float* in, float* out, uint64_t n, void* scratch, uint64_t scratch_bytes,
                              void* cuda_stream);

/* Allocation-free scan ----------------------------------------------------------------------------------- */
/* Same scan as ovl_scan_f32, for hosts that may not allocate device memory: for example a plugin running inside
 * an engine whose memory pool owns the whole GPU and forbids cudaMalloc from plugin code, or a latency-critical
 * loop that cannot afford the device-wide synchronisation an allocation implies.  The caller passes only inputs
 * and outputs; the tile descriptors live in a fixed array compiled into the library
 * (OVL_SCAN_STATIC_SCRATCH_BYTES of device memory, held by every GPU that loads the library until the process
 * exits).  This entry point has no counterpart in the reference.
 *
 *  - Limit: ovl_scan_f32_scratch_bytes(lines, n) must not exceed OVL_SCAN_STATIC_SCRATCH_BYTES (32767 slots of
 *    32 bytes: that many lines of up to 8192 elements, or about 134 million elements in longer lines, which are
 *    budgeted one slot per 4096 elements); larger requests return OVL_ERR_TOO_LARGE.
 *  - The first call on each device looks up the array's device address (with that device current); make that
 *    first call before starting any stream capture.  No call allocates or frees memory.
 *  - All calls share the one array, and it keeps whatever the previous call left in it: each call clears the part
 *    it needs on `cuda_stream` before its kernel.  Two calls that can overlap on the GPU (different streams, no
 *    dependency between them) race on the array; order them yourself.
 *  - Errors of the bounded device-side waits are reported as for ovl_scan_f32; read them with
 *    ovl_scan_f32_static_status() after the work on the stream has finished. */
#define OVL_SCAN_STATIC_SCRATCH_BYTES (1u << 20)
int ovl_scan_f32_static(int op, const float* in, float* out, uint64_t lines, uint64_t n, const double* carry,
                        void* cuda_stream);
/* Status word of the most recent ovl_scan_f32_static launch on the current device (synchronises the stream). */
int ovl_scan_f32_static_status(void* cuda_stream, int32_t* out_status);

#ifdef __cplusplus
}
#endif
#endif /* OVL_B200_H_ */
