/*
 * aixb200.h - C ABI of the B200 compute device for the AIX tensor library.
 *
 * One opaque handle (aixb200_device) stands for one GPU: a CUDA context, one
 * in-order stream, a caching allocator, a lazy recorder that fuses elementwise
 * op chains into runtime-compiled kernels, and fixed reduction / GEMM kernels.
 *
 * Every op entry point below replaces exactly one virtual of the reference's
 * abstract device class (Targets/AIXLib/aixDevice.hpp:30-84): same name, same
 * argument meaning, same ordering contract (calls take effect in program order;
 * results are observable by any later call and, on the host, after
 * aixb200_synchronize). Where the reference throws std::invalid_argument /
 * std::runtime_error, these functions return AIXB200_ERR_INVALID /
 * AIXB200_ERR_RUNTIME and leave a message in aixb200_last_error().
 *
 * The library never falls back to the CPU: without a usable GPU
 * aixb200_create() fails.
 */
#ifndef AIXB200_H
#define AIXB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AIXB200_MAX_RANK 8

/* Status codes. 0 is success; everything else leaves a message in aixb200_last_error(). */
enum
{
    AIXB200_OK            = 0,
    AIXB200_ERR_INVALID   = 1,   /* contract violation (reference: std::invalid_argument) */
    AIXB200_ERR_RUNTIME   = 2,   /* CUDA / NVRTC / NCCL / allocation failure (reference: std::runtime_error) */
    AIXB200_ERR_NOGPU     = 3,   /* no CUDA device or driver; there is no CPU fallback */
    AIXB200_ERR_TIMEOUT   = 4,   /* a bounded device- or host-side wait ran out */
};

/* Element types; numeric values equal aix::DataType (Targets/AIXLib/aixCore.hpp:44-55).
 * F16/BF16 are raw IEEE binary16 / bfloat16 bit patterns (Targets/AIXLib/aixFloat16.hpp). */
enum
{
    AIXB200_F64  = 0,
    AIXB200_F32  = 1,
    AIXB200_F16  = 2,
    AIXB200_BF16 = 3,
    AIXB200_I64  = 4,
    AIXB200_I32  = 5,
    AIXB200_I16  = 6,
    AIXB200_I8   = 7,
    AIXB200_U8   = 8,
    AIXB200_DTYPE_COUNT = 9
};

/* POD image of aix::DeviceTensorParams (Targets/AIXLib/aixCore.hpp:189-198).
 * `data` is the storage base, the view starts `offset` ELEMENTS into it; strides are in
 * elements and a stride of 0 is a broadcast dimension; rank 0 is a scalar (size 1).
 * `data` of an input may be device memory from aixb200_allocate or plain host memory
 * (it is staged to the GPU at call time); `data` of a result must come from
 * aixb200_allocate of the same device. isContiguous is derived from the strides. */
typedef struct aixb200_tensor
{
    void*    data;
    uint64_t offset;
    uint64_t size;
    uint32_t dtype;
    uint32_t rank;
    uint64_t shape[AIXB200_MAX_RANK];
    uint64_t strides[AIXB200_MAX_RANK];
} aixb200_tensor;

typedef struct aixb200_device aixb200_device;

/* Device configuration. Zero-initialise, then override; aixb200_default_config fills the defaults. */
typedef struct aixb200_config
{
    int32_t  ordinal;            /* CUDA device ordinal */
    int32_t  managed_memory;     /* 1: allocations are host-dereferenceable CUDA managed memory (what the C++
                                    aix::Device adapter needs, aixCore.hpp:435-440,491-499); 0: plain device memory */
    uint32_t flush_threshold;    /* pending elementwise ops before the planner runs (reference: 200, aixDeviceMetal.cpp:129) */
    int32_t  strict_math;        /* 1: no FMA contraction, IEEE division and square root, library expf/tanhf.
                                    0 (default): contraction allowed, 2-ulp division/sqrt, exp and tanh from hardware
                                    exp2/reciprocal; every f32 result stays within 1e-6 relative of the strict one.
                                    f16/bf16 values are rounded after every op in both modes. */
    int32_t  fusion;             /* 0 disables fusion: every recorded op becomes its own kernel */
    int32_t  disk_cache;         /* 1: keep compiled cubins in $AIXB200_CACHE_DIR (default ~/.cache/aixb200) */
    uint64_t cache_limit_bytes;  /* idle blocks kept by the allocator before it trims (0 = 3/4 of device memory) */
    void*    stream;             /* cudaStream_t to run on; NULL = the device creates its own non-blocking stream */
    int32_t  tf32x3_matmul;      /* f32 matmul: 1 (default) = split precision on the tensor cores - every operand is scaled by a
                                    power of two and cut into two fp16 terms, three fp16 passes accumulate in f32 (norm-wise error
                                    <= 1e-5); 0 = plain f32 FMA on the CUDA cores. The field keeps the name of the first scheme
                                    (TF32 main pass + bf16 cross terms), which remains behind AIXB200_GEMM_F32=hybrid. */
    int32_t  dry_run;            /* 1: no GPU is touched - ops are recorded, planned and compiled with NVRTC but not
                                    launched, and memory comes from malloc (host-logic tests on machines without a GPU) */
    /* Host-side fault injection for tests of the failure paths (nothing on the GPU faults): */
    uint64_t inject_alloc_limit_bytes; /* non-zero: the raw allocator reports out-of-memory once this many bytes are reserved */
    int32_t  inject_nvrtc_failures;    /* the next n kernel compilations fail as if NVRTC had returned an error */
    int32_t  reserved[3];
} aixb200_config;

void aixb200_default_config(aixb200_config* cfg);

/* ---- lifecycle ---- (reference: aix::createDevice, Targets/AIXLib/aixDevices.cpp:24-43) */
int  aixb200_create(int ordinal, aixb200_device** out);
int  aixb200_create_with_config(const aixb200_config* cfg, aixb200_device** out);
void aixb200_destroy(aixb200_device* dev);
/* Message of the last failed call on this device (dev may be NULL for creation failures). */
const char* aixb200_last_error(const aixb200_device* dev);
/* "B200" + the CUDA device name (reference: Device::name, aixDevice.hpp:36). */
const char* aixb200_name(const aixb200_device* dev);
/* Number of visible CUDA devices, or 0 when there is no driver. Never fails. */
int  aixb200_device_count(void);
const char* aixb200_version(void);

/* ---- memory ---- (reference: Device::allocate/deallocate, aixDevice.hpp:40-42; cache and deferred
 * frees: aixDeviceMetalCache.hpp:28-198, aixDeviceMetal.cpp:251-259) */
int aixb200_allocate(aixb200_device* dev, size_t bytes, void** out);
int aixb200_allocate_typed(aixb200_device* dev, size_t count, uint32_t dtype, void** out);
int aixb200_deallocate(aixb200_device* dev, void* memory);
int aixb200_empty_cache(aixb200_device* dev);                        /* Device::emptyCache, aixDevice.hpp:82 */
int aixb200_synchronize(aixb200_device* dev);                        /* Device::synchronize, aixDevice.hpp:83 */

/* ---- elementwise, recorded lazily and fused (aixDevice.hpp:44-48, 57-63) ---- */
int aixb200_add(aixb200_device* dev, const aixb200_tensor* a1, const aixb200_tensor* a2, const aixb200_tensor* result);
int aixb200_sub(aixb200_device* dev, const aixb200_tensor* a1, const aixb200_tensor* a2, const aixb200_tensor* result);
int aixb200_mul(aixb200_device* dev, const aixb200_tensor* a1, const aixb200_tensor* a2, const aixb200_tensor* result);
int aixb200_div(aixb200_device* dev, const aixb200_tensor* a1, const aixb200_tensor* a2, const aixb200_tensor* result);
int aixb200_unary(aixb200_device* dev, const aixb200_tensor* a1, const aixb200_tensor* result);   /* negate */
int aixb200_sqrt(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
int aixb200_sin(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
int aixb200_cos(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
int aixb200_tanh(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
int aixb200_log(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
int aixb200_exp(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
int aixb200_pow(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* exp, const aixb200_tensor* result);
/* fill: `scalar` points at ONE host value of type scalar_dtype, converted with saturation to the result type
 * (aixDevice.hpp:50; conversion rule aixDeviceCPU.cpp:96-117). fillMin writes numeric_limits<T>::lowest(). */
int aixb200_fill(aixb200_device* dev, const void* scalar, uint32_t scalar_dtype, const aixb200_tensor* result);
int aixb200_fill_min(aixb200_device* dev, const aixb200_tensor* result);                          /* aixDevice.hpp:51 */

/* ---- reductions (aixDevice.hpp:52, 60-62, 70-73) ---- */
int aixb200_sum(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
int aixb200_max(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
/* Same result as aixb200_sum, for callers that may not allocate GPU or host memory at the moment of the call - code
 * running under a fixed memory budget, inside a region where cudaMalloc is forbidden or would synchronise, or next to
 * another allocator that owns the whole device. No counterpart in the reference (its devices always allocate their
 * reduction temporaries, aixDeviceMetal.cpp:329-350). The partial sums live in a 32 KiB static __device__ array that is
 * part of this library's image: every GPU that loads the library holds it until the process exits.
 *  - `a` and `result` must already be device memory; host pointers are refused (staging would allocate).
 *  - at most AIXB200_SUM_STATIC_SCRATCH_MAX_ELEMENTS elements; larger inputs return AIXB200_ERR_INVALID.
 *  - recorded elementwise work must have been flushed (aixb200_synchronize) - otherwise AIXB200_ERR_INVALID, because
 *    flushing may compile and load a kernel.
 *  - the first call on a device resolves the array's address (cudaGetSymbolAddress); make that first call before any
 *    stream capture begins.
 *  - all calls on one GPU share the array: calls that overlap on the GPU (two streams, two device handles, two
 *    threads) race on it. Calls on one device handle are ordered by its stream and are safe.
 *  - an aixb200_all_reduce_async still in flight on `a` or `result` is waited for on the device's stream first (an event
 *    wait, no allocation), like in every other entry point. */
#define AIXB200_SUM_STATIC_SCRATCH_MAX_ELEMENTS (1ull << 30)
int aixb200_sum_static_scratch(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
int aixb200_argmax(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
int aixb200_argmax_indices(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result);
/* dst += sum over the broadcast dimensions of src (dst zeroed by the caller); dst = max(dst, ...) for max_to. */
int aixb200_reduce_to(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst);
int aixb200_max_to(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst);
int aixb200_argmax_to(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst, size_t dim);
int aixb200_argmax_indices_to(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst, size_t dim);

/* ---- contraction (aixDevice.hpp:63): result[M,N] = a[M,K] . b[K,N]; a and b may be arbitrary 2-D strided views ----
 * f32 on the tensor cores (tf32x3_matmul = 1) scales each operand by one power of two taken from its largest magnitude.
 * An operand that contains an infinity or a NaN is left unscaled; its finite elements above 65504 then overflow the fp16
 * terms, so rows and columns that the CPU device would still compute finitely can come out infinite or NaN as well.
 * Operands with non-finite elements that must keep their finite part exact need tf32x3_matmul = 0.
 * An f32 product on the tensor cores may be launched later than this call returns - at the latest by the next call that
 * is not a recorded elementwise op: `result + row vector` (nn::Linear's bias, aixNeuralNetwork.hpp:150-153), when it is
 * the next op recorded, `result` is already deallocated and no recorded op consumes the sum, runs inside the product's
 * kernel, which then writes only the sum; and `target += result` into a buffer whose zero-fill is still recorded (the
 * gradient accumulation after zeroGrad) makes a deallocated `result` land in `target` directly. Results and program order
 * are those of separate launches;
 * AIXB200_GEMM_EPILOGUE=0 in the environment launches every product from its own call, =2 folds a following tanh too. */
int aixb200_matmul(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* b, const aixb200_tensor* result);

/* ---- data movement (aixDevice.hpp:64-69, 74-81) ---- */
int aixb200_transpose(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* result, size_t dim0, size_t dim1);
/* Dtype-converting copy of `count` elements. src may be host or device memory. dst is device memory; as an
 * extension over the reference, copy_immediate also accepts a host dst (device-to-host read-back). */
int aixb200_copy(aixb200_device* dev, const void* src, uint32_t src_dtype, void* dst, uint32_t dst_dtype, size_t count);
int aixb200_copy_immediate(aixb200_device* dev, const void* src, uint32_t src_dtype, void* dst, uint32_t dst_dtype, size_t count);
int aixb200_contiguous(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst);
int aixb200_slice_set(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst,
                      size_t dim, size_t start, size_t end, size_t step);
int aixb200_tril(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst, int64_t diagonal);
int aixb200_triu(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst, int64_t diagonal);
int aixb200_index_select(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst,
                         const aixb200_tensor* indices, size_t dim);
int aixb200_index_add(aixb200_device* dev, const aixb200_tensor* src, const aixb200_tensor* dst,
                      const aixb200_tensor* indices, size_t dim);

/* ---- diagnostics (reference: fuse::FlushDiagnostics aixFuse.hpp:144-156; kernel cache counters
 * aixDeviceMetalKernelGen.hpp:51-53) ---- */
typedef struct aixb200_stats
{
    uint64_t ops_recorded;          /* elementwise ops recorded since creation */
    uint64_t flushes;
    uint64_t fused_kernels;         /* generated-kernel launches */
    uint64_t fused_ops;             /* recorded ops folded into those launches */
    uint64_t fills_absorbed;        /* fills turned into kernel scalars */
    uint64_t stores_elided;         /* intermediate results never written to memory */
    uint64_t kernel_cache_hits;
    uint64_t kernel_cache_misses;   /* == NVRTC compilations + disk-cache loads */
    uint64_t nvrtc_compiles;
    double   nvrtc_ms;              /* total time spent in NVRTC */
    uint64_t static_kernel_launches;/* reductions, GEMM, copies ... */
    uint64_t total_kernel_launches; /* every kernel this device put on its stream */
    uint64_t bytes_in_use;          /* handed out by allocate and not yet deallocated */
    uint64_t bytes_cached;          /* idle blocks held by the allocator */
    uint64_t bytes_reserved;        /* obtained from CUDA */
    uint64_t cuda_mallocs;          /* calls that reached the CUDA allocator */
    uint64_t h2d_bytes;             /* staged host->device */
    uint64_t d2h_bytes;
    uint64_t reductions_fused;      /* full sums / maxima folded into the kernel that produces their operand */
    uint64_t prepared_operand_hits; /* f32 matmul operands whose two-term fp16 form was still cached */
    uint64_t prepared_operand_builds; /* ... and those that had to be prepared (max pass + split) */
    uint64_t prepared_operand_max_known; /* ... of which the max pass was skipped: the producing kernel had left max|x| */
    uint64_t matmul_consumers_folded; /* recorded `product + row vector` and tanh ops that ran inside the product's kernel */
    uint64_t reserved[1];
} aixb200_stats;
int aixb200_get_stats(aixb200_device* dev, aixb200_stats* out);
/* CUDA C source of the most recently generated kernel (for inspection and tests); NULL if none yet. */
const char* aixb200_last_kernel_source(const aixb200_device* dev);

/* ---- device-side timing on the device's stream ---- */
typedef struct aixb200_event aixb200_event;
int aixb200_event_create(aixb200_device* dev, aixb200_event** out);
int aixb200_event_record(aixb200_device* dev, aixb200_event* ev);    /* flushes recorded work first */
int aixb200_event_elapsed_ms(aixb200_device* dev, aixb200_event* start, aixb200_event* stop, float* ms); /* waits for stop */
int aixb200_event_destroy(aixb200_device* dev, aixb200_event* ev);
/* Writes `bytes` of device memory so that nothing useful stays in L2 (timing hygiene between iterations). */
int aixb200_flush_l2(aixb200_device* dev);
/* Self-test of the bounded device-side waits: launches one tiny kernel (no TMA, no tensor-core work) that waits on an
 * mbarrier nobody arrives at and gives up after `limit_ns`. The kernel returns normally; it raises the device's error
 * word, and the next aixb200_synchronize returns AIXB200_ERR_TIMEOUT once, after which the device works as before.
 * This is the path the tensor-core matmul takes if one of its waits ever runs out. */
int aixb200_self_test_bounded_wait(aixb200_device* dev, uint64_t limit_ns);

/* ---- data-parallel exchange (no reference counterpart: the reference has no multi-device code) ---- */
#define AIXB200_COMM_ID_BYTES 128
int aixb200_comm_unique_id(void* id_out /* AIXB200_COMM_ID_BYTES */);
/* Creates the communicator (NCCL over NVLink / NVSwitch). Blocking by default. With the environment variable
 * AIXB200_COMM_INIT_TIMEOUT_MS set, initialisation is non-blocking and polled: if it has not completed by then (a rank
 * that never joins) the communicator is aborted and the call returns AIXB200_ERR_TIMEOUT instead of hanging. Every
 * collective, aixb200_comm_wait and aixb200_synchronize also query the communicator's asynchronous state first: an error
 * reported there (a peer that died, a network fault) aborts the communicator once and returns AIXB200_ERR_RUNTIME; later
 * collectives on it fail at once. */
int aixb200_comm_init(aixb200_device* dev, int rank, int nranks, const void* id);
/* Host-side fault injection for tests of those paths; process-wide, no GPU or NCCL involved. mode 0: the real NCCL;
 * 1: initialisation never completes; 2: everything succeeds until the communicator's state has been queried
 * `error_after_polls` times, then it reports a remote error. With a back end injected, aixb200_comm_init also works on a
 * dry-run device. aixb200_comm_injected_counters reads how often the stand-ins were initialised, polled and aborted. */
int aixb200_comm_inject_backend(int mode, int error_after_polls);
int aixb200_comm_injected_counters(int* inits, int* polls, int* aborts);
/* In-place sum all-reduce over `count` elements of dtype (F32, F64, BF16, F16, I32, I64) followed by a
 * multiplication by `scale` (1/nranks averages). Ordered after all work recorded so far. */
int aixb200_all_reduce(aixb200_device* dev, void* data, size_t count, uint32_t dtype, double scale);
/* Overlapped form: the same collective on a side stream, ordered after all work recorded so far. Work issued later on
 * the device's stream runs concurrently with it, except work that touches `data`: any later op whose operands or result
 * overlap a collective in flight is ordered after that collective (and only that one). aixb200_comm_wait() orders the
 * device's stream after every collective started this way (also implied by synchronize and by the blocking
 * all-reduce). */
int aixb200_all_reduce_async(aixb200_device* dev, void* data, size_t count, uint32_t dtype, double scale);
/* Sharded-optimizer pair, both in place on a buffer of `count` elements (a multiple of the number of ranks) and both
 * overlapped like aixb200_all_reduce_async. reduce_scatter: afterwards slice [r*count/R, (r+1)*count/R) of rank r's buffer
 * holds the sum over the ranks times `scale`; the other slices hold unspecified data. all_gather: every rank contributes
 * its own slice r and receives the others', so that all ranks hold identical buffers. A rank that updates only its slice
 * of a parameter between the two (its share of the optimizer state) does 1/R of the optimizer's work and moves half the
 * bytes of an all-reduce before the update can start. */
int aixb200_reduce_scatter_async(aixb200_device* dev, void* data, size_t count, uint32_t dtype, double scale);
int aixb200_all_gather_async(aixb200_device* dev, void* data, size_t count, uint32_t dtype);
/* Rank and size of the device's communicator (0 and 1 without one). */
int aixb200_comm_rank(aixb200_device* dev, int* rank, int* nranks);
int aixb200_comm_wait(aixb200_device* dev);
/* Joins only the collectives that touch [data, data + bytes): recorded work that does not depend on them is launched
 * first. An optimizer calls it before it starts on one parameter, so that the join falls between parameters. */
int aixb200_comm_wait_for(aixb200_device* dev, const void* data, size_t bytes);
int aixb200_comm_destroy(aixb200_device* dev);

#ifdef __cplusplus
}
#endif
#endif /* AIXB200_H */
