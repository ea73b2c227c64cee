// Library-internal declarations shared by the translation units of libb200dnn.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <unordered_map>
#include <unordered_set>
#include <utility>
#include <vector>

#include "../../include/b200dnn.h"

namespace b200 {

int fail(int code, const char* fmt, ...);  // records the thread's last error, returns code
int fail_cuda(cudaError_t e, const char* what);

#define B200_CUDA(call)                                         \
    do {                                                        \
        cudaError_t _e = (call);                                \
        if (_e != cudaSuccess) return ::b200::fail_cuda(_e, #call); \
    } while (0)

#define B200_REQUIRE(cond, code, ...)                        \
    do {                                                     \
        if (!(cond)) return ::b200::fail((code), __VA_ARGS__); \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct RetiredBlock {
    void* ptr;
    size_t bytes;
};

} // namespace b200

struct b200_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaDeviceProp prop{};
    int* d_status = nullptr;   // device status words: [0] first failed wait code
    int* sk_flags = nullptr;   // stream-K hand-off flags (zero between launches), SK_FLAG_COUNT ints, then
                               // GEMV_COUNTER_COUNT arrival counters (zero between launches)
    int64_t launches = 0;
    bool capturing = false;
    unsigned long long* gemm_trace = nullptr;  // device buffer of >= 32 slots while tracing, else null
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    cudaStream_t copy_stream = nullptr;   // the copy lane: host<->device copies that overlap the compute stream
    b200::EncodeTiledFn encode = nullptr;

    // cudaMalloc pool: free blocks by size, live blocks by pointer.
    std::mutex mu;
    std::multimap<size_t, void*> free_blocks;
    std::unordered_map<void*, size_t> live_blocks;
    size_t bytes_in_use = 0, bytes_reserved = 0;

    // Per-op bump workspace.
    void* ws_buf = nullptr;
    size_t ws_cap = 0, ws_used = 0;
    std::vector<b200::RetiredBlock> ws_retired;

    // Blocks a recorded graph has baked into its launches (pool blocks handed out and workspace
    // blocks used while capturing).  A pinned block that is freed waits in `held` instead of the
    // free list, so no later allocation can receive memory a replay will still write.
    std::vector<std::pair<void*, size_t>> capture_blocks;   // collected between graph_begin and graph_end
    std::unordered_map<void*, int> pinned;                  // block -> number of live graphs that use it
    std::unordered_map<void*, size_t> held;                 // freed while pinned: block -> size
    std::unordered_set<b200_graph*> graphs;                 // live graphs recorded on this context
};

constexpr int SK_FLAG_COUNT = 4096;
constexpr int GEMV_COUNTER_COUNT = 4096;   // arrival counters of the split matrix-vector product, after the flags

struct b200_event {
    cudaEvent_t ev = nullptr;
    int device = 0;
};

struct b200_graph {
    cudaGraphExec_t exec = nullptr;
    b200_ctx* ctx = nullptr;      // null once the context is gone
    std::vector<void*> pins;      // pool blocks this graph keeps out of circulation
};

namespace b200 {

// Encode a tiled tensor map of `rank` dims (innermost first).  strides_bytes has rank-1
// entries (the innermost stride is the element size).
int make_tmap(b200_ctx* ctx, CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base,
              const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
              CUtensorMapSwizzle swz);

int pool_alloc(b200_ctx* ctx, size_t bytes, void** out);
int pool_free(b200_ctx* ctx, void* p);
int ws_scratch(b200_ctx* ctx, size_t bytes, void** out);

// Attention over windows of at most 64 keys, E <= 64 (attention_window.cu).  Operands as the tensor-core
// path wants them: E contiguous, 16-byte aligned pointers and strides.
int attention_window_launch(b200_ctx* ctx, int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B, const b200_strided4* q,
                            const b200_strided4* k, const b200_strided4* v, const b200_strided4* o, int out_dtype,
                            float scale);

// GEMM with the bias broadcast along either axis (bias_per_n = 1: one value per column j,
// which is what a convolution lowered to a GEMM over pixels needs).  use_workspace = 0 keeps the
// planner to schedules that need no scratch memory (whole tiles only), so the call touches neither
// the workspace nor the pool.
int gemm_f16_run(b200_ctx* ctx, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* B,
                 int64_t ldb, const void* bias, int bias_per_n, void* out, int64_t ldo, int out_dtype,
                 int epilogue, int64_t nbatch, int64_t strideA, int64_t strideB, int64_t strideO,
                 int use_workspace = 1);

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Launch with the programmatic-serialization attribute (and a cluster width when > 1).  Only
// kernels that call grid_dep_wait() before their first global access may be launched this way.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dep(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              int cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

} // namespace b200
