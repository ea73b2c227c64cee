// Context, error reporting, the cudaMalloc pool, the per-op bump workspace, copies and
// the tensor-map encoder.  Host-side only; the one kernel here fills memory.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "internal.h"

namespace b200 {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int fail_cuda(cudaError_t e, const char* what) {
    return fail(B200_ECUDA, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

bool pdl_enabled() {
    static const bool on = getenv("B200_NO_PDL") == nullptr; // debugging aid: plain stream order when set
    return on;
}

static size_t round_up(size_t n, size_t a) { return (n + a - 1) / a * a; }

// Size classes: 256 B granules below 1 MiB, 2 MiB granules above, so a freed block is
// reusable by the next request of about the same size without splitting.
static size_t size_class(size_t bytes) {
    if (bytes == 0) bytes = 1;
    return bytes < (1u << 20) ? round_up(bytes, 256) : round_up(bytes, 2u << 20);
}

int pool_alloc(b200_ctx* ctx, size_t bytes, void** out) {
    size_t need = size_class(bytes);
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->free_blocks.lower_bound(need);
    // Take a free block only if it wastes at most 25 %.
    if (it != ctx->free_blocks.end() && it->first <= need + need / 4) {
        *out = it->second;
        ctx->live_blocks[it->second] = it->first;
        ctx->bytes_in_use += it->first;
        if (ctx->capturing) ctx->capture_blocks.emplace_back(it->second, it->first);
        ctx->free_blocks.erase(it);
        return B200_OK;
    }
    if (ctx->capturing)
        return fail(B200_ENOMEM, "pool: %zu bytes needed while capturing a graph; run the sequence once eagerly "
                                 "so the pool and workspace are warm", need);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, need);
    if (e != cudaSuccess) {
        // Give cached blocks back to the driver once and retry before reporting exhaustion.
        cudaGetLastError();
        for (auto& kv : ctx->free_blocks) {
            cudaFree(kv.second);
            ctx->bytes_reserved -= kv.first;
        }
        ctx->free_blocks.clear();
        e = cudaMalloc(&p, need);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(B200_ENOMEM, "pool: cudaMalloc(%zu) failed: %s", need, cudaGetErrorString(e));
        }
    }
    ctx->live_blocks[p] = need;
    ctx->bytes_in_use += need;
    ctx->bytes_reserved += need;
    *out = p;
    return B200_OK;
}

int pool_free(b200_ctx* ctx, void* p) {
    if (!p) return B200_OK;
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->live_blocks.find(p);
    if (it == ctx->live_blocks.end()) return fail(B200_EINVAL, "pool_free: %p is not a live pool block", p);
    // A block some live graph still writes on replay must not reach another owner: it waits in
    // `held` until the last such graph is destroyed.
    if (ctx->pinned.count(p)) ctx->held.emplace(p, it->second);
    else ctx->free_blocks.emplace(it->second, p);
    ctx->bytes_in_use -= it->second;
    ctx->live_blocks.erase(it);
    return B200_OK;
}

// graph_end: every block the capture touched becomes pinned by the new graph.
static void pin_capture_blocks(b200_ctx* ctx, b200_graph* g) {
    std::lock_guard<std::mutex> lk(ctx->mu);
    std::unordered_set<void*> seen;
    for (auto& bs : ctx->capture_blocks) {
        void* p = bs.first;
        if (!seen.insert(p).second) continue;
        g->pins.push_back(p);
        ctx->pinned[p]++;
        if (ctx->live_blocks.count(p) || ctx->held.count(p)) continue;
        // Handed out and returned while capturing: take it back out of the free list.
        auto range = ctx->free_blocks.equal_range(bs.second);
        for (auto it = range.first; it != range.second; ++it)
            if (it->second == p) {
                ctx->free_blocks.erase(it);
                ctx->held.emplace(p, bs.second);
                break;
            }
    }
    ctx->capture_blocks.clear();
    ctx->graphs.insert(g);
}

// graph_destroy: blocks no live graph uses any more go back into circulation.
static void unpin_blocks(b200_graph* g) {
    b200_ctx* ctx = g->ctx;
    if (!ctx) return;
    std::lock_guard<std::mutex> lk(ctx->mu);
    for (void* p : g->pins) {
        auto it = ctx->pinned.find(p);
        if (it == ctx->pinned.end()) continue;
        if (--it->second > 0) continue;
        ctx->pinned.erase(it);
        auto h = ctx->held.find(p);
        if (h != ctx->held.end()) {
            ctx->free_blocks.emplace(h->second, p);
            ctx->held.erase(h);
        }
    }
    g->pins.clear();
    ctx->graphs.erase(g);
}

static size_t pool_block_size(b200_ctx* ctx, void* p) {   // caller holds ctx->mu
    auto it = ctx->live_blocks.find(p);
    return it == ctx->live_blocks.end() ? 0 : it->second;
}

int ws_scratch(b200_ctx* ctx, size_t bytes, void** out) {
    size_t off = round_up(ctx->ws_used, 256);
    size_t need = off + bytes;
    if (!ctx->ws_buf || need > ctx->ws_cap) {
        // Retire, never release here: pointers handed out earlier in this op still point
        // into the old block and their kernels may not have run yet.
        if (ctx->ws_buf) ctx->ws_retired.push_back({ctx->ws_buf, ctx->ws_cap});
        size_t cap = need + need / 2;
        if (cap < (1u << 20)) cap = 1u << 20;
        void* p = nullptr;
        int rc = pool_alloc(ctx, cap, &p);
        if (rc) return rc;
        ctx->ws_buf = p;
        ctx->ws_cap = cap;
        // A fresh block starts at offset 0, as the reference's does: `off` was computed
        // against the old block but is a valid offset in the new, larger one.
    }
    ctx->ws_used = need;
    *out = static_cast<char*>(ctx->ws_buf) + off;
    if (ctx->capturing) {
        std::lock_guard<std::mutex> lk(ctx->mu);
        ctx->capture_blocks.emplace_back(ctx->ws_buf, pool_block_size(ctx, ctx->ws_buf));
    }
    return B200_OK;
}

int make_tmap(b200_ctx* ctx, CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base,
              const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
              CUtensorMapSwizzle swz) {
    cuuint64_t gdim[5];
    cuuint64_t gstr[5];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
        if (i + 1 < rank) gstr[i] = strides_bytes[i];
    }
    CUresult r = ctx->encode(map, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(B200_DECLINE_ALIGN,
                    "cuTensorMapEncodeTiled failed (%d): base %p rank %d dims %llu,%llu,%llu strides "
                    "%llu,%llu box %u,%u,%u",
                    (int)r, base, rank, (unsigned long long)gdim[0], (unsigned long long)(rank > 1 ? gdim[1] : 0),
                    (unsigned long long)(rank > 2 ? gdim[2] : 0), (unsigned long long)(rank > 1 ? gstr[0] : 0),
                    (unsigned long long)(rank > 2 ? gstr[1] : 0), bx[0], rank > 1 ? bx[1] : 0,
                    rank > 2 ? bx[2] : 0);
    }
    return B200_OK;
}

} // namespace b200

using namespace b200;

extern "C" {

const char* b200_last_error(void) { return g_err; }
const char* b200_version(void) { return "b200dnn-0.1 sm_100a"; }

int b200_ctx_create(int device, b200_ctx** out) {
    B200_REQUIRE(out != nullptr, B200_EINVAL, "ctx_create: out is null");
    int n = 0;
    B200_CUDA(cudaGetDeviceCount(&n));
    B200_REQUIRE(device >= 0 && device < n, B200_EINVAL, "ctx_create: device %d of %d", device, n);
    B200_CUDA(cudaSetDevice(device));
    b200_ctx* c = new b200_ctx();
    c->device = device;
    cudaError_t e = cudaGetDeviceProperties(&c->prop, device);
    if (e != cudaSuccess) { delete c; return fail_cuda(e, "cudaGetDeviceProperties"); }
    if (c->prop.major != 10) {
        int maj = c->prop.major, min = c->prop.minor;
        delete c;
        return fail(B200_ECUDA, "ctx_create: device %d is sm_%d%d; this library carries sm_100a code only",
                    device, maj, min);
    }
    e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete c; return fail_cuda(e, "cudaStreamCreate"); }
    e = cudaMalloc(&c->d_status, 256);
    if (e != cudaSuccess) { cudaStreamDestroy(c->stream); delete c; return fail_cuda(e, "cudaMalloc(status)"); }
    cudaMemsetAsync(c->d_status, 0, 256, c->stream);
    e = cudaMalloc(&c->sk_flags, (SK_FLAG_COUNT + GEMV_COUNTER_COUNT) * sizeof(int));
    if (e != cudaSuccess) { cudaFree(c->d_status); cudaStreamDestroy(c->stream); delete c; return fail_cuda(e, "cudaMalloc(flags)"); }
    // Zeroed on the context's own stream (a non-blocking stream does not wait for the legacy default
    // stream), and complete before the first launch can be issued.
    cudaMemsetAsync(c->sk_flags, 0, (SK_FLAG_COUNT + GEMV_COUNTER_COUNT) * sizeof(int), c->stream);
    cudaStreamSynchronize(c->stream);
    cudaEventCreate(&c->ev0);
    cudaEventCreate(&c->ev1);
    e = cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { b200_ctx_destroy(c); return fail_cuda(e, "cudaStreamCreate(copy lane)"); }
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
        b200_ctx_destroy(c);
        return fail(B200_ECUDA, "ctx_create: cuTensorMapEncodeTiled not available from the driver");
    }
    c->encode = reinterpret_cast<EncodeTiledFn>(fn);
    *out = c;
    return B200_OK;
}

int b200_ctx_destroy(b200_ctx* c) {
    if (!c) return B200_OK;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->copy_stream) { cudaStreamSynchronize(c->copy_stream); cudaStreamDestroy(c->copy_stream); }
    for (b200_graph* g : c->graphs) g->ctx = nullptr;   // a graph destroyed later has nothing left to unpin
    for (auto& kv : c->free_blocks) cudaFree(kv.second);
    for (auto& kv : c->live_blocks) cudaFree(kv.first);
    for (auto& kv : c->held) cudaFree(kv.first);
    if (c->d_status) cudaFree(c->d_status);
    if (c->sk_flags) cudaFree(c->sk_flags);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
    return B200_OK;
}

int b200_caps(b200_ctx* c, b200_caps_t* out) {
    B200_REQUIRE(c && out, B200_EINVAL, "caps: null argument");
    out->coopmat = 1;
    out->tile = 16;
    out->subgroup = 32;
    out->coopmatsubgroup = 32;
    out->sharedbudget = (int32_t)c->prop.sharedMemPerBlockOptin;
    out->workgrouplimit = c->prop.maxThreadsPerBlock;
    out->cores = c->prop.multiProcessorCount;
    out->warps = c->prop.maxThreadsPerMultiProcessor / 32;
    out->cc_major = c->prop.major;
    out->cc_minor = c->prop.minor;
    out->total_mem = (int64_t)c->prop.totalGlobalMem;
    return B200_OK;
}

int b200_sync(b200_ctx* c) {
    B200_REQUIRE(c, B200_EINVAL, "sync: null ctx");
    B200_CUDA(cudaStreamSynchronize(c->stream));
    B200_CUDA(cudaStreamSynchronize(c->copy_stream));
    int st = 0;
    B200_CUDA(cudaMemcpy(&st, c->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) {
        // A kernel that gave up may have left hand-off flags and arrival counters set: clear them with
        // the status word, on the context's stream, before anything else is launched.
        cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream);
        cudaMemsetAsync(c->sk_flags, 0, (SK_FLAG_COUNT + GEMV_COUNTER_COUNT) * sizeof(int), c->stream);
        cudaStreamSynchronize(c->stream);
        return fail(B200_EKERNEL, "a kernel gave up a bounded wait (device status %d)", st);
    }
    return B200_OK;
}

void* b200_stream(b200_ctx* c) { return c ? (void*)c->stream : nullptr; }
int64_t b200_launch_count(b200_ctx* c) { return c ? c->launches : 0; }

int b200_timer_start(b200_ctx* c) {
    B200_REQUIRE(c, B200_EINVAL, "timer_start: null ctx");
    B200_CUDA(cudaEventRecord(c->ev0, c->stream));
    return B200_OK;
}
int b200_timer_stop(b200_ctx* c, float* ms) {
    B200_REQUIRE(c && ms, B200_EINVAL, "timer_stop: null argument");
    B200_CUDA(cudaEventRecord(c->ev1, c->stream));
    B200_CUDA(cudaEventSynchronize(c->ev1));
    B200_CUDA(cudaEventElapsedTime(ms, c->ev0, c->ev1));
    return B200_OK;
}

int b200_graph_begin(b200_ctx* c) {
    B200_REQUIRE(c, B200_EINVAL, "graph_begin: null ctx");
    B200_REQUIRE(!c->capturing, B200_EINVAL, "graph_begin: already capturing");
    B200_CUDA(cudaSetDevice(c->device));
    B200_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    c->capturing = true;
    c->capture_blocks.clear();
    return B200_OK;
}
int b200_graph_end(b200_ctx* c, b200_graph** out) {
    B200_REQUIRE(c && out, B200_EINVAL, "graph_end: null argument");
    B200_REQUIRE(c->capturing, B200_EINVAL, "graph_end: not capturing");
    c->capturing = false;
    cudaGraph_t g = nullptr;
    B200_CUDA(cudaStreamEndCapture(c->stream, &g));
    cudaGraphExec_t ex = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) {
        c->capture_blocks.clear();
        return fail_cuda(e, "cudaGraphInstantiate");
    }
    b200_graph* r = new b200_graph();
    r->exec = ex;
    r->ctx = c;
    pin_capture_blocks(c, r);
    *out = r;
    return B200_OK;
}
int b200_graph_launch(b200_ctx* c, b200_graph* g) {
    B200_REQUIRE(c && g && g->exec, B200_EINVAL, "graph_launch: null argument");
    B200_CUDA(cudaGraphLaunch(g->exec, c->stream));
    return B200_OK;
}
int b200_graph_destroy(b200_graph* g) {
    if (g) {
        if (g->exec) cudaGraphExecDestroy(g->exec);
        unpin_blocks(g);
        delete g;
    }
    return B200_OK;
}

int b200_pool_alloc(b200_ctx* c, size_t bytes, void** dptr) {
    B200_REQUIRE(c && dptr, B200_EINVAL, "pool_alloc: null argument");
    B200_CUDA(cudaSetDevice(c->device));
    return pool_alloc(c, bytes, dptr);
}
int b200_pool_free(b200_ctx* c, void* dptr) {
    B200_REQUIRE(c, B200_EINVAL, "pool_free: null ctx");
    return pool_free(c, dptr);
}
int b200_pool_stats(b200_ctx* c, size_t* in_use, size_t* reserved) {
    B200_REQUIRE(c, B200_EINVAL, "pool_stats: null ctx");
    if (in_use) *in_use = c->bytes_in_use;
    if (reserved) *reserved = c->bytes_reserved;
    return B200_OK;
}

int b200_upload(b200_ctx* c, void* dst, const void* src, size_t bytes) {
    B200_REQUIRE(c && (bytes == 0 || (dst && src)), B200_EINVAL, "upload: null argument");
    if (bytes == 0) return B200_OK;
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
    B200_CUDA(cudaStreamSynchronize(c->stream));
    return B200_OK;
}
int b200_download(b200_ctx* c, void* dst, const void* src, size_t bytes) {
    B200_REQUIRE(c && (bytes == 0 || (dst && src)), B200_EINVAL, "download: null argument");
    if (bytes == 0) return B200_OK;
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
    B200_CUDA(cudaStreamSynchronize(c->stream));
    return B200_OK;
}
int b200_upload_async(b200_ctx* c, void* dst, const void* src, size_t bytes) {
    B200_REQUIRE(c && (bytes == 0 || (dst && src)), B200_EINVAL, "upload_async: null argument");
    if (bytes == 0) return B200_OK;
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
    return B200_OK;
}
int b200_download_async(b200_ctx* c, void* dst, const void* src, size_t bytes) {
    B200_REQUIRE(c && (bytes == 0 || (dst && src)), B200_EINVAL, "download_async: null argument");
    if (bytes == 0) return B200_OK;
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
    return B200_OK;
}
// ---- the copy lane and its events
static cudaStream_t lane_stream(b200_ctx* c, int lane) { return lane == B200_LANE_COPY ? c->copy_stream : c->stream; }

int b200_copy_lane_upload(b200_ctx* c, void* dst, const void* src, size_t bytes) {
    B200_REQUIRE(c && (bytes == 0 || (dst && src)), B200_EINVAL, "copy_lane_upload: null argument");
    if (bytes == 0) return B200_OK;
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->copy_stream));
    return B200_OK;
}
int b200_copy_lane_download(b200_ctx* c, void* dst, const void* src, size_t bytes) {
    B200_REQUIRE(c && (bytes == 0 || (dst && src)), B200_EINVAL, "copy_lane_download: null argument");
    if (bytes == 0) return B200_OK;
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->copy_stream));
    return B200_OK;
}
int b200_event_create(b200_ctx* c, b200_event** out) {
    B200_REQUIRE(c && out, B200_EINVAL, "event_create: null argument");
    B200_CUDA(cudaSetDevice(c->device));
    cudaEvent_t ev = nullptr;
    B200_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    b200_event* e = new b200_event();
    e->ev = ev;
    e->device = c->device;
    *out = e;
    return B200_OK;
}
int b200_event_destroy(b200_event* e) {
    if (e) {
        if (e->ev) cudaEventDestroy(e->ev);
        delete e;
    }
    return B200_OK;
}
int b200_event_record(b200_ctx* c, b200_event* e, int lane) {
    B200_REQUIRE(c && e && e->ev, B200_EINVAL, "event_record: null argument");
    B200_REQUIRE(lane == B200_LANE_COMPUTE || lane == B200_LANE_COPY, B200_EINVAL, "event_record: lane %d", lane);
    B200_REQUIRE(!(c->capturing && lane == B200_LANE_COMPUTE), B200_EINVAL, "event_record: the compute lane is being captured");
    B200_CUDA(cudaEventRecord(e->ev, lane_stream(c, lane)));
    return B200_OK;
}
int b200_lane_wait_event(b200_ctx* c, int lane, b200_event* e) {
    B200_REQUIRE(c && e && e->ev, B200_EINVAL, "lane_wait_event: null argument");
    B200_REQUIRE(lane == B200_LANE_COMPUTE || lane == B200_LANE_COPY, B200_EINVAL, "lane_wait_event: lane %d", lane);
    B200_REQUIRE(!(c->capturing && lane == B200_LANE_COMPUTE), B200_EINVAL, "lane_wait_event: the compute lane is being captured");
    B200_CUDA(cudaStreamWaitEvent(lane_stream(c, lane), e->ev, 0));
    return B200_OK;
}

int b200_copy(b200_ctx* c, void* dst, const void* src, size_t bytes) {
    B200_REQUIRE(c && (bytes == 0 || (dst && src)), B200_EINVAL, "copy: null argument");
    if (bytes == 0) return B200_OK;
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, c->stream));
    return B200_OK;
}
int b200_fill_bytes(b200_ctx* c, void* dst, int byte, size_t bytes) {
    B200_REQUIRE(c && (bytes == 0 || dst), B200_EINVAL, "fill_bytes: null argument");
    if (bytes == 0) return B200_OK;
    B200_CUDA(cudaMemsetAsync(dst, byte, bytes, c->stream));
    return B200_OK;
}
int b200_host_alloc(size_t bytes, void** hptr) {
    B200_REQUIRE(hptr, B200_EINVAL, "host_alloc: null argument");
    B200_CUDA(cudaMallocHost(hptr, bytes ? bytes : 1));
    return B200_OK;
}
int b200_host_free(void* hptr) {
    if (hptr) B200_CUDA(cudaFreeHost(hptr));
    return B200_OK;
}

int b200_workspace_reset(b200_ctx* c) {
    B200_REQUIRE(c, B200_EINVAL, "workspace_reset: null ctx");
    // Blocks retired by the previous op go back to the pool: work is in order on one
    // stream, so anything launched later runs after everything that could read them.
    for (auto& r : c->ws_retired) pool_free(c, r.ptr);
    c->ws_retired.clear();
    c->ws_used = 0;
    return B200_OK;
}
int b200_workspace_scratch(b200_ctx* c, size_t bytes, void** dptr) {
    B200_REQUIRE(c && dptr, B200_EINVAL, "workspace_scratch: null argument");
    B200_CUDA(cudaSetDevice(c->device));
    return ws_scratch(c, bytes, dptr);
}
int b200_workspace_stats(b200_ctx* c, size_t* used, size_t* cap, int* retired) {
    B200_REQUIRE(c, B200_EINVAL, "workspace_stats: null ctx");
    if (used) *used = c->ws_used;
    if (cap) *cap = c->ws_cap;
    if (retired) *retired = (int)c->ws_retired.size();
    return B200_OK;
}

int b200_timeline(b200_ctx* c, void* dptr) {
    B200_REQUIRE(c, B200_EINVAL, "timeline: null ctx");
    c->gemm_trace = static_cast<unsigned long long*>(dptr);
    return B200_OK;
}

int b200_shard_range(int64_t total, int world, int rank, int64_t align, int64_t* begin, int64_t* end) {
    B200_REQUIRE(begin && end && world > 0 && rank >= 0 && rank < world && total >= 0 && align > 0,
                 B200_EINVAL, "shard_range: bad argument");
    // Whole `align`-sized units are dealt out as evenly as possible (earlier ranks take
    // the remainder); the last, possibly partial, unit belongs to whichever rank holds it.
    int64_t units = (total + align - 1) / align;
    int64_t per = units / world, rem = units % world;
    int64_t ub = per * rank + (rank < rem ? rank : rem);
    int64_t ue = ub + per + (rank < rem ? 1 : 0);
    int64_t b = ub * align, e = ue * align;
    *begin = b < total ? b : total;
    *end = e < total ? e : total;
    return B200_OK;
}

} // extern "C"
