/*
 * b200dnn — C ABI of the B200 (sm_100a) dense hot path that sits behind the
 * DNNKernels op-dispatch API (matmul!, sdpa!, layernorm!, convolution!, scratch!).
 *
 * Conventions
 *   - Every entry point returns an int status: 0 = ok, otherwise a B200_E* /
 *     B200_DECLINE_* code; nothing throws or aborts across the boundary.
 *     b200_last_error() returns the message of the last failure on this thread.
 *   - All array arguments are raw DEVICE pointers owned by the caller unless the
 *     name says "host".  The library keeps no caller pointer past the stream work
 *     of the call.  Work is asynchronous on the context's stream, in call order.
 *   - Arrays are column-major with the reversed torch shape (the reference's
 *     layout): a "(M,K) ld" matrix has element (i,k) at i + ld*k.
 *   - fp16 is IEEE binary16; accumulation is fp32 everywhere.
 *   - "reference" citations are file:line in the reference project
 *     (DNNKernels/src/...).
 */
#ifndef B200DNN_H
#define B200DNN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- status codes */
enum {
    B200_OK = 0,
    B200_EINVAL = 1,         /* null pointer / negative extent / bad enum            */
    B200_ECUDA = 2,          /* a CUDA runtime or driver call failed                 */
    B200_ENOMEM = 3,         /* pool or workspace exhausted                          */
    B200_EKERNEL = 4,        /* a kernel reported a bounded wait that ran out        */
    /* Planner refusals, the vocabulary of Decline(reason) (kernelplans.jl:21-35). */
    B200_DECLINE_OPERANDS = 16,  /* :operands  dtype/rank the fast path does not take */
    B200_DECLINE_EXTENT = 17,    /* :extent    an extent the tiling cannot cover      */
    B200_DECLINE_ALIGN = 18,     /* :wrapped   stride/pointer a TMA map cannot express*/
    B200_DECLINE_BIAS = 19,      /* :bias      a bias/mask of a shape the op cannot take */
    B200_DECLINE_ELTYPE = 20,    /* :eltype                                            */
    B200_DECLINE_TILING = 21     /* :tiling    no tile shape fits                      */
};

enum { B200_F16 = 0, B200_F32 = 1 };
/* actfn(name) (ops.jl:1684-1685): identity / relu_epi / geluexact, plus gelutanh. */
enum { B200_EPI_NONE = 0, B200_EPI_RELU = 1, B200_EPI_GELU = 2, B200_EPI_GELU_TANH = 3 };

typedef struct b200_ctx b200_ctx;

/* Device facts, the B200 answer to caps(backend)/DeviceCaps (context.jl:55-68). */
typedef struct {
    int32_t coopmat;         /* 1: tensor-core path present                           */
    int32_t tile;            /* MMA K granule in elements (16 for fp16)               */
    int32_t subgroup;        /* 32                                                     */
    int32_t coopmatsubgroup; /* 32                                                     */
    int32_t sharedbudget;    /* bytes of shared memory one CTA may use                */
    int32_t workgrouplimit;  /* 1024                                                   */
    int32_t cores;           /* SM count                                               */
    int32_t warps;           /* resident warps per SM                                  */
    int32_t cc_major, cc_minor;
    int64_t total_mem;
} b200_caps_t;

/* ------------------------------------------------------- context (Ctx, context.jl:240-331) */
int b200_ctx_create(int device, b200_ctx** out);
int b200_ctx_destroy(b200_ctx* ctx);
int b200_caps(b200_ctx* ctx, b200_caps_t* out);
/* KernelAbstractions.synchronize(backend): block until the context's stream is idle,
 * then report any device-side error flag raised by a kernel since the last sync. */
int b200_sync(b200_ctx* ctx);
const char* b200_last_error(void);
const char* b200_version(void);   /* KERNELS_VERSION analogue (DNNKernels.jl:26-72) */
void* b200_stream(b200_ctx* ctx); /* the cudaStream_t the context launches on      */
/* Number of kernels this library has launched on the context since creation.       */
int64_t b200_launch_count(b200_ctx* ctx);

/* Self-test of the bounded waits (no reference counterpart): launches one warp that waits, with a limit
 * of limit_ns (at most 100 ms), on a barrier nothing ever arrives at.  The wait runs out, the kernel
 * returns normally, and the next b200_sync reports B200_EKERNEL and clears the status, after which the
 * context works as before.  gave_up_dev (device int, may be NULL) receives 1 when the wait gave up. */
int b200_selftest_bounded_wait(b200_ctx* ctx, int64_t limit_ns, int* gave_up_dev);

/* CUDA-event timer on the context's stream (Diagnostics.optimes, context.jl:162-221). */
int b200_timer_start(b200_ctx* ctx);
int b200_timer_stop(b200_ctx* ctx, float* ms_out); /* records, synchronises, reads */

/* Capture / replay of a launch sequence (Lava capture / replay!, SAM2Runner/src/sam2.jl:90-115):
 * everything launched on the context between begin and end is recorded into a CUDA graph
 * instead of running; replay launches the whole sequence with one call.  The static slab and
 * the warmed-up workspace make every device address repeat, which is the precondition.  Run
 * the sequence once eagerly first: the pool must not need cudaMalloc while capturing.
 * A graph bakes device addresses into its launches.  Pool blocks handed out and workspace blocks used
 * while capturing stay out of circulation until the graph is destroyed (a b200_pool_free of one is
 * honoured then), so later allocations and workspace growth cannot receive memory a replay still
 * writes.  Every caller-owned buffer the captured calls were given must outlive the graph as well. */
typedef struct b200_graph b200_graph;
int b200_graph_begin(b200_ctx* ctx);
int b200_graph_end(b200_ctx* ctx, b200_graph** out);
int b200_graph_launch(b200_ctx* ctx, b200_graph* g);
int b200_graph_destroy(b200_graph* g);

/* ------------------------------------- memory (Mantle pool / toback, driver.jl:81-115) */
/* 256-byte aligned device block from the context's cudaMalloc pool (size-class free
 * lists; blocks return to the pool on free, to the driver on ctx destroy). */
int b200_pool_alloc(b200_ctx* ctx, size_t bytes, void** dptr);
int b200_pool_free(b200_ctx* ctx, void* dptr);
int b200_pool_stats(b200_ctx* ctx, size_t* bytes_in_use, size_t* bytes_reserved);
int b200_upload(b200_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int b200_download(b200_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes); /* syncs */
int b200_upload_async(b200_ctx* ctx, void* dst_dev, const void* src_pinned_host, size_t bytes);
int b200_download_async(b200_ctx* ctx, void* dst_pinned_host, const void* src_dev, size_t bytes);
int b200_copy(b200_ctx* ctx, void* dst_dev, const void* src_dev, size_t bytes);
int b200_fill_bytes(b200_ctx* ctx, void* dst_dev, int byte, size_t bytes);
int b200_host_alloc(size_t bytes, void** hptr); /* pinned host memory */
int b200_host_free(void* hptr);

/* The copy lane (new surface, no reference counterpart: the reference uploads with toback and reads results with
 * Array(), both blocking).  A second stream of the context for pinned-host <-> device copies, so that the input
 * of the next pass goes up and the result of the previous one comes down while the compute stream runs the
 * current pass.  Order between the two lanes is what the caller states with events: record an event on one lane,
 * make the other lane wait for it.  An event may be re-recorded; a wait refers to the record before it.
 * b200_sync waits for both lanes. */
enum { B200_LANE_COMPUTE = 0, B200_LANE_COPY = 1 };
typedef struct b200_event b200_event;
int b200_copy_lane_upload(b200_ctx* ctx, void* dst_dev, const void* src_pinned_host, size_t bytes);
int b200_copy_lane_download(b200_ctx* ctx, void* dst_pinned_host, const void* src_dev, size_t bytes);
int b200_event_create(b200_ctx* ctx, b200_event** out);
int b200_event_destroy(b200_event* e);
int b200_event_record(b200_ctx* ctx, b200_event* e, int lane);
int b200_lane_wait_event(b200_ctx* ctx, int lane, b200_event* e);

/* Per-op bump workspace: Workspace / reset! / scratch! (workspace.jl:19-106).
 * Offsets are 256-byte aligned; growth allocates max(need*1.5, 1 MiB) and RETIRES the
 * old block until the next reset, exactly as the reference does, so pointers handed
 * out earlier in the same op stay valid. */
int b200_workspace_reset(b200_ctx* ctx);
int b200_workspace_scratch(b200_ctx* ctx, size_t bytes, void** dptr);
int b200_workspace_stats(b200_ctx* ctx, size_t* used, size_t* capacity, int* retired);

/* ------------------------------------------------------------------------- GEMM */
/*
 * out(M,N) = epi(T(bias[i] + sum_k A(M,K)[i,k] * B(K,N)[k,j])), per batch plane.
 * Replaces matmul!/matmul_coopmat! (matmul.jl:78-100,235-273), the external
 * Lava.coopmat_gemm! it calls (matmul.jl:264,269), padcols_kernel! and
 * mm_epilogue_kernel! (matmul.jl:182-217), and batchedmatmul! (matmul.jl:364-392)
 * through nbatch/strides.  bias is (M,) fp16 or NULL and starts the fp32 accumulator;
 * the activation is applied to the value already rounded to out_dtype.
 * A is (M,K) with M contiguous (the dense weight hoistpermutes leaves), B is (K,N)
 * with K contiguous (the activations).  No padding of any extent is required; lda,
 * ldb, ldo and the plane strides are in elements.
 */
int b200_gemm_f16(b200_ctx* ctx, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                  const void* B, int64_t ldb, const void* bias, void* out, int64_t ldo,
                  int out_dtype, int epilogue, int64_t nbatch, int64_t strideA, int64_t strideB,
                  int64_t strideO);
/* mm_coopmat_plan (matmul.jl:172-179): B200_OK if the tensor-core kernel takes the
 * shape, else the Decline reason.  Callable before out is allocated. */
int b200_gemm_f16_supported(int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldo,
                            int out_dtype);
/* The tile plan the GEMM would run with (MMCoopMatPlan, kernelplans.jl:382-385). */
typedef struct {
    int32_t block_m, block_n, block_k, stages;
    int32_t tiles_m, tiles_n, ctas;
    int32_t smem_bytes;
} b200_gemm_plan_t;
int b200_gemm_f16_plan(b200_ctx* ctx, int64_t M, int64_t N, int64_t K, int64_t nbatch,
                       b200_gemm_plan_t* plan);

/* The one-token product of matmul! (MMGemvPlan + Lava.gemv!, matmul.jl:103-137):
 * out[m] = epi(T(bias[m] + sum_k A[m,k] x[k])), A (M,K) column-major with leading dimension lda
 * (M contiguous), x (K), bias (M) or NULL, all of in_dtype (B200_F32 as in the reference, or
 * B200_F16); out (M) of out_dtype (fp32, or fp16 for fp16 operands); fp32 accumulation.  Any lda >= M
 * and any element-aligned A are read as aligned 16-byte vectors, which may include the other bytes of
 * the 16-byte blocks the array's first and last elements sit in.  Scratch for a split along K comes from
 * the context workspace. */
int b200_gemv(b200_ctx* ctx, int64_t M, int64_t K, const void* A, int64_t lda, const void* x,
              const void* bias, int in_dtype, void* out, int out_dtype, int epilogue);

/* Diagnostics: while dptr (a device buffer of 256 uint64, zeroed by the caller) is set, worker 0 of
 * every GEMM launch records a timeline into it — globaltimer nanoseconds at [slot] and the SM's cycle
 * counter at [64 + slot]; slots: 0 entry, 1 set-up done, 3 first operand stage landed, 4.. all UMMAs
 * of the worker's tile 0, 1, 2, 3+ issued, 8.. their accumulators complete, 12.. their epilogues
 * done, 16 exit; [128 + w] is the time worker w (w < 120) left.  NULL stops it.  The ratio of the two
 * clocks over the main loop gives the SM clock the kernel really ran at. */
int b200_timeline(b200_ctx* ctx, void* dptr);

/* -------------------------------------------------------------------- attention */
/*
 * Fused non-causal scaled-dot-product attention, single pass, online softmax.
 * Replaces sdpa!/sdpaflashcm! + attn_flash_cm! + attn_flash_cm_merge!
 * (attention.jl:773-776, flash.jl:459-1036,1398-1484), the scalar attn_flash!
 * (flash.jl:160-271, via out_dtype = B200_F32) and the toLE_tiled_* / densify layout
 * passes (attention.jl:342-396), which are unnecessary here because q/k/v are read
 * through their strides.  q,k,v are (E,L,H,B) fp16 with element strides
 * s = {sE,sL,sH,sB}, sE == 1; out is dense (E,Lq,H,B) in out_dtype.
 * scale multiplies the fp32 scores; softmax is fp32; P is rounded to fp16 before P*V.
 */
typedef struct {
    const void* ptr;
    int64_t stride[4]; /* elements: E, L, H, B */
} b200_strided4;
int b200_attention_f16(b200_ctx* ctx, int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                       const b200_strided4* q, const b200_strided4* k, const b200_strided4* v,
                       void* out, int out_dtype, float scale);
/* Same, with out as an (E,Lq,H,B) view of arbitrary L/H/B strides (E contiguous).  Writing the
 * token-major layout the next addmm reads — strides {1, E*H, E, E*H*Lq} — folds the
 * clone/contiguous that follows sdpa in the exported graphs (execute.jl:257-277) into the store. */
int b200_attention_f16_strided(b200_ctx* ctx, int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                               const b200_strided4* q, const b200_strided4* k, const b200_strided4* v,
                               const b200_strided4* out, int out_dtype, float scale);
/* Same, with the additive mask of _scaled_dot_product_efficient_attention (ops.jl:1365-1375,
 * attention.jl:55-59): bias is fp16 in the graph's own (Lk,Lq,H,B) order, stride[] = element strides
 * along Lk, Lq, H, B with 0 on a broadcast (size-1) axis; bias == NULL or bias->ptr == NULL means no
 * mask.  The mask is added to the scaled fp32 score; -inf entries block a key, and a row whose keys
 * are all blocked comes out as zeros (attn_softmax, attention.jl:73-100).  The reference declines a
 * bias on its fused path (flashcm_plan -> Decline(:bias)) and runs three passes; here it stays fused. */
int b200_attention_f16_bias(b200_ctx* ctx, int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                            const b200_strided4* q, const b200_strided4* k, const b200_strided4* v,
                            const b200_strided4* bias, const b200_strided4* out, int out_dtype, float scale);
/* flashcm_plan (flash.jl:1322-1374): B200_OK or the Decline reason (has_bias is accepted and ignored:
 * a mask does not decline here). */
int b200_attention_f16_supported(int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B,
                                 const int64_t* qstride, const int64_t* kstride,
                                 const int64_t* vstride, int has_bias);

/* Which way a call will run: 0 the fused tensor-core kernel (FlashCMPlan's place), 1 two batched GEMMs with a
 * softmax between them (sdpa_coopmat! + attn_softmax_rows!, attention.jl:528-705: head dims 136..4096 in
 * multiples of 8, E contiguous), 2 the scalar kernel.  Every route takes the additive mask. */
int b200_attention_f16_route(int64_t E, int64_t Lq, int64_t Lk, int64_t H, int64_t B, const int64_t* qstride,
                             const int64_t* kstride, const int64_t* vstride);

/* ------------------------------------------------------------------- layer norm */
/*
 * layernorm!/layernorm_kernel! (layernorm.jl:44-135): a is (C, groups) contiguous,
 * in_dtype/out_dtype fp16 or fp32; gamma/beta are (C,) in in_dtype or NULL; mean and
 * rstd are fp32 (groups,).  fp32 statistics, variance about the mean.
 */
int b200_layernorm(b200_ctx* ctx, int64_t groups, int64_t C, const void* a, int in_dtype, void* out,
                   int out_dtype, float* mean, float* rstd, const void* gamma, const void* beta,
                   float eps);

/*
 * add.Tensor (+ clamp.default) + native_layer_norm in one launch, fp16:
 *     x <- clamp(fp16(x + h), lo, hi)   (clamp only if use_clamp);   out <- LN(x)
 * The reference runs these as separate graph ops (ops.jl:186-197,323-335,575-647; its own
 * fusion of element-wise chains is fuse.jl).  Results are bit-identical to the three ops in
 * sequence; x is updated in place, x/h/out are (C, groups) contiguous.
 */
int b200_add_layernorm_f16(b200_ctx* ctx, int64_t groups, int64_t C, void* x, const void* h, int use_clamp,
                           float lo, float hi, void* out, float* mean, float* rstd, const void* gamma,
                           const void* beta, float eps);

/* ------------------------------------------------------- convolution as a GEMM */
/*
 * im2col_kernel! (conv_coopmat.jl:246-289): col (MP,CRSP) fp16 column-major from
 * x (W,H,Cin,N); rows >= NPQ, columns >= KW*KH*Cin and out-of-image taps are zero.  MP (the
 * padded row count) must be a multiple of 8 and col 16-byte aligned: rows leave in 16-byte stores.
 */
int b200_im2col_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW,
                    int64_t KH, int64_t sx, int64_t sy, int64_t px, int64_t py, int64_t dx,
                    int64_t dy, int64_t MP, int64_t CRSP, const void* x, void* col);
/*
 * convolution! for one group (conv.jl:100-145) lowered as convolution_coopmat!
 * (conv_coopmat.jl:341-392) does: [im2col unless 1x1/s1/p0] + GEMM with the bias and
 * activation fused, written straight into out (OW,OH,Cout,N) — no fp32 plane and no
 * conv_epilogue_kernel! pass.  x (W,H,Cin,N), w (KW,KH,Cin,Cout) fp16.  Scratch comes
 * from the context's workspace.
 */
int b200_conv2d_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW,
                    int64_t KH, int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py,
                    int64_t dx, int64_t dy, const void* x, const void* w, const void* bias,
                    void* out, int out_dtype, int epilogue);

/* The same with groups >= 1 (conv.jl:26-51,100-145; the reference runs grouped convolutions on its direct kernel):
 * w is (KW,KH,Cin/groups,Cout); each group is lowered like the ungrouped convolution, on its own channel slices. */
int b200_conv2d_grouped_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW,
                            int64_t KH, int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py,
                            int64_t dx, int64_t dy, int64_t groups, const void* x, const void* w, const void* bias,
                            void* out, int out_dtype, int epilogue);
/*
 * convolutiontranspose! (conv.jl:247-290): x (W,H,Cin,N), w (KW,KH,Cout/groups,Cin) — the transposed weight carries
 * its channel axes the other way round — out (OW,OH,Cout,N) with OW = (W-1)*sx - 2*px + dx*(KW-1) + opx + 1.  The
 * non-overlapping case (stride equal to the kernel, no padding, dilation or output padding, one group: shufflecase,
 * conv.jl:219-222) is a GEMM over (W*H) x Cin x (KW*KH*Cout) followed by the depth-to-space scatter (shuffleout,
 * conv.jl:232-246); everything else is the deterministic gather (convtranspose2d, conv.jl:147-190).  Scratch comes
 * from the context's workspace.
 */
int b200_convtranspose2d_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW,
                             int64_t KH, int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py,
                             int64_t dx, int64_t dy, int64_t opx, int64_t opy, int64_t groups, const void* x,
                             const void* w, const void* bias, void* out, int out_dtype);

/*
 * The same convolution for callers that must not allocate device memory when they call: a
 * server whose own allocator took the whole GPU at start-up, or a loop that may not make a
 * device-synchronising call such as cudaMalloc/cudaFree.  (No counterpart in the reference;
 * b200_conv2d_f16 above is the entry point that replaces the reference's convolution.)
 * The im2col matrix and the padded weight live in a fixed 32 MiB array built into the library
 * (each GPU that loads the library holds it until the process exits) instead of the workspace,
 * and the call makes no cudaMalloc, cudaFree or other allocating call.  Same arguments and
 * results as b200_conv2d_f16.
 *   - Limit: padded weight (only when KW*KH*Cin is not a multiple of 8: roundup8(KW*KH*Cin)*Cout*2
 *     bytes, rounded up to 256) + im2col matrix (only when not 1x1/stride 1/no padding:
 *     roundup8(OW*OH)*KW*KH*Cin*2 bytes) must fit in 32 MiB; otherwise B200_ENOMEM with the sizes
 *     in b200_last_error().  The 1024x1024x3, 7x7 stride-4 stem needs 19.3 MB.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress);
 *     make that first call before starting any stream capture.
 *   - All calls on a GPU share the one array and it keeps the previous call's bytes.  Each call
 *     rewrites every byte it later reads, so stale contents are harmless, but two calls whose
 *     kernels overlap on the GPU (different contexts/streams on one device) race on it.
 */
int b200_conv2d_f16_noalloc(b200_ctx* ctx, int64_t W, int64_t H, int64_t Cin, int64_t N, int64_t KW,
                            int64_t KH, int64_t Cout, int64_t sx, int64_t sy, int64_t px, int64_t py,
                            int64_t dx, int64_t dy, const void* x, const void* w, const void* bias,
                            void* out, int out_dtype, int epilogue);

/* ------------------------------------------- encoder glue ops (bandwidth-bound) */
/* add.Tensor, clamp.default, gelu.default on fp16 (ops.jl:186-197,323-335,1698-1702). */
int b200_add_f16(b200_ctx* ctx, const void* a, const void* b, void* out, int64_t n);
int b200_clamp_f16(b200_ctx* ctx, const void* a, void* out, int64_t n, float lo, float hi);
int b200_act_f16(b200_ctx* ctx, const void* a, void* out, int64_t n, int epilogue);
/* _to_copy.default between fp16 and fp32 on dense arrays (ops.jl:342-358); round to nearest even
 * on the way down, exact on the way up; equal dtypes are a device copy. */
int b200_cast(b200_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n);
/* max_pool2d_with_indices.default, values only (ops.jl:1329-1343, kernels/resample.jl:121-141):
 * out[ox,oy,c,n] = max of x over the kx*ky window at (ox*sx-px, oy*sy-py), positions outside the
 * image skipped.  x is (W,H,C,N) and out (OW,OH,C,N), OW = (W+2px-kx)/sx+1, each indexed through
 * element strides {x, y, c, n}: {1,W,W*H,W*H*C} is the reference's planar layout, {C,C*W,1,C*W*H} a
 * channels-last token array (eight channels per thread when that axis is contiguous in both). */
int b200_maxpool2d_f16(b200_ctx* ctx, int64_t W, int64_t H, int64_t C, int64_t N, const void* x,
                       const int64_t* xstride, void* out, const int64_t* ostride, int64_t kx, int64_t ky,
                       int64_t sx, int64_t sy, int64_t px, int64_t py);
/* permutedims!/contiguous of a 4-D array (execute.jl:257-277): out dense with shape
 * shape[0..3] (fastest first), element (i0,i1,i2,i3) read from
 * src[i0*s[0]+i1*s[1]+i2*s[2]+i3*s[3]]; elsize 2 or 4 bytes. */
int b200_permute4(b200_ctx* ctx, const void* src, void* out, const int64_t* shape,
                  const int64_t* stride, int elsize);

/* ---------------------------------------------------------------- sharding layer */
/*
 * New surface (no reference counterpart): independent units (images, sequences, GEMM
 * rows) are split into contiguous ranges, rank r of world gets [begin,end), with split
 * points rounded to a multiple of align so a GEMM shard starts on a tile boundary.
 */
int b200_shard_range(int64_t total, int world, int rank, int64_t align, int64_t* begin,
                     int64_t* end);

#ifdef __cplusplus
}
#endif
#endif /* B200DNN_H */
