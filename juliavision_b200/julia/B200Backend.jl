# B200Backend.jl — the reference-side binding of libb200dnn.so.
#
# Drop this file into DNNKernels/src and `include("B200Backend.jl")` after kernelplans.jl.
# It adds a backend, a device array, the caps answer, new plan types and one method per
# entry point (`matmul!`, `sdpa!`, `layernorm!`, `convolution!`, `scratch!`, `toback`), which is
# the extension rule the package states: a new path is a new plan type plus a new method
# (kernels/extern/matmul.jl:97-100, kernels/extern/attention.jl:767-771, kernelplans.jl:1-19).
# Nothing else in the package changes: `execute!`, the rewrite passes, `planslab` and `dest`
# keep working because `B200Array` is a dense column-major array like `LavaArray`.
#
# No Julia toolchain exists where this file was written, so it has not been executed; the
# identical call sequence is exercised through the same C symbols by the Python mirror in
# juliavision_b200/*.py and its tests.

module B200

using ..DNNKernels: Ctx, Decline, MMGemvPlan, accum, actfn, geluexact, gelutanh, relu_epi
import ..DNNKernels: matmul!, mmplan, mm_gemv_plan, batchedmatmul!, sdpa!, sdpaplan, layernorm!, convolution!,
                     maxpool2d!, scratch!, toback, caps, slabview
import KernelAbstractions

const LIB = get(ENV, "B200DNN_LIB", "libb200dnn.so")

# ------------------------------------------------------------------ status handling
const OK = Cint(0)
const DECLINE = Dict(16 => :operands, 17 => :extent, 18 => :wrapped, 19 => :bias, 20 => :eltype, 21 => :tiling)
lasterror() = unsafe_string(ccall((:b200_last_error, LIB), Cstring, ()))
check(rc::Cint) = rc == OK ? nothing : error("b200dnn status $rc: $(lasterror())")

# ------------------------------------------------------------------ backend / arrays
mutable struct B200Backend <: KernelAbstractions.GPU
    handle::Ptr{Cvoid}
    device::Int
    function B200Backend(device::Integer = 0)
        h = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall((:b200_ctx_create, LIB), Cint, (Cint, Ref{Ptr{Cvoid}}), device, h))
        b = new(h[], device)
        finalizer(x -> ccall((:b200_ctx_destroy, LIB), Cint, (Ptr{Cvoid},), x.handle), b)
    end
end

"""Dense column-major device array; `parent` keeps the pool block or slab alive."""
struct B200Array{T,N} <: DenseArray{T,N}
    ptr::Ptr{T}
    dims::NTuple{N,Int}
    backend::B200Backend
    parent::Any
end
Base.size(a::B200Array) = a.dims
Base.pointer(a::B200Array) = a.ptr
Base.strides(a::B200Array) = Base.size_to_strides(1, a.dims...)
KernelAbstractions.get_backend(a::B200Array) = a.backend
KernelAbstractions.synchronize(b::B200Backend) = check(ccall((:b200_sync, LIB), Cint, (Ptr{Cvoid},), b.handle))

mutable struct PoolBlock
    backend::B200Backend
    ptr::Ptr{Cvoid}
end
function KernelAbstractions.allocate(b::B200Backend, ::Type{T}, dims::Integer...) where {T}
    p = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:b200_pool_alloc, LIB), Cint, (Ptr{Cvoid}, Csize_t, Ref{Ptr{Cvoid}}), b.handle,
                max(prod(dims), 1) * sizeof(T), p))
    blk = PoolBlock(b, p[])
    finalizer(x -> ccall((:b200_pool_free, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}), x.backend.handle, x.ptr), blk)
    B200Array{T,length(dims)}(Ptr{T}(p[]), Int.(dims), b, blk)
end

"""`toback(backend, a)` (driver.jl:108-115): upload a host array."""
function toback(b::B200Backend, a::AbstractArray{T}) where {T}
    h = Array(a)
    d = KernelAbstractions.allocate(b, T, size(h)...)
    check(ccall((:b200_upload, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Csize_t), b.handle, d.ptr, h,
                sizeof(h)))
    d
end
function Base.Array(a::B200Array{T,N}) where {T,N}
    h = Array{T,N}(undef, a.dims)
    check(ccall((:b200_download, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Csize_t), a.backend.handle, h,
                a.ptr, sizeof(h)))
    h
end

"""`slabview(T, slab, dims, off)` (execute.jl:173-179): a typed view at a byte offset of a slab."""
slabview(::Type{T}, slab::B200Array{UInt8,1}, dims, off::Integer) where {T} =
    B200Array{T,length(dims)}(Ptr{T}(slab.ptr + off), Int.(Tuple(dims)), slab.backend, slab)

"""`scratch!(ws, backend, T, dims...)` (workspace.jl:63-96) served by the library's bump workspace."""
function scratch!(::Any, b::B200Backend, ::Type{T}, dims::Integer...) where {T}
    p = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:b200_workspace_scratch, LIB), Cint, (Ptr{Cvoid}, Csize_t, Ref{Ptr{Cvoid}}), b.handle,
                prod(dims) * sizeof(T), p))
    B200Array{T,length(dims)}(Ptr{T}(p[]), Int.(dims), b, nothing)
end
resetworkspace!(b::B200Backend) = check(ccall((:b200_workspace_reset, LIB), Cint, (Ptr{Cvoid},), b.handle))

# ------------------------------------------------------------------ caps (context.jl:55-68)
struct CapsC
    coopmat::Int32; tile::Int32; subgroup::Int32; coopmatsubgroup::Int32; sharedbudget::Int32
    workgrouplimit::Int32; cores::Int32; warps::Int32; cc_major::Int32; cc_minor::Int32; total_mem::Int64
end
struct B200Caps
    coopmat::Bool; tile::Int; subgroup::Int; coopmatsubgroup::Int; sharedbudget::Int
    workgrouplimit::Int; cores::Int; warps::Int
end
function caps(b::B200Backend)
    c = Ref{CapsC}()
    check(ccall((:b200_caps, LIB), Cint, (Ptr{Cvoid}, Ref{CapsC}), b.handle, c))
    B200Caps(c[].coopmat != 0, c[].tile, c[].subgroup, c[].coopmatsubgroup, c[].sharedbudget,
             c[].workgrouplimit, c[].cores, c[].warps)
end

# ------------------------------------------------------------------ plans
"""Tensor-core GEMM plan; no padded extent — ragged M/N/K are TMA-clipped tiles."""
struct MMTilePlan end
"""fp16 operands a tensor map cannot express: the scalar kernel (mm2's arithmetic) on the GPU."""
struct MMScalarPlan end
"""Fused single-pass attention on tcgen05."""
struct FlashTCPlan end
struct AttnScalarPlan end
struct TwoGemmPlan end     # head dims above 128 (multiples of 8): the two-GEMM route inside the library

dtcode(::Type{Float16}) = Cint(0)
dtcode(::Type{Float32}) = Cint(1)
epicode(epi) = epi === geluexact ? Cint(2) : epi === relu_epi ? Cint(1) : epi === gelutanh ? Cint(3) :
               epi === identity ? Cint(0) : error("no fused form for epilogue $epi")

"""Root pointer + strides of a wrapper stack over a B200Array (the job of `stridedroot`,
attention.jl:321-337): `nothing` when the stack is not a strided view."""
function rootstrides(a)
    a isa B200Array && return (pointer(a), strides(a))
    try
        return (pointer(a), strides(a))     # SubArray / PermutedDimsArray / ReshapedArray of dense parents
    catch
        return nothing
    end
end

# ------------------------------------------------------------------ matmul! (matmul.jl:78-100)
function mmplan(dev::B200Caps, out, A, B, bias)
    if size(B, 2) == 1                       # one token: the matrix-vector kernel (fp32 as in the reference, or fp16)
        g = mm_gemv_plan(dev, out, A, B, bias)
        g isa MMGemvPlan && return g
    end
    eltype(A) === Float16 && eltype(B) === Float16 || return Decline(:operands)
    eltype(out) in (Float16, Float32) || return Decline(:eltype)
    ra, rb, ro = rootstrides(A), rootstrides(B), rootstrides(out)
    (ra === nothing || rb === nothing || ro === nothing) && return Decline(:wrapped)
    (ra[2][1] == 1 && rb[2][1] == 1 && ro[2][1] == 1) || return Decline(:wrapped)
    M, K = size(A); N = size(B, 2)
    rc = ccall((:b200_gemm_f16_supported, LIB), Cint, (Int64, Int64, Int64, Int64, Int64, Int64, Cint),
               M, N, K, ra[2][2], rb[2][2], ro[2][2], dtcode(eltype(out)))
    rc == OK && return MMTilePlan()
    rc == 18 && return MMScalarPlan()
    Decline(get(DECLINE, Int(rc), :extent))
end

function matmul!(ctx, ::Union{MMTilePlan,MMScalarPlan}, out, A, B, bias, epi; gemm = NamedTuple())
    M, K = size(A); N = size(B, 2)
    check(ccall((:b200_gemm_f16, LIB), Cint,
                (Ptr{Cvoid}, Int64, Int64, Int64, Ptr{Cvoid}, Int64, Ptr{Cvoid}, Int64, Ptr{Cvoid}, Ptr{Cvoid},
                 Int64, Cint, Cint, Int64, Int64, Int64, Int64),
                ctx.backend.handle, M, N, K, pointer(A), stride(A, 2), pointer(B), stride(B, 2),
                bias === nothing ? C_NULL : pointer(bias), pointer(out), stride(out, 2), dtcode(eltype(out)),
                epicode(epi), 1, 0, 0, 0))
    out
end
# No CPU path behind this backend: a refusal is an error, not a slower route.
matmul!(ctx::Ctx{B200Backend}, d::Decline, out, A, B, bias, epi; gemm = NamedTuple()) =
    error("matmul!: Decline(:$(d.reason)) on the B200 backend")

function batchedmatmul!(ctx::Ctx{B200Backend}, out, A, B)
    M, K, nb = size(A); N = size(B, 2)
    check(ccall((:b200_gemm_f16, LIB), Cint,
                (Ptr{Cvoid}, Int64, Int64, Int64, Ptr{Cvoid}, Int64, Ptr{Cvoid}, Int64, Ptr{Cvoid}, Ptr{Cvoid},
                 Int64, Cint, Cint, Int64, Int64, Int64, Int64),
                ctx.backend.handle, M, N, K, pointer(A), stride(A, 2), pointer(B), stride(B, 2), C_NULL,
                pointer(out), stride(out, 2), dtcode(eltype(out)), 0, nb, stride(A, 3), stride(B, 3),
                stride(out, 3)))
    out
end

# ------------------------------------------------------------------ sdpa! (attention.jl:712-834)
struct Strided4
    ptr::Ptr{Cvoid}
    stride::NTuple{4,Int64}
end
s4(a) = (r = rootstrides(a); Strided4(Ptr{Cvoid}(r[1]), Int64.(r[2])))

# An additive mask does not decline here: the fused kernel adds it (b200_attention_f16_bias).  It must
# be Float16 and broadcast to (Lk, Lq, H, B), the graph's own order (attention.jl:55-59).
function sdpaplan(ctx::Ctx{B200Backend}, q, k, v, bias)
    if bias !== nothing
        eltype(bias) === Float16 || return (Decline(:eltype), k, v)
        all(i -> size(bias, i) in (1, (size(k, 2), size(q, 2), size(q, 3), size(q, 4))[i]), 1:4) ||
            return (Decline(:bias), k, v)
    end
    all(x -> eltype(x) === Float16, (q, k, v)) || return (Decline(:eltype), k, v)
    any(x -> rootstrides(x) === nothing, (q, k, v)) && return (Decline(:wrapped), k, v)
    E, Lq, H, B = size(q); Lk = size(k, 2)
    st(x) = collect(Int64.(rootstrides(x)[2]))
    rc = ccall((:b200_attention_f16_supported, LIB), Cint,
               (Int64, Int64, Int64, Int64, Int64, Ptr{Int64}, Ptr{Int64}, Ptr{Int64}, Cint),
               E, Lq, Lk, H, B, st(q), st(k), st(v), 0)
    rc == OK && return (FlashTCPlan(), k, v)
    if rc in (18, 21)
        # head dims above 128: S = K'Q, softmax over the keys, O = V P on the GEMM kernel (route 1), else scalar
        route = ccall((:b200_attention_f16_route, LIB), Cint,
                      (Int64, Int64, Int64, Int64, Int64, Ptr{Int64}, Ptr{Int64}, Ptr{Int64}),
                      E, Lq, Lk, H, B, st(q), st(k), st(v))
        return (route == 1 ? TwoGemmPlan() : AttnScalarPlan(), k, v)
    end
    (Decline(get(DECLINE, Int(rc), :extent)), k, v)
end

function sdpa!(ctx, ::Union{FlashTCPlan,TwoGemmPlan,AttnScalarPlan}, out, q, k, v, bias, scale)
    E, Lq, H, B = size(q); Lk = size(k, 2)
    out === nothing && (out = KernelAbstractions.allocate(ctx.backend, accum(eltype(q)), E, Lq, H, B))
    # `out` may be any (E, Lq, H, B) view with E contiguous: a token-major destination folds the
    # clone that follows sdpa in the exported graphs into the store.
    if bias === nothing
        check(ccall((:b200_attention_f16_strided, LIB), Cint,
                    (Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Ref{Strided4}, Ref{Strided4}, Ref{Strided4},
                     Ref{Strided4}, Cint, Cfloat),
                    ctx.backend.handle, E, Lq, Lk, H, B, s4(q), s4(k), s4(v), s4(out), dtcode(eltype(out)),
                    Float32(scale)))
    else
        b = s4(bias)   # a size-1 axis broadcasts: stride 0
        b = Strided4(b.ptr, ntuple(i -> size(bias, i) == 1 ? Int64(0) : b.stride[i], 4))
        check(ccall((:b200_attention_f16_bias, LIB), Cint,
                    (Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Ref{Strided4}, Ref{Strided4}, Ref{Strided4},
                     Ref{Strided4}, Ref{Strided4}, Cint, Cfloat),
                    ctx.backend.handle, E, Lq, Lk, H, B, s4(q), s4(k), s4(v), b, s4(out), dtcode(eltype(out)),
                    Float32(scale)))
    end
    out
end

# ------------------------------------------------------------------ layernorm! (layernorm.jl:125-135)
function layernorm!(ctx::Ctx{B200Backend}, out, mean, rstd, a, γ, β, C::Integer, eps::Real)
    groups = length(a) ÷ C
    check(ccall((:b200_layernorm, LIB), Cint,
                (Ptr{Cvoid}, Int64, Int64, Ptr{Cvoid}, Cint, Ptr{Cvoid}, Cint, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
                 Ptr{Cvoid}, Cfloat),
                ctx.backend.handle, groups, C, pointer(a), dtcode(eltype(a)), pointer(out), dtcode(eltype(out)),
                pointer(mean), pointer(rstd), γ === nothing ? C_NULL : pointer(γ),
                β === nothing ? C_NULL : pointer(β), Float32(eps)))
    out
end

# x .= clamp.(x .+ h); layernorm!(out, mean, rstd, x, ...) in one launch: the target of a load-time
# rewrite that folds add.Tensor (+ clamp.default) into the native_layer_norm that follows.
function addlayernorm!(ctx::Ctx{B200Backend}, out, mean, rstd, x, h, γ, β, C::Integer, eps::Real; clamp = nothing)
    lo, hi = clamp === nothing ? (0f0, 0f0) : Float32.(clamp)
    check(ccall((:b200_add_layernorm_f16, LIB), Cint,
                (Ptr{Cvoid}, Int64, Int64, Ptr{Cvoid}, Ptr{Cvoid}, Cint, Cfloat, Cfloat, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
                 Ptr{Cvoid}, Ptr{Cvoid}, Cfloat),
                ctx.backend.handle, length(x) ÷ C, C, pointer(x), pointer(h), clamp === nothing ? 0 : 1, lo, hi,
                pointer(out), pointer(mean), pointer(rstd), γ === nothing ? C_NULL : pointer(γ),
                β === nothing ? C_NULL : pointer(β), Float32(eps)))
    out
end

# ------------------------------------------------------------------ matmul!(::MMGemvPlan) (matmul.jl:103-137)
function mm_gemv_plan(dev::B200Caps, out, A, B, bias)
    T = eltype(A)
    (T === Float32 || T === Float16) && eltype(B) === T || return Decline(:operands)
    size(B, 2) == 1 || return Decline(:notvector)
    bias === nothing || (bias isa AbstractVector && length(bias) == size(A, 1)) || return Decline(:bias)
    MMGemvPlan()
end
function matmul!(ctx::Ctx{B200Backend}, ::MMGemvPlan, out, A, B, bias, epi; gemm = NamedTuple())
    M, K = size(A)
    check(ccall((:b200_gemv, LIB), Cint,
                (Ptr{Cvoid}, Int64, Int64, Ptr{Cvoid}, Int64, Ptr{Cvoid}, Ptr{Cvoid}, Cint, Ptr{Cvoid}, Cint, Cint),
                ctx.backend.handle, M, K, pointer(A), stride(A, 2), pointer(B),
                bias === nothing ? C_NULL : pointer(bias), dtcode(eltype(A)), pointer(out), dtcode(eltype(out)),
                epicode(epi)))
    out
end

# ------------------------------------------------------------------ maxpool2d!, _to_copy (resample.jl:141, ops.jl:342-358)
function maxpool2d!(ctx::Ctx{B200Backend}, out, x, k, s, p)
    xs, os = rootstrides(x), rootstrides(out)     # any (x, y, c, n) view: the NCHW permutes need no copy
    W, H, C, N = size(x)
    check(ccall((:b200_maxpool2d_f16, LIB), Cint,
                (Ptr{Cvoid}, Int64, Int64, Int64, Int64, Ptr{Cvoid}, Ptr{Int64}, Ptr{Cvoid}, Ptr{Int64}, Int64, Int64, Int64,
                 Int64, Int64, Int64),
                ctx.backend.handle, W, H, C, N, Ptr{Cvoid}(xs[1]), collect(Int64.(xs[2])), Ptr{Cvoid}(os[1]),
                collect(Int64.(os[2])), k[1], k[2], s[1], s[2], p[1], p[2]))
    out
end
function tocopy!(ctx::Ctx{B200Backend}, out, a)
    check(ccall((:b200_cast, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}, Cint, Ptr{Cvoid}, Cint, Int64),
                ctx.backend.handle, pointer(a), dtcode(eltype(a)), pointer(out), dtcode(eltype(out)), length(a)))
    out
end

# ------------------------------------------------------------------ capture / replay! (SAM2Runner/src/sam2.jl:90-115)
# Run the ops once (sizes the pool and the workspace), then record them; replay! launches the graph.
function capture(f, b::B200Backend)
    f(); KernelAbstractions.synchronize(b)
    check(ccall((:b200_graph_begin, LIB), Cint, (Ptr{Cvoid},), b.handle))
    f()
    g = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:b200_graph_end, LIB), Cint, (Ptr{Cvoid}, Ref{Ptr{Cvoid}}), b.handle, g))
    g[]
end
replay!(b::B200Backend, g::Ptr{Cvoid}) = check(ccall((:b200_graph_launch, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}), b.handle, g))

# ------------------------------------------------------------------ convolution! (conv.jl:100-145)
function convolution!(ctx::Ctx{B200Backend}, out, x, w, bias, stride, padding, dilation, groups; act = :none)
    W, H, Cin, N = size(x); KW, KH, _, Cout = size(w)
    check(ccall((:b200_conv2d_grouped_f16, LIB), Cint,
                (Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64,
                 Int64, Int64, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Cint, Cint),
                ctx.backend.handle, W, H, Cin, N, KW, KH, Cout, stride[1], stride[2], padding[1], padding[2],
                dilation[1], dilation[2], groups, pointer(x), pointer(w), bias === nothing ? C_NULL : pointer(bias),
                pointer(out), dtcode(eltype(out)), act === :relu ? 1 : act === :gelu ? 2 : 0))
    out
end

# ------------------------------------------------------------------ convolutiontranspose! (conv.jl:247-290)
# shufflecase (stride == kernel, nothing else set, one group) runs as a GEMM + depth-to-space inside the
# library; every other geometry as the deterministic gather.  w is (KW, KH, Cout ÷ groups, Cin).
function convolutiontranspose!(ctx::Ctx{B200Backend}, out, x, w, bias, stride, padding, dilation, outpad, groups)
    W, H, Cin, N = size(x); KW, KH, Cog, _ = size(w)
    check(ccall((:b200_convtranspose2d_f16, LIB), Cint,
                (Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64, Int64,
                 Int64, Int64, Int64, Int64, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Cint),
                ctx.backend.handle, W, H, Cin, N, KW, KH, Cog * groups, stride[1], stride[2], padding[1], padding[2],
                dilation[1], dilation[2], outpad[1], outpad[2], groups, pointer(x), pointer(w),
                bias === nothing ? C_NULL : pointer(bias), pointer(out), dtcode(eltype(out))))
    out
end

# ------------------------------------------------------------------ Diagnostics (context.jl:162-221)
# optimes: bracket an op with the context's event timer (milliseconds on the device).
function optime(f, b::B200Backend)
    check(ccall((:b200_timer_start, LIB), Cint, (Ptr{Cvoid},), b.handle))
    f()
    ms = Ref{Cfloat}(0)
    check(ccall((:b200_timer_stop, LIB), Cint, (Ptr{Cvoid}, Ref{Cfloat}), b.handle, ms))
    Float64(ms[])
end
launchcount(b::B200Backend) = ccall((:b200_launch_count, LIB), Int64, (Ptr{Cvoid},), b.handle)

end # module
