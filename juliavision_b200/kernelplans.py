"""Plan objects: one decision per call, made before the output is allocated, so that holding
a plan means the kernel runs (the rule of the reference's kernelplans.jl:1-35 and
flash.jl:1428-1432).  A refusal is a `Decline(reason)` with the reference's vocabulary.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Decline:
    """Structured refusal (kernelplans.jl:21-35). reason is one of :operands, :extent, :wrapped,
    :bias, :eltype, :tiling, :notvector."""
    reason: str


@dataclass(frozen=True)
class MMTilePlan:
    """Tensor-core GEMM plan; stands where MMCoopMatPlan(NP, tile) stood (kernelplans.jl:382-385).
    No padded extent: ragged M/N/K are covered by TMA-clipped tiles."""
    block_m: int
    block_n: int
    block_k: int
    stages: int
    tiles_m: int
    tiles_n: int
    ctas: int
    smem_bytes: int


@dataclass(frozen=True)
class MMScalarPlan:
    """fp16 operands a tensor map cannot express (unaligned leading dimension or pointer): the
    one-thread-per-output kernel with mm2's arithmetic (matmul.jl:17-28), still on the GPU."""
    reason: str


@dataclass(frozen=True)
class MMGemvPlan:
    """One column of B — "batch 1" in the reversed layout (mm_gemv_plan, matmul.jl:103-130): the
    bandwidth-bound matrix-vector kernel.  The reference takes it for fp32 operands only; here fp16
    operands take it too, since a 128-token tile would be almost empty."""


@dataclass(frozen=True)
class FlashTCPlan:
    """Fused single-pass attention on tcgen05; stands where FlashCMPlan stood
    (kernelplans.jl:54-324). BR/BC are the query/key block, EP the padded head dim (64 for E <= 64: two
    query tiles per CTA; 128 for 64 < E <= 128, which covers the reference's own E = 72: one tile per
    CTA, every operand two swizzle atoms along E).  Holding this
    plan means the call runs; inside it the library still chooses how: whole query-tile pairs, a key
    split with a merge for few queries over many keys, and for many windows of at most 64 keys a
    small-tile kernel (64 queries of one window and head per CTA) instead of the 128-row tiles."""
    BR: int = 128
    BC: int = 128
    EP: int = 64
    nsplit: int = 1


@dataclass(frozen=True)
class TwoGemmPlan:
    """Attention as two batched tensor-core GEMMs with a row softmax between them; stands where
    CoopMatSDPAPlan(chunk, EP, nbatch) stood (sdpa_coopmat!, attention.jl:585-705): head dims the fused
    kernel's tensor memory cannot hold (E > 128).  Only K is copied (transposed); scores in fp32."""
    nbatch: int = 1


@dataclass(frozen=True)
class AttnScalarPlan:
    """Fused attention for head dims / strides the tensor-core kernel declines."""
    reason: str
