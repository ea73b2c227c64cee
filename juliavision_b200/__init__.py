"""juliavision_b200 — the B200 (sm_100a) dense hot path of DNNKernels behind its own op API.

Host-side mirror of the reference's kernel entry points (`matmul!`, `batchedmatmul!`, `sdpa`,
`sdpa!`, `layernorm!`, `convolution!`, `scratch!`, `caps`, `toback`) over the C ABI of
libb200dnn.so.  Importing the package does not need a GPU; creating a `Ctx` does, and there
is no fallback if the library is missing.
"""
from ._lib import B200Error, SO_PATH, lib
from .attention import sdpa, sdpa_, sdpaplan
from .context import Ctx, DeviceArray, DeviceCaps, Workspace, caps
from .conv import convolution_, convolutiontranspose_, convsize, convtransposesize, onebyone, shufflecase
from .elementwise import act_, add_, clamp_, maxpool2d_, to_copy_
from .execute import Diagnostics, Model, execute_, foldgelu, foldincasts, foldoutcasts, hoistpermutes
from .graph import Buffer, Graph, Op, evalshape, loadgraph
from .kernelplans import AttnScalarPlan, Decline, FlashTCPlan, MMGemvPlan, MMScalarPlan, MMTilePlan, TwoGemmPlan
from .layernorm import add_layernorm_, layernorm_, native_layer_norm
from .matmul import batchedmatmul_, matmul_, mmplan
from .rewrites import foldbatchnorm, foldrelu, hoistcasts, weightsource
from .safetensors import readsafetensors, safetensorsnames
from .plan import Slab, alignup, checkslab, lifetimes, place, planslab
from .shard import gather_shards, shard_range, shard_range_py
from .streaming import Event, StreamedPass

__all__ = [
    "B200Error", "SO_PATH", "lib", "sdpa", "sdpa_", "sdpaplan", "Ctx", "DeviceArray", "DeviceCaps", "Workspace",
    "caps", "convolution_", "convsize", "onebyone", "act_", "add_", "clamp_", "AttnScalarPlan", "Decline",
    "FlashTCPlan", "MMScalarPlan", "MMTilePlan", "layernorm_", "add_layernorm_", "native_layer_norm", "batchedmatmul_", "matmul_",
    "mmplan", "Model", "execute_", "hoistpermutes", "foldgelu", "Buffer", "Graph", "Op", "evalshape", "loadgraph",
    "Slab", "alignup", "checkslab", "lifetimes", "place", "planslab", "shard_range", "shard_range_py", "gather_shards",
    "maxpool2d_", "to_copy_", "MMGemvPlan", "foldoutcasts", "foldincasts", "foldbatchnorm", "foldrelu", "hoistcasts", "weightsource", "readsafetensors", "safetensorsnames",
    "Event", "StreamedPass", "Diagnostics", "TwoGemmPlan", "convolutiontranspose_", "convtransposesize", "shufflecase",
]
