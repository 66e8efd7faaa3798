"""quadbit_b200: the two-level NVFP4 GEMM path (2:4-sparse and dense) of quadbit for
B200 (sm_100a) — hand-written tcgen05 / TMA kernels behind the reference's module API
and ctypes C-ABI."""
from ._lib import EXPORTED, QuadbitError, load  # noqa: F401
from .linear import DenseNVLinear, QBSparse, QuadbitLinear, quantize_act  # noqa: F401
from .mlp import FusedSparseMLP, register_fused_mlp_op  # noqa: F401,E402
from .moe import SparseMoE, load_sparse_moe  # noqa: F401,E402
from . import vllm_hook  # noqa: F401,E402
from .llama import LlamaConfig, LlamaPrefill  # noqa: F401,E402
from .tp import PeerBuffer, TPContext  # noqa: F401,E402
