"""Model blocks built on the fused kernels: the Llama tensor-parallel MLP and the Mixtral expert-parallel MoE."""
from .llama import LlamaMLP, LlamaMLPModule, reference_mlp  # noqa: F401
from .mixtral import MixtralMoEBlock, MixtralMoEModule  # noqa: F401
