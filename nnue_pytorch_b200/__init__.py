"""nnue_pytorch_b200: sm_100a kernels for the sparse feature-transformer hot
path of nnue-pytorch, behind the reference's own operator interface."""

from .composed_feature_transformer import ComposedFeatureTransformer
from .double_ft_functions import double_feature_transform
from .fused_ft_functions import FusedDoubleFtFunction
from .sparse_linear_functions import SparseLinearFunction

__all__ = [
    "ComposedFeatureTransformer",
    "FusedDoubleFtFunction",
    "SparseLinearFunction",
    "double_feature_transform",
]
