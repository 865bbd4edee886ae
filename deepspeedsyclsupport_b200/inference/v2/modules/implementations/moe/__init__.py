from .cutlass_multi_gemm import DSMultiGemmMoE
from .grouped_topk_moe import DSGroupedTopKMoE
