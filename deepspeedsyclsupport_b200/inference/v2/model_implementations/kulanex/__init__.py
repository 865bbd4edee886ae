from .container import KulanexDeltaContainer, KulanexNonTransformerContainer, KulanexParallelContainer
from .model import KulanexInferenceModel, KulanexSpec
from .policy import KulanexPolicy
