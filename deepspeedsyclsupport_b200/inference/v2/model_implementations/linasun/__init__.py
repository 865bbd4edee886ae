from .container import LinasunNonTransformerContainer, LinasunTransformerContainer
from .model import LinasunInferenceModel, LinasunSpec
from .policy import LinasunPolicy
