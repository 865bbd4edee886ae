from .channel_delta import DSChannelDeltaRule
from .matrix_memory import DSMatrixMemory
