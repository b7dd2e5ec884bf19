from .channel_delta import DSChannelDeltaRule
from .matrix_memory import DSMatrixMemory
from .tied_gate_linear import DSTiedGateLinearAttention
