from .channel_delta import DSChannelDeltaRule
from .matrix_memory import DSMatrixMemory
from .min_gru import DSMinGRU
from .tied_gate_linear import DSTiedGateLinearAttention
