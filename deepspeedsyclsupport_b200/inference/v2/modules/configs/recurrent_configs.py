"""Configuration of the recurrent token mixers: layers that carry a fixed-size state per sequence instead of a growing cache."""
from ...inference_utils import DtypeEnum
from ..ds_module import DSModuleConfig


class DSMatrixMemoryConfig(DSModuleConfig):
    """Matrix memory with exponential gating per head: S <- a S + b k v^T, n <- a n + b k with a log-space input gate i and forget gate f
    (both soft-capped: cap tanh(. / cap), f through logsigmoid) stabilised by a running maximum m that starts at 0; read-out
    S^T q / (max(|n . q|, exp(-m)) + 1e-6), q scaled by key_size^-1/2; then a per-head RMS norm, a weight and a sigmoid output gate."""
    n_heads: int
    key_size: int
    value_size: int
    gate_cap: float
    eps: float = 1e-6  # of the per-head norm of the read-out
    out_scale: float = 1.0  # the result is multiplied by this before it is rounded (mixers that are summed with weights)
    max_sequences: int
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16


class DSDeltaRuleConfig(DSModuleConfig):
    """Gated delta rule with one decay per head and key channel: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    q, k, v pass a short causal convolution and silu; q and k are unit vectors per head (q also times key_size^-1/2);
    g = exp(-exp(A_log) softplus(a + dt_bias)); the read-out gets a per-head RMS norm with a weight shared by the heads and a sigmoid gate."""
    n_heads: int
    n_heads_qk: int  # query / key heads; value head h reads q / k head h // (n_heads / n_heads_qk)
    key_size: int
    value_size: int
    conv_taps: int
    eps: float = 1e-6
    out_scale: float = 1.0
    max_sequences: int
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16


class DSTiedGateConfig(DSModuleConfig):
    """Linear attention whose forget gate also decides what is written (there is no key projection): per head, q = silu(W_q h),
    f = lower + (1 - lower) sigmoid(W_f h + b) per key channel, S <- diag(f) S + (1 - f) v^T, o = S^T q; the read-out gets a per-head RMS norm
    with a weight shared by the heads (no output gate)."""
    n_heads: int
    key_size: int
    value_size: int
    eps: float = 1e-6
    out_scale: float = 1.0
    max_sequences: int
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16


class DSMinGRUConfig(DSModuleConfig):
    """Minimal gated recurrence with one number of state per channel; the gates read only the current token: z = sigmoid(W_z h + b_z),
    u = W_x h + b_x, candidate c = u + 1/2 where u >= 0 and sigmoid(u) below, S <- (1 - z) S + z c, output S silu(W_g h) (before the output
    projection).  The state is fp32 and starts at zero."""
    width: int
    max_sequences: int
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16
