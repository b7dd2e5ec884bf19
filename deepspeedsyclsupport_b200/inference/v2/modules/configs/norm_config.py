"""Configuration of the pre- / post-norm modules (parity: inference/v2/modules/configs/norm_config.py:12-32)."""
from pydantic import field_validator

from ...inference_utils import DtypeEnum, NormTypeEnum
from ..ds_module import DSModuleConfig


class DSNormConfig(DSModuleConfig):
    """One config serves DSPreNormBase and DSPostNormBase.  `residual_dtype` is the dtype of the residual stream the norm adds into,
    `input_dtype` that of the incoming hidden states, `output_dtype` that of the normalised result."""
    type: NormTypeEnum  # layer_norm | rms_norm
    channels: int  # width of the normalised (last) dimension
    eps: float = 1e-5
    residual_dtype: DtypeEnum = DtypeEnum.fp16
    input_dtype: DtypeEnum = DtypeEnum.fp16
    output_dtype: DtypeEnum = DtypeEnum.fp16
    # norms whose weight is zero-centred multiply by (weight + weight_offset)
    weight_offset: float = 0.0
    # "sandwich" blocks norm a sublayer's output before it is added to the residual: x += norm(branch) * (w_b + offset), and the
    # same pass produces the next sublayer's input norm(x) * (w + offset).  The residual stream is then kept in fp32.
    sandwich: bool = False
    # sandwich blocks only: the normed branch is multiplied by this before it joins the stream (x += branch_mult * norm(branch) * ...)
    branch_mult: float = 1.0
    # "shared input" blocks: ONE norm per layer whose output every sublayer of the layer reads; the sublayers' outputs join the fp32 stream as
    # a plain sum in the pass that forms the next layer's norm.  The row is normed in `groups` equal consecutive parts, each divided by its
    # own root mean square, before the weight is applied.
    shared_input: bool = False
    groups: int = 1
    # "post sum" blocks: the norm sits BEHIND the residual sum and its result IS the new stream: x <- norm(stream_mult * x + sublayer(x)) * w.
    # The sublayers read the stream itself; the stream is kept in fp32 and handed on in the activation dtype as well.
    post_sum: bool = False
    stream_mult: float = 1.0

    @field_validator("channels")
    @classmethod
    def _positive_width(cls, v):
        if v <= 0:
            raise ValueError(f"channels must be positive, got {v}")
        return v

    @field_validator("eps")
    @classmethod
    def _positive_eps(cls, v):
        if not v > 0:
            raise ValueError(f"eps must be positive, got {v}")
        return v

    @property
    def is_rms(self) -> bool:
        return NormTypeEnum(self.type) == NormTypeEnum.RMSNorm
