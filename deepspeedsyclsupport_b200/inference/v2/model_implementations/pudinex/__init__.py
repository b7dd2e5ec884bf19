from .container import PudinexAttentionContainer, PudinexNonTransformerContainer, PudinexTiedGateContainer
from .model import PudinexInferenceModel, PudinexSpec
from .policy import PudinexPolicy
