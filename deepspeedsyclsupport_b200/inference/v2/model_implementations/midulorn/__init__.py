from .model import MidulornInferenceModel, MidulornSpec  # noqa: F401
from .policy import MidulornPolicy  # noqa: F401
