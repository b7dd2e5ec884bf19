"""Policy of the Midulorn family: config.json with "architecture": "Midulorn"; layer tensors live under `l<i>.`."""
import re

from ..inference_policy_base import ContainerMap, InferenceV2Policy
from .model import MidulornInferenceModel, MidulornSpec


class _MidulornMap(ContainerMap):
    """Layer tensors are named `l<i>.<rest>` (no dot between the prefix and the index)."""

    def set_transformer_params(self, prefixes, containers) -> None:
        self._prefix, self._transformer = "l", containers
        self._rx = re.compile(r"^l(\d+)\.(.*)$")


class MidulornPolicy(InferenceV2Policy):
    model_types = ("midulorn", )

    def spec(self) -> MidulornSpec:
        return MidulornSpec.from_config(self._model_config)

    def instantiate_model(self, engine_config, mp_group, device=None):
        return MidulornInferenceModel(self.spec(), tp_group=mp_group, dtype=self._dtype, device=device, engine_config=engine_config)

    def build_container_map(self) -> ContainerMap:
        cmap = _MidulornMap()
        cmap.set_transformer_params("l", self.model.layers)
        cmap.set_non_transformer_params(self.model.non_transformer)
        return cmap

    def finish_loading(self, cmap: ContainerMap) -> None:
        self.model.check_populated()
