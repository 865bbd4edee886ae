"""Token mixers that carry a fixed-size state per sequence (recurrent memories, short convolutions) instead of, or beside, a paged cache.
The reference engine has no such interface (its models are attention-only); it sits beside `DSSelfAttentionBase`."""
from typing import Any, Dict, List, Type

import torch

from ..ds_module import DSModuleBase, DSModuleConfig
from ..module_registry import DSModuleRegistryBase


class DSRecurrentMixerBase(DSModuleBase):
    """Consumes the fused projections of a ragged batch, advances every sequence's state by its new tokens (prompt portions and single
    decode tokens alike) and writes the mixer's output before the output projection."""

    @staticmethod
    def config_class() -> Type[DSModuleConfig]:
        return DSModuleConfig

    def __init__(self, config: DSModuleConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)

    def state_specs(self, prefix: str) -> List:
        """`StateBufferSpec`s of what one sequence carries between steps, named `<prefix>.<buffer>`."""
        raise NotImplementedError()

    def forward(self, *args, **kwargs) -> torch.Tensor:
        raise NotImplementedError()


class DSRecurrentRegistry(DSModuleRegistryBase):
    registry: Dict = {}

    @staticmethod
    def associated_class() -> Type[DSModuleBase]:
        return DSRecurrentMixerBase
