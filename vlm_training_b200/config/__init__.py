from .schema import Config, DataSection, ModelSection, ModelType, TrainingSection, WandbSection
from .manager import ConfigManager, to_flat_dict

__all__ = ["Config", "ConfigManager", "DataSection", "ModelSection", "ModelType",
           "TrainingSection", "WandbSection", "to_flat_dict"]
