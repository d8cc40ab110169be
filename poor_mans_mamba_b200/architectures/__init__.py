"""Architecture descriptions.  Importing the package registers them."""
from ..config.falcon_h1 import FalconH1Config
from ..config.registry import register_architecture
from . import falcon_h1

register_architecture("falcon_h1", FalconH1Config.from_dict, falcon_h1.model_spec,
                      aliases=("FalconH1ForCausalLM",))
