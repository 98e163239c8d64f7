"""Architecture descriptions.  Importing the package registers them."""
from ..config.boketar import BoketarConfig
from ..config.falcon_h1 import FalconH1Config
from ..config.gikovik import GikovikConfig
from ..config.registry import register_architecture
from ..config.sorovik import SorovikConfig
from ..config.tafesun import TafesunConfig
from . import boketar, falcon_h1, gikovik, sorovik, tafesun

register_architecture("falcon_h1", FalconH1Config.from_dict, falcon_h1.model_spec,
                      aliases=("FalconH1ForCausalLM",))
register_architecture("Boketar", BoketarConfig.from_dict, boketar.model_spec, aliases=("boketar",),
                      reads_tensor_shapes=True)
register_architecture("Tafesun", TafesunConfig.from_dict, tafesun.model_spec, aliases=("tafesun",))
register_architecture("Gikovik", GikovikConfig.from_dict, gikovik.model_spec, aliases=("gikovik",))
register_architecture("Sorovik", SorovikConfig.from_dict, sorovik.model_spec, aliases=("sorovik",))
