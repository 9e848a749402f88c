"""arcq_vit_b200: B200 (sm_100a) back end for the ARCQ packed inference path.

The directory name carries a hyphen; import it through ``__graft_entry__.import_package()``
(or any ``importlib`` loader that registers it as ``arcq_vit_b200``).
"""
from . import _cabi, codebook, ops, packing, sharding, staging  # noqa: F401
from .staging import WeightStager, attach_weight_stager  # noqa: F401
from .convert import (convert_arcq_linear_to_packed, count_packed_linear, load_packed_state_dict,  # noqa: F401
                      to_on_the_fly)
from .packed_linear import ARCQPackedLinear, ARCQPackedLinearOnTheFly, quantize_weight  # noqa: F401
from .vit import (DEIT_CONFIGS, GraphedModel, HostPipeline, VisionTransformer, create_vit, pack_linear,  # noqa: F401
                  pack_model_with_codebooks, quantise_model, quantised_linear_names)

__version__ = "0.1.0"
