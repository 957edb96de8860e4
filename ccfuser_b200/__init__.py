"""B200-native fused expert-parallel MoE layer library."""
from .config import MoEConfig
from .errors import MoECommError, MoECommTimeout, MoEOverflow
from .experts import Experts, ExpertLinear, scan_expert_params
from .gates import BaseGate, NaiveGate, zipf_router_bias
from .layers import MoELayer, MixMOE, MixMOETransformerMLP

from .parallel.placement import placement_cost, plan_placement, rebalance_experts
from .utils.checkpoint import (ep_state_dict, import_reference_state, load_ep_checkpoint, reshard_expert_state,
                               save_ep_checkpoint)

__version__ = "0.1.0"
__all__ = ["MoEConfig", "MoELayer", "MixMOE", "MixMOETransformerMLP", "NaiveGate", "BaseGate", "Experts",
           "ExpertLinear", "scan_expert_params", "zipf_router_bias", "MoECommError", "MoECommTimeout",
           "MoEOverflow", "ep_state_dict", "save_ep_checkpoint", "load_ep_checkpoint", "reshard_expert_state",
           "import_reference_state", "plan_placement", "placement_cost", "rebalance_experts"]
