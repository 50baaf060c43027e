from .modeling_rwkv import RwkvConfig, RwkvForCausalLM, RwkvModel, RwkvState

__all__ = ["RwkvConfig", "RwkvForCausalLM", "RwkvModel", "RwkvState"]
