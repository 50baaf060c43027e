from .modeling_mamba import (FalconMambaConfig, FalconMambaForCausalLM, FalconMambaModel, Mamba2Cache, Mamba2Config,  # noqa: F401
                             Mamba2ForCausalLM, Mamba2Model, MambaCache, MambaConfig, MambaForCausalLM, MambaModel)

__all__ = ["MambaConfig", "MambaModel", "MambaForCausalLM", "FalconMambaConfig", "FalconMambaModel",
           "FalconMambaForCausalLM", "MambaCache", "Mamba2Config", "Mamba2Model", "Mamba2ForCausalLM", "Mamba2Cache"]
