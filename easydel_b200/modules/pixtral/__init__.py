from .modeling_pixtral import PixtralTransformer, PixtralVisionConfig, PixtralVisionModel, grid_rotary

__all__ = ["PixtralTransformer", "PixtralVisionConfig", "PixtralVisionModel", "grid_rotary"]
