from .modeling_mistral3 import (Mistral3Config, Mistral3ForConditionalGeneration, Mistral3MultiModalProjector,
                                Mistral3PatchMerger)

__all__ = ["Mistral3Config", "Mistral3ForConditionalGeneration", "Mistral3MultiModalProjector", "Mistral3PatchMerger"]
