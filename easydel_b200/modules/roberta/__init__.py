from .modeling_roberta import (RobertaConfig, RobertaForMaskedLM, RobertaForSequenceClassification,  # noqa: F401
                               RobertaForTokenClassification, RobertaModel)

__all__ = ["RobertaConfig", "RobertaModel", "RobertaForMaskedLM", "RobertaForSequenceClassification",
           "RobertaForTokenClassification"]
