"""``eLargeModel``: one declarative config that drives model loading, training, evaluation and serving
(easydel/infra/elarge/model.py:136-2392, builders.py, types/*, scripts/elarge.py)."""

from .model import DEFAULTS, eLargeModel, normalize_config, validate_config  # noqa: F401
