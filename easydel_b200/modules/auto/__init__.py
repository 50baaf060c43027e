from .auto_modeling import *  # noqa: F401,F403
from .auto_modeling import resolve_model_class  # noqa: F401
