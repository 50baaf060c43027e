from .esurge_eval import eSurgeLMEvalAdapter, run_lm_eval  # noqa: F401
