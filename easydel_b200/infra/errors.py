"""Framework exceptions (names follow easydel/infra/errors.py)."""


class EasyDeLRuntimeError(RuntimeError):
    """Generic runtime failure inside the framework."""


class EasyDeLSyntaxRuntimeError(EasyDeLRuntimeError):
    """A configuration combination that can never run."""


class EasyDeLTimerError(EasyDeLRuntimeError):
    """Raised when ``training_time_limit`` elapses (the trainer saves and stops)."""


class EasyDeLBreakRequest(EasyDeLRuntimeError):
    """Cooperative request to stop the training loop and return the partial output."""


class EasyDeLPreemptionSignal(EasyDeLRuntimeError):
    """Raised after a coordinated checkpoint when the job has been told to vacate."""


class EasyDeLBlockWiseFFNError(EasyDeLRuntimeError):
    """Block-wise FFN chunk size does not divide the sequence."""


class EasyDeLNotImplementedFeatureError(NotImplementedError):
    """A feature of the reference that this build states it does not provide."""
