"""Error kinds of the engine, one class per kind of the reference's error enum
(src/error.rs:8-46).  Every error that leaves the package is one of these."""


class EngineError(Exception):
    """Base class."""


class ConfigError(EngineError):
    """config.json or an engine option is missing, malformed or out of range."""


class Unsupported(EngineError):
    """The configuration is well-formed but names something not implemented."""


class WeightError(EngineError):
    """A weight file is malformed, or tensors are missing, unexpected or misshaped."""


class ShapeError(EngineError):
    """An operator was given sizes it does not take."""


class ResourceExhausted(EngineError):
    """Queue full or cache pages exhausted for good."""


class Unavailable(EngineError):
    """The engine (or its compiled extension) is not usable."""


class StepFailed(EngineError):
    """A step ran and its result cannot be trusted: an activation or a logit was not finite, a token
    id fell outside the table, or a kernel gave up on a bounded wait.  Nothing of the step was
    committed (src/model/native.rs:272-306)."""

    def __init__(self, message: str, words=()):
        super().__init__(message)
        self.words = tuple(words)
