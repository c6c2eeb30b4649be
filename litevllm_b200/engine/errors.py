"""Error taxonomy of the runtime (reference: vllm/engine/errors.py:4-29).  The HTTP layer maps
InvalidRequestError -> 400, other RequestRejectedError -> 429, EngineFatalError -> 503."""


class LiteRuntimeError(RuntimeError):
    pass


class RequestRejectedError(LiteRuntimeError):
    """Admission refused (queue full, queue timeout, capability missing)."""

    def __init__(self, message: str, reason: str = "rejected"):
        super().__init__(message)
        self.reason = reason


class InvalidRequestError(RequestRejectedError):
    def __init__(self, message: str):
        super().__init__(message, reason="invalid")


class EngineFatalError(RequestRejectedError):
    def __init__(self, message: str):
        super().__init__(message, reason="fatal")


class RequestAbortedError(LiteRuntimeError):
    pass


class BackgroundLoopError(LiteRuntimeError):
    pass


class ExecutionStepError(LiteRuntimeError):
    pass


class RankFailureError(LiteRuntimeError):
    """A worker rank stopped answering (heartbeat lost) or reported a device status error."""
