"""Exception taxonomy of the public API; the HTTP server maps each class to a status code
(same class names as the reference, pocketllm/api/errors.py:6-27)."""


class PocketLLMError(Exception):
    """Base class of every error raised on purpose by this package."""


class ConfigurationError(PocketLLMError, ValueError):
    """Bad engine arguments or request parameters (HTTP 400)."""


class BackendUnavailableError(PocketLLMError, RuntimeError):
    """The native engine cannot be loaded or is not ready (HTTP 503)."""


class UnsupportedFeatureError(PocketLLMError, NotImplementedError):
    """The request asks for something the loaded model runtime cannot do (HTTP 501)."""


class RequestCancelledError(PocketLLMError):
    """The request was cancelled by the client (HTTP 499)."""


class TensorParallelSupervisorError(PocketLLMError, RuntimeError):
    """A tensor-parallel rank failed to start, never became ready, or died."""
