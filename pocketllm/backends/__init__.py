from .base import BackendBase
from .factory import create_backend, detect_model_format, select_backend
from .native_backend import NativeBackend

__all__ = ["BackendBase", "NativeBackend", "create_backend", "detect_model_format", "select_backend"]
