from .metrics import Metrics
from .openai import make_server, serve

__all__ = ["Metrics", "make_server", "serve"]
