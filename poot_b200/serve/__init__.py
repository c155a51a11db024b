"""OpenAI-compatible serving: continuous-batching engine thread, std-only HTTP server, metrics."""
from .config import ServeConfig, parse_args
from .http import ApiError, Server, ServerState, sampling_from_request
from .metrics import Metrics
from .scheduler import EngineDead, Job, ServeEngine
