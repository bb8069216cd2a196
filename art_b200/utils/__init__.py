from .format_message import format_message
from .get_model_step import get_model_step
from .iterate_dataset import iterate_dataset
from .limit_concurrency import limit_concurrency
from .log_http_errors import log_http_errors
from .retry import retry

__all__ = ["format_message", "get_model_step", "iterate_dataset", "limit_concurrency", "log_http_errors", "retry"]
