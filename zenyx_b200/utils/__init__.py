from .logging import get_logger, set_log_level, setup_logging

__all__ = ["setup_logging", "get_logger", "set_log_level"]
