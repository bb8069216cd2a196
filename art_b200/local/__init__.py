from .backend import LocalBackend

__all__ = ["LocalBackend"]
