from . import functional, native

__all__ = ["functional", "native"]
