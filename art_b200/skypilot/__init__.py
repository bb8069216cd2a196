from .backend import SkyPilotBackend, stop_server

__all__ = ["SkyPilotBackend", "stop_server"]
