from .api_server import eSurgeApiServer, create_app  # noqa: F401
