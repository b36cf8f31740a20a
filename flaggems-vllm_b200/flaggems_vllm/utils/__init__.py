from . import device_info  # noqa: F401
