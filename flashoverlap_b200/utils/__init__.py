from . import config, layout  # noqa: F401
