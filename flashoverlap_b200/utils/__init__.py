from . import config, layout, timing  # noqa: F401
