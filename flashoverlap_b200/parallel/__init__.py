from . import bootstrap, cpu_model  # noqa: F401
