from . import bootstrap, cpu_model, launch  # noqa: F401
