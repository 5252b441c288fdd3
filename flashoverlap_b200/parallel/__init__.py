from . import bootstrap, cpu_model, launch, symm  # noqa: F401
