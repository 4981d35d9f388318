from .model import Rutusun, RutusunArgs, rutusun_configs  # noqa: F401
