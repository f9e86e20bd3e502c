from .jsonc import loads as jsonc_loads, load as jsonc_load  # noqa: F401
from .model import BenchConfig, load_config  # noqa: F401
