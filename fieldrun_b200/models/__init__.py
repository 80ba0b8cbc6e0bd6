"""Built-in architectures; importing this package registers them."""
from . import bakasun, bamasun, depelix, fotanex, minimax_m2  # noqa: F401
