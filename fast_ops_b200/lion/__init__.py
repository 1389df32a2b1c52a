from .lion_optimizer import Lion, lion_update  # noqa: F401
from .zero1 import FlatLayout  # noqa: F401
