"""Architectures.  Importing this package registers every architecture the library has."""
from .model import LayerCall, Model
from . import lfm2  # noqa: F401  (registers Lfm2ForCausalLM)
from . import ponusun  # noqa: F401  (registers Ponusun)
from . import zosurax  # noqa: F401  (registers Zosurax)
from . import kerotar  # noqa: F401  (registers Kerotar)
from . import pirisun  # noqa: F401  (registers Pirisun)
