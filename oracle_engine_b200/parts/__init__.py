"""Parts of a layer and the model built from them; importing the package registers the
built-in parts (see registry.py for the interfaces)."""
from . import registry, spec                                                   # noqa: F401
from . import attention, block, embedding, feedforward, norms, positions      # noqa: F401
