"""Parts a model is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401
from .base import register_part, unregister_part  # noqa: F401
