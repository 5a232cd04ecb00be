"""The built-in architectures; importing this package registers them."""
from . import buguzen, lefatar, llama, sazepel  # noqa: F401
