"""The built-in architectures; importing this package registers them."""
from . import buguzen, lefatar, llama, mavidra, sazepel  # noqa: F401
