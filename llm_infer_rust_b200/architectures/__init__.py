"""Importing this package registers the architectures that ship with the engine."""
from . import kefetar, lufizen, mukenex, qwen3, torinex  # noqa: F401
