"""Importing this package registers every architecture the engine has."""
from . import busadra, ditalorn, lulenex, qwen3, zabonex  # noqa: F401
