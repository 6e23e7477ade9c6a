"""Architectures: importing this package registers them."""
from . import bapavik, gebilorn, lilunex, llama, rogisun  # noqa: F401
from .decoder import DecoderModel  # noqa: F401
