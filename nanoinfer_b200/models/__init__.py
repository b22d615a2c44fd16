"""Architectures: each module registers its config parser and tensor naming."""
from . import llama, runevik, tazulix, vuvalorn  # noqa: F401
