"""Architectures: each module registers its config parser and tensor naming."""
from . import llama, mobatar, runevik, tazulix, vuvalorn  # noqa: F401
