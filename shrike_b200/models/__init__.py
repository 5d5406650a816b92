"""Architectures this engine serves.  Importing the package registers them."""

from . import kavedra, qwen2, sadodra, setotar, vupitar  # noqa: F401
