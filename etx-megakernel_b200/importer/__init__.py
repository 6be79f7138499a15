from . import argblock, spec

__all__ = ["argblock", "spec"]
